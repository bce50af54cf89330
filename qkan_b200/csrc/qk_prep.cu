// Small set-up and finishing kernels around the two hot kernels:
//   prep         : per-edge constant table(s) (trig of theta, merged phases, folded mask) and
//                  bias[o] = sum_i postact_bias * postact_weights * mask, one launch
//   finish_grads : fixed-order sum of the per-batch-tile partials into the
//                  reference's parameter layouts
// (the column sums of grad_y that the postact-bias terms need are taken inside the backward kernel)
#include "qk_kernels.cuh"

namespace qk {

// Constants of edge (o, i) into the generic table and, when wanted, into the frozen-preact forward's table
// (same layout; its rows (pw_l, c_l) hold (cos c_l, sin c_l)).
__device__ void prep_edge(const PrepArgs& a, int o, int i) {
    const int R = a.reps, RK = a.rk;
    const int K = table_stride(RK);
    float* t = a.table + ((size_t)o * a.ipad + i) * K;
    float* tx = a.table_x ? a.table_x + ((size_t)o * a.ipad + i) * K : nullptr;
    auto put = [&](int row, float v) {
        t[row] = v;
        if (tx) tx[row] = v;
    };
    if (i >= a.in_dim) {
        for (int k = 0; k < K; ++k) put(k, 0.f);
        if (a.basew_c) a.basew_c[(size_t)o * a.ipad + i] = 0.f;
        return;
    }
    const size_t e = (size_t)o * a.in_dim + i;
    const size_t q = a.group > 0 ? (size_t)(i % a.group) : e;  // entry of theta / preacts this edge reads
    const float m = a.mask ? ld_param(a.mask, a.param_dtype, e) : 1.f;
    const float w = a.postw ? ld_param(a.postw, a.param_dtype, e) * m : 1.f;
    const float bw = a.basew ? ld_param(a.basew, a.param_dtype, e) * m : 0.f;
    if (a.basew_c) a.basew_c[(size_t)o * a.ipad + i] = bw;  // the base-term backward reads it as a dense matrix
    // rpz always encodes pw*x + pb (src/qkan/solver/exact.py:75-76)
    const bool ptr = (a.flags & QK_PREACT_TRAINABLE) != 0 || a.ansatz == QK_ANSATZ_RPZ;

    if (a.ansatz == QK_ANSATZ_REAL) {
        // alpha = A x + C; C is reduced to [-pi, pi] in double so the SFU sees a small argument
        const float* th = a.theta + q * R;
        double A = 0.0, C = 1.5707963267948966;
        for (int l = 0; l < R; ++l) {
            A += ptr ? (double)a.pw[q * R + l] : 1.0;
            C += (ptr ? (double)a.pb[q * R + l] : 0.0) - (double)th[l] - 3.141592653589793;
        }
        C -= 6.283185307179586 * rint(C / 6.283185307179586);
        for (int k = 0; k < K; ++k) put(k, 0.f);
        put(0, (float)A);
        put(1, (float)C);
        put(t_w(0), w);
        put(t_bw(0), bw);
        return;
    }

    const bool pz = a.ansatz == QK_ANSATZ_PZ;
    const int ts = pz ? 2 : 1;  // floats of theta per layer
    const float* th = a.theta + q * (R + 1) * ts;
    auto th_ry = [&](int l) { return pz ? th[2 * l + 1] : th[l]; };   // Ry angle of layer l
    auto th_rz = [&](int l) { return pz ? th[2 * l] : 0.f; };          // Rz angle of layer l (pz only)
    float s00, c00, sa0, ca0;
    sincosf(th_rz(0), &s00, &c00);
    sincosf(th_ry(0), &sa0, &ca0);
    // start vector: Ry(theta_ry[0]) Rz(theta_rz[0]) applied to (1,0,0)
    put(t_vx0(), c00 * ca0);
    put(t_vy0(), s00);
    put(t_vz0(), -c00 * sa0);
    put(t_ca0(RK), ca0);
    put(t_sa0(RK), sa0);
    for (int l = 0; l < RK; ++l) {
        if (l < R) {
            put(t_pw(l), ptr ? a.pw[q * R + l] : 1.f);
            put(t_c(l), (ptr ? a.pb[q * R + l] : 0.f) + th_rz(l + 1));
            if (tx) {  // frozen preacts, angle x + c_l: that forward wants cos/sin of c_l
                float s, c;
                sincosf(th_rz(l + 1), &s, &c);
                tx[t_pw(l)] = c;
                tx[t_c(l)] = s;
            }
        } else {  // identity padding
            put(t_pw(l), 0.f);
            put(t_c(l), 0.f);
        }
        if (l >= 1) {
            float s = 0.f, c = 1.f;
            if (l < R) sincosf(th_ry(l), &s, &c);
            put(t_ca(RK, l), c);
            put(t_sa(RK, l), s);
        }
    }
    float sf, cf;
    sincosf(th_ry(R), &sf, &cf);
    put(t_cf(RK), cf);
    put(t_sf(RK), sf);
    put(t_w(RK), w);
    put(t_bw(RK), bw);
}

// One CTA per output: its threads walk the input columns, write each edge's constants and add up
// bias[o] = sum_i postact_bias * postact_weights * mask in a fixed order (thread-strided partial sums, then a
// shared-memory tree): run-to-run reproducible.
constexpr int kPrepThreads = 128;
__global__ void __launch_bounds__(kPrepThreads) prep_kernel(PrepArgs a) {
    __shared__ float sm[kPrepThreads];
    const int o = blockIdx.x;
    const bool want_bias = a.bias != nullptr;
    const bool use_pb = want_bias && a.postb && (a.flags & QK_USE_POSTACT_BIAS);
    float s = 0.f;
    for (int i = threadIdx.x; i < a.ipad; i += kPrepThreads) {
        prep_edge(a, o, i);
        if (use_pb && i < a.in_dim) {
            const size_t e = (size_t)o * a.in_dim + i;
            const float m = a.mask ? ld_param(a.mask, a.param_dtype, e) : 1.f;
            const float w = a.postw ? ld_param(a.postw, a.param_dtype, e) * m : 1.f;
            s = fmaf(ld_param(a.postb, a.param_dtype, e), w, s);
        }
    }
    if (!want_bias) return;
    sm[threadIdx.x] = s;
    __syncthreads();
    for (int d = kPrepThreads / 2; d >= 1; d >>= 1) {
        if (threadIdx.x < d) sm[threadIdx.x] += sm[threadIdx.x + d];
        __syncthreads();
    }
    if (threadIdx.x == 0) a.bias[o] = sm[0];
}

// Block = 32 input columns (one lane each) x `blockDim.y` tile slices. Every slice adds the per-tile
// partials t = slice, slice + slices, ... of each accumulator row; slice 0 then adds the slice sums in
// order and writes the gradients. Fixed order throughout: run-to-run bitwise reproducible. The sums across
// tiles run in double (the kernel is bound by reading the partials, not by these adds): near a minimum the
// batch sum cancels to a small value, and optimisers that difference gradients (LBFGS) feel its rounding.
__global__ void finish_grads_kernel(FinishArgs a) {
    // [slices][nacc + 2][32]; the extra rows are the base-term kernel's partials and the column sums of grad_y
    extern __shared__ double part[];
    const int lane = threadIdx.x, slice = threadIdx.y, slices = blockDim.y;
    const int i = blockIdx.x * kWarp + lane;  // < ipad
    const int o = blockIdx.y;
    const int R = a.reps, RK = a.rk;
    const int nacc = a.nacc, nrow = a.nacc + 2;
    const size_t tile_stride = (size_t)a.out_dim * nacc * a.ipad;
    const float* p0 = a.partials + ((size_t)o * nacc) * a.ipad + i;
    // one accumulator row after the other (four rows at a time, i.e. four times the loads in flight per thread,
    // measured TWICE as slow at 65536 x 256 -> 256: 0.44 against 0.21 ms)
    for (int k = 0; k < nacc; ++k) {
        const float* p = p0 + (size_t)k * a.ipad;
        double s = 0.0;
        for (int t = slice; t < a.ntiles; t += slices) s += (double)p[(size_t)t * tile_stride];
        part[(slice * nrow + k) * kWarp + lane] = s;
    }
    {
        double s = 0.0;
        if (a.base_partials) {
            const float* bp = a.base_partials + (size_t)o * a.ipad + i;
            for (int t = slice; t < a.base_tiles; t += slices) s += (double)bp[(size_t)t * a.out_dim * a.ipad];
        }
        part[(slice * nrow + nacc) * kWarp + lane] = s;
    }
    {
        // sum_b grad_y[b,o] from the per-tile column sums (the same value in every lane)
        double s = 0.0;
        if (a.colpart)
            for (int t = slice; t < a.ntiles; t += slices) s += (double)a.colpart[(size_t)t * a.out_dim + o];
        part[(slice * nrow + nacc + 1) * kWarp + lane] = s;
    }
    __syncthreads();
    if (slice != 0 || i >= a.in_dim) return;
    const size_t e = (size_t)o * a.in_dim + i;
    const bool ptr = (a.flags & QK_PREACT_TRAINABLE) != 0 || a.ansatz == QK_ANSATZ_RPZ;
    const bool use_pb = (a.flags & QK_USE_POSTACT_BIAS) != 0 && a.postb != nullptr;
    auto total = [&](int k) {
        double s = 0.0;
        for (int w = 0; w < slices; ++w) s += part[(w * nrow + k) * kWarp + lane];
        return (float)s;
    };
    if (a.ansatz == QK_ANSATZ_REAL) {
        // d alpha / d theta_l = -1, / d pb_l = 1, / d pw_l = x for every layer l
        const float s1 = (a.gtheta || a.gpb) ? total(0) : 0.f;
        const float s2 = a.gpw ? total(1) : 0.f;
        for (int l = 0; l < R; ++l) {
            if (a.gtheta) a.gtheta[e * R + l] = -s1;
            if (a.gpb) a.gpb[e * R + l] = ptr ? s1 : 0.f;
            if (a.gpw) a.gpw[e * R + l] = ptr ? s2 : 0.f;
        }
    } else if (a.ansatz == QK_ANSATZ_RPZ) {
        if (a.gtheta) {
            float* g = a.gtheta + e * (R + 1);
            for (int l = 0; l < R; ++l) g[l] = total(a_ry(l));
            g[R] = total(a_ry(RK));
        }
        if (a.gpb)
            for (int l = 0; l < R; ++l) a.gpb[e * R + l] = total(a_c(RK, l));
        if (a.gpw)
            for (int l = 0; l < R; ++l) a.gpw[e * R + l] = total(a_pwx(RK, l));
    } else {
        if (a.gtheta) {
            float* g = a.gtheta + e * (R + 1) * 2;
            g[0] = total(a_t00(RK));
            for (int l = 0; l < R; ++l) g[2 * l + 1] = total(a_ry(l));
            g[2 * R + 1] = total(a_ry(RK));
            for (int l = 0; l < R; ++l) g[2 * (l + 1)] = total(a_c(RK, l));
        }
        if (a.gpb)
            for (int l = 0; l < R; ++l) a.gpb[e * R + l] = ptr ? total(a_c(RK, l)) : 0.f;
        if (a.gpw)
            for (int l = 0; l < R; ++l) a.gpw[e * R + l] = ptr ? total(a_pwx(RK, l)) : 0.f;
    }
    if (a.gpostw || a.gpostb || a.gbasew) {
        const float cs = (use_pb && a.colpart) ? total(nacc + 1) : 0.f;
        float m = a.mask ? ld_param(a.mask, a.param_dtype, e) : 1.f;
        if (a.gpostw) {
            float pbv = use_pb ? ld_param(a.postb, a.param_dtype, e) : 0.f;
            a.gpostw[e] = m * fmaf(pbv, cs, total(a_w(RK)));
        }
        if (a.gpostb) {
            float w = a.postw ? ld_param(a.postw, a.param_dtype, e) * m : 1.f;
            a.gpostb[e] = use_pb ? w * cs : 0.f;
        }
        if (a.gbasew) a.gbasew[e] = m * total(nacc);
    }
}

// One CTA per (group entry k, component c): threads take the (o, j) pairs, i = k + j*group, in a fixed
// strided order and a shared-memory tree adds them, so the result is run-to-run reproducible.
__global__ void group_reduce_kernel(const float* __restrict__ src, float* __restrict__ dst, int out_dim,
                                    int in_dim, int group, int per) {
    __shared__ float sm[256];
    const int k = blockIdx.x, c = blockIdx.y;
    const int nj = (in_dim - k + group - 1) / group;  // inputs i = k, k+group, ... < in_dim
    const long long n = (long long)out_dim * nj;
    float s = 0.f;
    for (long long idx = threadIdx.x; idx < n; idx += blockDim.x) {
        const int o = (int)(idx / nj), j = (int)(idx - (long long)o * nj);
        s += src[((size_t)o * in_dim + k + (size_t)j * group) * per + c];
    }
    sm[threadIdx.x] = s;
    __syncthreads();
    for (int d = 128; d >= 1; d >>= 1) {
        if (threadIdx.x < d) sm[threadIdx.x] += sm[threadIdx.x + d];
        __syncthreads();
    }
    if (threadIdx.x == 0) dst[(size_t)k * per + c] = sm[0];
}

cudaError_t launch_group_reduce(const float* src, float* dst, int out_dim, int in_dim, int group, int per,
                                cudaStream_t st) {
    dim3 grid(group, per);
    group_reduce_kernel<<<grid, 256, 0, st>>>(src, dst, out_dim, in_dim, group, per);
    return cudaPeekAtLastError();
}

template <typename IO>
__global__ void sum_gx_kernel(const float* __restrict__ part, IO* __restrict__ gx, size_t n, int nslices) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    float s = 0.f;
    for (int z = 0; z < nslices; ++z) s += part[(size_t)z * n + idx];
    st_from_float(gx + idx, s);
}

cudaError_t launch_sum_gx(const float* part, void* gx, int io_dtype, size_t n, int nslices, cudaStream_t st) {
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (io_dtype == QK_BF16)
        sum_gx_kernel<<<blocks, 256, 0, st>>>(part, static_cast<__nv_bfloat16*>(gx), n, nslices);
    else
        sum_gx_kernel<<<blocks, 256, 0, st>>>(part, static_cast<float*>(gx), n, nslices);
    return cudaPeekAtLastError();
}

cudaError_t launch_prep(const PrepArgs& a, cudaStream_t st) {
    prep_kernel<<<a.out_dim, kPrepThreads, 0, st>>>(a);
    return cudaPeekAtLastError();
}

cudaError_t launch_finish(const FinishArgs& a, cudaStream_t st) {
    // as many tile slices as there are tiles to share out, within 48 KB of shared memory; a grid that leaves SMs
    // idle anyway (narrow layers) takes 16 slices, i.e. half as long a chain of dependent loads per thread
    int slices = (long)(a.ipad / kWarp) * a.out_dim < 2 * 148 ? 16 : 8;
    const int most_tiles = a.ntiles > a.base_tiles ? a.ntiles : a.base_tiles;
    while (slices > 1 && (slices / 2 >= most_tiles || (size_t)slices * (a.nacc + 2) * kWarp * sizeof(double) > 48 * 1024))
        slices /= 2;
    dim3 grid(a.ipad / kWarp, a.out_dim), block(kWarp, slices);
    finish_grads_kernel<<<grid, block, (size_t)slices * (a.nacc + 2) * kWarp * sizeof(double), st>>>(a);
    return cudaPeekAtLastError();
}

}  // namespace qk
