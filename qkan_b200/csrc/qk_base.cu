// Backward of the base term  y += silu(x) @ (base_weight * mask)^T  of the layer epilogue
// (reference: src/qkan/qkan.py:755, 784; the reference's fused epilogue leaves these two products to a
// library GEMM, src/qkan/qkan_epilogue.py:517-522):
//   grad_base_weight[o,i] = mask[o,i] * sum_b grad_y[b,o] * silu(x[b,i])
//   grad_x[b,i]          += silu'(x[b,i]) * sum_o grad_y[b,o] * base_weight[o,i] * mask[o,i]
// Both are dense (B x O x I) contractions, 2 FMAs per edge and row together, and they are computed as two
// register-tiled float32 matrix products inside ONE launch (float32 on the FP32 pipe: the products meet the
// 1e-5 parity bound without a split-precision scheme):
//   * CTAs of the first kind own a (rows x columns) tile of grad_x and walk all outputs;
//   * CTAs of the second kind own an (outputs x columns) tile of grad_base_weight and walk one slab of batch
//     rows; the slabs' results go to scratch as partials and finish_grads adds them in slab order (no atomics,
//     bitwise reproducible).
// A CTA is 16 x 16 threads; a thread holds an F x F block of the tile (F = 8 for 128 x 128 tiles, 4 for 64 x 64)
// as packed column pairs. Operands are staged k-major in shared memory, double buffered, the next tile fetched
// into registers (one 128-bit load per thread and operand) during the multiply: F*F/2 packed FMAs per F/2
// 128-bit shared loads and F register moves (the broadcast operand's pairs) in the inner loop. Staging A as ready
// (a, a) pairs instead (no moves, F/4 more shared loads) measured 1 % slower, scalar FMAs the same.
#include "qk_kernels.cuh"
#include "qk_packed.cuh"

namespace qk {

namespace {

constexpr int kBaseThreads = 256;
// The 16 x 16 thread grid of a CTA: a warp covers 4 (ty) x 8 (tx) of it, so that its shared loads of B touch 8
// distinct 16-byte groups and those of A four.
__device__ __forceinline__ int base_tx() { return ((threadIdx.x / 32) % 2) * 8 + threadIdx.x % 8; }
__device__ __forceinline__ int base_ty() { return (threadIdx.x / 64) * 4 + (threadIdx.x % 32) / 8; }

__device__ __forceinline__ float sigmoid_f(float v) { return 1.f / (1.f + expf(-v)); }

// Four consecutive values starting at p (16-byte aligned for float, 8-byte for bfloat16).
__device__ __forceinline__ void ld4(const float* p, float (&v)[4], bool read_only) {
    const float4 q = read_only ? __ldg(reinterpret_cast<const float4*>(p)) : *reinterpret_cast<const float4*>(p);
    v[0] = q.x, v[1] = q.y, v[2] = q.z, v[3] = q.w;
}
__device__ __forceinline__ void ld4(const __nv_bfloat16* p, float (&v)[4], bool read_only) {
    const uint2 q = read_only ? __ldg(reinterpret_cast<const uint2*>(p)) : *reinterpret_cast<const uint2*>(p);
    v[0] = __uint_as_float(q.x << 16), v[1] = __uint_as_float(q.x & 0xffff0000u);
    v[2] = __uint_as_float(q.y << 16), v[3] = __uint_as_float(q.y & 0xffff0000u);
}
__device__ __forceinline__ void st4(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void st4(__nv_bfloat16* p, const float (&v)[4]) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
    uint2 q;
    q.x = *reinterpret_cast<const unsigned*>(&lo);
    q.y = *reinterpret_cast<const unsigned*>(&hi);
    *reinterpret_cast<uint2*>(p) = q;
}

// Columns c .. c+3 of one matrix row (`row` points at its first element) as floats; zero for a row outside the
// problem and for columns >= cmax. `vec`: rows of this matrix may be read four columns at a time.
template <typename P>
__device__ __forceinline__ float4 load4(const P* row, bool row_ok, int c, int cmax, bool vec) {
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (row_ok) {
        if (vec && c + 3 < cmax) {
            ld4(row + c, v, true);
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (c + j < cmax) v[j] = ld_as_float(row + c + j);
        }
    }
    return make_float4(v[0], v[1], v[2], v[3]);
}

template <int T>
struct BaseTile {
    static constexpr int F = T / 16;        // edge of a thread's block
    static constexpr int TK = 1024 / T;     // depth of a staged operand tile: four values per thread and operand
    static constexpr int LDA = T + 4;       // staged row of A, 128-bit aligned, banks spread
    static constexpr int LDB = T + 4;       // staged row of B
};

// One CTA's product  acc[m][n] = sum_k A(k, m) * B(k, n)  over `nk` staged tiles of depth TK. fetch_*(kt) returns
// the thread's four values of operand tile kt (global loads only, so that they stay in flight during the multiply);
// stage_*(dst, v) puts them into the staged tile `dst` (A at [k * LDA + m], B at [k * LDB + n]).
template <int T, typename FA, typename FB, typename SA, typename SB>
__device__ __forceinline__ void tile_product(int nk, FA fetch_a, FB fetch_b, SA stage_a, SB stage_b,
                                             float (&As)[2][BaseTile<T>::TK * BaseTile<T>::LDA],
                                             float (&Bs)[2][BaseTile<T>::TK * BaseTile<T>::LDB],
                                             f2 (&acc)[T / 16][T / 32]) {
    using C = BaseTile<T>;
    constexpr int F = C::F;
    const int tx = base_tx(), ty = base_ty();
#pragma unroll
    for (int m = 0; m < F; ++m)
#pragma unroll
        for (int n = 0; n < F / 2; ++n) acc[m][n] = pk(0.f);
    if (nk <= 0) return;
    float4 ra = fetch_a(0), rb = fetch_b(0);
    stage_a(As[0], ra);
    stage_b(Bs[0], rb);
    __syncthreads();
    for (int kt = 0, buf = 0; kt < nk; ++kt, buf ^= 1) {
        const bool more = kt + 1 < nk;
        if (more) {
            ra = fetch_a(kt + 1);
            rb = fetch_b(kt + 1);
        }
        // 128-wide tiles: not unrolled (one step's F/2 loads and F*F/2 packed FMAs already fill the register budget of
        // two CTAs per SM); 64-wide tiles (small, latency-bound problems): unrolled, the shared loads run ahead
#pragma unroll(F == 8 ? 1 : C::TK)
        for (int k = 0; k < C::TK; ++k) {
            f2 a2[F], b2[F / 2];
#pragma unroll
            for (int h = 0; h < F / 4; ++h) {
                const float4 a4 = *reinterpret_cast<const float4*>(&As[buf][k * C::LDA + h * 64 + ty * 4]);
                const float4 b4 = *reinterpret_cast<const float4*>(&Bs[buf][k * C::LDB + h * 64 + tx * 4]);
                a2[4 * h] = pk(a4.x), a2[4 * h + 1] = pk(a4.y), a2[4 * h + 2] = pk(a4.z), a2[4 * h + 3] = pk(a4.w);
                b2[2 * h] = make_float2(b4.x, b4.y), b2[2 * h + 1] = make_float2(b4.z, b4.w);
            }
#pragma unroll
            for (int m = 0; m < F; ++m)
#pragma unroll
                for (int n = 0; n < F / 2; ++n) acc[m][n] = fma2(a2[m], b2[n], acc[m][n]);
        }
        // the other buffer was last read before the barrier that ended the previous round
        if (more) {
            stage_a(As[buf ^ 1], ra);
            stage_b(Bs[buf ^ 1], rb);
        }
        __syncthreads();
    }
}

template <typename IO, int T>
__global__ void __launch_bounds__(kBaseThreads, 2) base_backward_kernel(BaseBwdArgs a) {
    using C = BaseTile<T>;
    constexpr int F = C::F, TK = C::TK, LDA = C::LDA, LDB = C::LDB;
    __shared__ __align__(16) float As[2][TK * LDA];
    __shared__ __align__(16) float Bs[2][TK * LDB];
    const int tx = base_tx(), ty = base_ty();
    const IO* __restrict__ x = static_cast<const IO*>(a.x);
    const IO* __restrict__ gy = static_cast<const IO*>(a.gy);
    const int tiles_i = (a.ipad + T - 1) / T, tiles_o = (a.out_dim + T - 1) / T;
    const int weight_ctas = a.partials ? a.slabs * tiles_o * tiles_i : 0;
    f2 acc[F][F / 2];
    // a thread's four values of a row-major operand tile (TK rows of T columns): row kr, columns c4 .. c4+3
    const int kr = threadIdx.x / (T / 4), c4 = (threadIdx.x % (T / 4)) * 4;
    auto stage_a_rows = [&](float* dst, const float4& v) {  // A(k = kr, m = c4 .. c4+3)
        *reinterpret_cast<float4*>(dst + kr * LDA + c4) = v;
    };

    if ((int)blockIdx.x < weight_ctas) {
        // grad_base_weight tile (outputs o0.., columns i0..) over the batch rows of one slab:
        // A(k = row, m = output) = grad_y, B(k = row, n = column) = silu(x); both lie row-major
        const int ti = blockIdx.x % tiles_i, to = (blockIdx.x / tiles_i) % tiles_o, slab = blockIdx.x / (tiles_i * tiles_o);
        const int i0 = ti * T, o0 = to * T, r0 = slab * a.slab_rows, r1 = min(a.batch, r0 + a.slab_rows);
        auto fetch_a = [&](int kt) {
            const int r = r0 + kt * TK + kr;
            return load4(gy + (size_t)r * a.out_dim, r < r1, o0 + c4, a.out_dim, a.vec_gy != 0);
        };
        auto fetch_b = [&](int kt) {
            const int r = r0 + kt * TK + kr;
            return load4(x + (size_t)r * a.in_dim, r < r1, i0 + c4, a.in_dim, a.vec4 != 0);
        };
        auto stage_b = [&](float* dst, const float4& v) {
            *reinterpret_cast<float4*>(dst + kr * LDB + c4) =
                make_float4(v.x * sigmoid_f(v.x), v.y * sigmoid_f(v.y), v.z * sigmoid_f(v.z), v.w * sigmoid_f(v.w));
        };
        tile_product<T>((r1 - r0 + TK - 1) / TK, fetch_a, fetch_b, stage_a_rows, stage_b, As, Bs, acc);
#pragma unroll
        for (int m = 0; m < F; ++m) {
            const int o = o0 + (m / 4) * 64 + ty * 4 + m % 4;
            if (o >= a.out_dim) continue;
#pragma unroll
            for (int h = 0; h < F / 4; ++h) {
                const int i = i0 + h * 64 + tx * 4;  // ipad is a multiple of 32: a group of four is inside or outside
                if (i < a.ipad)
                    *reinterpret_cast<float4*>(a.partials + ((size_t)slab * a.out_dim + o) * a.ipad + i) =
                        make_float4(acc[m][2 * h].x, acc[m][2 * h].y, acc[m][2 * h + 1].x, acc[m][2 * h + 1].y);
            }
        }
        return;
    }

    // grad_x tile (rows b0.., columns i0..) over all outputs: A(k = output, m = row) = grad_y, read along its rows
    // (row ma, outputs k4 .. k4+3 of the depth) and staged transposed; B(k = output, n = column) = base_weight * mask
    const int bid = blockIdx.x - weight_ctas;
    const int i0 = (bid % tiles_i) * T, b0 = (bid / tiles_i) * T;
    const int ma = threadIdx.x / (TK / 4), k4 = (threadIdx.x % (TK / 4)) * 4;
    auto fetch_a = [&](int kt) {
        const int b = b0 + ma;
        return load4(gy + (size_t)b * a.out_dim, b < a.batch, kt * TK + k4, a.out_dim, a.vec_gy != 0);
    };
    auto stage_a = [&](float* dst, const float4& v) {
        float* p = dst + k4 * LDA + ma;
        p[0] = v.x, p[LDA] = v.y, p[2 * LDA] = v.z, p[3 * LDA] = v.w;
    };
    auto fetch_b = [&](int kt) {  // rows of the dense base-weight matrix are ipad long and 128-byte aligned
        const int o = kt * TK + kr;
        return load4(a.basew + (size_t)o * a.ipad, o < a.out_dim, i0 + c4, a.ipad, true);
    };
    auto stage_b = [&](float* dst, const float4& v) { *reinterpret_cast<float4*>(dst + kr * LDB + c4) = v; };
    tile_product<T>((a.out_dim + TK - 1) / TK, fetch_a, fetch_b, stage_a, stage_b, As, Bs, acc);

    IO* __restrict__ gx = static_cast<IO*>(a.gx);
    auto dsilu = [](float v) {
        const float sg = sigmoid_f(v);
        return sg * (1.f + v * (1.f - sg));
    };
#pragma unroll
    for (int m = 0; m < F; ++m) {
        const int b = b0 + (m / 4) * 64 + ty * 4 + m % 4;
        if (b >= a.batch) continue;
#pragma unroll
        for (int h = 0; h < F / 4; ++h) {
            const int i = i0 + h * 64 + tx * 4;
            if (i >= a.in_dim) continue;
            const size_t at = (size_t)b * a.in_dim + i;
            const float s[4] = {acc[m][2 * h].x, acc[m][2 * h].y, acc[m][2 * h + 1].x, acc[m][2 * h + 1].y};
            // grad_x is read and written by this kernel: plain loads for it (the read-only path is for data the
            // kernel never writes). With bfloat16 activations the circuit share was rounded once when the backward
            // stored it and the sum is rounded again here (half an ulp each, inside the bf16 bound).
            if (a.vec4 && i + 3 < a.in_dim) {
                float xv[4], g[4];
                ld4(x + at, xv, true);
                ld4(gx + at, g, false);
#pragma unroll
                for (int j = 0; j < 4; ++j) g[j] = fmaf(dsilu(xv[j]), s[j], g[j]);
                st4(gx + at, g);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (i + j < a.in_dim)
                        st_from_float(gx + at + j, fmaf(dsilu(ld_as_float(x + at + j)), s[j], ld_rw_as_float(gx + at + j)));
            }
        }
    }
}

}  // namespace

BasePlan base_plan(int batch, int in_dim, int out_dim) {
    BasePlan p{};
    const int ipad = round_up(in_dim, 32);
    // 128 x 128 tiles (two CTAs resident per SM) unless the grad_x tiles would then leave SMs without work
    const long big = (long)((batch + 127) / 128) * ((ipad + 127) / 128);
    p.tile = big >= 2 * 148 ? 128 : 64;
    const int wave = 148 * (p.tile == 128 ? 2 : 3);
    const long weight_tiles = (long)((out_dim + p.tile - 1) / p.tile) * ((ipad + p.tile - 1) / p.tile);
    // Slabs of batch rows for grad_base_weight: about one wave of CTAs (they are the long ones and are launched
    // first, the grad_x tiles fill in behind them), no shorter than 16 rows (small problems are latency-bound: many
    // short slabs mean short chains of dependent tiles and a flat summation tree), and no longer than 4096 rows so
    // that a float32 running sum stays well inside the parity bound.
    long slabs = weight_tiles > 0 ? wave / weight_tiles : 1;
    const long most = (batch + 15) / 16, least = (batch + 4095) / 4096;
    if (slabs > most) slabs = most;
    if (slabs < least) slabs = least;
    if (slabs < 1) slabs = 1;
    const int rows = (int)((batch + slabs - 1) / slabs);
    p.slab_rows = 16;  // a power of two: whole staged tiles
    while (p.slab_rows < rows) p.slab_rows *= 2;
    p.slabs = (batch + p.slab_rows - 1) / p.slab_rows;
    if (p.slabs < 1) p.slabs = 1;
    return p;
}

cudaError_t launch_base_backward(const BaseBwdArgs& args, int io_dtype, cudaStream_t st) {
    BaseBwdArgs a = args;
    const BasePlan p = base_plan(a.batch, a.in_dim, a.out_dim);
    a.slab_rows = p.slab_rows;
    a.slabs = p.slabs;
    const size_t el = io_dtype == QK_BF16 ? 2 : 4;
    a.vec4 = a.in_dim % 4 == 0 && (uintptr_t)a.x % (4 * el) == 0 && (uintptr_t)a.gx % (4 * el) == 0;
    a.vec_gy = a.out_dim % 4 == 0 && (uintptr_t)a.gy % (4 * el) == 0;
    const long tiles_i = (a.ipad + p.tile - 1) / p.tile;
    const long weight_ctas = a.partials ? (long)p.slabs * ((a.out_dim + p.tile - 1) / p.tile) * tiles_i : 0;
    const long gx_ctas = a.gx ? (long)((a.batch + p.tile - 1) / p.tile) * tiles_i : 0;
    const long grid = weight_ctas + gx_ctas;
    if (grid == 0) return cudaSuccess;
    if (grid > 0x7fffffffL) return cudaErrorInvalidConfiguration;
    if (io_dtype == QK_BF16) {
        if (p.tile == 128) base_backward_kernel<__nv_bfloat16, 128><<<(unsigned)grid, kBaseThreads, 0, st>>>(a);
        else base_backward_kernel<__nv_bfloat16, 64><<<(unsigned)grid, kBaseThreads, 0, st>>>(a);
    } else {
        if (p.tile == 128) base_backward_kernel<float, 128><<<(unsigned)grid, kBaseThreads, 0, st>>>(a);
        else base_backward_kernel<float, 64><<<(unsigned)grid, kBaseThreads, 0, st>>>(a);
    }
    return cudaPeekAtLastError();
}

}  // namespace qk
