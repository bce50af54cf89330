// Backward of the base term  y += silu(x) @ (base_weight * mask)^T  of the layer epilogue
// (reference: src/qkan/qkan.py:755, 784; the reference's fused epilogue leaves these two products to a
// library GEMM, src/qkan/qkan_epilogue.py:517-522):
//   grad_base_weight[o,i] = mask[o,i] * sum_b grad_y[b,o] * silu(x[b,i])
//   grad_x[b,i]          += silu'(x[b,i]) * sum_o grad_y[b,o] * base_weight[o,i] * mask[o,i]
// Both are (B x O x I) contractions with 2 FMAs per edge and row. They run here, after the circuit backward,
// with the same mapping (lane = input column, CTA = rows x 32 columns, all outputs walked): silu(x) of the
// thread's rows and the running sums for grad_x stay in registers, grad_y is staged transposed eight outputs
// at a time and read back as 128-bit broadcasts, and the batch sum of grad_base_weight is reduced over the
// warps in shared memory and written as one partial per (row tile, output) for finish_grads.
#include "qk_kernels.cuh"
#include "qk_packed.cuh"

namespace qk {

namespace {

constexpr int kBaseWarps = 8;
constexpr int kBaseChunk = 8;  // outputs per staged grad_y chunk; equal to the warp count (one output per warp below)

__device__ __forceinline__ float sigmoid_f(float v) { return 1.f / (1.f + expf(-v)); }

#ifndef QK_BASE_MINB
#define QK_BASE_MINB 3
#endif
#ifndef QK_BASE_UNROLL
#define QK_BASE_UNROLL 2
#endif
#define QK_PRAGMA(x) _Pragma(#x)
#define QK_UNROLL(n) QK_PRAGMA(unroll n)

template <typename IO, int RPW>
__global__ void __launch_bounds__(kBaseWarps * kWarp, QK_BASE_MINB) base_backward_kernel(BaseBwdArgs a) {
    constexpr int TB = kBaseWarps * RPW;  // rows per CTA
    constexpr int LD = TB + 4;            // staged row length: keeps 128-bit alignment, spreads the banks
    __shared__ __align__(16) float gy_s[2][kBaseChunk][LD];
    __shared__ float bw_s[2][kBaseChunk][kWarp];
    __shared__ float red_s[kBaseWarps][kBaseChunk][kWarp];
    const int lane = threadIdx.x % kWarp, w = threadIdx.x / kWarp;
    const int bt = blockIdx.x, b0 = bt * TB, row0 = w * RPW;
    const int i = blockIdx.y * kWarp + lane;
    const bool col_ok = i < a.in_dim;
    const IO* __restrict__ x = static_cast<const IO*>(a.x);
    const IO* __restrict__ gy = static_cast<const IO*>(a.gy);

    // silu(x) and the running grad_x sums of the thread's rows, held as row pairs (two rows per instruction on
    // the packed float32 operations; the staged grad_y vector delivers the matching pairs)
    f2 sl2[RPW / 2], gxb2[RPW / 2];
#pragma unroll
    for (int r = 0; r < RPW; r += 2) {
        float v[2];
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int b = b0 + row0 + r + k;
            const float xv = (b < a.batch && col_ok) ? ld_as_float(x + (size_t)b * a.in_dim + i) : 0.f;
            v[k] = xv * sigmoid_f(xv);
        }
        sl2[r / 2] = make_float2(v[0], v[1]);
        gxb2[r / 2] = pk(0.f);
    }

    // Software pipeline over chunks of 8 outputs: the next chunk's grad_y tile and base weights are fetched
    // into registers while the current chunk is being multiplied, then stored to the other shared buffer.
    constexpr int PER_THREAD = TB * kBaseChunk / (kBaseWarps * kWarp);  // staged grad_y values per thread
    float gy_next[PER_THREAD], bw_next;
    auto fetch = [&](int oc) {
        const int nch = min(kBaseChunk, a.out_dim - oc);
#pragma unroll
        for (int q = 0; q < PER_THREAD; ++q) {
            const int idx = threadIdx.x + q * (kBaseWarps * kWarp);
            const int r = idx / kBaseChunk, c = idx % kBaseChunk;
            gy_next[q] = (b0 + r < a.batch && c < nch) ? ld_as_float(gy + (size_t)(b0 + r) * a.out_dim + oc + c) : 0.f;
        }
        // thread (w, lane) fetches the weight of output oc + w for column i (one output per warp)
        bw_next = (w < nch && col_ok) ? a.table[((size_t)(oc + w) * a.ipad + i) * a.ks + a.bw_row] : 0.f;
    };
    fetch(0);
    int buf = 0;
    for (int oc = 0; oc < a.out_dim; oc += kBaseChunk, buf ^= 1) {
        const int nch = min(kBaseChunk, a.out_dim - oc);
#pragma unroll
        for (int q = 0; q < PER_THREAD; ++q) {
            const int idx = threadIdx.x + q * (kBaseWarps * kWarp);
            gy_s[buf][idx % kBaseChunk][idx / kBaseChunk] = gy_next[q];
        }
        bw_s[buf][w][lane] = bw_next;
        __syncthreads();
        if (oc + kBaseChunk < a.out_dim) fetch(oc + kBaseChunk);
QK_UNROLL(QK_BASE_UNROLL)
        for (int c = 0; c < kBaseChunk; ++c) {
            const float bw = bw_s[buf][c][lane];
            const f2 bw2 = pk(bw);
            f2 sa = pk(0.f), sb = pk(0.f);  // two independent chains for the batch sum
#pragma unroll
            for (int r = 0; r < RPW; r += 4) {
                const float4 g = *reinterpret_cast<const float4*>(&gy_s[buf][c][row0 + r]);
                const f2 g01 = make_float2(g.x, g.y), g23 = make_float2(g.z, g.w);
                gxb2[r / 2] = fma2(g01, bw2, gxb2[r / 2]);
                gxb2[r / 2 + 1] = fma2(g23, bw2, gxb2[r / 2 + 1]);
                sa = fma2(g01, sl2[r / 2], sa);
                sb = fma2(g23, sl2[r / 2 + 1], sb);
            }
            const float s0 = sa.x, s1 = sa.y, s2 = sb.x, s3 = sb.y;
            // written after this chunk's staging barrier, i.e. after the last chunk's reads
            red_s[w][c][lane] = (s0 + s1) + (s2 + s3);
        }
        __syncthreads();
        // warp w adds output oc + w over the warps (fixed order): this row tile's partial of grad_base_weight
        if (a.partials && w < nch) {
            float s = 0.f;
#pragma unroll
            for (int ww = 0; ww < kBaseWarps; ++ww) s += red_s[ww][w][lane];
            a.partials[((size_t)bt * a.out_dim + oc + w) * a.ipad + i] = s;
        }
    }

    if (a.gx && col_ok) {
        IO* __restrict__ gx = static_cast<IO*>(a.gx);
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
            const int b = b0 + row0 + r;
            if (b < a.batch) {
                const size_t at = (size_t)b * a.in_dim + i;
                const float v = ld_as_float(x + at);
                const float sg = sigmoid_f(v);
                const float dsl = sg * (1.f + v * (1.f - sg));
                // grad_x is read and written by this kernel: a plain load (the read-only path is for data the
                // kernel never writes). With bfloat16 activations the circuit share was rounded once when the
                // backward stored it and the sum is rounded again here (half an ulp each, inside the bf16 bound).
                const float acc = (r & 1) ? gxb2[r / 2].y : gxb2[r / 2].x;
                st_from_float(gx + at, fmaf(dsl, acc, ld_rw_as_float(gx + at)));
            }
        }
    }
}

}  // namespace

int base_rows_per_cta(int batch, int in_dim) {
    // 128-row tiles (16 rows per warp, three CTAs resident per SM) unless that leaves SMs without work
    // (small batches): then 64-row tiles
    const long big = (long)((batch + 127) / 128) * ((in_dim + kWarp - 1) / kWarp);
    return big >= 3 * 148 ? 128 : 64;
}

cudaError_t launch_base_backward(const BaseBwdArgs& a, int io_dtype, cudaStream_t st) {
    const int tb = base_rows_per_cta(a.batch, a.in_dim);
    dim3 grid((a.batch + tb - 1) / tb, a.ipad / kWarp);
    const int threads = kBaseWarps * kWarp;
    if (io_dtype == QK_BF16) {
        if (tb == 128) base_backward_kernel<__nv_bfloat16, 16><<<grid, threads, 0, st>>>(a);
        else base_backward_kernel<__nv_bfloat16, 8><<<grid, threads, 0, st>>>(a);
    } else {
        if (tb == 128) base_backward_kernel<float, 16><<<grid, threads, 0, st>>>(a);
        else base_backward_kernel<float, 8><<<grid, threads, 0, st>>>(a);
    }
    return cudaPeekAtLastError();
}

}  // namespace qk
