// Per-edge activation scale: the standard deviation over the batch of every edge's output
//   v[b,o,i] = (postacts[b,o,i] + postact_bias[o,i]) * postact_weights[o,i] * mask[o,i]
//            + silu(x[b,i]) * base_weight[o,i] * mask[o,i]
// without materialising the (B,O,I) tensor. The reference gets the same numbers for its activation-scale
// regulariser and its pruning scores by calling forward_no_sum and torch.std on the result
// (src/qkan/qkan.py:835-891, 1280-1302); that tensor is 2.4 GB per layer at 8192 x 768 x 768 in float32.
//
// Mapping (the backward's): a lane owns one input column i, a CTA owns 32 columns and `groups * rpg` batch rows
// (one warp per group) and walks every output o. A thread keeps the edge constants in registers and adds up
// d and d^2 over its rows, with d = v - K and K = the edge's value on batch row 0: shifting by a sample of the
// data keeps the one-pass variance sum((d)^2) - (sum d)^2 / n free of the cancellation a large mean would cause,
// and K is the same in every CTA, so the per-tile sums simply add. Block reduction through shared memory, one
// partial pair per (tile, o), then stats_finish_kernel adds the tiles in a fixed order and takes the root.
#pragma once
#include "qk_kernels.cuh"

namespace qk {

struct StatsArgs {
    int batch, in_dim, out_dim, ipad;
    int groups, rpg, tb, grid_b;
    int fast, base;
    const void* x;
    const float* table;
    float* partials;  // [grid_b][out_dim][2][ipad]
};

__device__ __forceinline__ float stats_silu(float v) { return v / (1.f + __expf(-v)); }

template <int R>
__device__ __forceinline__ float edge_value(const EdgeFwd<R>& e, float x, float sx, bool fast, bool base) {
    float vx, vy, vz, ir, rr;
    float p = fast ? edge_forward<R, true, false, false>(e, x, nullptr, nullptr, vx, vy, vz, ir, rr)
                   : edge_forward<R, false, false, false>(e, x, nullptr, nullptr, vx, vy, vz, ir, rr);
    float v = p * e.w;
    if (base) v = fmaf(sx, e.bw, v);
    return v;
}

template <int R, typename IO>
__global__ void __launch_bounds__(256) stats_kernel(StatsArgs a) {
    extern __shared__ __align__(16) float smem[];
    const int groups = a.groups, rpg = a.rpg, tb = a.tb;
    float* x_s = smem;                          // [tb][32] x, thread-private columns
    float* s_s = x_s + (size_t)tb * kWarp;      // [tb][32] silu(x)
    float* red_s = s_s + (size_t)tb * kWarp;    // [2 buffers][groups][2][32]
    const int lane = threadIdx.x % kWarp, grp = threadIdx.x / kWarp;
    const int bt = blockIdx.x, b0 = bt * tb;
    const int i0 = blockIdx.y * kWarp, i = i0 + lane;
    constexpr int KS = table_stride(R);
    const IO* __restrict__ x = static_cast<const IO*>(a.x);
    const bool fast = a.fast != 0, base = a.base != 0;
    const int row0 = grp * rpg;
    const bool col_ok = i < a.in_dim;
    // rows past the batch are marked and skipped (their value must not enter the sums)
    int nrows = a.batch - (b0 + row0);
    nrows = nrows < 0 ? 0 : (nrows > rpg ? rpg : nrows);
    for (int j = 0; j < nrows; ++j) {
        const float v = col_ok ? ld_as_float(x + (size_t)(b0 + row0 + j) * a.in_dim + i) : 0.f;
        x_s[(row0 + j) * kWarp + lane] = v;
        s_s[(row0 + j) * kWarp + lane] = base ? stats_silu(v) : 0.f;
    }
    const float xk = col_ok ? ld_as_float(x + i) : 0.f;  // batch row 0: the shift sample
    const float sk = base ? stats_silu(xk) : 0.f;

    for (int o = 0; o < a.out_dim; ++o) {
        EdgeFwd<R> e;
        e.load(a.table + ((size_t)o * a.ipad + i) * KS);
        const float K = edge_value<R>(e, xk, sk, fast, base);
        float s1[2] = {0.f, 0.f}, s2[2] = {0.f, 0.f};
        const float* xp = x_s + row0 * kWarp + lane;
        const float* sp = s_s + row0 * kWarp + lane;
        int j = 0;
        for (; j + 2 <= nrows; j += 2) {
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const float d = edge_value<R>(e, xp[(j + u) * kWarp], sp[(j + u) * kWarp], fast, base) - K;
                s1[u] += d;
                s2[u] = fmaf(d, d, s2[u]);
            }
        }
        if (j < nrows) {
            const float d = edge_value<R>(e, xp[j * kWarp], sp[j * kWarp], fast, base) - K;
            s1[0] += d;
            s2[0] = fmaf(d, d, s2[0]);
        }
        float* red = red_s + (size_t)(o & 1) * groups * 2 * kWarp;
        red[(grp * 2 + 0) * kWarp + lane] = s1[0] + s1[1];
        red[(grp * 2 + 1) * kWarp + lane] = s2[0] + s2[1];
        __syncthreads();
        if (grp < 2) {  // warp 0 adds the sums, warp 1 the sums of squares, over the groups in order
            float s = 0.f;
            for (int g = 0; g < groups; ++g) s += red[(g * 2 + grp) * kWarp + lane];
            a.partials[(((size_t)bt * a.out_dim + o) * 2 + grp) * a.ipad + i] = s;
        }
    }
}

template <int R>
cudaError_t launch_stats_d(const StatsArgs& a, int io_dtype, cudaStream_t st) {
    const size_t smem = ((size_t)a.tb * kWarp * 2 + (size_t)2 * a.groups * 2 * kWarp) * sizeof(float);
    dim3 grid(a.grid_b, a.ipad / kWarp);
    static unsigned long long opted_in[2] = {0, 0};
    if (io_dtype == QK_BF16) {
        auto kern = stats_kernel<R, __nv_bfloat16>;
        cudaError_t err = opt_in_smem(kern, &opted_in[1]);
        if (err != cudaSuccess) return err;
        kern<<<grid, a.groups * kWarp, smem, st>>>(a);
    } else {
        auto kern = stats_kernel<R, float>;
        cudaError_t err = opt_in_smem(kern, &opted_in[0]);
        if (err != cudaSuccess) return err;
        kern<<<grid, a.groups * kWarp, smem, st>>>(a);
    }
    return cudaPeekAtLastError();
}

}  // namespace qk
