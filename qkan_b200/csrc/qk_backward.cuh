// Fused backward: grad_x and the batch-summed gradients of every per-edge
// parameter, from recomputed circuit states (nothing is checkpointed).
// Replaces what autograd derives for the reference's solver + epilogue
// (src/qkan/solver/exact.py:90-134, src/qkan/qkan.py:776-785; fused reference
// counterparts: src/qkan/csrc/cute_kernels.cu:216-508 and
// src/qkan/qkan_epilogue.py:187-309).
//
// Mapping: a lane owns one input column i; a CTA owns 32 columns and
// `groups * rpg` batch rows (one warp per group of rpg rows) and walks every
// output o. For the current edge (o,i) a thread keeps the edge constants and
// the 3R+3 gradient accumulators in registers while it runs through its rows,
// so the sum over the batch needs no cross-lane traffic; grad_x[b,i]
// accumulates over o in a thread-private shared-memory column. After each o
// the groups' accumulators are summed through shared memory (block-level
// reduction) and written as this batch tile's partial; finish_grads then sums
// the tiles in a fixed order (cross-CTA reduction, bitwise reproducible).
// The base term silu(x) @ base_weight has its own kernel (qk_base.cu): it is two small GEMMs, and carrying
// silu(x) and silu'(x) through this kernel's shared-memory tile cost it a resident CTA.
#pragma once
#include <type_traits>

#include "qk_kernels.cuh"
#include "qk_packed.cuh"

namespace qk {

// Returns gx0 + d/dx of this edge (gx0 is the grad_x accumulated over the outputs walked so far).
// `acc(k)` is a reference to accumulator k (a float array, or one half of a packed pair).
template <int R, bool FAST, bool EDGES, bool PRECISE, class Acc>
__device__ __forceinline__ float edge_backward_to(const EdgeFwd<R>& e, float x, float g, float gx0, Acc acc) {
    if constexpr (R == 0) {
        // "real" ansatz: p = f(alpha), alpha = A x + C. acc(0) = sum dL/dalpha, acc(1) = sum dL/dalpha * x
        float s, c, r = 1.f;
        const float p = real_forward<FAST, PRECISE>(e, x, s, c, r);
        const float gp = EDGES ? g : g * e.w;
        if (!EDGES) acc(a_w(0)) = fmaf(g, p, acc(a_w(0)));
        float dp = -s;
        if (FAST) {
            // d/dalpha [cos * (1+|sin|)^(-1/2)] = -sin r - (1/2) cos^2 r^3 sign(sin)
            const float sgn = s > 0.f ? 1.f : (s < 0.f ? -1.f : 0.f);
            dp = -fmaf((0.5f * c) * c, (r * r) * (r * sgn), s * r);
        }
        const float ga = gp * dp;
        acc(0) += ga;
        acc(1) = fmaf(ga, x, acc(1));
        return fmaf(ga, e.a, gx0);
    } else {
    float cs[R], sn[R], vx, vy, vz, inv_rho, r;
    const float p = edge_forward<R, FAST, true, PRECISE>(e, x, cs, sn, vx, vy, vz, inv_rho, r);
    const float gp = EDGES ? g : g * e.w;
    if (!EDGES) acc(a_w(R)) = fmaf(g, p, acc(a_w(R)));
    // w = v x a, a = cotangent of the final Bloch vector (its z component of w is 0)
    float wx, wy, wz;
    if (FAST) {
        // a = (q vx, q vy, az), az = gp r, q = -gp r^3 vz / (2 rho); then v x a = (vy k, -vx k, 0), k = az - vz q
        // with p = vz r:  k = gp r (1 + p^2 / (2 rho))
        const float k = (gp * r) * fmaf((0.5f * p) * p, inv_rho, 1.0f);
        wx = vy * k;
        wy = -(vx * k);
    } else {
        wx = vy * gp;
        wy = -(vx * gp);
    }
    acc(a_ry(R)) += wy;  // final Ry(theta[R,1])
    wz = wx * e.sf;
    wx = wx * e.cf;
    float gx = gx0;
#pragma unroll
    for (int l = R - 1; l >= 0; --l) {
        // merged Rz(pw_l x + c_l): its angle gradient is wz
        acc(a_c(R, l)) += wz;
        acc(a_pwx(R, l)) = fmaf(wz, x, acc(a_pwx(R, l)));
        gx = fmaf(wz, e.pw[l], gx);
        float nx = fmaf(wy, sn[l], wx * cs[l]);
        float ny = fmaf(-wx, sn[l], wy * cs[l]);
        wx = nx;
        wy = ny;
        acc(a_ry(l)) += wy;  // Ry(theta[l,1])
        if (l > 0) {
            float mx = fmaf(-wz, e.sa[l], wx * e.ca[l]);
            float mz = fmaf(wx, e.sa[l], wz * e.ca[l]);
            wx = mx;
            wz = mz;
        } else {
            wz = fmaf(wx, e.sa[0], wz * e.ca[0]);
        }
    }
    acc(a_t00(R)) += wz;  // Rz(theta[0,0])
    return gx;
    }
}

template <int R, bool FAST, bool EDGES, int NACC, bool PRECISE>
__device__ __forceinline__ float edge_backward(const EdgeFwd<R>& e, float x, float g, float gx0,
                                               float (&acc)[NACC]) {
    return edge_backward_to<R, FAST, EDGES, PRECISE>(e, x, g, gx0, [&](int k) -> float& { return acc[k]; });
}

constexpr int kGyChunk = 8;  // outputs whose grad_y columns are staged together

// Two batch rows per instruction on the packed float32 operations (qk_packed.cuh): 1 = on (the special-function
// variants with at least one repetition), 0 = the scalar form everywhere.
#ifndef QK_PACKED_F32
#define QK_PACKED_F32 1
#endif
// With four rows in flight: 1 = rows 0,1 as a packed pair and rows 2,3 as scalar rows, 0 = two packed pairs.
// The counters show the packed operations on one half of the FMA pipe only, so scalar rows were tried for the
// other half: measured slower (backward call 14.82 ms against 14.30 at the headline shape; 14.87 / 15.29 with
// register caps 128 / 96), so it stays off.
#ifndef QK_BWD_HYBRID
#define QK_BWD_HYBRID 0
#endif

// grad_y[b0 .. b0+tb, oc .. oc+nch) into shared memory, transposed ([output][row]); rows past the batch read as 0.
// QK_BWD_STAGE_NOINLINE = 1 keeps it out of line (the main loop's register allocation then does not depend on it).
#ifndef QK_BWD_STAGE_NOINLINE
#define QK_BWD_STAGE_NOINLINE 1
#endif
#if QK_BWD_STAGE_NOINLINE
#define QK_STAGE_LINKAGE static __device__ __noinline__
#else
#define QK_STAGE_LINKAGE static __device__ __forceinline__
#endif
template <typename IO>
QK_STAGE_LINKAGE void stage_grad_y(const IO* __restrict__ gsrc, int batch, int out_dim, int b0, int oc, int nch, int tb,
                                   float* __restrict__ gy_s) {
    if (std::is_same<IO, float>::value && nch == kGyChunk && (out_dim & 3) == 0 &&
        (reinterpret_cast<uintptr_t>(gsrc) & 15) == 0) {
        // full chunk of float32 rows from a 16-byte aligned grad_y: two 128-bit loads per row
        // (oc and out_dim are multiples of 4, so every row segment is aligned too)
        for (int idx = threadIdx.x; idx < tb * 2; idx += blockDim.x) {
            const int r = idx >> 1, h = idx & 1;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (b0 + r < batch)
                v = __ldg(reinterpret_cast<const float4*>(
                    reinterpret_cast<const float*>(gsrc) + (size_t)(b0 + r) * out_dim + oc + 4 * h));
            float* dst = gy_s + (4 * h) * tb + r;
            dst[0] = v.x;
            dst[tb] = v.y;
            dst[2 * tb] = v.z;
            dst[3 * tb] = v.w;
        }
    } else {
        for (int idx = threadIdx.x; idx < tb * kGyChunk; idx += blockDim.x) {
            const int r = idx / kGyChunk, c = idx % kGyChunk;
            float v = 0.f;
            if (b0 + r < batch && c < nch) v = ld_as_float(gsrc + (size_t)(b0 + r) * out_dim + oc + c);
            gy_s[c * tb + r] = v;
        }
    }
}

// Register cap of the short circuits (up to 3 repetitions): two CTAs of 256 threads stay resident per SM and the
// compiler spends the rest on scheduling; 4 to 8 repetitions are capped at 128 (still two CTAs: uncapped, the
// 8-repetition kernel took 152 registers, lost its second CTA and a fifth of its speed); the padded 12- and
// 16-repetition instantiations need more than that. The cap,
// the block-size bound beside it and the inlining of the column sums are a measured optimum of the instruction
// schedule, not limits the code needs. Backward call at 65536 x 256 -> 256, 3 repetitions (ms), scalar form: cap 96
// with the block-size bound and inlined sums 14.95; without the bound 15.25; sums out of line 15.42; cap 88 15.46,
// 104 15.32, 112 15.00, 128 15.53. Packed form (two rows per instruction): cap 80 14.92, 96 14.50, 112 14.29,
// 128 14.40.
#ifndef QK_BWD_SHORT_MAXNREG
#define QK_BWD_SHORT_MAXNREG 112
#endif
#ifdef QK_BWD_COLSUM_INLINE
#define QK_COLSUM_LINKAGE static __device__ __forceinline__
#else
#define QK_COLSUM_LINKAGE static __device__ __noinline__
#endif

// Column sums of one batch tile's staged grad_y rows (the postact-bias terms need sum_b grad_y[b,o]): taken by
// the CTAs of column block 0 only, one warp per output, lane-strided partial sums and a shuffle tree (fixed
// order); finish_grads adds the tiles in order. Out of line, like the staging of grad_y: with the packed main loop
// that measured 1 % faster than inlining both (14.18 against 14.31 ms at the headline shape; in the scalar build it
// was the other way round by 3 %, through nothing but a different instruction schedule of the hot loop).
QK_COLSUM_LINKAGE void tile_column_sums(float* __restrict__ dst, const float* gy_s, int nch, int groups, int tb) {
    const int lane = threadIdx.x % kWarp, grp = threadIdx.x / kWarp;
    for (int c = grp; c < nch; c += groups) {
        float s = 0.f;
        for (int r = lane; r < tb; r += kWarp) s += gy_s[c * tb + r];
#pragma unroll
        for (int d = 16; d >= 1; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
        if (lane == 0) dst[c] = s;
    }
}

template <int R, bool FAST, typename IO, bool EDGES, int RU, bool PRECISE, bool OSLICE>
__global__ void __launch_bounds__(256) __maxnreg__(R <= 3 ? QK_BWD_SHORT_MAXNREG : (R <= 8 ? 128 : 255)) backward_kernel(BwdArgs a) {
    constexpr int NACC = acc_rows(R);
    // floats per tile row: 32 (x, grad_x) pairs; a pair is one 64-bit access
    constexpr int ROW = 64;
    extern __shared__ __align__(16) float smem[];
    const int groups = a.cfg.groups, rpg = a.cfg.rpg, tb = a.cfg.tb;
    float* xg_s = smem;                                  // [tb][ROW]
    float* gy_s = xg_s + (size_t)tb * ROW;               // [kGyChunk][tb]   (fused mode)
    float* red_s = gy_s + (EDGES ? 0 : (size_t)kGyChunk * tb);  // [2][groups][NACC][32]
    const int lane = threadIdx.x % kWarp, grp = threadIdx.x / kWarp;
    const int bt = blockIdx.x;
    const int b0 = bt * tb;
    const int i0 = blockIdx.y * kWarp;
    const int i = i0 + lane;
    constexpr int KS = table_stride(R);
    const IO* __restrict__ x = static_cast<const IO*>(a.x);
    const IO* __restrict__ gsrc = static_cast<const IO*>(EDGES ? a.gpostacts : a.gy);
    const int row0 = grp * rpg;
    float* const my = xg_s + (size_t)row0 * ROW + 2 * lane;  // this thread's column of its group's rows

    for (int j = 0; j < rpg; ++j) {
        const int row = row0 + j;
        float v = 0.f;
        if (b0 + row < a.batch && i < a.in_dim) v = ld_as_float(x + (size_t)(b0 + row) * a.in_dim + i);
        *reinterpret_cast<float2*>(my + j * ROW) = make_float2(v, 0.f);
    }
    // a thread only ever touches its own column of its own group's rows: no barrier needed for xg_s

    // OSLICE: blockIdx.z selects a slice of the outputs (small batches: more CTAs in flight; see
    // BwdCfg::osplit). A separate instantiation, so that the unsliced kernel keeps its bound in the
    // constant bank instead of a register.
    const int o_begin = OSLICE ? blockIdx.z * a.cfg.ochunk : 0;
    const int o_end = OSLICE ? min(a.out_dim, o_begin + a.cfg.ochunk) : a.out_dim;
    for (int oc = o_begin; oc < o_end; oc += kGyChunk) {
        const int nch = min(kGyChunk, o_end - oc);
        if (!EDGES) {
            stage_grad_y<IO>(gsrc, a.batch, a.out_dim, b0, oc, nch, tb, gy_s);
            __syncthreads();
            if (a.colpart && blockIdx.y == 0)
                tile_column_sums(a.colpart + (size_t)bt * a.out_dim + oc, gy_s, nch, groups, tb);
        }
        for (int ol = 0; ol < nch; ++ol) {
            const int o = oc + ol;
            EdgeFwd<R> e;
            e.load(a.table + ((size_t)o * a.ipad + i) * KS);
            float acc[NACC];
            // (from 7 repetitions on, the constants as register pairs no longer fit beside two resident CTAs)
            constexpr bool kPacked = QK_PACKED_F32 != 0 && !PRECISE && R >= 1 && R <= 6 && (RU % 2) == 0;
            const float* gyp = gy_s + ol * tb + row0;
            float* p = my;
            if constexpr (kPacked) {
                EdgePk<R> e2;
                e2.from(e);
                f2 acc2[NACC];
#pragma unroll
                for (int k = 0; k < NACC; ++k) acc2[k] = pk(0.f);
#pragma unroll 1
                for (int j = 0; j < rpg; j += RU, p += RU * ROW) {
                    float xv[RU], gxo[RU], g[RU];
#pragma unroll
                    for (int u = 0; u < RU; ++u) {
                        const float2 xg = *reinterpret_cast<const float2*>(p + u * ROW);
                        xv[u] = xg.x;
                        gxo[u] = xg.y;
                        if (EDGES) {
                            const int b = b0 + row0 + j + u;
                            g[u] = 0.f;
                            if (b < a.batch && i < a.in_dim)
                                g[u] = ld_as_float(gsrc + ((size_t)b * a.out_dim + o) * a.in_dim + i);
                        }
                    }
                    if (!EDGES && RU == 2) {
                        const float2 gv = *reinterpret_cast<const float2*>(gyp + j);
                        g[0] = gv.x;
                        g[RU - 1] = gv.y;
                    }
                    if (!EDGES && RU == 4) {
                        const float4 gv = *reinterpret_cast<const float4*>(gyp + j);
                        g[0] = gv.x;
                        g[1 % RU] = gv.y;
                        g[2 % RU] = gv.z;
                        g[3 % RU] = gv.w;
                    }
#pragma unroll
                    for (int u = 0; u < RU; u += 2) {
                        if (QK_BWD_HYBRID != 0 && RU == 4 && u == 2) {
                            p[u * ROW + 1] = edge_backward_to<R, FAST, EDGES, false>(
                                e, xv[u], g[u], gxo[u], [&](int k) -> float& { return acc2[k].x; });
                            p[(u + 1) * ROW + 1] = edge_backward_to<R, FAST, EDGES, false>(
                                e, xv[u + 1], g[u + 1], gxo[u + 1], [&](int k) -> float& { return acc2[k].y; });
                            continue;
                        }
                        const f2 gx2 = edge_backward2<R, FAST, EDGES, NACC>(
                            e2, make_float2(xv[u], xv[u + 1]), make_float2(g[u], g[u + 1]),
                            make_float2(gxo[u], gxo[u + 1]), acc2);
                        p[u * ROW + 1] = gx2.x;
                        p[(u + 1) * ROW + 1] = gx2.y;
                    }
                }
#pragma unroll
                for (int k = 0; k < NACC; ++k) acc[k] = acc2[k].x + acc2[k].y;
            } else {
#pragma unroll
                for (int k = 0; k < NACC; ++k) acc[k] = 0.f;
#pragma unroll 1
                for (int j = 0; j < rpg; j += RU, p += RU * ROW) {
                    float xv[RU], gxo[RU], g[RU];
#pragma unroll
                    for (int u = 0; u < RU; ++u) {
                        const float2 xg = *reinterpret_cast<const float2*>(p + u * ROW);
                        xv[u] = xg.x;
                        gxo[u] = xg.y;
                        if (EDGES) {
                            const int b = b0 + row0 + j + u;
                            g[u] = 0.f;
                            if (b < a.batch && i < a.in_dim)
                                g[u] = ld_as_float(gsrc + ((size_t)b * a.out_dim + o) * a.in_dim + i);
                        } else if (RU != 2 && RU != 4) {
                            g[u] = gyp[j + u];
                        }
                    }
                    // tb, row0 and j are multiples of RU, so the staged grad_y values of these rows
                    // are one aligned vector (same address in every lane: a broadcast load)
                    if (!EDGES && RU == 2) {
                        const float2 gv = *reinterpret_cast<const float2*>(gyp + j);
                        g[0] = gv.x;
                        g[RU - 1] = gv.y;
                    }
                    if (!EDGES && RU == 4) {
                        const float4 gv = *reinterpret_cast<const float4*>(gyp + j);
                        g[0] = gv.x;
                        g[1 % RU] = gv.y;
                        g[2 % RU] = gv.z;
                        g[3 % RU] = gv.w;
                    }
#pragma unroll
                    for (int u = 0; u < RU; ++u) {
                        p[u * ROW + 1] = edge_backward<R, FAST, EDGES, NACC, PRECISE>(e, xv[u], g[u], gxo[u], acc);
                    }
                }
            }
            // block-level reduction over the row groups, then this tile's partial
            float* red = red_s + (size_t)(o & 1) * groups * NACC * 32;
#pragma unroll
            for (int k = 0; k < NACC; ++k) red[(grp * NACC + k) * 32 + lane] = acc[k];
            __syncthreads();
            // warp `grp` sums accumulators grp, grp + groups, ... over the groups (fixed order) for its 32 columns
            float* const part = a.partials + ((size_t)bt * a.out_dim + o) * NACC * a.ipad + i0 + lane;
            for (int k = grp; k < NACC; k += groups) {
                const float* r = red + k * 32 + lane;
                float s = 0.f;
                for (int gi = 0; gi < groups; ++gi) s += r[gi * NACC * 32];
                part[(size_t)k * a.ipad] = s;
            }
        }
    }

    if (OSLICE && a.gx) {
        // this output slice's share of grad_x; sum_gx_kernel adds the slices in order
        float* __restrict__ gxp = a.gx_part + (size_t)blockIdx.z * a.batch * a.in_dim;
        for (int j = 0; j < rpg; ++j) {
            const int row = row0 + j;
            if (b0 + row < a.batch && i < a.in_dim) gxp[(size_t)(b0 + row) * a.in_dim + i] = my[j * ROW + 1];
        }
    } else if (!OSLICE && a.gx) {
        IO* __restrict__ gx = static_cast<IO*>(a.gx);
        for (int j = 0; j < rpg; ++j) {
            const int row = row0 + j;
            if (b0 + row < a.batch && i < a.in_dim)
                st_from_float(gx + (size_t)(b0 + row) * a.in_dim + i, my[j * ROW + 1]);
        }
    }
}

template <int R, bool FAST, typename IO, bool EDGES>
static cudaError_t launch_bwd_t(const BwdArgs& a, cudaStream_t st) {
    // variant 0 / 1: four / two rows in flight; 2: full-precision math; 3 / 4: sliced outputs (plain / full precision)
    int variant = a.cfg.ru == 4 ? 0 : 1;
    auto kern = a.cfg.ru == 4 ? backward_kernel<R, FAST, IO, EDGES, 4, false, false>
                              : backward_kernel<R, FAST, IO, EDGES, 2, false, false>;
    if constexpr (std::is_same<IO, float>::value) {  // the full-precision variant exists for float32 I/O
        if (a.precise) {
            kern = backward_kernel<R, FAST, IO, EDGES, 2, true, false>;
            variant = 2;
        }
    }
    if (a.cfg.osplit > 1) {
        // sliced outputs: one row-interleave per repetition count (rows per group are multiples of 4)
        constexpr int RU_S = (R > 8) ? 2 : 4;
        kern = backward_kernel<R, FAST, IO, EDGES, RU_S, false, true>;
        variant = 3;
        if constexpr (std::is_same<IO, float>::value) {
            if (a.precise) {
                kern = backward_kernel<R, FAST, IO, EDGES, 2, true, true>;
                variant = 4;
            }
        }
    }
    // Every instantiation is opted in to the tile choosers' shared-memory cap once per device, not per launch:
    // host threads launching different shapes of one instantiation would otherwise race on the attribute.
    static unsigned long long opted_in[5] = {0, 0, 0, 0, 0};
    cudaError_t err = opt_in_smem(kern, &opted_in[variant]);
    if (err != cudaSuccess) return err;
    dim3 grid(a.cfg.grid_b, a.cfg.grid_i, a.cfg.osplit);
    kern<<<grid, a.cfg.groups * kWarp, a.cfg.smem, st>>>(a);
    return cudaPeekAtLastError();
}

template <int R, bool FAST, typename IO>
static cudaError_t launch_bwd_r(const BwdArgs& a, cudaStream_t st) {
    if (a.gpostacts) return launch_bwd_t<R, FAST, IO, true>(a, st);
    return launch_bwd_t<R, FAST, IO, false>(a, st);
}

template <int R>
cudaError_t launch_bwd_d(const BwdArgs& a, bool fast, int io_dtype, cudaStream_t st) {
    if (io_dtype == QK_BF16) {
        return fast ? launch_bwd_r<R, true, __nv_bfloat16>(a, st) : launch_bwd_r<R, false, __nv_bfloat16>(a, st);
    }
    return fast ? launch_bwd_r<R, true, float>(a, st) : launch_bwd_r<R, false, float>(a, st);
}

}  // namespace qk
