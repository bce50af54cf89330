// Fused forward: y[b,o] = sum_i (p[b,o,i] + PB[o,i]) * W[o,i] + sum_i silu(x[b,i]) * BW[o,i]
// with p the circuit readout of edge (o,i) on row b. Replaces the solver call,
// the mask fold and the epilogue of QKANLayer._forward_train / _forward_eval
// (reference: src/qkan/qkan.py:727-785; fused reference counterparts:
// src/qkan/csrc/cute_kernels.cu:96-210 and src/qkan/qkan_epilogue.py:61-165).
//
// Mapping: a lane owns one input column i, a warp owns one output o at a time,
// and both walk the CTA's batch rows. The edge's constants sit in registers,
// the x tile is staged once in shared memory with coalesced loads, and the sum
// over in_dim is a warp-shuffle transpose-reduction done once per 32 rows.
#pragma once
#include <type_traits>

#include "qk_kernels.cuh"
#include "qk_packed.cuh"

namespace qk {

// v[j] holds this lane's value for row j (j = 0..31). On return v[0] of lane L
// is the sum over all lanes of their v[L]: 31 shuffles for 32 sums.
__device__ __forceinline__ float transpose_reduce32(float (&v)[32], int lane) {
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) {
        const bool up = (lane & s) != 0;
#pragma unroll
        for (int j = 0; j < s; ++j) {
            float send = up ? v[j] : v[j + s];
            float keep = up ? v[j + s] : v[j];
            v[j] = keep + __shfl_xor_sync(0xffffffffu, send, s);
        }
    }
    return v[0];
}

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + expf(-v)); }

// Staging of one x tile (tb rows x w columns from column ic0) into shared memory: a warp takes whole rows; its lanes
// read 16 bytes each (4 float32 / 8 bfloat16 values), so a row segment is fetched with coalesced 128-bit loads. Rows
// whose segments are not 16-byte aligned (in_dim not a multiple of the vector, or an unaligned x) and the ragged right
// edge take the element-wise path. XTRIG stores (cos x, sin x), BASE also silu(x). Out of line on purpose: the
// register allocation of the kernel's main loop then does not depend on this code.
template <typename IO, bool BASE, bool XTRIG>
static __device__ __noinline__ void stage_x_tile(const IO* __restrict__ x, int batch, int in_dim, int b0, int ic0, int w,
                                                 int tb, int ich, float* __restrict__ x_s, float* __restrict__ b_s) {
    const int warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    const int nwarps = blockDim.x / kWarp;
    constexpr int VEC = 16 / (int)sizeof(IO);
    const bool vec_ok = (in_dim % VEC) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
    auto put = [&](int r, int c, float v) {
        if (XTRIG) {
            float sx, cx;
            precise_sincos(v, sx, cx);
            reinterpret_cast<float2*>(x_s)[r * ich + c] = make_float2(cx, sx);
        } else {
            x_s[r * ich + c] = v;
        }
        if (BASE) b_s[r * ich + c] = silu_f(v);
    };
    for (int r = warp; r < tb; r += nwarps) {
        const bool row_ok = b0 + r < batch;
        const IO* xr = x + (size_t)(b0 + r) * in_dim + ic0;
        for (int c = lane * VEC; c < w; c += kWarp * VEC) {
            if (vec_ok && row_ok && ic0 + c + VEC <= in_dim) {
                const uint4 q = __ldg(reinterpret_cast<const uint4*>(xr + c));
                if constexpr (sizeof(IO) == 4) {
                    put(r, c, __uint_as_float(q.x));
                    put(r, c + 1, __uint_as_float(q.y));
                    put(r, c + 2, __uint_as_float(q.z));
                    put(r, c + 3, __uint_as_float(q.w));
                } else {
                    const unsigned wd[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                    for (int k = 0; k < 4; ++k) {  // bfloat16 is the upper half of a float32
                        put(r, c + 2 * k, __uint_as_float(wd[k] << 16));
                        put(r, c + 2 * k + 1, __uint_as_float(wd[k] & 0xffff0000u));
                    }
                }
            } else {
#pragma unroll
                for (int k = 0; k < VEC; ++k) {
                    float v = 0.f;
                    if (row_ok && ic0 + c + k < in_dim) v = ld_as_float(xr + c + k);
                    put(r, c + k, v);
                }
            }
        }
    }
}

// One row pair in QK_FWD_POLY_EVERY of a lane's 32-row block (one row, in the scalar form) evaluates the sin/cos of
// its first QK_FWD_POLY_GATES data gates on the FMA pipe (poly_sincos) instead of the special-function unit, which
// bounds this kernel; 0 switches that off. Packed form (two rows per instruction), forward ms at 65536 x 256 -> 256,
// 3 repetitions: off 8.37; one gate of every pair 8.07 (kept), of every 2nd pair 8.19, of every 4th 8.34; two gates
// of every pair 9.56, of every 2nd 8.59; all three of every 3rd 8.59. Scalar form: Measured at 65536 x 256 -> 256, 3 repetitions (forward, ms): off 8.72; one gate of every 4th row 8.57,
// of every 3rd 8.66, of every 2nd 8.61, of every row 9.12; two gates of every 4th row 8.58, of every 2nd 9.14;
// all gates of every 8th row 8.66, of every 6th 8.72, of every 4th 8.86, of every 3rd 9.06. The unit is 84 % busy
// without it, yet moving more than a twelfth of the calls off it loses again: the kernel is as much bound by
// its queue to that unit, which the shuffles and shared-memory reads share, as by the unit itself.
#ifndef QK_PACKED_F32
#define QK_PACKED_F32 1
#endif
#ifndef QK_FWD_POLY_EVERY
#define QK_FWD_POLY_EVERY 1
#endif
#ifndef QK_XTRIG_PACKED
#define QK_XTRIG_PACKED 1
#endif
// 1: a lane adds up its columns of the staged chunk (all 32-column blocks) in its 32 row registers before the
// shuffle reduction over the lanes, so that reduction (about 4 instructions per edge and row) is paid once per
// chunk instead of once per 32-column block; the constants of a column block are then fetched once per 32 rows.
// 0: one shuffle reduction per 32-column block. Measured at 65536 x 256 -> 256, 3 repetitions (forward, ms): 8.06 -> 7.76
// trainable preacts, 8.43 -> 8.01 with the base term, 7.33 -> 7.22 (scalar) / 6.75 (packed) frozen preacts.
#ifndef QK_FWD_SUM_COLUMNS
#define QK_FWD_SUM_COLUMNS 1
#endif
// One row pair in QK_FWD_SCALAR_EVERY is evaluated as two scalar rows; 0 = every pair packed. Measured at the
// headline shape (forward, ms): 0: 8.05; every 4th 8.09, every 3rd 8.17, every 2nd 8.30: mixing does not pay.
#ifndef QK_FWD_SCALAR_EVERY
#define QK_FWD_SCALAR_EVERY 0
#endif
#ifndef QK_FWD_POLY_GATES
#define QK_FWD_POLY_GATES 1
#endif
#ifdef QK_FWD_MAXNREG
#define QK_FWD_REGCAP __maxnreg__(QK_FWD_MAXNREG)
#else
#define QK_FWD_REGCAP __launch_bounds__(512)
#endif

// XTRIG: the x tile holds (cos x, sin x) pairs and the data gates use the angle-addition form
// (frozen preacts, see edge_forward_xtrig).
template <int R, bool FAST, typename IO, bool BASE, bool EDGES, bool PRECISE, bool XTRIG>
__global__ void QK_FWD_REGCAP forward_kernel(FwdArgs a) {
    extern __shared__ __align__(16) float smem[];
    const int tb = a.cfg.tb, ot = a.cfg.ot, ich = a.cfg.ich;
    const int ldy = tb + 1;
    constexpr int XW = XTRIG ? 2 : 1;            // floats per staged x element
    float* x_s = smem;                           // [tb][ich] (x) or [tb][ich][2] (cos x, sin x)
    float* y_s = x_s + (size_t)tb * ich * XW;    // [ot][tb+1]
    float* b_s = y_s + (EDGES ? 0 : (size_t)ot * ldy);  // [tb][ich] silu(x), BASE only
    const int b0 = blockIdx.x * tb;
    const int o0 = blockIdx.y * ot;
    const int ot_eff = min(ot, a.out_dim - o0);
    const int warp = threadIdx.x / kWarp, lane = threadIdx.x % kWarp;
    const int nwarps = blockDim.x / kWarp;
    constexpr int KS = table_stride(R);
    const IO* __restrict__ x = static_cast<const IO*>(a.x);

    if (!EDGES)
        for (int idx = threadIdx.x; idx < ot * ldy; idx += blockDim.x) y_s[idx] = 0.f;

    for (int ic0 = 0; ic0 < a.ipad; ic0 += ich) {
        const int w = min(ich, a.ipad - ic0);  // multiple of 32
        __syncthreads();
        stage_x_tile<IO, BASE, XTRIG>(x, a.batch, a.in_dim, b0, ic0, w, tb, ich, x_s, b_s);
        __syncthreads();
        const int nsub = w / kWarp;
        for (int ol = warp; ol < ot_eff; ol += nwarps) {
            const int o = o0 + ol;
            constexpr bool kSumCols = QK_FWD_SUM_COLUMNS != 0 && !EDGES;
            for (int rg_outer = 0; rg_outer < (kSumCols ? tb : 1); rg_outer += 32) {
            float v[32];
            if constexpr (kSumCols) {
#pragma unroll
                for (int r = 0; r < 32; ++r) v[r] = 0.f;
            }
            for (int sub = 0; sub < nsub; ++sub) {
                const int col = sub * kWarp + lane;
                const int i = ic0 + col;
                EdgeFwd<R> e;
                e.load(a.table + ((size_t)o * a.ipad + i) * KS);
                const float bw = e.bw;
                // (the frozen-preact form: packed 6.75 against 7.22 ms scalar once the columns are summed before the
                // shuffle reduction; with one reduction per column block the two were equal, 7.31 / 7.32 ms)
                constexpr bool kPacked = QK_PACKED_F32 != 0 && !PRECISE && (!XTRIG || QK_XTRIG_PACKED != 0) && R >= 1 && R <= 12;
                constexpr int kPolyGates = R < QK_FWD_POLY_GATES ? R : QK_FWD_POLY_GATES;
                constexpr int kEvery = QK_FWD_POLY_EVERY > 0 ? QK_FWD_POLY_EVERY : 1;
                EdgePk<R> e2;
                if constexpr (kPacked) e2.from(e);
                for (int rg = kSumCols ? rg_outer : 0; rg < (kSumCols ? rg_outer + 32 : tb); rg += 32) {
                    if constexpr (kPacked) {
                        // two rows per instruction (qk_packed.cuh); pair q = r / 2 takes its first kPolyGates data
                        // gates from the polynomial when q % kEvery == kEvery - 1
#pragma unroll
                        for (int r = 0; r < 32; r += 2) {
                            f2 p2;
                            if constexpr (XTRIG) {
                                const float2 t0 = reinterpret_cast<const float2*>(x_s)[(rg + r) * ich + col];
                                const float2 t1 = reinterpret_cast<const float2*>(x_s)[(rg + r + 1) * ich + col];
                                constexpr int kScalarEveryX = QK_FWD_SCALAR_EVERY > 0 ? QK_FWD_SCALAR_EVERY : 1;
                                if (QK_FWD_SCALAR_EVERY > 0 && ((r / 2) % kScalarEveryX) == kScalarEveryX - 1) {
                                    p2.x = edge_forward_xtrig<R, FAST>(e, t0.x, t0.y);
                                    p2.y = edge_forward_xtrig<R, FAST>(e, t1.x, t1.y);
                                } else {
                                    p2 = edge_forward_xtrig2<R, FAST>(e2, make_float2(t0.x, t1.x), make_float2(t0.y, t1.y));
                                }
                            } else {
                                const f2 x2 = make_float2(x_s[(rg + r) * ich + col], x_s[(rg + r + 1) * ich + col]);
                                constexpr int kScalarEvery = QK_FWD_SCALAR_EVERY > 0 ? QK_FWD_SCALAR_EVERY : 1;
                                if (QK_FWD_SCALAR_EVERY > 0 && ((r / 2) % kScalarEvery) == kScalarEvery - 1) {
                                    float sx, sy, sz, si, sr;
                                    p2.x = edge_forward<R, FAST, false, false>(e, x2.x, nullptr, nullptr, sx, sy, sz, si, sr);
                                    p2.y = edge_forward<R, FAST, false, false>(e, x2.y, nullptr, nullptr, sx, sy, sz, si, sr);
                                } else {
                                f2 vx, vy, vz, ir, rr;
                                if (QK_FWD_POLY_EVERY > 0 && ((r / 2) % kEvery) == kEvery - 1)
                                    p2 = edge_forward2<R, FAST, false, kPolyGates>(e2, x2, nullptr, nullptr, nullptr, vx, vy, vz, ir, rr);
                                else
                                    p2 = edge_forward2<R, FAST, false, 0>(e2, x2, nullptr, nullptr, nullptr, vx, vy, vz, ir, rr);
                                }
                            }
                            if (EDGES) {
                                v[r] = p2.x;
                                v[r + 1] = p2.y;
                            } else {
                                f2 val = kSumCols ? fma2(p2, e2.w, make_float2(v[r], v[r + 1])) : mul2(p2, e2.w);
                                if (BASE)
                                    val = fma2(make_float2(b_s[(rg + r) * ich + col], b_s[(rg + r + 1) * ich + col]), pk(bw), val);
                                v[r] = val.x;
                                v[r + 1] = val.y;
                            }
                        }
                    } else {
#pragma unroll
                    for (int r = 0; r < 32; ++r) {
                        float p;
                        if constexpr (XTRIG) {
                            const float2 t = reinterpret_cast<const float2*>(x_s)[(rg + r) * ich + col];
                            p = edge_forward_xtrig<R, FAST>(e, t.x, t.y);
                        } else {
                            float xv = x_s[(rg + r) * ich + col];
                            float vx, vy, vz, ir, rr;
                            constexpr int kPolyGates = R < QK_FWD_POLY_GATES ? R : QK_FWD_POLY_GATES;
                            if (QK_FWD_POLY_EVERY > 0 && (r % (QK_FWD_POLY_EVERY > 0 ? QK_FWD_POLY_EVERY : 1)) == QK_FWD_POLY_EVERY - 1)
                                p = edge_forward<R, FAST, false, PRECISE, kPolyGates>(e, xv, nullptr, nullptr, vx, vy, vz, ir, rr);
                            else
                                p = edge_forward<R, FAST, false, PRECISE>(e, xv, nullptr, nullptr, vx, vy, vz, ir, rr);
                        }
                        if (EDGES) {
                            v[r] = p;
                        } else {
                            float val = kSumCols ? fmaf(p, e.w, v[r]) : p * e.w;
                            if (BASE) val = fmaf(b_s[(rg + r) * ich + col], bw, val);
                            v[r] = val;
                        }
                    }
                    }
                    if (EDGES) {
                        IO* out = static_cast<IO*>(a.postacts);
                        if (i < a.in_dim) {
#pragma unroll
                            for (int r = 0; r < 32; ++r)
                                if (b0 + rg + r < a.batch)
                                    st_from_float(out + ((size_t)(b0 + rg + r) * a.out_dim + o) * a.in_dim + i,
                                                  v[r]);
                        }
                    } else if (!kSumCols) {
                        float s = transpose_reduce32(v, lane);
                        y_s[ol * ldy + rg + lane] += s;
                    }
                }
            }
            if constexpr (kSumCols) {
                float s = transpose_reduce32(v, lane);
                y_s[ol * ldy + rg_outer + lane] += s;
            }
            }
        }
    }
    if (EDGES) return;
    __syncthreads();
    IO* __restrict__ y = static_cast<IO*>(a.y);
    for (int idx = threadIdx.x; idx < tb * ot_eff; idx += blockDim.x) {
        int r = idx / ot_eff, ol = idx - r * ot_eff;
        if (b0 + r < a.batch)
            st_from_float(y + (size_t)(b0 + r) * a.out_dim + o0 + ol,
                          y_s[ol * ldy + r] + a.bias[o0 + ol]);
    }
}

template <int R, bool FAST, typename IO, bool BASE, bool EDGES>
static cudaError_t launch_fwd_t(const FwdArgs& a, cudaStream_t st) {
    int variant = 0;  // 0: special-function unit, 1: full-precision math, 2: frozen-preact form
    auto kern = forward_kernel<R, FAST, IO, BASE, EDGES, false, false>;
    if constexpr (std::is_same<IO, float>::value) {  // the full-precision variant exists for float32 I/O
        if (a.precise) {
            kern = forward_kernel<R, FAST, IO, BASE, EDGES, true, false>;
            variant = 1;
        }
    }
    if constexpr (R >= 1 && R <= 8) {  // frozen-preact form (no identity padding possible beyond 8)
        if (a.xtrig) {
            kern = forward_kernel<R, FAST, IO, BASE, EDGES, false, true>;
            variant = 2;
        }
    }
    // opted in to the tile chooser's shared-memory cap once per device (see the backward launcher)
    static unsigned long long opted_in[3] = {0, 0, 0};
    cudaError_t err = opt_in_smem(kern, &opted_in[variant]);
    if (err != cudaSuccess) return err;
    dim3 grid(a.cfg.grid_b, a.cfg.grid_o);
    kern<<<grid, a.cfg.threads, a.cfg.smem, st>>>(a);
    return cudaPeekAtLastError();
}

template <int R, bool FAST, typename IO>
static cudaError_t launch_fwd_r(const FwdArgs& a, bool has_base, cudaStream_t st) {
    if (a.postacts) return launch_fwd_t<R, FAST, IO, false, true>(a, st);
    if (has_base) return launch_fwd_t<R, FAST, IO, true, false>(a, st);
    return launch_fwd_t<R, FAST, IO, false, false>(a, st);
}

template <int R>
cudaError_t launch_fwd_d(const FwdArgs& a, bool fast, int io_dtype, bool has_base,
                                cudaStream_t st) {
    if (io_dtype == QK_BF16) {
        return fast ? launch_fwd_r<R, true, __nv_bfloat16>(a, has_base, st)
                    : launch_fwd_r<R, false, __nv_bfloat16>(a, has_base, st);
    }
    return fast ? launch_fwd_r<R, true, float>(a, has_base, st)
                : launch_fwd_r<R, false, float>(a, has_base, st);
}

}  // namespace qk
