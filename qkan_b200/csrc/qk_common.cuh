// Shared definitions of the sm_100a QKANLayer kernels: the per-edge constant
// table, the Bloch-vector circuit evaluation and its reverse sweep.
//
// Mathematics (pz_encoding; reference: src/qkan/solver/exact.py:90-134 with the
// gates of src/qkan/torch_qc.py:76-121 and the readout of :261-277).
// The reference evolves two complex amplitudes through H, then per repetition
// Rz(theta[l,0]) Ry(theta[l,1]) Rz(enc_l), then Rz(theta[R,0]) Ry(theta[R,1]),
// and reads |a|-|b| (fast) or |a|^2-|b|^2 (Born). Here the same state is the
// real Bloch vector v = (vx,vy,vz):
//   H|0>            -> v = (1,0,0)
//   Rz(phi)         -> rotation of (vx,vy) by +phi
//   Ry(phi)         -> (vx,vz) <- (vx cos + vz sin, vz cos - vx sin)
//   Born readout    -> vz
//   fast readout    -> vz * rsqrt(1 + sqrt(vx^2+vy^2))
// Adjacent Rz gates are merged: Rz(enc_l) Rz(theta[l+1,0]) = Rz(pw_l x + c_l) with
// c_l = pb_l + theta[l+1,0]; the leading Rz(theta[0,0]) Ry(theta[0,1]) acts on a
// constant and is folded into the start vector.
// Backward: with a the cotangent of v, the vector w = v x a transforms by the
// same rotations as v, and the derivative with respect to a gate's angle is the
// component of w along that gate's axis. One 3-vector is therefore swept back
// through the gates (4 flops per gate) and no intermediate state is stored.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/qkan_b200.h"

namespace qk {

constexpr int kWarp = 32;
constexpr int kMaxReps = 16;

// The kernels are instantiated for these repetition counts. A circuit with more than 8
// repetitions runs in the next larger instantiation, padded with identity gates (zero
// angles, zero preact weight). 0 is the instantiation of the "real" ansatz, whose whole
// circuit collapses to one data-dependent angle (see EdgeFwd<0>).
__host__ __device__ constexpr int compiled_reps(int ansatz, int reps) {
    return ansatz == QK_ANSATZ_REAL ? 0 : (reps <= 8 ? reps : (reps <= 12 ? 12 : 16));
}

// ---- per-edge constant table -------------------------------------------------
// table[((o * ipad) + i) * KS + k], float32: the KS = table_stride(R) constants of one edge are
// contiguous (a multiple of four floats, read as 128-bit loads), ipad = in_dim rounded up to 32.
__host__ __device__ constexpr int t_vx0() { return 0; }
__host__ __device__ constexpr int t_vy0() { return 1; }
__host__ __device__ constexpr int t_vz0() { return 2; }
__host__ __device__ constexpr int t_pw(int l) { return 3 + 2 * l; }
__host__ __device__ constexpr int t_c(int l) { return 4 + 2 * l; }
__host__ __device__ constexpr int t_ca(int R, int l) { return 3 + 2 * R + 2 * (l - 1); }  // l >= 1
__host__ __device__ constexpr int t_sa(int R, int l) { return 4 + 2 * R + 2 * (l - 1); }  // l >= 1
__host__ __device__ constexpr int t_cf(int R) { return 4 * R + 1; }
__host__ __device__ constexpr int t_sf(int R) { return 4 * R + 2; }
__host__ __device__ constexpr int t_w(int R) { return 4 * R + 3; }    // postact_weights * mask
__host__ __device__ constexpr int t_ca0(int R) { return 4 * R + 4; }  // cos/sin theta[0,1] (backward)
__host__ __device__ constexpr int t_sa0(int R) { return 4 * R + 5; }
__host__ __device__ constexpr int t_bw(int R) { return 4 * R + 6; }  // base_weight * mask
__host__ __device__ constexpr int table_rows(int R) { return 4 * R + 7; }
__host__ __device__ constexpr int table_stride(int R) { return (table_rows(R) + 3) / 4 * 4; }

// accumulators of the backward, per edge, summed over the batch
//   [0,R]      d/d theta[l,1]              (l = R is the final Ry)
//   R+1+l      d/d c_l  = d/d theta[l+1,0] = d/d preacts_bias[l]
//   2R+1+l     sum g_l * x = d/d preacts_weight[l]
//   3R+1       d/d theta[0,0]
//   3R+2       sum grad_y * postact  (-> d/d postact_weights)
//   3R+3       sum grad_y * silu(x)  (-> d/d base_weight), only with the base term
__host__ __device__ constexpr int a_ry(int l) { return l; }
__host__ __device__ constexpr int a_c(int R, int l) { return R + 1 + l; }
__host__ __device__ constexpr int a_pwx(int R, int l) { return 2 * R + 1 + l; }
__host__ __device__ constexpr int a_t00(int R) { return 3 * R + 1; }
__host__ __device__ constexpr int a_w(int R) { return 3 * R + 2; }
__host__ __device__ constexpr int acc_rows(int R) { return 3 * R + 3; }

inline __host__ __device__ int round_up(int v, int m) { return (v + m - 1) / m * m; }
inline __host__ __device__ size_t align256(size_t v) { return (v + 255) & ~size_t(255); }

// ---- typed loads / stores ----------------------------------------------------
template <typename T>
__device__ __forceinline__ float ld_as_float(const T* p);
template <>
__device__ __forceinline__ float ld_as_float<float>(const float* p) {
    return __ldg(p);
}
template <>
__device__ __forceinline__ float ld_as_float<__nv_bfloat16>(const __nv_bfloat16* p) {
    return __bfloat162float(__ldg(p));
}
// plain (coherent) loads for buffers the same kernel also writes
__device__ __forceinline__ float ld_rw_as_float(const float* p) { return *p; }
__device__ __forceinline__ float ld_rw_as_float(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T>
__device__ __forceinline__ void st_from_float(T* p, float v);
template <>
__device__ __forceinline__ void st_from_float<float>(float* p, float v) {
    *p = v;
}
template <>
__device__ __forceinline__ void st_from_float<__nv_bfloat16>(__nv_bfloat16* p, float v) {
    *p = __float2bfloat16_rn(v);
}

__device__ __forceinline__ float ld_param(const void* p, int dtype, size_t idx) {
    return dtype == QK_BF16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p)[idx])
                            : static_cast<const float*>(p)[idx];
}

// ---- fast math ---------------------------------------------------------------
// sin/cos of the data angle on the special-function unit. The angles are
// pw*x + c with |c| <= ~2*pi and moderate |pw*x|; the unit's absolute error is
// ~4e-7 there, well inside the 1e-5 normalised tolerance of the layer outputs.
// PRECISE selects the full-precision library routines instead: their error is ~1 ulp and varies
// smoothly with the argument, which quasi-Newton optimisers (LBFGS on small fits) rely on when they
// difference gradients; the SFU path is ~4x faster per call and is the default for large layers.
// sin and cos to ~1 ulp on the FMA pipe: three-term Cody-Waite reduction by pi/2 (exact products for
// |a| < ~1e4, graceful beyond) and the classic degree-7 / degree-8 minimax polynomials on [-pi/4, pi/4].
// Kept branch-free and small so that the full-precision kernel variants stay compact.
__device__ __forceinline__ void precise_sincos(float a, float& s, float& c) {
    const float j = rintf(a * 0.63661977236758134f);
    float r = fmaf(j, -1.5703125f, a);
    r = fmaf(j, -4.837512969970703125e-4f, r);
    r = fmaf(j, -7.54978995489188216e-8f, r);
    const float z = r * r;
    float ps = fmaf(z, -1.9515295891e-4f, 8.3321608736e-3f);
    ps = fmaf(ps, z, -1.6666654611e-1f);
    ps = fmaf(ps * z, r, r);  // sin(r)
    float pc = fmaf(z, 2.443315711809948e-5f, -1.388731625493765e-3f);
    pc = fmaf(pc, z, 4.166664568298827e-2f);
    pc = fmaf(pc * z, z, fmaf(z, -0.5f, 1.0f));  // cos(r)
    const int q = (int)j;
    const float ss = (q & 1) ? pc : ps;
    const float cc = (q & 1) ? ps : pc;
    s = (q & 2) ? -ss : ss;
    c = ((q + 1) & 2) ? -cc : cc;
}

// sin and cos on the FMA pipe at the special-function unit's accuracy (abs. error ~1.5e-7 for |a| up to a few
// pi): reduction by pi with the round-to-nearest-integer constant, odd / even minimax polynomials on
// [-pi/2, pi/2], sign from the parity of the multiple. 17 FP32 / integer instructions and no special-function
// call: the forward is bound by that unit (2 calls per data gate), so it evaluates a share of its rows this way
// to put its idle FMA issue slots to work.
__device__ __forceinline__ void poly_sincos(float a, float& s, float& c) {
    const float t = fmaf(a, 0.318309886183790672f, 12582912.0f);  // 1.5 * 2^23: the multiple lands in the low mantissa bits
    const float j = t - 12582912.0f;
    float r = fmaf(j, -3.14159274101257324f, a);
    r = fmaf(j, 8.74227765734758577e-8f, r);  // (float)pi - pi
    const unsigned sign = __float_as_uint(t) << 31;
    const float z = r * r;
    float ps = fmaf(z, 2.593941034e-06f, -1.980381325e-04f);
    ps = fmaf(ps, z, 8.332978007e-03f);
    ps = fmaf(ps, z, -1.666665547e-01f);
    ps = fmaf(ps * z, r, r);
    float pc = fmaf(z, 2.313151009e-05f, -1.385326930e-03f);
    pc = fmaf(pc, z, 4.166365739e-02f);
    pc = fmaf(pc, z, -4.999992083e-01f);
    pc = fmaf(pc, z, 1.0f);
    s = __uint_as_float(__float_as_uint(ps) ^ sign);
    c = __uint_as_float(__float_as_uint(pc) ^ sign);
}

template <bool PRECISE>
__device__ __forceinline__ void qk_sincos(float a, float& s, float& c) {
    if constexpr (PRECISE) {
        precise_sincos(a, s, c);
    } else {
        asm("sin.approx.ftz.f32 %0, %1;" : "=f"(s) : "f"(a));
        asm("cos.approx.ftz.f32 %0, %1;" : "=f"(c) : "f"(a));
    }
}
template <bool PRECISE>
__device__ __forceinline__ float qk_rsqrt(float a) {
    if constexpr (PRECISE) {
        return 1.0f / sqrtf(a);
    } else {
        float r;
        asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(a));
        return r;
    }
}
template <bool PRECISE>
__device__ __forceinline__ float qk_sqrt(float a) {
    if constexpr (PRECISE) {
        return sqrtf(a);
    } else {
        float r;
        asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(a));
        return r;
    }
}

// ---- per-edge constants in registers -----------------------------------------
// 128-bit loads of one edge's KS contiguous constants into registers
template <int KS>
__device__ __forceinline__ void load_edge_row(const float* __restrict__ t, float (&v)[KS]) {
    const float4* __restrict__ t4 = reinterpret_cast<const float4*>(t);
#pragma unroll
    for (int q = 0; q < KS / 4; ++q) {
        const float4 f = __ldg(t4 + q);
        v[4 * q + 0] = f.x;
        v[4 * q + 1] = f.y;
        v[4 * q + 2] = f.z;
        v[4 * q + 3] = f.w;
    }
}

template <int R>
struct EdgeFwd {
    float vx0, vy0, vz0;
    float pw[R], c[R];
    float ca[R], sa[R];  // index 0 is used by the backward only
    float cf, sf, w, bw;

    // t points at this edge's row of the table
    __device__ __forceinline__ void load(const float* __restrict__ t) {
        float v[table_stride(R)];
        load_edge_row(t, v);
        vx0 = v[t_vx0()];
        vy0 = v[t_vy0()];
        vz0 = v[t_vz0()];
#pragma unroll
        for (int l = 0; l < R; ++l) {
            pw[l] = v[t_pw(l)];
            c[l] = v[t_c(l)];
        }
#pragma unroll
        for (int l = 1; l < R; ++l) {
            ca[l] = v[t_ca(R, l)];
            sa[l] = v[t_sa(R, l)];
        }
        ca[0] = v[t_ca0(R)];
        sa[0] = v[t_sa0(R)];
        cf = v[t_cf(R)];
        sf = v[t_sf(R)];
        w = v[t_w(R)];
        bw = v[t_bw(R)];
    }
};

// "real" ansatz (reference: src/qkan/solver/exact.py:216-257): every gate is an Ry or a reflection
// in the x-z plane, so the circuit is one rotation by alpha = A x + C with A = sum_l pw_l (or reps)
// and C = pi/2 + sum_l (pb_l - theta_l - pi); readout cos(alpha) (Born) or
// cos(alpha) rsqrt(1 + |sin(alpha)|) (fast). Table rows: 0 = A, 1 = C reduced to [-pi,pi], 3 = weight.
template <>
struct EdgeFwd<0> {
    float a, c, w, bw;
    __device__ __forceinline__ void load(const float* __restrict__ t) {
        float v[table_stride(0)];
        load_edge_row(t, v);
        a = v[0];
        c = v[1];
        w = v[t_w(0)];
        bw = v[t_bw(0)];
    }
};

template <bool FAST, bool PRECISE>
__device__ __forceinline__ float real_forward(const EdgeFwd<0>& e, float x, float& s, float& c, float& r) {
    qk_sincos<PRECISE>(fmaf(e.a, x, e.c), s, c);
    if (!FAST) return c;
    r = qk_rsqrt<PRECISE>(1.0f + fabsf(s));
    return c * r;
}

// Forward of one edge for one batch row: returns the readout p (before bias and weight).
// When KEEP is true the data-gate sin/cos and the final Bloch vector are returned for the backward.
// POLY > 0: the first POLY data gates take their sin/cos from poly_sincos (FMA pipe) instead of the special-function unit.
template <int R, bool FAST, bool KEEP, bool PRECISE, int POLY = 0>
__device__ __forceinline__ float edge_forward(const EdgeFwd<R>& e, float x, float* cs, float* sn,
                                              float& vx, float& vy, float& vz, float& inv_rho,
                                              float& r) {
    if constexpr (R == 0) {
        float s, c;
        return real_forward<FAST, PRECISE>(e, x, s, c, r);
    } else {
    vx = e.vx0;
    vy = e.vy0;
    vz = e.vz0;
#pragma unroll
    for (int l = 0; l < R; ++l) {
        if (l > 0) {  // Ry(theta[l,1])
            float nx = fmaf(vz, e.sa[l], vx * e.ca[l]);
            float nz = fmaf(-vx, e.sa[l], vz * e.ca[l]);
            vx = nx;
            vz = nz;
        }
        float s, c;
        if (!PRECISE && l < POLY)
            poly_sincos(fmaf(e.pw[l], x, e.c[l]), s, c);
        else
            qk_sincos<PRECISE>(fmaf(e.pw[l], x, e.c[l]), s, c);  // merged Rz(pw_l x + pb_l + theta[l+1,0])
        if (KEEP) {
            cs[l] = c;
            sn[l] = s;
        }
        float nx = fmaf(-vy, s, vx * c);
        float ny = fmaf(vx, s, vy * c);
        vx = nx;
        vy = ny;
    }
    {  // final Ry(theta[R,1])
        float nx = fmaf(vz, e.sf, vx * e.cf);
        float nz = fmaf(-vx, e.sf, vz * e.cf);
        vx = nx;
        vz = nz;
    }
    if (!FAST) return vz;
    // rho^2 with a 1e-30 floor folded into the sum (keeps 1/rho finite at the poles at no extra cost)
    float s2 = fmaf(vx, vx, fmaf(vy, vy, 1e-30f));
    if (KEEP) {
        inv_rho = qk_rsqrt<PRECISE>(s2);
        r = qk_rsqrt<PRECISE>(fmaf(s2, inv_rho, 1.0f));
    } else {
        r = qk_rsqrt<PRECISE>(1.0f + qk_sqrt<PRECISE>(s2));
    }
    return vz * r;
    }
}

// Forward for frozen preacts (the data angle is x + c_l): sin/cos of x are taken once per (row, column)
// when the tile is staged, and every data gate gets its angle by the addition formulas from the
// per-edge constants (cos c_l, sin c_l) that the table holds in place of (pw_l, c_l) in this mode.
// No special-function call is left in the loop except the readout.
template <int R, bool FAST>
__device__ __forceinline__ float edge_forward_xtrig(const EdgeFwd<R>& e, float cx, float sx) {
    float vx = e.vx0, vy = e.vy0, vz = e.vz0;
#pragma unroll
    for (int l = 0; l < R; ++l) {
        if (l > 0) {  // Ry(theta[l,1])
            float nx = fmaf(vz, e.sa[l], vx * e.ca[l]);
            float nz = fmaf(-vx, e.sa[l], vz * e.ca[l]);
            vx = nx;
            vz = nz;
        }
        const float c = fmaf(-sx, e.c[l], cx * e.pw[l]);  // cos(x + c_l)
        const float s = fmaf(cx, e.c[l], sx * e.pw[l]);   // sin(x + c_l)
        float nx = fmaf(-vy, s, vx * c);
        float ny = fmaf(vx, s, vy * c);
        vx = nx;
        vy = ny;
    }
    {
        float nx = fmaf(vz, e.sf, vx * e.cf);
        float nz = fmaf(-vx, e.sf, vz * e.cf);
        vx = nx;
        vz = nz;
    }
    if (!FAST) return vz;
    const float s2 = fmaf(vx, vx, vy * vy);
    return vz * qk_rsqrt<false>(1.0f + qk_sqrt<false>(s2));
}

}  // namespace qk
