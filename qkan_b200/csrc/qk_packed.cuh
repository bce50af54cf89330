// Two batch rows per instruction: the circuit evaluation and its reverse sweep on Blackwell's packed
// float32 arithmetic (fma.rn.f32x2 / mul.f32x2 / add.f32x2: one issue slot carries the operation for two values
// held in an aligned register pair). Both hot kernels are bound by issue slots rather than by the FMA pipe's lanes,
// and every batch row of an edge runs the same instruction stream on the same per-edge constants, so rows
// (u, u+1) of a lane ride in the two halves of each pair. The per-edge constants are broadcast into pairs once
// per edge; the special-function calls (sin, cos, rsqrt, sqrt) stay scalar, one per half. Every packed operation
// rounds each half exactly as the scalar fmaf / multiply / add it replaces, and the operation order is that of
// edge_forward / edge_backward in qk_common.cuh / qk_backward.cuh, so every per-row value (readout, grad_x share)
// is bit-identical to the scalar form; the batch sums of the parameter gradients add the even and the odd rows
// separately before joining them (a different, equally fixed order). Reference counterparts: src/qkan/csrc/cute_kernels.cu:96-210 (forward), :216-508 (backward).
#pragma once
#include "qk_common.cuh"

namespace qk {

typedef float2 f2;

__device__ __forceinline__ f2 pk(float a) { return make_float2(a, a); }
__device__ __forceinline__ f2 mul2(f2 a, f2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ f2 fma2(f2 a, f2 b, f2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ f2 add2(f2 a, f2 b) { return __fadd2_rn(a, b); }
// Negation of both halves. QK_NEG_XOR = 1 flips the sign bits with integer operations (ALU pipe) instead of
// leaving the choice to the compiler; measured 1 % slower in the backward (14.43 against 14.30 ms), so it is off.
#ifndef QK_NEG_XOR
#define QK_NEG_XOR 0
#endif
__device__ __forceinline__ f2 neg2(f2 a) {
#if QK_NEG_XOR
    return make_float2(__uint_as_float(__float_as_uint(a.x) ^ 0x80000000u),
                       __uint_as_float(__float_as_uint(a.y) ^ 0x80000000u));
#else
    return make_float2(-a.x, -a.y);
#endif
}

__device__ __forceinline__ void sincos2(f2 a, f2& s, f2& c) {
    qk_sincos<false>(a.x, s.x, c.x);
    qk_sincos<false>(a.y, s.y, c.y);
}
__device__ __forceinline__ f2 rsqrt2(f2 a) { return make_float2(qk_rsqrt<false>(a.x), qk_rsqrt<false>(a.y)); }
__device__ __forceinline__ f2 sqrt2(f2 a) { return make_float2(qk_sqrt<false>(a.x), qk_sqrt<false>(a.y)); }

// poly_sincos on both halves: the FMA-pipe work packed, the sign bits per half
__device__ __forceinline__ void poly_sincos2(f2 a, f2& s, f2& c) {
    const f2 magic = pk(12582912.0f);
    const f2 t = fma2(a, pk(0.318309886183790672f), magic);
    const f2 j = add2(t, pk(-12582912.0f));
    f2 r = fma2(j, pk(-3.14159274101257324f), a);
    r = fma2(j, pk(8.74227765734758577e-8f), r);
    const unsigned sx = __float_as_uint(t.x) << 31, sy = __float_as_uint(t.y) << 31;
    const f2 z = mul2(r, r);
    f2 ps = fma2(z, pk(2.593941034e-06f), pk(-1.980381325e-04f));
    ps = fma2(ps, z, pk(8.332978007e-03f));
    ps = fma2(ps, z, pk(-1.666665547e-01f));
    ps = fma2(mul2(ps, z), r, r);
    f2 pc = fma2(z, pk(2.313151009e-05f), pk(-1.385326930e-03f));
    pc = fma2(pc, z, pk(4.166365739e-02f));
    pc = fma2(pc, z, pk(-4.999992083e-01f));
    pc = fma2(pc, z, pk(1.0f));
    s = make_float2(__uint_as_float(__float_as_uint(ps.x) ^ sx), __uint_as_float(__float_as_uint(ps.y) ^ sy));
    c = make_float2(__uint_as_float(__float_as_uint(pc.x) ^ sx), __uint_as_float(__float_as_uint(pc.y) ^ sy));
}

// The edge's constants broadcast into register pairs (and the negated sines the rotations need, since the
// packed operations have no negate modifier).
template <int R>
struct EdgePk {
    f2 vx0, vy0, vz0;
    static constexpr int N = R > 0 ? R : 1;
    f2 pw[N], c[N];
    f2 ca[N], sa[N], nsa[N];  // index 0: backward only
    f2 cf, sf, nsf, w;
    __device__ __forceinline__ void from(const EdgeFwd<R>& e) {
        vx0 = pk(e.vx0);
        vy0 = pk(e.vy0);
        vz0 = pk(e.vz0);
#pragma unroll
        for (int l = 0; l < R; ++l) {
            pw[l] = pk(e.pw[l]);
            c[l] = pk(e.c[l]);
            ca[l] = pk(e.ca[l]);
            sa[l] = pk(e.sa[l]);
            nsa[l] = pk(-e.sa[l]);
        }
        cf = pk(e.cf);
        sf = pk(e.sf);
        nsf = pk(-e.sf);
        w = pk(e.w);
    }
};

// Forward of one edge for two batch rows (see edge_forward). KEEP: the data-gate cos / sin / -sin and the final
// Bloch vector are returned for the backward. POLY: the first POLY data gates take sin/cos from the polynomial.
template <int R, bool FAST, bool KEEP, int POLY>
__device__ __forceinline__ f2 edge_forward2(const EdgePk<R>& e, f2 x, f2* cs, f2* sn, f2* nsn, f2& vx, f2& vy,
                                            f2& vz, f2& inv_rho, f2& r) {
    vx = e.vx0;
    vy = e.vy0;
    vz = e.vz0;
#pragma unroll
    for (int l = 0; l < R; ++l) {
        if (l > 0) {  // Ry(theta[l,1])
            const f2 nx = fma2(vz, e.sa[l], mul2(vx, e.ca[l]));
            const f2 nz = fma2(vx, e.nsa[l], mul2(vz, e.ca[l]));
            vx = nx;
            vz = nz;
        }
        f2 s, c;
        if (l < POLY)
            poly_sincos2(fma2(e.pw[l], x, e.c[l]), s, c);
        else
            sincos2(fma2(e.pw[l], x, e.c[l]), s, c);  // merged Rz(pw_l x + pb_l + theta[l+1,0])
        const f2 ns = neg2(s);
        if (KEEP) {
            cs[l] = c;
            sn[l] = s;
            nsn[l] = ns;
        }
        const f2 nx = fma2(vy, ns, mul2(vx, c));
        const f2 ny = fma2(vx, s, mul2(vy, c));
        vx = nx;
        vy = ny;
    }
    {  // final Ry(theta[R,1])
        const f2 nx = fma2(vz, e.sf, mul2(vx, e.cf));
        const f2 nz = fma2(vx, e.nsf, mul2(vz, e.cf));
        vx = nx;
        vz = nz;
    }
    if (!FAST) return vz;
    const f2 s2 = fma2(vx, vx, fma2(vy, vy, pk(1e-30f)));
    if (KEEP) {
        inv_rho = rsqrt2(s2);
        r = rsqrt2(fma2(s2, inv_rho, pk(1.0f)));
    } else {
        r = rsqrt2(add2(pk(1.0f), sqrt2(s2)));
    }
    return mul2(vz, r);
}

// Frozen-preact forward for two rows (see edge_forward_xtrig): cx / sx hold cos x / sin x of the two rows and the
// table rows (pw_l, c_l) hold (cos c_l, sin c_l).
template <int R, bool FAST>
__device__ __forceinline__ f2 edge_forward_xtrig2(const EdgePk<R>& e, f2 cx, f2 sx) {
    f2 vx = e.vx0, vy = e.vy0, vz = e.vz0;
    const f2 nsx = neg2(sx);
#pragma unroll
    for (int l = 0; l < R; ++l) {
        if (l > 0) {
            const f2 nx = fma2(vz, e.sa[l], mul2(vx, e.ca[l]));
            const f2 nz = fma2(vx, e.nsa[l], mul2(vz, e.ca[l]));
            vx = nx;
            vz = nz;
        }
        const f2 c = fma2(nsx, e.c[l], mul2(cx, e.pw[l]));  // cos(x + c_l)
        const f2 s = fma2(cx, e.c[l], mul2(sx, e.pw[l]));   // sin(x + c_l)
        const f2 ns = neg2(s);
        const f2 nx = fma2(vy, ns, mul2(vx, c));
        const f2 ny = fma2(vx, s, mul2(vy, c));
        vx = nx;
        vy = ny;
    }
    {
        const f2 nx = fma2(vz, e.sf, mul2(vx, e.cf));
        const f2 nz = fma2(vx, e.nsf, mul2(vz, e.cf));
        vx = nx;
        vz = nz;
    }
    if (!FAST) return vz;
    const f2 s2 = fma2(vx, vx, mul2(vy, vy));
    return mul2(vz, rsqrt2(add2(pk(1.0f), sqrt2(s2))));
}

// Backward of one edge for two batch rows (see edge_backward): returns gx0 + d/dx; the accumulators hold the two
// rows' sums in their halves (added together once per edge by the caller).
template <int R, bool FAST, bool EDGES, int NACC>
__device__ __forceinline__ f2 edge_backward2(const EdgePk<R>& e, f2 x, f2 g, f2 gx0, f2 (&acc)[NACC]) {
    f2 cs[R], sn[R], nsn[R], vx, vy, vz, inv_rho, r;
    const f2 p = edge_forward2<R, FAST, true, 0>(e, x, cs, sn, nsn, vx, vy, vz, inv_rho, r);
    const f2 gp = EDGES ? g : mul2(g, e.w);
    if (!EDGES) acc[a_w(R)] = fma2(g, p, acc[a_w(R)]);
    f2 wx, wy, wz;
    if (FAST) {
        const f2 k = mul2(mul2(gp, r), fma2(mul2(mul2(pk(0.5f), p), p), inv_rho, pk(1.0f)));
        wx = mul2(vy, k);
        wy = neg2(mul2(vx, k));
    } else {
        wx = mul2(vy, gp);
        wy = neg2(mul2(vx, gp));
    }
    acc[a_ry(R)] = add2(acc[a_ry(R)], wy);  // final Ry(theta[R,1])
    wz = mul2(wx, e.sf);
    wx = mul2(wx, e.cf);
    f2 gx = gx0;
#pragma unroll
    for (int l = R - 1; l >= 0; --l) {
        acc[a_c(R, l)] = add2(acc[a_c(R, l)], wz);
        acc[a_pwx(R, l)] = fma2(wz, x, acc[a_pwx(R, l)]);
        gx = fma2(wz, e.pw[l], gx);
        const f2 nx = fma2(wy, sn[l], mul2(wx, cs[l]));
        const f2 ny = fma2(wx, nsn[l], mul2(wy, cs[l]));
        wx = nx;
        wy = ny;
        acc[a_ry(l)] = add2(acc[a_ry(l)], wy);  // Ry(theta[l,1])
        if (l > 0) {
            const f2 mx = fma2(wz, e.nsa[l], mul2(wx, e.ca[l]));
            const f2 mz = fma2(wx, e.sa[l], mul2(wz, e.ca[l]));
            wx = mx;
            wz = mz;
        } else {
            wz = fma2(wx, e.sa[0], mul2(wz, e.ca[0]));
        }
    }
    acc[a_t00(R)] = add2(acc[a_t00(R)], wz);  // Rz(theta[0,0])
    return gx;
}

}  // namespace qk
