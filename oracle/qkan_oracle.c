/*
 * TEST INFRASTRUCTURE — CPU restatement of the reference QKANLayer hot path.
 *
 * This file is the checker, never the product: only the test-suite, the
 * smoke check and the benchmark's CPU-baseline leg may load it. The CUDA
 * library must never link or call it.
 *
 * It restates, gate by gate and with complex amplitudes (NOT the Bloch-vector
 * form the CUDA kernels use), what the reference computes for the
 * "pz_encoding", "rpz_encoding" and "real" ansaetze:
 *
 *   circuits     src/qkan/solver/exact.py:90-134 (_pz_encoding), 136-168 (_rpz_encoding), 216-257 (_real)
 *   X, Z gates   src/qkan/torch_qc.py:337-349
 *   preact enc   src/qkan/solver/exact.py:77-87    (encoded_x = pw*x + pb)
 *   H gate       src/qkan/torch_qc.py:108-121      (h_gate)
 *   Rz gate      src/qkan/torch_qc.py:92-105       (diag(e^{-i phi/2}, e^{+i phi/2}))
 *   Ry gate      src/qkan/torch_qc.py:76-89        ([[c,-s],[s,c]], c = cos(phi/2))
 *   readout      src/qkan/torch_qc.py:261-277      (|a|-|b| fast, |a|^2-|b|^2 Born)
 *   epilogue     src/qkan/qkan.py:750-785          (sum_i (postacts+pb)*pw*mask + silu(x) @ (bw*mask)^T)
 *
 * The backward is a hand-written reverse-mode sweep over the same gate list
 * with every intermediate state kept, which is what torch autograd does for
 * the reference's exact solver.
 *
 * Parity pinned: the reference holds no golden vectors for this path, so the
 * pin is the reference itself executed on CPU; tests/golden/ holds its
 * outputs and tests/test_oracle.py checks this file against them.
 *
 * Compiled twice: with -DORACLE_F64 (double, symbols *_f64) and without
 * (float, symbols *_f32). Array layouts are the reference's natural-rank,
 * row-major layouts:
 *   x (B,I)  theta (O,I,R+1,2) [rpz: (O,I,R+1,1), real: (O,I,R,1)]  preacts_weight/bias (O,I,R)
 *   postact_weights/postact_bias/base_weight/mask (O,I)  y (B,O)
 */
#include <math.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#ifdef ORACLE_F64
typedef double real;
#define FN(name) name##_f64
#define R_COS cos
#define R_SIN sin
#define R_SQRT sqrt
#define R_EXP exp
#else
typedef float real;
#define FN(name) name##_f32
#define R_COS cosf
#define R_SIN sinf
#define R_SQRT sqrtf
#define R_EXP expf
#endif

#define QO_PREACT_TRAINABLE 1u
#define QO_FAST_MEASURE 2u
#define QO_USE_POSTACT_BIAS 4u

#define QO_MAX_REPS 64

typedef struct {
    real a0r, a0i, a1r, a1i;
} amp_t;

/* Rz(phi) = diag(e^{-i phi/2}, e^{+i phi/2})  (torch_qc.py:92-105) */
static inline amp_t apply_rz(amp_t s, real phi) {
    real er = R_COS(phi / 2), ei = -R_SIN(phi / 2);
    amp_t o;
    o.a0r = s.a0r * er - s.a0i * ei;
    o.a0i = s.a0r * ei + s.a0i * er;
    o.a1r = s.a1r * er + s.a1i * ei;
    o.a1i = -s.a1r * ei + s.a1i * er;
    return o;
}

/* Ry(phi) = [[c,-s],[s,c]]  (torch_qc.py:76-89) */
static inline amp_t apply_ry(amp_t s, real phi) {
    real c = R_COS(phi / 2), sn = R_SIN(phi / 2);
    amp_t o;
    o.a0r = c * s.a0r - sn * s.a1r;
    o.a0i = c * s.a0i - sn * s.a1i;
    o.a1r = sn * s.a0r + c * s.a1r;
    o.a1i = sn * s.a0i + c * s.a1i;
    return o;
}

/* reverse of Rz: cotangent of the input and d/dphi, given the gate INPUT s */
static inline amp_t rz_vjp(amp_t s, real phi, amp_t bar, real *gphi) {
    real er = R_COS(phi / 2), ei = -R_SIN(phi / 2);
    real der = (real)0.5 * ei;  /* d cos(phi/2)/dphi = -sin(phi/2)/2 */
    real dei = -(real)0.5 * er; /* d(-sin(phi/2))/dphi = -cos(phi/2)/2 */
    *gphi = bar.a0r * (s.a0r * der - s.a0i * dei) + bar.a0i * (s.a0r * dei + s.a0i * der) +
            bar.a1r * (s.a1r * der + s.a1i * dei) + bar.a1i * (-s.a1r * dei + s.a1i * der);
    amp_t o;
    o.a0r = bar.a0r * er + bar.a0i * ei;
    o.a0i = -bar.a0r * ei + bar.a0i * er;
    o.a1r = bar.a1r * er - bar.a1i * ei;
    o.a1i = bar.a1r * ei + bar.a1i * er;
    return o;
}

static inline amp_t ry_vjp(amp_t s, real phi, amp_t bar, real *gphi) {
    real c = R_COS(phi / 2), sn = R_SIN(phi / 2);
    real dc = -(real)0.5 * sn, ds = (real)0.5 * c;
    *gphi = bar.a0r * (dc * s.a0r - ds * s.a1r) + bar.a0i * (dc * s.a0i - ds * s.a1i) +
            bar.a1r * (ds * s.a0r + dc * s.a1r) + bar.a1i * (ds * s.a0i + dc * s.a1i);
    amp_t o;
    o.a0r = c * bar.a0r + sn * bar.a1r;
    o.a0i = c * bar.a0i + sn * bar.a1i;
    o.a1r = -sn * bar.a0r + c * bar.a1r;
    o.a1i = -sn * bar.a0i + c * bar.a1i;
    return o;
}

static inline real measure(amp_t s, int fast) {
    real n0 = s.a0r * s.a0r + s.a0i * s.a0i, n1 = s.a1r * s.a1r + s.a1i * s.a1i;
    return fast ? R_SQRT(n0) - R_SQRT(n1) : n0 - n1;
}

/* cotangent of the amplitudes for readout cotangent g (torch: d|z| = z/|z|, 0 at z = 0) */
static inline amp_t measure_vjp(amp_t s, int fast, real g) {
    amp_t b;
    if (fast) {
        real m0 = R_SQRT(s.a0r * s.a0r + s.a0i * s.a0i);
        real m1 = R_SQRT(s.a1r * s.a1r + s.a1i * s.a1i);
        real i0 = m0 > 0 ? g / m0 : 0, i1 = m1 > 0 ? -g / m1 : 0;
        b.a0r = s.a0r * i0;
        b.a0i = s.a0i * i0;
        b.a1r = s.a1r * i1;
        b.a1i = s.a1i * i1;
    } else {
        b.a0r = 2 * g * s.a0r;
        b.a0i = 2 * g * s.a0i;
        b.a1r = -2 * g * s.a1r;
        b.a1i = -2 * g * s.a1i;
    }
    return b;
}

static inline real silu(real v) { return v / (1 + R_EXP(-v)); }
static inline real silu_grad(real v) {
    real s = 1 / (1 + R_EXP(-v));
    return s * (1 + v * (1 - s));
}

/*
 * Gate lists of the three ansaetze (bits 8-9 of flags: 0 pz, 1 rpz, 2 real).
 *   pz   exact.py:90-134   per rep Rz(th[l,0]) Ry(th[l,1]) Rz(enc_l); then Rz(th[R,0]) Ry(th[R,1]); theta (R+1,2)
 *   rpz  exact.py:136-168  per rep Ry(th[l]) Rz(enc_l); then Ry(th[R]); theta (R+1,1); enc always pw*x+pb
 *   real exact.py:216-257  per rep X Ry(th[l]) Z Ry(enc_l); no final layer; theta (R,1)
 */
enum { G_RZ = 0, G_RY = 1, G_X = 2, G_Z = 3 };
enum { SRC_NONE = -1, SRC_THETA = 0, SRC_ENC = 1 };
typedef struct {
    int kind, src, idx;
} gate_t;

#define QO_ANSATZ(flags) (((flags) >> 8) & 3u)
#define QO_MAX_GATES (4 * QO_MAX_REPS + 4)

static int theta_per_edge(int ansatz, int R) { return ansatz == 0 ? 2 * (R + 1) : (ansatz == 1 ? R + 1 : R); }

static int build_gates(int ansatz, int R, gate_t *g) {
    int n = 0;
    for (int l = 0; l < R; ++l) {
        if (ansatz == 0) {
            g[n++] = (gate_t){G_RZ, SRC_THETA, 2 * l};
            g[n++] = (gate_t){G_RY, SRC_THETA, 2 * l + 1};
            g[n++] = (gate_t){G_RZ, SRC_ENC, l};
        } else if (ansatz == 1) {
            g[n++] = (gate_t){G_RY, SRC_THETA, l};
            g[n++] = (gate_t){G_RZ, SRC_ENC, l};
        } else {
            g[n++] = (gate_t){G_X, SRC_NONE, 0};
            g[n++] = (gate_t){G_RY, SRC_THETA, l};
            g[n++] = (gate_t){G_Z, SRC_NONE, 0};
            g[n++] = (gate_t){G_RY, SRC_ENC, l};
        }
    }
    if (ansatz == 0) {
        g[n++] = (gate_t){G_RZ, SRC_THETA, 2 * R};
        g[n++] = (gate_t){G_RY, SRC_THETA, 2 * R + 1};
    } else if (ansatz == 1) {
        g[n++] = (gate_t){G_RY, SRC_THETA, R};
    }
    return n;
}

static inline int uses_preacts(unsigned flags) {
    return (flags & QO_PREACT_TRAINABLE) || QO_ANSATZ(flags) == 1; /* exact.py:75-76 */
}

static inline real gate_angle(const gate_t *g, real x, const real *th, const real *pw, const real *pb,
                              unsigned flags) {
    if (g->src == SRC_THETA) return th[g->idx];
    return uses_preacts(flags) ? pw[g->idx] * x + pb[g->idx] : x; /* exact.py:87,121-124 */
}

/* One edge, forward. states (n_gates+1 entries, gate inputs then the final state) may be NULL. */
static inline real edge_forward(real x, const real *th, const real *pw, const real *pb,
                                const gate_t *gates, int n_gates, unsigned flags, amp_t *states) {
    const real h = (real)0.70710678118654752440;
    amp_t s = {h, 0, h, 0}; /* H|0> */
    for (int k = 0; k < n_gates; ++k) {
        const gate_t *g = gates + k;
        if (states) states[k] = s;
        if (g->kind == G_RZ) {
            s = apply_rz(s, gate_angle(g, x, th, pw, pb, flags));
        } else if (g->kind == G_RY) {
            s = apply_ry(s, gate_angle(g, x, th, pw, pb, flags));
        } else if (g->kind == G_X) { /* torch_qc.py:337-343 */
            amp_t t = {s.a1r, s.a1i, s.a0r, s.a0i};
            s = t;
        } else { /* Z, torch_qc.py:345-349 */
            s.a1r = -s.a1r;
            s.a1i = -s.a1i;
        }
    }
    if (states) states[n_gates] = s;
    return measure(s, (flags & QO_FAST_MEASURE) != 0);
}

/* postacts (B,O,I): what the reference solver returns (solver/_base.py contract). */
int FN(qkan_oracle_postacts)(int B, int I, int O, int R, unsigned flags, const real *x,
                             const real *theta, const real *pw, const real *pb, real *postacts) {
    if (R < 0 || R > QO_MAX_REPS || QO_ANSATZ(flags) > 2) return -1;
    gate_t gates[QO_MAX_GATES];
    const int ng = build_gates(QO_ANSATZ(flags), R, gates);
    const int tpe = theta_per_edge(QO_ANSATZ(flags), R);
#pragma omp parallel for schedule(static)
    for (int b = 0; b < B; ++b)
        for (int o = 0; o < O; ++o)
            for (int i = 0; i < I; ++i) {
                size_t e = (size_t)o * I + i;
                postacts[((size_t)b * O + o) * I + i] = edge_forward(
                    x[(size_t)b * I + i], theta + e * tpe, pw + e * R, pb + e * R, gates, ng, flags, NULL);
            }
    return 0;
}

/* Layer forward: y (B,O).  qkan.py:750-785 (train route; the eval route folds the same terms). */
int FN(qkan_oracle_forward)(int B, int I, int O, int R, unsigned flags, const real *x,
                            const real *theta, const real *pw, const real *pb, const real *postw,
                            const real *postb, const real *basew, const real *mask, real *y) {
    if (R < 0 || R > QO_MAX_REPS || QO_ANSATZ(flags) > 2) return -1;
    const int use_pb = (flags & QO_USE_POSTACT_BIAS) && postb;
    gate_t gates[QO_MAX_GATES];
    const int ng = build_gates(QO_ANSATZ(flags), R, gates);
    const int tpe = theta_per_edge(QO_ANSATZ(flags), R);
#pragma omp parallel for schedule(static)
    for (int b = 0; b < B; ++b)
        for (int o = 0; o < O; ++o) {
            real acc = 0;
            for (int i = 0; i < I; ++i) {
                size_t e = (size_t)o * I + i;
                real xv = x[(size_t)b * I + i];
                real m = mask ? mask[e] : 1;
                real p = edge_forward(xv, theta + e * tpe, pw + e * R, pb + e * R, gates, ng, flags, NULL);
                if (use_pb) p += postb[e];
                acc += p * (postw[e] * m);
                if (basew) acc += silu(xv) * (basew[e] * m);
            }
            y[(size_t)b * O + o] = acc;
        }
    return 0;
}

/*
 * Layer backward. Any gradient pointer may be NULL (not wanted). gpostacts,
 * when given, replaces the epilogue: the cotangent of postacts (B,O,I) is
 * read from it and postw/postb/basew/mask/gy are ignored (solver contract).
 * Parallel over o; grad_x is accumulated per thread and reduced at the end.
 */
int FN(qkan_oracle_backward)(int B, int I, int O, int R, unsigned flags, const real *x,
                             const real *theta, const real *pw, const real *pb, const real *postw,
                             const real *postb, const real *basew, const real *mask,
                             const real *gy, const real *gpostacts, real *gx, real *gtheta,
                             real *gpw, real *gpb, real *gpostw, real *gpostb, real *gbasew) {
    if (R < 0 || R > QO_MAX_REPS || QO_ANSATZ(flags) > 2) return -1;
    const int use_pb = (flags & QO_USE_POSTACT_BIAS) && postb;
    const int fast = (flags & QO_FAST_MEASURE) != 0;
    const int ptr = uses_preacts(flags);
    gate_t gates[QO_MAX_GATES];
    const int ng = build_gates(QO_ANSATZ(flags), R, gates);
    const int tpe = theta_per_edge(QO_ANSATZ(flags), R);
    size_t nE = (size_t)O * I;
    if (gtheta) memset(gtheta, 0, nE * tpe * sizeof(real));
    if (gpw) memset(gpw, 0, nE * R * sizeof(real));
    if (gpb) memset(gpb, 0, nE * R * sizeof(real));
    if (gpostw) memset(gpostw, 0, nE * sizeof(real));
    if (gpostb) memset(gpostb, 0, nE * sizeof(real));
    if (gbasew) memset(gbasew, 0, nE * sizeof(real));
    if (gx) memset(gx, 0, (size_t)B * I * sizeof(real));
    int nthreads = 1;
#ifdef _OPENMP
    nthreads = omp_get_max_threads();
#endif
    real *gx_priv = NULL;
    if (gx && nthreads > 1) {
        gx_priv = (real *)calloc((size_t)nthreads * B * I, sizeof(real));
        if (!gx_priv) return -2;
    }
#pragma omp parallel
    {
        int tid = 0;
#ifdef _OPENMP
        tid = omp_get_thread_num();
#endif
        real *gxl = gx ? (gx_priv ? gx_priv + (size_t)tid * B * I : gx) : NULL;
        amp_t states[QO_MAX_GATES + 1];
#pragma omp for schedule(static)
        for (int o = 0; o < O; ++o)
            for (int i = 0; i < I; ++i) {
                size_t e = (size_t)o * I + i;
                const real *th = theta + e * tpe;
                const real *pwe = pw + e * R, *pbe = pb + e * R;
                real m = mask ? mask[e] : 1;
                real W = gpostacts ? 0 : postw[e] * m;
                for (int b = 0; b < B; ++b) {
                    real xv = x[(size_t)b * I + i];
                    real p = edge_forward(xv, th, pwe, pbe, gates, ng, flags, states);
                    real gp;
                    real gxv = 0;
                    if (gpostacts) {
                        gp = gpostacts[((size_t)b * O + o) * I + i];
                    } else {
                        real g = gy[(size_t)b * O + o];
                        gp = g * W;
                        if (gpostw) gpostw[e] += g * (p + (use_pb ? postb[e] : 0)) * m;
                        if (gpostb && use_pb) gpostb[e] += g * W;
                        if (basew) {
                            if (gbasew) gbasew[e] += g * silu(xv) * m;
                            gxv += g * basew[e] * m * silu_grad(xv);
                        }
                    }
                    /* reverse sweep over the gate list */
                    amp_t bar = measure_vjp(states[ng], fast, gp);
                    for (int k = ng - 1; k >= 0; --k) {
                        const gate_t *gt = gates + k;
                        real g = 0;
                        if (gt->kind == G_RZ) {
                            bar = rz_vjp(states[k], gate_angle(gt, xv, th, pwe, pbe, flags), bar, &g);
                        } else if (gt->kind == G_RY) {
                            bar = ry_vjp(states[k], gate_angle(gt, xv, th, pwe, pbe, flags), bar, &g);
                        } else if (gt->kind == G_X) {
                            amp_t t = {bar.a1r, bar.a1i, bar.a0r, bar.a0i};
                            bar = t;
                            continue;
                        } else {
                            bar.a1r = -bar.a1r;
                            bar.a1i = -bar.a1i;
                            continue;
                        }
                        if (gt->src == SRC_THETA) {
                            if (gtheta) gtheta[e * tpe + gt->idx] += g;
                        } else if (ptr) {
                            if (gpw) gpw[e * R + gt->idx] += g * xv;
                            if (gpb) gpb[e * R + gt->idx] += g;
                            gxv += g * pwe[gt->idx];
                        } else {
                            gxv += g;
                        }
                    }
                    if (gxl) gxl[(size_t)b * I + i] += gxv;
                }
            }
    }
    if (gx_priv) {
        for (int t = 0; t < nthreads; ++t)
            for (size_t j = 0; j < (size_t)B * I; ++j) gx[j] += gx_priv[(size_t)t * B * I + j];
        free(gx_priv);
    }
    return 0;
}

/* Launchers such as torchrun export OMP_NUM_THREADS=1; the baseline timing asks for all cores explicitly. */
void FN(qkan_oracle_set_num_threads)(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int FN(qkan_oracle_num_threads)(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
