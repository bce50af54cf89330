/*
 * qkan_b200 — C ABI of the sm_100a QKANLayer kernels (pz_encoding, rpz_encoding and real ansaetze).
 *
 * Every entry point takes plain device pointers and sizes, launches on the
 * stream it is given, never synchronises, never allocates and never throws.
 * Return value: 0 on success, a negative QK_ERR_* code otherwise;
 * qk_last_error() then returns a thread-local description.
 *
 * Tensor layouts are the reference's natural-rank, row-major layouts
 * (src/qkan/qkan.py:259-347):
 *   x (B,I)  y (B,O)  theta (O,I,R+1,2) [see QkAnsatz]  preacts_weight/bias (O,I,R)
 *   postact_weights / postact_bias / base_weight / mask (O,I)
 * theta and preacts are always float32. x, y and their gradients use
 * QkDesc.io_dtype; the four (O,I) tensors use QkDesc.param_dtype. All
 * gradient outputs of parameters are float32.
 */
#ifndef QKAN_B200_H_
#define QKAN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define QK_ABI_VERSION 4

enum QkDtype { QK_F32 = 0, QK_BF16 = 1 };

/*
 * Circuit family (QKANLayer `ansatz=`). theta layouts follow src/qkan/qkan.py:259-274:
 *   QK_ANSATZ_PZ   "pz_encoding"  theta (O,I,R+1,2)   src/qkan/solver/exact.py:90-134
 *   QK_ANSATZ_RPZ  "rpz_encoding" theta (O,I,R+1,1)   src/qkan/solver/exact.py:136-168
 *                  (always encodes preacts_weight*x + preacts_bias, whatever QK_PREACT_TRAINABLE says)
 *   QK_ANSATZ_REAL "real"         theta (O,I,R,1)     src/qkan/solver/exact.py:216-257
 */
enum QkAnsatz { QK_ANSATZ_PZ = 0, QK_ANSATZ_RPZ = 1, QK_ANSATZ_REAL = 2 };

enum QkFlags {
    QK_PREACT_TRAINABLE = 1u, /* encode pw*x+pb; otherwise x itself (exact.py:87,121-124) */
    QK_FAST_MEASURE = 2u,     /* |a|-|b| readout; otherwise |a|^2-|b|^2 (torch_qc.py:261-277) */
    QK_USE_POSTACT_BIAS = 4u, /* add postact_bias before the weight (qkan.py:776-783) */
    QK_PRECISE_MATH = 8u,     /* sin/cos/sqrt by the full-precision routines instead of the special-function
                                 unit: ~1 ulp and smooth in the argument, as torch's own sin/cos in the
                                 reference are; meant for small fits driven by LBFGS. Honoured for QK_F32
                                 activations; with QK_BF16 activations the flag is accepted and has no effect
                                 (bfloat16 rounding of x and y is four orders of magnitude coarser) */
    QK_SINGLE_TABLE = 16u     /* frozen preacts (QK_PREACT_TRAINABLE off): do not build the second per-edge table
                                 that the angle-addition forward reads; the generic forward kernel runs instead
                                 (about a fifth slower there) and qk_tables_bytes() is nearly halved. For callers short
                                 of scratch; qk_pz_forward_noalloc sets it by itself when that makes a layer fit */
};

enum QkError {
    QK_OK = 0,
    QK_ERR_BAD_ARGUMENT = -1,
    QK_ERR_UNSUPPORTED = -2,
    QK_ERR_WORKSPACE = -3,
    QK_ERR_LAUNCH = -4
};

typedef struct QkDesc {
    int32_t batch;       /* B */
    int32_t in_dim;      /* I */
    int32_t out_dim;     /* O */
    int32_t reps;        /* 1 <= R <= 16 */
    int32_t io_dtype;    /* QkDtype of x, y, grad_y, grad_x */
    int32_t param_dtype; /* QkDtype of postact_weights, postact_bias, base_weight, mask */
    uint32_t flags;      /* QkFlags */
    int32_t ansatz;      /* QkAnsatz */
    int32_t group;       /* 0: theta / preacts hold one entry per edge, shapes (O,I,...).
                            g > 0: grouped parameters (QKANLayer `group=g`, src/qkan/qkan.py:246-308):
                            theta is (g,...) and preacts are (g,R); edge (o,i) uses entry i mod g for every o
                            (the broadcast of src/qkan/solver/exact.py:68-86), and grad_theta / grad_preacts_*
                            come back in the grouped shapes, summed over the edges that share an entry. */
} QkDesc;

/* ABI version of the loaded library (compare with QK_ABI_VERSION). */
int qk_abi_version(void);

/* Thread-local text of the last error returned on this thread ("" if none). */
const char* qk_last_error(void);

/*
 * Bytes of device scratch the forward / backward need for this problem.
 * The caller owns the scratch (any 256-byte aligned device allocation) and
 * may reuse it between calls on the same stream. The first qk_tables_bytes() bytes
 * hold the prepared state described further down; the backward's share follows it.
 */
size_t qk_forward_workspace_bytes(const QkDesc* desc);
size_t qk_backward_workspace_bytes(const QkDesc* desc);

/*
 * Fused layer forward: replaces the body of QKANLayer._forward_train /
 * _forward_eval after the optional batch-norm (src/qkan/qkan.py:727-785):
 * solver call (src/qkan/solver/exact.py:90-134) + mask fold + epilogue
 *   y[b,o] = sum_i (postacts[b,o,i] + postact_bias[o,i]) * postact_weights[o,i] * mask[o,i]
 *          + sum_i silu(x[b,i]) * base_weight[o,i] * mask[o,i]
 * without materialising postacts. postact_bias, base_weight and mask may be
 * NULL (zero, zero, ones).
 */
int qk_pz_forward(const QkDesc* desc, const void* x, const float* theta,
                  const float* preacts_weight, const float* preacts_bias,
                  const void* postact_weights, const void* postact_bias, const void* base_weight,
                  const void* mask, void* y, void* workspace, size_t workspace_bytes,
                  void* cuda_stream);

/*
 * Fused layer backward: what torch autograd derives for the reference's
 * exact solver plus epilogue (src/qkan/solver/exact.py:90-134,
 * src/qkan/qkan.py:776-785; the fused reference counterparts are
 * src/qkan/csrc/cute_kernels.cu:216-508 and src/qkan/qkan_epilogue.py:187-309).
 * Every gradient pointer may be NULL when that gradient is not wanted.
 * Parameter gradients are summed over the batch in a fixed order
 * (run-to-run bitwise reproducible) and are OVERWRITTEN, not accumulated.
 */
int qk_pz_backward(const QkDesc* desc, const void* x, const float* theta,
                   const float* preacts_weight, const float* preacts_bias,
                   const void* postact_weights, const void* postact_bias, const void* base_weight,
                   const void* mask, const void* grad_y, void* grad_x, float* grad_theta,
                   float* grad_preacts_weight, float* grad_preacts_bias,
                   float* grad_postact_weights, float* grad_postact_bias, float* grad_base_weight,
                   void* workspace, size_t workspace_bytes, void* cuda_stream);

/*
 * The same layer step with its set-up hoisted out, four launches in all (prepare, forward, backward, finish).
 *
 * qk_pz_forward and qk_pz_backward each begin with a set-up kernel that turns the parameters into per-edge
 * constants (sin/cos of theta, merged phases, postact_weights * mask, base_weight * mask, the folded bias vector): work the
 * reference redoes inside every CTA (src/qkan/csrc/cute_kernels.cu:96-140, its shared-memory trig cache).
 * A caller that runs forward and backward with unchanged parameters - every training step does - can build
 * that state once with qk_pz_prepare into a buffer of qk_tables_bytes() bytes (depends on in_dim, out_dim,
 * reps, ansatz, flags, group; not on batch) and pass it to both *_prepared calls. The buffer is valid until a
 * parameter value changes. qk_backward_scratch_bytes() is the backward's scratch without the tables.
 * `with_base_term` must be non-zero exactly when qk_pz_prepare was given a base_weight.
 * postact_weights / postact_bias / mask are read again by the backward's finishing kernel.
 */
size_t qk_tables_bytes(const QkDesc* desc);
size_t qk_backward_scratch_bytes(const QkDesc* desc);

int qk_pz_prepare(const QkDesc* desc, const float* theta, const float* preacts_weight,
                  const float* preacts_bias, const void* postact_weights, const void* postact_bias,
                  const void* base_weight, const void* mask, void* tables, size_t tables_bytes,
                  void* cuda_stream);

int qk_pz_forward_prepared(const QkDesc* desc, const void* x, const void* tables, size_t tables_bytes,
                           int with_base_term, void* y, void* cuda_stream);

int qk_pz_backward_prepared(const QkDesc* desc, const void* x, const void* tables, size_t tables_bytes,
                            const void* postact_weights, const void* postact_bias, const void* mask,
                            int with_base_term, const void* grad_y, void* grad_x, float* grad_theta,
                            float* grad_preacts_weight, float* grad_preacts_bias,
                            float* grad_postact_weights, float* grad_postact_bias, float* grad_base_weight,
                            void* scratch, size_t scratch_bytes, void* cuda_stream);

/*
 * Per-edge activation scale: edge_std[o,i] = unbiased standard deviation over the batch of the edge output
 *   (postacts[b,o,i] + postact_bias[o,i]) * postact_weights[o,i] * mask[o,i] + silu(x[b,i]) * base_weight[o,i] * mask[o,i]
 * i.e. torch.std(QKANLayer.forward_no_sum(x), dim=0) of the reference (src/qkan/qkan.py:835-891), which its
 * save_act pass computes for the activation-scale regulariser and pruning (src/qkan/qkan.py:1280-1302). The
 * (B,O,I) tensor is never formed: per-tile sums of the shifted values and their squares are reduced in a fixed
 * order. `tables` comes from qk_pz_prepare with the same parameters; edge_std is float32 (O,I); fewer than two
 * rows give NaN as torch.std does.
 */
size_t qk_edge_stats_scratch_bytes(const QkDesc* desc);
int qk_pz_edge_stats(const QkDesc* desc, const void* x, const void* tables, size_t tables_bytes,
                     int with_base_term, float* edge_std, void* scratch, size_t scratch_bytes,
                     void* cuda_stream);

/*
 * Solver plug-in contract (src/qkan/solver/_base.py:29-51, call site
 * src/qkan/qkan.py:699-714): per-edge activations postacts (B,O,I) in
 * io_dtype, and the matching backward from grad_postacts (B,O,I). Used by
 * forward_no_sum / save_act (src/qkan/qkan.py:835-891, 1280-1302) and when
 * the kernels are registered as a solver inside the reference's own layer.
 */
int qk_pz_postacts_forward(const QkDesc* desc, const void* x, const float* theta,
                           const float* preacts_weight, const float* preacts_bias,
                           void* postacts, void* workspace, size_t workspace_bytes,
                           void* cuda_stream);

int qk_pz_postacts_backward(const QkDesc* desc, const void* x, const float* theta,
                            const float* preacts_weight, const float* preacts_bias,
                            const void* grad_postacts, void* grad_x, float* grad_theta,
                            float* grad_preacts_weight, float* grad_preacts_bias,
                            void* workspace, size_t workspace_bytes, void* cuda_stream);

/*
 * Forward for callers that cannot allocate device memory (no counterpart in the
 * reference; it exists for the hosts this library is embedded in).
 *
 * Who needs it: a process whose device memory is wholly owned by another
 * runtime's pool, or a serving loop in which cudaMalloc - a call that
 * synchronises the whole device - is banned after start-up. Such a caller has
 * no workspace to pass, so this variant of qk_pz_forward keeps its scratch in a
 * fixed array that is part of the library image: qk_noalloc_max_scratch_bytes()
 * bytes (8 MiB) of device memory on every GPU that loads the library, held
 * until the process exits. The call itself allocates nothing and frees nothing.
 *
 * Limits and rules:
 *  - the problem must satisfy qk_forward_workspace_bytes(desc) <=
 *    qk_noalloc_max_scratch_bytes(); larger ones return QK_ERR_WORKSPACE and
 *    qk_noalloc_last_error() says how many bytes were needed;
 *  - the first call on each device looks the array's address up (a one-time
 *    runtime query); make that first call during start-up, before any stream
 *    capture is begun;
 *  - all calls on a device share the one array and it keeps whatever the last
 *    call left there. The forward rewrites everything it reads, so no clearing
 *    is needed, but two calls that can overlap on the GPU (different streams
 *    with no ordering between them) race on it: keep them on one stream or
 *    order them with events.
 * Inputs, outputs and results are those of qk_pz_forward.
 */
size_t qk_noalloc_max_scratch_bytes(void);
const char* qk_noalloc_last_error(void);
int qk_pz_forward_noalloc(const QkDesc* desc, const void* x, const float* theta,
                          const float* preacts_weight, const float* preacts_bias,
                          const void* postact_weights, const void* postact_bias,
                          const void* base_weight, const void* mask, void* y, void* cuda_stream);

/*
 * Developer overrides of the tile choice, process-wide; no counterpart in the reference (its batch-tile
 * heuristic, src/qkan/_kernel_utils.py:18-31, is fixed). 0 restores the library's own choice. On first use the
 * values are seeded once from the environment variables QK_BWD_GROUPS, QK_BWD_RPG, QK_BWD_RU, QK_BWD_OSPLIT,
 * QK_NO_XTRIG, QK_DEBUG, QK_FWD_THREADS, QK_FWD_TB, QK_FWD_OT and QK_FWD_ICH; the launch path itself never reads the
 * environment. Workspace sizes depend on the
 * tile choice: query them after setting an override, and do not change one between a size query and its call.
 */
enum QkDebugKey {
    QK_DBG_BWD_GROUPS = 0, /* warps (row groups) per backward CTA; needs QK_DBG_BWD_RPG too */
    QK_DBG_BWD_RPG = 1,    /* rows per group */
    QK_DBG_BWD_RU = 2,     /* rows a thread keeps in flight (2 or 4) */
    QK_DBG_BWD_OSPLIT = 3, /* output slices of the backward (grid.z) */
    QK_DBG_NO_XTRIG = 4,   /* non-zero: frozen-preact forward uses the generic kernel */
    QK_DBG_VERBOSE = 5,    /* non-zero: print the chosen tiles to stderr */
    QK_DBG_FWD_THREADS = 6, /* threads per forward CTA (multiple of 32, <= 512); needs the next two as well */
    QK_DBG_FWD_TB = 7,      /* batch rows per forward CTA (multiple of 32) */
    QK_DBG_FWD_OT = 8,      /* outputs per forward CTA */
    QK_DBG_FWD_ICH = 9      /* input columns the forward stages at a time (256, 128 or 64) */
};
void qk_debug_set(int key, int value);

#ifdef __cplusplus
}
#endif
#endif /* QKAN_B200_H_ */
