// C ABI of the library (see include/qkan_b200.h): argument validation,
// workspace carving and the kernel launch sequence. No torch types, no
// allocation, no synchronisation. A layer step is four launches: set-up (tables + bias), forward,
// backward, gradient finish (one more with the base term on, one more per sliced / grouped extra).
#include <cstdarg>
#include <cstdio>
#include <cstdlib>

#include "qk_kernels.cuh"

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int check_desc(const QkDesc* d) {
    if (!d) return fail(QK_ERR_BAD_ARGUMENT, "desc is NULL");
    if (d->batch < 0 || d->in_dim < 0 || d->out_dim < 0)
        return fail(QK_ERR_BAD_ARGUMENT, "negative dimension (B=%d I=%d O=%d)", d->batch, d->in_dim,
                    d->out_dim);
    if (d->reps < 1) return fail(QK_ERR_BAD_ARGUMENT, "reps must be >= 1 (got %d)", d->reps);
    if (d->reps > qk::kMaxReps)
        return fail(QK_ERR_UNSUPPORTED, "reps=%d exceeds the compiled maximum of %d", d->reps,
                    qk::kMaxReps);
    if (d->ansatz != QK_ANSATZ_PZ && d->ansatz != QK_ANSATZ_RPZ && d->ansatz != QK_ANSATZ_REAL)
        return fail(QK_ERR_BAD_ARGUMENT, "ansatz %d is not a QkAnsatz value", d->ansatz);
    if (d->io_dtype != QK_F32 && d->io_dtype != QK_BF16)
        return fail(QK_ERR_BAD_ARGUMENT, "io_dtype %d is neither QK_F32 nor QK_BF16", d->io_dtype);
    if (d->param_dtype != QK_F32 && d->param_dtype != QK_BF16)
        return fail(QK_ERR_BAD_ARGUMENT, "param_dtype %d is neither QK_F32 nor QK_BF16",
                    d->param_dtype);
    if (d->flags & ~(QK_PREACT_TRAINABLE | QK_FAST_MEASURE | QK_USE_POSTACT_BIAS | QK_PRECISE_MATH | QK_SINGLE_TABLE))
        return fail(QK_ERR_BAD_ARGUMENT, "unknown flag bits 0x%x", d->flags);
    if (d->group < 0) return fail(QK_ERR_BAD_ARGUMENT, "group must be >= 0 (got %d)", d->group);
    if (d->group > 65535) return fail(QK_ERR_UNSUPPORTED, "group %d exceeds 65535", d->group);
    if ((long long)d->out_dim > 65535)
        return fail(QK_ERR_UNSUPPORTED, "out_dim %d exceeds 65535", d->out_dim);
    return QK_OK;
}

// Forward with frozen preacts of the pz circuit: data angles are x + const and are evaluated by angle
// addition from (cos x, sin x) staged once per tile. Not combined with QK_PRECISE_MATH or with padded
// (> 8) circuits. (The same form was measured for the backward and was 3-5 % slower there: the backward is
// bound by issue slots, not by the special-function unit, so it keeps the generic kernel.)
bool use_xtrig(const QkDesc& d) {
    const int rk = qk::compiled_reps(d.ansatz, d.reps);
    return d.ansatz == QK_ANSATZ_PZ && !(d.flags & (QK_PREACT_TRAINABLE | QK_PRECISE_MATH | QK_SINGLE_TABLE)) &&
           rk >= 1 && rk <= 8 && !qk::debug_get(qk::kDbgNoXtrig);
}

// The prepared state of a layer: per-edge constant table, folded bias vector and, for the frozen-preact
// forward, that kernel's own table. Depends on the layer's shape and flags only, not on the batch.
struct Tables {
    int ipad;
    bool xtrig;
    size_t table_off, bias_off, tablex_off, basew_off, total;
};

// Scratch of one backward call: per-tile column sums of grad_y, per-tile gradient partials, the base-term
// kernel's partials, the grad_x shares of sliced launches, per-edge gradients ahead of a group reduction.
struct Scratch {
    qk::BwdCfg cfg;
    int base_tiles;
    size_t colpart_off, partials_off, basepart_off, gxpart_off, gtheta_off, gpw_off, gpb_off, total;
};

size_t theta_per_entry(const QkDesc& d) {
    return d.ansatz == QK_ANSATZ_PZ ? (size_t)(d.reps + 1) * 2
                                    : (d.ansatz == QK_ANSATZ_RPZ ? (size_t)d.reps + 1 : (size_t)d.reps);
}

Tables tables_layout(const QkDesc& d) {
    Tables l{};
    l.ipad = qk::round_up(d.in_dim, 32);
    l.xtrig = use_xtrig(d);
    const size_t table =
        qk::align256((size_t)d.out_dim * qk::table_stride(qk::compiled_reps(d.ansatz, d.reps)) * l.ipad * sizeof(float));
    l.table_off = 0;
    l.bias_off = table;
    l.total = l.bias_off + qk::align256((size_t)d.out_dim * sizeof(float));
    if (l.xtrig) {
        l.tablex_off = l.total;
        l.total += table;
    }
    // base_weight * mask once more as a dense [out_dim][ipad] matrix (operand of the base-term backward)
    l.basew_off = l.total;
    l.total += qk::align256((size_t)d.out_dim * l.ipad * sizeof(float));
    return l;
}

Scratch scratch_layout(const QkDesc& d) {
    Scratch l{};
    const int ipad = qk::round_up(d.in_dim, 32);
    l.cfg = qk::choose_bwd_cfg(d);
    l.colpart_off = 0;
    l.partials_off = qk::align256((size_t)l.cfg.grid_b * d.out_dim * sizeof(float));
    l.total = l.partials_off + qk::align256((size_t)l.cfg.grid_b * d.out_dim * l.cfg.nacc * ipad * sizeof(float));
    l.base_tiles = qk::base_plan(d.batch, d.in_dim, d.out_dim).slabs;
    l.basepart_off = l.total;
    l.total += qk::align256((size_t)l.base_tiles * d.out_dim * ipad * sizeof(float));
    if (l.cfg.osplit > 1) {
        l.gxpart_off = l.total;
        l.total += qk::align256((size_t)l.cfg.osplit * d.batch * d.in_dim * sizeof(float));
    }
    if (d.group > 0) {
        const size_t nE = (size_t)d.out_dim * d.in_dim;
        l.gtheta_off = l.total;
        l.gpw_off = l.gtheta_off + qk::align256(nE * theta_per_entry(d) * sizeof(float));
        l.gpb_off = l.gpw_off + qk::align256(nE * d.reps * sizeof(float));
        l.total = l.gpb_off + qk::align256(nE * d.reps * sizeof(float));
    }
    return l;
}

bool empty(const QkDesc& d) { return d.batch == 0 || d.in_dim == 0 || d.out_dim == 0; }
// the prepared state has no batch axis: only a layer without edges has nothing to prepare
bool no_edges(const QkDesc& d) { return d.in_dim == 0 || d.out_dim == 0; }

int cuda_fail(cudaError_t e, const char* what) {
    return fail(QK_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
}

int check_buffer(const void* p, size_t have, size_t need, const char* what) {
    if (!p || have < need)
        return fail(QK_ERR_WORKSPACE, "%s too small: need %zu bytes, got %zu", what, need, p ? have : (size_t)0);
    if ((uintptr_t)p % 256) return fail(QK_ERR_WORKSPACE, "%s must be 256-byte aligned", what);
    return QK_OK;
}

// `edges`: solver-contract mode (no epilogue: weight 1, no bias, no base term, no mask)
int run_prepare(const QkDesc* desc, const float* theta, const float* pw, const float* pb, const void* postw,
                const void* postb, const void* basew, const void* mask, bool edges, void* tables,
                size_t tables_bytes, cudaStream_t st) {
    int rc = check_desc(desc);
    if (rc) return rc;
    const QkDesc& d = *desc;
    if (no_edges(d)) return QK_OK;
    if (!theta || !pw || !pb) return fail(QK_ERR_BAD_ARGUMENT, "theta/preacts pointer is NULL");
    if (!edges && !postw) return fail(QK_ERR_BAD_ARGUMENT, "postact_weights is NULL");
    const Tables l = tables_layout(d);
    rc = check_buffer(tables, tables_bytes, l.total, "tables");
    if (rc) return rc;
    char* tb = static_cast<char*>(tables);
    qk::PrepArgs p{};
    p.in_dim = d.in_dim;
    p.out_dim = d.out_dim;
    p.reps = d.reps;
    p.rk = qk::compiled_reps(d.ansatz, d.reps);
    p.ansatz = d.ansatz;
    p.ipad = l.ipad;
    p.flags = d.flags;
    p.param_dtype = d.param_dtype;
    p.group = d.group;
    p.theta = theta;
    p.pw = pw;
    p.pb = pb;
    p.postw = edges ? nullptr : postw;
    p.postb = edges ? nullptr : postb;
    p.basew = edges ? nullptr : basew;
    p.mask = edges ? nullptr : mask;
    p.table = reinterpret_cast<float*>(tb + l.table_off);
    p.table_x = l.xtrig ? reinterpret_cast<float*>(tb + l.tablex_off) : nullptr;
    p.bias = edges ? nullptr : reinterpret_cast<float*>(tb + l.bias_off);
    p.basew_c = p.basew ? reinterpret_cast<float*>(tb + l.basew_off) : nullptr;
    cudaError_t e = qk::launch_prep(p, st);
    if (e != cudaSuccess) return cuda_fail(e, "prep launch");
    return QK_OK;
}

int run_forward_prepared(const QkDesc* desc, const void* x, const void* tables, size_t tables_bytes,
                         bool has_base, void* y, void* postacts, cudaStream_t st) {
    int rc = check_desc(desc);
    if (rc) return rc;
    const QkDesc& d = *desc;
    const bool edges = postacts != nullptr;
    if (empty(d)) {
        // y (B,O) of an in_dim == 0 layer is all zeros; the other empty shapes have no output
        if (!edges && d.in_dim == 0 && d.batch > 0 && d.out_dim > 0 && y) {
            size_t es = d.io_dtype == QK_BF16 ? 2 : 4;
            cudaError_t e = cudaMemsetAsync(y, 0, (size_t)d.batch * d.out_dim * es, st);
            if (e != cudaSuccess) return cuda_fail(e, "memset y");
        }
        return QK_OK;
    }
    if (!x) return fail(QK_ERR_BAD_ARGUMENT, "x is NULL");
    if (!edges && !y) return fail(QK_ERR_BAD_ARGUMENT, "y is NULL");
    const Tables l = tables_layout(d);
    rc = check_buffer(tables, tables_bytes, l.total, "tables");
    if (rc) return rc;
    const char* tb = static_cast<const char*>(tables);
    has_base = has_base && !edges;

    qk::FwdArgs f{};
    f.batch = d.batch;
    f.in_dim = d.in_dim;
    f.out_dim = d.out_dim;
    f.ipad = l.ipad;
    f.precise = (d.flags & QK_PRECISE_MATH) != 0;
    f.xtrig = l.xtrig;
    f.cfg = qk::choose_fwd_cfg(d, edges, has_base, l.xtrig);
    if (qk::debug_get(qk::kDbgVerbose))
        fprintf(stderr, "[qk] forward B=%d I=%d O=%d R=%d: tile %d rows x %d outputs, grid %d x %d, smem %zu\n",
                d.batch, d.in_dim, d.out_dim, d.reps, f.cfg.tb, f.cfg.ot, f.cfg.grid_b, f.cfg.grid_o, f.cfg.smem);
    f.x = x;
    f.table = reinterpret_cast<const float*>(tb + (l.xtrig ? l.tablex_off : l.table_off));
    f.bias = reinterpret_cast<const float*>(tb + l.bias_off);
    f.y = y;
    f.postacts = postacts;
    cudaError_t e = qk::launch_forward(f, qk::compiled_reps(d.ansatz, d.reps), (d.flags & QK_FAST_MEASURE) != 0,
                                       d.io_dtype, has_base, st);
    if (e != cudaSuccess) return cuda_fail(e, "forward launch");
    return QK_OK;
}

int run_backward_prepared(const QkDesc* desc, const void* x, const void* tables, size_t tables_bytes,
                          const void* postw, const void* postb, const void* mask, bool has_base,
                          const void* gy, const void* gpostacts, void* gx, float* gtheta, float* gpw,
                          float* gpb, float* gpostw, float* gpostb, float* gbasew, void* scratch,
                          size_t scratch_bytes, cudaStream_t st) {
    int rc = check_desc(desc);
    if (rc) return rc;
    const QkDesc& d = *desc;
    const bool edges = gpostacts != nullptr;
    const size_t nE = (size_t)d.out_dim * d.in_dim;
    if (empty(d)) {
        // no rows (or no edges): every requested gradient is zero
        cudaError_t e = cudaSuccess;
        size_t es = d.io_dtype == QK_BF16 ? 2 : 4;
        if (gx && (size_t)d.batch * d.in_dim) e = cudaMemsetAsync(gx, 0, (size_t)d.batch * d.in_dim * es, st);
        const size_t nQ = d.group > 0 ? (size_t)d.group : nE;  // entries of theta / preacts
        if (e == cudaSuccess && gtheta && nQ) e = cudaMemsetAsync(gtheta, 0, nQ * theta_per_entry(d) * 4, st);
        if (e == cudaSuccess && gpw && nQ) e = cudaMemsetAsync(gpw, 0, nQ * d.reps * 4, st);
        if (e == cudaSuccess && gpb && nQ) e = cudaMemsetAsync(gpb, 0, nQ * d.reps * 4, st);
        if (e == cudaSuccess && gpostw && nE) e = cudaMemsetAsync(gpostw, 0, nE * 4, st);
        if (e == cudaSuccess && gpostb && nE) e = cudaMemsetAsync(gpostb, 0, nE * 4, st);
        if (e == cudaSuccess && gbasew && nE) e = cudaMemsetAsync(gbasew, 0, nE * 4, st);
        if (e != cudaSuccess) return cuda_fail(e, "memset gradients");
        return QK_OK;
    }
    if (!x) return fail(QK_ERR_BAD_ARGUMENT, "x is NULL");
    if (!edges && (!postw || !gy)) return fail(QK_ERR_BAD_ARGUMENT, "postact_weights or grad_y is NULL");
    has_base = has_base && !edges;
    const Tables tl = tables_layout(d);
    rc = check_buffer(tables, tables_bytes, tl.total, "tables");
    if (rc) return rc;
    const Scratch l = scratch_layout(d);
    rc = check_buffer(scratch, scratch_bytes, l.total, "workspace");
    if (rc) return rc;
    const float* table = reinterpret_cast<const float*>(static_cast<const char*>(tables) + tl.table_off);
    char* wsb = static_cast<char*>(scratch);
    const int rk = qk::compiled_reps(d.ansatz, d.reps);

    const bool use_pb = !edges && (d.flags & QK_USE_POSTACT_BIAS) && postb;
    const bool need_colsum = use_pb && (gpostw || gpostb);
    float* colpart = reinterpret_cast<float*>(wsb + l.colpart_off);

    qk::BwdArgs b{};
    b.batch = d.batch;
    b.in_dim = d.in_dim;
    b.out_dim = d.out_dim;
    b.ipad = tl.ipad;
    b.precise = (d.flags & QK_PRECISE_MATH) != 0;
    b.cfg = l.cfg;
    if (qk::debug_get(qk::kDbgVerbose))
        fprintf(stderr, "[qk] backward B=%d I=%d O=%d R=%d: %d groups x %d rows, grid %d x %d x %d output slices of %d, smem %zu, ru %d\n",
                d.batch, d.in_dim, d.out_dim, d.reps, b.cfg.groups, b.cfg.rpg, b.cfg.grid_b, b.cfg.grid_i,
                b.cfg.osplit, b.cfg.ochunk, b.cfg.smem, b.cfg.ru);
    b.x = x;
    b.gy = gy;
    b.gpostacts = gpostacts;
    b.table = table;
    b.gx = gx;
    b.gx_part = b.cfg.osplit > 1 ? reinterpret_cast<float*>(wsb + l.gxpart_off) : nullptr;
    b.partials = reinterpret_cast<float*>(wsb + l.partials_off);
    b.colpart = need_colsum ? colpart : nullptr;
    cudaError_t e = qk::launch_backward(b, rk, (d.flags & QK_FAST_MEASURE) != 0, d.io_dtype, st);
    if (e != cudaSuccess) return cuda_fail(e, "backward launch");
    if (gx && b.cfg.osplit > 1) {
        e = qk::launch_sum_gx(b.gx_part, gx, d.io_dtype, (size_t)d.batch * d.in_dim, b.cfg.osplit, st);
        if (e != cudaSuccess) return cuda_fail(e, "grad_x slice sum launch");
    }
    // base term: its two contractions run as a kernel of their own and add their part of grad_x in place
    float* base_partials = reinterpret_cast<float*>(wsb + l.basepart_off);
    const bool base_pass = has_base && (gx || gbasew);
    if (base_pass) {
        qk::BaseBwdArgs ba{};
        ba.batch = d.batch;
        ba.in_dim = d.in_dim;
        ba.out_dim = d.out_dim;
        ba.ipad = tl.ipad;
        ba.x = x;
        ba.gy = gy;
        ba.basew = reinterpret_cast<const float*>(static_cast<const char*>(tables) + tl.basew_off);
        ba.gx = gx;
        ba.partials = gbasew ? base_partials : nullptr;
        e = qk::launch_base_backward(ba, d.io_dtype, st);
        if (e != cudaSuccess) return cuda_fail(e, "base-term backward launch");
    }

    if (gtheta || gpw || gpb || gpostw || gpostb || gbasew) {
        qk::FinishArgs f{};
        f.in_dim = d.in_dim;
        f.out_dim = d.out_dim;
        f.reps = d.reps;
        f.rk = rk;
        f.ansatz = d.ansatz;
        f.ipad = tl.ipad;
        f.nacc = b.cfg.nacc;
        f.ntiles = b.cfg.grid_b;
        f.base_tiles = has_base && gbasew ? l.base_tiles : 0;
        f.base_partials = f.base_tiles ? base_partials : nullptr;
        f.flags = d.flags;
        f.param_dtype = d.param_dtype;
        f.partials = b.partials;
        f.colpart = need_colsum ? colpart : nullptr;
        f.postw = edges ? nullptr : postw;
        f.postb = edges ? nullptr : postb;
        f.mask = edges ? nullptr : mask;
        // grouped parameters: per-edge gradients go to scratch and are summed per entry afterwards
        const bool grouped = d.group > 0;
        f.gtheta = grouped && gtheta ? reinterpret_cast<float*>(wsb + l.gtheta_off) : gtheta;
        f.gpw = grouped && gpw ? reinterpret_cast<float*>(wsb + l.gpw_off) : gpw;
        f.gpb = grouped && gpb ? reinterpret_cast<float*>(wsb + l.gpb_off) : gpb;
        f.gpostw = edges ? nullptr : gpostw;
        f.gpostb = edges ? nullptr : gpostb;
        f.gbasew = edges ? nullptr : gbasew;
        e = qk::launch_finish(f, st);
        if (e != cudaSuccess) return cuda_fail(e, "finish launch");
        if (grouped) {
            const int per_theta = (int)theta_per_entry(d);
            if (gtheta) e = qk::launch_group_reduce(f.gtheta, gtheta, d.out_dim, d.in_dim, d.group, per_theta, st);
            if (e == cudaSuccess && gpw)
                e = qk::launch_group_reduce(f.gpw, gpw, d.out_dim, d.in_dim, d.group, d.reps, st);
            if (e == cudaSuccess && gpb)
                e = qk::launch_group_reduce(f.gpb, gpb, d.out_dim, d.in_dim, d.group, d.reps, st);
            if (e != cudaSuccess) return cuda_fail(e, "group reduction launch");
        }
    }
    return QK_OK;
}

// one-workspace entry points: [tables | scratch]
int run_forward(const QkDesc* desc, const void* x, const float* theta, const float* pw, const float* pb,
                const void* postw, const void* postb, const void* basew, const void* mask, void* y,
                void* postacts, void* ws, size_t ws_bytes, cudaStream_t st) {
    int rc = check_desc(desc);
    if (rc) return rc;
    const bool edges = postacts != nullptr;
    if (!empty(*desc)) {
        if (!x || !theta || !pw || !pb) return fail(QK_ERR_BAD_ARGUMENT, "x/theta/preacts pointer is NULL");
        if (!edges && (!postw || !y)) return fail(QK_ERR_BAD_ARGUMENT, "postact_weights or y is NULL");
        rc = check_buffer(ws, ws_bytes, tables_layout(*desc).total, "workspace");
        if (rc) return rc;
        rc = run_prepare(desc, theta, pw, pb, postw, postb, basew, mask, edges, ws, ws_bytes, st);
        if (rc) return rc;
    }
    return run_forward_prepared(desc, x, ws, ws_bytes, basew != nullptr, y, postacts, st);
}

int run_backward(const QkDesc* desc, const void* x, const float* theta, const float* pw, const float* pb,
                 const void* postw, const void* postb, const void* basew, const void* mask, const void* gy,
                 const void* gpostacts, void* gx, float* gtheta, float* gpw, float* gpb, float* gpostw,
                 float* gpostb, float* gbasew, void* ws, size_t ws_bytes, cudaStream_t st) {
    int rc = check_desc(desc);
    if (rc) return rc;
    const bool edges = gpostacts != nullptr;
    size_t toff = 0;
    if (!empty(*desc)) {
        if (!x || !theta || !pw || !pb) return fail(QK_ERR_BAD_ARGUMENT, "x/theta/preacts pointer is NULL");
        if (!edges && (!postw || !gy)) return fail(QK_ERR_BAD_ARGUMENT, "postact_weights or grad_y is NULL");
        toff = tables_layout(*desc).total;
        const size_t need = toff + scratch_layout(*desc).total;
        rc = check_buffer(ws, ws_bytes, need, "workspace");
        if (rc) return rc;
        rc = run_prepare(desc, theta, pw, pb, postw, postb, basew, mask, edges, ws, toff, st);
        if (rc) return rc;
    }
    return run_backward_prepared(desc, x, ws, toff, postw, postb, mask, basew != nullptr, gy, gpostacts, gx,
                                 gtheta, gpw, gpb, gpostw, gpostb, gbasew,
                                 ws ? static_cast<char*>(ws) + toff : nullptr, ws_bytes >= toff ? ws_bytes - toff : 0,
                                 st);
}

}  // namespace

extern "C" {

int qk_abi_version(void) { return QK_ABI_VERSION; }

const char* qk_last_error(void) { return g_err; }

size_t qk_forward_workspace_bytes(const QkDesc* desc) {
    if (check_desc(desc)) return 0;
    if (empty(*desc)) return 256;
    return tables_layout(*desc).total;
}

size_t qk_backward_workspace_bytes(const QkDesc* desc) {
    if (check_desc(desc)) return 0;
    if (empty(*desc)) return 256;
    return tables_layout(*desc).total + scratch_layout(*desc).total;
}

size_t qk_tables_bytes(const QkDesc* desc) {
    if (check_desc(desc)) return 0;
    if (no_edges(*desc)) return 256;
    return tables_layout(*desc).total;
}

size_t qk_backward_scratch_bytes(const QkDesc* desc) {
    if (check_desc(desc)) return 0;
    if (empty(*desc)) return 256;
    return scratch_layout(*desc).total;
}

int qk_pz_prepare(const QkDesc* desc, const float* theta, const float* pw, const float* pb,
                  const void* postw, const void* postb, const void* basew, const void* mask, void* tables,
                  size_t tables_bytes, void* stream) {
    return run_prepare(desc, theta, pw, pb, postw, postb, basew, mask, false, tables, tables_bytes,
                       static_cast<cudaStream_t>(stream));
}

int qk_pz_forward_prepared(const QkDesc* desc, const void* x, const void* tables, size_t tables_bytes,
                           int with_base_term, void* y, void* stream) {
    return run_forward_prepared(desc, x, tables, tables_bytes, with_base_term != 0, y, nullptr,
                                static_cast<cudaStream_t>(stream));
}

int qk_pz_backward_prepared(const QkDesc* desc, const void* x, const void* tables, size_t tables_bytes,
                            const void* postw, const void* postb, const void* mask, int with_base_term,
                            const void* gy, void* gx, float* gtheta, float* gpw, float* gpb, float* gpostw,
                            float* gpostb, float* gbasew, void* scratch, size_t scratch_bytes, void* stream) {
    return run_backward_prepared(desc, x, tables, tables_bytes, postw, postb, mask, with_base_term != 0, gy,
                                 nullptr, gx, gtheta, gpw, gpb, gpostw, gpostb, gbasew, scratch, scratch_bytes,
                                 static_cast<cudaStream_t>(stream));
}

size_t qk_edge_stats_scratch_bytes(const QkDesc* desc) {
    if (check_desc(desc)) return 0;
    if (empty(*desc)) return 256;
    return qk::stats_scratch_bytes(desc->batch, desc->in_dim, desc->out_dim);
}

int qk_pz_edge_stats(const QkDesc* desc, const void* x, const void* tables, size_t tables_bytes,
                     int with_base_term, float* edge_std, void* scratch, size_t scratch_bytes, void* stream) {
    int rc = check_desc(desc);
    if (rc) return rc;
    const QkDesc& d = *desc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (no_edges(d)) return QK_OK;
    if (!edge_std) return fail(QK_ERR_BAD_ARGUMENT, "edge_std is NULL");
    if (d.batch == 0) {  // the deviation of no rows is not a number, as torch.std answers
        cudaError_t e = cudaMemsetAsync(edge_std, 0xff, (size_t)d.out_dim * d.in_dim * sizeof(float), st);
        if (e != cudaSuccess) return cuda_fail(e, "memset edge_std");
        return QK_OK;
    }
    if (!x) return fail(QK_ERR_BAD_ARGUMENT, "x is NULL");
    const Tables tl = tables_layout(d);
    rc = check_buffer(tables, tables_bytes, tl.total, "tables");
    if (rc) return rc;
    rc = check_buffer(scratch, scratch_bytes, qk::stats_scratch_bytes(d.batch, d.in_dim, d.out_dim), "workspace");
    if (rc) return rc;
    cudaError_t e = qk::launch_edge_stats(
        x, d.io_dtype, reinterpret_cast<const float*>(static_cast<const char*>(tables) + tl.table_off), d.batch,
        d.in_dim, d.out_dim, qk::compiled_reps(d.ansatz, d.reps), (d.flags & QK_FAST_MEASURE) != 0,
        with_base_term != 0, edge_std, static_cast<float*>(scratch), st);
    if (e != cudaSuccess) return cuda_fail(e, "edge statistics launch");
    return QK_OK;
}

void qk_debug_set(int key, int value) { qk::debug_set(key, value); }

int qk_pz_forward(const QkDesc* desc, const void* x, const float* theta, const float* pw,
                  const float* pb, const void* postw, const void* postb, const void* basew,
                  const void* mask, void* y, void* ws, size_t ws_bytes, void* stream) {
    return run_forward(desc, x, theta, pw, pb, postw, postb, basew, mask, y, nullptr, ws, ws_bytes,
                       static_cast<cudaStream_t>(stream));
}

int qk_pz_backward(const QkDesc* desc, const void* x, const float* theta, const float* pw,
                   const float* pb, const void* postw, const void* postb, const void* basew,
                   const void* mask, const void* gy, void* gx, float* gtheta, float* gpw,
                   float* gpb, float* gpostw, float* gpostb, float* gbasew, void* ws,
                   size_t ws_bytes, void* stream) {
    return run_backward(desc, x, theta, pw, pb, postw, postb, basew, mask, gy, nullptr, gx, gtheta,
                        gpw, gpb, gpostw, gpostb, gbasew, ws, ws_bytes,
                        static_cast<cudaStream_t>(stream));
}

int qk_pz_postacts_forward(const QkDesc* desc, const void* x, const float* theta, const float* pw,
                           const float* pb, void* postacts, void* ws, size_t ws_bytes,
                           void* stream) {
    if (!postacts && desc && !empty(*desc)) return fail(QK_ERR_BAD_ARGUMENT, "postacts is NULL");
    if (!postacts) return check_desc(desc);
    return run_forward(desc, x, theta, pw, pb, nullptr, nullptr, nullptr, nullptr, nullptr, postacts,
                       ws, ws_bytes, static_cast<cudaStream_t>(stream));
}

int qk_pz_postacts_backward(const QkDesc* desc, const void* x, const float* theta, const float* pw,
                            const float* pb, const void* gpostacts, void* gx, float* gtheta,
                            float* gpw, float* gpb, void* ws, size_t ws_bytes, void* stream) {
    if (!gpostacts && desc && !empty(*desc)) return fail(QK_ERR_BAD_ARGUMENT, "grad_postacts is NULL");
    if (!gpostacts) {
        // empty problem: zero the requested gradients through the common path
        static const char dummy = 0;
        return run_backward(desc, x, theta, pw, pb, nullptr, nullptr, nullptr, nullptr, nullptr,
                            &dummy, gx, gtheta, gpw, gpb, nullptr, nullptr, nullptr, ws, ws_bytes,
                            static_cast<cudaStream_t>(stream));
    }
    return run_backward(desc, x, theta, pw, pb, nullptr, nullptr, nullptr, nullptr, nullptr,
                        gpostacts, gx, gtheta, gpw, gpb, nullptr, nullptr, nullptr, ws, ws_bytes,
                        static_cast<cudaStream_t>(stream));
}

}  // extern "C"
