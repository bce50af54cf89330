// Tile-shape selection and the dispatch on the repetition count. The kernels
// themselves are instantiated once per R in qk_forward_inst.cu / qk_backward_inst.cu.
#include <cstdlib>

#include "qk_kernels.cuh"

namespace qk {

constexpr int kGyChunkHost = 8;  // must match kGyChunk of the backward kernel

// Developer tuning knob: integer environment override, read once per process.
static int tune_int(const char* name, int dflt) {
    const char* v = getenv(name);
    return v && *v ? atoi(v) : dflt;
}

template <int R>
cudaError_t launch_fwd_d(const FwdArgs& a, bool fast, int io_dtype, bool has_base, cudaStream_t st);
template <int R>
cudaError_t launch_bwd_d(const BwdArgs& a, bool fast, int io_dtype, bool has_base, cudaStream_t st);

#define QK_DECL(R)                                                                              \
    extern template cudaError_t launch_fwd_d<R>(const FwdArgs&, bool, int, bool, cudaStream_t); \
    extern template cudaError_t launch_bwd_d<R>(const BwdArgs&, bool, int, bool, cudaStream_t);
QK_DECL(1) QK_DECL(2) QK_DECL(3) QK_DECL(4) QK_DECL(5) QK_DECL(6) QK_DECL(7) QK_DECL(8)
#undef QK_DECL

FwdCfg choose_fwd_cfg(const QkDesc& d, bool edges, bool base) {
    FwdCfg c;
    const int ipad = round_up(d.in_dim, 32);
    c.threads = 512;
    c.ich = ipad < 256 ? ipad : 256;
    c.ot = d.out_dim < 256 ? d.out_dim : 256;
    c.tb = 64;
    // small problems: shrink the tile until the grid covers the machine twice
    auto ctas = [&](int tb, int ot) {
        return (long)((d.batch + tb - 1) / tb) * ((d.out_dim + ot - 1) / ot);
    };
    if (ctas(c.tb, c.ot) < 296) c.tb = 32;
    while (ctas(c.tb, c.ot) < 296 && c.ot > 16) c.ot = (c.ot + 1) / 2;
    c.grid_b = (d.batch + c.tb - 1) / c.tb;
    c.grid_o = (d.out_dim + c.ot - 1) / c.ot;
    // x tile + y tile + (with the base term) silu(x) tile
    c.smem = (size_t)c.tb * c.ich * 4 * (base ? 2 : 1) + (edges ? 0 : (size_t)c.ot * (c.tb + 1) * 4);
    return c;
}

BwdCfg choose_bwd_cfg(const QkDesc& d, bool base) {
    const int nacc = acc_rows(d.reps, base);
    const int grid_i = (d.in_dim + 31) / 32;
    const size_t budget = 200 * 1024;
    // (row groups = warps per CTA, rows per group), largest tile first; 8x32 runs two CTAs per SM
    static const int cand[][2] = {{8, 32}, {8, 16}, {4, 16}, {8, 8}, {4, 8}, {2, 8}, {1, 8}};
    BwdCfg best{};
    long best_ctas = -1;
    const int force_groups = tune_int("QK_BWD_GROUPS", 0), force_rpg = tune_int("QK_BWD_RPG", 0);
    if (force_groups > 0 && force_rpg > 0) {  // developer override of the tile shape
        const int tb = force_groups * force_rpg;
        size_t smem = (size_t)tb * 32 * 4 * (base ? 4 : 2) + (size_t)kGyChunkHost * tb * 4 +
                      (size_t)2 * force_groups * nacc * 32 * 4;
        return BwdCfg{force_groups, force_rpg, tb, (d.batch + tb - 1) / tb, grid_i, nacc, smem,
                      tune_int("QK_BWD_RU", 4)};
    }
    for (auto& c : cand) {
        const int groups = c[0], rpg = c[1], tb = groups * rpg;
        size_t smem = (size_t)tb * 32 * 4 * (base ? 4 : 2) + (size_t)kGyChunkHost * tb * 4 +
                      (size_t)2 * groups * nacc * 32 * 4;
        if (smem > budget) continue;
        const int grid_b = (d.batch + tb - 1) / tb;
        const long ctas = (long)grid_b * grid_i;
        BwdCfg cur{groups, rpg, tb, grid_b, grid_i, nacc, smem, tune_int("QK_BWD_RU", 4)};
        if (ctas >= 296) return cur;  // first (largest) tile that still fills the machine twice
        if (ctas > best_ctas) {
            best = cur;
            best_ctas = ctas;
        }
    }
    return best;
}


cudaError_t launch_forward(const FwdArgs& a, int reps, bool fast, int io_dtype, bool has_base,
                           cudaStream_t st) {
    switch (reps) {
        case 1: return launch_fwd_d<1>(a, fast, io_dtype, has_base, st);
        case 2: return launch_fwd_d<2>(a, fast, io_dtype, has_base, st);
        case 3: return launch_fwd_d<3>(a, fast, io_dtype, has_base, st);
        case 4: return launch_fwd_d<4>(a, fast, io_dtype, has_base, st);
        case 5: return launch_fwd_d<5>(a, fast, io_dtype, has_base, st);
        case 6: return launch_fwd_d<6>(a, fast, io_dtype, has_base, st);
        case 7: return launch_fwd_d<7>(a, fast, io_dtype, has_base, st);
        case 8: return launch_fwd_d<8>(a, fast, io_dtype, has_base, st);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_backward(const BwdArgs& a, int reps, bool fast, int io_dtype, bool has_base,
                            cudaStream_t st) {
    switch (reps) {
        case 1: return launch_bwd_d<1>(a, fast, io_dtype, has_base, st);
        case 2: return launch_bwd_d<2>(a, fast, io_dtype, has_base, st);
        case 3: return launch_bwd_d<3>(a, fast, io_dtype, has_base, st);
        case 4: return launch_bwd_d<4>(a, fast, io_dtype, has_base, st);
        case 5: return launch_bwd_d<5>(a, fast, io_dtype, has_base, st);
        case 6: return launch_bwd_d<6>(a, fast, io_dtype, has_base, st);
        case 7: return launch_bwd_d<7>(a, fast, io_dtype, has_base, st);
        case 8: return launch_bwd_d<8>(a, fast, io_dtype, has_base, st);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace qk
