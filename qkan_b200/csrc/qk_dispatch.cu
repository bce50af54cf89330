// Tile-shape selection and the dispatch on the repetition count. The kernels
// themselves are instantiated once per R in qk_forward_inst.cu / qk_backward_inst.cu.
#include <atomic>
#include <cstdlib>
#include <initializer_list>
#include <mutex>

#include "qk_kernels.cuh"

namespace qk {

constexpr int kGyChunkHost = 8;  // must match kGyChunk of the backward kernel

// Developer overrides of the tile choice (0 = none). They are process-wide values set through qk_debug_set;
// the first use seeds them, once, from the environment variables of the same names (QK_BWD_GROUPS, QK_BWD_RPG,
// QK_BWD_RU, QK_BWD_OSPLIT, QK_NO_XTRIG, QK_DEBUG, QK_FWD_THREADS, QK_FWD_TB, QK_FWD_OT, QK_FWD_ICH), so the launch path
// itself never reads the environment.
static std::atomic<int> g_debug[kDbgCount];
static std::once_flag g_debug_once;

static void debug_seed() {
    static const char* const names[kDbgCount] = {"QK_BWD_GROUPS", "QK_BWD_RPG", "QK_BWD_RU",
                                                 "QK_BWD_OSPLIT", "QK_NO_XTRIG", "QK_DEBUG",
                                                 "QK_FWD_THREADS", "QK_FWD_TB", "QK_FWD_OT", "QK_FWD_ICH"};
    for (int k = 0; k < kDbgCount; ++k) {
        const char* v = getenv(names[k]);
        g_debug[k].store(v && *v ? (atoi(v) != 0 ? atoi(v) : 1) : 0, std::memory_order_relaxed);
    }
}

int debug_get(int key) {
    std::call_once(g_debug_once, debug_seed);
    return key >= 0 && key < kDbgCount ? g_debug[key].load(std::memory_order_relaxed) : 0;
}

void debug_set(int key, int value) {
    std::call_once(g_debug_once, debug_seed);
    if (key >= 0 && key < kDbgCount) g_debug[key].store(value, std::memory_order_relaxed);
}

static int tune_int(int key, int dflt) {
    const int v = debug_get(key);
    return v > 0 ? v : dflt;
}

template <int R>
cudaError_t launch_fwd_d(const FwdArgs& a, bool fast, int io_dtype, bool has_base, cudaStream_t st);
template <int R>
cudaError_t launch_bwd_d(const BwdArgs& a, bool fast, int io_dtype, cudaStream_t st);

#define QK_DECL(R)                                                                              \
    extern template cudaError_t launch_fwd_d<R>(const FwdArgs&, bool, int, bool, cudaStream_t); \
    extern template cudaError_t launch_bwd_d<R>(const BwdArgs&, bool, int, cudaStream_t);
QK_DECL(0) QK_DECL(1) QK_DECL(2) QK_DECL(3) QK_DECL(4) QK_DECL(5) QK_DECL(6) QK_DECL(7) QK_DECL(8) QK_DECL(12) QK_DECL(16)
#undef QK_DECL

constexpr int kSmCount = 148;
constexpr size_t kSmemPerSm = 227 * 1024;

// Tile shapes are chosen with a small cost model: the busiest SM gets ceil(CTAs / 148) CTAs, a
// CTA's time grows with the edges x rows it owns plus its per-edge set-up, and too few resident
// warps cannot keep the issue slots busy. The largest tile wins ties (fewest partials / re-reads).
FwdCfg choose_fwd_cfg(const QkDesc& d, bool edges, bool base, bool xtrig) {
    const int ipad = round_up(d.in_dim, 32);
    FwdCfg best{};
    double best_cost = -1.0;
    const int f_threads = tune_int(kDbgFwdThreads, 0), f_tb = tune_int(kDbgFwdTb, 0), f_ot = tune_int(kDbgFwdOt, 0);
    if (f_threads > 0 && f_tb > 0 && f_ot > 0) {  // developer override
        FwdCfg c{};
        c.threads = f_threads;
        const int ich_o = tune_int(kDbgFwdIch, 256);
        c.ich = ipad < ich_o ? ipad : ich_o;
        c.tb = round_up(f_tb, 32);
        c.ot = d.out_dim < f_ot ? d.out_dim : f_ot;
        c.grid_b = (d.batch + c.tb - 1) / c.tb;
        c.grid_o = (d.out_dim + c.ot - 1) / c.ot;
        c.smem = (size_t)c.tb * c.ich * 4 * ((xtrig ? 2 : 1) + (base ? 1 : 0)) + (edges ? 0 : (size_t)c.ot * (c.tb + 1) * 4);
        if (c.smem <= (size_t)kSmemCap) return c;
    }
    const int f_ich = tune_int(kDbgFwdIch, 0);
    for (int tb : {64, 32}) {
        // columns staged at a time: 256 unless the tile would not fit (the frozen-preact form stages two floats per
        // element and the base term a third), then 128 or 64, so that the 64-row tile stays available
        for (int ich_want : {256, 128, 64}) {
            if (f_ich > 0 && ich_want != f_ich) continue;
            if (ich_want < 256 && ipad <= ich_want) continue;  // same tile as the wider candidate
            for (int ot = 256; ot >= 1; ot /= 2) {
                FwdCfg c{};
                c.threads = 512;
                c.ich = ipad < ich_want ? ipad : ich_want;
                c.tb = tb;
                c.ot = d.out_dim < ot ? d.out_dim : ot;
                if (c.ot < 16 && c.ot < d.out_dim) continue;  // fewer outputs than warps: idle warps
                c.grid_b = (d.batch + tb - 1) / tb;
                c.grid_o = (d.out_dim + c.ot - 1) / c.ot;
                c.smem = (size_t)tb * c.ich * 4 * ((xtrig ? 2 : 1) + (base ? 1 : 0)) +
                         (edges ? 0 : (size_t)c.ot * (tb + 1) * 4);
                if (c.smem > 200 * 1024) continue;
                const long ctas = (long)c.grid_b * c.grid_o;
                const long per_sm = (ctas + kSmCount - 1) / kSmCount;  // one CTA of 16 warps per SM at a time
                // constant loads per (o, 32 columns); warps that own a single output each stay in step
                // between barriers and expose that load latency together
                const double per_warp = c.ot / 16.0 < 1.0 ? 1.0 : c.ot / 16.0;
                const double setup = 1.0 + (0.6 + 8.0 / per_warp) / tb;
                const double restage = 1.0 + 0.01 * (256.0 / ich_want - 1.0);  // more staging rounds and barriers
                const double cost = (double)per_sm * tb * c.ot * setup * restage;
                if (best_cost < 0 || cost < best_cost * 0.999) {
                    best = c;
                    best_cost = cost;
                }
            }
        }
    }
    return best;
}

BwdCfg choose_bwd_cfg(const QkDesc& d) {
    const int rk = compiled_reps(d.ansatz, d.reps);
    const int nacc = acc_rows(rk);
    const int grid_i = (d.in_dim + 31) / 32;
    const int ru = tune_int(kDbgBwdRu, rk > 8 ? 2 : 4);  // long circuits: fewer rows in flight, no spills
    auto make = [&](int groups, int rpg) {
        const int tb = groups * rpg;
        size_t smem = (size_t)tb * 32 * 4 * 2 + (size_t)kGyChunkHost * tb * 4 +
                      (size_t)2 * groups * nacc * 32 * 4;
        return BwdCfg{groups, rpg, tb, (d.batch + tb - 1) / tb, grid_i, nacc, smem, ru, 1, round_up(d.out_dim, kGyChunkHost)};
    };
    auto slice = [&](BwdCfg c, int want) {  // cut the outputs into about `want` slices of a multiple of 8
        c.ochunk = round_up((d.out_dim + want - 1) / want, kGyChunkHost);
        c.osplit = (d.out_dim + c.ochunk - 1) / c.ochunk;
        return c;
    };
    const int force_groups = tune_int(kDbgBwdGroups, 0), force_rpg = tune_int(kDbgBwdRpg, 0);
    const int force_osplit = tune_int(kDbgBwdOsplit, 0);
    if (force_groups > 0 && force_rpg > 0)  // developer override
        return slice(make(force_groups, force_rpg), force_osplit > 0 ? force_osplit : 1);
    // (row groups = warps per CTA, rows per group), largest tile first
    static const int cand[][2] = {{8, 32}, {8, 16}, {4, 32}, {4, 16}, {8, 8}, {2, 32}, {4, 8}, {2, 16}, {2, 8}, {1, 8}};
    // registers per thread as compiled: up to 3 repetitions the kernel is built for two CTAs of 256 threads per
    // SM, which lets the compiler spend ~96 registers on scheduling (measured -2 % at 3 repetitions, -5 % at 1;
    // longer circuits were 1-2 % faster with the compiler's own choice)
    const int regs_est = rk > 8 ? 255 : (rk <= 3 ? 48 + 14 * rk : 34 + 11 * rk);
    const int ipad = round_up(d.in_dim, 32);
    // seconds per (row x 32 columns x output) on one SM: ~(28 R + 20) instructions at 0.72 IPC x 4 schedulers
    const double t_unit = (28.0 * rk + 20.0) / (4 * 0.72 * 1.965e9);
    const double partial_cap = 8.0 * 1024 * 1024 * 1024;  // bytes of per-tile partials we are willing to hold
    BwdCfg best{};
    double best_cost = -1.0;
    for (int pass = 0; pass < 2 && best_cost < 0; ++pass) {
        for (auto& c : cand) {
            // output slices (grid.z) give the CTA count a finer grain: fewer partly filled waves; their price
            // is one more pass over grad_x and a tile prologue per slice
            for (int want = 1; want <= 8; want *= 2) {
                if (want > 1 && (d.out_dim < 32 || force_osplit > 0)) break;
                BwdCfg cur = slice(make(c[0], c[1]), want);
                if (want > 1 && cur.osplit <= want / 2) continue;  // same slicing as a smaller `want`
                if (cur.smem > 200 * 1024) continue;
                const double partial_bytes = (double)cur.grid_b * d.out_dim * nacc * ipad * 4.0;
                if (pass == 0 && partial_bytes > partial_cap) continue;  // second pass lifts the cap if nothing fits
                const long ctas = (long)cur.grid_b * grid_i * cur.osplit;
                long resident = (long)(kSmemPerSm / (cur.smem + 1024));
                const long by_regs = 65536 / ((long)regs_est * cur.groups * 32);
                if (by_regs < resident) resident = by_regs;
                if (resident < 1) resident = 1;
                const long per_sm = (ctas + kSmCount - 1) / kSmCount;
                const long live = per_sm < resident ? per_sm : resident;
                const double warps = (double)live * cur.groups;
                const double occupancy =
                    warps >= 16 ? 1.0 : (warps >= 8 ? 1.0 + 0.04 * (16 - warps) : 1.32 + 0.2 * (8 - warps));
                const double setup = 1.0 + 0.09 * 32.0 / cur.rpg;       // per-edge set-up and reduction per row
                const double small_cta = 1.0 + 0.02 * (8.0 / cur.groups - 1.0);  // (0.06 fits 16384 x 256 x 256 better but costs 512 x 512 at 1 repetition 15 %)
                const int o_cta = cur.osplit > 1 ? cur.ochunk : d.out_dim;
                // a partly filled last wave costs less than a full one (its CTAs have the SM's issue slots to
                // themselves): count it half-way between its share and a whole wave
                const double waves = 0.5 * ((double)ctas / kSmCount + (double)per_sm);
                // measured: a sliced launch costs a few per cent more than its share of the work, more so for
                // short circuits (8192 x 512 x 512, 1 repetition: +4 % where the wave count predicted -12 %)
                const double slice_tax = cur.osplit > 1 ? 1.0 + 0.12 / (rk + 0.5) : 1.0;
                const double compute = waves * cur.tb * o_cta * t_unit * setup * occupancy * small_cta * slice_tax;
                const double partials = 2.0 * partial_bytes / 6.0e12;  // written here, read by finish_grads
                const double sliced = cur.osplit > 1 ? 4.0e-6 + (double)(cur.osplit + 1) * d.batch * d.in_dim * 4.0 / 3.0e12
                                                     : 0.0;
                const double cost = compute + partials + sliced;
                if (best_cost < 0 || cost < best_cost * 0.999) {
                    best = cur;
                    best_cost = cost;
                }
            }
        }
    }
    if (force_osplit > 0) return slice(best, force_osplit);
    // Small batches: the choice above leaves fewer than 16 warps per SM, and a CTA's time is then the
    // dependent chain of one output after the other (constant load, rows, reduction), not issue slots.
    // Smaller tiles and output slices put more chains in flight. Per output a warp spends about
    // 0.8 us + its rows x 0.175 us (measured at 3 repetitions, scaled by the instruction count).
    if ((long)best.grid_b * grid_i * best.osplit * best.groups >= kSmCount * 16 || d.batch <= 0) return best;
    static const int small[][2] = {{8, 16}, {8, 8}, {4, 8}, {8, 4}, {4, 4}, {2, 8}, {2, 4}};
    const double chain0 = 0.8e-6, chain_row = 0.175e-6 * (28.0 * rk + 20.0) / 104.0;
    best_cost = -1.0;
    for (auto& c : small) {
        if (c[1] % ru) continue;
        for (int want = 1; want <= 64; want *= 2) {
            if (want > 1 && d.out_dim < 32) break;  // too few outputs to be worth a second pass over grad_x
            BwdCfg cur = slice(make(c[0], c[1]), want);
            if (cur.osplit < want && want > 1 && cur.osplit <= want / 2) continue;  // same slicing as a smaller `want`
            long resident = (long)(kSmemPerSm / (cur.smem + 1024));
            const long by_regs = 65536 / ((long)regs_est * cur.groups * 32);
            if (by_regs < resident) resident = by_regs;
            if (resident > 32) resident = 32;
            if (resident < 1) resident = 1;
            const long ctas = (long)cur.grid_b * grid_i * cur.osplit;
            const long per_sm = (ctas + kSmCount - 1) / kSmCount;
            const long live = per_sm < resident ? per_sm : resident;
            const long waves = (per_sm + resident - 1) / resident;
            const double setup = 1.0 + 0.09 * 32.0 / cur.rpg;
            const double issue = (double)live * cur.tb * t_unit * setup;   // the SM's issue slots shared by its CTAs
            const double chain = chain0 + cur.rpg * chain_row;
            const double per_output = issue > chain ? issue : chain;
            const double partial_bytes = (double)cur.grid_b * d.out_dim * nacc * ipad * 4.0;
            const double gx_bytes = cur.osplit > 1 ? (double)(cur.osplit + 1) * d.batch * d.in_dim * 4.0 : 0.0;
            const double cost = (double)waves * cur.ochunk * per_output + (2.0 * partial_bytes + gx_bytes) / 3.0e12 +
                                (cur.osplit > 1 ? 4.0e-6 : 0.0);  // + the launch that adds the grad_x shares
            if (best_cost < 0 || cost < best_cost * 0.999) {
                best = cur;
                best_cost = cost;
            }
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
        case 12: return launch_fwd_d<12>(a, fast, io_dtype, has_base, st);
        case 16: return launch_fwd_d<16>(a, fast, io_dtype, has_base, st);
        case 0: return launch_fwd_d<0>(a, fast, io_dtype, has_base, st);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_backward(const BwdArgs& a, int reps, bool fast, int io_dtype, cudaStream_t st) {
    switch (reps) {
        case 1: return launch_bwd_d<1>(a, fast, io_dtype, st);
        case 2: return launch_bwd_d<2>(a, fast, io_dtype, st);
        case 3: return launch_bwd_d<3>(a, fast, io_dtype, st);
        case 4: return launch_bwd_d<4>(a, fast, io_dtype, st);
        case 5: return launch_bwd_d<5>(a, fast, io_dtype, st);
        case 6: return launch_bwd_d<6>(a, fast, io_dtype, st);
        case 7: return launch_bwd_d<7>(a, fast, io_dtype, st);
        case 8: return launch_bwd_d<8>(a, fast, io_dtype, st);
        case 12: return launch_bwd_d<12>(a, fast, io_dtype, st);
        case 16: return launch_bwd_d<16>(a, fast, io_dtype, st);
        case 0: return launch_bwd_d<0>(a, fast, io_dtype, st);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace qk
