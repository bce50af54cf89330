// Argument blocks and host-side launchers shared by the translation units.
#pragma once

#include "qk_common.cuh"

namespace qk {

struct PrepArgs {
    int in_dim, out_dim, reps, ipad;
    int rk;      // compiled_reps(ansatz, reps): the table is laid out for this repetition count
    int ansatz;  // QkAnsatz
    int group;   // > 0: theta / preacts are grouped, edge (o,i) reads entry i % group
    unsigned flags;
    int param_dtype;
    const float* theta;
    const float* pw;
    const float* pb;
    const void* postw;  // nullptr => weight 1 (solver-contract mode)
    const void* postb;
    const void* basew;
    const void* mask;
    float* table;    // generic table (backward, and every forward but the frozen-preact one)
    float* table_x;  // frozen-preact forward's table: rows (pw_l, c_l) hold (cos c_l, sin c_l); nullptr => not wanted
    float* bias;     // nullptr => not computed
    float* basew_c;  // [out_dim][ipad] base_weight * mask for the base-term backward; nullptr => not wanted
};

struct FinishArgs {
    int in_dim, out_dim, reps, ipad, nacc, ntiles;
    int base_tiles;               // row tiles of the base-term kernel (0: no base term)
    const float* base_partials;   // [base_tiles][out_dim][ipad] partial sums of grad_base_weight
    int rk, ansatz;
    unsigned flags;
    int param_dtype;
    const float* partials;
    const float* colpart;  // [ntiles][out_dim] per-tile column sums of grad_y (nullptr: postact-bias terms off)
    const void* postw;
    const void* postb;
    const void* mask;
    float* gtheta;
    float* gpw;
    float* gpb;
    float* gpostw;
    float* gpostb;
    float* gbasew;
};

// Tile shape of the forward: a CTA owns `tb` batch rows and `ot` outputs and
// walks the input dimension in chunks of `ich` (multiple of 32) columns.
struct FwdCfg {
    int tb, ot, ich, threads;
    int grid_b, grid_o;
    size_t smem;
};

// Tile shape of the backward: a CTA owns `groups * rpg` batch rows and 32 input
// columns (one lane per column) and walks all outputs.
struct BwdCfg {
    int groups, rpg, tb;
    int grid_b, grid_i;
    int nacc;
    size_t smem;
    int ru;  // rows a thread interleaves in its inner loop (2 or 4)
    // Small batches leave most SMs idle when a CTA walks all outputs, so the outputs are cut into
    // `osplit` slices of `ochunk` (a multiple of 8) handled by different CTAs (grid.z). Each slice writes
    // its share of grad_x to scratch and sum_gx adds the shares in order.
    int osplit, ochunk;
};

struct FwdArgs {
    int batch, in_dim, out_dim, ipad;
    int precise;  // QK_PRECISE_MATH requested (honoured for float32 I/O)
    int xtrig;    // use the frozen-preact kernel (table built with PrepArgs.xtrig)
    FwdCfg cfg;
    const void* x;
    const float* table;
    const float* bias;
    void* y;         // (B,O), fused mode
    void* postacts;  // (B,O,I), solver-contract mode (y unused)
};

struct BwdArgs {
    int batch, in_dim, out_dim, ipad;
    int precise;  // QK_PRECISE_MATH requested (honoured for float32 I/O)
    BwdCfg cfg;
    const void* x;
    const void* gy;         // (B,O) fused mode
    const void* gpostacts;  // (B,O,I) solver-contract mode (gy unused)
    const float* table;
    void* gx;  // may be nullptr
    float* gx_part;  // [osplit][B][I] float scratch, used when cfg.osplit > 1
    float* partials;
    float* colpart;  // [grid_b][out_dim] column sums of this tile's grad_y rows (written by the CTAs of column block 0); may be nullptr
};

// Backward of the base term (qk_base.cu): runs after the circuit backward, adds its part to grad_x in place.
struct BaseBwdArgs {
    int batch, in_dim, out_dim, ipad;
    int slab_rows, slabs;  // filled by the launcher from base_plan()
    int vec4;              // filled by the launcher: x / grad_x may be moved four columns at a time
    int vec_gy;            // filled by the launcher: so may grad_y
    const void* x;
    const void* gy;
    const float* basew;  // [out_dim][ipad] base_weight * mask, written by prep
    void* gx;            // read-modify-write; nullptr: grad_x not wanted
    float* partials;     // [slabs][out_dim][ipad]; nullptr: grad_base_weight not wanted
};

// Tiling of the base-term backward: tile edge (128 or 64) and the slabs of batch rows whose partial sums of
// grad_base_weight go to scratch.
struct BasePlan {
    int tile, slab_rows, slabs;
};
BasePlan base_plan(int batch, int in_dim, int out_dim);

FwdCfg choose_fwd_cfg(const QkDesc& d, bool edges, bool base, bool xtrig);

// Developer overrides (qk_debug_set in the C ABI; first use also reads the QK_* environment variables once).
enum DebugKey { kDbgBwdGroups = 0, kDbgBwdRpg, kDbgBwdRu, kDbgBwdOsplit, kDbgNoXtrig, kDbgVerbose, kDbgFwdThreads, kDbgFwdTb, kDbgFwdOt, kDbgFwdIch, kDbgCount };
int debug_get(int key);
void debug_set(int key, int value);

// Largest dynamic shared memory any tile chooser hands out; each kernel instantiation is opted in to it once per device.
constexpr int kSmemCap = 200 * 1024;
// Opts `kern` in to kSmemCap bytes of dynamic shared memory on the current device, once: `mask` is that
// instantiation's own set of devices already done. The attribute is set before the bit, so a second host thread
// either sees the bit (attribute in place) or sets the same value again. A cudaDeviceReset() forgets the attribute
// but not the bit: a process that resets a device must not call the library on it afterwards.
template <typename K>
inline cudaError_t opt_in_smem(K kern, unsigned long long* mask) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const unsigned long long bit = 1ull << (dev & 63);
    if (__atomic_load_n(mask, __ATOMIC_ACQUIRE) & bit) return cudaSuccess;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemCap);
    if (e == cudaSuccess) __atomic_fetch_or(mask, bit, __ATOMIC_RELEASE);
    return e;
}
BwdCfg choose_bwd_cfg(const QkDesc& d);
cudaError_t launch_base_backward(const BaseBwdArgs& a, int io_dtype, cudaStream_t st);

cudaError_t launch_prep(const PrepArgs& a, cudaStream_t st);
// per-edge standard deviation over the batch of the edge outputs (qk_stats.cu); scratch: stats_scratch_bytes()
size_t stats_scratch_bytes(int batch, int in_dim, int out_dim);
cudaError_t launch_edge_stats(const void* x, int io_dtype, const float* table, int batch, int in_dim, int out_dim,
                              int rk, bool fast, bool base, float* out_std, float* scratch, cudaStream_t st);
cudaError_t launch_finish(const FinishArgs& a, cudaStream_t st);
// gx[n] = sum over the output slices of part[s][n], in slice order, stored in the I/O dtype
cudaError_t launch_sum_gx(const float* part, void* gx, int io_dtype, size_t n, int nslices, cudaStream_t st);
// dst[k*per + c] = sum over o and over i == k (mod group) of src[(o*in_dim + i)*per + c], fixed order
cudaError_t launch_group_reduce(const float* src, float* dst, int out_dim, int in_dim, int group, int per,
                                cudaStream_t st);
cudaError_t launch_forward(const FwdArgs& a, int reps, bool fast, int io_dtype, bool has_base,
                           cudaStream_t st);
cudaError_t launch_backward(const BwdArgs& a, int reps, bool fast, int io_dtype, cudaStream_t st);

}  // namespace qk
