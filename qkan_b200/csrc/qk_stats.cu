// Host side of the per-edge activation scale (see qk_stats.cuh): tile choice, dispatch on the repetition
// count, and the kernel that adds the per-tile sums and takes the root.
#include <cmath>

#include "qk_stats.cuh"

namespace qk {

template <int R>
cudaError_t launch_stats_d(const StatsArgs& a, int io_dtype, cudaStream_t st);
#define QK_DECL(R) extern template cudaError_t launch_stats_d<R>(const StatsArgs&, int, cudaStream_t);
QK_DECL(0) QK_DECL(1) QK_DECL(2) QK_DECL(3) QK_DECL(4) QK_DECL(5) QK_DECL(6) QK_DECL(7) QK_DECL(8) QK_DECL(12) QK_DECL(16)
#undef QK_DECL

// Rows per CTA: 256 (8 warps x 32 rows) when that still gives every SM two CTAs, else smaller tiles, down to
// 8 warps x 4 rows, so that small batches spread over the machine.
void choose_stats_tile(int batch, int in_dim, int* groups, int* rpg) {
    const long col_blocks = (in_dim + 31) / 32;
    *groups = 8;
    for (int r : {32, 16, 8, 4}) {
        *rpg = r;
        const long ctas = ((batch + 8L * r - 1) / (8L * r)) * col_blocks;
        if (ctas >= 2 * 148) break;
    }
}

size_t stats_scratch_bytes(int batch, int in_dim, int out_dim) {
    int groups, rpg;
    choose_stats_tile(batch, in_dim, &groups, &rpg);
    const size_t tiles = (batch + (size_t)groups * rpg - 1) / ((size_t)groups * rpg);
    return align256(tiles * out_dim * 2 * round_up(in_dim, 32) * sizeof(float));
}

// std[o,i] = sqrt(max(0, (S2 - S1^2 / n) / (n - 1))) with S1, S2 the tile sums added in tile order;
// NaN for fewer than two rows, as torch.std gives.
__global__ void stats_finish_kernel(const float* __restrict__ partials, float* __restrict__ out, int ntiles,
                                    int batch, int in_dim, int out_dim, int ipad) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x, o = blockIdx.y;
    if (i >= in_dim) return;
    double s1 = 0.0, s2 = 0.0;
    for (int t = 0; t < ntiles; ++t) {
        const float* p = partials + (((size_t)t * out_dim + o) * 2) * ipad + i;
        s1 += (double)p[0];
        s2 += (double)p[ipad];
    }
    float r = nanf("");
    if (batch >= 2) {
        const double var = (s2 - s1 * s1 / batch) / (batch - 1);
        r = (float)sqrt(var > 0.0 ? var : 0.0);
    }
    out[(size_t)o * in_dim + i] = r;
}

cudaError_t launch_edge_stats(const void* x, int io_dtype, const float* table, int batch, int in_dim, int out_dim,
                              int rk, bool fast, bool base, float* out_std, float* scratch, cudaStream_t st) {
    StatsArgs a{};
    a.batch = batch;
    a.in_dim = in_dim;
    a.out_dim = out_dim;
    a.ipad = round_up(in_dim, 32);
    choose_stats_tile(batch, in_dim, &a.groups, &a.rpg);
    a.tb = a.groups * a.rpg;
    a.grid_b = (batch + a.tb - 1) / a.tb;
    a.fast = fast;
    a.base = base;
    a.x = x;
    a.table = table;
    a.partials = scratch;
    cudaError_t e;
    switch (rk) {
        case 0: e = launch_stats_d<0>(a, io_dtype, st); break;
        case 1: e = launch_stats_d<1>(a, io_dtype, st); break;
        case 2: e = launch_stats_d<2>(a, io_dtype, st); break;
        case 3: e = launch_stats_d<3>(a, io_dtype, st); break;
        case 4: e = launch_stats_d<4>(a, io_dtype, st); break;
        case 5: e = launch_stats_d<5>(a, io_dtype, st); break;
        case 6: e = launch_stats_d<6>(a, io_dtype, st); break;
        case 7: e = launch_stats_d<7>(a, io_dtype, st); break;
        case 8: e = launch_stats_d<8>(a, io_dtype, st); break;
        case 12: e = launch_stats_d<12>(a, io_dtype, st); break;
        case 16: e = launch_stats_d<16>(a, io_dtype, st); break;
        default: return cudaErrorInvalidValue;
    }
    if (e != cudaSuccess) return e;
    dim3 grid((in_dim + 127) / 128, out_dim);
    stats_finish_kernel<<<grid, 128, 0, st>>>(scratch, out_std, a.grid_b, batch, in_dim, out_dim, a.ipad);
    return cudaPeekAtLastError();
}

}  // namespace qk
