// Forward entry point for hosts that cannot give the library a scratch buffer.
//
// The regular forward needs a few megabytes of device scratch (the per-edge
// constant table and the folded bias vector) which the caller allocates. Some
// callers have no way to do that: a serving process whose device memory is
// entirely owned by another runtime's pool, or a latency-critical loop in which
// cudaMalloc (a device-wide synchronising call) is forbidden once start-up is
// over. For them the scratch lives in a fixed array inside the library image.
//
// The array below is device memory that exists once per GPU that loads this
// library and stays resident until the process exits. In host code its name is
// only a stand-in symbol, not a device address, so the address is looked up
// with cudaGetSymbolAddress once per device (with that device current) and it
// is that pointer which is handed to the kernels.
#include <cstdio>
#include <mutex>

#include "qk_common.cuh"

namespace {

constexpr size_t kStaticScratchBytes = size_t(8) << 20;  // 8 MiB per GPU
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

std::mutex g_mutex;
void* g_scratch_ptr[kMaxDevices] = {};
thread_local char g_static_err[256] = "";

}  // namespace

extern "C" {

size_t qk_noalloc_max_scratch_bytes(void) { return kStaticScratchBytes; }

const char* qk_noalloc_last_error(void) { return g_static_err; }

int qk_pz_forward_noalloc(const QkDesc* desc, const void* x, const float* theta,
                          const float* preacts_weight, const float* preacts_bias,
                          const void* postact_weights, const void* postact_bias,
                          const void* base_weight, const void* mask, void* y, void* cuda_stream) {
    g_static_err[0] = 0;
    size_t need = qk_forward_workspace_bytes(desc);
    if (need == 0) {
        // the descriptor itself was rejected: let the regular entry point name the reason, so that both entry
        // points answer a bad or unsupported descriptor with the same code (it fails before touching memory)
        const int rc = qk_pz_forward(desc, x, theta, preacts_weight, preacts_bias, postact_weights,
                                     postact_bias, base_weight, mask, y, nullptr, 0, cuda_stream);
        snprintf(g_static_err, sizeof(g_static_err), "%s", qk_last_error());
        return rc != QK_OK ? rc : QK_ERR_BAD_ARGUMENT;
    }
    QkDesc single = *desc;
    if (need > kStaticScratchBytes) {
        // a frozen-preact layer keeps two tables; with one (and the generic forward kernel) it may still fit
        single.flags |= QK_SINGLE_TABLE;
        const size_t need_single = qk_forward_workspace_bytes(&single);
        if (need_single != 0 && need_single <= kStaticScratchBytes) {
            desc = &single;
            need = need_single;
        }
    }
    if (need > kStaticScratchBytes) {
        snprintf(g_static_err, sizeof(g_static_err),
                 "problem needs %zu bytes of scratch but the built-in array holds %zu; "
                 "use qk_pz_forward with a caller-owned workspace",
                 need, kStaticScratchBytes);
        return QK_ERR_WORKSPACE;
    }
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        snprintf(g_static_err, sizeof(g_static_err), "cudaGetDevice: %s (device %d)",
                 cudaGetErrorString(e), dev);
        return QK_ERR_LAUNCH;
    }
    void* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        if (!g_scratch_ptr[dev]) {
            // first call on this device: resolve the array's device address (device `dev` is current)
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, g_static_scratch);
            if (e != cudaSuccess || !p) {
                snprintf(g_static_err, sizeof(g_static_err), "cudaGetSymbolAddress: %s",
                         cudaGetErrorString(e));
                return QK_ERR_LAUNCH;
            }
            g_scratch_ptr[dev] = p;
        }
        scratch = g_scratch_ptr[dev];
    }
    // Every byte of scratch the forward reads is rewritten by its own set-up kernels on the
    // same stream first, so nothing has to be cleared between calls.
    int rc = qk_pz_forward(desc, x, theta, preacts_weight, preacts_bias, postact_weights,
                           postact_bias, base_weight, mask, y, scratch, kStaticScratchBytes,
                           cuda_stream);
    if (rc != QK_OK) snprintf(g_static_err, sizeof(g_static_err), "%s", qk_last_error());
    return rc;
}

}  // extern "C"
