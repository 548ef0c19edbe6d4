// Weight/bias gradient for callers that cannot allocate device memory.
//
// pdw_dwconv_bwd_weight needs a scratch buffer for the per-thread-block fp32 partial sums and asks
// the caller to bring it.  Some callers have no way to do that: a plugin loaded into a host process
// whose device allocator it cannot reach, a server that gave its whole memory budget to its own
// pool at start-up and forbids cudaMalloc afterwards, or a latency-critical loop in which a call
// into the driver's allocator may block.  For them this file keeps the scratch inside the library
// image: a fixed 8 MiB array in device global memory.  Every GPU on which the library's code is
// loaded carries that array until the process exits.
#include <mutex>

#include "common.cuh"

namespace {

// The scratch itself.  In host code this name is only a handle for the runtime's symbol table, not
// a device address; the address used by the kernels is looked up below, per device.
static __device__ __align__(256) unsigned char g_static_scratch[PDW_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
void* g_scratch_ptr[kMaxDevices] = {nullptr};
std::mutex g_scratch_mutex;

// Device address of the array on the CURRENT device; resolved once per device.
int static_scratch_for_current_device(void** out) {
    int dev = 0;
    PDW_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return PDW_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (g_scratch_ptr[dev] == nullptr) {
        void* ptr = nullptr;
        PDW_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_static_scratch));
        if (ptr == nullptr) return pdw::cuda_fail(cudaErrorInvalidSymbol);
        g_scratch_ptr[dev] = ptr;
    }
    *out = g_scratch_ptr[dev];
    return PDW_OK;
}

}  // namespace

extern "C" int pdw_dwconv_bwd_weight_static(const void* x, const void* grad_out, void* dw, void* dbias,
                                            const pdw_conv_geom* g, int dtype, int out_fp32, int32_t* status_word,
                                            void* stream) {
    if (g == nullptr) return PDW_ERR_NULL_POINTER;
    const size_t need = pdw_dwconv_bwd_weight_workspace(g, dtype);
    if (need > (size_t)PDW_STATIC_SCRATCH_BYTES) return PDW_ERR_TOO_LARGE;
    void* scratch = nullptr;
    const int rc = static_scratch_for_current_device(&scratch);
    if (rc != PDW_OK) return rc;
    // Same kernels, same launch plan, same arithmetic as the caller-workspace entry point: only the
    // home of the partial sums differs.  Every partial the second-level kernel reads is written by the
    // first-level kernel of the same call, so nothing in the array has to be cleared between calls.
    return pdw_dwconv_bwd_weight(x, grad_out, dw, dbias, g, dtype, out_fp32, scratch, PDW_STATIC_SCRATCH_BYTES,
                                 status_word, stream);
}
