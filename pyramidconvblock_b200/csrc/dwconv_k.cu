// Instantiates the tiled depthwise-convolution kernels for ONE filter width.
// Compiled once per supported width with -DPDW_K=<K> so that the widths build in parallel.
#include "dwconv_stream.cuh"

#ifndef PDW_K
#error "compile with -DPDW_K=<filter width>"
#endif

namespace pdw {

#define PDW_CAT2(a, b) a##b
#define PDW_CAT(a, b) PDW_CAT2(a, b)

template <typename T>
static int tiled_for_type(const TiledArgs& a) {
    const int ct = tuning(1);
    if constexpr (sizeof(T) == 2) {
        if (tuning(0) && ct == 16 && tuning(7) && aligned_to(a.w, 16)) {
            const int rc = launch_stream<T, PDW_K>(a);
            if (rc != PDW_ERR_UNSUPPORTED) return rc;
        }
        if (tuning(0)) return ct == 32 ? launch_tiled<T, PDW_K, 32, 1>(a) : launch_tiled<T, PDW_K, 16, 1>(a);
    }
    return ct == 32 ? launch_tiled<T, PDW_K, 32, 0>(a) : launch_tiled<T, PDW_K, 16, 0>(a);
}

static int tiled_entry(const TiledArgs& a) {
    switch (a.dtype) {
        case PDW_F32: return tiled_for_type<float>(a);
        case PDW_F16: return tiled_for_type<__half>(a);
        case PDW_BF16: return tiled_for_type<__nv_bfloat16>(a);
    }
    return PDW_ERR_BAD_DTYPE;
}

template <typename T>
static int wgrad_for_type(const WgradArgs& a) {
    const int ct = tuning(1);
    if constexpr (sizeof(T) == 2) {
        if (tuning(0)) return ct == 32 ? launch_wgrad<T, PDW_K, 32, 1>(a) : launch_wgrad<T, PDW_K, 16, 1>(a);
    }
    return ct == 32 ? launch_wgrad<T, PDW_K, 32, 0>(a) : launch_wgrad<T, PDW_K, 16, 0>(a);
}

static int wgrad_entry(const WgradArgs& a) {
    switch (a.dtype) {
        case PDW_F32: return wgrad_for_type<float>(a);
        case PDW_F16: return wgrad_for_type<__half>(a);
        case PDW_BF16: return wgrad_for_type<__nv_bfloat16>(a);
    }
    return PDW_ERR_BAD_DTYPE;
}

static size_t wgrad_workspace(int B, int OH, int OW, int C, int KH, int dtype) {
    WgradPlan plan{};
    const int esize = (int)dtype_size(dtype);
    const bool ok = tuning(1) == 32 ? plan_wgrad<32, PDW_K>(B, OH, OW, C, KH, esize, sm_count(), &plan)
                                    : plan_wgrad<16, PDW_K>(B, OH, OW, C, KH, esize, sm_count(), &plan);
    return ok ? plan.workspace_bytes : 0;
}

extern const KernelSet PDW_CAT(kernel_set_k, PDW_K) = {PDW_K, tiled_entry, wgrad_entry, wgrad_workspace};

}  // namespace pdw
