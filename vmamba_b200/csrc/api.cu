// extern "C" entry points of libss2d_b200.so (declared in include/ss2d_b200.h).
#include <atomic>

#include "common.cuh"

namespace ss2d {
int selective_scan_fwd(const ss2d_scan_params* p, cudaStream_t st);
int selective_scan_bwd(const ss2d_scan_bwd_params* p, cudaStream_t st);
long long selective_scan_bwd_workspace_bytes(const ss2d_scan_bwd_params* p);
int cross_scan(const ss2d_cross_params* p, cudaStream_t st);
int cross_merge(const ss2d_cross_params* p, cudaStream_t st);
int cross_scan_ex(const ss2d_cross_ex_params* p, cudaStream_t st);
int cross_merge_ex(const ss2d_cross_ex_params* p, cudaStream_t st);
int layer_norm_cf(const ss2d_norm_params* p, cudaStream_t st);
long long core_workspace_bytes(const ss2d_core_params* p);
int core_fwd(const ss2d_core_params* p, cudaStream_t st);
int core_supported(const ss2d_core_params* p);
int core_fwd_static(const ss2d_core_params* p, cudaStream_t st);
long long core_static_capacity();
int route_expand(const ss2d_expand_params* p, cudaStream_t st);
int mlp_supported(const ss2d_mlp_params* p);
int mlp_fwd(const ss2d_mlp_params* p, cudaStream_t st);
long long route_expand_workspace_bytes(const ss2d_expand_params* p);
int stem_conv_norm_act(const ss2d_stem_params* p, cudaStream_t st);
int pixels_norm_to_planes(const ss2d_relayout_params* p, cudaStream_t st);
int planes_to_pixels(const ss2d_relayout_params* p, cudaStream_t st);
int bias_act(const ss2d_pointwise_params* p, cudaStream_t st);
int dwconv3x3_act(const ss2d_pointwise_params* p, cudaStream_t st);

static std::atomic<long long> g_launches{0};
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
int check_launch() { return cudaPeekAtLastError() == cudaSuccess ? SS2D_OK : SS2D_ECUDA; }
}  // namespace ss2d

extern "C" {

int ss2d_selective_scan_fwd(const ss2d_scan_params* p, void* stream) {
    return ss2d::selective_scan_fwd(p, (cudaStream_t)stream);
}
int ss2d_selective_scan_bwd(const ss2d_scan_bwd_params* p, void* stream) {
    return ss2d::selective_scan_bwd(p, (cudaStream_t)stream);
}
int64_t ss2d_selective_scan_bwd_workspace_bytes(const ss2d_scan_bwd_params* p) { return ss2d::selective_scan_bwd_workspace_bytes(p); }
int ss2d_cross_scan(const ss2d_cross_params* p, void* stream) { return ss2d::cross_scan(p, (cudaStream_t)stream); }
int ss2d_cross_merge(const ss2d_cross_params* p, void* stream) { return ss2d::cross_merge(p, (cudaStream_t)stream); }
int ss2d_cross_scan_ex(const ss2d_cross_ex_params* p, void* stream) { return ss2d::cross_scan_ex(p, (cudaStream_t)stream); }
int ss2d_cross_merge_ex(const ss2d_cross_ex_params* p, void* stream) { return ss2d::cross_merge_ex(p, (cudaStream_t)stream); }
int ss2d_layer_norm_cf(const ss2d_norm_params* p, void* stream) { return ss2d::layer_norm_cf(p, (cudaStream_t)stream); }
int64_t ss2d_core_workspace_bytes(const ss2d_core_params* p) { return ss2d::core_workspace_bytes(p); }
int ss2d_core_fwd(const ss2d_core_params* p, void* stream) { return ss2d::core_fwd(p, (cudaStream_t)stream); }
int ss2d_core_supported(const ss2d_core_params* p) { return ss2d::core_supported(p); }
int ss2d_core_fwd_static(const ss2d_core_params* p, void* stream) { return ss2d::core_fwd_static(p, (cudaStream_t)stream); }
int64_t ss2d_core_static_capacity(void) { return ss2d::core_static_capacity(); }

int ss2d_route_expand(const ss2d_expand_params* p, void* stream) { return ss2d::route_expand(p, (cudaStream_t)stream); }
int64_t ss2d_route_expand_workspace_bytes(const ss2d_expand_params* p) { return ss2d::route_expand_workspace_bytes(p); }

int ss2d_bias_act(const ss2d_pointwise_params* p, void* stream) { return ss2d::bias_act(p, (cudaStream_t)stream); }
int ss2d_dwconv3x3_act(const ss2d_pointwise_params* p, void* stream) { return ss2d::dwconv3x3_act(p, (cudaStream_t)stream); }

int ss2d_stem_conv_norm_act(const ss2d_stem_params* p, void* stream) { return ss2d::stem_conv_norm_act(p, (cudaStream_t)stream); }
int ss2d_pixels_norm_to_planes(const ss2d_relayout_params* p, void* stream) { return ss2d::pixels_norm_to_planes(p, (cudaStream_t)stream); }
int ss2d_planes_to_pixels(const ss2d_relayout_params* p, void* stream) { return ss2d::planes_to_pixels(p, (cudaStream_t)stream); }

int ss2d_mlp_supported(const ss2d_mlp_params* p) { return ss2d::mlp_supported(p); }
int ss2d_mlp_fwd(const ss2d_mlp_params* p, void* stream) { return ss2d::mlp_fwd(p, (cudaStream_t)stream); }

int ss2d_version(void) { return SS2D_ABI_VERSION; }
int64_t ss2d_launch_count(void) { return ss2d::g_launches.load(std::memory_order_relaxed); }

const char* ss2d_strerror(int status) {
    switch (status) {
        case SS2D_OK: return "ok";
        case SS2D_EINVAL_NULL: return "a required pointer is NULL";
        case SS2D_EINVAL_SHAPE: return "invalid or inconsistent sizes";
        case SS2D_EINVAL_DTYPE: return "unsupported dtype combination";
        case SS2D_EINVAL_ALIGN: return "pointer not aligned to its element size";
        case SS2D_EINVAL_STRIDE: return "stride too small for the given sizes";
        case SS2D_ENOTSUP: return "request not supported by this build";
        case SS2D_ECUDA: return "CUDA runtime error at kernel launch";
        case SS2D_EWORKSPACE: return "workspace missing or too small";
        case SS2D_ETOOBIG: return "problem larger than the library's built-in scratch (B*D*H*W > ss2d_core_static_capacity())";
        default: return "unknown status";
    }
}

}  // extern "C"
