// extern "C" entry points of libss2d_b200.so (declared in include/ss2d_b200.h).
#include <atomic>
#include <cstdlib>
#include <initializer_list>

#include <nvtx3/nvToolsExt.h>

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
int linear_supported(const ss2d_linear_params* p);
int linear_fwd(const ss2d_linear_params* p, cudaStream_t st);
long long route_expand_workspace_bytes(const ss2d_expand_params* p);
int stem_conv_norm_act(const ss2d_stem_params* p, cudaStream_t st);
int pixels_norm_to_planes(const ss2d_relayout_params* p, cudaStream_t st);
int planes_to_pixels(const ss2d_relayout_params* p, cudaStream_t st);
int bias_act(const ss2d_pointwise_params* p, cudaStream_t st);
int dwconv3x3_act(const ss2d_pointwise_params* p, cudaStream_t st);

static std::atomic<long long> g_launches{0};
static std::atomic<int> g_debug_checks{[] { const char* v = std::getenv("SS2D_DEBUG_CHECKS"); return (v && v[0] == '1') ? 1 : 0; }()};

// SS2D_OK, or SS2D_EINVAL_DEVICE when debug checks are on and one of the pointers is not memory of the current GPU.
static int pointers_on_current_device(std::initializer_list<const void*> ptrs) {
    if (!g_debug_checks.load(std::memory_order_relaxed)) return SS2D_OK;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return SS2D_ECUDA;
    for (const void* q : ptrs) {
        if (!q) continue;
        cudaPointerAttributes at;
        if (cudaPointerGetAttributes(&at, q) != cudaSuccess) { cudaGetLastError(); return SS2D_EINVAL_DEVICE; }
        if (at.type != cudaMemoryTypeDevice && at.type != cudaMemoryTypeManaged) return SS2D_EINVAL_DEVICE;
        if (at.type == cudaMemoryTypeDevice && at.device != dev) return SS2D_EINVAL_DEVICE;
    }
    return SS2D_OK;
}
// NVTX range around an entry point (SS2D_NVTX=1 at load time): the boundary calls show up by name in a timeline.
static const bool g_nvtx = [] { const char* v = std::getenv("SS2D_NVTX"); return v && v[0] == '1'; }();
struct Range {
    explicit Range(const char* name) { if (g_nvtx) nvtxRangePushA(name); }
    ~Range() { if (g_nvtx) nvtxRangePop(); }
};
#define SS2D_CHECK_PTRS(...)                                          \
    do {                                                              \
        const int rc_ = ss2d::pointers_on_current_device({__VA_ARGS__}); \
        if (rc_ != SS2D_OK) return rc_;                               \
    } while (0)

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
int check_launch() { return cudaPeekAtLastError() == cudaSuccess ? SS2D_OK : SS2D_ECUDA; }
}  // namespace ss2d

extern "C" {

int ss2d_set_debug_checks(int on) { return ss2d::g_debug_checks.exchange(on ? 1 : 0); }

int ss2d_selective_scan_fwd(const ss2d_scan_params* p, void* stream) {
    ss2d::Range nvtx_("ss2d_selective_scan_fwd");
    if (p) SS2D_CHECK_PTRS(p->u, p->delta, p->A, p->B, p->C, p->D, p->delta_bias, p->out, p->checkpoints);
    return ss2d::selective_scan_fwd(p, (cudaStream_t)stream);
}
int ss2d_selective_scan_bwd(const ss2d_scan_bwd_params* p, void* stream) {
    ss2d::Range nvtx_("ss2d_selective_scan_bwd");
    if (p) SS2D_CHECK_PTRS(p->u, p->delta, p->A, p->B, p->C, p->D, p->delta_bias, p->dout, p->du, p->ddelta, p->dA, p->dB, p->dC,
                           p->dD, p->ddelta_bias, p->workspace, p->checkpoints);
    return ss2d::selective_scan_bwd(p, (cudaStream_t)stream);
}
int64_t ss2d_selective_scan_bwd_workspace_bytes(const ss2d_scan_bwd_params* p) { return ss2d::selective_scan_bwd_workspace_bytes(p); }
int ss2d_cross_scan(const ss2d_cross_params* p, void* stream) {
    ss2d::Range nvtx_("ss2d_cross_scan");
    if (p) SS2D_CHECK_PTRS(p->in, p->out);
    return ss2d::cross_scan(p, (cudaStream_t)stream);
}
int ss2d_cross_merge(const ss2d_cross_params* p, void* stream) {
    ss2d::Range nvtx_("ss2d_cross_merge");
    if (p) SS2D_CHECK_PTRS(p->in, p->out);
    return ss2d::cross_merge(p, (cudaStream_t)stream);
}
int ss2d_cross_scan_ex(const ss2d_cross_ex_params* p, void* stream) {
    ss2d::Range nvtx_("ss2d_cross_scan_ex");
    if (p) SS2D_CHECK_PTRS(p->in, p->out);
    return ss2d::cross_scan_ex(p, (cudaStream_t)stream);
}
int ss2d_cross_merge_ex(const ss2d_cross_ex_params* p, void* stream) {
    ss2d::Range nvtx_("ss2d_cross_merge_ex");
    if (p) SS2D_CHECK_PTRS(p->in, p->out);
    return ss2d::cross_merge_ex(p, (cudaStream_t)stream);
}
int ss2d_layer_norm_cf(const ss2d_norm_params* p, void* stream) {
    ss2d::Range nvtx_("ss2d_layer_norm_cf");
    if (p) SS2D_CHECK_PTRS(p->in, p->add, p->add_bias, p->sum_out, p->weight, p->bias, p->out);
    return ss2d::layer_norm_cf(p, (cudaStream_t)stream);
}
int64_t ss2d_core_workspace_bytes(const ss2d_core_params* p) { return ss2d::core_workspace_bytes(p); }
int ss2d_core_fwd(const ss2d_core_params* p, void* stream) {
    ss2d::Range nvtx_("ss2d_core_fwd");
    if (p) SS2D_CHECK_PTRS(p->x, p->delta[0], p->delta[1], p->delta[2], p->delta[3], p->Bm[0], p->Bm[1], p->Bm[2], p->Bm[3], p->Cm[0], p->Cm[1],
                           p->Cm[2], p->Cm[3], p->A, p->Dskip, p->delta_bias, p->ln_weight, p->ln_bias, p->y, p->workspace);
    return ss2d::core_fwd(p, (cudaStream_t)stream);
}
int ss2d_core_supported(const ss2d_core_params* p) { return ss2d::core_supported(p); }
int ss2d_core_fwd_static(const ss2d_core_params* p, void* stream) {
    ss2d::Range nvtx_("ss2d_core_fwd_static");
    if (p) SS2D_CHECK_PTRS(p->x, p->delta[0], p->delta[1], p->delta[2], p->delta[3], p->Bm[0], p->Bm[1], p->Bm[2], p->Bm[3], p->Cm[0], p->Cm[1],
                           p->Cm[2], p->Cm[3], p->A, p->Dskip, p->delta_bias, p->ln_weight, p->ln_bias, p->y);
    return ss2d::core_fwd_static(p, (cudaStream_t)stream);
}
int64_t ss2d_core_static_capacity(void) { return ss2d::core_static_capacity(); }

int ss2d_route_expand(const ss2d_expand_params* p, void* stream) {
    ss2d::Range nvtx_("ss2d_route_expand"); return ss2d::route_expand(p, (cudaStream_t)stream); }
int64_t ss2d_route_expand_workspace_bytes(const ss2d_expand_params* p) { return ss2d::route_expand_workspace_bytes(p); }

int ss2d_bias_act(const ss2d_pointwise_params* p, void* stream) {
    ss2d::Range nvtx_("ss2d_bias_act"); return ss2d::bias_act(p, (cudaStream_t)stream); }
int ss2d_dwconv3x3_act(const ss2d_pointwise_params* p, void* stream) {
    ss2d::Range nvtx_("ss2d_dwconv3x3_act"); return ss2d::dwconv3x3_act(p, (cudaStream_t)stream); }

int ss2d_stem_conv_norm_act(const ss2d_stem_params* p, void* stream) {
    ss2d::Range nvtx_("ss2d_stem_conv_norm_act"); return ss2d::stem_conv_norm_act(p, (cudaStream_t)stream); }
int ss2d_pixels_norm_to_planes(const ss2d_relayout_params* p, void* stream) {
    ss2d::Range nvtx_("ss2d_pixels_norm_to_planes"); return ss2d::pixels_norm_to_planes(p, (cudaStream_t)stream); }
int ss2d_planes_to_pixels(const ss2d_relayout_params* p, void* stream) {
    ss2d::Range nvtx_("ss2d_planes_to_pixels"); return ss2d::planes_to_pixels(p, (cudaStream_t)stream); }

int ss2d_mlp_supported(const ss2d_mlp_params* p) { return ss2d::mlp_supported(p); }
int ss2d_mlp_fwd(const ss2d_mlp_params* p, void* stream) {
    ss2d::Range nvtx_("ss2d_mlp_fwd");
    if (p) SS2D_CHECK_PTRS(p->x, p->w1, p->b1, p->w2, p->y);
    return ss2d::mlp_fwd(p, (cudaStream_t)stream);
}

int ss2d_linear_supported(const ss2d_linear_params* p) { return ss2d::linear_supported(p); }
int ss2d_linear_fwd(const ss2d_linear_params* p, void* stream) {
    ss2d::Range nvtx_("ss2d_linear_fwd");
    if (p) SS2D_CHECK_PTRS(p->x, p->w, p->bias, p->out);
    return ss2d::linear_fwd(p, (cudaStream_t)stream);
}

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
        case SS2D_EINVAL_DEVICE: return "debug checks: a pointer is host memory or memory of another GPU than the current one";
        case SS2D_ETOOBIG: return "problem larger than the library's built-in scratch (B*D*H*W > ss2d_core_static_capacity())";
        default: return "unknown status";
    }
}

}  // extern "C"
