// CrossScan / CrossMerge as stand-alone tensor-to-tensor operators (channel-first).
//
// Every route is an index map  (h, w) -> l  that is contiguous either along w ("row-like")
// or along h ("column-like").  A CTA owns one 32x32 tile of one (b, c) plane: the tile is read
// (scan) or written (merge) with w fastest, column-like routes go through a padded shared-memory
// transpose so that both the global reads and the global writes of every route are coalesced.
// Data movement only: results are bit-identical to indexing.
#include "common.cuh"

namespace ss2d {

constexpr int kTile = 32;
constexpr int kRowsPerPass = 8;   // CTA = 32 x 8 threads, four passes per tile

struct RouteMap {
    // l = base + sh * h + sw * w ; col_like: |sh| == 1 (contiguous along h)
    long long base, sh, sw;
    int col_like;
};

__host__ __device__ inline RouteMap route_map(int scans, int k, long long H, long long W) {
    const long long L = H * W;
    RouteMap m;
    auto row_f = [&]() { m.base = 0; m.sh = W; m.sw = 1; m.col_like = 0; };
    auto row_r = [&]() { m.base = L - 1; m.sh = -W; m.sw = -1; m.col_like = 0; };
    auto col_f = [&]() { m.base = 0; m.sh = 1; m.sw = H; m.col_like = 1; };
    auto col_r = [&]() { m.base = L - 1; m.sh = -1; m.sw = -H; m.col_like = 1; };
    if (scans == 0) { if (k == 0) row_f(); else if (k == 1) col_f(); else if (k == 2) row_r(); else col_r(); }
    else if (scans == 1) row_f();
    else if (scans == 2) { if (k < 2) row_f(); else row_r(); }
    else {
        // rotations: k=1 -> l = (W-1-w)*H + h ; k=3 -> l = w*H + (H-1-h)
        if (k == 0) row_f();
        else if (k == 1) { m.base = (W - 1) * H; m.sh = 1; m.sw = -H; m.col_like = 1; }
        else if (k == 2) row_r();
        else { m.base = H - 1; m.sh = -1; m.sw = H; m.col_like = 1; }
    }
    return m;
}

struct CrossArgs {
    const void* in;
    void* out;
    long long C, H, W, tiles_h, tiles_w, n_tiles;
    RouteMap route[4];
};

template <typename T>
__global__ void __launch_bounds__(kTile * kRowsPerPass) cross_scan_kernel(const CrossArgs a) {
    __shared__ T tile[kTile][kTile + 1];
    const long long t = blockIdx.x;
    const long long tw = t % a.tiles_w, th = (t / a.tiles_w) % a.tiles_h, plane = t / (a.tiles_w * a.tiles_h);
    const long long b = plane / a.C, c = plane % a.C, L = a.H * a.W;
    const T* __restrict__ x = (const T*)a.in + plane * L;
    const long long h0 = th * kTile, w0 = tw * kTile;
    const int tx = threadIdx.x, ty = threadIdx.y;
#pragma unroll
    for (int j = 0; j < kTile; j += kRowsPerPass) {
        const long long h = h0 + ty + j, w = w0 + tx;
        if (h < a.H && w < a.W) tile[ty + j][tx] = x[h * a.W + w];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const RouteMap m = a.route[k];
        T* __restrict__ y = (T*)a.out + ((b * 4 + k) * a.C + c) * L;
#pragma unroll
        for (int j = 0; j < kTile; j += kRowsPerPass) {
            // row-like: thread x index runs along w; column-like: along h (transposed read)
            const int lh = m.col_like ? tx : ty + j, lw = m.col_like ? ty + j : tx;
            const long long h = h0 + lh, w = w0 + lw;
            if (h < a.H && w < a.W) y[m.base + m.sh * h + m.sw * w] = tile[lh][lw];
        }
    }
}

// Rounds to the storage type after every addition, as elementwise tensor additions do.
template <typename T> __device__ __forceinline__ T add_t(T x, T y) { return from_f<T>(to_f<T>(x) + to_f<T>(y)); }

template <typename T>
__global__ void __launch_bounds__(kTile * kRowsPerPass) cross_merge_kernel(const CrossArgs a, const int scans) {
    __shared__ T tile[4][kTile][kTile + 1];
    const long long t = blockIdx.x;
    const long long tw = t % a.tiles_w, th = (t / a.tiles_w) % a.tiles_h, plane = t / (a.tiles_w * a.tiles_h);
    const long long b = plane / a.C, c = plane % a.C, L = a.H * a.W;
    const long long h0 = th * kTile, w0 = tw * kTile;
    const int tx = threadIdx.x, ty = threadIdx.y;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const RouteMap m = a.route[k];
        const T* __restrict__ ys = (const T*)a.in + ((b * 4 + k) * a.C + c) * L;
#pragma unroll
        for (int j = 0; j < kTile; j += kRowsPerPass) {
            const int lh = m.col_like ? tx : ty + j, lw = m.col_like ? ty + j : tx;
            const long long h = h0 + lh, w = w0 + lw;
            if (h < a.H && w < a.W) tile[k][lh][lw] = ys[m.base + m.sh * h + m.sw * w];
        }
    }
    __syncthreads();
    T* __restrict__ y = (T*)a.out + plane * L;
#pragma unroll
    for (int j = 0; j < kTile; j += kRowsPerPass) {
        const long long h = h0 + ty + j, w = w0 + tx;
        if (h < a.H && w < a.W) {
            const T v0 = tile[0][ty + j][tx], v1 = tile[1][ty + j][tx], v2 = tile[2][ty + j][tx], v3 = tile[3][ty + j][tx];
            T r;
            if (scans == 0 || scans == 2) r = add_t(add_t(v0, v2), add_t(v1, v3));   // (y0+y2) + (y1+y3)
            else if (scans == 3) r = add_t(add_t(add_t(v0, v1), v2), v3);            // ((y0+y1)+y2)+y3
            else r = from_f<T>(((to_f<T>(v0) + to_f<T>(v1)) + to_f<T>(v2)) + to_f<T>(v3));   // one reduction, rounded once
            y[h * a.W + w] = r;
        }
    }
}

static int fill_args(const ss2d_cross_params* p, CrossArgs& a) {
    if (!p) return SS2D_EINVAL_NULL;
    if (!p->in || !p->out) return SS2D_EINVAL_NULL;
    if (!dtype_ok(p->dtype)) return SS2D_EINVAL_DTYPE;
    if (p->scans < 0 || p->scans > 3) return SS2D_ENOTSUP;
    if (p->B <= 0 || p->C <= 0 || p->H <= 0 || p->W <= 0) return SS2D_EINVAL_SHAPE;
    const size_t s = dtype_size(p->dtype);
    if (!aligned_to(p->in, s) || !aligned_to(p->out, s)) return SS2D_EINVAL_ALIGN;
    a.in = p->in; a.out = p->out;
    a.C = p->C; a.H = p->H; a.W = p->W;
    a.tiles_h = (p->H + kTile - 1) / kTile;
    a.tiles_w = (p->W + kTile - 1) / kTile;
    a.n_tiles = a.tiles_h * a.tiles_w * p->B * p->C;
    if (a.n_tiles > 0x7fffffffLL) return SS2D_EINVAL_SHAPE;
    for (int k = 0; k < 4; ++k) a.route[k] = route_map(p->scans, k, p->H, p->W);
    return SS2D_OK;
}

int cross_scan(const ss2d_cross_params* p, cudaStream_t st) {
    CrossArgs a;
    const int rc = fill_args(p, a);
    if (rc != SS2D_OK) return rc;
    const dim3 blk(kTile, kRowsPerPass);
    if (p->dtype == SS2D_F32) cross_scan_kernel<float><<<(unsigned)a.n_tiles, blk, 0, st>>>(a);
    else cross_scan_kernel<uint16_t><<<(unsigned)a.n_tiles, blk, 0, st>>>(a);   // 16-bit types: bits are moved as-is
    count_launch();
    return check_launch();
}

int cross_merge(const ss2d_cross_params* p, cudaStream_t st) {
    CrossArgs a;
    const int rc = fill_args(p, a);
    if (rc != SS2D_OK) return rc;
    const dim3 blk(kTile, kRowsPerPass);
    if (p->dtype == SS2D_F32) cross_merge_kernel<float><<<(unsigned)a.n_tiles, blk, 0, st>>>(a, p->scans);
    else if (p->dtype == SS2D_BF16) cross_merge_kernel<__nv_bfloat16><<<(unsigned)a.n_tiles, blk, 0, st>>>(a, p->scans);
    else cross_merge_kernel<__half><<<(unsigned)a.n_tiles, blk, 0, st>>>(a, p->scans);
    count_launch();
    return check_launch();
}

}  // namespace ss2d
