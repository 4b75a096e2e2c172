// CrossScan / CrossMerge as stand-alone tensor-to-tensor operators (channel-first).
//
// Every route is an index map  (h, w) -> l  that is contiguous either along w ("row-like")
// or along h ("column-like").  A CTA owns one 32x32 tile of one (b, c) plane: the tile is read
// (scan) or written (merge) with w fastest, column-like routes go through a padded shared-memory
// transpose so that both the global reads and the global writes of every route are coalesced.
// Data movement only: results are bit-identical to indexing.
#include <algorithm>

#include "common.cuh"

namespace ss2d {

constexpr int kTile = 32;
constexpr int kRowsPerPass = 4;   // CrossScan tile kernel: CTA = 32 x 4 threads, eight passes per tile
constexpr int kMergeRows = 2;     // CrossMerge tile kernel: CTA = 32 x 2 threads (512 planes of 256 x 256: scan 143 / 131 / 142 us, merge 250 / 226 / 197 us with 8 / 4 / 2 rows)

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

// Index arithmetic inside a plane is 32-bit (the callers bound H * W and the tile count by 2^31): with 64-bit
// divisions and products the kernels issued about 200 instructions per element and were bound by that.
template <typename T>
__global__ void __launch_bounds__(kTile * kRowsPerPass) cross_scan_kernel(const CrossArgs a) {
    __shared__ T tile[kTile][kTile + 1];
    const unsigned t = blockIdx.x, tiles_w = (unsigned)a.tiles_w, tiles_h = (unsigned)a.tiles_h, C = (unsigned)a.C;
    const unsigned tw = t % tiles_w, rest = t / tiles_w, th = rest % tiles_h, plane = rest / tiles_h;
    const unsigned b = plane / C, c = plane - b * C;
    const int H = (int)a.H, W = (int)a.W, L = H * W;
    const T* __restrict__ x = (const T*)a.in + (long long)plane * L;
    const int h0 = (int)th * kTile, w0 = (int)tw * kTile;
    const int tx = threadIdx.x, ty = threadIdx.y;
#pragma unroll
    for (int j = 0; j < kTile; j += kRowsPerPass) {
        const int h = h0 + ty + j, w = w0 + tx;
        if (h < H && w < W) tile[ty + j][tx] = x[h * W + w];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int base = (int)a.route[k].base, sh = (int)a.route[k].sh, sw = (int)a.route[k].sw;
        const bool col_like = a.route[k].col_like != 0;
        T* __restrict__ y = (T*)a.out + ((long long)(b * 4 + k) * C + c) * L;
#pragma unroll
        for (int j = 0; j < kTile; j += kRowsPerPass) {
            // row-like: thread x index runs along w; column-like: along h (transposed read)
            const int lh = col_like ? tx : ty + j, lw = col_like ? ty + j : tx;
            const int h = h0 + lh, w = w0 + lw;
            if (h < H && w < W) y[base + sh * h + sw * w] = tile[lh][lw];
        }
    }
}

// 16-bit maps with even H and W: a thread moves PAIRS of elements as one 32-bit word.  A 2-byte access per lane runs the
// load/store unit at a fraction of its rate (the kernel above reached 0.24 of the copy bandwidth on 256 x 256 bf16
// planes).  Tile: 64 x 64 elements = 32 words along the fast index of either orientation; a reversed route writes the
// pair at the mirrored address with its halves swapped.
constexpr int kPairTile = 64;
__global__ void __launch_bounds__(256) cross_scan_pair_kernel(const CrossArgs a) {
    __shared__ __align__(4) uint16_t tile[kPairTile][kPairTile + 2];       // pitch 33 words
    const unsigned t = blockIdx.x, tiles_w = (unsigned)a.tiles_w, tiles_h = (unsigned)a.tiles_h, C = (unsigned)a.C;
    const unsigned tw = t % tiles_w, rest = t / tiles_w, th = rest % tiles_h, plane = rest / tiles_h;
    const unsigned b = plane / C, c = plane - b * C;
    const int H = (int)a.H, W = (int)a.W, L = H * W;
    const uint16_t* __restrict__ x = (const uint16_t*)a.in + (long long)plane * L;
    const int h0 = (int)th * kPairTile, w0 = (int)tw * kPairTile;
    const int tx = threadIdx.x, ty = threadIdx.y;          // 32 x 8
#pragma unroll
    for (int j = 0; j < kPairTile; j += 8) {
        const int h = h0 + ty + j, w = w0 + 2 * tx;
        if (h < H && w < W) *reinterpret_cast<uint32_t*>(&tile[ty + j][2 * tx]) = *reinterpret_cast<const uint32_t*>(x + h * W + w);
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int base = (int)a.route[k].base, sh = (int)a.route[k].sh, sw = (int)a.route[k].sw;
        const bool col_like = a.route[k].col_like != 0;
        uint16_t* __restrict__ y = (uint16_t*)a.out + ((long long)(b * 4 + k) * C + c) * L;
#pragma unroll
        for (int j = 0; j < kPairTile; j += 8) {
            // the pair runs along w (row-like) or along h (column-like); `step` is the route's stride along the pair
            const int lh = col_like ? 2 * tx : ty + j, lw = col_like ? ty + j : 2 * tx;
            const int h = h0 + lh, w = w0 + lw;
            if (h < H && w < W) {
                const uint32_t e0 = col_like ? tile[lh][lw] : tile[lh][lw];
                const uint32_t e1 = col_like ? tile[lh + 1][lw] : tile[lh][lw + 1];
                const int step = col_like ? sh : sw;               // +1 or -1
                const int l0 = base + sh * h + sw * w;
                if (step > 0) *reinterpret_cast<uint32_t*>(y + l0) = e0 | (e1 << 16);
                else *reinterpret_cast<uint32_t*>(y + l0 - 1) = e1 | (e0 << 16);
            }
        }
    }
}

// Rounds to the storage type after every addition, as elementwise tensor additions do.
template <typename T> __device__ __forceinline__ T add_t(T x, T y) { return from_f<T>(to_f<T>(x) + to_f<T>(y)); }

template <typename T>
__global__ void __launch_bounds__(kTile * kMergeRows) cross_merge_kernel(const CrossArgs a, const int scans) {
    __shared__ T tile[2][kTile][kTile + 1];               // the column-like routes (at most two); the others are read in place
    const unsigned t = blockIdx.x, tiles_w = (unsigned)a.tiles_w, tiles_h = (unsigned)a.tiles_h, C = (unsigned)a.C;
    const unsigned tw = t % tiles_w, rest = t / tiles_w, th = rest % tiles_h, plane = rest / tiles_h;
    const unsigned b = plane / C, c = plane - b * C;
    const int H = (int)a.H, W = (int)a.W, L = H * W;
    const int h0 = (int)th * kTile, w0 = (int)tw * kTile;
    const int tx = threadIdx.x, ty = threadIdx.y;
    int slot[4], nslots = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) slot[k] = a.route[k].col_like ? nslots++ : -1;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        if (slot[k] < 0) continue;
        const int base = (int)a.route[k].base, sh = (int)a.route[k].sh, sw = (int)a.route[k].sw;
        const T* __restrict__ ys = (const T*)a.in + ((long long)(b * 4 + k) * C + c) * L;
#pragma unroll
        for (int j = 0; j < kTile; j += kMergeRows) {
            const int lh = tx, lw = ty + j;               // thread x index runs along h: the route's contiguous direction
            const int h = h0 + lh, w = w0 + lw;
            if (h < H && w < W) tile[slot[k]][lh][lw] = ys[base + sh * h + sw * w];
        }
    }
    // the row-like routes' values of this thread's output elements: their loads fly together with the ones above
    T direct[4][kTile / kMergeRows];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        if (slot[k] >= 0) continue;
        const int base = (int)a.route[k].base, sh = (int)a.route[k].sh, sw = (int)a.route[k].sw;
        const T* __restrict__ ys = (const T*)a.in + ((long long)(b * 4 + k) * C + c) * L;
#pragma unroll
        for (int j = 0; j < kTile; j += kMergeRows) {
            const int h = h0 + ty + j, w = w0 + tx;
            if (h < H && w < W) direct[k][j / kMergeRows] = ys[base + sh * h + sw * w];
        }
    }
    __syncthreads();
    T* __restrict__ y = (T*)a.out + (long long)plane * L;
#pragma unroll
    for (int j = 0; j < kTile; j += kMergeRows) {
        const int h = h0 + ty + j, w = w0 + tx;
        if (h < H && w < W) {
            T v[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) v[k] = slot[k] >= 0 ? tile[slot[k]][ty + j][tx] : direct[k][j / kMergeRows];
            T r;
            if (scans == 0 || scans == 2) r = add_t(add_t(v[0], v[2]), add_t(v[1], v[3]));   // (y0+y2) + (y1+y3)
            else if (scans == 3) r = add_t(add_t(add_t(v[0], v[1]), v[2]), v[3]);            // ((y0+y1)+y2)+y3
            else r = from_f<T>(((to_f<T>(v[0]) + to_f<T>(v[1])) + to_f<T>(v[2])) + to_f<T>(v[3]));   // one reduction, rounded once
            y[h * W + w] = r;
        }
    }
}

// ---- whole-plane variants for maps that fit in shared memory ------------------------------------------
// The tile kernels above leave most of a 32x32 tile idle on small maps (14x14, 7x7) and move one
// element per lane.  Here a CTA owns PP whole planes: they are copied into shared memory with
// flat vector loads, and every route is then produced (scan) or consumed (merge) as a flat run of
// vectors in ITS OWN index order, so all global traffic is contiguous 16-byte vectors; the
// permutation happens on the shared-memory side.
struct PlaneArgs {
    const void* in;
    void* out;
    long long planes;          // B * C
    int C, H, W, L, PP, nvec;  // nvec = L / PV
    RouteMap route[4];
    unsigned magic_H, magic_W, magic_nvec;
};

__device__ __forceinline__ int mdiv_u(int n, unsigned magic) { return magic ? (int)__umulhi((unsigned)n, magic) : n; }

// the same map with 32-bit fields (positions inside a plane fit): keeps 64-bit products out of the inner loops
struct RouteMapI { int base, sh, sw, col_like; };
__device__ __forceinline__ RouteMapI narrow(const RouteMap& m) { return RouteMapI{(int)m.base, (int)m.sh, (int)m.sw, (int)m.col_like}; }

// source position (flat h*W + w) read by step l of a route
__device__ __forceinline__ int route_src(const RouteMapI& m, int l, int H, int W, unsigned magic_H) {
    if (!m.col_like) return m.sw > 0 ? l : (int)m.base - l;            // row-major, forward or reversed
    // l = base + sh*h + sw*w with |sh| = 1, |sw| = H: recover (h, w)
    const int t = (int)(m.sw > 0 ? 0 : -m.sw * (W - 1));                // offset so that the w term is non-negative
    int r = l - (int)m.base + t + (m.sh < 0 ? (H - 1) : 0);            // = hh + H * ww with hh, ww in range
    const int ww = mdiv_u(r, magic_H), hh = r - ww * H;
    const int h = m.sh > 0 ? hh : H - 1 - hh;
    const int w = m.sw > 0 ? ww : W - 1 - ww;
    return h * W + w;
}

// Shared-memory planes have an odd line pitch (W | 1 for a row-major plane, H | 1 for a column-major one): the gathers of
// the permutation then walk down a line with consecutive lanes in different banks.  With the natural pitch (56 for a
// 56 x 56 map) 32 lanes fell into 4 banks and the kernels ran at a third of the copy bandwidth.
template <typename T, int PV>
__global__ void __launch_bounds__(256) cross_scan_plane_kernel(const PlaneArgs a) {
    extern __shared__ __align__(16) unsigned char smraw[];
    T* sm = reinterpret_cast<T*>(smraw);                   // [PP][H][Wp]
    const long long plane0 = (long long)blockIdx.x * a.PP;
    const int np = (int)min((long long)a.PP, a.planes - plane0);
    const int L = a.L, n = np * a.nvec, W = a.W, H = a.H, Wp = W | 1, Lp = H * Wp;
    const T* __restrict__ x = (const T*)a.in + plane0 * L;
    RouteMapI rm[4];
    bool any_col = false;
#pragma unroll
    for (int k = 0; k < 4; ++k) { rm[k] = narrow(a.route[k]); any_col = any_col || rm[k].col_like; }
    // ---- every vector of x: straight out for the row-major routes (as it is, or mirrored with its elements reversed),
    //      into the padded shared plane for the column-major ones
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int pl = mdiv_u(i, a.magic_nvec), p0 = (i - pl * a.nvec) * PV;
        const unsigned plane = (unsigned)plane0 + (unsigned)pl;                // B * C < 2^31 (checked by the caller)
        const unsigned b = plane / (unsigned)a.C, c = plane - b * (unsigned)a.C;
        const typename Vec<T, PV>::Raw r = Vec<T, PV>::load_raw(x + (long long)i * PV);
        const T* e = reinterpret_cast<const T*>(&r);
        typename Vec<T, PV>::Raw rev;
        T* er = reinterpret_cast<T*>(&rev);
#pragma unroll
        for (int j = 0; j < PV; ++j) er[j] = e[PV - 1 - j];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (rm[k].col_like) continue;
            T* dst = (T*)a.out + ((long long)(b * 4 + k) * a.C + c) * L;
            if (rm[k].sw > 0) Vec<T, PV>::store_raw(dst + p0, r);
            else Vec<T, PV>::store_raw(dst + (L - PV - p0), rev);
        }
        if (any_col) {
            int h = mdiv_u(p0, a.magic_W), w = p0 - h * W;
            T* dst = sm + pl * Lp;
#pragma unroll
            for (int j = 0; j < PV; ++j) {
                dst[h * Wp + w] = e[j];
                if (++w == W) { w = 0; ++h; }
            }
        }
    }
    if (!any_col) return;                                  // uniform over the grid
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const RouteMapI m = rm[k];
        if (!m.col_like) continue;
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            const int pl = mdiv_u(i, a.magic_nvec), l0 = (i - pl * a.nvec) * PV;
            const unsigned plane = (unsigned)plane0 + (unsigned)pl;
            const unsigned b = plane / (unsigned)a.C, c = plane - b * (unsigned)a.C;
            typename Vec<T, PV>::Raw r;
            T* e = reinterpret_cast<T*>(&r);
            const T* src = sm + pl * Lp;
            // column-major route: l - base = sh * h + sw * w with |sh| = 1, |sw| = H; walk h first
            const int t = (int)(m.sw > 0 ? 0 : -m.sw * (W - 1));
            const int r0 = l0 - m.base + t + (m.sh < 0 ? (H - 1) : 0);     // = hh + H * ww with hh, ww in range
            int ww = mdiv_u(r0, a.magic_H), hh = r0 - ww * H;
#pragma unroll
            for (int j = 0; j < PV; ++j) {
                const int h = m.sh > 0 ? hh : H - 1 - hh, w = m.sw > 0 ? ww : W - 1 - ww;
                e[j] = src[h * Wp + w];
                if (++hh == H) { hh = 0; ++ww; }
            }
            Vec<T, PV>::store_raw((T*)a.out + ((long long)(b * 4 + k) * a.C + c) * L + l0, r);
        }
    }
}

// Row-major routes (forward or reversed) are read straight from global memory as the vectors the output wants; only
// the column-major routes (at most two) pass through shared memory, each plane in its own order with an odd line pitch.
template <typename T, int PV>
__global__ void __launch_bounds__(256) cross_merge_plane_kernel(const PlaneArgs a, const int scans) {
    extern __shared__ __align__(16) unsigned char smraw[];
    T* sm = reinterpret_cast<T*>(smraw);                   // [2][PP][W][H | 1]
    const long long plane0 = (long long)blockIdx.x * a.PP;
    const int np = (int)min((long long)a.PP, a.planes - plane0);
    const int L = a.L, n = np * a.nvec, W = a.W, H = a.H;
    const int Hp = H | 1, Lp = W * Hp;
    RouteMapI rm[4];
    int slot[4], nslots = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        rm[k] = narrow(a.route[k]);
        slot[k] = -1;
        if (rm[k].col_like) {
            slot[k] = nslots++;
            const int b_lo = rm[k].base % H, b_hi = rm[k].base / H;
            rm[k].base = b_lo + Hp * b_hi;
            rm[k].sw = rm[k].sw > 0 ? Hp : -Hp;
        }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        if (slot[k] < 0) continue;
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            const int pl = mdiv_u(i, a.magic_nvec), l0 = (i - pl * a.nvec) * PV;
            const unsigned plane = (unsigned)plane0 + (unsigned)pl;
            const unsigned b = plane / (unsigned)a.C, c = plane - b * (unsigned)a.C;
            const typename Vec<T, PV>::Raw r = Vec<T, PV>::load_raw((const T*)a.in + ((long long)(b * 4 + k) * a.C + c) * L + l0);
            const T* e = reinterpret_cast<const T*>(&r);
            int line = mdiv_u(l0, a.magic_H), pos = l0 - line * H;
            T* dst = sm + (slot[k] * a.PP + pl) * Lp;
#pragma unroll
            for (int j = 0; j < PV; ++j) {
                dst[line * Hp + pos] = e[j];
                if (++pos == H) { pos = 0; ++line; }
            }
        }
    }
    __syncthreads();
    T* __restrict__ y = (T*)a.out + plane0 * L;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int pl = mdiv_u(i, a.magic_nvec), p0 = (i - pl * a.nvec) * PV;
        const unsigned plane = (unsigned)plane0 + (unsigned)pl;
        const unsigned b = plane / (unsigned)a.C, c = plane - b * (unsigned)a.C;
        T v[4][PV];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (slot[k] >= 0) continue;
            const T* src = (const T*)a.in + ((long long)(b * 4 + k) * a.C + c) * L;
            const bool fwd = rm[k].sw > 0;
            const typename Vec<T, PV>::Raw r = Vec<T, PV>::load_raw(src + (fwd ? p0 : L - PV - p0));
            const T* e = reinterpret_cast<const T*>(&r);
#pragma unroll
            for (int j = 0; j < PV; ++j) v[k][j] = e[fwd ? j : PV - 1 - j];
        }
        int h = mdiv_u(p0, a.magic_W), w = p0 - h * W;
#pragma unroll
        for (int j = 0; j < PV; ++j) {
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (slot[k] >= 0) v[k][j] = sm[(slot[k] * a.PP + pl) * Lp + rm[k].base + rm[k].sh * h + rm[k].sw * w];
            if (++w == W) { w = 0; ++h; }
        }
        typename Vec<T, PV>::Raw r;
        T* e = reinterpret_cast<T*>(&r);
#pragma unroll
        for (int j = 0; j < PV; ++j) {
            if (scans == 0 || scans == 2) e[j] = add_t(add_t(v[0][j], v[2][j]), add_t(v[1][j], v[3][j]));
            else if (scans == 3) e[j] = add_t(add_t(add_t(v[0][j], v[1][j]), v[2][j]), v[3][j]);
            else e[j] = from_f<T>(((to_f<T>(v[0][j]) + to_f<T>(v[1][j])) + to_f<T>(v[2][j])) + to_f<T>(v[3][j]));
        }
        Vec<T, PV>::store_raw(y + (long long)i * PV, r);
    }
}

// returns false when the map is too large for the whole-plane kernels
template <typename T>
static bool plan_plane(const ss2d_cross_params* p, int copies, PlaneArgs& a, int& pv, size_t& smem) {
    const long long L = p->H * p->W;
    // shared-memory room of one plane with its odd line pitch (the merge keeps planes of either orientation)
    const long long Lp = copies == 1 ? p->H * (p->W | 1) : p->W * (p->H | 1);    // scan: x row-major; merge: column-major routes
    if (Lp * (long long)sizeof(T) * copies > 64 * 1024) return false;
    pv = 16 / (int)sizeof(T);
    auto fit = [&](long long x) { while (pv > 1 && (x % pv) != 0) pv >>= 1; };
    fit(L);
    fit((long long)(reinterpret_cast<uintptr_t>(p->in) / sizeof(T)));
    fit((long long)(reinterpret_cast<uintptr_t>(p->out) / sizeof(T)));
    long long PP = (4096 + L - 1) / L;        // about 4096 elements per CTA
    while (PP > 1 && PP * Lp * (long long)sizeof(T) * copies > 64 * 1024) --PP;
    a.in = p->in; a.out = p->out; a.planes = p->B * p->C; a.C = (int)p->C; a.H = (int)p->H; a.W = (int)p->W;
    a.L = (int)L; a.PP = (int)PP; a.nvec = (int)(L / pv);
    for (int k = 0; k < 4; ++k) a.route[k] = route_map(p->scans, k, p->H, p->W);
    auto magic = [](long long d) { return d > 1 ? (unsigned)(((1ULL << 32) + (unsigned long long)d - 1) / (unsigned long long)d) : 0u; };
    a.magic_H = magic(p->H); a.magic_W = magic(p->W); a.magic_nvec = magic(a.nvec);
    smem = (size_t)PP * Lp * sizeof(T) * copies;
    return (a.planes + PP - 1) / PP <= 0x7fffffffLL;
}

template <typename T, int PV>
static int launch_scan_plane(const PlaneArgs& a, size_t smem, cudaStream_t st) {
    auto k = cross_scan_plane_kernel<T, PV>;
    if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return SS2D_ECUDA;
    k<<<(unsigned)((a.planes + a.PP - 1) / a.PP), 256, smem, st>>>(a);
    count_launch();
    return check_launch();
}
template <typename T, int PV>
static int launch_merge_plane(const PlaneArgs& a, int scans, size_t smem, cudaStream_t st) {
    auto k = cross_merge_plane_kernel<T, PV>;
    if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return SS2D_ECUDA;
    k<<<(unsigned)((a.planes + a.PP - 1) / a.PP), 256, smem, st>>>(a, scans);
    count_launch();
    return check_launch();
}
template <typename T>
static int scan_plane_v(const PlaneArgs& a, int pv, size_t smem, cudaStream_t st) {
    if constexpr (sizeof(T) == 2) { if (pv == 8) return launch_scan_plane<T, 8>(a, smem, st); }
    if (pv >= 4) return launch_scan_plane<T, 4>(a, smem, st);
    if (pv == 2) return launch_scan_plane<T, 2>(a, smem, st);
    return launch_scan_plane<T, 1>(a, smem, st);
}
template <typename T>
static int merge_plane_v(const PlaneArgs& a, int scans, int pv, size_t smem, cudaStream_t st) {
    if constexpr (sizeof(T) == 2) { if (pv == 8) return launch_merge_plane<T, 8>(a, scans, smem, st); }
    if (pv >= 4) return launch_merge_plane<T, 4>(a, scans, smem, st);
    if (pv == 2) return launch_merge_plane<T, 2>(a, scans, smem, st);
    return launch_merge_plane<T, 1>(a, scans, smem, st);
}

static int fill_args(const ss2d_cross_params* p, CrossArgs& a) {
    if (!p) return SS2D_EINVAL_NULL;
    if (!p->in || !p->out) return SS2D_EINVAL_NULL;
    if (!dtype_ok(p->dtype)) return SS2D_EINVAL_DTYPE;
    if (p->scans < 0 || p->scans > 3) return SS2D_ENOTSUP;
    if (p->B <= 0 || p->C <= 0 || p->H <= 0 || p->W <= 0) return SS2D_EINVAL_SHAPE;
    if (p->H * p->W > 0x3fffffffLL || p->C > 0x7fffffffLL || p->B * p->C > 0x7fffffffLL) return SS2D_EINVAL_SHAPE;   // 32-bit indices inside a plane
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
    // 16-bit maps with even sides: the pair kernel for every map that fills most of a 64 x 64 tile (0.87 of the copy
    // bandwidth on 256 x 256 planes against 0.60 for the whole-plane kernel on 128 x 128 ones)
    const bool pairs = p->dtype != SS2D_F32 && p->H % 2 == 0 && p->W % 2 == 0 && aligned_to(p->in, 4) && aligned_to(p->out, 4);
    if (!(pairs && p->H >= 48 && p->W >= 48)) {
        PlaneArgs pa; int pv; size_t smem;
        if (p->dtype == SS2D_F32) { if (plan_plane<float>(p, 1, pa, pv, smem)) return scan_plane_v<float>(pa, pv, smem, st); }
        else if (plan_plane<uint16_t>(p, 1, pa, pv, smem)) return scan_plane_v<uint16_t>(pa, pv, smem, st);
    }
    if (pairs) {
        CrossArgs q = a;
        q.tiles_h = (p->H + kPairTile - 1) / kPairTile;
        q.tiles_w = (p->W + kPairTile - 1) / kPairTile;
        q.n_tiles = q.tiles_h * q.tiles_w * p->B * p->C;
        cross_scan_pair_kernel<<<(unsigned)q.n_tiles, dim3(32, 8), 0, st>>>(q);
        count_launch();
        return check_launch();
    }
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
    {
        PlaneArgs pa; int pv; size_t smem;
        if (p->dtype == SS2D_F32) { if (plan_plane<float>(p, 2, pa, pv, smem)) return merge_plane_v<float>(pa, p->scans, pv, smem, st); }
        else if (p->dtype == SS2D_BF16) { if (plan_plane<__nv_bfloat16>(p, 2, pa, pv, smem)) return merge_plane_v<__nv_bfloat16>(pa, p->scans, pv, smem, st); }
        else if (plan_plane<__half>(p, 2, pa, pv, smem)) return merge_plane_v<__half>(pa, p->scans, pv, smem, st);
    }
    const dim3 blk(kTile, kMergeRows);
    if (p->dtype == SS2D_F32) cross_merge_kernel<float><<<(unsigned)a.n_tiles, blk, 0, st>>>(a, p->scans);
    else if (p->dtype == SS2D_BF16) cross_merge_kernel<__nv_bfloat16><<<(unsigned)a.n_tiles, blk, 0, st>>>(a, p->scans);
    else cross_merge_kernel<__half><<<(unsigned)a.n_tiles, blk, 0, st>>>(a, p->scans);
    count_launch();
    return check_launch();
}

// ------------------------------------------------------------------------------------------------
// Layout and one-by-one variants (channel-last x and / or routes; every route reading its own map):
// index-only variants of the two operators, off the benchmarked path.  One thread per (image, pixel,
// channel) handles the four routes; the fastest thread index follows the contiguous axis of the
// routes tensor (pixels for channel-first routes, channels for channel-last ones).
struct CrossExArgs {
    const void* in;
    void* out;
    RouteMap route[4];
    long long B, C, H, W, L, total;
    int x_cf, r_cf, one_by_one, scans;       // x / routes channel-first; every route has its own map
    int flat_1b1_copy;                       // one_by_one, scans 1: the four maps pass through unchanged
};

__device__ __forceinline__ long long x_index(const CrossExArgs& a, long long b, int k, long long c, long long p) {
    const long long K = a.one_by_one ? 4 : 1, kk = a.one_by_one ? k : 0;
    return a.x_cf ? ((b * K + kk) * a.C + c) * a.L + p : ((b * a.L + p) * K + kk) * a.C + c;
}
__device__ __forceinline__ long long r_index(const CrossExArgs& a, long long b, int k, long long c, long long l) {
    return a.r_cf ? ((b * 4 + k) * a.C + c) * a.L + l : ((b * a.L + l) * 4 + k) * a.C + c;
}
__device__ __forceinline__ void ex_decompose(const CrossExArgs& a, long long i, long long& b, long long& c, long long& p) {
    if (a.r_cf) { p = i % a.L; const long long t = i / a.L; c = t % a.C; b = t / a.C; }
    else { c = i % a.C; const long long t = i / a.C; p = t % a.L; b = t / a.L; }
}

template <typename T>
__global__ void __launch_bounds__(256) cross_scan_ex_kernel(const CrossExArgs a) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < a.total; i += (long long)gridDim.x * blockDim.x) {
        long long b, c, p;
        ex_decompose(a, i, b, c, p);
        const long long h = p / a.W, w = p - h * a.W;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const RouteMap& m = a.route[k];
            const long long l = a.flat_1b1_copy ? p : m.base + m.sh * h + m.sw * w;
            ((T*)a.out)[r_index(a, b, k, c, l)] = ((const T*)a.in)[x_index(a, b, k, c, p)];
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256) cross_merge_ex_kernel(const CrossExArgs a) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < a.total; i += (long long)gridDim.x * blockDim.x) {
        long long b, c, p;
        ex_decompose(a, i, b, c, p);
        const long long h = p / a.W, w = p - h * a.W;
        T v[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const RouteMap& m = a.route[k];
            const long long l = a.flat_1b1_copy ? p : m.base + m.sh * h + m.sw * w;
            v[k] = ((const T*)a.in)[r_index(a, b, k, c, l)];
        }
        if (a.one_by_one) {
#pragma unroll
            for (int k = 0; k < 4; ++k) ((T*)a.out)[x_index(a, b, k, c, p)] = v[k];
        } else {
            T r;
            if (a.scans == 0 || a.scans == 2) r = add_t(add_t(v[0], v[2]), add_t(v[1], v[3]));
            else if (a.scans == 3) r = add_t(add_t(add_t(v[0], v[1]), v[2]), v[3]);
            else r = from_f<T>(((to_f<T>(v[0]) + to_f<T>(v[1])) + to_f<T>(v[2])) + to_f<T>(v[3]));
            ((T*)a.out)[x_index(a, b, 0, c, p)] = r;
        }
    }
}

static int fill_ex(const ss2d_cross_ex_params* p, CrossExArgs& a) {
    if (!p) return SS2D_EINVAL_NULL;
    if (!p->in || !p->out) return SS2D_EINVAL_NULL;
    if (!dtype_ok(p->dtype)) return SS2D_EINVAL_DTYPE;
    if (p->scans < 0 || p->scans > 3) return SS2D_ENOTSUP;
    if (p->B <= 0 || p->C <= 0 || p->H <= 0 || p->W <= 0) return SS2D_EINVAL_SHAPE;
    if (p->scans == 3 && p->H != p->W) return SS2D_EINVAL_SHAPE;
    if (p->H * p->W > 0x3fffffffLL) return SS2D_EINVAL_SHAPE;
    // one map per route with a channel-last side: the route sets the reference's GPU kernel defines (csm_triton.py:313-336:
    // 0, 1 and 2; its torch branch for 2 indexes the wrong axes, csm_triton.py:117-123, and neither path has 3)
    if (p->one_by_one && !(p->in_channel_first && p->out_channel_first) && p->scans > 2) return SS2D_ENOTSUP;
    const size_t s = dtype_size(p->dtype);
    if (!aligned_to(p->in, s) || !aligned_to(p->out, s)) return SS2D_EINVAL_ALIGN;
    a.in = p->in; a.out = p->out;
    a.B = p->B; a.C = p->C; a.H = p->H; a.W = p->W; a.L = p->H * p->W; a.total = p->B * p->C * a.L;
    a.x_cf = p->in_channel_first ? 1 : 0; a.r_cf = p->out_channel_first ? 1 : 0;
    a.one_by_one = p->one_by_one ? 1 : 0; a.scans = p->scans;
    a.flat_1b1_copy = (p->one_by_one && p->scans == 1) ? 1 : 0;
    for (int k = 0; k < 4; ++k) a.route[k] = route_map(p->scans, k, p->H, p->W);
    return SS2D_OK;
}

template <typename T, bool kScan>
static int launch_ex(const CrossExArgs& a, cudaStream_t st) {
    long long ctas = (a.total + 255) / 256;
    if (ctas > 148LL * 32) ctas = 148LL * 32;
    if constexpr (kScan) cross_scan_ex_kernel<T><<<(unsigned)ctas, 256, 0, st>>>(a);
    else cross_merge_ex_kernel<T><<<(unsigned)ctas, 256, 0, st>>>(a);
    count_launch();
    return check_launch();
}

int cross_scan_ex(const ss2d_cross_ex_params* p, cudaStream_t st) {
    CrossExArgs a;
    const int rc = fill_ex(p, a);
    if (rc != SS2D_OK) return rc;
    if (p->dtype == SS2D_F32) return launch_ex<float, true>(a, st);
    return launch_ex<unsigned short, true>(a, st);           // 16-bit types: a copy does not look inside
}

int cross_merge_ex(const ss2d_cross_ex_params* p, cudaStream_t st) {
    CrossExArgs a;
    const int rc = fill_ex(p, a);
    if (rc != SS2D_OK) return rc;
    if (p->dtype == SS2D_F32) return launch_ex<float, false>(a, st);
    if (p->dtype == SS2D_BF16) return launch_ex<__nv_bfloat16, false>(a, st);
    return launch_ex<__half, false>(a, st);
}

}  // namespace ss2d
