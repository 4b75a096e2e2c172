// LayerNorm over the channel axis of a channel-first map, fp32 statistics, with an optional fused
// residual update:   s = in (+ add) (+ add_bias[d]);   [sum_out = s];   out = LN_D(s) * weight + bias.
//
// An "item" is PV consecutive pixels of one image; items are numbered across the whole batch so
// that every lane of every warp has work whatever the map size (L = 49 or 196 pixels per image
// would otherwise leave most of a tile empty).  threadIdx.x runs along the TX items of a CTA (a
// warp's global access is one contiguous run of PV*TX elements per channel, two channels per
// warp), threadIdx.y splits the D channels.  Mean and variance are the two-pass kind (sum of squared deviations), like the torch
// operator this replaces; values stay in registers between the passes when D / NTY fits, else
// they are re-read (from L1/L2).
#include "common.cuh"

namespace ss2d {

struct NormArgs {
    const float* in;
    const void* add;
    const float* add_bias;
    float* sum_out;
    const float *w, *b;
    void* out;
    long long bs, cs;        // element strides between images and between channels (pixels are contiguous)
    long long obs, ocs;      // the same for `out`
    int D, L, nv, items;     // nv = L / PV items per image, items = B * nv
    float eps;
    int skip_norm;           // 1: out = s converted, no statistics (a fused add + cast + layout change)
};

template <typename Tio, int NTY, int CACHE, int PV, int TX>
__global__ void __launch_bounds__(TX * NTY) layer_norm_cf_kernel(const NormArgs a) {
    __shared__ float red[NTY][TX][PV];
    const int tx = threadIdx.x, ty = threadIdx.y;
    const int item = blockIdx.x * TX + tx;
    const bool live = item < a.items;
    const int bimg = live ? item / a.nv : 0;
    const long long pix = (long long)(live ? (item - bimg * a.nv) : 0) * PV;
    const long long base = (long long)bimg * a.bs + pix;
    const float* __restrict__ src = a.in + base;
    const Tio* __restrict__ addp = a.add ? (const Tio*)a.add + base : nullptr;
    const int D = a.D;

    auto fetch = [&](int d, float (&v)[PV]) {
        if (!live) {
#pragma unroll
            for (int i = 0; i < PV; ++i) v[i] = 0.f;
            return;
        }
        const long long off = (long long)d * a.cs;
        if (a.in) Vec<float, PV>::load_plain(src + off, v);      // `in` may alias `sum_out`: no read-only path
        else {
#pragma unroll
            for (int i = 0; i < PV; ++i) v[i] = 0.f;
        }
        if (addp) {
            float t[PV];
            Vec<Tio, PV>::load(addp + off, t);
#pragma unroll
            for (int i = 0; i < PV; ++i) v[i] += t[i];
        }
        if (a.add_bias) {
            const float bb = __ldg(a.add_bias + d);
#pragma unroll
            for (int i = 0; i < PV; ++i) v[i] += bb;
        }
        if (a.sum_out) Vec<float, PV>::store(a.sum_out + base + off, v);
    };
    auto reduce_over_ty = [&](float (&v)[PV]) {
#pragma unroll
        for (int i = 0; i < PV; ++i) red[ty][tx][i] = v[i];
        __syncthreads();
#pragma unroll
        for (int i = 0; i < PV; ++i) {
            float s = 0.f;
#pragma unroll
            for (int j = 0; j < NTY; ++j) s += red[j][tx][i];
            v[i] = s;
        }
        __syncthreads();
    };

    float cache[CACHE > 0 ? CACHE : 1][PV];
    float s[PV];
#pragma unroll
    for (int i = 0; i < PV; ++i) s[i] = 0.f;
    if constexpr (CACHE > 0) {
        // All loads are issued before anything is stored: `sum_out` may be the buffer `in`, so a store
        // in between would order every later load behind it and leave one load in flight per warp.
        typename Vec<Tio, PV>::Raw addraw[CACHE];
#pragma unroll
        for (int c = 0; c < CACHE; ++c) {
            const int d = ty + c * NTY;
            if (live && d < D && a.in) Vec<float, PV>::load_plain(src + (long long)d * a.cs, cache[c]);
            else {
#pragma unroll
                for (int i = 0; i < PV; ++i) cache[c][i] = 0.f;
            }
        }
        if (addp) {
#pragma unroll
            for (int c = 0; c < CACHE; ++c) {
                const int d = ty + c * NTY;
                if (live && d < D) addraw[c] = Vec<Tio, PV>::load_raw(addp + (long long)d * a.cs);
            }
        }
#pragma unroll
        for (int c = 0; c < CACHE; ++c) {
            const int d = ty + c * NTY;
            if (live && d < D) {
                if (addp) {
                    float tv[PV];
                    Vec<Tio, PV>::unpack(addraw[c], tv);
#pragma unroll
                    for (int i = 0; i < PV; ++i) cache[c][i] += tv[i];
                }
                if (a.add_bias) {
                    const float bb = __ldg(a.add_bias + d);
#pragma unroll
                    for (int i = 0; i < PV; ++i) cache[c][i] += bb;
                }
            }
#pragma unroll
            for (int i = 0; i < PV; ++i) s[i] += cache[c][i];
        }
        if (a.sum_out && live) {
#pragma unroll
            for (int c = 0; c < CACHE; ++c) {
                const int d = ty + c * NTY;
                if (d < D) Vec<float, PV>::store(a.sum_out + base + (long long)d * a.cs, cache[c]);
            }
        }
    } else {
        for (int d = ty; d < D; d += NTY) {
            float v[PV];
            fetch(d, v);
#pragma unroll
            for (int i = 0; i < PV; ++i) s[i] += v[i];
        }
    }
    const bool norm = a.skip_norm == 0;      // uniform over the grid
    if (norm) reduce_over_ty(s);
    float mean[PV], q[PV];
#pragma unroll
    for (int i = 0; i < PV; ++i) { mean[i] = norm ? s[i] / (float)D : 0.f; q[i] = 0.f; }
    // after the first pass the sum lives in sum_out (if any): re-reads must not add again
    const float* __restrict__ again = a.sum_out ? a.sum_out + base : nullptr;
    auto refetch = [&](int d, float (&v)[PV]) {
        if (!live) {
#pragma unroll
            for (int i = 0; i < PV; ++i) v[i] = 0.f;
            return;
        }
        const long long off = (long long)d * a.cs;
        if (again) { Vec<float, PV>::load_plain(again + off, v); return; }
        if (a.in) Vec<float, PV>::load_plain(src + off, v);
        else {
#pragma unroll
            for (int i = 0; i < PV; ++i) v[i] = 0.f;
        }
        if (addp) {
            float t[PV];
            Vec<Tio, PV>::load(addp + off, t);
#pragma unroll
            for (int i = 0; i < PV; ++i) v[i] += t[i];
        }
        if (a.add_bias) {
            const float bb = __ldg(a.add_bias + d);
#pragma unroll
            for (int i = 0; i < PV; ++i) v[i] += bb;
        }
    };
    if (norm) {
        if constexpr (CACHE > 0) {
#pragma unroll
            for (int c = 0; c < CACHE; ++c) {
                if (ty + c * NTY < D) {
#pragma unroll
                    for (int i = 0; i < PV; ++i) { const float t = cache[c][i] - mean[i]; q[i] = fmaf(t, t, q[i]); }
                }
            }
        } else {
            for (int d = ty; d < D; d += NTY) {
                float v[PV];
                refetch(d, v);
#pragma unroll
                for (int i = 0; i < PV; ++i) { const float t = v[i] - mean[i]; q[i] = fmaf(t, t, q[i]); }
            }
        }
        reduce_over_ty(q);
    }
    if (!live) return;
    float rstd[PV];
#pragma unroll
    for (int i = 0; i < PV; ++i) rstd[i] = norm ? rsqrtf(q[i] / (float)D + a.eps) : 1.f;
    Tio* __restrict__ dst = (Tio*)a.out + (long long)bimg * a.obs + pix;
    auto emit = [&](int d, const float (&v)[PV]) {
        const float g = (norm && a.w) ? __ldg(a.w + d) : 1.f, be = (norm && a.b) ? __ldg(a.b + d) : 0.f;
        float o[PV];
#pragma unroll
        for (int i = 0; i < PV; ++i) o[i] = fmaf((v[i] - mean[i]) * rstd[i], g, be);
        Vec<Tio, PV>::store(dst + (long long)d * a.ocs, o);
    };
    if constexpr (CACHE > 0) {
#pragma unroll
        for (int c = 0; c < CACHE; ++c) {
            const int d = ty + c * NTY;
            if (d < D) emit(d, cache[c]);
        }
    } else {
        for (int d = ty; d < D; d += NTY) {
            float v[PV];
            refetch(d, v);
            emit(d, v);
        }
    }
}

// 16 items per CTA: CTAs of 128 to 512 threads, several per SM, so that the load phase of one overlaps the
// reduction / store phase of another (32 items per CTA, up to 1024 threads, was 12 % slower over a backbone
// forward); a warp's access is still one run of 16 * PV pixels per channel.
constexpr int kItemsPerCta = 16;

template <typename Tio, int NTY, int CACHE, int PV>
static void launch_one(const NormArgs& a, cudaStream_t st) {
    layer_norm_cf_kernel<Tio, NTY, CACHE, PV, kItemsPerCta>
        <<<(unsigned)((a.items + kItemsPerCta - 1) / kItemsPerCta), dim3(kItemsPerCta, NTY), 0, st>>>(a);
}

template <typename Tio>
static void launch_norm(NormArgs a, int pv, long long B, cudaStream_t st) {
    const int D = a.D;
    // registers hold CACHE * PV values per thread: at most 48 while D <= 192, at most 24 beyond
    // (more threads per CTA: keep about 64 registers per thread so that several CTAs share an SM)
    if (D > 32 * 32) pv = 1;
    else if (D > 16 * 12 && pv > 2) pv = 2;
    a.nv = a.L / pv;
    a.items = (int)(B * a.nv);
    if (D <= 8 * 12) {
        if (pv == 4) launch_one<Tio, 8, 12, 4>(a, st); else if (pv == 2) launch_one<Tio, 8, 12, 2>(a, st); else launch_one<Tio, 8, 12, 1>(a, st);
    } else if (D <= 16 * 12) {
        if (pv == 4) launch_one<Tio, 16, 12, 4>(a, st); else if (pv == 2) launch_one<Tio, 16, 12, 2>(a, st); else launch_one<Tio, 16, 12, 1>(a, st);
    } else if (D <= 32 * 12) {
        if (pv == 2) launch_one<Tio, 32, 12, 2>(a, st); else launch_one<Tio, 32, 12, 1>(a, st);
    } else if (D <= 32 * 24) {
        if (pv == 2) launch_one<Tio, 32, 24, 2>(a, st); else launch_one<Tio, 32, 24, 1>(a, st);
    } else if (D <= 32 * 32) {
        if (pv == 2) launch_one<Tio, 32, 32, 2>(a, st); else launch_one<Tio, 32, 32, 1>(a, st);
    } else if (D <= 32 * 48) {
        launch_one<Tio, 32, 48, 1>(a, st);
    } else if (D <= 32 * 64) {
        launch_one<Tio, 32, 64, 1>(a, st);
    } else {      // more channels than 512 threads can keep in registers: statistics pass, then re-read (from L2)
        launch_one<Tio, 32, 0, 1>(a, st);
    }
}

int layer_norm_cf(const ss2d_norm_params* p, cudaStream_t st) {
    if (!p) return SS2D_EINVAL_NULL;
    if ((!p->in && !p->add) || !p->out) return SS2D_EINVAL_NULL;
    if (!dtype_ok(p->io_dtype)) return SS2D_EINVAL_DTYPE;
    if (p->B <= 0 || p->D <= 0 || p->L <= 0) return SS2D_EINVAL_SHAPE;
    if (p->D > 0x7fffffffLL || p->B * p->L > 0x7fffffffLL) return SS2D_EINVAL_SHAPE;
    const long long bs = p->batch_stride ? p->batch_stride : p->D * p->L;
    const long long cs = p->channel_stride ? p->channel_stride : p->L;
    const long long obs = p->out_batch_stride ? p->out_batch_stride : bs;
    const long long ocs = p->out_channel_stride ? p->out_channel_stride : cs;
    if (cs < p->L || (p->B > 1 && bs < p->L) || ocs < p->L || (p->B > 1 && obs < p->L)) return SS2D_EINVAL_STRIDE;
    const size_t so = dtype_size(p->io_dtype);
    if (!aligned_to(p->in, 4) || !aligned_to(p->out, so) || !aligned_to(p->weight, 4) || !aligned_to(p->bias, 4) ||
        !aligned_to(p->add, so) || !aligned_to(p->add_bias, 4) || !aligned_to(p->sum_out, 4))
        return SS2D_EINVAL_ALIGN;
    int pv = 4;
    auto fit = [&](long long x) { if (x < 0) x = -x; while (pv > 1 && (x % pv) != 0) pv >>= 1; };
    fit(p->L); fit(bs); fit(cs); fit(obs); fit(ocs);
    if (p->in) fit((long long)(reinterpret_cast<uintptr_t>(p->in) / 4));
    fit((long long)(reinterpret_cast<uintptr_t>(p->out) / so));
    if (p->add) fit((long long)(reinterpret_cast<uintptr_t>(p->add) / so));
    if (p->sum_out) fit((long long)(reinterpret_cast<uintptr_t>(p->sum_out) / 4));
    NormArgs a;
    a.in = (const float*)p->in; a.add = p->add; a.add_bias = (const float*)p->add_bias; a.sum_out = (float*)p->sum_out;
    a.w = (const float*)p->weight; a.b = (const float*)p->bias; a.out = p->out;
    a.bs = bs; a.cs = cs; a.obs = obs; a.ocs = ocs; a.D = (int)p->D; a.L = (int)p->L; a.eps = p->eps; a.nv = 0; a.items = 0;
    a.skip_norm = p->skip_norm ? 1 : 0;
    if (p->io_dtype == SS2D_F32) launch_norm<float>(a, pv, p->B, st);
    else if (p->io_dtype == SS2D_BF16) launch_norm<__nv_bfloat16>(a, pv, p->B, st);
    else launch_norm<__half>(a, pv, p->B, st);
    count_launch();
    return check_launch();
}

}  // namespace ss2d
