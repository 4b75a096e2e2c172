// 1x1 projection of a channel-major map on the 5th-generation tensor cores:  out (M, N) = W (M, K) . x (K, N) (+ bias),
// N = B*H*W pixels contiguous in every row.  This is x_proj of the SS2D core computed on the un-scanned map (a 1x1
// projection commutes with the pixel permutation of CrossScan: vmamba.py:1536-1538, the grouped conv1d over the four
// routes is one matrix of 4 (R + 2N) rows here) and, with a bias, Linear2d.forward (vmamba.py:1062-1075).
//
// The output is skinny (M = 32 .. 104 rows against K = 96 .. 384 channels read for the x_proj shapes), so the kernel is
// bound by reading x once.  A persistent CTA per SM walks tiles of 128 pixels.  W stays in shared memory for the life of
// the CTA ([K / 32][M rows][64 B], K-major, loaded once by TMA); the x tile arrives in slices of up to 96 channels
// through a ring of TMA stages (two boxes of 64 pixels x slice rows: the "MN-major" operand form, pixels contiguous, no
// transpose anywhere); tcgen05.mma accumulates a tile into one of two TMEM accumulators (128 pixels x M fp32), so the
// tensor core works on tile t + 1 while eight warps move tile t from TMEM to global memory.  Warp 0 issues TMA, warp 1
// the MMAs.  What was measured on the way (VMamba-T stage 0, 32 x 96 . 96 x 401 408, CUDA-graph timing, inputs
// beyond L2): W re-fetched per slice and three TMA operations per 32-channel slice 36 us (a TMA operation costs the
// issuing thread about 170 cycles whatever its size); guarded 2-byte stores 2.6 k cycles per tile of 32 rows (with two
// or three warps per scheduler nothing hides a branch); branch-free 2-byte stores 25 us (a 2-byte store per lane runs
// the load/store unit at about 13 cycles per instruction); staging the tile for TMA stores 24 us (the TMA unit moves a
// 128-byte row in about 7.5 cycles, loads and stores alike: 17 bytes per clock and SM); 4-byte stores of pixel pairs
// 23.6 us = 4.4 TB/s.  The library GEMM takes 18.9 us on the same problem.
//
// Every wait on an mbarrier is bounded: when one runs out the kernel raises an error flag in mapped host memory, every
// role leaves its loop, TMEM is released and the kernel returns; the host reports SS2D_ECUDA on the next call.
#include "tc05.cuh"

namespace ss2d {

namespace {

using namespace tc05;

constexpr int kTilePx = 128;
constexpr int kMaxStages = 12;
constexpr int kSmemBudget = 200 * 1024;                    // W (resident) + the ring of x slices
constexpr int kEpiWarps = 8, kFirstEpiWarp = 4;
constexpr int kThreads = 32 * (kFirstEpiWarp + kEpiWarps);
constexpr int kSmemBytes = kSmemBudget + 1024 /* barriers */ + 1024 /* alignment slack */;

enum { BAR_W = 0, BAR_FULL = 1, BAR_EMPTY = 1 + kMaxStages, BAR_ACC_FULL = 1 + 2 * kMaxStages, BAR_ACC_EMPTY = 3 + 2 * kMaxStages,
       BAR_COUNT = 5 + 2 * kMaxStages };

struct LinearArgs {
    const float* bias;      // (M) or NULL
    void* out;
    long long N, out_row_stride;
    int M, Mpad, K, tiles;
    int kslice;             // channels per ring stage (a multiple of 32 that divides K)
    int stages, stage_bytes, w_bytes;
    int* error_flag;
};

template <typename T, bool kBias>
__global__ void __launch_bounds__(kThreads, 1)
linear_cf_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW, const LinearArgs a) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* ring = sm + a.w_bytes;                      // W first: [K / 32][Mpad rows][64 B], 64-byte swizzle
    uint64_t* bars = reinterpret_cast<uint64_t*>(sm + kSmemBudget);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + BAR_COUNT);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int Mpad = a.Mpad, nstages = a.stages, stage_bytes = a.stage_bytes, KS = a.kslice;
    const int nslices = a.K / KS;
    // two accumulators of Mpad columns; the allocation is a power of two of at least 32 columns
    uint32_t tmem_cols = 32;
    while ((int)tmem_cols < 2 * Mpad) tmem_cols <<= 1;

    if (threadIdx.x == 0) {
        mbar_init(bars + BAR_W, 1);
        for (int s = 0; s < nstages; ++s) { mbar_init(bars + BAR_FULL + s, 1); mbar_init(bars + BAR_EMPTY + s, 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(bars + BAR_ACC_FULL + i, 1); mbar_init(bars + BAR_ACC_EMPTY + i, kEpiWarps); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) { tmem_alloc(tmem_slot, tmem_cols); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const int ntiles_mine = (a.tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            mbar_expect_tx(bars + BAR_W, (uint32_t)a.w_bytes);
            for (int kc = 0; kc < a.K / 32; ++kc) tma_load_2d(sm + kc * Mpad * 64, &tmW, kc * 32, 0, bars + BAR_W);
            const uint32_t stage_tx = (uint32_t)KS * 256;
            int s = 0, round = 0;                              // ring position
            bool ok = true;
            for (int it = 0; ok && it < ntiles_mine; ++it) {
                const long long p0 = (long long)(blockIdx.x + (long long)it * gridDim.x) * kTilePx;
                for (int ks = 0; ks < nslices; ++ks) {
                    if (round > 0 && !mbar_wait_prompt(bars + BAR_EMPTY + s, (round - 1) & 1, abort_flag)) { ok = false; break; }
                    unsigned char* st = ring + s * stage_bytes;
                    mbar_expect_tx(bars + BAR_FULL + s, stage_tx);
                    tma_load_2d(st, &tmX, (int)p0, ks * KS, bars + BAR_FULL + s);
                    tma_load_2d(st + KS * 128, &tmX, (int)p0 + 64, ks * KS, bars + BAR_FULL + s);
                    if (++s == nstages) { s = 0; ++round; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            const uint32_t idesc = instr_desc(Fmt<T>::id, true, kTilePx, Mpad);
            const uint32_t sbase = smem_u32(sm), rbase = smem_u32(ring);
            const uint64_t db0 = smem_desc(sbase, 16, 512, kSw64);             // W: K-major rows of 64 bytes
            const uint32_t w_pair = (uint32_t)(Mpad * 64) >> 4;                // descriptor step between 32-channel slices of W
            int s = 0, round = 0;
            bool ok = mbar_wait_prompt(bars + BAR_W, 0, abort_flag);
            for (int it = 0; ok && it < ntiles_mine; ++it) {
                const int ab = it & 1;
                if (it >= 2) ok = mbar_wait_prompt(bars + BAR_ACC_EMPTY + ab, ((it >> 1) - 1) & 1, abort_flag);
                if (!ok) break;
                tc_fence_after();
                for (int ks = 0; ks < nslices; ++ks) {
                    if (!mbar_wait_prompt(bars + BAR_FULL + s, round & 1, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t da = smem_desc(rbase + s * stage_bytes, KS * 128, 1024, kSw128);   // x slice: MN-major, 64-pixel blocks
                    const int kk0 = ks * (KS / 16);
                    for (int k = 0; k < KS / 16; ++k) {
                        const int kk = kk0 + k;
                        tc_mma(tmem + ab * Mpad, da + (uint64_t)((k * 2048) >> 4), db0 + (uint64_t)((kk >> 1) * w_pair + (kk & 1) * 2), idesc,
                               kk > 0 ? 1u : 0u);
                    }
                    tc_commit(bars + BAR_EMPTY + s);           // the stage is free once these MMAs have read it
                    if (++s == nstages) { s = 0; ++round; }
                }
                if (ok) tc_commit(bars + BAR_ACC_FULL + ab);
            }
        }
    } else if (warp >= kFirstEpiWarp) {
        // ---------------------------------------------------------------- epilogue warps
        // No test inside the column loop: with two or three warps per scheduler nothing hides the latency of a branch
        // (a guarded form of this loop took 2.6 k cycles per tile of 32 columns, this one 0.4 k).
        const int ew = warp - kFirstEpiWarp;
        const int quarter = warp & 3;                          // TMEM lanes this warp may read: 32 * (warp id % 4) ...
        const int colh = ew >> 2;                              // ... and its half of the output rows
        const int row = quarter * 32 + lane;                   // pixel of the tile
        const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
        const int half_cols = Mpad / 2;                        // Mpad is a multiple of 16, M of 8
        const int c_begin = colh * half_cols, c_end = min(c_begin + half_cols, a.M);
        const long long N = a.N, ors = a.out_row_stride;
        const float* __restrict__ bias = a.bias;
        // A lane holds one pixel of every output row; a 2-byte store per lane and row runs the load/store unit at a
        // fraction of its rate (128 such stores per tile took as long as the tile's loads).  Neighbouring lanes
        // therefore trade halves: the even lane of a pair writes both pixels of the even row, the odd lane both pixels
        // of the odd row, four bytes each.
        const int odd = lane & 1;
        const unsigned sel = odd ? 0x3276u : 0x5410u;
        T* __restrict__ out = (T*)a.out + (quarter * 32 + (lane & ~1));
        bool ok = true;
        for (int it = 0; ok && it < ntiles_mine; ++it) {
            const int ab = it & 1;
            const long long p0 = (long long)(blockIdx.x + (long long)it * gridDim.x) * kTilePx;
            ok = mbar_wait_prompt(bars + BAR_ACC_FULL + ab, (it >> 1) & 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
            const bool live = p0 + row < N;                    // N is a multiple of 8: a pair of pixels is inside or outside
            T* __restrict__ dst = out + (live ? p0 : 0) + (long long)(c_begin + odd) * ors;
            for (int c0 = c_begin; c0 < c_end; c0 += 8) {
                uint32_t r[8];
                tmem_ld8(lane_base + ab * Mpad + c0, r);
                tmem_ld_wait();
                uint32_t w[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float lo = __uint_as_float(r[2 * q]) + (kBias ? __ldg(bias + c0 + 2 * q) : 0.f);
                    const float hi = __uint_as_float(r[2 * q + 1]) + (kBias ? __ldg(bias + c0 + 2 * q + 1) : 0.f);
                    const uint32_t own = Half2Of<T>::pack(lo, hi);
                    const uint32_t other = __shfl_xor_sync(0xffffffffu, own, 1);
                    w[q] = __byte_perm(own, other, sel);
                }
                if (live) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) *reinterpret_cast<uint32_t*>(dst + (long long)(2 * q) * ors) = w[q];
                }
                dst += 8 * ors;
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bars + BAR_ACC_EMPTY + ab);
        }
    }
    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, tmem_cols); }
    if (threadIdx.x == 0 && *abort_flag) atomicExch(a.error_flag, 1);
}

// Ring geometry for a problem, or false when W leaves no room for three stages.  The widest
// slice that fits is taken: a TMA operation costs the issuing thread about 170 cycles whatever its size.
static bool plan_linear(long long M, long long K, LinearArgs& a) {
    a.Mpad = (int)((M + 15) / 16 * 16);
    a.w_bytes = (int)((a.Mpad * K * 2 + 1023) / 1024 * 1024);
    const int room = kSmemBudget - a.w_bytes;
    for (int ks : {96, 64, 32}) {
        if (K % ks != 0) continue;
        a.kslice = ks;
        a.stage_bytes = ks * 256;                              // two 64-pixel halves of ks rows of 128 bytes
        a.stages = room / a.stage_bytes;
        if (a.stages > kMaxStages) a.stages = kMaxStages;
        if (a.stages >= 3) return true;
    }
    return false;
}

template <typename T>
int launch_linear(const ss2d_linear_params* p, cudaStream_t st) {
    LinearArgs a;
    if (!plan_linear(p->M, p->K, a)) return SS2D_ENOTSUP;
    CUtensorMap tmX, tmW;
    // x: (K, N) with row pitch x_row_stride; W: (M, K) dense.  Rows of W beyond M (the padding of the MMA's N) are
    // outside the tensor and arrive as zeros.
    if (!make_map_pitched(&tmX, Fmt<T>::tm, p->x, p->K, p->N, p->x_row_stride ? p->x_row_stride : p->N, a.kslice, 64,
                          CU_TENSOR_MAP_SWIZZLE_128B)) return SS2D_ECUDA;
    if (!make_map_pitched(&tmW, Fmt<T>::tm, p->w, p->M, p->K, p->K, a.Mpad, 32, CU_TENSOR_MAP_SWIZZLE_64B)) return SS2D_ECUDA;
    int* host_flag = error_flag_for_current_device();
    if (!host_flag) return SS2D_ECUDA;
    if (*host_flag) return SS2D_ECUDA;                     // an earlier launch on this device gave up on a wait
    int* dev_flag = nullptr;
    if (cudaHostGetDevicePointer((void**)&dev_flag, host_flag, 0) != cudaSuccess) return SS2D_ECUDA;
    static bool attr_ok[64][2] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    const int hb = p->bias ? 1 : 0;
    auto kern = hb ? linear_cf_kernel<T, true> : linear_cf_kernel<T, false>;
    if (!attr_ok[dev & 63][hb]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess) return SS2D_ECUDA;
        attr_ok[dev & 63][hb] = true;
    }
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return SS2D_ECUDA;
    a.bias = (const float*)p->bias; a.out = p->out; a.N = p->N;
    a.out_row_stride = p->out_row_stride ? p->out_row_stride : p->N;
    a.M = (int)p->M; a.K = (int)p->K;
    a.tiles = (int)((p->N + kTilePx - 1) / kTilePx);
    a.error_flag = dev_flag;
    const int grid = a.tiles < sms ? a.tiles : sms;
    kern<<<grid, kThreads, kSmemBytes, st>>>(tmX, tmW, a);
    count_launch();
    return check_launch();
}

}  // namespace

int linear_supported(const ss2d_linear_params* p) {
    if (!p) return SS2D_EINVAL_NULL;
    if (!p->x || !p->w || !p->out) return SS2D_EINVAL_NULL;
    if (p->dtype != SS2D_BF16 && p->dtype != SS2D_F16) return SS2D_ENOTSUP;     // fp32 maps: the library GEMM
    if (p->M <= 0 || p->K <= 0 || p->N <= 0) return SS2D_EINVAL_SHAPE;
    if (p->M > 256 || p->M % 8 != 0 || p->K % 32 != 0) return SS2D_ENOTSUP;
    { LinearArgs g; if (!plan_linear(p->M, p->K, g)) return SS2D_ENOTSUP; }      // W must leave room for the ring
    const long long xs = p->x_row_stride ? p->x_row_stride : p->N, os = p->out_row_stride ? p->out_row_stride : p->N;
    if (xs < p->N || os < p->N) return SS2D_EINVAL_STRIDE;
    if (xs % 8 != 0 || os % 2 != 0 || p->N % 8 != 0 || p->N > 0x7fffff00LL) return SS2D_ENOTSUP;   // 16-byte row pitch for TMA, paired stores
    if (!aligned_to(p->x, 16) || !aligned_to(p->w, 16) || !aligned_to(p->out, 4) || (p->bias && !aligned_to(p->bias, 4)))
        return SS2D_EINVAL_ALIGN;
    return SS2D_OK;
}

int linear_fwd(const ss2d_linear_params* p, cudaStream_t st) {
    const int rc = linear_supported(p);
    if (rc != SS2D_OK) return rc;
    if (p->dtype == SS2D_BF16) return launch_linear<__nv_bfloat16>(p, st);
    return launch_linear<__half>(p, st);
}

}  // namespace ss2d
