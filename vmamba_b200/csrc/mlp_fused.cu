// Fused MLP of a VSS block on the 5th-generation tensor cores:  y = W2 . gelu(W1 . x + b1)  on a channel-major
// map x (C, N) of N = B*H*W pixels, the 4C-wide hidden activations never leaving the SM.  Replaces fc1, the bias +
// GELU pass and fc2 of Mlp.forward (vmamba.py:1151-1167); the fc2 bias joins the residual update in the LayerNorm
// kernel that consumes y.
//
// One persistent CTA per SM walks tiles of 128 pixels.  Per tile and per chunk of 64 hidden units:
//   GEMM 1   H^T (128 px x 64)   = X^T (128 px x C) . W1_chunk^T (C x 64)      tcgen05.mma, accumulator in TMEM
//   epilogue H^T -> registers (tcgen05.ld) -> + b1 -> GELU -> bf16 -> shared memory, laid out as an MMA operand
//   GEMM 2   Y^T (128 px x C)   += G (128 px x 64) . W2_chunk^T (64 x C)       accumulator in TMEM over all chunks
// then Y^T -> registers -> 16-bit -> global, channel-major.  X^T is read straight from the channel-major map: a TMA
// box of 64 pixels x C channels is the "MN-major" operand form of the tensor core (pixels contiguous), so no transpose
// happens anywhere.  Both weight matrices stay in shared memory for the life of the CTA (C = 96: 144 KB), loaded once
// by TMA; x tiles are double-buffered TMA loads.  Warp 0 issues TMA, warp 1 the MMAs of GEMM 1, warp 2 those of GEMM 2
// (one lane each, each blocking on its own barriers: a single issuing thread that polled both streams spent its time
// on descriptor arithmetic and polling, sharing a scheduler with four epilogue warps), sixteen warps run the epilogues
// in two groups that take alternate chunks.  TMEM holds two H chunks and two Y tiles, so the tensor core works on
// chunk j+1 and on the next tile while the epilogue warps are busy; the Y tile is written out one chunk into the next
// tile.  The epilogue is what bounds the kernel (128 x 4C GELUs per tile, about 11 fp32 operations each, against the
// 2.4 k cycles of the tile's MMAs), which is why erf is a polynomial on the FMA pipe (gelu error <= 7.5e-4) and not the
// exp / reciprocal form: two MUFU operations per value alone would take 2.6 times as long as the tile's MMAs.
//
// Every wait on an mbarrier is bounded: when one runs out, the kernel raises an error flag in global memory, every role
// leaves its loop, TMEM is released and the kernel returns; the host reports SS2D_ECUDA on the next status query.
#include "activations.cuh"
#include "tc05.cuh"

namespace ss2d {

namespace {

using namespace tc05;

constexpr int kTilePx = 128;       // pixels per tile = M of the MMAs
constexpr int kHC = 64;            // hidden units per chunk = N of GEMM 1, K of GEMM 2
constexpr int kEpiWarps = 16;
constexpr int kFirstEpiWarp = 4;   // warps 0..3: TMA producer, GEMM 1 issuer, GEMM 2 issuer, (spare)
constexpr int kThreads = 32 * (kFirstEpiWarp + kEpiWarps);
struct MlpArgs {
    const float* b1;
    void* y;
    long long N;
    int tiles;
    int* error_flag;
};

// Shared memory of the C-channel kernel (byte offsets from a 1024-aligned base)
template <int C> struct MlpSmem {
    static constexpr int HID = 4 * C, NCH = HID / kHC, KC1 = C / 32;     // hidden width, chunks, 32-wide K slices of W1
    static constexpr int kW1 = 0;                                        // [KC1][HID rows][64 B], 64-byte swizzle
    static constexpr int kW1Bytes = KC1 * HID * 64;
    static constexpr int kW2 = kW1 + kW1Bytes;                           // [NCH][C rows][128 B], 128-byte swizzle
    static constexpr int kW2Block = C * 128, kW2Bytes = NCH * kW2Block;
    static constexpr int kX = kW2 + kW2Bytes;                            // [2 stages][2 halves][C rows][128 B]
    static constexpr int kXHalf = C * 128, kXStage = 2 * kXHalf;
    static constexpr int kG = kX + 2 * kXStage;                          // [2][128 rows][128 B]
    static constexpr int kGBuf = kTilePx * 128;
    static constexpr int kBars = kG + 2 * kGBuf;
    static constexpr int kBias = kBars + 256;                            // fc1 bias, fp32
    static constexpr int kTotal = kBias + HID * 4;
    static_assert(C % 32 == 0 && (C * 128) % 1024 == 0, "operand blocks must be whole swizzle atoms");
};

enum { BAR_W = 0, BAR_XF = 1, BAR_XE = 3, BAR_HF = 5, BAR_HE = 7, BAR_GF = 9, BAR_GE = 11, BAR_YF = 13, BAR_YE = 15, BAR_COUNT = 17 };

template <typename T, int C>
__global__ void __launch_bounds__(kThreads, 1)
mlp_fused_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW1,
                 const __grid_constant__ CUtensorMap tmW2, const MlpArgs a) {
    using S = MlpSmem<C>;
    constexpr int NCH = S::NCH;
    constexpr int kTmemCols = 512;
    constexpr int kColH = 0, kColY = 2 * kHC;                  // TMEM columns: two H chunks, then two Y tiles of C columns
    static_assert(kColY + 2 * C <= kTmemCols, "TMEM holds two H chunks and two Y tiles");
    extern __shared__ unsigned char smem_raw[];
    unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(sm + S::kBars);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + BAR_COUNT);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        mbar_init(bars + BAR_W, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(bars + BAR_XF + i, 1); mbar_init(bars + BAR_XE + i, 1);
            mbar_init(bars + BAR_HF + i, 1); mbar_init(bars + BAR_HE + i, kEpiWarps / 2);
            mbar_init(bars + BAR_GF + i, kEpiWarps / 2); mbar_init(bars + BAR_GE + i, 1);
            mbar_init(bars + BAR_YF + i, 1); mbar_init(bars + BAR_YE + i, kEpiWarps);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int i = threadIdx.x; i < S::HID; i += kThreads) reinterpret_cast<float*>(sm + S::kBias)[i] = __ldg(a.b1 + i);
    if (warp == 1) { tmem_alloc(tmem_slot, kTmemCols); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const int ntiles_mine = (a.tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            mbar_expect_tx(bars + BAR_W, S::kW1Bytes + S::kW2Bytes);
            for (int kc = 0; kc < S::KC1; ++kc)
                for (int r0 = 0; r0 < S::HID; r0 += 192)
                    tma_load_2d(sm + S::kW1 + (kc * S::HID + r0) * 64, &tmW1, kc * 32, r0, bars + BAR_W);
            for (int j = 0; j < NCH; ++j) tma_load_2d(sm + S::kW2 + j * S::kW2Block, &tmW2, j * kHC, 0, bars + BAR_W);
            for (int it = 0; it < ntiles_mine; ++it) {
                const int s = it & 1;
                if (it >= 2 && !mbar_wait(bars + BAR_XE + s, ((it >> 1) - 1) & 1, abort_flag)) break;
                const long long p0 = (long long)(blockIdx.x + (long long)it * gridDim.x) * kTilePx;
                mbar_expect_tx(bars + BAR_XF + s, S::kXStage);
                tma_load_2d(sm + S::kX + s * S::kXStage, &tmX, (int)p0, 0, bars + BAR_XF + s);
                tma_load_2d(sm + S::kX + s * S::kXStage + S::kXHalf, &tmX, (int)p0 + 64, 0, bars + BAR_XF + s);
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- GEMM 1 issuer
        // H^T (chunk c) = X^T . W1_c^T as soon as the x tile is there and the epilogue has read chunk c - 2 out of the H
        // buffer.  Chunks are numbered across tiles.  The thread's instruction stream is kept short (descriptors are
        // a constant plus an offset): it shares its scheduler with four epilogue warps.
        if (lane == 0) {
            constexpr uint32_t idesc1 = instr_desc(Fmt<T>::id, true, kTilePx, kHC);
            const uint32_t sbase = smem_u32(sm);
            const uint64_t a_base = smem_desc(sbase + S::kX, S::kXHalf, 1024, kSw128);
            const uint64_t b_base = smem_desc(sbase + S::kW1, 16, 512, kSw64);
            bool ok = mbar_wait(bars + BAR_W, 0, abort_flag);
            const int total = ntiles_mine * NCH;
            for (int c1 = 0, it = 0, j = 0; ok && c1 < total; ++c1) {
                const int s = it & 1, b = c1 & 1;
                if (j == 0) ok = mbar_wait(bars + BAR_XF + s, (it >> 1) & 1, abort_flag);
                if (ok && c1 >= 2) ok = mbar_wait(bars + BAR_HE + b, ((c1 >> 1) - 1) & 1, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint64_t da0 = a_base + (uint64_t)((s * S::kXStage) >> 4);
                const uint64_t db0 = b_base + (uint64_t)((j * kHC * 64) >> 4);
#pragma unroll
                for (int k = 0; k < C / 16; ++k)               // 16 channels per instruction
                    tc_mma(tmem + kColH + b * kHC, da0 + (uint64_t)((k * 2048) >> 4),
                           db0 + (uint64_t)((((k >> 1) * S::HID) * 64 + (k & 1) * 32) >> 4), idesc1, k > 0 ? 1u : 0u);
                tc_commit(bars + BAR_HF + b);
                if (j == NCH - 1) tc_commit(bars + BAR_XE + s);        // the x tile has been read by all its MMAs
                if (++j == NCH) { j = 0; ++it; }
            }
        }
    } else if (warp == 2) {
        // ---------------------------------------------------------------- GEMM 2 issuer
        // Y^T (+)= G_c . W2_c^T as soon as the epilogue has written G_c (and, at the start of a tile, read the Y tile
        // that used this accumulator two tiles ago).
        if (lane == 0) {
            constexpr uint32_t idesc2 = instr_desc(Fmt<T>::id, false, kTilePx, C);
            const uint32_t sbase = smem_u32(sm);
            const uint64_t a_base = smem_desc(sbase + S::kG, 16, 1024, kSw128);
            const uint64_t b_base = smem_desc(sbase + S::kW2, 16, 1024, kSw128);
            bool ok = mbar_wait(bars + BAR_W, 0, abort_flag);
            const int total = ntiles_mine * NCH;
            for (int c2 = 0, it = 0, j = 0; ok && c2 < total; ++c2) {
                const int yb = it & 1, b = c2 & 1;
                ok = mbar_wait(bars + BAR_GF + b, (c2 >> 1) & 1, abort_flag);
                if (ok && j == 0 && it >= 2) ok = mbar_wait(bars + BAR_YE + yb, ((it >> 1) - 1) & 1, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint64_t da0 = a_base + (uint64_t)((b * S::kGBuf) >> 4);
                const uint64_t db0 = b_base + (uint64_t)((j * S::kW2Block) >> 4);
#pragma unroll
                for (int k = 0; k < kHC / 16; ++k)
                    tc_mma(tmem + kColY + yb * C, da0 + (uint64_t)((k * 32) >> 4), db0 + (uint64_t)((k * 32) >> 4), idesc2,
                           (j > 0 || k > 0) ? 1u : 0u);
                tc_commit(bars + BAR_GE + b);                  // the G buffer is free once these MMAs have read it
                if (j == NCH - 1) tc_commit(bars + BAR_YF + yb);
                if (++j == NCH) { j = 0; ++it; }
            }
        }
    } else if (warp >= kFirstEpiWarp) {
        // ---------------------------------------------------------------- epilogue warps
        // Two groups of eight warps; group 0 takes the even chunks (H / G buffer 0), group 1 the odd ones, so that the
        // waits of one group (TMEM load, proxy fence, hand-over to the MMA warp) are covered by the arithmetic of the other.
        const int ew = warp - kFirstEpiWarp;
        const int grp = ew >> 3;
        const int quarter = warp & 3;                          // TMEM lanes this warp may read: 32 * (warp id % 4) ...
        const int colh = (ew >> 2) & 1;                        // ... and its half of a chunk's columns
        const int row = quarter * 32 + lane;                   // pixel of the tile
        const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
        const float* bias_s = reinterpret_cast<const float*>(sm + S::kBias);
        T* __restrict__ yout = (T*)a.y;
        static_assert(NCH % 2 == 0, "chunks alternate between the two epilogue groups");
        constexpr int CQ = C / 4;                                       // channels per warp: (group, column half) picks a quarter
        static_assert(CQ % 8 == 0, "a warp reads its channels in groups of 8 columns");
        const int cq0 = (grp * 2 + colh) * CQ;
        bool ok = true;
        // Y^T of tile `it` -> 16-bit -> global, channel-major.  Called one chunk into the NEXT tile, when the tile's last
        // GEMM 2 has long finished and the tensor core already has the next tile's chunks to work on.
        auto y_epilogue = [&](int it) {
            const int yb = it & 1;
            const long long p0 = (long long)(blockIdx.x + (long long)it * gridDim.x) * kTilePx;
            if (!mbar_wait(bars + BAR_YF + yb, (it >> 1) & 1, abort_flag)) return false;
            tc_fence_after();
            // A 2-byte store per lane and channel runs the load/store unit at a fraction of its rate: neighbouring lanes
            // trade halves, the even lane of a pair writes both pixels of the even channel, the odd lane both pixels of
            // the odd channel, four bytes each (N is a multiple of 8: a pair of pixels is inside the map or outside).
            const bool live = p0 + row < a.N;
            const int odd = lane & 1;
            const unsigned sel = odd ? 0x3276u : 0x5410u;
            T* __restrict__ ycol_ptr = yout + (long long)(cq0 + odd) * a.N + p0 + (row & ~1);
#pragma unroll
            for (int c0 = 0; c0 < CQ; c0 += 8) {
                uint32_t r[8];
                tmem_ld8(lane_base + kColY + yb * C + cq0 + c0, r);
                tmem_ld_wait();
                uint32_t w[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const uint32_t own = Half2Of<T>::pack(__uint_as_float(r[2 * q]), __uint_as_float(r[2 * q + 1]));
                    w[q] = __byte_perm(own, __shfl_xor_sync(0xffffffffu, own, 1), sel);
                }
                if (live) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) *reinterpret_cast<uint32_t*>(ycol_ptr + (long long)(c0 + 2 * q) * a.N) = w[q];
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bars + BAR_YE + yb);             // the Y tile is in registers / on its way out
            return true;
        };
        for (int it = 0; ok && it < ntiles_mine; ++it) {
            for (int j = grp; ok && j < NCH; j += 2) {
                const int g = it * NCH + j, b = grp;           // global chunk index; its buffers
                ok = mbar_wait(bars + BAR_HF + b, (g >> 1) & 1, abort_flag);
                if (!ok) break;
                tc_fence_after();
                uint32_t r0[16], r1[16];
                const uint32_t col = kColH + b * kHC + colh * 32;
                tmem_ld16(lane_base + col, r0);
                tmem_ld16(lane_base + col + 16, r1);
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bars + BAR_HE + b);          // the H chunk is in registers
                const float4* bias = reinterpret_cast<const float4*>(bias_s + j * kHC + colh * 32);
                uint32_t packed[16];
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const float4 bq = bias[q];
                    const uint32_t* src = q < 4 ? r0 + 4 * q : r1 + 4 * (q - 4);
                    const float2 lo = gelu_pair_poly(__fadd2_rn(make_float2(__uint_as_float(src[0]), __uint_as_float(src[1])), make_float2(bq.x, bq.y)));
                    const float2 hi = gelu_pair_poly(__fadd2_rn(make_float2(__uint_as_float(src[2]), __uint_as_float(src[3])), make_float2(bq.z, bq.w)));
                    packed[2 * q] = Half2Of<T>::pack(lo.x, lo.y);
                    packed[2 * q + 1] = Half2Of<T>::pack(hi.x, hi.y);
                }
                if (g >= 2) ok = mbar_wait(bars + BAR_GE + b, ((g >> 1) - 1) & 1, abort_flag);
                if (!ok) break;
                // G as a K-major operand with the 128-byte swizzle: row = pixel, 16-byte unit u of the row at u ^ (row % 8)
                unsigned char* grow = sm + S::kG + b * S::kGBuf + row * 128;
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int unit = (colh * 4 + u) ^ (row & 7);
                    *reinterpret_cast<uint4*>(grow + unit * 16) = make_uint4(packed[4 * u], packed[4 * u + 1], packed[4 * u + 2], packed[4 * u + 3]);
                }
                fence_async_smem();                                     // generic-proxy writes -> visible to the tensor core
                __syncwarp();
                if (lane == 0) mbar_arrive(bars + BAR_GF + b);
                if (j == grp && it > 0) ok = y_epilogue(it - 1);
            }
        }
        if (ok && ntiles_mine > 0) y_epilogue(ntiles_mine - 1);
    }
    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, kTmemCols); }
    if (threadIdx.x == 0 && *abort_flag) atomicExch(a.error_flag, 1);
}

// ---- host ------------------------------------------------------------------------------------------------------------
template <typename T, int C>
int launch_mlp(const ss2d_mlp_params* p, cudaStream_t st) {
    using S = MlpSmem<C>;
    CUtensorMap tmX, tmW1, tmW2;
    const long long N = p->N;
    if (!make_map(&tmX, Fmt<T>::tm, p->x, C, N, C, 64, CU_TENSOR_MAP_SWIZZLE_128B)) return SS2D_ECUDA;
    if (!make_map(&tmW1, Fmt<T>::tm, p->w1, 4 * C, C, 192, 32, CU_TENSOR_MAP_SWIZZLE_64B)) return SS2D_ECUDA;
    if (!make_map(&tmW2, Fmt<T>::tm, p->w2, C, 4 * C, C, 64, CU_TENSOR_MAP_SWIZZLE_128B)) return SS2D_ECUDA;
    int* host_flag = error_flag_for_current_device();
    if (!host_flag) return SS2D_ECUDA;
    if (*host_flag) return SS2D_ECUDA;                     // an earlier launch on this device gave up on a wait
    int* dev_flag = nullptr;
    if (cudaHostGetDevicePointer((void**)&dev_flag, host_flag, 0) != cudaSuccess) return SS2D_ECUDA;
    auto kern = mlp_fused_kernel<T, C>;
    constexpr int smem = S::kTotal + 1024;
    static bool attr_ok[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_ok[dev & 63]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return SS2D_ECUDA;
        attr_ok[dev & 63] = true;
    }
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return SS2D_ECUDA;
    MlpArgs a;
    a.b1 = (const float*)p->b1; a.y = p->y; a.N = N;
    a.tiles = (int)((N + kTilePx - 1) / kTilePx);
    a.error_flag = dev_flag;
    const int grid = a.tiles < sms ? a.tiles : sms;
    kern<<<grid, kThreads, smem, st>>>(tmX, tmW1, tmW2, a);
    count_launch();
    return check_launch();
}

}  // namespace

int mlp_supported(const ss2d_mlp_params* p) {
    if (!p) return SS2D_EINVAL_NULL;
    if (!p->x || !p->w1 || !p->b1 || !p->w2 || !p->y) return SS2D_EINVAL_NULL;
    if (p->dtype != SS2D_BF16 && p->dtype != SS2D_F16) return SS2D_ENOTSUP;     // fp32 maps: the library GEMMs
    if (p->C <= 0 || p->N <= 0) return SS2D_EINVAL_SHAPE;
    if (p->hidden != 4 * p->C) return SS2D_ENOTSUP;
    if (p->C != 96) return SS2D_ENOTSUP;                                         // widths whose weights fit one SM
    if (p->N % 8 != 0 || p->N > 0x7fffff00LL) return SS2D_ENOTSUP;               // 16-byte row pitch for TMA
    if (!aligned_to(p->x, 16) || !aligned_to(p->y, 4) || !aligned_to(p->w1, 16) || !aligned_to(p->w2, 16) || !aligned_to(p->b1, 16))
        return SS2D_EINVAL_ALIGN;
    return SS2D_OK;
}

int mlp_fwd(const ss2d_mlp_params* p, cudaStream_t st) {
    const int rc = mlp_supported(p);
    if (rc != SS2D_OK) return rc;
    if (p->dtype == SS2D_BF16) return launch_mlp<__nv_bfloat16, 96>(p, st);
    return launch_mlp<__half, 96>(p, st);
}

}  // namespace ss2d
