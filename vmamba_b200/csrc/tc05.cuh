// 5th-generation tensor-core plumbing shared by the tcgen05 kernels of this library: mbarrier and TMA wrappers with
// bounded waits, TMEM allocation and loads, shared-memory operand descriptors, tensor-map construction, and the
// per-device error flag a kernel raises when one of its waits runs out.
#pragma once
#include <cuda.h>

#include <mutex>

#include "common.cuh"

namespace ss2d {
namespace tc05 {

constexpr unsigned kSpinLimit = 1u << 18;

// ---- PTX wrappers --------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One attempt: the thread sleeps until the phase completes or about `kWaitSliceNs` have passed, so a waiting warp
// issues a handful of instructions per slice instead of spinning against the warps that have arithmetic to do.
constexpr uint32_t kWaitSliceNs = 20000;
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n"
        " mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        " selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(kWaitSliceNs) : "memory");
    return ok != 0;
}
// Bounded wait (at most kSpinLimit slices, a few seconds).  Returns false when the limit ran out or another role has
// already given up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    for (unsigned i = 0; i < kSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}

// The same for the threads of a load-bound pipeline (TMA producer, MMA issuer, the epilogue's hand-over): attempts
// without a sleep hint.  Bounded by time: every 256 missed attempts the global nanosecond timer is read, and two seconds
// after the first miss the wait gives up (error flag, as above).
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool mbar_wait_prompt(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    unsigned long long t0 = 0;
    for (unsigned i = 0;; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n .reg .pred p;\n"
            " mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            " selp.u32 %0, 1, 0, p;\n}"
            : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
        if (ok) return true;
        if ((i & 255) == 255) {
            if (*abort_flag) return false;
            const unsigned long long now = global_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > 2000000000ull) break;
        }
    }
    *abort_flag = 1;
    return false;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::); }
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// D (TMEM) (+)= A (smem descriptor) . B (smem descriptor); 16-bit inputs, fp32 accumulation
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns: lane i of the warp gets row (quarter base + i)
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- operand descriptors (the layouts TMA writes with its 128- / 64-byte swizzle) --------------------------------------
// Shared-memory matrix descriptor: start address, leading and stride byte offsets (all >> 4), descriptor version 1,
// swizzle mode.  For the swizzled layouts used here:
//   K-major  (rows of 64 / 32 contraction elements): stride offset = 8 rows (1024 / 512 bytes), leading offset unused
//   MN-major (rows of 64 M elements, one row per contraction index): stride offset = 8 rows of the contraction
//            (1024 bytes), leading offset = distance between blocks of 64 M elements
constexpr uint64_t kSw128 = 2ull << 61, kSw64 = 4ull << 61;
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lead_bytes, uint32_t stride_bytes, uint64_t swizzle) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | ((uint64_t)((lead_bytes >> 4) & 0x3fffu) << 16) |
           ((uint64_t)((stride_bytes >> 4) & 0x3fffu) << 32) | (1ull << 46) | swizzle;
}
// Instruction descriptor: fp32 accumulator, 16-bit A / B of format `fmt` (0 fp16, 1 bf16), A MN-major or K-major, B K-major
__host__ __device__ constexpr uint32_t instr_desc(int fmt, bool a_mn_major, int M, int N) {
    return (1u << 4) | ((uint32_t)fmt << 7) | ((uint32_t)fmt << 10) | ((a_mn_major ? 1u : 0u) << 15) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

template <typename T> struct Fmt;
template <> struct Fmt<__nv_bfloat16> { static constexpr int id = 1; static constexpr CUtensorMapDataType tm = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; };
template <> struct Fmt<__half> { static constexpr int id = 0; static constexpr CUtensorMapDataType tm = CU_TENSOR_MAP_DATA_TYPE_FLOAT16; };

// ---- host ------------------------------------------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeFn encode_fn() {
    static EncodeFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeFn>(p);
    }();
    return fn;
}

// 2-D map of a row-major (rows, cols) matrix of 16-bit elements: box (box_rows, box_cols), inner dimension = columns
inline bool make_map(CUtensorMap* m, CUtensorMapDataType dt, const void* base, long long rows, long long cols, int box_rows, int box_cols,
              CUtensorMapSwizzle sw) {
    EncodeFn enc = encode_fn();
    if (!enc) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return enc(m, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
               CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The same for rows `pitch` elements apart (pitch >= cols, a multiple of 8 elements)
inline bool make_map_pitched(CUtensorMap* m, CUtensorMapDataType dt, const void* base, long long rows, long long cols, long long pitch,
                             int box_rows, int box_cols, CUtensorMapSwizzle sw) {
    EncodeFn enc = encode_fn();
    if (!enc) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)pitch * 2};
    const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return enc(m, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
               CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

inline int* error_flag_for_current_device() {
    static std::mutex mu;
    static int* flags[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (!flags[dev]) {
        // mapped, pinned host memory: the kernel can raise the flag and the host can read it without a copy
        int* h = nullptr;
        if (cudaHostAlloc((void**)&h, sizeof(int), cudaHostAllocMapped) != cudaSuccess) return nullptr;
        *h = 0;
        flags[dev] = h;
    }
    return flags[dev];
}

}  // namespace tc05
}  // namespace ss2d
