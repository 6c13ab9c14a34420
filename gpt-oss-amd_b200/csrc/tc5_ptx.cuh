// PTX wrappers shared by the tcgen05 expert GEMMs (gemm_tc5_pair.cuh, gemm_tc5_ts.cuh):
// mbarrier, TMA / bulk copies, tensor-memory allocation, tcgen05.mma / commit / ld,
// shared-memory and instruction descriptors, bounded waits.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace moe {
namespace tc5 {

constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;  // 2 s
constexpr uint32_t WAIT_SUSPEND_NS = 20000;                 // one suspended test of a barrier lasts at most this

constexpr int STEP_CHUNKS = 6;  // 64-column chunks per pipeline step of the small-batch GEMM

struct TensorMaps {
    CUtensorMap box[4];   // token-row boxes of 32, 64, 128 (and 256, unused) rows x 64 columns
    // the same rows seen as [chunk of 64 columns][row][64 columns]: boxes of 32 and 64 rows x
    // STEP_CHUNKS chunks, so that one copy brings the activation tiles of a whole step
    CUtensorMap box3[2];
};

// ---------------------------------------------------------------------------
// PTX wrappers

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done;
}

// The same test, but the thread may stay suspended in hardware for up to `ns`
// nanoseconds waiting for the phase to complete (it resumes at once when it does).
// A role that waits in a loop of plain tests takes issue slots from the warps that
// have work -- above all from the single warp that issues the MMAs, whose chain of a
// few dozen instructions per step then sets the pace of the whole pipeline.
__device__ __forceinline__ uint32_t mbar_try_wait_suspend(uint32_t bar, uint32_t parity, uint32_t ns) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"(ns)
        : "memory");
    return done;
}

// One lane of a converged warp (the same one every time).
__device__ __forceinline__ uint32_t elect_one_sync() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred;
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait.  Returns false when the time limit passed or another role has
// raised the abort flag; the first to time out records `code`.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status, int code,
                                          volatile int* abort_flag) {
    if (mbar_try_wait(bar, parity))
        return true;
    unsigned long long t_start = 0;
    for (uint32_t it = 1;; ++it) {
        if (mbar_try_wait_suspend(bar, parity, WAIT_SUSPEND_NS))
            return true;
        if ((it & 15u) == 0) {
            if (*abort_flag)
                return false;
            const unsigned long long now = global_timer_ns();
            if (t_start == 0)
                t_start = now;
            else if (now - t_start > WAIT_LIMIT_NS)
                break;
        }
    }
    report_status(status, code);
    *abort_flag = 1;
    return false;
}

// The same bounded wait as a loop of plain tests (no suspension): for the one warp whose
// reaction time sets the pace of the pipeline, the MMA issuer (measured on one GPU, two
// runs each: 16384-token step 3.019 -> 2.995 ms, decode step 3.703 -> 3.692 ms; the same
// change on the sixteen decode warps costs 2 %).
__device__ __forceinline__ bool mbar_wait_hot(uint32_t bar, uint32_t parity, int* status, int code,
                                              volatile int* abort_flag) {
    unsigned long long t_start = 0;
    for (uint32_t it = 1;; ++it) {
        if (mbar_try_wait(bar, parity))
            return true;
        if ((it & 255u) == 0) {
            if (*abort_flag)
                return false;
            const unsigned long long now = global_timer_ns();
            if (t_start == 0)
                t_start = now;
            else if (now - t_start > WAIT_LIMIT_NS)
                break;
        }
    }
    report_status(status, code);
    *abort_flag = 1;
    return false;
}

// After an abort: give a copy that was already issued a bounded time to land
// before the CTA exits.
__device__ __forceinline__ void drain_wait(uint32_t bar, uint32_t parity) {
    const unsigned long long t0 = global_timer_ns();
    while (!mbar_try_wait(bar, parity)) {
        if (global_timer_ns() - t0 > 100000000ull)  // 0.1 s
            break;
    }
}

__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// Orders earlier generic-proxy accesses to global memory (here: rows that another
// GPU stored and this thread has just seen flagged) before later async-proxy ones
// (TMA loads) of this thread.
__device__ __forceinline__ void fence_proxy_async_global() {
    asm volatile("fence.proxy.async.global;" ::: "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes,
                                          uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst),
                 "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}

// D[tmem] (+)= A[smem desc] . B[smem desc]^T, bf16 x bf16 -> fp32, issued by one thread.
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Arrives on `bar` when every tcgen05.mma issued so far by this thread is done.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}

// 32 lanes x 32 consecutive fp32 columns: thread i of the warp gets lane
// (taddr.lane + i), registers = columns.  No wait: pair with tmem_ld_wait().
__device__ __forceinline__ void tmem_ld_32x32_issue(uint32_t taddr, uint32_t r[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Sum over the NACC K-split accumulators (BN columns apart) of 32 columns.
template <int NACC, int BN>
__device__ __forceinline__ void tmem_ld_sum(uint32_t taddr, float v[32]) {
    uint32_t r[32];
    tmem_ld_32x32_issue(taddr, r);
    tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 32; i++)
        v[i] = __uint_as_float(r[i]);
#pragma unroll
    for (int a = 1; a < NACC; a++) {
        tmem_ld_32x32_issue(taddr + (uint32_t)(a * BN), r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i++)
            v[i] += __uint_as_float(r[i]);
    }
}

// Shared-memory matrix descriptor: K-major tile whose rows are 128 bytes
// (64 bf16), 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t make_sw128_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);        // start address
    d |= (uint64_t)1 << 16;                              // leading byte offset (unused for SW128 K-major)
    d |= (uint64_t)(1024 >> 4) << 32;                    // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                              // descriptor version (sm_100)
    d |= (uint64_t)2 << 61;                              // SWIZZLE_128B
    return d;
}

// Instruction descriptor: bf16 x bf16 -> fp32, both operands K-major, M = 128.
__device__ __forceinline__ uint32_t make_idesc(int n) {
    return (1u << 4)                       // D format fp32
           | (1u << 7)                     // A format bf16
           | (1u << 10)                    // B format bf16
           | ((uint32_t)(n >> 3) << 17)    // N / 8
           | ((uint32_t)(TILE_M >> 4) << 24);  // M / 16
}


#if defined(MOE_B200_TEST_AIDS) && defined(TC5_TRACE)
// Test-aids builds only (-DMOE_B200_TEST_AIDS -DTC5_TRACE=<MODE>): SM-clock timestamps of the
// pipeline hand-offs of CTA 0.
constexpr int TRACE_STEPS = 512, TRACE_SLOTS = 16;
__device__ long long g_trace[TRACE_STEPS * TRACE_SLOTS];
#define TRACE(step, slot)                                                   \
    do {                                                                    \
        if (MODE == TC5_TRACE && blockIdx.x == 0 && (step) < TRACE_STEPS)                      \
            g_trace[(step) * TRACE_SLOTS + (slot)] = clock64();             \
    } while (0)
#else
#define TRACE(step, slot) do { } while (0)
#endif
#define TRACE_D(step, slot) TRACE(step, slot)

#define RING_ADVANCE(s, ph, depth) \
    do {                           \
        if (++(s) == (depth)) {    \
            (s) = 0;               \
            (ph) ^= 1u;            \
        }                          \
    } while (0)

}  // namespace tc5
}  // namespace moe
