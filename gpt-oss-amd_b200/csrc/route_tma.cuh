// Router kernel fed by TMA: the same computation, block shape, warp layout and
// summation order as route_tc_kernel (route.cuh) -- router GEMM + bias + top-K +
// softmax + per-block histogram, src/hip/gemms/gemm_router.hip:7-190,
// src/hip/topk.hip:5-72, src/hip/softmax.hip:5-51 -- with the ring stages filled by
// tiled bulk copies instead of 16-byte cp.async copies.
//
// Why: the cp.async version is a latency chain.  ncu on it (2048 tokens, 128
// experts): no unit above 30 % busy, 46 GB/s of L2 reads per SM; eight warps issuing
// 16-byte copies cannot keep more in flight.  Here one thread issues two tiled copies
// per 64-column chunk (the block's token rows, all router rows: up to 40 KB) and an
// mbarrier counts their bytes; rows past the batch and past E arrive as zeros from the
// tensor map's bounds, so nothing is zero-filled by hand.
//
// Stage layout: 128-byte rows (64 bf16), token rows first, then router rows, written
// with the 128-byte swizzle: the 16-byte segment j of row r sits at segment
// j ^ (r & 7).  The fragment loads of mma.m16n8k16 then touch 32 distinct banks (rows
// g = 0..7 of a fragment read segments (2 kk) ^ g, all different).
//
// The ring needs no "empty" barriers: the block meets at one __syncthreads per chunk
// (as the cp.async version does), after which the stage of the previous chunk is free
// and thread 0 refills it.  The wait for a stage is bounded in time; a wait that runs
// out records DS_TIMEOUT_ROUTE in the status word and the block leaves without
// writing results.
//
// Used by the handle's forward path for bf16 rows on a 16-byte boundary; the
// handle-free entry point and unaligned inputs keep route_tc_kernel.
#pragma once
#include "route.cuh"
#include "tc5_ptx.cuh"

namespace moe {

constexpr int DS_TIMEOUT_ROUTE = 0x108;  // a router stage did not arrive in time

template <int NT, int MT>
__host__ __device__ constexpr int route_tma_stage_bytes() {
    return (16 * MT + 32 * NT) * 128;
}

// Stages: as many as fit in ~200 KB (short blocks: one block per SM, the deeper the
// ring the fewer load round trips in the chain), at most 32; the 64-token blocks of
// large batches stay under half of it so that two blocks share an SM.
template <int NT, int MT>
__host__ __device__ constexpr int route_tma_stages() {
    constexpr int budget = (MT == 4 ? 100 : 200) * 1024;
    constexpr int fit = budget / route_tma_stage_bytes<NT, MT>();
    return fit > 32 ? 32 : (fit < 3 ? 3 : fit);
}

template <int NT, int MT>
constexpr size_t route_tma_smem_bytes() {
    size_t tiles = (size_t)route_tma_stages<NT, MT>() * route_tma_stage_bytes<NT, MT>();
    size_t logits = (size_t)(16 * MT) * (32 * NT) * 4;
    // + histogram, barriers, abort flag, and room to align the stages to 1024 bytes
    return (tiles > logits ? tiles : logits) + 256 * sizeof(int) + 32 * 8 + 16 + 1024;
}

// map_x: bf16 [T, H], box {64 columns, 16 MT rows}; map_w: bf16 [E, H], box {64, 32 NT}.
// Grid: ceil(T / (16 MT)) blocks of RTHREADS threads.
template <int NT, int MT>
__global__ void __launch_bounds__(RTHREADS)
route_tma_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                 int T, int H, const float* __restrict__ b_router, int E, int K,
                 float* __restrict__ score_out, int* __restrict__ topk_i, float* __restrict__ topk_w,
                 int* __restrict__ blk_hist, int* __restrict__ status) {
    using namespace tc5;
    constexpr int RBT = 16 * MT;     // tokens of this block
    constexpr int EP = NT * 32;      // padded expert count
    constexpr int N_TILES = NT * 4;  // n8 tiles over the experts
    constexpr int NG = 8 / MT;       // 8 warps = MT m-tiles x NG expert groups
    constexpr int NTW = (N_TILES + NG - 1) / NG;
    constexpr int S = route_tma_stages<NT, MT>();
    constexpr int STAGE = route_tma_stage_bytes<NT, MT>();
    constexpr size_t tiles_b = (size_t)S * STAGE;
    constexpr size_t lg_b = (size_t)RBT * EP * 4;
    static_assert(S >= 3 && S <= 32, "ring depth");

    extern __shared__ unsigned char smem_dyn[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~static_cast<uintptr_t>(1023));
    unsigned char* tiles = smem;
    float* lg = reinterpret_cast<float*>(smem);  // [RBT][EP], reuses the stages after the K loop
    int* hist = reinterpret_cast<int*>(smem + (tiles_b > lg_b ? tiles_b : lg_b));
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(hist + 256);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 32);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t4 = lane & 3;
    const int mb = warp % MT, ng = warp / MT;  // this warp's m-tile and expert group
    const int t0 = blockIdx.x * RBT;
    pdl_trigger();
    for (int i = tid; i < 256; i += RTHREADS)
        hist[i] = 0;
    if (tid == 0) {
        *abort_flag = 0;
        for (int s = 0; s < S; s++)
            mbar_init(smem_u32(bars + s), 1);
        fence_barrier_init();
    }
    __syncthreads();
    pdl_wait();  // the rows may come from the kernel before this one

    // Every block walks the K chunks in its own rotation: all blocks read the same
    // router rows, and in lock step they would all ask the same L2 lines at once.
    const int n_chunks = H / RMK;  // H is a multiple of 64
    const int c_rot = (int)((blockIdx.x * 7u) % (unsigned)n_chunks);
    auto issue = [&](int c) {  // thread 0: both copies of the block's c-th chunk into its stage
        int k = c + c_rot;
        if (k >= n_chunks)
            k -= n_chunks;
        const int s = c % S;
        const uint32_t bar = smem_u32(bars + s);
        const uint32_t dst = smem_u32(tiles + (size_t)s * STAGE);
        mbar_expect_tx(bar, (uint32_t)STAGE);
        tma_load_2d(dst, &map_x, bar, k * RMK, t0);
        tma_load_2d(dst + RBT * 128, &map_w, bar, k * RMK, 0);
    };
    if (tid == 0) {
        for (int c = 0; c < S - 1 && c < n_chunks; c++)
            issue(c);
    }

    float run[NTW][4];
#pragma unroll
    for (int n = 0; n < NTW; n++)
#pragma unroll
        for (int i = 0; i < 4; i++)
            run[n][i] = 0.f;

    // byte offsets of this lane's fragment words inside a stage: row * 128 + swizzled segment
    const uint32_t a_row = (uint32_t)(mb * 16 + g) * 128u + (uint32_t)t4 * 4u;
    const uint32_t seg_x = (uint32_t)g;  // (row & 7) of every row this lane reads

    bool ok = true;
    for (int c = 0; c < n_chunks; c++) {
        const bool mine = mbar_wait(smem_u32(bars + (c % S)), (uint32_t)(c / S) & 1u, status,
                                    DS_TIMEOUT_ROUTE, abort_flag);
        // everybody has chunk c, and chunk c-1 is consumed; a block leaves together
        if (__syncthreads_or(!mine)) {
            ok = false;
            break;
        }
        if (tid == 0 && c + S - 1 < n_chunks)
            issue(c + S - 1);  // into the stage chunk c-1 just left
        const unsigned char* xs = tiles + (size_t)(c % S) * STAGE;
        const unsigned char* ws = xs + RBT * 128;
        float acc[NTW][4];
#pragma unroll
        for (int n = 0; n < NTW; n++)
#pragma unroll
            for (int i = 0; i < 4; i++)
                acc[n][i] = 0.f;
        if (ng * NTW < N_TILES) {
#pragma unroll
            for (int kk = 0; kk < RMK / 16; kk++) {
                const uint32_t s_lo = ((uint32_t)(2 * kk) ^ seg_x) << 4, s_hi = ((uint32_t)(2 * kk + 1) ^ seg_x) << 4;
                uint32_t af[4];
                af[0] = *reinterpret_cast<const uint32_t*>(xs + a_row + s_lo);
                af[1] = *reinterpret_cast<const uint32_t*>(xs + a_row + 8 * 128 + s_lo);
                af[2] = *reinterpret_cast<const uint32_t*>(xs + a_row + s_hi);
                af[3] = *reinterpret_cast<const uint32_t*>(xs + a_row + 8 * 128 + s_hi);
#pragma unroll
                for (int n = 0; n < NTW; n++) {
                    const int nt = ng * NTW + n;
                    if (nt < N_TILES) {
                        const unsigned char* pb = ws + (uint32_t)(nt * 8 + g) * 128u + (uint32_t)t4 * 4u;
                        uint32_t bf[2];
                        bf[0] = *reinterpret_cast<const uint32_t*>(pb + s_lo);
                        bf[1] = *reinterpret_cast<const uint32_t*>(pb + s_hi);
                        route_mma_16816(acc[n], af, bf);
                    }
                }
            }
        }
#pragma unroll
        for (int n = 0; n < NTW; n++)
#pragma unroll
            for (int i = 0; i < 4; i++)
                run[n][i] += acc[n][i];
    }
    if (!ok) {
        // copies already issued may still be in flight: give them a bounded time to land
        // before the block's shared memory goes away
        if (tid == 0) {
            const unsigned long long t_0 = global_timer_ns();
            while (global_timer_ns() - t_0 < 100000000ull)
                __nanosleep(1000);
        }
        __syncthreads();
        return;
    }
    __syncthreads();  // every copy has landed and is consumed; lg aliases the stages
#pragma unroll
    for (int n = 0; n < NTW; n++) {
        const int nt = ng * NTW + n;
        if (nt < N_TILES) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int row = mb * 16 + g + 8 * (i >> 1);
                const int e = nt * 8 + 2 * t4 + (i & 1);
                lg[row * EP + e] = (e < E) ? run[n][i] + b_router[e] : -INFINITY;
            }
        }
    }
    __syncthreads();
    if (score_out) {
        for (int i = tid; i < RBT * E; i += RTHREADS) {
            const int r = i / E, e = i - r * E;
            if (t0 + r < T)
                score_out[(size_t)(t0 + r) * E + e] = lg[r * EP + e];
        }
    }
    for (int r = warp; r < RBT; r += RTHREADS / 32) {
        const int t = t0 + r;
        if (t >= T)
            break;
        float v[NT];
#pragma unroll
        for (int j = 0; j < NT; j++)
            v[j] = lg[r * EP + lane + 32 * j];
        select_topk_softmax<NT>(v, lane, K, t, topk_i, topk_w, hist);
    }
    __syncthreads();
    for (int e = tid; e < E; e += RTHREADS)
        blk_hist[(size_t)blockIdx.x * E + e] = hist[e];
}

}  // namespace moe
