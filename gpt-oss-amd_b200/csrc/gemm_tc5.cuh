// Grouped expert GEMMs on the 5th-generation tensor cores (tcgen05, sm_100a).
//
//   MODE 0: h[rows, I]  = SwiGLU(x[rows, H] . W1_e^T + b1_e)      (bf16 out)
//           moe_mlp1_swiglu, src/hip/moe.hip:9-258
//   MODE 1: y[rows, H]  = h[rows, I] . W2_e^T + b2_e              (fp32 out)
//           moe_mlp2_store / moe_mlp2_scatter, src/hip/moe.hip:261-800
//
// One persistent CTA per SM walks a device-built list of (expert, m-tile,
// n-tile) work items; no value is read back by the host (the reference sizes
// its grids from a per-layer device->host copy, src/forward.cpp:340-345,381).
//
// Orientation: D[128 weight rows, N token rows] = W_tile . X_tile^T, i.e. the
// weight tile is the UMMA A operand (M = 128 TMEM lanes) and the token rows are
// the B operand (N = 16..BN columns), so a ragged expert only narrows N.
//
// Shared-memory rings:
//   W ring   packed MXFP4 chunks (4352 B each), deep: covers the HBM latency
//            bulk copy -> decode warps
//   AB ring  STAGES slots, each a decoded bf16 weight tile (16 KB, written by
//            the decode warps) plus an activation tile (BN x 128 B, written by
//            TMA); ONE `full` barrier per slot collects the decode warps'
//            arrivals and the TMA transaction bytes, ONE `empty` barrier per
//            slot is signalled by tcgen05.commit, so the MMA-issuing thread does
//            one wait and one commit per pipeline step.
// This is the single-CTA kernel for LARGE batches (BN = 256 token rows per tile:
// a decoded weight tile feeds 256 token rows, the best ratio of decode work to
// FLOPs that two accumulator sets in tensor memory allow), selected with
// gemm_impl = MOE_B200_GEMM_TCGEN05_1CTA; the default runs large batches on CTA
// pairs (gemm_tc5_pair.cuh, same structure, half the activation bytes per SM) and
// calls with few rows per expert on gemm_tc5_swap.cuh, where the token rows are on
// the TMEM lanes instead.  The geometry stays a template (Geo<BN>): MT weight
// tiles per item and NACC K-split accumulators are 1 here.
//
// Warp roles:
//   warp 0       W producer        warp 1   B producer (TMA)
//   warp 2       allocates tensor memory, issues tcgen05.mma, commits
//   next 4*G     decode packed MXFP4 -> bf16 into the 128B-swizzled A slot, G
//                groups of four warps working on G pipeline steps at once
//   last 4*MT    epilogue: tcgen05.ld, bias, SwiGLU / store
//
// Every mbarrier wait is bounded in time; a wait that runs out records a code
// in the handle's status word, raises a CTA-wide abort flag and all roles fall
// through to the common exit where tensor memory is released.
#pragma once
#include "gemm_mma.cuh"  // swiglu()
#include "tc5_ptx.cuh"

namespace moe {
namespace tc5 {

constexpr int A_TILE_BYTES = TILE_M * 128;  // one decoded weight tile: 128 rows x 64 bf16, SW128
constexpr int MMA_WARP = 2;
constexpr int DEQ_WARP0 = 3;
constexpr int MAX_LOCAL_EXPERTS = 256;
constexpr int EPI_STAGE_BYTES = 2048;  // per epilogue warp: 32 token rows x 16 features bf16 (padded) or 16 token rows x 32 columns fp32

// Geometry per tile width BN (token rows per work item):
//   MT      weight tiles (of 128 rows) per work item.  The activation tile is
//           what a CTA pulls through L2 at every step; feeding two weight tiles
//           from it halves that traffic per FLOP, which is what bounds the
//           prefill-shaped GEMM (L2 -> SM bandwidth, not the tensor pipe)
//   G       decode groups (of four warps); group g decodes pipeline steps g, g+G, ...
//   STAGES  depth of the AB ring     WS  depth of the packed-weight ring.  Both are
//           multiples of G, so the successive fills of a slot are consumed by the same
//           group in program order: an mbarrier parity wait cannot tell phase n from
//           phase n-2, so a waiter must never run two phases ahead of a slot
//   NACC    K-split accumulators per weight tile (narrow tiles: back-to-back
//           MMAs into one accumulator are a dependent chain)
//   SETS    accumulator sets in tensor memory (2 = the MMAs of the next work
//           item overlap the epilogue of this one)
// SETS * MT * NACC * BN = 512 columns in every case.
template <int BN>
struct Geo;
template <>
struct Geo<256> {
    static constexpr int MT = 1, G = 4, STAGES = 4, WS = 4, NACC = 1, SETS = 2;
};

template <int BN>
__host__ __device__ constexpr int n_threads() {
    return (DEQ_WARP0 + 4 * Geo<BN>::G + 4 * Geo<BN>::MT) * 32;  // 608 or 736
}
template <int BN>
__host__ __device__ constexpr int n_barriers() {
    return 2 * Geo<BN>::WS + 2 * Geo<BN>::STAGES + 2 * Geo<BN>::SETS;
}
template <int BN>
__host__ __device__ constexpr int smem_bytes() {
    return Geo<BN>::STAGES * (Geo<BN>::MT * A_TILE_BYTES + BN * 128) +
           Geo<BN>::WS * Geo<BN>::MT * CHUNK_BYTES + 4 * Geo<BN>::MT * EPI_STAGE_BYTES +
           n_barriers<BN>() * 8 +
           (MAX_LOCAL_EXPERTS + 1) * 3 * 4 + 64 + 1024;  // + tile tables + holder/flag + alignment slack
}

struct TileInfo {
    int e, mt0, n_mt, row0, valid_n, n_mma, box_idx, box_rows;
};

// The tile tables live in shared memory (copied once per CTA): every role
// decodes every work item it touches, and a binary search over global memory
// costs several L2 round trips.
struct TileTables {
    const int* off;         // [E + 1]
    const int* cnt;         // [E]
    const int* tile_start;  // [E + 1]
};

// Work items ordered [expert][m_item][n_tile]: the n-tiles that share weight
// chunks run on neighbouring CTAs at the same time and meet in L2.  An m_item
// is MT consecutive weight tiles (the last one of a matrix may hold fewer).
template <int BN>
__device__ __forceinline__ TileInfo decode_tile(int tile, int m_tiles, int m_items,
                                                const TileTables& tt, int E) {
    int lo = 0, hi = E;
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (tt.tile_start[mid] * m_items <= tile)
            lo = mid;
        else
            hi = mid;
    }
    TileInfo ti;
    ti.e = lo;
    const int ntl = tt.tile_start[lo + 1] - tt.tile_start[lo];
    const int r = tile - tt.tile_start[lo] * m_items;
    const int mi = r / ntl;
    ti.mt0 = mi * Geo<BN>::MT;
    ti.n_mt = min(Geo<BN>::MT, m_tiles - ti.mt0);
    const int n0 = (r - mi * ntl) * BN;
    ti.row0 = tt.off[lo] + n0;
    ti.valid_n = min(BN, tt.cnt[lo] - n0);
    ti.n_mma = max(16, (ti.valid_n + 15) & ~15);
    ti.box_idx = ti.n_mma <= 32 ? 0 : ti.n_mma <= 64 ? 1 : ti.n_mma <= 128 ? 2 : 3;
    ti.box_rows = 32 << ti.box_idx;
    return ti;
}

template <int MODE, int BN>
__global__ void __launch_bounds__(n_threads<BN>(), 1)
expert_gemm_tc5_kernel(const __grid_constant__ TensorMaps maps, const uint8_t* __restrict__ chunks,
                       size_t expert_stride, int k_stages, int m_tiles,
                       const float* __restrict__ bias, int bias_stride,
                       const int* __restrict__ g_off, const int* __restrict__ g_cnt,
                       const int* __restrict__ g_tile_start, int E, void* __restrict__ outp,
                       int out_ld, int out_rows_valid, const int* __restrict__ row_dst,
                       float* const* __restrict__ row_ptr, float alpha, float limit,
                       int* __restrict__ status) {
    constexpr int MT = Geo<BN>::MT, STAGES = Geo<BN>::STAGES, WS = Geo<BN>::WS;
    constexpr int NACC = Geo<BN>::NACC, SETS = Geo<BN>::SETS;
    constexpr int THREADS = n_threads<BN>();
    constexpr int A_SLOT_BYTES = MT * A_TILE_BYTES;
    constexpr int B_SLOT_BYTES = BN * 128;
    constexpr int W_SLOT_BYTES = MT * CHUNK_BYTES;
    constexpr int SET_COLS = MT * NACC * BN;  // columns of one accumulator set
    constexpr int TMEM_COLS = SETS * SET_COLS;
    constexpr int EPI_WARPS = 4 * MT;
    constexpr int DEQ_GROUPS = Geo<BN>::G;
    constexpr int EPI_WARP0 = DEQ_WARP0 + 4 * DEQ_GROUPS;  // any four consecutive warps cover the four TMEM lane quarters
    static_assert(TMEM_COLS == 512, "the accumulator sets fill tensor memory");
    static_assert(STAGES % DEQ_GROUPS == 0 && WS % DEQ_GROUPS == 0,
                  "a slot's successive fills must belong to one decode group");

    extern __shared__ unsigned char smem_dyn[];
    // slots need 1024-byte alignment for the 128-byte swizzle
    unsigned char* smem = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
    unsigned char* a_ring = smem;
    unsigned char* b_ring = a_ring + STAGES * A_SLOT_BYTES;
    unsigned char* w_ring = b_ring + STAGES * B_SLOT_BYTES;
    unsigned char* epi_stage = w_ring + WS * W_SLOT_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(epi_stage + EPI_WARPS * EPI_STAGE_BYTES);
    int* s_tables = reinterpret_cast<int*>(bars + n_barriers<BN>());
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(s_tables + 3 * (MAX_LOCAL_EXPERTS + 1));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

    const uint32_t bar0 = smem_u32(bars);
    auto bar_w_full = [&](int s) { return bar0 + 8u * (uint32_t)s; };
    auto bar_w_empty = [&](int s) { return bar0 + 8u * (uint32_t)(WS + s); };
    auto bar_full = [&](int s) { return bar0 + 8u * (uint32_t)(2 * WS + s); };
    auto bar_empty = [&](int s) { return bar0 + 8u * (uint32_t)(2 * WS + STAGES + s); };
    auto bar_tmem_full = [&](int b) { return bar0 + 8u * (uint32_t)(2 * WS + 2 * STAGES + b); };
    auto bar_tmem_empty = [&](int b) { return bar0 + 8u * (uint32_t)(2 * WS + 2 * STAGES + SETS + b); };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < WS; s++) {
            mbar_init(bar_w_full(s), 1);
            mbar_init(bar_w_empty(s), 4);  // one elected arrival per warp of the decoding group
        }
        for (int s = 0; s < STAGES; s++) {
            mbar_init(bar_full(s), 4 + 1);  // four decode warps + the TMA producer's expect_tx
            mbar_init(bar_empty(s), 1);     // tcgen05.commit
        }
        for (int b = 0; b < SETS; b++) {
            mbar_init(bar_tmem_full(b), 1);
            mbar_init(bar_tmem_empty(b), EPI_WARPS);  // one per epilogue warp
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    for (int i = threadIdx.x; i <= E; i += THREADS) {
        s_tables[i] = g_off[i];
        s_tables[(MAX_LOCAL_EXPERTS + 1) + i] = (i < E) ? g_cnt[i] : 0;
        s_tables[2 * (MAX_LOCAL_EXPERTS + 1) + i] = g_tile_start[i];
    }
    if (warp == MMA_WARP)
        tmem_alloc(smem_u32(tmem_holder), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_holder;
    TileTables tt;
    tt.off = s_tables;
    tt.cnt = s_tables + (MAX_LOCAL_EXPERTS + 1);
    tt.tile_start = s_tables + 2 * (MAX_LOCAL_EXPERTS + 1);

    const int m_items = (m_tiles + MT - 1) / MT;
    const int total_tiles = tt.tile_start[E] * m_items;

    if (warp == 0) {
        // ------------------------- packed-weight producer ----------------------
        if (lane == 0) {
            int s = 0, armed = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                const TileInfo ti = decode_tile<BN>(tile, m_tiles, m_items, tt, E);
                const uint8_t* wsrc = chunks + (size_t)ti.e * expert_stride +
                                      (size_t)ti.mt0 * k_stages * CHUNK_BYTES;
                for (int ks = 0; ks < k_stages; ks++) {
                    ok = mbar_wait(bar_w_empty(s), ph ^ 1u, status, DS_TIMEOUT_EMPTY, abort_flag);
                    if (!ok)
                        break;
                    mbar_expect_tx(bar_w_full(s), (uint32_t)(ti.n_mt * CHUNK_BYTES));
                    for (int j = 0; j < ti.n_mt; j++)
                        bulk_load(smem_u32(w_ring + s * W_SLOT_BYTES + j * CHUNK_BYTES),
                                  wsrc + ((size_t)j * k_stages + ks) * CHUNK_BYTES, CHUNK_BYTES,
                                  bar_w_full(s));
                    armed = min(armed + 1, WS);
                    RING_ADVANCE(s, ph, WS);
                }
            }
            if (!ok) {
                for (int i = 0; i < armed; i++) {  // walk back over the copies in flight
                    if (--s < 0) {
                        s = WS - 1;
                        ph ^= 1u;
                    }
                    drain_wait(bar_w_full(s), ph);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------- activation-tile producer --------------------
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                const TileInfo ti = decode_tile<BN>(tile, m_tiles, m_items, tt, E);
                for (int ks = 0; ks < k_stages; ks++) {
                    ok = mbar_wait(bar_empty(s), ph ^ 1u, status, DS_TIMEOUT_EMPTY, abort_flag);
                    if (!ok)
                        break;
                    mbar_expect_tx(bar_full(s), (uint32_t)ti.box_rows * 128u);
                    tma_load_2d(smem_u32(b_ring + s * B_SLOT_BYTES), &maps.box[ti.box_idx],
                                bar_full(s), ks * KSTAGE, ti.row0);
                    RING_ADVANCE(s, ph, STAGES);
                }
            }
        }
    } else if (warp == MMA_WARP) {
        // ------------------------------ MMA issuer ----------------------------
        // The whole warp runs the loop with no lane-divergent code but the elected
        // issue itself: uniform control flow keeps the descriptors in uniform
        // registers, where tcgen05.mma reads them from.  The barrier of the NEXT step
        // is tested before the MMAs of this step are issued, so that its latency
        // overlaps the issue instead of adding to the per-step chain of this warp.
        // The operands in shared memory need no tcgen05 fence: TMA completes through
        // the mbarrier and the decode warps fence the async proxy before they arrive.
        int s = 0;
        uint32_t ph = 0;
        bool ok = true;
        int it = 0;
        bool ready = false;  // full[s] already seen complete for phase ph
        for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++it) {
            const TileInfo ti = decode_tile<BN>(tile, m_tiles, m_items, tt, E);
            const int set = it % SETS, round = it / SETS;
            ok = mbar_wait(bar_tmem_empty(set), (uint32_t)(round & 1) ^ 1u, status,
                           DS_TIMEOUT_TMEM_EMPTY, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok)
                break;
            tc_fence_after();  // the epilogue's tcgen05.ld of this set came before
            const uint32_t d_set = tmem_base + (uint32_t)(set * SET_COLS);
            const uint32_t idesc = make_idesc(ti.n_mma);
            for (int ks = 0; ks < k_stages; ks++) {
                if (!ready) {
                    ok = mbar_wait(bar_full(s), ph, status, DS_TIMEOUT_FULL_A, abort_flag);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok)
                        break;
                }
                if (lane == 0)
                    TRACE(it * k_stages + ks, 4);
                int s_next = s;
                uint32_t ph_next = ph;
                RING_ADVANCE(s_next, ph_next, STAGES);
                const uint32_t peek = mbar_try_wait(bar_full(s_next), ph_next);
                const uint64_t a_desc = make_sw128_desc(smem_u32(a_ring + s * A_SLOT_BYTES));
                const uint64_t b_desc = make_sw128_desc(smem_u32(b_ring + s * B_SLOT_BYTES));
                if (elect_one_sync()) {
#pragma unroll
                    for (int j = 0; j < MT; j++) {
                        if (j < ti.n_mt) {
#pragma unroll
                            for (int kk = 0; kk < KSTAGE / 16; kk++) {
                                // K-split: MMA kk goes to accumulator kk % NACC of weight tile
                                // j; each accumulator's first MMA of the work item overwrites
                                const int acc = j * NACC + kk % NACC;
                                const uint32_t accumulate = (ks == 0 && kk < NACC) ? 0u : 1u;
                                umma_bf16(d_set + (uint32_t)(acc * BN),
                                          a_desc + (uint64_t)(j * (A_TILE_BYTES >> 4) + kk * 2),
                                          b_desc + (uint64_t)(kk * 2), idesc, accumulate);
                            }
                        }
                    }
                    umma_commit(bar_empty(s));  // frees the slot when these MMAs have read it
                }
                if (lane == 0)
                    TRACE(it * k_stages + ks, 5);
                ready = __all_sync(0xffffffffu, peek != 0);
                s = s_next;
                ph = ph_next;
            }
            if (ok && elect_one_sync())
                umma_commit(bar_tmem_full(set));
            __syncwarp();
        }
    } else if (warp < EPI_WARP0) {
        // ------------------------------ MXFP4 decode --------------------------
        // DEQ_GROUPS groups of 4 warps; group g decodes the pipeline steps
        // g, g + DEQ_GROUPS, ... so that several steps are in flight at once (one
        // step is a chain of waits, loads and dependent ALU instructions, longer
        // than the MMAs of a step).  A thread owns row r of each weight tile of
        // the work item and decodes both of its 32-column blocks.
        const int u = threadIdx.x - DEQ_WARP0 * 32;
        const int g = u >> 7;
        const int r = u & (TILE_M - 1);
        const uint32_t a_row_off = (uint32_t)((r >> 3) * 1024 + (r & 7) * 128);
        const int my_tiles = (int)blockIdx.x < total_tiles
                                 ? (total_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
        const int total_steps = my_tiles * k_stages;
        bool ok = true;
        int cached_lt = -1, n_mt = MT;
        for (int i = g; ok && i < total_steps; i += DEQ_GROUPS) {
            if (MT > 1) {
                const int lt = i / k_stages;
                if (lt != cached_lt) {
                    cached_lt = lt;
                    n_mt = decode_tile<BN>((int)blockIdx.x + lt * (int)gridDim.x, m_tiles, m_items, tt, E).n_mt;
                }
            }
            const int sw = i % WS, sa = i % STAGES;
            const uint32_t phw = (uint32_t)(i / WS) & 1u, pha = (uint32_t)(i / STAGES) & 1u;
            ok = mbar_wait(bar_w_full(sw), phw, status, DS_TIMEOUT_FULL_W, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok)
                break;
            if (MT == 1) {
                // decode into registers first, release the packed chunk, and only then
                // wait for the A slot: the ALU work overlaps the MMAs still reading it
                const unsigned char* wst = w_ring + sw * W_SLOT_BYTES;
                const uint4 q0 = *reinterpret_cast<const uint4*>(wst + r * 16);
                const uint4 q1 = *reinterpret_cast<const uint4*>(wst + PLANE_BYTES + r * 16);
                const uint32_t sc = *reinterpret_cast<const uint16_t*>(wst + 2 * PLANE_BYTES + r * 2);
                const uint32_t mult0 = mxfp4_scale_mult(sc & 0xFFu);
                const uint32_t mult1 = mxfp4_scale_mult(sc >> 8);
                const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
                uint32_t d[8][4];
#pragma unroll
                for (int c = 0; c < 8; c++)
                    mxfp4_decode_word(w[c], c < 4 ? mult0 : mult1, d[c]);
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(bar_w_empty(sw));
                ok = mbar_wait(bar_empty(sa), pha ^ 1u, status, DS_TIMEOUT_EMPTY, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok)
                    break;
                unsigned char* arow = a_ring + sa * A_SLOT_BYTES + a_row_off;
#pragma unroll
                for (int c = 0; c < 8; c++)
                    *reinterpret_cast<uint4*>(arow + ((c ^ (r & 7)) * 16)) =
                        make_uint4(d[c][0], d[c][1], d[c][2], d[c][3]);
                fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor core
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(bar_full(sa));
            } else {
                ok = mbar_wait(bar_empty(sa), pha ^ 1u, status, DS_TIMEOUT_EMPTY, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok)
                    break;
#pragma unroll
                for (int j = 0; j < MT; j++) {
                    if (j < n_mt) {
                        const unsigned char* wst = w_ring + sw * W_SLOT_BYTES + j * CHUNK_BYTES;
                        const uint4 q0 = *reinterpret_cast<const uint4*>(wst + r * 16);
                        const uint4 q1 = *reinterpret_cast<const uint4*>(wst + PLANE_BYTES + r * 16);
                        const uint32_t sc = *reinterpret_cast<const uint16_t*>(wst + 2 * PLANE_BYTES + r * 2);
                        const uint32_t mult0 = mxfp4_scale_mult(sc & 0xFFu);
                        const uint32_t mult1 = mxfp4_scale_mult(sc >> 8);
                        const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
                        unsigned char* arow = a_ring + sa * A_SLOT_BYTES + j * A_TILE_BYTES + a_row_off;
#pragma unroll
                        for (int c = 0; c < 8; c++) {
                            uint32_t d[4];
                            mxfp4_decode_word(w[c], c < 4 ? mult0 : mult1, d);
                            *reinterpret_cast<uint4*>(arow + ((c ^ (r & 7)) * 16)) =
                                make_uint4(d[0], d[1], d[2], d[3]);
                        }
                    }
                }
                fence_proxy_async_smem();
                __syncwarp();
                // one arrival per warp: hundreds of per-thread arrivals on one mbarrier
                // serialise in shared memory
                if (lane == 0) {
                    mbar_arrive(bar_full(sa));
                    mbar_arrive(bar_w_empty(sw));
                }
            }
        }
    } else {
        // ------------------------------ epilogue ------------------------------
        const int j = (warp - EPI_WARP0) >> 2;  // weight tile of the work item this warp drains
        const int q = warp & 3;                 // TMEM lane quarter this warp may read
        const int row = q * 32 + lane;          // row inside the weight tile
        bool ok = true;
        int it = 0;
        for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++it) {
            const TileInfo ti = decode_tile<BN>(tile, m_tiles, m_items, tt, E);
            const int set = it % SETS, round = it / SETS;
            ok = mbar_wait(bar_tmem_full(set), (uint32_t)(round & 1), status, DS_TIMEOUT_TMEM_FULL,
                           abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok)
                break;
            if (warp == EPI_WARP0 && lane == 0)
                TRACE(it * k_stages, 10);
            tc_fence_after();
            if (j < ti.n_mt) {
                const float* be = bias + (size_t)ti.e * bias_stride;
                const int m = (ti.mt0 + j) * TILE_M + row;
                const uint32_t t_addr = tmem_base + ((uint32_t)(q * 32) << 16) +
                                        (uint32_t)(set * SET_COLS + j * NACC * BN);
                if (MODE == 0) {
                    // Lanes 2p / 2p+1 hold the gate / up row of feature pair p.  After one
                    // exchange the even lane finishes columns c0..c0+15 of that feature and
                    // the odd lane columns c0+16..c0+31.  The warp's 32 token rows x 16
                    // features are transposed through shared memory so that every global
                    // store writes 16 bytes per lane: 2-byte stores cost ~170 cycles per
                    // warp instruction here, 16 of them per 32 columns.
                    uint16_t* h = static_cast<uint16_t*>(outp);
                    unsigned char* stage = epi_stage + (warp - EPI_WARP0) * EPI_STAGE_BYTES;
                    uint16_t* stage16 = reinterpret_cast<uint16_t*>(stage);
                    const float bm = be[m];  // 2I is a multiple of TILE_M: always in range
                    const int jf0 = ((ti.mt0 + j) * TILE_M + q * 32) >> 1;  // first of this warp's 16 features
                    const bool odd = (lane & 1) != 0;
                    // token rows 16..31 sit 64 bytes further: no bank conflict between the halves
                    const int st_idx = (odd ? 16 * 16 + 32 : 0) + (lane >> 1);
                    for (int c0 = 0; c0 < ti.n_mma; c0 += 32) {
                        float v[32];
                        tmem_ld_sum<NACC, BN>(t_addr + (uint32_t)c0, v);
#pragma unroll
                        for (int c = 0; c < 16; c++) {
                            const float mine_lo = v[c] + bm, mine_hi = v[c + 16] + bm;
                            const float send = odd ? mine_lo : mine_hi;
                            const float recv = __shfl_xor_sync(0xffffffffu, send, 1);
                            const float gate = odd ? recv : mine_lo;
                            const float up = odd ? mine_hi : recv;
                            stage16[st_idx + c * 16] =
                                (uint16_t)float_to_bf16_bits(swiglu(gate, up, alpha, limit));
                        }
                        __syncwarp();
#pragma unroll
                        for (int p = 0; p < 2; p++) {
                            const int tok = (lane >> 1) + 16 * p, hf = lane & 1;
                            const uint4 val = *reinterpret_cast<const uint4*>(
                                stage + tok * 32 + hf * 16 + p * 64);
                            const int col = c0 + tok, jf = jf0 + hf * 8;
                            if (col < ti.valid_n && jf < out_rows_valid)
                                *reinterpret_cast<uint4*>(h + (size_t)(ti.row0 + col) * out_ld + jf) = val;
                        }
                        __syncwarp();
                    }
                } else {
                    // A lane holds one output column m for 32 token rows; 16 token rows
                    // at a time are transposed through shared memory so that a lane stores
                    // 16 bytes and a warp instruction four whole 128-byte row segments
                    // (a global store costs this kernel ~170 cycles per warp instruction
                    // whatever its width: one per token row made the epilogue longer
                    // than the main loop).
                    float* y = static_cast<float*>(outp);
                    unsigned char* stage = epi_stage + (warp - EPI_WARP0) * EPI_STAGE_BYTES;
                    float* stage32 = reinterpret_cast<float*>(stage);
                    const float bm = (m < out_rows_valid) ? be[m] : 0.f;
                    const int m4 = (ti.mt0 + j) * TILE_M + q * 32 + (lane & 7) * 4;  // columns this lane stores
                    const bool m4_ok = m4 < out_rows_valid;                          // the width is a multiple of 4
                    for (int c0 = 0; c0 < ti.n_mma; c0 += 32) {
                        float v[32];
                        tmem_ld_sum<NACC, BN>(t_addr + (uint32_t)c0, v);
#pragma unroll
                        for (int half = 0; half < 2; half++) {
#pragma unroll
                            for (int c = 0; c < 16; c++)
                                stage32[c * 32 + lane] = v[half * 16 + c] + bm;
                            __syncwarp();
#pragma unroll
                            for (int p = 0; p < 4; p++) {
                                const int tok = (lane >> 3) + 4 * p;
                                const float4 val =
                                    *reinterpret_cast<const float4*>(stage + (lane + 32 * p) * 16);
                                const int col = c0 + half * 16 + tok;
                                if (col < ti.valid_n && m4_ok) {
                                    // result row: on another GPU (peer mode), at a remapped row
                                    // (received order), or in place
                                    const int rr = ti.row0 + col;
                                    float* yrow = row_ptr ? row_ptr[rr]
                                                          : y + (size_t)(row_dst ? row_dst[rr] : rr) * out_ld;
                                    *reinterpret_cast<float4*>(yrow + m4) = val;
                                }
                            }
                            __syncwarp();
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(bar_tmem_empty(set));
            if (warp == EPI_WARP0 && lane == 0)
                TRACE(it * k_stages, 11);
        }
    }

    // common exit: every role comes here, finished or aborted
    tc_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

}  // namespace tc5
}  // namespace moe
