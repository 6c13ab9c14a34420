// Grouped expert GEMMs for LARGE batches on CTA PAIRS (tcgen05.mma.cta_group::2).
//
//   MODE 0: h[rows, I]  = SwiGLU(x[rows, H] . W1_e^T + b1_e)      (bf16 out)
//           moe_mlp1_swiglu, src/hip/moe.hip:9-258
//   MODE 1: y[rows, H]  = h[rows, I] . W2_e^T + b2_e              (fp32 out)
//           moe_mlp2_store / moe_mlp2_scatter, src/hip/moe.hip:261-800
//
// One persistent cluster of two CTAs per SM pair walks a device-built list of
// work items; no value is read back by the host (the reference sizes its grids
// from a per-layer device->host copy, src/forward.cpp:340-345,381).
//
// Orientation: D[weight rows, token rows] = W_tile . X_tile^T: the decoded weight
// tile is the UMMA A operand (TMEM lanes), the token rows the B operand, so a
// ragged expert only narrows N.  A single CTA doing this is bound by the
// activation bytes it pulls through L2 (32 KB per 64 columns of K, ~47 B/cycle/SM).
// Here a cluster of two CTAs works on one item (expert, PAIR of 128-row weight tiles, tile of 256 token rows) with
// one 256 x 256 x 16 MMA per instruction: each CTA decodes its own weight tile
// (A operand, its 128 TMEM lanes) and loads only HALF of the token tile (B
// operand: the tensor core reads rows 0..N/2-1 from the leader's shared memory and
// N/2..N-1 from the peer's), so the activation bytes per SM and per FLOP halve,
// and the MMA warp's per-step chain (one wait, four MMAs, one commit) feeds two
// SMs.
//
// Per CTA: W ring (packed chunks), A ring (decoded weights, 4 slots), B ring (half
// activation tiles of 16 KB, 8 slots) and a ring of NB barrier pairs indexed by
// the step number.  Cross-CTA synchronisation:
//   full[i]   the leader's barrier collects its own decode warps and TMA bytes plus
//             ONE arrival from the peer: the peer's warp 2 (it issues no MMAs)
//             waits for the peer's own full[i] and forwards it with a remote arrive
//   empty[i]  tcgen05.commit with cluster multicast: arrives in both CTAs
//   tmem_full / tmem_empty   multicast commit / the peer's epilogue warps arrive on
//             the leader's barrier remotely
// Both CTAs allocate and free tensor memory (cta_group::2) and meet at a cluster
// barrier before they exit, so no remote arrive can reach a CTA that has gone.
//
// Every mbarrier wait is bounded in time; a wait that runs out records a code in
// the handle's status word, raises a CTA-wide abort flag and all roles fall
// through to the common exit where tensor memory is released.
#pragma once
#include "peer_io.cuh"
#include "tc5_ptx.cuh"

namespace moe {
namespace tc5 {
namespace pair {

constexpr int BN = 256;                      // token rows per item
constexpr int BNH = BN / 2;                  // rows of the activation tile each CTA loads
constexpr int A_SLOT_BYTES = TILE_M * 128;   // decoded weight tile: 128 rows x 64 bf16, SW128
constexpr int B_SLOT_BYTES = BNH * 128;      // half activation tile
constexpr int MMA_WARP = 2;
constexpr int DEQ_WARP0 = 3;
constexpr int G = 4;                         // decode groups of four warps
// A slots, B slots, barrier pairs, packed-weight slots (deeper W / B rings measured: no change)
constexpr int SA = 4, SB = 8, NB = 8, WS = 4;
constexpr int SETS = 2;
constexpr int TMEM_COLS = SETS * BN;         // 512
constexpr int EPI_WARP0 = DEQ_WARP0 + 4 * G;
constexpr int N_THREADS = (EPI_WARP0 + 4) * 32;  // 736
constexpr int MAX_LOCAL_EXPERTS = 256;
constexpr int EPI_STAGE_BYTES = 2048;
constexpr int N_BARRIERS = 2 * WS + 2 * NB + 2 * SETS;
constexpr int SMEM_BYTES = SA * A_SLOT_BYTES + SB * B_SLOT_BYTES + WS * CHUNK_BYTES + 4 * EPI_STAGE_BYTES +
                           N_BARRIERS * 8 + (MAX_LOCAL_EXPERTS + 1) * 3 * 4 + 64 + 1024;
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory per CTA");
static_assert(SA % G == 0 && WS % G == 0 && NB % SA == 0 && NB % SB == 0 && NB % G == 0,
              "a slot's successive fills must belong to one decode group");

// ---- cluster / cta_group::2 PTX ------------------------------------------------

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on the barrier at the same shared-memory offset in CTA `rank` of the cluster.
__device__ __forceinline__ void mbar_arrive_remote(uint32_t bar, uint32_t rank) {
    asm volatile(
        "{\n\t.reg .b32 ra;\n\t"
        "mapa.shared::cluster.u32 ra, %0, %1;\n\t"
        "mbarrier.arrive.shared::cluster.b64 _, [ra];\n\t}"
        ::"r"(bar), "r"(rank) : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst),
                 "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem, 256 lanes over the pair] (+)= A . B^T, issued by one thread of the leader CTA.
__device__ __forceinline__ void umma2_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                           uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives on `bar` in BOTH CTAs when every MMA issued so far by this thread is done.
__device__ __forceinline__ void umma2_commit_both(uint32_t bar) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(bar), "h"((uint16_t)3) : "memory");
}
// Instruction descriptor: bf16 x bf16 -> fp32, both operands K-major, M = 256 over the pair.
__device__ __forceinline__ uint32_t make_idesc2(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

struct TileInfo {
    int e;        // local expert
    int mp;       // pair of weight tiles: tiles 2 mp and 2 mp + 1
    int row0;     // first token row of the item
    int valid_n;  // token rows of the item (1..256)
    int n_mma;    // rows the MMA computes (a multiple of 32)
    int box_idx;  // TMA box for this CTA's half: 32 << box_idx rows
};

struct TileTables {
    const int* off;         // [E + 1]
    const int* cnt;         // [E]
    const int* tile_start;  // [E + 1]  prefix of ceil(cnt / BN)
};

// Items ordered [expert][weight-tile pair][token tile]: the token tiles that share
// weight chunks run on neighbouring clusters at the same time and meet in L2.
__device__ __forceinline__ TileInfo decode_tile(int tile, int m_pairs, const TileTables& tt, int E) {
    int lo = 0, hi = E;
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (tt.tile_start[mid] * m_pairs <= tile)
            lo = mid;
        else
            hi = mid;
    }
    TileInfo ti;
    ti.e = lo;
    const int ntl = tt.tile_start[lo + 1] - tt.tile_start[lo];
    const int r = tile - tt.tile_start[lo] * m_pairs;
    ti.mp = r / ntl;
    // The expert's rows are cut into ntl = ceil(cnt / BN) items of EQUAL size (rounded up
    // to the MMA's granule) instead of full items plus a remainder: every item costs a
    // full pass of weight decoding whatever its rows, so three items of 176 rows finish
    // sooner than 256 + 256 + 16 (the decode of a step hides behind a shorter MMA).
    const int cnt = tt.cnt[lo];
    int rows = BN;
    if (ntl > 1) {
        const int q = ((cnt + ntl - 1) / ntl + 31) & ~31;
        if (q < BN && (ntl - 1) * q < cnt)
            rows = q;
    }
    const int n0 = (r - ti.mp * ntl) * rows;
    ti.row0 = tt.off[lo] + n0;
    ti.valid_n = min(rows, cnt - n0);
    ti.n_mma = max(32, (ti.valid_n + 31) & ~31);
    const int nh = ti.n_mma >> 1;
    ti.box_idx = nh <= 32 ? 0 : nh <= 64 ? 1 : 2;
    return ti;
}

// m_tiles: 128-row weight tiles per expert matrix.  Launched with cluster
// dimensions (2, 1, 1); gridDim.x is even.
template <int MODE>
__global__ void __launch_bounds__(N_THREADS, 1)
expert_gemm_pair_kernel(const __grid_constant__ TensorMaps maps, const uint8_t* __restrict__ chunks,
                        size_t expert_stride, int k_stages, int m_tiles,
                        const float* __restrict__ bias, const float* __restrict__ rscale,
                        int bias_stride,
                        const int* __restrict__ g_off, const int* __restrict__ g_cnt,
                        const int* __restrict__ g_tile_start, int E, void* __restrict__ outp,
                        int out_ld, int out_rows_valid, const int* __restrict__ row_dst,
                        const __grid_constant__ peer::GemmPeerIO pio, float alpha, float limit,
                        int* __restrict__ status) {
    extern __shared__ unsigned char smem_dyn[];
    // slots need 1024-byte alignment for the 128-byte swizzle; the offsets are the
    // same in both CTAs of the pair (the tensor core applies the leader's
    // descriptors to the peer's shared memory)
    unsigned char* smem = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
    unsigned char* a_ring = smem;
    unsigned char* b_ring = a_ring + SA * A_SLOT_BYTES;
    unsigned char* w_ring = b_ring + SB * B_SLOT_BYTES;
    unsigned char* epi_stage = w_ring + WS * CHUNK_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(epi_stage + 4 * EPI_STAGE_BYTES);
    int* s_tables = reinterpret_cast<int*>(bars + N_BARRIERS);
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(s_tables + 3 * (MAX_LOCAL_EXPERTS + 1));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

    const uint32_t bar0 = smem_u32(bars);
    auto bar_w_full = [&](int s) { return bar0 + 8u * (uint32_t)s; };
    auto bar_w_empty = [&](int s) { return bar0 + 8u * (uint32_t)(WS + s); };
    auto bar_full = [&](int s) { return bar0 + 8u * (uint32_t)(2 * WS + s); };
    auto bar_empty = [&](int s) { return bar0 + 8u * (uint32_t)(2 * WS + NB + s); };
    auto bar_tmem_full = [&](int b) { return bar0 + 8u * (uint32_t)(2 * WS + 2 * NB + b); };
    auto bar_tmem_empty = [&](int b) { return bar0 + 8u * (uint32_t)(2 * WS + 2 * NB + SETS + b); };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();  // 0 = leader: issues the MMAs
    const bool leader = rank == 0;

    pdl_trigger();
    if (threadIdx.x == 0) {
        for (int s = 0; s < WS; s++) {
            mbar_init(bar_w_full(s), 1);
            mbar_init(bar_w_empty(s), 4);  // one elected arrival per warp of the decoding group
        }
        for (int s = 0; s < NB; s++) {
            // four decode warps + the TMA producer's expect_tx (+ the peer's forward on the leader)
            mbar_init(bar_full(s), leader ? 4 + 1 + 1 : 4 + 1);
            mbar_init(bar_empty(s), 1);  // tcgen05.commit (multicast)
        }
        for (int b = 0; b < SETS; b++) {
            mbar_init(bar_tmem_full(b), 1);   // tcgen05.commit (multicast)
            mbar_init(bar_tmem_empty(b), 8);  // leader only: one per epilogue warp of both CTAs
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == MMA_WARP)
        tmem_alloc2(smem_u32(tmem_holder), TMEM_COLS);
    // everything above is this CTA's own set-up; what follows reads the plan, the token
    // rows and the intermediate that earlier kernels of the call wrote
    pdl_wait();
    for (int i = threadIdx.x; i <= E; i += N_THREADS) {
        s_tables[i] = g_off[i];
        s_tables[(MAX_LOCAL_EXPERTS + 1) + i] = (i < E) ? g_cnt[i] : 0;
        s_tables[2 * (MAX_LOCAL_EXPERTS + 1) + i] = g_tile_start[i];
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // the peer's barriers exist before anyone signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_holder;
    TileTables tt;
    tt.off = s_tables;
    tt.cnt = s_tables + (MAX_LOCAL_EXPERTS + 1);
    tt.tile_start = s_tables + 2 * (MAX_LOCAL_EXPERTS + 1);

    const int m_pairs = (m_tiles + 1) / 2;
    const int total_tiles = tt.tile_start[E] * m_pairs;
    const int pair_id = (int)blockIdx.x >> 1, n_pairs = (int)gridDim.x >> 1;
    // this CTA's weight tile of item (.., mp, ..) is 2 mp + rank; the last pair of a
    // matrix with an odd tile count has no tile for the peer: it decodes the
    // leader's tile again (the MMA needs defined operands) and stores nothing
    auto my_tile = [&](int mp) { return min(2 * mp + (int)rank, m_tiles - 1); };

    if (warp == 0) {
        // ------------------------- packed-weight producer ----------------------
        if (lane == 0) {
            int s = 0, armed = 0;
            uint32_t ph = 0;
            bool ok = true;
            int wstep = 0;
            (void)wstep;
            for (int tile = pair_id; ok && tile < total_tiles; tile += n_pairs) {
                const TileInfo ti = decode_tile(tile, m_pairs, tt, E);
                const uint8_t* wsrc = chunks + (size_t)ti.e * expert_stride +
                                      (size_t)my_tile(ti.mp) * k_stages * CHUNK_BYTES;
                for (int ks = 0; ks < k_stages; ks++) {
                    ok = mbar_wait(bar_w_empty(s), ph ^ 1u, status, DS_TIMEOUT_EMPTY, abort_flag);
                    if (!ok)
                        break;
                    TRACE(wstep, 0);
                    mbar_expect_tx(bar_w_full(s), (uint32_t)CHUNK_BYTES);
                    bulk_load(smem_u32(w_ring + s * CHUNK_BYTES), wsrc + (size_t)ks * CHUNK_BYTES,
                              CHUNK_BYTES, bar_w_full(s));
                    armed = min(armed + 1, WS);
                    TRACE(wstep, 1);
                    ++wstep;
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
        // ------------------------- activation producer (this CTA's half) -------
        if (lane == 0) {
            // step i: slot i % SB, barrier i % NB; the slot is free when step i - SB is done
            int i = 0, sb = 0, nb = 0, eb = 0;
            uint32_t phe = 0;
            bool ok = true;
            if (MODE == 0 && pio.wait_flags) {
                // expert-parallel peer mode: the rows of this GEMM are stored by the other
                // GPUs; wait (bounded) until every rank has delivered, then order those
                // generic-proxy writes before this thread's TMA loads
                for (int p = 0; ok && p < pio.G; p++)
                    ok = peer::wait_flag(pio.wait_flags + p, pio.seq, status);
                __threadfence_system();
                fence_proxy_async_global();
                if (!ok)
                    *abort_flag = 1;
            }
            for (int tile = pair_id; ok && tile < total_tiles; tile += n_pairs) {
                const TileInfo ti = decode_tile(tile, m_pairs, tt, E);
                const int half_row0 = ti.row0 + (int)rank * (ti.n_mma >> 1);
                for (int ks = 0; ks < k_stages; ks++, i++) {
                    if (i >= SB) {
                        ok = mbar_wait(bar_empty(eb), phe, status, DS_TIMEOUT_EMPTY, abort_flag);
                        if (!ok)
                            break;
                        RING_ADVANCE(eb, phe, NB);
                    }
                    TRACE(i, 2);
                    mbar_expect_tx(bar_full(nb), (uint32_t)(32 << ti.box_idx) * 128u);
                    tma_load_2d(smem_u32(b_ring + sb * B_SLOT_BYTES), &maps.box[ti.box_idx],
                                bar_full(nb), ks * KSTAGE, half_row0);
                    TRACE(i, 3);
                    if (++sb == SB)
                        sb = 0;
                    if (++nb == NB)
                        nb = 0;
                }
            }
            if (!ok && i > 0) {
                // after an abort: give the copies in flight 0.1 s to land before the CTA
                // exits (their barriers also count decode arrivals that may never come,
                // so there is nothing to wait on but the clock)
                const unsigned long long t0 = global_timer_ns();
                while (global_timer_ns() - t0 < 100000000ull)
                    __nanosleep(1000);
            }
        }
    } else if (warp == MMA_WARP) {
        int sa = 0, sb = 0, nb = 0;  // step i: A slot i % SA, B slot i % SB, barriers i % NB
        uint32_t ph = 0;             // (i / NB) & 1
        bool ok = true;
        if (!leader) {
            // ------------------------- peer: forward full[i] to the leader -------
            int it = 0;
            for (int tile = pair_id; ok && tile < total_tiles; tile += n_pairs, ++it) {
                for (int ks = 0; ks < k_stages; ks++) {
                    ok = mbar_wait_hot(bar_full(nb), ph, status, DS_TIMEOUT_FULL_A, abort_flag);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok)
                        break;
                    if (elect_one_sync())
                        mbar_arrive_remote(bar_full(nb), 0);
                    RING_ADVANCE(nb, ph, NB);
                }
            }
        } else {
            // ------------------------- leader: MMA issuer --------------------------
            // The whole warp runs the loop with no lane-divergent code but the elected
            // issue; the barrier of the NEXT step is tested before the MMAs of this
            // step are issued, so that its latency overlaps the issue.
            int it = 0;
            bool ready = false;  // full[nb] already seen complete for phase ph
            for (int tile = pair_id; ok && tile < total_tiles; tile += n_pairs, ++it) {
                const TileInfo ti = decode_tile(tile, m_pairs, tt, E);
                const int set = it % SETS, round = it / SETS;
                ok = mbar_wait(bar_tmem_empty(set), (uint32_t)(round & 1) ^ 1u, status,
                               DS_TIMEOUT_TMEM_EMPTY, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok)
                    break;
                tc_fence_after();  // the epilogues' tcgen05.ld of this set came before
                const uint32_t d_tmem = tmem_base + (uint32_t)(set * BN);
                const uint32_t idesc = make_idesc2(ti.n_mma);
                for (int ks = 0; ks < k_stages; ks++) {
                    if (!ready) {
                        ok = mbar_wait_hot(bar_full(nb), ph, status, DS_TIMEOUT_FULL_A, abort_flag);
                        ok = __all_sync(0xffffffffu, ok);
                        if (!ok)
                            break;
                    }
                    if (lane == 0)
                        TRACE(it * k_stages + ks, 4);
                    int nb_next = nb;
                    uint32_t ph_next = ph;
                    RING_ADVANCE(nb_next, ph_next, NB);
                    const uint32_t peek = mbar_try_wait(bar_full(nb_next), ph_next);
                    const uint64_t a_desc = make_sw128_desc(smem_u32(a_ring + sa * A_SLOT_BYTES));
                    const uint64_t b_desc = make_sw128_desc(smem_u32(b_ring + sb * B_SLOT_BYTES));
                    if (elect_one_sync()) {
#pragma unroll
                        for (int kk = 0; kk < KSTAGE / 16; kk++)
                            umma2_bf16(d_tmem, a_desc + (uint64_t)(kk * 2), b_desc + (uint64_t)(kk * 2),
                                       idesc, (ks | kk) != 0 ? 1u : 0u);
                        umma2_commit_both(bar_empty(nb));  // frees the slots of both CTAs
                    }
                    if (lane == 0)
                        TRACE(it * k_stages + ks, 5);
                    ready = __all_sync(0xffffffffu, peek != 0);
                    nb = nb_next;
                    ph = ph_next;
                    if (++sa == SA)
                        sa = 0;
                    if (++sb == SB)
                        sb = 0;
                }
                if (ok && elect_one_sync())
                    umma2_commit_both(bar_tmem_full(set));
                __syncwarp();
            }
        }
    } else if (warp < EPI_WARP0) {
        // ------------------------------ MXFP4 decode --------------------------
        // Four groups of 4 warps; group g decodes the pipeline steps g, g + 4, ...
        // Thread r owns row r of this CTA's weight tile: packed chunk -> registers
        // (before the wait for the A slot, so that the ALU work overlaps the MMAs
        // still reading it) -> 128B-swizzled bf16 row.
        const int u = threadIdx.x - DEQ_WARP0 * 32;
        const int g = u >> 7;
        const int r = u & (TILE_M - 1);
        const uint32_t a_row_off = (uint32_t)((r >> 3) * 1024 + (r & 7) * 128);
        const int my_tiles = pair_id < total_tiles ? (total_tiles - 1 - pair_id) / n_pairs + 1 : 0;
        const int total_steps = my_tiles * k_stages;
        bool ok = true;
        for (int i = g; ok && i < total_steps; i += G) {
            // A slot i % SA is free when step i - SA is done: barrier (i - SA) % NB
            const int sw = i % WS, sa = i % SA, nb = i % NB, eb = (i - SA + NB) % NB;
            const uint32_t phw = (uint32_t)(i / WS) & 1u, phe = (uint32_t)((i - SA) / NB) & 1u;
            ok = mbar_wait(bar_w_full(sw), phw, status, DS_TIMEOUT_FULL_W, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok)
                break;
            if ((u & 127) == 0)
                TRACE(i, 6);
            const unsigned char* wst = w_ring + sw * CHUNK_BYTES;
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
            if ((u & 127) == 0)
                TRACE(i, 7);
            if (i >= SA)
                ok = mbar_wait(bar_empty(eb), phe, status, DS_TIMEOUT_EMPTY, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok)
                break;
            if ((u & 127) == 0)
                TRACE(i, 8);
            unsigned char* arow = a_ring + sa * A_SLOT_BYTES + a_row_off;
#pragma unroll
            for (int c = 0; c < 8; c++)
                *reinterpret_cast<uint4*>(arow + ((c ^ (r & 7)) * 16)) =
                    make_uint4(d[c][0], d[c][1], d[c][2], d[c][3]);
            fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor core
            __syncwarp();
            // one arrival per warp: hundreds of per-thread arrivals on one mbarrier
            // serialise in shared memory
            if (lane == 0)
                mbar_arrive(bar_full(nb));
            if ((u & 127) == 0)
                TRACE(i, 9);
        }
    } else {
        // ------------------------------ epilogue ------------------------------
        // Each CTA drains its own 128 TMEM lanes (its weight tile) of the set.
        const int q = warp & 3;         // TMEM lane quarter this warp may read
        const int row = q * 32 + lane;  // row inside the weight tile
        unsigned char* stage = epi_stage + (warp - EPI_WARP0) * EPI_STAGE_BYTES;
        bool ok = true;
        int it = 0;
        for (int tile = pair_id; ok && tile < total_tiles; tile += n_pairs, ++it) {
            const TileInfo ti = decode_tile(tile, m_pairs, tt, E);
            const int set = it % SETS, round = it / SETS;
            ok = mbar_wait(bar_tmem_full(set), (uint32_t)(round & 1), status, DS_TIMEOUT_TMEM_FULL,
                           abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok)
                break;
            if (warp == EPI_WARP0 && lane == 0)
                TRACE(it * k_stages, 10);
            tc_fence_after();
            const int mt = 2 * ti.mp + (int)rank;
            if (mt < m_tiles) {
                const float* be = bias + (size_t)ti.e * bias_stride;
                const float* rse = rscale + (size_t)ti.e * bias_stride;  // 2^shift of every weight row
                const int m = mt * TILE_M + row;
                const uint32_t t_addr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(set * BN);
                if (MODE == 0) {
                    // Lanes 2p / 2p+1 hold the gate / up row of feature pair p.  After one
                    // exchange the even lane finishes columns c0..c0+15 of that feature and
                    // the odd lane columns c0+16..c0+31; the warp's 32 token rows x 16
                    // features are transposed through shared memory so that every global
                    // store writes 16 bytes per lane.
                    uint16_t* h = static_cast<uint16_t*>(outp);
                    uint16_t* stage16 = reinterpret_cast<uint16_t*>(stage);
                    const float bm = be[m], rs = rse[m];  // 2I is a multiple of TILE_M: always in range
                    const int jf0 = (mt * TILE_M + q * 32) >> 1;  // first of this warp's 16 features
                    const bool odd = (lane & 1) != 0;
                    // token rows 16..31 sit 64 bytes further: no bank conflict between the halves
                    const int st_idx = (odd ? 16 * 16 + 32 : 0) + (lane >> 1);
                    for (int c0 = 0; c0 < ti.n_mma; c0 += 32) {
                        float v[32];
                        tmem_ld_sum<1, BN>(t_addr + (uint32_t)c0, v);
#pragma unroll
                        for (int c = 0; c < 16; c++) {
                            const float mine_lo = fmaf(v[c], rs, bm), mine_hi = fmaf(v[c + 16], rs, bm);
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
                    // A lane holds one output column m for 32 token rows; 16 token rows at
                    // a time are transposed through shared memory so that a lane stores 16
                    // bytes and a warp instruction four whole 128-byte row segments.
                    float* y = static_cast<float*>(outp);
                    float* stage32 = reinterpret_cast<float*>(stage);
                    const float bm = (m < out_rows_valid) ? be[m] : 0.f;
                    const float rs = (m < out_rows_valid) ? rse[m] : 1.f;
                    const int m4 = mt * TILE_M + q * 32 + (lane & 7) * 4;  // columns this lane stores
                    const bool m4_ok = m4 < out_rows_valid;                // the width is a multiple of 4
                    for (int c0 = 0; c0 < ti.n_mma; c0 += 32) {
                        float v[32];
                        tmem_ld_sum<1, BN>(t_addr + (uint32_t)c0, v);
#pragma unroll
                        for (int half = 0; half < 2; half++) {
#pragma unroll
                            for (int c = 0; c < 16; c++)
                                stage32[c * 32 + lane] = fmaf(v[half * 16 + c], rs, bm);
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
                                    float* yrow;
                                    if (pio.ret) {
                                        const int2 a = pio.ret[rr];
                                        yrow = pio.yrecv[a.x] + (size_t)a.y * out_ld;
                                    } else {
                                        yrow = y + (size_t)(row_dst ? row_dst[rr] : rr) * out_ld;
                                    }
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
            if (lane == 0) {
                if (leader)
                    mbar_arrive(bar_tmem_empty(set));
                else
                    mbar_arrive_remote(bar_tmem_empty(set), 0);
            }
            if (warp == EPI_WARP0 && lane == 0)
                TRACE(it * k_stages, 11);
        }
        if (MODE == 1 && pio.ticket)
            __threadfence_system();  // this thread's peer stores, before the CTA is counted below
    }

    // common exit: every role comes here, finished or aborted.  The cluster barrier
    // keeps both CTAs (their shared memory and tensor memory) alive until the other
    // one has stopped signalling.
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == MMA_WARP) {
        tc_fence_after();
        tmem_dealloc2(tmem_base, TMEM_COLS);
    }
    if (MODE == 1 && pio.ticket && threadIdx.x == 0) {
        // the last CTA to get here raises "results delivered" at every rank
        if (atomicAdd(pio.ticket, 1) == (int)gridDim.x - 1) {
            *pio.ticket = 0;
            __threadfence_system();
            for (int p = 0; p < pio.G; p++)
                *reinterpret_cast<volatile int*>(pio.done_flags[p]) = pio.seq;
        }
    }
}

}  // namespace pair
}  // namespace tc5
}  // namespace moe
