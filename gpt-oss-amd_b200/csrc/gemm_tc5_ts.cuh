// Grouped expert GEMMs for SMALL batches (few token rows per expert), tcgen05,
// decoded weights in TENSOR MEMORY.
//
//   MODE 0: h[rows, I]  = SwiGLU(x[rows, H] . W1_e^T + b1_e)      (bf16 out)
//           moe_mlp1_swiglu, src/hip/moe.hip:9-258
//   MODE 1: y[rows, H]  = h[rows, I] . W2_e^T + b2_e              (fp32 out)
//           moe_mlp2_store / moe_mlp2_scatter, src/hip/moe.hip:261-800
//
// Same inputs, outputs, resident weight layout and rounding points as
// gemm_tc5_pair.cuh.  A decode-shaped call (a few dozen rows per expert) streams
// every expert's packed weights once and does almost no arithmetic: it should run
// at the speed of HBM.  What stops a kernel that decodes the weights into SHARED
// memory is the shared-memory pipe, not HBM: per 64 columns of K a 128-row weight
// tile costs 16 KB of decode stores plus 16 KB of tensor-core reads there, on top
// of the packed bytes going in and out (measured on the shared-memory version of
// this kernel: LSU + tensor-core wavefronts above 70 % of the pipe at a third of
// the HBM rate).  Here the decoded tile never touches shared memory:
//
//   D[128 weight rows, N token rows] = W_tile . X_tile^T
//
// with the decoded weights as the UMMA A operand IN TENSOR MEMORY (tcgen05.mma
// "TS" form: lane = weight row, one 32-bit column = two consecutive bf16 of K,
// written by the decode warps with tcgen05.st straight from registers) and the
// token rows as the B operand in shared memory (N = 32 or 64, a TMA box).  The
// tensor work is small (the four MMAs of a 128 x 32 x 64 chunk issue in ~100
// cycles), shared memory carries only the packed bytes and the small activation tile.
//
// One persistent CTA per SM walks work items (expert, 128-row weight tile, tile
// of up to 64 token rows).  A pipeline STEP covers CS = 6 chunks of 64 K-columns
// (384 columns, 26 KB of packed weights: one bulk copy, the chunks of a weight
// tile are contiguous).  Two measurements set that size.  (1) Bulk copies of one
// chunk (4352 B) stream at 2.6 TB/s over the whole GPU however deep the ring is,
// copies of three chunks or more at 6.1 TB/s: a copy has a fixed cost.  (2) The
// MMA-issuing warp needs ~25 cycles per tcgen05.mma at N = 32 (the tensor pipe's
// own rate) but ~800 cycles per step around them -- one barrier test, one commit
// and a little bookkeeping, each a round trip through a memory pipe that sixteen
// decode warps keep busy -- and it is the only warp that can issue them.  Rings:
//   W ring   packed MXFP4 steps in shared memory (bulk copies; covers HBM latency)
//   A ring   SA = 2 slots of 192 tensor-memory columns (decoded weights)
//   B ring   activation tiles in shared memory (one 3-d TMA box per step, no
//            multicast), handed out in units of 24 KB: a step of an item with up to
//            32 token rows takes one unit, with up to 64 rows two
// and NB barrier pairs indexed by the step number: full[i % NB] collects the
// decode warps' arrivals and the TMA bytes of step i, empty[i % NB] is signalled
// by tcgen05.commit when the MMAs of step i are done.
//
// Warp roles:
//   warp 0      W producer          warp 1   B producer (TMA)
//   warp 2      allocates tensor memory, issues tcgen05.mma, commits
//   next 16     decode packed MXFP4 -> bf16 -> tensor memory: two groups of eight
//               warps, group g decodes steps g, g + 2, ...; two warps share a
//               quarter of the rows, one takes the even chunks of the step, the
//               other the odd ones, so that a slot is refilled in half the time
//   last 4      epilogue: tcgen05.ld, bias, SwiGLU / store
//
// Every mbarrier wait is bounded in time; a wait that runs out records a code in
// the handle's status word, raises a CTA-wide abort flag and all roles fall
// through to the common exit where tensor memory is released.
#pragma once
#include "peer_io.cuh"
#include "tc5_ptx.cuh"

namespace moe {
namespace tc5 {
namespace ts {

constexpr int BN = 64;                       // most token rows per work item (UMMA N)
constexpr int CS = STEP_CHUNKS;              // chunks of 64 K-columns per pipeline step
constexpr int B_UNIT_BYTES = CS * 32 * 128;  // activation tiles of one step for 32 token rows (32 rows x 64 bf16 per chunk, SW128)
constexpr int SBU = 4;                       // units in the B ring
constexpr int W_SLOT_BYTES = CS * CHUNK_BYTES;
constexpr int A_SUB_COLS = KSTAGE / 2;       // one decoded chunk in tensor memory: 128 lanes x 32 columns of bf16x2
constexpr int A_SLOT_COLS = CS * A_SUB_COLS;
constexpr int MMA_WARP = 2;
constexpr int DEQ_WARP0 = 3;
constexpr int G = 2;                         // decode groups
constexpr int GW = 8;                        // warps per decode group: two per quarter of the rows
//   SA  A slots (tensor memory)   SB  activation slots   WS  packed slots   NB  barrier pairs
// SA and WS are multiples of G, so the successive fills of a slot are handled by one
// group in program order (an mbarrier parity wait cannot tell phase n from phase n-2).
constexpr int SA = 2, NB = 4, WS = 4;
constexpr int SETS = 2;                      // accumulator sets: the MMAs of item i+1 overlap the epilogue of item i
constexpr int TMEM_A0 = SETS * BN;           // first tensor-memory column of the A slots
constexpr int TMEM_COLS = 512;
static_assert(TMEM_A0 + SA * A_SLOT_COLS <= TMEM_COLS, "tensor memory");
static_assert(SA % G == 0 && WS % G == 0 && NB % SA == 0 && NB % G == 0 && NB >= SBU,
              "a slot's successive fills must belong to one decode group");
constexpr int EPI_WARP0 = DEQ_WARP0 + GW * G;
constexpr int N_THREADS = (EPI_WARP0 + 4) * 32;  // 736
constexpr int MAX_LOCAL_EXPERTS = 256;
constexpr int EPI_STAGE_BYTES = 2048;
constexpr int N_BARRIERS = 2 * WS + 2 * NB + 2 * SETS;
constexpr int SMEM_BYTES = SBU * B_UNIT_BYTES + WS * W_SLOT_BYTES + 4 * EPI_STAGE_BYTES + N_BARRIERS * 8 +
                           (MAX_LOCAL_EXPERTS + 1) * 3 * 4 + 64 + 1024;
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory per CTA");

// D[tmem] (+)= A[tmem] . B[smem desc]^T: A is 128 lanes x 8 columns (16 bf16 of K per lane).
// The shared-memory descriptor comes as its two 32-bit halves: stepping through a tile
// only changes the start-address field in the low half, one 32-bit add per MMA in the
// issuing warp's chain instead of a 64-bit one.
__device__ __forceinline__ void umma_ts_bf16(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_desc_lo,
                                             uint32_t b_desc_hi, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 bd;\n\t"
        "mov.b64 bd, {%2, %3};\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], bd, %4, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_desc_lo), "r"(b_desc_hi), "r"(idesc), "r"(accumulate) : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp writes lane (taddr.lane + i).
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t a[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(a[4]), "r"(a[5]), "r"(a[6]), "r"(a[7]),
          "r"(a[8]), "r"(a[9]), "r"(a[10]), "r"(a[11]), "r"(a[12]), "r"(a[13]), "r"(a[14]), "r"(a[15]),
          "r"(a[16]), "r"(a[17]), "r"(a[18]), "r"(a[19]), "r"(a[20]), "r"(a[21]), "r"(a[22]), "r"(a[23]),
          "r"(a[24]), "r"(a[25]), "r"(a[26]), "r"(a[27]), "r"(a[28]), "r"(a[29]), "r"(a[30]), "r"(a[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

struct TileInfo {
    int e;        // local expert
    int mt;       // 128-row weight tile
    int row0;     // first token row of the item
    int valid_n;  // token rows of the item (1..64)
    int n_mma;    // rows the MMA computes (a multiple of 32)
    int box_idx;  // TMA box: 32 << box_idx rows
};

struct TileTables {
    const int* off;         // [E + 1]
    const int* cnt;         // [E]
    const int* tile_start;  // [E + 1]  prefix of ceil(cnt / BN)
};

// Items ordered [expert][weight tile][token tile]: the token tiles that share
// packed weights run on neighbouring CTAs at the same time and meet in L2.
__device__ __forceinline__ TileInfo decode_tile(int tile, int m_tiles, const TileTables& tt, int E) {
    int lo = 0, hi = E;
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (tt.tile_start[mid] * m_tiles <= tile)
            lo = mid;
        else
            hi = mid;
    }
    TileInfo ti;
    ti.e = lo;
    const int ntl = tt.tile_start[lo + 1] - tt.tile_start[lo];
    const int r = tile - tt.tile_start[lo] * m_tiles;
    ti.mt = r / ntl;
    const int n0 = (r - ti.mt * ntl) * BN;
    ti.row0 = tt.off[lo] + n0;
    ti.valid_n = min(BN, tt.cnt[lo] - n0);
    ti.n_mma = max(32, (ti.valid_n + 31) & ~31);
    ti.box_idx = ti.n_mma <= 32 ? 0 : 1;
    return ti;
}

// m_tiles: 128-row weight tiles per expert matrix (rows padded to 128 in the resident
// layout); out_rows_valid: features (MODE 0) or output columns (MODE 1) that exist.
template <int MODE>
__global__ void __launch_bounds__(N_THREADS, 1)
expert_gemm_ts_kernel(const __grid_constant__ TensorMaps maps, const uint8_t* __restrict__ chunks,
                      size_t expert_stride, int k_stages, int m_tiles,
                      const float* __restrict__ bias, const float* __restrict__ rscale,
                        int bias_stride,
                      const int* __restrict__ g_off, const int* __restrict__ g_cnt,
                      const int* __restrict__ g_tile_start, int E, void* __restrict__ outp,
                      int out_ld, int out_rows_valid, const int* __restrict__ row_dst,
                      const __grid_constant__ peer::GemmPeerIO pio, float alpha, float limit,
                      int* __restrict__ status) {
    extern __shared__ unsigned char smem_dyn[];
    // slots need 1024-byte alignment for the 128-byte swizzle
    unsigned char* smem = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
    unsigned char* b_ring = smem;
    unsigned char* w_ring = b_ring + SBU * B_UNIT_BYTES;
    unsigned char* epi_stage = w_ring + WS * W_SLOT_BYTES;
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

    pdl_trigger();
    if (threadIdx.x == 0) {
        for (int s = 0; s < WS; s++) {
            mbar_init(bar_w_full(s), 1);
            mbar_init(bar_w_empty(s), GW);  // one elected arrival per warp of the decoding group
        }
        for (int s = 0; s < NB; s++) {
            mbar_init(bar_full(s), GW + 1);  // the decode warps of a group + the TMA producer's expect_tx
            mbar_init(bar_empty(s), 1);     // tcgen05.commit
        }
        for (int b = 0; b < SETS; b++) {
            mbar_init(bar_tmem_full(b), 1);
            mbar_init(bar_tmem_empty(b), 4);  // one per epilogue warp
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == MMA_WARP)
        tmem_alloc(smem_u32(tmem_holder), TMEM_COLS);
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
    tc_fence_after();
    const uint32_t tmem_base = *tmem_holder;
    TileTables tt;
    tt.off = s_tables;
    tt.cnt = s_tables + (MAX_LOCAL_EXPERTS + 1);
    tt.tile_start = s_tables + 2 * (MAX_LOCAL_EXPERTS + 1);

    const int total_tiles = tt.tile_start[E] * m_tiles;
    const int n_steps = (k_stages + CS - 1) / CS;  // pipeline steps per work item; the last may hold fewer chunks

    if (warp == 0) {
        // ------------------------- packed-weight producer ----------------------
        if (lane == 0) {
            int s = 0, armed = 0;
            uint32_t ph = 0;
            bool ok = true;
            int wstep = 0;
            (void)wstep;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                const TileInfo ti = decode_tile(tile, m_tiles, tt, E);
                const uint8_t* wsrc = chunks + (size_t)ti.e * expert_stride +
                                      (size_t)ti.mt * k_stages * CHUNK_BYTES;
                for (int st = 0; st < n_steps; st++) {
                    ok = mbar_wait(bar_w_empty(s), ph ^ 1u, status, DS_TIMEOUT_EMPTY, abort_flag);
                    if (!ok)
                        break;
                    TRACE(wstep, 0);
                    // the chunks of a weight tile are contiguous: one copy per step
                    const uint32_t bytes = (uint32_t)(min(CS, k_stages - st * CS) * CHUNK_BYTES);
                    mbar_expect_tx(bar_w_full(s), bytes);
                    bulk_load(smem_u32(w_ring + s * W_SLOT_BYTES), wsrc + (size_t)st * W_SLOT_BYTES, bytes,
                              bar_w_full(s));
                    TRACE(wstep, 1);
                    ++wstep;
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
            // step i: barrier i % NB; its tiles take one or two units of the B ring (one copy:
            // a 3-d box of CS chunks).  Before a step is issued, step i - Q must be done, where Q
            // is how many steps the ring is sure to hold: SBU while the last SBU steps all took
            // one unit, SBU / 2 otherwise.  Steps finish in order, so the producer consumes the
            // empty barriers in step order.
            int i = 0, nb = 0, bu = 0, waited = 0, ones_run = 0;
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
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                const TileInfo ti = decode_tile(tile, m_tiles, tt, E);
                const int need = ti.n_mma >> 5;  // units per step: 1 or 2
                for (int st = 0; st < n_steps; st++, i++) {
                    if (need == 2 && (bu & 1))
                        bu = (bu + 1) & (SBU - 1);
                    ones_run = (need == 1) ? ones_run + 1 : 0;
                    const int last = i - (ones_run > SBU ? SBU : SBU / 2);
                    while (ok && waited <= last) {
                        ok = mbar_wait(bar_empty(waited % NB), (uint32_t)(waited / NB) & 1u, status,
                                       DS_TIMEOUT_EMPTY, abort_flag);
                        waited++;
                    }
                    if (!ok)
                        break;
                    TRACE(i, 2);
                    // the whole box is delivered (chunks past the end of K arrive as zeros)
                    mbar_expect_tx(bar_full(nb), (uint32_t)(CS * ti.n_mma) * 128u);
                    tma_load_3d(smem_u32(b_ring + bu * B_UNIT_BYTES), &maps.box3[ti.box_idx], bar_full(nb), 0,
                                ti.row0, st * CS);
                    TRACE(i, 3);
                    bu = (bu + need) & (SBU - 1);
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
        // ------------------------------ MMA issuer ----------------------------
        // The whole warp runs the loop with no lane-divergent code but the elected issue.
        // This warp's chain per step (one barrier test, the MMAs, one commit, a little
        // bookkeeping) is what paces the kernel once the rings are deep enough -- the
        // operands of a step are ready thousands of cycles before it gets to them -- so
        // it carries nothing else: one plain wait per step, no look-ahead test.
        int sa = 0, bu = 0, nb = 0;  // step i: A slot i % SA, barriers i % NB, B units as the producer hands them out
        uint32_t ph = 0;             // (i / NB) & 1
        bool ok = true;
        int it = 0;
        for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++it) {
            const TileInfo ti = decode_tile(tile, m_tiles, tt, E);
            const int set = it % SETS, round = it / SETS;
            ok = mbar_wait(bar_tmem_empty(set), (uint32_t)(round & 1) ^ 1u, status,
                           DS_TIMEOUT_TMEM_EMPTY, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok)
                break;
            tc_fence_after();  // the epilogue's tcgen05.ld of this set came before
            if (lane == 0)
                TRACE(it * n_steps, 12);
            const uint32_t d_tmem = tmem_base + (uint32_t)(set * BN);
            const uint32_t idesc = make_idesc(ti.n_mma);
            const int need = ti.n_mma >> 5;                    // B units per step
            const uint32_t sub_step = (uint32_t)ti.n_mma * 8u;  // one chunk's tile in descriptor units of 16 bytes
            for (int st = 0; st < n_steps; st++) {
                ok = mbar_wait_hot(bar_full(nb), ph, status, DS_TIMEOUT_FULL_A, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok)
                    break;
                if (lane == 0)
                    TRACE(it * n_steps + st, 4);
                tc_fence_after();  // the decode warps' tcgen05.st of this step came before
                const uint32_t a_tmem = tmem_base + (uint32_t)(TMEM_A0 + sa * A_SLOT_COLS);
                if (need == 2 && (bu & 1))
                    bu = (bu + 1) & (SBU - 1);
                const uint64_t b_desc = make_sw128_desc(smem_u32(b_ring + bu * B_UNIT_BYTES));
                const uint32_t b_lo = (uint32_t)b_desc, b_hi = (uint32_t)(b_desc >> 32);
                const int nch = min(CS, k_stages - st * CS);
                if (elect_one_sync()) {
                    TRACE(it * n_steps + st, 13);
#pragma unroll
                    for (int j = 0; j < CS; j++) {
                        if (j < nch) {
#pragma unroll
                            for (int kk = 0; kk < KSTAGE / 16; kk++)
                                umma_ts_bf16(d_tmem, a_tmem + (uint32_t)(j * A_SUB_COLS + kk * 8),
                                             b_lo + (uint32_t)j * sub_step + (uint32_t)(kk * 2), b_hi, idesc,
                                             (st | j | kk) != 0 ? 1u : 0u);
                        }
                    }
                    TRACE(it * n_steps + st, 14);
                    umma_commit(bar_empty(nb));  // frees both slots when these MMAs have read them
                }
                if (lane == 0)
                    TRACE(it * n_steps + st, 5);
                RING_ADVANCE(nb, ph, NB);
                if (++sa == SA)
                    sa = 0;
                bu = (bu + need) & (SBU - 1);
            }
            if (ok && elect_one_sync())
                umma_commit(bar_tmem_full(set));
            __syncwarp();
        }
    } else if (warp < EPI_WARP0) {
        // ------------------------------ MXFP4 decode --------------------------
        // Group g decodes the pipeline steps g, g + G, ...  A warp may write the
        // tensor-memory lanes 32 * (warp id % 4) .. + 31: those are its weight rows.
        // Packed chunk -> registers (before the wait for the A slot, so that the ALU
        // work overlaps the MMAs still reading it) -> tcgen05.st.
        const int u = threadIdx.x - DEQ_WARP0 * 32;
        const int g = u / (GW * 32);
        const int half = ((u >> 5) % GW) >> 2;  // 0: this warp takes chunks 0, 2, 4 of a step; 1: chunks 1, 3, 5
        const int r = (warp & 3) * 32 + lane;
        const uint32_t a_lane = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)TMEM_A0;
        const int my_tiles = (int)blockIdx.x < total_tiles
                                 ? (total_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
        const int total_steps = my_tiles * n_steps;
        bool ok = true;
        for (int i = g; ok && i < total_steps; i += G) {
            // A slot i % SA is free when step i - SA is done: barrier (i - SA) % NB
            const int sw = i % WS, sa = i % SA, nb = i % NB, eb = (i - SA + NB) % NB;
            const uint32_t phw = (uint32_t)(i / WS) & 1u, phe = (uint32_t)((i - SA) / NB) & 1u;
            const int st = i % n_steps;  // step inside its work item
            const int nch = min(CS, k_stages - st * CS);
            ok = mbar_wait(bar_w_full(sw), phw, status, DS_TIMEOUT_FULL_W, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok)
                break;
            if ((u & (GW * 32 - 1)) == 0)
                TRACE(i, 6);
            const unsigned char* wst = w_ring + sw * W_SLOT_BYTES;
            const uint32_t a_slot = a_lane + (uint32_t)(sa * A_SLOT_COLS);
            bool slot_free = false;
            for (int j = half; j < nch; j += 2) {
                const unsigned char* wc = wst + j * CHUNK_BYTES;
                const uint4 q0 = *reinterpret_cast<const uint4*>(wc + r * 16);
                const uint4 q1 = *reinterpret_cast<const uint4*>(wc + PLANE_BYTES + r * 16);
                const uint32_t sc = *reinterpret_cast<const uint16_t*>(wc + 2 * PLANE_BYTES + r * 2);
                if (j + 2 >= nch) {
                    // this warp's last packed bytes of the step are in registers
                    __syncwarp();
                    if (lane == 0)
                        mbar_arrive(bar_w_empty(sw));
                }
                const uint32_t mult0 = mxfp4_scale_mult(sc & 0xFFu);
                const uint32_t mult1 = mxfp4_scale_mult(sc >> 8);
                const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
                uint32_t d[8][4];  // d[c][p] = bf16x2 of columns 8c + 2p, 8c + 2p + 1: tensor-memory column 4c + p
#pragma unroll
                for (int c = 0; c < 8; c++)
                    mxfp4_decode_word(w[c], c < 4 ? mult0 : mult1, d[c]);
                if (!slot_free) {
                    // the first chunk is decoded before the wait for the A slot, so that the
                    // ALU work overlaps the MMAs still reading it
                    if ((u & (GW * 32 - 1)) == 0)
                        TRACE(i, 7);
                    if (i >= SA)
                        ok = mbar_wait(bar_empty(eb), phe, status, DS_TIMEOUT_EMPTY, abort_flag);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok)
                        break;
                    if ((u & (GW * 32 - 1)) == 0)
                        TRACE(i, 8);
                    tc_fence_after();  // the MMAs that read this slot are done (commit -> empty)
                    slot_free = true;
                }
                tmem_st_32x32(a_slot + (uint32_t)(j * A_SUB_COLS), &d[0][0]);
            }
            if (!ok)
                break;
            if (half >= nch) {
                // a step with a single chunk leaves the odd-chunk warps without work: they
                // still release the packed slot and still wait for step i - SA, so that no
                // warp ever arrives twice within one phase of a barrier
                __syncwarp();
                if (lane == 0)
                    mbar_arrive(bar_w_empty(sw));
                if (i >= SA)
                    ok = mbar_wait(bar_empty(eb), phe, status, DS_TIMEOUT_EMPTY, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok)
                    break;
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(bar_full(nb));
            if ((u & (GW * 32 - 1)) == 0)
                TRACE(i, 9);
        }
    } else {
        // ------------------------------ epilogue ------------------------------
        // A lane holds one weight row (TMEM lane) for 32 token rows at a time.
        const int q = warp & 3;         // TMEM lane quarter this warp may read
        const int row = q * 32 + lane;  // row inside the weight tile
        unsigned char* stage = epi_stage + (warp - EPI_WARP0) * EPI_STAGE_BYTES;
        bool ok = true;
        int it = 0;
        for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++it) {
            const TileInfo ti = decode_tile(tile, m_tiles, tt, E);
            const int set = it % SETS, round = it / SETS;
            ok = mbar_wait(bar_tmem_full(set), (uint32_t)(round & 1), status, DS_TIMEOUT_TMEM_FULL,
                           abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok)
                break;
            if (warp == EPI_WARP0 && lane == 0)
                TRACE(it * n_steps, 10);
            tc_fence_after();
            const int mt = ti.mt;
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
                        stage16[st_idx + c * 16] = (uint16_t)float_to_bf16_bits(swiglu(gate, up, alpha, limit));
                    }
                    __syncwarp();
#pragma unroll
                    for (int p = 0; p < 2; p++) {
                        const int tok = (lane >> 1) + 16 * p, hf = lane & 1;
                        const uint4 val = *reinterpret_cast<const uint4*>(stage + tok * 32 + hf * 16 + p * 64);
                        const int col = c0 + tok, jf = jf0 + hf * 8;
                        if (col < ti.valid_n && jf < out_rows_valid)
                            *reinterpret_cast<uint4*>(h + (size_t)(ti.row0 + col) * out_ld + jf) = val;
                    }
                    __syncwarp();
                }
            } else {
                // A lane holds one output column m for 32 token rows; 16 token rows at a
                // time are transposed through shared memory so that a lane stores 16
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
                            const float4 val = *reinterpret_cast<const float4*>(stage + (lane + 32 * p) * 16);
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
            tc_fence_before();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(bar_tmem_empty(set));
            if (warp == EPI_WARP0 && lane == 0)
                TRACE(it * n_steps, 11);
        }
        if (MODE == 1 && pio.ticket)
            __threadfence_system();  // this thread's peer stores, before the CTA is counted below
    }

    // common exit: every role comes here, finished or aborted
    tc_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
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

}  // namespace ts
}  // namespace tc5
}  // namespace moe
