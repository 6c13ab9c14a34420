// Grouped expert GEMMs for SMALL batches (few token rows per expert), tcgen05.
//
//   MODE 0: h[rows, I]  = SwiGLU(x[rows, H] . W1_e^T + b1_e)      (bf16 out)
//           moe_mlp1_swiglu, src/hip/moe.hip:9-258
//   MODE 1: y[rows, H]  = h[rows, I] . W2_e^T + b2_e              (fp32 out)
//           moe_mlp2_store / moe_mlp2_scatter, src/hip/moe.hip:261-800
//
// Same inputs, outputs, weight layout and rounding points as gemm_tc5_pair.cuh, with
// the operand roles the other way round:
//   D[128 token rows, 256 weight rows] = X_tile . W_tile^T
// The token rows are the UMMA A operand (M = 128 TMEM lanes, fetched by TMA, a
// box of 32/64/128 rows), the decoded weights the B operand (N = 256, or 128 for
// the last tile of a matrix).  With a handful of rows per expert the call is
// bound by streaming the packed weights and by the MMA-issuing warp's serial
// chain (one barrier test, four MMAs, one commit per 64 columns of K): here every
// tcgen05.mma covers 256 weight rows instead of 128, i.e. twice the weight bytes
// per step of that chain.  The price is twice the decode work per FLOP (a decoded
// weight tile is used by 128 token rows, not 256), which is why large batches
// use gemm_tc5_pair.cuh.
//
// One persistent CTA per SM walks work items (expert, tile of 256 weight rows,
// tile of 128 token rows).  Rings in shared memory:
//   W ring   packed MXFP4 chunks (2 x 4352 B per step), deep: covers HBM latency
//   D ring   decoded bf16 weights (256 rows x 128 B, 128B swizzle)
//   X ring   activation tiles written by TMA (no multicast)
// and a ring of NB barrier pairs indexed by the step number: full[i % NB]
// collects the decode warps' arrivals and the TMA bytes of step i, empty[i % NB]
// is signalled by tcgen05.commit when the MMAs of step i are done; the producers
// wait for empty[(i - depth) % NB].
//
// Warp roles:
//   warp 0       W producer        warp 1   X producer (TMA)
//   warp 2       allocates tensor memory, issues tcgen05.mma, commits
//   next 12      decode packed MXFP4 -> bf16: three groups of four warps, group g
//                decodes steps g, g+3, ...; a thread owns one row of each of the
//                two 128-row chunks of the step
//   last 4       epilogue: tcgen05.ld, bias, SwiGLU / store.  A thread owns a
//                token row; gate/up pairs are adjacent accumulator columns
//
// Every mbarrier wait is bounded in time; a wait that runs out records a code
// in the handle's status word, raises a CTA-wide abort flag and all roles fall
// through to the common exit where tensor memory is released.
#pragma once
#include "peer_io.cuh"
#include "tc5_ptx.cuh"

namespace moe {
namespace tc5 {
namespace swp {

constexpr int BM = 128;                     // token rows per work item (UMMA M)
constexpr int BNW = 256;                    // weight rows per work item (UMMA N)
constexpr int X_SLOT_BYTES = BM * 128;      // 128 rows x 64 bf16, SW128
constexpr int D_SLOT_BYTES = BNW * 128;     // 256 rows x 64 bf16, SW128
constexpr int W_SLOT_BYTES = 2 * CHUNK_BYTES;
constexpr int MMA_WARP = 2;
constexpr int DEQ_WARP0 = 3;
constexpr int MAX_LOCAL_EXPERTS = 256;
constexpr int SETS = 2;                     // accumulator sets: the MMAs of item i+1 overlap the epilogue of item i
constexpr int TMEM_COLS = SETS * BNW;       // 512: all of tensor memory

//   G    decode groups     SD  decoded-weight slots     SX  activation slots
//   WS   packed slots      NB  barrier pairs (a multiple of SD, SX and G)
// SD and WS are multiples of G, so the successive fills of a slot are handled by
// one group in program order: an mbarrier parity wait cannot tell phase n from
// phase n-2, so a waiter must never run two phases ahead of a barrier.
constexpr int G = 3, SD = 3, SX = 3, WS = 6, NB = 3;
static_assert(SD % G == 0 && WS % G == 0 && NB % SD == 0 && NB % SX == 0 && NB % G == 0,
              "a slot's successive fills must belong to one decode group");

constexpr int EPI_WARP0 = DEQ_WARP0 + 4 * G;     // any four consecutive warps cover the four TMEM lane quarters
constexpr int N_THREADS = (EPI_WARP0 + 4) * 32;  // 608
constexpr int N_BARRIERS = 2 * WS + 2 * NB + 2 * SETS;
constexpr int SMEM_BYTES = SD * D_SLOT_BYTES + SX * X_SLOT_BYTES + WS * W_SLOT_BYTES + N_BARRIERS * 8 +
                           (MAX_LOCAL_EXPERTS + 1) * 3 * 4 + 64 + 1024;  // + tile tables + holder/flag + alignment slack
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory per CTA");

struct TileInfo {
    int e;        // local expert
    int wt;       // tile of 256 weight rows
    int n_mt;     // 128-row chunks of the weight tile that exist (1 or 2)
    int row0;     // first token row (in the expert-grouped buffer)
    int valid_m;  // token rows of this item (1..128)
    int box_idx;  // TMA box: 32 << box_idx rows
};

// The tile tables live in shared memory (copied once per CTA): every role
// decodes every work item it touches, and a binary search over global memory
// costs several L2 round trips.
struct TileTables {
    const int* off;         // [E + 1]
    const int* cnt;         // [E]
    const int* tile_start;  // [E + 1]  prefix of ceil(cnt / BM)
};

// Work items ordered [expert][weight tile][token tile]: the token tiles that
// share packed weights run on neighbouring CTAs at the same time and meet in L2.
__device__ __forceinline__ TileInfo decode_tile(int tile, int m_tiles, int w_tiles,
                                                const TileTables& tt, int E) {
    int lo = 0, hi = E;
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (tt.tile_start[mid] * w_tiles <= tile)
            lo = mid;
        else
            hi = mid;
    }
    TileInfo ti;
    ti.e = lo;
    const int ntl = tt.tile_start[lo + 1] - tt.tile_start[lo];
    const int r = tile - tt.tile_start[lo] * w_tiles;
    ti.wt = r / ntl;
    ti.n_mt = min(2, m_tiles - 2 * ti.wt);
    const int m0 = (r - ti.wt * ntl) * BM;
    ti.row0 = tt.off[lo] + m0;
    ti.valid_m = min(BM, tt.cnt[lo] - m0);
    ti.box_idx = ti.valid_m <= 32 ? 0 : ti.valid_m <= 64 ? 1 : 2;
    return ti;
}

// m_tiles: 128-row chunks per expert matrix (rows padded to 128 in the resident
// layout); out_rows_valid: features (MODE 0) or output columns (MODE 1) that exist.
template <int MODE>
__global__ void __launch_bounds__(N_THREADS, 1)
expert_gemm_swap_kernel(const __grid_constant__ TensorMaps maps, const uint8_t* __restrict__ chunks,
                       size_t expert_stride, int k_stages, int m_tiles,
                       const float* __restrict__ bias, int bias_stride,
                       const int* __restrict__ g_off, const int* __restrict__ g_cnt,
                       const int* __restrict__ g_tile_start, int E, void* __restrict__ outp,
                       int out_ld, int out_rows_valid, const int* __restrict__ row_dst,
                       const __grid_constant__ peer::GemmPeerIO pio, float alpha, float limit,
                       int* __restrict__ status) {
    extern __shared__ unsigned char smem_dyn[];
    // slots need 1024-byte alignment for the 128-byte swizzle
    unsigned char* smem = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
    unsigned char* d_ring = smem;
    unsigned char* x_ring = d_ring + SD * D_SLOT_BYTES;
    unsigned char* w_ring = x_ring + SX * X_SLOT_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(w_ring + WS * W_SLOT_BYTES);
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

    if (threadIdx.x == 0) {
        for (int s = 0; s < WS; s++) {
            mbar_init(bar_w_full(s), 1);
            mbar_init(bar_w_empty(s), 4);  // one elected arrival per warp of the decoding group
        }
        for (int s = 0; s < NB; s++) {
            mbar_init(bar_full(s), 4 + 1);  // four decode warps + the TMA producer's expect_tx
            mbar_init(bar_empty(s), 1);     // tcgen05.commit
        }
        for (int b = 0; b < SETS; b++) {
            mbar_init(bar_tmem_full(b), 1);
            mbar_init(bar_tmem_empty(b), 4);  // one per epilogue warp
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    for (int i = threadIdx.x; i <= E; i += N_THREADS) {
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

    const int w_tiles = (m_tiles + 1) / 2;
    const int total_tiles = tt.tile_start[E] * w_tiles;

    if (warp == 0) {
        // ------------------------- packed-weight producer ----------------------
        if (lane == 0) {
            int s = 0, armed = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                const TileInfo ti = decode_tile(tile, m_tiles, w_tiles, tt, E);
                const uint8_t* wsrc = chunks + (size_t)ti.e * expert_stride +
                                      (size_t)(2 * ti.wt) * k_stages * CHUNK_BYTES;
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
            // step i: slot i % SX, barrier i % NB; the slot is free when step i - SX is done
            int i = 0, sx = 0, nb = 0, eb = 0;
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
            for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
                const TileInfo ti = decode_tile(tile, m_tiles, w_tiles, tt, E);
                for (int ks = 0; ks < k_stages; ks++, i++) {
                    if (i >= SX) {
                        ok = mbar_wait(bar_empty(eb), phe, status, DS_TIMEOUT_EMPTY, abort_flag);
                        if (!ok)
                            break;
                        RING_ADVANCE(eb, phe, NB);
                    }
                    mbar_expect_tx(bar_full(nb), (uint32_t)(32 << ti.box_idx) * 128u);
                    tma_load_2d(smem_u32(x_ring + sx * X_SLOT_BYTES), &maps.box[ti.box_idx],
                                bar_full(nb), ks * KSTAGE, ti.row0);
                    if (++sx == SX)
                        sx = 0;
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
        // The whole warp runs the loop with NO lane-divergent code but the elected
        // issue itself: uniform control flow keeps the descriptors in uniform
        // registers, where tcgen05.mma reads them from, and a `lane == 0` branch costs
        // this warp more than the four MMAs of a step (measured: ~470 cycles per step
        // for one divergent barrier test).  The barrier of the NEXT step is tested
        // before the MMAs of this step are issued, so that its latency overlaps the
        // issue instead of adding to the per-step chain of this warp.  The operands in
        // shared memory need no tcgen05 fence: TMA completes through the mbarrier and
        // the decode warps fence the async proxy before they arrive.
        int sd = 0, sx = 0, nb = 0;  // step i: D slot i % SD, X slot i % SX, barriers i % NB
        uint32_t ph = 0;             // (i / NB) & 1
        bool ok = true;
        int it = 0;
        bool ready = false;  // full[nb] already seen complete for phase ph
        for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++it) {
            const TileInfo ti = decode_tile(tile, m_tiles, w_tiles, tt, E);
            const int set = it % SETS, round = it / SETS;
            ok = mbar_wait(bar_tmem_empty(set), (uint32_t)(round & 1) ^ 1u, status,
                           DS_TIMEOUT_TMEM_EMPTY, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok)
                break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + (uint32_t)(set * BNW);
            const uint32_t idesc = make_idesc(ti.n_mt * TILE_M);
            for (int ks = 0; ks < k_stages; ks++) {
                if (!ready) {
                    ok = mbar_wait(bar_full(nb), ph, status, DS_TIMEOUT_FULL_A, abort_flag);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok)
                        break;
                }
                // test the next step's barrier now, look at the answer after the issue
                int nb_next = nb;
                uint32_t ph_next = ph;
                RING_ADVANCE(nb_next, ph_next, NB);
                const uint32_t peek = mbar_try_wait(bar_full(nb_next), ph_next);
                const uint64_t a_desc = make_sw128_desc(smem_u32(x_ring + sx * X_SLOT_BYTES));
                const uint64_t b_desc = make_sw128_desc(smem_u32(d_ring + sd * D_SLOT_BYTES));
                if (elect_one_sync()) {
#pragma unroll
                    for (int kk = 0; kk < KSTAGE / 16; kk++)
                        umma_bf16(d_tmem, a_desc + (uint64_t)(kk * 2), b_desc + (uint64_t)(kk * 2),
                                  idesc, (ks | kk) != 0 ? 1u : 0u);
                    umma_commit(bar_empty(nb));  // frees both slots when these MMAs have read them
                }
                ready = __all_sync(0xffffffffu, peek != 0);
                nb = nb_next;
                ph = ph_next;
                if (++sd == SD)
                    sd = 0;
                if (++sx == SX)
                    sx = 0;
            }
            if (ok && elect_one_sync())
                umma_commit(bar_tmem_full(set));
            __syncwarp();
        }
    } else if (warp < EPI_WARP0) {
        // ------------------------------ MXFP4 decode --------------------------
        // G groups of 4 warps; group g decodes the pipeline steps g, g + G, ... so
        // that several steps are in flight at once (one step is a chain of waits,
        // loads and dependent ALU instructions).  Thread r owns row r of both
        // 128-row chunks of the step.  Chunk 0 is decoded into registers before the
        // wait for the D slot, so that the ALU work overlaps the MMAs still reading
        // the slot.
        const int u = threadIdx.x - DEQ_WARP0 * 32;
        const int g = u >> 7;
        const int r = u & (TILE_M - 1);
        const uint32_t d_row_off = (uint32_t)((r >> 3) * 1024 + (r & 7) * 128);
        const int my_tiles = (int)blockIdx.x < total_tiles
                                 ? (total_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
        const int total_steps = my_tiles * k_stages;
        bool ok = true;
        int cached_lt = -1, n_mt = 2;
        for (int i = g; ok && i < total_steps; i += G) {
            const int lt = i / k_stages;
            if (lt != cached_lt) {
                cached_lt = lt;
                n_mt = decode_tile((int)blockIdx.x + lt * (int)gridDim.x, m_tiles, w_tiles, tt, E).n_mt;
            }
            // D slot i % SD is free when step i - SD is done: barrier (i - SD) % NB
            const int sw = i % WS, sd = i % SD, nb = i % NB, eb = (i - SD + NB) % NB;
            const uint32_t phw = (uint32_t)(i / WS) & 1u, phe = (uint32_t)((i - SD) / NB) & 1u;
            ok = mbar_wait(bar_w_full(sw), phw, status, DS_TIMEOUT_FULL_W, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok)
                break;
            const unsigned char* wst = w_ring + sw * W_SLOT_BYTES;
            uint32_t d[8][4];
            {
                const uint4 q0 = *reinterpret_cast<const uint4*>(wst + r * 16);
                const uint4 q1 = *reinterpret_cast<const uint4*>(wst + PLANE_BYTES + r * 16);
                const uint32_t sc = *reinterpret_cast<const uint16_t*>(wst + 2 * PLANE_BYTES + r * 2);
                const uint32_t mult0 = mxfp4_scale_mult(sc & 0xFFu);
                const uint32_t mult1 = mxfp4_scale_mult(sc >> 8);
                const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
                for (int c = 0; c < 8; c++)
                    mxfp4_decode_word(w[c], c < 4 ? mult0 : mult1, d[c]);
            }
            // the second chunk's packed bytes wait in registers as well
            uint4 p0 = make_uint4(0, 0, 0, 0), p1 = p0;
            uint32_t sc2 = 0;
            if (n_mt > 1) {
                p0 = *reinterpret_cast<const uint4*>(wst + CHUNK_BYTES + r * 16);
                p1 = *reinterpret_cast<const uint4*>(wst + CHUNK_BYTES + PLANE_BYTES + r * 16);
                sc2 = *reinterpret_cast<const uint16_t*>(wst + CHUNK_BYTES + 2 * PLANE_BYTES + r * 2);
            }
            __syncwarp();
            if (lane == 0)
                mbar_arrive(bar_w_empty(sw));
            if (i >= SD)
                ok = mbar_wait(bar_empty(eb), phe, status, DS_TIMEOUT_EMPTY, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok)
                break;
            unsigned char* drow = d_ring + sd * D_SLOT_BYTES + d_row_off;
#pragma unroll
            for (int c = 0; c < 8; c++)
                *reinterpret_cast<uint4*>(drow + ((c ^ (r & 7)) * 16)) =
                    make_uint4(d[c][0], d[c][1], d[c][2], d[c][3]);
            if (n_mt > 1) {
                const uint32_t mult0 = mxfp4_scale_mult(sc2 & 0xFFu);
                const uint32_t mult1 = mxfp4_scale_mult(sc2 >> 8);
                const uint32_t w[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
                unsigned char* drow2 = drow + TILE_M * 128;  // rows 128..255 of the slot
#pragma unroll
                for (int c = 0; c < 8; c++) {
                    uint32_t e4[4];
                    mxfp4_decode_word(w[c], c < 4 ? mult0 : mult1, e4);
                    *reinterpret_cast<uint4*>(drow2 + ((c ^ (r & 7)) * 16)) =
                        make_uint4(e4[0], e4[1], e4[2], e4[3]);
                }
            }
            fence_proxy_async_smem();  // generic-proxy writes -> visible to the tensor core
            __syncwarp();
            // one arrival per warp: hundreds of per-thread arrivals on one mbarrier
            // serialise in shared memory
            if (lane == 0)
                mbar_arrive(bar_full(nb));
        }
    } else {
        // ------------------------------ epilogue ------------------------------
        // Thread = token row (TMEM lane), registers = 32 consecutive weight rows.
        const int q = warp & 3;         // TMEM lane quarter this warp may read
        const int row = q * 32 + lane;  // token row inside the item
        bool ok = true;
        int it = 0;
        for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++it) {
            const TileInfo ti = decode_tile(tile, m_tiles, w_tiles, tt, E);
            const int set = it % SETS, round = it / SETS;
            ok = mbar_wait(bar_tmem_full(set), (uint32_t)(round & 1), status, DS_TIMEOUT_TMEM_FULL,
                           abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok)
                break;
            tc_fence_after();
            const int n_cols = ti.n_mt * TILE_M;  // accumulator columns that were computed
            const int n0 = ti.wt * BNW;           // first weight row of the item
            const float* be = bias + (size_t)ti.e * bias_stride + n0;
            const uint32_t t_addr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(set * BNW);
            const bool row_ok = row < ti.valid_m;
            if (MODE == 0) {
                // columns 2p / 2p+1 are the gate / up row of feature n0/2 + p (the
                // checkpoint interleaves them): 32 columns -> 16 features = 32 bytes
                uint16_t* hrow = static_cast<uint16_t*>(outp) + (size_t)(ti.row0 + row) * out_ld + (n0 >> 1);
                for (int c0 = 0; c0 < n_cols; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld_32x32_issue(t_addr + (uint32_t)c0, v);
                    float b[32];
#pragma unroll
                    for (int c = 0; c < 32; c += 4) {  // 2I is a multiple of 128: always in range
                        const float4 t4 = __ldg(reinterpret_cast<const float4*>(be + c0 + c));
                        b[c] = t4.x, b[c + 1] = t4.y, b[c + 2] = t4.z, b[c + 3] = t4.w;
                    }
                    tmem_ld_wait();
                    uint32_t o[8];
#pragma unroll
                    for (int p = 0; p < 16; p += 2) {
                        const float f0 = swiglu(__uint_as_float(v[2 * p]) + b[2 * p],
                                                __uint_as_float(v[2 * p + 1]) + b[2 * p + 1], alpha, limit);
                        const float f1 = swiglu(__uint_as_float(v[2 * p + 2]) + b[2 * p + 2],
                                                __uint_as_float(v[2 * p + 3]) + b[2 * p + 3], alpha, limit);
                        o[p >> 1] = pack_bf16x2(f0, f1);
                    }
                    const int f_first = (n0 + c0) >> 1;
                    if (row_ok) {
                        if (f_first < out_rows_valid)
                            *reinterpret_cast<uint4*>(hrow + (c0 >> 1)) = make_uint4(o[0], o[1], o[2], o[3]);
                        if (f_first + 8 < out_rows_valid)
                            *reinterpret_cast<uint4*>(hrow + (c0 >> 1) + 8) = make_uint4(o[4], o[5], o[6], o[7]);
                    }
                }
            } else {
                // result row: on another GPU (peer mode), at a remapped row (received
                // order), or in place
                float* yrow = nullptr;
                if (row_ok) {
                    const int rr = ti.row0 + row;
                    if (pio.ret) {
                        const int2 a = pio.ret[rr];
                        yrow = pio.yrecv[a.x] + (size_t)a.y * out_ld;
                    } else {
                        yrow = static_cast<float*>(outp) + (size_t)(row_dst ? row_dst[rr] : rr) * out_ld;
                    }
                    yrow += n0;
                }
                for (int c0 = 0; c0 < n_cols; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld_32x32_issue(t_addr + (uint32_t)c0, v);
                    tmem_ld_wait();
                    if (row_ok) {
#pragma unroll
                        for (int c = 0; c < 32; c += 4) {
                            if (n0 + c0 + c < out_rows_valid) {  // the width is a multiple of 4
                                const float4 t4 = __ldg(reinterpret_cast<const float4*>(be + c0 + c));
                                *reinterpret_cast<float4*>(yrow + c0 + c) =
                                    make_float4(__uint_as_float(v[c]) + t4.x, __uint_as_float(v[c + 1]) + t4.y,
                                                __uint_as_float(v[c + 2]) + t4.z, __uint_as_float(v[c + 3]) + t4.w);
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(bar_tmem_empty(set));
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

}  // namespace swp
}  // namespace tc5
}  // namespace moe
