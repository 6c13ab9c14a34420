// Router GEMM + bias, top-k, softmax over the selected logits and the per-block
// expert histogram -- one kernel; and the fp32 -> bf16 cast of the block input,
// with the RMSNorm in front of the block folded in when asked.
//
// Replaces gemm_router (src/hip/gemms/gemm_router.hip:7-190), topk_kernel
// (src/hip/topk.hip:5-57), softmax_kernel (src/hip/softmax.hip:5-44), the
// histogram half of count_tokens_per_expert (src/hip/scheduler.hip:11-31) and,
// when a norm weight is given, rmsnorm (src/hip/rmsnorm.hip:3-37,
// src/forward.cpp:315; CPU: src/run.cpp:306-319).
//
// Router: one kernel family for every batch size.  A block owns RB = 16 * MT
// token rows (MT = 1, 2 or 4, picked by the host so that a small batch still
// spreads over the GPU) and all experts; warp-level tensor-core MMAs (mma.sync
// bf16, fp32 accumulate) over K chunks of 64 columns.  Token rows and router
// matrix (every block reads all of it, from L2) stream through a deep cp.async
// ring -- the kernel is a chain of H / 64 dependent chunks per block, so what
// matters is how many chunks are in flight: as many stages as shared memory holds
// (up to 12), one __syncthreads per chunk.  Input rows are bf16: fp32 input goes
// through rows_to_bf16_kernel first.
//
// Numerics.  The expert indices must equal those of the CPU engine, which sums
// float products in a double (src/run.cpp:341-354), for every token whose
// top-(K+1) logits are not within 1e-6 of each other.  Activations and router
// weights are bf16, so each product is exact in fp32; the tensor core sums one
// chunk of 64 terms into a FRESH accumulator and the chunk results are added to
// a running fp32 sum with round-to-nearest adds on the CUDA cores, so no long
// accumulation happens inside the tensor core; then the fp32 bias is added
// (src/run.cpp:635-637).  Measured at H = 2880, E = 128: |logit error| < 2e-6,
// no index mismatch.  Ties go to the lower expert index (src/hip/topk.hip:30-49).
//
// RMSNorm (optional, in rows_to_bf16_kernel) follows the CPU engine bit for bit:
// the squares are rounded to float and summed in double, 1.0f / sqrtf((float)(ss /
// H + 1e-5f)) in IEEE float arithmetic, and o = weight * (scale * x) evaluated in
// double and rounded to float once (src/run.cpp:306-319); that float is then
// rounded to bf16, the block's input precision (src/hip/BLAS.hip:32-40).  Only the
// order of the double additions differs (1e-16).
#pragma once
#include "common.cuh"

namespace moe {

constexpr int RB = 64;           // most tokens per routing block (MT = 4); sizes the permute kernels' shared arrays
constexpr int RMK = 64;          // K chunk: terms the tensor core sums before a round-to-nearest add
constexpr int RMLD = RMK + 8;    // bf16 per smem row: conflict-free fragment loads
constexpr int RTHREADS = 256;

// Stages of the cp.async ring.  16-token blocks (small batches: at most a block per SM,
// each a chain of H / 64 dependent chunks whose length in time is the number of load
// round trips) take as many as fit in ~200 KB of shared memory, at most 28.  The 32- and
// 64-token blocks of larger batches stay under half of it so that two blocks share an SM
// and 8192 or 16384 tokens (256 blocks) run as one wave.  Measured, E = 128: 8192 tokens
// 0.080 ms with 8 stages and one block per SM, 0.060 with 4 stages and two; 16384 tokens
// 0.113 ms with 3 stages and two blocks per SM, 0.172 with 7 stages and one.
// A CTA of a K-splitting cluster (CS > 1) walks only 1/CS of the chunks: 8 stages cover them.
template <int NT, int MT, int CS = 1>
__host__ __device__ constexpr int route_tc_stages() {
    constexpr int stage_bytes = (16 * MT + 32 * NT) * RMLD * 2;
    constexpr int budget = (MT >= 2 && CS == 1 ? 100 : 200) * 1024;
    constexpr int fit = budget / stage_bytes;
    constexpr int cap = CS > 1 ? 8 : (MT == 1 ? 28 : 12);
    return fit > cap ? cap : (fit < 3 ? 3 : fit);
}

// Shared memory of one block: the stages (reused for the logits after the K loop)
// plus the histogram.
template <int NT, int MT, int CS = 1>
constexpr size_t route_tc_smem_bytes() {
    size_t tiles = (size_t)route_tc_stages<NT, MT, CS>() * (16 * MT + 32 * NT) * RMLD * 2;
    size_t logits = (size_t)(16 * MT) * (32 * NT) * 4;
    return (tiles > logits ? tiles : logits) + 256 * sizeof(int);
}

// One warp: v[j] holds the logit of expert lane + 32 j (-inf past E).  Selects
// the K largest (ties to the lower index, src/hip/topk.hip:30-49), applies the
// softmax over the selected logits (src/run.cpp:641, src/hip/softmax.hip:5-44),
// stores indices and weights of token t and counts the experts in `hist`
// (shared memory, integer adds: order-independent).
template <int NT>
__device__ __forceinline__ void select_topk_softmax(float v[NT], int lane, int K, int t,
                                                    int* __restrict__ topk_i,
                                                    float* __restrict__ topk_w, int* hist) {
    float sel_v[8];
    int sel_i[8];
#pragma unroll
    for (int kk = 0; kk < 8; kk++) {
        if (kk < K) {
            float bv = v[0];
            int bi = lane;
#pragma unroll
            for (int j = 1; j < NT; j++)
                if (v[j] > bv) {
                    bv = v[j];
                    bi = lane + 32 * j;
                }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                float ov = __shfl_xor_sync(0xffffffffu, bv, off);
                int oi = __shfl_xor_sync(0xffffffffu, bi, off);
                if (ov > bv || (ov == bv && oi < bi)) {
                    bv = ov;
                    bi = oi;
                }
            }
            sel_v[kk] = bv;
            sel_i[kk] = bi;
            if ((bi & 31) == lane) {
#pragma unroll
                for (int j = 0; j < NT; j++)
                    if (j == (bi >> 5))
                        v[j] = -INFINITY;
            }
        }
    }
    float ex[8], sum = 0.f;
#pragma unroll
    for (int kk = 0; kk < 8; kk++)
        if (kk < K) {
            ex[kk] = expf(sel_v[kk] - sel_v[0]);
            sum += ex[kk];
        }
    if (lane == 0) {
#pragma unroll
        for (int kk = 0; kk < 8; kk++)
            if (kk < K) {
                topk_i[(size_t)t * K + kk] = sel_i[kk];
                topk_w[(size_t)t * K + kk] = ex[kk] / sum;
                atomicAdd(&hist[sel_i[kk]], 1);
            }
    }
}

__device__ __forceinline__ void route_mma_16816(float c[4], const uint32_t a[4], const uint32_t b[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gsrc) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// The CPU engine's rmsnorm element (src/run.cpp:317): weight * (scale * x) in
// double, rounded to float once; `scale` is the float 1/sqrtf(...) widened.
__device__ __forceinline__ float rms_apply(float x, float w, float scale) {
    return (float)((double)w * ((double)scale * (double)x));
}

// x f32 [T, H] -> out bf16 [T, H] (round to nearest even, src/hip/BLAS.hip:32-40),
// with the RMSNorm of src/run.cpp:306-319 applied first when rms_w is given
// (weight [H], f32 or bf16).  One block per row; the row stays in registers
// between the sum of squares and the scaling (H <= 8192).
constexpr int RCAST_THREADS = 256;
constexpr int RCAST_MAX_VEC = 8;  // float4 per thread: H <= 8192

__global__ void __launch_bounds__(RCAST_THREADS)
rows_to_bf16_kernel(const float* __restrict__ x, int T, int H, const void* __restrict__ rms_w,
                    int rms_w_is_f32, uint16_t* __restrict__ out) {
    __shared__ double s_part[RCAST_THREADS / 32];
    __shared__ float s_scale;
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, tid = threadIdx.x;
    if (t >= T)
        return;
    const int nvec = H / 4;
    const float4* row = reinterpret_cast<const float4*>(x + (size_t)t * H);
    float4 v[RCAST_MAX_VEC];
#pragma unroll
    for (int i = 0; i < RCAST_MAX_VEC; i++) {
        const int k = tid + i * RCAST_THREADS;
        v[i] = (k < nvec) ? row[k] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float scale = 1.f;
    if (rms_w) {
        // float products summed in double (src/run.cpp:308-311)
        double ss = 0.0;
#pragma unroll
        for (int i = 0; i < RCAST_MAX_VEC; i++) {
            ss += (double)(v[i].x * v[i].x);
            ss += (double)(v[i].y * v[i].y);
            ss += (double)(v[i].z * v[i].z);
            ss += (double)(v[i].w * v[i].w);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1)
            ss += __shfl_xor_sync(0xffffffffu, ss, off);
        if ((tid & 31) == 0)
            s_part[tid >> 5] = ss;
        __syncthreads();
        if (tid == 0) {
            double tot = 0.0;
            for (int w = 0; w < RCAST_THREADS / 32; w++)
                tot += s_part[w];
            tot /= (double)H;
            tot += (double)1e-5f;
            s_scale = __fdiv_rn(1.0f, __fsqrt_rn((float)tot));
        }
        __syncthreads();
        scale = s_scale;
    }
    uint2* orow = reinterpret_cast<uint2*>(out + (size_t)t * H);
#pragma unroll
    for (int i = 0; i < RCAST_MAX_VEC; i++) {
        const int k = tid + i * RCAST_THREADS;
        if (k < nvec) {
            float4 q = v[i];
            if (rms_w) {
                float w0, w1, w2, w3;
                if (rms_w_is_f32) {
                    const float4 wq = reinterpret_cast<const float4*>(rms_w)[k];
                    w0 = wq.x, w1 = wq.y, w2 = wq.z, w3 = wq.w;
                } else {
                    const uint2 wq = reinterpret_cast<const uint2*>(rms_w)[k];
                    w0 = __uint_as_float(wq.x << 16), w1 = __uint_as_float(wq.x & 0xFFFF0000u);
                    w2 = __uint_as_float(wq.y << 16), w3 = __uint_as_float(wq.y & 0xFFFF0000u);
                }
                q.x = rms_apply(q.x, w0, scale), q.y = rms_apply(q.y, w1, scale);
                q.z = rms_apply(q.z, w2, scale), q.w = rms_apply(q.w, w3, scale);
            }
            orow[k] = make_uint2(pack_bf16x2(q.x, q.y), pack_bf16x2(q.z, q.w));
        }
    }
}

// NT = number of 32-expert tiles (E <= 32 NT), MT = number of 16-token tiles per block.
//   x          [T, H] bf16 (XF32: f32)      score_out  optional [T, E] logits
// XF32: the token rows are fp32 and are rounded to bf16 on their way into shared
// memory, through registers one chunk ahead instead of the cp.async ring (slower:
// a chunk then costs a global-load latency).  Only the handle-free entry point,
// which has nowhere to put a bf16 copy of the rows, uses it.
// Grid: ceil(T / (16 MT)) blocks of RTHREADS threads.
//
// CS > 1 (batches that do not fill the GPU): a thread-block CLUSTER of CS CTAs shares one block of
// tokens and splits K -- CTA r of the cluster takes the chunks r, r + CS, ... -- so the
// chain of dependent chunks is CS times shorter and CS times as many SMs pull the rows.
// Each CTA leaves its partial sums in its own shared memory; after a cluster barrier
// CTA 0 adds them in rank order through distributed shared memory (a fixed order: the
// result does not depend on timing), then does bias, top-K, softmax and the histogram
// as before.  The grid is CS x the number of token blocks.
__device__ __forceinline__ uint32_t route_cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void route_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The four floats at the same shared-memory address in CTA `rank` of the cluster.  Volatile (it
// stays behind the cluster barrier, itself a volatile asm) but without a memory clobber:
// the loads of one element from all ranks are independent and overlap -- a remote
// shared-memory load takes several hundred cycles.
__device__ __forceinline__ float4 route_ld_remote(const float4* p, uint32_t rank) {
    float4 v;
    const uint32_t la = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile(
        "{\n\t.reg .b32 ra;\n\t"
        "mapa.shared::cluster.u32 ra, %4, %5;\n\t"
        "ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [ra];\n\t}"
        : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(la), "r"(rank));
    return v;
}

template <int NT, int MT, bool XF32, int CS = 1>
__global__ void __launch_bounds__(RTHREADS)
route_tc_kernel(const void* __restrict__ xv, int T, int H, const uint16_t* __restrict__ w_router,
                const float* __restrict__ b_router, int E, int K, float* __restrict__ score_out,
                int* __restrict__ topk_i, float* __restrict__ topk_w, int* __restrict__ blk_hist) {
    const uint16_t* x = static_cast<const uint16_t*>(xv);
    constexpr int RBT = 16 * MT;                 // tokens of this block
    constexpr int EP = NT * 32;                  // padded expert count
    constexpr int N_TILES = NT * 4;              // n8 tiles over the experts
    // 8 warps = MT m-tiles x NG expert groups; a warp owns NTW n8 tiles of one m-tile
    constexpr int NG = 8 / MT;
    constexpr int NTW = (N_TILES + NG - 1) / NG;
    constexpr int S = route_tc_stages<NT, MT, CS>();
    constexpr int ROWS = RBT + EP;               // rows of a stage: token rows, then router rows
    constexpr int STAGE_ELEMS = ROWS * RMLD;
    constexpr size_t tiles_b = (size_t)S * STAGE_ELEMS * 2;
    constexpr size_t lg_b = (size_t)RBT * EP * 4;
    constexpr int SEGS = (ROWS * 8 + RTHREADS - 1) / RTHREADS;  // 16-byte segments per thread and chunk
    static_assert(S >= 3, "the ring needs at least three stages");
    static_assert(CS == 1 || !XF32, "the K split takes bf16 rows");

    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint16_t* tiles = reinterpret_cast<uint16_t*>(smem_raw);
    float* lg = reinterpret_cast<float*>(smem_raw);  // [RBT][EP], reuses the tiles after the K loop
    int* hist = reinterpret_cast<int*>(smem_raw + (tiles_b > lg_b ? tiles_b : lg_b));

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t4 = lane & 3;
    const int mb = warp % MT, ng = warp / MT;  // this warp's m-tile and expert group
    const int crank = CS > 1 ? (int)route_cluster_rank() : 0;  // this CTA's share of K
    const int tblk = (int)blockIdx.x / CS;                      // its block of tokens
    const int t0 = tblk * RBT;
    pdl_trigger();
    for (int i = tid; i < 256; i += RTHREADS)
        hist[i] = 0;

    // Source row of every 16-byte segment this thread copies per chunk (fixed for the
    // whole kernel); rows past the batch / past E are never copied: zeroed once here.
    const uint16_t* seg_src[SEGS];
    int seg_dst[SEGS];
#pragma unroll
    for (int s = 0; s < SEGS; s++) {
        const int seg = tid + s * RTHREADS, row = seg >> 3, sg = seg & 7;
        seg_src[s] = nullptr;
        seg_dst[s] = row * RMLD + sg * 8;
        if (seg < ROWS * 8) {
            if (row < RBT) {
                if (!XF32 && t0 + row < T)
                    seg_src[s] = x + (size_t)(t0 + row) * H + sg * 8;
            } else if (row - RBT < E) {
                seg_src[s] = w_router + (size_t)(row - RBT) * H + sg * 8;
            }
            if (!seg_src[s] && !(XF32 && row < RBT)) {
                for (int st = 0; st < S; st++)
                    *reinterpret_cast<uint4*>(tiles + st * STAGE_ELEMS + seg_dst[s]) = make_uint4(0, 0, 0, 0);
            }
        }
    }
    // Every block walks the K chunks in its own rotation: all blocks read the same
    // router rows, and in lock step they would all ask the same L2 lines at once.
    const int n_chunks_all = H / RMK;  // H is a multiple of 64
    const int n_chunks = (n_chunks_all - crank + CS - 1) / CS;  // this CTA's: crank, crank + CS, ... (may be 0)
    const int c_rot = n_chunks > 0 ? (int)(((unsigned)tblk * 7u) % (unsigned)n_chunks) : 0;
    auto chunk_col = [&](int c) {
        int k = c + c_rot;
        if (k >= n_chunks)
            k -= n_chunks;
        return (crank + k * CS) * RMK;
    };
    auto issue = [&](int c) {  // cp.async of the c-th chunk of this block into its stage
        uint16_t* st = tiles + (c % S) * STAGE_ELEMS;
        const int col = chunk_col(c);
#pragma unroll
        for (int s = 0; s < SEGS; s++)
            if (seg_src[s])
                cp_async_16(st + seg_dst[s], seg_src[s] + col);
    };

    // XF32 only: token rows through registers
    constexpr int XSEG = (RBT * 8 + RTHREADS - 1) / RTHREADS;
    uint4 xr[XSEG];
    auto x_fetch = [&](int c) {
#pragma unroll
        for (int s = 0; s < XSEG; s++) {
            const int seg = tid + s * RTHREADS, row = seg >> 3, sg = seg & 7;
            uint4 q = make_uint4(0, 0, 0, 0);
            if (seg < RBT * 8 && t0 + row < T) {
                const float4* p = reinterpret_cast<const float4*>(
                    static_cast<const float*>(xv) + (size_t)(t0 + row) * H + chunk_col(c) + sg * 8);
                const float4 a = p[0], b = p[1];
                q = make_uint4(pack_bf16x2(a.x, a.y), pack_bf16x2(a.z, a.w), pack_bf16x2(b.x, b.y),
                               pack_bf16x2(b.z, b.w));
            }
            xr[s] = q;
        }
    };
    auto x_stash = [&](int c) {
        uint16_t* st = tiles + (c % S) * STAGE_ELEMS;
#pragma unroll
        for (int s = 0; s < XSEG; s++) {
            const int seg = tid + s * RTHREADS, row = seg >> 3, sg = seg & 7;
            if (seg < RBT * 8)
                *reinterpret_cast<uint4*>(st + row * RMLD + sg * 8) = xr[s];
        }
    };

    float run[NTW][4];
#pragma unroll
    for (int n = 0; n < NTW; n++)
#pragma unroll
        for (int i = 0; i < 4; i++)
            run[n][i] = 0.f;

    pdl_wait();  // the rows may come from the kernel before this one
#pragma unroll
    for (int c = 0; c < S - 1; c++) {
        if (c < n_chunks)
            issue(c);
        cp_async_commit();
    }
    if (XF32) {
        x_fetch(0);
        x_stash(0);
        if (n_chunks > 1)
            x_fetch(1);
    }
    for (int c = 0; c < n_chunks; c++) {
        cp_async_wait<S - 2>();  // this thread's copies of chunk c have landed
        __syncthreads();         // everybody's have, and chunk c-1 is consumed
        if (c + S - 1 < n_chunks)
            issue(c + S - 1);    // into the stage chunk c-1 just left
        cp_async_commit();
        if (XF32) {
            if (c + 1 < n_chunks)
                x_stash(c + 1);  // its stage was last read for chunk c + 1 - S
            if (c + 2 < n_chunks)
                x_fetch(c + 2);
        }
        const uint16_t* xs = tiles + (c % S) * STAGE_ELEMS;
        const uint16_t* ws = xs + RBT * RMLD;
        float acc[NTW][4];
#pragma unroll
        for (int n = 0; n < NTW; n++)
#pragma unroll
            for (int i = 0; i < 4; i++)
                acc[n][i] = 0.f;
        if (ng * NTW < N_TILES) {
#pragma unroll
            for (int kk = 0; kk < RMK / 16; kk++) {
                uint32_t af[4];
                const uint16_t* pa = xs + (mb * 16 + g) * RMLD + kk * 16 + 2 * t4;
                af[0] = *reinterpret_cast<const uint32_t*>(pa);
                af[1] = *reinterpret_cast<const uint32_t*>(pa + 8 * RMLD);
                af[2] = *reinterpret_cast<const uint32_t*>(pa + 8);
                af[3] = *reinterpret_cast<const uint32_t*>(pa + 8 * RMLD + 8);
#pragma unroll
                for (int n = 0; n < NTW; n++) {
                    const int nt = ng * NTW + n;
                    if (nt < N_TILES) {
                        const uint16_t* pb = ws + (nt * 8 + g) * RMLD + kk * 16 + 2 * t4;
                        uint32_t bf[2];
                        bf[0] = *reinterpret_cast<const uint32_t*>(pb);
                        bf[1] = *reinterpret_cast<const uint32_t*>(pb + 8);
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
    cp_async_wait<0>();
    __syncthreads();  // tiles dead; lg aliases them
#pragma unroll
    for (int n = 0; n < NTW; n++) {
        const int nt = ng * NTW + n;
        if (nt < N_TILES) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int row = mb * 16 + g + 8 * (i >> 1);
                const int e = nt * 8 + 2 * t4 + (i & 1);
                if (CS > 1)
                    lg[row * EP + e] = run[n][i];  // this CTA's share of the sum
                else
                    lg[row * EP + e] = (e < E) ? run[n][i] + b_router[e] : -INFINITY;
            }
        }
    }
    if (CS > 1) {
        route_cluster_sync();  // every CTA's partial sums are in its shared memory
        if (crank == 0) {
            constexpr int N4 = RBT * EP / 4;  // float4 elements of the logits tile
            float4* lg4 = reinterpret_cast<float4*>(lg);
            for (int i0 = tid; i0 < N4; i0 += 2 * RTHREADS) {
                // two elements per round: their remote loads are in flight together
                float4 part[2][CS];
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    const int i = i0 + j * RTHREADS;
                    if (i < N4) {
                        part[j][0] = lg4[i];
#pragma unroll
                        for (int r = 1; r < CS; r++)
                            part[j][r] = route_ld_remote(lg4 + i, (uint32_t)r);
                    }
                }
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    const int i = i0 + j * RTHREADS;
                    if (i < N4) {
                        float4 v = part[j][0];
#pragma unroll
                        for (int r = 1; r < CS; r++) {  // rank order: the sum does not depend on timing
                            v.x += part[j][r].x;
                            v.y += part[j][r].y;
                            v.z += part[j][r].z;
                            v.w += part[j][r].w;
                        }
                        const int e = (4 * i) % EP;  // EP is a multiple of 4: the four share a token row
                        v.x = (e + 0 < E) ? v.x + b_router[e + 0] : -INFINITY;
                        v.y = (e + 1 < E) ? v.y + b_router[e + 1] : -INFINITY;
                        v.z = (e + 2 < E) ? v.z + b_router[e + 2] : -INFINITY;
                        v.w = (e + 3 < E) ? v.w + b_router[e + 3] : -INFINITY;
                        lg4[i] = v;
                    }
                }
            }
        }
        route_cluster_sync();  // the other CTAs' shared memory has been read: they may leave
        if (crank != 0)
            return;
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
        blk_hist[(size_t)tblk * E + e] = hist[e];
}

}  // namespace moe
