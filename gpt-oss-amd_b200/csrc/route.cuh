// Router GEMM + bias, top-k, softmax over the selected logits, the per-block
// expert histogram and (optionally) the RMSNorm in front of the block -- one kernel.
//
// Replaces gemm_router (src/hip/gemms/gemm_router.hip:7-190), topk_kernel
// (src/hip/topk.hip:5-57), softmax_kernel (src/hip/softmax.hip:5-44), the
// histogram half of count_tokens_per_expert (src/hip/scheduler.hip:11-31) and,
// when a norm weight is given, rmsnorm (src/hip/rmsnorm.hip:3-37,
// src/forward.cpp:315; CPU: src/run.cpp:306-319).
//
// One kernel family for every batch size: a block owns RB = 16 * MT token rows
// (MT = 1, 2 or 4, picked by the host so that a small batch still spreads over
// the GPU) and all experts; warp-level tensor-core MMAs (mma.sync bf16, fp32
// accumulate) over K chunks of 64 columns.  The router matrix streams through a
// three-stage cp.async ring (every block reads all of it, from L2), the token
// rows go through registers one chunk ahead (fp32 input is rounded to bf16 there,
// and the norm is applied there): one __syncthreads per chunk, loads of chunk
// c + 2 in flight under the MMAs of chunk c.
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
// RMSNorm (optional) follows the CPU engine bit for bit: the squares are rounded
// to float and summed in double, 1.0f / sqrtf((float)(ss / H + 1e-5f)) in IEEE
// float arithmetic, and o = weight * (scale * x) evaluated in double and rounded
// to float once (src/run.cpp:306-319); that float is then rounded to bf16, the
// block's input precision (src/hip/BLAS.hip:32-40), and also written out for the
// permute kernel.  Only the order of the double additions differs (1e-16).
#pragma once
#include "common.cuh"

namespace moe {

constexpr int RB = 64;           // most tokens per routing block (MT = 4); sizes the permute kernels' shared arrays
constexpr int RMK = 64;          // K chunk: terms the tensor core sums before a round-to-nearest add
constexpr int RMLD = RMK + 8;    // bf16 per smem row: conflict-free fragment loads
constexpr int RSTAGES = 3;       // router-matrix stages in flight
constexpr int RTHREADS = 256;

// Shared memory of one block: RSTAGES x (token tile + router tile), reused for
// the logits after the K loop, plus the histogram.
template <int NT, int MT>
constexpr size_t route_tc_smem_bytes() {
    size_t tiles = (size_t)RSTAGES * (16 * MT + 32 * NT) * RMLD * 2;
    size_t logits = (size_t)(16 * MT) * (32 * NT) * 4;
    return (tiles > logits ? tiles : logits) + 256 * sizeof(int) + 16 * MT * sizeof(float);
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

// NT = number of 32-expert tiles (E <= 32 NT), MT = number of 16-token tiles per block.
//   x            [T, H] f32 or bf16 (the block input, or with `rms_w` the residual stream)
//   rms_w        optional norm weight [H] (f32 or bf16 by rms_w_is_f32); needs f32 x
//   xn_out       with rms_w: the normalised rows as bf16 [T, H] (what the block consumes)
//   score_out    optional [T, E] logits
// Grid: ceil(T / (16 MT)) blocks of RTHREADS threads.
template <int NT, int MT>
__global__ void __launch_bounds__(RTHREADS)
route_tc_kernel(const void* __restrict__ x, int x_is_f32, int T, int H,
                const uint16_t* __restrict__ w_router, const float* __restrict__ b_router, int E, int K,
                const void* __restrict__ rms_w, int rms_w_is_f32, uint16_t* __restrict__ xn_out,
                float* __restrict__ score_out, int* __restrict__ topk_i, float* __restrict__ topk_w,
                int* __restrict__ blk_hist) {
    constexpr int RBT = 16 * MT;                 // tokens of this block
    constexpr int EP = NT * 32;                  // padded expert count
    constexpr int N_TILES = NT * 4;              // n8 tiles over the experts
    // 8 warps = MT m-tiles x NG expert groups; a warp owns NTW n8 tiles of one m-tile
    constexpr int NG = 8 / MT;
    constexpr int NTW = (N_TILES + NG - 1) / NG;
    constexpr int STAGE_ELEMS = (RBT + EP) * RMLD;
    constexpr size_t tiles_b = (size_t)RSTAGES * STAGE_ELEMS * 2;
    constexpr size_t lg_b = (size_t)RBT * EP * 4;
    constexpr int XSEG = (RBT * 8 + RTHREADS - 1) / RTHREADS;  // 16-byte x segments per thread and chunk
    constexpr int WSEG = EP * 8 / RTHREADS;                    // 16-byte router segments per thread and chunk (= NT)

    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint16_t* tiles = reinterpret_cast<uint16_t*>(smem_raw);
    float* lg = reinterpret_cast<float*>(smem_raw);  // [RBT][EP], reuses the tiles after the K loop
    int* hist = reinterpret_cast<int*>(smem_raw + (tiles_b > lg_b ? tiles_b : lg_b));
    float* s_scale = reinterpret_cast<float*>(hist + 256);  // [RBT] rmsnorm scales

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t4 = lane & 3;
    const int mb = warp % MT, ng = warp / MT;  // this warp's m-tile and expert group
    const int t0 = blockIdx.x * RBT;
    for (int i = tid; i < 256; i += RTHREADS)
        hist[i] = 0;

    const bool normed = rms_w != nullptr;
    if (normed) {
        // sum of squares of each row: float products summed in double (src/run.cpp:308-311)
        for (int r = warp; r < RBT; r += RTHREADS / 32) {
            double ss = 0.0;
            if (t0 + r < T) {
                const float4* row = reinterpret_cast<const float4*>(static_cast<const float*>(x) + (size_t)(t0 + r) * H);
                for (int v = lane; v < H / 4; v += 32) {
                    const float4 q = row[v];
                    ss += (double)(q.x * q.x);
                    ss += (double)(q.y * q.y);
                    ss += (double)(q.z * q.z);
                    ss += (double)(q.w * q.w);
                }
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1)
                ss += __shfl_xor_sync(0xffffffffu, ss, off);
            if (lane == 0) {
                ss /= (double)H;
                ss += (double)1e-5f;
                s_scale[r] = __fdiv_rn(1.0f, __fsqrt_rn((float)ss));
            }
        }
        __syncthreads();
    }

    // ---- loads of one chunk
    auto w_issue = [&](int c) {  // cp.async of router chunk c into its stage
        uint16_t* ws = tiles + (c % RSTAGES) * STAGE_ELEMS + RBT * RMLD;
#pragma unroll
        for (int s = 0; s < WSEG; s++) {
            const int seg = tid + s * RTHREADS, row = seg >> 3, sg = seg & 7;
            uint16_t* dst = ws + row * RMLD + sg * 8;
            if (row < E)
                cp_async_16(dst, w_router + (size_t)row * H + c * RMK + sg * 8);
            else
                *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        }
    };
    uint4 xr[XSEG];
    auto x_fetch = [&](int c) {  // token rows of chunk c -> registers (bf16, normed if asked)
#pragma unroll
        for (int s = 0; s < XSEG; s++) {
            const int seg = tid + s * RTHREADS, row = seg >> 3, sg = seg & 7;
            uint4 q = make_uint4(0, 0, 0, 0);
            if (seg < RBT * 8 && t0 + row < T) {
                const size_t off = (size_t)(t0 + row) * H + c * RMK + sg * 8;
                if (x_is_f32) {
                    const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(x) + off);
                    float4 a = p[0], b = p[1];
                    if (normed) {
                        const float sc = s_scale[row];
                        float w[8];
                        if (rms_w_is_f32) {
                            const float4* pw = reinterpret_cast<const float4*>(static_cast<const float*>(rms_w) + c * RMK + sg * 8);
                            const float4 wa = pw[0], wb = pw[1];
                            w[0] = wa.x, w[1] = wa.y, w[2] = wa.z, w[3] = wa.w;
                            w[4] = wb.x, w[5] = wb.y, w[6] = wb.z, w[7] = wb.w;
                        } else {
                            const uint4 wq = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(rms_w) + c * RMK + sg * 8);
                            const uint32_t ww[4] = {wq.x, wq.y, wq.z, wq.w};
#pragma unroll
                            for (int i = 0; i < 4; i++) {
                                w[2 * i] = __uint_as_float(ww[i] << 16);
                                w[2 * i + 1] = __uint_as_float(ww[i] & 0xFFFF0000u);
                            }
                        }
                        a.x = rms_apply(a.x, w[0], sc), a.y = rms_apply(a.y, w[1], sc);
                        a.z = rms_apply(a.z, w[2], sc), a.w = rms_apply(a.w, w[3], sc);
                        b.x = rms_apply(b.x, w[4], sc), b.y = rms_apply(b.y, w[5], sc);
                        b.z = rms_apply(b.z, w[6], sc), b.w = rms_apply(b.w, w[7], sc);
                    }
                    q = make_uint4(pack_bf16x2(a.x, a.y), pack_bf16x2(a.z, a.w), pack_bf16x2(b.x, b.y),
                                   pack_bf16x2(b.z, b.w));
                    if (normed)
                        *reinterpret_cast<uint4*>(xn_out + off) = q;
                } else {
                    q = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(x) + off);
                }
            }
            xr[s] = q;
        }
    };
    auto x_stash = [&](int c) {
        uint16_t* xs = tiles + (c % RSTAGES) * STAGE_ELEMS;
#pragma unroll
        for (int s = 0; s < XSEG; s++) {
            const int seg = tid + s * RTHREADS, row = seg >> 3, sg = seg & 7;
            if (seg < RBT * 8)
                *reinterpret_cast<uint4*>(xs + row * RMLD + sg * 8) = xr[s];
        }
    };

    float run[NTW][4];
#pragma unroll
    for (int n = 0; n < NTW; n++)
#pragma unroll
        for (int i = 0; i < 4; i++)
            run[n][i] = 0.f;

    const int n_chunks = H / RMK;  // H is a multiple of 64
    // prologue: router chunks 0 .. RSTAGES-2 in flight, token chunk 0 in its stage, chunk 1 in registers
#pragma unroll
    for (int c = 0; c < RSTAGES - 1; c++) {
        if (c < n_chunks)
            w_issue(c);
        cp_async_commit();
    }
    x_fetch(0);
    x_stash(0);
    if (n_chunks > 1)
        x_fetch(1);
    for (int c = 0; c < n_chunks; c++) {
        cp_async_wait<RSTAGES - 2>();  // this thread's copies of router chunk c have landed
        __syncthreads();               // everybody's have, token chunk c is stored, chunk c-1 is consumed
        if (c + RSTAGES - 1 < n_chunks)
            w_issue(c + RSTAGES - 1);  // into the stage chunk c-1 just left
        cp_async_commit();
        if (c + 1 < n_chunks)
            x_stash(c + 1);            // its stage was last read for chunk c + 1 - RSTAGES
        if (c + 2 < n_chunks)
            x_fetch(c + 2);
        const uint16_t* xs = tiles + (c % RSTAGES) * STAGE_ELEMS;
        const uint16_t* ws = xs + RBT * RMLD;
        float acc[NTW][4];
#pragma unroll
        for (int n = 0; n < NTW; n++)
#pragma unroll
            for (int i = 0; i < 4; i++)
                acc[n][i] = 0.f;
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
