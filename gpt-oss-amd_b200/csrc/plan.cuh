// Token -> expert permutation, tile tables for the grouped GEMMs, and the
// routing-weighted combine.
//
// Replaces count_tokens_per_expert / exclusive_scan_expert_offsets /
// compact_by_expert_kernel / gather_rows* / classify_and_build_queues
// (src/hip/scheduler.hip:11-184), the host-side grid sizing of
// src/forward.cpp:383-460, and the atomicAdd combine + vecadd_and_zero
// (src/hip/moe.hip:464-509, src/hip/vecadd.hip:19-38).
//
// Differences by design: the order of rows inside an expert is the token order
// (deterministic; the reference's atomic compaction is not), no value is read
// back by the host, and the combine adds a token's K contributions in
// ascending expert order -- the order the CPU engine uses (src/run.cpp:645-705).
#pragma once
#include "common.cuh"
#include "route.cuh"

namespace moe {

// One block of 256 threads.  blk_hist [nblk, E] -> cnt[E], off[E+1] (rows sorted by
// expert), blk_base[nblk, E] (first row of block b's assignments to expert e), and the
// GEMM tile table tile_start[E+1] = prefix of ceil(cnt/bn).  s_cnt[256] (shared)
// holds the counts for every thread when the function returns.
// A thread walks one expert's column of the histogram (coalesced across the threads
// of a warp); with fewer than 129 experts the 256 threads split the routing blocks
// into 256 / E parts, which shortens the chain of dependent steps accordingly.
__device__ __forceinline__ void plan_body(const int* __restrict__ blk_hist, int nblk, int E, int bn,
                                          int* __restrict__ cnt, int* __restrict__ off,
                                          int* __restrict__ tile_start, int* __restrict__ blk_base,
                                          int* s_cnt) {
    __shared__ int s_off[257];
    __shared__ int s_part[256];
    const int P = max(1, 256 / E);  // parts of the block range
    const int part = (int)threadIdx.x / E, e = (int)threadIdx.x - part * E;
    const bool active = part < P;
    const int b_lo = active ? (int)((long long)nblk * part / P) : 0;
    const int b_hi = active ? (int)((long long)nblk * (part + 1) / P) : 0;
    int sum = 0;
    for (int b = b_lo; b < b_hi; b++)
        sum += blk_hist[(size_t)b * E + e];
    if (active)
        s_part[threadIdx.x] = sum;
    __syncthreads();
    if ((int)threadIdx.x < E) {
        int total = 0;
        for (int p = 0; p < P; p++)
            total += s_part[p * E + threadIdx.x];
        s_cnt[threadIdx.x] = total;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int o = 0, t = 0;
        for (int i = 0; i < E; i++) {
            s_off[i] = o;
            off[i] = o;
            tile_start[i] = t;
            cnt[i] = s_cnt[i];
            o += s_cnt[i];
            t += (s_cnt[i] + bn - 1) / bn;
        }
        s_off[E] = o;
        off[E] = o;
        tile_start[E] = t;
    }
    __syncthreads();
    if (active) {
        int run = s_off[e];
        for (int p = 0; p < part; p++)
            run += s_part[p * E + e];
        for (int b = b_lo; b < b_hi; b++) {
            blk_base[(size_t)b * E + e] = run;
            run += blk_hist[(size_t)b * E + e];
        }
    }
    __syncthreads();
}

__global__ void __launch_bounds__(256)
plan_kernel(const int* __restrict__ blk_hist, int nblk, int E, int bn, int* __restrict__ cnt,
            int* __restrict__ off, int* __restrict__ tile_start, int* __restrict__ blk_base) {
    __shared__ int s_cnt[256];
    pdl_trigger();
    pdl_wait();
    plan_body(blk_hist, nblk, E, bn, cnt, off, tile_start, blk_base, s_cnt);
}

// Most routing blocks for which the permute kernel plans by itself (below).
constexpr int PLAN_FUSED_MAX_BLOCKS = 32;

// Stable placement of every (token, k) assignment into its expert's row range
// and the row gather x[token] -> xs[row] as bf16 (fp32 input is rounded here:
// src/hip/BLAS.hip:32-40).  grid = (routing blocks of RB tokens, S): the S
// blocks of a routing block split its assignments, so that a batch of a few
// thousand tokens still puts several blocks on every SM (the copy is bound by
// loads in flight, not by the arithmetic).
// Small batches (blk_hist != nullptr, at most PLAN_FUSED_MAX_BLOCKS routing blocks):
// no plan kernel runs before this one; every block sums the per-block histograms
// itself (a few KB from L2) to find the first row of its own routing block for every
// expert, and block (0, 0) writes cnt / off / tile_start for the GEMMs.  One launch
// and one dependent kernel start less on the latency-bound decode path.
__global__ void __launch_bounds__(256)
permute_kernel(const void* __restrict__ x, int x_is_f32, int T, int H, int K, int E, int rb,
               const int* __restrict__ topk_i, const int* __restrict__ blk_base,
               int* __restrict__ slot_of, int* __restrict__ row_token,
               uint16_t* __restrict__ xs_out, int* __restrict__ status,
               const int* __restrict__ blk_hist, int nblk, int bn, int* __restrict__ cnt,
               int* __restrict__ off, int* __restrict__ tile_start) {
    __shared__ int s_base[256];
    pdl_trigger();
    pdl_wait();
    if (blk_hist) {
        __shared__ int s_tot[256];
        const int e = threadIdx.x;
        int before = 0;
        if (e < E) {
            int total = 0;
            for (int b = 0; b < nblk; b++) {
                const int v = blk_hist[(size_t)b * E + e];
                before += (b < (int)blockIdx.x) ? v : 0;
                total += v;
            }
            s_tot[e] = total;
        }
        __syncthreads();
        if (threadIdx.x < 32) {
            // exclusive prefix over the experts (and over their tile counts), one warp
            const bool writer = blockIdx.x == 0 && blockIdx.y == 0;
            int carry_o = 0, carry_t = 0;
            for (int e0 = 0; e0 < E; e0 += 32) {
                const int i = e0 + (int)threadIdx.x;
                const int c = i < E ? s_tot[i] : 0;
                const int nt = (c + bn - 1) / bn;
                int so = c, stl = nt;
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
                    const int uo = __shfl_up_sync(0xffffffffu, so, d), ut = __shfl_up_sync(0xffffffffu, stl, d);
                    if ((int)threadIdx.x >= d) {
                        so += uo;
                        stl += ut;
                    }
                }
                if (i < E) {
                    s_base[i] = carry_o + so - c;
                    if (writer) {
                        cnt[i] = c;
                        off[i] = carry_o + so - c;
                        tile_start[i] = carry_t + stl - nt;
                    }
                }
                carry_o += __shfl_sync(0xffffffffu, so, 31);
                carry_t += __shfl_sync(0xffffffffu, stl, 31);
            }
            if (writer && threadIdx.x == 0) {
                off[E] = carry_o;
                tile_start[E] = carry_t;
            }
        }
        __syncthreads();
        if (e < E)
            s_base[e] += before;
        __syncthreads();
    }
    __shared__ int s_e[RB * 8];
    __shared__ int s_pos[RB * 8];
    const int t0 = blockIdx.x * rb;  // rb <= RB tokens per block, the routing kernel's block size
    const int n_assign = rb * K;
    for (int a = threadIdx.x; a < n_assign; a += blockDim.x) {
        const int t = t0 + a / K;
        int e = -1;
        if (t < T) {
            e = topk_i[(size_t)t0 * K + a];
            if (e < 0 || e >= E) {
                report_status(status, DS_BAD_EXPERT);
                e = -1;
            }
        }
        s_e[a] = e;
    }
    __syncthreads();
    // the gridDim.y blocks of a routing block split its TOKENS (all K assignments of a
    // token stay together: its row is read once and stored K times)
    const int tok_per = (rb + gridDim.y - 1) / gridDim.y;
    const int tl_lo = blockIdx.y * tok_per, tl_hi = min(rb, tl_lo + tok_per);
    const int a_lo = tl_lo * K, a_hi = tl_hi * K;
    for (int a = a_lo + threadIdx.x; a < a_hi; a += blockDim.x) {
        const int e = s_e[a];
        int pos = -1;
        if (e >= 0) {
            int rank = 0;
            for (int j = 0; j < a; j++)
                rank += (s_e[j] == e);
            pos = (blk_hist ? s_base[e] : blk_base[(size_t)blockIdx.x * E + e]) + rank;
            slot_of[(size_t)t0 * K + a] = pos;
            row_token[pos] = t0 + a / K;
        }
        s_pos[a] = pos;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int vec_per_row = H / 8;  // 8 bf16 = 16 bytes
    // a warp takes a quarter of a token's row at a time: a block that holds only a few
    // tokens still keeps all its warps busy
    constexpr int NSEG = 4;
    const int seg_len = (vec_per_row + NSEG - 1) / NSEG;
    for (int item = tl_lo * NSEG + warp; item < tl_hi * NSEG; item += nwarps) {
        const int tl = item / NSEG, seg = item - tl * NSEG;
        const int t = t0 + tl;
        if (t >= T)
            break;
        const int v_lo = seg * seg_len, v_hi = min(vec_per_row, v_lo + seg_len);
        uint4* dst[8];
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const int pos = k < K ? s_pos[tl * K + k] : -1;
            dst[k] = pos >= 0 ? reinterpret_cast<uint4*>(xs_out + (size_t)pos * H) : nullptr;
        }
        if (x_is_f32) {
            const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(x) + (size_t)t * H);
            for (int v = v_lo + lane; v < v_hi; v += 32) {
                const float4 p = src[2 * v], q = src[2 * v + 1];
                const uint4 r = make_uint4(pack_bf16x2(p.x, p.y), pack_bf16x2(p.z, p.w),
                                           pack_bf16x2(q.x, q.y), pack_bf16x2(q.z, q.w));
#pragma unroll
                for (int k = 0; k < 8; k++)
                    if (dst[k])
                        dst[k][v] = r;
            }
        } else {
            const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(x) + (size_t)t * H);
            for (int v = v_lo + lane; v < v_hi; v += 32) {
                const uint4 r = src[v];
#pragma unroll
                for (int k = 0; k < 8; k++)
                    if (dst[k])
                        dst[k][v] = r;
            }
        }
    }
}

// out[t,:] (+)= sum over the token's K assignments, ascending expert index, of
// topk_w * y[slot,:].  One block per token.
// Expert-parallel peer mode: `wait_flags` points at this rank's G "results
// delivered" flags; the block first waits (bounded) until every rank has stored
// its result rows into y.  The grid then has at least one block even for T == 0:
// the wait is also what keeps this rank from starting the next call while a peer
// still reads what this call sent it.
__global__ void __launch_bounds__(256)
combine_kernel(const float* __restrict__ y, int T, int H, int K, const int* __restrict__ topk_i,
               const float* __restrict__ topk_w, const int* __restrict__ slot_of,
               float* __restrict__ out, int accumulate, const int* __restrict__ wait_flags, int G,
               int seq, int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    if (wait_flags) {
        if ((int)threadIdx.x < G) {
            const volatile int* f = wait_flags + threadIdx.x;
            unsigned long long t_start = 0;
            while ((int)(*f - seq) < 0) {
                if (*reinterpret_cast<volatile int*>(status) != 0)
                    break;
                unsigned long long now;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                if (t_start == 0)
                    t_start = now;
                else if (now - t_start > 2000000000ull) {
                    report_status(status, 0x301);  // peer::DS_TIMEOUT_PEER
                    break;
                }
                __nanosleep(100);
            }
            __threadfence_system();
        }
        __syncthreads();
    }
    const int t = blockIdx.x;
    if (t >= T)
        return;
    int ex[8], sl[8];
    float wt[8];
#pragma unroll
    for (int k = 0; k < 8; k++) {
        if (k < K) {
            ex[k] = topk_i[(size_t)t * K + k];
            sl[k] = slot_of[(size_t)t * K + k];
            wt[k] = topk_w[(size_t)t * K + k];
        } else {
            ex[k] = 0x7fffffff;
            sl[k] = 0;
            wt[k] = 0.f;
        }
    }
    // sort by expert index (K <= 8): odd-even transposition network on registers
#pragma unroll
    for (int pass = 0; pass < 8; pass++) {
#pragma unroll
        for (int i = (pass & 1); i + 1 < 8; i += 2) {
            if (ex[i] > ex[i + 1]) {
                int te = ex[i]; ex[i] = ex[i + 1]; ex[i + 1] = te;
                int ts = sl[i]; sl[i] = sl[i + 1]; sl[i + 1] = ts;
                float tw = wt[i]; wt[i] = wt[i + 1]; wt[i + 1] = tw;
            }
        }
    }
    const int nvec = H / 4;
    float4* o = reinterpret_cast<float4*>(out + (size_t)t * H);
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int k = 0; k < 8; k++) {
            if (k < K) {
                const float4 yv = reinterpret_cast<const float4*>(y + (size_t)sl[k] * H)[v];
                acc.x = fmaf(yv.x, wt[k], acc.x);
                acc.y = fmaf(yv.y, wt[k], acc.y);
                acc.z = fmaf(yv.z, wt[k], acc.z);
                acc.w = fmaf(yv.w, wt[k], acc.w);
            }
        }
        if (accumulate) {
            float4 p = o[v];
            acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
        }
        o[v] = acc;
    }
}

}  // namespace moe
