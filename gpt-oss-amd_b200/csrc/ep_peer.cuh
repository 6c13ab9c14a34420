// Expert-parallel exchange over peer memory (NVLink / NVSwitch), fused into the
// kernels on either side of it -- no NCCL call, no host wait, no extra pass.
//
//   dispatch  the permute kernel stores each token row straight into the
//             destination GPU's expert-grouped GEMM input (plain peer stores),
//             together with the row's return address
//   return    the down-projection GEMM's epilogue stores each result row
//             straight into the owner GPU's combine input
//
// Replaces, like csrc/ep.cuh, the reference's host-driven scheme
// (src/forward.cpp:515-992: pack copies, hipMemcpyPeerAsync, remote launches,
// host event waits, per-(shard, expert) accumulate launches).
//
// Synchronisation: three flag barriers per call (counts published, rows
// delivered, results delivered).  A flag is an int in the receiver's control
// buffer, written by the peer with the call's sequence number after a
// system-scope fence, and polled by one thread with a time limit; a wait that
// runs out records DS_TIMEOUT_PEER in the status word and the kernel returns
// (later kernels of the call then work on stale data; the host sees the status).
// Buffers are reused by the next call only after the last barrier of this
// one, which every rank passes after all ranks finished reading them.
//
// All loads and stores to peer memory are ordinary ld/st; there is no TMA
// multicast and no multimem here.
#pragma once
#include "common.cuh"
#include "route.cuh"

namespace moe {
namespace peer {

constexpr int MAX_RANKS = 8;
constexpr unsigned long long PEER_WAIT_NS = 2000000000ull;  // 2 s
constexpr int DS_TIMEOUT_PEER = 0x301;

// Control buffer of a rank (ints): [G*E] counts of every rank, then three rows
// of G flags (counts / dispatch / return).
struct Table {
    uint16_t* xgrp[MAX_RANKS];  // [rows_cap, H] bf16: GEMM input, grouped by local expert
    float* yrecv[MAX_RANKS];    // [max_tokens*K, H] f32: combine input in assignment order
    int* ctrl[MAX_RANKS];
    int2* ret[MAX_RANKS];       // [rows_cap]: (owner rank, owner assignment) of each row
};

__device__ __forceinline__ unsigned long long timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ int shard_first(int E, int G, int d) {
    const int base = E / G, rem = E % G;
    return d * base + (d < rem ? d : rem);
}
__device__ __forceinline__ int shard_owner(int E, int G, int e) {
    const int base = E / G, rem = E % G;
    const int cut = (base + 1) * rem;
    return e < cut ? e / (base + 1) : rem + (e - cut) / base;
}

// Bounded poll of flag `slot` until it reaches `seq`.
__device__ __forceinline__ bool wait_flag(const int* flag, int seq, int* status) {
    const volatile int* f = flag;
    const unsigned long long t0 = timer_ns();
    while ((int)(*f - seq) < 0) {
        if (timer_ns() - t0 > PEER_WAIT_NS) {
            report_status(status, DS_TIMEOUT_PEER);
            return false;
        }
        __nanosleep(200);
    }
    return true;
}

// One block.  Copies this rank's per-expert counts into every rank's control
// buffer, then raises the counts flag there.
__global__ void __launch_bounds__(256)
publish_counts_kernel(const int* __restrict__ cnt, int E, int G, int rank, Table tb, int seq) {
    for (int i = threadIdx.x; i < G * E; i += blockDim.x) {
        const int p = i / E, e = i - p * E;
        tb.ctrl[p][rank * E + e] = cnt[e];
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < G) {
        volatile int* f = tb.ctrl[threadIdx.x] + G * E + rank;
        *f = seq;
    }
}

// One block.  Waits for every rank's counts, then builds (a) the tables of the
// rows this rank computes, grouped by local expert, and (b) for every global
// expert the row at which this rank's segment starts in the owner's buffer:
// rows of expert e at its owner are ordered by source rank.
__global__ void __launch_bounds__(256)
wait_counts_plan_kernel(int E, int G, int rank, int bn, Table tb, int seq, int* __restrict__ g_cnt,
                        int* __restrict__ g_off, int* __restrict__ g_tile_start,
                        int* __restrict__ send_base, int* __restrict__ status) {
    __shared__ int s_tot[256];
    __shared__ int s_ok;
    const int* ctrl = tb.ctrl[rank];
    if (threadIdx.x == 0)
        s_ok = 1;
    __syncthreads();
    if (threadIdx.x < G) {
        if (!wait_flag(ctrl + G * E + threadIdx.x, seq, status))
            s_ok = 0;
    }
    __syncthreads();
    __threadfence_system();
    const volatile int* cnt_all = ctrl;
    const int e = threadIdx.x;
    if (e < E) {
        int t = 0;
        for (int p = 0; p < G; p++)
            t += cnt_all[p * E + e];
        s_tot[e] = s_ok ? t : 0;
    }
    __syncthreads();
    const int first = shard_first(E, G, rank), n_local = shard_first(E, G, rank + 1) - first;
    if (threadIdx.x == 0) {
        int o = 0, t = 0;
        for (int i = 0; i < n_local; i++) {
            const int c = s_tot[first + i];
            g_cnt[i] = c;
            g_off[i] = o;
            g_tile_start[i] = t;
            o += c;
            t += (c + bn - 1) / bn;
        }
        g_off[n_local] = o;
        g_tile_start[n_local] = t;
    }
    if (e < E) {
        const int d = shard_owner(E, G, e);
        int base = 0;
        for (int i = shard_first(E, G, d); i < e; i++)
            base += s_tot[i];
        for (int p = 0; p < rank; p++)
            base += cnt_all[p * E + e];
        send_base[e] = base;
    }
}

// The permute kernel of plan.cuh with the destination on another GPU: stable
// placement of every (token, k) assignment, row copied as bf16 into the owner's
// expert-grouped buffer, return address beside it.  grid = (routing blocks, S).
__global__ void __launch_bounds__(256)
permute_to_peers_kernel(const void* __restrict__ x, int x_is_f32, int T, int H, int K, int E, int G,
                        int rank, int rb, const int* __restrict__ topk_i,
                        const int* __restrict__ blk_base, const int* __restrict__ off,
                        const int* __restrict__ send_base, Table tb, int* __restrict__ slot_of,
                        int* __restrict__ status) {
    __shared__ int s_e[RB * 8];
    __shared__ int s_row[RB * 8];
    const int t0 = blockIdx.x * rb;
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
    const int per = (n_assign + gridDim.y - 1) / gridDim.y;  // gridDim.y blocks share a routing block
    const int a_lo = blockIdx.y * per, a_hi = min(n_assign, a_lo + per);
    for (int a = a_lo + threadIdx.x; a < a_hi; a += blockDim.x) {
        const int e = s_e[a];
        int row = -1;
        if (e >= 0) {
            int r = 0;
            for (int j = 0; j < a; j++)
                r += (s_e[j] == e);
            // position inside this rank's rows of expert e, then inside the owner's buffer
            row = send_base[e] + (blk_base[(size_t)blockIdx.x * E + e] - off[e]) + r;
            const int d = shard_owner(E, G, e);
            const int asg = t0 * K + a;
            tb.ret[d][row] = make_int2(rank, asg);
            slot_of[asg] = asg;  // results come back in assignment order
        }
        s_row[a] = row;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int vec_per_row = H / 8;
    for (int a = a_lo + warp; a < a_hi; a += nwarps) {
        const int row = s_row[a];
        if (row < 0)
            continue;
        const int t = t0 + a / K;
        uint4* dst = reinterpret_cast<uint4*>(tb.xgrp[shard_owner(E, G, s_e[a])] + (size_t)row * H);
        if (x_is_f32) {
            const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(x) + (size_t)t * H);
            for (int v = lane; v < vec_per_row; v += 32) {
                float4 p = src[2 * v], q = src[2 * v + 1];
                dst[v] = make_uint4(pack_bf16x2(p.x, p.y), pack_bf16x2(p.z, p.w),
                                    pack_bf16x2(q.x, q.y), pack_bf16x2(q.z, q.w));
            }
        } else {
            const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(x) + (size_t)t * H);
            for (int v = lane; v < vec_per_row; v += 32)
                dst[v] = src[v];
        }
    }
}

// One warp.  Flag barrier `which` (1 = rows delivered, 2 = results delivered):
// everything this GPU wrote before is fenced at system scope, every rank is told,
// and every rank's word is awaited.
__global__ void __launch_bounds__(32)
barrier_kernel(int which, int E, int G, int rank, Table tb, int seq, int* __restrict__ status) {
    __threadfence_system();
    if (threadIdx.x < G) {
        volatile int* f = tb.ctrl[threadIdx.x] + G * E + which * G + rank;
        *f = seq;
        wait_flag(tb.ctrl[rank] + G * E + which * G + threadIdx.x, seq, status);
    }
    __syncwarp();
    __threadfence_system();
}

// Address of the owner's result row for every row this rank computes.
__global__ void __launch_bounds__(256)
row_pointers_kernel(const int* __restrict__ g_off, int n_local, int H, Table tb, int rank,
                    float** __restrict__ row_ptr) {
    const int rows = g_off[n_local];
    const int2* ret = tb.ret[rank];
    for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += gridDim.x * blockDim.x) {
        const int2 a = ret[r];
        row_ptr[r] = tb.yrecv[a.x] + (size_t)a.y * H;
    }
}

}  // namespace peer
}  // namespace moe
