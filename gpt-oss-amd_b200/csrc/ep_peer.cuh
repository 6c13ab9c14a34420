// Expert-parallel exchange over peer memory (NVLink / NVSwitch), fused into the
// kernels on either side of it -- no NCCL call, no host wait, no extra pass and
// no extra launch: an expert-parallel call is the same six kernels as a
// single-GPU call.
//
//   counts    the plan kernel stores this rank's per-expert row counts into every
//             rank's control buffer and raises the "counts" flag there
//   dispatch  the permute kernel waits for every rank's counts, works out where
//             its rows go, and stores each token row straight into the owner
//             GPU's expert-grouped GEMM input (plain peer stores) with the row's
//             return address beside it; its last block raises "rows delivered"
//   compute   the gate/up GEMM's activation producer waits for "rows delivered"
//             of every rank before its first load
//   return    the down GEMM's epilogue stores each result row straight into the
//             token owner's combine input; its last CTA raises "results
//             delivered", which the owner's combine kernel waits for
//
// Replaces, like csrc/ep.cuh, the reference's host-driven scheme
// (src/forward.cpp:515-992: pack copies, hipMemcpyPeerAsync, remote launches,
// host event waits, per-(shard, expert) accumulate launches).
//
// A flag is an int in the receiver's control buffer, written by the peer with
// the call's sequence number after a system-scope fence, and polled with a time
// limit; a wait that runs out records DS_TIMEOUT_PEER in the status word, later
// waits of the call return at once, the call's remaining kernels compute
// nothing that leaves this GPU, and the host sees the status.  Buffer reuse:
// a rank starts the next call's peer stores only after its own combine kernel,
// which has seen "results delivered" from every rank, i.e. every rank has
// finished reading what the previous call stored there.
//
// All loads and stores to peer memory are ordinary ld/st; there is no TMA
// multicast and no multimem here, and every TMA load reads local memory.
#pragma once
#include "common.cuh"
#include "peer_io.cuh"
#include "plan.cuh"
#include "route.cuh"

namespace moe {
namespace peer {

// Waits (threads 0..G-1) for the G flags of kind `which` in this rank's control
// buffer; every thread of the block gets the verdict.  Ends with a system-scope
// fence: what the peers stored before raising their flags is visible.
__device__ __forceinline__ bool block_wait_flags(const int* my_ctrl, int E, int G, int which, int seq,
                                                 int* status, int* s_ok) {
    if (threadIdx.x == 0)
        *s_ok = 1;
    __syncthreads();
    if ((int)threadIdx.x < G) {
        if (!wait_flag(my_ctrl + G * E + which * G + threadIdx.x, seq, status))
            *s_ok = 0;
        __threadfence_system();
    }
    __syncthreads();
    return *s_ok != 0;
}

// The plan kernel of plan.cuh (one block) that also publishes this rank's
// per-expert counts to every rank and raises the counts flag there.
__global__ void __launch_bounds__(256)
plan_publish_kernel(const int* __restrict__ blk_hist, int nblk, int E, int bn, int* __restrict__ cnt,
                    int* __restrict__ off, int* __restrict__ tile_start, int* __restrict__ blk_base,
                    int G, int rank, Table tb, int seq) {
    __shared__ int s_cnt[256];
    pdl_trigger();
    pdl_wait();
    plan_body(blk_hist, nblk, E, bn, cnt, off, tile_start, blk_base, s_cnt);
    // s_cnt is complete for every thread here (plan_body ends behind a barrier)
    for (int i = threadIdx.x; i < G * E; i += blockDim.x) {
        const int p = i / E, e = i - p * E;
        tb.ctrl[p][rank * E + e] = s_cnt[e];
    }
    __threadfence_system();
    __syncthreads();
    if ((int)threadIdx.x < G) {
        volatile int* f = flag_slot(tb.ctrl[threadIdx.x], E, G, FLAG_COUNTS, rank);
        *f = seq;
    }
}

// The permute kernel of plan.cuh with the destination on another GPU.
//   1. wait for every rank's counts
//   2. per global expert: the row at which this rank's segment starts in the
//      owner's buffer (rows of expert e at its owner are ordered by source rank)
//   3. block (0,0): the tile tables of the rows THIS rank computes
//   4. stable placement of every (token, k) assignment; the row goes as bf16 into
//      the owner's expert-grouped buffer, its return address beside it
//   5. the last block to finish raises "rows delivered" at every rank
// grid = (max(routing blocks, 1), S); runs with T == 0 too (steps 1-3 and 5).
__global__ void __launch_bounds__(256)
permute_to_peers_kernel(const void* __restrict__ x, int x_is_f32, int T, int H, int K, int E, int G,
                        int rank, int rb, int bn, int rows_cap, const int* __restrict__ topk_i,
                        const int* __restrict__ blk_base, const int* __restrict__ off, Table tb,
                        int seq, int* __restrict__ slot_of, int* __restrict__ g_cnt,
                        int* __restrict__ g_off, int* __restrict__ g_tile_start,
                        int* __restrict__ ticket, int* __restrict__ status) {
    __shared__ int s_e[RB * 8];
    __shared__ int s_row[RB * 8];
    __shared__ int s_tot[256];
    __shared__ int s_base[256];
    __shared__ int s_ok;
    pdl_trigger();
    pdl_wait();
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
    const int* ctrl = tb.ctrl[rank];
    bool ok = block_wait_flags(ctrl, E, G, FLAG_COUNTS, seq, status, &s_ok);
    const volatile int* cnt_all = ctrl;
    const int e = threadIdx.x;
    if (e < E) {
        int t = 0;
        for (int p = 0; p < G; p++)
            t += cnt_all[p * E + e];
        s_tot[e] = ok ? t : 0;
    }
    __syncthreads();
    if ((int)threadIdx.x < G) {
        // no receive buffer may overflow (cannot happen when every rank was created
        // with the same max_tokens, which moe_b200_ep_peer_enable checks)
        long long rows = 0;
        for (int i = shard_first(E, G, threadIdx.x); i < shard_first(E, G, threadIdx.x + 1); i++)
            rows += s_tot[i];
        if (rows > rows_cap) {
            report_status(status, DS_BAD_PLAN);
            s_ok = 0;
        }
    }
    __syncthreads();
    ok = s_ok != 0;
    const int first = shard_first(E, G, rank), n_local = shard_first(E, G, rank + 1) - first;
    if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) {
        int o = 0, t = 0;
        for (int i = 0; i < n_local; i++) {
            const int c = ok ? s_tot[first + i] : 0;
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
        s_base[e] = base;
    }
    __syncthreads();
    if (ok && t0 < T) {
        const int per = (n_assign + gridDim.y - 1) / gridDim.y;  // gridDim.y blocks share a routing block
        const int a_lo = blockIdx.y * per, a_hi = min(n_assign, a_lo + per);
        for (int a = a_lo + threadIdx.x; a < a_hi; a += blockDim.x) {
            const int ea = s_e[a];
            int row = -1;
            if (ea >= 0) {
                int r = 0;
                for (int j = 0; j < a; j++)
                    r += (s_e[j] == ea);
                // position inside this rank's rows of the expert, then inside the owner's buffer
                row = s_base[ea] + (blk_base[(size_t)blockIdx.x * E + ea] - off[ea]) + r;
                const int asg = t0 * K + a;
                tb.ret[shard_owner(E, G, ea)][row] = make_int2(rank, asg);
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
    // every thread's peer stores are fenced at system scope before the block is counted
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int n_blocks = gridDim.x * gridDim.y;
        s_ok = (atomicAdd(ticket, 1) == n_blocks - 1) ? 1 : 0;
    }
    __syncthreads();
    if (s_ok) {  // the last block: all rows of this rank are on their way
        if (threadIdx.x == 0)
            *ticket = 0;
        __threadfence_system();
        if ((int)threadIdx.x < G) {
            volatile int* f = flag_slot(tb.ctrl[threadIdx.x], E, G, FLAG_ROWS, rank);
            *f = seq;
        }
    }
}

}  // namespace peer
}  // namespace moe
