// Types and device helpers shared by the peer-memory exchange (ep_peer.cuh) and the
// expert GEMMs that take part in it: flag layout, bounded flag waits, and what a
// GEMM kernel needs to know about the other ranks.
#pragma once
#include "common.cuh"

namespace moe {
namespace peer {

constexpr int MAX_RANKS = 8;
constexpr unsigned long long PEER_WAIT_NS = 2000000000ull;  // 2 s
constexpr int DS_TIMEOUT_PEER = 0x301;  // a rank did not join the call in time
constexpr int DS_BAD_PLAN = 0x302;      // the ranks' row counts exceed a receive buffer

constexpr int FLAG_COUNTS = 0, FLAG_ROWS = 1, FLAG_RESULTS = 2;

// Control buffer of a rank (ints): [G*E] counts of every rank, then three rows
// of G flags (counts / rows delivered / results delivered), one per source rank.
struct Table {
    uint16_t* xgrp[MAX_RANKS];  // [rows_cap, H] bf16: GEMM input, grouped by local expert
    float* yrecv[MAX_RANKS];    // [max_tokens*K, H] f32: combine input in assignment order
    int* ctrl[MAX_RANKS];
    int2* ret[MAX_RANKS];       // [rows_cap]: (owner rank, owner assignment) of each row
};

// What the expert GEMMs need in peer mode (all zero otherwise).
struct GemmPeerIO {
    const int* wait_flags;       // gate/up GEMM: this rank's "rows delivered" flags [G]
    float* yrecv[MAX_RANKS];     // down GEMM: every rank's combine input
    const int2* ret;             // down GEMM: return address of each row computed here
    int* done_flags[MAX_RANKS];  // down GEMM: where to raise "results delivered" (one per rank)
    int* ticket;                 // down GEMM: counts CTAs that finished storing
    int G, seq;
};

__device__ __forceinline__ unsigned long long timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__host__ __device__ __forceinline__ int shard_first(int E, int G, int d) {
    const int base = E / G, rem = E % G;
    return d * base + (d < rem ? d : rem);
}
__device__ __forceinline__ int shard_owner(int E, int G, int e) {
    const int base = E / G, rem = E % G;
    const int cut = (base + 1) * rem;
    return e < cut ? e / (base + 1) : rem + (e - cut) / base;
}

__host__ __device__ __forceinline__ int* flag_slot(int* ctrl, int E, int G, int which, int src) {
    return ctrl + G * E + which * G + src;
}

// Bounded poll of a flag until it reaches `seq`.  Gives up at once when the
// status word already holds a code: one wait of the call has failed, the rest
// would only add their own two seconds.
__device__ __forceinline__ bool wait_flag(const int* flag, int seq, int* status) {
    const volatile int* f = flag;
    if ((int)(*f - seq) >= 0)
        return true;
    const unsigned long long t0 = timer_ns();
    while ((int)(*f - seq) < 0) {
        if (*reinterpret_cast<volatile int*>(status) != 0)
            return false;
        if (timer_ns() - t0 > PEER_WAIT_NS) {
            report_status(status, DS_TIMEOUT_PEER);
            return false;
        }
        __nanosleep(100);
    }
    return true;
}

}  // namespace peer
}  // namespace moe
