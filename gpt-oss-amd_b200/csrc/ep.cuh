// Expert-parallel exchange: token dispatch and result return as NCCL
// all-to-all(v) over NVLink, with the local grouped GEMMs in between.
//
// Replaces the reference's host-driven scheme (src/forward.cpp:515-992): per
// shard a mutex, a pack of D2D copies, hipMemcpyPeerAsync of fp32 rows and
// weights, kernels launched on the remote device by the token owner's thread,
// peer copies back and one accumulate launch per (shard, expert).  Here every
// rank runs the same call; rows travel as bf16 (5760 B instead of 11520 B at
// H = 2880), results come back as fp32 rows in the sender's own order, and the
// sender applies the routing weights in its combine kernel.
//
// Per call and rank:
//   all-gather of the per-expert row counts  -> one host wait (the sizes of the
//   sends are host arguments of ncclSend/ncclRecv)
//   all-to-all of rows, regroup by local expert, GEMMs, all-to-all back.
#pragma once
#include <nccl.h>

#include <functional>
#include <string>
#include <vector>

#include "../../include/moe_b200.h"
#include "common.cuh"
#include "ep_peer.cuh"

namespace moe {
namespace ep {

struct State {
    ncclComm_t comm = nullptr;
    int* cnt_all = nullptr;       // [G, E] per-expert send counts of every rank
    uint16_t* xrecv = nullptr;    // [rows_cap, H] received rows, grouped by source rank
    uint16_t* xgrp = nullptr;     // [rows_cap, H] the same rows grouped by local expert
    float* ysend = nullptr;       // [rows_cap, H] results in xrecv order
    float* yrecv = nullptr;       // [max_tokens*K, H] results in this rank's send order
    int* g_cnt = nullptr;         // [n_local]
    int* g_off = nullptr;         // [n_local + 1]
    int* g_tile_start = nullptr;  // [n_local + 1]
    int* gather_src = nullptr;    // [rows_cap] grouped row -> xrecv row
    int* recv_off_dev = nullptr;  // [G]
    int* h_cnt_all = nullptr;     // pinned [G, E]
    std::vector<int> send_cnt, send_off, recv_cnt, recv_off;

    // peer-memory mode (ep_peer.cuh)
    int* ctrl = nullptr;          // [G*E counts][3*G flags]; cnt_all aliases its start
    char* arena = nullptr;        // one allocation holding xgrp, yrecv, ctrl, ret (peer-visible)
    size_t arena_off[4] = {0, 0, 0, 0};
    int2* ret = nullptr;          // [rows_cap] return address of each received row
    int* tickets = nullptr;       // [2] finished-block counters (permute kernel, down GEMM)
    size_t arena_bytes = 0;
    int rows_cap = 0;
    bool nccl_buffers = false;    // xrecv / ysend / gather_src exist (NCCL mode only)
    peer::Table table{};
    std::vector<void*> opened;    // cudaIpcOpenMemHandle mappings to close
    bool peer_enabled = false;
    int seq = 0;                  // call sequence number carried by the flags
};

typedef std::function<int(const uint16_t* xin, int rows_upper, int bn, const int* g_off,
                          const int* g_cnt, const int* g_tile_start, float* yout, const int* row_dst)>
    GemmLauncher;
typedef std::function<int(int rows)> PickBn;  // GEMM n-tile width for a call with `rows` local rows
typedef std::function<void(int stage, bool begin)> StageMark;

// Pure host arithmetic (also exported through the C ABI for tests): from the
// [G, E] matrix of per-expert send counts, the rows this rank sends to / gets
// from every peer and where they start.  Rows are sorted by global expert and
// shards are contiguous (src/model.cpp:104-114), so a peer's rows are one
// contiguous range.
inline void plan_exchange(int E, int G, int rank, const int* cnt_all, int* send_cnt, int* send_off,
                          int* recv_cnt, int* recv_off) {
    int my_first = 0, my_n = 0;
    moe_b200_shard_range(E, G, rank, &my_first, &my_n);
    int so = 0, ro = 0;
    for (int p = 0; p < G; p++) {
        int pf = 0, pn = 0;
        moe_b200_shard_range(E, G, p, &pf, &pn);
        int s = 0, r = 0;
        for (int e = pf; e < pf + pn; e++)
            s += cnt_all[(size_t)rank * E + e];
        for (int e = my_first; e < my_first + my_n; e++)
            r += cnt_all[(size_t)p * E + e];
        send_cnt[p] = s;
        send_off[p] = so;
        recv_cnt[p] = r;
        recv_off[p] = ro;
        so += s;
        ro += r;
    }
}

// Tables of the rows this rank computes, grouped by local expert.  One block.
__global__ void __launch_bounds__(256)
regroup_plan_kernel(const int* __restrict__ cnt_all, int E, int G, int first, int n_local, int bn,
                    int* __restrict__ g_cnt, int* __restrict__ g_off, int* __restrict__ g_tile_start) {
    __shared__ int s_cnt[256];
    const int le = threadIdx.x;
    if (le < n_local) {
        int c = 0;
        for (int p = 0; p < G; p++)
            c += cnt_all[(size_t)p * E + first + le];
        s_cnt[le] = c;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int o = 0, t = 0;
        for (int i = 0; i < n_local; i++) {
            g_cnt[i] = s_cnt[i];
            g_off[i] = o;
            g_tile_start[i] = t;
            o += s_cnt[i];
            t += (s_cnt[i] + bn - 1) / bn;
        }
        g_off[n_local] = o;
        g_tile_start[n_local] = t;
    }
}

// gather_src[grouped row] = received row.  grid (n_local, G): one block per
// (local expert, source rank) segment; inside a segment the sender's order is
// kept, and segments of an expert are ordered by source rank.
__global__ void __launch_bounds__(128)
regroup_index_kernel(const int* __restrict__ cnt_all, int E, int G, int first, int n_local,
                     const int* __restrict__ recv_off, const int* __restrict__ g_off,
                     int* __restrict__ gather_src) {
    const int le = blockIdx.x, p = blockIdx.y;
    const int n = cnt_all[(size_t)p * E + first + le];
    if (n == 0)
        return;
    int src = recv_off[p];
    for (int i = 0; i < le; i++)
        src += cnt_all[(size_t)p * E + first + i];
    int dst = g_off[le];
    for (int q = 0; q < p; q++)
        dst += cnt_all[(size_t)q * E + first + le];
    for (int i = threadIdx.x; i < n; i += blockDim.x)
        gather_src[dst + i] = src + i;
}

// xgrp[r, :] = xrecv[gather_src[r], :], 16 bytes per thread.
__global__ void __launch_bounds__(256)
regroup_rows_kernel(const uint16_t* __restrict__ xrecv, const int* __restrict__ gather_src, int rows,
                    int H, uint16_t* __restrict__ xgrp) {
    const int vec = H / 8;
    const int warps_per_block = blockDim.x >> 5;
    const int lane = threadIdx.x & 31;
    for (int r = blockIdx.x * warps_per_block + (threadIdx.x >> 5); r < rows;
         r += gridDim.x * warps_per_block) {
        const uint4* s = reinterpret_cast<const uint4*>(xrecv + (size_t)gather_src[r] * H);
        uint4* d = reinterpret_cast<uint4*>(xgrp + (size_t)r * H);
        for (int v = lane; v < vec; v += 32)
            d[v] = s[v];
    }
}

template <typename T>
inline int ep_alloc(T** p, size_t n, std::vector<void*>& allocs, size_t& bytes, std::string& err) {
    void* q = nullptr;
    size_t b = n * sizeof(T);
    if (b == 0)
        b = sizeof(T);
    cudaError_t e = cudaMalloc(&q, b);
    if (e != cudaSuccess) {
        err = std::string("cudaMalloc (expert-parallel buffers): ") + cudaGetErrorString(e);
        return MOE_B200_ERR_CUDA;
    }
    allocs.push_back(q);
    bytes += b;
    *p = static_cast<T*>(q);
    return 0;
}

inline int allocate(State& s, const moe_b200_config& c, int n_local, int first, int rows_cap,
                    std::vector<void*>& allocs, size_t& bytes, std::string& err) {
    (void)first;
    const size_t H = c.hidden_dim, E = c.n_experts, G = c.ep_size;
    const size_t TK = (size_t)c.max_tokens * c.experts_per_token;
    int st;
    // The buffers a peer writes (xgrp, yrecv, ctrl, ret) share ONE allocation, so that one
    // IPC handle exports them and a peer maps them with one call.
    auto up = [](size_t b) { return (b + 255) / 256 * 256; };
    s.arena_off[0] = 0;                                                      // xgrp
    s.arena_off[1] = s.arena_off[0] + up((size_t)rows_cap * H * sizeof(uint16_t));  // yrecv
    s.arena_off[2] = s.arena_off[1] + up(TK * H * sizeof(float));            // ctrl
    s.arena_off[3] = s.arena_off[2] + up((G * E + 3 * G + 16) * sizeof(int));  // ret
    s.arena_bytes = s.arena_off[3] + up((size_t)rows_cap * sizeof(int2));
    s.rows_cap = rows_cap;
    if ((st = ep_alloc(&s.arena, s.arena_bytes, allocs, bytes, err)))
        return st;
    s.xgrp = reinterpret_cast<uint16_t*>(s.arena + s.arena_off[0]);
    s.yrecv = reinterpret_cast<float*>(s.arena + s.arena_off[1]);
    s.ctrl = reinterpret_cast<int*>(s.arena + s.arena_off[2]);
    s.ret = reinterpret_cast<int2*>(s.arena + s.arena_off[3]);
    if ((st = ep_alloc(&s.tickets, 2, allocs, bytes, err)) ||
        (st = ep_alloc(&s.g_cnt, n_local, allocs, bytes, err)) ||
        (st = ep_alloc(&s.g_off, n_local + 1, allocs, bytes, err)) ||
        (st = ep_alloc(&s.g_tile_start, n_local + 1, allocs, bytes, err)))
        return st;
    s.cnt_all = s.ctrl;
    if (cudaMemset(s.ctrl, 0, (G * E + 3 * G + 16) * sizeof(int)) != cudaSuccess ||
        cudaMemset(s.tickets, 0, 2 * sizeof(int)) != cudaSuccess) {
        err = "cudaMemset failed";
        return MOE_B200_ERR_CUDA;
    }
    return 0;
}

// The buffers only the NCCL exchange uses (received rows in source order, results in
// the same order, the regroup index): allocated by moe_b200_ep_init, so that a handle
// in peer-memory mode does not carry them.
inline int allocate_nccl(State& s, const moe_b200_config& c, std::vector<void*>& allocs, size_t& bytes,
                         std::string& err) {
    if (s.nccl_buffers)
        return 0;
    const size_t H = c.hidden_dim, E = c.n_experts, G = c.ep_size;
    int st;
    if ((st = ep_alloc(&s.xrecv, (size_t)s.rows_cap * H, allocs, bytes, err)) ||
        (st = ep_alloc(&s.ysend, (size_t)s.rows_cap * H, allocs, bytes, err)) ||
        (st = ep_alloc(&s.gather_src, s.rows_cap, allocs, bytes, err)) ||
        (st = ep_alloc(&s.recv_off_dev, G, allocs, bytes, err)))
        return st;
    if (cudaMallocHost(reinterpret_cast<void**>(&s.h_cnt_all), G * E * sizeof(int)) != cudaSuccess) {
        err = "cudaMallocHost failed";
        return MOE_B200_ERR_CUDA;
    }
    s.send_cnt.assign(G, 0);
    s.send_off.assign(G, 0);
    s.recv_cnt.assign(G, 0);
    s.recv_off.assign(G, 0);
    s.nccl_buffers = true;
    return 0;
}

inline void shutdown(State& s) {
    for (void* p : s.opened)
        cudaIpcCloseMemHandle(p);
    s.opened.clear();
    s.peer_enabled = false;
    if (s.comm) {
        ncclCommDestroy(s.comm);
        s.comm = nullptr;
    }
    if (s.h_cnt_all) {
        cudaFreeHost(s.h_cnt_all);
        s.h_cnt_all = nullptr;
    }
}

inline int unique_id(char out[128], std::string& err) {
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is expected to be 128 bytes");
    ncclUniqueId id;
    ncclResult_t r = ncclGetUniqueId(&id);
    if (r != ncclSuccess) {
        err = std::string("ncclGetUniqueId: ") + ncclGetErrorString(r);
        return MOE_B200_ERR_NCCL;
    }
    memcpy(out, &id, 128);
    return 0;
}

inline int init(State& s, const char id_bytes[128], int G, int rank, std::string& err) {
    if (s.comm)
        return 0;
    ncclUniqueId id;
    memcpy(&id, id_bytes, 128);
    ncclResult_t r = ncclCommInitRank(&s.comm, G, id, rank);
    if (r != ncclSuccess) {
        s.comm = nullptr;
        err = std::string("ncclCommInitRank: ") + ncclGetErrorString(r);
        return MOE_B200_ERR_NCCL;
    }
    return 0;
}

#define EP_NCCL(expr)                                                        \
    do {                                                                     \
        ncclResult_t _r = (expr);                                            \
        if (_r != ncclSuccess) {                                             \
            err = std::string(#expr) + ": " + ncclGetErrorString(_r);        \
            return MOE_B200_ERR_NCCL;                                        \
        }                                                                    \
    } while (0)
#define EP_CUDA(expr)                                                        \
    do {                                                                     \
        cudaError_t _e = (expr);                                             \
        if (_e != cudaSuccess) {                                             \
            err = std::string(#expr) + ": " + cudaGetErrorString(_e);        \
            return MOE_B200_ERR_CUDA;                                        \
        }                                                                    \
    } while (0)

// cnt: this rank's per-(global)-expert row counts; xs: its rows sorted by
// expert.  On return *y_out points at the fp32 result rows in the same order
// as xs.
inline int exchange_and_compute(State& s, const moe_b200_config& c, int n_local, int first,
                                const PickBn& pick_bn, int T, const int* cnt, const uint16_t* xs, const GemmLauncher& gemms,
                                const StageMark& mark, const float** y_out, cudaStream_t st,
                                int* launches, std::string& err) {
    (void)T;
    const int E = c.n_experts, G = c.ep_size, rank = c.ep_rank, H = c.hidden_dim;
    mark(MOE_B200_STAGE_DISPATCH, true);
    EP_NCCL(ncclAllGather(cnt, s.cnt_all, (size_t)E, ncclInt32, s.comm, st));
    EP_CUDA(cudaMemcpyAsync(s.h_cnt_all, s.cnt_all, (size_t)G * E * sizeof(int),
                            cudaMemcpyDeviceToHost, st));
    EP_CUDA(cudaStreamSynchronize(st));
    plan_exchange(E, G, rank, s.h_cnt_all, s.send_cnt.data(), s.send_off.data(), s.recv_cnt.data(),
                  s.recv_off.data());
    const int rows = s.recv_off[G - 1] + s.recv_cnt[G - 1];
    const int bn = pick_bn(rows);
    EP_CUDA(cudaMemcpyAsync(s.recv_off_dev, s.recv_off.data(), (size_t)G * sizeof(int),
                            cudaMemcpyHostToDevice, st));

    EP_NCCL(ncclGroupStart());
    for (int p = 0; p < G; p++) {
        if (s.send_cnt[p] > 0)
            EP_NCCL(ncclSend(xs + (size_t)s.send_off[p] * H, (size_t)s.send_cnt[p] * H, ncclBfloat16,
                             p, s.comm, st));
        if (s.recv_cnt[p] > 0)
            EP_NCCL(ncclRecv(s.xrecv + (size_t)s.recv_off[p] * H, (size_t)s.recv_cnt[p] * H,
                             ncclBfloat16, p, s.comm, st));
    }
    EP_NCCL(ncclGroupEnd());
    mark(MOE_B200_STAGE_DISPATCH, false);

    mark(MOE_B200_STAGE_REGROUP, true);
    regroup_plan_kernel<<<1, 256, 0, st>>>(s.cnt_all, E, G, first, n_local, bn, s.g_cnt, s.g_off,
                                           s.g_tile_start);
    *launches += 1;
    if (rows > 0) {
        regroup_index_kernel<<<dim3(n_local, G), 128, 0, st>>>(s.cnt_all, E, G, first, n_local,
                                                              s.recv_off_dev, s.g_off, s.gather_src);
        int blocks = (rows + 7) / 8;
        if (blocks > 148 * 8)
            blocks = 148 * 8;
        regroup_rows_kernel<<<blocks, 256, 0, st>>>(s.xrecv, s.gather_src, rows, H, s.xgrp);
        *launches += 2;
    }
    mark(MOE_B200_STAGE_REGROUP, false);
    if (rows > 0) {
        int gst = gemms(s.xgrp, rows, bn, s.g_off, s.g_cnt, s.g_tile_start, s.ysend, s.gather_src);
        if (gst)
            return gst;
    }

    mark(MOE_B200_STAGE_RETURN, true);
    EP_NCCL(ncclGroupStart());
    for (int p = 0; p < G; p++) {
        if (s.recv_cnt[p] > 0)
            EP_NCCL(ncclSend(s.ysend + (size_t)s.recv_off[p] * H, (size_t)s.recv_cnt[p] * H,
                             ncclFloat32, p, s.comm, st));
        if (s.send_cnt[p] > 0)
            EP_NCCL(ncclRecv(s.yrecv + (size_t)s.send_off[p] * H, (size_t)s.send_cnt[p] * H,
                             ncclFloat32, p, s.comm, st));
    }
    EP_NCCL(ncclGroupEnd());
    mark(MOE_B200_STAGE_RETURN, false);
    *y_out = s.yrecv;
    return 0;
}

// ---------------------------------------------------------------------------
// Peer-memory mode

constexpr int PEER_BUFFERS = 4;  // xgrp, yrecv, ctrl, ret
static_assert(sizeof(cudaIpcMemHandle_t) == MOE_B200_EP_IPC_BYTES, "IPC handle size");

// What follows the IPC handle in an export blob.  Peers store into the arena at
// addresses computed from THEIR configuration, so every field must agree between
// the ranks before any mapping is used.
struct PeerBlobInfo {
    unsigned long long off[PEER_BUFFERS];  // byte offsets of xgrp, yrecv, ctrl, ret
    unsigned long long arena_bytes;
    int hidden, n_experts, top_k, max_tokens, rows_cap, ep_size, ep_rank, version;
};
constexpr int PEER_BLOB_VERSION = 2;
static_assert(sizeof(cudaIpcMemHandle_t) + sizeof(PeerBlobInfo) <= MOE_B200_EP_PEER_EXPORT_BYTES,
              "export blob size");

inline PeerBlobInfo peer_blob_info(const State& s, const moe_b200_config& c) {
    PeerBlobInfo b{};
    for (int i = 0; i < PEER_BUFFERS; i++)
        b.off[i] = s.arena_off[i];
    b.arena_bytes = s.arena_bytes;
    b.hidden = c.hidden_dim;
    b.n_experts = c.n_experts;
    b.top_k = c.experts_per_token;
    b.max_tokens = c.max_tokens;
    b.rows_cap = s.rows_cap;
    b.ep_size = c.ep_size;
    b.ep_rank = c.ep_rank;
    b.version = PEER_BLOB_VERSION;
    return b;
}

// blob: the arena's IPC handle, then PeerBlobInfo.
inline int peer_export(State& s, const moe_b200_config& c, char* out, std::string& err) {
    memset(out, 0, MOE_B200_EP_PEER_EXPORT_BYTES);
    cudaIpcMemHandle_t h;
    EP_CUDA(cudaIpcGetMemHandle(&h, s.arena));
    memcpy(out, &h, sizeof(h));
    const PeerBlobInfo b = peer_blob_info(s, c);
    memcpy(out + sizeof(h), &b, sizeof(b));
    return 0;
}

// all: [G][MOE_B200_EP_PEER_EXPORT_BYTES], the exports of every rank in rank order.
// Every blob is checked against this rank's own configuration BEFORE any peer
// memory is mapped: a rank created with other sizes would receive stores past the
// end of its buffers.
inline int peer_enable(State& s, const moe_b200_config& c, const char* all, std::string& err) {
    const int G = c.ep_size, rank = c.ep_rank;
    if (G > peer::MAX_RANKS) {
        err = "peer-memory mode supports at most 8 ranks";
        return MOE_B200_ERR_UNSUPPORTED;
    }
    if (c.n_experts > 256) {
        err = "peer-memory mode supports at most 256 experts";
        return MOE_B200_ERR_UNSUPPORTED;
    }
    if (s.peer_enabled)
        return 0;
    const PeerBlobInfo mine = peer_blob_info(s, c);
    for (int p = 0; p < G; p++) {
        PeerBlobInfo b;
        memcpy(&b, all + (size_t)p * MOE_B200_EP_PEER_EXPORT_BYTES + MOE_B200_EP_IPC_BYTES, sizeof(b));
        const char* what = nullptr;
        if (b.version != PEER_BLOB_VERSION)
            what = "blob version";
        else if (b.ep_rank != p)
            what = "rank order of the blobs";
        else if (b.ep_size != mine.ep_size)
            what = "ep_size";
        else if (b.hidden != mine.hidden)
            what = "hidden_dim";
        else if (b.n_experts != mine.n_experts)
            what = "n_experts";
        else if (b.top_k != mine.top_k)
            what = "experts_per_token";
        else if (b.max_tokens != mine.max_tokens)
            what = "max_tokens";
        else if (b.rows_cap != mine.rows_cap || b.arena_bytes != mine.arena_bytes ||
                 memcmp(b.off, mine.off, sizeof(b.off)) != 0)
            what = "exchange buffer layout";
        if (what) {
            err = std::string("peer export of rank ") + std::to_string(p) + " does not match this rank: " +
                  what + " differs (every rank must be created with the same hidden_dim, n_experts, "
                         "experts_per_token, max_tokens and ep_size)";
            return MOE_B200_ERR_INVALID;
        }
    }
    for (int p = 0; p < G; p++) {
        const char* blob = all + (size_t)p * MOE_B200_EP_PEER_EXPORT_BYTES;
        char* base = s.arena;
        if (p != rank) {
            cudaIpcMemHandle_t h;
            memcpy(&h, blob, sizeof(h));
            void* q = nullptr;
            EP_CUDA(cudaIpcOpenMemHandle(&q, h, cudaIpcMemLazyEnablePeerAccess));
            s.opened.push_back(q);
            base = static_cast<char*>(q);
        }
        s.table.xgrp[p] = reinterpret_cast<uint16_t*>(base + mine.off[0]);
        s.table.yrecv[p] = reinterpret_cast<float*>(base + mine.off[1]);
        s.table.ctrl[p] = reinterpret_cast<int*>(base + mine.off[2]);
        s.table.ret[p] = reinterpret_cast<int2*>(base + mine.off[3]);
    }
    s.peer_enabled = true;
    return 0;
}

}  // namespace ep
}  // namespace moe
