// Host side of the C ABI declared in include/moe_b200.h.
#include "../../include/moe_b200.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "batcher.hpp"
#include "common.cuh"
#include "ep.cuh"
#include "expert_file.hpp"
#ifdef MOE_B200_TEST_AIDS
#include "gemm_mma.cuh"
#endif
#include "gemm_tc5_pair.cuh"
#include "gemm_tc5_ts.cuh"
#include "mxfp4.cuh"
#include "plan.cuh"
#include "route.cuh"

using namespace moe;

namespace {

std::string g_create_error;

struct LayerWeights {
    uint16_t* w_router = nullptr;  // [E, H] bf16
    float* b_router = nullptr;     // [E]
    uint8_t* w1 = nullptr;         // [n_local][m_tiles1][ks1][CHUNK_BYTES]
    uint8_t* w2 = nullptr;         // [n_local][m_tiles2][ks2][CHUNK_BYTES]
    float* bias1 = nullptr;        // [n_local, 2I]
    float* bias2 = nullptr;        // [n_local, H]
    float* rscale1 = nullptr;      // [n_local, 2I]  2^shift of every gate/up weight row (mxfp4_row_shift_kernel)
    float* rscale2 = nullptr;      // [n_local, H]
    bool router_set = false;
    std::vector<char> expert_set;
};

}  // namespace

struct moe_b200_request_queue_s {
    moe::sched::RequestQueue q;
};
struct moe_b200_batcher_s {
    moe::sched::Batcher b;
};

struct moe_b200_handle_s {
    moe_b200_config cfg{};
    int first_expert = 0, n_local = 0;
    int m_tiles1 = 0, m_tiles2 = 0, ks1 = 0, ks2 = 0;
    size_t stride1 = 0, stride2 = 0;  // bytes per expert
    int n_sms = 0;
    int rows_cap = 0;                 // rows the grouped buffers can hold
    int nblk_cap = 0;
    std::vector<LayerWeights> layers;
    std::vector<void*> allocs;
    size_t device_bytes = 0;

    // routing + permutation workspace
    int* topk_i = nullptr;
    float* topk_w = nullptr;
    int* blk_hist = nullptr;
    int* blk_base = nullptr;
    int* cnt = nullptr;         // [E] rows per (global) expert, send order
    int* off = nullptr;         // [E+1]
    int* tile_start = nullptr;  // [E+1] (ep_size == 1: the GEMM tile table)
    int* slot_of = nullptr;     // [T*K] row of each assignment in send order
    int* row_token = nullptr;   // [T*K]
    uint16_t* xs = nullptr;     // [T*K, H] bf16 rows sorted by expert (send order)
    uint16_t* xn = nullptr;     // [T, H] bf16 block input when the norm in front of it is fused
    uint16_t* hbuf = nullptr;   // [rows_cap, I] bf16
    float* ybuf = nullptr;      // [rows_cap, H] fp32
    int* status = nullptr;

    // host staging for moe_b200_forward_host
    void* t_dev = nullptr;
    float* out_dev = nullptr;
    cudaStream_t own_stream = nullptr;
    cudaStream_t in_stream = nullptr, out_stream = nullptr;  // host-buffer entry point: copies beside the compute
    std::vector<cudaEvent_t> host_ev;                       // two per token chunk

    // upload staging (one expert matrix)
    uint8_t* stage_blocks = nullptr;
    uint8_t* stage_scales = nullptr;
    int* stage_shift = nullptr;  // exponent shift of every row of the matrix being re-tiled

    tc5::TensorMaps maps_x{}, maps_h{};  // TMA maps over the GEMM inputs
    int pair_grid = 0;       // CTAs of the pair GEMM (2 x resident clusters)
    int smem_attr_done = 0;  // bit set: shared-memory opt-in of a kernel family done on this device

    ep::State ep;

    // per-stage timing: event pairs for `prof_armed` forwards
    std::vector<cudaEvent_t> prof_ev;
    int prof_armed = 0, prof_next = 0, prof_call = -1;
    bool prof_external = false;  // the host-buffer entry point picked prof_call for the forward it wraps

    std::string err;
    int last_launches = 0;
};

namespace {

moe_b200_status fail(moe_b200_handle h, moe_b200_status st, const std::string& msg) {
    if (h)
        h->err = msg;
    else
        g_create_error = msg;
    return st;
}

#define CU_TRY(h, expr)                                                                     \
    do {                                                                                    \
        cudaError_t _e = (expr);                                                            \
        if (_e != cudaSuccess)                                                              \
            return fail(h, MOE_B200_ERR_CUDA,                                               \
                        std::string(#expr) + ": " + cudaGetErrorString(_e));                \
    } while (0)

// Records the begin / end event of a stage of the forward being profiled.
void prof_mark(moe_b200_handle h, int stage, bool begin, cudaStream_t st) {
    if (h->prof_call < 0)
        return;
    cudaEventRecord(h->prof_ev[((size_t)h->prof_call * MOE_B200_N_STAGES + stage) * 2 + (begin ? 0 : 1)], st);
}

bool is_device_pointer(const void* p) {
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}

// Programmatic dependent launch (pdl_wait / pdl_trigger in common.cuh) for the kernels
// of a small-batch single-GPU call: each may start its set-up while the kernel before
// it drains.  MOE_B200_NO_PDL=1 in the environment switches it off (a debugging aid:
// the kernels then run strictly one after the other, as on every other path).
bool pdl_enabled() {
    static const bool on = std::getenv("MOE_B200_NO_PDL") == nullptr;
    return on;
}

template <typename... KArgs, typename... Args>
cudaError_t launch_kernel(bool pdl, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                          cudaStream_t st, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

template <typename T>
moe_b200_status dev_alloc(moe_b200_handle h, T** p, size_t n_elems) {
    void* q = nullptr;
    size_t bytes = n_elems * sizeof(T);
    if (bytes == 0)
        bytes = sizeof(T);
    CU_TRY(h, cudaMalloc(&q, bytes));
    h->allocs.push_back(q);
    h->device_bytes += bytes;
    *p = static_cast<T*>(q);
    return MOE_B200_OK;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

moe_b200_status make_maps(moe_b200_handle h, tc5::TensorMaps* maps, void* base, int cols, int rows) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    CU_TRY(h, cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
    if (!fn || qres != cudaDriverEntryPointSuccess)
        return fail(h, MOE_B200_ERR_CUDA, "cuTensorMapEncodeTiled not available in this driver");
    EncodeTiledFn encode = reinterpret_cast<EncodeTiledFn>(fn);
    for (int i = 0; i < 4; i++) {
        cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
        cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
        cuuint32_t box[2] = {(cuuint32_t)KSTAGE, (cuuint32_t)(32 << i)};
        cuuint32_t estr[2] = {1, 1};
        CUresult r = encode(&maps->box[i], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides,
                            box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS)
            return fail(h, MOE_B200_ERR_CUDA,
                        "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
    }
    for (int i = 0; i < 2; i++) {
        // [chunk][row][64 columns]: the chunk axis has the smallest stride (128 bytes)
        cuuint64_t dims[3] = {(cuuint64_t)KSTAGE, (cuuint64_t)rows, (cuuint64_t)(cols / KSTAGE)};
        cuuint64_t strides[2] = {(cuuint64_t)cols * 2, (cuuint64_t)KSTAGE * 2};
        cuuint32_t box[3] = {(cuuint32_t)KSTAGE, (cuuint32_t)(32 << i), (cuuint32_t)tc5::STEP_CHUNKS};
        cuuint32_t estr[3] = {1, 1, 1};
        CUresult r = encode(&maps->box3[i], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, base, dims, strides,
                            box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS)
            return fail(h, MOE_B200_ERR_CUDA,
                        "cuTensorMapEncodeTiled (3-d) failed with code " + std::to_string((int)r));
    }
    return MOE_B200_OK;
}

moe_b200_status check_layer(moe_b200_handle h, int layer) {
    if (!h)
        return MOE_B200_ERR_INVALID;
    if (layer < 0 || layer >= h->cfg.n_layers)
        return fail(h, MOE_B200_ERR_INVALID, "layer index out of range");
    return MOE_B200_OK;
}

constexpr int TC5_BN = 256;                   // token rows per tile of the large-batch GEMM
constexpr int SMALL_MAX_ROWS_PER_EXPERT = 64; // at most this many rows per expert on average: small-batch GEMM

// Token rows per routing block (16 x the router kernel's MT).  Measured (E = 128, route
// stage in ms; block height, CTAs per cluster): 2048 tokens (16,1) 0.030, (32,1) 0.042,
// (32,2) 0.031, (64,1) 0.079, (64,4) 0.053; 4096 tokens (16,1) 0.054, (32,1) 0.042,
// (32,2) 0.053, (64,2) 0.062: a block's time grows with its height (more 16-byte
// copies per thread and chunk in the same dependent chain), so a batch takes the
// shortest blocks that still run as one wave, and tall blocks only when it must.
// `nt` = ceil(E / 32).
int route_block_tokens(int T, int nt) {
    if (T <= 2368)
        return 16;
    if (T <= 9472 || nt > 4)  // 8 expert tiles: at most 32 rows per block (registers)
        return 32;
    return 64;
}

// cudaFuncAttributeMaxDynamicSharedMemorySize belongs to (device, kernel), not to a
// handle.  The router kernel's shared memory depends only on its template
// parameters, so every caller -- any handle's forward and the handle-free
// moe_b200_route_noalloc -- asks for the same value; it is set once per device and
// instantiation through this one function and never lowered.
constexpr int MAX_DEVICES = 64;
int g_route_attr[MAX_DEVICES];  // bit per (NT, MT, XF32) instantiation

struct RouteArgs {
    const void* x;  // bf16 rows (f32 with x_is_f32: the handle-free entry point only)
    int x_is_f32, T, H;
    const uint16_t* w_router;
    const float* b_router;
    int E, K;
    float* score_out;
    int* topk_i;
    float* topk_w;
    int* blk_hist;
    bool pdl;                  // launch as a programmatic dependent of the kernel before it
    int n_sms;                 // SMs of the device, or 0: never split K over a cluster
};

template <int NT, int MT, bool XF32>
cudaError_t launch_route_tc(int dev, const RouteArgs& a, cudaStream_t st) {
    constexpr int bit = 1 << (((NT == 1 ? 0 : NT == 2 ? 1 : NT == 4 ? 2 : 3) * 3 + (MT == 1 ? 0 : MT == 2 ? 1 : 2)) * 2 +
                              (XF32 ? 1 : 0));
    if (dev < 0 || dev >= MAX_DEVICES)
        return cudaErrorInvalidDevice;
    if (!(g_route_attr[dev] & bit)) {
        cudaError_t e = cudaFuncSetAttribute(route_tc_kernel<NT, MT, XF32>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)route_tc_smem_bytes<NT, MT>());
        if (e != cudaSuccess)
            return e;
        g_route_attr[dev] |= bit;
    }
    const int nblk = ceil_div(a.T, 16 * MT);
    // a launch that failed must not be followed by kernels that consume its output
    const cudaError_t e = launch_kernel(a.pdl, route_tc_kernel<NT, MT, XF32>, dim3(nblk), dim3(RTHREADS),
                                        route_tc_smem_bytes<NT, MT>(), st, a.x, a.T, a.H, a.w_router, a.b_router,
                                        a.E, a.K, a.score_out, a.topk_i, a.topk_w, a.blk_hist);
    return e != cudaSuccess ? e : cudaGetLastError();
}

int g_route_cs_attr[MAX_DEVICES];  // bit per (NT, CS) instantiation of the K-split router

// Small batches: a cluster of CS CTAs per block of 16 tokens splits K (route.cuh).
template <int NT, int CS>
cudaError_t launch_route_split(int dev, const RouteArgs& a, cudaStream_t st) {
    constexpr int bit = 1 << ((NT == 1 ? 0 : NT == 2 ? 1 : NT == 4 ? 2 : 3) * 3 + (CS == 2 ? 0 : CS == 4 ? 1 : 2));
    if (dev < 0 || dev >= MAX_DEVICES)
        return cudaErrorInvalidDevice;
    auto kernel = route_tc_kernel<NT, 1, false, CS>;
    if (!(g_route_cs_attr[dev] & bit)) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)route_tc_smem_bytes<NT, 1, CS>());
        if (e != cudaSuccess)
            return e;
        g_route_cs_attr[dev] |= bit;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ceil_div(a.T, 16) * CS);
    cfg.blockDim = dim3(RTHREADS);
    cfg.dynamicSmemBytes = route_tc_smem_bytes<NT, 1, CS>();
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CS;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = a.pdl ? 2 : 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, a.x, a.T, a.H, a.w_router, a.b_router, a.E, a.K,
                                             a.score_out, a.topk_i, a.topk_w, a.blk_hist);
    return e != cudaSuccess ? e : cudaGetLastError();
}

template <int NT>
cudaError_t launch_route_short(int dev, const RouteArgs& a, cudaStream_t st) {
    // as many CTAs per token block as still fit one wave
    const int nblk = ceil_div(a.T, 16);
    if (nblk * 8 <= a.n_sms)
        return launch_route_split<NT, 8>(dev, a, st);
    if (nblk * 4 <= a.n_sms)
        return launch_route_split<NT, 4>(dev, a, st);
    if (nblk * 2 <= a.n_sms)
        return launch_route_split<NT, 2>(dev, a, st);
    return launch_route_tc<NT, 1, false>(dev, a, st);
}

// rb = rows per routing block as route_block_tokens() chose them (fp32 rows: 16).
cudaError_t launch_route(int dev, const RouteArgs& a, int rb, cudaStream_t st) {
    const int nt = ceil_div(a.E, 32);
    if (a.x_is_f32) {
        if (rb != 16)
            return cudaErrorInvalidValue;
        if (nt <= 1)
            return launch_route_tc<1, 1, true>(dev, a, st);
        if (nt <= 2)
            return launch_route_tc<2, 1, true>(dev, a, st);
        if (nt <= 4)
            return launch_route_tc<4, 1, true>(dev, a, st);
        return launch_route_tc<8, 1, true>(dev, a, st);
    }
#define ROUTE_CASE(NT_)                                         \
    do {                                                        \
        if (rb == 16)                                           \
            return launch_route_short<NT_>(dev, a, st);         \
        if (rb == 32)                                           \
            return launch_route_tc<NT_, 2, false>(dev, a, st);  \
    } while (0)
    if (nt <= 1) {
        ROUTE_CASE(1);
        return launch_route_tc<1, 4, false>(dev, a, st);
    }
    if (nt <= 2) {
        ROUTE_CASE(2);
        return launch_route_tc<2, 4, false>(dev, a, st);
    }
    if (nt <= 4) {
        ROUTE_CASE(4);
        return launch_route_tc<4, 4, false>(dev, a, st);
    }
    ROUTE_CASE(8);
#undef ROUTE_CASE
    return cudaErrorInvalidValue;
}

// Large batches on CTA pairs (gemm_tc5_pair.cuh): cluster launch, one cluster per SM pair.
template <int MODE>
moe_b200_status launch_pair_kernel(moe_b200_handle h, int grid, cudaStream_t st,
                                   const tc5::TensorMaps& maps, const uint8_t* chunks, size_t stride,
                                   int ks, int m_tiles, const float* bias, const float* rscale,
                                   int bias_stride,
                                   const int* g_off, const int* g_cnt, const int* g_tile_start, int EL,
                                   void* out, int out_ld, int out_valid, const int* row_dst,
                                   const peer::GemmPeerIO& pio) {
    namespace pr = tc5::pair;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(pr::N_THREADS);
    cfg.dynamicSmemBytes = pr::SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    CU_TRY(h, cudaLaunchKernelEx(&cfg, pr::expert_gemm_pair_kernel<MODE>, maps, chunks, stride, ks, m_tiles,
                                 bias, rscale, bias_stride, g_off, g_cnt, g_tile_start, EL, out, out_ld,
                                 out_valid,
                                 row_dst, pio, h->cfg.swiglu_alpha, h->cfg.swiglu_limit, h->status));
    return MOE_B200_OK;
}

moe_b200_status launch_pair(moe_b200_handle h, const LayerWeights& lw, const tc5::TensorMaps& maps_x,
                            const int* g_off, const int* g_cnt, const int* g_tile_start, float* yout,
                            const int* row_dst, const peer::GemmPeerIO& pio, cudaStream_t st) {
    const moe_b200_config& c = h->cfg;
    const int H = c.hidden_dim, I = c.intermediate_dim, EL = h->n_local;
    namespace pr = tc5::pair;
    if (!(h->smem_attr_done & 4)) {
        CU_TRY(h, cudaFuncSetAttribute(pr::expert_gemm_pair_kernel<0>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, pr::SMEM_BYTES));
        CU_TRY(h, cudaFuncSetAttribute(pr::expert_gemm_pair_kernel<1>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, pr::SMEM_BYTES));
        // clusters that can be resident at once: a persistent kernel must not launch more
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * (h->n_sms / 2));
        cfg.blockDim = dim3(pr::N_THREADS);
        cfg.dynamicSmemBytes = pr::SMEM_BYTES;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int n_clusters = 0;
        CU_TRY(h, cudaOccupancyMaxActiveClusters(&n_clusters, pr::expert_gemm_pair_kernel<0>, &cfg));
        if (n_clusters < 1)
            return fail(h, MOE_B200_ERR_CUDA, "no CTA pair of the expert GEMM fits on this device");
        h->pair_grid = 2 * std::min(n_clusters, h->n_sms / 2);
        h->smem_attr_done |= 4;
    }
    prof_mark(h, MOE_B200_STAGE_GEMM1, true, st);
    moe_b200_status s1 = launch_pair_kernel<0>(h, h->pair_grid, st, maps_x, lw.w1, h->stride1, h->ks1,
                                               h->m_tiles1, lw.bias1, lw.rscale1, 2 * I, g_off, g_cnt,
                                               g_tile_start, EL, h->hbuf, I, I, nullptr, pio);
    if (s1)
        return s1;
    prof_mark(h, MOE_B200_STAGE_GEMM1, false, st);
    prof_mark(h, MOE_B200_STAGE_GEMM2, true, st);
    s1 = launch_pair_kernel<1>(h, h->pair_grid, st, h->maps_h, lw.w2, h->stride2, h->ks2, h->m_tiles2,
                               lw.bias2, lw.rscale2, H, g_off, g_cnt, g_tile_start, EL, yout, H, H, row_dst,
                               pio);
    if (s1)
        return s1;
    prof_mark(h, MOE_B200_STAGE_GEMM2, false, st);
    h->last_launches += 2;
    return MOE_B200_OK;
}

// Small batches, decoded weights in tensor memory (gemm_tc5_ts.cuh).
moe_b200_status launch_ts(moe_b200_handle h, const LayerWeights& lw, const tc5::TensorMaps& maps_x,
                          const int* g_off, const int* g_cnt, const int* g_tile_start, float* yout,
                          const int* row_dst, const peer::GemmPeerIO& pio, cudaStream_t st) {
    const moe_b200_config& c = h->cfg;
    const int H = c.hidden_dim, I = c.intermediate_dim, EL = h->n_local;
    namespace ts = tc5::ts;
    if (!(h->smem_attr_done & 32)) {
        CU_TRY(h, cudaFuncSetAttribute(ts::expert_gemm_ts_kernel<0>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, ts::SMEM_BYTES));
        CU_TRY(h, cudaFuncSetAttribute(ts::expert_gemm_ts_kernel<1>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, ts::SMEM_BYTES));
        h->smem_attr_done |= 32;
    }
    prof_mark(h, MOE_B200_STAGE_GEMM1, true, st);
    const bool pdl = c.ep_size == 1 && pdl_enabled();
    CU_TRY(h, launch_kernel(pdl, ts::expert_gemm_ts_kernel<0>, dim3(h->n_sms), dim3(ts::N_THREADS),
                            ts::SMEM_BYTES, st, maps_x, lw.w1, h->stride1, h->ks1, h->m_tiles1, lw.bias1,
                            lw.rscale1, 2 * I, g_off, g_cnt, g_tile_start, EL, (void*)h->hbuf, I, I,
                            (const int*)nullptr, pio, c.swiglu_alpha, c.swiglu_limit, h->status));
    prof_mark(h, MOE_B200_STAGE_GEMM1, false, st);
    prof_mark(h, MOE_B200_STAGE_GEMM2, true, st);
    CU_TRY(h, launch_kernel(pdl, ts::expert_gemm_ts_kernel<1>, dim3(h->n_sms), dim3(ts::N_THREADS),
                            ts::SMEM_BYTES, st, h->maps_h, lw.w2, h->stride2, h->ks2, h->m_tiles2, lw.bias2,
                            lw.rscale2, H, g_off, g_cnt, g_tile_start, EL, (void*)yout, H, H, row_dst, pio,
                            c.swiglu_alpha, c.swiglu_limit, h->status));
    prof_mark(h, MOE_B200_STAGE_GEMM2, false, st);
    h->last_launches += 2;
    return MOE_B200_OK;
}

// The two grouped GEMMs over `g_*` tables describing rows grouped by local
// expert; `bn` is the number of token rows per tile the tables were built for
// (pick_bn), which also selects the kernel.
moe_b200_status launch_gemms(moe_b200_handle h, const LayerWeights& lw, const uint16_t* xin,
                             const tc5::TensorMaps& maps_x, int rows_upper, int bn,
                             const int* g_off,
                             const int* g_cnt, const int* g_tile_start, float* yout,
                             const int* row_dst, const peer::GemmPeerIO& pio, cudaStream_t st) {
    const moe_b200_config& c = h->cfg;
    const int H = c.hidden_dim, I = c.intermediate_dim, EL = h->n_local;
#ifdef MOE_B200_TEST_AIDS
    if (c.gemm_impl == MOE_B200_GEMM_MMA_SYNC) {
        if (pio.ret)
            return fail(h, MOE_B200_ERR_UNSUPPORTED,
                        "the cross-check GEMM does not take part in the peer-memory exchange");
        const int n_tiles_upper = rows_upper / V0_BN + EL;
        dim3 g1(n_tiles_upper, h->m_tiles1), g2(n_tiles_upper, h->m_tiles2);
        prof_mark(h, MOE_B200_STAGE_GEMM1, true, st);
        expert_gemm_mma_kernel<0><<<g1, 256, 0, st>>>(lw.w1, h->stride1, h->ks1, lw.bias1, lw.rscale1, 2 * I,
                                                      xin,
                                                      H, g_off, g_cnt, g_tile_start, EL, h->hbuf, I,
                                                      I, nullptr, c.swiglu_alpha, c.swiglu_limit);
        prof_mark(h, MOE_B200_STAGE_GEMM1, false, st);
        prof_mark(h, MOE_B200_STAGE_GEMM2, true, st);
        expert_gemm_mma_kernel<1><<<g2, 256, 0, st>>>(lw.w2, h->stride2, h->ks2, lw.bias2, lw.rscale2, H,
                                                      h->hbuf,
                                                      I, g_off, g_cnt, g_tile_start, EL, yout, H, H,
                                                      row_dst, c.swiglu_alpha, c.swiglu_limit);
        prof_mark(h, MOE_B200_STAGE_GEMM2, false, st);
        h->last_launches += 2;
        return MOE_B200_OK;
    }
#endif
    (void)xin;
    (void)rows_upper;
    (void)H;
    (void)I;
    (void)EL;
    if (bn == tc5::ts::BN)
        return launch_ts(h, lw, maps_x, g_off, g_cnt, g_tile_start, yout, row_dst, pio, st);
    if (bn == TC5_BN)
        return launch_pair(h, lw, maps_x, g_off, g_cnt, g_tile_start, yout, row_dst, pio, st);
    return fail(h, MOE_B200_ERR_INVALID, "tile tables were built for another tile height");
}

// Blocks per routing block of the permute kernels: about sixteen blocks per SM (measured at
// 16384 tokens: 0.136 ms with four, 0.108 ms with sixteen), at least one row per warp.
int permute_split(moe_b200_handle h, int nblk, int n_assign) {
    const int want = (16 * h->n_sms + nblk - 1) / (nblk > 0 ? nblk : 1);
    return std::max(1, std::min({want, 8, n_assign / 8}));
}

// Token rows per GEMM tile for a call that has `rows` rows spread over the local
// experts; the tile tables are built for it and it selects the kernel: few rows per
// expert (bound by streaming the weights) -> the single-CTA kernel with the decoded
// weights in tensor memory, 64 token rows per tile; otherwise CTA pairs and 256
// token rows per tile.  Any choice is correct for any distribution of rows.
int pick_bn(moe_b200_handle h, int rows) {
#ifdef MOE_B200_TEST_AIDS
    if (h->cfg.gemm_impl == MOE_B200_GEMM_MMA_SYNC)
        return V0_BN;
#endif
    const int per_expert = rows / (h->n_local > 0 ? h->n_local : 1);
    return per_expert <= SMALL_MAX_ROWS_PER_EXPERT ? tc5::ts::BN : TC5_BN;
}

moe_b200_status check_shard(moe_b200_handle h, int first_expert, int n) {
    if (n <= 0 || first_expert < h->first_expert || first_expert + n > h->first_expert + h->n_local)
        return fail(h, MOE_B200_ERR_INVALID,
                    "experts [" + std::to_string(first_expert) + ", " +
                        std::to_string(first_expert + n) + ") are not inside this rank's shard [" +
                        std::to_string(h->first_expert) + ", " +
                        std::to_string(h->first_expert + h->n_local) + ")");
    return MOE_B200_OK;
}

// Upload of packed experts: everything is queued on one stream (copy -> re-tile ->
// next copy into the same staging buffer are ordered by it) and the host waits once,
// in upload_finish.  Rows whose scale bytes the shifted one-multiply decode cannot hold are
// reported through a flag word of their own, so that an older wait code in the
// status word cannot mask them.
moe_b200_status upload_begin(moe_b200_handle h) {
    CU_TRY(h, cudaMemsetAsync(h->status + 1, 0, sizeof(int), h->own_stream));
    return MOE_B200_OK;
}

moe_b200_status upload_expert(moe_b200_handle h, int layer, int le, const uint8_t* b1, const uint8_t* s1,
                              const float* c1, const uint8_t* b2, const uint8_t* s2, const float* c2) {
    LayerWeights& lw = h->layers[layer];
    const int H = h->cfg.hidden_dim, I = h->cfg.intermediate_dim;
    const int G1 = H / 32, G2 = I / 32;
    const size_t nb1 = (size_t)2 * I * G1 * 16, ns1 = (size_t)2 * I * G1;
    const size_t nb2 = (size_t)H * G2 * 16, ns2 = (size_t)H * G2;
    cudaStream_t s = h->own_stream;
    int* bad_scale = h->status + 1;
    if (!(is_device_pointer(b1) && is_device_pointer(s1))) {
        CU_TRY(h, cudaMemcpyAsync(h->stage_blocks, b1, nb1, cudaMemcpyHostToDevice, s));
        CU_TRY(h, cudaMemcpyAsync(h->stage_scales, s1, ns1, cudaMemcpyHostToDevice, s));
        b1 = h->stage_blocks;
        s1 = h->stage_scales;
    }
    mxfp4_row_shift_kernel<<<(2 * I + 7) / 8, 256, 0, s>>>(b1, s1, 2 * I, G1, h->stage_shift,
                                                           lw.rscale1 + (size_t)le * 2 * I, bad_scale);
    mxfp4_retile_kernel<<<dim3(h->ks1, h->m_tiles1), TILE_M, 0, s>>>(b1, s1, 2 * I, G1, h->stage_shift,
                                                                     lw.w1 + le * h->stride1);
    if (!(is_device_pointer(b2) && is_device_pointer(s2))) {
        CU_TRY(h, cudaMemcpyAsync(h->stage_blocks, b2, nb2, cudaMemcpyHostToDevice, s));
        CU_TRY(h, cudaMemcpyAsync(h->stage_scales, s2, ns2, cudaMemcpyHostToDevice, s));
        b2 = h->stage_blocks;
        s2 = h->stage_scales;
    }
    mxfp4_row_shift_kernel<<<(H + 7) / 8, 256, 0, s>>>(b2, s2, H, G2, h->stage_shift,
                                                       lw.rscale2 + (size_t)le * H, bad_scale);
    mxfp4_retile_kernel<<<dim3(h->ks2, h->m_tiles2), TILE_M, 0, s>>>(b2, s2, H, G2, h->stage_shift,
                                                                     lw.w2 + le * h->stride2);
    CU_TRY(h, cudaMemcpyAsync(lw.bias1 + (size_t)le * 2 * I, c1, (size_t)2 * I * 4, cudaMemcpyDefault, s));
    CU_TRY(h, cudaMemcpyAsync(lw.bias2 + (size_t)le * H, c2, (size_t)H * 4, cudaMemcpyDefault, s));
    return MOE_B200_OK;
}

moe_b200_status upload_finish(moe_b200_handle h, int layer, int first_expert, int n) {
    LayerWeights& lw = h->layers[layer];
    CU_TRY(h, cudaGetLastError());
    int sw = 0;
    CU_TRY(h, cudaMemcpyAsync(&sw, h->status + 1, sizeof(int), cudaMemcpyDeviceToHost, h->own_stream));
    CU_TRY(h, cudaStreamSynchronize(h->own_stream));
    for (int i = 0; i < n; i++)
        lw.expert_set[first_expert + i - h->first_expert] = (sw == 0);
    if (sw != 0)
        return fail(h, MOE_B200_ERR_UNSUPPORTED,
                    "a weight row whose blocks' e8m0 scale bytes span more than 128 binades was found "
                    "(blocks of zeros do not count); one row of the in-kernel decode covers 128");
    return MOE_B200_OK;
}

}  // namespace

// ---------------------------------------------------------------------------

extern "C" {

const char* moe_b200_version(void) {
#ifdef MOE_B200_TEST_AIDS
    return "moe_b200 0.2 sm_100a test-aids";
#else
    return "moe_b200 0.2 sm_100a";
#endif
}

void moe_b200_shard_range(int n_experts, int ep_size, int ep_rank, int* first_expert, int* n_local) {
    // src/model.cpp:104-114: contiguous blocks, remainder to the low ranks
    if (ep_size <= 0) {
        if (first_expert)
            *first_expert = 0;
        if (n_local)
            *n_local = 0;
        return;
    }
    const int base = n_experts / ep_size, rem = n_experts % ep_size;
    const int local = base + (ep_rank < rem ? 1 : 0);
    const int first = ep_rank * base + (ep_rank < rem ? ep_rank : rem);
    if (first_expert)
        *first_expert = first;
    if (n_local)
        *n_local = local;
}

moe_b200_status moe_b200_create(const moe_b200_config* cfg, moe_b200_handle* out) {
    if (!cfg || !out)
        return fail(nullptr, MOE_B200_ERR_INVALID, "null argument");
    *out = nullptr;
    const moe_b200_config& c = *cfg;
    if (c.hidden_dim <= 0 || c.hidden_dim % 64 || c.intermediate_dim <= 0 || c.intermediate_dim % 64)
        return fail(nullptr, MOE_B200_ERR_INVALID, "hidden_dim and intermediate_dim must be positive multiples of 64");
    if (c.n_experts <= 0 || c.n_experts > 256)
        return fail(nullptr, MOE_B200_ERR_INVALID, "n_experts must be in 1..256");
    if (c.experts_per_token <= 0 || c.experts_per_token > 8 || c.experts_per_token > c.n_experts)
        return fail(nullptr, MOE_B200_ERR_INVALID, "experts_per_token must be in 1..min(8, n_experts)");
    if (c.n_layers <= 0 || c.max_tokens <= 0)
        return fail(nullptr, MOE_B200_ERR_INVALID, "n_layers and max_tokens must be positive");
    if (c.ep_size <= 0 || c.ep_rank < 0 || c.ep_rank >= c.ep_size || c.ep_size > c.n_experts)
        return fail(nullptr, MOE_B200_ERR_INVALID, "bad ep_rank / ep_size");
#ifdef MOE_B200_TEST_AIDS
    if (c.gemm_impl != MOE_B200_GEMM_TCGEN05 && c.gemm_impl != MOE_B200_GEMM_MMA_SYNC)
        return fail(nullptr, MOE_B200_ERR_INVALID, "unknown gemm_impl");
#else
    if (c.gemm_impl != MOE_B200_GEMM_TCGEN05)
        return fail(nullptr, MOE_B200_ERR_INVALID,
                    "gemm_impl must be MOE_B200_GEMM_TCGEN05 (the cross-check kernel exists only in "
                    "the test-aids build)");
#endif

    int n_dev = 0;
    if (cudaGetDeviceCount(&n_dev) != cudaSuccess || n_dev == 0) {
        cudaGetLastError();
        return fail(nullptr, MOE_B200_ERR_NO_DEVICE, "no CUDA device; this library has no CPU path");
    }
    if (c.device < 0 || c.device >= n_dev)
        return fail(nullptr, MOE_B200_ERR_INVALID, "device ordinal out of range");
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, c.device) != cudaSuccess)
        return fail(nullptr, MOE_B200_ERR_CUDA, "cudaGetDeviceProperties failed");
    if (prop.major != 10)
        return fail(nullptr, MOE_B200_ERR_NO_DEVICE,
                    "device is sm_" + std::to_string(prop.major * 10 + prop.minor) +
                        "; the kernels are built for sm_100a only");

    moe_b200_handle h = new (std::nothrow) moe_b200_handle_s();
    if (!h)
        return fail(nullptr, MOE_B200_ERR_INVALID, "out of host memory");
    h->cfg = c;
    h->n_sms = prop.multiProcessorCount;
    moe_b200_shard_range(c.n_experts, c.ep_size, c.ep_rank, &h->first_expert, &h->n_local);
    const int H = c.hidden_dim, I = c.intermediate_dim, E = c.n_experts, K = c.experts_per_token;
    h->m_tiles1 = ceil_div(2 * I, TILE_M);
    h->m_tiles2 = ceil_div(H, TILE_M);
    h->ks1 = H / KSTAGE;
    h->ks2 = I / KSTAGE;
    h->stride1 = (size_t)h->m_tiles1 * h->ks1 * CHUNK_BYTES;
    h->stride2 = (size_t)h->m_tiles2 * h->ks2 * CHUNK_BYTES;
    h->rows_cap = c.max_tokens * K * c.ep_size;
    {
        // most routing blocks any batch up to max_tokens can have
        const int nt = ceil_div(E, 32);
        const int steps[3] = {std::min(c.max_tokens, 2368), std::min(c.max_tokens, 9472), c.max_tokens};
        h->nblk_cap = 1;
        for (int i = 0; i < 3; i++)
            h->nblk_cap = std::max(h->nblk_cap, ceil_div(steps[i], route_block_tokens(steps[i], nt)));
    }

    moe_b200_status st = MOE_B200_OK;
    auto bail = [&](moe_b200_status s) {
        std::string e = h->err;
        moe_b200_destroy(h);
        g_create_error = e;
        return s;
    };
    if (cudaSetDevice(c.device) != cudaSuccess)
        return bail(fail(h, MOE_B200_ERR_CUDA, "cudaSetDevice failed"));

    h->layers.resize(c.n_layers);
    for (auto& lw : h->layers) {
        lw.expert_set.assign(h->n_local, 0);
        if ((st = dev_alloc(h, &lw.w_router, (size_t)E * H)) || (st = dev_alloc(h, &lw.b_router, E)) ||
            (st = dev_alloc(h, &lw.w1, h->stride1 * h->n_local)) ||
            (st = dev_alloc(h, &lw.w2, h->stride2 * h->n_local)) ||
            (st = dev_alloc(h, &lw.bias1, (size_t)h->n_local * 2 * I)) ||
            (st = dev_alloc(h, &lw.bias2, (size_t)h->n_local * H)) ||
            (st = dev_alloc(h, &lw.rscale1, (size_t)h->n_local * 2 * I)) ||
            (st = dev_alloc(h, &lw.rscale2, (size_t)h->n_local * H)))
            return bail(st);
    }
    const size_t TK = (size_t)c.max_tokens * K;
    if ((st = dev_alloc(h, &h->topk_i, TK)) || (st = dev_alloc(h, &h->topk_w, TK)) ||
        (st = dev_alloc(h, &h->blk_hist, (size_t)h->nblk_cap * E)) ||
        (st = dev_alloc(h, &h->blk_base, (size_t)h->nblk_cap * E)) ||
        (st = dev_alloc(h, &h->cnt, E)) || (st = dev_alloc(h, &h->off, E + 1)) ||
        (st = dev_alloc(h, &h->tile_start, E + 1)) || (st = dev_alloc(h, &h->slot_of, TK)) ||
        (st = dev_alloc(h, &h->row_token, TK)) || (st = dev_alloc(h, &h->xs, TK * H)) ||
        (st = dev_alloc(h, &h->xn, (size_t)c.max_tokens * H)) ||
        (st = dev_alloc(h, &h->hbuf, (size_t)h->rows_cap * I)) ||
        (st = dev_alloc(h, &h->status, 2)) ||
        (st = dev_alloc(h, (float**)&h->t_dev, (size_t)c.max_tokens * H)) ||
        (st = dev_alloc(h, &h->out_dev, (size_t)c.max_tokens * H)) ||
        (st = dev_alloc(h, &h->stage_blocks, (size_t)2 * I * (H / 32) * 16 > (size_t)H * (I / 32) * 16
                                                 ? (size_t)2 * I * (H / 32) * 16
                                                 : (size_t)H * (I / 32) * 16)) ||
        (st = dev_alloc(h, &h->stage_scales, (size_t)2 * I * (H / 32) > (size_t)H * (I / 32)
                                                 ? (size_t)2 * I * (H / 32)
                                                 : (size_t)H * (I / 32))) ||
        (st = dev_alloc(h, &h->stage_shift, (size_t)(2 * I > H ? 2 * I : H))))
        return bail(st);
    // fp32 rows of the down GEMM before the combine: only the single-GPU path keeps
    // them here (expert-parallel results go to the token owner's receive buffer)
    if (c.ep_size == 1 && (st = dev_alloc(h, &h->ybuf, (size_t)h->rows_cap * H)))
        return bail(st);
    if (cudaMemset(h->status, 0, 2 * sizeof(int)) != cudaSuccess ||
        cudaStreamCreateWithFlags(&h->own_stream, cudaStreamNonBlocking) != cudaSuccess)
        return bail(fail(h, MOE_B200_ERR_CUDA, "stream / memset failed"));
    if (c.ep_size > 1) {
        st = (moe_b200_status)ep::allocate(h->ep, c, h->n_local, h->first_expert, h->rows_cap,
                                           h->allocs, h->device_bytes, h->err);
        if (st)
            return bail(st);
    }
    {
        void* x_base = (c.ep_size > 1) ? (void*)h->ep.xgrp : (void*)h->xs;
        const int x_rows = (c.ep_size > 1) ? h->rows_cap : (int)TK;
        if ((st = make_maps(h, &h->maps_x, x_base, H, x_rows)) ||
            (st = make_maps(h, &h->maps_h, h->hbuf, I, h->rows_cap)))
            return bail(st);
    }
    *out = h;
    return MOE_B200_OK;
}

moe_b200_status moe_b200_destroy(moe_b200_handle h) {
    if (!h)
        return MOE_B200_OK;
    cudaSetDevice(h->cfg.device);
    cudaDeviceSynchronize();
    ep::shutdown(h->ep);
    for (void* p : h->allocs)
        cudaFree(p);
    for (cudaEvent_t e : h->prof_ev)
        cudaEventDestroy(e);
    if (h->own_stream)
        cudaStreamDestroy(h->own_stream);
    if (h->in_stream)
        cudaStreamDestroy(h->in_stream);
    if (h->out_stream)
        cudaStreamDestroy(h->out_stream);
    for (cudaEvent_t e : h->host_ev)
        cudaEventDestroy(e);
    cudaGetLastError();
    delete h;
    return MOE_B200_OK;
}

moe_b200_status moe_b200_set_router(moe_b200_handle h, int layer, const void* w_bf16,
                                    const float* bias) {
    moe_b200_status st = check_layer(h, layer);
    if (st)
        return st;
    if (!w_bf16 || !bias)
        return fail(h, MOE_B200_ERR_INVALID, "null router pointer");
    CU_TRY(h, cudaSetDevice(h->cfg.device));
    LayerWeights& lw = h->layers[layer];
    const size_t E = h->cfg.n_experts, H = h->cfg.hidden_dim;
    CU_TRY(h, cudaMemcpy(lw.w_router, w_bf16, E * H * 2, cudaMemcpyDefault));
    CU_TRY(h, cudaMemcpy(lw.b_router, bias, E * 4, cudaMemcpyDefault));
    lw.router_set = true;
    return MOE_B200_OK;
}

moe_b200_status moe_b200_set_experts_mxfp4(moe_b200_handle h, int layer, int first_expert, int n,
                                           const uint8_t* blocks1, const uint8_t* scales1,
                                           const float* bias1, const uint8_t* blocks2,
                                           const uint8_t* scales2, const float* bias2) {
    moe_b200_status st = check_layer(h, layer);
    if (st)
        return st;
    if (!blocks1 || !scales1 || !bias1 || !blocks2 || !scales2 || !bias2)
        return fail(h, MOE_B200_ERR_INVALID, "null expert pointer");
    if ((st = check_shard(h, first_expert, n)))
        return st;
    CU_TRY(h, cudaSetDevice(h->cfg.device));
    const int H = h->cfg.hidden_dim, I = h->cfg.intermediate_dim;
    const size_t nb1 = (size_t)2 * I * (H / 32) * 16, ns1 = (size_t)2 * I * (H / 32);
    const size_t nb2 = (size_t)H * (I / 32) * 16, ns2 = (size_t)H * (I / 32);
    if ((st = upload_begin(h)))
        return st;
    for (int i = 0; i < n; i++) {
        if ((st = upload_expert(h, layer, first_expert + i - h->first_expert, blocks1 + i * nb1,
                                scales1 + i * ns1, bias1 + (size_t)i * 2 * I, blocks2 + i * nb2,
                                scales2 + i * ns2, bias2 + (size_t)i * H)))
            return st;
    }
    return upload_finish(h, layer, first_expert, n);
}

moe_b200_status moe_b200_expert_file_info(const char* path, int* n_layers, int* n_experts,
                                          int* hidden_dim, int* intermediate_dim,
                                          int* experts_per_token, float* swiglu_limit,
                                          unsigned long long* file_bytes) {
    if (!path)
        return fail(nullptr, MOE_B200_ERR_INVALID, "null path");
    efile::Mapping m;
    const std::string err = efile::open_file(path, m);
    if (!err.empty())
        return fail(nullptr, MOE_B200_ERR_INVALID, err);
    const efile::RefConfig& c = m.hdr.config;
    if (n_layers)
        *n_layers = c.n_layers;
    if (n_experts)
        *n_experts = c.n_experts;
    if (hidden_dim)
        *hidden_dim = c.hidden_dim;
    if (intermediate_dim)
        *intermediate_dim = c.intermediate_dim;
    if (experts_per_token)
        *experts_per_token = c.experts_per_token;
    if (swiglu_limit)
        *swiglu_limit = c.swiglu_limit;
    if (file_bytes)
        *file_bytes = m.hdr.file_bytes;
    return MOE_B200_OK;
}

moe_b200_status moe_b200_load_experts_file(moe_b200_handle h, const char* path, int file_layer, int layer) {
    moe_b200_status st = check_layer(h, layer);
    if (st)
        return st;
    if (!path)
        return fail(h, MOE_B200_ERR_INVALID, "null path");
    efile::Mapping m;
    const std::string err = efile::open_file(path, m);
    if (!err.empty())
        return fail(h, MOE_B200_ERR_INVALID, err);
    const efile::RefConfig& fc = m.hdr.config;
    const moe_b200_config& c = h->cfg;
    if (fc.hidden_dim != c.hidden_dim || fc.intermediate_dim != c.intermediate_dim ||
        fc.n_experts != c.n_experts || fc.experts_per_token != c.experts_per_token)
        return fail(h, MOE_B200_ERR_INVALID,
                    std::string(path) + ": dimensions differ from the handle's (file: H " +
                        std::to_string(fc.hidden_dim) + ", I " + std::to_string(fc.intermediate_dim) + ", E " +
                        std::to_string(fc.n_experts) + ", K " + std::to_string(fc.experts_per_token) + ")");
    if (file_layer < 0 || file_layer >= fc.n_layers)
        return fail(h, MOE_B200_ERR_INVALID, "the file has no such layer");
    CU_TRY(h, cudaSetDevice(c.device));
    const int H = c.hidden_dim, I = c.intermediate_dim, E = c.n_experts;
    const unsigned char* r = efile::router_of(m, file_layer);
    if ((st = moe_b200_set_router(h, layer, r, reinterpret_cast<const float*>(r + (size_t)E * H * 2))))
        return st;
    // only the records of this rank's shard are touched (and so paged in)
    const efile::RecordLayout rl = efile::record_layout(H, I);
    if ((st = upload_begin(h)))
        return st;
    for (int le = 0; le < h->n_local; le++) {
        const unsigned char* rec = efile::record_of(m, file_layer, h->first_expert + le);
        if ((st = upload_expert(h, layer, le, rec + rl.blocks1, rec + rl.scales1,
                                reinterpret_cast<const float*>(rec + rl.bias1), rec + rl.blocks2,
                                rec + rl.scales2, reinterpret_cast<const float*>(rec + rl.bias2))))
            return st;
    }
    return upload_finish(h, layer, h->first_expert, h->n_local);  // waits for the copies: the mapping can go
}

}  // extern "C"

namespace {

// The block.  With `rms_w` the input is the fp32 residual stream: the router kernel
// applies the norm, writes the normalised rows as bf16 into the handle's workspace
// and the permute kernel gathers from there.
moe_b200_status forward_impl(moe_b200_handle h, int layer, const void* t, int t_dtype, const void* rms_w,
                             int rms_w_dtype, int n_tokens, float* out, int accumulate,
                             float* router_score_out, int* topk_i_out, float* topk_w_out,
                             moe_b200_stream stream) {
    moe_b200_status st = check_layer(h, layer);
    if (st)
        return st;
    const moe_b200_config& c = h->cfg;
    if (n_tokens < 0 || n_tokens > c.max_tokens)
        return fail(h, MOE_B200_ERR_INVALID, "n_tokens outside [0, max_tokens]");
    if (t_dtype != MOE_B200_DTYPE_F32 && t_dtype != MOE_B200_DTYPE_BF16)
        return fail(h, MOE_B200_ERR_INVALID, "unknown activation dtype");
    if (rms_w && (rms_w_dtype != MOE_B200_DTYPE_F32 && rms_w_dtype != MOE_B200_DTYPE_BF16))
        return fail(h, MOE_B200_ERR_INVALID, "unknown norm weight dtype");
    if (rms_w && t_dtype != MOE_B200_DTYPE_F32)
        return fail(h, MOE_B200_ERR_INVALID, "the fused norm takes the fp32 residual stream");
    if (n_tokens > 0 && (!t || !out))
        return fail(h, MOE_B200_ERR_INVALID, "null activation / output pointer");
    // the kernels move rows 16 bytes at a time: a pointer off that boundary would be a
    // misaligned-address fault on the GPU, so it is refused here
    if (n_tokens > 0 && ((reinterpret_cast<uintptr_t>(t) | reinterpret_cast<uintptr_t>(out) |
                          reinterpret_cast<uintptr_t>(rms_w)) & 15u) != 0)
        return fail(h, MOE_B200_ERR_INVALID,
                    "activation, output and norm-weight pointers must be 16-byte aligned");
    LayerWeights& lw = h->layers[layer];
    if (!lw.router_set)
        return fail(h, MOE_B200_ERR_NOT_LOADED, "router weights of this layer were not set");
    for (char s : lw.expert_set)
        if (!s)
            return fail(h, MOE_B200_ERR_NOT_LOADED, "not every local expert of this layer was set");
    if (c.ep_size > 1 && !h->ep.comm && !h->ep.peer_enabled)
        return fail(h, MOE_B200_ERR_NCCL,
                    "ep_size > 1 but neither moe_b200_ep_init nor moe_b200_ep_peer_enable was called");
    const bool peer_mode = c.ep_size > 1 && h->ep.peer_enabled;
    CU_TRY(h, cudaSetDevice(c.device));
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const int T = n_tokens, H = c.hidden_dim, E = c.n_experts, K = c.experts_per_token;
    const int rb = route_block_tokens(T, ceil_div(E, 32));
    const int nblk = ceil_div(T, rb);
    const int bn_local = pick_bn(h, T * K);  // ep_size == 1: the GEMMs run on this rank's own rows
    // Programmatic dependent launch pays for small batches (decode20b: 4.20 -> 4.05 ms per
    // step) and costs about 1 % on large ones (the next kernel's waiting blocks share the
    // SMs of a GEMM that is bound by instruction issue), so it follows the GEMM choice.
    const bool pdl = c.ep_size == 1 && pdl_enabled() && bn_local == tc5::ts::BN;
    h->last_launches = 0;
    if (!h->prof_external)
        h->prof_call = (h->prof_next < h->prof_armed) ? h->prof_next++ : -1;

    if (T > 0) {
        prof_mark(h, MOE_B200_STAGE_ROUTE, true, s);
        if (t_dtype == MOE_B200_DTYPE_F32) {
            // fp32 rows (the engine's s->t, or with rms_w its residual stream) become the
            // bf16 rows every later kernel reads: one pass, norm folded in when asked
            if (H > 4 * RCAST_THREADS * RCAST_MAX_VEC)
                return fail(h, MOE_B200_ERR_UNSUPPORTED, "fp32 input is supported up to hidden_dim 8192");
            CU_TRY(h, launch_kernel(pdl, rows_to_bf16_kernel, dim3(T), dim3(RCAST_THREADS), 0, s,
                                    static_cast<const float*>(t), T, H, rms_w,
                                    (int)(rms_w_dtype == MOE_B200_DTYPE_F32), h->xn));
            h->last_launches++;
            t = h->xn;
            t_dtype = MOE_B200_DTYPE_BF16;
        }
        RouteArgs ra{t, 0, T, H, lw.w_router, lw.b_router, E, K, router_score_out, h->topk_i, h->topk_w,
                     h->blk_hist, pdl, h->n_sms};
        CU_TRY(h, launch_route(c.device, ra, rb, s));
        prof_mark(h, MOE_B200_STAGE_ROUTE, false, s);
        h->last_launches++;
    }
    // plan + permute also run for T == 0 on an expert-parallel rank (nblk == 0
    // gives all-zero counts), so that the exchange below always has its inputs
    const peer::GemmPeerIO no_peer{};
    const float* y_for_combine = h->ybuf;
    const int* combine_wait = nullptr;
    int seq = 0;
    if (peer_mode) {
        // exchange fused into the plan / permute kernels, the GEMMs and the combine (ep_peer.cuh)
        ep::State& es = h->ep;
        const int G = c.ep_size, rank = c.ep_rank;
        seq = ++es.seq;
        const int bn = pick_bn(h, (T > 0 ? T : c.max_tokens) * K);  // rows here are not known on the host
        prof_mark(h, MOE_B200_STAGE_PLAN, true, s);
        peer::plan_publish_kernel<<<1, 256, 0, s>>>(h->blk_hist, nblk, E, bn_local, h->cnt, h->off,
                                                    h->tile_start, h->blk_base, G, rank, es.table, seq);
        prof_mark(h, MOE_B200_STAGE_PLAN, false, s);
        prof_mark(h, MOE_B200_STAGE_DISPATCH, true, s);
        const int gx = nblk > 0 ? nblk : 1;
        peer::permute_to_peers_kernel<<<dim3(gx, T > 0 ? permute_split(h, nblk, rb * K) : 1), 256, 0, s>>>(
            t, t_dtype == MOE_B200_DTYPE_F32, T, H, K, E, G, rank, rb, bn, h->rows_cap, h->topk_i,
            h->blk_base, h->off, es.table, seq, h->slot_of, es.g_cnt, es.g_off, es.g_tile_start,
            es.tickets, h->status);
        prof_mark(h, MOE_B200_STAGE_DISPATCH, false, s);
        h->last_launches += 2;
        peer::GemmPeerIO pio{};
        pio.wait_flags = peer::flag_slot(es.table.ctrl[rank], E, G, peer::FLAG_ROWS, 0);
        pio.ret = es.table.ret[rank];
        for (int p = 0; p < G; p++) {
            pio.yrecv[p] = es.table.yrecv[p];
            pio.done_flags[p] = peer::flag_slot(es.table.ctrl[p], E, G, peer::FLAG_RESULTS, rank);
        }
        pio.ticket = es.tickets + 1;
        pio.G = G;
        pio.seq = seq;
        st = launch_gemms(h, lw, es.xgrp, h->maps_x, h->rows_cap, bn, es.g_off, es.g_cnt,
                          es.g_tile_start, nullptr, nullptr, pio, s);
        if (st)
            return st;
        y_for_combine = es.yrecv;
        combine_wait = peer::flag_slot(es.table.ctrl[rank], E, G, peer::FLAG_RESULTS, 0);
    } else {
        // small batches: the permute kernel plans by itself (one launch less on the
        // latency-bound path); otherwise a one-block plan kernel runs first
        const bool fused_plan = T > 0 && nblk <= PLAN_FUSED_MAX_BLOCKS;
        if (fused_plan) {
            prof_mark(h, MOE_B200_STAGE_PLAN, true, s);  // an empty stage, not a stale one
            prof_mark(h, MOE_B200_STAGE_PLAN, false, s);
        } else {
            prof_mark(h, MOE_B200_STAGE_PLAN, true, s);
            CU_TRY(h, launch_kernel(pdl, plan_kernel, dim3(1), dim3(256), 0, s, h->blk_hist, nblk, E, bn_local,
                                    h->cnt, h->off, h->tile_start, h->blk_base));
            prof_mark(h, MOE_B200_STAGE_PLAN, false, s);
            h->last_launches++;
        }
        if (T > 0) {
            prof_mark(h, MOE_B200_STAGE_PERMUTE, true, s);
            CU_TRY(h, launch_kernel(pdl, permute_kernel, dim3(nblk, permute_split(h, nblk, rb * K)), dim3(256), 0,
                                    s, t, (int)(t_dtype == MOE_B200_DTYPE_F32), T, H, K, E, rb, h->topk_i,
                                    h->blk_base, h->slot_of, h->row_token, h->xs, h->status,
                                    fused_plan ? h->blk_hist : nullptr, nblk, bn_local, h->cnt, h->off,
                                    h->tile_start));
            prof_mark(h, MOE_B200_STAGE_PERMUTE, false, s);
            h->last_launches++;
        }
        if (c.ep_size == 1) {
            if (T > 0) {
                st = launch_gemms(h, lw, h->xs, h->maps_x, T * K, bn_local, h->off, h->cnt, h->tile_start,
                                  h->ybuf, nullptr, no_peer, s);
                if (st)
                    return st;
            }
        } else {
            ep::GemmLauncher gl = [&](const uint16_t* xin, int rows_upper, int bn, const int* g_off,
                                      const int* g_cnt, const int* g_tile_start, float* yout,
                                      const int* row_dst) -> int {
                return (int)launch_gemms(h, lw, xin, h->maps_x, rows_upper, bn, g_off, g_cnt,
                                         g_tile_start, yout, row_dst, no_peer, s);
            };
            ep::PickBn pick = [&](int rows) { return pick_bn(h, rows); };
            int launches = 0;
            ep::StageMark mark = [&](int stage, bool begin) { prof_mark(h, stage, begin, s); };
            st = (moe_b200_status)ep::exchange_and_compute(h->ep, c, h->n_local, h->first_expert, pick,
                                                           T, h->cnt, h->xs, gl, mark, &y_for_combine, s,
                                                           &launches, h->err);
            h->last_launches += launches;
            if (st)
                return st;
        }
    }

    if (T > 0 || combine_wait) {
        // peer mode launches it for T == 0 as well: the wait inside is what orders this
        // rank's next call behind the peers' reads of this one
        prof_mark(h, MOE_B200_STAGE_COMBINE, true, s);
        CU_TRY(h, launch_kernel(pdl, combine_kernel, dim3(T > 0 ? T : 1), dim3(256), 0, s, y_for_combine, T, H,
                                K, h->topk_i, h->topk_w, h->slot_of, out, accumulate, combine_wait, c.ep_size,
                                seq, h->status));
        prof_mark(h, MOE_B200_STAGE_COMBINE, false, s);
        h->last_launches++;
    }
    if (T > 0) {
        if (topk_i_out)
            CU_TRY(h, cudaMemcpyAsync(topk_i_out, h->topk_i, (size_t)T * K * 4, cudaMemcpyDeviceToDevice, s));
        if (topk_w_out)
            CU_TRY(h, cudaMemcpyAsync(topk_w_out, h->topk_w, (size_t)T * K * 4, cudaMemcpyDeviceToDevice, s));
    }
    CU_TRY(h, cudaGetLastError());
    return MOE_B200_OK;
}

}  // namespace

extern "C" {

moe_b200_status moe_b200_forward(moe_b200_handle h, int layer, const void* t, int t_dtype,
                                 int n_tokens, float* out, int accumulate, float* router_score_out,
                                 int* topk_i_out, float* topk_w_out, moe_b200_stream stream) {
    return forward_impl(h, layer, t, t_dtype, nullptr, 0, n_tokens, out, accumulate, router_score_out,
                        topk_i_out, topk_w_out, stream);
}

moe_b200_status moe_b200_forward_norm(moe_b200_handle h, int layer, const float* x, const void* rms_weight,
                                      int rms_weight_dtype, int n_tokens, float* out, int accumulate,
                                      float* router_score_out, int* topk_i_out, float* topk_w_out,
                                      moe_b200_stream stream) {
    if (!rms_weight)
        return fail(h, MOE_B200_ERR_INVALID, "null norm weight");
    return forward_impl(h, layer, x, MOE_B200_DTYPE_F32, rms_weight, rms_weight_dtype, n_tokens, out,
                        accumulate, router_score_out, topk_i_out, topk_w_out, stream);
}

moe_b200_status moe_b200_forward_host(moe_b200_handle h, int layer, const void* t_host, int t_dtype,
                                      int n_tokens, float* out_host, int* topk_i_host,
                                      float* topk_w_host) {
    moe_b200_status st = check_layer(h, layer);
    if (st)
        return st;
    if (n_tokens < 0 || n_tokens > h->cfg.max_tokens)
        return fail(h, MOE_B200_ERR_INVALID, "n_tokens outside [0, max_tokens]");
    if (n_tokens > 0 && (!t_host || !out_host))
        return fail(h, MOE_B200_ERR_INVALID, "null host pointer");
    CU_TRY(h, cudaSetDevice(h->cfg.device));
    const size_t H = h->cfg.hidden_dim, K = h->cfg.experts_per_token;
    const size_t esz = (t_dtype == MOE_B200_DTYPE_F32) ? 4 : 2;
    cudaStream_t s = h->own_stream;
    // The block is independent per token, and a row's result does not depend on which
    // rows share its tile (the K loop has a fixed order), so a large batch is cut into
    // token chunks whose host->device copy, compute and device->host copy overlap on
    // three streams: the copies (PCIe, the fp32 result above all) take longer than the
    // compute.  A chunk keeps >= 128 rows per expert (measured at 16384 tokens, 128 experts:
    // 5.97-6.38 ms per step with four chunks, 6.42-7.43 with two).
    // Not with expert parallelism: every call is collective there and the ranks' token
    // counts differ.
    int chunk = n_tokens;
    if (h->cfg.ep_size == 1) {
        const int min_chunk = std::max(2048, (int)((128 * (size_t)h->cfg.n_experts + K - 1) / K));
        if (n_tokens >= 2 * min_chunk) {
            const int n_chunks = std::min(8, n_tokens / min_chunk);
            chunk = ((n_tokens + n_chunks - 1) / n_chunks + 63) / 64 * 64;
        }
    }
    if (chunk >= n_tokens) {
        // one pass; with profiling armed the two copies are timed as stages of the call
        h->prof_call = (h->prof_next < h->prof_armed) ? h->prof_next++ : -1;
        h->prof_external = true;
        struct Release {
            moe_b200_handle h;
            ~Release() { h->prof_external = false; }
        } release{h};
        prof_mark(h, MOE_B200_STAGE_H2D, true, s);
        if (n_tokens > 0)
            CU_TRY(h, cudaMemcpyAsync(h->t_dev, t_host, (size_t)n_tokens * H * esz, cudaMemcpyHostToDevice, s));
        prof_mark(h, MOE_B200_STAGE_H2D, false, s);
        st = moe_b200_forward(h, layer, h->t_dev, t_dtype, n_tokens, h->out_dev, 0, nullptr, nullptr,
                              nullptr, reinterpret_cast<moe_b200_stream>(s));
        if (st)
            return st;
        prof_mark(h, MOE_B200_STAGE_D2H, true, s);
        if (n_tokens > 0) {
            CU_TRY(h, cudaMemcpyAsync(out_host, h->out_dev, (size_t)n_tokens * H * 4, cudaMemcpyDeviceToHost, s));
            if (topk_i_host)
                CU_TRY(h, cudaMemcpyAsync(topk_i_host, h->topk_i, (size_t)n_tokens * K * 4, cudaMemcpyDeviceToHost, s));
            if (topk_w_host)
                CU_TRY(h, cudaMemcpyAsync(topk_w_host, h->topk_w, (size_t)n_tokens * K * 4, cudaMemcpyDeviceToHost, s));
        }
        prof_mark(h, MOE_B200_STAGE_D2H, false, s);
        CU_TRY(h, cudaStreamSynchronize(s));
        return MOE_B200_OK;
    }
    const int n_chunks = (n_tokens + chunk - 1) / chunk;
    if (!h->in_stream) {
        CU_TRY(h, cudaStreamCreateWithFlags(&h->in_stream, cudaStreamNonBlocking));
        CU_TRY(h, cudaStreamCreateWithFlags(&h->out_stream, cudaStreamNonBlocking));
    }
    while ((int)h->host_ev.size() < 2 * n_chunks) {
        cudaEvent_t e;
        CU_TRY(h, cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        h->host_ev.push_back(e);
    }
    const char* t_src = static_cast<const char*>(t_host);
    char* t_dst = static_cast<char*>(h->t_dev);
    for (int c = 0; c < n_chunks; c++) {
        const size_t t0 = (size_t)c * chunk, n = std::min((size_t)chunk, (size_t)n_tokens - t0);
        CU_TRY(h, cudaMemcpyAsync(t_dst + t0 * H * esz, t_src + t0 * H * esz, n * H * esz,
                                  cudaMemcpyHostToDevice, h->in_stream));
        CU_TRY(h, cudaEventRecord(h->host_ev[2 * c], h->in_stream));
    }
    for (int c = 0; c < n_chunks; c++) {
        const size_t t0 = (size_t)c * chunk, n = std::min((size_t)chunk, (size_t)n_tokens - t0);
        CU_TRY(h, cudaStreamWaitEvent(s, h->host_ev[2 * c], 0));
        st = moe_b200_forward(h, layer, t_dst + t0 * H * esz, t_dtype, (int)n, h->out_dev + t0 * H, 0, nullptr,
                              nullptr, nullptr, reinterpret_cast<moe_b200_stream>(s));
        if (st)
            return st;
        // the routing side outputs live in the workspace the next chunk reuses: copy them here
        if (topk_i_host)
            CU_TRY(h, cudaMemcpyAsync(topk_i_host + t0 * K, h->topk_i, n * K * 4, cudaMemcpyDeviceToHost, s));
        if (topk_w_host)
            CU_TRY(h, cudaMemcpyAsync(topk_w_host + t0 * K, h->topk_w, n * K * 4, cudaMemcpyDeviceToHost, s));
        CU_TRY(h, cudaEventRecord(h->host_ev[2 * c + 1], s));
        CU_TRY(h, cudaStreamWaitEvent(h->out_stream, h->host_ev[2 * c + 1], 0));
        CU_TRY(h, cudaMemcpyAsync(out_host + t0 * H, h->out_dev + t0 * H, n * H * 4, cudaMemcpyDeviceToHost,
                                  h->out_stream));
    }
    CU_TRY(h, cudaStreamSynchronize(s));
    CU_TRY(h, cudaStreamSynchronize(h->out_stream));
    return MOE_B200_OK;
}

moe_b200_status moe_b200_ep_unique_id(char id_out[128]) {
    std::string err;
    moe_b200_status st = (moe_b200_status)ep::unique_id(id_out, err);
    if (st)
        g_create_error = err;
    return st;
}

moe_b200_status moe_b200_ep_peer_export(moe_b200_handle h, char* blob_out) {
    if (!h || !blob_out)
        return MOE_B200_ERR_INVALID;
    if (h->cfg.ep_size <= 1)
        return fail(h, MOE_B200_ERR_INVALID, "handle was created with ep_size == 1");
    CU_TRY(h, cudaSetDevice(h->cfg.device));
    return (moe_b200_status)ep::peer_export(h->ep, h->cfg, blob_out, h->err);
}

moe_b200_status moe_b200_ep_peer_enable(moe_b200_handle h, const char* all_blobs) {
    if (!h || !all_blobs)
        return MOE_B200_ERR_INVALID;
    if (h->cfg.ep_size <= 1)
        return fail(h, MOE_B200_ERR_INVALID, "handle was created with ep_size == 1");
    CU_TRY(h, cudaSetDevice(h->cfg.device));
    return (moe_b200_status)ep::peer_enable(h->ep, h->cfg, all_blobs, h->err);
}

moe_b200_status moe_b200_ep_init(moe_b200_handle h, const char id[128]) {
    if (!h || !id)
        return MOE_B200_ERR_INVALID;
    if (h->cfg.ep_size <= 1)
        return fail(h, MOE_B200_ERR_INVALID, "handle was created with ep_size == 1");
    CU_TRY(h, cudaSetDevice(h->cfg.device));
    moe_b200_status st = (moe_b200_status)ep::allocate_nccl(h->ep, h->cfg, h->allocs, h->device_bytes, h->err);
    if (st)
        return st;
    return (moe_b200_status)ep::init(h->ep, id, h->cfg.ep_size, h->cfg.ep_rank, h->err);
}

void moe_b200_ep_plan(int n_experts, int ep_size, int ep_rank, const int* cnt_all, int* send_cnt,
                      int* send_off, int* recv_cnt, int* recv_off) {
    ep::plan_exchange(n_experts, ep_size, ep_rank, cnt_all, send_cnt, send_off, recv_cnt, recv_off);
}

int moe_b200_ep_peer_sequence(moe_b200_handle h) { return h ? h->ep.seq : 0; }

moe_b200_status moe_b200_ep_peer_resync(moe_b200_handle h, int sequence) {
    if (!h)
        return MOE_B200_ERR_INVALID;
    if (!h->ep.peer_enabled)
        return fail(h, MOE_B200_ERR_INVALID, "the peer-memory exchange is not enabled on this handle");
    if (sequence < h->ep.seq)
        return fail(h, MOE_B200_ERR_INVALID, "the sequence number can only move forward");
    CU_TRY(h, cudaSetDevice(h->cfg.device));
    CU_TRY(h, cudaDeviceSynchronize());
    // finished-block counters of a call that was cut short start from zero again
    CU_TRY(h, cudaMemset(h->ep.tickets, 0, 2 * sizeof(int)));
    h->ep.seq = sequence;
    return MOE_B200_OK;
}

moe_b200_status moe_b200_request_queue_create(int n_requests, const int* const* prompt_tokens,
                                              const int* prompt_lens, int* const* output_tokens,
                                              int max_seq_len, moe_b200_request_queue* out) {
    if (!out)
        return fail(nullptr, MOE_B200_ERR_INVALID, "null argument");
    *out = nullptr;
    if (n_requests < 0 || max_seq_len <= 0 || (n_requests > 0 && (!prompt_tokens || !prompt_lens)))
        return fail(nullptr, MOE_B200_ERR_INVALID, "bad request queue arguments");
    for (int r = 0; r < n_requests; r++)
        if (prompt_lens[r] < 1 || !prompt_tokens[r])  // src/getp/run.cpp:505-508
            return fail(nullptr, MOE_B200_ERR_INVALID,
                        "request " + std::to_string(r) + " has no prompt token");
    moe_b200_request_queue q = new (std::nothrow) moe_b200_request_queue_s();
    if (!q)
        return fail(nullptr, MOE_B200_ERR_INVALID, "out of host memory");
    q->q.n_requests = n_requests;
    q->q.max_seq_len = max_seq_len;
    q->q.prompt_tokens = prompt_tokens;
    q->q.prompt_lens = prompt_lens;
    q->q.output_tokens = output_tokens;
    *out = q;
    return MOE_B200_OK;
}

void moe_b200_request_queue_destroy(moe_b200_request_queue q) { delete q; }

moe_b200_status moe_b200_batcher_create(moe_b200_request_queue q, int n_slots, int continuous,
                                        moe_b200_batcher* out) {
    if (!q || !out || n_slots <= 0)
        return fail(nullptr, MOE_B200_ERR_INVALID, "bad batcher arguments");
    moe_b200_batcher b = new (std::nothrow) moe_b200_batcher_s();
    if (!b)
        return fail(nullptr, MOE_B200_ERR_INVALID, "out of host memory");
    b->b.q = &q->q;
    b->b.n_slots = n_slots;
    b->b.continuous = continuous != 0;
    b->b.slots.assign(n_slots, moe::sched::Slot());
    b->b.row_slot.reserve(n_slots);
    *out = b;
    return MOE_B200_OK;
}

void moe_b200_batcher_destroy(moe_b200_batcher b) { delete b; }

int moe_b200_batcher_begin_step(moe_b200_batcher b, int* tokens, int* positions, int* slots,
                                int* needs_sample) {
    if (!b || !tokens || !positions || !slots || b->b.step_open)
        return -1;
    return moe::sched::begin_step(b->b, tokens, positions, slots, needs_sample);
}

moe_b200_status moe_b200_batcher_end_step(moe_b200_batcher b, const int* sampled) {
    if (!b || !sampled || !b->b.step_open)
        return fail(nullptr, MOE_B200_ERR_INVALID, "end_step without a step in flight");
    moe::sched::end_step(b->b, sampled);
    return MOE_B200_OK;
}

void moe_b200_batcher_stats(moe_b200_batcher b, long long* steps, long long* rows, long long* tokens_out) {
    if (!b)
        return;
    if (steps)
        *steps = b->b.steps;
    if (rows)
        *rows = b->b.rows;
    if (tokens_out)
        *tokens_out = b->b.tokens_out;
}

size_t moe_b200_device_bytes(moe_b200_handle h) { return h ? h->device_bytes : 0; }

const char* moe_b200_last_error(moe_b200_handle h) {
    return h ? h->err.c_str() : g_create_error.c_str();
}

moe_b200_status moe_b200_device_status(moe_b200_handle h, int* status_word) {
    if (!h || !status_word)
        return MOE_B200_ERR_INVALID;
    CU_TRY(h, cudaSetDevice(h->cfg.device));
    CU_TRY(h, cudaDeviceSynchronize());
    CU_TRY(h, cudaMemcpy(status_word, h->status, sizeof(int), cudaMemcpyDeviceToHost));
    if (*status_word != 0)  // read and clear: the next report starts from a clean word
        CU_TRY(h, cudaMemset(h->status, 0, sizeof(int)));
    if (*status_word != 0)
        return fail(h, MOE_B200_ERR_DEVICE,
                    "device status word = 0x" + [&] {
                        char b[16];
                        snprintf(b, sizeof b, "%x", *status_word);
                        return std::string(b);
                    }());
    return MOE_B200_OK;
}

moe_b200_status moe_b200_profile(moe_b200_handle h, int n_calls) {
    if (!h || n_calls < 0 || n_calls > 4096)
        return fail(h, MOE_B200_ERR_INVALID, "n_calls must be in 0..4096");
    CU_TRY(h, cudaSetDevice(h->cfg.device));
    const size_t need = (size_t)n_calls * MOE_B200_N_STAGES * 2;
    while (h->prof_ev.size() < need) {
        cudaEvent_t e;
        CU_TRY(h, cudaEventCreate(&e));
        h->prof_ev.push_back(e);
    }
    h->prof_armed = n_calls;
    h->prof_next = 0;
    h->prof_call = -1;
    return MOE_B200_OK;
}

moe_b200_status moe_b200_profile_read(moe_b200_handle h, int call, float* ms) {
    if (!h || !ms || call < 0 || call >= h->prof_next)
        return fail(h, MOE_B200_ERR_INVALID, "no profiled forward with this index");
    for (int s = 0; s < MOE_B200_N_STAGES; s++) {
        const size_t i = ((size_t)call * MOE_B200_N_STAGES + s) * 2;
        float v = 0.f;
        if (cudaEventElapsedTime(&v, h->prof_ev[i], h->prof_ev[i + 1]) != cudaSuccess) {
            cudaGetLastError();  // stage did not run in that call
            v = 0.f;
        }
        ms[s] = v;
    }
    return MOE_B200_OK;
}

int moe_b200_last_launch_count(moe_b200_handle h) { return h ? h->last_launches : 0; }

moe_b200_status moe_b200_last_expert_counts(moe_b200_handle h, int* counts) {
    if (!h || !counts)
        return MOE_B200_ERR_INVALID;
    CU_TRY(h, cudaSetDevice(h->cfg.device));
    CU_TRY(h, cudaDeviceSynchronize());
    const int* src = (h->cfg.ep_size > 1) ? h->ep.g_cnt : h->cnt;
    CU_TRY(h, cudaMemcpy(counts, src, (size_t)h->n_local * sizeof(int), cudaMemcpyDeviceToHost));
    return MOE_B200_OK;
}

moe_b200_status moe_b200_mxfp4_unpack(const uint8_t* blocks, const uint8_t* scales, long long rows,
                                      int G, uint16_t* out_bf16, moe_b200_stream stream) {
    if (!blocks || !scales || !out_bf16 || rows < 0 || G <= 0)
        return fail(nullptr, MOE_B200_ERR_INVALID, "bad argument to moe_b200_mxfp4_unpack");
    const long long n_blocks = rows * G;
    if (n_blocks == 0)
        return MOE_B200_OK;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
        cudaGetLastError();
        return fail(nullptr, MOE_B200_ERR_NO_DEVICE, "no CUDA device; this library has no CPU path");
    }
    long long want = (n_blocks + 255) / 256;
    int grid = (int)(want < (long long)sms * 8 ? want : (long long)sms * 8);
    mxfp4_unpack_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(blocks, scales,
                                                                                   n_blocks, out_bf16);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
        return fail(nullptr, MOE_B200_ERR_CUDA, cudaGetErrorString(e));
    return MOE_B200_OK;
}

moe_b200_status moe_b200_last_intermediate(moe_b200_handle h, int n_tokens, uint16_t* out_bf16,
                                           moe_b200_stream stream) {
    if (!h || !out_bf16 || n_tokens < 0 || n_tokens > h->cfg.max_tokens)
        return fail(h, MOE_B200_ERR_INVALID, "bad argument to moe_b200_last_intermediate");
    if (h->cfg.ep_size != 1)
        return fail(h, MOE_B200_ERR_UNSUPPORTED, "only available with ep_size == 1");
    const int rows = n_tokens * h->cfg.experts_per_token;
    if (rows == 0)
        return MOE_B200_OK;
    CU_TRY(h, cudaSetDevice(h->cfg.device));
    int blocks = (rows + 7) / 8;
    ep::regroup_rows_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        h->hbuf, h->slot_of, rows, h->cfg.intermediate_dim, out_bf16);
    CU_TRY(h, cudaGetLastError());
    return MOE_B200_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// moe_b200_route_noalloc: the routing kernels with their scratch in the library
// image instead of a handle's workspace.

namespace {

constexpr int NA_MAX_BLOCKS = MOE_B200_ROUTE_NOALLOC_MAX_TOKENS / 16;  // routing blocks of 16 tokens
constexpr int NA_HIST_INTS = NA_MAX_BLOCKS * MOE_B200_ROUTE_NOALLOC_MAX_EXPERTS;
constexpr int NA_SCRATCH_INTS = 2 * NA_HIST_INTS + MOE_B200_ROUTE_NOALLOC_MAX_EXPERTS + 1;
constexpr int NA_MAX_DEVICES = MAX_DEVICES;

// [0, NA_HIST_INTS)              per-block expert histograms (router kernel -> plan kernel)
// [NA_HIST_INTS, 2*NA_HIST_INTS) per-block row bases (written by the plan kernel, unused here)
// [2*NA_HIST_INTS, ...)          tile table of the plan kernel (unused here)
// About 0.26 MB per GPU.  In host code this name is only a stand-in for the
// symbol, not a device address: kernels get the pointer cudaGetSymbolAddress
// returns for the current device.
static __device__ __align__(256) int g_route_noalloc_scratch[NA_SCRATCH_INTS];

int* g_na_scratch_ptr[NA_MAX_DEVICES];  // per device, filled by the first call there

}  // namespace

extern "C" {

moe_b200_status moe_b200_route_noalloc(const void* t, int t_dtype, int n_tokens, int hidden_dim,
                                       const void* w_router_bf16, const float* b_router,
                                       int n_experts, int experts_per_token, int* topk_i_out,
                                       float* topk_w_out, int* expert_counts_out,
                                       int* expert_offsets_out, moe_b200_stream stream) {
    if (!t || !w_router_bf16 || !b_router || !topk_i_out || !topk_w_out || !expert_counts_out ||
        !expert_offsets_out)
        return fail(nullptr, MOE_B200_ERR_INVALID, "moe_b200_route_noalloc: null pointer");
    if (t_dtype != MOE_B200_DTYPE_F32 && t_dtype != MOE_B200_DTYPE_BF16)
        return fail(nullptr, MOE_B200_ERR_INVALID, "moe_b200_route_noalloc: unknown activation dtype");
    if (((reinterpret_cast<uintptr_t>(t) | reinterpret_cast<uintptr_t>(w_router_bf16)) & 15u) != 0)
        return fail(nullptr, MOE_B200_ERR_INVALID,
                    "moe_b200_route_noalloc: activation and router pointers must be 16-byte aligned");
    if (n_tokens <= 0 || n_tokens > MOE_B200_ROUTE_NOALLOC_MAX_TOKENS)
        return fail(nullptr, MOE_B200_ERR_INVALID,
                    "moe_b200_route_noalloc: n_tokens must be in 1.." +
                        std::to_string(MOE_B200_ROUTE_NOALLOC_MAX_TOKENS) +
                        " (the scratch array is fixed-size; use a handle for larger batches)");
    if (n_experts <= 0 || n_experts > MOE_B200_ROUTE_NOALLOC_MAX_EXPERTS)
        return fail(nullptr, MOE_B200_ERR_INVALID,
                    "moe_b200_route_noalloc: n_experts must be in 1.." +
                        std::to_string(MOE_B200_ROUTE_NOALLOC_MAX_EXPERTS));
    if (hidden_dim <= 0 || hidden_dim % 64 || hidden_dim > MOE_B200_ROUTE_NOALLOC_MAX_HIDDEN)
        return fail(nullptr, MOE_B200_ERR_INVALID,
                    "moe_b200_route_noalloc: hidden_dim must be a multiple of 64 up to " +
                        std::to_string(MOE_B200_ROUTE_NOALLOC_MAX_HIDDEN));
    if (experts_per_token <= 0 || experts_per_token > 8 || experts_per_token > n_experts)
        return fail(nullptr, MOE_B200_ERR_INVALID, "moe_b200_route_noalloc: K must be in 1..min(8, n_experts)");
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        cudaGetLastError();
        return fail(nullptr, MOE_B200_ERR_NO_DEVICE, "no CUDA device; this library has no CPU path");
    }
    if (dev < 0 || dev >= NA_MAX_DEVICES)
        return fail(nullptr, MOE_B200_ERR_INVALID, "moe_b200_route_noalloc: device ordinal too large");
    if (!g_na_scratch_ptr[dev]) {
        // set-up, once per device, with that device current: the symbol's address there
        int* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_route_noalloc_scratch);
        if (e != cudaSuccess || !p) {
            cudaGetLastError();
            return fail(nullptr, e == cudaErrorNoDevice ? MOE_B200_ERR_NO_DEVICE : MOE_B200_ERR_CUDA,
                        std::string("cudaGetSymbolAddress(route scratch): ") + cudaGetErrorString(e));
        }
        g_na_scratch_ptr[dev] = p;
    }
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    int* scratch = g_na_scratch_ptr[dev];
    int* blk_hist = scratch;
    int* blk_base = scratch + NA_HIST_INTS;
    int* tile_start = scratch + 2 * NA_HIST_INTS;
    const int rb = 16;  // NA_MAX_BLOCKS is sized for it
    const int nblk = ceil_div(n_tokens, rb);
    RouteArgs ra{t, t_dtype == MOE_B200_DTYPE_F32, n_tokens, hidden_dim,
                 static_cast<const uint16_t*>(w_router_bf16), b_router, n_experts, experts_per_token,
                 nullptr, topk_i_out, topk_w_out, blk_hist, false, 0};
    CU_TRY(nullptr, launch_route(dev, ra, rb, st));
    plan_kernel<<<1, 256, 0, st>>>(blk_hist, nblk, n_experts, 1, expert_counts_out, expert_offsets_out,
                                   tile_start, blk_base);
    CU_TRY(nullptr, cudaGetLastError());
    return MOE_B200_OK;
}

moe_b200_status moe_b200_unpack_resident(moe_b200_handle h, int layer, int local_expert, int which,
                                         uint16_t* out_bf16, moe_b200_stream stream) {
    moe_b200_status st = check_layer(h, layer);
    if (st)
        return st;
    if (local_expert < 0 || local_expert >= h->n_local || (which != 1 && which != 2) || !out_bf16)
        return fail(h, MOE_B200_ERR_INVALID, "bad argument to moe_b200_unpack_resident");
    LayerWeights& lw = h->layers[layer];
    if (!lw.expert_set[local_expert])
        return fail(h, MOE_B200_ERR_NOT_LOADED, "expert was not set");
    CU_TRY(h, cudaSetDevice(h->cfg.device));
    const int H = h->cfg.hidden_dim, I = h->cfg.intermediate_dim;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    if (which == 1)
        mxfp4_unpack_resident_kernel<<<dim3(h->ks1, h->m_tiles1), TILE_M, 0, s>>>(
            lw.w1 + local_expert * h->stride1, lw.rscale1 + (size_t)local_expert * 2 * I, 2 * I, H, out_bf16);
    else
        mxfp4_unpack_resident_kernel<<<dim3(h->ks2, h->m_tiles2), TILE_M, 0, s>>>(
            lw.w2 + local_expert * h->stride2, lw.rscale2 + (size_t)local_expert * H, H, I, out_bf16);
    CU_TRY(h, cudaGetLastError());
    return MOE_B200_OK;
}

}  // extern "C"

#if defined(MOE_B200_TEST_AIDS) && defined(TC5_TRACE)
// Debug builds only (not declared in the header): reads the hand-off timestamps.
extern "C" int moe_b200_debug_trace_read(long long* out, int n) {
    cudaDeviceSynchronize();
    const size_t bytes = sizeof(long long) * (size_t)n;
    return (int)cudaMemcpyFromSymbol(out, moe::tc5::g_trace, bytes);
}
#endif
