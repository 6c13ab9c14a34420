// Router GEMM + bias, top-k, softmax over the selected logits, and the
// per-block expert histogram -- one kernel.
//
// Replaces gemm_router (src/hip/gemms/gemm_router.hip:7-190), topk_kernel
// (src/hip/topk.hip:5-57), softmax_kernel (src/hip/softmax.hip:5-44) and the
// histogram half of count_tokens_per_expert (src/hip/scheduler.hip:11-31).
//
// Numerics.  The expert indices must equal those of the CPU engine, which sums
// float products in a double (src/run.cpp:341-354), for every token whose
// top-(K+1) logits are not within 1e-6 of each other.  Activations and router
// weights are bf16, so each product is exact in fp32; the sum is formed as
// fp32 FMA chains of RKC terms whose results are added in double and rounded
// to fp32 once, then the fp32 bias is added (src/run.cpp:635-637).  The error
// left is a few 1e-8, far inside the tie window.  Ties go to the lower expert
// index (src/hip/topk.hip:30-49).
#pragma once
#include "common.cuh"

namespace moe {

constexpr int RB = 64;         // tokens per routing block
constexpr int RKC = 32;        // K chunk
constexpr int RLD = RKC + 4;   // padded row length in floats (conflict-free float4 reads)
constexpr int RTHREADS = 256;

template <int NT>
constexpr size_t route_smem_bytes() {
    size_t gemm = (size_t)(RB + NT * 32) * RLD * sizeof(float);
    size_t logits = (size_t)RB * (NT * 32) * sizeof(float);
    return (gemm > logits ? gemm : logits) + 256 * sizeof(int);
}

__device__ __forceinline__ void load8_as_bf16_floats(const void* base, size_t elem_off, bool f32,
                                                     bool valid, float out[8]) {
    if (!valid) {
#pragma unroll
        for (int i = 0; i < 8; i++)
            out[i] = 0.f;
        return;
    }
    if (f32) {
        const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(base) + elem_off);
        float4 a = p[0], b = p[1];
        float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 8; i++)
            out[i] = bf16_bits_to_float(float_to_bf16_bits(v[i]));
    } else {
        uint4 q = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(base) + elem_off);
        uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            out[2 * i] = __uint_as_float(w[i] << 16);
            out[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
        }
    }
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

// NT = number of 32-expert tiles (E <= 32*NT).
template <int NT>
__global__ void __launch_bounds__(RTHREADS)
route_kernel(const void* __restrict__ x, int x_is_f32, int T, int H,
             const uint16_t* __restrict__ w_router, const float* __restrict__ b_router, int E, int K,
             float* __restrict__ score_out, int* __restrict__ topk_i, float* __restrict__ topk_w,
             int* __restrict__ blk_hist) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* xs = reinterpret_cast<float*>(smem_raw);  // [RB][RLD]
    float* ws = xs + RB * RLD;                       // [NT*32][RLD]
    float* lg = reinterpret_cast<float*>(smem_raw);  // [RB][NT*32], reuses xs/ws after the GEMM
    constexpr size_t gemm_b = (size_t)(RB + NT * 32) * RLD * sizeof(float);
    constexpr size_t lg_b = (size_t)RB * (NT * 32) * sizeof(float);
    int* hist = reinterpret_cast<int*>(smem_raw + (gemm_b > lg_b ? gemm_b : lg_b));

    const int tid = threadIdx.x;
    const int t0 = blockIdx.x * RB;
    const int tp = tid >> 3, eq = tid & 7;
    const bool f32 = x_is_f32 != 0;

    for (int i = tid; i < 256; i += RTHREADS)
        hist[i] = 0;

    float acc[2][NT * 4];
    double tot[2][NT * 4];
#pragma unroll
    for (int a = 0; a < 2; a++)
#pragma unroll
        for (int j = 0; j < NT * 4; j++) {
            acc[a][j] = 0.f;
            tot[a][j] = 0.0;
        }

    // staging registers for the next chunk
    constexpr int WSEG = (NT * 128 + RTHREADS - 1) / RTHREADS;  // 16-byte w segments per thread
    float xr[8];
    float wr[WSEG][8];
    const int xrow = tid >> 2, xseg = tid & 3;
    auto fetch = [&](int k0) {
        load8_as_bf16_floats(x, (size_t)(t0 + xrow) * H + k0 + xseg * 8, f32, (t0 + xrow) < T, xr);
#pragma unroll
        for (int s = 0; s < WSEG; s++) {
            int seg = tid + s * RTHREADS;
            int row = seg >> 2, sg = seg & 3;
            bool ok = (seg < NT * 128) && (row < E);
            load8_as_bf16_floats(w_router, (size_t)row * H + k0 + sg * 8, false, ok, wr[s]);
        }
    };
    auto stash = [&]() {
        float4* xd = reinterpret_cast<float4*>(xs + xrow * RLD + xseg * 8);
        xd[0] = make_float4(xr[0], xr[1], xr[2], xr[3]);
        xd[1] = make_float4(xr[4], xr[5], xr[6], xr[7]);
#pragma unroll
        for (int s = 0; s < WSEG; s++) {
            int seg = tid + s * RTHREADS;
            if (seg < NT * 128) {
                int row = seg >> 2, sg = seg & 3;
                float4* wd = reinterpret_cast<float4*>(ws + row * RLD + sg * 8);
                wd[0] = make_float4(wr[s][0], wr[s][1], wr[s][2], wr[s][3]);
                wd[1] = make_float4(wr[s][4], wr[s][5], wr[s][6], wr[s][7]);
            }
        }
    };

    const int n_chunks = H / RKC;
    fetch(0);
    for (int c = 0; c < n_chunks; c++) {
        __syncthreads();  // previous chunk's reads done
        stash();
        __syncthreads();
        if (c + 1 < n_chunks)
            fetch((c + 1) * RKC);
#pragma unroll
        for (int k4 = 0; k4 < RKC / 4; k4++) {
            const float4 xa = *reinterpret_cast<const float4*>(xs + (2 * tp) * RLD + k4 * 4);
            const float4 xb = *reinterpret_cast<const float4*>(xs + (2 * tp + 1) * RLD + k4 * 4);
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float4 wv =
                        *reinterpret_cast<const float4*>(ws + (nt * 32 + eq + 8 * j) * RLD + k4 * 4);
                    float a0 = acc[0][nt * 4 + j], a1 = acc[1][nt * 4 + j];
                    a0 = fmaf(xa.x, wv.x, a0);
                    a0 = fmaf(xa.y, wv.y, a0);
                    a0 = fmaf(xa.z, wv.z, a0);
                    a0 = fmaf(xa.w, wv.w, a0);
                    a1 = fmaf(xb.x, wv.x, a1);
                    a1 = fmaf(xb.y, wv.y, a1);
                    a1 = fmaf(xb.z, wv.z, a1);
                    a1 = fmaf(xb.w, wv.w, a1);
                    acc[0][nt * 4 + j] = a0;
                    acc[1][nt * 4 + j] = a1;
                }
        }
#pragma unroll
        for (int a = 0; a < 2; a++)
#pragma unroll
            for (int j = 0; j < NT * 4; j++) {
                tot[a][j] += (double)acc[a][j];
                acc[a][j] = 0.f;
            }
    }
    __syncthreads();  // xs/ws dead; lg aliases them

    constexpr int EP = NT * 32;
#pragma unroll
    for (int a = 0; a < 2; a++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int e = nt * 32 + eq + 8 * j;
                float s = (float)tot[a][nt * 4 + j];
                s += (e < E) ? b_router[e] : 0.f;
                lg[(2 * tp + a) * EP + e] = (e < E) ? s : -INFINITY;
            }
    __syncthreads();

    if (score_out) {
        for (int i = tid; i < RB * E; i += RTHREADS) {
            int r = i / E, e = i - r * E;
            if (t0 + r < T)
                score_out[(size_t)(t0 + r) * E + e] = lg[r * EP + e];
        }
    }

    // top-K + softmax: one warp per token, RB/8 tokens per warp
    const int warp = tid >> 5, lane = tid & 31;
    for (int r = warp; r < RB; r += RTHREADS / 32) {
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

// ---------------------------------------------------------------------------
// Small-batch variant: RBS tokens per block, one warp per token, so that a
// decode-sized batch (a few hundred tokens) still fills the GPU.  The token rows
// and eight router rows at a time sit in shared memory as bf16; every lane owns
// the 16-byte vectors lane, lane+32, ... of the K axis and keeps eight fp32
// partial sums (chains of H/32 exact products), which a shuffle tree adds.
constexpr int RBS = 8;     // tokens (= warps) per block
constexpr int RGE = 8;     // experts staged per pass

inline size_t route_small_smem_bytes(int H) { return (size_t)(RBS + RGE) * H * 2 + 256 * sizeof(int); }

template <int NT>
__global__ void __launch_bounds__(RBS * 32)
route_small_kernel(const void* __restrict__ x, int x_is_f32, int T, int H,
                   const uint16_t* __restrict__ w_router, const float* __restrict__ b_router, int E,
                   int K, float* __restrict__ score_out, int* __restrict__ topk_i,
                   float* __restrict__ topk_w, int* __restrict__ blk_hist) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint16_t* xs = reinterpret_cast<uint16_t*>(smem_raw);  // [RBS][H]
    uint16_t* ws = xs + (size_t)RBS * H;                   // [RGE][H]
    int* hist = reinterpret_cast<int*>(ws + (size_t)RGE * H);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int t0 = blockIdx.x * RBS;
    const int vec = H / 8;
    for (int i = tid; i < 256; i += RBS * 32)
        hist[i] = 0;
    // stage the block's token rows as bf16
    for (int i = tid; i < RBS * vec; i += RBS * 32) {
        const int r = i / vec, v = i - r * vec;
        uint4 q = make_uint4(0, 0, 0, 0);
        if (t0 + r < T) {
            if (x_is_f32) {
                const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(x) +
                                                                  (size_t)(t0 + r) * H) + 2 * v;
                const float4 a = p[0], b = p[1];
                q = make_uint4(pack_bf16x2(a.x, a.y), pack_bf16x2(a.z, a.w), pack_bf16x2(b.x, b.y),
                               pack_bf16x2(b.z, b.w));
            } else {
                q = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(x) + (size_t)(t0 + r) * H)[v];
            }
        }
        reinterpret_cast<uint4*>(xs + (size_t)r * H)[v] = q;
    }
    float logit[NT];
#pragma unroll
    for (int j = 0; j < NT; j++)
        logit[j] = -INFINITY;
    const int t = t0 + warp;
    for (int e0 = 0; e0 < E; e0 += RGE) {
        __syncthreads();  // previous group consumed (first pass: xs staged)
        for (int i = tid; i < RGE * vec; i += RBS * 32) {
            const int r = i / vec, v = i - r * vec;
            uint4 q = make_uint4(0, 0, 0, 0);
            if (e0 + r < E)
                q = reinterpret_cast<const uint4*>(w_router + (size_t)(e0 + r) * H)[v];
            reinterpret_cast<uint4*>(ws + (size_t)r * H)[v] = q;
        }
        __syncthreads();
        float acc[RGE];
#pragma unroll
        for (int g = 0; g < RGE; g++)
            acc[g] = 0.f;
        for (int v = lane; v < vec; v += 32) {
            const uint4 xq = reinterpret_cast<const uint4*>(xs + (size_t)warp * H)[v];
            const uint32_t xw[4] = {xq.x, xq.y, xq.z, xq.w};
            float xf[8];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                xf[2 * i] = __uint_as_float(xw[i] << 16);
                xf[2 * i + 1] = __uint_as_float(xw[i] & 0xFFFF0000u);
            }
#pragma unroll
            for (int g = 0; g < RGE; g++) {
                const uint4 wq = reinterpret_cast<const uint4*>(ws + (size_t)g * H)[v];
                const uint32_t ww[4] = {wq.x, wq.y, wq.z, wq.w};
                float a = acc[g];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    a = fmaf(xf[2 * i], __uint_as_float(ww[i] << 16), a);
                    a = fmaf(xf[2 * i + 1], __uint_as_float(ww[i] & 0xFFFF0000u), a);
                }
                acc[g] = a;
            }
        }
#pragma unroll
        for (int g = 0; g < RGE; g++) {
            float a = acc[g];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1)
                a += __shfl_xor_sync(0xffffffffu, a, off);
            const int e = e0 + g;
            if (e < E && (e & 31) == lane) {
                const float sc = a + b_router[e];
#pragma unroll
                for (int j = 0; j < NT; j++)
                    if (j == (e >> 5))
                        logit[j] = sc;
            }
        }
    }
    if (t < T) {
        if (score_out) {
#pragma unroll
            for (int j = 0; j < NT; j++)
                if (lane + 32 * j < E)
                    score_out[(size_t)t * E + lane + 32 * j] = logit[j];
        }
        select_topk_softmax<NT>(logit, lane, K, t, topk_i, topk_w, hist);
    }
    __syncthreads();
    for (int e = tid; e < E; e += RBS * 32)
        blk_hist[(size_t)blockIdx.x * E + e] = hist[e];
}

// ---------------------------------------------------------------------------
// Large-batch variant on the warp-level tensor-core path (mma.sync bf16, fp32
// accumulate): the router is 0.4 % of the block's FLOPs but at 16k tokens x 128
// experts it is 6 GFMA, too much for the fp32 pipes.
//
// Exactness of the expert indices: products of bf16 values are exact; what
// differs from the CPU engine's double sum is the accumulation.  The tensor core
// sums one K chunk of RMK = 64 terms into a fresh accumulator; the chunk results
// are added to a running fp32 sum with round-to-nearest adds on the CUDA cores,
// so no long accumulation happens inside the tensor core.  The index test
// against the oracle (ties within 1e-6 excluded) is what admits this kernel.
constexpr int RMK = 64;          // K chunk
constexpr int RMLD = RMK + 8;    // bf16 per smem row: conflict-free fragment loads

__device__ __forceinline__ void route_mma_16816(float c[4], const uint32_t a[4], const uint32_t b[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

template <int NT>
__global__ void __launch_bounds__(RTHREADS)
route_mma_kernel(const void* __restrict__ x, int x_is_f32, int T, int H,
                 const uint16_t* __restrict__ w_router, const float* __restrict__ b_router, int E,
                 int K, float* __restrict__ score_out, int* __restrict__ topk_i,
                 float* __restrict__ topk_w, int* __restrict__ blk_hist) {
    constexpr int EP = NT * 32;      // padded expert count
    constexpr int NTW = NT * 2;      // n8 tiles per warp (half of the experts)
    constexpr size_t tiles_b = (size_t)(RB + EP) * RMLD * 2;
    constexpr size_t lg_b = (size_t)RB * EP * 4;
    __shared__ __align__(16) unsigned char smem_raw[(tiles_b > lg_b ? tiles_b : lg_b)];
    __shared__ int hist[256];
    uint16_t* xs = reinterpret_cast<uint16_t*>(smem_raw);  // [RB][RMLD]
    uint16_t* ws = xs + RB * RMLD;                         // [EP][RMLD]
    float* lg = reinterpret_cast<float*>(smem_raw);        // [RB][EP] after the GEMM

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t4 = lane & 3;
    const int mb = warp & 3, nh = warp >> 2;
    const int t0 = blockIdx.x * RB;
    for (int i = tid; i < 256; i += RTHREADS)
        hist[i] = 0;

    float run[NTW][4];
#pragma unroll
    for (int n = 0; n < NTW; n++)
#pragma unroll
        for (int i = 0; i < 4; i++)
            run[n][i] = 0.f;

    // staging registers: 16-byte segments of the next chunk
    constexpr int XSEG = RB * 8 / RTHREADS;  // 2
    constexpr int WSEG = EP * 8 / RTHREADS;  // NT
    uint4 xr[XSEG], wr[WSEG];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int s = 0; s < XSEG; s++) {
            const int seg = tid + s * RTHREADS, row = seg >> 3, sg = seg & 7;
            uint4 q = make_uint4(0, 0, 0, 0);
            if (t0 + row < T) {
                if (x_is_f32) {
                    const float4* p = reinterpret_cast<const float4*>(
                        static_cast<const float*>(x) + (size_t)(t0 + row) * H + k0 + sg * 8);
                    const float4 a = p[0], b = p[1];
                    q = make_uint4(pack_bf16x2(a.x, a.y), pack_bf16x2(a.z, a.w), pack_bf16x2(b.x, b.y),
                                   pack_bf16x2(b.z, b.w));
                } else {
                    q = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(x) +
                                                        (size_t)(t0 + row) * H + k0 + sg * 8);
                }
            }
            xr[s] = q;
        }
#pragma unroll
        for (int s = 0; s < WSEG; s++) {
            const int seg = tid + s * RTHREADS, row = seg >> 3, sg = seg & 7;
            wr[s] = (row < E) ? *reinterpret_cast<const uint4*>(w_router + (size_t)row * H + k0 + sg * 8)
                              : make_uint4(0, 0, 0, 0);
        }
    };
    auto stash = [&]() {
#pragma unroll
        for (int s = 0; s < XSEG; s++) {
            const int seg = tid + s * RTHREADS, row = seg >> 3, sg = seg & 7;
            *reinterpret_cast<uint4*>(xs + row * RMLD + sg * 8) = xr[s];
        }
#pragma unroll
        for (int s = 0; s < WSEG; s++) {
            const int seg = tid + s * RTHREADS, row = seg >> 3, sg = seg & 7;
            *reinterpret_cast<uint4*>(ws + row * RMLD + sg * 8) = wr[s];
        }
    };

    const int n_chunks = H / RMK;  // H is a multiple of 64
    fetch(0);
    for (int c = 0; c < n_chunks; c++) {
        __syncthreads();
        stash();
        __syncthreads();
        if (c + 1 < n_chunks)
            fetch((c + 1) * RMK);
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
                const uint16_t* pb = ws + (nh * (EP / 2) + n * 8 + g) * RMLD + kk * 16 + 2 * t4;
                uint32_t bf[2];
                bf[0] = *reinterpret_cast<const uint32_t*>(pb);
                bf[1] = *reinterpret_cast<const uint32_t*>(pb + 8);
                route_mma_16816(acc[n], af, bf);
            }
        }
#pragma unroll
        for (int n = 0; n < NTW; n++)
#pragma unroll
            for (int i = 0; i < 4; i++)
                run[n][i] += acc[n][i];
    }
    __syncthreads();  // tiles dead; lg aliases them
#pragma unroll
    for (int n = 0; n < NTW; n++)
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int row = mb * 16 + g + 8 * (i >> 1);
            const int e = nh * (EP / 2) + n * 8 + 2 * t4 + (i & 1);
            lg[row * EP + e] = (e < E) ? run[n][i] + b_router[e] : -INFINITY;
        }
    __syncthreads();
    if (score_out) {
        for (int i = tid; i < RB * E; i += RTHREADS) {
            const int r = i / E, e = i - r * E;
            if (t0 + r < T)
                score_out[(size_t)(t0 + r) * E + e] = lg[r * EP + e];
        }
    }
    for (int r = warp; r < RB; r += RTHREADS / 32) {
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
