// Grouped expert GEMMs on warp-level mma.sync -- the CROSS-CHECK implementation.
//
// Same inputs, outputs, weight layout and rounding points as the tcgen05
// kernels (gemm_tc5_pair.cuh, gemm_tc5_ts.cuh), written as plainly as possible
// (single-buffered, no TMA, no tensor memory) so that the two can be compared on
// the device at sizes where the CPU oracle is too slow.  Compiled only into the
// test-aids build of the library (-DMOE_B200_TEST_AIDS), where
// moe_b200_config.gemm_impl = MOE_B200_GEMM_MMA_SYNC selects it; the shipped
// library has the tcgen05 kernels only.
//
// MODE 0: gate/up projection + bias + clamped SwiGLU -> h bf16 [rows, I]
//         (moe_mlp1_swiglu, src/hip/moe.hip:9-258; SwiGLU src/run.cpp:673-689)
// MODE 1: down projection + bias -> y fp32 [rows, H]
//         (moe_mlp2_store, src/hip/moe.hip:538-800; the routing weight is
//         applied by the combine kernel)
#pragma once
#include "common.cuh"

namespace moe {

constexpr int V0_BN = 64;
constexpr int V0_LD = 72;  // bf16 per smem row: 36 words -> conflict-free fragment loads

__device__ __forceinline__ void mma_bf16_16816(float c[4], const uint32_t a[4], const uint32_t b[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// Locates the expert of n-tile `nt` in the prefix table tile_start[E+1].
__device__ __forceinline__ int find_expert(const int* __restrict__ tile_start, int E, int nt) {
    int lo = 0, hi = E;  // invariant: tile_start[lo] <= nt < tile_start[hi]
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (tile_start[mid] <= nt)
            lo = mid;
        else
            hi = mid;
    }
    return lo;
}

template <int MODE>
__global__ void __launch_bounds__(256)
expert_gemm_mma_kernel(const uint8_t* __restrict__ chunks, size_t expert_stride, int k_stages,
                       const float* __restrict__ bias, const float* __restrict__ rscale, int bias_stride,
                       const uint16_t* __restrict__ xin, int K, const int* __restrict__ g_off,
                       const int* __restrict__ g_cnt, const int* __restrict__ g_tile_start, int E,
                       void* __restrict__ outp, int out_ld, int out_rows_valid,
                       const int* __restrict__ row_dst, float alpha, float limit) {
    __shared__ __align__(16) uint16_t As[TILE_M * V0_LD];
    __shared__ __align__(16) uint16_t Bs[V0_BN * V0_LD];

    const int nt_global = blockIdx.x;
    if (nt_global >= g_tile_start[E])
        return;
    const int e = find_expert(g_tile_start, E, nt_global);
    const int n0 = (nt_global - g_tile_start[e]) * V0_BN;
    const int cnt = g_cnt[e];
    const int row0 = g_off[e] + n0;
    const int valid_n = min(V0_BN, cnt - n0);
    const int mt = blockIdx.y;
    const int m_tiles = gridDim.y;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int pi = warp & 3, nh = warp >> 2;

    float acc[2][4][4];
#pragma unroll
    for (int a = 0; a < 2; a++)
#pragma unroll
        for (int b = 0; b < 4; b++)
#pragma unroll
            for (int c = 0; c < 4; c++)
                acc[a][b][c] = 0.f;

    const uint8_t* wbase = chunks + (size_t)e * expert_stride + (size_t)mt * k_stages * CHUNK_BYTES;
    const int ar = tid >> 1, ab = tid & 1;
    const int a_srow = (MODE == 0) ? ((ar >> 1) + 64 * (ar & 1)) : ar;

    for (int ks = 0; ks < k_stages; ks++) {
        const uint8_t* chunk = wbase + (size_t)ks * CHUNK_BYTES;
        {
            const uint4 q = *reinterpret_cast<const uint4*>(chunk + ab * PLANE_BYTES + ar * 16);
            const uint32_t mult = mxfp4_scale_mult(chunk[2 * PLANE_BYTES + ar * 2 + ab]);
            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
            uint4* dst = reinterpret_cast<uint4*>(As + a_srow * V0_LD + ab * 32);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                uint32_t d[4];
                mxfp4_decode_word(w[j], mult, d);
                dst[j] = make_uint4(d[0], d[1], d[2], d[3]);
            }
        }
#pragma unroll
        for (int s = 0; s < 2; s++) {
            const int seg = tid + s * 256;
            const int row = seg >> 3, sg = seg & 7;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (row < valid_n)
                v = *reinterpret_cast<const uint4*>(xin + (size_t)(row0 + row) * K + ks * KSTAGE + sg * 8);
            *reinterpret_cast<uint4*>(Bs + row * V0_LD + sg * 8) = v;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 4; kk++) {
            uint32_t af[2][4];
#pragma unroll
            for (int a = 0; a < 2; a++) {
                const int rb = (pi + 4 * a) * 16;
                const uint16_t* p = As + (rb + g) * V0_LD + kk * 16 + 2 * t;
                af[a][0] = *reinterpret_cast<const uint32_t*>(p);
                af[a][1] = *reinterpret_cast<const uint32_t*>(p + 8 * V0_LD);
                af[a][2] = *reinterpret_cast<const uint32_t*>(p + 8);
                af[a][3] = *reinterpret_cast<const uint32_t*>(p + 8 * V0_LD + 8);
            }
#pragma unroll
            for (int nb = 0; nb < 4; nb++) {
                const uint16_t* p = Bs + (nh * 32 + nb * 8 + g) * V0_LD + kk * 16 + 2 * t;
                uint32_t bf[2];
                bf[0] = *reinterpret_cast<const uint32_t*>(p);
                bf[1] = *reinterpret_cast<const uint32_t*>(p + 8);
                mma_bf16_16816(acc[0][nb], af[0], bf);
                mma_bf16_16816(acc[1][nb], af[1], bf);
            }
        }
        __syncthreads();
    }

    const float* be = bias + (size_t)e * bias_stride;
    const float* rse = rscale + (size_t)e * bias_stride;
    if (MODE == 0) {
        // acc[0] = gate rows, acc[1] = matching up rows (smem rows p and 64+p)
        uint16_t* h = static_cast<uint16_t*>(outp);
#pragma unroll
        for (int half = 0; half < 2; half++) {
            const int p = pi * 16 + g + 8 * half;    // pair index inside the tile
            const int j = mt * (TILE_M / 2) + p;     // feature
            if (j >= out_rows_valid)
                continue;
            const float bg = be[mt * TILE_M + 2 * p], bu = be[mt * TILE_M + 2 * p + 1];
            const float sg = rse[mt * TILE_M + 2 * p], su = rse[mt * TILE_M + 2 * p + 1];
#pragma unroll
            for (int nb = 0; nb < 4; nb++)
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    const int col = nh * 32 + nb * 8 + 2 * t + c;
                    if (col < valid_n) {
                        const float v = swiglu(fmaf(acc[0][nb][2 * half + c], sg, bg),
                                               fmaf(acc[1][nb][2 * half + c], su, bu), alpha, limit);
                        h[(size_t)(row0 + col) * out_ld + j] = (uint16_t)float_to_bf16_bits(v);
                    }
                }
        }
    } else {
        float* y = static_cast<float*>(outp);
#pragma unroll
        for (int a = 0; a < 2; a++)
#pragma unroll
            for (int half = 0; half < 2; half++) {
                const int m = mt * TILE_M + (pi + 4 * a) * 16 + g + 8 * half;
                if (m >= out_rows_valid)
                    continue;
                const float bm = be[m], rs = rse[m];
#pragma unroll
                for (int nb = 0; nb < 4; nb++)
#pragma unroll
                    for (int c = 0; c < 2; c++) {
                        const int col = nh * 32 + nb * 8 + 2 * t + c;
                        if (col < valid_n) {
                            float* yrow = y + (size_t)(row_dst ? row_dst[row0 + col] : (row0 + col)) * out_ld;
                            yrow[m] = fmaf(acc[a][nb][2 * half + c], rs, bm);
                        }
                    }
            }
    }
    (void)m_tiles;
}

}  // namespace moe
