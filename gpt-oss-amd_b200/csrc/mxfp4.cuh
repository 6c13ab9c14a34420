// MXFP4 kernels outside the GEMMs: exact unpack of checkpoint-layout tensors,
// re-tiling into the resident layout at upload, and a decode of resident
// weights through the GEMM's own decode function (for bit-exactness tests).
#pragma once
#include "common.cuh"

namespace moe {

// blocks [rows, G, 16] u8, scales [rows, G] u8 -> out [rows, 32*G] bf16 bits.
// One thread per 16-byte block: 16 B in, 64 B out.  Pure HBM-bound byte work:
// 17 B read + 64 B written per block.
__global__ void mxfp4_unpack_kernel(const uint8_t* __restrict__ blocks,
                                    const uint8_t* __restrict__ scales, long long n_blocks,
                                    uint16_t* __restrict__ out) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < n_blocks; i += stride) {
        const uint4 q = *reinterpret_cast<const uint4*>(blocks + i * 16);
        const uint32_t sb = scales[i];
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
        uint4* o = reinterpret_cast<uint4*>(out + i * 32);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            uint32_t r[4];
#pragma unroll
            for (int p = 0; p < 4; p++) {
                uint32_t lo = mxfp4_decode_exact((w[j] >> (8 * p)) & 0xFu, sb);
                uint32_t hi = mxfp4_decode_exact((w[j] >> (8 * p + 4)) & 0xFu, sb);
                r[p] = lo | (hi << 16);
            }
            o[j] = make_uint4(r[0], r[1], r[2], r[3]);
        }
    }
}

// Checkpoint layout of ONE expert matrix -> resident chunks.
// grid (k_stages, m_tiles), block TILE_M threads (thread = row of the tile).
__global__ void mxfp4_retile_kernel(const uint8_t* __restrict__ blocks,
                                    const uint8_t* __restrict__ scales, int rows, int G,
                                    uint8_t* __restrict__ chunks, int* __restrict__ status) {
    const int ks = blockIdx.x, mt = blockIdx.y, r = threadIdx.x;
    const int row = mt * TILE_M + r;
    uint8_t* chunk = chunks + ((size_t)mt * gridDim.x + ks) * CHUNK_BYTES;
#pragma unroll
    for (int b = 0; b < 2; b++) {
        const int g = ks * 2 + b;
        uint4 q = make_uint4(0, 0, 0, 0);
        uint32_t sb = 127;
        if (row < rows && g < G) {
            q = *reinterpret_cast<const uint4*>(blocks + ((size_t)row * G + g) * 16);
            sb = scales[(size_t)row * G + g];
            if (sb > (uint32_t)MAX_SCALE_BYTE)
                report_status(status, DS_BAD_SCALE);
        }
        q.x = mxfp4_retile_word(q.x);
        q.y = mxfp4_retile_word(q.y);
        q.z = mxfp4_retile_word(q.z);
        q.w = mxfp4_retile_word(q.w);
        *reinterpret_cast<uint4*>(chunk + b * PLANE_BYTES + r * 16) = q;
        chunk[2 * PLANE_BYTES + r * 2 + b] = (uint8_t)sb;
    }
}

// Resident chunks of one expert matrix -> row-major bf16 [rows, K] through
// mxfp4_decode_word, the function the GEMM main loops call.
// grid (k_stages, m_tiles), block TILE_M threads.
__global__ void mxfp4_unpack_resident_kernel(const uint8_t* __restrict__ chunks, int rows, int K,
                                             uint16_t* __restrict__ out) {
    const int ks = blockIdx.x, mt = blockIdx.y, r = threadIdx.x;
    const int row = mt * TILE_M + r;
    if (row >= rows)
        return;
    const uint8_t* chunk = chunks + ((size_t)mt * gridDim.x + ks) * CHUNK_BYTES;
#pragma unroll
    for (int b = 0; b < 2; b++) {
        const int col0 = ks * KSTAGE + b * 32;
        if (col0 >= K)
            continue;
        const uint4 q = *reinterpret_cast<const uint4*>(chunk + b * PLANE_BYTES + r * 16);
        const uint32_t mult = mxfp4_scale_mult(chunk[2 * PLANE_BYTES + r * 2 + b]);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
        uint4* o = reinterpret_cast<uint4*>(out + (size_t)row * K + col0);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            uint32_t d[4];
            mxfp4_decode_word(w[j], mult, d);
            o[j] = make_uint4(d[0], d[1], d[2], d[3]);
        }
    }
}

}  // namespace moe
