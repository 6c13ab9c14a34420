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

// The GEMMs' one-multiply decode covers resident scale bytes 0..MAX_SCALE_BYTE.  A
// checkpoint may hold any e8m0 byte (the reference's dequantize_fp4 takes them all,
// tools/model_export/gpt-oss-20b/export_model_bin.py:125-129), so every weight ROW gets
// an exponent shift: shift = max(0, largest scale byte of the row - MAX_SCALE_BYTE), the
// resident bytes are the checkpoint's minus the shift, and the GEMM epilogue multiplies
// the row's fp32 accumulator by 2^shift (exact: a power of two).  A row is representable
// when the scale bytes of its blocks that hold a non-zero code span at most
// MAX_SCALE_BYTE binades; a row that does not is reported (DS_BAD_SCALE).  Blocks of
// zeros keep their zeros under any scale.
// One warp per row.  row_shift[rows] (ints, scratch for the re-tile kernel that follows
// on the same stream) and row_scale[rows] = 2^shift.
__global__ void mxfp4_row_shift_kernel(const uint8_t* __restrict__ blocks,
                                       const uint8_t* __restrict__ scales, int rows, int G,
                                       int* __restrict__ row_shift, float* __restrict__ row_scale,
                                       int* __restrict__ status) {
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows)
        return;
    int hi = 0, lo = 255;
    for (int g = lane; g < G; g += 32) {
        const uint4 q = *reinterpret_cast<const uint4*>(blocks + ((size_t)row * G + g) * 16);
        if (((q.x | q.y | q.z | q.w) & 0x77777777u) != 0) {  // some magnitude is not zero
            const int sb = scales[(size_t)row * G + g];
            hi = max(hi, sb);
            lo = min(lo, sb);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, o));
        lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, o));
    }
    if (lane == 0) {
        const int shift = max(0, hi - MAX_SCALE_BYTE);
        if (lo < shift)
            report_status(status, DS_BAD_SCALE);
        row_shift[row] = shift;
        row_scale[row] = __uint_as_float((uint32_t)(127 + shift) << 23);
    }
}

// Checkpoint layout of ONE expert matrix -> resident chunks.
// grid (k_stages, m_tiles), block TILE_M threads (thread = row of the tile).
__global__ void mxfp4_retile_kernel(const uint8_t* __restrict__ blocks,
                                    const uint8_t* __restrict__ scales, int rows, int G,
                                    const int* __restrict__ row_shift, uint8_t* __restrict__ chunks) {
    const int ks = blockIdx.x, mt = blockIdx.y, r = threadIdx.x;
    const int row = mt * TILE_M + r;
    const int shift = row < rows ? row_shift[row] : 0;
    uint8_t* chunk = chunks + ((size_t)mt * gridDim.x + ks) * CHUNK_BYTES;
#pragma unroll
    for (int b = 0; b < 2; b++) {
        const int g = ks * 2 + b;
        uint4 q = make_uint4(0, 0, 0, 0);
        int sb = 127;
        if (row < rows && g < G) {
            q = *reinterpret_cast<const uint4*>(blocks + ((size_t)row * G + g) * 16);
            // only a block of zeros can leave the range (mxfp4_row_shift_kernel checked the rest)
            sb = min(max((int)scales[(size_t)row * G + g] - shift, 0), MAX_SCALE_BYTE);
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
// mxfp4_decode_word, the function the GEMM main loops call, times the row's 2^shift
// (what the GEMM epilogue applies to the accumulator).
// grid (k_stages, m_tiles), block TILE_M threads.
__global__ void mxfp4_unpack_resident_kernel(const uint8_t* __restrict__ chunks,
                                             const float* __restrict__ row_scale, int rows, int K,
                                             uint16_t* __restrict__ out) {
    const int ks = blockIdx.x, mt = blockIdx.y, r = threadIdx.x;
    const int row = mt * TILE_M + r;
    if (row >= rows)
        return;
    const float rs = row_scale[row];
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
            if (rs != 1.f) {
#pragma unroll
                for (int p = 0; p < 4; p++) {
                    const float lo = __uint_as_float(d[p] << 16) * rs;
                    const float hi = __uint_as_float(d[p] & 0xFFFF0000u) * rs;
                    d[p] = pack_bf16x2(lo, hi);
                }
            }
            o[j] = make_uint4(d[0], d[1], d[2], d[3]);
        }
    }
}

}  // namespace moe
