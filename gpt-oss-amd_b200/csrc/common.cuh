// Shared definitions of the MoE kernels: resident weight layout, MXFP4 decode,
// status codes.  sm_100a only.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace moe {

// ---------------------------------------------------------------------------
// Resident ("re-tiled") MXFP4 layout of one expert matrix W[rows, K]
// (rows = 2I for mlp1, H for mlp2; K = H or I).
//
// The matrix is cut into tiles of TILE_M rows x KSTAGE columns.  One tile is a
// contiguous CHUNK_BYTES chunk, chunks ordered [m_tile][k_stage], so a GEMM CTA
// streams its weights with one bulk copy per pipeline stage:
//
//   [0    , 2048)  plane 0: row r's MXFP4 block for columns [0,32)  at r*16
//   [2048 , 4096)  plane 1: row r's MXFP4 block for columns [32,64) at r*16
//   [4096 , 4352)  scales : row r's two e8m0 bytes at r*2
//
// Inside a 16-byte block the four 32-bit words each cover 8 consecutive
// columns; the 32 bits of a word are the 32 bits of its eight e2m1 codes, moved
// to the positions from which mxfp4_decode_word (below) needs the fewest shifts
// and masks: even columns in the low half, odd columns in the high half, so
// columns (2p, 2p+1) sit 16 bits apart and land in one bf16x2 register.  Every
// bit is still a bit of an e2m1 code and every scale an e8m0 byte: 4.25 bits per
// weight, as in the checkpoint.  Rows past the end of the matrix are zero codes.
constexpr int TILE_M = 128;
constexpr int KSTAGE = 64;
constexpr int PLANE_BYTES = TILE_M * 16;
constexpr int CHUNK_BYTES = 2 * PLANE_BYTES + TILE_M * 2;  // 4352
constexpr int MAX_SCALE_BYTE = 128;  // largest e8m0 byte the one-multiply decode covers

// Device status word (one int per handle).  0 = fine.  A bounded wait that ran
// out stores one of these (first writer wins) and the kernel winds down.
enum DeviceStatus : int {
    DS_OK = 0,
    DS_TIMEOUT_FULL_W = 0x101,    // dequant warps waiting for packed weights
    DS_TIMEOUT_FULL_A = 0x102,    // MMA warp waiting for decoded weights
    DS_TIMEOUT_FULL_B = 0x103,    // MMA warp waiting for the activation tile
    DS_TIMEOUT_EMPTY = 0x104,     // producer waiting for a free stage
    DS_TIMEOUT_TMEM_FULL = 0x105, // epilogue waiting for the accumulator
    DS_TIMEOUT_TMEM_EMPTY = 0x106,// MMA warp waiting for a drained accumulator
    DS_BAD_SCALE = 0x201,         // a scale byte above MAX_SCALE_BYTE was uploaded (own flag word)
    DS_BAD_EXPERT = 0x202,        // router produced an expert index out of range
};

__device__ __forceinline__ void report_status(int* status, int code) {
    if (status)
        atomicCAS(status, 0, code);
}

// ---------------------------------------------------------------------------
// bf16 helpers

__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits16) {
    return __uint_as_float(bits16 << 16);
}

// fp32 -> bf16 bits, round to nearest even (what __float2bfloat16 does in the
// reference, src/hip/BLAS.hip:32-40).
__device__ __forceinline__ uint32_t float_to_bf16_bits(float f) {
    return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(f));
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    return float_to_bf16_bits(lo) | (float_to_bf16_bits(hi) << 16);
}

// ---------------------------------------------------------------------------
// In-kernel MXFP4 decode (the GEMM main loops and unpack_resident use this).
//
// An e2m1 code s|e1 e0|m placed with its magnitude bits at bf16 bits [8:6] is
// the bf16 number  value * 2^-126  (exponent field = e, top mantissa bit = m;
// e = 0 lands on the bf16 subnormals exactly as 0 / 0.5 are the e2m1
// subnormals).  One bf16x2 multiply by 2^(scale_byte - 1) then yields
// value * 2^(scale_byte - 127) exactly: both factors have at most two
// significant bits.  The multiplier is representable for scale bytes 0..128.

// bf16x2 multiplier for a scale byte (both halves).
__device__ __forceinline__ uint32_t mxfp4_scale_mult(uint32_t scale_byte) {
    return ((scale_byte + 126u) << 7) * 0x00010001u;
}

__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
    __nv_bfloat162 x = *reinterpret_cast<__nv_bfloat162*>(&a);
    __nv_bfloat162 y = *reinterpret_cast<__nv_bfloat162*>(&b);
    __nv_bfloat162 r = __hmul2(x, y);
    return *reinterpret_cast<uint32_t*>(&r);
}

// Resident word: the eight e2m1 codes of eight consecutive columns, bit-scattered so
// that the decode needs as few shifts and masks as the bf16 layout allows.  Even columns
// belong to the low 16-bit half of an output, odd columns to the high half; the codes of
// columns (2p, 2p+1) make output p.  A code s|e1 e0|m must end up with e1 e0 m at
// bits [8:6] and s at bit 15 of its half, so a code that one rotation of the word by r
// puts in place sits on the bits {a, a+1, a+2, a+9} (+16 for the other half, mod 32)
// with a = 6 - r.  Modulo 16 that pattern fits three times but never four (enumerated);
// of all layouts the one below decodes in the fewest operations: three codes on the
// pattern (a = 0, 4, 10), the fourth with e1, e0, s already in place and only its m
// one rotation away.
//   output 0: m e0 e1 s at bits  0  1  2  9 | 16 17 18 25   (low-half code | high-half code)
//   output 1:                    4  5  6 13 | 20 21 22 29
//   output 2:                   10 11 12 19 | 26 27 28  3
//   output 3:                   30  7  8 15 | 14 23 24 31
// Per word: 4 shifts or rotations, 5 logic operations, 4 bf16x2 multiplies (a
// nibble-per-code word needs 7 + 8 + 4).
// Bit of the resident word that holds bit `b` (0 = m, 1 = e0, 2 = e1, 3 = s) of the code
// of output `o`, half `h`: the table above, five bits per entry.
__host__ __device__ constexpr int mxfp4_resident_pos(int o, int h, int b) {
    constexpr unsigned long long LO[4] = {  // four positions per (output, low half), 8 bits each
        0x09020100ull, 0x0D060504ull, 0x130C0B0Aull, 0x0F08071Eull};
    constexpr unsigned long long HI[4] = {
        0x19121110ull, 0x1D161514ull, 0x031C1B1Aull, 0x1F18170Eull};
    return (int)(((h ? HI[o] : LO[o]) >> (8 * b)) & 0xFFull);
}

__device__ __forceinline__ void mxfp4_decode_word(uint32_t w, uint32_t mult, uint32_t out[4]) {
    const uint32_t CODE = 0x81C081C0u;  // sign and magnitude of a code in place, both halves
    const uint32_t M_BIT = 0x00400040u;
    const uint32_t b0 = (w << 6) & CODE;
    const uint32_t b1 = (w << 2) & CODE;
    const uint32_t b2 = __funnelshift_r(w, w, 4) & CODE;
    const uint32_t r8 = __funnelshift_l(w, w, 8);
    const uint32_t b3 = ((r8 & M_BIT) | (w & ~M_BIT)) & CODE;  // a bit-select, then the mask
    out[0] = bf16x2_mul(b0, mult);
    out[1] = bf16x2_mul(b1, mult);
    out[2] = bf16x2_mul(b2, mult);
    out[3] = bf16x2_mul(b3, mult);
}

// Checkpoint word (nibble i = column i; bits of a nibble: m, e0, e1, s) -> resident word.
__host__ __device__ __forceinline__ uint32_t mxfp4_retile_word(uint32_t w) {
    uint32_t r = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const uint32_t c = (w >> (4 * i)) & 0xFu;
#pragma unroll
        for (int b = 0; b < 4; b++)
            r |= ((c >> b) & 1u) << mxfp4_resident_pos(i >> 1, i & 1, b);
    }
    return r;
}

// Exact decode of one element for ANY scale byte, integer arithmetic only:
// the bf16 bit pattern of LUT[code] * 2^(scale_byte-127) as the reference's
// dequantize_fp4 produces it
// (tools/model_export/gpt-oss-20b/export_model_bin.py:75-133), including the
// bf16 subnormals at scale byte 0 and the overflow to inf at 254/255.
__host__ __device__ __forceinline__ uint32_t mxfp4_decode_exact(uint32_t code, uint32_t scale_byte) {
    uint32_t sign = (code & 8u) << 12;
    uint32_t m = code & 7u;
    if (m == 0)
        return sign;
    uint32_t mant = (m >= 2) ? (m & 1u) : 0u;
    int biased = (int)scale_byte + ((m >= 2) ? (int)(m >> 1) - 1 : -1);
    if (biased >= 255)
        return sign | 0x7F80u;
    if (biased >= 1)
        return sign | ((uint32_t)biased << 7) | (mant << 6);
    // subnormal result: (2 + mant) * 2^(biased - 128), unit 2^-133
    return sign | ((2u + mant) << (biased + 5));
}

__host__ __device__ __forceinline__ int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Programmatic dependent launch.  A kernel launched with the programmatic-serialization
// attribute may start while the kernel before it on the stream is still running; it
// does its own set-up (shared-memory init, barriers, tensor-memory allocation) and calls
// pdl_wait() before it touches anything that kernel wrote -- the wait returns when the
// whole previous grid has completed and its memory is visible.  pdl_trigger() lets the
// NEXT kernel start its own set-up early; it orders nothing.  Both are no-ops in a
// kernel launched the ordinary way.  Every kernel of the forward path calls both, in
// this order, before its first global access that depends on an earlier kernel, and
// writes nothing to global memory before the wait.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Clamped SwiGLU (src/run.cpp:673-689, src/hip/moe.hip:186-191): the gate has no
// lower clamp.
__device__ __forceinline__ float swiglu(float gate, float up, float alpha, float limit) {
    const float g = fminf(gate, limit);
    const float u = fminf(fmaxf(up, -limit), limit);
    // fast reciprocal: the IEEE division costs ~90 cycles per value in the epilogue
    const float sig = __fdividef(1.0f, 1.0f + __expf(-alpha * g));
    return g * sig * (u + 1.0f);
}

}  // namespace moe
