/*
 * moe_oracle.c -- CPU restatement of the gpt-oss-amd MoE feed-forward block.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA path: it is
 * linked/loaded by tests/, by the smoke check and by the cpu_baseline /
 * reference legs of bench.py, and by nothing else.  The shipped library
 * (libmoe_b200.so) never calls into it and has no CPU fallback.
 *
 * Parity status: PINNED.  Every function below is checked (a) against the
 * reference's own compiled CPU code (oracle/_ref, built from the reference
 * sources by oracle/Makefile) bit-for-bit on seeded inputs, and (b) for the
 * MXFP4 decode, against an exhaustive 16x256 table and random tensors produced
 * by running the reference's dequantize_fp4 (tests/golden/).
 *
 * Each function names the reference lines it restates (paths are relative to
 * the reference project root).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------------ */
/* bf16 helpers                                                              */

/* float -> bf16 bits, round-to-nearest-even, NaN -> 0x7FC0.  This is the
 * conversion torch applies when dequantize_fp4 stores its fp32 product into a
 * bf16 tensor (tools/model_export/gpt-oss-20b/export_model_bin.py:106,129),
 * and the __float2bfloat16 rounding the HIP path applies to activations
 * (src/hip/BLAS.hip:32-40). */
static inline uint16_t f32_to_bf16_bits(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u)
        return 0x7fc0;
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}

static inline float bf16_bits_to_f32(uint16_t b) {
    uint32_t u = ((uint32_t)b) << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

float oracle_round_bf16(float f) { return bf16_bits_to_f32(f32_to_bf16_bits(f)); }

void oracle_round_bf16_array(float* x, long long n) {
    for (long long i = 0; i < n; i++)
        x[i] = oracle_round_bf16(x[i]);
}

/* ------------------------------------------------------------------------ */
/* MXFP4 decode: tools/model_export/gpt-oss-20b/export_model_bin.py:75-133
 * (identical copy in tools/model_export/gpt-oss-120b/export_model_bin.py:90-148).
 *
 *   out[.., 2b]   = LUT[blk & 0xF] * 2^(scale-127)
 *   out[.., 2b+1] = LUT[blk >> 4 ] * 2^(scale-127)
 *
 * torch.ldexp scales exactly (no intermediate overflow): the result is the
 * real number LUT[code] * 2^(scale-127) rounded to bf16.  So scale byte 255
 * (exp = +128) gives 0 for codes 0/8, +/-2^127 for +/-0.5 and +/-inf for the
 * rest; scale byte 0 (exp = -127) gives bf16 subnormals.  The golden table
 * (tests/golden/mxfp4_table.npz, produced by running the reference function)
 * pins all 16 x 256 cases.
 */
static const float FP4_LUT[16] = {+0.0f, +0.5f, +1.0f, +1.5f, +2.0f, +3.0f, +4.0f, +6.0f,
                                  -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};

/* LUT[code] * 2^(scale_byte-127), exact in fp32 except for overflow to inf
 * (ldexpf scales without forming 2^e on its own). */
static inline float mxfp4_value(int code, int scale_byte) {
    return ldexpf(FP4_LUT[code & 15], (scale_byte & 255) - 127);
}

/* bf16 bit pattern of one decoded element (code in 0..15, scale byte 0..255). */
uint16_t oracle_mxfp4_decode_bits(int code, int scale_byte) {
    return f32_to_bf16_bits(mxfp4_value(code, scale_byte));
}

/* blocks: [rows, G, 16] uint8; scales: [rows, G] uint8; out: [rows, 32*G] bf16 bits.
 * Low nibble = even element (export_model_bin.py:122-127). */
void oracle_mxfp4_dequant_bf16(const uint8_t* blocks, const uint8_t* scales, long long rows, int G,
                               uint16_t* out) {
#pragma omp parallel for
    for (long long r = 0; r < rows; r++) {
        for (int g = 0; g < G; g++) {
            const uint8_t* blk = blocks + (r * G + g) * 16;
            int sc = scales[r * G + g];
            uint16_t* o = out + (r * G + g) * 32;
            for (int b = 0; b < 16; b++) {
                o[2 * b] = f32_to_bf16_bits(mxfp4_value(blk[b] & 15, sc));
                o[2 * b + 1] = f32_to_bf16_bits(mxfp4_value(blk[b] >> 4, sc));
            }
        }
    }
}

/* Same decode widened to fp32: what the exported .bin holds and the CPU engine
 * reads (the exporter casts the bf16 tensor to float32 when writing). */
void oracle_mxfp4_dequant_f32(const uint8_t* blocks, const uint8_t* scales, long long rows, int G,
                              float* out) {
#pragma omp parallel for
    for (long long r = 0; r < rows; r++) {
        for (int g = 0; g < G; g++) {
            const uint8_t* blk = blocks + (r * G + g) * 16;
            int sc = scales[r * G + g];
            float* o = out + (r * G + g) * 32;
            for (int b = 0; b < 16; b++) {
                o[2 * b] = bf16_bits_to_f32(f32_to_bf16_bits(mxfp4_value(blk[b] & 15, sc)));
                o[2 * b + 1] = bf16_bits_to_f32(f32_to_bf16_bits(mxfp4_value(blk[b] >> 4, sc)));
            }
        }
    }
}

/* ------------------------------------------------------------------------ */
/* matmul: src/run.cpp:341-354.  W (d,n) @ x (n,) -> xout (d,), float products
 * summed left to right in a double, OpenMP over output rows. */
void oracle_matmul(float* xout, const float* x, const float* w, int n, int d) {
    int i;
#pragma omp parallel for private(i)
    for (i = 0; i < d; i++) {
        double val = 0.0f;
        for (int j = 0; j < n; j++) {
            val += w[1ll * i * n + j] * x[j];
        }
        xout[i] = val;
    }
}

/* softmax: src/run.cpp:321-339 (double max and sum, expf of a float argument). */
void oracle_softmax(float* x, int size) {
    double max_val = x[0];
    for (int i = 1; i < size; i++) {
        if (x[i] > max_val)
            max_val = x[i];
    }
    double sum = 0.0f;
    for (int i = 0; i < size; i++) {
        x[i] = expf(x[i] - max_val);
        sum += x[i];
    }
    for (int i = 0; i < size; i++) {
        x[i] /= sum;
    }
}

/* topk: src/run.cpp:356-404 -- qsort of (value, index) pairs, descending by
 * value; order among equal values is whatever qsort leaves. */
typedef struct {
    float value;
    int index;
} OraclePair;

static int oracle_compare_desc(const void* a, const void* b) {
    float diff = ((const OraclePair*)b)->value - ((const OraclePair*)a)->value;
    if (diff > 0)
        return 1;
    if (diff < 0)
        return -1;
    return 0;
}

void oracle_topk(float* topk_values, int* topk_indices, const float* router_score, int num_experts,
                 int experts_per_token) {
    OraclePair* pairs = (OraclePair*)malloc(sizeof(OraclePair) * (size_t)num_experts);
    for (int i = 0; i < num_experts; ++i) {
        pairs[i].value = router_score[i];
        pairs[i].index = i;
    }
    qsort(pairs, (size_t)num_experts, sizeof(OraclePair), oracle_compare_desc);
    for (int i = 0; i < experts_per_token; ++i) {
        topk_values[i] = pairs[i].value;
        topk_indices[i] = pairs[i].index;
    }
    free(pairs);
}

/* SwiGLU: src/run.cpp:673-689 (and src/hip/moe.hip:186-191, which differs only
 * in using the fast __expf).  Gate has no lower clamp. */
static inline float oracle_swiglu(float gate, float up, float alpha, float limit) {
    float val = gate;
    float up_val = up;
    if (val > limit)
        val = limit;
    if (up_val > limit)
        up_val = limit;
    if (up_val < -limit)
        up_val = -limit;
    val *= (1.0f / (1.0f + expf(-alpha * val)));
    val *= (up_val + 1.0f);
    return val;
}

/* ------------------------------------------------------------------------ */
/* The MoE block of forward(): src/run.cpp:628-707, applied to T tokens one at a
 * time exactly as the engine does (the residual add at :710-712 is left to the
 * caller).
 *
 * Weights are fp32 (the decoded MXFP4 values) and are passed per expert so a
 * caller can materialise only the experts its tokens use:
 *   w1[e] -> [2I, H] gate/up row-interleaved, b1[e] -> [2I]
 *   w2[e] -> [H, I],                         b2[e] -> [H]
 * An expert that is selected but whose pointer is NULL makes the call fail
 * with -(e+1).
 *
 * round_mode 0: the CPU engine's numerics (fp32 activations throughout).
 * round_mode 1: the HIP engine's rounding points restated on the CPU: the block
 *   input is rounded to bf16 before the router and MLP1 GEMMs
 *   (src/hip/gemms/gemm_router.hip:67, src/hip/moe.hip:90 via BLAS.hip:32-40)
 *   and the SwiGLU output is rounded to bf16 before MLP2 (src/hip/moe.hip:343).
 *
 * Outputs (any may be NULL): router_score [T,E], topk_i [T,K], topk_v [T,K]
 * (after softmax), e_agg [T,H], and h [T,K,I]: the SwiGLU output that enters
 * MLP2 (after the bf16 rounding in round_mode 1) of the expert at position k of
 * the token's top-k list -- used to tell bf16 rounding flips of h apart from
 * real errors.
 */
int oracle_moe_forward(int T, int H, int I, int E, int K, float alpha, float limit, int round_mode,
                       const float* t_in, const float* w_router, const float* b_router,
                       const float* const* w1, const float* const* b1, const float* const* w2,
                       const float* const* b2, float* router_score_out, int* topk_i_out,
                       float* topk_v_out, float* e_agg_out, float* h_out) {
    float* t = (float*)malloc(sizeof(float) * (size_t)H);
    float* router_score = (float*)malloc(sizeof(float) * (size_t)E);
    float* topk_v = (float*)malloc(sizeof(float) * (size_t)K);
    int* topk_i = (int*)malloc(sizeof(int) * (size_t)K);
    float* mlp1_out = (float*)malloc(sizeof(float) * (size_t)(2 * I));
    float* gate = (float*)malloc(sizeof(float) * (size_t)I);
    float* up = (float*)malloc(sizeof(float) * (size_t)I);
    float* gate_up = (float*)malloc(sizeof(float) * (size_t)I);
    float* tb2 = (float*)malloc(sizeof(float) * (size_t)H);
    float* e_agg = (float*)malloc(sizeof(float) * (size_t)H);
    int status = 0;

    for (int tok = 0; tok < T && status == 0; tok++) {
        memcpy(t, t_in + (size_t)tok * H, sizeof(float) * (size_t)H);
        if (round_mode == 1)
            oracle_round_bf16_array(t, H);

        /* router: run.cpp:630-637 */
        oracle_matmul(router_score, t, w_router, H, E);
        for (int i = 0; i < E; i++)
            router_score[i] += b_router[i];
        /* run.cpp:639-641 */
        oracle_topk(topk_v, topk_i, router_score, E, K);
        oracle_softmax(topk_v, K);

        /* run.cpp:644-707: experts visited in index order */
        memset(e_agg, 0, sizeof(float) * (size_t)H);
        for (int e = 0; e < E; e++) {
            float expert_w = 0;
            int in_topk = 0, k_pos = 0;
            for (int idx = 0; idx < K; idx++) {
                if (topk_i[idx] == e) {
                    in_topk = 1;
                    k_pos = idx;
                    expert_w = topk_v[idx];
                    break;
                }
            }
            if (!in_topk)
                continue;
            if (!w1[e] || !b1[e] || !w2[e] || !b2[e]) {
                status = -(e + 1);
                break;
            }
            oracle_matmul(mlp1_out, t, w1[e], H, 2 * I);
            for (int i = 0; i < 2 * I; i++)
                mlp1_out[i] += b1[e][i];
            for (int j = 0; j < I; j++) {
                gate[j] = mlp1_out[2 * j];
                up[j] = mlp1_out[2 * j + 1];
            }
            for (int i = 0; i < I; i++)
                gate_up[i] = oracle_swiglu(gate[i], up[i], alpha, limit);
            if (round_mode == 1)
                oracle_round_bf16_array(gate_up, I);
            if (h_out)
                memcpy(h_out + ((size_t)tok * K + k_pos) * I, gate_up, sizeof(float) * (size_t)I);
            oracle_matmul(tb2, gate_up, w2[e], I, H);
            for (int i = 0; i < H; i++)
                tb2[i] += b2[e][i];
            for (int i = 0; i < H; i++)
                e_agg[i] += tb2[i] * expert_w;
        }

        if (router_score_out)
            memcpy(router_score_out + (size_t)tok * E, router_score, sizeof(float) * (size_t)E);
        if (topk_i_out)
            memcpy(topk_i_out + (size_t)tok * K, topk_i, sizeof(int) * (size_t)K);
        if (topk_v_out)
            memcpy(topk_v_out + (size_t)tok * K, topk_v, sizeof(float) * (size_t)K);
        if (e_agg_out)
            memcpy(e_agg_out + (size_t)tok * H, e_agg, sizeof(float) * (size_t)H);
    }

    free(t);
    free(router_score);
    free(topk_v);
    free(topk_i);
    free(mlp1_out);
    free(gate);
    free(up);
    free(gate_up);
    free(tb2);
    free(e_agg);
    return status;
}

/* One expert applied to a list of rows (no routing): y[r] = MLP2(SwiGLU(MLP1(x[r]))),
 * the inner part of run.cpp:658-700.  Used by the expert-parallel tests, where a
 * rank computes only the experts it owns on rows it received. */
void oracle_expert_rows(int n_rows, int H, int I, float alpha, float limit, int round_mode,
                        const float* x, const float* w1, const float* b1, const float* w2,
                        const float* b2, float* y) {
    float* t = (float*)malloc(sizeof(float) * (size_t)H);
    float* mlp1_out = (float*)malloc(sizeof(float) * (size_t)(2 * I));
    float* gate_up = (float*)malloc(sizeof(float) * (size_t)I);
    for (int r = 0; r < n_rows; r++) {
        memcpy(t, x + (size_t)r * H, sizeof(float) * (size_t)H);
        if (round_mode == 1)
            oracle_round_bf16_array(t, H);
        oracle_matmul(mlp1_out, t, w1, H, 2 * I);
        for (int i = 0; i < 2 * I; i++)
            mlp1_out[i] += b1[i];
        for (int j = 0; j < I; j++)
            gate_up[j] = oracle_swiglu(mlp1_out[2 * j], mlp1_out[2 * j + 1], alpha, limit);
        if (round_mode == 1)
            oracle_round_bf16_array(gate_up, I);
        float* yr = y + (size_t)r * H;
        oracle_matmul(yr, gate_up, w2, I, H);
        for (int i = 0; i < H; i++)
            yr[i] += b2[i];
    }
    free(t);
    free(mlp1_out);
    free(gate_up);
}

/* Routing only (run.cpp:630-641) for T tokens: lets a caller find out which
 * experts a batch selects before it materialises their fp32 weights. */
void oracle_route(int T, int H, int E, int K, int round_mode, const float* t_in,
                  const float* w_router, const float* b_router, float* router_score_out,
                  int* topk_i_out, float* topk_v_out) {
    float* t = (float*)malloc(sizeof(float) * (size_t)H);
    float* router_score = (float*)malloc(sizeof(float) * (size_t)E);
    for (int tok = 0; tok < T; tok++) {
        memcpy(t, t_in + (size_t)tok * H, sizeof(float) * (size_t)H);
        if (round_mode == 1)
            oracle_round_bf16_array(t, H);
        oracle_matmul(router_score, t, w_router, H, E);
        for (int i = 0; i < E; i++)
            router_score[i] += b_router[i];
        oracle_topk(topk_v_out + (size_t)tok * K, topk_i_out + (size_t)tok * K, router_score, E, K);
        oracle_softmax(topk_v_out + (size_t)tok * K, K);
        if (router_score_out)
            memcpy(router_score_out + (size_t)tok * E, router_score, sizeof(float) * (size_t)E);
    }
    free(t);
    free(router_score);
}

/* The RMSNorm in front of the block (src/run.cpp:306-319; call src/run.cpp:626,
 * GPU engine src/forward.cpp:315): squares rounded to float and summed in double,
 * 1.0f / sqrtf of the mean plus 1e-5f in float, then weight * (ss * x) evaluated in
 * double and stored as float.  rows x size. */
void oracle_rmsnorm(float* o, const float* x, const float* weight, int rows, int size) {
    int r, j;
    for (r = 0; r < rows; r++) {
        const float* xr = x + (size_t)r * size;
        float* orow = o + (size_t)r * size;
        double ss = 0.0f;
        for (j = 0; j < size; j++) {
            ss += xr[j] * xr[j];
        }
        ss /= size;
        ss += 1e-5f;
        ss = 1.0f / sqrtf(ss);
        for (j = 0; j < size; j++) {
            orow[j] = weight[j] * (ss * xr[j]);
        }
    }
}

int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* OpenMP threads of the calling thread's later parallel regions, whatever
 * OMP_NUM_THREADS the process inherited (the reference's run.sh sets its own
 * count the same way, run.sh:6). */
void oracle_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0)
        omp_set_num_threads(n);
#else
    (void)n;
#endif
}
