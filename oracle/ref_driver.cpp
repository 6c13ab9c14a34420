// ref_driver.cpp -- C entry points around the reference engine's own CPU code.
//
// TEST INFRASTRUCTURE ONLY (checker and timed CPU baseline; never on the
// product path).
//
// This file is not compiled on its own.  oracle/Makefile streams the
// reference's src/run.cpp (read in place, with its two `#include "getp/..."`
// lines -- the HIP engine -- dropped, and -DTESTING so it has no main) into the
// compiler and appends this file to the same translation unit, so everything
// below calls the reference's compiled functions directly:
//   matmul  (src/run.cpp:341-354)      topk (src/run.cpp:373-404)
//   softmax (src/run.cpp:321-339)      forward (src/run.cpp:503-720)
//   memory_map_weights (src/run.cpp:196-235), malloc_run_state (:120-167)
// The result, oracle/_ref/libref_moe.so, is git-ignored.

#include <omp.h>

#include <vector>

extern "C" {

// Thin exports of the reference's own building blocks.
void ref_matmul(float* xout, float* x, float* w, int n, int d) { matmul(xout, x, w, n, d); }
void ref_softmax(float* x, int size) { softmax(x, size); }
void ref_topk(float* v, int* i, float* score, int E, int K) { topk(v, i, score, E, K); }
// The reference's own rmsnorm (src/run.cpp:306-319), row by row.
void ref_rmsnorm(float* o, float* x, float* weight, int rows, int size) {
    for (int r = 0; r < rows; r++)
        rmsnorm(o + (size_t)r * size, x + (size_t)r * size, weight, size);
}
int ref_num_threads(void) { return omp_get_max_threads(); }
// Threads of the calling thread's later parallel regions, whatever OMP_NUM_THREADS
// the process inherited.
void ref_set_num_threads(int n) {
    if (n > 0)
        omp_set_num_threads(n);
}

// The MoE block of the reference forward() (src/run.cpp:628-707) for T tokens,
// token at a time, experts in index order.  Only the ~40 lines of glue between
// the reference's matmul/topk/softmax calls are restated here; the arithmetic
// that dominates runs in the reference's functions.  Weights per expert as in
// the engine: w1[e] [2I,H] (gate/up rows interleaved), w2[e] [H,I].
// round_bf16 != 0 additionally rounds the block input and the SwiGLU output to
// bf16 (the HIP engine's rounding points, src/hip/BLAS.hip:32-40,
// src/hip/moe.hip:90,343).
static inline float drv_round_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) {
        u = 0x7fc00000u;
    } else {
        u += 0x7fffu + ((u >> 16) & 1u);
        u &= 0xffff0000u;
    }
    float r;
    memcpy(&r, &u, 4);
    return r;
}

int ref_moe_forward(int T, int H, int I, int E, int K, float limit, int round_bf16, const float* t_in,
                    float* w_router, const float* b_router, float* const* w1,
                    const float* const* b1, float* const* w2, const float* const* b2,
                    float* router_score_out, int* topk_i_out, float* topk_v_out, float* e_agg_out) {
    std::vector<float> t(H), score(E), topk_v(K), mlp1_out(2 * I), gate(I), up(I), gate_up(I),
        tb2(H), e_agg(H);
    std::vector<int> topk_i(K);
    for (int tok = 0; tok < T; tok++) {
        memcpy(t.data(), t_in + (size_t)tok * H, sizeof(float) * H);
        if (round_bf16)
            for (int i = 0; i < H; i++)
                t[i] = drv_round_bf16(t[i]);
        matmul(score.data(), t.data(), w_router, H, E);
        for (int i = 0; i < E; i++)
            score[i] += b_router[i];
        topk(topk_v.data(), topk_i.data(), score.data(), E, K);
        softmax(topk_v.data(), K);
        memset(e_agg.data(), 0, sizeof(float) * H);
        for (int e = 0; e < E; e++) {
            float expert_w = 0;
            int in_topk = 0;
            for (int idx = 0; idx < K; idx++) {
                if (topk_i[idx] == e) {
                    in_topk = 1;
                    expert_w = topk_v[idx];
                    break;
                }
            }
            if (!in_topk)
                continue;
            if (!w1[e] || !w2[e])
                return -(e + 1);
            matmul(mlp1_out.data(), t.data(), w1[e], H, 2 * I);
            for (int i = 0; i < 2 * I; i++)
                mlp1_out[i] += b1[e][i];
            for (int j = 0; j < I; j++) {
                gate[j] = mlp1_out[2 * j];
                up[j] = mlp1_out[2 * j + 1];
            }
            const float alpha = 1.702f;
            for (int i = 0; i < I; i++) {
                float val = gate[i];
                float up_val = up[i];
                if (val > limit)
                    val = limit;
                if (up_val > limit)
                    up_val = limit;
                if (up_val < -limit)
                    up_val = -limit;
                val *= (1.0f / (1.0f + expf(-alpha * val)));
                val *= (up_val + 1.0f);
                gate_up[i] = round_bf16 ? drv_round_bf16(val) : val;
            }
            matmul(tb2.data(), gate_up.data(), w2[e], I, H);
            for (int i = 0; i < H; i++)
                tb2[i] += b2[e][i];
            for (int i = 0; i < H; i++)
                e_agg[i] += tb2[i] * expert_w;
        }
        if (router_score_out)
            memcpy(router_score_out + (size_t)tok * E, score.data(), sizeof(float) * E);
        if (topk_i_out)
            memcpy(topk_i_out + (size_t)tok * K, topk_i.data(), sizeof(int) * K);
        if (topk_v_out)
            memcpy(topk_v_out + (size_t)tok * K, topk_v.data(), sizeof(float) * K);
        if (e_agg_out)
            memcpy(e_agg_out + (size_t)tok * H, e_agg.data(), sizeof(float) * H);
    }
    return 0;
}

// Whole-path cross-check: run the UNMODIFIED reference forward() on a one-layer
// model built in memory and return what its RunState holds for the MoE block of
// that layer: t (the block input, post-RMSNorm), router_score, topk_i, topk_v,
// e_agg.  Token i's embedding row is x_rows[i]; the attention output projection
// is zero so the residual stream reaching the FFN norm is the embedding itself;
// norm scales are 1.  Expert weights are dense fp32 [E,2I,H] / [E,H,I] as in
// the exported .bin (memory_map_weights order).
int ref_forward_moe_probe(int T, int H, int I, int E, int K, float limit, const float* x_rows,
                          const float* w_router, const float* b_router, const float* w1,
                          const float* b1, const float* w2, const float* b2, float* t_out,
                          float* router_score_out, int* topk_i_out, float* topk_v_out,
                          float* e_agg_out) {
    Transformer tr;
    memset(&tr, 0, sizeof(tr));
    Config* c = &tr.config;
    c->vocab_size = T;
    c->hidden_dim = H;
    c->n_experts = E;
    c->experts_per_token = K;
    c->intermediate_dim = I;
    c->n_layers = 1;
    c->head_dim = 64;
    c->n_attn_heads = 2;
    c->n_kv_heads = 1;
    c->seq_len = 4;
    c->initial_context_length = 4096;
    c->rope_theta = 150000.0f;
    c->rope_scaling_factor = 32.0f;
    c->sliding_window = 0;
    c->swiglu_limit = limit;

    const long long qkv_rows = (long long)c->head_dim * (c->n_attn_heads + 2 * c->n_kv_heads);
    const long long attn_dim = (long long)c->head_dim * c->n_attn_heads;
    long long n = 0;
    n += 2ll * T * H;                 // embedding, unembedding
    n += 3ll * H;                     // attn norm, ffn norm, out norm
    n += qkv_rows * H + qkv_rows;     // w_qkv, b_qkv
    n += attn_dim * H + H;            // w_o, b_o
    n += c->n_attn_heads;             // sinks
    n += 1ll * H * E + E;             // router
    n += 2ll * E * I * H + 2ll * E * I; // mlp1
    n += 1ll * E * H * I + 1ll * E * H; // mlp2
    float* blob = reinterpret_cast<float*>(calloc((size_t)n, sizeof(float)));
    if (!blob)
        return -1;
    memory_map_weights(&tr.weights, c, blob);
    TransformerWeights* w = &tr.weights;
    memcpy(w->token_embedding_table, x_rows, sizeof(float) * (size_t)T * H);
    for (int i = 0; i < H; i++) {
        w->rms_attn_w[i] = 1.0f;
        w->rms_ffn_w[i] = 1.0f;
        w->rms_out_w[i] = 1.0f;
    }
    // w_qkv, b_qkv, w_o, b_o, sinks, unembedding stay zero.
    memcpy(w->w_router, w_router, sizeof(float) * (size_t)H * E);
    memcpy(w->b_router, b_router, sizeof(float) * (size_t)E);
    memcpy(w->w_mlp1, w1, sizeof(float) * (size_t)2 * E * I * H);
    memcpy(w->b_mlp1, b1, sizeof(float) * (size_t)2 * E * I);
    memcpy(w->w_mlp2, w2, sizeof(float) * (size_t)E * H * I);
    memcpy(w->b_mlp2, b2, sizeof(float) * (size_t)E * H);
    malloc_run_state(&tr.state, c);
    RunState* s = &tr.state;
    for (int tok = 0; tok < T; tok++) {
        forward(&tr, tok, 0);
        memcpy(t_out + (size_t)tok * H, s->t, sizeof(float) * H);
        memcpy(router_score_out + (size_t)tok * E, s->router_score, sizeof(float) * E);
        memcpy(topk_i_out + (size_t)tok * K, s->topk_i, sizeof(int) * K);
        memcpy(topk_v_out + (size_t)tok * K, s->topk_v, sizeof(float) * K);
        memcpy(e_agg_out + (size_t)tok * H, s->e_agg, sizeof(float) * H);
    }
    free_run_state(s);
    free(blob);
    return 0;
}

} // extern "C"
