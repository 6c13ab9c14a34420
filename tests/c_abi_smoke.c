/*
 * The engine-side binding of include/moe_b200.h as a plain-C (C99) translation
 * unit: what a maintainer of the engine writes in place of the MoE block of
 * src/forward.cpp:317-514 -- one handle created at warm-up, router and packed
 * experts uploaded per layer, one call per layer and batch.
 *
 *   c_abi_smoke [out.bin]
 *
 * Without a GPU it checks the pure-host entry points and that create fails with
 * MOE_B200_ERR_NO_DEVICE ("no device" is printed).  With a GPU it runs a small
 * layer on inputs from a fixed linear congruential generator through the
 * host-buffer entry point and, when a path is given, writes
 *   int32 T, H, E, K, I;  x, w_router (bf16 bits);  b_router;  blocks1, scales1,
 *   bias1, blocks2, scales2, bias2;  int32 topk_i[T*K];  float topk_w[T*K];
 *   float out[T*H]
 * (inputs as it passed them, outputs as it got them) for the test that runs the
 * same inputs through the oracle (tests/test_gpu_parity.py::test_plain_c_caller).
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "moe_b200.h"

enum { H = 128, I = 64, E = 8, K = 2, T = 24 };

static unsigned int lcg_state = 12345u;
static unsigned int lcg(void) {
    lcg_state = lcg_state * 1664525u + 1013904223u;
    return lcg_state >> 8;
}

/* bf16 bits of a small value in [-1, 1) with 7 significant bits: exact in bf16 */
static unsigned short small_bf16(void) {
    int v = (int)(lcg() % 255u) - 127; /* -127..127 */
    float f = (float)v / 128.0f;
    unsigned int u;
    memcpy(&u, &f, 4);
    return (unsigned short)(u >> 16);
}

static int fail(const char* what, moe_b200_handle h) {
    printf("FAILED: %s: %s\n", what, moe_b200_last_error(h));
    return 1;
}

int main(int argc, char** argv) {
    int first = -1, n = -1, r, p;
    moe_b200_config cfg;
    moe_b200_handle h = NULL;
    moe_b200_status st;

    printf("%s\n", moe_b200_version());

    /* src/model.cpp:104-114: 10 experts over 4 ranks -> 3, 3, 2, 2 */
    {
        static const int want_first[4] = {0, 3, 6, 8}, want_n[4] = {3, 3, 2, 2};
        for (r = 0; r < 4; r++) {
            moe_b200_shard_range(10, 4, r, &first, &n);
            if (first != want_first[r] || n != want_n[r]) {
                printf("FAILED: shard_range rank %d -> (%d, %d)\n", r, first, n);
                return 1;
            }
        }
    }
    /* two ranks, four experts: what rank 0 sends to rank 1 is what rank 1 expects from rank 0 */
    {
        int cnt_all[2][4] = {{1, 2, 3, 4}, {5, 6, 7, 8}};
        int sc[2][2], so[2][2], rc[2][2], ro[2][2];
        for (r = 0; r < 2; r++)
            moe_b200_ep_plan(4, 2, r, &cnt_all[0][0], sc[r], so[r], rc[r], ro[r]);
        for (r = 0; r < 2; r++)
            for (p = 0; p < 2; p++)
                if (sc[r][p] != rc[p][r]) {
                    printf("FAILED: ep_plan is not symmetric\n");
                    return 1;
                }
        if (sc[0][0] != 3 || sc[0][1] != 7 || so[0][1] != 3 || rc[1][0] != 7 || rc[1][1] != 15) {
            printf("FAILED: ep_plan values\n");
            return 1;
        }
    }

    memset(&cfg, 0, sizeof cfg);
    cfg.hidden_dim = H;
    cfg.intermediate_dim = I;
    cfg.n_experts = E;
    cfg.experts_per_token = K;
    cfg.n_layers = 1;
    cfg.swiglu_alpha = 1.702f;
    cfg.swiglu_limit = 7.0f;
    cfg.max_tokens = T;
    cfg.ep_rank = 0;
    cfg.ep_size = 1;
    cfg.device = 0;
    cfg.gemm_impl = MOE_B200_GEMM_TCGEN05;

    /* bad arguments come back as codes, never as exit() */
    cfg.hidden_dim = 100;
    if (moe_b200_create(&cfg, &h) != MOE_B200_ERR_INVALID || h != NULL)
        return fail("create accepted hidden_dim = 100", NULL);
    cfg.hidden_dim = H;

    st = moe_b200_create(&cfg, &h);
    if (st == MOE_B200_ERR_NO_DEVICE) {
        printf("no device: %s\n", moe_b200_last_error(NULL));
        printf("c_abi_smoke ok\n");
        return 0;
    }
    if (st != MOE_B200_OK)
        return fail("create", NULL);

    {
        /* warm-up: router + packed MXFP4 experts of layer 0, from host memory */
        static unsigned short w_router[E * H];
        static float b_router[E];
        static unsigned char blocks1[E * 2 * I * (H / 32) * 16], scales1[E * 2 * I * (H / 32)];
        static unsigned char blocks2[E * H * (I / 32) * 16], scales2[E * H * (I / 32)];
        static float bias1[E * 2 * I], bias2[E * H];
        static unsigned short x[T * H];
        static float out[T * H], topk_w[T * K];
        static int topk_i[T * K];
        size_t i;
        int word = -1;

        for (i = 0; i < sizeof w_router / 2; i++)
            w_router[i] = small_bf16();
        for (i = 0; i < E; i++)
            b_router[i] = (float)((int)(lcg() % 64u) - 32) / 64.0f;
        for (i = 0; i < sizeof blocks1; i++)
            blocks1[i] = (unsigned char)(lcg() & 0xFFu);
        for (i = 0; i < sizeof scales1; i++)
            scales1[i] = (unsigned char)(119u + lcg() % 5u); /* 2^-8 .. 2^-4 */
        for (i = 0; i < sizeof blocks2; i++)
            blocks2[i] = (unsigned char)(lcg() & 0xFFu);
        for (i = 0; i < sizeof scales2; i++)
            scales2[i] = (unsigned char)(119u + lcg() % 5u);
        for (i = 0; i < E * 2 * I; i++)
            bias1[i] = (float)((int)(lcg() % 64u) - 32) / 2048.0f;
        for (i = 0; i < E * H; i++)
            bias2[i] = (float)((int)(lcg() % 64u) - 32) / 2048.0f;
        for (i = 0; i < T * H; i++)
            x[i] = small_bf16();

        if (moe_b200_set_router(h, 0, w_router, b_router) != MOE_B200_OK)
            return fail("set_router", h);
        if (moe_b200_set_experts_mxfp4(h, 0, 0, E, blocks1, scales1, bias1, blocks2, scales2, bias2) !=
            MOE_B200_OK)
            return fail("set_experts_mxfp4", h);
        /* a layer that was not loaded is an error code */
        if (moe_b200_forward_host(h, 1, x, MOE_B200_DTYPE_BF16, T, out, NULL, NULL) != MOE_B200_ERR_INVALID)
            return fail("forward_host accepted layer 1", h);

        /* the block: s->t in, e_agg out (src/forward.cpp:317-514 in one call) */
        if (moe_b200_forward_host(h, 0, x, MOE_B200_DTYPE_BF16, T, out, topk_i, topk_w) != MOE_B200_OK)
            return fail("forward_host", h);
        if (moe_b200_device_status(h, &word) != MOE_B200_OK || word != 0)
            return fail("device_status", h);
        for (i = 0; i < T * K; i++)
            if (topk_i[i] < 0 || topk_i[i] >= E)
                return fail("expert index out of range", h);
        for (i = 0; i < T * H; i++)
            if (!(out[i] == out[i]) || out[i] > 1e30f || out[i] < -1e30f)
                return fail("non-finite output", h);
        printf("launches %d, device bytes %lu\n", moe_b200_last_launch_count(h),
               (unsigned long)moe_b200_device_bytes(h));
        if (argc > 1) {
            FILE* f = fopen(argv[1], "wb");
            int hdr[5];
            hdr[0] = T, hdr[1] = H, hdr[2] = E, hdr[3] = K, hdr[4] = I;
            if (!f)
                return fail("cannot open the output file", h);
            fwrite(hdr, sizeof hdr, 1, f);
            fwrite(x, sizeof x, 1, f);
            fwrite(w_router, sizeof w_router, 1, f);
            fwrite(b_router, sizeof b_router, 1, f);
            fwrite(blocks1, sizeof blocks1, 1, f);
            fwrite(scales1, sizeof scales1, 1, f);
            fwrite(bias1, sizeof bias1, 1, f);
            fwrite(blocks2, sizeof blocks2, 1, f);
            fwrite(scales2, sizeof scales2, 1, f);
            fwrite(bias2, sizeof bias2, 1, f);
            fwrite(topk_i, sizeof topk_i, 1, f);
            fwrite(topk_w, sizeof topk_w, 1, f);
            fwrite(out, sizeof out, 1, f);
            fclose(f);
        }
    }
    if (moe_b200_destroy(h) != MOE_B200_OK)
        return fail("destroy", NULL);
    printf("c_abi_smoke ok\n");
    return 0;
}
