"""CPU tests that pin the oracle (oracle/moe_oracle.c) before anything trusts it:
against the golden vectors produced by running the reference, and -- when the
reference-derived library oracle/_ref/libref_moe.so is present -- bit for bit
against the reference's own compiled CPU functions on fresh seeded inputs."""
import os

import numpy as np
import pytest

import gpt_oss_amd_b200.synth as synth
from oracle import oracle


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


def test_mxfp4_table_matches_reference_function(golden_dir):
    table = _load(golden_dir, "mxfp4_table.npz")["table"]
    assert table.shape == (16, 256)
    mine = oracle.mxfp4_decode_table()
    assert np.array_equal(mine, table)
    # spot facts the table pins: -0.0 survives, +/-0.5 is the e2m1 subnormal
    assert table[8, 127] == 0x8000 and table[1, 127] == 0x3F00 and table[15, 127] == 0xC0C0


def test_mxfp4_random_matches_reference_function(golden_dir):
    r = _load(golden_dir, "mxfp4_random.npz")
    for tag in ("full", "cfg"):
        out = oracle.mxfp4_dequant_bf16(r[f"blocks_{tag}"], r[f"scales_{tag}"])
        assert np.array_equal(out, r[f"out_{tag}"]), tag
        f32 = oracle.mxfp4_dequant_f32(r[f"blocks_{tag}"], r[f"scales_{tag}"])
        same = synth.bf16_bits_to_f32(r[f"out_{tag}"])
        assert np.array_equal(f32.view(np.uint32), same.view(np.uint32))


def test_nibble_order_low_is_even():
    blocks = np.zeros((1, 1, 16), dtype=np.uint8)
    blocks[0, 0, 0] = 0x72  # low nibble 2 -> 1.0, high nibble 7 -> 6.0
    scales = np.full((1, 1), 127, dtype=np.uint8)
    out = oracle.mxfp4_dequant_f32(blocks, scales)
    assert out[0, 0] == 1.0 and out[0, 1] == 6.0 and not out[0, 2:].any()


def _small_case(golden_dir):
    g = _load(golden_dir, "moe_small.npz")
    x = synth.bf16_bits_to_f32(g["x_bits"])
    wr = synth.bf16_bits_to_f32(g["w_router_bits"])
    cache = oracle.ExpertCache(g["blocks1"], g["scales1"], g["bias1"], g["blocks2"], g["scales2"],
                               g["bias2"])
    return g, x, wr, cache


@pytest.mark.parametrize("mode,tag", [(0, "f32"), (1, "bf16")])
def test_moe_block_matches_reference_golden(golden_dir, mode, tag):
    g, x, wr, cache = _small_case(golden_dir)
    r = oracle.moe_forward(x, wr, g["b_router"], cache, top_k=int(g["top_k"]), round_mode=mode)
    assert np.array_equal(r["topk_i"], g[f"{tag}_topk_i"])
    for k in ("router_score", "topk_v", "e_agg"):
        assert np.array_equal(r[k].view(np.uint32), g[f"{tag}_{k}"].view(np.uint32)), k


def test_glue_matches_unmodified_reference_forward(golden_dir):
    """The reference forward() run whole on a one-layer model; its MoE block
    input `t` fed to the restated block must give its e_agg bit for bit."""
    g, _, wr, cache = _small_case(golden_dir)
    r = oracle.moe_forward(g["probe_t"], wr, g["b_router"], cache, top_k=int(g["top_k"]),
                           round_mode=0)
    assert np.array_equal(r["topk_i"], g["probe_topk_i"])
    for k in ("router_score", "topk_v", "e_agg"):
        assert np.array_equal(r[k].view(np.uint32), g[f"probe_{k}"].view(np.uint32)), k


@pytest.mark.skipif(not oracle.have_reference(), reason="oracle/_ref not built on this machine")
@pytest.mark.parametrize("mode", [0, 1])
def test_port_equals_reference_library_on_fresh_inputs(mode):
    shape = synth.MoEShape(hidden=192, intermediate=96, n_experts=16, top_k=4)
    lw = synth.make_layer(shape, seed=123)
    x = synth.bf16_bits_to_f32(synth.make_tokens(9, shape.hidden, seed=5))
    wr = synth.bf16_bits_to_f32(lw.w_router)
    cache = oracle.ExpertCache(lw.blocks1, lw.scales1, lw.bias1, lw.blocks2, lw.scales2, lw.bias2)
    a = oracle.moe_forward(x, wr, lw.b_router, cache, round_mode=mode, impl="port")
    b = oracle.moe_forward(x, wr, lw.b_router, cache, round_mode=mode, impl="reference")
    assert np.array_equal(a["topk_i"], b["topk_i"])
    for k in ("router_score", "topk_v", "e_agg"):
        assert np.array_equal(a[k].view(np.uint32), b[k].view(np.uint32)), k


def test_swiglu_clamps_and_gate_has_no_lower_clamp():
    # one expert, identity-like weights are awkward in MXFP4; test through expert_rows
    H, I = 32, 32
    w1 = np.zeros((2 * I, H), dtype=np.float32)
    b1 = np.zeros(2 * I, dtype=np.float32)
    w2 = np.eye(H, I, dtype=np.float32)
    b2 = np.zeros(H, dtype=np.float32)
    b1[0], b1[1] = 100.0, 100.0  # gate, up both clamp to 7
    b1[2], b1[3] = -100.0, -100.0  # gate unclamped below, up clamps to -7
    x = np.zeros((1, H), dtype=np.float32)
    y = oracle.expert_rows(x, w1, b1, w2, b2, round_mode=0)
    sig = 1.0 / (1.0 + np.exp(np.float32(-1.702 * 7.0)))
    assert np.isclose(y[0, 0], 7.0 * sig * 8.0, rtol=1e-6)
    assert y[0, 1] == 0.0 or abs(y[0, 1]) < 1e-30  # -100 * sigmoid(-170.2) * (-6) ~ 0


def test_rmsnorm_port_equals_reference_function():
    """oracle_rmsnorm against the reference's compiled rmsnorm (src/run.cpp:306-319),
    bit for bit, and against the formula in numpy."""
    rng = np.random.default_rng(5)
    x = (rng.standard_normal((7, 2880)) * rng.uniform(0.1, 30, size=(7, 1))).astype(np.float32)
    w = (1.0 + 0.1 * rng.standard_normal(2880)).astype(np.float32)
    mine = oracle.rmsnorm(x, w)
    ss = (x.astype(np.float32) ** 2).astype(np.float64).sum(axis=1) / 2880 + np.float64(np.float32(1e-5))
    scale = (np.float32(1.0) / np.sqrt(ss.astype(np.float32))).astype(np.float64)
    want = (w.astype(np.float64) * (scale[:, None] * x.astype(np.float64))).astype(np.float32)
    assert np.abs(mine - want).max() <= 1e-6 * np.abs(want).max()
    if oracle.have_reference():
        ref = oracle.rmsnorm(x, w, impl="reference")
        assert np.array_equal(mine.view(np.uint32), ref.view(np.uint32))
