"""GPU parity tests (run on a B200 with -m gpu).  Everything goes through the C
ABI; the CPU oracle (already pinned by the CPU tests) is the checker.

Rules: MXFP4 decode bit-exact; top-k expert indices identical except for tokens
whose logits tie within 1e-6; outputs within rel-L2 2e-3 and max-abs 2e-2 of the
bf16-weight / fp32-accumulate numerics."""
import os

import numpy as np
import pytest
import torch

import gpt_oss_amd_b200 as pkg
from gpt_oss_amd_b200 import capi, synth
from oracle import oracle
from parity_util import compare, oracle_case, run_gpu

pytestmark = pytest.mark.gpu

IMPLS = [pytest.param(capi.GEMM_MMA_SYNC, id="mma_sync"), pytest.param(capi.GEMM_TCGEN05, id="tcgen05"),
         pytest.param(capi.GEMM_TCGEN05_1CTA, id="tcgen05_1cta")]


def _bits(t):
    return t.cpu().numpy().view(np.uint16)


# --------------------------------------------------------------------------
# MXFP4 decode


def test_mxfp4_unpack_exhaustive_table(golden_dir):
    table = np.load(os.path.join(golden_dir, "mxfp4_table.npz"))["table"]  # [16, 256]
    pattern = np.array([(2 * i + 1) << 4 | (2 * i) for i in range(8)] * 2, dtype=np.uint8)
    blocks = torch.from_numpy(np.tile(pattern, (256, 1, 1))).cuda()
    scales = torch.arange(256, dtype=torch.uint8).reshape(256, 1).cuda()
    out = _bits(pkg.mxfp4_unpack(blocks, scales))  # [256, 32]
    assert np.array_equal(out[:, :16].T, table)
    assert np.array_equal(out[:, 16:].T, table)


def test_mxfp4_unpack_random_golden(golden_dir):
    r = np.load(os.path.join(golden_dir, "mxfp4_random.npz"))
    for tag in ("full", "cfg"):
        out = _bits(pkg.mxfp4_unpack(torch.from_numpy(r[f"blocks_{tag}"]).cuda(),
                                     torch.from_numpy(r[f"scales_{tag}"]).cuda()))
        assert np.array_equal(out, r[f"out_{tag}"]), tag


def test_mxfp4_unpack_full_size_matrix():
    g = torch.Generator().manual_seed(3)
    blocks = torch.randint(0, 256, (5760, 90, 16), generator=g, dtype=torch.uint8)
    scales = (127 + torch.randint(-8, -3, (5760, 90), generator=g)).to(torch.uint8)
    out = _bits(pkg.mxfp4_unpack(blocks.cuda(), scales.cuda()))
    assert np.array_equal(out, oracle.mxfp4_dequant_bf16(blocks.numpy(), scales.numpy()))


@pytest.mark.parametrize("lo,hi", [(-8, -4), (-127, 1)])
def test_resident_decode_is_bit_exact(lo, hi):
    """The decode the GEMM main loops use (one bf16x2 multiply per pair), applied
    to the re-tiled resident weights, against the oracle -- benchmark scale range
    and the whole supported range of scale bytes 0..128."""
    shape = pkg.MoEShape(hidden=192, intermediate=128, n_experts=4, top_k=2)
    lw = synth.make_layer(shape, seed=11, scale_lo=lo, scale_hi=hi)
    with pkg.MoEEngine(shape, max_tokens=8) as eng:
        eng.load_layer(0, lw)
        for e in range(shape.n_experts):
            w1 = _bits(eng.unpack_resident(0, e, 1))
            w2 = _bits(eng.unpack_resident(0, e, 2))
            assert np.array_equal(w1, oracle.mxfp4_dequant_bf16(lw.blocks1[e], lw.scales1[e]))
            assert np.array_equal(w2, oracle.mxfp4_dequant_bf16(lw.blocks2[e], lw.scales2[e]))


def test_scale_bytes_above_128_are_rejected():
    shape = pkg.MoEShape(hidden=128, intermediate=64, n_experts=4, top_k=2)
    lw = synth.make_layer(shape, seed=1)
    lw.scales2[1, 3, 0] = 129
    with pkg.MoEEngine(shape, max_tokens=8) as eng:
        with pytest.raises(capi.MoEError) as ei:
            eng.load_layer(0, lw)
        assert ei.value.status == capi.ERR_UNSUPPORTED
        assert eng.device_status() == 0


# --------------------------------------------------------------------------
# the block


def test_golden_small_layer(golden_dir):
    """The committed fixture computed by the reference's own CPU functions."""
    g = np.load(os.path.join(golden_dir, "moe_small.npz"))
    shape = pkg.MoEShape(hidden=int(g["hidden"]), intermediate=int(g["intermediate"]),
                         n_experts=int(g["n_experts"]), top_k=int(g["top_k"]))
    lw = synth.LayerWeights(shape, g["w_router_bits"], g["b_router"], g["blocks1"], g["scales1"],
                            g["bias1"], g["blocks2"], g["scales2"], g["bias2"])
    ref = {"router_score": g["bf16_router_score"], "topk_i": g["bf16_topk_i"],
           "topk_v": g["bf16_topk_v"], "e_agg": g["bf16_e_agg"]}
    for impl in (capi.GEMM_MMA_SYNC, capi.GEMM_TCGEN05):
        res = run_gpu(shape, lw, g["x_bits"], impl)
        del res["h_bits"]  # the fixture holds no intermediate: plain comparison
        compare(res, ref, shape.top_k, f"golden impl {impl}")
        assert np.abs(res["score"] - ref["router_score"]).max() < 1e-5


CASES = [
    # (H, I, E, K, T)   ragged and empty experts, single token, E not a multiple of 32
    (128, 64, 8, 4, 1),
    (128, 64, 8, 4, 3),
    (192, 128, 4, 2, 64),
    (256, 192, 32, 4, 65),
    (128, 128, 40, 4, 130),
    (320, 64, 128, 4, 257),
    (128, 64, 8, 1, 33),
    (128, 64, 16, 8, 17),
    (128, 64, 32, 4, 2500),   # above the small-batch routing threshold
    (128, 64, 128, 4, 2100),
    (320, 192, 4, 2, 700),    # large-batch GEMM kernel with partial weight tiles
]


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("H,I,E,K,T", CASES)
def test_block_matches_oracle(H, I, E, K, T, impl):
    shape = pkg.MoEShape(hidden=H, intermediate=I, n_experts=E, top_k=K)
    lw = synth.make_layer(shape, seed=H + E + T)
    x_bits = synth.make_tokens(T, H, seed=T)
    ref = oracle_case(lw, x_bits)
    res = run_gpu(shape, lw, x_bits, impl)
    compare(res, ref, K, f"{(H, I, E, K, T)}")
    assert sum(res["counts"]) == T * K
    hist = np.bincount(ref["topk_i"].reshape(-1), minlength=E)
    assert list(hist) == res["counts"]


@pytest.mark.parametrize("impl", IMPLS)
def test_fp32_input_and_accumulate(impl):
    shape = pkg.MoEShape(hidden=128, intermediate=64, n_experts=8, top_k=4)
    lw = synth.make_layer(shape, seed=5)
    x_bits = synth.make_tokens(40, 128, seed=9)
    ref = oracle_case(lw, x_bits)
    base = np.random.default_rng(0).standard_normal((40, 128)).astype(np.float32)
    res = run_gpu(shape, lw, x_bits, impl, dtype="f32", accumulate_into=base)
    # out = base + e_agg, the residual add of the engine (src/hip/vecadd.hip:19-38)
    assert np.abs((res["out"] - base) - ref["e_agg"]).max() <= 2e-2


@pytest.mark.parametrize("impl", IMPLS)
def test_all_tokens_to_one_expert(impl):
    """Maximum skew: a router bias that sends every token to the same experts."""
    shape = pkg.MoEShape(hidden=128, intermediate=64, n_experts=8, top_k=2)
    lw = synth.make_layer(shape, seed=2)
    lw.b_router[:] = -50.0
    lw.b_router[5] = 50.0
    lw.b_router[2] = 40.0
    x_bits = synth.make_tokens(300, 128, seed=4)
    ref = oracle_case(lw, x_bits)
    res = run_gpu(shape, lw, x_bits, impl)
    compare(res, ref, 2, "one expert")
    assert res["counts"][5] == 300 and res["counts"][2] == 300


def test_config0_full_size_layer():
    """gpt-oss-20b-shaped layer, 64 tokens (the reference's CPU-runnable case)."""
    shape = pkg.MoEShape()  # H = I = 2880, E = 32, K = 4
    lw = synth.make_layer(shape, seed=0)
    x_bits = synth.make_tokens(64, shape.hidden, seed=0)
    ref = oracle_case(lw, x_bits)
    for impl in (capi.GEMM_MMA_SYNC, capi.GEMM_TCGEN05):
        res = run_gpu(shape, lw, x_bits, impl)
        m = compare(res, ref, 4, f"config 0 impl {impl}")
        print("config0", impl, m)


def test_tcgen05_equals_mma_sync_at_prefill_size():
    """Too large for the CPU oracle: the two GEMM implementations must agree
    (same rounding points, only the fp32 summation order differs), with a token
    sample checked against the oracle."""
    shape = pkg.MoEShape()
    lw = synth.make_layer(shape, seed=21, zipf_s=1.1, zipf_gain=1.0)
    T = 2048
    x_bits = synth.make_tokens(T, shape.hidden, seed=21)
    a = run_gpu(shape, lw, x_bits, capi.GEMM_MMA_SYNC)
    b = run_gpu(shape, lw, x_bits, capi.GEMM_TCGEN05)
    assert np.array_equal(a["topk_i"], b["topk_i"])
    d = a["out"].astype(np.float64) - b["out"].astype(np.float64)
    assert np.linalg.norm(d) / np.linalg.norm(a["out"].astype(np.float64)) < 5e-4
    assert max(a["counts"]) > 2 * (T * 4 / 32)  # the skew is real
    sample = np.arange(0, T, T // 16)
    ref = oracle_case(lw, x_bits[sample])
    sub = {k: b[k][sample] for k in ("out", "topk_i", "topk_w", "h_bits")}
    print("prefill sample", compare(sub, ref, 4, "prefill sample"))


# --------------------------------------------------------------------------
# error behaviour of the ABI


def test_error_codes():
    shape = pkg.MoEShape(hidden=128, intermediate=64, n_experts=8, top_k=4)
    lw = synth.make_layer(shape, seed=1)
    with pkg.MoEEngine(shape, max_tokens=8) as eng:
        t = torch.zeros(4, 128, dtype=torch.bfloat16, device="cuda")
        with pytest.raises(capi.MoEError) as ei:
            eng.forward(0, t)
        assert ei.value.status == capi.ERR_NOT_LOADED
        eng.load_layer(0, lw)
        with pytest.raises(capi.MoEError) as ei:
            eng.forward(0, torch.zeros(9, 128, dtype=torch.bfloat16, device="cuda"))
        assert ei.value.status == capi.ERR_INVALID
        with pytest.raises(capi.MoEError) as ei:
            eng.forward(3, t)
        assert ei.value.status == capi.ERR_INVALID
        out = eng.forward(0, t[:0])  # empty batch is fine
        assert out.shape == (0, 128)
        eng.forward(0, t)
        assert eng.device_status() == 0


def test_forward_host_matches_device_path():
    shape = pkg.MoEShape(hidden=128, intermediate=64, n_experts=8, top_k=4)
    lw = synth.make_layer(shape, seed=3)
    x_bits = synth.make_tokens(50, 128, seed=3)
    with pkg.MoEEngine(shape, max_tokens=64) as eng:
        eng.load_layer(0, lw)
        t = torch.from_numpy(x_bits.view(np.int16)).view(torch.bfloat16)
        dev = eng.forward(0, t.cuda()).cpu()
        out = torch.empty(50, 128, dtype=torch.float32).pin_memory()
        eng.forward_host(0, t.pin_memory(), out)
        assert torch.equal(out, dev)


def test_forward_host_chunked_equals_device_path():
    """Large batches go through the host-buffer entry point in token chunks whose
    copies overlap the compute: same bits as one call on device buffers."""
    shape = pkg.MoEShape(hidden=128, intermediate=64, n_experts=8, top_k=4)
    lw = synth.make_layer(shape, seed=4)
    T = 5000  # two chunks of 2560 tokens
    x_bits = synth.make_tokens(T, 128, seed=4)
    with pkg.MoEEngine(shape, max_tokens=T) as eng:
        eng.load_layer(0, lw)
        t = torch.from_numpy(x_bits.view(np.int16)).view(torch.bfloat16)
        dev, _, ti, tw = eng.forward(0, t.cuda(), side=True)
        dev, ti, tw = dev.cpu(), ti.cpu(), tw.cpu()
        out = torch.empty(T, 128, dtype=torch.float32).pin_memory()
        eng.forward_host(0, t.pin_memory(), out)
        assert torch.equal(out, dev)
        assert eng.device_status() == 0


def test_router_indices_at_full_width_large_batch():
    """The tensor-core router (batches above the small-batch threshold) at the
    real hidden size and 128 experts: indices against the CPU engine's
    double-accumulated router, ties within 1e-6 excluded."""
    from parity_util import tie_mask

    shape = pkg.MoEShape(hidden=2880, intermediate=64, n_experts=128, top_k=4)
    lw = synth.make_layer(shape, seed=77)
    T = 4096
    x_bits = synth.make_tokens(T, shape.hidden, seed=77)
    scores, ti, tv = oracle.route(synth.bf16_bits_to_f32(x_bits), synth.bf16_bits_to_f32(lw.w_router),
                                  lw.b_router, 4, round_mode=1)
    res = run_gpu(shape, lw, x_bits, capi.GEMM_TCGEN05)
    ok = ~tie_mask(scores, 4)
    err = np.abs(res["score"] - scores).max()
    mism = int((res["topk_i"][ok] != ti[ok]).any(axis=1).sum())
    print("router: max |logit error|", err, "ties excluded", int((~ok).sum()), "mismatches", mism)
    assert mism == 0
    assert err < 2e-6
    assert np.abs(res["topk_w"][ok] - tv[ok]).max() < 1e-5
