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
from parity_util import compare, compare_sampled, oracle_case, run_gpu

pytestmark = pytest.mark.gpu

# GEMM_MMA_SYNC is the plain warp-MMA cross-check kernel of the test-aids build
IMPLS = [pytest.param(capi.GEMM_MMA_SYNC, id="mma_sync"), pytest.param(capi.GEMM_TCGEN05, id="tcgen05")]


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


@pytest.mark.parametrize("lo,hi", [(-8, -4), (-127, 1), (0, 128), (-127, 128)])
def test_resident_decode_is_bit_exact(lo, hi):
    """The decode the GEMM main loops use (one bf16x2 multiply per pair, times the
    row's exponent shift), applied to the re-tiled resident weights, against the
    oracle -- benchmark scale range, scale bytes 0..128 (no shift), 127..255 and
    the whole range 0..255 with every row's spread held to 128 binades."""
    shape = pkg.MoEShape(hidden=192, intermediate=128, n_experts=4, top_k=2)
    lw = synth.make_layer(shape, seed=11, scale_lo=lo, scale_hi=hi)
    if hi - lo > 128:
        # every row draws its own window of 129 consecutive scale bytes
        rng = np.random.default_rng(5)
        for sc in (lw.scales1, lw.scales2):
            base = rng.integers(0, 256 - 128, size=sc.shape[:2] + (1,))
            sc[...] = (base + rng.integers(0, 129, size=sc.shape)).astype(np.uint8)
        assert lw.scales1.max() > 200 and lw.scales1.min() < 20
    with pkg.MoEEngine(shape, max_tokens=8) as eng:
        eng.load_layer(0, lw)
        for e in range(shape.n_experts):
            w1 = _bits(eng.unpack_resident(0, e, 1))
            w2 = _bits(eng.unpack_resident(0, e, 2))
            assert np.array_equal(w1, oracle.mxfp4_dequant_bf16(lw.blocks1[e], lw.scales1[e]))
            assert np.array_equal(w2, oracle.mxfp4_dequant_bf16(lw.blocks2[e], lw.scales2[e]))


def test_row_with_scale_spread_above_128_is_rejected():
    """One weight row may span 128 binades of block scales; a block of zeros does not count."""
    shape = pkg.MoEShape(hidden=128, intermediate=64, n_experts=4, top_k=2)
    lw = synth.make_layer(shape, seed=1)
    lw.scales2[1, 3, 0] = 200
    lw.scales2[1, 3, 1] = 71
    lw.blocks2[1, 3, 1, :] = 0x11   # non-zero codes under the small scale
    with pkg.MoEEngine(shape, max_tokens=8) as eng:
        with pytest.raises(capi.MoEError) as ei:
            eng.load_layer(0, lw)
        assert ei.value.status == capi.ERR_UNSUPPORTED
        assert eng.device_status() == 0
        lw.blocks2[1, 3, 1, :] = 0x80   # only zeros (of either sign) under it: representable
        eng.load_layer(0, lw)
        w2 = _bits(eng.unpack_resident(0, 1, 2))
        assert np.array_equal(w2, oracle.mxfp4_dequant_bf16(lw.blocks2[1], lw.scales2[1]))


@pytest.mark.parametrize("impl", IMPLS)
def test_block_with_large_scale_bytes(impl):
    """Scale bytes above 128 on the GEMM path (rows kept with an exponent shift).
    Gate/up matrix: every block scale raised by 2^10 (bytes 129..133) and the tokens
    scaled down by 2^10, so the pre-activations keep their usual size: against the
    oracle.  Down matrix: raising every block scale by 2^9 (bytes 128..132, rows with and
    without a shift) must multiply the output by exactly 2^9 (zero bias)."""
    shape = pkg.MoEShape(hidden=128, intermediate=64, n_experts=8, top_k=2)
    lw = synth.make_layer(shape, seed=21)
    lw.scales1 += 10
    assert lw.scales1.min() == 129
    x_bits = synth.bf16_bits(torch.from_numpy(synth.bf16_bits_to_f32(synth.make_tokens(96, 128, seed=2)) * 2.0 ** -10))
    ref = oracle_case(lw, x_bits)
    res = run_gpu(shape, lw, x_bits, impl)
    print(compare(res, ref, 2, "scales1 + 10"))
    lw.bias2[...] = 0
    small = run_gpu(shape, lw, x_bits, impl, want_h=False)["out"]
    lw.scales2 += 9
    assert lw.scales2.min() == 128 and lw.scales2.max() == 132
    big = run_gpu(shape, lw, x_bits, impl, want_h=False)["out"]
    assert np.array_equal(big, small * np.float32(512.0))


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
    (128, 64, 128, 4, 4000),  # large-batch (CTA-pair) GEMM kernel with 128 experts, 125 rows each
    (192, 128, 128, 4, 9000), # the same above 256 rows per expert: several token tiles per expert
    (128, 64, 64, 4, 9600),   # 64-token routing blocks (above 9472 tokens)
]


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("H,I,E,K,T", CASES)
def test_block_matches_oracle(H, I, E, K, T, impl):
    shape = pkg.MoEShape(hidden=H, intermediate=I, n_experts=E, top_k=K)
    lw = synth.make_layer(shape, seed=H + E + T)
    x_bits = synth.make_tokens(T, H, seed=T)
    ref = oracle_case(lw, x_bits)
    res = run_gpu(shape, lw, x_bits, impl)
    print((H, I, E, K, T), compare(res, ref, K, f"{(H, I, E, K, T)}"))
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
    sub = {k: b[k][sample] for k in ("out", "topk_i", "topk_w", "h_bits")}
    print("prefill sample", compare_sampled(sub, lw, x_bits[sample], lw.w_router, lw.b_router, 4,
                                            "prefill sample"))


def _sample_rows(T, n, seed):
    """n distinct token rows of a batch of T: the first and last rows (tile edges)
    plus a seeded draw from the rest."""
    rng = np.random.default_rng(seed)
    mid = rng.choice(np.arange(1, T - 1), size=n - 2, replace=False)
    return np.sort(np.concatenate([[0, T - 1], mid]))


def test_config3_headline_shape_sampled():
    """The benchmarked configuration itself: gpt-oss-120b-shaped layer, E = 128,
    H = I = 2880, 16384 tokens, uniform routing -- the CTA-pair GEMM with 128-expert
    tile tables and several token tiles per expert.  All 16384 tokens run on the GPU;
    a 32-token sample goes through the CPU oracle (which decodes only the experts
    those tokens touch) with the full rule set, h-flip accounting included."""
    shape = pkg.MoEShape(n_experts=128)
    T = 16384
    lw = synth.make_layer(shape, seed=0)
    x_bits = synth.make_tokens(T, shape.hidden, seed=0)
    res = run_gpu(shape, lw, x_bits, capi.GEMM_TCGEN05)
    assert sum(res["counts"]) == T * 4
    assert min(res["counts"]) > 256  # every expert has more than one token tile
    sample = _sample_rows(T, 32, seed=3)
    sub = {k: res[k][sample] for k in ("out", "topk_i", "topk_w", "h_bits")}
    m = compare_sampled(sub, lw, x_bits[sample], lw.w_router, lw.b_router, 4, "config 3 sample")
    print("config3", m)
    # and every token against the cross-check GEMM (same rounding points, other summation order)
    x = run_gpu(shape, lw, x_bits, capi.GEMM_MMA_SYNC, want_h=False)
    assert np.array_equal(x["topk_i"], res["topk_i"])
    d = x["out"].astype(np.float64) - res["out"].astype(np.float64)
    rel = np.linalg.norm(d) / np.linalg.norm(x["out"].astype(np.float64))
    print("config3 tcgen05 vs mma_sync: rel-L2", rel, "max-abs", np.abs(d).max())
    assert rel < 5e-4
    # the router at this size is the tensor-core kernel: all 16384 index rows against the oracle
    scores, ti, _ = oracle.route(synth.bf16_bits_to_f32(x_bits), synth.bf16_bits_to_f32(lw.w_router),
                                 lw.b_router, 4, round_mode=1)
    from parity_util import tie_mask
    ok = ~tie_mask(scores, 4)
    assert int((res["topk_i"][ok] != ti[ok]).any(axis=1).sum()) == 0
    assert list(np.bincount(ti.reshape(-1), minlength=128)) == res["counts"] or (~ok).any()


def test_config2_zipf_prefill_sampled():
    """gpt-oss-20b-shaped layer, 8192 tokens, Zipf(1.1) router bias scaled so that the
    busiest expert draws about 4x the mean load (the skewed configuration): the
    grouped GEMM with tiles from 1 to ~17 per expert.  32-token oracle sample."""
    shape = pkg.MoEShape()
    T = 8192
    lw = synth.make_layer(shape, seed=0, zipf_s=1.1, zipf_gain=synth.ZIPF_GAIN_4X)
    x_bits = synth.make_tokens(T, shape.hidden, seed=0)
    res = run_gpu(shape, lw, x_bits, capi.GEMM_TCGEN05)
    skew = max(res["counts"]) / (sum(res["counts"]) / len(res["counts"]))
    assert 3.5 < skew < 4.5, skew
    sample = _sample_rows(T, 32, seed=5)
    sub = {k: res[k][sample] for k in ("out", "topk_i", "topk_w", "h_bits")}
    m = compare_sampled(sub, lw, x_bits[sample], lw.w_router, lw.b_router, 4, "config 2 sample")
    print("config2 skew", skew, m)


def test_config1_decode_batch_three_layers():
    """The decode-shaped configuration: 256 tokens per step through stacked
    gpt-oss-20b-shaped layers with independent seeds (three of the 24), 32 rows per
    expert -- the small-batch GEMM.  Every token of every layer against the oracle."""
    shape = pkg.MoEShape()
    T, layers = 256, 3
    x_bits = synth.make_tokens(T, shape.hidden, seed=0)
    with pkg.MoEEngine(shape, n_layers=layers, max_tokens=T) as eng:
        lws = []
        for layer in range(layers):
            lw = synth.make_layer(shape, seed=layer)
            eng.load_layer(layer, lw)
            lws.append(lw)
        t = torch.from_numpy(x_bits.view(np.int16)).cuda().view(torch.bfloat16)
        for layer in range(layers):
            out, sc, ti, tw = eng.forward(layer, t, side=True)
            h_bits = eng.last_intermediate(T)
            torch.cuda.synchronize()
            assert eng.device_status() == 0
            res = {"out": out.cpu().numpy(), "topk_i": ti.cpu().numpy(), "topk_w": tw.cpu().numpy(),
                   "h_bits": h_bits.cpu().numpy().view(np.uint16)}
            ref = oracle_case(lws[layer], x_bits)
            print("config1 layer", layer, compare(res, ref, 4, f"config 1 layer {layer}"))
            ref["cache"].drop()


@pytest.mark.parametrize("w_dtype", ["f32", "bf16"])
@pytest.mark.parametrize("H,I,E,T", [(256, 128, 32, 300), (2880, 64, 128, 1500), (2880, 2880, 32, 96)])
def test_fused_rmsnorm_in_front_of_the_block(H, I, E, T, w_dtype):
    """moe_b200_forward_norm: the FFN RMSNorm (src/forward.cpp:315, src/run.cpp:306-319)
    fused into the router kernel.  The oracle is the reference's rmsnorm followed by the
    block; the fused norm reproduces the CPU engine's arithmetic, so the expert indices
    must match like everywhere else.  Also the engine's in-place residual update
    x += MoE(rmsnorm(x)) with out aliasing x."""
    shape = pkg.MoEShape(hidden=H, intermediate=I, n_experts=E, top_k=4)
    lw = synth.make_layer(shape, seed=H + T)
    g = torch.Generator().manual_seed(T)
    x = (torch.randn(T, H, generator=g) * (0.5 + 4.0 * torch.rand(T, 1, generator=g))).float()
    w = (1.0 + 0.2 * torch.randn(H, generator=g)).float()
    w_dev = w.cuda().to(torch.bfloat16) if w_dtype == "bf16" else w.cuda()
    w_ref = w_dev.float().cpu().numpy()
    impl = "reference" if oracle.have_reference() else "port"
    xn = oracle.rmsnorm(x.numpy(), w_ref, impl=impl)
    x_bits = synth.bf16_bits(torch.from_numpy(xn))
    ref = oracle_case(lw, x_bits)
    with pkg.MoEEngine(shape, max_tokens=T) as eng:
        eng.load_layer(0, lw)
        out, sc, ti, tw = eng.forward_norm(0, x.cuda(), w_dev, side=True)
        h_bits = eng.last_intermediate(T)
        torch.cuda.synchronize()
        res = {"out": out.cpu().numpy(), "topk_i": ti.cpu().numpy(), "topk_w": tw.cpu().numpy(),
               "h_bits": h_bits.cpu().numpy().view(np.uint16)}
        print("fused norm", (H, I, E, T, w_dtype), compare(res, ref, 4, "fused norm"))
        assert np.abs(sc.cpu().numpy() - ref["router_score"]).max() < 1e-5
        # the same rows through the separate path: normalised bf16 rows in, identical bits out
        t = torch.from_numpy(x_bits.view(np.int16)).cuda().view(torch.bfloat16)
        assert torch.equal(eng.forward(0, t), out)
        # in place: x += MoE(rmsnorm(x))
        xr = x.cuda().clone()
        eng.forward_norm(0, xr, w_dev, out=xr, accumulate=True)
        torch.cuda.synchronize()
        assert torch.equal(xr, x.cuda() + out)
        assert eng.device_status() == 0


def test_plain_c_caller(tmp_path):
    """tests/c_abi_smoke.c -- a C99 program that includes only include/moe_b200.h and
    links the shipped library, i.e. the engine-side binding as code -- runs a small
    layer through the host-buffer entry point; its outputs are checked against the
    oracle on the inputs it used."""
    import subprocess

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe, dump = tmp_path / "c_abi_smoke", tmp_path / "out.bin"
    lib_dir = os.path.dirname(capi.LIB_PATH)
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Wextra", "-Werror", "-pedantic",
                    "-I", os.path.join(root, "include"), os.path.join(root, "tests", "c_abi_smoke.c"),
                    "-L", lib_dir, "-l:libmoe_b200.so", f"-Wl,-rpath,{lib_dir}", "-o", str(exe)],
                   check=True, capture_output=True, text=True)
    run = subprocess.run([str(exe), str(dump)], capture_output=True, text=True)
    assert run.returncode == 0 and "c_abi_smoke ok" in run.stdout, run.stdout + run.stderr
    assert "no device" not in run.stdout
    raw = open(dump, "rb").read()
    T, H, E, K, I = np.frombuffer(raw, dtype=np.int32, count=5)
    pos = [20]

    def take(dtype, *shape):
        n = int(np.prod(shape)) * np.dtype(dtype).itemsize
        a = np.frombuffer(raw, dtype=dtype, count=int(np.prod(shape)), offset=pos[0]).reshape(shape)
        pos[0] += n
        return a

    x_bits, w_router = take(np.uint16, T, H), take(np.uint16, E, H)
    b_router = take(np.float32, E)
    blocks1, scales1, bias1 = take(np.uint8, E, 2 * I, H // 32, 16), take(np.uint8, E, 2 * I, H // 32), take(np.float32, E, 2 * I)
    blocks2, scales2, bias2 = take(np.uint8, E, H, I // 32, 16), take(np.uint8, E, H, I // 32), take(np.float32, E, H)
    res = {"topk_i": take(np.int32, T, K), "topk_w": take(np.float32, T, K), "out": take(np.float32, T, H)}
    assert pos[0] == len(raw)
    shape = pkg.MoEShape(hidden=int(H), intermediate=int(I), n_experts=int(E), top_k=int(K))
    lw = synth.LayerWeights(shape, w_router, b_router, blocks1, scales1, bias1, blocks2, scales2, bias2)
    ref = oracle_case(lw, x_bits)
    ref.pop("h")
    print("plain C caller", compare(res, ref, int(K), "plain C caller"))


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


def test_unaligned_pointers_are_refused():
    """Rows move 16 bytes at a time; a pointer off that boundary is an argument error,
    not a fault on the GPU."""
    shape = pkg.MoEShape(hidden=128, intermediate=64, n_experts=4, top_k=2)
    lw = synth.make_layer(shape, seed=1)
    with pkg.MoEEngine(shape, max_tokens=16) as eng:
        eng.load_layer(0, lw)
        flat = torch.zeros(8 * 128 + 8, dtype=torch.bfloat16, device="cuda")
        good = flat[:8 * 128].view(8, 128)
        bad = flat[1:1 + 8 * 128].view(8, 128)
        eng.forward(0, good)
        with pytest.raises(capi.MoEError) as ei:
            eng.forward(0, bad)
        assert ei.value.status == capi.ERR_INVALID
        out_flat = torch.zeros(8 * 128 + 4, dtype=torch.float32, device="cuda")
        with pytest.raises(capi.MoEError):
            eng.forward(0, good, out=out_flat[1:1 + 8 * 128].view(8, 128))
        torch.cuda.synchronize()
        assert eng.device_status() == 0


@pytest.mark.parametrize("T", [40, 300, 1000, 3000])
def test_block_is_bit_reproducible(T):
    """Same inputs, same bits: the router's K split over a cluster adds its partial sums in
    rank order, placement is stable, the combine adds in ascending expert order -- nothing
    depends on timing.  The batch sizes cover clusters of 8, 4 and 2 CTAs and none."""
    shape = pkg.MoEShape(hidden=320, intermediate=128, n_experts=40, top_k=4)
    lw = synth.make_layer(shape, seed=17)
    x_bits = synth.make_tokens(T, shape.hidden, seed=T)
    a = run_gpu(shape, lw, x_bits, capi.GEMM_TCGEN05)
    b = run_gpu(shape, lw, x_bits, capi.GEMM_TCGEN05)
    for key in ("out", "score", "topk_i", "topk_w", "h_bits"):
        assert np.array_equal(a[key], b[key]), key
