"""Shared helpers of the GPU parity tests: run the CUDA path through the C ABI
and the CPU oracle on the same seeded inputs and compare under the stated
tolerances (the rules themselves live in oracle/parity.py, which the parity
record of bench.py uses too).

Every comparison returns -- and the tests print -- both the RAW max-abs error
and the one left after removing the effect of identified one-ulp bf16 flips of
the intermediate h; the raw figure has its own asserted ceiling.
"""
import numpy as np
import torch

import gpt_oss_amd_b200 as pkg
from gpt_oss_amd_b200 import synth
from oracle import oracle, parity
from oracle.parity import tie_mask  # noqa: F401  (re-exported for the tests)

REL_L2_TOL = parity.REL_L2_TOL
MAX_ABS_TOL = parity.MAX_ABS_TOL
RAW_MAX_ABS_CEILING = parity.RAW_MAX_ABS_CEILING


def expert_cache(lw):
    return oracle.ExpertCache(lw.blocks1, lw.scales1, lw.bias1, lw.blocks2, lw.scales2, lw.bias2,
                              first_expert=lw.first_expert)


def oracle_case(lw, x_bits, round_mode=1, impl="port", cache=None):
    shape = lw.shape
    x = synth.bf16_bits_to_f32(x_bits)
    wr = synth.bf16_bits_to_f32(lw.w_router)
    cache = cache or expert_cache(lw)
    ref = oracle.moe_forward(x, wr, lw.b_router, cache, top_k=shape.top_k, alpha=shape.alpha,
                             limit=shape.limit, round_mode=round_mode, impl=impl,
                             want_h=(impl == "port"))
    ref["cache"] = cache
    return ref


def compare(res, ref, top_k, label=""):
    """Asserts the parity rules; returns the measured figures (rel_l2,
    max_abs_raw, max_abs_adjusted, h_flips, ...).  `res`: dict from run_gpu;
    `ref`: dict from oracle_case."""
    m = parity.finish(parity.merge([parity.measure(res, ref, top_k)]))
    assert m["ok"], f"{label}: {m['why']}"
    return m


def compare_sampled(res, lw_or_loader, x_bits, w_router_bits, b_router, top_k, label="", group=8):
    """Like compare() for a token sample of a full-size layer: the oracle decodes
    only the experts each group of tokens touches.  `lw_or_loader`: LayerWeights
    holding all experts packed, or a function e -> packed arrays of expert e."""
    if callable(lw_or_loader):
        loader = lw_or_loader
    else:
        lw = lw_or_loader
        loader = lambda e: tuple(a[e - lw.first_expert:e - lw.first_expert + 1] for a in (
            lw.blocks1, lw.scales1, lw.bias1, lw.blocks2, lw.scales2, lw.bias2))
    m = parity.compare_sampled(res, x_bits, w_router_bits, b_router, loader, top_k, group=group)
    assert m["ok"], f"{label}: {m['why']}"
    return m


def run_gpu(shape, lw, x_bits, gemm_impl, dtype="bf16", max_tokens=None, accumulate_into=None,
            want_h=True):
    T = x_bits.shape[0]
    eng = pkg.MoEEngine(shape, n_layers=1, max_tokens=max_tokens or max(T, 1), gemm_impl=gemm_impl)
    try:
        eng.load_layer(0, lw)
        xb = torch.from_numpy(x_bits.view(np.int16)).cuda().view(torch.bfloat16)
        t = xb if dtype == "bf16" else xb.float()
        if accumulate_into is not None:
            out = torch.from_numpy(accumulate_into.copy()).cuda()
            eng.forward(0, t, out=out, accumulate=True)
            _, sc, ti, tw = eng.forward(0, t, side=True)
        else:
            out, sc, ti, tw = eng.forward(0, t, side=True)
        h_bits = eng.last_intermediate(T) if want_h else None
        torch.cuda.synchronize()
        status = eng.device_status()
        assert status == 0, f"device status word 0x{status:x}"
        res = {"out": out.cpu().numpy(), "score": sc.cpu().numpy(), "topk_i": ti.cpu().numpy(),
               "topk_w": tw.cpu().numpy(), "launches": eng.last_launch_count(),
               "counts": eng.last_expert_counts()}
        if want_h:
            res["h_bits"] = h_bits.cpu().numpy().view(np.uint16)
        return res
    finally:
        eng.close()
