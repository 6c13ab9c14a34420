"""Shared helpers of the GPU parity tests: run the CUDA path through the C ABI
and the CPU oracle on the same seeded inputs and compare under the stated
tolerances."""
import numpy as np
import torch

import gpt_oss_amd_b200 as pkg
from gpt_oss_amd_b200 import synth
from oracle import oracle

#: tolerances of the output comparison against the bf16-weight / fp32-accumulate
#: numerics (oracle round_mode 1)
REL_L2_TOL = 2e-3
MAX_ABS_TOL = 2e-2
TIE_EPS = 1e-6


def oracle_case(lw, x_bits, round_mode=1, impl="port"):
    shape = lw.shape
    x = synth.bf16_bits_to_f32(x_bits)
    wr = synth.bf16_bits_to_f32(lw.w_router)
    cache = oracle.ExpertCache(lw.blocks1, lw.scales1, lw.bias1, lw.blocks2, lw.scales2, lw.bias2)
    return oracle.moe_forward(x, wr, lw.b_router, cache, top_k=shape.top_k, alpha=shape.alpha,
                              limit=shape.limit, round_mode=round_mode, impl=impl)


def tie_mask(router_score, top_k):
    """True for tokens whose top-(K+1) logits have two neighbours closer than
    TIE_EPS: their expert order is not defined and they are excluded."""
    s = np.sort(router_score.astype(np.float64), axis=1)[:, ::-1]
    k = min(top_k + 1, s.shape[1])
    gaps = s[:, : k - 1] - s[:, 1:k]
    return (gaps < TIE_EPS).any(axis=1)


def compare(out_gpu, topk_i_gpu, topk_w_gpu, ref, top_k, label=""):
    """Asserts the parity rules; returns the measured figures."""
    ties = tie_mask(ref["router_score"], top_k)
    ok = ~ties
    mism = (topk_i_gpu[ok] != ref["topk_i"][ok]).any(axis=1).sum()
    assert mism == 0, f"{label}: {mism} tokens with different expert indices (ties excluded: {ties.sum()})"
    if topk_w_gpu is not None:
        assert np.abs(topk_w_gpu[ok] - ref["topk_v"][ok]).max() < 1e-5, label
    a, b = out_gpu[ok].astype(np.float64), ref["e_agg"][ok].astype(np.float64)
    rel = np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30)
    mx = np.abs(a - b).max() if a.size else 0.0
    assert np.isfinite(a).all(), label
    assert rel <= REL_L2_TOL, f"{label}: rel-L2 {rel:.3e}"
    assert mx <= MAX_ABS_TOL, f"{label}: max-abs {mx:.3e}"
    return {"rel_l2": rel, "max_abs": mx, "ties": int(ties.sum())}


def run_gpu(shape, lw, x_bits, gemm_impl, dtype="bf16", max_tokens=None, accumulate_into=None):
    T = x_bits.shape[0]
    eng = pkg.MoEEngine(shape, n_layers=1, max_tokens=max_tokens or max(T, 1), gemm_impl=gemm_impl)
    try:
        eng.load_layer(0, lw)
        xb = torch.from_numpy(x_bits.view(np.int16)).cuda().view(torch.bfloat16)
        t = xb if dtype == "bf16" else xb.float()
        if accumulate_into is not None:
            out = torch.from_numpy(accumulate_into.copy()).cuda()
            eng.forward(0, t, out=out, accumulate=True)
            sc = ti = tw = None
            out2, sc, ti, tw = eng.forward(0, t, side=True)
        else:
            out, sc, ti, tw = eng.forward(0, t, side=True)
        torch.cuda.synchronize()
        status = eng.device_status()
        assert status == 0, f"device status word 0x{status:x}"
        res = {"out": out.cpu().numpy(), "score": sc.cpu().numpy(), "topk_i": ti.cpu().numpy(),
               "topk_w": tw.cpu().numpy(), "launches": eng.last_launch_count(),
               "counts": eng.last_expert_counts()}
        return res
    finally:
        eng.close()
