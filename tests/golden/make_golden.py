"""Generate the golden fixtures in this directory by RUNNING THE REFERENCE.

Needs the reference checkout (its location: the MOE_REFERENCE_ROOT environment
variable, else the default below) and ``make -C oracle ref``; the fixtures it writes are
committed so the tests need neither.

* ``mxfp4_table.npz``   -- every (e2m1 code, e8m0 scale byte) pair decoded by the
  reference's ``dequantize_fp4`` (tools/model_export/gpt-oss-20b/
  export_model_bin.py:95-133), as bf16 bit patterns ``table[16, 256]``.
* ``mxfp4_random.npz``  -- random blocks/scales (full scale-byte range and the
  benchmark range) with the reference's bf16 output bits.
* ``moe_small.npz``     -- a small MoE layer (packed MXFP4 experts) with the
  outputs of the reference's compiled CPU functions: ``ref_moe_forward`` in both
  rounding modes, and the unmodified ``forward()`` probed on a one-layer model.

Run:  python tests/golden/make_golden.py
"""
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
REF = os.environ.get("MOE_REFERENCE_ROOT", "/root/reference")


def load_reference_dequant():
    path = os.path.join(REF, "tools", "model_export", "gpt-oss-20b", "export_model_bin.py")
    spec = importlib.util.spec_from_file_location("ref_export_model_bin", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.dequantize_fp4


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def main():
    dequantize_fp4 = load_reference_dequant()

    # exhaustive table: one block per scale byte whose 32 elements are codes 0..15 twice
    pattern = np.array([(2 * i + 1) << 4 | (2 * i) for i in range(8)] * 2, dtype=np.uint8)
    blocks = np.tile(pattern, (256, 1, 1))  # [256, 1, 16]
    scales = np.arange(256, dtype=np.uint8).reshape(256, 1)
    out = bits(dequantize_fp4(torch.from_numpy(blocks), torch.from_numpy(scales)))  # [256, 32]
    assert (out[:, :16] == out[:, 16:]).all()
    table = out[:, :16].T.copy()  # [code, scale]
    np.savez_compressed(os.path.join(HERE, "mxfp4_table.npz"), table=table)

    g = torch.Generator().manual_seed(20240611)
    b_full = torch.randint(0, 256, (48, 6, 16), generator=g, dtype=torch.uint8)
    s_full = torch.randint(0, 256, (48, 6), generator=g, dtype=torch.uint8)
    b_cfg = torch.randint(0, 256, (64, 4, 16), generator=g, dtype=torch.uint8)
    s_cfg = (127 + torch.randint(-8, -3, (64, 4), generator=g)).to(torch.uint8)
    np.savez_compressed(
        os.path.join(HERE, "mxfp4_random.npz"),
        blocks_full=b_full.numpy(), scales_full=s_full.numpy(),
        out_full=bits(dequantize_fp4(b_full, s_full)),
        blocks_cfg=b_cfg.numpy(), scales_cfg=s_cfg.numpy(),
        out_cfg=bits(dequantize_fp4(b_cfg, s_cfg)),
    )

    # small MoE layer through the reference's compiled CPU code
    import gpt_oss_amd_b200.synth as synth
    from oracle import oracle

    assert oracle.have_reference(), "run `make -C oracle ref` first"
    shape = synth.MoEShape(hidden=128, intermediate=64, n_experts=8, top_k=4)
    lw = synth.make_layer(shape, seed=7)
    T = 12
    x_bits = synth.make_tokens(T, shape.hidden, seed=7)
    x = synth.bf16_bits_to_f32(x_bits)
    wr = synth.bf16_bits_to_f32(lw.w_router)
    cache = oracle.ExpertCache(lw.blocks1, lw.scales1, lw.bias1, lw.blocks2, lw.scales2, lw.bias2)
    r0 = oracle.moe_forward(x, wr, lw.b_router, cache, round_mode=0, impl="reference")
    r1 = oracle.moe_forward(x, wr, lw.b_router, cache, round_mode=1, impl="reference")
    w1 = np.stack([cache.w1(e) for e in range(shape.n_experts)])
    w2 = np.stack([cache.w2(e) for e in range(shape.n_experts)])
    probe = oracle.reference_forward_probe(x, wr, lw.b_router, w1, lw.bias1, w2, lw.bias2)
    np.savez_compressed(
        os.path.join(HERE, "moe_small.npz"),
        hidden=shape.hidden, intermediate=shape.intermediate, n_experts=shape.n_experts,
        top_k=shape.top_k, x_bits=x_bits, w_router_bits=lw.w_router, b_router=lw.b_router,
        blocks1=lw.blocks1, scales1=lw.scales1, bias1=lw.bias1,
        blocks2=lw.blocks2, scales2=lw.scales2, bias2=lw.bias2,
        f32_router_score=r0["router_score"], f32_topk_i=r0["topk_i"], f32_topk_v=r0["topk_v"],
        f32_e_agg=r0["e_agg"],
        bf16_router_score=r1["router_score"], bf16_topk_i=r1["topk_i"], bf16_topk_v=r1["topk_v"],
        bf16_e_agg=r1["e_agg"],
        probe_t=probe["t"], probe_router_score=probe["router_score"], probe_topk_i=probe["topk_i"],
        probe_topk_v=probe["topk_v"], probe_e_agg=probe["e_agg"],
    )
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
