"""Writer (and a numpy reader) of the packed expert file that
``moe_b200_load_experts_file`` maps: the MoE weights of a model kept as the
checkpoint has them -- e2m1 blocks, e8m0 scales, fp32 biases -- expert-major,
one page-aligned record per (layer, expert), so that an expert-parallel rank
maps and uploads only its own shard.

This is the MoE half of the reference's exporter
(tools/model_export/gpt-oss-20b/export_model_bin.py): where that script calls
``dequantize_fp4`` on every ``mlp1_weight`` / ``mlp2_weight`` tensor and writes
fp32 (lines 95-133, 246-270), this writer stores the ``.blocks`` / ``.scales``
tensors unchanged.  Everything that is not MoE stays in the engine's ``.bin``
(src/run.cpp:196-235); a copy of its 15-field config header (src/run.cpp:26-46) is
kept in this file so the two can be checked against each other.

Byte layout: csrc/expert_file.hpp.
"""
from __future__ import annotations

import struct
from typing import Iterable

import numpy as np

from .synth import LayerWeights, MoEShape

MAGIC = b"MOEB200\0"
VERSION = 1
HEADER_BYTES = 4096
_HDR = struct.Struct("<8sII11i2fifI5Q")  # magic, version, header_bytes, RefConfig, reserved, 5 offsets

#: the reference's Config fields that are not MoE dimensions (src/run.cpp:26-46), with the
#: gpt-oss values the benchmark configurations name; override through ``extra_config``
DEFAULT_CONFIG = dict(vocab_size=201088, head_dim=64, n_attn_heads=64, n_kv_heads=8, seq_len=1024,
                      initial_context_length=4096, rope_theta=150000.0, rope_scaling_factor=32.0,
                      sliding_window=128)


def _round_up(v: int, a: int) -> int:
    return (v + a - 1) // a * a


def record_layout(H: int, I: int) -> dict:
    """Byte offsets of the six arrays inside a record and the record size."""
    o, r = 0, {}
    for name, n in (("blocks1", 2 * I * (H // 32) * 16), ("scales1", 2 * I * (H // 32)), ("bias1", 2 * I * 4),
                    ("blocks2", H * (I // 32) * 16), ("scales2", H * (I // 32)), ("bias2", H * 4)):
        r[name] = o
        o = _round_up(o + n, 16)
    r["bytes"] = _round_up(o, 4096)
    return r


def router_layer_bytes(H: int, E: int) -> int:
    return _round_up(E * H * 2 + E * 4, 256)


def _header(shape: MoEShape, n_layers: int, extra: dict) -> tuple[bytes, dict]:
    H, I, E = shape.hidden, shape.intermediate, shape.n_experts
    cfg = dict(DEFAULT_CONFIG)
    cfg.update(extra or {})
    rl = record_layout(H, I)
    router_off = HEADER_BYTES
    rbytes = router_layer_bytes(H, E)
    expert_off = _round_up(router_off + rbytes * n_layers, 4096)
    file_bytes = expert_off + rl["bytes"] * n_layers * E
    raw = _HDR.pack(MAGIC, VERSION, HEADER_BYTES, cfg["vocab_size"], H, E, shape.top_k, I, n_layers,
                    cfg["head_dim"], cfg["n_attn_heads"], cfg["n_kv_heads"], cfg["seq_len"],
                    cfg["initial_context_length"], float(cfg["rope_theta"]),
                    float(cfg["rope_scaling_factor"]), cfg["sliding_window"], float(shape.limit), 0,
                    router_off, rbytes, expert_off, rl["bytes"], file_bytes)
    return raw, dict(router_off=router_off, router_layer_bytes=rbytes, expert_off=expert_off,
                     record=rl, file_bytes=file_bytes)


def write_expert_file(path: str, shape: MoEShape, layers: Iterable[LayerWeights], n_layers: int,
                      extra_config: dict | None = None) -> int:
    """Writes ``n_layers`` layers (each a LayerWeights holding ALL experts of the layer,
    in checkpoint layout) and returns the file size.  Layers are consumed one at a
    time, so a model never has to be in memory whole."""
    H, I, E = shape.hidden, shape.intermediate, shape.n_experts
    raw, lay = _header(shape, n_layers, extra_config)
    rl = lay["record"]
    with open(path, "wb") as f:
        f.write(raw)
        f.truncate(lay["file_bytes"])
        count = 0
        for layer, lw in enumerate(layers):
            assert lw.first_expert == 0 and lw.blocks1.shape == (E, 2 * I, H // 32, 16), "a whole layer, please"
            assert lw.scales1.shape == (E, 2 * I, H // 32) and lw.blocks2.shape == (E, H, I // 32, 16)
            f.seek(lay["router_off"] + lay["router_layer_bytes"] * layer)
            f.write(np.ascontiguousarray(lw.w_router, dtype=np.uint16).tobytes())
            f.write(np.ascontiguousarray(lw.b_router, dtype=np.float32).tobytes())
            for e in range(E):
                base = lay["expert_off"] + rl["bytes"] * (layer * E + e)
                for name, arr, dt in (("blocks1", lw.blocks1, np.uint8), ("scales1", lw.scales1, np.uint8),
                                      ("bias1", lw.bias1, np.float32), ("blocks2", lw.blocks2, np.uint8),
                                      ("scales2", lw.scales2, np.uint8), ("bias2", lw.bias2, np.float32)):
                    f.seek(base + rl[name])
                    f.write(np.ascontiguousarray(arr[e], dtype=dt).tobytes())
            count += 1
        assert count == n_layers, f"{count} layers written, {n_layers} announced"
    return lay["file_bytes"]


def read_header(path: str) -> dict:
    with open(path, "rb") as f:
        raw = f.read(_HDR.size)
    v = _HDR.unpack(raw)
    if v[0] != MAGIC or v[1] != VERSION:
        raise ValueError(f"{path}: not a packed expert file")
    names = ["vocab_size", "hidden_dim", "n_experts", "experts_per_token", "intermediate_dim", "n_layers",
             "head_dim", "n_attn_heads", "n_kv_heads", "seq_len", "initial_context_length", "rope_theta",
             "rope_scaling_factor", "sliding_window", "swiglu_limit"]
    cfg = dict(zip(names, v[3:18]))
    return dict(config=cfg, header_bytes=v[2], router_off=v[19], router_layer_bytes=v[20],
                expert_off=v[21], record_bytes=v[22], file_bytes=v[23])


def read_layer(path: str, layer: int, first: int = 0, n: int | None = None) -> LayerWeights:
    """Experts [first, first + n) of one layer back as LayerWeights (memory-mapped
    reads of just those records): the numpy twin of the library's loader."""
    h = read_header(path)
    c = h["config"]
    H, I, E = c["hidden_dim"], c["intermediate_dim"], c["n_experts"]
    n = E - first if n is None else n
    rl = record_layout(H, I)
    assert rl["bytes"] == h["record_bytes"]
    mm = np.memmap(path, dtype=np.uint8, mode="r")
    r0 = h["router_off"] + h["router_layer_bytes"] * layer
    w_router = np.array(mm[r0:r0 + E * H * 2]).view(np.uint16).reshape(E, H)
    b_router = np.array(mm[r0 + E * H * 2:r0 + E * H * 2 + E * 4]).view(np.float32)

    def take(name, shape, dt):
        out = np.empty((n,) + shape, dtype=dt)
        nbytes = int(np.prod(shape)) * np.dtype(dt).itemsize
        for i in range(n):
            base = h["expert_off"] + rl["bytes"] * (layer * E + first + i) + rl[name]
            out[i] = np.array(mm[base:base + nbytes]).view(dt).reshape(shape)
        return out

    shape = MoEShape(hidden=H, intermediate=I, n_experts=E, top_k=c["experts_per_token"],
                     limit=c["swiglu_limit"])
    return LayerWeights(shape, w_router, b_router,
                        take("blocks1", (2 * I, H // 32, 16), np.uint8), take("scales1", (2 * I, H // 32), np.uint8),
                        take("bias1", (2 * I,), np.float32), take("blocks2", (H, I // 32, 16), np.uint8),
                        take("scales2", (H, I // 32), np.uint8), take("bias2", (H,), np.float32),
                        first_expert=first)
