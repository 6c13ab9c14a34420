"""Packed expert file (the on-disk form of the MoE weights): writer -> reader round
trips on the CPU, the library's header check, and -- on a GPU -- that a layer loaded
from a file is bit for bit the layer loaded from arrays, for a whole layer and for
an expert-parallel shard."""
import ctypes
import os

import numpy as np
import pytest
import torch

import gpt_oss_amd_b200 as pkg
from gpt_oss_amd_b200 import capi, expert_file, synth

SHAPE = dict(hidden=192, intermediate=128, n_experts=6, top_k=2)


def _write(tmp_path, n_layers=3, shape_kw=SHAPE):
    shape = pkg.MoEShape(**shape_kw)
    layers = [synth.make_layer(shape, seed=10 + i) for i in range(n_layers)]
    path = str(tmp_path / "experts.moe4")
    size = expert_file.write_expert_file(path, shape, iter(layers), n_layers)
    assert os.path.getsize(path) == size
    return shape, layers, path


def _info(path):
    L = capi.lib()
    ints = [ctypes.c_int() for _ in range(5)]
    lim, nbytes = ctypes.c_float(), ctypes.c_ulonglong()
    st = L.moe_b200_expert_file_info(path.encode(), *[ctypes.byref(i) for i in ints], ctypes.byref(lim),
                                     ctypes.byref(nbytes))
    return st, [i.value for i in ints], lim.value, nbytes.value


def test_writer_reader_round_trip(tmp_path):
    shape, layers, path = _write(tmp_path)
    h = expert_file.read_header(path)
    assert h["config"]["hidden_dim"] == 192 and h["config"]["n_layers"] == 3
    assert h["record_bytes"] % 4096 == 0 and h["expert_off"] % 4096 == 0
    # the copy of the engine's 15-field header carries the non-MoE fields too
    assert h["config"]["vocab_size"] == 201088 and h["config"]["sliding_window"] == 128
    assert abs(h["config"]["swiglu_limit"] - 7.0) < 1e-6
    for layer, lw in enumerate(layers):
        for first, n in ((0, None), (4, 2), (1, 3)):  # whole layer and two shards
            got = expert_file.read_layer(path, layer, first, n)
            sl = slice(first, None if n is None else first + n)
            assert np.array_equal(got.w_router, lw.w_router) and np.array_equal(got.b_router, lw.b_router)
            for name in ("blocks1", "scales1", "bias1", "blocks2", "scales2", "bias2"):
                assert np.array_equal(getattr(got, name), getattr(lw, name)[sl]), (layer, first, name)
    # packed: 4.25 bits per weight plus biases, not the 32 of the fp32 .bin
    weights = 3 * 6 * (2 * 128 * 192 + 192 * 128)
    assert os.path.getsize(path) < weights * 4 / 4


def test_library_reads_and_validates_the_header(tmp_path):
    shape, layers, path = _write(tmp_path)
    st, ints, lim, nbytes = _info(path)
    assert st == capi.OK
    assert ints == [3, 6, 192, 128, 2] and abs(lim - 7.0) < 1e-6
    assert nbytes == os.path.getsize(path)
    # truncated file, foreign file, missing file: refused with a reason, never a crash
    raw = open(path, "rb").read()
    cut = str(tmp_path / "cut.moe4")
    open(cut, "wb").write(raw[:len(raw) - 5000])
    assert _info(cut)[0] == capi.ERR_INVALID
    assert b"truncated" in capi.lib().moe_b200_last_error(None)
    bad = str(tmp_path / "bad.moe4")
    open(bad, "wb").write(b"NOTMAGIC" + raw[8:])
    assert _info(bad)[0] == capi.ERR_INVALID
    assert _info(str(tmp_path / "nope.moe4"))[0] == capi.ERR_INVALID
    # a header whose offsets do not follow from its dimensions
    forged = bytearray(raw)
    forged[16 + 4:16 + 8] = (256).to_bytes(4, "little")  # hidden_dim 192 -> 256
    fp = str(tmp_path / "forged.moe4")
    open(fp, "wb").write(bytes(forged))
    assert _info(fp)[0] == capi.ERR_INVALID


@pytest.mark.gpu
def test_file_loaded_layer_equals_array_loaded_layer(tmp_path):
    shape, layers, path = _write(tmp_path)
    x_bits = synth.make_tokens(70, shape.hidden, seed=1)
    t = torch.from_numpy(x_bits.view(np.int16)).cuda().view(torch.bfloat16)
    with pkg.MoEEngine(shape, n_layers=2, max_tokens=128) as a, pkg.MoEEngine(shape, n_layers=2, max_tokens=128) as b:
        a.load_layer(0, layers[2])
        a.load_layer(1, layers[0])
        b.load_layer_file(path, 2, 0)  # file layer 2 -> handle layer 0
        b.load_layer_file(path, 0, 1)
        for layer in range(2):
            for e in range(shape.n_experts):
                for which in (1, 2):
                    assert torch.equal(a.unpack_resident(layer, e, which), b.unpack_resident(layer, e, which))
            oa, sa, ia, wa = a.forward(layer, t, side=True)
            ob, sb, ib, wb = b.forward(layer, t, side=True)
            assert torch.equal(oa, ob) and torch.equal(sa, sb) and torch.equal(ia, ib) and torch.equal(wa, wb)
        assert a.device_status() == 0 and b.device_status() == 0
        # wrong dimensions and a layer the file does not have are refused
        with pytest.raises(capi.MoEError) as ei:
            b.load_layer_file(path, 3, 0)
        assert ei.value.status == capi.ERR_INVALID
    other = pkg.MoEShape(hidden=256, intermediate=128, n_experts=6, top_k=2)
    with pkg.MoEEngine(other, max_tokens=8) as c:
        with pytest.raises(capi.MoEError) as ei:
            c.load_layer_file(path, 0, 0)
        assert ei.value.status == capi.ERR_INVALID


@pytest.mark.gpu
def test_expert_parallel_rank_loads_only_its_shard(tmp_path):
    """A handle created as rank 1 of 4 uploads experts [2, 4) of 6 (src/model.cpp:104-114:
    2, 2, 1, 1) and nothing else; one GPU is enough, no exchange is set up."""
    shape, layers, path = _write(tmp_path, n_layers=1)
    with pkg.MoEEngine(shape, max_tokens=16, ep_rank=1, ep_size=4) as eng:
        assert (eng.first_expert, eng.n_local) == (2, 2)
        eng.load_layer_file(path, 0)
        with pkg.MoEEngine(shape, max_tokens=16) as whole:
            whole.load_layer(0, layers[0])
            for le in range(2):
                for which in (1, 2):
                    assert torch.equal(eng.unpack_resident(0, le, which), whole.unpack_resident(0, 2 + le, which))
