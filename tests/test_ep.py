"""Expert-parallel path (N > 1).

* CPU (gloo, world size 2 and 3): the exchange protocol of csrc/ep.cuh -- sort
  by global expert, all-gather of counts, the host plan of moe_b200_ep_plan,
  dispatch, regroup by local expert, return in the sender's order, combine --
  restated over gloo with the oracle computing the experts, against a
  single-process oracle run.
* GPU (needs >= 2 devices): one process per GPU, the exchange inside the
  library over NCCL and over peer memory, against the oracle and against the
  single-GPU run.
"""
import os
import socket
import tempfile

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

import ep_workers
import gpt_oss_amd_b200 as pkg
from gpt_oss_amd_b200 import capi, synth
from parity_util import compare, oracle_case, run_gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


SHAPE = dict(hidden=128, intermediate=64, n_experts=10, top_k=4)


@pytest.mark.parametrize("world", [2, 3])
def test_exchange_protocol_over_gloo(world):
    T, seed = 41, 3
    shape = pkg.MoEShape(**SHAPE)
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(ep_workers.cpu_worker, args=(world, _free_port(), SHAPE, T, seed, d), nprocs=world,
                 join=True)
        parts = [np.load(os.path.join(d, f"cpu_rank{r}.npz")) for r in range(world)]
    out = np.concatenate([p["out"] for p in parts])
    topk_i = np.concatenate([p["topk_i"] for p in parts])
    assert [int(p["start"]) for p in parts] == list(ep_workers.split_tokens(T, world)[:-1])
    lw = synth.make_layer(shape, seed)
    ref = oracle_case(lw, synth.make_tokens(T, shape.hidden, seed))
    assert np.array_equal(topk_i, ref["topk_i"])
    # same arithmetic per row; only the combine's fused multiply-add differs
    assert np.abs(out - ref["e_agg"]).max() <= 1e-5 * max(1.0, np.abs(ref["e_agg"]).max())


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["nccl", "peer"])
@pytest.mark.parametrize("impl", [capi.GEMM_MMA_SYNC, capi.GEMM_TCGEN05])
def test_expert_parallel_on_gpus(impl, mode):
    world = min(torch.cuda.device_count(), 8)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    if impl == capi.GEMM_MMA_SYNC and mode == "peer":
        pytest.skip("the cross-check GEMM does not take part in the peer-memory exchange")
    T, seed = 300, 5
    shape_kw = dict(hidden=256, intermediate=128, n_experts=16, top_k=4)
    shape = pkg.MoEShape(**shape_kw)
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(ep_workers.gpu_worker, args=(world, _free_port(), shape_kw, T, seed, d, impl, mode),
                 nprocs=world, join=True)
        parts = [dict(np.load(os.path.join(d, f"gpu_rank{r}.npz"))) for r in range(world)]
    assert all(int(p["status"]) == 0 for p in parts)
    res = {k: np.concatenate([p[k] for p in parts]) for k in ("out", "topk_i", "topk_w")}
    lw = synth.make_layer(shape, seed)
    x_bits = synth.make_tokens(T, shape.hidden, seed)
    ref = oracle_case(lw, x_bits)
    ref.pop("h")
    m = compare(res, ref, shape.top_k, f"ep{world}-{mode}")
    print("ep", world, m)
    # every rank computed exactly its shard's rows
    hist = np.bincount(ref["topk_i"].reshape(-1), minlength=shape.n_experts)
    assert list(np.concatenate([p["counts"] for p in parts])) == list(hist)
    # second call (last rank without tokens): the other ranks' results do not change
    for r in range(world - 1):
        assert np.allclose(parts[r]["out2"], parts[r]["out"], rtol=0, atol=2e-3)
    assert parts[-1]["out2"].shape[0] == 0
    # third call, everybody again: the same bits as the first
    for r in range(world):
        assert np.array_equal(parts[r]["out3"], parts[r]["out"])
    # and the expert-parallel result agrees with the single-GPU result of the same library
    # (not bit for bit: fewer rows per expert pick a narrower GEMM tile, whose K loop is
    # split over more accumulators, and a differently rounded h element can flip in bf16)
    single = run_gpu(shape, lw, x_bits, impl)
    d = single["out"].astype(np.float64) - res["out"].astype(np.float64)
    assert np.linalg.norm(d) / np.linalg.norm(single["out"].astype(np.float64)) <= 1e-4
    assert np.abs(d).max() <= 2e-3


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["nccl", "peer"])
def test_expert_parallel_full_width_pair_kernel(mode):
    """gpt-oss-120b-shaped layer (E = 128, H = I = 2880), 4096 tokens over all the GPUs
    of the box: 128 rows per expert, i.e. the CTA-pair GEMM under expert parallelism.
    Every rank checks eight of its own tokens against the CPU oracle."""
    import json

    world = min(torch.cuda.device_count(), 8)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    T, seed = 4096, 0
    shape_kw = dict(hidden=2880, intermediate=2880, n_experts=128, top_k=4)
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(ep_workers.gpu_worker,
                 args=(world, _free_port(), shape_kw, T, seed, d, capi.GEMM_TCGEN05, mode, 8),
                 nprocs=world, join=True)
        parts = [dict(np.load(os.path.join(d, f"gpu_rank{r}.npz"))) for r in range(world)]
    assert all(int(p["status"]) == 0 for p in parts)
    assert sum(int(p["counts"].sum()) for p in parts) == T * 4
    for r, p in enumerate(parts):
        m = json.loads(str(p["figures"]))
        print("ep full width", mode, "rank", r, m)
        assert m["ok"], m["why"]
        assert np.array_equal(p["out3"], p["out"])


@pytest.mark.gpu
def test_missing_rank_is_reported_not_hung():
    """A rank that does not join an expert-parallel call: the host-made failure.  The
    other rank's bounded flag waits run out, the status word says which wait, nothing
    faults and the context stays usable; after the ranks have re-aligned their call
    counters the next joint call is right."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    shape_kw = dict(hidden=128, intermediate=64, n_experts=8, top_k=2)
    T, seed = 40, 1
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(ep_workers.gpu_missing_rank_worker, args=(2, _free_port(), shape_kw, T, seed, d),
                 nprocs=2, join=True)
        parts = [dict(np.load(os.path.join(d, f"miss_rank{r}.npz"))) for r in range(2)]
    r0 = parts[0]
    assert int(r0["status"]) == 0x301  # DS_TIMEOUT_PEER (csrc/peer_io.cuh)
    assert bool(r0["usable"])
    assert list(r0["seqs"]) == [1, 0]
    assert all(int(p["status_after"]) == 0 for p in parts)
    shape = pkg.MoEShape(**shape_kw)
    lw = synth.make_layer(shape, seed)
    ref = oracle_case(lw, synth.make_tokens(T, shape.hidden, seed))
    ref.pop("h")
    res = {k: np.concatenate([p[k] for p in parts]) for k in ("out", "topk_i", "topk_w")}
    print("after resync", compare(res, ref, shape.top_k, "after resync"))


@pytest.mark.gpu
def test_peer_enable_rejects_a_rank_with_other_sizes():
    """Peers store into each other's buffers at addresses computed from their own
    configuration, so a blob from a rank created with another max_tokens (or hidden
    size, expert count, ...) must be refused before anything is mapped.  One GPU is
    enough: the forged second blob is never opened."""
    import ctypes
    import struct

    shape = pkg.MoEShape(hidden=128, intermediate=64, n_experts=8, top_k=2)
    with pkg.MoEEngine(shape, max_tokens=64, ep_rank=0, ep_size=2) as eng:
        mine = eng.ep_peer_export()
        assert len(mine) == capi.EP_PEER_EXPORT_BYTES
        # blob = 64-byte IPC handle, 4 offsets + arena size (u64), then ints:
        # hidden, n_experts, top_k, max_tokens, rows_cap, ep_size, ep_rank, version
        ints_at = 64 + 5 * 8
        ints = list(struct.unpack_from("8i", mine, ints_at))
        assert ints[:4] == [128, 8, 2, 64] and ints[5:7] == [2, 0]

        def forged(**kw):
            v = list(ints)
            v[6] = 1  # pretend to be rank 1
            for k, x in kw.items():
                v[{"hidden": 0, "n_experts": 1, "top_k": 2, "max_tokens": 3, "rank": 6}[k]] = x
            b = bytearray(mine)
            struct.pack_into("8i", b, ints_at, *v)
            return bytes(b)

        for kw in (dict(max_tokens=32), dict(hidden=256), dict(n_experts=16), dict(top_k=4), dict(rank=0)):
            with pytest.raises(capi.MoEError) as ei:
                eng.ep_peer_enable([mine, forged(**kw)])
            assert ei.value.status == capi.ERR_INVALID, kw
        # and the handle is still not in peer mode: a forward is refused, not run
        t = torch.zeros(4, 128, dtype=torch.bfloat16, device="cuda")
        with pytest.raises(capi.MoEError):
            eng.forward(0, t)
