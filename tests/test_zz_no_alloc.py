"""moe_b200_route_noalloc: routing with the scratch memory inside the library.

Some callers of this library cannot allocate device memory at the moment they
need a routing decision -- a serving loop that handed its whole memory budget
to its own pools at warm-up and cannot afford the device-wide synchronisation
of cudaMalloc between decode steps, or a host application that only lets a
plug-in work on buffers it passes in.  For them the library has one entry point
that needs no handle: the per-block histograms the routing kernels use as
scratch live in a fixed array in the library image (about 0.26 MB per GPU, at
most 2048 tokens and 256 experts per call).

This test calls it through the C ABI twice in a row on different batches --
the array keeps the first call's contents, and the second, smaller batch must
not see them -- and compares expert indices, routing weights and per-expert
counts with what the handle-based moe_b200_forward reports for the same inputs,
and with the CPU oracle's router.  A second test interleaves it with handles of
other hidden sizes: the routing kernel's shared-memory limit is a per-device
setting that all of them share.  It is the last test file on purpose, and passes
on its own in a fresh process.
"""
import ctypes

import numpy as np
import pytest
import torch

import gpt_oss_amd_b200 as pkg
from gpt_oss_amd_b200 import capi, synth
from oracle import oracle
from oracle.parity import tie_mask

pytestmark = pytest.mark.gpu


def _vp(t):
    return ctypes.c_void_p(t.data_ptr())


def _route_noalloc(t, w_router, b_router, E, K):
    T, H = t.shape
    ti = torch.empty(T, K, dtype=torch.int32, device="cuda")
    tw = torch.empty(T, K, dtype=torch.float32, device="cuda")
    cnt = torch.empty(E, dtype=torch.int32, device="cuda")
    off = torch.empty(E + 1, dtype=torch.int32, device="cuda")
    dt = capi.DTYPE_BF16 if t.dtype == torch.bfloat16 else capi.DTYPE_F32
    s = torch.cuda.current_stream()
    capi.check(capi.lib().moe_b200_route_noalloc(_vp(t), dt, T, H, _vp(w_router), _vp(b_router), E, K,
                                                 _vp(ti), _vp(tw), _vp(cnt), _vp(off),
                                                 ctypes.c_void_p(s.cuda_stream)))
    torch.cuda.synchronize()
    return ti.cpu().numpy(), tw.cpu().numpy(), cnt.cpu().numpy(), off.cpu().numpy()


def test_route_noalloc_matches_forward_on_two_calls_in_a_row():
    shape = pkg.MoEShape(hidden=256, intermediate=64, n_experts=40, top_k=4)
    lw = synth.make_layer(shape, seed=31)
    w_router = torch.from_numpy(lw.w_router.view(np.int16)).cuda()
    b_router = torch.from_numpy(lw.b_router).cuda()
    with pkg.MoEEngine(shape, max_tokens=1024) as eng:
        eng.load_layer(0, lw)
        for call, (T, seed, dtype) in enumerate([(1000, 1, torch.bfloat16), (37, 2, torch.float32)]):
            x_bits = synth.make_tokens(T, shape.hidden, seed=seed)
            t = torch.from_numpy(x_bits.view(np.int16)).cuda().view(torch.bfloat16).to(dtype)
            _, _, ref_i, ref_w = eng.forward(0, t, side=True)
            torch.cuda.synchronize()
            ref_cnt = np.array(eng.last_expert_counts())
            ti, tw, cnt, off = _route_noalloc(t, w_router, b_router, shape.n_experts, shape.top_k)
            # the same router on the same inputs; the handle's path may split K over a
            # cluster of CTAs (another order of the fp32 chunk sums): last-bit differences
            assert np.array_equal(ti, ref_i.cpu().numpy()), f"call {call}"
            assert np.abs(tw - ref_w.cpu().numpy()).max() < 1e-6, f"call {call}"
            assert np.array_equal(cnt, ref_cnt), f"call {call}"
            assert cnt.sum() == T * shape.top_k
            assert np.array_equal(off, np.concatenate([[0], np.cumsum(cnt)])), f"call {call}"
            # and against the CPU engine's router (double-accumulated logits, ties excluded)
            scores, o_i, o_w = oracle.route(synth.bf16_bits_to_f32(x_bits),
                                            synth.bf16_bits_to_f32(lw.w_router), lw.b_router,
                                            shape.top_k, round_mode=1)
            ok = ~tie_mask(scores, shape.top_k)
            assert np.array_equal(ti[ok], o_i[ok]), f"call {call}"
            assert np.abs(tw[ok] - o_w[ok]).max() < 1e-5, f"call {call}"
            if ok.all():
                assert np.array_equal(cnt, np.bincount(o_i.reshape(-1), minlength=shape.n_experts))


def test_route_noalloc_interleaved_with_handles_of_other_hidden_sizes():
    """The shared-memory opt-in of the routing kernel belongs to the device, not to a
    caller: a handle with a small hidden size used between two allocation-free calls
    at a large one must not shrink the limit under the second call."""
    E, K = 32, 4
    big = pkg.MoEShape(hidden=2880, intermediate=64, n_experts=E, top_k=K)
    small = pkg.MoEShape(hidden=256, intermediate=64, n_experts=E, top_k=K)
    lw_big = synth.make_layer(big, seed=41)
    w_router = torch.from_numpy(lw_big.w_router.view(np.int16)).cuda()
    b_router = torch.from_numpy(lw_big.b_router).cuda()
    x_bits = synth.make_tokens(200, big.hidden, seed=41)
    t = torch.from_numpy(x_bits.view(np.int16)).cuda().view(torch.bfloat16)
    first = _route_noalloc(t, w_router, b_router, E, K)
    lw_small = synth.make_layer(small, seed=42)
    with pkg.MoEEngine(small, max_tokens=64) as eng:
        eng.load_layer(0, lw_small)
        ts = torch.from_numpy(synth.make_tokens(50, small.hidden, seed=42).view(np.int16)).cuda()
        eng.forward(0, ts.view(torch.bfloat16))
        torch.cuda.synchronize()
        assert eng.device_status() == 0
        second = _route_noalloc(t, w_router, b_router, E, K)
    for a, b in zip(first, second):
        assert np.array_equal(a, b)
    with pkg.MoEEngine(big, max_tokens=256) as eng:
        eng.load_layer(0, lw_big)
        _, _, ref_i, ref_w = eng.forward(0, t, side=True)
        torch.cuda.synchronize()
        assert np.array_equal(second[0], ref_i.cpu().numpy())
        # the handle's router may split K over a cluster of CTAs: last-bit differences
        assert np.abs(second[1] - ref_w.cpu().numpy()).max() < 1e-6


def test_route_noalloc_rejects_sizes_beyond_its_fixed_scratch():
    t = torch.zeros(8, 128, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(8, 128, dtype=torch.int16, device="cuda")
    b = torch.zeros(8, dtype=torch.float32, device="cuda")
    o = torch.zeros(4096, dtype=torch.int32, device="cuda")
    L = capi.lib()

    def call(T=8, H=128, E=8, K=4):
        return L.moe_b200_route_noalloc(_vp(t), capi.DTYPE_BF16, T, H, _vp(w), _vp(b), E, K, _vp(o),
                                        _vp(o), _vp(o), _vp(o), None)

    assert call(T=2049) == capi.ERR_INVALID
    assert b"2048" in L.moe_b200_last_error(None)
    assert call(E=257) == capi.ERR_INVALID
    assert call(H=6208) == capi.ERR_INVALID
    assert call(H=100) == capi.ERR_INVALID
    assert call(K=9) == capi.ERR_INVALID
    assert L.moe_b200_route_noalloc(None, capi.DTYPE_BF16, 8, 128, _vp(w), _vp(b), 8, 4, _vp(o), _vp(o),
                                    _vp(o), _vp(o), None) == capi.ERR_INVALID
