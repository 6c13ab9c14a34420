"""CPU-side checks of the C-ABI library: it loads, exports every symbol the
header declares, its pure-host functions agree with the reference's rules, and
its compute entry points refuse to run without a GPU (no CPU fallback)."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

import gpt_oss_amd_b200 as pkg
from gpt_oss_amd_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "moe_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)  # drop comments
    declared = set(re.findall(r"\b(moe_b200_[a-z0-9_]+)\s*\(", header))
    assert declared == set(capi.SYMBOLS), declared ^ set(capi.SYMBOLS)
    L = capi.lib()
    for name in declared:
        assert hasattr(L, name), name
    assert b"sm_100a" in L.moe_b200_version()


def test_shard_range_matches_reference_rule():
    # src/model.cpp:104-114: base = E / ep, remainder to the low ranks, contiguous
    for E, G in [(128, 8), (128, 1), (32, 2), (10, 4), (7, 3), (256, 8)]:
        seen = []
        for r in range(G):
            first, n = capi.shard_range(E, G, r)
            base, rem = divmod(E, G)
            assert n == base + (1 if r < rem else 0)
            assert first == r * base + min(r, rem)
            seen += list(range(first, first + n))
        assert seen == list(range(E))


def test_ep_plan_is_consistent_across_ranks():
    rng = np.random.default_rng(0)
    E, G = 10, 4
    cnt_all = rng.integers(0, 9, size=(G, E))
    plans = [capi.ep_plan(E, G, r, cnt_all) for r in range(G)]
    for r in range(G):
        send_cnt, send_off, recv_cnt, recv_off = plans[r]
        assert sum(send_cnt) == cnt_all[r].sum()
        assert send_off == list(np.concatenate([[0], np.cumsum(send_cnt)[:-1]]))
        assert recv_off == list(np.concatenate([[0], np.cumsum(recv_cnt)[:-1]]))
        for p in range(G):
            assert send_cnt[p] == plans[p][2][r]  # what r sends to p is what p expects from r
            first, n = capi.shard_range(E, G, p)
            assert send_cnt[p] == cnt_all[r, first:first + n].sum()


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_compute_entry_points_fail_loudly_without_a_gpu():
    shape = pkg.MoEShape(hidden=128, intermediate=64, n_experts=8, top_k=4)
    with pytest.raises(capi.MoEError) as ei:
        pkg.MoEEngine(shape, max_tokens=16)
    assert ei.value.status == capi.ERR_NO_DEVICE
    st = capi.lib().moe_b200_mxfp4_unpack(ctypes.c_void_p(16), ctypes.c_void_p(16), 1, 1,
                                          ctypes.c_void_p(16), None)
    assert st == capi.ERR_NO_DEVICE


def test_create_rejects_bad_configs():
    L = capi.lib()
    h = ctypes.c_void_p()
    for kw in [dict(hidden_dim=100), dict(n_experts=300), dict(experts_per_token=9),
               dict(ep_size=2, ep_rank=2), dict(max_tokens=0), dict(gemm_impl=5), dict(gemm_impl=1)]:
        base = dict(hidden_dim=128, intermediate_dim=64, n_experts=8, experts_per_token=4,
                    n_layers=1, swiglu_alpha=1.702, swiglu_limit=7.0, max_tokens=16, ep_rank=0,
                    ep_size=1, device=0, gemm_impl=0)
        base.update(kw)
        cfg = capi.Config(**base)
        assert L.moe_b200_create(ctypes.byref(cfg), ctypes.byref(h)) == capi.ERR_INVALID, kw
        assert L.moe_b200_last_error(None)


def test_test_aids_build_is_separate_from_the_shipped_library():
    """The cross-check GEMM exists only in the test-aids build: the shipped library
    refuses gemm_impl = 1 (checked above); the test-aids build gets past the argument
    checks with it and, on a machine without a GPU, stops at the missing device."""
    L = capi.lib(test_aids=True)
    assert b"test-aids" in L.moe_b200_version()
    assert b"test-aids" not in capi.lib().moe_b200_version()
    for name in capi.SYMBOLS:
        assert hasattr(L, name), name
    if not torch.cuda.is_available():
        cfg = capi.Config(hidden_dim=128, intermediate_dim=64, n_experts=8, experts_per_token=4,
                          n_layers=1, swiglu_alpha=1.702, swiglu_limit=7.0, max_tokens=16, ep_rank=0,
                          ep_size=1, device=0, gemm_impl=capi.GEMM_MMA_SYNC)
        h = ctypes.c_void_p()
        assert L.moe_b200_create(ctypes.byref(cfg), ctypes.byref(h)) == capi.ERR_NO_DEVICE


def test_header_compiles_as_c99_and_links(tmp_path):
    """tests/c_abi_smoke.c is the engine-side binding as code: a plain-C translation
    unit that includes include/moe_b200.h, compiled with -std=c99 -Wall -Werror and
    linked against the shipped library.  It runs the pure-host entry points and, on a
    machine without a GPU, checks that create fails with MOE_B200_ERR_NO_DEVICE."""
    import subprocess

    exe = tmp_path / "c_abi_smoke"
    lib_dir = os.path.dirname(capi.LIB_PATH)
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Wextra", "-Werror", "-pedantic",
                    "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "c_abi_smoke.c"),
                    "-L", lib_dir, "-l:libmoe_b200.so", f"-Wl,-rpath,{lib_dir}", "-o", str(exe)],
                   check=True, capture_output=True, text=True)
    res = subprocess.run([str(exe)], capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "c_abi_smoke ok" in res.stdout
    if not torch.cuda.is_available():
        assert "no device" in res.stdout


def test_retile_word_roundtrip_semantics():
    """The resident nibble order keeps every e2m1 code: even columns in the low
    half-word, odd columns in the high half-word (csrc/common.cuh)."""
    def retile(w):
        nib = [(w >> (4 * i)) & 0xF for i in range(8)]
        lo = sum(nib[2 * p] << (4 * p) for p in range(4))
        hi = sum(nib[2 * p + 1] << (4 * p) for p in range(4))
        return lo | (hi << 16)
    w = 0x76543210
    assert retile(w) == 0x75316420
