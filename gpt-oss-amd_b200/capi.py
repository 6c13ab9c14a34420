"""ctypes bindings of libmoe_b200.so -- one Python function per C entry point of
include/moe_b200.h, nothing more.  Loading the library needs no GPU; every
entry point that computes fails with MOE_B200_ERR_NO_DEVICE without one (there
is no CPU fallback)."""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("MOE_B200_LIB") or os.path.join(_HERE, "libmoe_b200.so")
#: the same sources compiled with -DMOE_B200_TEST_AIDS (adds the cross-check GEMM); tests only
TEST_AIDS_LIB_PATH = os.path.join(_HERE, "libmoe_b200_testaids.so")

OK, ERR_INVALID, ERR_CUDA, ERR_NO_DEVICE, ERR_NOT_LOADED, ERR_DEVICE, ERR_NCCL, ERR_UNSUPPORTED = range(8)
DTYPE_F32, DTYPE_BF16 = 0, 1
GEMM_TCGEN05 = 0
GEMM_MMA_SYNC = 1  # exists in the test-aids build only
EP_PEER_EXPORT_BYTES = 256

#: every symbol include/moe_b200.h declares
SYMBOLS = [
    "moe_b200_shard_range", "moe_b200_create", "moe_b200_destroy", "moe_b200_set_router",
    "moe_b200_set_experts_mxfp4", "moe_b200_forward", "moe_b200_forward_norm", "moe_b200_forward_host",
    "moe_b200_ep_unique_id", "moe_b200_ep_init", "moe_b200_ep_plan", "moe_b200_device_bytes",
    "moe_b200_last_error", "moe_b200_device_status", "moe_b200_last_launch_count",
    "moe_b200_last_expert_counts", "moe_b200_mxfp4_unpack", "moe_b200_unpack_resident",
    "moe_b200_version", "moe_b200_profile", "moe_b200_profile_read",
    "moe_b200_last_intermediate", "moe_b200_route_noalloc",
    "moe_b200_ep_peer_export", "moe_b200_ep_peer_enable", "moe_b200_ep_peer_sequence",
    "moe_b200_ep_peer_resync", "moe_b200_expert_file_info", "moe_b200_load_experts_file",
    "moe_b200_request_queue_create", "moe_b200_request_queue_destroy", "moe_b200_batcher_create",
    "moe_b200_batcher_destroy", "moe_b200_batcher_begin_step", "moe_b200_batcher_end_step",
    "moe_b200_batcher_stats",
]
N_STAGES = 11
STAGE_NAMES = ["route", "plan", "permute", "dispatch", "regroup", "gemm1", "gemm2", "return",
               "combine", "h2d", "d2h"]


class Config(ctypes.Structure):
    _fields_ = [
        ("hidden_dim", ctypes.c_int), ("intermediate_dim", ctypes.c_int),
        ("n_experts", ctypes.c_int), ("experts_per_token", ctypes.c_int),
        ("n_layers", ctypes.c_int), ("swiglu_alpha", ctypes.c_float),
        ("swiglu_limit", ctypes.c_float), ("max_tokens", ctypes.c_int),
        ("ep_rank", ctypes.c_int), ("ep_size", ctypes.c_int), ("device", ctypes.c_int),
        ("gemm_impl", ctypes.c_int),
    ]


class MoEError(RuntimeError):
    def __init__(self, status: int, text: str):
        super().__init__(f"moe_b200 status {status}: {text}")
        self.status = status


_libs = {}


def _bind(L: ctypes.CDLL) -> ctypes.CDLL:
    vp, ci = ctypes.c_void_p, ctypes.c_int
    ip = ctypes.POINTER(ctypes.c_int)
    L.moe_b200_shard_range.argtypes = [ci, ci, ci, ip, ip]
    L.moe_b200_shard_range.restype = None
    L.moe_b200_create.argtypes = [ctypes.POINTER(Config), ctypes.POINTER(vp)]
    L.moe_b200_destroy.argtypes = [vp]
    L.moe_b200_set_router.argtypes = [vp, ci, vp, vp]
    L.moe_b200_set_experts_mxfp4.argtypes = [vp, ci, ci, ci, vp, vp, vp, vp, vp, vp]
    L.moe_b200_forward.argtypes = [vp, ci, vp, ci, ci, vp, ci, vp, vp, vp, vp]
    L.moe_b200_forward_norm.argtypes = [vp, ci, vp, vp, ci, ci, vp, ci, vp, vp, vp, vp]
    L.moe_b200_forward_host.argtypes = [vp, ci, vp, ci, ci, vp, vp, vp]
    L.moe_b200_ep_unique_id.argtypes = [ctypes.c_char_p]
    L.moe_b200_ep_init.argtypes = [vp, ctypes.c_char_p]
    L.moe_b200_ep_plan.argtypes = [ci, ci, ci, ip, ip, ip, ip, ip]
    L.moe_b200_ep_plan.restype = None
    L.moe_b200_device_bytes.argtypes = [vp]
    L.moe_b200_device_bytes.restype = ctypes.c_size_t
    L.moe_b200_last_error.argtypes = [vp]
    L.moe_b200_last_error.restype = ctypes.c_char_p
    L.moe_b200_device_status.argtypes = [vp, ip]
    L.moe_b200_last_launch_count.argtypes = [vp]
    L.moe_b200_last_expert_counts.argtypes = [vp, ip]
    L.moe_b200_mxfp4_unpack.argtypes = [vp, vp, ctypes.c_longlong, ci, vp, vp]
    L.moe_b200_unpack_resident.argtypes = [vp, ci, ci, ci, vp, vp]
    L.moe_b200_version.restype = ctypes.c_char_p
    L.moe_b200_last_intermediate.argtypes = [vp, ci, vp, vp]
    L.moe_b200_route_noalloc.argtypes = [vp, ci, ci, ci, vp, vp, ci, ci, vp, vp, vp, vp, vp]
    L.moe_b200_ep_peer_export.argtypes = [vp, ctypes.c_char_p]
    L.moe_b200_ep_peer_enable.argtypes = [vp, ctypes.c_char_p]
    L.moe_b200_ep_peer_sequence.argtypes = [vp]
    L.moe_b200_ep_peer_resync.argtypes = [vp, ci]
    fp = ctypes.POINTER(ctypes.c_float)
    L.moe_b200_expert_file_info.argtypes = [ctypes.c_char_p, ip, ip, ip, ip, ip, fp,
                                            ctypes.POINTER(ctypes.c_ulonglong)]
    L.moe_b200_load_experts_file.argtypes = [vp, ctypes.c_char_p, ci, ci]
    ipp = ctypes.POINTER(ip)
    llp = ctypes.POINTER(ctypes.c_longlong)
    L.moe_b200_request_queue_create.argtypes = [ci, ipp, ip, ipp, ci, ctypes.POINTER(vp)]
    L.moe_b200_request_queue_destroy.argtypes = [vp]
    L.moe_b200_request_queue_destroy.restype = None
    L.moe_b200_batcher_create.argtypes = [vp, ci, ci, ctypes.POINTER(vp)]
    L.moe_b200_batcher_destroy.argtypes = [vp]
    L.moe_b200_batcher_destroy.restype = None
    L.moe_b200_batcher_begin_step.argtypes = [vp, ip, ip, ip, ip]
    L.moe_b200_batcher_end_step.argtypes = [vp, ip]
    L.moe_b200_batcher_stats.argtypes = [vp, llp, llp, llp]
    L.moe_b200_batcher_stats.restype = None
    L.moe_b200_profile.argtypes = [vp, ci]
    L.moe_b200_profile_read.argtypes = [vp, ci, ctypes.POINTER(ctypes.c_float)]
    return L


def lib(test_aids: bool = False) -> ctypes.CDLL:
    """The loaded library (``test_aids``: the variant with the cross-check GEMM,
    for tests).  Raises if it has not been built: nothing here falls back to
    another implementation."""
    path = TEST_AIDS_LIB_PATH if test_aids else LIB_PATH
    if path not in _libs:
        if not os.path.isfile(path):
            raise FileNotFoundError(
                f"{path} is missing: build it with `python gpt-oss-amd_b200/build.py` "
                "(needs nvcc); there is no fallback implementation")
        _libs[path] = _bind(ctypes.CDLL(path))
    return _libs[path]


def check(status: int, handle=None, L: ctypes.CDLL | None = None) -> None:
    if status != OK:
        text = (L or lib()).moe_b200_last_error(handle).decode("utf-8", "replace")
        raise MoEError(status, text)


def shard_range(n_experts: int, ep_size: int, ep_rank: int) -> tuple[int, int]:
    first, n = ctypes.c_int(), ctypes.c_int()
    lib().moe_b200_shard_range(n_experts, ep_size, ep_rank, ctypes.byref(first), ctypes.byref(n))
    return first.value, n.value


def ep_plan(n_experts: int, ep_size: int, ep_rank: int, cnt_all):
    """cnt_all: [ep_size][n_experts] ints -> (send_cnt, send_off, recv_cnt, recv_off) lists."""
    flat = [int(v) for row in cnt_all for v in row]
    arr = (ctypes.c_int * len(flat))(*flat)
    outs = [(ctypes.c_int * ep_size)() for _ in range(4)]
    lib().moe_b200_ep_plan(n_experts, ep_size, ep_rank, arr, *outs)
    return tuple(list(o) for o in outs)
