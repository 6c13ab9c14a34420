"""Host-side mirror of the engine's MoE interface over the C ABI.

``MoEEngine`` plays the part of the MoE fields of ``OssTransformerHybrid`` /
``OssRunState`` (include/model.hpp:132-180,232-237): it owns one handle per GPU,
takes the router and the packed MXFP4 experts of each layer (``set_router`` /
``set_experts`` <-> the expert part of copy_transformer_to_device,
src/model.cpp:365-399) and runs the block (``forward`` <-> src/forward.cpp:317-992).
PyTorch is used only for device memory and streams; all compute goes through
``libmoe_b200.so``.  If the library is missing or no sm_100 GPU is present the
calls raise -- there is no other implementation to fall back to.
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from . import capi
from .synth import LayerWeights, MoEShape


def _ptr(x):
    """Device/host address of a tensor / array (None -> NULL)."""
    if x is None:
        return None
    if isinstance(x, torch.Tensor):
        assert x.is_contiguous()
        return ctypes.c_void_p(x.data_ptr())
    if isinstance(x, np.ndarray):
        assert x.flags["C_CONTIGUOUS"]
        return ctypes.c_void_p(x.ctypes.data)
    raise TypeError(type(x))


class MoEEngine:
    def __init__(self, shape: MoEShape, n_layers: int = 1, max_tokens: int = 256, ep_rank: int = 0,
                 ep_size: int = 1, device: int = 0, gemm_impl: int = capi.GEMM_TCGEN05):
        self.shape = shape
        self.n_layers = n_layers
        self.max_tokens = max_tokens
        self.ep_rank, self.ep_size = ep_rank, ep_size
        self.device = device
        self.first_expert, self.n_local = capi.shard_range(shape.n_experts, ep_size, ep_rank)
        cfg = capi.Config(shape.hidden, shape.intermediate, shape.n_experts, shape.top_k, n_layers,
                          shape.alpha, shape.limit, max_tokens, ep_rank, ep_size, device, gemm_impl)
        # a handle belongs to the library that created it: the shipped one, or (for the
        # cross-check GEMM of the parity tests) its test-aids build
        self._lib = capi.lib(test_aids=(gemm_impl != capi.GEMM_TCGEN05))
        h = ctypes.c_void_p()
        capi.check(self._lib.moe_b200_create(ctypes.byref(cfg), ctypes.byref(h)), None, self._lib)
        self._h = h

    # -- lifetime ---------------------------------------------------------
    def close(self):
        if getattr(self, "_h", None):
            self._lib.moe_b200_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    # -- weights ----------------------------------------------------------
    def set_router(self, layer: int, w_bf16_bits, bias):
        capi.check(self._lib.moe_b200_set_router(self._h, layer, _ptr(w_bf16_bits), _ptr(bias)),
                   self._h, self._lib)

    def set_experts(self, layer: int, first_expert: int, blocks1, scales1, bias1, blocks2, scales2,
                    bias2):
        n = blocks1.shape[0]
        capi.check(self._lib.moe_b200_set_experts_mxfp4(
            self._h, layer, first_expert, n, _ptr(blocks1), _ptr(scales1), _ptr(bias1),
            _ptr(blocks2), _ptr(scales2), _ptr(bias2)), self._h, self._lib)

    def load_layer(self, layer: int, lw: LayerWeights):
        """Router plus the part of this rank's contiguous expert shard that
        ``lw`` holds (it may hold the whole layer or just the shard)."""
        self.set_router(layer, np.ascontiguousarray(lw.w_router), np.ascontiguousarray(lw.b_router))
        a = max(self.first_expert, lw.first_expert)
        b = min(self.first_expert + self.n_local, lw.first_expert + lw.blocks1.shape[0])
        if b > a:
            i, j = a - lw.first_expert, b - lw.first_expert
            self.set_experts(layer, a, *(np.ascontiguousarray(x[i:j]) for x in (
                lw.blocks1, lw.scales1, lw.bias1, lw.blocks2, lw.scales2, lw.bias2)))

    def load_layer_file(self, path: str, file_layer: int, layer: int | None = None):
        """Router + this rank's expert shard of one layer from a packed expert file
        (``expert_file.write_expert_file``): the library maps the file itself."""
        capi.check(self._lib.moe_b200_load_experts_file(
            self._h, path.encode(), file_layer, file_layer if layer is None else layer), self._h, self._lib)

    # -- the block --------------------------------------------------------
    def forward(self, layer: int, t: torch.Tensor, out: torch.Tensor | None = None,
                accumulate: bool = False, side: bool = False, stream=None):
        """t: CUDA [T, H] bf16 or fp32.  Returns out (fp32 [T, H]) or, with
        ``side=True``, (out, router_score, topk_i, topk_w)."""
        assert t.is_cuda and t.dim() == 2 and t.shape[1] == self.shape.hidden
        T = t.shape[0]
        dt = capi.DTYPE_BF16 if t.dtype == torch.bfloat16 else capi.DTYPE_F32
        assert t.dtype in (torch.bfloat16, torch.float32)
        if out is None:
            assert not accumulate
            out = torch.empty(T, self.shape.hidden, dtype=torch.float32, device=t.device)
        sc = ti = tw = None
        if side:
            sc = torch.empty(T, self.shape.n_experts, dtype=torch.float32, device=t.device)
            ti = torch.empty(T, self.shape.top_k, dtype=torch.int32, device=t.device)
            tw = torch.empty(T, self.shape.top_k, dtype=torch.float32, device=t.device)
        s = stream if stream is not None else torch.cuda.current_stream(t.device)
        capi.check(self._lib.moe_b200_forward(
            self._h, layer, _ptr(t.contiguous()), dt, T, _ptr(out), int(accumulate), _ptr(sc),
            _ptr(ti), _ptr(tw), ctypes.c_void_p(s.cuda_stream)), self._h, self._lib)
        return (out, sc, ti, tw) if side else out

    def forward_norm(self, layer: int, x: torch.Tensor, rms_weight: torch.Tensor,
                     out: torch.Tensor | None = None, accumulate: bool = False, side: bool = False,
                     stream=None):
        """The block with the RMSNorm in front of it fused in.  x: CUDA fp32 [T, H], the
        residual stream; rms_weight: CUDA [H] fp32 or bf16.  ``out`` may be ``x`` itself
        (with ``accumulate=True``: x += MoE(rmsnorm(x)), the engine's residual update)."""
        assert x.is_cuda and x.dtype == torch.float32 and x.dim() == 2 and x.shape[1] == self.shape.hidden
        assert rms_weight.is_cuda and rms_weight.numel() == self.shape.hidden
        assert rms_weight.dtype in (torch.bfloat16, torch.float32)
        T = x.shape[0]
        wdt = capi.DTYPE_BF16 if rms_weight.dtype == torch.bfloat16 else capi.DTYPE_F32
        if out is None:
            assert not accumulate
            out = torch.empty(T, self.shape.hidden, dtype=torch.float32, device=x.device)
        sc = ti = tw = None
        if side:
            sc = torch.empty(T, self.shape.n_experts, dtype=torch.float32, device=x.device)
            ti = torch.empty(T, self.shape.top_k, dtype=torch.int32, device=x.device)
            tw = torch.empty(T, self.shape.top_k, dtype=torch.float32, device=x.device)
        s = stream if stream is not None else torch.cuda.current_stream(x.device)
        capi.check(self._lib.moe_b200_forward_norm(
            self._h, layer, _ptr(x.contiguous()), _ptr(rms_weight.contiguous()), wdt, T, _ptr(out),
            int(accumulate), _ptr(sc), _ptr(ti), _ptr(tw), ctypes.c_void_p(s.cuda_stream)), self._h, self._lib)
        return (out, sc, ti, tw) if side else out

    def forward_host(self, layer: int, t_host, out_host, topk_i_host=None, topk_w_host=None):
        """Host buffers in and out (torch CPU tensors, ideally pinned, or numpy)."""
        T = t_host.shape[0]
        if isinstance(t_host, torch.Tensor):
            dt = capi.DTYPE_BF16 if t_host.dtype == torch.bfloat16 else capi.DTYPE_F32
        else:
            dt = capi.DTYPE_BF16 if t_host.dtype == np.uint16 else capi.DTYPE_F32
        capi.check(self._lib.moe_b200_forward_host(
            self._h, layer, _ptr(t_host), dt, T, _ptr(out_host), _ptr(topk_i_host),
            _ptr(topk_w_host)), self._h, self._lib)
        return out_host

    # -- expert parallel ----------------------------------------------------
    @staticmethod
    def ep_unique_id() -> bytes:
        buf = ctypes.create_string_buffer(128)
        capi.check(capi.lib().moe_b200_ep_unique_id(buf))
        return buf.raw

    def ep_init(self, unique_id: bytes):
        capi.check(self._lib.moe_b200_ep_init(self._h, unique_id), self._h, self._lib)

    def ep_peer_export(self) -> bytes:
        buf = ctypes.create_string_buffer(capi.EP_PEER_EXPORT_BYTES)
        capi.check(self._lib.moe_b200_ep_peer_export(self._h, buf), self._h, self._lib)
        return buf.raw

    def ep_peer_enable(self, blobs_in_rank_order: list[bytes]):
        """Map the peers' exchange buffers: the exchange then runs inside the
        kernels over NVLink peer memory instead of NCCL."""
        capi.check(self._lib.moe_b200_ep_peer_enable(self._h, b"".join(blobs_in_rank_order)), self._h, self._lib)

    def ep_peer_sequence(self) -> int:
        return int(self._lib.moe_b200_ep_peer_sequence(self._h))

    def ep_peer_resync(self, sequence: int):
        capi.check(self._lib.moe_b200_ep_peer_resync(self._h, int(sequence)), self._h, self._lib)

    def ep_connect(self, dist, mode: str = "peer"):
        """Collective over the torch.distributed process group ``dist`` (any
        backend): set up the expert-parallel exchange, 'peer' or 'nccl'."""
        if mode == "peer":
            blobs = [None] * self.ep_size
            dist.all_gather_object(blobs, self.ep_peer_export())
            self.ep_peer_enable(blobs)
        else:
            ids = [self.ep_unique_id() if self.ep_rank == 0 else None]
            dist.broadcast_object_list(ids, src=0)
            self.ep_init(ids[0])

    # -- introspection ------------------------------------------------------
    def device_status(self) -> int:
        w = ctypes.c_int()
        st = self._lib.moe_b200_device_status(self._h, ctypes.byref(w))
        if st not in (capi.OK, capi.ERR_DEVICE):
            capi.check(st, self._h, self._lib)
        return w.value

    def device_bytes(self) -> int:
        return int(self._lib.moe_b200_device_bytes(self._h))

    def last_launch_count(self) -> int:
        return int(self._lib.moe_b200_last_launch_count(self._h))

    def last_expert_counts(self) -> list[int]:
        arr = (ctypes.c_int * self.n_local)()
        capi.check(self._lib.moe_b200_last_expert_counts(self._h, arr), self._h, self._lib)
        return list(arr)

    def last_intermediate(self, n_tokens: int) -> torch.Tensor:
        """bf16 bits [n_tokens, K, I] of the SwiGLU output that entered the down
        projection in the last forward (ep_size == 1)."""
        K, I = self.shape.top_k, self.shape.intermediate
        out = torch.empty(n_tokens, K, I, dtype=torch.int16, device=f"cuda:{self.device}")
        s = torch.cuda.current_stream(out.device)
        capi.check(self._lib.moe_b200_last_intermediate(self._h, n_tokens, _ptr(out),
                                                         ctypes.c_void_p(s.cuda_stream)), self._h, self._lib)
        return out

    def profile(self, n_calls: int):
        """Arm per-stage CUDA-event timing for the next n_calls forwards."""
        capi.check(self._lib.moe_b200_profile(self._h, n_calls), self._h, self._lib)

    def profile_read(self, call: int) -> dict:
        """Stage name -> milliseconds of the call-th profiled forward (after a
        synchronise of the stream it ran on)."""
        ms = (ctypes.c_float * capi.N_STAGES)()
        capi.check(self._lib.moe_b200_profile_read(self._h, call, ms), self._h, self._lib)
        return dict(zip(capi.STAGE_NAMES, (float(v) for v in ms)))

    def unpack_resident(self, layer: int, local_expert: int, which: int) -> torch.Tensor:
        H, I = self.shape.hidden, self.shape.intermediate
        shape = (2 * I, H) if which == 1 else (H, I)
        out = torch.empty(shape, dtype=torch.int16, device=f"cuda:{self.device}")
        s = torch.cuda.current_stream(out.device)
        capi.check(self._lib.moe_b200_unpack_resident(self._h, layer, local_expert, which, _ptr(out),
                                                       ctypes.c_void_p(s.cuda_stream)), self._h, self._lib)
        return out


class RequestQueue:
    """The requests of a serving run, shared by the batchers of all ranks: encoded
    prompts in, generated tokens out (the Requests buffers of src/getp/eval.cpp:10-40)."""

    def __init__(self, prompts: list, max_seq_len: int):
        self.n = len(prompts)
        self.max_seq_len = max_seq_len
        self._prompts = [np.ascontiguousarray(p, dtype=np.int32) for p in prompts]
        self._lens = np.array([len(p) for p in self._prompts], dtype=np.int32)
        self.outputs = np.zeros((max(self.n, 1), max_seq_len + 1), dtype=np.int32)
        ip = ctypes.POINTER(ctypes.c_int)
        self._pp = (ip * max(self.n, 1))(*[p.ctypes.data_as(ip) for p in self._prompts])
        self._op = (ip * max(self.n, 1))(*[self.outputs[r].ctypes.data_as(ip) for r in range(max(self.n, 1))])
        h = ctypes.c_void_p()
        capi.check(capi.lib().moe_b200_request_queue_create(
            self.n, self._pp, self._lens.ctypes.data_as(ip), self._op, max_seq_len, ctypes.byref(h)))
        self._h = h

    def close(self):
        if getattr(self, "_h", None):
            capi.lib().moe_b200_request_queue_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()


class TokenBatcher:
    """One rank's view of the serving loop: which (token, position, slot) rows go into
    the next forward() (moe_b200_batcher_*; src/getp/run.cpp:573-617,661-736)."""

    def __init__(self, queue: RequestQueue, n_slots: int, continuous: bool = True):
        self.queue, self.n_slots = queue, n_slots
        h = ctypes.c_void_p()
        capi.check(capi.lib().moe_b200_batcher_create(queue._h, n_slots, int(continuous), ctypes.byref(h)))
        self._h = h
        self._buf = [np.zeros(n_slots, dtype=np.int32) for _ in range(4)]

    def begin_step(self):
        """-> (tokens, positions, slots, needs_sample) arrays of the step's rows, or None."""
        ip = ctypes.POINTER(ctypes.c_int)
        n = capi.lib().moe_b200_batcher_begin_step(self._h, *[b.ctypes.data_as(ip) for b in self._buf])
        if n < 0:
            raise RuntimeError("begin_step while a step is in flight")
        if n == 0:
            return None
        return tuple(b[:n].copy() for b in self._buf)

    def end_step(self, sampled):
        s = np.ascontiguousarray(sampled, dtype=np.int32)
        capi.check(capi.lib().moe_b200_batcher_end_step(self._h, s.ctypes.data_as(ctypes.POINTER(ctypes.c_int))))

    def stats(self) -> dict:
        v = [ctypes.c_longlong() for _ in range(3)]
        capi.lib().moe_b200_batcher_stats(self._h, *[ctypes.byref(x) for x in v])
        return {"steps": v[0].value, "rows": v[1].value, "tokens_out": v[2].value}

    def close(self):
        if getattr(self, "_h", None):
            capi.lib().moe_b200_batcher_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()


def mxfp4_unpack(blocks: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """blocks CUDA u8 [..., G, 16], scales CUDA u8 [..., G] -> bf16 bits (int16) [..., 32 G]."""
    assert blocks.is_cuda and scales.is_cuda and blocks.dtype == torch.uint8
    G = blocks.shape[-2]
    rows = blocks.numel() // (G * 16)
    out = torch.empty(*blocks.shape[:-2], 32 * G, dtype=torch.int16, device=blocks.device)
    s = torch.cuda.current_stream(blocks.device)
    capi.check(capi.lib().moe_b200_mxfp4_unpack(_ptr(blocks.contiguous()), _ptr(scales.contiguous()),
                                                rows, G, _ptr(out), ctypes.c_void_p(s.cuda_stream)))
    return out
