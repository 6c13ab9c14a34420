"""ctypes/numpy front end of the CPU checkers.

TEST INFRASTRUCTURE ONLY: imported by tests/, by ``__graft_entry__.smoke`` and by
the ``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``; never by the
package that ships.

Two back ends with the same interface:

* ``port``      -- ``libmoe_oracle.so``, the plain-C restatement in
  ``moe_oracle.c`` (always available),
* ``reference`` -- ``_ref/libref_moe.so``, the reference engine's own CPU
  functions compiled from its sources by ``make ref`` (available wherever that
  build was run; the built file travels with the tree).

``round_mode`` 0 keeps the CPU engine's fp32 activations; 1 adds the HIP
engine's bf16 rounding of the block input and of the SwiGLU output (the
numerics the output tolerance is stated against).
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_PORT_SO = os.path.join(_HERE, "libmoe_oracle.so")
_REF_SO = os.path.join(_HERE, "_ref", "libref_moe.so")

_f32p = ctypes.POINTER(ctypes.c_float)
_i32p = ctypes.POINTER(ctypes.c_int)
_u8p = ctypes.POINTER(ctypes.c_uint8)
_u16p = ctypes.POINTER(ctypes.c_uint16)


def build(with_reference: bool = True) -> None:
    """Compile the checkers (``make``; plus ``make ref`` when the reference
    sources are present on this machine)."""
    subprocess.run(["make", "-C", _HERE, "all"], check=True, capture_output=True)
    ref_root = os.environ.get("MOE_REFERENCE_ROOT", "/root/reference")
    if with_reference and os.path.isfile(os.path.join(ref_root, "src", "run.cpp")):
        subprocess.run(["make", "-C", _HERE, "ref", f"REF={ref_root}"], check=True,
                       capture_output=True)


def have_reference() -> bool:
    return os.path.isfile(_REF_SO)


_port = None
_ref = None


def _lib_port():
    global _port
    if _port is None:
        if not os.path.isfile(_PORT_SO):
            build(with_reference=False)
        _port = ctypes.CDLL(_PORT_SO)
        _port.oracle_mxfp4_decode_bits.restype = ctypes.c_uint16
    return _port


def _lib_ref():
    global _ref
    if _ref is None:
        _ref = ctypes.CDLL(_REF_SO)
    return _ref


def _p(a, typ):
    return a.ctypes.data_as(typ)


def num_threads(impl: str = "port") -> int:
    return int(_lib_ref().ref_num_threads() if impl == "reference" else _lib_port().oracle_num_threads())


def host_cores() -> int:
    """Cores this process may run on (the affinity mask, not OMP_NUM_THREADS)."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def use_all_cores() -> int:
    """Make both checkers use every core this process may run on, whatever
    OMP_NUM_THREADS the launcher exported (torch.distributed.run exports 1).
    Returns the thread count set."""
    n = host_cores()
    _lib_port().oracle_set_num_threads(n)
    if have_reference():
        _lib_ref().ref_set_num_threads(n)
    return n


# ---------------------------------------------------------------------------
# MXFP4


def mxfp4_decode_table() -> np.ndarray:
    """[16 codes, 256 scale bytes] bf16 bit patterns from the C restatement."""
    lib = _lib_port()
    out = np.empty((16, 256), dtype=np.uint16)
    for c in range(16):
        for s in range(256):
            out[c, s] = lib.oracle_mxfp4_decode_bits(c, s)
    return out


def mxfp4_dequant_bf16(blocks: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """blocks [..., G, 16] u8, scales [..., G] u8 -> [..., 32*G] bf16 bits (u16)."""
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    scales = np.ascontiguousarray(scales, dtype=np.uint8)
    G = blocks.shape[-2]
    rows = int(np.prod(blocks.shape[:-2], dtype=np.int64))
    out = np.empty(blocks.shape[:-2] + (32 * G,), dtype=np.uint16)
    _lib_port().oracle_mxfp4_dequant_bf16(_p(blocks, _u8p), _p(scales, _u8p),
                                          ctypes.c_longlong(rows), G, _p(out, _u16p))
    return out


def mxfp4_dequant_f32(blocks: np.ndarray, scales: np.ndarray) -> np.ndarray:
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    scales = np.ascontiguousarray(scales, dtype=np.uint8)
    G = blocks.shape[-2]
    rows = int(np.prod(blocks.shape[:-2], dtype=np.int64))
    out = np.empty(blocks.shape[:-2] + (32 * G,), dtype=np.float32)
    _lib_port().oracle_mxfp4_dequant_f32(_p(blocks, _u8p), _p(scales, _u8p),
                                         ctypes.c_longlong(rows), G, _p(out, _f32p))
    return out


# ---------------------------------------------------------------------------
# the block


class ExpertCache:
    """fp32 (decoded) weights of the experts a batch touches, decoded on demand
    from packed MXFP4 so full-size layers need not be expanded whole."""

    def __init__(self, blocks1, scales1, bias1, blocks2, scales2, bias2, first_expert=0,
                 loader=None):
        """Arrays hold experts [first_expert, first_expert + n).  ``loader(e)``,
        if given, supplies the six packed arrays of a single expert that is not
        in the arrays (used when a full layer is too large to keep packed)."""
        self.blocks1, self.scales1, self._bias1 = blocks1, scales1, bias1
        self.blocks2, self.scales2, self._bias2 = blocks2, scales2, bias2
        self.first = first_expert
        self.loader = loader
        self.intermediate = (blocks2.shape[2] * 32) if blocks2 is not None else None
        self._w1 = {}
        self._w2 = {}
        self._b = {}

    def _have(self, e):
        return self.blocks1 is not None and self.first <= e < self.first + self.blocks1.shape[0]

    def _load(self, e):
        if e in self._w1:
            return
        if self._have(e):
            i = e - self.first
            b1, s1, c1, b2, s2, c2 = (self.blocks1[i], self.scales1[i], self._bias1[i],
                                      self.blocks2[i], self.scales2[i], self._bias2[i])
        else:
            b1, s1, c1, b2, s2, c2 = (a[0] for a in self.loader(e))
        self._w1[e] = mxfp4_dequant_f32(b1, s1)
        self._w2[e] = mxfp4_dequant_f32(b2, s2)
        self._b[e] = (np.ascontiguousarray(c1, dtype=np.float32),
                      np.ascontiguousarray(c2, dtype=np.float32))
        if self.intermediate is None:
            self.intermediate = self._w2[e].shape[1]

    def w1(self, e):
        self._load(e)
        return self._w1[e]

    def w2(self, e):
        self._load(e)
        return self._w2[e]

    def bias1(self, e):
        self._load(e)
        return self._b[e][0]

    def bias2(self, e):
        self._load(e)
        return self._b[e][1]

    def drop(self):
        self._w1.clear()
        self._w2.clear()
        self._b.clear()


def rmsnorm(x_f32, weight_f32, impl="port"):
    """The RMSNorm in front of the block (src/run.cpp:306-319), row by row -> [T, H]."""
    x = np.ascontiguousarray(x_f32, dtype=np.float32)
    w = np.ascontiguousarray(weight_f32, dtype=np.float32)
    T, H = x.shape
    o = np.empty_like(x)
    if impl == "reference":
        _lib_ref().ref_rmsnorm(_p(o, _f32p), _p(x, _f32p), _p(w, _f32p), T, H)
    else:
        _lib_port().oracle_rmsnorm(_p(o, _f32p), _p(x, _f32p), _p(w, _f32p), T, H)
    return o


def route(x_f32, w_router_f32, b_router, top_k, round_mode=1):
    """Router + top-k + softmax (src/run.cpp:630-641) -> (scores, topk_i, topk_v)."""
    x = np.ascontiguousarray(x_f32, dtype=np.float32)
    wr = np.ascontiguousarray(w_router_f32, dtype=np.float32)
    br = np.ascontiguousarray(b_router, dtype=np.float32)
    T, H = x.shape
    E = wr.shape[0]
    scores = np.empty((T, E), dtype=np.float32)
    ti = np.empty((T, top_k), dtype=np.int32)
    tv = np.empty((T, top_k), dtype=np.float32)
    _lib_port().oracle_route(T, H, E, top_k, round_mode, _p(x, _f32p), _p(wr, _f32p), _p(br, _f32p),
                             _p(scores, _f32p), _p(ti, _i32p), _p(tv, _f32p))
    return scores, ti, tv


def moe_forward(x_f32, w_router_f32, b_router, experts: ExpertCache, top_k=4, alpha=1.702,
                limit=7.0, round_mode=1, impl="port", want_h=False):
    """The MoE block for T tokens (src/run.cpp:628-707).  Returns a dict with
    ``router_score`` [T,E], ``topk_i`` [T,K], ``topk_v`` [T,K], ``e_agg`` [T,H] and,
    with ``want_h`` (port only), ``h`` [T,K,I], the input of MLP2 per selected expert."""
    x = np.ascontiguousarray(x_f32, dtype=np.float32)
    wr = np.ascontiguousarray(w_router_f32, dtype=np.float32)
    br = np.ascontiguousarray(b_router, dtype=np.float32)
    T, H = x.shape
    E = wr.shape[0]
    _, ti, _ = route(x, wr, br, top_k, round_mode)
    needed = sorted(set(int(e) for e in ti.reshape(-1)))
    PtrArr = ctypes.c_void_p * E
    w1p, b1p, w2p, b2p = PtrArr(), PtrArr(), PtrArr(), PtrArr()
    keep = []
    for e in needed:
        w1, w2 = experts.w1(e), experts.w2(e)
        b1, b2 = experts.bias1(e), experts.bias2(e)
        keep += [w1, w2, b1, b2]
        w1p[e], b1p[e], w2p[e], b2p[e] = (w1.ctypes.data, b1.ctypes.data, w2.ctypes.data,
                                          b2.ctypes.data)
    I = experts.intermediate
    scores = np.empty((T, E), dtype=np.float32)
    topk_i = np.empty((T, top_k), dtype=np.int32)
    topk_v = np.empty((T, top_k), dtype=np.float32)
    e_agg = np.empty((T, H), dtype=np.float32)
    h = np.empty((T, top_k, I), dtype=np.float32) if (want_h and impl == "port") else None
    if impl == "reference":
        if abs(alpha - 1.702) > 1e-9:
            raise ValueError("the reference hard-codes alpha = 1.702 (src/run.cpp:673)")
        st = _lib_ref().ref_moe_forward(T, H, I, E, top_k, ctypes.c_float(limit), round_mode,
                                        _p(x, _f32p), _p(wr, _f32p), _p(br, _f32p), w1p, b1p, w2p,
                                        b2p, _p(scores, _f32p), _p(topk_i, _i32p),
                                        _p(topk_v, _f32p), _p(e_agg, _f32p))
    else:
        st = _lib_port().oracle_moe_forward(T, H, I, E, top_k, ctypes.c_float(alpha),
                                            ctypes.c_float(limit), round_mode, _p(x, _f32p),
                                            _p(wr, _f32p), _p(br, _f32p), w1p, b1p, w2p, b2p,
                                            _p(scores, _f32p), _p(topk_i, _i32p),
                                            _p(topk_v, _f32p), _p(e_agg, _f32p),
                                            _p(h, _f32p) if h is not None else None)
    if st != 0:
        raise RuntimeError(f"oracle: expert {-st - 1} selected but not provided")
    res = {"router_score": scores, "topk_i": topk_i, "topk_v": topk_v, "e_agg": e_agg}
    if h is not None:
        res["h"] = h
    return res


def expert_rows(x_f32, w1, b1, w2, b2, alpha=1.702, limit=7.0, round_mode=1):
    """One expert applied to rows (inner part of src/run.cpp:658-700) -> [n, H]."""
    x = np.ascontiguousarray(x_f32, dtype=np.float32)
    n, H = x.shape
    I = w2.shape[1]
    y = np.empty((n, H), dtype=np.float32)
    w1 = np.ascontiguousarray(w1, dtype=np.float32)
    w2 = np.ascontiguousarray(w2, dtype=np.float32)
    b1 = np.ascontiguousarray(b1, dtype=np.float32)
    b2 = np.ascontiguousarray(b2, dtype=np.float32)
    _lib_port().oracle_expert_rows(n, H, I, ctypes.c_float(alpha), ctypes.c_float(limit),
                                   round_mode, _p(x, _f32p), _p(w1, _f32p), _p(b1, _f32p),
                                   _p(w2, _f32p), _p(b2, _f32p), _p(y, _f32p))
    return y


def reference_forward_probe(x_rows, w_router_f32, b_router, w1, b1, w2, b2, top_k=4, limit=7.0):
    """Run the unmodified reference ``forward()`` on a one-layer in-memory model
    and return its MoE-block state (``t`` = block input after RMSNorm)."""
    x = np.ascontiguousarray(x_rows, dtype=np.float32)
    T, H = x.shape
    E = w_router_f32.shape[0]
    I = w2.shape[2]
    arrs = [np.ascontiguousarray(a, dtype=np.float32) for a in (w_router_f32, b_router, w1, b1, w2, b2)]
    t = np.empty((T, H), dtype=np.float32)
    scores = np.empty((T, E), dtype=np.float32)
    topk_i = np.empty((T, top_k), dtype=np.int32)
    topk_v = np.empty((T, top_k), dtype=np.float32)
    e_agg = np.empty((T, H), dtype=np.float32)
    st = _lib_ref().ref_forward_moe_probe(T, H, I, E, top_k, ctypes.c_float(limit), _p(x, _f32p),
                                          *[_p(a, _f32p) for a in arrs], _p(t, _f32p),
                                          _p(scores, _f32p), _p(topk_i, _i32p), _p(topk_v, _f32p),
                                          _p(e_agg, _f32p))
    if st != 0:
        raise RuntimeError("reference probe failed")
    return {"t": t, "router_score": scores, "topk_i": topk_i, "topk_v": topk_v, "e_agg": e_agg}
