"""B200 (sm_100a) MoE feed-forward block for the gpt-oss-amd engine.

The product is the C-ABI library ``libmoe_b200.so`` (include/moe_b200.h) built
from ``csrc/``; this package holds its ctypes bindings (``capi``), a host-side
mirror of the engine's MoE interface (``moe.MoEEngine``), the synthetic input
generators of the benchmark configurations (``synth``), the writer of the packed
expert file the library loads (``expert_file``) and the build script.
"""
from . import capi, expert_file, synth  # noqa: F401
from .moe import MoEEngine, RequestQueue, TokenBatcher, mxfp4_unpack  # noqa: F401
from .synth import LayerWeights, MoEShape, make_layer, make_tokens  # noqa: F401
