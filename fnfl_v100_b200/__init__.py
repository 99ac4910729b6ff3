"""fnfl_v100_b200: B200 (sm_100a) kernels for the FNFL engine's fused per-layer row-wise path.

RMSNorm (hidden and per-head), SwiGLU fused with Q8_1 requantisation, NeoX partial RoPE fused with the Q8_0
quantise-and-append into the KV cache, and Q4_K / IQ3_XXS / Q8_0 token-embedding get_rows, behind the C ABI of
include/fnb200.h.

There is no fallback path: the first operator call loads fnfl_v100_b200/libfnb200.so and raises ImportError if
it has not been built (`python -m fnfl_v100_b200.build`).  `require()` does that check up front.
"""
from . import _lib, ops, shard, synth
from .chain import ChainConfig, PrefillChain


def require() -> None:
    """Load the CUDA library now; raises ImportError when it is missing."""
    _lib.lib()


__all__ = ["ops", "shard", "synth", "PrefillChain", "ChainConfig", "require"]
