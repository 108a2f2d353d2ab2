"""rlx_b200 — B200-native GGUF quantized-weight linear layer (drop-in for RLX's Op::DequantMatMul)."""
from .api import *  # noqa: F401,F403
from .api import __all__ as _api_all
from .gguf import GgufFile, GgufTensor  # noqa: F401

__all__ = list(_api_all) + ["GgufFile", "GgufTensor"]
