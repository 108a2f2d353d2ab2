"""rlx_b200 — B200-native GGUF quantized-weight linear layer (drop-in for RLX's Op::DequantMatMul)."""
from .api import *  # noqa: F401,F403
from .api import __all__  # noqa: F401
