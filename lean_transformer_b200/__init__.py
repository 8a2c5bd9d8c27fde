"""B200-native (sm_100a) LeanFFN and block-sparse linear layers behind the lean_transformer module API.

Everything that computes lives in ``libleanffn_b200.so`` (hand-written CUDA, C ABI in
``include/leanffn_b200.h``); importing this package loads that library and fails if it is missing.
"""
from . import _native  # noqa: F401  (loads the shared library; raises if it is absent)
from .blocksparse import *  # noqa: F401,F403
from .ffn import LeanFFN, _LeanFFN  # noqa: F401
from .attn import LeanSelfAttention, RotaryAttentionCore, RotaryEmbeddings, SimpleAttentionCore  # noqa: F401
from .fused_linear import linear_dropout_residual  # noqa: F401
from .ops import check_device_status  # noqa: F401
from .utils import ACT2FN, pad_to_multiple, resolve_activation  # noqa: F401

__version__ = "0.1.0"
