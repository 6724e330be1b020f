from .base import BaseTranscoder, mark_replicated, is_replicated
from .clt import CrossLayerTranscoder, pair_index, resolve_dtype
from .activations import BatchTopK, TokenTopK, JumpReLU

__all__ = [
    "BaseTranscoder", "CrossLayerTranscoder", "BatchTopK", "TokenTopK", "JumpReLU",
    "mark_replicated", "is_replicated", "pair_index", "resolve_dtype",
]
