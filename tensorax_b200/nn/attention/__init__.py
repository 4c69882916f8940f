from .layers import GroupedQueryAttention, MultiHeadAttention, ScaledDotProductAttention
from .utils import create_causal_mask, create_padding_mask

__all__ = [
    "ScaledDotProductAttention",
    "GroupedQueryAttention",
    "MultiHeadAttention",
    "create_causal_mask",
    "create_padding_mask",
]
