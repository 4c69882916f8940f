"""Attention layers of the reference's ``tensorax.nn`` (tensorax/nn/attention/)."""
from .attention import (  # noqa: F401
    GroupedQueryAttention,
    MultiHeadAttention,
    ScaledDotProductAttention,
    create_causal_mask,
    create_padding_mask,
)
