from .attn_engine import AttentionEngine, OnlineFunc
from .linear_attn_engine import LinearAttentionEngine

__all__ = ["AttentionEngine", "OnlineFunc", "LinearAttentionEngine"]
