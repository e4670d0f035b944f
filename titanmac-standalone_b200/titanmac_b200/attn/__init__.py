from .windowed_attention import WindowedAttention

__all__ = ["WindowedAttention"]
