"""titanmac_b200 — B200-native WindowedAttention path of TitanMAC (hand-written sm_100a CUDA behind a C ABI)."""

from .config import TitanMACConfig, WindowConfig
from .attn.windowed_attention import WindowedAttention
from . import _native

__all__ = ["TitanMACConfig", "WindowConfig", "WindowedAttention", "_native"]
