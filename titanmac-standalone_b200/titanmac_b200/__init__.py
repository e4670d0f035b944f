"""titanmac_b200 — B200-native WindowedAttention path of TitanMAC (hand-written sm_100a CUDA behind a C ABI)."""

from .config import TitanMACConfig, WindowConfig
from .attn.windowed_attention import WindowedAttention
from .attn.block_sparse_attention import BlockSparseAttention, create_block_sparse_attention
from .blocks.titan_block import MLPBlock, RMSNorm, TitanBlock
from .models.titanmac import TitanMAC
from .host_pipeline import HostPipeline
from . import _native

__all__ = ["TitanMACConfig", "WindowConfig", "WindowedAttention", "BlockSparseAttention",
           "create_block_sparse_attention", "TitanBlock", "RMSNorm", "MLPBlock", "TitanMAC",
           "HostPipeline", "_native"]
