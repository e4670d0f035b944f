"""Configuration objects read by the attention path.

``WindowConfig`` mirrors the reference's standalone attention config
(titans_core/attn/windowed_attention.py:16-34) and ``TitanMACConfig`` the model
config's architecture fields (titans_core/config.py:81-117, ``d_head`` :160-167,
``validate`` :198-245) with the same names and defaults.  Fields that only drive
the reference's neural memory and optimizers are not part of this path and are
absent; the reference's own config objects can be passed instead of these
anywhere in this package, because only attributes are read.
"""

from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Any, Dict


@dataclass
class WindowConfig:
    window_size: int
    num_heads: int
    head_dim: int
    n_persistent: int
    dropout: float = 0.0
    causal: bool = True


@dataclass
class TitanMACConfig:
    vocab_size: int = 128000
    d_model: int = 640
    n_heads: int = 10
    n_layers: int = 16
    d_ff: int = 2560
    max_seq_len: int = 4096
    window_size: int = 512
    n_persistent: int = 16
    # As in the reference (titans_core/config.py:91-92): True selects BlockSparseAttention (depthwise
    # convolutions on Q/K/V, block-granular window, global persistent rows), False WindowedAttention.
    # The ring-cache generation path (TitanMAC.prefill / decode_step / generate) needs False.
    use_block_sparse: bool = True
    block_size: int = 64
    dropout: float = 0.0
    tie_weights: bool = True
    norm_eps: float = 1e-5
    attention_dropout: float = 0.0
    causal: bool = True

    @property
    def d_head(self) -> int:
        if self.d_model % self.n_heads != 0:
            raise ValueError(f"d_model ({self.d_model}) must be divisible by n_heads ({self.n_heads})")
        return self.d_model // self.n_heads

    def validate(self) -> None:
        if self.d_model % self.n_heads != 0:
            raise ValueError(f"d_model ({self.d_model}) must be divisible by n_heads ({self.n_heads})")
        if self.n_persistent >= self.max_seq_len:
            raise ValueError(f"n_persistent ({self.n_persistent}) must be < max_seq_len ({self.max_seq_len})")
        if self.window_size < 0:
            raise ValueError(f"window_size must be non-negative, got {self.window_size}")
        for name in ("d_model", "d_ff", "n_heads", "n_layers"):
            if getattr(self, name) <= 0:
                raise ValueError(f"{name} must be positive, got {getattr(self, name)}")
        for name in ("dropout", "attention_dropout"):
            if not 0.0 <= getattr(self, name) <= 1.0:
                raise ValueError(f"{name} must be in [0, 1], got {getattr(self, name)}")

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)
