"""The block around the attention module: pre-norm residual wiring, RMSNorm and the MLP.

Mirrors titans_core/blocks/titan_block.py:41-102, blocks/norms.py:39-60 and
blocks/mlp.py:28-67 of the reference (same submodule names, so checkpoints load
unchanged).  The attention is this package's own code, and so is the element-wise work around
it on a GPU: RMSNorm with the preceding residual add folded in is one kernel
(``tmw_add_rmsnorm``); the linears are the library's tensor-core product ``tmw_linear`` with bias and the exact GELU
in its epilogue (a decode step's few rows: library GEMM plus the one-pass ``tmw_gelu``).
``use_block_sparse`` selects the attention class exactly as in the reference.
Under ``torch.no_grad()`` the fused kernels run; with grad mode on, norm and GELU fall back to the
differentiable PyTorch formulas and the windowed attention core uses its own backward kernel.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .. import _native
from ..attn.block_sparse_attention import BlockSparseAttention
from ..attn.windowed_attention import WindowedAttention


class RMSNorm(nn.Module):
    """``x / sqrt(mean(x^2) + eps) * scale`` (blocks/norms.py:55-58)."""

    def __init__(self, dim: int, eps: float = 1e-5):
        super().__init__()
        self.eps = eps
        self.scale = nn.Parameter(torch.ones(dim))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if _native.add_rmsnorm_supported(x) and not self._wants_grad(x):
            return _native.add_rmsnorm(x, None, self.scale, self.eps)[1]
        rms = torch.sqrt(torch.mean(x ** 2, dim=-1, keepdim=True) + self.eps)
        return x / rms * self.scale

    def _wants_grad(self, *tensors: torch.Tensor) -> bool:
        """The fused kernel has no backward: with grad mode on and a gradient due to an input or to the scale,
        the plain PyTorch formula runs instead (inference callers use ``torch.no_grad()``)."""
        return torch.is_grad_enabled() and (self.scale.requires_grad or any(t.requires_grad for t in tensors))

    def add_forward(self, x: torch.Tensor, residual: torch.Tensor, inplace: bool = False):
        """``h = x + residual`` and ``RMSNorm(h)`` together: returns ``(h, normed)``."""
        if _native.add_rmsnorm_supported(x) and not self._wants_grad(x, residual):
            return _native.add_rmsnorm(x, residual, self.scale, self.eps, inplace_sum=inplace)
        h = x + residual
        return h, self.forward(h)


class MLPBlock(nn.Module):
    """Linear(+bias) → exact GELU → Linear(+bias) (blocks/mlp.py:36-65)."""

    def __init__(self, d_model: int, d_ff: int, dropout: float = 0.0):
        super().__init__()
        self.d_model, self.d_ff, self.dropout_p = d_model, d_ff, dropout
        self.fc1 = nn.Linear(d_model, d_ff)
        self.fc2 = nn.Linear(d_ff, d_model)
        self.activation = nn.GELU()
        self.dropout = nn.Dropout(dropout) if dropout > 0 else nn.Identity()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if torch.is_grad_enabled() and (x.requires_grad or self.fc1.weight.requires_grad):
            return self.dropout(self.fc2(self.activation(self.fc1(x))))
        # inference: bias and the exact-erf GELU ride in the epilogue of the library's tensor-core product
        # (tmw_linear); few rows (a decode step) take the library GEMM and the one-pass GELU kernel
        h = _native.project(self.fc1, x, gelu=True)
        return self.dropout(_native.project(self.fc2, h))


class TitanBlock(nn.Module):
    """``x + Attention(RMSNorm(x))`` then ``x + MLP(RMSNorm(x))`` (titan_block.py:92-100)."""

    def __init__(self, config):
        super().__init__()
        self.config = config
        self.norm_attn = RMSNorm(config.d_model, eps=config.norm_eps)
        self.norm_mlp = RMSNorm(config.d_model, eps=config.norm_eps)
        if getattr(config, "use_block_sparse", False):  # same switch as titan_block.py:51-64
            self.attention = BlockSparseAttention(
                d_model=config.d_model, n_heads=config.n_heads, window_size=config.window_size,
                block_size=getattr(config, "block_size", 64), n_persistent=config.n_persistent,
                dropout=config.attention_dropout, causal=config.causal)
        else:
            self.attention = WindowedAttention(config)
        self.mlp = MLPBlock(d_model=config.d_model, d_ff=config.d_ff, dropout=config.dropout)

    def forward(self, x: torch.Tensor, attn_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        a = self.attention(self.norm_attn(x), attn_mask=attn_mask)
        x, h = self.norm_mlp.add_forward(x, a)
        return x + self.mlp(h)
