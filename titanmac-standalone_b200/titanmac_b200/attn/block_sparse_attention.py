"""Drop-in for the reference's ``BlockSparseAttention`` (its default attention class) on B200.

Same constructor arguments, attributes and ``state_dict`` keys (``qkv_proj.weight``,
``conv_q.weight``, ``conv_k.weight``, ``conv_v.weight`` of shape ``[d_model, 1, taps]``,
``out_proj.weight``) and ``forward(x, attn_mask=None)`` as
titans_core/attn/block_sparse_attention.py:27-343, and the same factory
``create_block_sparse_attention(config)`` (:346-368), so ``TitanBlock`` can pick it for
``use_block_sparse=True`` like the reference does (titans_core/blocks/titan_block.py:51-64).

What the reference does in Python — three transposed Conv1d calls, then a loop over query blocks
that concatenates each block's keys, builds a mask and runs a softmax — is two launches here:
``tmw_causal_dwconv`` over the whole QKV projection output (the three filters stacked) and
``tmw_prefill_block_sparse`` reading Q, K, V as strided views of the result.

Not supported (raises ``NotImplementedError``): ``causal=False`` and dropout in training mode.  With grad
mode on and a gradient due, the attention core runs as an autograd function (``tmw_prefill_block_sparse_lse`` /
``tmw_prefill_block_sparse_backward``), and so do the convolutions (``tmw_causal_dwconv_backward``).  Like the reference, a caller-supplied ``attn_mask`` is ignored (:218-219).
The ring-cache generation path of ``TitanMAC`` belongs to ``WindowedAttention`` only.
"""

from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn

from .. import _native


class _CausalDwConv(torch.autograd.Function):
    """``tmw_causal_dwconv`` with ``tmw_causal_dwconv_backward``: ``x [B, T, C]``, ``weight [C, taps]``."""

    @staticmethod
    def forward(ctx, x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        x, weight = x.contiguous(), weight.contiguous()
        ctx.save_for_backward(x, weight)
        return _native.causal_dwconv(x, weight)

    @staticmethod
    def backward(ctx, dy: torch.Tensor):
        x, weight = ctx.saved_tensors
        return _native.causal_dwconv_backward(x, weight, dy)


class _BlockSparseCore(torch.autograd.Function):
    """``qkv [B, L, 3, H, dh]`` (after the convolutions) → ``o [B, L, H, dh]``; backward through
    ``tmw_prefill_block_sparse_backward``."""

    @staticmethod
    def forward(ctx, qkv: torch.Tensor, window: int, block: int, n_persistent: int, scale: float, algo: int):
        qkv = qkv.contiguous()
        B, L, _, H, dh = qkv.shape
        q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))
        o = torch.empty((B, L, H, dh), dtype=qkv.dtype, device=qkv.device)
        lse = torch.empty((B * H * L,), dtype=torch.float32, device=qkv.device)
        _native.prefill(q, k, v, window, n_persistent, out=o.permute(0, 2, 1, 3), scale=scale, algo=algo,
                        window_block=block, lse=lse)
        ctx.save_for_backward(qkv, o, lse)
        ctx.args = (window, block, n_persistent, scale)
        return o

    @staticmethod
    def backward(ctx, d_o: torch.Tensor):
        qkv, o, lse = ctx.saved_tensors
        window, block, n_persistent, scale = ctx.args
        d_o = d_o.contiguous()
        dqkv = torch.empty_like(qkv)
        q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))
        dq, dk, dv = (dqkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))
        _native.prefill_backward(q, k, v, o.permute(0, 2, 1, 3), d_o.permute(0, 2, 1, 3), lse, dq, dk, dv, window,
                                 n_persistent, scale=scale, window_block=block)
        return dqkv, None, None, None, None, None


class BlockSparseAttention(nn.Module):
    def __init__(self, d_model: int, n_heads: int, window_size: int = 512, block_size: int = 64,
                 n_persistent: int = 0, dropout: float = 0.0, causal: bool = True, use_conv: bool = True,
                 conv_kernel: int = 4):
        super().__init__()
        if d_model % n_heads != 0:
            raise ValueError(f"d_model ({d_model}) must be divisible by n_heads ({n_heads})")
        self.d_model, self.n_heads, self.d_head = d_model, n_heads, d_model // n_heads
        self.window_size, self.block_size, self.n_persistent = window_size, block_size, n_persistent
        self.dropout_p, self.causal, self.use_conv = dropout, causal, use_conv
        self.qkv_proj = nn.Linear(d_model, 3 * d_model, bias=False)
        if use_conv:
            mk = lambda: nn.Conv1d(d_model, d_model, kernel_size=conv_kernel, padding=conv_kernel - 1,  # noqa: E731
                                   groups=d_model, bias=False)
            self.conv_q, self.conv_k, self.conv_v = mk(), mk(), mk()
        self.out_proj = nn.Linear(d_model, d_model, bias=False)
        self.dropout = nn.Dropout(dropout) if dropout > 0 else nn.Identity()
        self.scale = 1.0 / math.sqrt(self.d_head)
        self.algo = _native.ALGO_AUTO   # tmw_algo passed to the library (tests pin a kernel)
        self.core_events = None         # see WindowedAttention.core_events

    def stacked_conv_weight(self) -> torch.Tensor:
        """``[3 * d_model, taps]``: the three depthwise filters in the channel order of the QKV projection."""
        return torch.cat([self.conv_q.weight[:, 0], self.conv_k.weight[:, 0], self.conv_v.weight[:, 0]], dim=0)

    def forward(self, x: torch.Tensor, attn_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        if torch.is_grad_enabled() and (x.requires_grad or any(p.requires_grad for p in self.parameters())):
            return self._forward_train(x)
        with torch.no_grad():
            return self._forward(x)

    def _forward_train(self, x: torch.Tensor) -> torch.Tensor:
        """Grad mode: the projections are differentiable library calls; the depthwise convolutions and the attention
        core are autograd functions with their own backward kernels."""
        if not self.causal:
            raise NotImplementedError("causal=False is not supported")
        if self.training and self.dropout_p > 0:
            raise NotImplementedError("attention dropout in training mode is not supported")
        if not x.is_cuda:
            raise RuntimeError("BlockSparseAttention (B200) needs CUDA tensors; there is no CPU path")
        B, L, D = x.shape
        if self.n_persistent >= L:
            raise ValueError(f"n_persistent ({self.n_persistent}) must be < seq_len ({L})")
        qkv = self.qkv_proj(x)
        if self.use_conv:
            qkv = _CausalDwConv.apply(qkv, self.stacked_conv_weight())
        o = _BlockSparseCore.apply(qkv.reshape(B, L, 3, self.n_heads, self.d_head), self.window_size, self.block_size,
                                   self.n_persistent, self.scale, self.algo)
        return self.dropout(self.out_proj(o.view(B, L, D)))

    def _forward(self, x: torch.Tensor) -> torch.Tensor:
        if not self.causal:
            raise NotImplementedError("causal=False is not supported")
        if self.training and self.dropout_p > 0:
            raise NotImplementedError("attention dropout in training mode is not supported")
        if not x.is_cuda:
            raise RuntimeError("BlockSparseAttention (B200) needs CUDA tensors; there is no CPU path")
        B, L, D = x.shape
        if self.n_persistent >= L:
            raise ValueError(f"n_persistent ({self.n_persistent}) must be < seq_len ({L})")
        qkv = _native.project(self.qkv_proj, x)
        if self.use_conv:
            qkv = _native.causal_dwconv(qkv, self.stacked_conv_weight())
        v5 = qkv.view(B, L, 3, self.n_heads, self.d_head)
        q, k, v = (v5[:, :, i].permute(0, 2, 1, 3) for i in range(3))
        o = torch.empty((B, L, self.n_heads, self.d_head), dtype=qkv.dtype, device=qkv.device)
        if self.core_events is not None:
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
        _native.prefill(q, k, v, self.window_size, self.n_persistent, out=o.permute(0, 2, 1, 3), scale=self.scale,
                        algo=self.algo, window_block=self.block_size)
        if self.core_events is not None:
            end.record()
            self.core_events.append((start, end))
        return self.dropout(_native.project(self.out_proj, o.view(B, L, D)))


def create_block_sparse_attention(config) -> BlockSparseAttention:
    """From a ``TitanMACConfig``; block size ``config.block_size`` if present, else ``max(64, window_size // 8)``
    (block_sparse_attention.py:356-368)."""
    block_size = getattr(config, "block_size", max(64, config.window_size // 8))
    return BlockSparseAttention(d_model=config.d_model, n_heads=config.n_heads, window_size=config.window_size,
                                block_size=block_size, n_persistent=config.n_persistent,
                                dropout=config.attention_dropout, causal=config.causal)
