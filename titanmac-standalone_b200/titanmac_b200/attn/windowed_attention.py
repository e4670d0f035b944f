"""Drop-in for the reference's ``WindowedAttention`` module on B200.

Same constructor, attributes, ``state_dict`` keys (``qkv_proj.weight``,
``out_proj.weight``) and ``forward(x, attn_mask=None)`` as
titans_core/attn/windowed_attention.py:179-334, so the block's call site
(titans_core/blocks/titan_block.py:64 and :94) works unchanged.  What differs is
what happens inside ``forward``: no ``L×L`` mask is built or converted, and the
attention core is ``tmw_prefill`` from libtmw reading Q, K, V as strided views of
the projection output and writing straight into the head-concatenated layout.

Not supported (raises ``NotImplementedError``): a caller-supplied ``attn_mask``
(every caller in the reference passes ``None``), ``causal=False`` and dropout in
training mode.  When a gradient is wanted (grad mode on and the input or a weight
requires one) the attention core runs as an autograd function whose backward is
``tmw_prefill_backward``; otherwise nothing is saved.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import _native


class _WindowedCore(torch.autograd.Function):
    """``qkv [B, L, 3, H, dh]`` → ``o [B, L, H, dh]`` with ``tmw_prefill_lse`` / ``tmw_prefill_backward``."""

    @staticmethod
    def forward(ctx, qkv: torch.Tensor, window: int, n_persistent: int, algo: int) -> torch.Tensor:
        qkv = qkv.contiguous()
        B, L, _, H, dh = qkv.shape
        q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))
        o = torch.empty((B, L, H, dh), dtype=qkv.dtype, device=qkv.device)
        lse = torch.empty((B, H, L), dtype=torch.float32, device=qkv.device)
        _native.prefill(q, k, v, window, n_persistent, out=o.permute(0, 2, 1, 3), algo=algo, lse=lse)
        ctx.save_for_backward(qkv, o, lse)
        ctx.window, ctx.n_persistent = window, n_persistent
        return o

    @staticmethod
    def backward(ctx, d_o: torch.Tensor):
        qkv, o, lse = ctx.saved_tensors
        d_o = d_o.contiguous()
        dqkv = torch.empty_like(qkv)
        q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))
        dq, dk, dv = (dqkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))
        _native.prefill_backward(q, k, v, o.permute(0, 2, 1, 3), d_o.permute(0, 2, 1, 3), lse, dq, dk, dv,
                                 ctx.window, ctx.n_persistent)
        return dqkv, None, None, None


class WindowedAttention(nn.Module):
    """Causal sliding-window attention with persistent prefix rows.

    ``x`` is ``[B, L, d_model]`` whose first ``n_persistent`` rows are the
    persistent rows: they attend to one another only; every later row attends to
    all of them plus itself and its ``window_size`` predecessors.
    """

    def __init__(self, config):
        super().__init__()
        if hasattr(config, "num_heads"):  # WindowConfig
            self.d_model = config.num_heads * config.head_dim
            self.n_heads = config.num_heads
            self.d_head = config.head_dim
            self.window_size = config.window_size
            self.num_persistent = config.n_persistent
            self.causal = config.causal
            self.dropout_p = config.dropout
        else:  # TitanMACConfig
            self.d_model = config.d_model
            self.n_heads = config.n_heads
            self.d_head = config.d_head
            self.window_size = config.window_size
            self.num_persistent = config.n_persistent
            self.causal = config.causal
            self.dropout_p = config.attention_dropout

        assert self.d_model == self.n_heads * self.d_head, (
            f"d_model ({self.d_model}) must equal n_heads ({self.n_heads}) * d_head ({self.d_head})"
        )
        self.qkv_proj = nn.Linear(self.d_model, 3 * self.d_model, bias=False)
        self.out_proj = nn.Linear(self.d_model, self.d_model, bias=False)
        self.dropout = nn.Dropout(self.dropout_p) if self.dropout_p > 0 else nn.Identity()
        # tmw_algo passed to the library: 0 lets it choose, 1/2 pin a kernel (tests)
        self.algo = _native.ALGO_AUTO
        # when set to a list, forward() appends a (start, end) CUDA event pair around the
        # attention-core launch; used by the benchmark to time that kernel in place
        self.core_events = None

    # -- checks shared by forward() and the generation path -------------------------
    def _check_supported(self, x: torch.Tensor, attn_mask: Optional[torch.Tensor]) -> None:
        if attn_mask is not None:
            raise NotImplementedError("a caller-supplied attn_mask is not supported; pass None")
        if not self.causal:
            raise NotImplementedError("causal=False is not supported")
        if self.training and self.dropout_p > 0:
            raise NotImplementedError("attention dropout in training mode is not supported")
        if not x.is_cuda:
            raise RuntimeError("WindowedAttention (B200) needs CUDA tensors; there is no CPU path")

    def _check_lengths(self, seq_len: int) -> None:
        # same conditions and messages as build_band_mask in the reference
        if self.num_persistent >= seq_len:
            raise ValueError(
                f"num_persistent_tokens ({self.num_persistent}) must be < seq_len ({seq_len})"
            )
        if self.window_size < 0:
            raise ValueError(f"window_size must be non-negative, got {self.window_size}")

    def split_qkv(self, qkv: torch.Tensor):
        """``[B, L, 3D]`` → strided ``[B, H, L, dh]`` views of Q, K, V (no copies)."""
        B, L, _ = qkv.shape
        v5 = qkv.view(B, L, 3, self.n_heads, self.d_head)
        return tuple(v5[:, :, i].permute(0, 2, 1, 3) for i in range(3))

    def forward(self, x: torch.Tensor, attn_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        B, L, D = x.shape
        self._check_lengths(L)
        self._check_supported(x, attn_mask)
        if torch.is_grad_enabled() and (x.requires_grad or self.qkv_proj.weight.requires_grad
                                        or self.out_proj.weight.requires_grad):
            qkv = self.qkv_proj(x).view(B, L, 3, self.n_heads, self.d_head)
            o = _WindowedCore.apply(qkv, self.window_size, self.num_persistent, self.algo)
            return self.dropout(self.out_proj(o.view(B, L, D)))
        with torch.no_grad():
            return self._forward_no_grad(x)

    def _forward_no_grad(self, x: torch.Tensor) -> torch.Tensor:
        B, L, D = x.shape
        qkv = _native.project(self.qkv_proj, x)  # tmw_linear: [B, L, 3, H, dh] is just its row-major output
        q, k, v = self.split_qkv(qkv)
        # the output is allocated as [B, L, H, dh] so that "concat heads" is a view
        o = torch.empty((B, L, self.n_heads, self.d_head), dtype=qkv.dtype, device=qkv.device)
        if self.core_events is not None:
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
        _native.prefill(q, k, v, self.window_size, self.num_persistent, out=o.permute(0, 2, 1, 3),
                        algo=self.algo)
        if self.core_events is not None:
            end.record()
            self.core_events.append((start, end))
        return self.dropout(_native.project(self.out_proj, o.view(B, L, D)))
