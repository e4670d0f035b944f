"""CPU restatement of the reference's BlockSparseAttention (test infrastructure, not product code).

The reference's default attention class (titans_core/config.py:91 ``use_block_sparse=True``,
titans_core/attn/block_sparse_attention.py) differs from WindowedAttention in three ways, all
restated here from its forward (block_sparse_attention.py:223-343):

* a causal depthwise convolution of width 4 over the WHOLE row axis (persistent rows included)
  after the QKV projection, one filter per channel, separately for Q, K and V (:77-92, :241-256);
* the window's left edge is block-granular: the sequence row with sequence index ``t`` in block
  ``b = t // block_size`` sees the sequence keys ``max(0, b * block_size - window) .. t``
  (:299-311, causal part :147-156) plus every persistent key (:313-316);
* the ``Np`` persistent query rows see EVERY key, later rows included, with no mask (:283-291).

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU legs of ``bench.py`` may import this file.
Pinned against outputs of the unmodified reference: ``tests/golden/block_sparse_golden.npz``
(made by ``tests/golden/make_block_sparse_golden.py``).
"""

from __future__ import annotations

import math
from typing import Optional

import torch


def causal_dwconv(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``x [B, T, C]``, ``weight [C, K]`` → ``y[b, t, c] = sum_k weight[c, k] * x[b, t - (K-1) + k, c]``
    with zeros before the first row (Conv1d with padding K-1 trimmed to T, :247-251)."""
    B, T, C = x.shape
    K = weight.shape[1]
    xp = torch.cat([torch.zeros(B, K - 1, C, dtype=x.dtype), x], dim=1)
    y = torch.zeros_like(x)
    for k in range(K):
        y = y + xp[:, k:k + T] * weight[:, k]
    return y


def first_visible_key(t: int, window: int, block_size: int) -> int:
    """Sequence index of the first sequence key that the sequence row ``t`` sees (:299-305)."""
    return max(0, (t // block_size) * block_size - window)


def mask(seq_len: int, window: int, block_size: int, n_persistent: int) -> torch.Tensor:
    """Boolean ``[L, L]`` visibility over all rows (persistent rows first)."""
    L, Np = seq_len, n_persistent
    m = torch.zeros(L, L, dtype=torch.bool)
    m[:Np, :] = True            # persistent query rows: every key (:283-291)
    m[Np:, :Np] = True          # persistent keys for every sequence row (:313-316)
    for t in range(L - Np):
        m[Np + t, Np + first_visible_key(t, window, block_size):Np + t + 1] = True
    return m


def attention_core(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int, block_size: int,
                   n_persistent: int, scale: Optional[float] = None) -> torch.Tensor:
    """``q, k, v [B, H, L, dh]`` (after the convolutions) → ``[B, H, L, dh]``, fp32."""
    dh = q.shape[-1]
    scale = 1.0 / math.sqrt(dh) if scale is None else scale
    s = torch.matmul(q.float(), k.float().transpose(-1, -2)) * scale
    s = s.masked_fill(~mask(q.shape[2], window, block_size, n_persistent), float("-inf"))
    return torch.matmul(torch.softmax(s, dim=-1), v.float())


def module_forward(x: torch.Tensor, w_qkv: torch.Tensor, conv_q: torch.Tensor, conv_k: torch.Tensor,
                   conv_v: torch.Tensor, w_out: torch.Tensor, n_heads: int, window: int, block_size: int,
                   n_persistent: int, return_parts: bool = False):
    """The whole module in fp32.  ``conv_* [D, K]`` (the Conv1d weights ``[D, 1, K]`` squeezed)."""
    B, L, D = x.shape
    dh = D // n_heads
    qkv = x.float() @ w_qkv.float().t()
    q, k, v = qkv.chunk(3, dim=-1)
    q, k, v = causal_dwconv(q, conv_q.float()), causal_dwconv(k, conv_k.float()), causal_dwconv(v, conv_v.float())
    heads = lambda t: t.view(B, L, n_heads, dh).transpose(1, 2)  # noqa: E731
    o = attention_core(heads(q), heads(k), heads(v), window, block_size, n_persistent)
    y = o.transpose(1, 2).reshape(B, L, D) @ w_out.float().t()
    return (y, q, k, v, o) if return_parts else y


def live_pairs(seq_len: int, window: int, block_size: int, n_persistent: int) -> int:
    """Visible (query, key) pairs per (batch, head): the algorithmic work of the attention core."""
    Np, T = n_persistent, seq_len - n_persistent
    pairs = Np * seq_len + T * Np
    for t0 in range(0, T, block_size):
        lo = max(0, t0 - window)
        n = min(block_size, T - t0)
        pairs += n * (t0 - lo) + n * (n + 1) // 2
    return pairs


def module_forward_reference_cost(x: torch.Tensor, w_qkv: torch.Tensor, conv_q: torch.Tensor, conv_k: torch.Tensor,
                                  conv_v: torch.Tensor, w_out: torch.Tensor, n_heads: int, window: int,
                                  block_size: int, n_persistent: int) -> torch.Tensor:
    """The forward with the same cost structure as the reference on CPU (the timed CPU baseline only):
    library depthwise Conv1d calls on transposed tensors (block_sparse_attention.py:241-256), dense
    attention of the persistent rows over every key (:283-291), then a Python loop over query blocks that
    concatenates the block's keys, builds its mask and runs matmul / softmax / matmul (:294-343)."""
    import torch.nn.functional as F

    B, L, D = x.shape
    Np, dh, K = n_persistent, D // n_heads, conv_q.shape[1]
    qkv = F.linear(x, w_qkv)
    parts = []
    for t, w in zip(qkv.chunk(3, dim=-1), (conv_q, conv_k, conv_v)):
        y = F.conv1d(t.transpose(1, 2), w[:, None, :].to(t.dtype), padding=K - 1, groups=D)[:, :, :L]
        parts.append(y.transpose(1, 2).reshape(B, L, n_heads, dh).transpose(1, 2))
    q, k, v = parts
    scale = 1.0 / math.sqrt(dh)
    out = torch.empty(B, n_heads, L, dh, dtype=x.dtype)
    if Np > 0:
        s = torch.matmul(q[:, :, :Np], k.transpose(-2, -1)) * scale
        out[:, :, :Np] = torch.matmul(F.softmax(s, dim=-1), v)
    T = L - Np
    for b0 in range(0, T, block_size):
        b1 = min(b0 + block_size, T)
        c0 = max(0, b0 - window)
        kc = torch.cat([k[:, :, :Np], k[:, :, Np + c0:Np + b1]], dim=2)
        vc = torch.cat([v[:, :, :Np], v[:, :, Np + c0:Np + b1]], dim=2)
        m = torch.ones(b1 - b0, Np + b1 - c0, dtype=torch.bool)
        m[:, Np:] = torch.arange(b0, b1)[:, None] >= torch.arange(c0, b1)[None, :]
        s = (torch.matmul(q[:, :, Np + b0:Np + b1], kc.transpose(-2, -1)) * scale).masked_fill(~m, float("-inf"))
        out[:, :, Np + b0:Np + b1] = torch.matmul(F.softmax(s, dim=-1), vc)
    return F.linear(out.transpose(1, 2).reshape(B, L, D), w_out)
