"""CPU oracle for TitanMAC's WindowedAttention hot path.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain CPU PyTorch, what the reference module
``titans_core/attn/windowed_attention.py`` computes.  It exists so that the CUDA
path can be checked against something that does not share any code with it.  It
is imported only by the tests, by the smoke check and by the benchmark's CPU
baseline / reference arm; the shipped package never imports it and has no CPU
fallback.

Parity status: PINNED.  The functions below are checked against outputs of the
reference module itself (imported from the reference checkout when the golden
fixtures under ``tests/golden/`` were generated; the generating script sits
beside the fixtures).  The reference has no tests or golden vectors of its own
for this module.

Every function cites the reference lines it follows as ``file:line``.
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

# --------------------------------------------------------------------------- #
# Mask
# --------------------------------------------------------------------------- #


def validate_mask_args(seq_len: int, window_size: int, n_persistent: int) -> None:
    """Argument checks of ``build_band_mask`` (windowed_attention.py:97-103)."""
    if n_persistent >= seq_len:
        raise ValueError(
            f"num_persistent_tokens ({n_persistent}) must be < seq_len ({seq_len})"
        )
    if window_size < 0:
        raise ValueError(f"window_size must be non-negative, got {window_size}")


def visible(i: int, j: int, window_size: int, n_persistent: int, causal: bool = True) -> bool:
    """Scalar form of the mask: may query row ``i`` attend to key column ``j``?

    windowed_attention.py:113-118 — every row sees the persistent columns
    ``j < Np``; rows ``i < Np`` see nothing else (the ``if causal: pass`` block at
    :122-132 leaves ``mask[:Np, Np:]`` False, also when ``causal`` is False).
    windowed_attention.py:134-150 — sequence rows see ``|i-j| <= w`` and, when
    causal, ``i >= j``; both restricted to ``j >= Np``.
    """
    if j < n_persistent:
        return True
    if i < n_persistent:
        return False
    if abs(i - j) > window_size:
        return False
    if causal and j > i:
        return False
    return True


def band_mask(seq_len: int, window_size: int, n_persistent: int, causal: bool = True) -> torch.Tensor:
    """Dense boolean mask ``[L, L]`` (True = attend), windowed_attention.py:61-152."""
    validate_mask_args(seq_len, window_size, n_persistent)
    pos = torch.arange(seq_len)
    i = pos[:, None]
    j = pos[None, :]
    seq = (i >= n_persistent) & (j >= n_persistent) & ((i - j).abs() <= window_size)
    if causal:
        seq = seq & (i >= j)
    return (j < n_persistent) | seq


def live_pairs(seq_len: int, window_size: int, n_persistent: int) -> int:
    """Number of True entries of the causal mask, in closed form (no L×L array)."""
    validate_mask_args(seq_len, window_size, n_persistent)
    t = seq_len - n_persistent
    w = window_size
    full = max(0, t - w)  # rows with a complete window of w+1 keys
    ramp = min(t, w)  # rows 0..ramp-1 see t'+1 keys
    seq_pairs = ramp * (ramp + 1) // 2 + full * (w + 1)
    return seq_pairs + n_persistent * t + n_persistent * n_persistent


# --------------------------------------------------------------------------- #
# Attention core
# --------------------------------------------------------------------------- #


def attention_core_dense(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    window_size: int,
    n_persistent: int,
    causal: bool = True,
    scale: Optional[float] = None,
    compute_dtype: torch.dtype = torch.float32,
) -> torch.Tensor:
    """softmax(Q Kᵀ · scale + M) V over the dense mask.  q, k, v: ``[B, H, L, dh]``.

    windowed_attention.py:307-323: the boolean mask becomes an additive 0 / -inf
    mask and goes through scaled-dot-product attention with the default scale
    ``1/sqrt(dh)`` and no dropout in eval mode.  Written out here as explicit
    matmul → masked_fill → softmax → matmul so that it does not depend on the
    fused library routine.
    """
    B, H, L, dh = q.shape
    if scale is None:
        scale = 1.0 / math.sqrt(dh)
    mask = band_mask(L, window_size, n_persistent, causal)
    qf, kf, vf = (t.to(compute_dtype) for t in (q, k, v))
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.matmul(p, vf)


def attention_core_rows(
    q_rows: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    row0: int,
    window_size: int,
    n_persistent: int,
    scale: Optional[float] = None,
    compute_dtype: torch.dtype = torch.float32,
) -> torch.Tensor:
    """The same formula for the query rows ``[row0, row0+R)`` only (causal mask).

    ``q_rows``: ``[B, H, R, dh]``; ``k``, ``v``: ``[B, H, L, dh]`` with the
    persistent prefix at rows ``[0, Np)``.  Only the key columns that
    windowed_attention.py:113-150 can leave unmasked for these rows are
    touched — ``[0, Np) ∪ [row0 - w, row0 + R)`` — so this runs at sequence
    lengths where the reference's dense ``L×L`` mask cannot be allocated.
    """
    B, H, R, dh = q_rows.shape
    if scale is None:
        scale = 1.0 / math.sqrt(dh)
    Np, w = n_persistent, window_size
    lo = max(Np, row0 - w)
    hi = row0 + R
    cols = torch.cat([torch.arange(0, Np), torch.arange(lo, hi)]) if hi > lo else torch.arange(0, Np)
    i = torch.arange(row0, row0 + R)[:, None]
    j = cols[None, :]
    m = (j < Np) | ((i >= Np) & (j >= Np) & (j <= i) & (i - j <= w))
    qf = q_rows.to(compute_dtype)
    kf = k[:, :, cols].to(compute_dtype)
    vf = v[:, :, cols].to(compute_dtype)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    s = s.masked_fill(~m, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.matmul(p, vf)


def attention_core_blockwise(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    window_size: int,
    n_persistent: int,
    block: int = 1024,
    scale: Optional[float] = None,
    compute_dtype: torch.dtype = torch.float32,
) -> torch.Tensor:
    """All rows, evaluated ``block`` rows at a time through ``attention_core_rows``."""
    L = q.shape[2]
    validate_mask_args(L, window_size, n_persistent)
    out = torch.empty(q.shape, dtype=compute_dtype)
    for r0 in range(0, L, block):
        r1 = min(L, r0 + block)
        out[:, :, r0:r1] = attention_core_rows(
            q[:, :, r0:r1], k, v, r0, window_size, n_persistent, scale, compute_dtype
        )
    return out


# --------------------------------------------------------------------------- #
# Module forward
# --------------------------------------------------------------------------- #


def split_heads(qkv: torch.Tensor, n_heads: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``[B, L, 3D]`` → three ``[B, H, L, dh]`` tensors.

    windowed_attention.py:298-304: Q, K, V are the three consecutive thirds of
    the last axis; head ``h`` is columns ``[h·dh, (h+1)·dh)`` of its third.
    """
    B, L, D3 = qkv.shape
    D = D3 // 3
    dh = D // n_heads
    q, k, v = qkv.split(D, dim=-1)
    shape = (B, L, n_heads, dh)
    return tuple(t.reshape(shape).permute(0, 2, 1, 3) for t in (q, k, v))


def module_forward(
    x: torch.Tensor,
    w_qkv: torch.Tensor,
    w_out: torch.Tensor,
    n_heads: int,
    window_size: int,
    n_persistent: int,
    causal: bool = True,
    compute_dtype: torch.dtype = torch.float32,
    blockwise: bool = False,
) -> torch.Tensor:
    """Whole ``WindowedAttention.forward`` in eval mode (windowed_attention.py:277-334).

    ``x``: ``[B, L, D]`` whose first ``Np`` rows are the persistent prefix;
    ``w_qkv``: ``[3D, D]`` and ``w_out``: ``[D, D]`` (``nn.Linear`` weights, no
    bias, :233-236).  Inputs of any float dtype are promoted to
    ``compute_dtype`` — feeding bf16-rounded tensors gives the fp32 result for
    exactly those rounded values.
    """
    B, L, D = x.shape
    validate_mask_args(L, window_size, n_persistent)
    xf = x.to(compute_dtype)
    qkv = xf @ w_qkv.to(compute_dtype).t()  # :295
    q, k, v = split_heads(qkv, n_heads)  # :298-304
    if blockwise:
        assert causal
        o = attention_core_blockwise(q, k, v, window_size, n_persistent, compute_dtype=compute_dtype)
    else:
        o = attention_core_dense(q, k, v, window_size, n_persistent, causal, compute_dtype=compute_dtype)
    o = o.permute(0, 2, 1, 3).reshape(B, L, D)  # :327-328
    return o @ w_out.to(compute_dtype).t()  # :331


def module_forward_reference_cost(
    x: torch.Tensor,
    w_qkv: torch.Tensor,
    w_out: torch.Tensor,
    n_heads: int,
    window_size: int,
    n_persistent: int,
    mask_cache: Optional[dict] = None,
) -> torch.Tensor:
    """The forward with the same *cost structure* as the reference on CPU.

    Used only as the timed CPU baseline.  It does what the reference does per
    call in the input dtype: two bias-free linears, a dense ``L×L`` additive
    mask rebuilt from the cached boolean mask on every call
    (windowed_attention.py:311-313) and the library's fused
    scaled-dot-product attention over all ``L×L`` pairs (:318-323).  The
    boolean mask is cached per length like the module's ``_mask_cache``
    (:262-273).
    """
    import torch.nn.functional as F

    B, L, D = x.shape
    if mask_cache is None:
        mask_cache = {}
    if L not in mask_cache:
        mask_cache[L] = band_mask(L, window_size, n_persistent, True)
    mask = mask_cache[L]
    qkv = F.linear(x, w_qkv)
    q, k, v = split_heads(qkv, n_heads)
    add = torch.zeros(mask.shape, dtype=x.dtype)
    add.masked_fill_(~mask, float("-inf"))
    o = F.scaled_dot_product_attention(q, k, v, attn_mask=add, dropout_p=0.0, is_causal=False)
    o = o.transpose(1, 2).reshape(B, L, D)
    return F.linear(o, w_out)


# --------------------------------------------------------------------------- #
# Decode
# --------------------------------------------------------------------------- #


def decode_row(
    q_row: torch.Tensor,
    k_pers: torch.Tensor,
    v_pers: torch.Tensor,
    k_win: torch.Tensor,
    v_win: torch.Tensor,
    scale: Optional[float] = None,
    compute_dtype: torch.dtype = torch.float32,
) -> torch.Tensor:
    """One new token's attention output.

    The reference has no incremental decode: its generation helper re-runs the
    whole forward per token and keeps the last row (examples/train_math.py:146-161).
    That last row attends to the ``Np`` persistent keys plus the current token
    and its ``w`` predecessors (windowed_attention.py:136-150), so the decode
    oracle is the softmax over exactly those keys, in any order.

    ``q_row``: ``[B, H, dh]``; ``k_pers``/``v_pers``: ``[H, Np, dh]`` (shared by
    the batch) ; ``k_win``/``v_win``: ``[B, H, n, dh]`` — the ``n <= w+1`` most
    recent sequence keys including the current token.
    """
    B, H, dh = q_row.shape
    if scale is None:
        scale = 1.0 / math.sqrt(dh)
    qf = q_row.to(compute_dtype)[:, :, None, :]
    kp = k_pers.to(compute_dtype)[None].expand(B, -1, -1, -1)
    vp = v_pers.to(compute_dtype)[None].expand(B, -1, -1, -1)
    kk = torch.cat([kp, k_win.to(compute_dtype)], dim=2)
    vv = torch.cat([vp, v_win.to(compute_dtype)], dim=2)
    s = torch.matmul(qf, kk.transpose(-1, -2)) * scale
    p = torch.softmax(s, dim=-1)
    return torch.matmul(p, vv)[:, :, 0, :]


# --------------------------------------------------------------------------- #
# Seeded synthetic inputs (shared by tests, smoke and bench so that every
# consumer draws the same numbers in the same order)
# --------------------------------------------------------------------------- #


def layer_inputs(
    batch: int,
    seq_tokens: int,
    d_model: int,
    n_persistent: int,
    seed: int = 0,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``x [B, Np+T, D] ~ N(0,1)`` with a batch-shared persistent prefix, and
    ``w_qkv [3D, D]``, ``w_out [D, D] ~ N(0, 0.02)``; CPU fp32, fixed draw order.

    The prefix rows are identical for every batch element because that is what
    the model delivers at the block's call site: it prepends the same
    ``persistent_tokens`` parameter to each sequence (models/titanmac.py:608-619).
    """
    g = torch.Generator(device="cpu").manual_seed(seed)
    w_qkv = torch.randn(3 * d_model, d_model, generator=g) * 0.02
    w_out = torch.randn(d_model, d_model, generator=g) * 0.02
    pers = torch.randn(n_persistent, d_model, generator=g)
    seq = torch.randn(batch, seq_tokens, d_model, generator=g)
    x = torch.cat([pers[None].expand(batch, -1, -1), seq], dim=1).contiguous()
    return x, w_qkv, w_out


def qkv_inputs(
    batch: int, heads: int, length: int, head_dim: int, seed: int = 0
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Q, K, V ``[B, H, L, dh] ~ N(0,1)``, CPU fp32, fixed draw order."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    q = torch.randn(batch, heads, length, head_dim, generator=g)
    k = torch.randn(batch, heads, length, head_dim, generator=g)
    v = torch.randn(batch, heads, length, head_dim, generator=g)
    return q, k, v
