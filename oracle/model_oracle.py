"""CPU restatement of the reference's TitanBlock / TitanMAC forward around the windowed attention.

TEST INFRASTRUCTURE ONLY: imported by ``tests/`` (never by the package or by a timed region).  It exists so
that the model-level parity of benchmark configurations 3 and 4 (16 layers, 8192-token sequences, 2048 + 64
teacher-forced tokens) can be checked where the reference itself cannot run: its dense ``L x L`` mask and
scores do not fit in memory at those lengths, here the attention goes row block by row block through
``windowed_oracle.attention_core_blockwise`` (the same formula on the keys a block can see).

Restated from the reference project (paths inside it):
  titans_core/blocks/norms.py:55-58         RMSNorm: x / sqrt(mean(x^2) + eps) * scale
  titans_core/blocks/mlp.py:58-65           fc1 (+bias) -> exact (erf) GELU -> fc2 (+bias)
  titans_core/blocks/titan_block.py:92-100  x + attention(norm_attn(x)); x + mlp(norm_mlp(x))
  titans_core/models/titanmac.py:608-662    token + position embeddings on the sequence rows, the persistent
                                            tokens prepended, final norm, LM head over all rows, then the
                                            persistent rows dropped
Parity pinned: ``tests/test_oracle_golden.py`` holds ``model_forward`` / ``block_forward`` against the logits and
block outputs that the unmodified reference produced (``tests/golden/titanmac_golden.npz``).

All arithmetic is fp32 on the weights as given (round them to bf16 first to get "fp32 math on bf16-rounded
weights", the reference point of the 16-bit tolerance).
"""

from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch
import torch.nn.functional as F

from . import windowed_oracle as wo


def rms_norm(x: torch.Tensor, scale: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    """norms.py:55-58."""
    return x / torch.sqrt(torch.mean(x * x, dim=-1, keepdim=True) + eps) * scale


def attention_forward(x: torch.Tensor, w_qkv: torch.Tensor, w_out: torch.Tensor, n_heads: int, window: int,
                      n_persistent: int, block: int = 1024) -> torch.Tensor:
    """windowed_attention.py:295-332 with the attention core evaluated block-wise."""
    B, L, D = x.shape
    q, k, v = wo.split_heads(F.linear(x, w_qkv), n_heads)
    o = wo.attention_core_blockwise(q, k, v, window, n_persistent, block=block)
    return F.linear(o.permute(0, 2, 1, 3).reshape(B, L, D), w_out)


def block_forward(x: torch.Tensor, sd: Dict[str, torch.Tensor], prefix: str, n_heads: int, window: int,
                  n_persistent: int, eps: float = 1e-5) -> torch.Tensor:
    """titan_block.py:92-100 on the parameters ``sd[prefix + ...]`` (the reference's state_dict names)."""
    g = lambda name: sd[prefix + name].float()  # noqa: E731
    x = x + attention_forward(rms_norm(x, g("norm_attn.scale"), eps), g("attention.qkv_proj.weight"),
                              g("attention.out_proj.weight"), n_heads, window, n_persistent)
    h = rms_norm(x, g("norm_mlp.scale"), eps)
    h = F.gelu(F.linear(h, g("mlp.fc1.weight"), g("mlp.fc1.bias")))  # exact erf form, mlp.py:42
    return x + F.linear(h, g("mlp.fc2.weight"), g("mlp.fc2.bias"))


def model_forward(sd: Dict[str, torch.Tensor], ids: torch.Tensor, n_layers: int, n_heads: int, window: int,
                  n_persistent: int, eps: float = 1e-5, positions: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Logits ``[B, T, V]`` of ``ids [B, T]`` (titanmac.py:608-662), or ``[B, len(positions), V]`` for the given
    sequence positions only (the LM head is the most expensive product of the forward)."""
    B, T = ids.shape
    x = sd["embed_tokens.weight"].float()[ids] + sd["embed_positions.weight"].float()[:T][None]
    if n_persistent > 0:
        x = torch.cat([sd["persistent_tokens"].float()[None].expand(B, -1, -1), x], dim=1)
    for i in range(n_layers):
        x = block_forward(x, sd, f"layers.{i}.", n_heads, window, n_persistent, eps)
    x = x[:, n_persistent:]
    if positions is not None:
        x = x[:, list(positions)]
    return F.linear(rms_norm(x, sd["norm.scale"].float(), eps), sd["lm_head.weight"].float())
