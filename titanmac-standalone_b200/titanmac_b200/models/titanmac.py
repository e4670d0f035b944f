"""TitanMAC without neural memory: the model-level plumbing around the attention path.

``forward`` mirrors titans_core/models/titanmac.py:554-686 for
``use_neural_memory=False``: token + learned position embeddings, the persistent
tokens prepended to every sequence (:608-619), the block stack (:629-640), final
norm, tied LM head over all rows and the slice that drops the persistent rows
(:652-662), optional shifted cross-entropy (:674-684).  Parameter names match the
reference (``embed_tokens``, ``embed_positions``, ``persistent_tokens``,
``layers.N...``, ``norm``, ``lm_head``), so its checkpoints load.  Under
``torch.no_grad()`` the fused inference kernels run; with grad mode on the same call
is differentiable (the attention cores through their own backward kernels, norms and
GELU through PyTorch), so ``forward(ids, labels=...)["loss"].backward()`` trains.

``prefill`` / ``decode_step`` / ``generate`` are new: the reference has no KV cache,
its generation helper re-runs the whole forward for every new token
(examples/train_math.py:146-161).  Here a prompt is run once, every layer's last
``w+1`` keys/values go into a ring cache, the persistent keys/values (which do not
depend on the prompt) are kept once per layer, and each new token costs one pass of
``tmw_decode`` per layer.  A decode step returns the logits the reference's
re-forward would return for its last row.
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import _native
from ..blocks.titan_block import RMSNorm, TitanBlock


class TitanMAC(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.config = config
        config.validate()
        if getattr(config, "use_neural_memory", False):
            raise NotImplementedError("the neural-memory variants (MAC/MAG/MAL) are not part of this package")
        self.embed_tokens = nn.Embedding(config.vocab_size, config.d_model)
        self.embed_positions = nn.Embedding(config.max_seq_len, config.d_model)
        if config.n_persistent > 0:
            self.persistent_tokens = nn.Parameter(torch.zeros(config.n_persistent, config.d_model))
        else:
            self.register_parameter("persistent_tokens", None)
        self.layers = nn.ModuleList([TitanBlock(config) for _ in range(config.n_layers)])
        self.norm = RMSNorm(config.d_model, eps=config.norm_eps)
        self.lm_head = nn.Linear(config.d_model, config.vocab_size, bias=False)
        if config.tie_weights:
            self.lm_head.weight = self.embed_tokens.weight
        self._init_weights()
        self._graph = None

    def _init_weights(self) -> None:
        # titanmac.py:140-158: only embeddings, persistent tokens and an untied head are re-initialised
        nn.init.normal_(self.embed_tokens.weight, mean=0.0, std=0.02)
        nn.init.normal_(self.embed_positions.weight, mean=0.0, std=0.02)
        if self.persistent_tokens is not None:
            nn.init.normal_(self.persistent_tokens, mean=0.0, std=0.02)
        if not self.config.tie_weights:
            nn.init.normal_(self.lm_head.weight, mean=0.0, std=0.02)

    # ------------------------------------------------------------------ forward --
    def _embed(self, input_ids: torch.Tensor, first_position: int = 0) -> torch.Tensor:
        B, T = input_ids.shape
        positions = torch.arange(first_position, first_position + T, device=input_ids.device)
        x = self.embed_tokens(input_ids) + self.embed_positions(positions)[None]
        if self.persistent_tokens is not None and first_position == 0:
            x = torch.cat([self.persistent_tokens[None].expand(B, -1, -1), x], dim=1)
        return x

    def forward(self, input_ids: torch.Tensor, labels: Optional[torch.Tensor] = None,
                attention_mask: Optional[torch.Tensor] = None) -> Dict[str, torch.Tensor]:
        Np = self.config.n_persistent
        x = self._embed(input_ids)
        # Same wiring as TitanBlock.forward, with every residual add folded into the RMSNorm that follows it
        # (one kernel): the MLP output of a layer is added by the next layer's first norm, or by the final norm.
        pending = None
        for layer in self.layers:
            if pending is None:
                h = layer.norm_attn(x)
            else:
                x, h = layer.norm_attn.add_forward(x, pending, inplace=True)
            a = layer.attention(h, attn_mask=None)
            x, h = layer.norm_mlp.add_forward(x, a, inplace=True)
            pending = layer.mlp(h)
        h = self.norm(x) if pending is None else self.norm.add_forward(x, pending, inplace=True)[1]
        logits = _native.project(self.lm_head, h)
        logits = logits[:, Np:, :] if Np > 0 else logits
        out = {"logits": logits}
        if labels is not None:
            shift_logits = logits[..., :-1, :].contiguous()
            shift_labels = labels[..., 1:].contiguous()
            out["loss"] = F.cross_entropy(shift_logits.reshape(-1, self.config.vocab_size), shift_labels.reshape(-1),
                                          reduction="mean", ignore_index=-100)
        return out

    # --------------------------------------------------------------- generation --
    def _need_windowed(self) -> None:
        if getattr(self.config, "use_block_sparse", False):
            raise NotImplementedError(
                "the ring-cache generation path (prefill / decode_step / generate) is built for WindowedAttention; "
                "build the config with use_block_sparse=False (forward() works with either attention class)")

    def new_caches(self, batch: int, device, dtype) -> List[_native.RingCache]:
        self._need_windowed()
        c = self.config
        return [_native.RingCache(batch, c.n_heads, c.d_head, c.window_size, c.n_persistent, dtype, device)
                for _ in self.layers]

    @torch.no_grad()
    def prefill(self, input_ids: torch.Tensor, caches: Optional[List[_native.RingCache]] = None):
        """Run the prompt ``[B, T]`` once; returns (logits of the last prompt token ``[B, V]``, caches)."""
        self._need_windowed()
        B, T = input_ids.shape
        Np = self.config.n_persistent
        x = self._embed(input_ids)
        if caches is None:
            caches = self.new_caches(B, x.device, x.dtype)
        pending = None
        for layer, cache in zip(self.layers, caches):
            attn = layer.attention
            if pending is None:
                h = layer.norm_attn(x)
            else:
                x, h = layer.norm_attn.add_forward(x, pending, inplace=True)
            L = h.shape[1]
            attn._check_lengths(L)
            attn._check_supported(h, None)
            qkv = _native.project(attn.qkv_proj, h)
            q, k, v = attn.split_qkv(qkv)
            o = torch.empty((B, L, attn.n_heads, attn.d_head), dtype=qkv.dtype, device=qkv.device)
            _native.prefill(q, k, v, attn.window_size, attn.num_persistent, out=o.permute(0, 2, 1, 3), algo=attn.algo)
            # hand the keys/values over: the persistent rows are the same for every sequence
            if Np > 0:
                cache.set_persistent(k[0, :, :Np], v[0, :, :Np])
            cache.fill(k[:, :, Np:], v[:, :, Np:], t0=0)
            x, h = layer.norm_mlp.add_forward(x, _native.project(attn.out_proj, o.view(B, L, -1)), inplace=True)
            pending = layer.mlp(h)
        last = self.norm(x[:, -1]) if pending is None else self.norm.add_forward(x[:, -1], pending[:, -1])[1]
        logits = self.lm_head(last)
        return logits, caches

    @torch.no_grad()
    def decode_step(self, token_ids: torch.Tensor, pos: torch.Tensor, caches: List[_native.RingCache]) -> torch.Tensor:
        """One new token per sequence.  ``token_ids [B]``, ``pos [B] int32`` = its index in the sequence
        (the prompt occupied 0..T-1).  Returns logits ``[B, V]``; ``pos`` is not modified."""
        self._need_windowed()
        c = self.config
        B = token_ids.shape[0]
        x = self.embed_tokens(token_ids) + self.embed_positions(pos.long())
        pending = None
        for layer, cache in zip(self.layers, caches):
            attn = layer.attention
            if pending is None:
                h = layer.norm_attn(x)
            else:
                x, h = layer.norm_attn.add_forward(x, pending, inplace=True)
            qkv = attn.qkv_proj(h).view(B, 3, c.n_heads, c.d_head)
            o = cache.decode(qkv[:, 0], qkv[:, 1], qkv[:, 2], pos)
            x, h = layer.norm_mlp.add_forward(x, attn.out_proj(o.view(B, -1)), inplace=True)
            pending = layer.mlp(h)
        h = self.norm(x) if pending is None else self.norm.add_forward(x, pending, inplace=True)[1]
        return self.lm_head(h)

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, max_new_tokens: int, use_cuda_graph: bool = True) -> torch.Tensor:
        """Greedy continuation of ``input_ids [B, T]``; returns ``[B, T + max_new_tokens]``.

        The decode step is launch-bound (a dozen small kernels per layer), so it is captured once in a
        CUDA graph and replayed; token ids and positions live in static device buffers.
        """
        B, T = input_ids.shape
        if T + max_new_tokens > self.config.max_seq_len:
            raise ValueError("prompt + new tokens exceed max_seq_len (the position-embedding table)")
        logits, caches = self.prefill(input_ids)
        tok = logits.argmax(dim=-1)
        pos = torch.full((B,), T, dtype=torch.int32, device=input_ids.device)
        out = [input_ids, tok[:, None]]
        step = self.decode_step
        graph = None
        if use_cuda_graph and max_new_tokens > 2:
            static_tok, static_pos = tok.clone(), pos.clone()
            side = torch.cuda.Stream(input_ids.device)
            side.wait_stream(torch.cuda.current_stream(input_ids.device))
            with torch.cuda.stream(side):  # one eager step on the capture stream warms up cuBLAS workspaces
                static_logits = step(static_tok, static_pos, caches)
                static_tok.copy_(static_logits.argmax(dim=-1))
                static_pos += 1
            torch.cuda.current_stream(input_ids.device).wait_stream(side)
            out.append(static_tok.clone()[:, None])
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                static_logits = step(static_tok, static_pos, caches)
                static_tok.copy_(static_logits.argmax(dim=-1))
                static_pos += 1
            for _ in range(max_new_tokens - 2):
                graph.replay()
                out.append(static_tok.clone()[:, None])
        else:
            for _ in range(max_new_tokens - 1):
                logits = step(tok, pos, caches)
                tok = logits.argmax(dim=-1)
                pos = pos + 1
                out.append(tok[:, None])
        return torch.cat(out, dim=1)[:, : T + max_new_tokens]
