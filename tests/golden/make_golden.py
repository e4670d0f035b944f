"""Generate the golden fixtures in this directory from the reference itself.

Run once, where the reference checkout is available:

    python tests/golden/make_golden.py --reference /path/to/TitanMAC-Standalone

It imports the *unmodified* reference modules on CPU, runs them in fp32 on seeded
inputs and writes ``windowed_attention_golden.npz`` (layer cases) and
``titanmac_golden.npz`` (block / model cases).  The tests never import the
reference; they read these files.

What is recorded per layer case: the inputs (small cases) or a checksum of the
seeded inputs (the large fp32 config), the module output, and the tensors that
went into and came out of the reference's scaled-dot-product-attention call
(captured by wrapping that one function while the reference forward runs), plus
the row sums of the reference's boolean mask.
"""

from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle.windowed_oracle import layer_inputs  # noqa: E402  (seeded input recipe only)

# (name, batch, seq_tokens, heads, head_dim, window, n_persistent, seed, store_full)
LAYER_CASES = [
    ("tiny_w3", 2, 8, 2, 8, 3, 2, 11, True),
    ("ragged_w16", 2, 72, 3, 16, 16, 5, 12, True),
    ("self_only_w0", 1, 199, 2, 32, 0, 1, 13, True),
    ("window_exceeds_len", 2, 150, 2, 16, 300, 0, 14, True),
    ("one_persistent_row_short", 1, 1, 2, 16, 4, 3, 15, True),
    ("dh64_multi_tile", 1, 284, 2, 64, 64, 16, 16, True),
    ("dh128_multi_tile", 1, 244, 1, 128, 100, 16, 17, True),
    ("dh64_np8_w129", 2, 400, 1, 64, 129, 8, 18, True),
    # benchmark configuration 1: batch 2, T=512, d_model 512, 8 heads x 64, w=256, Np=16, seed 0
    ("config1_fp32", 2, 512, 8, 64, 256, 16, 0, False),
]

# cases that also keep the exact q, k, v the reference fed to its attention call
CORE_INPUT_CASES = ("tiny_w3", "ragged_w16", "dh64_multi_tile")

# rows kept for the large case: the persistent block, the first sequence rows, rows
# around the point where the window first fills, a stride through the middle, the end
def kept_rows(length: int, n_persistent: int, window: int) -> np.ndarray:
    rows = set(range(0, min(length, n_persistent + 24)))
    edge = n_persistent + window
    rows.update(r for r in range(edge - 4, edge + 5) if 0 <= r < length)
    rows.update(range(0, length, 7))
    rows.update(range(max(0, length - 8), length))
    return np.array(sorted(rows), dtype=np.int64)


def run_layer_cases(ref_attn, out: dict) -> None:
    import torch.nn.functional as F

    for name, B, T, H, dh, w, Np, seed, full in LAYER_CASES:
        D = H * dh
        x, w_qkv, w_out = layer_inputs(B, T, D, Np, seed)
        cfg = ref_attn.WindowConfig(window_size=w, num_heads=H, head_dim=dh, n_persistent=Np)
        mod = ref_attn.WindowedAttention(cfg).eval()
        with torch.no_grad():
            mod.qkv_proj.weight.copy_(w_qkv)
            mod.out_proj.weight.copy_(w_out)

        captured = {}
        real_sdpa = F.scaled_dot_product_attention

        def spy(q, k, v, attn_mask=None, dropout_p=0.0, is_causal=False, **kw):
            o = real_sdpa(q, k, v, attn_mask=attn_mask, dropout_p=dropout_p, is_causal=is_causal, **kw)
            captured.update(q=q.detach().clone(), k=k.detach().clone(), v=v.detach().clone(),
                            o=o.detach().clone(), mask=attn_mask.detach().clone())
            return o

        ref_attn.F.scaled_dot_product_attention = spy
        try:
            with torch.no_grad():
                y = mod(x)
        finally:
            ref_attn.F.scaled_dot_product_attention = real_sdpa

        L = Np + T
        bool_mask = torch.isfinite(captured["mask"])
        meta = np.array([B, T, H, dh, w, Np, seed], dtype=np.int64)
        out[f"{name}/meta"] = meta
        out[f"{name}/mask_row_sums"] = bool_mask.sum(1).numpy().astype(np.int64)
        checksum = np.array(
            [x.double().sum().item(), w_qkv.double().sum().item(), w_out.double().sum().item(),
             x.double().abs().sum().item()], dtype=np.float64)
        out[f"{name}/input_checksum"] = checksum
        if full:
            out[f"{name}/x"] = x.numpy()
            out[f"{name}/w_qkv"] = w_qkv.numpy()
            out[f"{name}/w_out"] = w_out.numpy()
            out[f"{name}/y"] = y.numpy()
            if name in CORE_INPUT_CASES:
                out[f"{name}/core_q"] = captured["q"].contiguous().numpy()
                out[f"{name}/core_k"] = captured["k"].contiguous().numpy()
                out[f"{name}/core_v"] = captured["v"].contiguous().numpy()
            out[f"{name}/core_o"] = captured["o"].contiguous().numpy()
        else:
            rows = kept_rows(L, Np, w)
            out[f"{name}/rows"] = rows
            out[f"{name}/y_rows"] = y[:, rows].numpy()
            out[f"{name}/core_o_rows"] = captured["o"][:, :, rows].contiguous().numpy()
        print(f"{name}: L={L} y_absmax={y.abs().max().item():.4f}")

    # error behaviour of the reference (windowed_attention.py:97-100, :229-230)
    cfg = ref_attn.WindowConfig(window_size=4, num_heads=2, head_dim=8, n_persistent=16)
    mod = ref_attn.WindowedAttention(cfg).eval()
    errs = []
    for L in (1, 16):
        try:
            mod(torch.zeros(1, L, 16))
            errs.append("none")
        except Exception as e:  # noqa: BLE001
            errs.append(type(e).__name__)
    out["errors/np_ge_len"] = np.array(errs)


def run_model_cases(out: dict) -> None:
    from titans_core.config import TitanMACConfig
    from titans_core.blocks.titan_block import TitanBlock
    from titans_core.models.titanmac import TitanMAC

    def reinit(module: torch.nn.Module, seed: int) -> None:
        g = torch.Generator(device="cpu").manual_seed(seed)
        with torch.no_grad():
            for pname, p in sorted(module.named_parameters()):
                if pname.endswith("scale"):
                    p.fill_(1.0)
                elif pname.endswith("bias"):
                    p.copy_(torch.randn(p.shape, generator=g) * 0.01)
                else:
                    p.copy_(torch.randn(p.shape, generator=g) * 0.02)

    # --- one TitanBlock, attention half and full block ---------------------------
    cfg = TitanMACConfig(vocab_size=97, d_model=128, n_heads=2, n_layers=1, d_ff=128, max_seq_len=256,
                         window_size=24, n_persistent=4, use_block_sparse=False)
    block = TitanBlock(cfg).eval()
    reinit(block, 21)
    g = torch.Generator(device="cpu").manual_seed(22)
    x = torch.randn(2, 4 + 90, 128, generator=g)
    with torch.no_grad():
        y = block(x)
    out["block/cfg"] = np.array([cfg.d_model, cfg.n_heads, cfg.d_ff, cfg.window_size, cfg.n_persistent], dtype=np.int64)
    out["block/x"] = x.numpy()
    out["block/y"] = y.numpy()
    for k, v in block.state_dict().items():
        out[f"block/sd/{k}"] = v.numpy()

    # --- small TitanMAC, logits over a teacher-forced sequence ------------------
    cfg = TitanMACConfig(vocab_size=101, d_model=128, n_heads=2, n_layers=2, d_ff=128, max_seq_len=128,
                         window_size=20, n_persistent=6, use_block_sparse=False)
    model = TitanMAC(cfg).eval()
    reinit(model, 31)
    g = torch.Generator(device="cpu").manual_seed(32)
    ids = torch.randint(0, cfg.vocab_size, (3, 70), generator=g)
    with torch.no_grad():
        logits = model(ids)["logits"]
    out["model/cfg"] = np.array([cfg.vocab_size, cfg.d_model, cfg.n_heads, cfg.n_layers, cfg.d_ff,
                                 cfg.max_seq_len, cfg.window_size, cfg.n_persistent], dtype=np.int64)
    out["model/ids"] = ids.numpy()
    out["model/logits"] = logits.numpy()
    for k, v in model.state_dict().items():
        out[f"model/sd/{k}"] = v.numpy()
    print("model logits absmax", logits.abs().max().item())


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project")
    args = ap.parse_args()
    sys.dont_write_bytecode = True
    sys.path.insert(0, args.reference)
    torch.manual_seed(0)
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    import titans_core.attn.windowed_attention as ref_attn

    layer = {}
    run_layer_cases(ref_attn, layer)
    np.savez_compressed(os.path.join(HERE, "windowed_attention_golden.npz"), **layer)
    model = {}
    run_model_cases(model)
    np.savez_compressed(os.path.join(HERE, "titanmac_golden.npz"), **model)
    for f in ("windowed_attention_golden.npz", "titanmac_golden.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)) // 1024, "KiB")


if __name__ == "__main__":
    main()
