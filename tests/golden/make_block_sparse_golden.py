"""Generate ``block_sparse_golden.npz`` from the reference's BlockSparseAttention itself.

    python tests/golden/make_block_sparse_golden.py --reference /path/to/TitanMAC-Standalone

Imports the unmodified reference class on CPU, runs it in fp32 on seeded inputs and records, per case,
the input, every weight (by state_dict key), the module output, the Q / K / V tensors after its
convolutions (forward hooks on the three Conv1d modules) and the attention output that enters its output
projection (forward pre-hook).  The tests read the file; they never import the reference.
"""

from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

# (name, batch, sequence tokens, heads, head_dim, window, block_size, n_persistent, seed)
CASES = [
    ("small_np4", 2, 90, 2, 32, 24, 8, 4, 41),
    ("dh64_multi_tile", 1, 300, 2, 64, 128, 64, 16, 42),
    ("no_persistent", 1, 50, 1, 16, 16, 16, 0, 43),
    ("window_not_multiple_of_block", 2, 77, 2, 16, 20, 8, 3, 44),
    ("dh128_default_block", 1, 260, 1, 128, 96, 64, 16, 45),
]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project")
    args = ap.parse_args()
    sys.dont_write_bytecode = True
    sys.path.insert(0, args.reference)
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    from titans_core.attn.block_sparse_attention import BlockSparseAttention

    out = {}
    for name, B, T, H, dh, w, bs, Np, seed in CASES:
        D = H * dh
        g = torch.Generator(device="cpu").manual_seed(seed)
        mod = BlockSparseAttention(d_model=D, n_heads=H, window_size=w, block_size=bs, n_persistent=Np).eval()
        with torch.no_grad():
            for pname, p in sorted(mod.named_parameters()):
                std = 0.3 if pname.startswith("conv_") else 1.0 / (D ** 0.5)
                p.copy_(torch.randn(p.shape, generator=g) * std)
        x = torch.randn(B, Np + T, D, generator=g)
        parts = {}
        hooks = [getattr(mod, n).register_forward_hook(
            lambda m, i, o, n=n: parts.__setitem__(n, o[:, :, :Np + T].transpose(1, 2).detach().clone()))
            for n in ("conv_q", "conv_k", "conv_v")]
        hooks.append(mod.out_proj.register_forward_pre_hook(lambda m, i: parts.__setitem__("attn", i[0].detach().clone())))
        with torch.no_grad():
            y = mod(x)
        for h in hooks:
            h.remove()
        out[f"{name}/meta"] = np.array([B, T, H, dh, w, bs, Np, seed], dtype=np.int64)
        out[f"{name}/x"] = x.numpy()
        out[f"{name}/y"] = y.numpy()
        for key, val in mod.state_dict().items():
            out[f"{name}/sd/{key}"] = val.numpy()
        for key in ("conv_q", "conv_k", "conv_v", "attn"):
            out[f"{name}/{key}"] = parts[key].numpy()
        print(name, "output absmax", float(y.abs().max()))
    path = os.path.join(HERE, "block_sparse_golden.npz")
    np.savez_compressed(path, **out)
    print(os.path.basename(path), os.path.getsize(path) // 1024, "KiB")


if __name__ == "__main__":
    main()
