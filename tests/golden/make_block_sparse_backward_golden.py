"""Generate ``block_sparse_backward_golden.npz``: gradients of the reference's BlockSparseAttention.

    python tests/golden/make_block_sparse_backward_golden.py --reference /path/to/TitanMAC-Standalone

Runs the unmodified reference class in fp32 on CPU on seeded inputs, backpropagates ``sum(y * g)`` for a seeded
``g`` and records the input, every weight, ``g``, the output and the gradients of the input and of every weight.
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
    ("small_np4", 2, 90, 2, 32, 24, 8, 4, 61),
    ("dh64_multi_tile", 1, 300, 2, 64, 128, 64, 16, 62),
    ("no_persistent", 1, 50, 1, 16, 16, 16, 0, 63),
    ("window_not_multiple_of_block", 2, 77, 2, 16, 20, 8, 3, 64),
    ("dh128", 1, 200, 1, 128, 96, 64, 16, 65),
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
        mod = BlockSparseAttention(d_model=D, n_heads=H, window_size=w, block_size=bs, n_persistent=Np)
        with torch.no_grad():
            for pname, p in sorted(mod.named_parameters()):
                std = 0.3 if pname.startswith("conv_") else 1.0 / (D ** 0.5)
                p.copy_(torch.randn(p.shape, generator=g) * std)
        x = torch.randn(B, Np + T, D, generator=g).requires_grad_(True)
        gy = torch.randn(B, Np + T, D, generator=g)
        y = mod(x)
        (y * gy).sum().backward()
        out[f"{name}/meta"] = np.array([B, T, H, dh, w, bs, Np, seed], dtype=np.int64)
        out[f"{name}/x"] = x.detach().numpy()
        out[f"{name}/g"] = gy.numpy()
        out[f"{name}/y"] = np.ascontiguousarray(y.detach().numpy())
        out[f"{name}/dx"] = np.ascontiguousarray(x.grad.numpy())
        for key, val in mod.state_dict().items():
            out[f"{name}/sd/{key}"] = val.numpy()
        for pname, p in mod.named_parameters():
            out[f"{name}/grad/{pname}"] = np.ascontiguousarray(p.grad.numpy())
        print(name, "dx absmax", float(x.grad.abs().max()))
    path = os.path.join(HERE, "block_sparse_backward_golden.npz")
    np.savez_compressed(path, **out)
    print(os.path.basename(path), os.path.getsize(path) // 1024, "KiB")


if __name__ == "__main__":
    main()
