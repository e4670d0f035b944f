"""Generate ``backward_golden.npz``: gradients of the reference's WindowedAttention, from the reference itself.

    python tests/golden/make_backward_golden.py --reference /path/to/TitanMAC-Standalone

Runs the unmodified reference module in fp32 on CPU on seeded inputs, backpropagates the scalar
``sum(y * g)`` for a seeded ``g`` and records the input, the weights, ``g``, the output and the gradients
with respect to the input and to both weights.  The tests read the file; they never import the reference.
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

# (name, batch, sequence tokens, heads, head_dim, window, n_persistent, seed)
CASES = [
    ("tiny_w3", 2, 8, 2, 8, 3, 2, 51),
    ("ragged_w16", 2, 72, 3, 16, 16, 5, 52),
    ("dh64_multi_tile", 1, 284, 2, 64, 64, 16, 53),
    ("dh128_w100", 1, 200, 1, 128, 100, 16, 54),
    ("no_persistent_w0", 1, 40, 2, 32, 0, 0, 55),
]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project")
    args = ap.parse_args()
    sys.dont_write_bytecode = True
    sys.path.insert(0, args.reference)
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    import titans_core.attn.windowed_attention as ref_attn

    out = {}
    for name, B, T, H, dh, w, Np, seed in CASES:
        D = H * dh
        x, w_qkv, w_out = layer_inputs(B, T, D, Np, seed)
        w_qkv, w_out = w_qkv * 5, w_out * 5  # larger weights: gradients well above rounding noise
        mod = ref_attn.WindowedAttention(ref_attn.WindowConfig(window_size=w, num_heads=H, head_dim=dh, n_persistent=Np))
        with torch.no_grad():
            mod.qkv_proj.weight.copy_(w_qkv)
            mod.out_proj.weight.copy_(w_out)
        x = x.clone().requires_grad_(True)
        g = torch.randn(x.shape, generator=torch.Generator().manual_seed(seed + 1000))
        y = mod(x)
        (y * g).sum().backward()
        out[f"{name}/meta"] = np.array([B, T, H, dh, w, Np, seed], dtype=np.int64)
        for key, val in (("x", x), ("w_qkv", w_qkv), ("w_out", w_out), ("g", g), ("y", y), ("dx", x.grad),
                         ("dw_qkv", mod.qkv_proj.weight.grad), ("dw_out", mod.out_proj.weight.grad)):
            out[f"{name}/{key}"] = np.ascontiguousarray(val.detach().numpy())
        print(name, "dx absmax", float(x.grad.abs().max()), "dw_qkv absmax", float(mod.qkv_proj.weight.grad.abs().max()))
    path = os.path.join(HERE, "backward_golden.npz")
    np.savez_compressed(path, **out)
    print(os.path.basename(path), os.path.getsize(path) // 1024, "KiB")


if __name__ == "__main__":
    main()
