"""Autograd through the CPU oracle reproduces the gradients of the reference module (golden fixture): this
pins the oracle as the checker of the backward kernels."""

import os

import numpy as np
import pytest
import torch

from oracle import windowed_oracle as wo

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def bz():
    return np.load(os.path.join(HERE, "golden", "backward_golden.npz"))


def test_oracle_autograd_matches_reference_gradients(bz):
    for name in sorted({k.split("/")[0] for k in bz.files}):
        B, T, H, dh, w, Np, _ = (int(v) for v in bz[f"{name}/meta"])
        t = lambda key: torch.from_numpy(bz[f"{name}/{key}"])  # noqa: E731
        x = t("x").clone().requires_grad_(True)
        w_qkv = t("w_qkv").clone().requires_grad_(True)
        w_out = t("w_out").clone().requires_grad_(True)
        y = wo.module_forward(x, w_qkv, w_out, H, w, Np)
        assert (y.detach() - t("y")).abs().max().item() <= 1e-5, name
        (y * t("g")).sum().backward()
        for got, key in ((x.grad, "dx"), (w_qkv.grad, "dw_qkv"), (w_out.grad, "dw_out")):
            want = t(key)
            assert (got - want).abs().max().item() <= 2e-5 * max(1.0, want.abs().max().item()), (name, key)


def test_block_sparse_oracle_autograd_matches_reference_gradients():
    """The same pin for the block-sparse class: autograd through its oracle gives the reference's gradients."""
    from oracle import block_sparse_oracle as bo

    z = np.load(os.path.join(HERE, "golden", "block_sparse_backward_golden.npz"))
    for name in sorted({k.split("/")[0] for k in z.files}):
        B, T, H, dh, w, bs, Np, _ = (int(v) for v in z[f"{name}/meta"])
        t = lambda key: torch.from_numpy(z[f"{name}/{key}"])  # noqa: E731
        x = t("x").clone().requires_grad_(True)
        prm = {k: t(f"sd/{k}").clone().requires_grad_(True)
               for k in ("qkv_proj.weight", "conv_q.weight", "conv_k.weight", "conv_v.weight", "out_proj.weight")}
        y = bo.module_forward(x, prm["qkv_proj.weight"], prm["conv_q.weight"][:, 0], prm["conv_k.weight"][:, 0],
                              prm["conv_v.weight"][:, 0], prm["out_proj.weight"], H, w, bs, Np)
        assert (y.detach() - t("y")).abs().max().item() <= 1e-5, name
        (y * t("g")).sum().backward()
        assert (x.grad - t("dx")).abs().max().item() <= 2e-5 * max(1.0, t("dx").abs().max().item()), name
        for k, p in prm.items():
            want = t(f"grad/{k}")
            assert (p.grad - want).abs().max().item() <= 2e-5 * max(1.0, want.abs().max().item()), (name, k)
