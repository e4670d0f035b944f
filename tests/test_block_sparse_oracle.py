"""The block-sparse oracle against outputs of the reference's own BlockSparseAttention (golden fixture)."""

import os

import numpy as np
import pytest
import torch

from oracle import block_sparse_oracle as bo

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def bs_golden():
    return np.load(os.path.join(HERE, "golden", "block_sparse_golden.npz"))


def cases(z):
    return sorted({k.split("/")[0] for k in z.files})


def load_case(z, name):
    B, T, H, dh, w, bs, Np, _ = (int(v) for v in z[f"{name}/meta"])
    t = lambda key: torch.from_numpy(z[f"{name}/{key}"])  # noqa: E731
    sd = {k[len(name) + 4:]: torch.from_numpy(z[k]) for k in z.files if k.startswith(f"{name}/sd/")}
    return dict(B=B, T=T, H=H, dh=dh, w=w, bs=bs, Np=Np, x=t("x"), y=t("y"), q=t("conv_q"), k=t("conv_k"),
                v=t("conv_v"), attn=t("attn"), sd=sd)


def test_fixture_has_the_reference_state_dict_keys(bs_golden):
    c = load_case(bs_golden, "small_np4")
    assert sorted(c["sd"]) == ["conv_k.weight", "conv_q.weight", "conv_v.weight", "out_proj.weight", "qkv_proj.weight"]
    assert c["sd"]["conv_q.weight"].shape == (c["H"] * c["dh"], 1, 4)


def test_oracle_matches_reference_outputs(bs_golden):
    for name in cases(bs_golden):
        c = load_case(bs_golden, name)
        sd = c["sd"]
        y, q, k, v, o = bo.module_forward(c["x"], sd["qkv_proj.weight"], sd["conv_q.weight"][:, 0],
                                          sd["conv_k.weight"][:, 0], sd["conv_v.weight"][:, 0],
                                          sd["out_proj.weight"], c["H"], c["w"], c["bs"], c["Np"], return_parts=True)
        assert (q - c["q"]).abs().max().item() <= 2e-6, name   # after the convolutions
        assert (k - c["k"]).abs().max().item() <= 2e-6, name
        assert (v - c["v"]).abs().max().item() <= 2e-6, name
        B, L, D = c["x"].shape
        assert (o.transpose(1, 2).reshape(B, L, D) - c["attn"]).abs().max().item() <= 2e-6, name
        assert (y - c["y"]).abs().max().item() <= 2e-6, name


def test_mask_properties():
    m = bo.mask(3 + 40, window=16, block_size=8, n_persistent=3)
    assert m[:3].all()                                  # persistent rows see everything
    assert m[3:, :3].all()                              # every row sees the persistent keys
    seq = m[3:, 3:]
    assert not torch.triu(seq, diagonal=1).any()        # causal
    counts = seq.sum(dim=1)
    assert counts[0] == 1 and counts.max() == 16 + 8    # between w + 1 and w + block_size keys once filled
    assert (counts[24:] >= 17).all()
    assert bo.first_visible_key(23, 16, 8) == 0 and bo.first_visible_key(24, 16, 8) == 8


def test_cost_faithful_restatement_and_pair_count_agree_with_the_oracle(bs_golden):
    for name in cases(bs_golden):
        c = load_case(bs_golden, name)
        sd = c["sd"]
        args = (c["x"], sd["qkv_proj.weight"], sd["conv_q.weight"][:, 0], sd["conv_k.weight"][:, 0],
                sd["conv_v.weight"][:, 0], sd["out_proj.weight"], c["H"], c["w"], c["bs"], c["Np"])
        assert (bo.module_forward_reference_cost(*args) - c["y"]).abs().max().item() <= 2e-6, name
        L = c["Np"] + c["T"]
        assert bo.live_pairs(L, c["w"], c["bs"], c["Np"]) == int(bo.mask(L, c["w"], c["bs"], c["Np"]).sum()), name
