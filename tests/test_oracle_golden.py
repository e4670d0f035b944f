"""The CPU oracles against the golden vectors generated from the reference itself."""

import numpy as np
import pytest
import torch

from conftest import CORE_CASES, FULL_CASES
from oracle import c_oracle
from oracle import windowed_oracle as wo


@pytest.mark.parametrize("case", FULL_CASES + ["config1_fp32"])
def test_mask_row_sums_match_reference(golden, case):
    m = golden.meta(case)
    ref = golden.np(case, "mask_row_sums")
    ours = wo.band_mask(m["L"], m["w"], m["Np"]).sum(1).numpy()
    assert np.array_equal(ours, ref)
    assert int(ref.sum()) == wo.live_pairs(m["L"], m["w"], m["Np"])
    step = max(1, m["L"] // 40)
    for p in list(range(0, m["L"], step)) + [m["L"] - 1]:
        assert c_oracle.row_count(p, m["L"], m["w"], m["Np"]) == ref[p]


def test_mask_known_answer():
    # L=10, w=3, Np=2: persistent rows see 2 keys, sequence rows 2 + min(t+1, 4)
    assert wo.band_mask(10, 3, 2).sum(1).tolist() == [2, 2, 3, 4, 5, 6, 6, 6, 6, 6]
    assert wo.visible(5, 2, 3, 2) and not wo.visible(6, 2, 3, 0) and not wo.visible(1, 2, 3, 2)


@pytest.mark.parametrize("case", FULL_CASES)
def test_module_forward_matches_reference(golden, case):
    m = golden.meta(case)
    y = wo.module_forward(golden[case, "x"], golden[case, "w_qkv"], golden[case, "w_out"], m["H"], m["w"], m["Np"])
    assert (y - golden[case, "y"]).abs().max().item() <= 2e-6
    yb = wo.module_forward(golden[case, "x"], golden[case, "w_qkv"], golden[case, "w_out"], m["H"], m["w"],
                           m["Np"], blockwise=True)
    assert (yb - golden[case, "y"]).abs().max().item() <= 2e-6
    yc = wo.module_forward_reference_cost(golden[case, "x"], golden[case, "w_qkv"], golden[case, "w_out"],
                                          m["H"], m["w"], m["Np"])
    assert (yc - golden[case, "y"]).abs().max().item() <= 2e-6


@pytest.mark.parametrize("case", CORE_CASES)
def test_core_matches_reference(golden, case):
    m = golden.meta(case)
    q, k, v, o = (golden[case, f"core_{n}"] for n in "qkvo")
    dense = wo.attention_core_dense(q, k, v, m["w"], m["Np"])
    assert (dense - o).abs().max().item() <= 2e-6
    block = wo.attention_core_blockwise(q, k, v, m["w"], m["Np"], block=37)
    assert (block - o).abs().max().item() <= 2e-6
    c = torch.from_numpy(c_oracle.attention(q, k, v, m["w"], m["Np"]))
    assert (c - o).abs().max().item() <= 2e-6
    f64 = wo.attention_core_dense(q, k, v, m["w"], m["Np"], compute_dtype=torch.float64)
    assert (f64.float() - o).abs().max().item() <= 2e-6


def test_core_rows_with_offsets_match_dense(golden):
    """A block of query rows against a K/V buffer that starts mid-sequence (the sharded layout)."""
    case = "dh64_multi_tile"
    m = golden.meta(case)
    q, k, v, o = (golden[case, f"core_{n}"] for n in "qkvo")
    Np, w = m["Np"], m["w"]
    r0, r1 = 150, 230
    lo = r0 - w
    kk = torch.cat([k[:, :, :Np], k[:, :, lo:r1]], dim=2)
    vv = torch.cat([v[:, :, :Np], v[:, :, lo:r1]], dim=2)
    c = torch.from_numpy(c_oracle.attention(q[:, :, r0:r1], kk, vv, w, Np, q_pos0=r0, k_pos0=lo))
    assert (c - o[:, :, r0:r1]).abs().max().item() <= 2e-6
    rows = wo.attention_core_rows(q[:, :, r0:r1], k, v, r0, w, Np)
    assert (rows - o[:, :, r0:r1]).abs().max().item() <= 2e-6


def test_config1_rows_match_reference(golden):
    case = "config1_fp32"
    m = golden.meta(case)
    x, w_qkv, w_out = wo.layer_inputs(m["B"], m["T"], m["D"], m["Np"], m["seed"])
    chk = golden.np(case, "input_checksum")
    ours = np.array([x.double().sum().item(), w_qkv.double().sum().item(), w_out.double().sum().item(),
                     x.double().abs().sum().item()])
    assert np.allclose(ours, chk, rtol=0, atol=1e-9), "seeded inputs differ from the ones the fixture was made with"
    rows = golden[case, "rows"]
    y = wo.module_forward(x, w_qkv, w_out, m["H"], m["w"], m["Np"])
    assert (y[:, rows] - golden[case, "y_rows"]).abs().max().item() <= 2e-6


def test_decode_row_is_last_row_of_full_forward(golden):
    case = "dh64_multi_tile"
    m = golden.meta(case)
    q, k, v, o = (golden[case, f"core_{n}"] for n in "qkvo")
    Np, w = m["Np"], m["w"]
    for pos in (Np, Np + 5, Np + w, Np + w + 1, m["L"] - 1):
        lo = max(Np, pos - w)
        out = wo.decode_row(q[:, :, pos], k[0, :, :Np], v[0, :, :Np], k[:, :, lo:pos + 1], v[:, :, lo:pos + 1])
        assert (out - o[:, :, pos]).abs().max().item() <= 2e-6


def test_reference_error_behaviour(golden):
    assert list(golden.np("errors", "np_ge_len")) == ["ValueError", "ValueError"]
    with pytest.raises(ValueError):
        wo.band_mask(16, 4, 16)
    with pytest.raises(ValueError):
        wo.band_mask(16, -1, 2)
    with pytest.raises(ValueError):
        wo.module_forward(torch.zeros(1, 3, 16), torch.zeros(48, 16), torch.zeros(16, 16), 2, 4, 3)


def _sd(golden_model, prefix):
    keys = [k[len(prefix) + 4:] for k in golden_model._z.files if k.startswith(prefix + "/sd/")]
    return {k: golden_model[prefix, "sd/" + k] for k in keys}


def test_model_oracle_block_matches_reference_block(golden_model):
    """oracle/model_oracle.py against the output the reference's TitanBlock produced."""
    from oracle import model_oracle as mo

    d_model, n_heads, d_ff, w, Np = (int(v) for v in golden_model.np("block", "cfg"))
    y = mo.block_forward(golden_model["block", "x"], _sd(golden_model, "block"), "", n_heads, w, Np)
    assert (y - golden_model["block", "y"]).abs().max().item() <= 2e-6


def test_model_oracle_logits_match_reference_model(golden_model):
    """... and against the logits of the reference's TitanMAC, whole and at sampled positions."""
    from oracle import model_oracle as mo

    V, d_model, n_heads, n_layers, d_ff, max_len, w, Np = (int(v) for v in golden_model.np("model", "cfg"))
    sd, ids, want = _sd(golden_model, "model"), golden_model["model", "ids"], golden_model["model", "logits"]
    got = mo.model_forward(sd, ids, n_layers, n_heads, w, Np)
    assert got.shape == want.shape
    assert (got - want).abs().max().item() <= 5e-6
    some = [0, 7, 41, ids.shape[1] - 1]
    assert (mo.model_forward(sd, ids, n_layers, n_heads, w, Np, positions=some) - want[:, some]).abs().max().item() <= 5e-6
