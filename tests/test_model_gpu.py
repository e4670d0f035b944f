"""Block and model plumbing around the attention path, and generation with the ring cache, against
outputs of the reference's TitanBlock / TitanMAC recorded in the golden fixture."""

import pytest
import torch

from titanmac_b200 import TitanBlock, TitanMAC, TitanMACConfig

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def load_sd(golden_model, prefix):
    keys = [k[len(prefix) + 4:] for k in golden_model._z.files if k.startswith(prefix + "/sd/")]
    return {k: golden_model[prefix, "sd/" + k] for k in keys}


def block_cfg(g):
    d_model, n_heads, d_ff, w, Np = (int(v) for v in g.np("block", "cfg"))
    return TitanMACConfig(vocab_size=97, d_model=d_model, n_heads=n_heads, n_layers=1, d_ff=d_ff, max_seq_len=256,
                          window_size=w, n_persistent=Np, use_block_sparse=False)


def model_cfg(g):
    V, d_model, n_heads, n_layers, d_ff, max_len, w, Np = (int(v) for v in g.np("model", "cfg"))
    return TitanMACConfig(vocab_size=V, d_model=d_model, n_heads=n_heads, n_layers=n_layers, d_ff=d_ff,
                          max_seq_len=max_len, window_size=w, n_persistent=Np, use_block_sparse=False)


def test_block_matches_reference(golden_model):
    block = TitanBlock(block_cfg(golden_model)).eval()
    sd = load_sd(golden_model, "block")
    assert sorted(sd) == sorted(block.state_dict())
    block.load_state_dict(sd)
    y = block.to(DEV)(golden_model["block", "x"].to(DEV)).cpu()
    assert (y - golden_model["block", "y"]).abs().max().item() <= 2e-5


def test_config_selects_the_attention_class_like_the_reference():
    from titanmac_b200 import BlockSparseAttention, WindowedAttention

    assert isinstance(TitanBlock(TitanMACConfig(d_model=128, n_heads=2, d_ff=128)).attention, BlockSparseAttention)
    assert isinstance(TitanBlock(TitanMACConfig(d_model=128, n_heads=2, d_ff=128, use_block_sparse=False)).attention,
                      WindowedAttention)
    model = TitanMAC(TitanMACConfig(vocab_size=50, d_model=128, n_heads=2, n_layers=1, d_ff=128, max_seq_len=64))
    with pytest.raises(NotImplementedError):  # the ring-cache path belongs to the windowed class
        model.new_caches(1, DEV, torch.bfloat16)


def test_model_forward_matches_reference_logits(golden_model):
    model = TitanMAC(model_cfg(golden_model)).eval()
    sd = load_sd(golden_model, "model")
    assert sorted(sd) == sorted(model.state_dict())
    model.load_state_dict(sd)
    model = model.to(DEV)
    ids = golden_model["model", "ids"].to(DEV)
    out = model(ids, labels=ids)
    want = golden_model["model", "logits"]
    assert out["logits"].shape == want.shape
    assert (out["logits"].cpu() - want).abs().max().item() <= 5e-5
    assert torch.isfinite(out["loss"])


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 6e-2)])
def test_prefill_then_decode_equals_full_forward(golden_model, dtype, tol):
    """Teacher-forced: after a prompt of 40 tokens, every decode step's logits equal the reference's logits
    for that position of the full sequence (causality)."""
    model = TitanMAC(model_cfg(golden_model)).eval()
    model.load_state_dict(load_sd(golden_model, "model"))
    model = model.to(device=DEV, dtype=dtype)
    ids = golden_model["model", "ids"].to(DEV)
    want = golden_model["model", "logits"]
    T0 = 40
    logits, caches = model.prefill(ids[:, :T0])
    assert (logits.float().cpu() - want[:, T0 - 1]).abs().max().item() <= tol
    for t in range(T0, ids.shape[1]):
        pos = torch.full((ids.shape[0],), t, dtype=torch.int32, device=DEV)
        logits = model.decode_step(ids[:, t], pos, caches)
        assert (logits.float().cpu() - want[:, t]).abs().max().item() <= tol, t


def test_generate_with_and_without_cuda_graph_agree(golden_model):
    model = TitanMAC(model_cfg(golden_model)).eval()
    model.load_state_dict(load_sd(golden_model, "model"))
    model = model.to(DEV)
    ids = golden_model["model", "ids"].to(DEV)[:, :30]
    a = model.generate(ids, 20, use_cuda_graph=False)
    b = model.generate(ids, 20, use_cuda_graph=True)
    assert a.shape == (ids.shape[0], 50) and torch.equal(a[:, :30], ids)
    assert torch.equal(a, b)
    with pytest.raises(ValueError):
        model.generate(ids, 1000)
