"""Host-side behaviour of the drop-in module that needs no GPU: construction, state_dict
compatibility and the exceptions the reference raises in the same situations."""

import pytest
import torch

from titanmac_b200 import TitanMACConfig, WindowConfig, WindowedAttention, _native


def test_constructor_accepts_both_config_kinds():
    a = WindowedAttention(WindowConfig(window_size=8, num_heads=4, head_dim=16, n_persistent=2))
    assert (a.d_model, a.n_heads, a.d_head, a.window_size, a.num_persistent, a.causal, a.dropout_p) == (
        64, 4, 16, 8, 2, True, 0.0)
    b = WindowedAttention(TitanMACConfig(d_model=640, n_heads=10, window_size=512, n_persistent=16))
    assert (b.d_model, b.n_heads, b.d_head, b.window_size, b.num_persistent) == (640, 10, 64, 512, 16)
    assert isinstance(b.dropout, torch.nn.Identity)


def test_state_dict_keys_and_shapes_match_the_reference_module():
    m = WindowedAttention(TitanMACConfig(d_model=128, n_heads=2))
    sd = m.state_dict()
    assert list(sd) == ["qkv_proj.weight", "out_proj.weight"]
    assert sd["qkv_proj.weight"].shape == (384, 128) and sd["out_proj.weight"].shape == (128, 128)


def test_config_errors():
    with pytest.raises(ValueError):
        TitanMACConfig(d_model=641, n_heads=10).d_head
    with pytest.raises(ValueError):
        TitanMACConfig(d_model=641, n_heads=10).validate()
    with pytest.raises(ValueError):
        TitanMACConfig(n_persistent=5000).validate()
    with pytest.raises(ValueError):
        TitanMACConfig(window_size=-1).validate()
    TitanMACConfig().validate()

    class Odd:  # d_model that is not heads * d_head trips the module's own assertion
        d_model, n_heads, d_head, window_size, n_persistent, causal, attention_dropout = 100, 3, 32, 4, 1, True, 0.0

    with pytest.raises(AssertionError):
        WindowedAttention(Odd())


def test_forward_raises_like_the_reference_before_any_device_work():
    m = WindowedAttention(WindowConfig(window_size=4, num_heads=2, head_dim=8, n_persistent=16)).eval()
    for L in (1, 16):  # n_persistent >= length
        with pytest.raises(ValueError, match="must be < seq_len"):
            m(torch.zeros(1, L, 16))
    neg = WindowedAttention(WindowConfig(window_size=-1, num_heads=2, head_dim=8, n_persistent=1)).eval()
    with pytest.raises(ValueError, match="non-negative"):
        neg(torch.zeros(1, 8, 16))


def test_unsupported_modes_and_missing_device_fail_loudly():
    m = WindowedAttention(WindowConfig(window_size=4, num_heads=2, head_dim=8, n_persistent=1)).eval()
    x = torch.zeros(1, 8, 16)
    with pytest.raises(NotImplementedError):
        m(x, attn_mask=torch.ones(8, 8, dtype=torch.bool))
    with pytest.raises(RuntimeError, match="no CPU path"):
        m(x)
    nc = WindowedAttention(WindowConfig(window_size=4, num_heads=2, head_dim=8, n_persistent=1, causal=False))
    with pytest.raises(NotImplementedError):
        nc(x)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        _native.prefill(torch.zeros(1, 1, 8, 8), torch.zeros(1, 1, 8, 8), torch.zeros(1, 1, 8, 8), 4, 1)
