"""The block-sparse drop-in (convolution kernel, block-granular window, global persistent rows) against
outputs of the reference's own BlockSparseAttention (golden fixture) and against the oracle."""

import os

import numpy as np
import pytest
import torch

from oracle import block_sparse_oracle as bo
from titanmac_b200 import BlockSparseAttention, TitanMACConfig, _native, create_block_sparse_attention

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def z():
    return np.load(os.path.join(HERE, "golden", "block_sparse_golden.npz"))


def names(z):
    return sorted({k.split("/")[0] for k in z.files})


def build(z, name, dtype):
    B, T, H, dh, w, bs, Np, _ = (int(v) for v in z[f"{name}/meta"])
    mod = BlockSparseAttention(d_model=H * dh, n_heads=H, window_size=w, block_size=bs, n_persistent=Np).eval()
    sd = {k[len(name) + 4:]: torch.from_numpy(z[k]) for k in z.files if k.startswith(f"{name}/sd/")}
    assert sorted(sd) == sorted(mod.state_dict())   # same keys and shapes as the reference's checkpoint
    mod.load_state_dict(sd)
    return mod.to(device=DEV, dtype=dtype), (B, T, H, dh, w, bs, Np)


def test_convolution_kernel_matches_reference_conv_outputs(z):
    for name in names(z):
        mod, (B, T, H, dh, w, bs, Np) = build(z, name, torch.float32)
        x = torch.from_numpy(z[f"{name}/x"]).to(DEV)
        y = _native.causal_dwconv(mod.qkv_proj(x), mod.stacked_conv_weight())
        D = H * dh
        for i, key in enumerate(("conv_q", "conv_k", "conv_v")):
            want = torch.from_numpy(z[f"{name}/{key}"])
            assert (y[:, :, i * D:(i + 1) * D].cpu() - want).abs().max().item() <= 2e-5, (name, key)


@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_convolution_kernel_other_widths_and_dtypes(taps):
    g = torch.Generator().manual_seed(taps)
    x = torch.randn(2, 150, 3 * 64, generator=g)
    w = torch.randn(3 * 64, taps, generator=g) * 0.5
    want = bo.causal_dwconv(x, w)
    assert (_native.causal_dwconv(x.to(DEV), w.to(DEV)).cpu() - want).abs().max().item() <= 1e-5
    got = _native.causal_dwconv(x.to(torch.bfloat16).to(DEV), w.to(torch.bfloat16).to(DEV)).float().cpu()
    want16 = bo.causal_dwconv(x.to(torch.bfloat16).float(), w.to(torch.bfloat16).float())
    assert (got - want16).abs().max().item() <= 3e-2


def test_module_fp32_matches_reference_output(z):
    for name in names(z):
        mod, _ = build(z, name, torch.float32)
        y = mod(torch.from_numpy(z[f"{name}/x"]).to(DEV)).cpu()
        assert (y - torch.from_numpy(z[f"{name}/y"])).abs().max().item() <= 2e-5, name


@pytest.mark.parametrize("algo", [_native.ALGO_SIMT, _native.ALGO_TCGEN05])
def test_core_16bit_both_kernels(z, algo):
    for name in ("dh64_multi_tile", "dh128_default_block"):
        B, T, H, dh, w, bs, Np, _ = (int(v) for v in z[f"{name}/meta"])
        q, k, v = (torch.from_numpy(z[f"{name}/{key}"]).contiguous().view(B, Np + T, H, dh).transpose(1, 2).to(torch.bfloat16)
                   for key in ("conv_q", "conv_k", "conv_v"))
        want = bo.attention_core(q.float(), k.float(), v.float(), w, bs, Np)
        got = _native.prefill(q.to(DEV), k.to(DEV), v.to(DEV), w, Np, algo=algo, window_block=bs).float().cpu()
        assert (got - want).abs().max().item() <= 2e-2, name
    _native.poll_status(torch.device(DEV))


@pytest.mark.parametrize("dh,H,B,T,w,bs,Np", [
    (64, 2, 2, 1500, 512, 64, 16),    # the default model's layer geometry (block = max(64, 512 // 8))
    (64, 1, 1, 700, 100, 32, 5),      # window not a multiple of the block, ragged length
    (128, 2, 1, 900, 256, 128, 0),    # no persistent rows
    (64, 1, 1, 300, 0, 16, 3),        # window 0: the row's own block only
    (64, 2, 1, 1000, 2048, 256, 16),  # window longer than the sequence, block larger than a key tile
])
def test_core_bf16_against_oracle_larger_shapes(dh, H, B, T, w, bs, Np):
    g = torch.Generator().manual_seed(dh + T)
    q, k, v = (torch.randn(B, H, Np + T, dh, generator=g).to(torch.bfloat16) for _ in range(3))
    want = bo.attention_core(q.float(), k.float(), v.float(), w, bs, Np)
    for algo in (_native.ALGO_TCGEN05, _native.ALGO_SIMT):
        got = _native.prefill(q.to(DEV), k.to(DEV), v.to(DEV), w, Np, algo=algo, window_block=bs).float().cpu()
        assert (got - want).abs().max().item() <= 2e-2, algo
    _native.poll_status(torch.device(DEV))


def test_factory_and_errors():
    mod = create_block_sparse_attention(TitanMACConfig(d_model=128, n_heads=2, window_size=1024, n_persistent=4))
    assert (mod.block_size, mod.window_size, mod.n_persistent) == (64, 1024, 4)   # config.block_size wins
    with pytest.raises(ValueError):
        BlockSparseAttention(d_model=130, n_heads=4)
    q = torch.zeros(1, 1, 40, 64, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(_native.TmwError):   # whole sequences only
        _native.prefill(q[:, :, 8:], q, q, 8, 0, q_pos0=8, window_block=8)
