"""Backward of the windowed attention core (tmw_prefill_lse + tmw_prefill_backward) through the module's
autograd function: gradients against those of the reference module (golden fixture) and against autograd
through the CPU oracle."""

import os

import numpy as np
import pytest
import torch

from oracle import windowed_oracle as wo
from titanmac_b200 import TitanBlock, TitanMACConfig, WindowConfig, WindowedAttention, _native

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def bz():
    return np.load(os.path.join(HERE, "golden", "backward_golden.npz"))


def test_module_gradients_match_reference_fp32(bz):
    for name in sorted({k.split("/")[0] for k in bz.files}):
        B, T, H, dh, w, Np, _ = (int(v) for v in bz[f"{name}/meta"])
        t = lambda key: torch.from_numpy(bz[f"{name}/{key}"])  # noqa: E731
        mod = WindowedAttention(WindowConfig(window_size=w, num_heads=H, head_dim=dh, n_persistent=Np))
        with torch.no_grad():
            mod.qkv_proj.weight.copy_(t("w_qkv"))
            mod.out_proj.weight.copy_(t("w_out"))
        mod = mod.to(DEV)
        x = t("x").to(DEV).requires_grad_(True)
        y = mod(x)
        assert (y.detach().cpu() - t("y")).abs().max().item() <= 2e-5, name
        (y * t("g").to(DEV)).sum().backward()
        for got, key in ((x.grad, "dx"), (mod.qkv_proj.weight.grad, "dw_qkv"), (mod.out_proj.weight.grad, "dw_out")):
            want = t(key)
            err = (got.cpu() - want).abs().max().item()
            assert err <= 3e-5 * max(1.0, want.abs().max().item()), (name, key, err)
    _native.poll_status(torch.device(DEV))


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 4e-2)])
@pytest.mark.parametrize("dh,H,B,L,w,Np", [(64, 2, 2, 16 + 500, 128, 16), (128, 1, 1, 8 + 300, 64, 8),
                                           (32, 3, 1, 90, 200, 0), (16, 1, 2, 5 + 70, 0, 5),
                                           (64, 1, 1, 16 + 1500, 300, 16),   # windows over several tiles, ragged tail
                                           (64, 2, 1, 700, 256, 0),          # no persistent keys
                                           (64, 1, 1, 130 + 400, 100, 130),  # persistent keys over two tiles
                                           (128, 2, 1, 16 + 900, 512, 16)])
def test_core_gradients_against_oracle_autograd(dtype, tol, dh, H, B, L, w, Np):
    q, k, v = (t.to(dtype) for t in wo.qkv_inputs(B, H, L, dh, seed=dh + L))
    g = torch.randn(B, H, L, dh, generator=torch.Generator().manual_seed(1)).to(dtype)
    qr, kr, vr = (t.float().clone().requires_grad_(True) for t in (q, k, v))
    o_ref = wo.attention_core_dense(qr, kr, vr, w, Np)
    (o_ref * g.float()).sum().backward()

    qd, kd, vd = (t.to(DEV) for t in (q, k, v))
    lse = torch.empty(B, H, L, dtype=torch.float32, device=DEV)
    # (the tensor-core FORWARD kernel keeps the persistent keys in one tile of at most 128)
    for algo in ([_native.ALGO_SIMT] if dtype == torch.float32 or dh not in (64, 128) or Np > 128
                 else [_native.ALGO_SIMT, _native.ALGO_TCGEN05]):
        o = _native.prefill(qd, kd, vd, w, Np, algo=algo, lse=lse)      # [B, H, L, dh] view of [B, L, H, dh]
        # lse is log2-domain: log2 sum_j exp2(s * scale * log2 e)
        s = torch.matmul(qr.detach(), kr.detach().transpose(-1, -2)) / dh ** 0.5
        s = s.masked_fill(~wo.band_mask(L, w, Np), float("-inf"))
        want_lse = torch.logsumexp(s, dim=-1) * 1.4426950408889634
        assert (lse.cpu() - want_lse).abs().max().item() <= (1e-4 if dtype == torch.float32 else 3e-2), algo
        d_o = torch.empty_like(o)
        d_o.copy_(g.to(DEV))
        # CUDA-core kernels; for 16-bit types and head_dim 64 / 128 also the warp-level tensor-core kernels and the
        # tcgen05 kernels (which is what the library picks by itself there)
        tensor_core = dtype != torch.float32 and dh in (64, 128)
        for bwd_algo in ((_native.ALGO_SIMT, _native.ALGO_MMA, _native.ALGO_TCGEN05, _native.ALGO_AUTO) if tensor_core
                         else (_native.ALGO_SIMT, _native.ALGO_AUTO)):
            dq, dk, dv = torch.empty_like(qd), torch.empty_like(kd), torch.empty_like(vd)
            _native.prefill_backward(qd, kd, vd, o, d_o, lse, dq, dk, dv, w, Np, algo=bwd_algo)
            for got, want, nm in ((dq, qr.grad, "dq"), (dk, kr.grad, "dk"), (dv, vr.grad, "dv")):
                err = (got.float().cpu() - want).abs().max().item()
                assert err <= tol * max(1.0, want.abs().max().item()), (nm, algo, bwd_algo, err)
    _native.poll_status(torch.device(DEV))


def test_tcgen05_backward_captured_in_a_cuda_graph_and_replayed():
    """The tcgen05 backward takes its scratch memory (the rows' lse and D between its two launches) from a
    stream-ordered pool: the call must also work while a stream is being captured, and every replay of the graph
    must give the gradients of an eager call - bit for bit, the launches are deterministic."""
    B, H, L, dh, w, Np = 2, 2, 16 + 700, 64, 200, 16
    q, k, v = (t.to(torch.bfloat16).to(DEV) for t in wo.qkv_inputs(B, H, L, dh, seed=5))
    lse = torch.empty(B, H, L, dtype=torch.float32, device=DEV)
    o = _native.prefill(q, k, v, w, Np, lse=lse)
    d_o = torch.randn(B, L, H, dh, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16).to(DEV).permute(0, 2, 1, 3)
    want = [torch.empty_like(q) for _ in range(3)]
    _native.prefill_backward(q, k, v, o, d_o, lse, *want, w, Np, algo=_native.ALGO_TCGEN05)
    got = [torch.zeros_like(q) for _ in range(3)]
    side = torch.cuda.Stream(device=DEV)
    side.wait_stream(torch.cuda.current_stream(DEV))
    with torch.cuda.stream(side):
        _native.prefill_backward(q, k, v, o, d_o, lse, *got, w, Np, algo=_native.ALGO_TCGEN05)  # warm-up
    torch.cuda.current_stream(DEV).wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        _native.prefill_backward(q, k, v, o, d_o, lse, *got, w, Np, algo=_native.ALGO_TCGEN05)
    for _ in range(3):
        for t in got:
            t.zero_()
        graph.replay()
        torch.cuda.synchronize()
        for a, b, nm in zip(got, want, ("dq", "dk", "dv")):
            assert torch.equal(a, b), nm
    _native.poll_status(torch.device(DEV))


def test_block_trains_end_to_end():
    """One TitanBlock with the windowed class under grad mode: every parameter and the input get a gradient,
    and the forward value equals the inference path's."""
    cfg = TitanMACConfig(d_model=128, n_heads=2, d_ff=256, window_size=32, n_persistent=4, use_block_sparse=False)
    block = TitanBlock(cfg).to(DEV)
    x = torch.randn(2, 4 + 100, 128, device=DEV, requires_grad=True)
    y = block(x)
    y.square().mean().backward()
    assert x.grad is not None and torch.isfinite(x.grad).all()
    for name, prm in block.named_parameters():
        assert prm.grad is not None and torch.isfinite(prm.grad).all(), name
    with torch.no_grad():
        y2 = block(x.detach())
    assert (y.detach() - y2).abs().max().item() <= 1e-4


def test_block_sparse_module_gradients_match_reference_fp32():
    from titanmac_b200 import BlockSparseAttention

    z = np.load(os.path.join(HERE, "golden", "block_sparse_backward_golden.npz"))
    for name in sorted({k.split("/")[0] for k in z.files}):
        B, T, H, dh, w, bs, Np, _ = (int(v) for v in z[f"{name}/meta"])
        t = lambda key: torch.from_numpy(z[f"{name}/{key}"])  # noqa: E731
        mod = BlockSparseAttention(d_model=H * dh, n_heads=H, window_size=w, block_size=bs, n_persistent=Np)
        mod.load_state_dict({k[len(name) + 4:]: torch.from_numpy(z[k]) for k in z.files if k.startswith(f"{name}/sd/")})
        mod = mod.to(DEV)
        x = t("x").to(DEV).requires_grad_(True)
        y = mod(x)
        assert (y.detach().cpu() - t("y")).abs().max().item() <= 2e-5, name
        (y * t("g").to(DEV)).sum().backward()
        err = (x.grad.cpu() - t("dx")).abs().max().item()
        assert err <= 3e-5 * max(1.0, t("dx").abs().max().item()), (name, "dx", err)
        for pname, prm in mod.named_parameters():
            want = t(f"grad/{pname}")
            err = (prm.grad.cpu() - want).abs().max().item()
            assert err <= 3e-5 * max(1.0, want.abs().max().item()), (name, pname, err)
    _native.poll_status(torch.device(DEV))


@pytest.mark.parametrize("dh,H,B,T,w,bs,Np", [(64, 2, 1, 700, 128, 64, 16), (128, 1, 1, 400, 100, 32, 5),
                                               (64, 1, 2, 300, 0, 16, 0),
                                               (64, 1, 1, 1500, 512, 64, 16),    # windows over several tiles, ragged tail
                                               (64, 1, 1, 600, 100, 48, 130),    # persistent rows over two tiles, odd block
                                               (128, 1, 1, 900, 256, 64, 16)])
def test_block_sparse_core_gradients_bf16_both_backward_kernels(dh, H, B, T, w, bs, Np):
    from oracle import block_sparse_oracle as bo

    L = Np + T
    gen = torch.Generator().manual_seed(dh + T)
    q, k, v, g = (torch.randn(B, H, L, dh, generator=gen).to(torch.bfloat16) for _ in range(4))
    qr, kr, vr = (t.float().clone().requires_grad_(True) for t in (q, k, v))
    (bo.attention_core(qr, kr, vr, w, bs, Np) * g.float()).sum().backward()
    qd, kd, vd = (t.to(DEV) for t in (q, k, v))
    lse = torch.empty(B * H * L, dtype=torch.float32, device=DEV)
    o = _native.prefill(qd, kd, vd, w, Np, window_block=bs, lse=lse)
    d_o = torch.empty_like(o)
    d_o.copy_(g.to(DEV))
    # CUDA cores, warp-level tensor cores, tcgen05, and what the library picks by itself (tcgen05)
    for bwd_algo in (_native.ALGO_SIMT, _native.ALGO_MMA, _native.ALGO_TCGEN05, _native.ALGO_AUTO):
        dq, dk, dv = torch.empty_like(qd), torch.empty_like(kd), torch.empty_like(vd)
        _native.prefill_backward(qd, kd, vd, o, d_o, lse, dq, dk, dv, w, Np, algo=bwd_algo, window_block=bs)
        for got, want, nm in ((dq, qr.grad, "dq"), (dk, kr.grad, "dk"), (dv, vr.grad, "dv")):
            err = (got.float().cpu() - want).abs().max().item()
            assert err <= 4e-2 * max(1.0, want.abs().max().item()), (nm, bwd_algo, err)
    _native.poll_status(torch.device(DEV))


@pytest.mark.parametrize("block_sparse", [False, True])
def test_model_trains_end_to_end(block_sparse):
    """The whole model under grad mode, with either attention class: the loss is finite, every parameter gets a
    finite gradient, and the logits equal those of the inference path."""
    from titanmac_b200 import TitanMAC

    torch.manual_seed(0)
    cfg = TitanMACConfig(vocab_size=97, d_model=128, n_heads=2, n_layers=2, d_ff=256, max_seq_len=128, window_size=32,
                         n_persistent=4, use_block_sparse=block_sparse, block_size=16)
    model = TitanMAC(cfg).to(DEV)
    ids = torch.randint(0, 97, (2, 100), device=DEV)
    out = model(ids, labels=ids)
    assert torch.isfinite(out["loss"])
    out["loss"].backward()
    for name, prm in model.named_parameters():
        assert prm.grad is not None and torch.isfinite(prm.grad).all(), name
    with torch.no_grad():
        ref = model(ids)["logits"]
    assert (out["logits"].detach() - ref).abs().max().item() <= 2e-3


@pytest.mark.parametrize("taps", [1, 4, 6])
def test_convolution_backward_against_oracle_autograd(taps):
    from oracle import block_sparse_oracle as bo

    gen = torch.Generator().manual_seed(taps)
    x = torch.randn(2, 150, 3 * 64, generator=gen)
    w = torch.randn(3 * 64, taps, generator=gen) * 0.5
    dy = torch.randn(2, 150, 3 * 64, generator=gen)
    xr, wr = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    (bo.causal_dwconv(xr, wr) * dy).sum().backward()
    dx, dw = _native.causal_dwconv_backward(x.to(DEV), w.to(DEV), dy.to(DEV))
    assert (dx.cpu() - xr.grad).abs().max().item() <= 1e-5
    assert (dw.cpu() - wr.grad).abs().max().item() <= 1e-4 * max(1.0, wr.grad.abs().max().item())
    dx16, dw16 = _native.causal_dwconv_backward(x.to(torch.bfloat16).to(DEV), w.to(torch.bfloat16).to(DEV),
                                                dy.to(torch.bfloat16).to(DEV))
    assert (dx16.float().cpu() - xr.grad).abs().max().item() <= 6e-2
    assert (dw16.float().cpu() - wr.grad).abs().max().item() <= 2e-2 * max(1.0, wr.grad.abs().max().item())
