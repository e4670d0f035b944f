"""Parity at the full sizes of benchmark configurations 3, 4 and 5, where the dense reference cannot run: sampled
row blocks (first, last, around every boundary of a 2/4/8-way sequence split) against the CPU oracle, the
sharded layout against the unsharded result, and size-independent properties of a softmax average."""

import pytest
import torch

from oracle import windowed_oracle as wo
from titanmac_b200 import _native

DEV = "cuda:0"
TOL = 2e-2


def device_inputs(B, H, L, dh, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    qkv = torch.randn(B, L, 3, H, dh, generator=g, device=DEV, dtype=torch.float32).to(torch.bfloat16)
    return tuple(qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))


def check_rows(o, q, k, v, w, Np, r0, rows):
    """Rows [r0, r0+rows) of the device result against the oracle fed only the keys those rows can see."""
    L = q.shape[2]
    r1 = min(L, r0 + rows)
    lo = max(Np, r0 - w)
    kk = torch.cat([k[:, :, :Np], k[:, :, lo:r1]], dim=2).float().cpu()
    vv = torch.cat([v[:, :, :Np], v[:, :, lo:r1]], dim=2).float().cpu()
    qq = q[:, :, r0:r1].float().cpu()
    # same formula on the slice: position of the first non-persistent key row of the slice is `lo`
    s = torch.matmul(qq, kk.transpose(-1, -2)) / (q.shape[-1] ** 0.5)
    i = torch.arange(r0, r1)[:, None]
    j = torch.cat([torch.arange(0, Np), torch.arange(lo, r1)])[None, :]
    pers_col = torch.cat([torch.ones(Np, dtype=torch.bool), torch.zeros(r1 - lo, dtype=torch.bool)])[None, :]
    mask = torch.where(i < Np, pers_col.expand(len(i), -1), pers_col | ((j <= i) & (i - j <= w) & (j >= Np)))
    s = s.masked_fill(~mask, float("-inf"))
    ref = torch.matmul(torch.softmax(s, dim=-1), vv)
    err = (o[:, :, r0:r1].float().cpu() - ref).abs().max().item()
    assert err <= TOL, (r0, err)


def test_slice_formula_equals_the_pinned_oracle():
    """The sliced formula used above is the oracle's (which is pinned to the reference) on a small case.
    Runs without a GPU."""
    q, k, v = wo.qkv_inputs(1, 2, 7 + 90, 16, seed=4)
    full = wo.attention_core_dense(q, k, v, 13, 7)
    for r0 in (0, 5, 7, 30, 80):
        check_rows(full, q, k, v, 13, 7, r0, 16)


@pytest.mark.gpu
def test_config5_full_length_sampled_blocks_and_shard_boundaries():
    H, dh, w, Np, T = 16, 128, 1024, 16, 131072
    L = Np + T
    q, k, v = device_inputs(1, H, L, dh, seed=5)
    o = _native.prefill(q, k, v, w, Np, algo=_native.ALGO_TCGEN05)
    _native.poll_status(torch.device(DEV))
    starts = {0, Np, L - 128}
    for n in (2, 4, 8):
        for r in range(1, n):
            b = Np + r * T // n
            starts.update({b - 128, b})
    for r0 in sorted(starts):
        check_rows(o, q, k, v, w, Np, r0, 128)
    assert torch.isfinite(o.float()).all()
    assert o.float().abs().max() <= v.float().abs().max() + 1e-2  # a softmax average stays inside its values
    # the same rows through the sequence-sharded layout (persistent | halo | own) of rank 3 of 4
    r0, r1 = Np + 3 * T // 4, L
    lo = r0 - w
    kk = torch.cat([k[:, :, :Np], k[:, :, lo:r1]], dim=2).contiguous()
    vv = torch.cat([v[:, :, :Np], v[:, :, lo:r1]], dim=2).contiguous()
    part = _native.prefill(q[:, :, r0:r1], kk, vv, w, Np, q_pos0=r0, k_pos0=lo, algo=_native.ALGO_TCGEN05)
    assert (part.float() - o[:, :, r0:r1].float()).abs().max().item() <= 1e-2


@pytest.mark.gpu
def test_config3_shape_sampled_blocks():
    B, H, dh, w, Np, T = 2, 10, 64, 512, 16, 8192
    L = Np + T
    q, k, v = device_inputs(B, H, L, dh, seed=3)
    o = _native.prefill(q, k, v, w, Np, algo=_native.ALGO_TCGEN05)
    for r0 in (0, Np, 500, 4096, L - 100):
        check_rows(o, q, k, v, w, Np, r0, 100)
    o2 = _native.prefill(q, k, v, w, Np, algo=_native.ALGO_SIMT)
    assert (o.float() - o2.float()).abs().max().item() <= TOL


@pytest.mark.gpu
def test_config4_full_batch_decode_step_sampled_sequences():
    """One decode step at B=256, 10 heads x 64, w=512, Np=16 on full rings; a sample of sequences against the
    oracle, and the ring afterwards holds the new token in its slot and nothing else changed."""
    B, H, dh, w, Np = 256, 10, 64, 512, 16
    g = torch.Generator(device=DEV).manual_seed(4)
    cache = _native.RingCache(B, H, dh, w, Np, torch.bfloat16, DEV)
    for t_ in (cache.k_ring, cache.v_ring, cache.k_pers, cache.v_pers):
        t_.copy_(torch.randn(t_.shape, generator=g, device=DEV))
    qkv = torch.randn(B, 3, H, dh, generator=g, device=DEV).to(torch.bfloat16)
    t = 2048 + 77
    pos = torch.full((B,), t, dtype=torch.int32, device=DEV)
    k_before, v_before = cache.k_ring.clone(), cache.v_ring.clone()
    out = cache.decode(qkv[:, 0], qkv[:, 1], qkv[:, 2], pos)
    _native.poll_status(torch.device(DEV))
    slot = t % (w + 1)
    sample = [0, 1, 100, 255]
    k_win = k_before[sample].clone()
    v_win = v_before[sample].clone()
    k_win[:, :, slot] = qkv[sample, 1]
    v_win[:, :, slot] = qkv[sample, 2]
    ref = wo.decode_row(qkv[sample, 0].float().cpu(), cache.k_pers.float().cpu(), cache.v_pers.float().cpu(),
                        k_win.float().cpu(), v_win.float().cpu())
    assert (out[sample].float().cpu() - ref).abs().max().item() <= TOL
    k_before[:, :, slot] = qkv[:, 1]
    v_before[:, :, slot] = qkv[:, 2]
    assert torch.equal(cache.k_ring, k_before) and torch.equal(cache.v_ring, v_before)


@pytest.mark.gpu
@pytest.mark.parametrize("block", [0, 64])
def test_config2_full_size_backward_invariants(block):
    """Backward at the full size of benchmark configuration 2 (dense autograd over 4112 x 4112 pairs is the
    thing being replaced), through identities that hold for any mask because every row of P sums to one:
      sum_j dV_j = sum_i dO_i                       (dV = P^T dO)
      sum_i Q_i . dQ_i = sum_j K_j . dK_j           (both are scale * sum_ij dS_ij Q_i . K_j)
      backward(2 dO) = 2 backward(dO)               (linear in dO)
    per (sequence, head), for the windowed mask and the block-sparse one."""
    B, H, dh, w, Np, T = 8, 10, 64, 512, 16, 4096
    L = Np + T
    q, k, v = device_inputs(B, H, L, dh, seed=21)
    like = lambda t: torch.empty_strided(t.shape, t.stride(), dtype=t.dtype, device=DEV)  # noqa: E731
    lse = torch.empty((B, H, L), dtype=torch.float32, device=DEV)
    o = _native.prefill(q, k, v, w, Np, window_block=block, lse=lse)
    d_o = like(o).copy_(device_inputs(B, H, L, dh, seed=22)[0])
    grads = []
    for mul in (1.0, 2.0):
        dq, dk, dv = like(q), like(k), like(v)
        _native.prefill_backward(q, k, v, o, like(o).copy_(d_o.float() * mul), lse, dq, dk, dv, w, Np, window_block=block)
        grads.append((dq.float(), dk.float(), dv.float()))
    _native.poll_status(torch.device(DEV))
    dq, dk, dv = grads[0]
    # column sums over 4112 bf16-rounded rows: compare relative to the size of the terms summed
    lhs, rhs = dv.sum(dim=2), d_o.float().sum(dim=2)
    assert ((lhs - rhs).abs().max() / d_o.float().abs().sum(dim=2).max()).item() < 3e-4
    a = (q.float() * dq).sum(dim=(2, 3))
    b = (k.float() * dk).sum(dim=(2, 3))
    denom = (q.float() * dq).abs().sum(dim=(2, 3))
    assert ((a - b).abs() / denom).max().item() < 1e-3
    for g1, g2 in zip(grads[0], grads[1]):
        assert ((2 * g1 - g2).abs().max() / g2.abs().max()).item() < 1e-2  # one bf16 rounding of each side
    assert all(torch.isfinite(g).all().item() for g in grads[0])
