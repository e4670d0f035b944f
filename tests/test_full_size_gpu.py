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


# ---------------------------------------------------------------------------------------------------------
# Model-level parity at the full sizes of benchmark configurations 3 and 4, and every row of configuration 2
# ---------------------------------------------------------------------------------------------------------
MODEL_TOL = 6e-2        # bf16 model logits (|logit| ~ 2) against fp32 math on the same bf16-rounded weights
# what this code has been observed to stay under (3.0e-2 over the 65 positions of the decode test; one bf16 step
# of a logit of magnitude 2 to 4 is 1.6e-2); the observed value is part of every assertion message
MODEL_REGRESSION = 4.5e-2


def default_model(max_seq_len, seed=0):
    """The reference's default 16-layer model (d_model 640, 10 heads, window 512, 16 persistent tokens, vocabulary
    50 000, tied head) with every weight N(0, 0.02) from a seeded CPU generator, biases 0, norm scales 1; returns
    the bf16 module on the GPU and its weights as fp32 copies OF THE bf16 VALUES for the oracle."""
    from titanmac_b200 import TitanMAC, TitanMACConfig

    cfg = TitanMACConfig(vocab_size=50000, d_model=640, n_heads=10, n_layers=16, d_ff=2560, max_seq_len=max_seq_len,
                         window_size=512, n_persistent=16, use_block_sparse=False)
    g = torch.Generator(device="cpu").manual_seed(seed)
    model = TitanMAC(cfg).eval()
    with torch.no_grad():
        for name, prm in model.named_parameters():
            if name.endswith("scale"):
                prm.fill_(1.0)
            elif name.endswith("bias"):
                prm.zero_()
            else:
                prm.copy_(torch.randn(prm.shape, generator=g) * 0.02)
    model = model.to(device=DEV, dtype=torch.bfloat16)
    sd = {k: v.float().cpu() for k, v in model.state_dict().items()}
    return model, sd, cfg


@pytest.mark.gpu
def test_config3_model_logits_of_one_8192_token_sequence():
    """One sequence of benchmark configuration 3 through all 16 layers: logits at sampled positions against the model
    oracle (pinned to the reference's TitanMAC on the small fixture) in fp32 on the bf16-rounded weights."""
    from oracle import model_oracle as mo

    torch.set_grad_enabled(False)
    model, sd, cfg = default_model(8192)
    T = 8192
    ids = torch.randint(0, cfg.vocab_size, (1, T), generator=torch.Generator().manual_seed(3))
    logits = model(ids.to(DEV))["logits"]
    _native.poll_status(torch.device(DEV))
    assert logits.shape == (1, T, cfg.vocab_size)
    positions = [0, 1, 495, 496, 497, 511, 512, 513, 1024, 4095, 4096, 6000, T - 2, T - 1]
    ref = mo.model_forward(sd, ids, cfg.n_layers, cfg.n_heads, cfg.window_size, cfg.n_persistent, cfg.norm_eps,
                           positions=positions)
    err = (logits[:, positions].float().cpu() - ref).abs().max().item()
    assert err <= MODEL_TOL, f"observed max-abs logit error {err:.3e} (|logit| max {ref.abs().max().item():.2f})"
    assert err <= MODEL_REGRESSION, f"observed max-abs logit error {err:.3e} above the regression bound"


@pytest.mark.gpu
def test_config4_decode_steps_equal_one_teacher_forced_forward():
    """benchmark configuration 4 at full batch: 256 sequences, a prompt of 2048 tokens, then 64 single-token steps on the
    ring caches.  For two sampled sequences ONE teacher-forced oracle forward over the 2048 + 64 tokens gives
    the logits that every step must return (causality): the last prompt position and all 64 steps are compared."""
    from oracle import model_oracle as mo

    torch.set_grad_enabled(False)
    B, T0, steps = 256, 2048, 64
    model, sd, cfg = default_model(T0 + steps)
    ids = torch.randint(0, cfg.vocab_size, (B, T0 + steps), generator=torch.Generator().manual_seed(4))
    ids_dev = ids.to(DEV)
    sample = [0, B - 1]
    caches = model.new_caches(B, DEV, torch.bfloat16)
    got = []
    for b0 in range(0, B, 32):  # the prompt in slices of the batch (bounds the activation footprint)
        sub = model.new_caches(32, DEV, torch.bfloat16)
        lg, _ = model.prefill(ids_dev[b0:b0 + 32, :T0], sub)
        for full, part in zip(caches, sub):
            full.k_ring[b0:b0 + 32].copy_(part.k_ring); full.v_ring[b0:b0 + 32].copy_(part.v_ring)
            full.k_pers.copy_(part.k_pers); full.v_pers.copy_(part.v_pers)
        for s in sample:
            if b0 <= s < b0 + 32:
                got.append((s, lg[s - b0].float().cpu()))
    first = torch.stack([x for _, x in sorted(got, key=lambda t: t[0])])
    step_logits = []
    for t in range(T0, T0 + steps):
        pos = torch.full((B,), t, dtype=torch.int32, device=DEV)
        step_logits.append(model.decode_step(ids_dev[:, t], pos, caches)[sample].float().cpu())
    _native.poll_status(torch.device(DEV))
    ours = torch.cat([first[:, None], torch.stack(step_logits, dim=1)], dim=1)  # positions T0-1 .. T0+steps-1
    ref = mo.model_forward(sd, ids[sample], cfg.n_layers, cfg.n_heads, cfg.window_size, cfg.n_persistent,
                           cfg.norm_eps, positions=list(range(T0 - 1, T0 + steps)))
    err = (ours - ref).abs().max(dim=-1).values  # per (sequence, position)
    worst = err.max().item()
    assert worst <= MODEL_TOL, f"observed max-abs logit error {worst:.3e} at step {int(err.max(dim=0).values.argmax())}"
    assert worst <= MODEL_REGRESSION, f"observed max-abs logit error {worst:.3e} above the regression bound"


@pytest.mark.gpu
def test_config2_every_row_of_two_batch_elements():
    """benchmark configuration 2 (L = 16 + 4096, 10 heads x 64, window 512): ALL rows of the first and the last batch element
    of the tensor-core kernel's output against the oracle's block-wise evaluation."""
    B, T, D, H, w, Np = 8, 4096, 640, 10, 512, 16
    x, w_qkv, _ = wo.layer_inputs(B, T, D, Np, seed=0)
    qkv = torch.nn.functional.linear(x.to(torch.bfloat16).to(DEV), w_qkv.to(torch.bfloat16).to(DEV))
    L = Np + T
    q, k, v = (qkv.view(B, L, 3, H, 64)[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    o = _native.prefill(q, k, v, w, Np, algo=_native.ALGO_TCGEN05)
    _native.poll_status(torch.device(DEV))
    for b in (0, B - 1):
        qc, kc, vc = (t[b:b + 1].float().cpu() for t in (q, k, v))
        ref = wo.attention_core_blockwise(qc, kc, vc, w, Np, block=512)
        err = (o[b:b + 1].float().cpu() - ref).abs().max().item()
        assert err <= TOL, f"batch element {b}: observed max-abs error {err:.3e}"
        assert err <= 5e-3, f"batch element {b}: observed max-abs error {err:.3e} above the regression bound"
