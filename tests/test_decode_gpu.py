"""Parity of the ring-cache decode path (through the C ABI) with the reference's decode semantics:
the output for a new token equals the last row of a full forward over everything seen so far."""

import pytest
import torch

from oracle import windowed_oracle as wo
from titanmac_b200 import _native

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def run_decode(q, k, v, w, Np, prefill_tokens, dtype):
    """q,k,v: [B,H,L,dh] CPU.  Prefill the ring with the first tokens, then decode the rest one by one."""
    B, H, L, dh = q.shape
    cache = _native.RingCache(B, H, dh, w, Np, dtype, DEV)
    qd, kd, vd = (t.to(dtype).to(DEV) for t in (q, k, v))
    cache.set_persistent(kd[0, :, :Np], vd[0, :, :Np])
    if prefill_tokens > 0:
        cache.fill(kd[:, :, Np:Np + prefill_tokens], vd[:, :, Np:Np + prefill_tokens], t0=0)
    outs = []
    for t in range(prefill_tokens, L - Np):
        pos = torch.full((B,), t, dtype=torch.int32, device=DEV)
        outs.append(cache.decode(qd[:, :, Np + t], kd[:, :, Np + t], vd[:, :, Np + t], pos).clone())
    return torch.stack(outs, dim=2)  # [B,H,steps,dh]


def test_decode_fp32_equals_last_row_of_reference_forward(golden):
    case = "dh64_multi_tile"   # L=300, w=64, Np=16: the ring wraps several times
    m = golden.meta(case)
    q, k, v, o = (golden[case, f"core_{n}"] for n in "qkvo")
    for pre in (0, 10, 100):
        got = run_decode(q, k, v, m["w"], m["Np"], pre, torch.float32).cpu()
        want = o[:, :, m["Np"] + pre:]
        assert (got - want).abs().max().item() <= 1e-5, pre


@pytest.mark.parametrize("dh,w,Np,B,H,L,pre", [
    (64, 512, 16, 3, 10, 16 + 700, 600),   # default model geometry, ring wraps
    (128, 100, 16, 2, 2, 16 + 230, 0),
    (32, 7, 0, 2, 3, 60, 3),               # no persistent keys
    (16, 0, 2, 1, 2, 2 + 20, 1),           # self-only window
    (256, 20, 4, 1, 1, 4 + 50, 25),
    (8, 5, 1, 2, 1, 1 + 30, 0),
])
def test_decode_bf16_matches_fp32_oracle(dh, w, Np, B, H, L, pre):
    q, k, v = wo.qkv_inputs(B, H, L, dh, seed=dh + w)
    q, k, v = (t.to(torch.bfloat16) for t in (q, k, v))
    k[1:, :, :Np] = k[:1, :, :Np]  # persistent rows are shared by the batch
    v[1:, :, :Np] = v[:1, :, :Np]
    got = run_decode(q, k, v, w, Np, pre, torch.bfloat16).float().cpu()
    want = wo.attention_core_rows(q[:, :, Np + pre:], k, v, Np + pre, w, Np)
    assert (got - want).abs().max().item() <= 2e-2


@pytest.mark.parametrize("dh,w,Np,B,H,steps,pre,dtype", [
    (64, 40, 5, 80, 8, 60, 0, torch.bfloat16),    # 640 pairs: one pair per two-warp CTA
    (64, 19, 3, 170, 8, 12, 25, torch.bfloat16),  # 1360 pairs: one warp per pair, two pairs per CTA
    (64, 45, 16, 20, 5, 70, 0, torch.bfloat16),   # 100 pairs: four warps share a pair
    (128, 30, 2, 16, 8, 40, 10, torch.float16),   # 128 pairs, head_dim 128, four warps
    (64, 37, 16, 100, 10, 30, 30, torch.bfloat16),
    (128, 21, 0, 75, 8, 50, 3, torch.float16),    # no persistent keys, ring shorter than one chunk at first
    (128, 33, 7, 160, 4, 20, 40, torch.bfloat16),
])
def test_decode_streaming_kernel_many_pairs(dh, w, Np, B, H, steps, pre, dtype):
    """16-bit caches with more than half a pair per SM run the shared-memory streaming variant in one of its
    three launch shapes: same contract - first tokens, a ring that is not full yet, several wraps of the ring."""
    L = Np + pre + steps
    q, k, v = (t.to(dtype) for t in wo.qkv_inputs(B, H, L, dh, seed=dh + w + B))
    k[1:, :, :Np] = k[:1, :, :Np]
    v[1:, :, :Np] = v[:1, :, :Np]
    got = run_decode(q, k, v, w, Np, pre, dtype).float().cpu()
    want = wo.attention_core_rows(q[:, :, Np + pre:].float(), k.float(), v.float(), Np + pre, w, Np)
    assert (got - want).abs().max().item() <= 2e-2
    _native.poll_status(torch.device(DEV))


def test_decode_ragged_positions_and_strided_inputs():
    """Sequences at different positions in one call; q/k/v taken as strided views of one [B, 3D] buffer."""
    dh, w, Np, B, H = 64, 50, 4, 4, 3
    L = Np + 200
    q, k, v = (t.to(torch.bfloat16) for t in wo.qkv_inputs(B, H, L, dh, seed=9))
    k[1:, :, :Np] = k[:1, :, :Np]
    v[1:, :, :Np] = v[:1, :, :Np]
    ts = [0, 49, 50, 137]
    cache = _native.RingCache(B, H, dh, w, Np, torch.bfloat16, DEV)
    cache.set_persistent(k[0, :, :Np].to(DEV), v[0, :, :Np].to(DEV))
    for b, t in enumerate(ts):  # history of sequence b: tokens 0..t-1
        if t > 0:
            cb = _native.RingCache(1, H, dh, w, Np, torch.bfloat16, DEV)
            cb.fill(k[b:b + 1, :, Np:Np + t].to(DEV), v[b:b + 1, :, Np:Np + t].to(DEV))
            cache.k_ring[b].copy_(cb.k_ring[0])
            cache.v_ring[b].copy_(cb.v_ring[0])
    qkv = torch.empty(B, 3, H, dh, dtype=torch.bfloat16, device=DEV)
    for b, t in enumerate(ts):
        qkv[b, 0], qkv[b, 1], qkv[b, 2] = q[b, :, Np + t].to(DEV), k[b, :, Np + t].to(DEV), v[b, :, Np + t].to(DEV)
    pos = torch.tensor(ts, dtype=torch.int32, device=DEV)
    got = cache.decode(qkv[:, 0], qkv[:, 1], qkv[:, 2], pos).float().cpu()
    for b, t in enumerate(ts):
        want = wo.attention_core_rows(q[b:b + 1, :, Np + t:Np + t + 1], k[b:b + 1], v[b:b + 1], Np + t, w, Np)
        assert (got[b] - want[0, :, 0]).abs().max().item() <= 2e-2, (b, t)
        assert torch.equal(cache.k_ring[b, :, t % (w + 1)].cpu(), k[b, :, Np + t])


def test_cache_fill_keeps_only_the_window():
    dh, w, B, H = 16, 4, 1, 1
    k = torch.arange(12, dtype=torch.float32).view(1, 1, 12, 1).expand(B, H, 12, dh).contiguous().to(DEV)
    cache = _native.RingCache(B, H, dh, w, 0, torch.float32, DEV)
    cache.fill(k, k, t0=3)  # tokens 3..14; the ring of 5 slots keeps tokens 10..14
    ring = cache.k_ring[0, 0, :, 0].cpu().tolist()
    assert sorted(ring) == [7.0, 8.0, 9.0, 10.0, 11.0]       # row i holds value i = token 3+i
    for tok in range(10, 15):
        assert ring[tok % 5] == float(tok - 3)


@pytest.mark.parametrize("splits", [0, 1, 3, 16])
def test_split_and_unsplit_decode_agree(splits):
    """The split launch (partials in scratch memory + merge kernel) returns what the one-CTA-per-pair launch
    returns, for every split count, with ragged positions (some splits of short sequences are empty)."""
    dh, w, Np, B, H = 64, 200, 16, 5, 3
    L = Np + 400
    q, k, v = (t.to(torch.bfloat16) for t in wo.qkv_inputs(B, H, L, dh, seed=21))
    k[1:, :, :Np] = k[:1, :, :Np]
    v[1:, :, :Np] = v[:1, :, :Np]
    ts = [0, 1, 57, 200, 399]
    outs = []
    for s in (splits, 0):
        cache = _native.RingCache(B, H, dh, w, Np, torch.bfloat16, DEV)
        cache.splits = s
        cache.set_persistent(k[0, :, :Np].to(DEV), v[0, :, :Np].to(DEV))
        for b, t in enumerate(ts):
            if t > 0:
                cb = _native.RingCache(1, H, dh, w, Np, torch.bfloat16, DEV)
                cb.fill(k[b:b + 1, :, Np:Np + t].to(DEV), v[b:b + 1, :, Np:Np + t].to(DEV))
                cache.k_ring[b].copy_(cb.k_ring[0])
                cache.v_ring[b].copy_(cb.v_ring[0])
        qn = torch.stack([q[b, :, Np + t] for b, t in enumerate(ts)]).to(DEV)
        kn = torch.stack([k[b, :, Np + t] for b, t in enumerate(ts)]).to(DEV)
        vn = torch.stack([v[b, :, Np + t] for b, t in enumerate(ts)]).to(DEV)
        pos = torch.tensor(ts, dtype=torch.int32, device=DEV)
        outs.append((cache.decode(qn, kn, vn, pos).float().cpu(), cache.k_ring.clone().cpu()))
    assert (outs[0][0] - outs[1][0]).abs().max().item() <= 4e-3   # same math, different merge order
    assert torch.equal(outs[0][1], outs[1][1])                    # the new token landed in the same slots
    for b, t in enumerate(ts):
        want = wo.attention_core_rows(q[b:b + 1, :, Np + t:Np + t + 1], k[b:b + 1], v[b:b + 1], Np + t, w, Np)
        assert (outs[0][0][b] - want[0, :, 0]).abs().max().item() <= 2e-2


def test_negative_position_is_reported_not_written_out_of_bounds():
    """pos is a device array the host cannot check: a negative entry is treated as position 0 by the kernels and
    comes back from tmw_poll_status as an invalid argument."""
    B, H, dh, w, Np = 3, 2, 64, 16, 4
    cache = _native.RingCache(B, H, dh, w, Np, torch.bfloat16, DEV)
    for t_ in (cache.k_ring, cache.v_ring, cache.k_pers, cache.v_pers):
        t_.normal_()
    guard_k = cache.k_ring.clone()
    x = torch.randn(B, 3, H, dh, device=DEV).to(torch.bfloat16)
    pos = torch.tensor([5, -7, 2], dtype=torch.int32, device=DEV)
    out = cache.decode(x[:, 0], x[:, 1], x[:, 2], pos)
    with pytest.raises(_native.TmwError) as e:
        _native.poll_status(torch.device(DEV))
    assert e.value.status == _native.TMW_ERR_INVALID_ARGUMENT
    assert torch.isfinite(out.float()).all()
    # only the slots of positions 5, 0 (the negative one) and 2 changed
    changed = (cache.k_ring != guard_k).any(dim=-1).any(dim=1)  # [B, slots]
    assert changed.nonzero().tolist() == [[0, 5], [1, 0], [2, 2]]
    _native.poll_status(torch.device(DEV))  # the status word was cleared
