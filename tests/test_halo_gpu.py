"""Device-side halo path of the sequence-sharded prefill (tmw_halo_push, tmw_prefill_halo) on one GPU: the push
kernel fills the [persistent | halo] part of a rank's K/V buffer and raises the flags, the attention kernel
polls them; a flag that nobody raises makes the bounded wait expire and the call report TMW_ERR_DEVICE_TIMEOUT
while the context stays usable.  (The multi-GPU form, with the buffers of other processes mapped through CUDA
IPC, is exercised by bench.py on two and more GPUs, where sampled blocks are held against the oracle.)"""

import pytest
import torch

from oracle import windowed_oracle as wo
from titanmac_b200 import _native

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def sharded_case(dh, seed):
    """Rows [r0, r1) of a sequence as one rank sees them: its buffers [persistent | halo | own] start out with
    garbage in the first two parts."""
    L, w, Np, H = 1500, 200, 16, 2
    q, k, v = (t.to(torch.bfloat16).to(DEV) for t in wo.qkv_inputs(1, H, L, dh, seed=seed))
    r0, r1 = Np + 700, L
    lo = r0 - w
    # row-major buffers [1, rows, H, dh] like the sharded layout; NaN where other ranks will write
    rows = Np + w + (r1 - r0)
    kbuf = torch.full((1, rows, H, dh), float("nan"), dtype=torch.bfloat16, device=DEV)
    vbuf = torch.full_like(kbuf, float("nan"))
    kbuf[:, Np + w:] = k[:, :, r0:r1].permute(0, 2, 1, 3)
    vbuf[:, Np + w:] = v[:, :, r0:r1].permute(0, 2, 1, 3)
    src_k = k.permute(0, 2, 1, 3).contiguous()  # what the producers hold: [1, L, H, dh]
    src_v = v.permute(0, 2, 1, 3).contiguous()
    return dict(q=q, k=k, v=v, kbuf=kbuf, vbuf=vbuf, src_k=src_k, src_v=src_v, r0=r0, r1=r1, lo=lo, w=w, Np=Np, H=H,
                dh=dh, L=L)


@pytest.mark.parametrize("dh", [64, 128])
def test_push_then_prefill_with_flags_equals_unsharded_rows(dh):
    c = sharded_case(dh, seed=7)
    Np, w, r0, r1, lo = c["Np"], c["w"], c["r0"], c["r1"], c["lo"]
    row_bytes = c["H"] * dh * 2
    flags = torch.zeros(4, dtype=torch.int32, device=DEV)
    for step in (1, 2):  # two steps in a row: the flags carry the step number
        # persistent rows (what rank 0 would push) and the halo (what the left neighbour would push)
        _native.halo_push([(c["src_k"].data_ptr(), c["kbuf"].data_ptr(), Np * row_bytes),
                           (c["src_v"].data_ptr(), c["vbuf"].data_ptr(), Np * row_bytes)], DEV,
                          signal_flag=flags.data_ptr(), signal_value=step)
        _native.halo_push([(c["src_k"].data_ptr() + lo * row_bytes, c["kbuf"].data_ptr() + Np * row_bytes, w * row_bytes),
                           (c["src_v"].data_ptr() + lo * row_bytes, c["vbuf"].data_ptr() + Np * row_bytes, w * row_bytes)],
                          DEV, wait_flag=flags.data_ptr() + 8, wait_value=step - 1,
                          signal_flag=flags.data_ptr() + 4, signal_value=step)
        hw = _native.HaloWait()
        hw.pers_flag, hw.halo_flag, hw.value, hw.halo_rows = flags.data_ptr(), flags.data_ptr() + 4, step, w
        out = _native.prefill(c["q"][:, :, r0:r1].contiguous(), c["kbuf"].permute(0, 2, 1, 3),
                              c["vbuf"].permute(0, 2, 1, 3), w, Np, q_pos0=r0, k_pos0=lo, halo_wait=hw)
        _native.halo_push([], DEV, signal_flag=flags.data_ptr() + 8, signal_value=step)  # acknowledgement
        _native.poll_status(DEV)
        assert flags[:3].tolist() == [step, step, step]
        ref = wo.attention_core_rows(c["q"][:, :, r0:r1].float().cpu(), c["k"].float().cpu(), c["v"].float().cpu(), r0, w, Np)
        err = (out.float().cpu() - ref).abs().max().item()
        assert err <= 2e-2, f"step {step}: observed max-abs error {err:.3e}"
        c["kbuf"][:, :Np + w] = float("nan")  # the next step must bring the rows again
        c["vbuf"][:, :Np + w] = float("nan")


def test_flag_that_is_never_raised_times_out_and_the_context_survives():
    c = sharded_case(64, seed=8)
    Np, w, r0, r1, lo = c["Np"], c["w"], c["r0"], c["r1"], c["lo"]
    c["kbuf"][:, :Np + w] = 0
    c["vbuf"][:, :Np + w] = 0
    flags = torch.zeros(2, dtype=torch.int32, device=DEV)
    hw = _native.HaloWait()
    hw.pers_flag, hw.halo_flag, hw.value, hw.halo_rows = flags.data_ptr(), flags.data_ptr() + 4, 1, w
    hw.wait_limit_cycles = 2_000_000  # about a millisecond
    _native.prefill(c["q"][:, :, r0:r1].contiguous(), c["kbuf"].permute(0, 2, 1, 3), c["vbuf"].permute(0, 2, 1, 3), w, Np,
                    q_pos0=r0, k_pos0=lo, halo_wait=hw)
    with pytest.raises(_native.TmwError) as e:
        _native.poll_status(DEV)
    assert e.value.status == _native.TMW_ERR_DEVICE_TIMEOUT
    # the same for a push that waits for an acknowledgement nobody sends: nothing is copied, nothing signalled
    dst = torch.zeros(64, dtype=torch.int32, device=DEV)
    src = torch.ones(64, dtype=torch.int32, device=DEV)
    _native.halo_push([(src.data_ptr(), dst.data_ptr(), 256)], DEV, wait_flag=flags.data_ptr(), wait_value=5,
                      signal_flag=flags.data_ptr() + 4, signal_value=9, wait_limit_cycles=2_000_000)
    with pytest.raises(_native.TmwError) as e:
        _native.poll_status(DEV)
    assert e.value.status == _native.TMW_ERR_DEVICE_TIMEOUT
    assert int(dst.sum()) == 0 and flags.tolist() == [0, 0]
    # status cleared, context usable: an ordinary call works
    o = _native.prefill(c["q"], c["k"], c["v"], w, Np)
    _native.poll_status(DEV)
    assert torch.isfinite(o.float()).all()


def test_push_argument_checks():
    buf = torch.zeros(64, dtype=torch.int32, device=DEV)
    with pytest.raises(_native.TmwError) as e:
        _native.halo_push([(buf.data_ptr() + 4, buf.data_ptr(), 16)], DEV)
    assert e.value.status == _native.TMW_ERR_INVALID_ARGUMENT
    with pytest.raises(_native.TmwError) as e:
        _native.halo_push([(buf.data_ptr(), buf.data_ptr() + 128, 24)], DEV)
    assert e.value.status == _native.TMW_ERR_INVALID_ARGUMENT
