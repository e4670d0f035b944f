"""The allocation-free split decode (`tmw_decode_split_static`) against `tmw_decode_split`.

Some hosts cannot allocate device memory around a decode step (a server that owns all of HBM through its
own pool, a loop that must not make a synchronising driver call).  For them the library keeps the scratch
memory of the split launch in a fixed built-in array.  This test calls that entry point through the C ABI
twice in a row on the same inputs and checks both results against the entry point that takes caller
scratch memory; it also checks that sizes beyond the built-in array are refused.  The file name makes
pytest collect it last.
"""

import ctypes

import pytest
import torch

from oracle import windowed_oracle as wo
from titanmac_b200 import _native

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _call(cache, fn_name, q, k_new, v_new, pos, splits, scratch=None):
    lib = _native.lib()
    out = torch.empty((cache.batch, cache.heads, cache.head_dim), dtype=cache.dtype, device=DEV)
    c = cache.desc()
    qs = (ctypes.c_int64 * 2)(q.stride(0), q.stride(1))
    ns = (ctypes.c_int64 * 2)(k_new.stride(0), k_new.stride(1))
    os_ = (ctypes.c_int64 * 2)(out.stride(0), out.stride(1))
    stream = torch.cuda.current_stream(DEV).cuda_stream
    if fn_name == "tmw_decode_split_static":
        rc = lib.tmw_decode_split_static(ctypes.byref(c), q.data_ptr(), k_new.data_ptr(), v_new.data_ptr(),
                                         out.data_ptr(), qs, ns, os_, pos.data_ptr(), splits, stream)
    else:
        rc = lib.tmw_decode_split(ctypes.byref(c), q.data_ptr(), k_new.data_ptr(), v_new.data_ptr(), out.data_ptr(),
                                  qs, ns, os_, pos.data_ptr(), splits, scratch.data_ptr(), scratch.numel() * 4, stream)
    return rc, out


def test_static_scratch_decode_matches_caller_scratch_decode_twice():
    dh, w, Np, B, H, splits = 64, 1500, 16, 2, 3, 6
    L = Np + 1800
    q, k, v = (t.to(torch.bfloat16) for t in wo.qkv_inputs(B, H, L, dh, seed=33))
    k[1:, :, :Np] = k[:1, :, :Np]
    v[1:, :, :Np] = v[:1, :, :Np]
    ts = [1700, 900]

    def fresh_cache():
        cache = _native.RingCache(B, H, dh, w, Np, torch.bfloat16, DEV)
        cache.set_persistent(k[0, :, :Np].to(DEV), v[0, :, :Np].to(DEV))
        for b, t in enumerate(ts):
            cb = _native.RingCache(1, H, dh, w, Np, torch.bfloat16, DEV)
            cb.fill(k[b:b + 1, :, Np:Np + t].to(DEV), v[b:b + 1, :, Np:Np + t].to(DEV))
            cache.k_ring[b].copy_(cb.k_ring[0])
            cache.v_ring[b].copy_(cb.v_ring[0])
        return cache

    qn = torch.stack([q[b, :, Np + t] for b, t in enumerate(ts)]).to(DEV)
    kn = torch.stack([k[b, :, Np + t] for b, t in enumerate(ts)]).to(DEV)
    vn = torch.stack([v[b, :, Np + t] for b, t in enumerate(ts)]).to(DEV)
    pos = torch.tensor(ts, dtype=torch.int32, device=DEV)

    ref_cache = fresh_cache()
    nbytes = _native.lib().tmw_decode_split_scratch_bytes(ctypes.byref(ref_cache.desc()), splits)
    scratch = torch.zeros(nbytes // 4, dtype=torch.float32, device=DEV)
    rc, want = _call(ref_cache, "tmw_decode_split", qn, kn, vn, pos, splits, scratch)
    assert rc == _native.TMW_OK

    static_cache = fresh_cache()
    for attempt in range(2):  # the second call finds the array as the first one left it
        rc, got = _call(static_cache, "tmw_decode_split_static", qn, kn, vn, pos, splits)
        assert rc == _native.TMW_OK, attempt
        torch.cuda.synchronize()
        assert (got.float() - want.float()).abs().max().item() <= 4e-3, attempt
    assert torch.equal(static_cache.k_ring, ref_cache.k_ring)  # the new token went into the same ring slots

    for b, t in enumerate(ts):  # and both agree with the oracle's last row
        ref = wo.attention_core_rows(q[b:b + 1, :, Np + t:Np + t + 1], k[b:b + 1], v[b:b + 1], Np + t, w, Np)
        assert (got[b].float().cpu() - ref[0, :, 0]).abs().max().item() <= 2e-2


def test_static_calls_follow_one_another_on_a_stream_without_synchronising():
    """Two calls with different geometries (6 splits over 6 pairs, then 3 splits over 2 pairs) issued back to back:
    the second reuses the built-in array as soon as the first has finished on the stream - the host does not
    wait in between."""
    dh, w, Np = 64, 1200, 8

    def case(B, H, t, seed):
        q, k, v = (x.to(torch.bfloat16) for x in wo.qkv_inputs(B, H, Np + t + 1, dh, seed=seed))
        k[1:, :, :Np] = k[:1, :, :Np]
        v[1:, :, :Np] = v[:1, :, :Np]

        def cache():
            c = _native.RingCache(B, H, dh, w, Np, torch.bfloat16, DEV)
            c.set_persistent(k[0, :, :Np].to(DEV), v[0, :, :Np].to(DEV))
            c.fill(k[:, :, Np:Np + t].to(DEV), v[:, :, Np:Np + t].to(DEV))
            return c

        new = tuple(x[:, :, Np + t].to(DEV) for x in (q, k, v))
        return cache, new, torch.full((B,), t, dtype=torch.int32, device=DEV)

    cases = [case(2, 3, 1500, 41) + (6,), case(1, 2, 1300, 42) + (3,)]
    want = []
    for cache, (qn, kn, vn), pos, splits in cases:
        c = cache()
        nbytes = _native.lib().tmw_decode_split_scratch_bytes(ctypes.byref(c.desc()), splits)
        scratch = torch.zeros(nbytes // 4, dtype=torch.float32, device=DEV)
        rc, out = _call(c, "tmw_decode_split", qn, kn, vn, pos, splits, scratch)
        assert rc == _native.TMW_OK
        want.append(out)
    caches = [cache() for cache, _, _, _ in cases]
    torch.cuda.synchronize()
    got = []
    for c, (_, (qn, kn, vn), pos, splits) in zip(caches, cases):  # no synchronisation between the two calls
        rc, out = _call(c, "tmw_decode_split_static", qn, kn, vn, pos, splits)
        assert rc == _native.TMW_OK
        got.append(out)
    torch.cuda.synchronize()
    for g, w_ in zip(got, want):
        assert (g.float() - w_.float()).abs().max().item() <= 4e-3


def test_static_scratch_decode_refuses_what_does_not_fit():
    lib = _native.lib()
    big = _native.RingCache(512, 10, 64, 8, 0, torch.bfloat16, DEV)  # 5120 pairs > 4096
    x = torch.zeros(512, 10, 64, dtype=torch.bfloat16, device=DEV)
    pos = torch.zeros(512, dtype=torch.int32, device=DEV)
    rc, _ = _call(big, "tmw_decode_split_static", x, x, x, pos, 2)
    assert rc == _native.TMW_ERR_TOO_LARGE
    assert b"built-in" in lib.tmw_last_cuda_error()
    wide = _native.RingCache(256, 10, 128, 8, 0, torch.bfloat16, DEV)  # 2560 pairs x 16 splits x 130 floats > 2 MiB
    x = torch.zeros(256, 10, 128, dtype=torch.bfloat16, device=DEV)
    rc, _ = _call(wide, "tmw_decode_split_static", x, x, x, pos[:256], 16)
    assert rc == _native.TMW_ERR_TOO_LARGE
