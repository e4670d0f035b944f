"""The C-ABI library loads, exports exactly what include/tmw.h declares, and its host-side
argument checks answer without touching a GPU (no compute call is made here)."""

import ctypes
import os
import re
import subprocess
import tempfile

import pytest

from conftest import ROOT
from titanmac_b200 import _native

HEADER = os.path.join(ROOT, "include", "tmw.h")


def declared_symbols():
    text = open(HEADER).read()
    return sorted(set(re.findall(r"TMW_API[^;()]*?\b(tmw_[a-z_0-9]+)\s*\(", text)))


def test_header_binding_and_exports_agree():
    declared = declared_symbols()
    assert declared, "no TMW_API declarations found"
    assert declared == sorted(_native.SIGNATURES)
    out = subprocess.run(["nm", "-D", "--defined-only", _native.LIB_PATH], capture_output=True, text=True, check=True)
    exported = sorted(line.split()[-1] for line in out.stdout.splitlines() if " T tmw_" in line)
    assert exported == declared
    lib = _native.lib()
    for name in declared:
        assert getattr(lib, name) is not None


def test_struct_layouts_match_the_header():
    src = r"""
    #include <stdio.h>
    #include <stddef.h>
    #include "tmw.h"
    int main(void) {
        printf("%zu %zu %zu %zu %zu\n", sizeof(tmw_prefill_desc), offsetof(tmw_prefill_desc, scale),
               offsetof(tmw_prefill_desc, q_stride), offsetof(tmw_prefill_desc, o_stride),
               offsetof(tmw_prefill_desc, k_pos0));
        printf("%zu %zu %zu %zu\n", sizeof(tmw_cache_desc), offsetof(tmw_cache_desc, k_ring),
               offsetof(tmw_cache_desc, v_pers), offsetof(tmw_cache_desc, scale));
        printf("%zu %zu %zu %zu\n", sizeof(tmw_linear_desc), offsetof(tmw_linear_desc, epilogue),
               offsetof(tmw_linear_desc, lda), offsetof(tmw_linear_desc, ldc));
        return 0;
    }
    """
    with tempfile.TemporaryDirectory() as d:
        c = os.path.join(d, "t.c")
        open(c, "w").write(src)
        exe = os.path.join(d, "t")
        subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), c, "-o", exe], check=True)
        lines = subprocess.run([exe], capture_output=True, text=True, check=True).stdout.split("\n")
    P, C = _native.PrefillDesc, _native.CacheDesc
    assert [int(v) for v in lines[0].split()] == [ctypes.sizeof(P), P.scale.offset, P.q_stride.offset,
                                                  P.o_stride.offset, P.k_pos0.offset]
    assert [int(v) for v in lines[1].split()] == [ctypes.sizeof(C), C.k_ring.offset, C.v_pers.offset, C.scale.offset]
    G = _native.LinearDesc
    assert [int(v) for v in lines[2].split()] == [ctypes.sizeof(G), G.epilogue.offset, G.lda.offset, G.ldc.offset]


def test_version_and_error_text():
    lib = _native.lib()
    assert lib.tmw_version() == 100
    assert lib.tmw_strerror(0) == b"ok"
    for code in range(-8, 0):
        assert lib.tmw_strerror(code) not in (b"ok", b"unknown status")
    assert lib.tmw_strerror(-99) == b"unknown status"


def _desc(**kw):
    d = _native.PrefillDesc()
    d.dtype, d.algo = _native.TMW_BF16, 0
    d.batch, d.heads, d.head_dim = 1, 1, 64
    d.q_rows = d.k_rows = 128
    d.window, d.n_persistent, d.q_pos0, d.k_pos0 = 16, 4, 0, 4
    for i, s in enumerate((0, 64, 64)):
        d.q_stride[i] = d.k_stride[i] = d.v_stride[i] = d.o_stride[i] = s
    for k, v in kw.items():
        setattr(d, k, v)
    return d


@pytest.mark.parametrize("kw,expected", [
    (dict(window=-1), _native.TMW_ERR_NEGATIVE_WINDOW),
    (dict(n_persistent=128, k_pos0=128), _native.TMW_ERR_PERSISTENT_GE_LEN),
    (dict(n_persistent=200, k_pos0=200), _native.TMW_ERR_PERSISTENT_GE_LEN),
    (dict(dtype=7), _native.TMW_ERR_UNSUPPORTED),
    (dict(k_pos0=2), _native.TMW_ERR_INVALID_ARGUMENT),
    (dict(q_rows=-1), _native.TMW_ERR_INVALID_ARGUMENT),
    (dict(algo=9), _native.TMW_ERR_INVALID_ARGUMENT),
    (dict(q_pos0=300), _native.TMW_ERR_KEY_RANGE),          # queries past the last key
    (dict(q_pos0=60, k_pos0=50), _native.TMW_ERR_KEY_RANGE),  # window starts before the first held key
])
def test_prefill_rejects_bad_descriptors_on_the_host(kw, expected):
    d = _desc(**kw)
    fake = ctypes.c_void_p(0x1000)  # never dereferenced: validation fails first
    assert _native.lib().tmw_prefill(ctypes.byref(d), fake, fake, fake, fake, None) == expected


def test_prefill_rejects_null_misaligned_and_odd_strides():
    lib = _native.lib()
    ok = ctypes.c_void_p(0x1000)
    d = _desc()
    assert lib.tmw_prefill(None, ok, ok, ok, ok, None) == _native.TMW_ERR_INVALID_ARGUMENT
    assert lib.tmw_prefill(ctypes.byref(d), None, ok, ok, ok, None) == _native.TMW_ERR_INVALID_ARGUMENT
    assert lib.tmw_prefill(ctypes.byref(d), ctypes.c_void_p(0x1004), ok, ok, ok, None) == _native.TMW_ERR_INVALID_ARGUMENT
    d = _desc()
    d.k_stride[2] = 63
    assert lib.tmw_prefill(ctypes.byref(d), ok, ok, ok, ok, None) == _native.TMW_ERR_INVALID_ARGUMENT
    # an empty problem is fine and launches nothing
    assert lib.tmw_prefill(ctypes.byref(_desc(batch=0)), None, None, None, None, None) == _native.TMW_OK


def test_cache_entry_points_reject_bad_arguments_on_the_host():
    lib = _native.lib()
    assert lib.tmw_cache_ring_bytes(_native.TMW_BF16, 256, 10, 64, 512) == 256 * 10 * 513 * 64 * 2
    assert lib.tmw_cache_ring_bytes(_native.TMW_F32, 2, 3, 16, 0) == 2 * 3 * 1 * 16 * 4
    assert lib.tmw_cache_ring_bytes(9, 1, 1, 64, 4) == 0
    c = _native.CacheDesc()
    c.dtype, c.batch, c.heads, c.head_dim, c.window, c.n_persistent = _native.TMW_BF16, 1, 1, 64, -2, 0
    s3 = (ctypes.c_int64 * 3)(0, 64, 64)
    s2 = (ctypes.c_int64 * 2)(64, 64)
    ok = ctypes.c_void_p(0x1000)
    assert lib.tmw_cache_fill(ctypes.byref(c), ok, ok, s3, s3, 4, 0, None) == _native.TMW_ERR_NEGATIVE_WINDOW
    c.window, c.head_dim = 4, 48
    assert lib.tmw_decode(ctypes.byref(c), ok, ok, ok, ok, s2, s2, s2, ok, None) == _native.TMW_ERR_UNSUPPORTED
    c.head_dim = 64  # rings are NULL
    assert lib.tmw_decode(ctypes.byref(c), ok, ok, ok, ok, s2, s2, s2, ok, None) == _native.TMW_ERR_INVALID_ARGUMENT


def test_split_decode_scratch_size_and_argument_checks():
    lib = _native.lib()
    c = _native.CacheDesc()
    c.dtype, c.batch, c.heads, c.head_dim, c.window, c.n_persistent = _native.TMW_BF16, 32, 10, 64, 512, 0
    c.k_ring = c.v_ring = 0x1000
    assert lib.tmw_decode_split_scratch_bytes(ctypes.byref(c), 4) == 32 * 10 * 4 * (64 + 2) * 4 + 32 * 10 * 4
    assert lib.tmw_decode_split_scratch_bytes(ctypes.byref(c), 0) == 0
    assert lib.tmw_decode_split_scratch_bytes(ctypes.byref(c), _native.MAX_DECODE_SPLITS + 1) == 0
    s2 = (ctypes.c_int64 * 2)(640, 64)
    ok = ctypes.c_void_p(0x1000)
    args = (ctypes.byref(c), ok, ok, ok, ok, s2, s2, s2, ok)
    assert lib.tmw_decode_split(*args, 0, ok, 1 << 30, None) == _native.TMW_ERR_INVALID_ARGUMENT   # splits
    assert lib.tmw_decode_split(*args, 4, None, 1 << 30, None) == _native.TMW_ERR_INVALID_ARGUMENT  # no scratch
    assert lib.tmw_decode_split(*args, 4, ok, 1024, None) == _native.TMW_ERR_TOO_LARGE            # scratch too small
