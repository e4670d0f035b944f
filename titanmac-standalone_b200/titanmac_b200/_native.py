"""ctypes binding of ``libtmw.so`` (C ABI declared in ``include/tmw.h``).

There is no other implementation behind these functions: if the shared library is
missing or a call fails, an exception is raised — nothing falls back to PyTorch
or to the CPU.
"""

from __future__ import annotations

import ctypes
import math
import os
from typing import Optional, Sequence

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtmw.so")

TMW_OK = 0
TMW_ERR_INVALID_ARGUMENT = -1
TMW_ERR_UNSUPPORTED = -2
TMW_ERR_PERSISTENT_GE_LEN = -3
TMW_ERR_NEGATIVE_WINDOW = -4
TMW_ERR_KEY_RANGE = -5
TMW_ERR_CUDA = -6
TMW_ERR_DEVICE_TIMEOUT = -7
TMW_ERR_TOO_LARGE = -8

TMW_F32, TMW_BF16, TMW_F16 = 0, 1, 2
ALGO_AUTO, ALGO_SIMT, ALGO_TCGEN05, ALGO_MMA = 0, 1, 2, 3

_DTYPES = {torch.float32: TMW_F32, torch.bfloat16: TMW_BF16, torch.float16: TMW_F16}


class TmwError(RuntimeError):
    """A libtmw call returned a status that has no more specific Python exception."""

    def __init__(self, status: int, text: str):
        super().__init__(f"libtmw: {text} (status {status})")
        self.status = status


class PrefillDesc(ctypes.Structure):
    _fields_ = [
        ("dtype", ctypes.c_int32),
        ("algo", ctypes.c_int32),
        ("batch", ctypes.c_int32),
        ("heads", ctypes.c_int32),
        ("head_dim", ctypes.c_int32),
        ("q_rows", ctypes.c_int32),
        ("k_rows", ctypes.c_int32),
        ("window", ctypes.c_int32),
        ("n_persistent", ctypes.c_int32),
        ("q_pos0", ctypes.c_int32),
        ("k_pos0", ctypes.c_int32),
        ("scale", ctypes.c_float),
        ("q_stride", ctypes.c_int64 * 3),
        ("k_stride", ctypes.c_int64 * 3),
        ("v_stride", ctypes.c_int64 * 3),
        ("o_stride", ctypes.c_int64 * 3),
    ]


class CacheDesc(ctypes.Structure):
    _fields_ = [
        ("dtype", ctypes.c_int32),
        ("batch", ctypes.c_int32),
        ("heads", ctypes.c_int32),
        ("head_dim", ctypes.c_int32),
        ("window", ctypes.c_int32),
        ("n_persistent", ctypes.c_int32),
        ("k_ring", ctypes.c_void_p),
        ("v_ring", ctypes.c_void_p),
        ("k_pers", ctypes.c_void_p),
        ("v_pers", ctypes.c_void_p),
        ("scale", ctypes.c_float),
    ]


class LinearDesc(ctypes.Structure):
    _fields_ = [
        ("dtype", ctypes.c_int32),
        ("m", ctypes.c_int32),
        ("n", ctypes.c_int32),
        ("k", ctypes.c_int32),
        ("epilogue", ctypes.c_int32),
        ("lda", ctypes.c_int64),
        ("ldw", ctypes.c_int64),
        ("ldc", ctypes.c_int64),
    ]


EPILOGUE_NONE, EPILOGUE_GELU = 0, 1
HALO_MAX_COPIES = 8


class HaloCopy(ctypes.Structure):
    _fields_ = [("src", ctypes.c_void_p), ("dst", ctypes.c_void_p), ("bytes", ctypes.c_size_t)]


class IpcMem(ctypes.Structure):
    _fields_ = [("handle", ctypes.c_ubyte * 64), ("offset", ctypes.c_uint64), ("size", ctypes.c_uint64)]


class HaloWait(ctypes.Structure):
    _fields_ = [
        ("pers_flag", ctypes.c_void_p),
        ("halo_flag", ctypes.c_void_p),
        ("value", ctypes.c_int32),
        ("halo_rows", ctypes.c_int32),
        ("wait_limit_cycles", ctypes.c_int64),
    ]


# name -> (restype, argtypes); the CPU test-suite checks that every symbol here is
# declared in include/tmw.h and exported by the library, and vice versa.
SIGNATURES = {
    "tmw_version": (ctypes.c_int, []),
    "tmw_strerror": (ctypes.c_char_p, [ctypes.c_int]),
    "tmw_last_cuda_error": (ctypes.c_char_p, []),
    "tmw_poll_status": (ctypes.c_int, [ctypes.c_void_p]),
    "tmw_prefill": (
        ctypes.c_int,
        [ctypes.POINTER(PrefillDesc), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
         ctypes.c_void_p],
    ),
    "tmw_prefill_lse": (
        ctypes.c_int,
        [ctypes.POINTER(PrefillDesc)] + [ctypes.c_void_p] * 6,
    ),
    "tmw_prefill_backward": (
        ctypes.c_int,
        [ctypes.POINTER(PrefillDesc)] + [ctypes.c_void_p] * 10,
    ),
    "tmw_prefill_block_sparse_lse": (
        ctypes.c_int,
        [ctypes.POINTER(PrefillDesc), ctypes.c_int32] + [ctypes.c_void_p] * 6,
    ),
    "tmw_prefill_block_sparse_backward": (
        ctypes.c_int,
        [ctypes.POINTER(PrefillDesc), ctypes.c_int32] + [ctypes.c_void_p] * 10,
    ),
    "tmw_prefill_block_sparse": (
        ctypes.c_int,
        [ctypes.POINTER(PrefillDesc), ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
         ctypes.c_void_p, ctypes.c_void_p],
    ),
    "tmw_causal_dwconv_backward": (
        ctypes.c_int,
        [ctypes.c_int32] * 5 + [ctypes.c_void_p] * 6,
    ),
    "tmw_causal_dwconv": (
        ctypes.c_int,
        [ctypes.c_int32] * 5 + [ctypes.c_void_p] * 4,
    ),
    "tmw_cache_ring_bytes": (ctypes.c_size_t, [ctypes.c_int32] * 5),
    "tmw_cache_fill": (
        ctypes.c_int,
        [ctypes.POINTER(CacheDesc), ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(ctypes.c_int64),
         ctypes.POINTER(ctypes.c_int64), ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p],
    ),
    "tmw_decode": (
        ctypes.c_int,
        [ctypes.POINTER(CacheDesc), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
         ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_int64),
         ctypes.c_void_p, ctypes.c_void_p],
    ),
    "tmw_decode_split_scratch_bytes": (ctypes.c_size_t, [ctypes.POINTER(CacheDesc), ctypes.c_int32]),
    "tmw_decode_split": (
        ctypes.c_int,
        [ctypes.POINTER(CacheDesc), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
         ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_int64),
         ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p],
    ),
    "tmw_decode_split_static": (
        ctypes.c_int,
        [ctypes.POINTER(CacheDesc), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
         ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_int64),
         ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p],
    ),
    "tmw_halo_push": (
        ctypes.c_int,
        [ctypes.POINTER(HaloCopy), ctypes.c_int32, ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p, ctypes.c_int32,
         ctypes.c_int64, ctypes.c_void_p],
    ),
    "tmw_enable_peer_access": (ctypes.c_int, [ctypes.c_int32]),
    "tmw_ipc_export": (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(IpcMem)]),
    "tmw_ipc_open": (ctypes.c_int, [ctypes.POINTER(IpcMem), ctypes.POINTER(ctypes.c_void_p)]),
    "tmw_ipc_close_all": (ctypes.c_int, []),
    "tmw_prefill_halo": (
        ctypes.c_int,
        [ctypes.POINTER(PrefillDesc)] + [ctypes.c_void_p] * 4 + [ctypes.POINTER(HaloWait), ctypes.c_void_p],
    ),
    "tmw_linear": (ctypes.c_int, [ctypes.POINTER(LinearDesc)] + [ctypes.c_void_p] * 5),
    "tmw_gelu": (ctypes.c_int, [ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
    "tmw_add_rmsnorm": (
        ctypes.c_int,
        [ctypes.c_int32, ctypes.c_int64, ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
         ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p],
    ),
}

MAX_DECODE_SPLITS = 16

_lib: Optional[ctypes.CDLL] = None


def lib() -> ctypes.CDLL:
    """Load ``libtmw.so`` from the package directory (once)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `make -C titanmac-standalone_b200/csrc -j` "
                "(nvcc, sm_100a).  There is no fallback implementation."
            )
        handle = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def check(status: int) -> None:
    """Map a libtmw status to the exception the reference raises in the same situation."""
    if status == TMW_OK:
        return
    text = lib().tmw_strerror(status).decode()
    if status in (TMW_ERR_PERSISTENT_GE_LEN, TMW_ERR_NEGATIVE_WINDOW):
        raise ValueError(text)  # build_band_mask raises ValueError for both
    if status in (TMW_ERR_CUDA, TMW_ERR_DEVICE_TIMEOUT):
        text += ": " + lib().tmw_last_cuda_error().decode()
    raise TmwError(status, text)


def _require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("libtmw works on CUDA tensors only; there is no CPU path")


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _bhrd_strides(t: torch.Tensor) -> Sequence[int]:
    if t.stride(3) != 1:
        raise ValueError("the head_dim axis must be contiguous")
    return (t.stride(0), t.stride(1), t.stride(2))


def prefill(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    window: int,
    n_persistent: int,
    out: Optional[torch.Tensor] = None,
    q_pos0: int = 0,
    k_pos0: Optional[int] = None,
    scale: float = 0.0,
    algo: int = ALGO_AUTO,
    window_block: int = 0,
    lse: Optional[torch.Tensor] = None,
    halo_wait: Optional[HaloWait] = None,
) -> torch.Tensor:
    """``tmw_prefill`` on ``[B, H, rows, dh]`` tensors (any strides with a contiguous last axis).

    ``halo_wait`` selects ``tmw_prefill_halo``: the kernel polls the given flags before it reads the persistent /
    halo rows of the K/V buffer (sequence-sharded ranks whose neighbours push those rows, see ``halo_push``).

    ``window_block > 0`` selects ``tmw_prefill_block_sparse``: the mask of the reference's
    BlockSparseAttention with that block size (whole sequences only).  ``lse`` (fp32 ``[B, H, rows]``,
    contiguous) receives every row's log-sum-exp (``tmw_prefill_lse``), which ``prefill_backward`` needs."""
    _require_cuda(q, k, v)
    if q.dtype not in _DTYPES or k.dtype != q.dtype or v.dtype != q.dtype:
        raise TypeError("q, k, v must share one dtype out of float32, bfloat16, float16")
    B, H, rq, dh = q.shape
    rk = k.shape[2]
    if out is None:
        out = torch.empty((B, rq, H, dh), dtype=q.dtype, device=q.device).permute(0, 2, 1, 3)
    d = PrefillDesc()
    d.dtype = _DTYPES[q.dtype]
    d.algo = algo
    d.batch, d.heads, d.head_dim = B, H, dh
    d.q_rows, d.k_rows = rq, rk
    d.window, d.n_persistent = window, n_persistent
    d.q_pos0 = q_pos0
    d.k_pos0 = n_persistent if k_pos0 is None else k_pos0
    d.scale = scale
    d.q_stride[:] = _bhrd_strides(q)
    d.k_stride[:] = _bhrd_strides(k)
    d.v_stride[:] = _bhrd_strides(v)
    d.o_stride[:] = _bhrd_strides(out)
    with torch.cuda.device(q.device):
        if halo_wait is not None:
            if lse is not None or window_block > 0:
                raise ValueError("halo_wait goes with the plain windowed prefill only")
            check(lib().tmw_prefill_halo(ctypes.byref(d), q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                         ctypes.byref(halo_wait), _stream_ptr(q.device)))
        elif lse is not None:
            if lse.dtype != torch.float32 or lse.numel() != B * H * rq or not lse.is_contiguous() or lse.device != q.device:
                raise ValueError("lse must be a contiguous fp32 tensor of B * H * rows elements on the same device")
            if window_block > 0:  # two planes: [B, H, rows - Np] then [B, H, Np]
                check(lib().tmw_prefill_block_sparse_lse(ctypes.byref(d), window_block, q.data_ptr(), k.data_ptr(),
                                                         v.data_ptr(), out.data_ptr(), lse.data_ptr(),
                                                         _stream_ptr(q.device)))
            else:
                check(lib().tmw_prefill_lse(ctypes.byref(d), q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                            lse.data_ptr(), _stream_ptr(q.device)))
        elif window_block > 0:
            check(lib().tmw_prefill_block_sparse(ctypes.byref(d), window_block, q.data_ptr(), k.data_ptr(),
                                                 v.data_ptr(), out.data_ptr(), _stream_ptr(q.device)))
        else:
            check(lib().tmw_prefill(ctypes.byref(d), q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                    _stream_ptr(q.device)))
    return out


def prefill_backward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, o: torch.Tensor, d_o: torch.Tensor,
                     lse: torch.Tensor, dq: torch.Tensor, dk: torch.Tensor, dv: torch.Tensor, window: int,
                     n_persistent: int, scale: float = 0.0, algo: int = ALGO_AUTO, window_block: int = 0) -> None:
    """``tmw_prefill_backward``: fills ``dq, dk, dv`` (same strides as ``q, k, v``) from ``d_o`` (same strides as
    ``o``), the saved output and the log-sum-exp of ``prefill(..., lse=...)``.  Whole sequences only."""
    _require_cuda(q, k, v, o, d_o, lse, dq, dk, dv)
    B, H, L, dh = q.shape
    for a, b_ in ((dq, q), (dk, k), (dv, v), (d_o, o)):
        if a.shape != b_.shape or a.stride() != b_.stride() or a.dtype != q.dtype:
            raise ValueError("dq, dk, dv, d_o must match q, k, v, o in shape, strides and dtype")
    if lse.dtype != torch.float32 or lse.numel() != B * H * L or not lse.is_contiguous():
        raise ValueError("lse must be the contiguous fp32 tensor that prefill(..., lse=...) filled")
    d = PrefillDesc()
    d.dtype = _DTYPES[q.dtype]
    d.algo = algo  # ALGO_SIMT pins the CUDA-core kernels, otherwise tensor cores for 16-bit types and head_dim 64 / 128
    d.batch, d.heads, d.head_dim = B, H, dh
    d.q_rows, d.k_rows = L, k.shape[2]
    d.window, d.n_persistent = window, n_persistent
    d.q_pos0, d.k_pos0, d.scale = 0, n_persistent, scale
    d.q_stride[:] = _bhrd_strides(q)
    d.k_stride[:] = _bhrd_strides(k)
    d.v_stride[:] = _bhrd_strides(v)
    d.o_stride[:] = _bhrd_strides(o)
    with torch.cuda.device(q.device):
        if window_block > 0:
            check(lib().tmw_prefill_block_sparse_backward(ctypes.byref(d), window_block, q.data_ptr(), k.data_ptr(),
                                                          v.data_ptr(), o.data_ptr(), d_o.data_ptr(), lse.data_ptr(),
                                                          dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                                          _stream_ptr(q.device)))
        else:
            check(lib().tmw_prefill_backward(ctypes.byref(d), q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                                             d_o.data_ptr(), lse.data_ptr(), dq.data_ptr(), dk.data_ptr(),
                                             dv.data_ptr(), _stream_ptr(q.device)))


def causal_dwconv(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``y[b, t, c] = sum_j weight[c, j] * x[b, t - (taps-1) + j, c]`` for ``x [B, T, C]`` contiguous and
    ``weight [C, taps]`` — the causal depthwise Conv1d of block_sparse_attention.py:241-256 without the
    transposes."""
    _require_cuda(x, weight)
    if x.dtype not in _DTYPES or weight.dtype != x.dtype or x.dim() != 3 or weight.dim() != 2:
        raise TypeError("causal_dwconv: x [B, T, C] and weight [C, taps] of one dtype out of fp32 / bf16 / fp16")
    if weight.shape[0] != x.shape[2]:
        raise ValueError("causal_dwconv: one filter per channel")
    x = x if x.is_contiguous() else x.contiguous()
    weight = weight if weight.is_contiguous() else weight.contiguous()
    y = torch.empty_like(x)
    B, T, C = x.shape
    if B == 0 or T == 0:
        return y
    with torch.cuda.device(x.device):
        check(lib().tmw_causal_dwconv(_DTYPES[x.dtype], B, T, C, weight.shape[1], x.data_ptr(), weight.data_ptr(),
                                      y.data_ptr(), _stream_ptr(x.device)))
    return y


class RingCache:
    """K/V ring of ``window + 1`` slots per (sequence, head) plus the batch-shared persistent K/V."""

    def __init__(self, batch: int, heads: int, head_dim: int, window: int, n_persistent: int,
                 dtype: torch.dtype, device: torch.device, scale: float = 0.0):
        if dtype not in _DTYPES:
            raise TypeError("dtype must be float32, bfloat16 or float16")
        if window < 0:
            raise ValueError(f"window_size must be non-negative, got {window}")
        self.batch, self.heads, self.head_dim = batch, heads, head_dim
        self.window, self.n_persistent = window, n_persistent
        self.slots = window + 1
        self.dtype, self.device, self.scale = dtype, torch.device(device), scale
        nbytes = lib().tmw_cache_ring_bytes(_DTYPES[dtype], batch, heads, head_dim, window)
        elems = nbytes // torch.empty((), dtype=dtype).element_size()
        assert elems == batch * heads * self.slots * head_dim
        self.k_ring = torch.zeros((batch, heads, self.slots, head_dim), dtype=dtype, device=device)
        self.v_ring = torch.zeros_like(self.k_ring)
        self.k_pers = torch.zeros((heads, n_persistent, head_dim), dtype=dtype, device=device)
        self.v_pers = torch.zeros_like(self.k_pers)
        # A handful of (sequence, head) pairs with a long window cannot fill the GPU with one CTA per pair:
        # then every pair's keys are split over several CTAs (tmw_decode_split) through a scratch buffer
        # owned by this object.  Measured on B200: it wins from about 2000 keys per pair and fewer pairs than
        # half the SMs; at window 512 the unsplit launch is faster for every batch size.
        self.splits = self.pick_splits(batch * heads, self.slots, self.device)
        self._scratch = None

    @staticmethod
    def pick_splits(pairs: int, slots: int, device) -> int:
        """0 = one CTA (or warp) per pair; otherwise the number of key ranges per pair."""
        sms = torch.cuda.get_device_properties(device).multi_processor_count if torch.cuda.is_available() else 148
        if pairs == 0 or 2 * pairs > sms or slots < 1024:
            return 0
        return max(2, min(MAX_DECODE_SPLITS, 2 * sms // pairs, slots // 128))

    def desc(self) -> CacheDesc:
        c = CacheDesc()
        c.dtype = _DTYPES[self.dtype]
        c.batch, c.heads, c.head_dim = self.batch, self.heads, self.head_dim
        c.window, c.n_persistent = self.window, self.n_persistent
        c.k_ring, c.v_ring = self.k_ring.data_ptr(), self.v_ring.data_ptr()
        c.k_pers = self.k_pers.data_ptr() if self.n_persistent > 0 else None
        c.v_pers = self.v_pers.data_ptr() if self.n_persistent > 0 else None
        c.scale = self.scale
        return c

    def set_persistent(self, k_pers: torch.Tensor, v_pers: torch.Tensor) -> None:
        """``[heads, Np, dh]`` keys/values of the persistent rows (identical for every sequence)."""
        self.k_pers.copy_(k_pers)
        self.v_pers.copy_(v_pers)

    def fill(self, k: torch.Tensor, v: torch.Tensor, t0: int = 0) -> None:
        """Load sequence K/V rows ``[B, H, rows, dh]`` (row i = token ``t0 + i``) into the ring."""
        _require_cuda(k, v)
        c = self.desc()
        ks = (ctypes.c_int64 * 3)(*_bhrd_strides(k))
        vs = (ctypes.c_int64 * 3)(*_bhrd_strides(v))
        with torch.cuda.device(self.device):
            check(lib().tmw_cache_fill(ctypes.byref(c), k.data_ptr(), v.data_ptr(), ks, vs, k.shape[2], t0,
                                       _stream_ptr(self.device)))

    def decode(self, q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, pos: torch.Tensor,
               out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One step: ``q, k_new, v_new [B, H, dh]``, ``pos [B] int32`` (token index of the new token)."""
        _require_cuda(q, k_new, v_new, pos)
        if pos.dtype != torch.int32:
            raise TypeError("pos must be int32")
        for t in (q, k_new, v_new):
            if t.stride(2) != 1:
                raise ValueError("the head_dim axis must be contiguous")
        if k_new.stride()[:2] != v_new.stride()[:2]:
            raise ValueError("k_new and v_new must share their strides")
        if out is None:
            out = torch.empty((self.batch, self.heads, self.head_dim), dtype=self.dtype, device=self.device)
        c = self.desc()
        qs = (ctypes.c_int64 * 2)(q.stride(0), q.stride(1))
        ns = (ctypes.c_int64 * 2)(k_new.stride(0), k_new.stride(1))
        os_ = (ctypes.c_int64 * 2)(out.stride(0), out.stride(1))
        with torch.cuda.device(self.device):
            if self.splits > 0:
                if self._scratch is None:
                    nbytes = lib().tmw_decode_split_scratch_bytes(ctypes.byref(c), self.splits)
                    self._scratch = torch.zeros(nbytes // 4, dtype=torch.float32, device=self.device)  # counters start at 0
                check(lib().tmw_decode_split(ctypes.byref(c), q.data_ptr(), k_new.data_ptr(), v_new.data_ptr(),
                                             out.data_ptr(), qs, ns, os_, pos.data_ptr(), self.splits,
                                             self._scratch.data_ptr(), self._scratch.numel() * 4,
                                             _stream_ptr(self.device)))
            else:
                check(lib().tmw_decode(ctypes.byref(c), q.data_ptr(), k_new.data_ptr(), v_new.data_ptr(),
                                       out.data_ptr(), qs, ns, os_, pos.data_ptr(), _stream_ptr(self.device)))
        return out


def causal_dwconv_backward(x: torch.Tensor, weight: torch.Tensor, dy: torch.Tensor):
    """Gradients of ``causal_dwconv``: returns ``(dx like x, dw [C, taps] in weight's dtype)``."""
    _require_cuda(x, weight, dy)
    x = x if x.is_contiguous() else x.contiguous()
    dy = dy if dy.is_contiguous() else dy.contiguous()
    weight = weight if weight.is_contiguous() else weight.contiguous()
    if dy.shape != x.shape or dy.dtype != x.dtype or weight.dtype != x.dtype:
        raise ValueError("causal_dwconv_backward: x, dy of one shape and dtype, weight of the same dtype")
    B, T, C = x.shape
    dx = torch.empty_like(x)
    dw = torch.zeros((C, weight.shape[1]), dtype=torch.float32, device=x.device)
    if B and T:
        with torch.cuda.device(x.device):
            check(lib().tmw_causal_dwconv_backward(_DTYPES[x.dtype], B, T, C, weight.shape[1], x.data_ptr(),
                                                   weight.data_ptr(), dy.data_ptr(), dx.data_ptr(), dw.data_ptr(),
                                                   _stream_ptr(x.device)))
    return dx, dw.to(weight.dtype)


def gelu_supported(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype in _DTYPES and x.numel() % 8 == 0 and x.is_contiguous()


def gelu(x: torch.Tensor, inplace: bool = False) -> torch.Tensor:
    """Exact (erf) GELU of a contiguous CUDA tensor — the nn.GELU() of titans_core/blocks/mlp.py:58-65."""
    _require_cuda(x)
    if x.dtype not in _DTYPES or not x.is_contiguous():
        raise TypeError("gelu: contiguous fp32 / bf16 / fp16 tensor expected")
    y = x if inplace else torch.empty_like(x)
    if x.numel() == 0:
        return y
    with torch.cuda.device(x.device):
        check(lib().tmw_gelu(_DTYPES[x.dtype], x.numel(), x.data_ptr(), y.data_ptr(), _stream_ptr(x.device)))
    return y


def enable_peer_access(device, peer_device) -> None:
    """Kernels running on ``device`` may then store into ``peer_device``'s memory (``tmw_enable_peer_access``)."""
    with torch.cuda.device(device):
        check(lib().tmw_enable_peer_access(torch.device(peer_device).index))


def ipc_export(t: torch.Tensor) -> bytes:
    """Description of the allocation behind a CUDA tensor for another process of this node (``tmw_ipc_export``)."""
    _require_cuda(t)
    mem = IpcMem()
    with torch.cuda.device(t.device):
        check(lib().tmw_ipc_export(t.data_ptr(), ctypes.byref(mem)))
    return bytes(mem)


def ipc_open(blob: bytes, device) -> int:
    """Address, valid for kernels running on ``device``, of the buffer another process exported (``tmw_ipc_open``)."""
    mem = IpcMem.from_buffer_copy(blob)
    out = ctypes.c_void_p()
    with torch.cuda.device(device):
        check(lib().tmw_ipc_open(ctypes.byref(mem), ctypes.byref(out)))
    return int(out.value)


def ipc_close_all() -> None:
    check(lib().tmw_ipc_close_all())


def halo_push(copies, device, wait_flag: int = 0, wait_value: int = 0, signal_flag: int = 0, signal_value: int = 0,
              wait_limit_cycles: int = 0) -> None:
    """``tmw_halo_push`` on the current stream of ``device``.  ``copies``: a list of ``(src_ptr, dst_ptr, nbytes)``
    (device addresses; ``dst`` may be a peer mapping); ``wait_flag`` / ``signal_flag``: device addresses of int32
    flags or 0.  More than ``HALO_MAX_COPIES`` copies are spread over several launches: the first one waits, the
    last one signals."""
    groups = [copies[i:i + HALO_MAX_COPIES] for i in range(0, len(copies), HALO_MAX_COPIES)] or [[]]
    with torch.cuda.device(device):
        for gi, group in enumerate(groups):
            arr = (HaloCopy * max(1, len(group)))()
            for j, (s, d_, n) in enumerate(group):
                arr[j].src, arr[j].dst, arr[j].bytes = s, d_, n
            first, last = gi == 0, gi == len(groups) - 1
            check(lib().tmw_halo_push(arr, len(group), wait_flag if first and wait_flag else None, wait_value,
                                      signal_flag if last and signal_flag else None, signal_value, wait_limit_cycles,
                                      _stream_ptr(device)))


def linear_supported(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether ``linear`` takes these operands: 16-bit CUDA tensors, rows of x contiguous, sizes multiples of 8."""
    return (x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and weight.dtype == x.dtype and x.dim() >= 2
            and weight.dim() == 2 and x.shape[-1] == weight.shape[1] and x.shape[-1] % 8 == 0
            and weight.shape[0] % 8 == 0 and weight.is_contiguous() and x.numel() > 0)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, gelu: bool = False,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ weight.T (+ bias)`` and, with ``gelu``, the exact GELU of that — ``torch.nn.functional.linear`` on
    the library's own tensor-core kernel (the projections of windowed_attention.py:295, 331 and the MLP of
    titans_core/blocks/mlp.py:58-65 with bias and activation in the epilogue)."""
    _require_cuda(x, weight)
    if not linear_supported(x, weight):
        raise TypeError("linear: bf16 / fp16 CUDA operands, contiguous weight [n, k], k and n multiples of 8")
    k, n = x.shape[-1], weight.shape[0]
    x2 = x.reshape(-1, k)
    if x2.stride(1) != 1 or x2.stride(0) % 8 != 0 or x2.data_ptr() % 16:
        x2 = x2.contiguous()
    if bias is not None:
        if bias.dtype != x.dtype or bias.shape != (n,) or not bias.is_cuda:
            raise TypeError("linear: bias must be a vector of n elements in the dtype of x")
        bias = bias if bias.is_contiguous() else bias.contiguous()
    m = x2.shape[0]
    if out is None:
        out = torch.empty(x.shape[:-1] + (n,), dtype=x.dtype, device=x.device)
    elif out.shape != x.shape[:-1] + (n,) or out.dtype != x.dtype or not out.is_contiguous():
        raise ValueError("linear: out must be contiguous, of x's dtype and shaped like x with n columns")
    desc = LinearDesc(dtype=_DTYPES[x.dtype], m=m, n=n, k=k, epilogue=EPILOGUE_GELU if gelu else EPILOGUE_NONE,
                      lda=x2.stride(0), ldw=weight.stride(0), ldc=n)
    with torch.cuda.device(x.device):
        check(lib().tmw_linear(ctypes.byref(desc), x2.data_ptr(), weight.data_ptr(),
                               bias.data_ptr() if bias is not None else None, out.data_ptr(),
                               _stream_ptr(x.device)))
    return out


# Products with at most this many rows (a decode step's: one row per sequence) stay with the library GEMM of
# torch.nn.functional.linear: they are launch- and latency-bound, and the tensor-core kernel above, built to
# stream tiles of 128 / 256 rows, measures about twice the library's few microseconds there.
LINEAR_MIN_ROWS = 257


def project(lin: "torch.nn.Linear", x: torch.Tensor, gelu: bool = False) -> torch.Tensor:
    """Forward of an ``nn.Linear`` (optionally followed by the exact GELU) on the inference path: the library's
    tensor-core kernel with bias and activation in its epilogue where it applies (16-bit CUDA operands, no
    gradient wanted, more rows than a decode step has), otherwise the module's own forward."""
    rows = x.numel() // x.shape[-1] if x.shape[-1] else 0
    if (rows >= LINEAR_MIN_ROWS and linear_supported(x, lin.weight)
            and (lin.bias is None or lin.bias.dtype == x.dtype)
            and not (torch.is_grad_enabled() and (x.requires_grad or lin.weight.requires_grad))):
        return linear(x, lin.weight, lin.bias, gelu=gelu)
    y = lin(x)
    if not gelu:
        return y
    if gelu_supported(y) and not (torch.is_grad_enabled() and y.requires_grad):
        return globals()["gelu"](y, inplace=True)
    return torch.nn.functional.gelu(y)


def add_rmsnorm_supported(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype in _DTYPES and x.shape[-1] % 8 == 0


def add_rmsnorm(x: torch.Tensor, residual: Optional[torch.Tensor], scale: torch.Tensor, eps: float,
                inplace_sum: bool = False):
    """``h = x + residual`` (``residual`` may be None), ``y = h / sqrt(mean(h^2) + eps) * scale`` in one
    pass (RMSNorm of titans_core/blocks/norms.py:55-58 with the residual add of titan_block.py:94-100
    folded in).  Returns ``(h, y)``; ``h`` is ``x`` itself when there is no residual, and is written into
    ``x`` when ``inplace_sum``."""
    _require_cuda(x, scale)
    dim = x.shape[-1]
    if x.dtype not in _DTYPES or scale.dtype != x.dtype or scale.shape != (dim,):
        raise TypeError("add_rmsnorm: fp32 / bf16 / fp16 rows and a scale vector of the same type and length")
    x = x if x.is_contiguous() else x.contiguous()
    scale = scale if scale.is_contiguous() else scale.contiguous()
    if residual is not None:
        if residual.shape != x.shape or residual.dtype != x.dtype or residual.device != x.device:
            raise ValueError("add_rmsnorm: x and residual must agree in shape, dtype and device")
        residual = residual if residual.is_contiguous() else residual.contiguous()
    y = torch.empty_like(x)
    h = x if (residual is None or inplace_sum) else torch.empty_like(x)
    rows = x.numel() // dim if dim else 0
    if rows == 0:  # nothing to do (and an empty tensor has no address to pass)
        return h, y
    with torch.cuda.device(x.device):
        check(lib().tmw_add_rmsnorm(_DTYPES[x.dtype], rows, dim, x.data_ptr(),
                                    residual.data_ptr() if residual is not None else None, scale.data_ptr(),
                                    float(eps), h.data_ptr() if residual is not None else None, y.data_ptr(),
                                    _stream_ptr(x.device)))
    return h, y


def poll_status(device: Optional[torch.device] = None) -> None:
    """Synchronise the current stream and raise if a kernel reported an expired bounded wait."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        check(lib().tmw_poll_status(_stream_ptr(dev)))


def default_scale(head_dim: int) -> float:
    return 1.0 / math.sqrt(head_dim)
