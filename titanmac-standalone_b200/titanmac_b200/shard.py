"""Sequence-sharded prefill: contiguous row blocks per rank, one K/V halo from the left.

The reference has no distributed code; this is the multi-GPU form of its attention
core for contexts that do not fit (or are too slow on) one GPU.  Rows are counted
over the whole length ``L = Np + T`` like in the module (the first ``Np`` rows are
the persistent rows, titans_core/attn/windowed_attention.py:113-118).  Rank 0 owns
rows ``[0, Np + T_0)``, rank ``r > 0`` owns a block of sequence rows.  A sequence row
``i`` needs the keys ``max(Np, i - w) .. i`` (windowed_attention.py:136-150) and the
``Np`` persistent keys, so a rank needs from its left neighbours only the ``w`` rows
before its first row, plus the persistent K/V from rank 0.

Everything lands in the rank's own HBM first — a K and a V buffer laid out as
``[persistent | halo | own rows]`` — and is then read by ordinary per-CTA TMA loads;
nothing is read from a peer's memory by the attention kernel.  The buffers are stored
row-major (``[B, rows, H, dh]``, the layout of the projection output), so a halo is a
contiguous range that is sent and received in place, all transfers of a step in one batch.
Optionally (``overlap=True``) the rows whose window lies inside the rank's own block are
launched before the halo arrives (on a side stream), the first ``w`` rows after it.

The planning and the exchange work on CPU tensors with the ``gloo`` backend as well
(that is how they are tested without GPUs); the attention calls need CUDA.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def shard_bounds(total_rows: int, n_persistent: int, world: int) -> List[Tuple[int, int]]:
    """Row ranges ``[r0, r1)`` per rank: the ``T = total_rows - Np`` sequence rows are split as evenly
    as possible into contiguous blocks; rank 0's block also contains the ``Np`` persistent rows."""
    if n_persistent >= total_rows:
        raise ValueError(f"num_persistent_tokens ({n_persistent}) must be < seq_len ({total_rows})")
    T = total_rows - n_persistent
    base, rem = divmod(T, world)
    bounds, start = [], n_persistent
    for r in range(world):
        n = base + (1 if r < rem else 0)
        bounds.append((0 if r == 0 else start, start + n))
        start += n
    return bounds


@dataclass(frozen=True)
class Transfer:
    src: int          # sending rank
    dst: int          # receiving rank
    src_row0: int     # first row (whole-length numbering) sent
    rows: int
    dst_offset: int   # row offset inside the receiver's halo region


def plan_halo(bounds: Sequence[Tuple[int, int]], window: int, n_persistent: int) -> List[Transfer]:
    """All halo transfers of one exchange.  Rank ``r > 0`` receives rows ``[max(Np, r0 - w), r0)``,
    which may span several left neighbours when a block is shorter than the window."""
    if window < 0:
        raise ValueError(f"window_size must be non-negative, got {window}")
    out: List[Transfer] = []
    for dst in range(1, len(bounds)):
        r0 = bounds[dst][0]
        lo = max(n_persistent, r0 - window)
        for src in range(dst):
            s0, s1 = max(bounds[src][0], lo), min(bounds[src][1], r0)
            if s1 > s0:
                out.append(Transfer(src, dst, s0, s1 - s0, s0 - lo))
    return out


def halo_rows(bounds: Sequence[Tuple[int, int]], rank: int, window: int, n_persistent: int) -> int:
    if rank == 0:
        return 0
    r0 = bounds[rank][0]
    return r0 - max(n_persistent, r0 - window)


class ShardedKV:
    """This rank's K/V buffers ``[B, H, Np + halo + own, dh]`` (views of row-major storage, so that every
    transfer is in place) and the positions that go with them.

    ``ShardedKV(k_own, v_own, ...)`` copies the rank's rows into fresh buffers.  ``ShardedKV.allocate(...)``
    only makes the buffers: the producer of K and V (the QKV projection) then writes this rank's rows straight
    into ``k_own`` / ``v_own`` — views of the buffers — and no copy of the rank's 2 x own x H x dh elements is
    made per call.
    """

    def __init__(self, k_own: torch.Tensor, v_own: torch.Tensor, total_rows: int, window: int, n_persistent: int,
                 group: Optional[dist.ProcessGroup] = None):
        B, H, _, dh = k_own.shape
        self._layout(total_rows, window, n_persistent, group)
        if k_own.shape[2] != self.r1 - self.r0 or v_own.shape != k_own.shape:
            raise ValueError(f"rank {self.rank} must hold rows [{self.r0}, {self.r1}) of K and V")
        self._buffers(B, H, dh, k_own.dtype, k_own.device)
        self.k[:, :, self.own_offset:] = k_own
        self.v[:, :, self.own_offset:] = v_own

    @classmethod
    def allocate(cls, batch: int, heads: int, head_dim: int, total_rows: int, window: int, n_persistent: int,
                 dtype: torch.dtype, device, group: Optional[dist.ProcessGroup] = None) -> "ShardedKV":
        self = cls.__new__(cls)
        self._layout(total_rows, window, n_persistent, group)
        self._buffers(batch, heads, head_dim, dtype, device)
        return self

    def _layout(self, total_rows: int, window: int, n_persistent: int, group) -> None:
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.window, self.n_persistent, self.total_rows = window, n_persistent, total_rows
        self.bounds = shard_bounds(total_rows, n_persistent, self.world)
        self.r0, self.r1 = self.bounds[self.rank]
        self.halo = halo_rows(self.bounds, self.rank, window, n_persistent)
        # rank 0: buffer == own rows (they start with the persistent rows); rank r > 0: [persistent | halo | own]
        self.own_offset = 0 if self.rank == 0 else n_persistent + self.halo
        self.k_pos0 = n_persistent if self.rank == 0 else self.r0 - self.halo  # position of buffer row Np
        self.q_pos0 = self.r0

    def _buffers(self, B: int, H: int, dh: int, dtype: torch.dtype, device) -> None:
        # Stored row-major, [B, rows, H, dh], like the output of the QKV projection: a range of rows of one
        # batch element is then one contiguous piece of memory that can be sent and received in place.
        # self.k / self.v are the [B, H, rows, dh] views the attention kernel takes.
        rows = self.own_offset + (self.r1 - self.r0)
        self._k_rows = torch.empty((B, rows, H, dh), dtype=dtype, device=device)
        self._v_rows = torch.empty((B, rows, H, dh), dtype=dtype, device=device)
        self.k = self._k_rows.permute(0, 2, 1, 3)
        self.v = self._v_rows.permute(0, 2, 1, 3)

    def _pieces(self, a: int, rows: int):
        """Contiguous views of buffer rows ``[a, a + rows)``: K then V of every batch element."""
        return [t[b, a:a + rows] for t in (self._k_rows, self._v_rows) for b in range(t.shape[0])]

    @property
    def k_own(self) -> torch.Tensor:
        return self.k[:, :, self.own_offset:]

    @property
    def v_own(self) -> torch.Tensor:
        return self.v[:, :, self.own_offset:]

    def exchange(self) -> None:
        """Persistent K/V from rank 0 and the halo rows from the left neighbours, into this rank's buffers:
        one batch of in-place sends and receives."""
        self._run(self._persistent_ops() + self._halo_ops())

    def exchange_persistent(self) -> None:
        self._run(self._persistent_ops())

    def exchange_halo(self) -> None:
        self._run(self._halo_ops())

    def _run(self, ops) -> None:
        if ops:
            for req in dist.batch_isend_irecv(ops):
                req.wait()

    def _persistent_ops(self):
        """Rank 0 sends its first ``Np`` rows to every other rank (they land in rows ``[0, Np)`` there)."""
        Np, ops = self.n_persistent, []
        if Np == 0 or self.world == 1:
            return ops
        if self.rank == 0:
            for dst in range(1, self.world):
                ops += [dist.P2POp(dist.isend, t, self._global(dst), group=self.group) for t in self._pieces(0, Np)]
        else:
            ops += [dist.P2POp(dist.irecv, t, self._global(0), group=self.group) for t in self._pieces(0, Np)]
        return ops

    def _halo_ops(self):
        Np, ops = self.n_persistent, []
        for tr in plan_halo(self.bounds, self.window, Np):
            if tr.src == self.rank:
                a = self.own_offset + (tr.src_row0 - self.r0)
                ops += [dist.P2POp(dist.isend, t, self._global(tr.dst), group=self.group)
                        for t in self._pieces(a, tr.rows)]
            elif tr.dst == self.rank:
                ops += [dist.P2POp(dist.irecv, t, self._global(tr.src), group=self.group)
                        for t in self._pieces(Np + tr.dst_offset, tr.rows)]
        return ops

    def _global(self, group_rank: int) -> int:
        return dist.get_global_rank(self.group, group_rank) if self.group is not None else group_rank


_side_streams = {}


def _side_stream(device: torch.device) -> "torch.cuda.Stream":
    key = (device.type, device.index)
    if key not in _side_streams:
        _side_streams[key] = torch.cuda.Stream(device)
    return _side_streams[key]


def sharded_prefill(q_own: torch.Tensor, k_own: Optional[torch.Tensor], v_own: Optional[torch.Tensor],
                    total_rows: int, window: int, n_persistent: int, group: Optional[dist.ProcessGroup] = None,
                    overlap: bool = False, algo: int = 0, kv: Optional[ShardedKV] = None) -> torch.Tensor:
    """Attention output for this rank's rows (``[B, H, own, dh]``), CUDA only.

    ``q_own, k_own, v_own``: ``[B, H, r1 - r0, dh]`` — this rank's rows of the whole-length tensors
    (rank 0's block starts with the persistent rows).  With ``kv`` (from :meth:`ShardedKV.allocate`, its
    ``k_own`` / ``v_own`` views already filled) ``k_own`` and ``v_own`` are ignored and nothing is copied.

    ``overlap=False``: one batch of sends / receives, then one launch (measured best for halos of a few MB:
    0.915 ms against 0.927 ms per step on two GPUs at 131 072 rows).  ``overlap=True``: the persistent rows
    first, then the rows that need no halo on a side stream while the halo travels, then the first
    ``window`` rows - for halos large enough that the transfer shows.
    """
    from . import _native

    if kv is None:
        kv = ShardedKV(k_own, v_own, total_rows, window, n_persistent, group)
    B, H, own, dh = q_own.shape
    out = torch.empty((B, own, H, dh), dtype=q_own.dtype, device=q_own.device).permute(0, 2, 1, 3)
    # rows whose window needs the halo: the first `window` rows of ranks > 0
    need_halo = min(own, window) if kv.rank > 0 else 0
    if not overlap or need_halo == 0 or need_halo == own:
        kv.exchange()
        _native.prefill(q_own, kv.k, kv.v, window, n_persistent, out=out, q_pos0=kv.q_pos0, k_pos0=kv.k_pos0, algo=algo)
        return out
    kv.exchange_persistent()  # 2 * B * H * Np * dh elements: needed by every row, so it goes first
    main = torch.cuda.current_stream(q_own.device)
    side = _side_stream(q_own.device)
    side.wait_stream(main)
    with torch.cuda.stream(side):  # interior rows: every key they need is already in this rank's block
        _native.prefill(q_own[:, :, need_halo:], kv.k, kv.v, window, n_persistent, out=out[:, :, need_halo:],
                        q_pos0=kv.q_pos0 + need_halo, k_pos0=kv.k_pos0, algo=algo)
    kv.exchange_halo()
    _native.prefill(q_own[:, :, :need_halo], kv.k, kv.v, window, n_persistent, out=out[:, :, :need_halo],
                    q_pos0=kv.q_pos0, k_pos0=kv.k_pos0, algo=algo)
    main.wait_stream(side)
    return out


# ------------------------------------------------------------------------------------------------------------
# The same step without a host-side collective: producers push, the attention kernel polls
# ------------------------------------------------------------------------------------------------------------
class _PeerBuffers:
    """Addresses (valid for kernels on this rank's GPU) of another rank's K rows, V rows and flag words, and the
    number of rows of its buffers."""

    def __init__(self, k_addr: int, v_addr: int, flags_addr: int, rows: int):
        self.k, self.v, self.flags, self.rows = k_addr, v_addr, flags_addr, rows


class PeerShardedKV(ShardedKV):
    """``ShardedKV`` whose persistent and halo regions are written by the OTHER ranks' GPUs.

    Every rank maps the buffers and flag words of the ranks it writes to (``tmw_ipc_export`` / ``tmw_ipc_open``,
    once at set-up; one process per GPU on one node).  A step is then, on each rank's stream and with no host-side collective:

      1. ``push()``     - the rank's last ``window`` rows of K and V go into the right neighbour's halo region
                          and (rank 0) the persistent rows into every other rank's buffer: ``tmw_halo_push``,
                          plain stores through the peer mapping, then a release store of the step number to the
                          destination's "ready" flag.  A push first waits until the destination has acknowledged
                          the previous step (it may still be reading the rows about to be overwritten).
      2. the attention launch with ``wait()`` - ``tmw_prefill_halo`` polls the ready flags right before the first
                          TMA load that touches pushed rows; tiles whose window is local start at once.
      3. ``ack()``      - after the attention kernel (stream order) the rank tells its producers that the step's
                          rows have been read.

    Restricted to shards at least one window long (the halo then comes from exactly one neighbour); shorter
    shards use the collective form (``ShardedKV.exchange``).  All device-side waits are bounded and surface
    as ``TMW_ERR_DEVICE_TIMEOUT`` through ``_native.poll_status``.
    """

    # flag words in every rank's own memory
    READY_PERS, READY_HALO, ACK_HALO, ACK_PERS0 = 0, 1, 2, 3  # ACK_PERS0 + d: rank d has read the persistent rows

    @classmethod
    def allocate(cls, batch: int, heads: int, head_dim: int, total_rows: int, window: int, n_persistent: int,
                 dtype: torch.dtype, device, group: Optional[dist.ProcessGroup] = None,
                 wait_limit_cycles: int = 0) -> "PeerShardedKV":
        self = cls.__new__(cls)
        self._layout(total_rows, window, n_persistent, group)
        for r in range(1, self.world):
            if halo_rows(self.bounds, r, window, n_persistent) > self.bounds[r - 1][1] - max(self.bounds[r - 1][0],
                                                                                            n_persistent):
                raise ValueError("PeerShardedKV needs shards of at least `window` rows (one halo source per rank)")
        self._buffers(batch, heads, head_dim, dtype, device)
        self.device = torch.device(device)
        self.wait_limit_cycles = wait_limit_cycles
        self.flags = torch.zeros(self.ACK_PERS0 + self.world, dtype=torch.int32, device=device)
        self.step = 0
        # exchange the mappings: every rank publishes its two buffers and its flags (tmw_ipc_export), and maps
        # those of the ranks it writes to with its own GPU current (tmw_ipc_open)
        from . import _native

        mine = (_native.ipc_export(self._k_rows), _native.ipc_export(self._v_rows), _native.ipc_export(self.flags),
                self._k_rows.shape[1])
        everyone = [None] * self.world
        dist.all_gather_object(everyone, mine, group=group)
        self._peer = {}
        need = set()
        if self.rank + 1 < self.world:
            need.add(self.rank + 1)           # halo goes to the right neighbour
        if self.rank > 0:
            need.update({self.rank - 1, 0})   # acknowledgements go to the left neighbour and to rank 0
        if self.rank == 0:
            need.update(range(1, self.world))  # persistent rows go to everyone
        for r in sorted(need):
            kb, vb, fb, rows = everyone[r]
            self._peer[r] = _PeerBuffers(_native.ipc_open(kb, self.device), _native.ipc_open(vb, self.device),
                                         _native.ipc_open(fb, self.device), rows)
        dist.barrier(group=group)
        return self

    def close(self) -> None:
        """Collective: every rank drops its mappings of the others' memory before anybody frees its own."""
        from . import _native

        torch.cuda.synchronize(self.device)
        self._peer.clear()
        _native.ipc_close_all()
        dist.barrier(group=self.group)

    def push(self) -> None:
        from . import _native

        self.step += 1
        e, Np = self.step, self.n_persistent
        row_bytes = self._k_rows.shape[2] * self._k_rows.shape[3] * self._k_rows.element_size()
        B, my_rows = self._k_rows.shape[0], self._k_rows.shape[1]
        my_flags = self.flags.data_ptr()

        def copies(dst: _PeerBuffers, src_row: int, dst_row: int, n: int):
            # buffer rows [src_row, src_row + n) of every batch element of K and V -> the destination's rows
            # [dst_row, dst_row + n)
            return [(base.data_ptr() + (b * my_rows + src_row) * row_bytes,
                     dst_base + (b * dst.rows + dst_row) * row_bytes, n * row_bytes)
                    for base, dst_base in ((self._k_rows, dst.k), (self._v_rows, dst.v)) for b in range(B)]

        if self.rank + 1 < self.world:
            dst = self._peer[self.rank + 1]
            n = halo_rows(self.bounds, self.rank + 1, self.window, Np)
            _native.halo_push(copies(dst, my_rows - n, Np, n), self.device,
                              wait_flag=my_flags + 4 * self.ACK_HALO, wait_value=e - 1,
                              signal_flag=dst.flags + 4 * self.READY_HALO, signal_value=e,
                              wait_limit_cycles=self.wait_limit_cycles)
        if self.rank == 0 and Np > 0:
            for d in range(1, self.world):
                dst = self._peer[d]
                _native.halo_push(copies(dst, 0, 0, Np), self.device,
                                  wait_flag=my_flags + 4 * (self.ACK_PERS0 + d), wait_value=e - 1,
                                  signal_flag=dst.flags + 4 * self.READY_PERS, signal_value=e,
                                  wait_limit_cycles=self.wait_limit_cycles)

    def wait(self):
        """The ``halo_wait`` argument of ``_native.prefill`` for the current step (None on rank 0)."""
        from . import _native

        if self.rank == 0:
            return None
        w = _native.HaloWait()
        w.pers_flag = self.flags.data_ptr() + 4 * self.READY_PERS if self.n_persistent > 0 else None
        w.halo_flag = self.flags.data_ptr() + 4 * self.READY_HALO if self.halo > 0 else None
        w.value, w.halo_rows, w.wait_limit_cycles = self.step, self.halo, self.wait_limit_cycles
        return w

    def ack(self) -> None:
        from . import _native

        if self.rank == 0:
            return
        e = self.step
        if self.halo > 0:
            _native.halo_push([], self.device, signal_flag=self._peer[self.rank - 1].flags + 4 * self.ACK_HALO,
                              signal_value=e)
        if self.n_persistent > 0:
            _native.halo_push([], self.device, signal_flag=self._peer[0].flags + 4 * (self.ACK_PERS0 + self.rank),
                              signal_value=e)


def pushed_prefill(q_own: torch.Tensor, kv: PeerShardedKV, algo: int = 0) -> torch.Tensor:
    """Attention output for this rank's rows with the halo pushed by the neighbours' GPUs: push, one attention
    launch that polls the flags, acknowledgement.  ``kv.k_own`` / ``kv.v_own`` hold this rank's rows."""
    from . import _native

    B, H, own, dh = q_own.shape
    out = torch.empty((B, own, H, dh), dtype=q_own.dtype, device=q_own.device).permute(0, 2, 1, 3)
    kv.push()
    _native.prefill(q_own, kv.k, kv.v, kv.window, kv.n_persistent, out=out, q_pos0=kv.q_pos0, k_pos0=kv.k_pos0,
                    algo=algo, halo_wait=kv.wait())
    kv.ack()
    return out
