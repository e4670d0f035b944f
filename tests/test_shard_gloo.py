"""Sequence sharding on CPU ranks (gloo): halo planning, the exchange itself, and that attention over each
rank's [persistent | halo | own] buffers reproduces the unsharded rows (checked with the plain-C oracle)."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import c_oracle
from oracle import windowed_oracle as wo
from titanmac_b200 import shard


def test_bounds_and_plan():
    b = shard.shard_bounds(16 + 100, 16, 4)
    assert b == [(0, 41), (41, 66), (66, 91), (91, 116)]
    assert shard.shard_bounds(5 + 7, 5, 3) == [(0, 8), (8, 10), (10, 12)]
    with pytest.raises(ValueError):
        shard.shard_bounds(16, 16, 2)
    # window shorter than a block: one neighbour each
    plan = shard.plan_halo(b, 10, 16)
    assert [(t.src, t.dst, t.src_row0, t.rows, t.dst_offset) for t in plan] == [
        (0, 1, 31, 10, 0), (1, 2, 56, 10, 0), (2, 3, 81, 10, 0)]
    # window longer than a block: rank 3 needs rows from ranks 1 and 2 (and the clip at Np for rank 1)
    plan = shard.plan_halo(b, 40, 16)
    got = {(t.src, t.dst): (t.src_row0, t.rows, t.dst_offset) for t in plan}
    assert got[(0, 1)] == (16, 25, 0)
    assert got[(0, 2)] == (26, 15, 0) and got[(1, 2)] == (41, 25, 15)
    assert got[(1, 3)] == (51, 15, 0) and got[(2, 3)] == (66, 25, 15)
    assert (0, 3) not in got
    assert shard.halo_rows(b, 3, 40, 16) == 40 and shard.halo_rows(b, 1, 40, 16) == 25
    with pytest.raises(ValueError):
        shard.plan_halo(b, -1, 16)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, L, w, Np, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        q, k, v = wo.qkv_inputs(1, 2, L, 16, seed=7)
        bounds = shard.shard_bounds(L, Np, world)
        r0, r1 = bounds[rank]
        kv = shard.ShardedKV(k[:, :, r0:r1].clone(), v[:, :, r0:r1].clone(), L, w, Np)
        kv.exchange()
        halo = shard.halo_rows(bounds, rank, w, Np)
        if rank == 0:
            want_k = k[:, :, :r1]
        else:
            want_k = torch.cat([k[:, :, :Np], k[:, :, r0 - halo:r1]], dim=2)
        assert torch.equal(kv.k, want_k), f"rank {rank}: K buffer differs"
        # the buffers made first and filled in place by the producer end up the same
        kv2 = shard.ShardedKV.allocate(1, 2, 16, L, w, Np, k.dtype, "cpu")
        kv2.k_own.copy_(k[:, :, r0:r1])
        kv2.v_own.copy_(v[:, :, r0:r1])
        kv2.exchange()
        assert torch.equal(kv2.k, kv.k) and torch.equal(kv2.v, kv.v), f"rank {rank}: allocate() path differs"
        assert (kv2.q_pos0, kv2.k_pos0, kv2.own_offset) == (kv.q_pos0, kv.k_pos0, kv.own_offset)
        assert kv.q_pos0 == r0 and kv.k_pos0 == (Np if rank == 0 else r0 - halo)
        o = c_oracle.attention(q[:, :, r0:r1], kv.k, kv.v, w, Np, q_pos0=kv.q_pos0, k_pos0=kv.k_pos0)
        np.save(os.path.join(out_dir, f"o{rank}.npy"), o)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,L,w,Np", [(2, 4 + 60, 9, 4), (3, 3 + 50, 30, 3), (2, 40, 5, 0)])
def test_exchange_and_sharded_attention_match_unsharded(tmp_path, world, L, w, Np):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, L, w, Np, str(tmp_path)), nprocs=world, join=True)
    q, k, v = wo.qkv_inputs(1, 2, L, 16, seed=7)
    full = wo.attention_core_dense(q, k, v, w, Np).numpy()
    got = np.concatenate([np.load(tmp_path / f"o{r}.npy") for r in range(world)], axis=2)
    assert got.shape == full.shape
    assert np.abs(got - full).max() <= 2e-6
