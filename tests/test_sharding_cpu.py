"""Host-side logic of the multi-GPU wrappers, run as two gloo ranks on CPU: column ranges and slices, the count
exchange, the row all-to-all, the regrouping permutation and the way back.  The per-rank compute is the numpy oracle
(tests may use it as the checker), so what is verified is that sharded == unsharded."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import kquant as kq
from quactlize_b200 import sharding, synth

WORLD = 2


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(fn, *args):
    port = _free_port()
    mp.spawn(_entry, args=(port, fn, args), nprocs=WORLD, join=True)


def _entry(rank, port, fn, args):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    try:
        fn(rank, *args)
    finally:
        dist.destroy_process_group()


def test_column_range_covers_everything():
    for n, world, mult in ((4096, 8, 1), (14336, 8, 256), (768, 4, 256), (10, 4, 1)):
        spans = [sharding.column_range(n, r, world, mult) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert all((hi - lo) % mult == 0 for lo, hi in spans)
        assert max(hi - lo for lo, hi in spans) - min(hi - lo for lo, hi in spans) <= mult
    with pytest.raises(ValueError):
        sharding.column_range(100, 0, 2, 256)
    with pytest.raises(ValueError):
        sharding.expert_range(10, 0, 4)


def _column_parallel(rank, qtype):
    n, k = 96, 512
    blocks = synth.kquant_blocks(qtype, n * k // 256, seed=5)
    x = synth.activations(1, k, seed=6)
    full = kq.vecdot_dense(blocks, x, n, k, qtype)
    mine = sharding.shard_blocks(torch.from_numpy(blocks), n, k, rank, WORLD)
    lo, hi = sharding.column_range(n, rank, WORLD)
    y = torch.from_numpy(kq.vecdot_dense(mine.numpy(), x, hi - lo, k, qtype).astype(np.float32)).reshape(1, -1)
    got = sharding.gather_columns(y, n)
    assert np.array_equal(got.numpy().reshape(-1), np.asarray(full, dtype=np.float32).reshape(-1))
    # planes and units slice along their own n axes to the same columns
    low, high, scale, zero = kq.prepare_gemv(blocks, n, k, qtype)
    sl = sharding.shard_planes([torch.from_numpy(np.ascontiguousarray(t)) for t in (low, high, scale, zero)], [1, 1, 2, 2], n, rank, WORLD)
    w_full = kq.gemv_artifact_dequantize(low, high, scale, zero, qtype).reshape(n, k)
    w_mine = kq.gemv_artifact_dequantize(*[t.numpy() for t in sl], qtype).reshape(hi - lo, k)
    assert np.array_equal(w_mine, w_full[lo:hi])


@pytest.mark.parametrize("qt", [12, 14])
def test_column_parallel_two_ranks(qt):
    _run(_column_parallel, qt)


def _expert_parallel(rank, uneven):
    experts, n, k, qtype = 4, 32, 256, 12
    blocks = synth.kquant_blocks(qtype, experts * n * k // 256, seed=9).reshape(experts, n * k // 256, -1)
    w = np.stack([kq.dequantize_f32(blocks[e], qtype).reshape(n, k) for e in range(experts)])
    rng = np.random.default_rng(100 + rank)
    counts = rng.integers(0, 6, size=experts)
    if uneven:
        counts[rank] = 0                                   # an expert nobody on this rank routes to
        if rank == 1:
            counts[:] = 0                                  # a rank with no rows at all
    rows = int(counts.sum())
    a = rng.normal(size=(rows, k)).astype(np.float32)
    owner = np.repeat(np.arange(experts), counts)
    want = np.stack([a[i] @ w[owner[i]].T for i in range(rows)]) if rows else np.zeros((0, n), np.float32)
    lo, hi = sharding.expert_range(experts, rank, WORLD)
    w_local = w[lo:hi]

    def compute(rows_t, offsets, max_rows):
        off = offsets.numpy()
        assert off[0] == 0 and off[-1] == rows_t.shape[0] and max_rows == (np.diff(off).max() if len(off) > 1 else 0)
        out = np.zeros((rows_t.shape[0], n), np.float32)
        for j in range(hi - lo):
            out[off[j]:off[j + 1]] = rows_t.numpy()[off[j]:off[j + 1]] @ w_local[j].T
        return torch.from_numpy(out)

    plan = sharding.plan_dispatch(torch.from_numpy(counts), experts)
    got = sharding.expert_parallel_apply(torch.from_numpy(a), torch.from_numpy(counts), experts, n, compute, plan=plan)
    assert got.shape == (rows, n)
    assert np.allclose(got.numpy(), want, rtol=1e-5, atol=1e-5)
    mine, ratio = sharding.imbalance(plan)
    assert mine == sum(plan.recv_rows) and ratio >= 1.0
    with pytest.raises(ValueError):
        sharding.plan_dispatch(torch.from_numpy(counts[:-1]), experts)


@pytest.mark.parametrize("uneven", [False, True])
def test_expert_parallel_two_ranks(uneven):
    _run(_expert_parallel, uneven)
