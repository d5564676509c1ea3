"""Host-side logic of the expert-parallel step on CPU: the route plan (pure index arithmetic, the same function the GPU
path runs on device tensors) for several simulated ranks, and its count exchange between two real gloo ranks."""
import os
import socket
import subprocess
import sys
import textwrap

import numpy as np
import pytest
import torch

from conftest import ROOT
from quactlize_b200 import ep


@pytest.mark.parametrize("world,experts,top_k,tokens", [(1, 8, 2, 50), (2, 8, 2, 64), (4, 8, 2, 33), (8, 128, 8, 16), (4, 128, 8, 1)])
def test_plan_routes_places_every_route_once_expert_major(world, experts, top_k, tokens):
    rng = np.random.default_rng(world * 1000 + experts + tokens)
    per = experts // world
    routes = [torch.from_numpy(np.argsort(rng.random((tokens + r, experts)), axis=1)[:, :top_k].reshape(-1).astype(np.int64)) for r in range(world)]
    counts_all = torch.stack([torch.bincount(f, minlength=experts) for f in routes]).to(torch.int32)
    tot = counts_all.sum(0)
    seen = [dict() for _ in range(world)]                       # owner -> {position: (source rank, expert, item index)}
    for r in range(world):
        order, dst_rank, dst_pos, local_off = ep.plan_routes(routes[r], counts_all, r)
        es = routes[r][order]
        assert bool((es[1:] >= es[:-1]).all())                   # items go out sorted by expert, i.e. by destination rank
        assert torch.equal(dst_rank.long(), es // per)
        assert local_off.dtype == torch.int32 and local_off.tolist() == [0] + tot[r * per:(r + 1) * per].cumsum(0).tolist()
        for i in range(order.numel()):
            o, p = int(dst_rank[i]), int(dst_pos[i])
            assert p not in seen[o]
            seen[o][p] = (r, int(es[i]), i)
    for o in range(world):
        total = int(tot[o * per:(o + 1) * per].sum())
        assert sorted(seen[o]) == list(range(total))            # a permutation: every row of the owner's buffer written once
        keys = [seen[o][p] for p in range(total)]
        assert keys == sorted(keys, key=lambda t: (t[1], t[0], t[2]))   # expert-major, then source rank, then the source's order


def test_plan_routes_with_idle_ranks_and_empty_experts():
    counts_all = torch.tensor([[3, 0, 0, 1], [0, 0, 0, 0]], dtype=torch.int32)
    order, dst_rank, dst_pos, local_off = ep.plan_routes(torch.tensor([3, 0, 0, 0]), counts_all, 0)
    assert order.tolist() == [1, 2, 3, 0] and dst_rank.tolist() == [0, 0, 0, 1] and dst_pos.tolist() == [0, 1, 2, 0]
    assert local_off.tolist() == [0, 3, 3]
    order, dst_rank, dst_pos, local_off = ep.plan_routes(torch.zeros(0, dtype=torch.int64), counts_all, 1)
    assert order.numel() == 0 and local_off.tolist() == [0, 0, 1]


CHILD = textwrap.dedent('''
    import os, sys, torch, torch.distributed as dist
    sys.path.insert(0, os.environ["QB_ROOT"])
    from quactlize_b200 import ep
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    experts, top_k = 8, 2
    g = torch.Generator().manual_seed(5 + rank)
    routes = torch.stack([torch.randperm(experts, generator=g)[:top_k] for _ in range(20 + 7 * rank)])
    flat = routes.reshape(-1)
    counts = torch.bincount(flat, minlength=experts).to(torch.int32)
    counts_all = torch.empty(world * experts, dtype=torch.int32)
    dist.all_gather_into_tensor(counts_all, counts)
    counts_all = counts_all.view(world, experts)
    order, dst_rank, dst_pos, local_off = ep.plan_routes(flat, counts_all, rank)
    # every rank tells every owner what it will write; owners check they are covered exactly once
    mine = [(int(dst_rank[i]), int(dst_pos[i])) for i in range(order.numel())]
    everyone = [None] * world
    dist.all_gather_object(everyone, mine)
    rows_here = sorted(p for lst in everyone for (o, p) in lst if o == rank)
    assert rows_here == list(range(int(local_off[-1]))), (rank, rows_here[:5], int(local_off[-1]))
    dist.barrier()
    if rank == 0:
        print("EP_PLAN_OK")
''')


def test_count_exchange_and_plan_between_two_gloo_ranks():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    import tempfile
    with tempfile.NamedTemporaryFile("w", suffix=".py", delete=False) as f:      # torchrun wants a script path
        f.write(CHILD)
        path = f.name
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), path]
    try:
        r = subprocess.run(cmd, env=dict(os.environ, QB_ROOT=ROOT), capture_output=True, text=True, timeout=300)
        assert r.returncode == 0 and "EP_PLAN_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
    finally:
        os.unlink(path)
