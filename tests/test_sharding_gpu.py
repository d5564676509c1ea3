"""Expert-parallel and column-parallel paths on real GPUs over NCCL, as child processes (one per GPU).  Skipped on a
single-GPU box; the host-side logic is covered on CPU by test_sharding_cpu.py."""
import json
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _torchrun(nproc, args):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port())] + args
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    return [json.loads(line) for line in r.stdout.splitlines() if line.startswith("{")]


def test_expert_parallel_layer_on_one_gpu():
    """World size 1: the whole step (plan, dispatch into this rank's own receive buffer, GEMMs, epilogue combine) must
    equal the plain grouped GEMMs bit for bit."""
    lines = _torchrun(1, ["-m", "quactlize_b200.bench_ep", "--small", "--tokens", "512", "--steps", "2"])
    rec = lines[-1]
    assert rec["bit_identical_to_single_gpu"] is True and rec["finite"] is True and rec["transport"] == "peer"
    assert rec["rows_total"] == 1024 and rec["ms_per_step"] > 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("transport", ["peer", "nccl"])
def test_expert_parallel_matches_single_gpu(transport):
    lines = _torchrun(2, ["-m", "quactlize_b200.bench_ep", "--small", "--tokens", "512", "--steps", "2", "--transport", transport])
    rec = lines[-1]
    assert rec["bit_identical_to_single_gpu"] is True and rec["finite"] is True
    assert rec["n_gpus"] == 2 and sum(rec["rows_per_rank"]) == 1024 and rec["tflops_aggregate"] > 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_bench_two_gpus_carries_the_expert_parallel_record():
    lines = _torchrun(2, ["bench.py", "--gpus", "2", "--steps", "3", "--warmup", "3", "--no-cpu"])
    line = lines[-1]
    assert line["n_gpus"] == 2 and line["scaling"] == "weak" and line["value"] > 0 and line["gpu_launches"] > 0
    assert line["ep_moe"]["bit_identical_to_single_gpu"] is True and line["ep_moe"]["n_gpus"] == 2


def test_plan_kernel_matches_the_index_arithmetic():
    """ep_count / ep_plan (one CTA each, on the device) against plan_routes for every rank of a simulated job: same owners,
    same local offsets, and per (expert) the same set of rows -- the order inside an expert is free."""
    import ctypes as C
    import numpy as np
    from quactlize_b200 import _lib, ep
    L = _lib.lib()
    dev = "cuda:0"
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: C.c_void_p(t.data_ptr())
    for world, experts, top_k, tokens in ((1, 8, 2, 40), (2, 8, 2, 300), (4, 128, 8, 17), (8, 8, 2, 512)):
        rng = np.random.default_rng(world + experts)
        per = experts // world
        routes = [torch.from_numpy(np.argsort(rng.random((tokens + 3 * r, experts)), axis=1)[:, :top_k].reshape(-1).astype(np.int64)).to(dev)
                  for r in range(world)]
        counts = []
        for f in routes:
            c = torch.empty(experts, dtype=torch.int32, device=dev)
            assert L.quactlize_b200_ep_count_dev_v1(p(f), f.numel(), experts, p(c), stream) == 0
            assert torch.equal(c.long(), torch.bincount(f, minlength=experts))
            counts.append(c)
        counts_all = torch.stack(counts).contiguous()
        for r in range(world):
            f = routes[r]
            n = f.numel()
            tok, rk, pos, ior = (torch.full((n,), -7, dtype=torch.int32, device=dev) for _ in range(4))
            off = torch.empty(per + 1, dtype=torch.int32, device=dev)
            assert L.quactlize_b200_ep_plan_dev_v1(p(f), p(counts_all), r, world, experts, n, top_k, p(tok), p(rk), p(pos), p(ior), p(off), stream) == 0
            order, dst_rank, dst_pos, local_off = ep.plan_routes(f, counts_all, r)
            assert torch.equal(off, local_off)
            assert sorted(ior.tolist()) == list(range(n))                          # every route has its own item
            item_expert = torch.empty(n, dtype=torch.int64, device=dev)
            item_expert[ior.long()] = f
            assert bool((item_expert[1:] >= item_expert[:-1]).all())               # items are in expert order
            assert torch.equal(rk.long(), item_expert // per)
            assert torch.equal(tok.long()[ior.long()], torch.arange(n, device=dev) // top_k)
            want = {}
            for e, q in zip(f[order].tolist(), dst_pos.tolist()):
                want.setdefault(e, set()).add(q)
            got = {}
            for e, q in zip(item_expert.tolist(), pos.tolist()):
                got.setdefault(e, set()).add(q)
            assert got == want


def test_rendezvous_gives_up_when_a_rank_never_arrives():
    """The meeting of the ranks through peer memory is a bounded wait: with a second "rank" whose epoch word nobody ever
    writes (two sync areas on this one GPU, only rank 0 launched), the kernel returns after its limit, the status word
    reports the expiry once, and a one-rank meeting afterwards passes."""
    import ctypes as C
    from quactlize_b200 import _lib
    L = _lib.lib()
    dev = torch.device("cuda", 0)
    nbytes = L.quactlize_b200_ep_sync_bytes(2, 8)
    assert nbytes == 1024 + 2 * 8 * 4
    areas = [torch.zeros(nbytes // 4, dtype=torch.int32, device=dev) for _ in range(2)]
    ptrs = torch.tensor([a.data_ptr() for a in areas], dtype=torch.int64, device=dev)
    counts = torch.arange(8, dtype=torch.int32, device=dev)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert L.quactlize_b200_device_wait_status() == 0
    assert L.quactlize_b200_ep_sync_dev_v1(C.c_void_p(ptrs.data_ptr()), 0, 2, 0, C.c_void_p(counts.data_ptr()), 8, stream) == 0
    torch.cuda.synchronize()                                             # returns after the 2 s limit, no hang
    assert L.quactlize_b200_device_wait_status() != 0                    # the expiry, reported once
    assert L.quactlize_b200_device_wait_status() == 0
    # rank 0's counts reached both tables, its epoch word both rows
    for a in areas:
        assert a[256:264].tolist() == list(range(8)) and int(a[0]) == 1
    one = torch.tensor([areas[0].data_ptr()], dtype=torch.int64, device=dev)
    assert L.quactlize_b200_ep_sync_dev_v1(C.c_void_p(one.data_ptr()), 0, 1, 1, None, 0, stream) == 0
    torch.cuda.synchronize()
    assert L.quactlize_b200_device_wait_status() == 0
    assert L.quactlize_b200_ep_sync_dev_v1(C.c_void_p(ptrs.data_ptr()), 2, 2, 0, None, 0, stream) == 20   # rank out of range
