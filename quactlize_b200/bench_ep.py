"""Expert-parallel MoE grouped GEMM over N GPUs of one node (one process per GPU, NCCL):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m quactlize_b200.bench_ep [--tokens 4096] [--experts 8] [--check]

Weak scaling: every rank brings `tokens` tokens (top-2 routed over ALL experts, Zipf(1.1) popularity) and owns
experts/N experts of a Mixtral-8x7B-shaped gate projection (hidden 4096 -> ffn 14336, int4 gs=128 scale+zero, bf16).
A step = count exchange + row all-to-all + local ragged tensor-core GEMM + all-to-all back.  Timed with CUDA events on
the current stream, max over ranks; rank 0 prints one JSON line.  --check compares against every expert computed
locally on a small shape."""
from __future__ import annotations

import argparse
import json
import os

import numpy as np
import torch
import torch.distributed as dist

import quactlize_b200 as qb
from quactlize_b200 import sharding, synth


def _weights(experts_lo, experts_hi, n, k, gs, dev):
    lows, scales, zeros = [], [], []
    for e in range(experts_lo, experts_hi):                   # seeded per GLOBAL expert: any rank can rebuild any expert
        rng = np.random.default_rng(1000 + e)
        lows.append(rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8))
        s = (np.abs(rng.normal(0, 0.02, size=(k // gs, n))) / 7).astype(np.float16)
        scales.append(s)
        zeros.append((-8.0 * s.astype(np.float32)).astype(np.float16))
    t = lambda xs: torch.from_numpy(np.stack(xs)).to(dev)
    return t(lows), t(scales), t(zeros)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=14336)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--check", action="store_true")
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    e, k, n, gs, top_k = args.experts, args.hidden, args.ffn, 128, 2
    lo, hi = sharding.expert_range(e, rank, world)
    low, scale, zero = _weights(lo, hi, n, k, gs, dev)
    counts = synth.zipf_rows_per_expert(args.tokens, e, top_k, seed=11 + rank)
    rows = int(counts.sum())
    a = torch.randn((rows, k), device=dev, dtype=torch.float32, generator=torch.Generator(dev).manual_seed(rank)).to(torch.bfloat16)
    counts_t = torch.from_numpy(np.asarray(counts, dtype=np.int64))

    def compute(rows_t, offsets, max_rows):
        return qb.gemm_plane(rows_t, low, None, scale, zero, 4, 0, gs, row_offsets=offsets)

    def step(plan=None):
        return sharding.expert_parallel_apply(a, counts_t, e, n, compute, plan=plan)

    out = step()
    if args.check:
        fl, fs, fz = _weights(0, e, n, k, gs, dev)
        off = torch.from_numpy(np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)).to(dev)
        ref = qb.gemm_plane(a, fl, None, fs, fz, 4, 0, gs, row_offsets=off)
        ok = torch.equal(out, ref)
        flag = torch.tensor([1 if ok else 0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if rank == 0:
            print(json.dumps({"check": "expert-parallel == single-GPU grouped GEMM, bit for bit", "ok": bool(flag.item())}), flush=True)
        assert ok
        del fl, fs, fz, ref
    plan = sharding.plan_dispatch(counts_t, e)
    mine, ratio = sharding.imbalance(plan)
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize(); dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()                                               # plans again every step: routing changes per step in real use
    e1.record()
    torch.cuda.synchronize(); dist.barrier()
    ms = torch.tensor([e0.elapsed_time(e1) / args.steps], device=dev)
    # compute-only time of the same local problem, for the split
    grouped = torch.randn((sum(plan.recv_rows), k), device=dev).to(torch.bfloat16)
    offd = plan.offsets.to(dev)
    for _ in range(3):
        compute(grouped, offd, plan.max_rows)
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    c0.record()
    for _ in range(args.steps):
        compute(grouped, offd, plan.max_rows)
    c1.record(); torch.cuda.synchronize()
    cms = torch.tensor([c0.elapsed_time(c1) / args.steps], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX); dist.all_reduce(cms, op=dist.ReduceOp.MAX)
    total_rows = torch.tensor([float(rows)], device=dev); dist.all_reduce(total_rows)
    if rank == 0:
        flops = 2.0 * float(total_rows) * n * k
        print(json.dumps({"config": f"expert-parallel MoE grouped W4A16 gs128 bf16 gate, E={e}, {args.tokens} tokens/rank top-2",
                          "n_gpus": world, "scaling": "weak", "ms_per_step": round(float(ms), 3),
                          "gemm_ms_max_rank": round(float(cms), 3), "TFLOPs_aggregate": round(flops / float(ms) / 1e9, 1),
                          "rows_total": int(total_rows), "rows_rank0": mine, "imbalance_max_over_mean": round(ratio, 3)}), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
