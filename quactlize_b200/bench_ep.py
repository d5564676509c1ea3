"""Expert-parallel MoE layer of benchmark configuration 4 over the GPUs of one node (one process per GPU, NCCL):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m quactlize_b200.bench_ep [--tokens 4096] [--steps 10] [--transport peer|nccl] [--small]

Mixtral-8x7B-shaped FFN: 8 experts, top-2, hidden 4096, ffn 14336, int4 gs=128 scale+zero, bf16; `tokens` tokens IN TOTAL
(strong scaling: each rank brings tokens/N of them and owns 8/N experts), router popularity Zipf(1.1).  A step is the
whole layer: plan (one all_gather of counts), dispatch, gate/up GEMM, silu*mul, down GEMM with the combine in its
epilogue, weighted top-k sum (quactlize_b200/ep.py).  Timed with CUDA events on the current stream, max over ranks;
the local GEMMs alone are timed on the same received rows for the split.  Before timing every rank recomputes the
layer for a sample of its own tokens with ALL experts held locally and compares bit for bit.
`run()` is what bench.py calls for its `ep_moe` sub-record."""
from __future__ import annotations

import argparse
import datetime
import json
import os

import numpy as np
import torch
import torch.distributed as dist

from quactlize_b200 import ep, sharding

GS, BITS, TOP_K = 128, 4, 2

# the decode-MoE configuration (128 experts, top-8, hidden 2048, intermediate 768, W2A16 gs=64) as keyword arguments of run()
CFG5 = {"experts": 128, "hidden": 2048, "ffn": 768, "top_k": 8, "bits": 2, "gs": 64, "alpha": 0.0}


def expert_weights(e: int, n: int, k: int, dev, tag: int, bits: int = BITS, gs: int = GS):
    """One expert's plane artifact, seeded by its GLOBAL id so any rank can rebuild any expert."""
    g = torch.Generator(device=dev).manual_seed(100003 * tag + e)
    low = torch.randint(0, 256, (n, k * bits // 8), dtype=torch.uint8, device=dev, generator=g)
    scale = (torch.randn((k // gs, n), device=dev, generator=g).abs() * (0.02 / 7)).to(torch.float16)
    return low, scale, (-float(2 ** (bits - 1)) * scale.float()).to(torch.float16)


def stack_experts(ids, n, k, dev, tag, bits: int = BITS, gs: int = GS):
    parts = [expert_weights(e, n, k, dev, tag, bits, gs) for e in ids]
    return tuple(torch.stack([p[i] for p in parts]).contiguous() for i in range(3))


def zipf_routes(tokens: int, experts: int, top_k: int, seed: int, alpha: float = 1.1) -> np.ndarray:
    """[tokens, top_k] distinct experts per token, popularity proportional to rank^-alpha (the ranking is the same on
    every rank of the job; the draws are per rank)."""
    w = 1.0 / np.arange(1, experts + 1, dtype=np.float64) ** alpha
    w = w[np.random.default_rng(11).permutation(experts)]
    g = -np.log(-np.log(np.random.default_rng(seed).random((tokens, experts))))
    return np.argsort(-(np.log(w)[None, :] + g), axis=1)[:, :top_k].astype(np.int64)


def run(dev, rank: int, world: int, steps: int = 10, peaks=None, sampler=None, tokens: int = 4096, experts: int = 8,
        hidden: int = 4096, ffn: int = 14336, transport: str = "peer", check_tokens: int = 48, top_k: int = TOP_K,
        bits: int = BITS, gs: int = GS, alpha: float = 1.1, graph: bool = True, sync: str = "peer") -> dict:
    if experts % world or tokens % world:
        return {"skipped": f"{experts} experts / {tokens} tokens do not divide over {world} ranks"}
    TOP_K, BITS, GS = top_k, bits, gs                        # noqa: N806 (shadow the module defaults below)
    lo, hi = sharding.expert_range(experts, rank, world)
    gate_up = stack_experts(range(lo, hi), 2 * ffn, hidden, dev, 1, bits, gs)
    down = stack_experts(range(lo, hi), hidden, ffn, dev, 2, bits, gs)
    t_r = tokens // world
    routes = torch.from_numpy(zipf_routes(t_r, experts, TOP_K, seed=1000 + rank, alpha=alpha)).to(dev)
    gen = torch.Generator(device=dev).manual_seed(77 + rank)
    x = torch.randn((t_r, hidden), device=dev, generator=gen).to(torch.bfloat16)
    wts = torch.softmax(torch.randn((t_r, TOP_K), device=dev, generator=gen), dim=1)
    capacity = tokens * TOP_K
    used = transport
    try:
        layer = ep.ExpertParallelFFN(gate_up, down, experts, TOP_K, BITS, GS, capacity, t_r * TOP_K, transport=transport, sync=sync)
    except RuntimeError as e:                                # IPC peer mapping unavailable: same step over NCCL all_to_all
        if transport != "peer":
            raise
        used = f"nccl (peer mapping failed: {str(e)[:80]})"
        layer = ep.ExpertParallelFFN(gate_up, down, experts, TOP_K, BITS, GS, capacity, t_r * TOP_K, transport="nccl")
    ok = torch.tensor([1 if layer.transport == transport else 0], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if int(ok.item()) == 0 and layer.transport == "peer":    # some rank fell back: everyone must
        layer.close()
        layer = ep.ExpertParallelFFN(gate_up, down, experts, TOP_K, BITS, GS, capacity, t_r * TOP_K, transport="nccl")
        used = "nccl (a peer fell back)"

    out = layer(x, routes, wts)
    torch.cuda.synchronize(dev)
    # ---- bit-equality with the single-GPU grouped GEMMs on a sample of this rank's tokens, all experts held locally
    nchk = min(check_tokens, t_r)
    full_gu = stack_experts(range(experts), 2 * ffn, hidden, dev, 1, bits, gs)
    full_dn = stack_experts(range(experts), hidden, ffn, dev, 2, bits, gs)
    flat = routes[:nchk].reshape(-1)
    order = torch.argsort(flat, stable=True)
    offs = torch.zeros(experts + 1, dtype=torch.int32, device=dev)
    offs[1:] = torch.bincount(flat, minlength=experts).cumsum(0).to(torch.int32)
    ref_rows = ep.local_ffn(x[:nchk][order // TOP_K].contiguous(), offs, full_gu, full_dn, BITS, GS)
    item_of_route = torch.empty_like(order)
    item_of_route[order] = torch.arange(order.numel(), device=dev)
    ref = ep.combine(ref_rows, item_of_route.to(torch.int32), wts[:nchk], nchk, TOP_K)
    same = torch.tensor([1 if torch.equal(ref, out[:nchk]) else 0], device=dev)
    finite = torch.tensor([1 if bool(torch.isfinite(out.float()).all()) else 0], device=dev)
    dist.all_reduce(same, op=dist.ReduceOp.MIN); dist.all_reduce(finite, op=dist.ReduceOp.MIN)
    del full_gu, full_dn, ref_rows
    torch.cuda.empty_cache()

    def timed(fn, n):
        for _ in range(3):
            fn()
        torch.cuda.synchronize(dev); dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize(dev); dist.barrier()
        t = torch.tensor([e0.elapsed_time(e1) / n], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # The step as a CUDA graph (kernels and NCCL collectives captured on one stream) where capture works, so the short
    # kernels of the exchange are not spaced by the host; the same step enqueued call by call otherwise.
    step, mode = (lambda: layer(x, routes, wts)), "eager"
    if graph:
        g, g_out = None, None
        try:
            side = torch.cuda.Stream(dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):                    # warm the step on a side stream, as capture requires
                for _ in range(2):
                    layer(x, routes, wts)
            torch.cuda.current_stream(dev).wait_stream(side)
            torch.cuda.synchronize(dev)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                g_out = layer(x, routes, wts)
            ok_here = 1
        except Exception:                                    # capture not possible here (e.g. the NCCL build): stay eager
            ok_here = 0
        torch.cuda.synchronize(dev)
        captured = torch.tensor([ok_here], device=dev)
        dist.all_reduce(captured, op=dist.ReduceOp.MIN)      # nobody replays (its collectives would wait) unless everybody captured
        if int(captured.item()) == 1:
            g.replay()
            torch.cuda.synchronize(dev)
            same_g = torch.tensor([1 if torch.equal(g_out, out) else 0], device=dev)
            dist.all_reduce(same_g, op=dist.ReduceOp.MIN)
            if int(same_g.item()) == 1:
                step, mode = g.replay, "cuda_graph"
    if sampler is not None:
        sampler.start()
    step_ms = timed(step, steps)
    clocks = sampler.stop() if sampler is not None else None
    eager_ms = timed(lambda: layer(x, routes, wts), steps) if mode == "cuda_graph" else step_ms
    # the local GEMMs alone, on the rows this rank really received (max over ranks = what bounds the step)
    local_off = layer.plan(routes).local_off
    my_rows = int(local_off[-1].item())
    rows_buf = layer.buf.rows if layer.buf is not None else torch.randn((max(my_rows, 1), hidden), device=dev).to(torch.bfloat16)
    gemm_ms = timed(lambda: ep.local_ffn(rows_buf, local_off, gate_up, down, BITS, GS), steps)
    plan_ms = timed(lambda: layer.plan(routes), steps)
    rows_t = torch.tensor([float(my_rows)], device=dev)
    mx, sm = rows_t.clone(), rows_t.clone()
    dist.all_reduce(mx, op=dist.ReduceOp.MAX); dist.all_reduce(sm, op=dist.ReduceOp.SUM)
    per_rank = [torch.zeros_like(rows_t) for _ in range(world)]
    dist.all_gather(per_rank, rows_t)
    layer.close()
    total_rows = float(sm.item())
    flops = 2.0 * total_rows * hidden * ffn * 3                           # gate, up and down over the real rows
    rec = {"workload": f"MoE FFN, {experts} experts top-{TOP_K}, hidden {hidden}, ffn {ffn}, int{BITS} gs{GS} scale+zero, bf16, "
                       f"{tokens} tokens in total (strong scaling), " + (f"Zipf({alpha}) router" if alpha else "uniform router"),
           "n_gpus": world, "transport": used, "collectives": ("none inside the step: route counts and three meetings of the ranks through epoch words in peer memory"
                           if getattr(layer, "sync", "nccl") == "peer" else
                           "all_gather(route counts) + 2 x all_reduce(1 element) as stream-ordered barriers")
           if layer.transport == "peer" else "all_gather(route counts) + 2 x all_to_all(rows)",
           "launch_mode": mode, "ms_per_step": round(step_ms, 4), "ms_per_step_eager": round(eager_ms, 4), "gemm_ms_max_rank": round(gemm_ms, 4), "plan_ms": round(plan_ms, 4),
           "exchange_and_combine_ms": round(max(step_ms - gemm_ms, 0.0), 4), "gemm_share_of_step": round(gemm_ms / step_ms, 4),
           "tflops_aggregate": round(flops / step_ms / 1e9, 1), "rows_total": int(total_rows),
           "rows_per_rank": [int(p.item()) for p in per_rank], "imbalance_max_over_mean": round(float(mx.item()) * world / total_rows, 3),
           "bit_identical_to_single_gpu": bool(same.item()), "finite": bool(finite.item()), "steps": steps, "clocks": clocks}
    if peaks:
        rec["frac_of_burst_peak_aggregate"] = round(flops / step_ms / 1e9 / (peaks["bf16"] * world), 4)
    return rec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--transport", default="peer", choices=["peer", "nccl"])
    ap.add_argument("--small", action="store_true", help="a small layer (hidden 512, ffn 768) for tests")
    ap.add_argument("--sync", default="peer", choices=["peer", "nccl"], help="how the ranks meet inside a step (peer transport)")
    ap.add_argument("--no-graph", action="store_true", help="enqueue the step call by call instead of replaying a CUDA graph")
    ap.add_argument("--cfg5", action="store_true", help="the decode-MoE configuration: 128 experts top-8, 2048/768, W2A16 gs=64")
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(minutes=5))   # a collective that is never joined ends the run, not the box's time
    kw = {"hidden": 512, "ffn": 768} if args.small else dict(CFG5) if args.cfg5 else {}
    rec = run(dev, rank, world, steps=args.steps, tokens=args.tokens, transport=args.transport, graph=not args.no_graph, sync=args.sync, **kw)
    if rank == 0:
        print(json.dumps(rec), flush=True)
    dist.destroy_process_group()
    if not rec.get("bit_identical_to_single_gpu", True):
        raise SystemExit(3)


if __name__ == "__main__":
    main()
