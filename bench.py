"""Headline benchmark: Q4_K decode GEMV at Llama-3-8B FFN shapes, reported as HBM GB/s on weight bytes, with every
other published configuration as a sub-record of the same JSON line.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--m 1] [--configs all|none|a,b,..]

One STEP is the FFN of one decode token through all 32 layers of a Llama-3-8B-shaped model: per layer a gate and an
up projection (K=4096 -> N=14336) and a down projection (K=14336 -> N=4096), each a raw-block Q4_K GEMV with one fp16
activation row -- 96 launches over 96 distinct weight buffers (3.17 GB, so every launch streams from HBM).  `value` is
weight bytes / device time with everything resident in HBM (the median of BATCHES timed batches of exactly K steps,
the band is reported); `e2e` is the same step through the host-pointer C-ABI entry (quactlize_ppu_vecdot_dense:
pinned host buffers, H2D + kernel + D2H inside the timed region).  Before anything is timed one weight per shape is
checked against the numpy oracle on a sample of output rows (`parity_max_rel`).

`configs` carries the other benchmark configurations (quactlize_b200/workloads.py), each timed the same way (CUDA
graph replay over distinct weight copies larger than L2, CUDA events, median of 5 batches with min-max), each with
its own clock record and its own parity figure.

Multi-GPU (torchrun, one rank per GPU): the headline is column-parallel over N with no data-path collective (every
rank owns a full-size N-shard, "weak"); the `ep_moe` sub-record is the expert-parallel MoE layer of configuration 4,
strong-scaled over the ranks with its dispatch and combine exchanges inside the timed step.

`--impl reference` times the reference's own CPU route for this path (routes.matmul_dequant_first: its host
gguf_dequantize + torch matmul, quactlize/routes.py:46-63) from the extension in oracle/_ref on the host cores.
"""
from __future__ import annotations

import argparse
import datetime
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QT = 12
BLOCK = 144
SHAPES = [(14336, 4096), (4096, 14336)]        # (N, K): gate/up and down
LAYERS = 32
DISTINCT = 4                                   # distinct host weights per shape (device buffers are all distinct)
WEIGHT_BYTES = 33030144                        # N*K/256*144 for either shape
BATCHES = 5


def _peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            j = json.load(open(p))
            return {"hbm": float(j["hbm_gbs"]), "bf16": float(j["bf16_tflops"]),
                    "bf16_sustained": float(j["bf16_tflops_sustained"]), "source": "measured"}
        except Exception:
            pass
    return {"hbm": 6650.0, "bf16": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


from quactlize_b200.clocks import ClockSampler  # noqa: E402


def _host_weights(seed):
    from quactlize_b200 import synth
    return {(n, k): [synth.kquant_blocks(QT, n * k // 256, seed=seed + 100 * si + c) for c in range(DISTINCT)]
            for si, (n, k) in enumerate(SHAPES)}


def _git_head():
    try:
        return subprocess.run(["git", "-C", ROOT, "rev-parse", "--short", "HEAD"], capture_output=True, text=True).stdout.strip() or None
    except Exception:
        return None


def sub_records(names, peaks):
    """Every other benchmark configuration: parity on an output sample, then device time, each with its own clocks."""
    from oracle import checks                      # the checker, outside every timed region
    from quactlize_b200 import workloads
    reg = workloads.registry()
    out = {}
    for name in names:
        if name not in reg:
            out[name] = {"error": "unknown configuration"}
            continue
        t0 = time.perf_counter()
        try:
            case = reg[name]()
            par = checks.compare(case.sample())
            torch.cuda.synchronize()
            sampler = ClockSampler(torch.cuda.current_device()).start()
            t = workloads.time_case(case, batches=BATCHES)
            clocks = sampler.stop()
            us = t["us"]
            rec = {"us": round(us, 3), "us_min": round(t["us_min"], 3), "us_max": round(t["us_max"], 3),
                   "launches": t["launches"], "copies": case.ncopies, "kernel": case.kernel,
                   "parity_max_rel": float(f"{par['max_rel']:.3g}"), "parity_elementwise_ok": par["elementwise_ok"],
                   "parity_checked": par["checked"], "clocks": clocks}
            if case.bound == "hbm":
                gbs = case.alg_bytes / us / 1e3
                rec.update({"bound": "hbm", "GBps": round(gbs, 1), "GBps_weight_bytes": round(case.weight_bytes / us / 1e3, 1),
                            "frac": round(gbs / peaks["hbm"], 4), "frac_of_nominal_8000": round(gbs / 8000.0, 4),
                            "algorithmic_bytes": case.alg_bytes,
                            "weight_bytes": case.weight_bytes})
            else:
                tf = case.flops / us / 1e6
                rec.update({"bound": "tensor", "tflops": round(tf, 1), "frac_of_nominal_2250": round(tf / 2250.0, 4),
                            "frac_burst": round(tf / peaks["bf16"], 4),
                            "frac_sustained": round(tf / peaks["bf16_sustained"], 4), "flops": case.flops})
            rec.update(case.notes)
            rec["wall_s"] = round(time.perf_counter() - t0, 2)
            out[name] = rec
            del case
        except Exception as e:                     # one failing configuration must not hide the others
            out[name] = {"error": f"{type(e).__name__}: {e}"[:300]}
        torch.cuda.empty_cache()
    return out


def run_b200(args):
    import torch.distributed as dist
    from oracle import checks
    from quactlize_b200 import _lib, synth

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(minutes=5))   # a collective that is never joined ends the run, not the box's time
    L = _lib.lib()
    m = args.m
    peaks = _peaks()

    host_w = _host_weights(seed=1234 + 7919 * rank)
    # the step's launches in layer order: gate, up, down of each layer, every one on its own device buffer
    base = {s: [torch.from_numpy(b).to(dev) for b in ws] for s, ws in host_w.items()}
    seq = []
    for layer in range(LAYERS):
        for j, s in enumerate((SHAPES[0], SHAPES[0], SHAPES[1])):
            idx = (2 * layer + j) if j < 2 else layer
            seq.append((s[0], s[1], base[s][idx % DISTINCT] if idx < DISTINCT else base[s][idx % DISTINCT].clone(), idx % DISTINCT))
    xs = {k: torch.from_numpy(synth.activations(m, k, seed=5 + k)).to(dev) for _, k in SHAPES}
    outs = [torch.empty((m, n), dtype=torch.float32, device=dev) for n, _, _, _ in seq]
    stream = torch.cuda.current_stream(dev)

    def step():
        sp = torch.cuda.current_stream(dev).cuda_stream        # the capture stream while a graph is being recorded
        for (n, k, w, _), o in zip(seq, outs):
            if m == 1:
                rc = L.quactlize_ppu_vecdot_dense_dev_v1(w.data_ptr(), BLOCK, xs[k].data_ptr(), o.data_ptr(), n, k // 256, QT, sp)
            else:
                rc = L.quactlize_b200_vecdot_rows_dev_v1(w.data_ptr(), BLOCK, xs[k].data_ptr(), o.data_ptr(), m, n, k // 256, QT, 0, sp)
            if rc:
                raise RuntimeError(f"GEMV enqueue failed rc={rc}")

    launches_per_step = len(seq)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    # ---- parity before timing: one weight per shape, a row sample against the numpy oracle ------------------------
    step(); torch.cuda.synchronize(dev)
    if L.quactlize_b200_device_wait_status() != 0:
        raise RuntimeError("a device wait gave up")
    parity = 0.0
    rng = np.random.default_rng(7)
    for (n, k, w, hi), o in zip(seq[:3], outs[:3]):
        rows = np.unique(np.concatenate([[0, n - 1], rng.integers(0, n, 254)]))
        sub = host_w[(n, k)][hi].reshape(n, k // 256, BLOCK)[rows].reshape(-1, BLOCK)
        r = checks.compare({"kind": "raw", "got": o.cpu().numpy()[:, rows], "blocks": sub, "x": xs[k].cpu().numpy(),
                            "n": len(rows), "k": k, "qtype": QT, "out": "fp32"})
        parity = max(parity, r["max_rel"])
    if not parity <= 1e-2:
        raise RuntimeError(f"parity check failed before timing: max-rel {parity}")
    first = {}
    for (n, k, _, hi), o in zip(seq, outs):           # buffers that hold the same weight must give the same output
        ref_o = first.setdefault((n, k, hi), o)
        if ref_o is not o and not torch.equal(ref_o, o):
            raise RuntimeError("two buffers holding the same weight gave different outputs")

    # The decode loop is launch-bound (each GEMV runs for a few microseconds), so one step is recorded once into a
    # CUDA graph and replayed; --no-graph times plain back-to-back enqueues instead.
    run_step = step
    if not args.no_graph:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        run_step = graph.replay
    warm = max(3, args.warmup)
    for _ in range(warm):
        run_step()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    batch_ms = sorted(timed(run_step, args.steps) for _ in range(BATCHES))
    clocks = sampler.stop() if rank == 0 else None
    ms = batch_ms[len(batch_ms) // 2]
    step_bytes = launches_per_step * WEIGHT_BYTES
    value = world * step_bytes * args.steps / (ms * 1e-3) / 1e9

    # ---- the same step with each layer's gate and up in ONE launch (they share the activation): 64 launches on the same
    # 96 buffers through the additive two-matrix entry; outputs must equal the per-matrix launches bit for bit
    fused = None
    if m == 1 and not args.no_graph:
        outs_f = [torch.empty_like(o) for o in outs]

        def fused_step():
            sp = torch.cuda.current_stream(dev).cuda_stream
            for layer in range(LAYERS):
                (n, k, wg, _), (_, _, wu, _), (nd, kd, wd, _) = seq[3 * layer], seq[3 * layer + 1], seq[3 * layer + 2]
                rc = L.quactlize_b200_vecdot_dense2_dev_v1(wg.data_ptr(), n, wu.data_ptr(), n, BLOCK, xs[k].data_ptr(),
                                                           outs_f[3 * layer].data_ptr(), outs_f[3 * layer + 1].data_ptr(), k // 256, QT, sp)
                rc = rc or L.quactlize_ppu_vecdot_dense_dev_v1(wd.data_ptr(), BLOCK, xs[kd].data_ptr(), outs_f[3 * layer + 2].data_ptr(),
                                                               nd, kd // 256, QT, sp)
                if rc:
                    raise RuntimeError(f"fused step enqueue failed rc={rc}")
        fused_step(); torch.cuda.synchronize(dev)
        same = all(torch.equal(a_, b_) for a_, b_ in zip(outs, outs_f))
        gf = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gf):
            fused_step()
        for _ in range(warm):
            gf.replay()
        fms = sorted(timed(gf.replay, args.steps) for _ in range(BATCHES))
        fm = fms[len(fms) // 2]
        fgbs = world * step_bytes * args.steps / (fm * 1e-3) / 1e9
        fused = {"what": "the same step with gate and up of a layer in one launch (quactlize_b200_vecdot_dense2_dev_v1): 64 launches",
                 "ms_per_step": round(fm / args.steps, 5), "value": round(fgbs, 2), "unit": "GB/s",
                 "frac": round(fgbs / world / peaks["hbm"], 4), "bit_identical_to_per_matrix_launches": bool(same),
                 "gpu_launches": BATCHES * args.steps * 2 * LAYERS}
        del outs_f

    # ---- end to end through the host-pointer ABI: pinned host weights, H2D + kernel + D2H per call -----------------
    pin_w = {s: [torch.from_numpy(b).pin_memory() for b in ws] for s, ws in host_w.items()}
    pin_x = {k: xs[k][:1].cpu().pin_memory() for _, k in SHAPES}
    pin_o = {n: torch.empty((1, n), dtype=torch.float32).pin_memory() for n, _ in SHAPES}

    def e2e_step():
        for n, k, _, hi in seq:
            rc = L.quactlize_ppu_vecdot_dense(pin_w[(n, k)][hi].data_ptr(), BLOCK, pin_x[k].data_ptr(), pin_o[n].data_ptr(), n, k // 256, QT)
            if rc:
                raise RuntimeError(f"host-pointer GEMV failed rc={rc}")

    e2e_steps = max(1, min(args.steps, 3))
    e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_val = world * step_bytes * e2e_steps / e2e_s / 1e9
    h2d = sum(WEIGHT_BYTES + k * 2 for _, k, _, _ in seq)
    d2h = sum(n * 4 for n, _, _, _ in seq)
    del pin_w

    ep = ep5 = None
    if world > 1 and args.configs != "none":
        from quactlize_b200 import bench_ep
        try:
            ep = bench_ep.run(dev, rank, world, steps=max(5, min(args.steps, 20)), peaks=peaks,
                              sampler=ClockSampler(local) if rank == 0 else None)
        except Exception as e:
            ep = {"error": f"{type(e).__name__}: {e}"[:300]}
        try:                                                 # the decode-MoE configuration, 1024 tokens in total
            ep5 = bench_ep.run(dev, rank, world, steps=max(5, min(args.steps, 20)), peaks=peaks, tokens=1024, **bench_ep.CFG5)
        except Exception as e:
            ep5 = {"error": f"{type(e).__name__}: {e}"[:300]}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    per_launch_ms = ms / (args.steps * launches_per_step)
    alg = WEIGHT_BYTES + m * (2 * 4096 + 14336) // 3 * 2 + m * (2 * 14336 + 4096) // 3 * 4     # weights + x + out, mean over gate, up, down
    achieved = alg / (per_launch_ms * 1e-3) / 1e9
    traffic, traffic_src = None, None
    tp = os.path.join(ROOT, "profiles", "q4k_gemv_traffic.json")
    if os.path.exists(tp) and m == 1:
        try:
            tj = json.load(open(tp))
            traffic, traffic_src = tj.get("dram_bytes_per_launch"), f"recorded: profiles/q4k_gemv_traffic.json ({tj.get('commit', 'commit not recorded')})"
        except Exception:
            traffic = None
    line = {
        "metric": "Q4_K decode GEMV HBM GB/s on weight bytes", "value": round(value, 2), "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": warm, "ms_per_step": round(ms / args.steps, 5),
        "ms_per_step_min": round(batch_ms[0] / args.steps, 5), "ms_per_step_max": round(batch_ms[-1] / args.steps, 5),
        "timed_batches": BATCHES,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp16 codes->HFMA2, fp32 accumulate",
        "data": "synthetic",
        "config": {"workload": f"GGUF Q4_K decode GEMV M={m}, Llama-3-8B FFN: one step = gate, up (K=4096->N=14336) and down "
                               f"(K=14336->N=4096) of {LAYERS} layers, {launches_per_step} launches on distinct weight buffers",
                   "parallelism": f"column-parallel x{world}",
                   "l2": f"inputs larger than L2: {launches_per_step * WEIGHT_BYTES / 1e9:.2f} GB of weights per step, each buffer read once per step"},
        "parity_max_rel": float(f"{parity:.3g}"),
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm"], 4), "frac_of_nominal_8000": round(achieved / 8000.0, 4),
                     "traffic": traffic, "traffic_source": traffic_src,
                     "peak_source": peaks["source"], "kernel": "q4k_gemv1_kernel" if m == 1 else "q4k_rows_kernel",
                     "algorithmic_bytes_per_launch": alg, "us_per_launch": round(per_launch_ms * 1e3, 3)},
        "e2e": {"value": round(e2e_val, 3), "unit": "GB/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                "api": "quactlize_ppu_vecdot_dense (host pointers, pinned)", "steps": e2e_steps},
        "gpu_launches": BATCHES * args.steps * launches_per_step, "launch_mode": "eager" if args.no_graph else "cuda_graph",
        "clocks": clocks, "commit": _git_head(),
    }
    if fused is not None:
        line["fused_gate_up_step"] = fused
    if ep is not None:
        line["ep_moe"] = ep
        line["ep_moe_cfg5"] = ep5
    if world == 1 and args.configs != "none":
        from quactlize_b200 import workloads
        names = sorted(workloads.registry()) if args.configs == "all" else args.configs.split(",")
        del seq, outs, base
        torch.cuda.empty_cache()
        line["configs"] = sub_records(names, peaks)
    if not args.no_cpu:
        line["cpu_baseline"] = cpu_reference(sample_copies=1)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def _ref_ops():
    """torch.ops.quactlize from the reference's own host extension (oracle/_ref), CPU arms only."""
    from oracle import build_ref
    lib = build_ref.build()
    if lib is None:
        return None
    os.environ["QUACTLIZE_PPU_LIB"] = "/nonexistent/force-the-reference-cpu-arm.so"
    torch.ops.load_library(lib)
    return torch.ops.quactlize


def cpu_reference(sample_copies=1):
    """The reference's CPU route (dequant-first: host gguf_dequantize, then a @ w.T) on `sample_copies` weights per shape."""
    q = _ref_ops()
    from quactlize_b200 import synth
    cores = torch.get_num_threads()
    total_bytes, t_deq, t_mm = 0, 0.0, 0.0
    if q is not None:
        for si, (n, k) in enumerate(SHAPES):
            for c in range(sample_copies):
                b = torch.from_numpy(synth.kquant_blocks(QT, n * k // 256, seed=99 + si + c))
                x = torch.from_numpy(synth.activations(1, k, seed=3))
                t0 = time.perf_counter()
                w = q.gguf_dequantize(b, QT).view(n, k)
                t1 = time.perf_counter()
                _ = x.to(w.dtype) @ w.t()
                t2 = time.perf_counter()
                t_deq += t1 - t0; t_mm += t2 - t1; total_bytes += b.numel()
        kind = "reference"
    else:
        from oracle import kquant as kq
        for si, (n, k) in enumerate(SHAPES):
            b = synth.kquant_blocks(QT, n * k // 256, seed=99 + si)
            x = synth.activations(1, k, seed=3)
            t0 = time.perf_counter()
            kq.vecdot_dense(b, x, n, k, QT)
            t_deq += time.perf_counter() - t0; total_bytes += b.size
        kind = "port"
    tot = t_deq + t_mm
    return {"value": round(total_bytes / tot / 1e9, 5), "unit": "GB/s", "cores": cores, "kind": kind,
            "sample": f"{sample_copies} weight(s) per shape ({total_bytes / 1e6:.0f} MB): dequantise {t_deq:.2f} s "
                      f"(serial host loop) + matmul {t_mm:.3f} s ({cores} threads)",
            "matmul_only_gbs": round(total_bytes / t_mm / 1e9, 3) if t_mm > 0 else None}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    q = _ref_ops()
    if q is None:
        print(json.dumps({"impl": "reference", "unavailable": "reference host extension not built (oracle/_ref missing)"}))
        return
    from quactlize_b200 import synth
    cores = torch.get_num_threads()
    mats = []
    for si, (n, k) in enumerate(SHAPES):
        mats.append((n, k, torch.from_numpy(synth.kquant_blocks(QT, n * k // 256, seed=99 + si)),
                     torch.from_numpy(synth.activations(1, k, seed=3))))

    def step():
        for n, k, b, x in mats:
            w = q.gguf_dequantize(b, QT).view(n, k)
            _ = x.to(w.dtype) @ w.t()

    warm = min(args.warmup, 1)
    steps = max(1, min(args.steps, 3))
    for _ in range(warm):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = time.perf_counter() - t0
    nbytes = sum(b.numel() for _, _, b, _ in mats)
    val = nbytes * steps / dt / 1e9
    print(json.dumps({
        "impl": "reference", "metric": "Q4_K decode GEMV HBM GB/s on weight bytes", "value": round(val, 5), "unit": "GB/s",
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": steps, "warmup": warm, "ms_per_step": round(dt / steps * 1e3, 2),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp16", "data": "synthetic",
        "config": {"workload": f"GGUF Q4_K decode GEMV M=1, Llama-3-8B FFN: one step = gate, up (K=4096->N=14336) and down "
                               f"(K=14336->N=4096) of {LAYERS} layers; each step here is a bounded sample of it, one weight per shape"},
        "cpu_baseline": {"value": round(val, 5), "unit": "GB/s", "cores": cores, "kind": "reference",
                         "sample": "routes.matmul_dequant_first on one weight per shape per step"},
        "e2e": {"value": round(val, 5), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--m", type=int, default=1, help="activation rows per GEMV (1 = the headline decode case)")
    ap.add_argument("--configs", default="all", help="sub-records: all, none, or a comma list of workloads.registry() names")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-graph", action="store_true", help="enqueue every launch instead of replaying a CUDA graph")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
