"""Headline benchmark: Q4_K decode GEMV at Llama-3-8B FFN shapes, reported as HBM GB/s on weight bytes.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--m 1]

One STEP is one pass of the decode hot path over one batch of synthetic layers: COPIES distinct gate/up-shaped
weights (K=4096 -> N=14336) and COPIES distinct down-shaped weights (K=14336 -> N=4096), each multiplied by one fp16
activation row.  The weights of a step total 2*COPIES*33 MB (> the 126 MB L2), so every launch streams from HBM.
`value` is weight bytes / device time with everything resident in HBM; `e2e` is the same work through the host-pointer
C-ABI entry (quactlize_ppu_vecdot_dense: pinned host buffers, H2D + kernel + D2H inside the timed region).

Multi-GPU (torchrun, one rank per GPU): column-parallel over N with no data-path collective -- every rank owns a
full-size N-shard (the global FFN is world x wider), so per-GPU work is fixed ("weak").

`--impl reference` times the reference's own CPU route for this path (routes.matmul_dequant_first: its host
gguf_dequantize + torch matmul, quactlize/routes.py:46-63) from the extension in oracle/_ref on the host cores.
"""
from __future__ import annotations

import argparse
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
COPIES = 4                                     # distinct weights per shape per step: 8 x 33.03 MB = 264 MB > L2
WEIGHT_BYTES = 33030144                        # N*K/256*144 for either shape


def _peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled during the timed region."""
    Q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx = float(r[1])
                for nme, v in zip(names, r[2:6]):
                    if v.lower().startswith("active"):
                        reasons.add(nme)
            except Exception:
                continue
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def _make_weights(seed):
    from quactlize_b200 import synth
    out = []
    for si, (n, k) in enumerate(SHAPES):
        for c in range(COPIES):
            out.append((n, k, synth.kquant_blocks(QT, n * k // 256, seed=seed + 100 * si + c)))
    return out


def run_b200(args):
    import torch.distributed as dist
    import quactlize_b200 as qb
    from quactlize_b200 import _lib, synth

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    L = _lib.lib()
    m = args.m

    host_w = _make_weights(seed=1234 + 7919 * rank)
    dev_w = [(n, k, torch.from_numpy(b).to(dev)) for n, k, b in host_w]
    xs = {k: torch.from_numpy(synth.activations(m, k, seed=5 + k)).to(dev) for _, k in SHAPES}
    outs = [torch.empty((m, n), dtype=torch.float32, device=dev) for n, _, _ in dev_w]
    stream = torch.cuda.current_stream(dev)

    def step():
        sp = torch.cuda.current_stream(dev).cuda_stream        # the capture stream while a graph is being recorded
        for (n, k, w), o in zip(dev_w, outs):
            if m == 1:
                rc = L.quactlize_ppu_vecdot_dense_dev_v1(w.data_ptr(), BLOCK, xs[k].data_ptr(), o.data_ptr(), n, k // 256, QT, sp)
            else:
                rc = L.quactlize_b200_vecdot_rows_dev_v1(w.data_ptr(), BLOCK, xs[k].data_ptr(), o.data_ptr(), m, n, k // 256, QT, 0, sp)
            if rc:
                raise RuntimeError(f"GEMV enqueue failed rc={rc}")

    launches_per_step = len(dev_w)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
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

    # parity spot check before timing (one weight per shape against the numpy oracle on a row sample happens in smoke();
    # here: finite outputs and a non-zero result)
    step(); torch.cuda.synchronize(dev)
    if L.quactlize_b200_device_wait_status() != 0 or not all(bool(torch.isfinite(o).all()) for o in outs):
        raise RuntimeError("GEMV produced non-finite output or a device wait gave up")

    # The decode loop is launch-bound (each GEMV runs for a few microseconds), so one step is recorded once into a
    # CUDA graph and replayed; --no-graph times plain back-to-back enqueues instead.
    run_step = step
    if not args.no_graph:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        run_step = graph.replay
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms = timed(run_step, args.steps, max(3, args.warmup))
    clocks = sampler.stop() if rank == 0 else None
    step_bytes = launches_per_step * WEIGHT_BYTES
    value = world * step_bytes * args.steps / (ms * 1e-3) / 1e9

    # ---- end to end through the host-pointer ABI: pinned host weights, H2D + kernel + D2H per call -----------------
    pin_w = [(n, k, torch.from_numpy(b).pin_memory()) for n, k, b in host_w]
    pin_x = {k: xs[k][:1].cpu().pin_memory() for _, k in SHAPES}
    pin_o = [torch.empty((1, n), dtype=torch.float32).pin_memory() for n, _, _ in pin_w]

    def e2e_step():
        for (n, k, w), o in zip(pin_w, pin_o):
            rc = L.quactlize_ppu_vecdot_dense(w.data_ptr(), BLOCK, pin_x[k].data_ptr(), o.data_ptr(), n, k // 256, QT)
            if rc:
                raise RuntimeError(f"host-pointer GEMV failed rc={rc}")

    e2e_steps = max(1, min(args.steps, 5))
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
    h2d = sum(w.numel() + pin_x[k].numel() * 2 for _, k, w in pin_w)
    d2h = sum(o.numel() * 4 for o in pin_o)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    peak, how = _peaks()
    per_launch_ms = ms / (args.steps * launches_per_step)
    alg = WEIGHT_BYTES + m * 14336 * 2 + m * 4096 * 4          # weights + x + out (mean over the two shapes)
    achieved = alg / (per_launch_ms * 1e-3) / 1e9
    traffic = None
    tp = os.path.join(ROOT, "profiles", "q4k_gemv_traffic.json")
    if os.path.exists(tp):
        try:
            traffic = json.load(open(tp)).get("dram_bytes_per_launch")
        except Exception:
            traffic = None
    line = {
        "metric": "Q4_K decode GEMV HBM GB/s on weight bytes", "value": round(value, 2), "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": round(ms / args.steps, 5),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp16 codes->HFMA2, fp32 accumulate",
        "data": "synthetic",
        "config": {"workload": f"GGUF Q4_K decode GEMV M={m}, Llama-3-8B FFN (K=4096->N=14336 and K=14336->N=4096), "
                               f"{COPIES} distinct weights per shape per step", "parallelism": f"column-parallel x{world}",
                   "l2": f"inputs larger than L2: {launches_per_step * WEIGHT_BYTES / 1e6:.0f} MB of weights per step, rotating"},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(achieved / peak, 4), "traffic": traffic, "peak_source": how,
                     "kernel": "q4k_gemv1_kernel", "algorithmic_bytes_per_launch": alg,
                     "us_per_launch": round(per_launch_ms * 1e3, 3)},
        "e2e": {"value": round(e2e_val, 3), "unit": "GB/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                "api": "quactlize_ppu_vecdot_dense (host pointers, pinned)"},
        "gpu_launches": args.steps * launches_per_step, "launch_mode": "eager" if args.no_graph else "cuda_graph",
        "clocks": clocks,
    }
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
        "config": {"workload": "GGUF Q4_K decode GEMV M=1, Llama-3-8B FFN (K=4096->N=14336 and K=14336->N=4096), "
                               "one weight per shape per step (bounded sample of the same workload)"},
        "cpu_baseline": {"value": round(val, 5), "unit": "GB/s", "cores": cores, "kind": "reference",
                         "sample": "routes.matmul_dequant_first on one weight per shape per step"},
        "e2e": {"value": round(val, 5), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--m", type=int, default=1, help="activation rows per GEMV (1 = the headline decode case)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-graph", action="store_true", help="enqueue every launch instead of replaying a CUDA graph")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
