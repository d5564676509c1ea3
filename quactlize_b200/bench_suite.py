"""Command line over the benchmark cases of quactlize_b200.workloads (every benchmark configuration at full size plus the
auxiliary ones: fused gate+up, a 264 MB Q4_K matrix, the raw blocks of the other formats, dequantise, the units pre-pass).

    python -m quactlize_b200.bench_suite --list
    python -m quactlize_b200.bench_suite --only cfg2_m8_4096to14336,cfg4_gate [--batches 5]
    python -m quactlize_b200.bench_suite --only cfg2_m4_4096to14336 --launches 4      # plain launches, for a profiler

Timed mode prints one JSON line per case: microseconds per launch (median of the batches with the min-max band; a CUDA
graph over all copies of the case, so every launch meets cold weights), the fraction of the measured peak that bounds the
case, and the SM clock with the throttle reasons sampled during the timed region.  `--launches N` skips the graph and the
timing and just makes N passes over the copies, which is what a one-kernel ncu capture wants.  The parity figure of each
case is bench.py's business (it owns the checker); this tool only measures."""
from __future__ import annotations

import argparse
import json
import os

import torch

from quactlize_b200 import workloads
from quactlize_b200.clocks import ClockSampler


def peaks() -> dict:
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        j = json.load(open(p))
        return {"hbm": float(j["hbm_gbs"]), "bf16": float(j["bf16_tflops"]), "bf16_sustained": float(j["bf16_tflops_sustained"]),
                "source": "measured"}
    except Exception:
        return {"hbm": 6650.0, "bf16": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


def record(case, t: dict, clocks, pk: dict) -> dict:
    us = t["us"]
    rec = {"case": case.name, "us": round(us, 3), "us_min": round(t["us_min"], 3), "us_max": round(t["us_max"], 3),
           "launches": t["launches"], "copies": case.ncopies, "kernel": case.kernel, "clocks": clocks, "peaks": pk["source"]}
    if case.bound == "hbm":
        gbs = case.alg_bytes / us / 1e3
        rec.update({"bound": "hbm", "GBps": round(gbs, 1), "frac": round(gbs / pk["hbm"], 4), "algorithmic_bytes": case.alg_bytes})
    else:
        tf = case.flops / us / 1e6
        rec.update({"bound": "tensor", "tflops": round(tf, 1), "frac_burst": round(tf / pk["bf16"], 4),
                    "frac_sustained": round(tf / pk["bf16_sustained"], 4)})
    rec.update(case.notes)
    return rec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="", help="comma-separated case names (see --list)")
    ap.add_argument("--list", action="store_true")
    ap.add_argument("--batches", type=int, default=5)
    ap.add_argument("--launches", type=int, default=0, help="no timing: this many plain passes over the case's copies")
    args = ap.parse_args()
    reg = workloads.registry()
    if args.list or not args.only:
        print("\n".join(sorted(reg)))
        return
    pk = peaks()
    dev = torch.cuda.current_device()
    for name in args.only.split(","):
        case = reg[name]()
        if args.launches:
            for _ in range(args.launches):
                for i in range(case.ncopies):
                    case.launch(i)
            torch.cuda.synchronize()
            print(json.dumps({"case": case.name, "plain_launches": args.launches * case.ncopies}), flush=True)
        else:
            sampler = ClockSampler(dev).start()
            t = workloads.time_case(case, batches=args.batches)
            print(json.dumps(record(case, t, sampler.stop(), pk)), flush=True)
        del case
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
