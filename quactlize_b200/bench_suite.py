"""Per-configuration device timings of the decode GEMV family (everything resident in HBM, CUDA events, CUDA-graph
replay over enough distinct weight copies to exceed the 126 MB L2).  One JSON line per configuration.

    python -m quactlize_b200.bench_suite [--only cfg1,cfg3] [--reps 30]

cfg1  W4A16 dense GEMV, M=1, K=N=4096, gs=128 (generic plane kernel, fp16)
cfg2  GGUF Q4_K raw-block GEMV, M in {1,4,8}, 4096->14336 and 14336->4096
cfg3  bit-plane k-quant GEMV (planes + packed units), M=1, K=4096, N in {4096,14336}, Q6_K / Q5_K / Q3_K
cfg4  prefill MoE grouped W4A16 GEMM (tensor cores), Mixtral-8x7B shapes; fpa = dense fpA_intB M=2048 N=K=4096
cfg5  decode MoE, 128 experts top-8, hidden 2048 / intermediate 768, W2A16 and W1A16 gs=64, bf16, 1..64 tokens
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np
import torch

import quactlize_b200 as qb
from quactlize_b200 import _lib, synth

DEV = "cuda:0"


def _peak():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(p))["hbm_gbs"])
    except Exception:
        return 6650.0


def _time_graph(fn, reps):
    """fn() enqueues one pass over all weight copies on the current stream; returns microseconds per pass."""
    fn(); torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / reps


def _emit(name, us_per_launch, bytes_per_launch, extra=None):
    gbs = bytes_per_launch / us_per_launch / 1e3
    line = {"config": name, "us_per_launch": round(us_per_launch, 3), "weight_bytes": int(bytes_per_launch),
            "GBps": round(gbs, 1), "frac_of_measured_peak": round(gbs / _peak(), 4)}
    if extra:
        line.update(extra)
    print(json.dumps(line), flush=True)


def _copies(nbytes):
    return max(2, int(np.ceil(300e6 / nbytes)))


def cfg1(reps):
    n = k = 4096
    nc = _copies(n * k // 2)
    ws = []
    for c in range(nc):
        low, scale, zero = synth.group_planes(1, n, k, 4, 128, seed=c)
        ws.append(tuple(torch.from_numpy(t).to(DEV) for t in (low, scale, zero)))
    x = torch.from_numpy(synth.activations(1, k, seed=1)).to(DEV)

    def run():
        for low, scale, zero in ws:
            qb.gemv_plane(x, low, None, scale, zero, 4, 0, 128)
    us = _time_graph(run, reps) / nc
    _emit("cfg1 W4A16 gs128 M=1 4096x4096", us, n * k // 2, {"scale_zero_bytes": 2 * (k // 128) * n * 2})


def cfg2(reps):
    for n, k in ((14336, 4096), (4096, 14336)):
        nb = n * k // 256 * 144
        nc = _copies(nb)
        ws = [torch.from_numpy(synth.kquant_blocks(12, n * k // 256, seed=c)).to(DEV) for c in range(nc)]
        for m in (1, 4, 8):
            x = torch.from_numpy(synth.activations(m, k, seed=1)).to(DEV)

            def run():
                for w in ws:
                    qb.gguf_vecdot_rows(w, x, n, k, 12)
            _emit(f"cfg2 Q4_K raw M={m} {k}->{n}", _time_graph(run, reps) / nc, nb)


def cfg3(reps):
    k = 4096
    for qt, name in ((14, "Q6_K"), (13, "Q5_K"), (11, "Q3_K")):
        for n in (4096, 14336):
            nb = n * k // 256 * synth.BLOCK_BYTES[qt]
            nc = _copies(nb)
            arts = []
            for c in range(nc):
                blocks = torch.from_numpy(synth.kquant_blocks(qt, n * k // 256, seed=c))
                arts.append(tuple(t.to(DEV) for t in qb.gguf_prepare_fully_quantized_dense(blocks, n, k, qt)))
            x = torch.from_numpy(synth.activations(1, k, seed=1)).to(DEV)

            def run():
                for low, high, units in arts:
                    qb.gguf_gemv_bc(x, low, high, units, qt)
            _emit(f"cfg3 {name} planes+units M=1 {k}->{n}", _time_graph(run, reps) / nc, nb)


def cfg5(reps):
    e, top_k, hidden, inter, gs = 128, 8, 2048, 768, 64
    for bits in (2, 1):
        mats = {"gate_up": (2 * inter, hidden), "down": (hidden, inter)}
        arts = {}
        for nm, (n, k) in mats.items():
            low, scale, zero = synth.group_planes(e, n, k, bits, gs, seed=bits)
            arts[nm] = tuple(torch.from_numpy(t).to(DEV) for t in (low, scale, zero)) + (n, k)
        for tokens in (1, 8, 64):
            routes = synth.uniform_routes(tokens, e, top_k, seed=tokens)
            counts = np.bincount(routes.reshape(-1), minlength=e)
            off = torch.from_numpy(np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)).to(DEV)
            rows = int(counts.sum())
            active = int((counts > 0).sum())
            mr = int(counts.max())
            for nm, (low, scale, zero, n, k) in arts.items():
                a = torch.from_numpy(synth.activations(rows, k, seed=3, dtype=np.float32)).to(torch.bfloat16).to(DEV)

                def run():
                    qb.gemv_plane(a, low, None, scale, zero, bits, 0, gs, row_offsets=off, max_rows=mr)
                wb = active * n * k * bits // 8
                _emit(f"cfg5 W{bits}A16 gs64 {nm} tokens={tokens} (rows {rows}, active experts {active}) [CUDA-core GEMV]",
                      _time_graph(run, reps), wb, {"scale_zero_bytes": active * 2 * (k // gs) * n * 2, "note": "weights L2-resident across replays"})

                def run_tc():
                    qb.gemm_plane(a, low, None, scale, zero, bits, 0, gs, row_offsets=off)
                _emit(f"cfg5 W{bits}A16 gs64 {nm} tokens={tokens} (rows {rows}, active experts {active}) [tensor-core grouped GEMM]",
                      _time_graph(run_tc, reps), wb, {"scale_zero_bytes": active * 2 * (k // gs) * n * 2, "note": "weights L2-resident across replays"})


def cfg4(reps):
    """Prefill MoE grouped W4A16 GEMM, Mixtral-8x7B-shaped: 8 experts, top-2, 4096 tokens (8192 gathered rows, Zipf(1.1)
    ragged), hidden 4096, ffn 14336, int4 gs=128 scale+zero, bf16 activations."""
    e, tokens, top_k, hidden, ffn, gs = 8, 4096, 2, 4096, 14336, 128
    counts = synth.zipf_rows_per_expert(tokens, e, top_k, seed=11)
    rows = int(counts.sum())
    off = torch.from_numpy(np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)).to(DEV)
    rng = np.random.default_rng(0)
    for nm, (n, k) in (("gate", (ffn, hidden)), ("down", (hidden, ffn))):
        low = torch.from_numpy(rng.integers(0, 256, size=(e, n, k // 2), dtype=np.uint8)).to(DEV)
        scale = torch.from_numpy((np.abs(rng.normal(0, 0.02, size=(e, k // gs, n))) / 7).astype(np.float16)).to(DEV)
        zero = (-8.0 * scale.float()).to(torch.float16)
        a = torch.randn((rows, k), device=DEV, dtype=torch.float32).to(torch.bfloat16)

        def run():
            qb.gemm_plane(a, low, None, scale, zero, 4, 0, gs, row_offsets=off)
        us = _time_graph(run, max(3, reps // 3))
        flops = 2.0 * rows * n * k
        print(json.dumps({"config": f"cfg4 MoE grouped W4A16 gs128 bf16 {nm} (E=8, rows {rows}, per-expert {counts.tolist()})",
                          "us_per_launch": round(us, 1), "TFLOPs": round(flops / us / 1e6, 1),
                          "frac_of_measured_bf16_peak": round(flops / us / 1e6 / 1652.4, 4)}), flush=True)
        del low, scale, zero, a
        torch.cuda.empty_cache()


def fpa(reps):
    """Dense fpA_intB at the reference's bench default: M=2048, N=K=4096, int4 gs=32, fp16."""
    m, n, k = 2048, 4096, 4096
    low, scale, zero = synth.group_planes(1, n, k, 4, 32, seed=5)
    a = torch.randn((m, k), device=DEV, dtype=torch.float16)
    lo_d, sc_d, ze_d = (torch.from_numpy(t).to(DEV) for t in (low, scale, zero))

    def run2():
        qb.gemm_plane(a, lo_d, None, sc_d, ze_d, 4, 0, 32)
    us = _time_graph(run2, reps)
    print(json.dumps({"config": "dense fpA_intB int4 gs32 fp16 M=2048 N=K=4096", "us_per_launch": round(us, 1),
                      "TFLOPs": round(2.0 * m * n * k / us / 1e6, 1)}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="cfg1,cfg2,cfg3,cfg5")
    ap.add_argument("--reps", type=int, default=30)
    args = ap.parse_args()
    _lib.lib()
    torch.cuda.set_device(0)
    for name in args.only.split(","):
        {"cfg1": cfg1, "cfg2": cfg2, "cfg3": cfg3, "cfg4": cfg4, "cfg5": cfg5, "fpa": fpa}[name](args.reps)
        torch.cuda.empty_cache()
    assert _lib.lib().quactlize_b200_device_wait_status() == 0


if __name__ == "__main__":
    main()
