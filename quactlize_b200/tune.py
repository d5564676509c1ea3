"""Offline tactic tuning over the library's compiled tactic inventory: sweep a model's real shapes once, write a table,
never search at run time.

Follows the behaviour of the reference's tools/tune.py (policy statements :28-41, bucket rule :258-272, runtime cache
:132-225), against THIS library's inventory:

  * the candidates are read from the library itself (quactlize_ppu_list_configs / _list_grouped_configs) and restricted,
    per shape, to what its own validity predicates admit (quactlize_ppu_*_config_valid_v1) -- a table can therefore never
    name a tactic the library does not contain or would decline;
  * M maps to its last positive power of two and ONLY bucket values that were measured are written: a request that
    maps to another bucket misses and takes the compiled default; a winner is never extended beyond its evidence;
  * a sweep that does not separate its candidates (the best two medians closer than the observed spread) records NO
    winner -- an absent tactic gets the default, a wrong one does not get noticed;
  * every table carries its provenance: the library file's hash, the hash of the inventory it was chosen from, the
    device, the workload, repetitions.

Routes tuned: `dense_fully_quantized` and `grouped_fully_quantized` (the tensor-core GEMMs on planes + packed units,
through their `_dev_v2` entries, which take a tactic name).  Timing: CUDA events on the current stream, candidates
interleaved across repetitions, median per candidate.

    python -m quactlize_b200.tune --model llama3-8b --route dense_fully_quantized --qtype 12 -o tactics.json \
        [--runtime-cache tactics.cache] [--m 16,64,256,1024,4096] [--reps 5]
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import sys
import tempfile
from typing import Callable, Dict, List, Optional, Sequence, Tuple

CACHE_SCHEMA = "quactlize-ppu-tactic-cache-v1"
BUCKET_POLICY = "last-positive-power-of-two(raw-total-tokens);store-only-profiled-buckets;v1"
ROUTE_SCHEMA = "route+normalized-op+qtype+n+k+group-size+m-bucket+experts+top-k;v2"
ROUTES = ("dense_fully_quantized", "grouped_fully_quantized")
_FNV_OFFSET, _FNV_PRIME = 14695981039346656037, 1099511628211

# model name -> (FFN projections [(op, n, k)], experts, top_k); shapes of the benchmark configurations
MODELS: Dict[str, dict] = {
    "llama3-8b": {"projections": [("ffn_gate", 14336, 4096), ("ffn_up", 14336, 4096), ("ffn_down", 4096, 14336)], "experts": 0, "topk": 0},
    "mixtral-8x7b": {"projections": [("ffn_moe_gate", 14336, 4096), ("ffn_moe_up", 14336, 4096), ("ffn_moe_down", 4096, 14336)],
                     "experts": 8, "topk": 2},
    "qwen3-30b-a3b": {"projections": [("ffn_moe_gate", 768, 2048), ("ffn_moe_up", 768, 2048), ("ffn_moe_down", 2048, 768)],
                      "experts": 128, "topk": 8},
}


def fnv1a64(data: bytes, value: int = _FNV_OFFSET) -> int:
    for b in data:
        value = ((value ^ b) * _FNV_PRIME) & ((1 << 64) - 1)
    return value


def _hash_field(value: int, text: str) -> int:
    return fnv1a64(text.encode() + b"\0", value)


class _ConfigV1(C.Structure):
    _fields_ = [("enable_cuda_kernel", C.c_bool), ("name", C.c_char_p), ("tile_m", C.c_int32), ("tile_n", C.c_int32),
                ("warp_m", C.c_int32), ("warp_n", C.c_int32), ("stages", C.c_int32)]


def load_inventory(lib) -> Tuple[List[dict], List[dict], str]:
    """(dense tactics, grouped tactics, canonical hash of both lists) as the loaded library reports them."""
    def read(symbol):
        fn = getattr(lib, symbol)
        fn.argtypes, fn.restype = [C.POINTER(C.POINTER(_ConfigV1))], C.c_int32
        ptr = C.POINTER(_ConfigV1)()
        count = fn(C.byref(ptr))
        if count < 0 or (count and not ptr):
            raise RuntimeError(f"{symbol} returned an invalid inventory")
        rows = []
        for i in range(count):
            r = ptr[i]
            if not r.name:
                raise RuntimeError(f"{symbol} config {i} has no name")
            rows.append({"enable_cuda_kernel": bool(r.enable_cuda_kernel), "name": r.name.decode(), "tile_m": r.tile_m,
                         "tile_n": r.tile_n, "warp_m": r.warp_m, "warp_n": r.warp_n, "stages": r.stages})
        return rows
    dense, grouped = read("quactlize_ppu_list_configs"), read("quactlize_ppu_list_grouped_configs")
    value = _FNV_OFFSET
    for family, rows in (("dense", dense), ("grouped", grouped)):
        value = _hash_field(_hash_field(value, family), str(len(rows)))
        for r in rows:
            value = _hash_field(value, "cuda" if r["enable_cuda_kernel"] else "tensor")
            for f in ("name", "tile_m", "tile_n", "warp_m", "warp_n", "stages"):
                value = _hash_field(value, str(r[f]))
    return dense, grouped, f"{value:016x}"


def m_bucket(m: int) -> int:
    """The last positive power of two not above m; no bucket (0) for non-positive m."""
    return 0 if m <= 0 else 1 << (m.bit_length() - 1)


def measured_buckets(by_m: Dict[int, str]) -> List[dict]:
    """Resolved measurements -> exact bucket winners.  Two measurements that fall in one bucket must agree."""
    out: Dict[int, dict] = {}
    for m in sorted(by_m):
        b = m_bucket(m)
        if b in out and out[b]["config"] != by_m[m]:
            raise ValueError(f"M={out[b]['measured_m']} and M={m} map to bucket {b} but disagree")
        out[b] = {"m_bucket": b, "measured_m": m, "config": by_m[m]}
    return [out[b] for b in sorted(out)]


def pick_winner(samples: Dict[str, Sequence[float]]) -> Tuple[Optional[str], str]:
    """Median time per candidate; the fastest wins only if it is SEPARATED from the runner-up: its slowest repetition
    is still faster than the runner-up's median.  Returns (name or None, note)."""
    if not samples:
        return None, "no valid candidate"
    if any(len(v) < 2 for v in samples.values()):
        return None, "one pass cannot rank"
    med = sorted((statistics.median(v), name) for name, v in samples.items())
    if len(med) == 1:
        return med[0][1], "only candidate"
    best, second = med[0], med[1]
    if max(samples[best[1]]) < second[0]:
        return best[1], "separated"
    return None, f"unresolved: {best[1]} {best[0]:.2f} us vs {second[1]} {second[0]:.2f} us overlap"


def valid_candidates(lib, route: str, inventory: List[dict], m: int, n: int, k: int, gs: int, qtype: int, experts: int, topk: int):
    """Tensor-core tactics of the inventory that the library's own predicate admits for this problem."""
    out = []
    for row in inventory:
        if row["enable_cuda_kernel"]:
            continue
        name = row["name"].encode()
        if route == "dense_fully_quantized":
            fn = lib.quactlize_ppu_dense_fully_quantized_config_valid_v1
            ok = fn(m, n, k, gs, qtype, name)
        else:
            rows = m * topk
            fn = lib.quactlize_ppu_grouped_fully_quantized_config_valid_v1
            ok = fn(rows, n, k, gs, experts, rows, qtype, name)
        if ok:
            out.append(row["name"])
    return out


def device_timer(lib, route: str, n: int, k: int, qtype: int, experts: int, topk: int) -> Callable[[int, str], float]:
    """A timer (m, tactic) -> microseconds for one shape, on cuda:0 with seeded synthetic weights."""
    import numpy as np
    import torch
    import quactlize_b200 as qb
    from . import synth
    dev = "cuda:0"
    e = max(experts, 1)
    blocks = torch.from_numpy(synth.kquant_blocks(qtype, e * n * k // 256, seed=n + k + qtype))
    if route == "dense_fully_quantized":
        low, high, units = (t.to(dev) for t in qb.gguf_prepare_fully_quantized_dense(blocks, n, k, qtype))
    else:
        low, high, units = (t.to(dev) for t in qb.gguf_prepare_fully_quantized_grouped(blocks, n, k, qtype, e))
    hp = high.data_ptr() if high.numel() else None
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def timer(m: int, tactic: str) -> float:
        rows = m if route == "dense_fully_quantized" else m * topk
        a = torch.from_numpy(synth.activations(rows, k, seed=m)).to(dev)
        out = torch.empty((rows, n), dtype=torch.float16, device=dev)
        if route == "dense_fully_quantized":
            need = lib.quactlize_ppu_dense_fully_quantized_workspace_bytes_v1(rows, n, k, qtype)
            ws = torch.empty(max(need, 1), dtype=torch.uint8, device=dev)
            call = lambda: lib.quactlize_ppu_dense_fully_quantized_dev_v2(a.data_ptr(), low.data_ptr(), hp, units.data_ptr(), out.data_ptr(),
                                                                          rows, n, k, qtype, ws.data_ptr(), need, stream, tactic.encode())
        else:
            counts = synth.zipf_rows_per_expert(m, e, topk, seed=m) if e > 1 else np.array([rows])
            off = torch.from_numpy(np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)).to(dev)
            mr = int(counts.max())
            need = lib.quactlize_ppu_grouped_fully_quantized_workspace_bytes_v1(max(mr, 1), n, k, e, qtype)
            ws = torch.empty(max(need, 1), dtype=torch.uint8, device=dev)
            call = lambda: lib.quactlize_ppu_grouped_fully_quantized_dev_v2(a.data_ptr(), low.data_ptr(), hp, units.data_ptr(), off.data_ptr(),
                                                                            out.data_ptr(), rows, n, k, e, max(mr, 1), qtype, ws.data_ptr(),
                                                                            need, stream, tactic.encode())
        for _ in range(2):
            if call():
                raise RuntimeError(f"tactic {tactic} refused M={m} N={n} K={k}")
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        inner = 5
        e0.record()
        for _ in range(inner):
            call()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / inner
    return timer


def tune(lib, model: str, route: str, qtype: int, ms: Sequence[int], reps: int,
         timer_for: Optional[Callable[[int, int], Callable[[int, str], float]]] = None) -> dict:
    """Sweep every distinct (n, k) of the model over `ms`; returns the table (resolved winners only, plus the raw
    medians and the notes of unresolved sweeps).  `timer_for(n, k)` supplies the timer (the device one by default)."""
    if reps < 2:
        raise ValueError("reps must be at least 2: one pass cannot separate candidates")
    if route not in ROUTES:
        raise ValueError(f"route must be one of {ROUTES}")
    cfg = MODELS[model]
    grouped = route == "grouped_fully_quantized"
    if grouped and not cfg["experts"]:
        raise ValueError(f"{model} has no experts; use the dense route")
    dense_inv, grouped_inv, inv_hash = load_inventory(lib)
    inventory = grouped_inv if grouped else dense_inv
    gs = 32 if qtype in (12, 13) else 16
    shapes = []
    for shape in sorted({(n, k) for _, n, k in cfg["projections"]}):
        n, k = shape
        timer = (timer_for or (lambda n_, k_: device_timer(lib, route, n_, k_, qtype, cfg["experts"], cfg["topk"])))(n, k)
        by_m, raw = {}, []
        for m in ms:
            cands = valid_candidates(lib, route, inventory, m, n, k, gs, qtype, cfg["experts"], cfg["topk"])
            samples: Dict[str, List[float]] = {c: [] for c in cands}
            for _ in range(reps):                          # interleave the candidates across repetitions
                for c in cands:
                    samples[c].append(timer(m, c))
            winner, note = pick_winner(samples)
            raw.append({"m": m, "note": note, "median_us": {c: round(statistics.median(v), 3) for c, v in samples.items() if v}})
            if winner is not None:
                by_m[m] = winner
        shapes.append({"n": n, "k": k, "buckets": measured_buckets(by_m), "sweeps": raw})
    return {"schema": "quactlize-b200-tactic-table-v1", "model": model, "route": route, "qtype": qtype, "group_size": gs,
            "reps": reps, "bucket_policy": BUCKET_POLICY, "config_space_fnv1a64": inv_hash,
            "candidates": [r["name"] for r in inventory if not r["enable_cuda_kernel"]], "shapes": shapes}


def write_runtime_cache(path: str, table: dict, lib_path: str, device: str) -> List[str]:
    """The strict winner-only cache in the reference's line format (tools/tune.py:192-209): provenance lines, then one
    `entry|...` line per (op, shape, bucket).  Written atomically.  Returns the lines."""
    model = table["model"]
    if any(ch in device for ch in "|=\r\n") or any(ch in model for ch in "|=\r\n"):
        raise ValueError("device/model provenance contains a cache delimiter")
    cfg = MODELS[model]
    grouped = table["route"] == "grouped_fully_quantized"
    ops: Dict[Tuple[int, int], List[str]] = {}
    for op, n, k in cfg["projections"]:
        ops.setdefault((n, k), []).append(op)
    entries = []
    for shape in table["shapes"]:
        for b in shape["buckets"]:
            for op in sorted(ops.get((shape["n"], shape["k"]), ())):
                entries.append(f"entry|route={table['route']}|op={op}|qtype={table['qtype']}|n={shape['n']}|k={shape['k']}|"
                               f"gs={table['group_size']}|m_bucket={b['m_bucket']}|experts={cfg['experts'] if grouped else 0}|"
                               f"top_k={cfg['topk'] if grouped else 0}|cuda=0|config={b['config']}")
    with open(lib_path, "rb") as f:
        elf = f"{fnv1a64(f.read()):016x}"
    lines = [f"schema={CACHE_SCHEMA}", f"bucket_policy={BUCKET_POLICY}", f"bucket_policy_fnv1a64={fnv1a64(BUCKET_POLICY.encode()):016x}",
             f"route_schema_fnv1a64={fnv1a64(ROUTE_SCHEMA.encode()):016x}", f"loaded_elf_fnv1a64={elf}",
             f"config_space_fnv1a64={table['config_space_fnv1a64']}", f"device={device}", f"workload={model}", *entries]
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    fd, tmp = tempfile.mkstemp(prefix=os.path.basename(path) + ".", dir=os.path.dirname(os.path.abspath(path)))
    try:
        with os.fdopen(fd, "w") as out:
            out.write("\n".join(lines) + "\n")
            out.flush()
            os.fsync(out.fileno())
        os.replace(tmp, path)
    except Exception:
        if os.path.exists(tmp):
            os.unlink(tmp)
        raise
    return lines


def lookup(cache_lines: Sequence[str], route: str, op: str, qtype: int, n: int, k: int, gs: int, m: int,
           experts: int = 0, top_k: int = 0, config_space: Optional[str] = None) -> Optional[str]:
    """The tactic a run-time caller should name for this problem, or None (= let the library choose): the entry of the
    exact bucket m falls in, nothing else.  A cache written against another inventory (config_space) never matches."""
    head = dict(l.split("=", 1) for l in cache_lines if "=" in l and not l.startswith("entry|"))
    if head.get("schema") != CACHE_SCHEMA or (config_space is not None and head.get("config_space_fnv1a64") != config_space):
        return None
    want = {"route": route, "op": op, "qtype": str(qtype), "n": str(n), "k": str(k), "gs": str(gs), "m_bucket": str(m_bucket(m)),
            "experts": str(experts), "top_k": str(top_k)}
    for l in cache_lines:
        if not l.startswith("entry|"):
            continue
        f = dict(p.split("=", 1) for p in l.split("|")[1:])
        if all(f.get(a) == b for a, b in want.items()):
            return f.get("config")
    return None


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="offline tactic tuning over the library's compiled inventory")
    ap.add_argument("--model", required=True, choices=sorted(MODELS))
    ap.add_argument("--route", default="dense_fully_quantized", choices=ROUTES)
    ap.add_argument("--qtype", type=int, default=12)
    ap.add_argument("--m", default="16,64,256,1024,4096", help="token counts to measure (each fills exactly its own bucket)")
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("-o", "--out", required=True)
    ap.add_argument("--runtime-cache", default="")
    args = ap.parse_args(argv)
    if args.reps < 2:
        print("--reps must be at least 2: one pass cannot separate candidates", file=sys.stderr)
        return 2
    import torch
    from . import _lib
    lib = _lib.lib()
    table = tune(lib, args.model, args.route, args.qtype, [int(x) for x in args.m.split(",")], args.reps)
    table["device"] = torch.cuda.get_device_name(0)
    with open(args.out, "w") as f:
        json.dump(table, f, indent=1)
    if args.runtime_cache:
        write_runtime_cache(args.runtime_cache, table, _lib.LIB_PATH, table["device"].replace("|", "/").replace("=", "-"))
    resolved = sum(len(s["buckets"]) for s in table["shapes"])
    print(json.dumps({"resolved_buckets": resolved, "shapes": len(table["shapes"]), "out": args.out}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
