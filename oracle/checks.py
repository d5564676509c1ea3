"""Checker for output samples of the benchmark cases.  TEST INFRASTRUCTURE: imported by tests/, by the smoke test and
by bench.py's parity check (outside every timed region) -- never by the product path.

A sample (quactlize_b200.workloads.Case.sample) is a small self-contained problem: the device's outputs for a seeded
subset of output columns / activation rows plus the host inputs that produce them.  The reference value is the
fp64-accumulated dequantise-then-matmul of oracle.kquant over those inputs.

Error figures:
  max_rel      max|got-ref| / max|ref| over the sample, non-finite = inf  (the reference's GEMV gate,
               tests/test_gemv_lowbit.cu:291-305 in its project; bound 4e-3 there, 1e-2 required here)
  elementwise  the reference's grouped-GEMM gate |err| <= atol + 5e-2*|ref| (tests/test_moe_grouped_real.cu:124), its
               absolute floor 1e-2 scaled to the magnitude of the sample (1e-2 * max(1, max|ref|/10)).
"""
from __future__ import annotations

import numpy as np

from oracle import kquant as kq

# asserted bounds per output type; the requirement is 1e-2 for every one of them
BOUND = {"fp32": 2e-3, "fp16": 3e-3, "bf16": 1e-2}


def reference(sample) -> np.ndarray:
    if sample["kind"] == "raw":
        return kq.vecdot_dense(sample["blocks"], sample["x"], sample["n"], sample["k"], sample["qtype"])
    if sample["kind"] == "planes":
        return kq.planes_matmul(sample["a"], sample["low"], sample["high"], sample["scale"], sample["zero"],
                                sample["bits_lo"], sample["bits_hi"], sample["group_size"], sample["row_offsets"],
                                sample.get("code_offset", 0))
    raise ValueError(sample["kind"])


def _compare_bits(sample) -> dict:
    """Integer / fp16-plane results are compared bit for bit (max_rel is 0 or inf)."""
    if sample["kind"] == "dequant_bits":
        want = kq.dequantize(sample["blocks"], sample["qtype"])
    else:
        sc, ze = kq.units_decode(sample["units"], sample["qtype"], sample["zmul"])
        want = np.stack([sc[0], ze[0]])
    got = np.asarray(sample["got"])
    same = got.shape == want.shape and np.array_equal(got.view(np.uint16), want.view(np.uint16))
    return {"max_rel": 0.0 if same else float("inf"), "elementwise_ok": bool(same), "checked": int(want.size), "bound": 0.0}


def compare(sample) -> dict:
    if sample["kind"] in ("dequant_bits", "units_bits"):
        return _compare_bits(sample)
    ref = reference(sample).astype(np.float64)
    got = np.asarray(sample["got"], dtype=np.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    mr = kq.max_rel(got, ref)
    top = float(np.max(np.abs(ref))) if ref.size else 0.0
    atol = 1e-2 * max(1.0, top / 10.0)
    ok = bool(np.all(np.isfinite(got)) and np.all(np.abs(got - ref) <= atol + 5e-2 * np.abs(ref)))
    return {"max_rel": mr, "elementwise_ok": ok, "checked": int(ref.size), "bound": BOUND[sample["out"]]}


def check(sample) -> dict:
    r = compare(sample)
    assert r["max_rel"] <= r["bound"], r
    assert r["elementwise_ok"], r
    return r
