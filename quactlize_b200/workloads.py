"""The benchmark configurations as runnable cases: seeded synthetic inputs at the full published sizes, resident on the
device, with everything a checker needs to verify a launch on a sample of its outputs.

A Case owns `ncopies` distinct copies of its weights (enough bytes that one pass over all of them exceeds the 126 MB
L2, so every launch streams from HBM), `launch(i)` enqueues one launch on copy i on torch's current stream, and
`sample()` runs copy 0 once and returns the outputs of a seeded subset of output columns (and activation rows)
together with the HOST inputs that produce them -- the subset is a self-contained small problem that a host
restatement of the format finishes in seconds.  Nothing here computes a reference: the checker lives with the tests.

    cfg1  W4A16 dense GEMV, M=1, K=N=4096, gs=128, fp16                 (generic plane kernel)
    cfg2  GGUF Q4_K raw-block GEMV, M in {1,4,8}, 4096->14336, 14336->4096
    cfg3  bit-plane k-quant GEMV (planes + packed units), M=1, K=4096, N in {4096,14336}, Q6_K / Q5_K / Q3_K
    cfg4  prefill MoE grouped W4A16 GEMM, 8 experts top-2, 4096 tokens Zipf(1.1), hidden 4096, ffn 14336, bf16
    cfg5  decode MoE, 128 experts top-8, hidden 2048, intermediate 768, W2A16 / W1A16 gs=64, bf16, 1..64 tokens
    fpa   dense fpA_intB GEMM, M=2048, N=K=4096, int4 gs=32, fp16
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

import numpy as np
import torch

import quactlize_b200 as qb
from quactlize_b200 import synth

L2_BYTES = 126e6
COLD_BYTES = 300e6            # distinct weight bytes one pass over a case's copies must touch
SAMPLE_COLS = 256


@dataclass
class Case:
    name: str
    bound: str                                   # "hbm" or "tensor": which roofline bounds the launch
    weight_bytes: int                            # packed weight bytes one launch reads (the published numerator)
    alg_bytes: int                               # weights + scale channel + activations + outputs of one launch
    flops: float
    ncopies: int
    launch: Callable[[int], None]
    sample: Callable[[], Dict]
    kernel: str = ""
    notes: Dict = field(default_factory=dict)


def _dev(t, dev):
    return torch.from_numpy(np.ascontiguousarray(t)).to(dev)


def _ncopies(nbytes: int) -> int:
    return max(2, int(np.ceil(COLD_BYTES / nbytes)))


def _cols(n: int, seed: int, count: int = SAMPLE_COLS) -> np.ndarray:
    """A seeded sample of output columns that always holds the first and the last one."""
    rng = np.random.default_rng(seed)
    c = rng.choice(n, size=min(count, n), replace=False)
    c[0], c[-1] = 0, n - 1
    return np.unique(c)


# ---------------------------------------------------------------------------------------------------------------------

def cfg1(dev="cuda:0", n: int = 4096) -> Case:
    k = 4096
    gs, bits = 128, 4
    low, scale, zero = synth.group_planes(1, n, k, bits, gs, seed=101)
    x = synth.activations(1, k, seed=102)
    nc = _ncopies(low.size)
    d0 = tuple(_dev(t, dev) for t in (low, scale, zero))
    copies = [d0] + [tuple(t.clone() for t in d0) for _ in range(nc - 1)]
    xd = _dev(x, dev)

    def launch(i):
        lo, sc, ze = copies[i]
        return qb.gemv_plane(xd, lo, None, sc, ze, bits, 0, gs)

    def sample():
        cols = _cols(n, 103)
        got = launch(0).float().cpu().numpy()[:, cols]
        return {"kind": "planes", "got": got, "a": x, "low": low[:, cols], "high": None, "scale": scale[:, :, cols],
                "zero": zero[:, :, cols], "bits_lo": bits, "bits_hi": 0, "group_size": gs, "row_offsets": None,
                "out": "fp16"}
    wb = n * k * bits // 8
    sz = 2 * (k // gs) * n * 2
    return Case(f"cfg1_w4a16_m1_{n}x4096", "hbm", wb, wb + sz + k * 2 + n * 2, 2.0 * n * k, nc, launch, sample,
                "rowthread_gemv_kernel", {"scale_zero_bytes": sz})


def cfg2(m: int, n: int, k: int, dev="cuda:0", qtype: int = 12) -> Case:
    bb = synth.BLOCK_BYTES[qtype]
    bpr = k // 256
    blocks = synth.kquant_blocks(qtype, n * bpr, seed=200 + n % 97 + m)
    x = synth.activations(m, k, seed=201 + m)
    nc = _ncopies(blocks.size)
    b0 = _dev(blocks, dev)
    copies = [b0] + [b0.clone() for _ in range(nc - 1)]
    xd = _dev(x, dev)

    def launch(i):
        return qb.gguf_vecdot_rows(copies[i], xd, n, k, qtype)

    def sample():
        cols = _cols(n, 202)
        got = launch(0).cpu().numpy()[:, cols]
        sub = blocks.reshape(n, bpr, bb)[cols].reshape(-1, bb)
        return {"kind": "raw", "got": got, "blocks": sub, "x": x, "n": len(cols), "k": k, "qtype": qtype, "out": "fp32"}
    wb = blocks.size
    name = {10: "q2k", 11: "q3k", 12: "q4k", 13: "q5k", 14: "q6k"}.get(qtype, f"qt{qtype}")
    kernel = "kquant_gemv_generic_kernel" if qtype != 12 else "q4k_gemv1_kernel" if m == 1 else "q4k_rows_kernel"
    return Case(f"cfg2_{name}_m{m}_{k}to{n}", "hbm", wb, wb + m * k * 2 + m * n * 4, 2.0 * m * n * k, nc, launch, sample, kernel)


def gate_up_two_buffers(dev="cuda:0") -> Case:
    """Gate and up projections of one layer (two separate Q4_K matrices 4096 -> 14336, one activation) in one launch."""
    n, k, qtype = 14336, 4096, 12
    bb, bpr = synth.BLOCK_BYTES[qtype], k // 256
    ga = synth.kquant_blocks(qtype, n * bpr, seed=231)
    up = synth.kquant_blocks(qtype, n * bpr, seed=232)
    x = synth.activations(1, k, seed=233)
    nc = _ncopies(ga.size + up.size)
    a0, u0 = _dev(ga, dev), _dev(up, dev)
    copies = [(a0, u0)] + [(a0.clone(), u0.clone()) for _ in range(nc - 1)]
    xd = _dev(x, dev)

    def launch(i):
        return qb.gguf_vecdot_dense2(copies[i][0], copies[i][1], xd, n, n, k, qtype)

    def sample():
        cols = _cols(n, 234)
        og, ou = launch(0)
        got = np.concatenate([og.cpu().numpy()[:, cols], ou.cpu().numpy()[:, cols]], axis=1)
        sub = np.concatenate([ga.reshape(n, bpr, bb)[cols], up.reshape(n, bpr, bb)[cols]]).reshape(-1, bb)
        return {"kind": "raw", "got": got, "blocks": sub, "x": x, "n": 2 * len(cols), "k": k, "qtype": qtype, "out": "fp32"}
    wb = ga.size + up.size
    return Case("q4k_m1_gate_up_two_buffers_4096to14336x2", "hbm", wb, wb + k * 2 + 2 * n * 4, 4.0 * n * k, nc, launch, sample,
                "q4k_gemv1_kernel")


def cfg3(qtype: int, n: int, dev="cuda:0") -> Case:
    k = 4096
    bb = synth.BLOCK_BYTES[qtype]
    bpr = k // 256
    blocks = synth.kquant_blocks(qtype, n * bpr, seed=300 + qtype + n % 89)
    x = synth.activations(1, k, seed=301)
    art = qb.gguf_prepare_fully_quantized_dense(torch.from_numpy(blocks), n, k, qtype)
    a0 = tuple(t.to(dev) for t in art)
    nc = _ncopies(blocks.size)
    copies = [a0] + [tuple(t.clone() for t in a0) for _ in range(nc - 1)]
    xd = _dev(x, dev)

    def launch(i):
        lo, hi, un = copies[i]
        return qb.gguf_gemv_bc(xd, lo, hi, un, qtype)

    def sample():
        cols = _cols(n, 302)
        got = launch(0).cpu().numpy()[:, cols]
        sub = blocks.reshape(n, bpr, bb)[cols].reshape(-1, bb)
        return {"kind": "raw", "got": got, "blocks": sub, "x": x, "n": len(cols), "k": k, "qtype": qtype, "out": "fp32"}
    wb = blocks.size                              # planes + units are byte-neutral: exactly the raw block bytes
    nm = {14: "q6k", 13: "q5k", 11: "q3k"}[qtype]
    return Case(f"cfg3_{nm}_m1_{k}to{n}", "hbm", wb, wb + k * 2 + n * 4, 2.0 * n * k, nc, launch, sample,
                "bc_gemv1_kernel")


def cfg4_counts(seed: int = 11) -> np.ndarray:
    return synth.zipf_rows_per_expert(4096, 8, 2, seed=seed)


def cfg4(which: str, dev="cuda:0", gemm: Optional[Callable] = None) -> Case:
    """which = "gate" (hidden 4096 -> ffn 14336) or "down" (14336 -> 4096).  `gemm` overrides the entry that runs it."""
    e, hidden, ffn, gs, bits = 8, 4096, 14336, 128, 4
    n, k = (ffn, hidden) if which == "gate" else (hidden, ffn)
    counts = cfg4_counts()
    rows = int(counts.sum())
    off = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    rng = np.random.default_rng(400 + (which == "down"))
    low = rng.integers(0, 256, size=(e, n, k // 2), dtype=np.uint8)
    scale = (np.abs(rng.normal(0, 0.02, size=(e, k // gs, n))) / 7).astype(np.float16)
    zero = (-8.0 * scale.astype(np.float32)).astype(np.float16)
    a = torch.from_numpy(synth.activations(rows, k, seed=401, dtype=np.float32)).to(torch.bfloat16)
    lo_d, sc_d, ze_d, a_d, off_d = _dev(low, dev), _dev(scale, dev), _dev(zero, dev), a.to(dev), _dev(off, dev)
    run = gemm or (lambda *args, **kw: qb.gemm_plane(*args, **kw))

    def launch(i):
        return run(a_d, lo_d, None, sc_d, ze_d, bits, 0, gs, row_offsets=off_d)

    def sample():
        cols = _cols(n, 402)
        rng2 = np.random.default_rng(403)
        pick, sub_off = [], [0]
        for x in range(e):                        # per expert: first row, last row (ragged tail tile), a few inside
            r0, r1 = int(off[x]), int(off[x + 1])
            if r1 > r0:
                inner = rng2.integers(r0, r1, size=min(6, r1 - r0))
                rr = np.unique(np.concatenate([[r0, r1 - 1], inner]))
                pick.append(rr)
                sub_off.append(sub_off[-1] + len(rr))
            else:
                sub_off.append(sub_off[-1])
        pick = np.concatenate(pick)
        out = launch(0)
        got = out[torch.from_numpy(pick).to(dev)].float().cpu().numpy()[:, cols]
        return {"kind": "planes", "got": got, "a": a[torch.from_numpy(pick)].float().numpy(), "low": low[:, cols],
                "high": None, "scale": scale[:, :, cols], "zero": zero[:, :, cols], "bits_lo": bits, "bits_hi": 0,
                "group_size": gs, "row_offsets": np.asarray(sub_off, np.int32), "out": "bf16"}
    wb = low.size
    flops = 2.0 * rows * n * k
    return Case(f"cfg4_moe_w4a16_{which}", "tensor", wb, wb + 2 * scale.nbytes + rows * k * 2 + rows * n * 2, flops, 1,
                launch, sample, "mixed_gemm_kernel", {"rows": rows, "rows_per_expert": counts.tolist()})


def cfg5(bits: int, which: str, tokens: int, dev="cuda:0", run: Optional[Callable] = None, max_banks: int = 48) -> Case:
    """Decode MoE: 128 experts, top-8 uniform routing, gate_up (2048 -> 2*768) or down (768 -> 2048), W{bits}A16 gs=64.

    One launch touches only the experts its tokens hit, so to stay cold a pass walks `ncopies` expert BANKS (each a
    full set of 128 experts, generated on the device), every launch with its own seeded routing.  Bank 0 is kept on
    the host as well: it is the one `sample()` checks."""
    e, top_k, hidden, inter, gs = 128, 8, 2048, 768, 64
    n, k = (2 * inter, hidden) if which == "gate_up" else (hidden, inter)
    per_expert = n * k * bits // 8
    sz_expert = 2 * (k // gs) * n * 2
    routes = [synth.uniform_routes(tokens, e, top_k, seed=500 + 31 * j + tokens) for j in range(max_banks)]
    counts = [np.bincount(r.reshape(-1), minlength=e) for r in routes]
    active0 = int((counts[0] > 0).sum())
    nb = int(min(max_banks, max(2, np.ceil(COLD_BYTES / (active0 * (per_expert + sz_expert))))))
    low0, scale0, zero0 = synth.group_planes(e, n, k, bits, gs, seed=510 + bits)
    g = torch.Generator(device=dev).manual_seed(520 + bits)
    banks = [tuple(_dev(t, dev) for t in (low0, scale0, zero0))]
    for _ in range(nb - 1):
        lo = torch.randint(0, 256, low0.shape, dtype=torch.uint8, device=dev, generator=g)
        sc = (torch.randn(scale0.shape, device=dev, generator=g).abs() * (0.02 / 7)).to(torch.float16)
        banks.append((lo, sc, (-(2.0 ** (bits - 1)) * sc.float()).to(torch.float16)))
    rows = tokens * top_k
    a = torch.from_numpy(synth.activations(rows, k, seed=530, dtype=np.float32)).to(torch.bfloat16)
    a_d = a.to(dev)
    offs = [np.concatenate([[0], np.cumsum(c)]).astype(np.int32) for c in counts[:nb]]
    offs_d = [_dev(o, dev) for o in offs]
    mrs = [int(c.max()) for c in counts[:nb]]
    fn = run or (lambda a_, lo, sc, ze, off, mr: qb.gemv_plane(a_, lo, None, sc, ze, bits, 0, gs, row_offsets=off, max_rows=mr))

    def launch(i):
        lo, sc, ze = banks[i]
        return fn(a_d, lo, sc, ze, offs_d[i], mrs[i])

    def sample():
        cols = _cols(n, 540, 128)
        got = launch(0).float().cpu().numpy()[:, cols]
        return {"kind": "planes", "got": got, "a": a.float().numpy(), "low": low0[:, cols], "high": None,
                "scale": scale0[:, :, cols], "zero": zero0[:, :, cols], "bits_lo": bits, "bits_hi": 0, "group_size": gs,
                "row_offsets": offs[0], "out": "bf16"}
    act = float(np.mean([(c > 0).sum() for c in counts[:nb]]))
    wb = int(act * per_expert)
    if run is not None:
        return Case(f"cfg5_w{bits}a16_{which}_t{tokens}_splitk", "hbm", wb, int(act * (per_expert + sz_expert)) + rows * k * 2 + rows * n * 2,
                    2.0 * rows * n * k, nb, launch, sample, "mixed_gemm_kernel (split-K) + splitk_reduce_kernel",
                    {"rows": rows, "active_experts_mean": round(act, 1), "banks": nb, "scale_zero_bytes": int(act * sz_expert)})
    return Case(f"cfg5_w{bits}a16_{which}_t{tokens}", "hbm", wb, int(act * (per_expert + sz_expert)) + rows * k * 2 + rows * n * 2,
                2.0 * rows * n * k, nb, launch, sample, "rowmma_gemv_kernel",
                {"rows": rows, "active_experts_mean": round(act, 1), "banks": nb, "scale_zero_bytes": int(act * sz_expert)})


def cfg5_splitk(bits: int, which: str, tokens: int, dev="cuda:0") -> Case:
    """cfg5 through the tensor-core split-K grouped GEMM (128 x 128 tiles, shallow rings, K slices chosen by the library)."""
    gs = 64
    return cfg5(bits, which, tokens, dev,
                run=lambda a_, lo, sc, ze, off, mr: qb.gemm_plane(a_, lo, None, sc, ze, bits, 0, gs, row_offsets=off, split_k=0))


def fpa(dev="cuda:0") -> Case:
    m, n, k, gs, bits = 2048, 4096, 4096, 32, 4
    low, scale, zero = synth.group_planes(1, n, k, bits, gs, seed=600)
    a = synth.activations(m, k, seed=601)
    lo_d, sc_d, ze_d, a_d = _dev(low, dev), _dev(scale, dev), _dev(zero, dev), _dev(a, dev)

    def launch(i):
        return qb.gemm_plane(a_d, lo_d, None, sc_d, ze_d, bits, 0, gs)

    def sample():
        cols = _cols(n, 602)
        rows = np.unique(np.concatenate([[0, m - 1], np.random.default_rng(603).integers(0, m, 30)]))
        got = launch(0)[torch.from_numpy(rows).to(dev)].float().cpu().numpy()[:, cols]
        return {"kind": "planes", "got": got, "a": a[rows], "low": low[:, cols], "high": None, "scale": scale[:, :, cols],
                "zero": zero[:, :, cols], "bits_lo": bits, "bits_hi": 0, "group_size": gs, "row_offsets": None, "out": "fp16"}
    wb = low.size
    return Case("fpa_int4_gs32_m2048_4096x4096", "tensor", wb, wb + 2 * scale.nbytes + m * k * 2 + m * n * 2,
                2.0 * m * n * k, 1, launch, sample, "mixed_gemm_kernel")


def aux_dequant(qtype: int = 12, n: int = 14336, k: int = 4096, dev="cuda:0") -> Case:
    """Raw blocks -> the fp16 weight (the materialisation the dequantise-then-dense route pays): bytes in + bytes out."""
    bb = synth.BLOCK_BYTES[qtype]
    blocks = synth.kquant_blocks(qtype, n * k // 256, seed=700 + qtype)
    b0 = _dev(blocks, dev)
    nc = _ncopies(blocks.size + n * k * 2)
    copies = [b0] + [b0.clone() for _ in range(nc - 1)]
    outs = [torch.empty((n * k // 256, 256), dtype=torch.float16, device=dev) for _ in range(nc)]
    L = qb._lib.lib()

    def launch(i):
        rc = L.quactlize_b200_dequantize_dev_v1(copies[i].data_ptr(), bb, outs[i].data_ptr(), n * k // 256, qtype,
                                                torch.cuda.current_stream().cuda_stream)
        if rc:
            raise RuntimeError(f"dequantize enqueue failed rc={rc}")
        return outs[i]

    def sample():
        rows = _cols(n * k // 256, 701, 512)
        got = launch(0)[torch.from_numpy(rows).to(dev)].cpu().numpy()
        return {"kind": "dequant_bits", "got": got, "blocks": blocks[rows], "qtype": qtype, "out": "fp16"}
    nm = {10: "q2k", 11: "q3k", 12: "q4k", 13: "q5k", 14: "q6k"}[qtype]
    wb = blocks.size
    return Case(f"aux_dequant_{nm}_{k}to{n}", "hbm", wb, wb + n * k * 2, 0.0, nc, launch, sample, "dequant_kernel")


def aux_units_prepass(qtype: int = 12, n: int = 14336, k: int = 4096, dev="cuda:0") -> Case:
    """Packed units -> fp16 scale/zero planes (the workspace pre-pass of the fully-quantized GEMM)."""
    blocks = synth.kquant_blocks(qtype, n * k // 256, seed=710 + qtype)
    units = qb.gguf_pack_units(torch.from_numpy(blocks), n, k, qtype)              # [1, U, n, bytes]
    u0 = units.to(dev)
    g = qb.kquant_geometry(qtype)
    out_bytes = 2 * (k // g.group_size) * n * 2
    nc = _ncopies(units.numel() + out_bytes)
    copies = [u0] + [u0.clone() for _ in range(nc - 1)]

    def launch(i):
        return qb.gguf_packed_scale_prepass(copies[i], qtype, 0)

    def sample():
        cols = _cols(n, 711)
        sc, ze = launch(0)
        got = np.stack([sc[0].cpu().numpy()[:, cols], ze[0].cpu().numpy()[:, cols]])
        return {"kind": "units_bits", "got": got, "units": units[0].numpy()[:, cols], "qtype": qtype, "zmul": 0, "out": "fp16"}
    nm = {10: "q2k", 11: "q3k", 12: "q4k", 13: "q5k", 14: "q6k"}[qtype]
    return Case(f"aux_units_prepass_{nm}_{k}to{n}", "hbm", units.numel(), units.numel() + out_bytes, 0.0, nc, launch, sample,
                "prepass_unit_kernel")


# ---------------------------------------------------------------------------------------------------------------------

FFN = [(14336, 4096), (4096, 14336)]


def registry() -> Dict[str, Callable[[], Case]]:
    """name -> builder of every benchmark case at its full size."""
    r: Dict[str, Callable[[], Case]] = {"cfg1": cfg1}
    for m in (1, 4, 8):
        for n, k in FFN:
            r[f"cfg2_m{m}_{k}to{n}"] = (lambda m=m, n=n, k=k: cfg2(m, n, k))
    for qt, nm in ((14, "q6k"), (13, "q5k"), (11, "q3k")):
        for n in (4096, 14336):
            r[f"cfg3_{nm}_{n}"] = (lambda qt=qt, n=n: cfg3(qt, n))
    for w in ("gate", "down"):
        r[f"cfg4_{w}"] = (lambda w=w: cfg4(w))
    for bits in (2, 1):
        for w in ("gate_up", "down"):
            for t in (1, 8, 64):
                r[f"cfg5_w{bits}_{w}_t{t}"] = (lambda bits=bits, w=w, t=t: cfg5(bits, w, t))
    for w in ("gate_up", "down"):                 # the same decode MoE through the split-K tensor-core grouped GEMM
        for t in (1, 8, 64):
            r[f"cfg5_w2_{w}_t{t}_splitk"] = (lambda w=w, t=t: cfg5_splitk(2, w, t))
    # beside the named configurations: gate and up of one layer as ONE launch (they share the activation: N = 28672),
    # a 264 MB Q4_K matrix (what the single-row kernel streams once the fixed cost of a launch is amortised), and the raw
    # blocks of the other four formats through the raw-block entry
    r["aux_w4a16_m1_32768x4096"] = (lambda: cfg1(n=32768))      # the plane GEMV on a 67 MB matrix
    r["aux_q4k_m1_gate_up_fused"] = (lambda: cfg2(1, 2 * 14336, 4096))
    r["aux_q4k_m1_gate_up_two_buffers"] = gate_up_two_buffers    # the same through the two-matrix entry, separate buffers
    r["aux_q4k_m1_stream_264mb"] = (lambda: cfg2(1, 8 * 14336, 4096))
    for qt, nm in ((10, "q2k"), (11, "q3k"), (13, "q5k"), (14, "q6k")):
        r[f"aux_raw_{nm}_m1_4096to14336"] = (lambda qt=qt: cfg2(1, 14336, 4096, qtype=qt))
    r["fpa"] = fpa
    r["aux_dequant_q4k"] = aux_dequant
    r["aux_dequant_q6k"] = (lambda: aux_dequant(14))
    r["aux_units_prepass_q4k"] = aux_units_prepass
    return r


def time_case(case: Case, batches: int = 5, target_ms: float = 25.0, max_reps: int = 400) -> Dict:
    """Device time of one launch: a CUDA graph of one pass over all copies, replayed; CUDA events on the current
    stream around each of `batches` timed batches; median with the min-max band (microseconds per launch)."""
    for i in range(case.ncopies):
        case.launch(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(case.ncopies):
            case.launch(i)
    for _ in range(3):
        g.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(); g.replay(); e1.record(); torch.cuda.synchronize()
    one = max(e0.elapsed_time(e1), 1e-3)
    reps = int(min(max_reps, max(1, round(target_ms / one))))
    us = []
    for _ in range(batches):
        e0.record()
        for _ in range(reps):
            g.replay()
        e1.record(); torch.cuda.synchronize()
        us.append(e0.elapsed_time(e1) * 1e3 / (reps * case.ncopies))
    us.sort()
    return {"us": us[len(us) // 2], "us_min": us[0], "us_max": us[-1], "launches": batches * reps * case.ncopies,
            "reps": reps}
