"""quactlize_b200 -- weight-only low-bit matmul for B200 (sm_100a) behind quactlize's Python surface.

The op names, argument order, shapes and error behaviour follow the reference's `quactlize/__init__.py` wrappers
(one function per `torch.ops.quactlize.*` op).  Underneath, every op calls the C-ABI device library
`libquactlize_b200.so` through ctypes:

  * CPU tensors go through the host-pointer entries (the library copies to the device, runs, copies back), exactly
    what the reference's host extension does through its dlopen seam;
  * CUDA tensors go through the `_dev` entries on torch's current stream: nothing is allocated or synchronised by the
    library, the result tensor is allocated by torch.

There is no CPU arm here: a missing library or CUDA device is an error, never a silent fallback.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from .formats import QuantType, kquant_geometry  # noqa: F401

__all__ = [
    "gguf_vecdot", "gguf_vecdot_dense", "gguf_vecdot_rows", "gguf_vecdot_moe", "gguf_dequantize", "gguf_scale_prepass",
    "gguf_packed_scale_prepass", "gguf_prepare_gemv", "gguf_prepare_fully_quantized_dense",
    "gguf_prepare_fully_quantized_grouped", "gguf_recover_fully_quantized", "gguf_gemv_scale_first",
    "gguf_gemv_scale_first_moe", "gguf_gemv_bc", "gguf_gemv_bc_moe", "gemv_plane", "gguf_backend", "gguf_pack_unit",
    "gguf_pack_units", "gguf_unit_decode", "gguf_scale_block_shape", "gguf_unpack", "planes_dequantize",
    "gguf_gemv_artifact_dequantize", "gguf_gemv_artifact_dequantize_scale", "gguf_dense_artifact_dequantize",
    "gguf_dense_artifact_dequantize_scale", "gguf_grouped_artifact_dequantize",
]


def _check(cond, msg):
    if not cond:
        raise RuntimeError(msg)


def _rc(rc, what):
    if rc != 0:
        raise RuntimeError(f"{what} failed in libquactlize_b200 (rc={rc}"
                           f"{'; runtime failure, see stderr' if rc == 41 else ''})")


def _p(t):
    return None if t is None or t.numel() == 0 else C.c_void_p(t.data_ptr())


def _stream(t):
    return C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _same_device(*ts):
    devs = {t.device for t in ts if t is not None and t.numel() > 0}
    _check(len(devs) == 1, f"all tensors must be on one device, got {sorted(str(d) for d in devs)}")
    return next(iter(devs))


def _u8(t, name, dim=None):
    _check(t.dtype == torch.uint8 and t.is_contiguous(), f"{name} must be contiguous uint8")
    if dim is not None:
        _check(t.dim() == dim, f"{name} must be {dim}-D, got {tuple(t.shape)}")


def _f16(x):
    _check(x.dtype in (torch.float16, torch.float32), "activations must be float16 or float32")
    return (x if x.dtype == torch.float16 else x.to(torch.float16)).contiguous()


def _geom(qtype):
    g = kquant_geometry(qtype)
    _check(g is not None, f"unsupported ggml type {qtype} -- expected one of Q2_K=10, Q3_K=11, Q4_K=12, Q5_K=13, Q6_K=14")
    return g


def gguf_backend() -> str:
    """Which backend serves the ops, as the reference reports it ("ppu (...)" / "cpu (...)"); here always the device
    library, or an ImportError from loading it."""
    _lib.lib()
    return f"b200 ({_lib.LIB_PATH})"


# ---------------------------------------------------------------------------------------------------------------------
# raw GGUF block consumers

def gguf_vecdot(blocks, x, qtype: int):
    """One dot product per raw block: blocks uint8 [rows,type_size], x fp16/fp32 [rows,256] -> fp32 [rows]."""
    g = _geom(qtype)
    _u8(blocks, "blocks", 2)
    _check(blocks.shape[1] == g.block_bytes, f"this format's raw GGUF block is {g.block_bytes} bytes, got {blocks.shape[1]}")
    _check(x.dim() == 2 and x.shape[1] == 256 and x.shape[0] == blocks.shape[0], "x must be [rows,256] matching blocks")
    dev = _same_device(blocks, x)
    x16 = _f16(x)
    rows = blocks.shape[0]
    out = torch.empty(rows, dtype=torch.float32, device=dev)
    if rows == 0:
        return out
    L = _lib.lib()
    if dev.type == "cpu":
        _rc(L.quactlize_ppu_vecdot(_p(blocks), g.block_bytes, _p(x16), _p(out), rows, 1, int(qtype)), "gguf_vecdot")
    else:
        with torch.cuda.device(dev):
            _rc(L.quactlize_b200_vecdot_dev_v1(_p(blocks), g.block_bytes, _p(x16), _p(out), rows, 1, int(qtype),
                                               _stream(blocks)), "gguf_vecdot")
    return out


def gguf_vecdot_rows(blocks, x, n: int, k: int, qtype: int, force_generic: bool = False):
    """Raw-block GEMV with m >= 1 shared activation rows: x [m,k] -> fp32 [m,n] (CUDA tensors)."""
    g = _geom(qtype)
    _u8(blocks, "blocks", 2)
    _check(n > 0 and k > 0 and k % 256 == 0, "n must be positive and k a positive multiple of 256")
    _check(blocks.shape == (n * (k // 256), g.block_bytes), f"blocks must be [{n * (k // 256)},{g.block_bytes}], got {tuple(blocks.shape)}")
    _check(x.dim() == 2 and x.shape[1] == k, "x must be [m,k]")
    dev = _same_device(blocks, x)
    _check(dev.type == "cuda", "gguf_vecdot_rows takes CUDA tensors")
    x16 = _f16(x)
    m = x.shape[0]
    out = torch.empty((m, n), dtype=torch.float32, device=dev)
    if m == 0:
        return out
    with torch.cuda.device(dev):
        _rc(_lib.lib().quactlize_b200_vecdot_rows_dev_v1(_p(blocks), g.block_bytes, _p(x16), _p(out), m, n, k // 256,
                                                         int(qtype), int(force_generic), _stream(blocks)), "gguf_vecdot_rows")
    return out


def gguf_vecdot_dense(blocks, x, n: int, k: int, qtype: int):
    """Dense decode GEMV: blocks [n*k/256,type_size], one activation x fp16/fp32 [1,k] -> fp32 [1,n]."""
    g = _geom(qtype)
    _u8(blocks, "blocks", 2)
    _check(x.dim() == 2 and x.shape[0] == 1 and x.shape[1] == k, "x must be fp16/fp32 [1,k]")
    _check(n > 0 and k > 0 and k % 256 == 0, "n must be positive and k a positive multiple of 256")
    bpr = k // 256
    _check(blocks.shape[0] == n * bpr, f"blocks need n*k/256 rows; got {blocks.shape[0]}")
    _check(blocks.shape[1] == g.block_bytes, f"this format's raw GGUF block is {g.block_bytes} bytes, got {blocks.shape[1]}")
    dev = _same_device(blocks, x)
    x16 = _f16(x)
    out = torch.empty((1, n), dtype=torch.float32, device=dev)
    L = _lib.lib()
    if dev.type == "cpu":
        _rc(L.quactlize_ppu_vecdot_dense(_p(blocks), g.block_bytes, _p(x16), _p(out), n, bpr, int(qtype)), "gguf_vecdot_dense")
    else:
        with torch.cuda.device(dev):
            _rc(L.quactlize_ppu_vecdot_dense_dev_v1(_p(blocks), g.block_bytes, _p(x16), _p(out), n, bpr, int(qtype),
                                                    _stream(blocks)), "gguf_vecdot_dense")
    return out


def gguf_vecdot_dense2(blocks_a, blocks_b, x, n_a: int, n_b: int, k: int, qtype: int):
    """Two dense decode GEMVs that share their activation, in one launch (additive; a layer's gate and up projections):
    blocks_a [n_a*k/256,type_size], blocks_b [n_b*k/256,type_size], x fp16/fp32 [1,k] -> (fp32 [1,n_a], fp32 [1,n_b]).
    Device tensors only."""
    g = _geom(qtype)
    _u8(blocks_a, "blocks_a", 2)
    _u8(blocks_b, "blocks_b", 2)
    _check(x.dim() == 2 and x.shape[0] == 1 and x.shape[1] == k, "x must be fp16/fp32 [1,k]")
    _check(n_a > 0 and n_b > 0 and k > 0 and k % 256 == 0, "n_a, n_b must be positive and k a positive multiple of 256")
    bpr = k // 256
    _check(blocks_a.shape[0] == n_a * bpr and blocks_b.shape[0] == n_b * bpr, "blocks need n*k/256 rows")
    _check(blocks_a.shape[1] == g.block_bytes and blocks_b.shape[1] == g.block_bytes,
           f"this format's raw GGUF block is {g.block_bytes} bytes")
    dev = _same_device(blocks_a, x)
    _check(dev.type == "cuda" and blocks_b.device == dev, "gguf_vecdot_dense2 takes tensors of one CUDA device")
    x16 = _f16(x)
    out_a = torch.empty((1, n_a), dtype=torch.float32, device=dev)
    out_b = torch.empty((1, n_b), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _rc(_lib.lib().quactlize_b200_vecdot_dense2_dev_v1(_p(blocks_a), n_a, _p(blocks_b), n_b, g.block_bytes, _p(x16), _p(out_a),
                                                           _p(out_b), bpr, int(qtype), _stream(blocks_a)), "gguf_vecdot_dense2")
    return out_a, out_b


def _offsets_info(row_offsets, experts, total_rows):
    _check(row_offsets.dtype == torch.int32 and row_offsets.dim() == 1 and row_offsets.numel() == experts + 1,
           "row_offsets must be int32 [experts+1]")
    off = row_offsets.detach().cpu()
    _check(int(off[0]) == 0, "row_offsets must start at zero")
    d = off[1:] - off[:-1]
    _check(bool((d >= 0).all()), "row_offsets must be nondecreasing")
    _check(int(off[-1]) == total_rows, f"row_offsets end at {int(off[-1])} but x has {total_rows} rows")
    return int(d.max()) if experts > 0 else 0


def gguf_vecdot_moe(blocks, x, row_offsets, qtype: int):
    """Ragged MoE decode over raw blocks: blocks [E,n*k/256,type_size], gathered x [rows,k], offsets int32 [E+1]
    -> fp32 [rows,n]."""
    g = _geom(qtype)
    _u8(blocks, "blocks", 3)
    _check(x.dim() == 2, "x must be fp16/fp32 [total_rows,k]")
    experts, k = blocks.shape[0], x.shape[1]
    _check(k > 0 and k % 256 == 0, "x's k must be a positive multiple of 256")
    bpr = k // 256
    _check(blocks.shape[1] % bpr == 0, "expert block count must be divisible by k/256")
    n = blocks.shape[1] // bpr
    _check(blocks.shape[2] == g.block_bytes, f"this format's raw GGUF block is {g.block_bytes} bytes, got {blocks.shape[2]}")
    total = x.shape[0]
    max_rows = _offsets_info(row_offsets, experts, total)
    dev = _same_device(blocks, x)
    x16 = _f16(x)
    out = torch.empty((total, n), dtype=torch.float32, device=dev)
    if total == 0:
        return out
    L = _lib.lib()
    off = row_offsets.to(dev).contiguous()
    if dev.type == "cpu":
        _rc(L.quactlize_ppu_vecdot_moe(_p(blocks), g.block_bytes, _p(x16), _p(off), _p(out), n, bpr, experts, total,
                                       max_rows, int(qtype)), "gguf_vecdot_moe")
    else:
        with torch.cuda.device(dev):
            _rc(L.quactlize_b200_vecdot_moe_dev_v1(_p(blocks), g.block_bytes, _p(x16), _p(off), _p(out), n, bpr, experts,
                                                   total, max_rows, int(qtype), _stream(blocks)), "gguf_vecdot_moe")
    return out


def gguf_dequantize(blocks, qtype: int):
    """Raw blocks [rows,type_size] -> fp16 [rows,256], bit-exact half(dl*q - ml)."""
    g = _geom(qtype)
    _u8(blocks, "blocks", 2)
    _check(blocks.shape[1] == g.block_bytes, f"this format's raw GGUF block is {g.block_bytes} bytes, got {blocks.shape[1]}")
    rows = blocks.shape[0]
    out = torch.empty((rows, 256), dtype=torch.float16, device=blocks.device)
    if rows == 0:
        return out
    L = _lib.lib()
    if blocks.device.type == "cpu":
        _rc(L.quactlize_ppu_dequantize(_p(blocks), g.block_bytes, _p(out), rows, int(qtype)), "gguf_dequantize")
    else:
        with torch.cuda.device(blocks.device):
            _rc(L.quactlize_b200_dequantize_dev_v1(_p(blocks), g.block_bytes, _p(out), rows, int(qtype), _stream(blocks)),
                "gguf_dequantize")
    return out


def gguf_scale_prepass(scale_blocks, d, dmin, qtype: int, zmul: int):
    """The format's scale blocks [rows,scale_bytes] + fp16 headers -> fp16 (scale, zero) [rows,groups]; zmul in {0,8}."""
    g = _geom(qtype)
    _u8(scale_blocks, "scale_blocks", 2)
    _check(scale_blocks.shape[1] == g.scale_bytes, f"scale_blocks second dim is {scale_blocks.shape[1]} but this format's scale block is {g.scale_bytes} bytes")
    _check(d.dtype == torch.float16 and d.dim() == 1 and d.shape[0] == scale_blocks.shape[0], "d must be float16 [rows]")
    has = dmin is not None and dmin.numel() > 0
    _check(not g.has_min or has, "this format has a min channel, so dmin is required")
    _check(zmul in (0, 8), f"zmul must be 0 or 8; got {zmul}")
    rows = scale_blocks.shape[0]
    sb, dd = scale_blocks.cpu(), d.cpu().contiguous()
    dm = dmin.cpu().contiguous() if has else None
    scale = torch.empty((rows, g.groups), dtype=torch.float16)
    zero = torch.empty_like(scale)
    _rc(_lib.lib().quactlize_ppu_prepass(_p(sb), g.scale_bytes, _p(dd), _p(dm), rows, _p(scale), _p(zero), g.groups,
                                         int(qtype), int(zmul)), "gguf_scale_prepass")
    return scale.to(scale_blocks.device), zero.to(scale_blocks.device)


def gguf_packed_scale_prepass(units, qtype: int, zmul: int = 0):
    """Packed units (dense [U,n,bytes] or grouped [E,U,n,bytes]) -> fp16 planes (scale, zero) [E, k/group_size, n]."""
    g = _geom(qtype)
    _u8(units, "units")
    _check(units.dim() in (3, 4), "packed units must be dense [unit,n,bytes] or grouped [experts,unit,n,bytes]")
    _check(zmul in (-32, -24, -4, 0, 8), f"zmul must be one of -32, -24, -4, 0, 8; got {zmul}")
    u4 = units if units.dim() == 4 else units.unsqueeze(0)
    experts, nu, n, ub = u4.shape
    _check(ub == g.unit_total, f"this format's copyable unit is {g.unit_total} bytes; got {ub}")
    _check(experts > 0 and nu > 0 and n > 0, "packed unit axes must be nonempty")
    k = nu * g.sb_per_unit * 256
    scale = torch.empty((experts, k // g.group_size, n), dtype=torch.float16, device=units.device)
    zero = torch.empty_like(scale)
    L = _lib.lib()
    if units.device.type == "cpu":
        _rc(L.quactlize_ppu_prepass_unit(_p(u4), _p(scale), _p(zero), n, k, experts, int(qtype), int(zmul)),
            "gguf_packed_scale_prepass")
    else:
        with torch.cuda.device(units.device):
            _rc(L.quactlize_b200_prepass_unit_dev_v1(_p(u4), _p(scale), _p(zero), n, k, experts, int(qtype), int(zmul),
                                                     _stream(units)), "gguf_packed_scale_prepass")
    return scale, zero


# ---------------------------------------------------------------------------------------------------------------------
# offline artifact producers (host work; the result follows the input's device)

def _blocks_cpu(blocks, n, k, g, experts=None):
    _u8(blocks, "blocks")
    _check(blocks.dim() in (2, 3), "blocks must be uint8 [N*K/256,type_size] or [E,N*K/256,type_size]")
    _check(n > 0 and k > 0 and k % 256 == 0, "n must be positive and k a positive multiple of 256")
    e = blocks.shape[0] if blocks.dim() == 3 else 1
    per = blocks.shape[1] if blocks.dim() == 3 else blocks.shape[0]
    if experts is not None:
        _check(blocks.dim() == 2 and blocks.shape[0] == experts * n * (k // 256),
               f"blocks should be [{experts * n * (k // 256)}, type_size] for {experts} experts of an ({n}, {k}) weight, got {tuple(blocks.shape)}")
        e, per = experts, n * (k // 256)
    _check(per == n * (k // 256), f"each expert needs {n * (k // 256)} raw blocks for n={n} k={k}; got {per}")
    _check(blocks.shape[-1] == g.block_bytes, f"this format's raw GGUF block is {g.block_bytes} bytes, got {blocks.shape[-1]}")
    return blocks.cpu().contiguous(), e


def gguf_prepare_gemv(blocks, n: int, k: int, qtype: int):
    """Raw blocks -> the resident scale-first artifact (low, high, scale, zero): Native code planes [E,n,...] and fp16
    planes [E,k/group_size,n]; `high` is empty for single-plane formats."""
    g = _geom(qtype)
    b, e = _blocks_cpu(blocks, n, k, g)
    low = torch.empty((e, n, k * g.lo_bits // 8), dtype=torch.uint8)
    high = torch.empty((e, n, k * g.hi_bits // 8), dtype=torch.uint8) if g.hi_bits else torch.empty((0,), dtype=torch.uint8)
    scale = torch.empty((e, k // g.group_size, n), dtype=torch.float16)
    zero = torch.empty_like(scale)
    _rc(_lib.lib().quactlize_b200_prepare_gemv(_p(b), _p(low), _p(high), _p(scale), _p(zero), n, k, e, int(qtype)),
        "gguf_prepare_gemv")
    dev = blocks.device
    return low.to(dev), high.to(dev), scale.to(dev), zero.to(dev)


def _prepare_fq(blocks, n, k, qtype, experts, dense):
    g = _geom(qtype)
    _check(n % 256 == 0 and k % 256 == 0, "fully-quantized preparation needs n and k multiples of 256")
    _check((k // 256) % g.sb_per_unit == 0, f"this format needs {g.sb_per_unit} superblocks per copyable unit")
    b, e = _blocks_cpu(blocks, n, k, g, experts)
    low = torch.empty((e, n, k * g.lo_bits // 8), dtype=torch.uint8)
    high = torch.empty((e, n, k * g.hi_bits // 8), dtype=torch.uint8) if g.hi_bits else torch.empty((0,), dtype=torch.uint8)
    nu = k // 256 // g.sb_per_unit
    units = torch.empty((e, nu, n, g.unit_total), dtype=torch.uint8)
    _rc(_lib.lib().quactlize_ppu_prepare_fully_quantized_v1(_p(b), _p(low), _p(high), _p(units), n, k, e, int(qtype)),
        "gguf_prepare_fully_quantized")
    if dense:
        units = units[0]
    dev = blocks.device
    return low.to(dev), high.to(dev), units.to(dev)


def gguf_prepare_fully_quantized_dense(blocks, n: int, k: int, qtype: int):
    """Raw blocks [n*k/256,type_size] -> (low [1,n,..], high, units [U,n,bytes]); nothing is expanded."""
    _check(blocks.dim() == 2, "dense preparation takes one [n*k/256,type_size] weight")
    return _prepare_fq(blocks, n, k, qtype, 1, True)


def gguf_prepare_fully_quantized_grouped(blocks, n: int, k: int, qtype: int, experts: int):
    """Raw blocks [E*n*k/256,type_size] (expert-major) -> (low [E,n,..], high, units [E,U,n,bytes])."""
    return _prepare_fq(blocks, n, k, qtype, int(experts), False)


def gguf_recover_fully_quantized(low, high, units, n: int, k: int, qtype: int):
    """Byte-exact inverse of the fully-quantized producers: (low, high, units) -> raw blocks [E*n*k/256,type_size]."""
    g = _geom(qtype)
    e = low.shape[0]
    lo, hi, un = low.cpu().contiguous(), high.cpu().contiguous(), units.cpu().contiguous()
    out = torch.empty((e * n * (k // 256), g.block_bytes), dtype=torch.uint8)
    _rc(_lib.lib().quactlize_ppu_recover_fully_quantized_v1(_p(lo), _p(hi), _p(un), _p(out), n, k, e, int(qtype)),
        "gguf_recover_fully_quantized")
    return out.to(low.device)


def gguf_pack_units(blocks, n: int, k: int, qtype: int, experts: int = 1):
    """Raw blocks -> packed scale units [E,U,n,bytes] only (any n).  Additive: the producer the fully-quantized artifact
    uses, reachable without building the code planes."""
    g = _geom(qtype)
    b, e = _blocks_cpu(blocks, n, k, g, experts)
    _check((k // 256) % g.sb_per_unit == 0, f"this format needs {g.sb_per_unit} superblocks per copyable unit")
    units = torch.empty((e, k // 256 // g.sb_per_unit, n, g.unit_total), dtype=torch.uint8)
    _rc(_lib.lib().quactlize_b200_pack_units(_p(b), _p(units), n, k, e, int(qtype)), "gguf_pack_units")
    return units.to(blocks.device)


_HDR_OFF = {10: (80, 82, 0), 11: (108, -1, 96), 12: (0, 2, 4), 13: (0, 2, 4), 14: (208, -1, 192)}   # d, dmin, scale block


def gguf_pack_unit(scale_blocks, d, dmin, qtype: int):
    """GGUF scale block (+ fp16 headers) -> the reordered, byte-neutral packed unit (the reference op of the same name,
    gguf_prepass_ops.cpp:1253-1311).

    2-D scale_blocks [rows,scale_bytes] with d (and dmin) [rows] -> the row-wise form [rows/P,unit_bytes] (P consecutive
    rows share a unit for Q3_K/Q6_K); 3-D [N,superblocks,scale_bytes] with headers [N,superblocks] -> the stored
    artifact [superblocks/P,N,unit_bytes]."""
    g = _geom(qtype)
    _u8(scale_blocks, "scale_blocks")
    _check(scale_blocks.dim() in (2, 3), "scale_blocks must be uint8 [rows,bytes] or [N,superblocks,bytes]")
    _check(scale_blocks.shape[-1] == g.scale_bytes, "scale_blocks last dim must be the SCALE block")
    _check(d.dtype == torch.float16, "d must be float16")
    artifact = scale_blocks.dim() == 3
    rows = scale_blocks.numel() // g.scale_bytes
    _check(d.numel() == rows and tuple(d.shape) == tuple(scale_blocks.shape[:-1]), "d must match scale_blocks' leading dimensions")
    has = dmin is not None and dmin.numel() > 0
    _check(not g.has_min or has, "this format has a min channel, so dmin is required")
    _check(not has or (dmin.dtype == torch.float16 and dmin.shape == d.shape), "dmin must be float16 with the same shape as d")
    ncols, nsb = (scale_blocks.shape[0], scale_blocks.shape[1]) if artifact else (1, rows)
    _check(nsb % g.sb_per_unit == 0, f"this format packs {g.sb_per_unit} superblocks per unit, so the superblock count "
                                     f"must be a multiple of that; got {nsb}")
    # the block-form producer reads the scale block and the headers at their raw offsets: build blocks holding only those
    d_off, m_off, s_off = _HDR_OFF[int(qtype)]
    raw = torch.zeros((rows, g.block_bytes), dtype=torch.uint8)
    raw[:, s_off:s_off + g.scale_bytes] = scale_blocks.reshape(rows, g.scale_bytes).cpu()
    raw[:, d_off:d_off + 2] = d.reshape(rows).cpu().contiguous().view(torch.uint8).reshape(rows, 2)
    if g.has_min:
        raw[:, m_off:m_off + 2] = dmin.reshape(rows).cpu().contiguous().view(torch.uint8).reshape(rows, 2)
    units = torch.empty((1, nsb // g.sb_per_unit, ncols, g.unit_total), dtype=torch.uint8)
    _rc(_lib.lib().quactlize_b200_pack_units(_p(raw), _p(units), ncols, nsb * 256, 1, int(qtype)), "gguf_pack_unit")
    out = units[0] if artifact else units[0, :, 0, :]
    return out.contiguous().to(scale_blocks.device)


def gguf_unit_decode(units, qtype: int, zmul: int):
    """Packed units -> (scale, zero) fp16, one row per SUPERBLOCK: [superblocks,groups] for the row-wise form
    [rows,unit_bytes], [N,superblocks,groups] for the artifact form [U,N,unit_bytes] (gguf_prepass_ops.cpp:1314-1359)."""
    g = _geom(qtype)
    _u8(units, "units")
    _check(units.dim() in (2, 3), "units must be uint8 [rows,unit] or artifact [unit_sb,N,unit]")
    _check(zmul in (-32, -24, -4, 0, 8), "zmul must be one of -32, -24, -4, 0, 8; it is the consumer's complete code correction")
    _check(units.shape[-1] == g.unit_total, f"this format's unit is {g.unit_total} bytes, got {units.shape[-1]}")
    u3 = units if units.dim() == 3 else units.unsqueeze(1)            # [U, N, bytes]
    scale, zero = gguf_packed_scale_prepass(u3, qtype, zmul)          # [1, U*P*groups, N]
    nu, n = u3.shape[0], u3.shape[1]
    shape = (nu * g.sb_per_unit, g.groups, n)
    s = scale.reshape(shape).permute(2, 0, 1).contiguous()
    z = zero.reshape(shape).permute(2, 0, 1).contiguous()
    return (s, z) if units.dim() == 3 else (s[0], z[0])


def gguf_scale_block_shape(qtype: int):
    """(scale block bytes, groups, group size, has_min, scale bias, signed) of a k-quant's SCALE block."""
    g = _geom(qtype)
    return [g.scale_bytes, g.groups, g.group_size, int(g.has_min), 32 if int(qtype) == 11 else 0, int(int(qtype) == 14)]


def _to_cuda(t):
    return t if t is None or t.is_cuda else t.cuda()


def gguf_unpack(blocks, qtype: int):
    """Raw blocks [rows,type_size] -> (codes int8 [rows,256], scale fp16 [rows,groups], zero fp16 [rows,groups]) with
    W = code*scale + zero; codes are signed for Q3_K (-4..3) and Q6_K (-32..31).  Runs on the device; CPU tensors are
    staged through it and the results come back on the CPU."""
    g = _geom(qtype)
    _u8(blocks, "blocks", 2)
    _check(blocks.shape[1] == g.block_bytes, f"this format's raw GGUF block is {g.block_bytes} bytes, got {blocks.shape[1]}")
    b = _to_cuda(blocks)
    rows = b.shape[0]
    codes = torch.empty((rows, 256), dtype=torch.int8, device=b.device)
    scale = torch.empty((rows, g.groups), dtype=torch.float16, device=b.device)
    zero = torch.empty_like(scale)
    if rows:
        with torch.cuda.device(b.device):
            _rc(_lib.lib().quactlize_b200_unpack_dev_v1(_p(b), g.block_bytes, _p(codes), _p(scale), _p(zero), rows, int(qtype),
                                                        _stream(b)), "gguf_unpack")
    return tuple(t.to(blocks.device) for t in (codes, scale, zero))


def planes_dequantize(low, high, scale, zero, bits_lo: int, bits_hi: int, group_size: int, code_shift: int = 0):
    """Additive: any plane artifact -> fp16 [E,n,k] = half(float(lo + 2^bits_lo*hi + code_shift)*scale + zero), the
    materialisation of the dequantise-then-dense route.  Device kernel; CPU tensors are staged through the device."""
    _u8(low, "low", 3)
    e, n = low.shape[0], low.shape[1]
    k = low.shape[2] * 8 // bits_lo
    if bits_hi:
        _u8(high, "high", 3)
        _check(tuple(high.shape) == (e, n, k * bits_hi // 8), "artifact high plane does not match its scale shape and qtype")
    _check(scale.dtype == torch.float16 and tuple(scale.shape) == (e, k // group_size, n), "scale must be fp16 [E,k/group_size,n]")
    _check(zero is None or (zero.dtype == torch.float16 and zero.shape == scale.shape), "zero must match scale")
    lo, hi, sc, ze = _to_cuda(low), _to_cuda(high) if bits_hi else None, _to_cuda(scale).contiguous(), _to_cuda(zero)
    out = torch.empty((e, n, k), dtype=torch.float16, device=lo.device)
    with torch.cuda.device(lo.device):
        _rc(_lib.lib().quactlize_b200_planes_dequantize_dev_v1(_p(lo), _p(hi) if bits_hi else None, _p(sc),
                                                               _p(ze.contiguous()) if ze is not None else None, _p(out), e, n, k,
                                                               bits_lo, bits_hi, group_size, int(code_shift), _stream(lo)),
            "plane dequantize")
    return out.to(low.device)


def _artifact_dequantize(low, high, scale, zero, qtype, placed):
    g = _geom(qtype)
    _check(low.dtype == torch.uint8 and high.dtype == torch.uint8, "artifact code planes must be uint8")
    _check(low.dim() == 3, "artifact low plane must be [experts,n,packed_k]")
    _check(scale.dtype == torch.float16 and zero.dtype == torch.float16, "artifact scale and zero must be fp16")
    _check(scale.dim() == 3 and scale.shape == zero.shape, "artifact scale and zero must have equal [experts,k/group_size,n] shapes")
    e, sk, n = scale.shape
    k = sk * g.group_size
    _check(tuple(low.shape) == (e, n, k * g.lo_bits // 8), "artifact low plane does not match its scale shape and qtype")
    if g.hi_bits == 0:
        _check(high.numel() == 0, "single-plane artifact must have an empty high plane")
    if placed:
        _check(n % 256 == 0 and k % 256 == 0, "placed artifact inverse needs n/k multiples of 256")
    return planes_dequantize(low, high if g.hi_bits else None, scale, zero, g.lo_bits, g.hi_bits, g.group_size,
                             code_shift=-8 if placed and g.lo_bits == 4 else 0)


def _artifact_dequantize_scale(scale, zero, qtype):
    _geom(qtype)
    _check(scale.dtype == torch.float16 and zero.dtype == torch.float16, "artifact scale and zero must be fp16")
    _check(scale.dim() == 3 and scale.shape == zero.shape, "artifact scale and zero must have equal [experts,k/group_size,n] shapes")
    _check(scale.numel() > 0, "artifact scale planes must be nonempty")
    return scale.transpose(1, 2).contiguous(), zero.transpose(1, 2).contiguous()


def gguf_gemv_artifact_dequantize(low, high, scale, zero, qtype: int):
    """Inverse of `gguf_prepare_gemv`: resident artifact -> fp16 [experts,n,k] (gguf_prepass_ops.cpp:1215-1218)."""
    return _artifact_dequantize(low, high, scale, zero, qtype, False)


def gguf_gemv_artifact_dequantize_scale(scale, zero, qtype: int):
    """The GEMV artifact's affine channels as stored, transposed to [experts,n,k/group_size] (gguf_prepass_ops.cpp:1207-1210)."""
    return _artifact_dequantize_scale(scale, zero, qtype)


def gguf_dense_artifact_dequantize(low, high, scale, zero, qtype: int):
    """Inverse of `gguf_prepare_dense`: int4-low codes decode as (code - 8) against the stored zero plane -> fp16 [1,n,k]."""
    return _artifact_dequantize(low, high, scale, zero, qtype, True)


def gguf_dense_artifact_dequantize_scale(scale, zero, qtype: int):
    """The dense artifact's affine channels as stored, [1,n,k/group_size]."""
    return _artifact_dequantize_scale(scale, zero, qtype)


def gguf_grouped_artifact_dequantize(low, high, scale, zero, qtype: int):
    """The per-expert form of `gguf_dense_artifact_dequantize` -> fp16 [experts,n,k]."""
    return _artifact_dequantize(low, high, scale, zero, qtype, True)


# ---------------------------------------------------------------------------------------------------------------------
# bit-plane GEMV

def _planes_check(a, low, high, g, k):
    _check(a.dim() == 2, "a must be fp16/fp32 [rows,k]")
    _u8(low, "low", 3)
    _check(k > 0 and k % 256 == 0, "a's k must be a positive multiple of 256")
    _check(low.shape[2] == k * g.lo_bits // 8, "low plane byte count disagrees with k/qtype")
    if g.hi_bits:
        _u8(high, "high", 3)
        _check(high.shape == (low.shape[0], low.shape[1], k * g.hi_bits // 8), "high plane shape disagrees with qtype")
    else:
        _check(high is None or high.numel() == 0, "single-plane format must have an empty high plane")


def _scale_first(a, low, high, scale, zero, row_offsets, qtype, grouped):
    g = _geom(qtype)
    k = a.shape[1] if a.dim() == 2 else 0
    _planes_check(a, low, high, g, k)
    e, n = low.shape[0], low.shape[1]
    _check(scale.dtype == torch.float16 and zero.dtype == torch.float16 and scale.shape == zero.shape and
           scale.shape == (e, k // g.group_size, n), "scale and zero must be fp16 [experts,k/group_size,n]")
    rows = a.shape[0]
    dev = _same_device(a, low, scale, zero)
    a16 = _f16(a)
    out = torch.empty((rows, n), dtype=torch.float16, device=dev)
    experts, max_rows, off = 0, rows, None
    if grouped:
        experts = e
        max_rows = _offsets_info(row_offsets, experts, rows)
        off = row_offsets.to(dev).contiguous()
    else:
        _check(e == 1, "dense artifact must have one expert dimension")
    if rows == 0:
        return out
    L = _lib.lib()
    scale, zero = scale.contiguous(), zero.contiguous()
    if dev.type == "cpu":
        _rc(L.quactlize_ppu_gemv_lowbit(_p(a16), _p(low), _p(high), _p(scale), _p(zero), _p(out), rows, n, k,
                                        g.group_size, int(qtype), experts, _p(off), max_rows), "scale-first GEMV")
    else:
        with torch.cuda.device(dev):
            if grouped:
                _rc(L.quactlize_b200_gemv_lowbit_moe_dev_v1(_p(a16), _p(low), _p(high), _p(scale), _p(zero), _p(out), rows,
                                                            n, k, g.group_size, int(qtype), experts, _p(off), max_rows,
                                                            _stream(a16)), "scale-first MoE GEMV")
            else:
                _check(n % 256 == 0, "the device-pointer scale-first entry needs n a multiple of 256")
                _rc(L.quactlize_ppu_gemv_lowbit_dev_v1(_p(a16), _p(low), _p(high), _p(scale), _p(zero), _p(out), rows, n, k,
                                                       g.group_size, int(qtype), _stream(a16), None), "scale-first GEMV")
    return out


def gguf_gemv_scale_first(a, low, high, scale, zero, qtype: int):
    """Dense GEMV over a resident `gguf_prepare_gemv` artifact -> fp16 [rows,n]."""
    return _scale_first(a, low, high, scale, zero, None, qtype, False)


def gguf_gemv_scale_first_moe(a, low, high, scale, zero, row_offsets, qtype: int):
    """Ragged MoE GEMV over a resident `gguf_prepare_gemv` artifact -> fp16 [rows,n]."""
    return _scale_first(a, low, high, scale, zero, row_offsets, qtype, True)


def _bc(a, low, high, units, row_offsets, qtype, grouped):
    g = _geom(qtype)
    k = a.shape[1] if a.dim() == 2 else 0
    _planes_check(a, low, high, g, k)
    e, n = low.shape[0], low.shape[1]
    _check(n > 0 and n % 256 == 0 and k % (256 * g.sb_per_unit) == 0, f"BC GEMV needs n multiple 256 and k multiple {256 * g.sb_per_unit}")
    _u8(units, "units")
    nu = k // 256 // g.sb_per_unit
    rows = a.shape[0]
    dev = _same_device(a, low, units)
    a16 = _f16(a)
    out = torch.empty((rows, n), dtype=torch.float32, device=dev)
    experts, max_rows, off = 0, 1, None
    if grouped:
        _check(units.shape == (e, nu, n, g.unit_total), f"grouped packed units must be [experts,copyable_unit,n,{g.unit_total}]")
        experts = e
        max_rows = _offsets_info(row_offsets, experts, rows)
        off = row_offsets.to(dev).contiguous()
    else:
        _check(rows == 1, "dense BC decode is GEMV and requires exactly one activation row")
        _check(e == 1, "dense BC artifact must have one expert dimension")
        _check(units.shape == (nu, n, g.unit_total), f"dense packed units must be [copyable_unit,n,{g.unit_total}]")
    if rows == 0:
        return out
    L = _lib.lib()
    if dev.type == "cpu":
        _rc(L.quactlize_ppu_bc_gemv(_p(a16), _p(low), _p(high), _p(units), _p(off), _p(out), rows, n, k, experts, max_rows,
                                    int(qtype)), "BC GEMV")
    else:
        with torch.cuda.device(dev):
            _rc(L.quactlize_ppu_bc_gemv_dev_v1(_p(a16), _p(low), _p(high), _p(units), _p(off), _p(out), rows, n, k, experts,
                                               max_rows, int(qtype), _stream(a16)), "BC GEMV")
    return out


def gguf_gemv_bc(a, low, high, units, qtype: int):
    """CUDA-core GEMV over the merged form: Native code planes plus packed scale units -> fp32 [1,n]."""
    return _bc(a, low, high, units, None, qtype, False)


def gguf_gemv_bc_moe(a, low, high, units, row_offsets, qtype: int):
    """The MoE arm; row_offsets is cumulative so an empty expert is representable -> fp32 [rows,n]."""
    return _bc(a, low, high, units, row_offsets, qtype, True)


def gemv_plane(a, low, high, scale, zero, bits_lo: int, bits_hi: int, group_size: int, code_offset: int = 0,
               row_offsets=None, out_dtype=None, max_rows=None):
    """Generic per-group plane GEMV (W4A16 / W2A16 / W1A16 ...): W = (lo + 2^bits_lo*hi + code_offset)*scale + zero.

    a fp16 or bf16 [rows,k] (CUDA); low uint8 [E,n,k*bits_lo/8]; scale (and optional zero) fp16 [E,k/group_size,n];
    dense when row_offsets is None (E == 1), else ragged with cumulative int32 offsets.  Returns [rows,n] in a's dtype
    unless out_dtype (torch.float16 / bfloat16 / float32) says otherwise.  Passing max_rows (an upper bound on any
    expert's row count) skips the host-side validation of a device-resident row_offsets, which would synchronise."""
    _check(a.is_cuda and a.dim() == 2 and a.dtype in (torch.float16, torch.bfloat16), "a must be a CUDA fp16/bf16 [rows,k] tensor")
    _u8(low, "low", 3)
    e, n, k = low.shape[0], low.shape[1], a.shape[1]
    _check(low.shape[2] == k * bits_lo // 8, "low plane byte count disagrees with k/bits")
    if bits_hi:
        _u8(high, "high", 3)
        _check(high.shape == (e, n, k * bits_hi // 8), "high plane shape disagrees with bits_hi")
    _check(scale.dtype == torch.float16 and scale.shape == (e, k // group_size, n), "scale must be fp16 [E,k/group_size,n]")
    _check(zero is None or (zero.dtype == torch.float16 and zero.shape == scale.shape), "zero must match scale")
    out_dtype = out_dtype or a.dtype
    ok = {torch.float16: 0, torch.float32: 1, torch.bfloat16: 2}[out_dtype]
    rows = a.shape[0]
    out = torch.empty((rows, n), dtype=out_dtype, device=a.device)
    experts, bound, off = 0, rows, None
    if row_offsets is not None:
        experts = e
        bound = int(max_rows) if max_rows is not None else _offsets_info(row_offsets, experts, rows)
        _check(0 < bound <= max(rows, 1), "max_rows must bound the rows of any one expert")
        off = row_offsets.to(a.device).contiguous()
    else:
        _check(e == 1, "dense artifact must have one expert dimension")
    if rows == 0:
        return out
    a = a.contiguous()
    with torch.cuda.device(a.device):
        _rc(_lib.lib().quactlize_b200_gemv_plane_dev_v1(
            _p(a), _p(low), _p(high) if bits_hi else None, _p(scale.contiguous()), _p(zero.contiguous()) if zero is not None else None,
            _p(out), rows, n, k, bits_lo, bits_hi, group_size, int(code_offset), 1 if a.dtype == torch.bfloat16 else 0, ok,
            experts, _p(off), bound, _stream(a)), "plane GEMV")
    return out


# ---------------------------------------------------------------------------------------------------------------------
# tensor-core mixed-input GEMM

def gemm_plane(a, low, high, scale, zero, bits_lo: int, bits_hi: int, group_size: int, code_offset: int = 0,
               row_offsets=None, split_k=None):
    """Generic per-group plane GEMM on the tensor cores: D = a @ W^T, W = (lo + 2^bits_lo*hi + code_offset)*scale + zero.

    a fp16/bf16 [rows,k] (CUDA); low uint8 [E,n,k*bits_lo/8]; scale (and optional zero) fp16 [E,k/group_size,n];
    dense when row_offsets is None (E == 1), else grouped with cumulative int32 offsets [E+1] on the device (rows
    gathered in expert order, empty experts allowed).  n % 128 == 0, k % 256 == 0.  Returns [rows,n] in a's dtype.

    split_k selects the decode form: 128 x 128 tiles with shallow rings and K split over that many slices (0 = as many
    as fill the SMs, at most 8; 1 = shallow rings only) whose fp32 partial planes a second small kernel sums."""
    _check(a.is_cuda and a.dim() == 2 and a.dtype in (torch.float16, torch.bfloat16), "a must be a CUDA fp16/bf16 [rows,k] tensor")
    _u8(low, "low", 3)
    e, n, k = low.shape[0], low.shape[1], a.shape[1]
    _check(low.shape[2] == k * bits_lo // 8, "low plane byte count disagrees with k/bits")
    if bits_hi:
        _u8(high, "high", 3)
        _check(high.shape == (e, n, k * bits_hi // 8), "high plane shape disagrees with bits_hi")
    _check(scale.dtype == torch.float16 and scale.shape == (e, k // group_size, n), "scale must be fp16 [E,k/group_size,n]")
    _check(zero is None or (zero.dtype == torch.float16 and zero.shape == scale.shape), "zero must match scale")
    rows = a.shape[0]
    out = torch.empty((rows, n), dtype=a.dtype, device=a.device)
    experts, off = 0, None
    if row_offsets is not None:
        _check(row_offsets.dtype == torch.int32 and row_offsets.numel() == e + 1, "row_offsets must be int32 [experts+1]")
        experts, off = e, row_offsets.to(a.device).contiguous()
    else:
        _check(e == 1, "dense artifact must have one expert dimension")
    if rows == 0:
        return out
    a = a.contiguous()
    if split_k is not None:
        L = _lib.lib()
        need = L.quactlize_b200_gemm_plane_splitk_workspace_bytes_v1(rows, n, int(split_k)) if int(split_k) != 1 else 0
        _check(need >= 0, "split_k must be between 0 and 64")
        ws = torch.empty(max(need, 16), dtype=torch.uint8, device=a.device)
        with torch.cuda.device(a.device):
            _rc(L.quactlize_b200_gemm_plane_splitk_dev_v1(
                _p(a), _p(low), _p(high) if bits_hi else None, _p(scale.contiguous()),
                _p(zero.contiguous()) if zero is not None else None, _p(out), rows, n, k, bits_lo, bits_hi, group_size,
                int(code_offset), 1 if a.dtype == torch.bfloat16 else 0, experts, _p(off), int(split_k), _p(ws), need,
                _stream(a)), "split-K plane GEMM")
        return out
    with torch.cuda.device(a.device):
        _rc(_lib.lib().quactlize_b200_gemm_plane_dev_v1(
            _p(a), _p(low), _p(high) if bits_hi else None, _p(scale.contiguous()),
            _p(zero.contiguous()) if zero is not None else None, _p(out), rows, n, k, bits_lo, bits_hi, group_size,
            int(code_offset), 1 if a.dtype == torch.bfloat16 else 0, experts, _p(off), _stream(a)), "plane GEMM")
    return out


def gguf_prepare_dense(blocks, n: int, k: int, qtype: int):
    """Scale-first dense artifact with the reference's dense contract (gguf_prepass_ops.cpp:884-922): Native planes and
    fp16 planes whose zero carries +8*scale for the int4-low formats, matching a converter that emits (low - 8)."""
    g = _geom(qtype)
    _check(blocks.dim() == 2, "dense preparation takes one [n*k/256,type_size] weight")
    _check(n % 256 == 0 and k % 256 == 0, "dense fpA tactic needs n and k multiples of 256")
    low, high, scale, zero = gguf_prepare_gemv(blocks, n, k, qtype)
    if g.lo_bits == 4:
        zero = (zero.float() + 8.0 * scale.float()).to(torch.float16)
    return low, high, scale, zero


def gguf_dense_scale_first(a, low, high, scale, zero, qtype: int):
    """Dense mixed-input GEMM over a resident `gguf_prepare_dense` artifact -> fp16 [m,n]."""
    g = _geom(qtype)
    k = a.shape[1] if a.dim() == 2 else 0
    _planes_check(a, low, high, g, k)
    n = low.shape[1]
    _check(low.shape[0] == 1 and n % 256 == 0, "dense fpA shape needs one expert and n a multiple of 256")
    _check(scale.dtype == torch.float16 and zero.dtype == torch.float16 and scale.shape == zero.shape == (1, k // g.group_size, n),
           "scale and zero must be fp16 [1,k/group_size,n]")
    m = a.shape[0]
    dev = _same_device(a, low, scale, zero)
    a16 = _f16(a)
    if m == 0:
        return torch.empty((0, n), dtype=torch.float16, device=dev)
    if dev.type == "cpu":
        out = torch.empty((m, n), dtype=torch.float16)
        _rc(_lib.lib().quactlize_ppu_dense_lowbit(_p(a16), _p(low), _p(high), _p(scale.contiguous()), _p(zero.contiguous()), _p(out), m, n, k,
                                                  g.group_size, int(qtype)), "scale-first dense GEMM")
        return out
    return gemm_plane(a16, low, high if g.hi_bits else None, scale, zero, g.lo_bits, g.hi_bits, g.group_size,
                      code_offset=-8 if g.lo_bits == 4 else 0)


def _fq_common(a, low, high, units, g, grouped):
    k = a.shape[1] if a.dim() == 2 else 0
    _planes_check(a, low, high, g, k)
    e, n = low.shape[0], low.shape[1]
    _check(n % 256 == 0 and k % (256 * g.sb_per_unit) == 0, f"fully-quantized GEMM needs n multiple 256 and k multiple {256 * g.sb_per_unit}")
    nu = k // 256 // g.sb_per_unit
    _u8(units, "units")
    want = (e, nu, n, g.unit_total) if grouped else (nu, n, g.unit_total)
    _check(tuple(units.shape) == want, f"packed units must be {list(want)} for this format, got {list(units.shape)}")
    return e, n, k


def gguf_dense_fully_quantized(a, low, high, units, qtype: int):
    """Dense GEMM reading the format's own packed scale bytes (planes + units) -> fp16 [m,n]."""
    g = _geom(qtype)
    e, n, k = _fq_common(a, low, high, units, g, False)
    _check(e == 1, "dense artifact must have one expert dimension")
    m = a.shape[0]
    dev = _same_device(a, low, units)
    a16 = _f16(a)
    out = torch.empty((m, n), dtype=torch.float16, device=dev)
    if m == 0:
        return out
    L = _lib.lib()
    if dev.type == "cpu":
        _rc(L.quactlize_ppu_dense_fully_quantized(_p(a16), _p(low), _p(high), _p(units), _p(out), m, n, k, int(qtype)),
            "fully-quantized dense GEMM")
    else:
        need = L.quactlize_ppu_dense_fully_quantized_workspace_bytes_v1(m, n, k, int(qtype))
        _check(need >= 0, "shape or format refused by the workspace query")
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
        with torch.cuda.device(dev):
            _rc(L.quactlize_ppu_dense_fully_quantized_dev_v1(_p(a16), _p(low), _p(high), _p(units), _p(out), m, n, k, int(qtype),
                                                             _p(ws), need, _stream(a16)), "fully-quantized dense GEMM")
    return out


def gguf_grouped_fully_quantized(a, low, high, units, rows_per_expert, qtype: int):
    """Grouped (MoE) GEMM on packed scale bytes; ragged rows, an expert may have none -> fp16 [total_rows,n]."""
    g = _geom(qtype)
    e, n, k = _fq_common(a, low, high, units, g, True)
    _check(rows_per_expert.dtype == torch.int32 and rows_per_expert.dim() == 1 and rows_per_expert.numel() == e,
           "rows_per_expert must be contiguous int32 [experts]")
    rp = rows_per_expert.detach().cpu().contiguous()
    _check(bool((rp >= 0).all()), "expert row counts must be nonnegative")
    total = int(rp.sum())
    _check(total == a.shape[0], f"rows_per_expert sums to {total} but a has {a.shape[0]} rows")
    dev = _same_device(a, low, units)
    a16 = _f16(a)
    out = torch.empty((total, n), dtype=torch.float16, device=dev)
    if total == 0:
        return out
    L = _lib.lib()
    if dev.type == "cpu":
        _rc(L.quactlize_ppu_grouped_fully_quantized(_p(a16), _p(low), _p(high), _p(units), _p(rp), _p(out), total, n, k, e, int(qtype)),
            "fully-quantized grouped GEMM")
    else:
        off = torch.cat((torch.zeros(1, dtype=torch.int64), rp.to(torch.int64).cumsum(0))).to(torch.int32).to(dev)
        mr = int(rp.max())
        need = L.quactlize_ppu_grouped_fully_quantized_workspace_bytes_v1(max(mr, 1), n, k, e, int(qtype))
        _check(need >= 0, "shape or format refused by the workspace query")
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
        with torch.cuda.device(dev):
            _rc(L.quactlize_ppu_grouped_fully_quantized_dev_v1(_p(a16), _p(low), _p(high), _p(units), _p(off), _p(out), total, n, k, e,
                                                               max(mr, 1), int(qtype), _p(ws), need, _stream(a16)), "fully-quantized grouped GEMM")
    return out


__all__ += ["gemm_plane", "gguf_prepare_dense", "gguf_dense_scale_first", "gguf_dense_fully_quantized", "gguf_grouped_fully_quantized"]
