"""The canonical K-pack carrier of the reference's artifact container, and its bridge to the Native planes that the
kernels of this library read.

K-pack is the on-disk plane order of `reference/gguf_kpack.py` (prepare_dense / prepare_grouped / recover_raw_blocks,
:241-302 for the bit maps): a plane of b bits is a [K/pack, N] array of little-endian 16-bit words, pack = 16/b, the codes
of one word being 8 apart in k.  Word index of code (n, k): kg*N + n with kg = (k // (8*pack))*8 + k % 8; slot
(k % (8*pack)) // 8.  Q5_K's 1-bit high plane has its own transpose.  Codes of the signed formats are offset-binary
(Q3_K +4, Q6_K +32); units are the byte-neutral packed units of `gguf_pack_unit`.

Everything here is index arithmetic on tensors (CPU or CUDA); the permutations are built once per shape and cached.
"""
from __future__ import annotations

from functools import lru_cache
from typing import Tuple

import torch

from . import gguf_prepare_fully_quantized_dense, gguf_prepare_fully_quantized_grouped, gguf_recover_fully_quantized
from .formats import QuantType, kquant_geometry


@lru_cache(maxsize=64)
def _maps(n: int, k: int, bits: int, q5_high: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    """(word index [N, K] int64, bit shift [N, K] int64) of every code of one expert's plane."""
    pack = 16 // bits
    kk = torch.arange(k, dtype=torch.int64)[None, :]
    nn = torch.arange(n, dtype=torch.int64)[:, None]
    if q5_high:
        ncol = (nn & ~15) | (nn & 7) | (((kk >> 7) & 1) << 3)
        kg = (kk // 256) * 16 + (((kk >> 6) & 1) << 3) + (kk & 7)
        slot = (((nn >> 3) & 1) << 3) | ((kk >> 3) & 7)
    else:
        ncol = nn.expand(n, k)
        kg = ((kk // (8 * pack)) * 8 + kk % 8).expand(n, k)
        slot = ((kk % (8 * pack)) // 8).expand(n, k)
    return (kg * n + ncol).contiguous(), (slot * bits).contiguous()


def _native_codes(plane: torch.Tensor, bits: int, k: int) -> torch.Tensor:
    """Native plane bytes [E, N, K*bits/8] -> codes [E, N, K] (element k at bit k*bits, LSB first)."""
    per = 8 // bits
    p = plane.to(torch.int64)
    parts = [(p >> (bits * i)) & ((1 << bits) - 1) for i in range(per)]
    return torch.stack(parts, dim=-1).reshape(plane.shape[0], plane.shape[1], k)


def _native_pack(codes: torch.Tensor, bits: int) -> torch.Tensor:
    per = 8 // bits
    c = codes.reshape(codes.shape[0], codes.shape[1], codes.shape[2] // per, per)
    out = torch.zeros(c.shape[:-1], dtype=torch.int64, device=codes.device)
    for i in range(per):
        out |= (c[..., i] & ((1 << bits) - 1)) << (bits * i)
    return out.to(torch.uint8)


def plane_from_native(plane: torch.Tensor, bits: int, n: int, k: int, q5_high: bool = False) -> torch.Tensor:
    """Native plane [E, N, K*bits/8] -> K-pack carrier bytes of the same shape."""
    if plane.numel() == 0:
        return plane
    e = plane.shape[0]
    idx, shift = (t.to(plane.device) for t in _maps(n, k, bits, q5_high))
    codes = _native_codes(plane, bits, k)
    words = torch.zeros((e, (k * bits // 16) * n), dtype=torch.int64, device=plane.device)
    words.scatter_add_(1, idx.reshape(1, -1).expand(e, -1), (codes << shift[None]).reshape(e, -1))   # slots are disjoint bits: add == or
    lo, hi = (words & 0xFF).to(torch.uint8), (words >> 8).to(torch.uint8)
    return torch.stack((lo, hi), dim=-1).reshape(e, n, k * bits // 8)


def plane_to_native(plane: torch.Tensor, bits: int, n: int, k: int, q5_high: bool = False) -> torch.Tensor:
    """K-pack carrier bytes [E, N, K*bits/8] -> Native plane of the same shape."""
    if plane.numel() == 0:
        return plane
    e = plane.shape[0]
    idx, shift = (t.to(plane.device) for t in _maps(n, k, bits, q5_high))
    b = plane.reshape(e, -1, 2).to(torch.int64)
    words = b[..., 0] | (b[..., 1] << 8)
    codes = (words[:, idx.reshape(-1)].reshape(e, n, k) >> shift[None]) & ((1 << bits) - 1)
    return _native_pack(codes, bits)


def _check(n: int, k: int, qtype: int):
    g = kquant_geometry(int(qtype))
    if n % 256 or k % 256 or (g.hi_bits and int(qtype) in (QuantType.Q3_K, QuantType.Q6_K) and k % 512):
        raise ValueError(f"K-pack needs n % 256 == 0 and k % 256 == 0 (k % 512 for Q3_K / Q6_K); got n={n}, k={k}")
    return g


def prepare_dense(blocks: torch.Tensor, n: int, k: int, qtype: int):
    """Raw blocks [n*k/256, type_size] -> (low, high, units) in the canonical K-pack carrier; units [k/256/P, n, bytes]."""
    g = _check(n, k, qtype)
    low, high, units = gguf_prepare_fully_quantized_dense(blocks, n, k, int(qtype))
    return (plane_from_native(low, g.lo_bits, n, k), plane_from_native(high, g.hi_bits, n, k, int(qtype) == QuantType.Q5_K) if g.hi_bits else high,
            units[0] if units.dim() == 4 else units)


def prepare_grouped(blocks: torch.Tensor, n: int, k: int, qtype: int, experts: int):
    """Expert-major raw blocks -> (low [E,...], high [E,...], units [E, k/256/P, n, bytes])."""
    g = _check(n, k, qtype)
    low, high, units = gguf_prepare_fully_quantized_grouped(blocks, n, k, int(qtype), int(experts))
    return (plane_from_native(low, g.lo_bits, n, k), plane_from_native(high, g.hi_bits, n, k, int(qtype) == QuantType.Q5_K) if g.hi_bits else high, units)


def to_native(low: torch.Tensor, high: torch.Tensor, units: torch.Tensor, n: int, k: int, qtype: int):
    """A K-pack artifact -> the (low, high, units) this library's GEMV / GEMM entries consume (Native planes, units [E,...])."""
    g = _check(n, k, qtype)
    u = units if units.dim() == 4 else units[None]
    return (plane_to_native(low, g.lo_bits, n, k), plane_to_native(high, g.hi_bits, n, k, int(qtype) == QuantType.Q5_K) if g.hi_bits else high, u)


def recover_raw_blocks(low: torch.Tensor, high: torch.Tensor, units: torch.Tensor, n: int, k: int, qtype: int) -> torch.Tensor:
    """K-pack artifact -> the official GGUF blocks, byte for byte."""
    nl, nh, u = to_native(low, high, units, n, k, qtype)
    return gguf_recover_fully_quantized(nl, nh, u, n, k, int(qtype))
