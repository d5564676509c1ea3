"""Artifacts placed by the reference's device library ("xplane" order) <-> the Native planes this library reads.

The reference's tensor-core producers (`gguf_prepare_dense`, `gguf_prepare_fully_quantized_*` through its device
library) store code planes in 64-column x TileK tiles with a bit permutation inside each tile; the inverse maps are
stated in quactlize/include/gguf_bc_vecdot.hpp:34-95.  `to_native` converts such planes at load so every kernel here can
consume them; `from_native` is the same map the other way (a weight prepared here can be handed to a consumer of the
placed order).  Scale units and fp16 planes are not placed: they pass through unchanged.
"""
from __future__ import annotations

import torch

from . import _lib
from .formats import kquant_geometry


def _convert(low, high, n: int, k: int, qtype: int, to_native: bool):
    g = kquant_geometry(int(qtype))
    if g is None:
        raise RuntimeError(f"unsupported ggml type {qtype}")
    if low.dtype != torch.uint8 or low.dim() != 3 or tuple(low.shape[1:]) != (n, k * g.lo_bits // 8):
        raise RuntimeError(f"low plane must be uint8 [E,{n},{k * g.lo_bits // 8}], got {tuple(low.shape)}")
    e = low.shape[0]
    if g.hi_bits and (high is None or tuple(high.shape) != (e, n, k * g.hi_bits // 8)):
        raise RuntimeError("high plane shape disagrees with the format")
    if n % 64 or k % 256:
        raise RuntimeError("placed planes need n a multiple of 64 and k a multiple of 256")
    lo_in = low.cpu().contiguous()
    hi_in = high.cpu().contiguous() if g.hi_bits else None
    lo_out = torch.empty_like(lo_in)
    hi_out = torch.empty_like(hi_in) if g.hi_bits else torch.empty((0,), dtype=torch.uint8)
    fn = _lib.lib().quactlize_b200_xplane_to_native if to_native else _lib.lib().quactlize_b200_native_to_xplane
    for x in range(e):                                             # the placement is per expert
        rc = fn(lo_in[x].data_ptr(), hi_in[x].data_ptr() if g.hi_bits else None, lo_out[x].data_ptr(),
                hi_out[x].data_ptr() if g.hi_bits else None, n, k, int(qtype))
        if rc:
            raise RuntimeError(f"xplane conversion failed (rc={rc})")
    return lo_out.to(low.device), hi_out.to(low.device)


def to_native(low, high, n: int, k: int, qtype: int):
    """Placed (low, high) planes [E,n,bytes] -> Native planes of the same shapes."""
    return _convert(low, high, n, k, qtype, True)


def from_native(low, high, n: int, k: int, qtype: int):
    """Native (low, high) planes [E,n,bytes] -> the reference's placed order."""
    return _convert(low, high, n, k, qtype, False)


def slot(qtype: int, high: bool, n: int, k: int, num_cols: int) -> int:
    """Placed code index of logical (n, k) in a plane of num_cols columns."""
    return int(_lib.lib().quactlize_b200_xplane_slot(int(qtype), int(bool(high)), n, k, num_cols))
