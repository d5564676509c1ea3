"""Importer for int4 weights stored in the GPTQ `mixed_gemm` layout of the reference's offline preprocessor.

The reference keeps a second family of int4 artifacts: a [K, N] matrix of signed nibbles, packed two per byte
(`pack_int4`) and rearranged by `preprocess_weights_to_layout(..., "mixed_gemm")` for an Ampere-style mixed-input MMA
(layout name mmarow32_tr_cl4_cvtword_bias).  Its consumer-side inverse is `restore_q4_mixed`
(quactlize/csrc/preprocess/thop/gguf_prepass_ops.cpp:1373-1410); this module restates that inverse with whole-array index
arithmetic and turns the result into the Native code plane this library's kernels read, so a checkpoint stored that way
can be served without going back to raw blocks.  The four stages of the stored layout, undone in reverse order:

  4. converter word order   inside every 8 nibbles, stored position d holds logical position 2d (d < 4) or 2(d-4)+1
  3. column interleave      32-bit words of 4 adjacent columns are interleaved in bands of 8 word-rows (64 k)
  2. sub-byte transpose     the matrix is held [N, K]
  1. MMA row permutation    inside every 32 rows of K, stored row w holds logical row 8*((w%8)//2) + w%2 + 2*(w//8)

Stored nibbles are UNSIGNED codes q (the layout's bias stage turned the signed q-8 back into q).
"""
from __future__ import annotations

import numpy as np
import torch

from . import gguf_packed_scale_prepass

_WORD_SRC = np.array([0, 2, 4, 6, 1, 3, 5, 7])                       # stored nibble d of a word -> logical nibble
_ROW_OF = np.array([8 * ((w % 8) // 2) + w % 2 + 2 * (w // 8) for w in range(32)])


def _nibbles(stored: np.ndarray) -> np.ndarray:
    b = stored.reshape(-1).view(np.uint8)
    out = np.empty(b.size * 2, np.uint8)
    out[0::2] = b & 0xF
    out[1::2] = b >> 4
    return out


def restore_q4_mixed(weight) -> torch.Tensor:
    """Stored `mixed_gemm` int4 weight, int8 [K, N/2] -> unsigned codes uint8 [K, N] in logical row-major order."""
    w = weight.detach().cpu().contiguous().numpy() if isinstance(weight, torch.Tensor) else np.ascontiguousarray(weight)
    if w.ndim != 2 or w.dtype not in (np.int8, np.uint8):
        raise ValueError("processed Q4 weight must be int8 [K,N/2]")
    k, n = w.shape[0], w.shape[1] * 2
    if k % 64 or n % 64:
        raise ValueError("mixed_gemm Q4 artifact needs K and N multiples of 64")
    s = _nibbles(w).reshape(-1, 8)
    words = np.empty_like(s)
    words[:, _WORD_SRC] = s                                           # stage 4: stored position d -> logical position
    vec_rows = k // 8
    nn, kr = np.meshgrid(np.arange(n), np.arange(vec_rows), indexing="ij")
    src = (nn // 4) * vec_rows * 4 + 4 * ((kr // 8) * 8) + 8 * (nn % 4) + kr % 8
    col = words[src.reshape(-1)].reshape(n, k)                        # stage 3: [N, K] nibbles
    perm = col.T                                                      # stage 2: [K, N]
    logical = np.empty_like(perm)
    rows = (np.arange(k) // 32) * 32
    logical[rows + _ROW_OF[np.arange(k) % 32]] = perm                 # stage 1: stored row w -> logical row r
    return torch.from_numpy(np.ascontiguousarray(logical))


def native_plane_from_codes(codes: torch.Tensor) -> torch.Tensor:
    """Unsigned 4-bit codes [K, N] -> this library's Native low plane uint8 [1, N, K/2] (element k of a row at bit 4k)."""
    c = codes.to(torch.uint8).t().contiguous()                        # [N, K]
    return (c[:, 0::2] | (c[:, 1::2] << 4)).unsqueeze(0).contiguous()


def import_mixed_gemm_q4(weight, units):
    """A stored Q4_K artifact of the reference's GPTQ route -- `weight` int8 [K, N/2] in the mixed_gemm layout, `units`
    uint8 [K/256, N, 16] packed scale units -- as (low, high, units) for `gguf_gemv_bc` / `gguf_dense_fully_quantized`."""
    codes = restore_q4_mixed(weight)
    k, n = codes.shape
    if units.dtype != torch.uint8 or tuple(units.shape) != (k // 256, n, 16):
        raise ValueError(f"Q4 artifact units must be uint8 [{k // 256},{n},16], got {tuple(units.shape)}")
    return native_plane_from_codes(codes), torch.empty((0,), dtype=torch.uint8), units.contiguous()


def gguf_q4_artifact_dequantize(weight, units, layout: str = "mixed_gemm") -> torch.Tensor:
    """The reference op of the same name (gguf_prepass_ops.cpp:1419-1452): both offline-shuffled Q4_K artifacts -> the
    float32 weight [K, N] = (code - 8) * scale + zero with the packed unit decoded at ZMul = 8."""
    if layout not in ("mixed_gemm", "mmarow32_tr_cl4_cvtword_bias"):
        raise RuntimeError(f"artifact consumer currently implements the mixed_gemm stored layout, got {layout}")
    codes = restore_q4_mixed(weight)
    k, n = codes.shape
    if k % 256 or tuple(units.shape) != (k // 256, n, 16):
        raise RuntimeError(f"weight K and unit superblocks disagree: K={k} units={tuple(units.shape)}")
    scale, zero = gguf_packed_scale_prepass(units, 12, 8)             # [1, K/32, N]
    s = scale[0].float().cpu().repeat_interleave(32, dim=0)
    z = zero[0].float().cpu().repeat_interleave(32, dim=0)
    return (codes.float() - 8.0) * s + z
