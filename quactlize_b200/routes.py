"""The host side of each route -- same names, argument order and error behaviour as the reference's
`quactlize/routes.py`, so a caller can switch packages without touching call sites.

Shape convention (quactlize/routes.py:19-23): a GGUF weight of logical shape (n, k) is n*(k/256) raw blocks in
ROW-MAJOR order -- block b of output row i sits at flat index i*(k/256)+b; grouped weights are expert-major.
Grouped activations are already gathered in expert order; `rows_per_expert` must sum to the activation rows and an
expert may have none.
"""
from __future__ import annotations

from typing import Optional

import torch

import quactlize_b200 as _pkg
from . import (gguf_dequantize, gguf_vecdot_dense, gguf_vecdot_moe, gguf_prepare_gemv, gguf_gemv_scale_first,
               gguf_gemv_scale_first_moe, gguf_packed_scale_prepass, gguf_gemv_bc, gguf_gemv_bc_moe,
               gguf_prepare_fully_quantized_dense, gguf_prepare_fully_quantized_grouped, gguf_vecdot_rows,
               gguf_prepare_dense, gguf_dense_scale_first, gguf_dense_fully_quantized, gguf_grouped_fully_quantized,
               gguf_gemv_artifact_dequantize, gguf_gemv_artifact_dequantize_scale, gguf_dense_artifact_dequantize,
               gguf_dense_artifact_dequantize_scale, gguf_grouped_artifact_dequantize)
from .formats import QuantType, placed_code_zmul, select_path


def _check_shape(blocks: torch.Tensor, n: int, k: int, qtype: int) -> None:
    if k % 256:
        raise ValueError(f"k={k} is not a multiple of the k-quant superblock (256)")
    want = n * (k // 256)
    if blocks.dim() != 2 or blocks.shape[0] != want:
        raise ValueError(f"blocks should be [{want}, type_size] for an ({n}, {k}) weight in {QuantType(qtype).name}, "
                         f"got {tuple(blocks.shape)}. Row-major: block b of row i sits at i*(k/256)+b")


def dequantize_weight(blocks, n: int, k: int, qtype: int):
    """Raw GGUF blocks -> the fp16 weight (n, k) (quactlize/routes.py:39-43)."""
    _check_shape(blocks, n, k, qtype)
    return gguf_dequantize(blocks, int(qtype)).view(n, k)


def matmul_dequant_first(a, blocks, n: int, k: int, qtype: int, weight: Optional[torch.Tensor] = None):
    """DEQUANT_FIRST, dense: expand to fp16 (bit-exact device kernel), then a library GEMM.  a (m,k) -> (m,n).
    `weight` hoists the materialisation out of a timing loop (quactlize/routes.py:46-63)."""
    if weight is None:
        weight = dequantize_weight(blocks, n, k, qtype)
    if a.shape[-1] != k:
        raise ValueError(f"activation has k={a.shape[-1]}, weight has k={k}")
    return a.to(weight.dtype) @ weight.t()


def matmul_dequant_first_grouped(a, blocks, n: int, k: int, qtype: int, num_experts: int, rows_per_expert):
    """DEQUANT_FIRST, grouped: one library GEMM per non-empty expert (quactlize/routes.py:66-90)."""
    if rows_per_expert.numel() != num_experts:
        raise ValueError(f"rows_per_expert has {rows_per_expert.numel()} entries, expected {num_experts}")
    total = int(rows_per_expert.sum().item())
    if total != a.shape[0]:
        raise ValueError(f"rows_per_expert sums to {total}, activation has {a.shape[0]} rows")
    per_expert = n * (k // 256)
    _check_shape(blocks, n * num_experts, k, qtype)
    out = a.new_empty((a.shape[0], n), dtype=torch.float16)
    start = 0
    for e in range(num_experts):
        rows = int(rows_per_expert[e].item())
        if rows == 0:
            continue
        w = dequantize_weight(blocks[e * per_expert:(e + 1) * per_expert], n, k, qtype)
        out[start:start + rows] = a[start:start + rows].to(torch.float16) @ w.t()
        start += rows
    return out


def matmul_native_gemv(a, blocks, n: int, k: int, qtype: int):
    """FULLY_QUANTIZED GEMV over raw blocks: a (1,k) fp16/fp32 -> (1,n) fp32 (quactlize/routes.py:93-104)."""
    _check_shape(blocks, n, k, qtype)
    if a.shape[0] != 1:
        raise ValueError(f"the GEMV band is m=1; got m={a.shape[0]}")
    return gguf_vecdot_dense(blocks, a.to(torch.float16).contiguous(), n, k, int(qtype))


def matmul_native_gemv_rows(a, blocks, n: int, k: int, qtype: int):
    """Additive: the same route for a small batch of rows, a (m,k) -> (m,n) fp32 (CUDA tensors)."""
    _check_shape(blocks, n, k, qtype)
    return gguf_vecdot_rows(blocks, a.to(torch.float16).contiguous(), n, k, int(qtype))


def _row_offsets(rows_per_expert, experts: int, total_rows: int):
    if rows_per_expert.numel() != experts:
        raise ValueError(f"rows_per_expert has {rows_per_expert.numel()} entries, expected {experts}")
    rows = rows_per_expert.to(dtype=torch.int64, device="cpu")
    if bool((rows < 0).any()):
        raise ValueError("rows_per_expert must be nonnegative")
    if int(rows.sum().item()) != total_rows:
        raise ValueError(f"rows_per_expert sums to {int(rows.sum().item())}, activation has {total_rows} rows")
    return torch.cat((torch.zeros(1, dtype=torch.int64), rows.cumsum(0))).to(torch.int32).contiguous()


def matmul_native_gemv_moe(a, blocks, n: int, k: int, qtype: int, num_experts: int, rows_per_expert):
    """FULLY_QUANTIZED MoE decode: raw blocks, gathered rows, one launch (quactlize/routes.py:118-132)."""
    if a.dim() != 2 or a.shape[1] != k:
        raise ValueError(f"activation must be [total_rows,{k}], got {tuple(a.shape)}")
    want = n * (k // 256)
    if blocks.dim() == 2:
        if blocks.shape[0] != num_experts * want:
            raise ValueError(f"flat blocks need {num_experts * want} rows, got {blocks.shape[0]}")
        blocks = blocks.view(num_experts, want, blocks.shape[1])
    if blocks.dim() != 3 or tuple(blocks.shape[:2]) != (num_experts, want):
        raise ValueError(f"blocks must be [{num_experts},{want},type_size], got {tuple(blocks.shape)}")
    offsets = _row_offsets(rows_per_expert, num_experts, a.shape[0])
    return gguf_vecdot_moe(blocks.contiguous(), a, offsets.to(a.device), int(qtype))


def prepare_scale_first(blocks, n: int, k: int, qtype: int):
    """Offline artifact of both scale-first decode shapes: (low, high, scale, zero) (quactlize/routes.py:135-148)."""
    return gguf_prepare_gemv(blocks, n, k, int(qtype))


def matmul_scale_first_gemv(a, artifact, qtype: int):
    """SCALE_FIRST GEMV over prebuilt planes -> fp16 (quactlize/routes.py:161-164)."""
    low, high, scale, zero = artifact
    return gguf_gemv_scale_first(a, low, high, scale, zero, int(qtype))


def matmul_scale_first_gemv_moe(a, artifact, qtype: int, rows_per_expert):
    """SCALE_FIRST ragged MoE GEMV (quactlize/routes.py:167-173)."""
    low, high, scale, zero = artifact
    offsets = _row_offsets(rows_per_expert, int(low.shape[0]), a.shape[0])
    return gguf_gemv_scale_first_moe(a, low, high, scale, zero, offsets.to(a.device), int(qtype))


def _unpack_fq(artifact, where: str):
    xs = list(artifact)
    if len(xs) != 3:
        raise ValueError(f"{where}: the artifact has {len(xs)} tensor(s); the contract is (low, high, units) -- three, "
                         f"with `high` an EMPTY tensor for a single-plane format. shapes seen: {[tuple(x.shape) for x in xs]}")
    return xs[0], xs[1], xs[2]


def has_op(name: str) -> bool:
    """Whether an op of the reference's registry exists in this build (quactlize/routes.py:228-243).  Here every op is
    a function of the package, so the package namespace is the registry."""
    return callable(getattr(_pkg, name, None))


def dequantize_scale_from_units(units, qtype: int, zmul: Optional[int] = None):
    """Packed scale units -> fp16 (scale, zero) planes [E, k/group_size, n] (quactlize/routes.py:262-288).

    zmul is the consumer's complete code correction and is DERIVED from the format when not given: the placed dense
    contract's table (Q2_K 0, Q3_K -4, Q4_K 8, Q5_K 8, Q6_K -24: int4-low codes convert as low-8, signed formats are
    stored offset-binary).  A consumer that reads the offset-binary plane codes directly (the plane GEMVs of this
    library) passes minus the format's code bias instead."""
    if zmul is None:
        zmul = placed_code_zmul(qtype)
    return gguf_packed_scale_prepass(units, int(qtype), int(zmul))


def dequantize_scale_first(artifact, qtype: int):
    """GEMV scale-first artifact -> fp16 [experts,n,k], without running a GEMV (quactlize/routes.py:151-153)."""
    return gguf_gemv_artifact_dequantize(*artifact, int(qtype))


def dequantize_scale_first_scales(artifact, qtype: int):
    """GEMV scale-first artifact -> the stored (scale, zero) planes as [experts,n,k/group_size] (quactlize/routes.py:156-158)."""
    return gguf_gemv_artifact_dequantize_scale(artifact[2], artifact[3], int(qtype))


def prepare_scale_first_dense(blocks, n: int, k: int, qtype: int, derive_from_bc: bool = True):
    """Offline artifact (low, high, scale, zero) of the dense scale-first GEMM (quactlize/routes.py:176-199).  By default
    the fp16 planes are DERIVED from the packed units of the fully-quantized artifact; derive_from_bc=False keeps the
    independent producer from raw blocks reachable (the two are compared bit for bit by the tests)."""
    _check_shape(blocks, n, k, qtype)
    if not derive_from_bc:
        return gguf_prepare_dense(blocks, n, k, int(qtype))
    low, high, units = gguf_prepare_fully_quantized_dense(blocks, n, k, int(qtype))
    scale, zero = dequantize_scale_from_units(units, qtype)
    return low, high, scale, zero


def dequantize_scale_first_dense(artifact, qtype: int):
    """Dense scale-first artifact -> fp16 [1,n,k], without running a GEMM (quactlize/routes.py:202-204)."""
    return gguf_dense_artifact_dequantize(*artifact, int(qtype))


def dequantize_scale_first_dense_scales(artifact, qtype: int):
    """Dense scale-first artifact -> the stored (scale, zero) planes [1,n,k/group_size] (quactlize/routes.py:207-209)."""
    return gguf_dense_artifact_dequantize_scale(artifact[2], artifact[3], int(qtype))


def dequantize_fully_quantized(artifact, qtype: int, grouped: bool = False):
    """(low, high, units) -> the fp16 weight [experts,n,k]: the scale planes derived from the units, then the
    scale-first dequantise-all -- a composition, not a second decoder (quactlize/routes.py:322-349)."""
    low, high, units = _unpack_fq(artifact, "dequantize_fully_quantized")
    scale, zero = dequantize_scale_from_units(units, qtype)
    op = gguf_grouped_artifact_dequantize if grouped else gguf_dense_artifact_dequantize
    return op(low, high, scale, zero, int(qtype))


def prepare_fully_quantized_dense(blocks, n: int, k: int, qtype: int, tile_k=None):
    """Offline artifact (low, high, units): code planes plus the packed scale unit, nothing expanded
    (quactlize/routes.py:344-364).  tile_k is accepted for call compatibility; planes here are tile-free."""
    _check_shape(blocks, n, k, int(qtype))
    return gguf_prepare_fully_quantized_dense(blocks, n, k, int(qtype))


def prepare_fully_quantized_grouped(blocks, n: int, k: int, qtype: int, experts: int):
    """The MoE artifact, expert-major blocks in, (low, high, units) out (quactlize/routes.py:378-388)."""
    want = experts * n * (k // 256)
    if blocks.dim() != 2 or blocks.shape[0] != want:
        raise ValueError(f"blocks should be [{want}, type_size] for {experts} experts of an ({n}, {k}) weight, "
                         f"got {tuple(blocks.shape)}")
    return gguf_prepare_fully_quantized_grouped(blocks, n, k, int(qtype), int(experts))


def matmul_bc_gemv(a, artifact, qtype: int):
    """Decode GEMV off the merged form (planes + packed units) -> fp32 [1,n] (quactlize/routes.py:291-305)."""
    low, high, units = _unpack_fq(artifact, "matmul_bc_gemv")
    return gguf_gemv_bc(a, low, high, units, int(qtype))


def matmul_bc_gemv_moe(a, artifact, qtype: int, num_experts: int, rows_per_expert):
    """The MoE arm of the merged-form GEMV (quactlize/routes.py:308-319)."""
    low, high, units = _unpack_fq(artifact, "matmul_bc_gemv_moe")
    offsets = _row_offsets(rows_per_expert, num_experts, a.shape[0])
    return gguf_gemv_bc_moe(a, low, high, units, offsets.to(a.device), int(qtype))


def matmul_fully_quantized_dense(a, artifact, qtype: int):
    """a @ w.T with nothing expanded: the tensor-core GEMM reads planes + packed units (quactlize/routes.py:367-375)."""
    low, high, units = _unpack_fq(artifact, "matmul_fully_quantized_dense")
    return gguf_dense_fully_quantized(a, low, high, units, int(qtype))


def matmul_fully_quantized_grouped(a, artifact, qtype: int, rows_per_expert):
    """The grouped GEMM on planes + packed units; rows are ragged and an expert may have none
    (quactlize/routes.py:391-399)."""
    low, high, units = _unpack_fq(artifact, "matmul_fully_quantized_grouped")
    return gguf_grouped_fully_quantized(a, low, high, units, rows_per_expert.to(torch.int32), int(qtype))


def matmul_scale_first_dense(a, artifact, qtype: int):
    """SCALE_FIRST/DENSE: packed codes and resident fp16 planes on the tensor cores (quactlize/routes.py:402-405)."""
    low, high, scale, zero = artifact
    return gguf_dense_scale_first(a, low, high, scale, zero, int(qtype))


def matmul_selected(a, artifact, qtype: int, fp16_planes: str = "workspace"):
    """Additive: run a dense matmul over a fully-quantized artifact (low, high, units) on the path `formats.select_path`
    names for this row count (quactlize/formats.py:175-219).  `gemv` is the merged-form decode GEMV (planes + units, no
    fp16 planes at all), `fused_native_scale` / `fused_fp16_scale` the tensor-core GEMM on the same bytes, and
    `dequant_then_dense` materialises the fp16 weight with the device dequantiser and hands it to a library GEMM --
    the fallback above the crossover.  Returns (path name, result); the result's dtype is the path's own."""
    low, high, units = _unpack_fq(artifact, "matmul_selected")
    path = select_path(QuantType(int(qtype)), int(a.shape[0]), True, fp16_planes)
    if path == "gemv":
        return path, matmul_bc_gemv(a, artifact, qtype)
    if path in ("fused_native_scale", "fused_fp16_scale"):
        return path, matmul_fully_quantized_dense(a, artifact, qtype)
    w = dequantize_fully_quantized(artifact, qtype)[0]
    return path, a.to(w.dtype) @ w.t()


ROUTES = {
    "dequant_first": matmul_dequant_first,
    "native_gemv": matmul_native_gemv,
    "native_gemv_moe": matmul_native_gemv_moe,
    "scale_first_gemv": matmul_scale_first_gemv,
    "scale_first_gemv_moe": matmul_scale_first_gemv_moe,
    "scale_first_dense": matmul_scale_first_dense,
    "bc_gemv": matmul_bc_gemv,
    "bc_gemv_moe": matmul_bc_gemv_moe,
    "fully_quantized_dense": matmul_fully_quantized_dense,
    "fully_quantized_grouped": matmul_fully_quantized_grouped,
}
