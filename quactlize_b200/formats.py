"""Format table and path selection -- the host-side surface of `quactlize.formats`, kept so callers can switch over.

Same names and semantics as the reference module (quactlize/formats.py): `QuantType` (ggml numbers), `BLOCKS`
(per-format block layout and storage arithmetic), the capability sets, `select_path`, `storage_growth`,
`needs_native_scale`, `fold_for`, `PlacedArrangement`, `placed_code_zmul`, `report`.  What differs is what the sets
mean on B200: every k-quant has a raw-block GEMV, a scale-first GEMV, a merged-artifact GEMV and the tensor-core GEMMs
in one library, and the placed arrangement of this library is the Native plane order (fold is always 1).
"""
from __future__ import annotations

from enum import IntEnum
from typing import Dict, FrozenSet, NamedTuple, Optional


class QuantType(IntEnum):
    """ggml type numbers (quactlize/formats.py:26-45); non-GGUF formats sit above the ggml range."""
    Q4_0 = 2
    Q4_1 = 3
    Q5_0 = 6
    Q5_1 = 7
    Q8_0 = 8
    Q2_K = 10
    Q3_K = 11
    Q4_K = 12
    Q5_K = 13
    Q6_K = 14
    GPTQ_INT4_SYM = 1000
    GPTQ_INT4_ASYM = 1001
    AWQ_INT4 = 1002


class BlockLayout(NamedTuple):
    """Bytes of one quantisation block: total, the part that encodes scales/mins, group size, affine or not
    (quactlize/formats.py:48-80)."""
    weights: int
    block_bytes: int
    scale_meta_bytes: int
    group_size: int
    has_min: bool

    @property
    def fp16_plane_bytes(self) -> int:
        return (self.weights // self.group_size) * 2 * (2 if self.has_min else 1)

    @property
    def bytes_on_fp16_scale_path(self) -> int:
        return self.block_bytes - self.scale_meta_bytes + self.fp16_plane_bytes

    @property
    def fp16_scale_growth(self) -> float:
        return self.bytes_on_fp16_scale_path / self.block_bytes - 1.0


BLOCKS: Dict[QuantType, BlockLayout] = {
    QuantType.Q4_0: BlockLayout(32, 18, 2, 32, False),
    QuantType.Q4_1: BlockLayout(32, 20, 4, 32, True),
    QuantType.Q5_0: BlockLayout(32, 22, 2, 32, False),
    QuantType.Q5_1: BlockLayout(32, 24, 4, 32, True),
    QuantType.Q8_0: BlockLayout(32, 34, 2, 32, False),
    QuantType.Q2_K: BlockLayout(256, 84, 20, 16, True),
    QuantType.Q3_K: BlockLayout(256, 110, 14, 16, False),
    QuantType.Q4_K: BlockLayout(256, 144, 16, 32, True),
    QuantType.Q5_K: BlockLayout(256, 176, 16, 32, True),
    QuantType.Q6_K: BlockLayout(256, 210, 18, 16, False),
}

NON_BLOCK_SCALE_GROWTH: Dict[QuantType, Optional[float]] = {
    QuantType.GPTQ_INT4_SYM: 0.0, QuantType.GPTQ_INT4_ASYM: None, QuantType.AWQ_INT4: None,
}


class KQuantGeometry(NamedTuple):
    """Everything the op wrappers need to validate shapes of one k-quant: raw block bytes, groups, plane widths, the
    scale block inside the raw block, and the packed-unit geometry (quactlize/include/gguf_packed_unit.hpp:39-107)."""
    block_bytes: int
    groups: int
    group_size: int
    lo_bits: int
    hi_bits: int
    has_min: bool
    scale_bytes: int
    code_bias: int
    sb_bytes: int
    sb_per_unit: int
    unit_total: int


def _geo(bb, groups, lo, hi, has_min, scale_bytes, bias, sbits, mbits):
    sb = (4 if has_min else 2) + groups * (sbits + mbits) // 8
    p = 1 if sb % 4 == 0 else 2
    return KQuantGeometry(bb, groups, 256 // groups, lo, hi, has_min, scale_bytes, bias, sb, p, sb * p)


_KQ = {
    10: _geo(84, 16, 2, 0, True, 16, 0, 4, 4),
    11: _geo(110, 16, 2, 1, False, 12, 4, 6, 0),
    12: _geo(144, 8, 4, 0, True, 12, 0, 6, 6),
    13: _geo(176, 8, 4, 1, True, 12, 0, 6, 6),
    14: _geo(210, 16, 4, 2, False, 16, 32, 8, 0),
}


def kquant_geometry(qtype) -> Optional[KQuantGeometry]:
    return _KQ.get(int(qtype))


_K = frozenset({QuantType.Q2_K, QuantType.Q3_K, QuantType.Q4_K, QuantType.Q5_K, QuantType.Q6_K})
#: single-token CUDA-core GEMV over a resident artifact (quactlize/formats.py:135-141)
GEMV: FrozenSet[QuantType] = frozenset({QuantType.GPTQ_INT4_SYM}) | _K
#: fused mixed-input tensor-core GEMM with fp16 scale planes
FUSED_FP16_SCALE: FrozenSet[QuantType] = frozenset({QuantType.GPTQ_INT4_SYM}) | _K
#: fused GEMM / GEMV reading the format's own packed scale bytes
FUSED_NATIVE_SCALE: FrozenSet[QuantType] = _K
#: dequantise to fp16, then a dense library GEMM
DEQUANT_THEN_DENSE: FrozenSet[QuantType] = _K

DENSE_CROSSOVER_ROWS = 512      # above this the dense path's extra pass over the weights is repaid (formats.py:166-169)
GEMV_MAX_ROWS = 1               # the decode band


def storage_growth(qtype: QuantType) -> Optional[float]:
    """Fractional growth of stored bytes if the format's scale metadata were replaced by fp16 planes; None when it is
    not a single ratio (quactlize/formats.py:222-227)."""
    if qtype in BLOCKS:
        return BLOCKS[qtype].fp16_scale_growth
    return NON_BLOCK_SCALE_GROWTH.get(qtype)


def needs_native_scale(qtype: QuantType, budget: float = 0.0) -> bool:
    """Whether the format must keep its own scale channel to respect the no-extra-storage rule (formats.py:334-341)."""
    g = storage_growth(qtype)
    return True if g is None else g > budget


def select_path(qtype: QuantType, num_rows: int, native_scale_available: bool = True, fp16_planes: str = "auto") -> str:
    """Which implementation runs this (format, row count): "gemv", "dequant_then_dense", "fused_native_scale" or
    "fused_fp16_scale"; raises NotImplementedError when none may.  fp16_planes says whether fp16 scale planes may
    exist: "auto" (only for formats whose scales already are fp16), "workspace" (transient planes allowed), "never"
    (quactlize/formats.py:175-219)."""
    if fp16_planes not in ("auto", "workspace", "never"):
        raise ValueError(f"fp16_planes must be auto, workspace or never; got {fp16_planes!r}")
    planes_ok = {"never": False, "workspace": True, "auto": not needs_native_scale(qtype)}[fp16_planes]
    if num_rows <= GEMV_MAX_ROWS and qtype in GEMV and planes_ok:
        return "gemv"
    if num_rows >= DENSE_CROSSOVER_ROWS and qtype in DEQUANT_THEN_DENSE and planes_ok:
        return "dequant_then_dense"
    if native_scale_available and qtype in FUSED_NATIVE_SCALE:
        return "fused_native_scale"
    if qtype in FUSED_FP16_SCALE and planes_ok:
        return "fused_fp16_scale"
    if qtype in DEQUANT_THEN_DENSE and planes_ok:
        return "dequant_then_dense"
    if not planes_ok and (qtype in FUSED_FP16_SCALE or qtype in DEQUANT_THEN_DENSE):
        g = storage_growth(qtype)
        raise NotImplementedError(
            f"{qtype.name} at {num_rows} rows has only fp16-scale-plane paths, and materialising those planes grows the "
            f"stored weight by {g if g is not None else float('nan'):.1%}. Pass fp16_planes='workspace' if the planes are "
            f"transient, or give the format a native scale channel.")
    raise NotImplementedError(f"{qtype.name} has no path at {num_rows} rows")


def fold_for(bits: int, tile_k: int) -> int:
    """N-fold factor the reference's PPU consumer derives from (bits, tile_k): 1 when a k-run of tile_k codes is at
    least 32 bytes, else 32 / run (quactlize/formats.py:250-279).  Kept for artifact manifests written by the
    reference; planes produced by this library are Native and unfolded."""
    run_bytes = tile_k * bits // 8
    if run_bytes >= 32:
        return 1
    if run_bytes == 0:
        raise ValueError(f"bits={bits} tile_k={tile_k}: the k-run is under one byte")
    if 32 % run_bytes:
        raise ValueError(f"bits={bits} tile_k={tile_k}: a {run_bytes}B run does not divide the 32B floor")
    return 32 // run_bytes


class PlacedArrangement(NamedTuple):
    """What an artifact records about its plane arrangement; fold is derived, never stored (formats.py:282-302)."""
    bits: int
    tile_k: int
    high_bits: int = 0

    @property
    def fold(self) -> int:
        return fold_for(self.bits, self.tile_k)

    @property
    def high_fold(self) -> int:
        return fold_for(self.high_bits, self.tile_k) if self.high_bits else 1

    def layout_is_tile_free(self) -> bool:
        return self.fold == 1 and self.high_fold == 1


#: zero-plane correction of the REFERENCE's placed dense arrangement (its int4 converter emits code-8):
#: quactlize/formats.py:315-321.  Used when deriving fp16 planes from packed units for its dense contract.
PLACED_CODE_ZMUL = {QuantType.Q2_K: 0, QuantType.Q3_K: -4, QuantType.Q4_K: 8, QuantType.Q5_K: 8, QuantType.Q6_K: -24}


def placed_code_zmul(qtype) -> int:
    q = QuantType(qtype)
    if q not in PLACED_CODE_ZMUL:
        raise NotImplementedError(f"{q.name} has no recorded placed-code correction")
    return PLACED_CODE_ZMUL[q]


def report() -> str:
    """One table: storage arithmetic and available paths per format."""
    rows = []
    for q in QuantType:
        g = storage_growth(q)
        growth = "n/a" if g is None else f"{g * 100:+5.1f}%"
        paths = [n for n, s in (("gemv", GEMV), ("native", FUSED_NATIVE_SCALE), ("fp16", FUSED_FP16_SCALE),
                                ("dense", DEQUANT_THEN_DENSE)) if q in s]
        blk = BLOCKS.get(q)
        size = f"{blk.block_bytes:>3}B/{blk.weights}w gs={blk.group_size}" if blk else "not a block format"
        rows.append(f"  {q.name:<15} {size:<20} fp16-scale growth {growth:>7}   native required: "
                    f"{'yes' if needs_native_scale(q) else 'no':<3} paths: {','.join(paths) or 'NONE'}")
    return "== quactlize_b200 formats ==\n" + "\n".join(rows)


if __name__ == "__main__":
    print(report())
