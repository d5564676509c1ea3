"""Importers for the reference's other stored weight forms, on CPU.

* GPTQ `mixed_gemm` int4 layout: pinned on a committed fixture the reference's own offline preprocessor produced
  (tests/golden/make_gptq_fixture.py): stored bytes -> the original codes, and its Q4_K artifact dequantise op.
* "xplane" placed planes: the bit maps are the ones its decode GEMV reads placed planes with; what can be checked
  without its device library is checked -- every map is a bijection, both directions invert each other byte for
  byte, and the Q4_K property its fast path states (a placed 32-code group is contiguous and its logical k is an 8x4
  transpose, quactlize/include/gguf_bc_vecdot.hpp:117-119,135) holds."""
import os

import numpy as np
import pytest
import torch

import quactlize_b200 as qb
from conftest import GOLDEN
from oracle import kquant as kq
from quactlize_b200 import gptq, synth, xplane


@pytest.fixture(scope="module")
def fix():
    return np.load(os.path.join(GOLDEN, "gptq_mixed_gemm_q4.npz"))


@pytest.mark.parametrize("tag", ["a", "b"])
def test_restore_q4_mixed_inverts_the_reference_preprocessor(fix, tag):
    got = gptq.restore_q4_mixed(torch.from_numpy(fix[f"stored_{tag}"]))
    assert got.dtype == torch.uint8 and np.array_equal(got.numpy(), fix[f"codes_{tag}"])


@pytest.mark.gpu
def test_q4_artifact_dequantize_matches_the_reference_op(fix):
    w = gptq.gguf_q4_artifact_dequantize(torch.from_numpy(fix["q4k_stored"]), torch.from_numpy(fix["q4k_units"]))
    assert w.dtype == torch.float32 and np.array_equal(w.numpy().view(np.uint32), fix["q4k_dequant"].view(np.uint32))
    with pytest.raises(RuntimeError):
        gptq.gguf_q4_artifact_dequantize(torch.from_numpy(fix["q4k_stored"]), torch.from_numpy(fix["q4k_units"]), "logical")


def test_imported_artifact_is_the_native_artifact(fix):
    blocks = fix["q4k_blocks"]
    n, k = 64, 512
    low, high, units = gptq.import_mixed_gemm_q4(torch.from_numpy(fix["q4k_stored"]), torch.from_numpy(fix["q4k_units"]))
    want_low, _, _, _ = qb.gguf_prepare_gemv(torch.from_numpy(blocks), n, k, 12)
    assert torch.equal(low, want_low) and high.numel() == 0
    assert np.array_equal(units.numpy(), kq.pack_units(blocks, n, k, 12)[0])
    raw = qb.gguf_pack_units(torch.from_numpy(blocks), n, k, 12)[0]
    assert torch.equal(units, raw)


@pytest.mark.parametrize("qtype,high", [(10, False), (11, False), (11, True), (12, False), (13, False), (13, True), (14, False), (14, True)])
def test_xplane_map_is_a_bijection(qtype, high):
    n, k = 128, 512
    slots = np.array([[xplane.slot(qtype, high, c, kk, n) for kk in range(k)] for c in range(n)])
    assert slots.min() == 0 and slots.max() == n * k - 1 and np.unique(slots).size == n * k
    # a tile of 64 columns x TileK codes stays inside its own 64 * TileK slots
    tk = 128 if qtype == 14 else 256
    t = slots[:64, :tk]
    if tk == 256:
        assert t.max() < 64 * 256
    else:                                           # two 128-code k-tiles share one 256-row band, interleaved by 128 rows
        assert np.unique(np.concatenate([slots[:64, :128].ravel(), slots[:64, 128:256].ravel()])).size == 64 * 256
        assert slots[:64, :256].max() < 64 * 256
    if kq.fmt(qtype).hi_bits == 0:
        assert xplane.slot(qtype, True, 0, 0, n) == -1           # the format has no high plane


def test_xplane_q4_group_is_contiguous_and_transposed():
    n = 64
    for col in (0, 5, 63):
        for g in range(8):
            base = xplane.slot(12, False, col, 32 * g, n)
            for p in range(32):
                logical_k = 32 * g + (p & 3) * 8 + (p >> 2)
                assert xplane.slot(12, False, col, logical_k, n) == base + p


def test_xplane_round_trip_every_format(qtype):
    e, n, k = 2, 256, 512
    blocks = synth.kquant_blocks(qtype, e * n * k // 256, seed=9 + qtype)
    low, high, _ = qb.gguf_prepare_fully_quantized_grouped(torch.from_numpy(blocks), n, k, qtype, e)
    plo, phi = xplane.from_native(low, high, n, k, qtype)
    assert plo.shape == low.shape and not torch.equal(plo, low)
    back_lo, back_hi = xplane.to_native(plo, phi, n, k, qtype)
    assert torch.equal(back_lo, low) and torch.equal(back_hi, high)
    # the placed plane holds the same multiset of codes per 64-column x 256-k tile as the Native one
    f = kq.fmt(qtype)
    codes_native = kq.plane_unpack(low.numpy()[0], f.lo_bits)                     # [n, k]
    flat = kq.plane_unpack(plo.numpy()[0].reshape(-1), f.lo_bits)
    for c, kk in ((0, 0), (63, 255), (64, 256), (255, 511), (17, 301)):
        assert flat[xplane.slot(qtype, False, c, kk, n)] == codes_native[c, kk]
    with pytest.raises(RuntimeError):
        xplane.to_native(low[:, :96], high, 96, k, qtype)
