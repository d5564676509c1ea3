"""Pins the numpy oracle: bit-for-bit against golden vectors produced by the reference's own host ops
(tests/golden/make_golden.py) and against the official gguf package's dequantiser."""
import os

import numpy as np
import pytest

from conftest import load_golden
from oracle import kquant as kq
from quactlize_b200 import synth


def _eq(a, b):
    a, b = np.asarray(a), np.asarray(b)
    assert a.shape == b.shape, (a.shape, b.shape)
    if a.dtype == np.float16:
        a, b = a.view(np.uint16), b.view(np.uint16)
    assert np.array_equal(a, b)


def test_dequantize_bit_exact(qtype):
    g = load_golden(qtype)
    _eq(kq.dequantize(g["blocks"], qtype), g["dequant"])


def test_unpack_bit_exact(qtype):
    g = load_golden(qtype)
    c, s, z = kq.unpack(g["blocks"], qtype)
    _eq(c, g["codes"]); _eq(s, g["scale_rows"]); _eq(z, g["zero_rows"])


def test_prepare_gemv_bit_exact(qtype):
    g = load_golden(qtype)
    low, high, scale, zero = kq.prepare_gemv(g["blocks"], int(g["n"]), int(g["k"]), qtype)
    _eq(low, g["low"]); _eq(high, g["high"]); _eq(scale, g["scale"]); _eq(zero, g["zero"])
    _eq(kq.gemv_artifact_dequantize(low, high, scale, zero, qtype), g["artifact_dequant"])


def test_units_bit_exact(qtype):
    g = load_golden(qtype)
    n, k = int(g["n"]), int(g["k"])
    units = kq.pack_units(g["blocks"], n, k, qtype)[0]
    _eq(units, g["units"])
    for zm in (-32, -24, -4, 0, 8):
        s, z = kq.units_decode(units, qtype, zm)
        _eq(s, g[f"unit_scale_z{zm}"]); _eq(z, g[f"unit_zero_z{zm}"])


def test_scale_prepass_bit_exact(qtype):
    g = load_golden(qtype)
    f = kq.fmt(qtype)
    b = g["blocks"]
    d, dmin = kq.d_dmin(b, qtype)
    for zm in (0, 8):
        s, z = kq.scale_prepass(b[:, f.scale_off:f.scale_off + f.scale_bytes], d, dmin, qtype, zm)
        _eq(s, g[f"prepass_scale_z{zm}"]); _eq(z, g[f"prepass_zero_z{zm}"])


def test_recover_round_trip(qtype):
    g = load_golden(qtype)
    n, k = int(g["n"]), int(g["k"])
    low, high, units = kq.prepare_fully_quantized(g["blocks"], n, k, qtype)
    _eq(kq.recover_blocks(low, high, units, n, k, qtype), g["blocks"])


def test_vecdot_dense_matches_reference_cpu_arm(qtype):
    g = load_golden(qtype)
    got = kq.vecdot_dense(g["blocks"], g["x"], int(g["n"]), int(g["k"]), qtype)
    assert kq.max_rel(got, g["vecdot_dense"]) < 2e-6
    # the merged artifact (planes + units) describes the same weight
    low, high, units = kq.prepare_fully_quantized(g["blocks"], int(g["n"]), int(g["k"]), qtype)
    assert kq.max_rel(kq.bc_matmul(g["x"], low, high, units, qtype), g["vecdot_dense"]) < 2e-6


def test_official_gguf_dequantizer(qtype):
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    blocks = synth.kquant_blocks(qtype, 257, seed=5 + qtype)
    ref = quants.dequantize(blocks.reshape(-1), gguf.GGMLQuantizationType(qtype)).reshape(-1, 256)
    got = kq.dequantize(blocks, qtype)
    _eq(got, ref.astype(np.float16))
    assert np.allclose(kq.dequantize_f32(blocks, qtype), ref, rtol=1e-6, atol=1e-9)


def test_planes_matmul_matches_dequant(qtype):
    g = load_golden(qtype)
    f = kq.fmt(qtype)
    n, k = int(g["n"]), int(g["k"])
    low, high, scale, zero = g["low"], g["high"], g["scale"], g["zero"]
    a = synth.activations(3, k, seed=9)
    w = kq.gemv_artifact_dequantize(low, high, scale, zero, qtype)[0].astype(np.float64)
    ref = a.astype(np.float64) @ w.T
    got = kq.planes_matmul(a, low, high, scale, zero, f.lo_bits, f.hi_bits, f.group_size)
    assert kq.max_rel(got, ref) < 2e-3


# ---- the reference's real-weight golden vectors for the tensor-core arithmetic (repacked by make_real_fixtures.py) ----

def _real(name):
    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", name))


def test_real_q2k_w2a16_gold():
    """tests/test_w2a16_real.cu:1-9: a Q2_K slice at its native gs=16, D = A @ (q*scale + zero)."""
    f = _real("real_q2k_w2a16.npz")
    ref = kq.planes_matmul(f["a"].astype(np.float32), f["low"], None, f["scale"], f["zero"], 2, 0, int(f["gs"]))
    assert kq.max_rel(ref, f["gold"].astype(np.float64)) < 2e-3


def test_real_q3k_two_plane_gold():
    """tests/test_q3_concat_real.cu:1-12: W = dl*(low2 + 4*high1 - 4); the fixture's split scales obey
    scale_hi = 4*scale_lo and zero_lo = -4*scale_lo exactly (powers of two), so one two-plane product reproduces it."""
    f = _real("real_q3k_two_plane.npz")
    assert np.array_equal(f["scale_hi"].astype(np.float32), 4 * f["scale_lo"].astype(np.float32))
    assert np.array_equal(f["zero_lo"].astype(np.float32), -4 * f["scale_lo"].astype(np.float32))
    ref = kq.planes_matmul(f["a"].astype(np.float32), f["low"], f["high"], f["scale_lo"], None, 2, 1, int(f["gs"]), code_offset=-4)
    assert kq.max_rel(ref, f["gold"].astype(np.float64)) < 2e-3


def test_real_q4k_blocks_gold():
    """tests/rwmoep_loader.hpp:12-22: real Q4_K columns in native form (codes, 6-bit sc/mn, fp16 d/dmin), repacked into
    raw 144-byte blocks; gold = A @ dequant(W)."""
    f = _real("real_q4k_blocks.npz")
    a, blocks, gold = f["a"], f["blocks"], f["gold"].astype(np.float64)
    n, k = gold.shape[1], a.shape[1]
    ref = a.astype(np.float64) @ kq.dequantize_f32(blocks, 12).reshape(n, k).T.astype(np.float64)
    assert kq.max_rel(ref, gold) < 2e-3
    # the official gguf dequantiser reads the repacked blocks the same way
    import gguf
    off = gguf.quants.dequantize(blocks, gguf.GGMLQuantizationType.Q4_K).reshape(n, k)
    assert np.array_equal(off.astype(np.float32), kq.dequantize_f32(blocks, 12).reshape(n, k))


# ---- canonical K-pack carrier: SHA-256 goldens of the reference (tests/test_reference_gguf_kpack.py:29-66) ----------------

KPACK_SHA256 = {
    10: ("17c5bc5ffa2c3796060988b43dcbe6b8ab15f1e0cfff8d1fc203163b511cf834", "e3b0c44298fc1c149afbf4c8996fb92427ae41e4649b934ca495991b7852b855",
         "8e74ce7f1c0a324e377025b52d041fe951adb73382476027c962c18f18182b06"),
    11: ("25d1cd007ac3b09944ee3fe7907f8a6c28b1648a805b125d72646ee2a4442673", "aeb7f677e045094859431309010b14a87131d0cd0227f263472145d0d2b12065",
         "681e897a5308d65fb365262bc53445b179a2ef685d951c430285a8ebb789a580"),
    12: ("3d4096663c410cf9fe53640b326327d3bc25af58c52a183a9fa9bd0c35652452", "e3b0c44298fc1c149afbf4c8996fb92427ae41e4649b934ca495991b7852b855",
         "1a9546a67e9b7a15374150f1c418d00f98b5aa48f25fe21f0231013e805f338a"),
    13: ("53f75fa3c1661bd764addd82ef2c183247a6244645d90e5ebc780f9ed6a41fe2", "c59f97a90cac811b5c7f5ac46cadc1f53a3ddd1a580ec8423c5f9d5584a1a4f4",
         "316e801f5b78e98e736a8640c15eaba740256fa9d14ec52578f45862f571d1ab"),
    14: ("a38cc40e0b4763215d7799a02ac61ba2f391a537729c04203c9c78275f54b27e", "c32f0a1246d31041c5cc6b1f316d7ce445f4f1dd41933ab309709989ed938ea7",
         "b679c272d8da7aec284aa4b9ee41aba5960c2e7861a70e264604ee7e5f8d1285"),
}


def test_kpack_carrier_matches_reference_sha256(qtype):
    """The reference binds its K-pack carrier to exact bytes with SHA-256 digests over a deterministic byte pattern
    (n=256, k=512, raw byte i = (i*73 + qtype*19 + 7) & 0xFF); the oracle's planes and units reproduce all three."""
    import hashlib
    f = kq.fmt(qtype)
    n, k = 256, 512
    rows = n * (k // 256)
    raw = ((np.arange(rows * f.block_bytes, dtype=np.int64) * 73 + qtype * 19 + 7) & 0xFF).astype(np.uint8).reshape(rows, f.block_bytes)
    low, high, units = kq.prepare_kpack(raw, n, k, qtype)
    got = tuple(hashlib.sha256(np.ascontiguousarray(t).tobytes()).hexdigest() for t in (low, high, units))
    assert got == KPACK_SHA256[qtype]
    assert np.array_equal(kq.recover_from_kpack(low, high, units, n, k, qtype), raw)
