"""The K-pack carrier of the package (quactlize_b200.kpack), on CPU: bytes against the reference's SHA-256 goldens
(tests/test_reference_gguf_kpack.py:29-105 of the reference), round trips, grouped = expert-major dense, and the bridge to
the Native planes the kernels read."""
import hashlib

import numpy as np
import pytest
import torch

import quactlize_b200 as qb
from quactlize_b200 import kpack
from oracle import kquant as kq
from test_oracle_pins import KPACK_SHA256


def _raw(qtype, n=256, k=512, experts=1):
    f = kq.fmt(qtype)
    rows = experts * n * (k // 256)
    v = ((np.arange(rows * f.block_bytes, dtype=np.int64) * 73 + qtype * 19 + 7) & 0xFF).astype(np.uint8)
    return torch.from_numpy(v.reshape(rows, f.block_bytes))


def _sha(t):
    return hashlib.sha256(t.contiguous().numpy().tobytes()).hexdigest()


def test_dense_is_byte_exact(qtype):
    raw = _raw(qtype)
    low, high, units = kpack.prepare_dense(raw, 256, 512, qtype)
    f = kq.fmt(qtype)
    assert low.shape == (1, 256, 512 * f.lo_bits // 8)
    assert units.shape == (2 // f.sb_per_unit, 256, f.unit_total)
    assert (_sha(low), _sha(high), _sha(units)) == KPACK_SHA256[qtype]
    assert torch.equal(kpack.recover_raw_blocks(low, high, units, 256, 512, qtype), raw)


@pytest.mark.parametrize("qt", [11, 13])
def test_grouped_adds_only_the_expert_axis(qt):
    raw = _raw(qt, experts=2)
    low, high, units = kpack.prepare_grouped(raw, 256, 512, qt, 2)
    per = 256 * 2
    for e in range(2):
        dl, dh, du = kpack.prepare_dense(raw[e * per:(e + 1) * per], 256, 512, qt)
        assert torch.equal(low[e], dl[0]) and torch.equal(high[e], dh[0]) and torch.equal(units[e], du)
    assert torch.equal(kpack.recover_raw_blocks(low, high, units, 256, 512, qt), raw)


def test_bridge_to_native_planes(qtype):
    raw = _raw(qtype, n=256, k=1024)
    low, high, units = kpack.prepare_dense(raw, 256, 1024, qtype)
    nl, nh, nu = kpack.to_native(low, high, units, 256, 1024, qtype)
    wl, wh, wu = qb.gguf_prepare_fully_quantized_dense(raw, 256, 1024, qtype)
    assert torch.equal(nl, wl) and torch.equal(nh, wh) and torch.equal(nu.reshape(wu.shape), wu)
    # and the oracle agrees with the package on the carrier itself
    ol, oh, _ = kq.prepare_kpack(raw.numpy(), 256, 1024, qtype)
    assert np.array_equal(low.numpy(), ol) and np.array_equal(high.numpy().reshape(-1), np.asarray(oh).reshape(-1))


def test_q4_word_is_a_k8_gather():
    """Low nibbles of official Q4_K bytes 16+k for k = 0, 8, 16, 24 of column 0 become slots 0..3 of word (kg=0, n=0)."""
    raw = torch.zeros((256, 144), dtype=torch.uint8)
    for slot, kk in enumerate((0, 8, 16, 24)):
        raw[0, 16 + kk] = slot + 1
    low, _, _ = kpack.prepare_dense(raw, 256, 256, 12)
    word = int(low.reshape(-1)[0]) | (int(low.reshape(-1)[1]) << 8)
    assert word == 0x4321


def test_geometry_is_checked():
    with pytest.raises(ValueError):
        kpack.prepare_dense(_raw(14, k=512)[:256], 256, 256, 14)      # Q6_K pairs two superblocks
    with pytest.raises(ValueError):
        kpack.prepare_dense(_raw(12)[:100], 100, 512, 12)
