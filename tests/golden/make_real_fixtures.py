"""Converts the reference's own real-weight golden vectors for the tensor-core path into fixtures that travel.

The reference's tests hold three files with activations, quantised weights cut from real checkpoints, the scale
channel and a gold output computed by its Python tooling (tests/test_w2a16_real.cu:1-9, tests/test_q3_concat_real.cu:1-12,
tests/rwmoep_loader.hpp:12-22 for the layouts).  This script re-expresses each in the layouts of this library --
Native bit planes [N][K*bits/8], fp16 scale/zero [K/gs][N], raw Q4_K blocks -- and stores them with the gold:

    python tests/golden/make_real_fixtures.py /path/to/reference/tests/data

Nothing is recomputed: codes, scales, activations and gold are the reference's bytes, only repacked.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import kquant as kq  # noqa: E402


class Reader:
    def __init__(self, path, offset):
        self.b = open(path, "rb").read()
        self.o = offset

    def take(self, dtype, n):
        size = n * np.dtype(dtype).itemsize
        a = np.frombuffer(self.b[self.o:self.o + size], dtype=dtype).copy()
        assert a.size == n, "short fixture"
        self.o += size
        return a

    def done(self):
        assert self.o == len(self.b), "trailing bytes: layout mismatch"


def native_plane(codes_nk, bits):
    """codes [N][K] (values < 2^bits) -> Native plane bytes [N][K*bits/8], element k at bit k*bits, LSB first."""
    n, k = codes_nk.shape
    per = 8 // bits
    c = codes_nk.reshape(n, k // per, per).astype(np.uint16)
    out = np.zeros((n, k // per), dtype=np.uint16)
    for j in range(per):
        out |= c[:, :, j] << (bits * j)
    return out.astype(np.uint8)


def q2k(src, dst):
    hdr = np.frombuffer(open(src, "rb").read(16), dtype=np.int32)
    m, n, k, gs = (int(x) for x in hdr)
    r = Reader(src, 16)
    a = r.take(np.float16, m * k).reshape(m, k)
    q = r.take(np.uint8, k * n).reshape(k, n)
    scale = r.take(np.float16, (k // gs) * n).reshape(k // gs, n)
    zero = r.take(np.float16, (k // gs) * n).reshape(k // gs, n)
    gold = r.take(np.float16, m * n).reshape(m, n)
    r.done()
    assert q.max() <= 3
    np.savez_compressed(dst, a=a, low=native_plane(q.T.copy(), 2)[None], scale=scale[None], zero=zero[None], gold=gold,
                        gs=np.int32(gs))


def q3k(src, dst):
    hdr = np.frombuffer(open(src, "rb").read(16), dtype=np.int32)
    m, n, k, gs = (int(x) for x in hdr)
    r = Reader(src, 16)
    a = r.take(np.float16, m * k).reshape(m, k)
    lo = r.take(np.uint8, k * n).reshape(k, n)
    hi = r.take(np.uint8, k * n).reshape(k, n)
    sg = (k // gs) * n
    sc_lo, zr_lo, sc_hi = (r.take(np.float16, sg).reshape(k // gs, n) for _ in range(3))
    gold = r.take(np.float16, m * n).reshape(m, n)
    r.done()
    assert lo.max() <= 3 and hi.max() <= 1
    np.savez_compressed(dst, a=a, low=native_plane(lo.T.copy(), 2)[None], high=native_plane(hi.T.copy(), 1)[None],
                        scale_lo=sc_lo[None], zero_lo=zr_lo[None], scale_hi=sc_hi[None], gold=gold, gs=np.int32(gs))


def q4k_blocks(codes_nk, sc, mn, d, dmin):
    """Raw Q4_K blocks [N*K/256][144] from codes [N][K] in 0..15, 6-bit sub-scales/mins [K/32][N], fp16 d/dmin [K/256][N]."""
    n, k = codes_nk.shape
    nb = k // 256
    blk = np.zeros((n, nb, 144), dtype=np.uint8)
    blk[:, :, 0:2] = d.T.copy().view(np.uint8).reshape(n, nb, 2)
    blk[:, :, 2:4] = dmin.T.copy().view(np.uint8).reshape(n, nb, 2)
    s = sc.T.reshape(n, nb, 8).astype(np.uint8)
    mm = mn.T.reshape(n, nb, 8).astype(np.uint8)
    for t in range(4):
        blk[:, :, 4 + t] = (s[:, :, t] & 63) | ((s[:, :, 4 + t] >> 4) << 6)
        blk[:, :, 8 + t] = (mm[:, :, t] & 63) | ((mm[:, :, 4 + t] >> 4) << 6)
        blk[:, :, 12 + t] = (s[:, :, 4 + t] & 15) | ((mm[:, :, 4 + t] & 15) << 4)
    c = codes_nk.reshape(n, nb, 4, 2, 32).astype(np.uint8)            # [pair of groups][nibble][j]
    blk[:, :, 16:144] = (c[:, :, :, 0, :] | (c[:, :, :, 1, :] << 4)).reshape(n, nb, 128)
    return blk.reshape(n * nb, 144)


def q4k(src, dst):
    raw = open(src, "rb").read(48)
    assert raw[:8] == b"RWMOEP\0\0"
    L, m, n, k, gs, mode, ktype, sb, z_mul, cvt_bias = (int(x) for x in np.frombuffer(raw[8:48], dtype=np.int32))
    assert (L, gs, mode, sb) == (1, 32, 1, 256)
    r = Reader(src, 48)
    a = r.take(np.float16, m * k).reshape(m, k)
    q = r.take(np.int8, n * k).reshape(n, k)
    sc = r.take(np.int8, (k // gs) * n).reshape(k // gs, n)
    mn = r.take(np.int8, (k // gs) * n).reshape(k // gs, n)
    d = r.take(np.float16, (k // sb) * n).reshape(k // sb, n)
    dmin = r.take(np.float16, (k // sb) * n).reshape(k // sb, n)
    gold = r.take(np.float16, m * n).reshape(m, n)
    r.done()
    blocks = q4k_blocks((q.astype(np.int16) + 8).astype(np.uint8), sc, mn, d, dmin)
    # the repacked blocks must mean exactly what the fixture's planes mean
    w = (d.astype(np.float32).repeat(8, 0) * sc).repeat(32, 0).T * (q.astype(np.float32) + 8) - \
        (dmin.astype(np.float32).repeat(8, 0) * mn).repeat(32, 0).T
    assert np.array_equal(kq.dequantize_f32(blocks, 12).reshape(n, k), w.astype(np.float32))
    np.savez_compressed(dst, a=a, blocks=blocks, gold=gold)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    data = sys.argv[1]
    q2k(os.path.join(data, "real_q2k_ffn_gate_L0.bin"), os.path.join(HERE, "real_q2k_w2a16.npz"))
    q3k(os.path.join(data, "real_q3k_concat.bin"), os.path.join(HERE, "real_q3k_two_plane.npz"))
    q4k(os.path.join(data, "q4k_packed.bin"), os.path.join(HERE, "real_q4k_blocks.npz"))
    for f in ("real_q2k_w2a16.npz", "real_q3k_two_plane.npz", "real_q4k_blocks.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)))
