"""GPU kernels against the reference's own real-weight golden outputs (fixtures repacked by
tests/golden/make_real_fixtures.py from the reference's tests/data).  Gates: the reference's element-wise
|err| <= 1e-2 + 5e-2*|gold| (tests/test_moe_grouped_real.cu:124) and max-rel <= 1e-2 (asserted at 6e-3; the gold itself
is rounded to fp16)."""
import os

import numpy as np
import pytest
import torch

import quactlize_b200 as qb
from oracle import kquant as kq
from quactlize_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def _gate(out, gold):
    got = out.float().cpu().numpy().astype(np.float64)
    gold = gold.astype(np.float64)
    assert np.all(np.isfinite(got))
    assert np.all(np.abs(got - gold) <= 1e-2 + 5e-2 * np.abs(gold))
    assert kq.max_rel(got, gold) < 6e-3
    torch.cuda.synchronize()
    assert _lib.lib().quactlize_b200_device_wait_status() == 0


def test_real_q2k_w2a16_tensor_core():
    f = np.load(os.path.join(GOLDEN, "real_q2k_w2a16.npz"))
    out = qb.gemm_plane(_t(f["a"]), _t(f["low"]), None, _t(f["scale"]), _t(f["zero"]), 2, 0, int(f["gs"]))
    _gate(out, f["gold"])


def test_real_q2k_w2a16_gemv_rows():
    f = np.load(os.path.join(GOLDEN, "real_q2k_w2a16.npz"))
    a = _t(f["a"][:4])
    out = torch.cat([qb.gemv_plane(a[i:i + 1], _t(f["low"]), None, _t(f["scale"]), _t(f["zero"]), 2, 0, int(f["gs"]))
                     for i in range(4)])
    _gate(out, f["gold"][:4])


def test_real_q3k_two_plane_tensor_core():
    f = np.load(os.path.join(GOLDEN, "real_q3k_two_plane.npz"))
    out = qb.gemm_plane(_t(f["a"]), _t(f["low"]), _t(f["high"]), _t(f["scale_lo"]), None, 2, 1, int(f["gs"]), code_offset=-4)
    _gate(out, f["gold"])


@pytest.mark.parametrize("route", ["vecdot_dense", "vecdot_rows", "gemv_bc", "dense_fully_quantized", "dense_scale_first"])
def test_real_q4k_blocks(route):
    f = np.load(os.path.join(GOLDEN, "real_q4k_blocks.npz"))
    a, blocks, gold = f["a"], f["blocks"], f["gold"]
    n, k = gold.shape[1], a.shape[1]
    bt = torch.from_numpy(blocks)
    if route == "vecdot_dense":                       # raw-block GEMV, one row (the headline kernel)
        _gate(qb.gguf_vecdot_dense(bt.to(DEV), _t(a[:1]), n, k, 12), gold[:1])
    elif route == "vecdot_rows":                      # all 16 rows (row-tiled kernels)
        _gate(qb.gguf_vecdot_rows(bt.to(DEV), _t(a), n, k, 12), gold)
    elif route == "dense_scale_first":                # scale-first dense artifact on the tensor cores
        art = [t.to(DEV) for t in qb.gguf_prepare_dense(bt, n, k, 12)]
        _gate(qb.gguf_dense_scale_first(_t(a), *art, 12), gold)
    else:                                             # merged artifact: planes + packed units
        low, high, units = (t.to(DEV) for t in qb.gguf_prepare_fully_quantized_dense(bt, n, k, 12))
        if route == "gemv_bc":
            _gate(qb.gguf_gemv_bc(_t(a[:1]), low, high, units, 12), gold[:1])
        else:
            _gate(qb.gguf_dense_fully_quantized(_t(a), low, high, units, 12), gold)
