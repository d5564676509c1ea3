"""The pair form of the tensor-core GEMM (cluster of two CTAs, tcgen05 cta_group::2, 512 x 256 tiles): opt-in through
QUACTLIZE_B200_GEMM_PAIR, must give what the oracle gives on dense and ragged grouped problems, and the same bits as the
single-CTA form (both accumulate every output in the same K order)."""
import os

import numpy as np
import pytest
import torch

import quactlize_b200 as qb
from oracle import kquant as kq
from quactlize_b200 import _lib, synth

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run(a, low, scale, zero, gs, off, pair):
    t = lambda v: torch.from_numpy(v).to(DEV)
    old = os.environ.pop("QUACTLIZE_B200_GEMM_PAIR", None)
    try:
        if pair:
            os.environ["QUACTLIZE_B200_GEMM_PAIR"] = "1"
        out = qb.gemm_plane(a.to(DEV), t(low), None, t(scale), t(zero), 4, 0, gs, row_offsets=None if off is None else t(off))
        torch.cuda.synchronize()
    finally:
        os.environ.pop("QUACTLIZE_B200_GEMM_PAIR", None)
        if old is not None:
            os.environ["QUACTLIZE_B200_GEMM_PAIR"] = old
    assert _lib.lib().quactlize_b200_device_wait_status() == 0
    return out


@pytest.mark.parametrize("m,n,k,gs,dtype,rows", [
    (512, 256, 256, 128, torch.bfloat16, None),
    (300, 256, 512, 128, torch.float16, None),
    (1024, 512, 1024, 64, torch.bfloat16, None),
    (700, 512, 2048, 32, torch.float16, None),
    (0, 512, 1024, 128, torch.bfloat16, [600, 0, 257, 1, 513, 200]),
    (0, 256, 768, 16, torch.bfloat16, [1100, 300]),
])
def test_pair_form_matches_oracle_and_single_cta_form(m, n, k, gs, dtype, rows):
    e = 1 if rows is None else len(rows)
    low, scale, zero = synth.group_planes(e, n, k, 4, gs, seed=m + n + k)
    total = m if rows is None else sum(rows)
    a = torch.from_numpy(synth.activations(total, k, seed=3, dtype=np.float32)).to(dtype)
    off = None if rows is None else np.concatenate([[0], np.cumsum(rows)]).astype(np.int32)
    ref = kq.planes_matmul(a.float().numpy(), low, None, scale, zero, 4, 0, gs, off)
    pair = _run(a, low, scale, zero, gs, off, True)
    single = _run(a, low, scale, zero, gs, off, False)
    assert kq.max_rel(pair.float().cpu().numpy(), ref) < (1e-2 if dtype == torch.bfloat16 else 3e-3)
    assert torch.equal(pair, single)
