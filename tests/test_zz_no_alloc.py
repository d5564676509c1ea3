"""The allocation-free dense GEMM entry (quactlize_b200_dense_fully_quantized_static_v1) against the regular
device-pointer entry, through the C ABI.  Collected last on purpose: it must pass after every other GPU test has used
the library, and alone in a fresh process.  Tolerance: the outputs of the two entries come from the same kernels on the
same planes, so they are compared for equality; the regular entry itself is held to max-rel 6e-3 against the oracle in
test_gemm_gpu.py, which is re-checked here."""
import ctypes

import numpy as np
import pytest
import torch

import quactlize_b200 as qb
from oracle import kquant as kq
from quactlize_b200 import _lib, synth

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SCRATCH_BYTES = 16 * 1024 * 1024


def _p(t):
    return ctypes.c_void_p(t.data_ptr() if t is not None and t.numel() else 0)


def _case(qtype, m, n, k, seed):
    blocks = synth.kquant_blocks(qtype, n * k // 256, seed=seed)
    low, high, units = qb.gguf_prepare_fully_quantized_dense(torch.from_numpy(blocks), n, k, qtype)
    a = synth.activations(m, k, seed=seed + 1)
    ref = a.astype(np.float64) @ kq.dequantize_f32(blocks, qtype).reshape(n, k).T
    return torch.from_numpy(a).to(DEV), low.to(DEV), high.to(DEV), units.to(DEV), ref


def _regular(L, a, low, high, units, m, n, k, qtype):
    need = L.quactlize_ppu_dense_fully_quantized_workspace_bytes_v1(m, n, k, qtype)
    ws = torch.empty(need, dtype=torch.uint8, device=DEV)
    out = torch.empty((m, n), dtype=torch.float16, device=DEV)
    rc = L.quactlize_ppu_dense_fully_quantized_dev_v1(_p(a), _p(low), _p(high), _p(units), _p(out), m, n, k, qtype, _p(ws), need,
                                                      ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    return out


def _static(L, a, low, high, units, m, n, k, qtype):
    out = torch.full((m, n), float("nan"), dtype=torch.float16, device=DEV)
    rc = L.quactlize_b200_dense_fully_quantized_static_v1(_p(a), _p(low), _p(high), _p(units), _p(out), m, n, k, qtype,
                                                          ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    return out


def test_static_scratch_entry_two_calls_in_a_row():
    L = _lib.lib()
    torch.cuda.set_device(0)
    # two different weights back to back: the second is smaller, so the array still holds planes of the first
    cases = [(14, 70, 512, 1024, 21), (12, 300, 256, 2048, 22)]
    prepared = [(_case(qt, m, n, k, seed), qt, m, n, k) for qt, m, n, k, seed in cases]
    torch.cuda.synchronize()
    got = [_static(L, a, low, high, units, m, n, k, qt) for (a, low, high, units, _), qt, m, n, k in prepared]
    torch.cuda.synchronize()
    for out, ((a, low, high, units, ref), qt, m, n, k) in zip(got, prepared):
        want = _regular(L, a, low, high, units, m, n, k, qt)
        torch.cuda.synchronize()
        res = out.float().cpu().numpy()
        assert np.all(np.isfinite(res))
        assert torch.equal(out, want)
        assert kq.max_rel(res, ref) < 6e-3
    # the same call again gives the same bytes
    (a, low, high, units, _), qt, m, n, k = prepared[0]
    again = _static(L, a, low, high, units, m, n, k, qt)
    torch.cuda.synchronize()
    assert torch.equal(again, got[0])
    assert L.quactlize_b200_device_wait_status() == 0


def test_static_scratch_entry_leaves_device_memory_untouched():
    """After a first (warm) call, further calls must not change the device's free memory at all: the entry owns no
    allocation, so cudaMemGetInfo (read through torch.cuda.mem_get_info) is identical before and after."""
    L = _lib.lib()
    torch.cuda.set_device(0)
    (a, low, high, units, _), (qt, m, n, k) = _case(13, 64, 512, 1024, 31), (13, 64, 512, 1024)
    out = torch.empty((m, n), dtype=torch.float16, device=DEV)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    call = lambda: L.quactlize_b200_dense_fully_quantized_static_v1(_p(a), _p(low), _p(high), _p(units), _p(out), m, n, k, qt, stream)
    assert call() == 0                                   # warm: symbol-address lookup, function attributes, module load
    torch.cuda.synchronize()
    free_before, total = torch.cuda.mem_get_info(0)
    for _ in range(3):
        assert call() == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info(0)
    assert free_after == free_before, (free_before, free_after, total)
    assert L.quactlize_b200_device_wait_status() == 0


def test_static_scratch_entry_refuses_what_does_not_fit():
    L = _lib.lib()
    n = k = 16384                                        # Q6_K: 2 planes * (k/16) * n fp16 = 64 MiB
    assert 4 * (k // 16) * n > SCRATCH_BYTES
    dummy = torch.zeros(64, dtype=torch.uint8, device=DEV)
    rc = L.quactlize_b200_dense_fully_quantized_static_v1(_p(dummy), _p(dummy), _p(dummy), _p(dummy), _p(dummy), 1, n, k, 14,
                                                          ctypes.c_void_p(0))
    assert rc == 37
    # refusals that come before any pointer is touched: unknown format, missing activation
    assert L.quactlize_b200_dense_fully_quantized_static_v1(_p(dummy), _p(dummy), _p(dummy), _p(dummy), _p(dummy), 1, 256, 256, 99,
                                                            ctypes.c_void_p(0)) == 33
    assert L.quactlize_b200_dense_fully_quantized_static_v1(None, _p(dummy), _p(dummy), _p(dummy), _p(dummy), 1, 256, 256, 14,
                                                            ctypes.c_void_p(0)) == 30
