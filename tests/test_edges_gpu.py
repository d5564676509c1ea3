"""Edge shapes of the hot path on the device: smallest sizes, ragged groups with every expert empty, unaligned device
pointers (the plain-load kernels take over), K at and beyond what the bulk-copy kernels hold in shared memory."""
import numpy as np
import pytest
import torch

import quactlize_b200 as qb
from oracle import kquant as kq
from quactlize_b200 import _lib, synth

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def _wait_ok():
    torch.cuda.synchronize()
    assert _lib.lib().quactlize_b200_device_wait_status() == 0


@pytest.mark.parametrize("qt", [10, 11, 12, 13, 14])
@pytest.mark.parametrize("n,k", [(1, 256), (8, 256), (9, 512), (17, 2048)])
@pytest.mark.parametrize("m", [1, 2, 9])
def test_smallest_raw_shapes(qt, n, k, m):
    blocks = synth.kquant_blocks(qt, n * k // 256, seed=qt + n + k + m)
    x = synth.activations(m, k, seed=3)
    out = qb.gguf_vecdot_rows(_cuda(blocks), _cuda(x), n, k, qt)
    assert out.shape == (m, n)
    assert kq.max_rel(out.cpu().numpy(), kq.vecdot_dense(blocks, x, n, k, qt)) < 4e-3
    _wait_ok()


@pytest.mark.parametrize("qt", [12, 14])
def test_moe_with_every_expert_empty_and_with_one_full(qt):
    n, k, e = 32, 1024, 4
    blocks = synth.kquant_blocks(qt, e * n * k // 256, seed=31 + qt).reshape(e, n * k // 256, -1)
    for rows in ([0, 0, 0, 0], [0, 0, 7, 0]):
        total = sum(rows)
        x = synth.activations(max(total, 1), k, seed=5)[:total]
        off = np.concatenate([[0], np.cumsum(rows)]).astype(np.int32)
        out = qb.gguf_vecdot_moe(_cuda(blocks), _cuda(x), _cuda(off), qt)
        assert out.shape == (total, n)
        if total:
            assert kq.max_rel(out.cpu().numpy(), kq.vecdot_moe(blocks, x, off, n, k, qt)) < 4e-3
    _wait_ok()


@pytest.mark.parametrize("qt", [12, 14])
@pytest.mark.parametrize("m", [1, 4])
def test_unaligned_device_pointers_take_the_plain_kernels(qt, m):
    """Blocks and activations that start off a 16-byte boundary: no bulk copy may be issued from them."""
    n, k = 64, 4096
    blocks = synth.kquant_blocks(qt, n * k // 256, seed=41 + qt)
    x = synth.activations(m, k, seed=6)
    bb = blocks.shape[1]
    raw = torch.zeros(blocks.size + 64, dtype=torch.uint8, device=DEV)
    raw[2:2 + blocks.size] = _cuda(blocks).reshape(-1)
    b_un = raw[2:2 + blocks.size].view(n * k // 256, bb)                # 2 bytes off
    xs = torch.zeros(m * k + 8, dtype=torch.float16, device=DEV)
    xs[1:1 + m * k] = _cuda(x).reshape(-1)
    x_un = xs[1:1 + m * k].view(m, k)                                    # 2 bytes off
    assert b_un.data_ptr() % 16 != 0 and x_un.data_ptr() % 16 != 0
    ref = kq.vecdot_dense(blocks, x, n, k, qt)
    for bt, xt in ((b_un, _cuda(x)), (_cuda(blocks), x_un), (b_un, x_un)):
        out = qb.gguf_vecdot_rows(bt, xt, n, k, qt)
        assert kq.max_rel(out.cpu().numpy(), ref) < 4e-3
    _wait_ok()


@pytest.mark.parametrize("k", [16384, 16640, 32768])
def test_long_rows(k):
    """K = 16384 is the most the single-row Q4_K kernel keeps in shared memory; longer rows go to another kernel."""
    n = 24
    blocks = synth.kquant_blocks(12, n * k // 256, seed=k % 97)
    x = synth.activations(2, k, seed=7)
    ref = kq.vecdot_dense(blocks, x, n, k, 12)
    for rows in (1, 2):
        out = qb.gguf_vecdot_rows(_cuda(blocks), _cuda(x[:rows]), n, k, 12)
        assert kq.max_rel(out.cpu().numpy(), ref[:rows]) < 4e-3
    b6 = synth.kquant_blocks(14, n * k // 256, seed=k % 89)
    out6 = qb.gguf_vecdot_rows(_cuda(b6), _cuda(x[:1]), n, k, 14)
    assert kq.max_rel(out6.cpu().numpy(), kq.vecdot_dense(b6, x[:1], n, k, 14)) < 4e-3
    _wait_ok()


def test_grouped_gemm_with_empty_groups_only_and_single_row_groups():
    n, k, bits, gs, e = 256, 512, 4, 128, 5
    low, scale, zero = synth.group_planes(e, n, k, bits, gs, seed=51)
    for rows in ([0, 0, 0, 0, 0], [1, 0, 1, 0, 1], [0, 0, 0, 0, 300]):
        total = sum(rows)
        a = synth.activations(max(total, 1), k, seed=8)[:total]
        off = np.concatenate([[0], np.cumsum(rows)]).astype(np.int32)
        out = qb.gemm_plane(_cuda(a), _cuda(low), None, _cuda(scale), _cuda(zero), bits, 0, gs, row_offsets=_cuda(off))
        assert out.shape == (total, n)
        if total:
            ref = kq.planes_matmul(a, low, None, scale, zero, bits, 0, gs, off)
            assert kq.max_rel(out.float().cpu().numpy(), ref) < 3e-3
    _wait_ok()


@pytest.mark.parametrize("qt", [11, 13, 14])
@pytest.mark.parametrize("k", [16384, 32768])
def test_merged_gemv_long_rows(qt, k):
    """K = 16384 is what the merged artifact's row-pair kernel still holds (four segments of sixteen superblocks); longer
    rows go to the row-thread kernel."""
    n = 256
    blocks = synth.kquant_blocks(qt, n * k // 256, seed=k % 83 + qt)
    low, high, units = qb.gguf_prepare_fully_quantized_dense(torch.from_numpy(blocks), n, k, qt)
    a = synth.activations(1, k, seed=9)
    out = qb.gguf_gemv_bc(_cuda(a), low.to(DEV), high.to(DEV), units.to(DEV), qt)
    assert kq.max_rel(out.cpu().numpy(), kq.vecdot_dense(blocks, a, n, k, qt)) < 4e-3
    _wait_ok()


@pytest.mark.parametrize("qt", [10, 14])
def test_merged_gemv_with_unaligned_units(qt):
    """Packed units that start 4 bytes off a 16-byte boundary: the row-pair kernel's 8-byte unit pieces would be misaligned,
    so another kernel takes the launch."""
    n, k = 256, 2048
    blocks = synth.kquant_blocks(qt, n * k // 256, seed=51 + qt)
    low, high, units = qb.gguf_prepare_fully_quantized_dense(torch.from_numpy(blocks), n, k, qt)
    raw = torch.zeros(units.numel() + 64, dtype=torch.uint8, device=DEV)
    raw[4:4 + units.numel()] = units.to(DEV).reshape(-1)
    u_un = raw[4:4 + units.numel()].view(units.shape)
    assert u_un.data_ptr() % 16 == 4
    a = synth.activations(1, k, seed=10)
    out = qb.gguf_gemv_bc(_cuda(a), low.to(DEV), high.to(DEV), u_un, qt)
    assert kq.max_rel(out.cpu().numpy(), kq.vecdot_dense(blocks, a, n, k, qt)) < 4e-3
    _wait_ok()
