"""GPU parity tests of the CUDA-core family, through the C ABI (ctypes) against the numpy oracle and the reference
goldens.  Integer/byte/fp16-plane results are bit-exact; GEMV outputs are within max-rel 1e-2 of an fp64-accumulated
dequant-then-matmul (asserted tighter, 2e-3, the reference's own gate is 4e-3: tests/test_gemv_lowbit.cu:299-305)."""
import numpy as np
import pytest
import torch

import quactlize_b200 as qb
from conftest import load_golden
from oracle import kquant as kq
from quactlize_b200 import _lib, synth

pytestmark = pytest.mark.gpu
TOL = 2e-3
DEV = "cuda:0"


def _cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def _bits(t):
    a = t.detach().cpu().numpy()
    return a.view(np.uint16) if a.dtype == np.float16 else a


def _wait_ok():
    torch.cuda.synchronize()
    assert _lib.lib().quactlize_b200_device_wait_status() == 0


# ---- bit-exact kernels ------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("where", ["cuda", "cpu"])
def test_dequantize_bit_exact(qtype, where):
    g = load_golden(qtype)
    b = torch.from_numpy(g["blocks"])
    out = qb.gguf_dequantize(b.to(DEV) if where == "cuda" else b, qtype)
    assert np.array_equal(_bits(out), g["dequant"].view(np.uint16))


def test_dequantize_large_matches_oracle(qtype):
    blocks = synth.kquant_blocks(qtype, 4099, seed=3 + qtype)
    out = qb.gguf_dequantize(_cuda(blocks), qtype)
    assert np.array_equal(_bits(out), kq.dequantize(blocks, qtype).view(np.uint16))


def test_scale_prepass_bit_exact(qtype):
    g = load_golden(qtype)
    f = kq.fmt(qtype)
    b = g["blocks"]
    d, dmin = kq.d_dmin(b, qtype)
    sb = torch.from_numpy(np.ascontiguousarray(b[:, f.scale_off:f.scale_off + f.scale_bytes]))
    for zm in (0, 8):
        s, z = qb.gguf_scale_prepass(sb, torch.from_numpy(d), torch.from_numpy(dmin) if f.has_min else None, qtype, zm)
        assert np.array_equal(_bits(s), g[f"prepass_scale_z{zm}"].view(np.uint16))
        assert np.array_equal(_bits(z), g[f"prepass_zero_z{zm}"].view(np.uint16))


@pytest.mark.parametrize("where", ["cuda", "cpu"])
def test_packed_scale_prepass_bit_exact(qtype, where):
    g = load_golden(qtype)
    u = torch.from_numpy(g["units"])
    u = u.to(DEV) if where == "cuda" else u
    for zm in (-32, -24, -4, 0, 8):
        s, z = qb.gguf_packed_scale_prepass(u, qtype, zm)
        assert np.array_equal(_bits(s), g[f"unit_scale_z{zm}"].view(np.uint16))
        assert np.array_equal(_bits(z), g[f"unit_zero_z{zm}"].view(np.uint16))


# ---- raw-block GEMV ---------------------------------------------------------------------------------------------------

def test_vecdot_dense_golden(qtype):
    g = load_golden(qtype)
    n, k = int(g["n"]), int(g["k"])
    for where in ("cuda", "cpu"):
        b, x = torch.from_numpy(g["blocks"]), torch.from_numpy(g["x"])
        if where == "cuda":
            b, x = b.to(DEV), x.to(DEV)
        out = qb.gguf_vecdot_dense(b, x, n, k, qtype)
        assert out.shape == (1, n) and out.dtype == torch.float32
        assert kq.max_rel(out.cpu().numpy(), g["vecdot_dense"]) < TOL
    _wait_ok()


def test_vecdot_per_block_rows(qtype):
    blocks = synth.kquant_blocks(qtype, 300, seed=11 + qtype)
    x = synth.activations(300, 256, seed=5)
    ref = np.einsum("rk,rk->r", kq.dequantize_f32(blocks, qtype), x.astype(np.float64))
    for where in ("cuda", "cpu"):
        b, xx = torch.from_numpy(blocks), torch.from_numpy(x)
        if where == "cuda":
            b, xx = b.to(DEV), xx.to(DEV)
        out = qb.gguf_vecdot(b, xx, qtype)
        assert kq.max_rel(out.cpu().numpy(), ref) < TOL


Q4_SHAPES = [(512, 4096), (96, 14336), (37, 256), (200, 768), (64, 11008 // 256 * 256), (1, 4096), (130, 8192)]


@pytest.mark.parametrize("n,k", Q4_SHAPES)
@pytest.mark.parametrize("m", [1, 2, 3, 4, 5, 7, 8])
def test_q4k_fast_kernel_vs_oracle(n, k, m):
    blocks = synth.kquant_blocks(12, n * k // 256, seed=n + k + m)
    x = synth.activations(m, k, seed=m + 1)
    x[0, :7] *= 30.0                                     # outliers exercise the power-of-two activation scaling
    ref = kq.vecdot_dense(blocks, x, n, k, 12)
    out = qb.gguf_vecdot_rows(_cuda(blocks), _cuda(x), n, k, 12)
    # 30x outlier activations: the fp16 group sums (8 products each) carry ~2^-11 of the outlier terms
    assert kq.max_rel(out.cpu().numpy(), ref) < 4e-3
    gen = qb.gguf_vecdot_rows(_cuda(blocks), _cuda(x), n, k, 12, force_generic=True)
    assert kq.max_rel(gen.cpu().numpy(), ref) < TOL
    _wait_ok()


KQ_SHAPES = [(256, 4096), (96, 14336), (37, 2048), (1, 4096), (130, 8192), (300, 6144)]


@pytest.mark.parametrize("n,k", KQ_SHAPES)
@pytest.mark.parametrize("m", [1, 3])
@pytest.mark.parametrize("qt", [10, 11, 13, 14])
def test_kquant_fast_kernel_vs_oracle(qt, n, k, m):
    """Q2_K / Q3_K / Q5_K / Q6_K raw blocks through the bulk-copy single-row kernel (rows that are a multiple of 16 bytes)."""
    blocks = synth.kquant_blocks(qt, n * k // 256, seed=n + k + m + qt)
    x = synth.activations(m, k, seed=m + 1)
    x[0, :7] *= 30.0
    ref = kq.vecdot_dense(blocks, x, n, k, qt)
    out = qb.gguf_vecdot_rows(_cuda(blocks), _cuda(x), n, k, qt)
    assert kq.max_rel(out.cpu().numpy(), ref) < 4e-3
    gen = qb.gguf_vecdot_rows(_cuda(blocks), _cuda(x), n, k, qt, force_generic=True)
    assert kq.max_rel(gen.cpu().numpy(), ref) < TOL
    _wait_ok()


@pytest.mark.parametrize("qt", [10, 11, 13, 14])
def test_kquant_fast_kernel_moe(qt):
    n, k, rows_per_expert = 64, 2048, [3, 0, 1, 5]
    e = len(rows_per_expert)
    blocks = synth.kquant_blocks(qt, e * n * k // 256, seed=23 + qt).reshape(e, n * k // 256, -1)
    x = synth.activations(sum(rows_per_expert), k, seed=8)
    off = np.concatenate([[0], np.cumsum(rows_per_expert)]).astype(np.int32)
    ref = kq.vecdot_moe(blocks, x, off, n, k, qt)
    out = qb.gguf_vecdot_moe(_cuda(blocks), _cuda(x), torch.from_numpy(off).to(DEV), qt)
    assert kq.max_rel(out.cpu().numpy(), ref) < 4e-3
    _wait_ok()


@pytest.mark.parametrize("qt", [12, 14])
@pytest.mark.parametrize("n_a,n_b,k", [(14336, 14336, 4096), (97, 53, 4096), (33, 1, 2048), (40, 24, 14336)])
def test_two_matrices_one_launch(qt, n_a, n_b, k):
    """gate and up in one launch: both outputs equal what one launch per matrix gives, bit for bit, and the oracle."""
    ba = synth.kquant_blocks(qt, n_a * k // 256, seed=n_a + qt)
    bb = synth.kquant_blocks(qt, n_b * k // 256, seed=n_b + qt + 1)
    x = synth.activations(1, k, seed=9)
    oa, ob = qb.gguf_vecdot_dense2(_cuda(ba), _cuda(bb), _cuda(x), n_a, n_b, k, qt)
    sa = qb.gguf_vecdot_dense(_cuda(ba), _cuda(x), n_a, k, qt)
    sb = qb.gguf_vecdot_dense(_cuda(bb), _cuda(x), n_b, k, qt)
    assert torch.equal(oa, sa) and torch.equal(ob, sb)
    cols = np.unique(np.concatenate([[0, n_a - 1], np.random.default_rng(1).integers(0, n_a, 64)]))
    sub = ba.reshape(n_a, k // 256, -1)[cols].reshape(-1, ba.shape[1])
    assert kq.max_rel(oa.cpu().numpy()[:, cols], kq.vecdot_dense(sub, x, len(cols), k, qt)) < TOL
    _wait_ok()


def test_q4k_activation_extremes():
    n, k = 64, 1024
    blocks = synth.kquant_blocks(12, n * k // 256, seed=9)
    for scale in (0.0, 1e-4, 1.0, 200.0, 6.0e4 / 8):
        x = (synth.activations(1, k, seed=2).astype(np.float32) * scale).astype(np.float16)
        ref = kq.vecdot_dense(blocks, x, n, k, 12)
        out = qb.gguf_vecdot_dense(_cuda(blocks), _cuda(x), n, k, 12).cpu().numpy()
        if scale == 0.0:
            assert np.all(out == 0.0)
        else:
            assert kq.max_rel(out, ref) < TOL


@pytest.mark.parametrize("m", [1, 3])
def test_generic_raw_kernel_all_formats(qtype, m):
    n, k = 70, 1536
    blocks = synth.kquant_blocks(qtype, n * k // 256, seed=qtype)
    x = synth.activations(m, k, seed=4)
    out = qb.gguf_vecdot_rows(_cuda(blocks), _cuda(x), n, k, qtype)
    assert kq.max_rel(out.cpu().numpy(), kq.vecdot_dense(blocks, x, n, k, qtype)) < TOL


@pytest.mark.parametrize("rows_per_expert", [[3, 0, 1, 9], [0, 0, 5], [1], [2, 2, 2, 2, 2, 2, 2, 2]])
def test_vecdot_moe_ragged(qtype, rows_per_expert):
    n, k = 48, 1024
    e = len(rows_per_expert)
    blocks = synth.kquant_blocks(qtype, e * n * k // 256, seed=17 + qtype).reshape(e, n * k // 256, -1)
    total = sum(rows_per_expert)
    x = synth.activations(total, k, seed=6)
    off = np.concatenate([[0], np.cumsum(rows_per_expert)]).astype(np.int32)
    ref = kq.vecdot_moe(blocks, x, off, n, k, qtype)
    for where in ("cuda", "cpu"):
        b, xx, oo = torch.from_numpy(blocks), torch.from_numpy(x), torch.from_numpy(off)
        if where == "cuda":
            b, xx, oo = b.to(DEV), xx.to(DEV), oo.to(DEV)
        out = qb.gguf_vecdot_moe(b, xx, oo, qtype)
        assert out.shape == (total, n)
        assert kq.max_rel(out.cpu().numpy(), ref) < TOL
    _wait_ok()


# ---- scale-first planes -----------------------------------------------------------------------------------------------

@pytest.mark.parametrize("n,k", [(256, 1024), (512, 4096), (256, 14336)])
def test_scale_first_gemv_dense(qtype, n, k):
    f = kq.fmt(qtype)
    blocks = synth.kquant_blocks(qtype, n * k // 256, seed=qtype + n)
    low, high, scale, zero = kq.prepare_gemv(blocks, n, k, qtype)
    a = synth.activations(2, k, seed=8)
    ref = kq.planes_matmul(a, low, high, scale, zero, f.lo_bits, f.hi_bits, f.group_size)
    args = [_cuda(a), _cuda(low), _cuda(high), _cuda(scale), _cuda(zero)]
    out = qb.gguf_gemv_scale_first(*args, qtype)
    assert out.dtype == torch.float16 and out.shape == (2, n)
    assert kq.max_rel(out.float().cpu().numpy(), ref) < TOL
    if n * k <= 256 * 4096:
        host = qb.gguf_gemv_scale_first(*[t.cpu() for t in args], qtype)
        assert kq.max_rel(host.float().numpy(), ref) < TOL
    _wait_ok()


def test_scale_first_gemv_moe(qtype):
    f = kq.fmt(qtype)
    n, k, rows = 64, 1024, [2, 0, 5, 4]                 # enough rows per expert for the four-rows-per-pass kernel
    e = len(rows)
    blocks = synth.kquant_blocks(qtype, e * n * k // 256, seed=qtype).reshape(e, n * k // 256, -1)
    low, high, scale, zero = kq.prepare_gemv(blocks, n, k, qtype)
    a = synth.activations(sum(rows), k, seed=8)
    off = np.concatenate([[0], np.cumsum(rows)]).astype(np.int32)
    ref = kq.planes_matmul(a, low, high, scale, zero, f.lo_bits, f.hi_bits, f.group_size, off)
    for where in ("cuda", "cpu"):
        ts = [torch.from_numpy(np.ascontiguousarray(t)) for t in (a, low, high, scale, zero, off)]
        if where == "cuda":
            ts = [t.to(DEV) for t in ts]
        out = qb.gguf_gemv_scale_first_moe(*ts, qtype)
        assert kq.max_rel(out.float().cpu().numpy(), ref) < TOL
    _wait_ok()


GENERIC = [(4, 128, 4096, 4096), (4, 32, 512, 1024), (4, 64, 256, 2048), (2, 64, 768, 2048), (2, 64, 2048, 768),
           (1, 64, 768, 2048), (1, 64, 2048, 768), (2, 32, 256, 512), (1, 128, 256, 1024), (4, 16, 256, 512)]


@pytest.mark.parametrize("bits,gs,n,k", GENERIC)
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_generic_plane_gemv_dense(bits, gs, n, k, dtype):
    low, scale, zero = synth.group_planes(1, n, k, bits, gs, seed=bits * gs)
    a32 = synth.activations(2, k, seed=3, dtype=np.float32)
    at = torch.from_numpy(a32).to(dtype)
    ref = kq.planes_matmul(at.float().numpy(), low, None, scale, zero, bits, 0, gs)
    out = qb.gemv_plane(at.to(DEV), _cuda(low), None, _cuda(scale), _cuda(zero), bits, 0, gs)
    assert out.dtype == dtype
    tol = TOL if dtype == torch.float16 else 6e-3          # bf16 output rounding
    assert kq.max_rel(out.float().cpu().numpy(), ref) < tol
    # folded zero-point form: W = (q - 2^(bits-1)) * scale, no zero plane
    out2 = qb.gemv_plane(at.to(DEV), _cuda(low), None, _cuda(scale), None, bits, 0, gs, code_offset=-(1 << (bits - 1)),
                         out_dtype=torch.float32)
    ref2 = kq.planes_matmul(at.float().numpy(), low, None, scale, None, bits, 0, gs, code_offset=-(1 << (bits - 1)))
    assert kq.max_rel(out2.cpu().numpy(), ref2) < TOL
    _wait_ok()


@pytest.mark.parametrize("bits,gs,n,k", [(4, 128, 4096, 4096), (4, 128, 2048, 4096), (4, 128, 64, 3072), (4, 128, 64, 8192),
                                         (2, 16, 64, 14336), (2, 64, 256, 14336), (1, 64, 1536, 2048), (4, 32, 72, 1024),
                                         (4, 128, 16384, 4096), (2, 64, 16384, 4096), (4, 64, 40, 512)])
def test_generic_plane_gemv_single_row_shapes(bits, gs, n, k):
    # one activation row through the row-thread kernel: several row blocks per CTA, K split over few / all warps, ragged
    # last stage of a ring (K not a multiple of 1024), n a multiple of 8 only (8-row tiles), of 16 (two weight rows per lane),
    # and large enough for the 32-row tiles (four weight rows per lane)
    low, scale, zero = synth.group_planes(1, n, k, bits, gs, seed=bits + n)
    x = synth.activations(1, k, seed=4)
    out = qb.gemv_plane(_cuda(x), _cuda(low), None, _cuda(scale), _cuda(zero), bits, 0, gs, out_dtype=torch.float32)
    assert kq.max_rel(out.cpu().numpy(), kq.planes_matmul(x, low, None, scale, zero, bits, 0, gs)) < TOL
    _wait_ok()


@pytest.mark.parametrize("rows", [[0, 3, 1, 0, 0, 8, 2, 1, 0, 0, 4, 0, 1, 1, 0, 2], [5, 0, 9, 4, 1, 8, 2, 3, 0, 6, 4, 7, 1, 5, 0, 2]],
                         ids=["row_per_pass", "four_rows_per_pass"])
@pytest.mark.parametrize("bits", [2, 1])
def test_generic_plane_gemv_decode_moe(bits, rows):
    # Qwen3-30B-A3B-like decode shape at reduced expert count: ragged rows, empty experts; the second row list has enough
    # rows per expert for the kernel that shares every weight tile among up to four rows
    e, n, k, gs = 16, 768, 2048, 64
    low, scale, zero = synth.group_planes(e, n, k, bits, gs, seed=bits)
    a = torch.from_numpy(synth.activations(sum(rows), k, seed=1, dtype=np.float32)).to(torch.bfloat16)
    off = np.concatenate([[0], np.cumsum(rows)]).astype(np.int32)
    ref = kq.planes_matmul(a.float().numpy(), low, None, scale, zero, bits, 0, gs, off)
    out = qb.gemv_plane(a.to(DEV), _cuda(low), None, _cuda(scale), _cuda(zero), bits, 0, gs, row_offsets=_cuda(off),
                        out_dtype=torch.float32)
    assert kq.max_rel(out.cpu().numpy(), ref) < TOL
    _wait_ok()


# ---- merged artifact (planes + packed units) ----------------------------------------------------------------------------

@pytest.mark.parametrize("n,k", [(256, 1024), (512, 4096)])
def test_bc_gemv_dense(qtype, n, k):
    blocks = synth.kquant_blocks(qtype, n * k // 256, seed=qtype * 3)
    low, high, units = qb.gguf_prepare_fully_quantized_dense(torch.from_numpy(blocks), n, k, qtype)
    a = synth.activations(1, k, seed=12)
    ref = kq.vecdot_dense(blocks, a, n, k, qtype)
    out = qb.gguf_gemv_bc(_cuda(a), low.to(DEV), high.to(DEV), units.to(DEV), qtype)
    assert out.dtype == torch.float32 and out.shape == (1, n)
    assert kq.max_rel(out.cpu().numpy(), ref) < TOL
    host = qb.gguf_gemv_bc(torch.from_numpy(a), low, high, units, qtype)
    assert kq.max_rel(host.numpy(), ref) < TOL
    _wait_ok()


@pytest.mark.parametrize("n,k", [(256, 9728), (1024, 14336), (4096, 512)])
def test_bc_gemv_dense_row_pair_segments(qtype, n, k):
    """K segments per row: 38 superblocks = three segments of 13 (a two-superblock unit straddles a segment boundary),
    56 = four of 14, and rows of two superblocks; more CTAs than SMs' worth of rows and fewer."""
    blocks = synth.kquant_blocks(qtype, n * k // 256, seed=qtype * 7 + n % 13)
    low, high, units = qb.gguf_prepare_fully_quantized_dense(torch.from_numpy(blocks), n, k, qtype)
    a = synth.activations(1, k, seed=14)
    rows = np.random.default_rng(3).choice(n, size=min(n, 192), replace=False)
    rows[:4] = [0, 1, n - 2, n - 1]
    bb = blocks.shape[1]
    ref = kq.vecdot_dense(blocks.reshape(n, -1, bb)[rows].reshape(-1, bb), a, len(rows), k, qtype)
    out = qb.gguf_gemv_bc(_cuda(a), low.to(DEV), high.to(DEV), units.to(DEV), qtype)
    assert kq.max_rel(out.cpu().numpy()[:, rows], ref) < TOL
    _wait_ok()


@pytest.mark.parametrize("rows", [[1, 0, 4, 2], [1, 0, 1, 1]], ids=["ragged", "one_row_each"])
def test_bc_gemv_moe(qtype, rows):
    n, k = 256, 1024
    e = len(rows)
    blocks = synth.kquant_blocks(qtype, e * n * k // 256, seed=qtype * 5)
    low, high, units = qb.gguf_prepare_fully_quantized_grouped(torch.from_numpy(blocks), n, k, qtype, e)
    a = synth.activations(sum(rows), k, seed=13)
    off = np.concatenate([[0], np.cumsum(rows)]).astype(np.int32)
    ref = kq.vecdot_moe(blocks.reshape(e, -1, blocks.shape[1]), a, off, n, k, qtype)
    out = qb.gguf_gemv_bc_moe(_cuda(a), low.to(DEV), high.to(DEV), units.to(DEV), _cuda(off), qtype)
    assert kq.max_rel(out.cpu().numpy(), ref) < TOL
    _wait_ok()


# ---- runtime contract ---------------------------------------------------------------------------------------------------

def test_injected_host_failures_leave_output_untouched():
    L = _lib.lib()
    g = load_golden(12)
    b = torch.from_numpy(g["blocks"])
    for kind in (1, 2, 3, 4, 6):
        out = torch.full((b.shape[0], 256), 7.0, dtype=torch.float16)
        L.quactlize_b200_rt_fail_next(kind)
        rc = L.quactlize_ppu_dequantize(b.data_ptr(), 144, out.data_ptr(), b.shape[0], 12)
        assert rc == 41 and L.quactlize_b200_rt_last_status() == kind
        assert bool((out == 7.0).all())
    out = qb.gguf_dequantize(b, 12)                       # the latch clears on the next call
    assert np.array_equal(_bits(out), g["dequant"].view(np.uint16))


@pytest.mark.parametrize("rows", [1, 3], ids=["row_thread", "mma"])
def test_dependent_launch_chain_reads_the_previous_output(rows):
    """Two GEMVs back to back on one stream, the second reading the first one's fp16 output as its activations, replayed
    from a CUDA graph.  The kernels are launched with programmatic stream serialisation, so the second may be scheduled
    while the first drains: its result is right only if nothing of its input is read before the dependency wait."""
    k1, n1, n2 = 512, 1024, 256
    l1, s1, z1 = synth.group_planes(1, n1, k1, 4, 64, seed=11)
    l2, s2, z2 = synth.group_planes(1, n2, n1, 4, 128, seed=12)
    s1 = (s1.astype(np.float32) * 0.05).astype(np.float16)          # keeps the intermediate well inside fp16
    z1 = (z1.astype(np.float32) * 0.05).astype(np.float16)
    d1, d2 = [_cuda(t) for t in (l1, s1, z1)], [_cuda(t) for t in (l2, s2, z2)]
    xs = [torch.from_numpy(synth.activations(rows, k1, seed=20 + i)).to(DEV) for i in range(4)]
    x = torch.empty_like(xs[0])

    def chain():
        mid = qb.gemv_plane(x, d1[0], None, d1[1], d1[2], 4, 0, 64)
        return mid, qb.gemv_plane(mid, d2[0], None, d2[1], d2[2], 4, 0, 128, out_dtype=torch.float32)

    x.copy_(xs[0]); chain(); torch.cuda.synchronize()                 # plans and tensor maps exist before the capture
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        mid, out = chain()
    for xi in xs:
        x.copy_(xi)
        g.replay(); g.replay()
        torch.cuda.synchronize()
        ref_mid = kq.planes_matmul(xi.float().cpu().numpy(), l1, None, s1, z1, 4, 0, 64).astype(np.float16)
        assert kq.max_rel(mid.float().cpu().numpy(), ref_mid.astype(np.float32)) < TOL
        ref = kq.planes_matmul(mid.float().cpu().numpy(), l2, None, s2, z2, 4, 0, 128)   # from the device's own intermediate
        assert kq.max_rel(out.cpu().numpy(), ref) < TOL
    _wait_ok()


@pytest.mark.parametrize("rows", [3, 5, 7, 8, 11])
@pytest.mark.parametrize("bits,gs,n,k", [(4, 128, 512, 1024), (2, 64, 288, 2048), (1, 64, 256, 1024)])
def test_generic_plane_gemv_dense_batches(bits, gs, n, k, rows):
    # small dense batches through the tensor-core kernel: every count of held activation rows (their skewed rows must leave
    # the regions behind them aligned), more rows than one group holds, n a multiple of 32 and of 16 only
    low, scale, zero = synth.group_planes(1, n, k, bits, gs, seed=bits * 7 + rows)
    x = synth.activations(rows, k, seed=9)
    out = qb.gemv_plane(_cuda(x), _cuda(low), None, _cuda(scale), _cuda(zero), bits, 0, gs, out_dtype=torch.float32)
    assert kq.max_rel(out.cpu().numpy(), kq.planes_matmul(x, low, None, scale, zero, bits, 0, gs)) < TOL
    _wait_ok()
