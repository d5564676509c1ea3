"""The route layer (quactlize_b200.routes) and the artifact inverse ops on the GPU, through the package's public functions
(each one call into the C ABI), against the numpy oracle and the reference-run goldens.  Decoded weights, codes and
fp16 planes are bit-exact; matmul results are within the bounds of oracle/checks.py."""
import numpy as np
import pytest
import torch

import quactlize_b200 as qb
from conftest import load_golden
from oracle import kquant as kq
from quactlize_b200 import _lib, formats, routes, synth

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _bits(t):
    a = t.detach().cpu().numpy()
    return a.view(np.uint16) if a.dtype == np.float16 else a


def test_unpack_bit_exact(qtype):
    g = load_golden(qtype)
    for where in ("cuda", "cpu"):
        b = torch.from_numpy(g["blocks"])
        c, s, z = qb.gguf_unpack(b.to(DEV) if where == "cuda" else b, qtype)
        assert c.dtype == torch.int8 and np.array_equal(c.cpu().numpy(), g["codes"])
        assert np.array_equal(_bits(s), g["scale_rows"].view(np.uint16))
        assert np.array_equal(_bits(z), g["zero_rows"].view(np.uint16))


def test_gemv_artifact_dequantize_bit_exact(qtype):
    g = load_golden(qtype)
    art = [torch.from_numpy(g[k]).to(DEV) for k in ("low", "high", "scale", "zero")]
    w = qb.gguf_gemv_artifact_dequantize(*art, qtype)
    assert np.array_equal(_bits(w), g["artifact_dequant"].view(np.uint16))
    s, z = qb.gguf_gemv_artifact_dequantize_scale(art[2], art[3], qtype)
    assert np.array_equal(_bits(s), np.ascontiguousarray(g["scale"].transpose(0, 2, 1)).view(np.uint16))
    assert np.array_equal(_bits(z), np.ascontiguousarray(g["zero"].transpose(0, 2, 1)).view(np.uint16))
    assert torch.equal(routes.dequantize_scale_first(art, qtype), w)


def test_unit_decode_matches_packed_prepass(qtype):
    g = load_golden(qtype)
    u = torch.from_numpy(g["units"]).to(DEV)                        # artifact form [U, n, bytes]
    for zm in (-32, -24, -4, 0, 8):
        s, z = qb.gguf_unit_decode(u, qtype, zm)                     # [n, superblocks, groups]
        n = u.shape[1]
        want_s = g[f"unit_scale_z{zm}"][0].reshape(-1, kq.fmt(qtype).groups, n).transpose(2, 0, 1)
        want_z = g[f"unit_zero_z{zm}"][0].reshape(-1, kq.fmt(qtype).groups, n).transpose(2, 0, 1)
        assert np.array_equal(_bits(s), np.ascontiguousarray(want_s).view(np.uint16))
        assert np.array_equal(_bits(z), np.ascontiguousarray(want_z).view(np.uint16))


def test_dense_artifact_two_producers_agree_and_invert(qtype):
    n, k = 256, 1024
    blocks = synth.kquant_blocks(qtype, n * k // 256, seed=31 + qtype)
    tb = torch.from_numpy(blocks)
    derived = routes.prepare_scale_first_dense(tb, n, k, qtype)                       # planes derived from the packed units
    direct = routes.prepare_scale_first_dense(tb, n, k, qtype, derive_from_bc=False)  # planes from raw blocks
    for a, b in zip(derived, direct):                 # equal as VALUES: where a sub-scale is 0 the two producers differ in the
        assert a.shape == b.shape and torch.equal(a, b)   # sign of the zero they store (each is bit-exact with its own golden)
    w = routes.dequantize_scale_first_dense([t.to(DEV) for t in derived], qtype)
    f = kq.fmt(qtype)
    want = kq.planes_dequantize(derived[0].numpy(), derived[1].numpy() if f.hi_bits else None, derived[2].numpy(),
                                derived[3].numpy(), f.lo_bits, f.hi_bits, f.group_size, code_offset=-8 if f.lo_bits == 4 else 0)
    assert np.array_equal(_bits(w), want.view(np.uint16))
    art = routes.prepare_fully_quantized_dense(tb, n, k, qtype)
    w2 = routes.dequantize_fully_quantized([t.to(DEV) for t in art], qtype)
    assert torch.equal(w2, w)
    assert kq.max_rel(w.float().cpu().numpy()[0], kq.dequantize_f32(blocks, qtype).reshape(n, k)) < 2e-3


@pytest.mark.parametrize("m", [1, 40, 600])
def test_every_dense_route_agrees_with_the_oracle(qtype, m):
    n, k = 256, 1024
    blocks = synth.kquant_blocks(qtype, n * k // 256, seed=5 + qtype + m)
    tb = torch.from_numpy(blocks)
    a = torch.from_numpy(synth.activations(m, k, seed=m)).to(DEV)
    ref = a.cpu().numpy().astype(np.float64) @ kq.dequantize_f32(blocks, qtype).reshape(n, k).T
    outs = {"dequant_first": routes.matmul_dequant_first(a, tb.to(DEV), n, k, qtype)}
    sfd = [t.to(DEV) for t in routes.prepare_scale_first_dense(tb, n, k, qtype)]
    outs["scale_first_dense"] = routes.matmul_scale_first_dense(a, sfd, qtype)
    fq = [t.to(DEV) for t in routes.prepare_fully_quantized_dense(tb, n, k, qtype)]
    outs["fully_quantized_dense"] = routes.matmul_fully_quantized_dense(a, fq, qtype)
    path, sel = routes.matmul_selected(a, fq, qtype)
    assert path == formats.select_path(formats.QuantType(qtype), m, True, "workspace")
    outs["selected:" + path] = sel
    if m == 1:
        outs["native_gemv"] = routes.matmul_native_gemv(a, tb.to(DEV), n, k, qtype)
        outs["bc_gemv"] = routes.matmul_bc_gemv(a, fq, qtype)
        outs["scale_first_gemv"] = routes.matmul_scale_first_gemv(a, [t.to(DEV) for t in routes.prepare_scale_first(tb, n, k, qtype)], qtype)
    for name, out in outs.items():
        assert tuple(out.shape) == (m, n), name
        assert kq.max_rel(out.float().cpu().numpy(), ref) < 6e-3, name
    assert m != 1 or path == "gemv"
    assert m != 600 or path == "dequant_then_dense"


def test_grouped_routes_agree_with_the_oracle(qtype):
    e, n, k = 4, 256, 1024
    rows = torch.tensor([70, 0, 3, 129], dtype=torch.int64)
    blocks = synth.kquant_blocks(qtype, e * n * k // 256, seed=77 + qtype)
    tb = torch.from_numpy(blocks)
    a = torch.from_numpy(synth.activations(int(rows.sum()), k, seed=9)).to(DEV)
    off = np.concatenate([[0], np.cumsum(rows.numpy())]).astype(np.int32)
    ref = kq.vecdot_moe(blocks.reshape(e, n * k // 256, -1), a.cpu().numpy(), off, n, k, qtype)
    fq = [t.to(DEV) for t in routes.prepare_fully_quantized_grouped(tb, n, k, qtype, e)]
    outs = {"fully_quantized_grouped": routes.matmul_fully_quantized_grouped(a, fq, qtype, rows),
            "dequant_first_grouped": routes.matmul_dequant_first_grouped(a, tb.to(DEV), n, k, qtype, e, rows),
            "native_gemv_moe": routes.matmul_native_gemv_moe(a, tb.to(DEV), n, k, qtype, e, rows),
            "bc_gemv_moe": routes.matmul_bc_gemv_moe(a, fq, qtype, e, rows)}
    for name, out in outs.items():
        assert kq.max_rel(out.float().cpu().numpy(), ref) < 6e-3, name
    wg = routes.dequantize_fully_quantized(fq, qtype, grouped=True)
    assert tuple(wg.shape) == (e, n, k)
    assert kq.max_rel(wg.float().cpu().numpy().reshape(e * n, k), kq.dequantize_f32(blocks, qtype).reshape(e * n, k)) < 2e-3


def test_route_error_behaviour():
    n, k, qt = 256, 512, 12
    blocks = torch.from_numpy(synth.kquant_blocks(qt, n * k // 256, seed=1))
    a = torch.zeros((2, k), dtype=torch.float16)
    with pytest.raises(ValueError):
        routes.matmul_native_gemv(a, blocks, n, k, qt)                       # the GEMV band is m = 1
    with pytest.raises(ValueError):
        routes.dequantize_weight(blocks, n + 1, k, qt)                       # block count disagrees with (n, k)
    with pytest.raises(ValueError):
        routes.matmul_bc_gemv(a[:1], (blocks, blocks), qt)                   # the artifact contract is three tensors
    with pytest.raises(ValueError):
        routes._row_offsets(torch.tensor([1, -1]), 2, 0)
    assert routes.has_op("gguf_dense_fully_quantized") and not routes.has_op("gguf_no_such_op")


def test_bounded_wait_that_runs_out_is_reported_and_recovers():
    """A wait on a barrier nothing arms gives up after its limit, the kernel returns normally, the status word reports it
    once, and the next real launch is unaffected."""
    L = _lib.lib()
    torch.cuda.synchronize()
    assert L.quactlize_b200_device_wait_status() == 0
    stream = torch.cuda.current_stream().cuda_stream
    assert L.quactlize_b200_debug_wait_probe(1_000_000, stream) == 0         # 1 ms
    torch.cuda.synchronize()                                                 # the kernel ended by itself
    assert L.quactlize_b200_device_wait_status() == 41
    assert L.quactlize_b200_rt_last_status() == 7                            # RtStatus::DeviceWait
    assert L.quactlize_b200_device_wait_status() == 0                        # read-and-clear
    assert L.quactlize_b200_debug_wait_probe(0, stream) == 20 and L.quactlize_b200_debug_wait_probe(10**9, stream) == 20
    n, k = 512, 4096
    blocks = synth.kquant_blocks(12, n * k // 256, seed=4)
    x = synth.activations(1, k, seed=5)
    out = qb.gguf_vecdot_dense(torch.from_numpy(blocks).to(DEV), torch.from_numpy(x).to(DEV), n, k, 12)
    assert kq.max_rel(out.cpu().numpy(), kq.vecdot_dense(blocks, x, n, k, 12)) < 2e-3
    # a host-pointer entry called while the word is set reports the failure (41) and leaves `out` untouched
    assert L.quactlize_b200_debug_wait_probe(1_000_000, stream) == 0
    torch.cuda.synchronize()
    hb, hx = torch.from_numpy(blocks), torch.from_numpy(x)
    ho = torch.full((1, n), 7.0, dtype=torch.float32)
    rc = L.quactlize_ppu_vecdot_dense(hb.data_ptr(), 144, hx.data_ptr(), ho.data_ptr(), n, k // 256, 12)
    assert rc == 41 and bool((ho == 7.0).all())
    rc = L.quactlize_ppu_vecdot_dense(hb.data_ptr(), 144, hx.data_ptr(), ho.data_ptr(), n, k // 256, 12)
    assert rc == 0 and kq.max_rel(ho.numpy(), kq.vecdot_dense(blocks, x, n, k, 12)) < 2e-3


def test_gemv_from_a_kpack_file(tmp_path):
    """A weight read back from a K-pack artifact file (the reference's augmented-GGUF container) feeds the merged-form
    GEMV and the tensor-core GEMM directly."""
    gguf = pytest.importorskip("gguf")
    from quactlize_b200 import kpack_file
    qt, n, k = 14, 256, 1024
    blocks = synth.kquant_blocks(qt, n * k // 256, seed=123)
    src, out = tmp_path / "w.gguf", tmp_path / "w.kpack.gguf"
    w = gguf.GGUFWriter(str(src), "llama")
    w.add_string("general.name", "one weight")
    w.add_tensor("blk.0.ffn_down.weight", blocks.reshape(n, -1), raw_dtype=gguf.GGMLQuantizationType.Q6_K)
    w.write_header_to_file(); w.write_kv_data_to_file(); w.write_tensors_to_file(); w.close()
    kpack_file.pack(str(src), str(out))
    low, high, units, n2, k2, qt2, e = kpack_file.load(str(out), "blk.0.ffn_down.weight")
    assert (n2, k2, qt2, e) == (n, k, qt, 1)
    x = synth.activations(1, k, seed=8)
    got = qb.gguf_gemv_bc(torch.from_numpy(x).to(DEV), low.to(DEV), high.to(DEV), units[0].to(DEV), qt)
    assert kq.max_rel(got.cpu().numpy(), kq.vecdot_dense(blocks, x, n, k, qt)) < 2e-3
    a = synth.activations(33, k, seed=9)
    gm = qb.gguf_dense_fully_quantized(torch.from_numpy(a).to(DEV), low.to(DEV), high.to(DEV), units[0].to(DEV), qt)
    assert kq.max_rel(gm.float().cpu().numpy(), kq.vecdot_dense(blocks, a, n, k, qt)) < 6e-3


def test_offline_tuner_on_the_device(tmp_path):
    """The tuner sweeps the compiled tactics on a small shape with the real device timer; whatever it resolves names a
    compiled tactic the library admits, and the cache it writes answers only the buckets that were measured."""
    from quactlize_b200 import tune
    L = _lib.lib()
    tune.MODELS["tiny-test"] = {"projections": [("ffn_gate", 512, 1024)], "experts": 0, "topk": 0}
    try:
        table = tune.tune(L, "tiny-test", "dense_fully_quantized", 12, [32, 1024], reps=3)
    finally:
        del tune.MODELS["tiny-test"]
    shape = table["shapes"][0]
    assert (shape["n"], shape["k"]) == (512, 1024) and len(shape["sweeps"]) == 2
    for sweep in shape["sweeps"]:
        assert set(sweep["median_us"]) == set(table["candidates"]) and all(v > 0 for v in sweep["median_us"].values())
    for b in shape["buckets"]:
        assert b["config"] in table["candidates"] and b["m_bucket"] in (32, 1024)
        assert L.quactlize_ppu_dense_fully_quantized_config_valid_v1(b["measured_m"], 512, 1024, 32, 12, b["config"].encode()) == 1
    torch.cuda.synchronize()
    assert L.quactlize_b200_device_wait_status() == 0
