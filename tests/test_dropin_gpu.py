"""Drop-in check: the REFERENCE's own host extension (built from its sources into oracle/_ref) dlopens this library
through QUACTLIZE_PPU_LIB and its ops forward to the B200 kernels.  Runs in a child process because the reference
caches its load attempt per process (quactlize/csrc/preprocess/thop/ppu_backend.cpp:51-64)."""
import os
import subprocess
import sys
import textwrap

import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu

CHILD = textwrap.dedent('''
    import glob, os, sys
    import numpy as np, torch
    sys.path.insert(0, os.environ["QB_ROOT"])
    from oracle import kquant as kq
    from quactlize_b200 import synth
    torch.ops.load_library(glob.glob(os.path.join(os.environ["QB_ROOT"], "oracle", "_ref", "quactlize_ref_C*.so"))[0])
    q = torch.ops.quactlize
    backend = q.gguf_backend()
    assert backend.startswith("ppu"), backend
    for qt in (10, 11, 12, 13, 14):
        n, k = 256, 1024
        blocks = synth.kquant_blocks(qt, n * k // 256, seed=qt)
        tb = torch.from_numpy(blocks)
        x = torch.from_numpy(synth.activations(1, k, seed=1))
        ref = kq.vecdot_dense(blocks, x.numpy(), n, k, qt)
        assert kq.max_rel(q.gguf_vecdot_dense(tb, x, n, k, qt).numpy(), ref) < 2e-3
        assert np.array_equal(q.gguf_dequantize(tb, qt).numpy().view(np.uint16), kq.dequantize(blocks, qt).view(np.uint16))
        low, high, scale, zero = q.gguf_prepare_gemv(tb, n, k, qt)
        f = kq.fmt(qt)
        out = q.gguf_gemv_scale_first(x, low, high, scale, zero, qt)
        ref2 = kq.planes_matmul(x.numpy(), low.numpy(), high.numpy(), scale.numpy(), zero.numpy(), f.lo_bits, f.hi_bits, f.group_size)
        assert kq.max_rel(out.float().numpy(), ref2) < 2e-3
        lo2, hi2, units = q.gguf_prepare_fully_quantized_dense(tb, n, k, qt)
        assert kq.max_rel(q.gguf_gemv_bc(x, lo2, hi2, units, qt).numpy(), ref) < 2e-3
        e, rows = 3, [2, 0, 1]
        eb = torch.from_numpy(synth.kquant_blocks(qt, e * n * k // 256, seed=qt + 50)).view(e, n * k // 256, -1)
        xa = torch.from_numpy(synth.activations(3, k, seed=2))
        off = torch.tensor([0, 2, 2, 3], dtype=torch.int32)
        refm = kq.vecdot_moe(eb.numpy(), xa.numpy(), off.numpy(), n, k, qt)
        assert kq.max_rel(q.gguf_vecdot_moe(eb, xa, off, qt).numpy(), refm) < 2e-3
        # ---- the tensor-core family through the reference's ops (dense scale-first, fully-quantized dense and grouped) ----
        m = 70
        am = torch.from_numpy(synth.activations(m, k, seed=3))
        refw = am.numpy().astype(np.float64) @ kq.dequantize_f32(blocks, qt).reshape(n, k).T
        dart = q.gguf_prepare_dense(tb, n, k, qt)
        got = q.gguf_dense_scale_first(am, *dart, qt)
        assert got.dtype == torch.float16 and kq.max_rel(got.float().numpy(), refw) < 6e-3
        wdq = q.gguf_dense_artifact_dequantize(*dart, qt)                 # placed inverse through recover_dense
        assert kq.max_rel(wdq[0].float().numpy(), kq.dequantize_f32(blocks, qt).reshape(n, k)) < 2e-3
        got = q.gguf_dense_fully_quantized(am, lo2, hi2, units, qt)
        assert kq.max_rel(got.float().numpy(), refw) < 6e-3
        sc_u, ze_u = q.gguf_packed_scale_prepass(units, qt, 0)
        sc_o, ze_o = kq.units_decode(units.numpy()[None], qt, 0)
        assert np.array_equal(sc_u.numpy().view(np.uint16), sc_o.view(np.uint16)) and np.array_equal(ze_u.numpy().view(np.uint16), ze_o.view(np.uint16))
        ge, grow = 3, [130, 0, 37]
        gb = synth.kquant_blocks(qt, ge * n * k // 256, seed=qt + 90)
        glo, ghi, gun = q.gguf_prepare_fully_quantized_grouped(torch.from_numpy(gb), n, k, qt, ge)
        ga = torch.from_numpy(synth.activations(sum(grow), k, seed=4))
        gout = q.gguf_grouped_fully_quantized(ga, glo, ghi, gun, torch.tensor(grow, dtype=torch.int32), qt)
        goff = np.concatenate([[0], np.cumsum(grow)]).astype(np.int32)
        gref = kq.vecdot_moe(gb.reshape(ge, n * k // 256, -1), ga.numpy(), goff, n, k, qt)
        assert kq.max_rel(gout.float().numpy(), gref) < 6e-3
        # scale-first and merged-form MoE GEMVs
        art_m = q.gguf_prepare_gemv(eb, n, k, qt)
        om = q.gguf_gemv_scale_first_moe(xa, *art_m, off, qt)
        refp = kq.planes_matmul(xa.numpy(), *[t.numpy() for t in art_m], f.lo_bits, f.hi_bits, f.group_size, off.numpy())
        assert kq.max_rel(om.float().numpy(), refp) < 2e-3
    print("DROPIN_OK", backend)
''')


def test_reference_extension_forwards_to_this_library():
    ref = [f for f in os.listdir(os.path.join(ROOT, "oracle", "_ref"))] if os.path.isdir(os.path.join(ROOT, "oracle", "_ref")) else []
    if not any(f.startswith("quactlize_ref_C") and f.endswith(".so") for f in ref):
        pytest.skip("reference host extension not built (oracle/build_ref.py needs the reference checkout)")
    env = dict(os.environ, QB_ROOT=ROOT, QUACTLIZE_PPU_LIB=os.path.join(ROOT, "quactlize_b200", "csrc", "libquactlize_b200.so"))
    r = subprocess.run([sys.executable, "-c", CHILD], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "DROPIN_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
