"""Generate the committed golden vectors by running the REFERENCE's own host ops on seeded inputs.

Run where the reference checkout exists:  python tests/golden/make_golden.py
It builds (or reuses) the reference host extension via oracle/build_ref.py, feeds it seeded raw k-quant blocks and
stores inputs plus the reference's outputs in tests/golden/kquant_<NAME>.npz.  The tests then check both the numpy
oracle and the CUDA kernels against these files without needing the reference checkout.

Ops recorded per format (all CPU arms of torch.ops.quactlize.*): gguf_dequantize, gguf_unpack, gguf_prepare_gemv,
gguf_gemv_artifact_dequantize, gguf_pack_unit (3-D artifact form), gguf_packed_scale_prepass for every accepted
zmul, gguf_scale_prepass (zmul 0 and 8), gguf_vecdot_dense (fp16 activation).
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import build_ref  # noqa: E402
from quactlize_b200 import synth  # noqa: E402

N, K = 32, 1024
NAMES = {10: "Q2_K", 11: "Q3_K", 12: "Q4_K", 13: "Q5_K", 14: "Q6_K"}
# (scale block offset, scale block bytes, d offset, dmin offset) inside the raw block
SLICES = {10: (0, 16, 80, 82), 11: (96, 12, 108, -1), 12: (4, 12, 0, 2), 13: (4, 12, 0, 2), 14: (192, 16, 208, -1)}


def main():
    lib = build_ref.build()
    if lib is None:
        raise SystemExit("reference checkout not present")
    os.environ["QUACTLIZE_PPU_LIB"] = "/nonexistent/so-the-cpu-arms-run.so"
    torch.ops.load_library(lib)
    q = torch.ops.quactlize
    assert q.gguf_backend().startswith("cpu")
    for qt, name in NAMES.items():
        blocks = synth.kquant_blocks(qt, N * K // 256, seed=1000 + qt)
        # a few hand-made edge blocks: zero block, all-ones block, negative d
        blocks[0, :] = 0
        blocks[1, :] = 0xFF
        so, sb, do, mo = SLICES[qt]
        blocks[1, do:do + 2] = np.array([0.0123], np.float16).view(np.uint8)
        if mo >= 0:
            blocks[1, mo:mo + 2] = np.array([0.0071], np.float16).view(np.uint8)
        blocks[2, do:do + 2] = np.array([-0.0042], np.float16).view(np.uint8)
        blocks[3, do:do + 2] = np.array([3.1e-6], np.float16).view(np.uint8)      # subnormal d
        tb = torch.from_numpy(blocks.copy())
        x = torch.from_numpy(synth.activations(1, K, seed=77 + qt))
        out = {"blocks": blocks, "x": x.numpy(), "n": N, "k": K}
        out["dequant"] = q.gguf_dequantize(tb, qt).numpy()
        c, s, z = q.gguf_unpack(tb, qt)
        out["codes"], out["scale_rows"], out["zero_rows"] = c.numpy(), s.numpy(), z.numpy()
        low, high, scale, zero = q.gguf_prepare_gemv(tb, N, K, qt)
        out["low"], out["high"], out["scale"], out["zero"] = low.numpy(), high.numpy(), scale.numpy(), zero.numpy()
        out["artifact_dequant"] = q.gguf_gemv_artifact_dequantize(low, high, scale, zero, qt).numpy()
        nsb = K // 256
        sblk = tb[:, so:so + sb].contiguous().view(N, nsb, sb)
        d = tb[:, do:do + 2].contiguous().view(torch.float16).view(N, nsb)
        dm = tb[:, mo:mo + 2].contiguous().view(torch.float16).view(N, nsb) if mo >= 0 else torch.empty(0, dtype=torch.float16)
        units = q.gguf_pack_unit(sblk, d, dm, qt)[0]
        out["units"] = units.numpy()
        for zm in (-32, -24, -4, 0, 8):
            sc, ze = q.gguf_packed_scale_prepass(units, qt, zm)
            out[f"unit_scale_z{zm}"], out[f"unit_zero_z{zm}"] = sc.numpy(), ze.numpy()
        for zm in (0, 8):
            sc, ze = q.gguf_scale_prepass(sblk.view(N * nsb, sb), d.reshape(-1), dm.reshape(-1) if mo >= 0 else dm, qt, zm)
            out[f"prepass_scale_z{zm}"], out[f"prepass_zero_z{zm}"] = sc.numpy(), ze.numpy()
        out["vecdot_dense"] = q.gguf_vecdot_dense(tb, x, N, K, qt).numpy()
        path = os.path.join(HERE, f"kquant_{name}.npz")
        np.savez_compressed(path, **out)
        print(name, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
