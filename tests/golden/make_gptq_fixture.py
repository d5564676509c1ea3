"""Generate tests/golden/gptq_mixed_gemm_q4.npz by running the REFERENCE's own offline preprocessor.

Run where the reference checkout exists:  python tests/golden/make_gptq_fixture.py
For two shapes (one non-square) seeded 4-bit codes go through the reference's pack_int4 and
preprocess_weights_to_layout(..., "mixed_gemm"); the stored bytes are recorded next to the codes.  For one Q4_K weight
the stored int4 matrix and the packed units are also fed to the reference's gguf_q4_artifact_dequantize and its float32
result recorded."""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import build_ref, kquant as kq  # noqa: E402
from quactlize_b200 import synth  # noqa: E402


def main():
    lib = build_ref.build()
    if lib is None:
        raise SystemExit("reference checkout not present")
    os.environ["QUACTLIZE_PPU_LIB"] = "/nonexistent/so-the-cpu-arms-run.so"
    torch.ops.load_library(lib)
    q = torch.ops.quactlize
    out = {}
    for tag, (k, n) in {"a": (128, 128), "b": (64, 192)}.items():
        codes = np.random.default_rng(7 + k + n).integers(0, 16, size=(k, n)).astype(np.uint8)
        packed = q.pack_int8_tensor_to_packed_int4(torch.from_numpy(codes.astype(np.int8) - 8))
        stored = q.preprocess_weights_to_layout(packed, torch.quint4x2, "mixed_gemm")
        out[f"codes_{tag}"], out[f"stored_{tag}"] = codes, stored.numpy()
    n, k = 64, 512
    blocks = synth.kquant_blocks(12, n * k // 256, seed=4242)
    codes = kq.codes(blocks, 12).reshape(n, k).T.astype(np.int8)              # [K, N]
    packed = q.pack_int8_tensor_to_packed_int4(torch.from_numpy(np.ascontiguousarray(codes) - 8))
    stored = q.preprocess_weights_to_layout(packed, torch.quint4x2, "mixed_gemm")
    tb = torch.from_numpy(blocks)
    nsb = k // 256
    sblk = tb[:, 4:16].contiguous().view(n, nsb, 12)
    d = tb[:, 0:2].contiguous().view(torch.float16).view(n, nsb)
    dm = tb[:, 2:4].contiguous().view(torch.float16).view(n, nsb)
    units = q.gguf_pack_unit(sblk, d, dm, 12)[0]
    out["q4k_blocks"], out["q4k_stored"], out["q4k_units"] = blocks, stored.numpy(), units.numpy()
    out["q4k_dequant"] = q.gguf_q4_artifact_dequantize(stored, units, "mixed_gemm").numpy()
    np.savez_compressed(os.path.join(HERE, "gptq_mixed_gemm_q4.npz"), **out)
    print({k_: v.shape for k_, v in out.items()})


if __name__ == "__main__":
    main()
