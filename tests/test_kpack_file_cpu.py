"""K-pack artifact files on CPU: a small synthetic GGUF (k-quant tensors of random blocks, one expert-major tensor, one
fp32 tensor, a few metadata keys) is packed, verified against itself and against the source, and loaded back in the
layout the kernels read."""
import numpy as np
import pytest
import torch

gguf = pytest.importorskip("gguf")

import quactlize_b200 as qb
from quactlize_b200 import kpack_file, synth

QT = {10: gguf.GGMLQuantizationType.Q2_K, 11: gguf.GGMLQuantizationType.Q3_K, 12: gguf.GGMLQuantizationType.Q4_K,
      13: gguf.GGMLQuantizationType.Q5_K, 14: gguf.GGMLQuantizationType.Q6_K}


def _source(path):
    w = gguf.GGUFWriter(str(path), "llama")
    w.add_uint32("llama.block_count", 1)
    w.add_string("general.name", "synthetic")
    w.add_array("test.ints", [1, 2, 3])
    tensors = {}
    for qt in (10, 11, 12, 13, 14):
        n, k = 256, 512
        b = synth.kquant_blocks(qt, n * k // 256, seed=qt)
        tensors[f"blk.0.w{qt}.weight"] = (qt, b, n, k, 1)
        w.add_tensor(f"blk.0.w{qt}.weight", b.reshape(n, -1), raw_dtype=QT[qt])
    e, n, k = 2, 256, 256
    b = synth.kquant_blocks(12, e * n * k // 256, seed=77)
    tensors["blk.0.experts.weight"] = (12, b, n, k, e)
    w.add_tensor("blk.0.experts.weight", b.reshape(e, n, -1), raw_dtype=QT[12])
    small = synth.kquant_blocks(12, 96 * 256 // 256, seed=5)            # n = 96: not convertible, copied verbatim
    w.add_tensor("blk.0.small.weight", small.reshape(96, -1), raw_dtype=QT[12])
    w.add_tensor("norm.weight", np.arange(8, dtype=np.float32))
    w.write_header_to_file(); w.write_kv_data_to_file(); w.write_tensors_to_file(); w.close()
    return tensors


def test_pack_verify_load(tmp_path):
    src, out = tmp_path / "m.gguf", tmp_path / "m.kpack.gguf"
    tensors = _source(src)
    manifest = kpack_file.pack(str(src), str(out))
    assert len(manifest["converted"]) == 6 and manifest["source_tensors"] == 8
    assert kpack_file.verify(str(out)) == {"converted": 6, "tensors": 2 + 5 * 3 - 2 + 2, "source_checked": False}
    assert kpack_file.verify(str(out), str(src))["source_checked"] is True
    r = gguf.GGUFReader(str(out))
    assert str(r.fields["general.name"].contents()) == "synthetic" and list(r.fields["test.ints"].contents()) == [1, 2, 3]
    for name, (qt, blocks, n, k, e) in tensors.items():
        low, high, units, n2, k2, qt2, e2 = kpack_file.load(str(out), name)
        assert (n2, k2, qt2, e2) == (n, k, qt, e)
        want = (qb.gguf_prepare_fully_quantized_dense(torch.from_numpy(blocks), n, k, qt) if e == 1
                else qb.gguf_prepare_fully_quantized_grouped(torch.from_numpy(blocks), n, k, qt, e))
        assert torch.equal(low, want[0]) and torch.equal(high, want[1]) and torch.equal(units.reshape(want[2].shape), want[2])


def test_verify_catches_a_flipped_bit(tmp_path):
    src, out = tmp_path / "m.gguf", tmp_path / "m.kpack.gguf"
    _source(src)
    kpack_file.pack(str(src), str(out), tensors=["blk.0.w12.weight"])
    r = gguf.GGUFReader(str(out))
    t = next(t for t in r.tensors if t.name.endswith(".low"))
    data = bytearray(open(out, "rb").read())
    data[int(t.data_offset) + 5] ^= 0x10
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(bytes(data))
    with pytest.raises(ValueError):
        kpack_file.verify(str(bad))
    with pytest.raises(ValueError):
        kpack_file.verify(str(src))                       # no manifest: not an artifact
