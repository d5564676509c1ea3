"""K-pack artifact files on CPU: a small synthetic GGUF (k-quant tensors of random blocks, one expert-major tensor, one
fp32 tensor, a few metadata keys) is packed, verified against itself and against the source, and loaded back in the
layout the kernels read.  The container is the reference's: where its checkout is present, its own pure-Python
`reference/gguf_kpack.py` is imported by path and must (a) verify a file packed here and (b) pack a file that loads
and verifies here."""
import importlib.util
import os

import numpy as np
import pytest
import torch

gguf = pytest.importorskip("gguf")

import quactlize_b200 as qb
from conftest import ROOT
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
    assert len(manifest["tensors"]) == 6 and len(manifest["source_tensors"]) == 8
    assert [r["source_name"] for r in manifest["tensors"]][:2] == ["blk.0.w10.weight", "blk.0.w11.weight"]
    assert manifest["tensors"][5]["grouped"] is True and manifest["tensors"][5]["experts"] == 2
    assert kpack_file.verify(str(out)) == manifest
    assert kpack_file.verify(str(out), str(src)) == manifest
    r = gguf.GGUFReader(str(out))
    assert len(r.tensors) == 8 + 6 * 2 + 3                              # every source tensor kept + low/units (+ high for three formats)
    assert str(r.fields["general.name"].contents()) == "synthetic" and list(r.fields["test.ints"].contents()) == [1, 2, 3]
    assert r.fields["quactlize.kpack.reference.schema"].contents() == "quactlize.kquant-kpack.reference-gguf"
    assert {t.name for t in r.tensors if t.name.startswith("__qkpack_ref.000002.")} == {"__qkpack_ref.000002.low", "__qkpack_ref.000002.units"}
    for name, (qt, blocks, n, k, e) in tensors.items():
        low, high, units, n2, k2, qt2, e2 = kpack_file.load(str(out), name)
        assert (n2, k2, qt2, e2) == (n, k, qt, e)
        want = (qb.gguf_prepare_fully_quantized_dense(torch.from_numpy(blocks), n, k, qt) if e == 1
                else qb.gguf_prepare_fully_quantized_grouped(torch.from_numpy(blocks), n, k, qt, e))
        assert torch.equal(low, want[0]) and torch.equal(high, want[1]) and torch.equal(units.reshape(want[2].shape), want[2])
    with pytest.raises(KeyError):
        kpack_file.load(str(out), "blk.0.small.weight")                 # kept, not converted
    with pytest.raises(FileExistsError):
        kpack_file.pack(str(src), str(out))
    with pytest.raises(ValueError):
        kpack_file.pack(str(src), str(tmp_path / "x.gguf"), tensors=["blk.0.small.weight"])   # named but not convertible
    with pytest.raises(ValueError):
        kpack_file.pack(str(out), str(tmp_path / "y.gguf"))             # the input already owns the namespace


def test_verify_catches_a_flipped_bit(tmp_path):
    src, out = tmp_path / "m.gguf", tmp_path / "m.kpack.gguf"
    _source(src)
    kpack_file.pack(str(src), str(out), tensors=["blk.0.w12.weight"])
    r = gguf.GGUFReader(str(out))
    for victim in (".low", "blk.0.w12.weight"):                          # a carrier, then the source tensor it must reproduce
        t = next(t for t in r.tensors if t.name.endswith(victim))
        data = bytearray(open(out, "rb").read())
        data[int(t.data_offset) + 5] ^= 0x10
        bad = tmp_path / f"bad{victim.replace('.', '_')}.gguf"
        bad.write_bytes(bytes(data))
        with pytest.raises(ValueError):
            kpack_file.verify(str(bad))
    with pytest.raises(ValueError):
        kpack_file.verify(str(src))                       # no manifest: not an artifact


REF_KPACK = os.path.join(os.environ.get("QUACTLIZE_REFERENCE_ROOT", os.path.join(os.path.dirname(ROOT), "reference")),
                         "reference", "gguf_kpack.py")


def _ref_module():
    spec = importlib.util.spec_from_file_location("ref_gguf_kpack", REF_KPACK)
    mod = importlib.util.module_from_spec(spec)
    import sys
    sys.modules["ref_gguf_kpack"] = mod                  # its dataclasses resolve their own module by name
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.skipif(not os.path.exists(REF_KPACK), reason="reference checkout not present")
def test_reference_verifier_accepts_a_file_packed_here(tmp_path):
    src, out = tmp_path / "m.gguf", tmp_path / "m.kpack.gguf"
    _source(src)
    ours = kpack_file.pack(str(src), str(out))
    theirs = _ref_module().verify_reference_gguf(str(out), source_path=str(src))
    assert theirs == ours


@pytest.mark.skipif(not os.path.exists(REF_KPACK), reason="reference checkout not present")
def test_file_packed_by_the_reference_loads_and_verifies_here(tmp_path):
    src, out = tmp_path / "m.gguf", tmp_path / "m.ref.gguf"
    tensors = _source(src)
    names = ["blk.0.w13.weight", "blk.0.w11.weight", "blk.0.experts.weight"]      # its packer is scalar Python: keep it to three
    theirs = _ref_module().pack_reference_gguf(str(src), str(out), tensor_names=names)
    assert kpack_file.verify(str(out), str(src)) == theirs
    for name in names:
        qt, blocks, n, k, e = tensors[name]
        low, high, units, *_ = kpack_file.load(str(out), name)
        want = (qb.gguf_prepare_fully_quantized_dense(torch.from_numpy(blocks), n, k, qt) if e == 1
                else qb.gguf_prepare_fully_quantized_grouped(torch.from_numpy(blocks), n, k, qt, e))
        assert torch.equal(low, want[0]) and torch.equal(high, want[1]) and torch.equal(units.reshape(want[2].shape), want[2])
    # and the same selection packed here is the same file content, carrier for carrier
    mine = tmp_path / "m.mine.gguf"
    assert kpack_file.pack(str(src), str(mine), tensors=names) == theirs
