"""K-pack artifact files: a GGUF whose k-quant weight tensors are replaced by K-pack carriers plus a manifest.

Mirrors the file mode of the reference's `reference/gguf_kpack.py` (pack_reference_gguf :1124-1230, verify_reference_gguf
:1099-1121): every convertible tensor (Q2_K..Q6_K, n % 256 == 0, k % 256 == 0, k % 512 == 0 for Q3_K / Q6_K; 2-D, or 3-D
expert-major) becomes three I8 tensors -- low plane, high plane, packed units, in the canonical K-pack order of
`quactlize_b200.kpack` -- and a manifest record with its geometry and the SHA-256 of the source bytes; every other tensor
and every metadata key is copied.  `verify` rebuilds the official blocks from the carriers and checks them against the
manifest (and against the source file when given), so the container is byte-neutral by construction.

    python -m quactlize_b200.kpack_file pack  model.gguf model.kpack.gguf
    python -m quactlize_b200.kpack_file verify model.kpack.gguf [model.gguf]

Needs the `gguf` package (reader / writer of the container format).
"""
from __future__ import annotations

import argparse
import hashlib
import json
import sys
from typing import Dict, Optional, Sequence

import numpy as np
import torch

from . import kpack
from .formats import QuantType, kquant_geometry

MANIFEST_KEY = "quactlize.kpack.manifest"
VERSION_KEY = "quactlize.kpack.version"
VERSION = 1
_KQ = {10, 11, 12, 13, 14}


def _gguf():
    try:
        import gguf
    except Exception as e:                                   # pragma: no cover
        raise RuntimeError("the gguf package is needed to read or write artifact files") from e
    return gguf


def _sha(b: bytes) -> str:
    return hashlib.sha256(b).hexdigest()


def _geometry(tensor, qtype: int):
    """(n, k, experts) of a GGUF tensor (dims are stored innermost first) or None when K-pack does not cover it."""
    dims = [int(x) for x in tensor.shape]
    if len(dims) == 2:
        k, n, e = dims[0], dims[1], 1
    elif len(dims) == 3:
        k, n, e = dims
    else:
        return None
    if n % 256 or k % 256 or (qtype in (QuantType.Q3_K, QuantType.Q6_K) and k % 512):
        return None
    return n, k, e


def _blocks(tensor, n: int, k: int, experts: int, qtype: int) -> torch.Tensor:
    g = kquant_geometry(qtype)
    raw = np.ascontiguousarray(np.asarray(tensor.data)).view(np.uint8).reshape(experts * n * (k // 256), g.block_bytes)
    return torch.from_numpy(raw.copy())


def _copy_metadata(reader, writer) -> None:
    gguf = _gguf()
    for key, field in reader.fields.items():
        if key.startswith("GGUF.") or key in ("general.architecture", MANIFEST_KEY, VERSION_KEY):
            continue
        vtype = field.types[0]
        sub = field.types[-1] if vtype == gguf.GGUFValueType.ARRAY else None
        writer.add_key_value(key, field.contents(), vtype, sub_type=sub)


def _architecture(reader) -> str:
    f = reader.fields.get("general.architecture")
    return str(f.contents()) if f is not None else "unknown"


def pack(source: str, out: str, tensors: Optional[Sequence[str]] = None) -> Dict:
    """Write `out` from the GGUF `source`; `tensors` restricts the conversion to the named tensors.  Returns the manifest."""
    gguf = _gguf()
    reader = gguf.GGUFReader(source)
    writer = gguf.GGUFWriter(out, _architecture(reader))
    _copy_metadata(reader, writer)
    records = []
    for index, t in enumerate(reader.tensors):
        qtype = int(t.tensor_type)
        geo = _geometry(t, qtype) if qtype in _KQ and (tensors is None or t.name in tensors) else None
        if geo is None:
            writer.add_tensor(t.name, np.asarray(t.data), raw_dtype=t.tensor_type)
            continue
        n, k, e = geo
        blocks = _blocks(t, n, k, e, qtype)
        low, high, units = (kpack.prepare_dense(blocks, n, k, qtype) if e == 1 else kpack.prepare_grouped(blocks, n, k, qtype, e))
        names = {}
        for part, ten in (("low", low), ("high", high), ("units", units)):
            if ten.numel() == 0:
                names[part] = None
                continue
            name = f"kpack.{index}.{part}"
            writer.add_tensor(name, ten.contiguous().numpy().view(np.int8))
            names[part] = {"name": name, "shape": list(ten.shape)}
        records.append({"index": index, "name": t.name, "qtype": qtype, "n": n, "k": k, "experts": e,
                        "source_sha256": _sha(blocks.numpy().tobytes()), "carriers": names})
    manifest = {"version": VERSION, "source_tensors": len(reader.tensors), "converted": records}
    writer.add_key_value(VERSION_KEY, VERSION, gguf.GGUFValueType.UINT32)
    writer.add_key_value(MANIFEST_KEY, json.dumps(manifest, sort_keys=True), gguf.GGUFValueType.STRING)
    writer.write_header_to_file()
    writer.write_kv_data_to_file()
    writer.write_tensors_to_file()
    writer.close()
    return manifest


def _manifest(reader) -> Dict:
    f = reader.fields.get(MANIFEST_KEY)
    if f is None:
        raise ValueError("not a K-pack artifact: no manifest")
    m = json.loads(str(f.contents()))
    if int(m.get("version", -1)) != VERSION:
        raise ValueError(f"unsupported K-pack artifact version {m.get('version')}")
    return m


def _carrier(by_name, spec, role: str) -> torch.Tensor:
    if spec is None:
        return torch.zeros((0,), dtype=torch.uint8)
    if spec["name"] not in by_name:
        raise ValueError(f"carrier {spec['name']} ({role}) is missing")
    a = np.ascontiguousarray(np.asarray(by_name[spec["name"]].data)).view(np.uint8).reshape(spec["shape"])
    return torch.from_numpy(a.copy())


def load(path: str, name: str):
    """One converted weight of an artifact file as (low, high, units, n, k, qtype, experts), planes in NATIVE order, i.e.
    what the GEMV / GEMM entries of this library consume."""
    gguf = _gguf()
    reader = gguf.GGUFReader(path)
    by_name = {t.name: t for t in reader.tensors}
    for rec in _manifest(reader)["converted"]:
        if rec["name"] == name:
            low, high, units = (_carrier(by_name, rec["carriers"][p], p) for p in ("low", "high", "units"))
            nl, nh, nu = kpack.to_native(low, high, units, rec["n"], rec["k"], rec["qtype"])
            return nl, nh, nu, rec["n"], rec["k"], rec["qtype"], rec["experts"]
    raise KeyError(name)


def verify(path: str, source: Optional[str] = None) -> Dict:
    """Rebuild the official blocks of every converted tensor and compare with the manifest (and the source file)."""
    gguf = _gguf()
    reader = gguf.GGUFReader(path)
    manifest = _manifest(reader)
    by_name = {t.name: t for t in reader.tensors}
    src = {t.name: t for t in gguf.GGUFReader(source).tensors} if source else None
    checked = 0
    for rec in manifest["converted"]:
        low, high, units = (_carrier(by_name, rec["carriers"][p], p) for p in ("low", "high", "units"))
        raw = kpack.recover_raw_blocks(low, high, units, rec["n"], rec["k"], rec["qtype"]).numpy().tobytes()
        if _sha(raw) != rec["source_sha256"]:
            raise ValueError(f"{rec['name']}: recovered blocks do not match the manifest digest")
        if src is not None:
            if rec["name"] not in src:
                raise ValueError(f"{rec['name']}: not in the source file")
            if np.ascontiguousarray(np.asarray(src[rec["name"]].data)).view(np.uint8).tobytes() != raw:
                raise ValueError(f"{rec['name']}: recovered blocks differ from the source file")
        checked += 1
    if src is not None:
        converted = {r["name"] for r in manifest["converted"]}
        for name, t in src.items():
            if name in converted:
                continue
            if name not in by_name or np.asarray(by_name[name].data).tobytes() != np.asarray(t.data).tobytes():
                raise ValueError(f"{name}: copied tensor differs from the source file")
    return {"converted": checked, "tensors": len(reader.tensors), "source_checked": source is not None}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="K-pack artifact files")
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("pack"); p.add_argument("source"); p.add_argument("out"); p.add_argument("--tensor", action="append")
    v = sub.add_parser("verify"); v.add_argument("path"); v.add_argument("source", nargs="?")
    args = ap.parse_args(argv)
    if args.cmd == "pack":
        m = pack(args.source, args.out, args.tensor)
        print(json.dumps({"converted": len(m["converted"]), "source_tensors": m["source_tensors"]}))
    else:
        print(json.dumps(verify(args.path, args.source)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
