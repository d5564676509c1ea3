"""K-pack artifact files in the reference's container: an AUGMENTED GGUF that keeps every source tensor and metadata
field and appends, for each converted k-quant weight, three I8 carrier tensors (low plane, high plane, packed units in
the canonical K-pack order of `quactlize_b200.kpack`) plus a versioned JSON manifest.

The container is the one `reference/gguf_kpack.py` of the reference project writes and verifies (schema and metadata
keys :73-79, carrier names :800-803, manifest fields :867-907 and :1206-1212, verification :1099-1121), so a file
packed here passes the reference's `verify_reference_gguf` and a file packed by the reference loads here:

    metadata   quactlize.kpack.reference.schema   = "quactlize.kquant-kpack.reference-gguf"   (string)
               quactlize.kpack.reference.version  = 1                                         (uint32)
               quactlize.kpack.reference.manifest = JSON, keys sorted, no whitespace          (string)
    carriers   __qkpack_ref.NNNNNN.low / .high / .units   (NNNNNN = index of the converted tensor, GGML I8)
    manifest   schema, schema_version,
               source_metadata [{index, name, types, sha256}]            every source metadata field, file order
               source_tensors  [{index, name, tensor_type, type_name, shape, nbytes, sha256}]
               tensors         [{index, source_index, source_name, qtype, n, k, experts, grouped, arrangement, carriers}]

Convertible: Q2_K..Q6_K tensors of GGUF shape [K, N] or [K, N, E] with N % 256 == 0 and K % 256 == 0 (K % 512 for Q3_K and
Q6_K, whose units pair two superblocks).  `verify` rebuilds the official blocks from the carriers and compares them
with the source tensor kept in the same file, byte for byte; `load` returns a weight in the NATIVE plane order the
GEMV / GEMM entries of this library read.

    python -m quactlize_b200.kpack_file pack   model.gguf model.kpack-reference.gguf [--tensor NAME ...]
    python -m quactlize_b200.kpack_file verify model.kpack-reference.gguf [--source model.gguf]

Needs the `gguf` package (reader / writer of the container format).
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import sys
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from . import kpack
from .formats import kquant_geometry

SCHEMA = "quactlize.kquant-kpack.reference-gguf"
SCHEMA_VERSION = 1
PREFIX = "quactlize.kpack.reference."
SCHEMA_KEY, VERSION_KEY, MANIFEST_KEY = PREFIX + "schema", PREFIX + "version", PREFIX + "manifest"
CARRIER_PREFIX = "__qkpack_ref."
_KQ = (10, 11, 12, 13, 14)
_ARR_FIELDS = ("version", "layout", "bits", "high_bits", "artifact_tile_k", "transport_tile_k", "group_size", "reserved",
               "mapping_id")


def _gguf():
    try:
        import gguf
    except Exception as e:                                   # pragma: no cover
        raise RuntimeError("the gguf package is needed to read or write artifact files") from e
    return gguf


def _sha(b: bytes) -> str:
    return hashlib.sha256(b).hexdigest()


def _bytes_of(array) -> bytes:
    return np.ascontiguousarray(array).view(np.uint8).reshape(-1).tobytes()


def arrangement(qtype: int) -> Dict[str, int]:
    """The serialized identity of the carrier bytes of one format (reference/gguf_kpack.py:175-187): arrangement
    version 2; Q4_K is layout 1 (4-bit K-pack, transport tile 64), the others layout 2 with a transport tile of
    16 * max codes-per-16-bit-word over the format's planes."""
    g = kquant_geometry(int(qtype))
    if int(qtype) == 12:
        vals = (2, 1, 4, 0, 0, 64, 32, 0, 0x51344B5034540001)
    else:
        packs = [16 // g.lo_bits] + ([16 // g.hi_bits] if g.hi_bits else [])
        vals = (2, 2, g.lo_bits, g.hi_bits, 0, 16 * max(packs), g.group_size, 0, 0x514B504B54000001)
    return dict(zip(_ARR_FIELDS, vals))


def _geometry(tensor, qtype: int):
    """(n, k, experts, grouped) of a GGUF tensor (dims are stored innermost first) or None when K-pack does not cover it."""
    dims = [int(x) for x in tensor.shape]
    if len(dims) not in (2, 3):
        return None
    k, n = dims[0], dims[1]
    e = dims[2] if len(dims) == 3 else 1
    per_unit = kquant_geometry(qtype).sb_per_unit
    if n <= 0 or n % 256 or k <= 0 or k % (256 * per_unit) or e <= 0:
        return None
    return n, k, e, len(dims) == 3


def _blocks(tensor, n: int, k: int, experts: int, qtype: int) -> torch.Tensor:
    g = kquant_geometry(qtype)
    raw = np.frombuffer(_bytes_of(tensor.data), dtype=np.uint8)
    want = experts * n * (k // 256) * g.block_bytes
    if raw.size != want:
        raise ValueError(f"{tensor.name}: GGUF payload has {raw.size} bytes, expected {want}")
    return torch.from_numpy(raw.reshape(-1, g.block_bytes).copy())


def _metadata(reader) -> Dict[str, object]:
    """Serialized model metadata: fields that carry value types, without the reader's own GGUF.* header counts."""
    return {name: f for name, f in reader.fields.items() if f.types and not name.startswith("GGUF.")}


def _field_sha(field) -> str:
    h = hashlib.sha256()
    for part in field.parts:
        raw = part.tobytes()
        h.update(len(raw).to_bytes(8, "little"))
        h.update(raw)
    return h.hexdigest()


def _carrier_name(index: int, part: str) -> str:
    return f"{CARRIER_PREFIX}{index:06d}.{part}"


def _shapes(n: int, k: int, e: int, grouped: bool, qtype: int):
    g = kquant_geometry(qtype)
    nu = (k // 256) // g.sb_per_unit
    return ([e, n, k * g.lo_bits // 8], [e, n, k * g.hi_bits // 8] if g.hi_bits else [0],
            [e, nu, n, g.unit_total] if grouped else [nu, n, g.unit_total])


def pack(source: str, out: str, tensors: Optional[Sequence[str]] = None) -> Dict:
    """Write the augmented GGUF `out` from `source`; `tensors` restricts the conversion to the named tensors (a named
    tensor that cannot be converted is an error; without names, tensors K-pack does not cover are simply kept).
    The file is verified before it gets its final name.  Returns the manifest."""
    gguf = _gguf()
    if os.path.abspath(source) == os.path.abspath(out):
        raise ValueError("input and output GGUF paths must differ")
    if os.path.lexists(out):
        raise FileExistsError(f"refusing to overwrite existing output {out}")
    reader = gguf.GGUFReader(source)
    if reader.endianess != gguf.GGUFEndian.LITTLE:
        raise ValueError("K-pack 16-bit carriers require a little-endian input GGUF")
    meta = _metadata(reader)
    clash = sorted(nm for nm in meta if nm.startswith(PREFIX)) + sorted(t.name for t in reader.tensors if t.name.startswith(CARRIER_PREFIX))
    if clash:
        raise ValueError("input already owns the K-pack reference namespace: " + ", ".join(clash[:8]))
    names = {t.name for t in reader.tensors}
    if tensors is not None:
        if len(set(tensors)) != len(tensors):
            raise ValueError("tensor names must not be repeated")
        missing = sorted(set(tensors) - names)
        if missing:
            raise ValueError("requested tensor(s) are absent: " + ", ".join(missing))
    selected = {}
    for t in reader.tensors:
        if tensors is not None and t.name not in tensors:
            continue
        qt = int(t.tensor_type)
        geo = _geometry(t, qt) if qt in _KQ else None
        if geo is None:
            if tensors is not None:
                raise ValueError(f"requested tensor {t.name!r} ({t.tensor_type.name}, shape {list(map(int, t.shape))}) is not convertible")
            continue
        selected[t.name] = geo
    if not selected:
        raise ValueError("input/selection contains no convertible Q2_K/Q3_K/Q4_K/Q5_K/Q6_K tensor")
    arch = reader.get_field("general.architecture")
    if arch is None or not isinstance(arch.contents(), str) or not arch.contents():
        raise ValueError("input GGUF has no general.architecture string")

    partial = f"{out}.partial.{os.getpid()}"
    writer = gguf.GGUFWriter(partial, arch.contents(), use_temp_file=True, endianess=gguf.GGUFEndian.LITTLE)
    writer.data_alignment = int(reader.alignment)
    try:
        for name, field in meta.items():
            if name == "general.architecture":               # written by the writer's constructor
                continue
            vtype = field.types[0]
            sub = field.types[-1] if vtype == gguf.GGUFValueType.ARRAY else None
            writer.add_key_value(name, field.contents(), vtype, sub_type=sub)
        source_records, index_of = [], {}
        for index, t in enumerate(reader.tensors):
            raw = _bytes_of(t.data)
            index_of[t.name] = index
            source_records.append({"index": index, "name": t.name, "tensor_type": int(t.tensor_type), "type_name": t.tensor_type.name,
                                   "shape": [int(x) for x in t.shape], "nbytes": len(raw), "sha256": _sha(raw)})
            writer.add_tensor(t.name, t.data, raw_shape=t.data.shape, raw_dtype=t.tensor_type, tensor_endianess=reader.endianess)
        converted: List[dict] = []
        for t in reader.tensors:
            if t.name not in selected:
                continue
            n, k, e, grouped = selected[t.name]
            qt = int(t.tensor_type)
            blocks = _blocks(t, n, k, e, qt)
            low, high, units = kpack.prepare_grouped(blocks, n, k, qt, e) if grouped else kpack.prepare_dense(blocks, n, k, qt)
            idx = len(converted)
            carriers = {}
            for part, ten, shape in zip(("low", "high", "units"), (low, high, units), _shapes(n, k, e, grouped, qt)):
                if ten.numel() == 0:
                    carriers[part] = None
                    continue
                data = ten.contiguous().reshape(shape).numpy().view(np.int8)      # I8 is GGUF's one-byte carrier type
                writer.add_tensor(_carrier_name(idx, part), data)
                carriers[part] = {"name": _carrier_name(idx, part), "shape": shape, "sha256": _sha(_bytes_of(data))}
            converted.append({"index": idx, "source_index": index_of[t.name], "source_name": t.name, "qtype": qt, "n": n, "k": k,
                              "experts": e, "grouped": grouped, "arrangement": arrangement(qt), "carriers": carriers})
        manifest = {"schema": SCHEMA, "schema_version": SCHEMA_VERSION,
                    "source_metadata": [{"index": i, "name": nm, "types": [int(v) for v in f.types], "sha256": _field_sha(f)}
                                        for i, (nm, f) in enumerate(meta.items())],
                    "source_tensors": source_records, "tensors": converted}
        writer.add_string(SCHEMA_KEY, SCHEMA)
        writer.add_uint32(VERSION_KEY, SCHEMA_VERSION)
        writer.add_string(MANIFEST_KEY, json.dumps(manifest, sort_keys=True, separators=(",", ":")))
        writer.write_header_to_file()
        writer.write_kv_data_to_file()
        writer.write_tensors_to_file()
    finally:
        writer.close()
    try:
        verify(partial, source)
        os.link(partial, out)
    finally:
        os.unlink(partial)
    return manifest


def _manifest(reader) -> Dict:
    gguf = _gguf()
    meta = _metadata(reader)
    reserved = {nm for nm in meta if nm.startswith(PREFIX)}
    if reserved != {SCHEMA_KEY, VERSION_KEY, MANIFEST_KEY}:
        raise ValueError("not a K-pack artifact: the reference metadata keys are missing or unexpected "
                         f"(found {sorted(reserved)})")
    s, v, m = (reader.get_field(x) for x in (SCHEMA_KEY, VERSION_KEY, MANIFEST_KEY))
    if s.types != [gguf.GGUFValueType.STRING] or s.contents() != SCHEMA:
        raise ValueError(f"{SCHEMA_KEY} is invalid")
    if v.types != [gguf.GGUFValueType.UINT32] or v.contents() != SCHEMA_VERSION:
        raise ValueError(f"unsupported K-pack artifact version {v.contents()}")
    if m.types != [gguf.GGUFValueType.STRING]:
        raise ValueError(f"{MANIFEST_KEY} is not a string")
    try:
        manifest = json.loads(m.contents())
    except (TypeError, json.JSONDecodeError) as e:
        raise ValueError("K-pack manifest is not valid JSON") from e
    want = {"schema", "schema_version", "source_metadata", "source_tensors", "tensors"}
    if not isinstance(manifest, dict) or set(manifest) != want:
        raise ValueError(f"K-pack manifest must contain exactly {sorted(want)}")
    if manifest["schema"] != SCHEMA or manifest["schema_version"] != SCHEMA_VERSION:
        raise ValueError("K-pack manifest schema/version is unsupported")
    for key in ("source_metadata", "source_tensors", "tensors"):
        if not isinstance(manifest[key], list) or not manifest[key]:
            raise ValueError(f"K-pack manifest has an empty {key} list")
    return manifest


def _carrier(by_name, record, name: str, shape: List[int], role: str) -> torch.Tensor:
    gguf = _gguf()
    if not isinstance(record, dict) or set(record) != {"name", "shape", "sha256"}:
        raise ValueError(f"{role} carrier record has the wrong fields")
    if record["name"] != name or record["shape"] != shape:
        raise ValueError(f"{role} carrier identity/shape is not canonical")
    t = by_name.get(name)
    if t is None or t.tensor_type != gguf.GGMLQuantizationType.I8:
        raise ValueError(f"{role} carrier {name} is missing or is not GGML I8")
    if list(t.data.shape) != shape:
        raise ValueError(f"{role} carrier {name}: GGUF shape disagrees with its manifest")
    raw = _bytes_of(t.data)
    if record["sha256"] != _sha(raw):
        raise ValueError(f"{role} carrier {name} checksum mismatch")
    return torch.from_numpy(np.frombuffer(raw, dtype=np.uint8).reshape(shape).copy())


def _record_artifact(by_name, rec, position: int):
    """(low, high, units) carriers of one manifest record, checked against the record and its source tensor's geometry."""
    src = by_name.get(rec.get("source_name"))
    if src is None:
        raise ValueError(f"converted tensor record {position}: source tensor {rec.get('source_name')!r} is not in the file")
    qt = rec["qtype"]
    if qt not in _KQ or qt != int(src.tensor_type):
        raise ValueError(f"converted tensor {src.name}: qtype disagrees with the source")
    geo = _geometry(src, qt)
    if geo is None or (rec["n"], rec["k"], rec["experts"], rec["grouped"]) != geo:
        raise ValueError(f"converted tensor {src.name}: geometry disagrees with the source")
    if rec["arrangement"] != arrangement(qt):
        raise ValueError(f"converted tensor {src.name}: arrangement is not canonical")
    n, k, e, grouped = geo
    carriers = rec["carriers"]
    if not isinstance(carriers, dict) or set(carriers) != {"low", "high", "units"}:
        raise ValueError(f"converted tensor {src.name}: carriers must name low/high/units exactly")
    lo_s, hi_s, un_s = _shapes(n, k, e, grouped, qt)
    low = _carrier(by_name, carriers["low"], _carrier_name(position, "low"), lo_s, "low")
    units = _carrier(by_name, carriers["units"], _carrier_name(position, "units"), un_s, "units")
    used = {_carrier_name(position, "low"), _carrier_name(position, "units")}
    if kquant_geometry(qt).hi_bits:
        high = _carrier(by_name, carriers["high"], _carrier_name(position, "high"), hi_s, "high")
        used.add(_carrier_name(position, "high"))
    else:
        if carriers["high"] is not None:
            raise ValueError(f"converted tensor {src.name}: format has no high plane")
        high = torch.zeros((0,), dtype=torch.uint8)
    return src, (low, high, units), geo, used


def verify(path: str, source: Optional[str] = None) -> Dict:
    """Check an augmented GGUF: the manifest's inventories against the file, every carrier's checksum, and the official
    blocks rebuilt from every artifact against the source tensor kept in the file; with `source`, also that every
    original tensor and metadata field is preserved byte for byte.  Returns the manifest."""
    gguf = _gguf()
    reader = gguf.GGUFReader(path)
    if reader.endianess != gguf.GGUFEndian.LITTLE:
        raise ValueError("K-pack 16-bit carriers require a little-endian GGUF")
    manifest = _manifest(reader)
    by_name = {t.name: t for t in reader.tensors}
    meta = {nm: f for nm, f in _metadata(reader).items() if not nm.startswith(PREFIX)}
    if len(manifest["source_metadata"]) != len(meta):
        raise ValueError("source metadata inventory length changed")
    for pos, rec in enumerate(manifest["source_metadata"]):
        f = meta.get(rec.get("name")) if isinstance(rec, dict) else None
        if f is None or rec.get("index") != pos or rec.get("types") != [int(v) for v in f.types] or rec.get("sha256") != _field_sha(f):
            raise ValueError(f"source metadata record {pos} does not match the file")
    source_names = set()
    for pos, rec in enumerate(manifest["source_tensors"]):
        t = by_name.get(rec.get("name")) if isinstance(rec, dict) else None
        if t is None or rec.get("index") != pos or rec["name"] in source_names or rec["name"].startswith(CARRIER_PREFIX):
            raise ValueError(f"source tensor record {pos} does not match the file")
        raw = _bytes_of(t.data)
        if (rec.get("tensor_type") != int(t.tensor_type) or rec.get("type_name") != t.tensor_type.name or
                rec.get("shape") != [int(x) for x in t.shape] or rec.get("nbytes") != len(raw) or rec.get("sha256") != _sha(raw)):
            raise ValueError(f"source tensor {rec['name']}: identity or byte payload changed")
        source_names.add(rec["name"])
    carriers, seen = set(), set()
    for pos, rec in enumerate(manifest["tensors"]):
        if not isinstance(rec, dict) or rec.get("index") != pos:
            raise ValueError(f"converted tensor record {pos} has a noncanonical identity")
        src, (low, high, units), (n, k, e, grouped), used = _record_artifact(by_name, rec, pos)
        si = rec.get("source_index")
        if si in seen or not isinstance(si, int) or si >= len(manifest["source_tensors"]) or manifest["source_tensors"][si]["name"] != src.name:
            raise ValueError(f"converted tensor record {pos} has an invalid source binding")
        seen.add(si)
        carriers |= used
        restored = kpack.recover_raw_blocks(low, high, units, n, k, rec["qtype"])
        want = _blocks(src, n, k, e, rec["qtype"])
        if not torch.equal(restored, want):
            raise ValueError(f"converted tensor {src.name}: recovered official GGUF blocks differ in {int((restored != want).sum())} bytes")
    if set(by_name) != source_names | carriers:
        raise ValueError("GGUF tensor inventory disagrees with the manifest")
    if source is not None:
        src_reader = gguf.GGUFReader(source)
        src_meta = _metadata(src_reader)
        if set(src_meta) != set(meta):
            raise ValueError("source metadata keys were not preserved")
        for nm, f in src_meta.items():
            if [int(v) for v in f.types] != [int(v) for v in meta[nm].types] or [p.tobytes() for p in f.parts] != [p.tobytes() for p in meta[nm].parts]:
                raise ValueError(f"source metadata {nm!r} was not preserved byte-exactly")
        for t in src_reader.tensors:
            o = by_name.get(t.name)
            if o is None or o.tensor_type != t.tensor_type or list(o.shape) != list(t.shape) or _bytes_of(o.data) != _bytes_of(t.data):
                raise ValueError(f"source tensor {t.name!r} was not preserved byte-exactly")
    return manifest


def load(path: str, name: str):
    """One converted weight of an artifact file as (low, high, units, n, k, qtype, experts): planes in NATIVE order and
    units [E, U, n, bytes], i.e. what the GEMV / GEMM entries of this library consume.  Works on files packed here and on
    files packed by the reference."""
    gguf = _gguf()
    reader = gguf.GGUFReader(path)
    by_name = {t.name: t for t in reader.tensors}
    for pos, rec in enumerate(_manifest(reader)["tensors"]):
        if rec.get("source_name") == name:
            _, (low, high, units), (n, k, e, _), _ = _record_artifact(by_name, rec, pos)
            nl, nh, nu = kpack.to_native(low, high, units, n, k, rec["qtype"])
            return nl, nh, nu, n, k, rec["qtype"], e
    raise KeyError(name)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="K-pack artifact files (the reference's augmented-GGUF container)")
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("pack"); p.add_argument("source"); p.add_argument("out"); p.add_argument("--tensor", action="append")
    v = sub.add_parser("verify"); v.add_argument("path"); v.add_argument("--source")
    args = ap.parse_args(argv)
    try:
        m = pack(args.source, args.out, args.tensor) if args.cmd == "pack" else verify(args.path, args.source)
    except (ValueError, FileExistsError, RuntimeError) as e:
        print(f"KPACK_REFERENCE_GGUF FAIL {e}", file=sys.stderr)
        return 1
    print(f"KPACK_REFERENCE_GGUF PASS action={args.cmd} converted={len(m['tensors'])} source_tensors={len(m['source_tensors'])}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
