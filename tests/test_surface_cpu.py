"""The kept Python surface (formats / routes) against the reference's own pure-Python modules, imported by path from its
checkout.  Skipped when the checkout is absent (it does not travel to the GPU box).  Every (format, rows, flag)
combination must select the same path or raise the same exception type; tables and derived quantities must agree."""
import importlib.util
import inspect
import os

import pytest

from quactlize_b200 import formats as ours

from conftest import ROOT

REF_ROOT = os.environ.get("QUACTLIZE_REFERENCE_ROOT") or os.path.join(os.path.dirname(ROOT), "reference")
REF_FORMATS = os.path.join(REF_ROOT, "quactlize", "formats.py")

pytestmark = pytest.mark.skipif(not os.path.exists(REF_FORMATS), reason="reference checkout not present")


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.fixture(scope="module")
def ref():
    return _load(REF_FORMATS, "ref_quactlize_formats")


def _outcome(fn, *args, **kw):
    try:
        return ("ok", fn(*args, **kw))
    except Exception as e:                             # the TYPE of the refusal is part of the contract
        return ("raises", type(e).__name__)


def test_quant_types_and_block_table_agree(ref):
    assert {m.name: int(m) for m in ours.QuantType} == {m.name: int(m) for m in ref.QuantType}
    assert set(map(int, ours.BLOCKS)) == set(map(int, ref.BLOCKS))
    for q in ref.BLOCKS:
        a, b = ours.BLOCKS[ours.QuantType(int(q))], ref.BLOCKS[q]
        assert tuple(a) == tuple(b), q
        assert a.fp16_plane_bytes == b.fp16_plane_bytes and a.bytes_on_fp16_scale_path == b.bytes_on_fp16_scale_path
        assert a.fp16_scale_growth == b.fp16_scale_growth


def test_select_path_agrees_everywhere(ref):
    rows = [0, 1, 2, 8, 64, 511, 512, 513, 4096]
    for q in ref.QuantType:
        for r in rows:
            for native in (True, False):
                for planes in ("auto", "workspace", "never", "bogus"):
                    want = _outcome(ref.select_path, q, r, native, planes)
                    got = _outcome(ours.select_path, ours.QuantType(int(q)), r, native, planes)
                    assert got == want, (q.name, r, native, planes)


def test_storage_growth_and_native_scale_agree(ref):
    for q in ref.QuantType:
        o = ours.QuantType(int(q))
        assert ours.storage_growth(o) == ref.storage_growth(q)
        for budget in (0.0, 0.05, 0.5):
            assert ours.needs_native_scale(o, budget) == ref.needs_native_scale(q, budget)
    assert ours.DENSE_CROSSOVER_ROWS == ref.DENSE_CROSSOVER_ROWS and ours.GEMV_MAX_ROWS == ref.GEMV_MAX_ROWS
    for name in ("GEMV", "FUSED_NATIVE_SCALE", "FUSED_FP16_SCALE", "DEQUANT_THEN_DENSE"):
        assert set(map(int, getattr(ours, name))) == set(map(int, getattr(ref, name))), name


def test_fold_and_placed_arrangement_agree(ref):
    for bits in (1, 2, 3, 4, 5, 6, 8):
        for tk in (1, 2, 4, 8, 16, 32, 48, 64, 128, 256, 512):
            assert _outcome(ours.fold_for, bits, tk) == _outcome(ref.fold_for, bits, tk), (bits, tk)
    for bits, tk, hb in ((4, 256, 0), (4, 32, 1), (2, 64, 1), (1, 64, 0), (4, 128, 2), (2, 512, 0)):
        a, b = ours.PlacedArrangement(bits, tk, hb), ref.PlacedArrangement(bits, tk, hb)
        assert (a.fold, a.high_fold, a.layout_is_tile_free()) == (b.fold, b.high_fold, b.layout_is_tile_free())
    assert {int(k): v for k, v in ours.PLACED_CODE_ZMUL.items()} == {int(k): v for k, v in ref.PLACED_CODE_ZMUL.items()}
    for q in ref.QuantType:
        assert _outcome(ours.placed_code_zmul, int(q)) == _outcome(ref.placed_code_zmul, int(q))


def test_route_surface_has_every_reference_route():
    """Same public names and the same positional parameters as the reference's routes module (read as text: importing
    it needs the reference's compiled extension)."""
    import ast
    from quactlize_b200 import routes
    src = open(os.path.join(REF_ROOT, "quactlize", "routes.py")).read()
    tree = ast.parse(src)
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and not node.name.startswith("_"):
            assert hasattr(routes, node.name), f"routes.{node.name} is missing"
            want = [a.arg for a in node.args.args]
            got = list(inspect.signature(getattr(routes, node.name)).parameters)[:len(want)]
            assert got == want, (node.name, got, want)
    ref_routes = None
    for node in tree.body:
        if isinstance(node, ast.Assign) and getattr(node.targets[0], "id", "") == "ROUTES":
            ref_routes = [k.value for k in node.value.keys]
    assert ref_routes and all(k in routes.ROUTES for k in ref_routes)


def test_op_surface_has_every_reference_gguf_op():
    """Every gguf_* wrapper of the reference's package (quactlize/__init__.py) exists here with the same parameters."""
    import ast
    import quactlize_b200 as qb
    tree = ast.parse(open(os.path.join(REF_ROOT, "quactlize", "__init__.py")).read())
    skipped = {"gguf_q4_artifact_dequantize"}          # consumes the GPTQ mixed_gemm layout: lives in quactlize_b200.gptq
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name.startswith("gguf_") and node.name not in skipped:
            assert hasattr(qb, node.name), f"quactlize_b200.{node.name} is missing"
            want = [a.arg for a in node.args.args]
            got = list(inspect.signature(getattr(qb, node.name)).parameters)[:len(want)]
            assert got == want, (node.name, got, want)
