"""The offline tuner's host logic on CPU, with an injected timer (no GPU): candidates come from the library's own
inventory and validity predicates, M maps to the last positive power of two, only measured buckets are stored, an
unresolved sweep records nothing, the run-time cache round-trips and never matches another bucket or inventory."""
import pytest

from quactlize_b200 import _lib, tune


def test_bucket_rule():
    assert [tune.m_bucket(m) for m in (-3, 0, 1, 2, 3, 4, 63, 64, 65, 4095, 4096)] == [0, 0, 1, 2, 2, 4, 32, 64, 64, 2048, 4096]
    assert tune.measured_buckets({16: "a", 64: "b", 100: "b"}) == [
        {"m_bucket": 16, "measured_m": 16, "config": "a"}, {"m_bucket": 64, "measured_m": 100, "config": "b"}]
    with pytest.raises(ValueError):
        tune.measured_buckets({64: "a", 100: "b"})                       # one bucket, two answers


def test_winner_must_be_separated():
    assert tune.pick_winner({"a": [10.0, 10.2, 10.1], "b": [12.0, 12.5, 12.2]}) == ("a", "separated")
    name, note = tune.pick_winner({"a": [10.0, 13.0, 10.1], "b": [12.0, 12.5, 12.2]})
    assert name is None and note.startswith("unresolved")
    assert tune.pick_winner({"a": [10.0]})[0] is None                     # one pass cannot rank
    assert tune.pick_winner({"a": [10.0, 10.1]}) == ("a", "only candidate")
    assert tune.pick_winner({})[0] is None


def test_inventory_and_tune_with_a_fake_timer(tmp_path):
    lib = _lib.lib()
    dense, grouped, h = tune.load_inventory(lib)
    names = [r["name"] for r in dense if not r["enable_cuda_kernel"]]
    assert names == ["256x256x64:tcgen05", "128x128x64:tcgen05"] and len(h) == 16
    assert any(r["enable_cuda_kernel"] for r in dense) and any(r["enable_cuda_kernel"] for r in grouped)
    calls = []

    def timer_for(n, k):
        def timer(m, tactic):
            calls.append((n, k, m, tactic))
            big = tactic.startswith("256")
            if m == 300:                                                  # a tie: must stay unresolved
                return 50.0
            return (40.0 if big else 60.0) if m >= 512 else (30.0 if not big else 45.0)
        return timer

    table = tune.tune(lib, "llama3-8b", "dense_fully_quantized", 12, [16, 300, 1024], reps=3, timer_for=timer_for)
    assert table["config_space_fnv1a64"] == h and table["candidates"] == names
    assert [s["n"] for s in table["shapes"]] == [4096, 14336]
    for s in table["shapes"]:
        assert s["buckets"] == [{"m_bucket": 16, "measured_m": 16, "config": "128x128x64:tcgen05"},
                                {"m_bucket": 1024, "measured_m": 1024, "config": "256x256x64:tcgen05"}]
        assert [w["note"].split(":")[0] for w in s["sweeps"]] == ["separated", "unresolved", "separated"]
    # candidates were interleaved: the first two calls are different tactics of the same M
    assert calls[0][3] != calls[1][3] and calls[0][2] == calls[1][2]

    cache = tmp_path / "t.cache"
    lines = tune.write_runtime_cache(str(cache), table, _lib.LIB_PATH, "NVIDIA B200")
    assert cache.read_text().splitlines() == lines and lines[0] == "schema=quactlize-ppu-tactic-cache-v1"
    assert sum(l.startswith("entry|") for l in lines) == 2 * 3            # two buckets x three projections
    look = lambda m, **kw: tune.lookup(lines, "dense_fully_quantized", "ffn_down", 12, 4096, 14336, 32, m, **kw)
    assert look(16) == look(31) == "128x128x64:tcgen05" and look(1024) == look(2047) == "256x256x64:tcgen05"
    assert look(300) is None and look(32) is None and look(2048) is None  # unmeasured buckets miss: compiled default
    assert look(16, config_space="0" * 16) is None                        # a cache from another inventory never matches
    assert tune.lookup(lines, "dense_fully_quantized", "ffn_down", 13, 4096, 14336, 32, 16) is None
    with pytest.raises(ValueError):
        tune.write_runtime_cache(str(cache), table, _lib.LIB_PATH, "bad|device")
    with pytest.raises(ValueError):
        tune.tune(lib, "llama3-8b", "grouped_fully_quantized", 12, [16], reps=2, timer_for=timer_for)
    with pytest.raises(ValueError):
        tune.tune(lib, "llama3-8b", "dense_fully_quantized", 12, [16], reps=1, timer_for=timer_for)


def test_grouped_route_uses_the_grouped_predicate():
    lib = _lib.lib()
    seen = []
    table = tune.tune(lib, "mixtral-8x7b", "grouped_fully_quantized", 12, [64], reps=2,
                      timer_for=lambda n, k: (lambda m, t: seen.append((m, t)) or {"128x128x64:tcgen05": 10.0, "256x256x64:tcgen05": 20.0}.get(t, 15.0)))
    assert {t for _, t in seen} == {"256x256x64:tcgen05", "128x128x64:tcgen05", "128x128x64:tcgen05:splitk"}
    assert all(s["buckets"][0]["config"] == "128x128x64:tcgen05" for s in table["shapes"])
