"""Auto-tuner: symbols and spaces, the batch-size / checkpoint-ratio search
with early stop, the JSON database, log parsers, dialect registry and the CLI
driving a (fake) training script."""
import json
import textwrap

import pytest

from slapo_b200.autotune import tune as T
from slapo_b200.framework_dialect import (get_all_dialects, get_dialect_cls,
                                          register_framework_dialect)


def test_symbol_and_space():
    space = T.Space()
    bs = space.create_symbol("batch_size", [4, 8, 16])
    assert not bs.is_fixed() and len(bs) == 3
    sym = space.next()
    assert sym is bs
    sym.fix_at(1)
    assert bs.is_fixed() and bs.value == 8
    assert bs > 4 and bs >= 8 and bs < 16 and bs <= 8
    # re-creating a fixed symbol keeps it; an unfixed one takes the new candidates
    assert space.create_symbol("batch_size", [1]) is bs
    ck = space.create_symbol("ckpt", [1.0, 0.5])
    ck2 = space.create_symbol("ckpt", [0.25])
    assert ck2.vals == [0.25] and space.space["ckpt"] is ck2 and ck is not ck2
    clone = space.clone()
    clone.space["batch_size"].fix_at(0)
    assert bs.value == 8
    space.reset()
    assert not bs.is_fixed() and space.next() is bs
    assert space.next().name == "ckpt" and space.next() is None


def test_space_enumeration_with_dependent_symbols():
    def update(args, space):
        bs = space.create_symbol("batch_size", [8, 16])
        # candidates of the second symbol depend on the first
        space.create_symbol("ckpt", [1.0] if bs.is_fixed() and bs.value == 16 else [1.0, 0.5])
        return space

    space = update({}, T.Space())
    points = space.enumerate({}, update)
    assert {(p["batch_size"], p["ckpt"]) for p in points} == {(8, 1.0), (8, 0.5), (16, 1.0)}
    assert space.log_space({}, update) == 3


def _memory_model(cfg, limit=100.0):
    """Memory grows with the batch and shrinks with checkpointing; throughput
    grows with the batch and drops with checkpointing."""
    mem = cfg["batch_size"] * (4.0 - 3.0 * cfg["ckpt_ratio"])
    if mem > limit:
        return 0.0
    return cfg["batch_size"] / (1.0 + 0.3 * cfg["ckpt_ratio"])


def test_tune_finds_the_best_feasible_point():
    best, thr, trace = T.tune({}, lambda a: (8, 64, 8), _memory_model,
                              ckpt_ratios=[1.0, 0.92, 0.84, 0.67, 0.5, 0.34, 0.25, 0.0], patience=100)
    feasible = [(bs, r) for bs in range(8, 65, 8)
                for r in [1.0, 0.92, 0.84, 0.67, 0.5, 0.34, 0.25, 0.0]
                if _memory_model({"batch_size": bs, "ckpt_ratio": r}) > 0]
    want = max(feasible, key=lambda p: _memory_model({"batch_size": p[0], "ckpt_ratio": p[1]}))
    assert (best["batch_size"], best["ckpt_ratio"]) == want
    assert thr == pytest.approx(_memory_model({"batch_size": want[0], "ckpt_ratio": want[1]}))
    assert len(trace) < len(feasible)          # a search, not a sweep
    assert trace[0][0] == {"batch_size": 64, "ckpt_ratio": 1.0}


def test_tune_early_stop_and_oom_at_max_batch():
    calls = []

    def flat(cfg):
        calls.append(dict(cfg))
        return 10.0            # never improves after the first point

    T.tune({}, lambda a: (1, 64, 1), flat, patience=5)
    assert len(calls) == 6     # first point + 5 non-improving evaluations

    best, thr, _ = T.tune({}, lambda a: (8, 64, 8), lambda c: _memory_model(c, limit=30.0),
                          patience=100)
    assert best["batch_size"] <= 24 and thr > 0


def test_database_roundtrip(tmp_path):
    path = tmp_path / "db.json"
    db = T.Database(str(path))
    db.load()
    db.commit("(batch_size: 8)", {"thrpt": 1.5, "error_code": 0})
    again = T.Database(str(path))
    again.load()
    assert again.db["(batch_size: 8)"]["thrpt"] == 1.5
    mem = T.Database(None)
    mem.load()
    mem.commit("k", {"x": 1})   # in-memory only
    assert mem.db["k"] == {"x": 1}


def test_log_parsers(tmp_path):
    native = tmp_path / "n.log"
    native.write_text("\n".join(json.dumps({"samples_per_sec": v, "max_mem_mb": 1000 + v,
                                            "param_per_gpu_m": 335.0}) for v in (5, 10, 12)))
    params, thr, mem, code = get_dialect_cls("log_parser", "native").parse_log(str(native))
    assert (params, thr, mem, code) == (335.0, 11.0, 1012.0, 0)
    oom = tmp_path / "oom.log"
    oom.write_text("torch.OutOfMemoryError: CUDA out of memory.")
    assert get_dialect_cls("log_parser", "native").parse_log(str(oom))[3] == 1
    bad = tmp_path / "bad.log"
    bad.write_text("Traceback (most recent call last):")
    assert get_dialect_cls("log_parser", "native").parse_log(str(bad))[3] == 2
    ds = tmp_path / "ds.log"
    ds.write_text("step=10 SamplesPerSec=100.0 MaxMemAllocated=2.0GB\n"
                  "step=20 SamplesPerSec=120.0 MaxMemAllocated=2.5GB\n")
    _, thr, mem, code = get_dialect_cls("log_parser", "deepspeed").parse_log(str(ds))
    assert thr == 110.0 and mem == 2.5 * 1024 and code == 0
    mg = tmp_path / "mg.log"
    mg.write_text("global batch size: 32\n elapsed time per iteration (ms): 900.0 |\n"
                  " elapsed time per iteration (ms): 1000.0 | max allocated: 1234.0\n")
    _, thr, mem, code = get_dialect_cls("log_parser", "megatron").parse_log(str(mg))
    assert thr == pytest.approx(32.0) and mem == 1234.0 and code == 0


def test_dialect_registry():
    assert "native" in get_all_dialects("log_parser")
    assert "native" in get_all_dialects("runtime_engine")

    @register_framework_dialect("unit_test_target", "log_parser")
    class P:
        @staticmethod
        def parse_log(path):
            return 0.0, 1.0, 0.0, 0

    assert get_dialect_cls("log_parser", "unit_test_target") is P
    with pytest.raises(Exception):
        get_dialect_cls("log_parser", "missing_target")
    # allow_none falls back to the dialect registered for target None, if there is one
    fallback = get_all_dialects("runtime_engine").get(None)
    if fallback is not None:
        assert get_dialect_cls("runtime_engine", "missing_target", allow_none=True) is fallback
    with pytest.raises(Exception):
        register_framework_dialect("x", "not_a_dialect_kind")(P)


def test_cli_end_to_end(tmp_path, monkeypatch):
    cfg = tmp_path / "cfg.py"
    cfg.write_text(textwrap.dedent("""
        def get_bs_range(args):
            return (4, 16, 4)
    """))
    script = tmp_path / "train.py"
    script.write_text(textwrap.dedent("""
        import json, sys
        args = dict(zip(sys.argv[1::2], sys.argv[2::2]))
        bs, ratio = int(args["--batch"]), float(args["--ckpt"])
        if bs * (4 - 3 * ratio) > 30:
            print("torch.OutOfMemoryError: CUDA out of memory."); sys.exit(1)
        for _ in range(3):
            print(json.dumps({"samples_per_sec": bs / (1 + 0.3 * ratio), "max_mem_mb": 1.0}))
    """))
    db = tmp_path / "db.json"
    monkeypatch.chdir(tmp_path)
    T.main(["--config", str(cfg), "--db", str(db), str(script),
            "--batch", "batch_size", "--ckpt", "ckpt_ratio"])
    records = json.loads(db.read_text())
    assert records, "the CLI evaluated nothing"
    ok = [v for v in records.values() if v["error_code"] == 0]
    oom = [v for v in records.values() if v["error_code"] == 1]
    assert ok and oom
    assert max(v["thrpt"] for v in ok) > 0
