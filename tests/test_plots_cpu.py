"""The plotting scripts under benchmark/plot run on records of every supported form and write
well-formed SVG (no matplotlib needed)."""
import json
import os
import subprocess
import sys
import xml.dom.minidom

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PLOT = os.path.join(ROOT, "benchmark", "plot")


def _run(script, *args):
    res = subprocess.run([sys.executable, os.path.join(PLOT, script), *args], capture_output=True,
                         text=True, cwd=ROOT)
    assert res.returncode == 0, res.stderr
    return res.stdout


def _bench_line(model, impl, gpus, value, label=None):
    rec = {"metric": "train samples/sec", "value": value, "n_gpus": gpus, "impl": impl,
           "config": {"model": model, "parallelism": f"tp{gpus}"}}
    if label:
        rec["label"] = label
    return json.dumps(rec)


def _check_svg(path):
    doc = xml.dom.minidom.parse(str(path))
    assert doc.documentElement.tagName == "svg"
    return doc


def test_single_device_and_single_node(tmp_path):
    src = tmp_path / "results.jsonl"
    lines = ["some log text"]
    for n, nat, ref in ((1, 520.0, 430.0), (2, 773.0, 494.0), (4, 1129.0, 590.0), (8, 1557.0, 770.0)):
        lines += [_bench_line("bert-large", "native", n, nat), _bench_line("bert-large", "reference", n, ref)]
    lines.append(json.dumps({"model": "opt-2.7b", "samples_per_sec": 42.7, "tp": 1, "pp": 1, "dp": 1}))
    src.write_text("\n".join(lines) + "\n")
    out = _run("single_device.py", str(src), str(tmp_path / "sd.svg"))
    assert "bert-large: native 520.0, reference 430.0" in out and "opt-2.7b" in out
    assert len(_check_svg(tmp_path / "sd.svg").getElementsByTagName("rect")) >= 4
    out = _run("single_node.py", str(src), str(tmp_path / "sn.svg"))
    assert "8 GPUs 1557.0 samples/s (eff 0.37)" in out
    assert len(_check_svg(tmp_path / "sn.svg").getElementsByTagName("polyline")) == 3


def test_sweep_tsv_is_read(tmp_path):
    src = tmp_path / "sweep.tsv"
    src.write_text("model\tgpus\tlayout\tsamples_per_sec\n"
                   "gpt-neo-2.7b\t4\ttp2dp2\t107.4\ngpt-neo-2.7b\t8\ttp4dp2\t140.7\n"
                   "t5-large\t8\ttp4dp2\toom\n")
    out = _run("single_node.py", str(src), str(tmp_path / "x.svg"))
    assert "gpt-neo-2.7b (native): 4 GPUs 107.4" in out and "t5-large" not in out


def test_ablation(tmp_path):
    src = tmp_path / "ab.jsonl"
    src.write_text("\n".join([
        _bench_line("bert-large", "native", 8, 1242.0, "peer-load reductions"),
        _bench_line("bert-large", "native", 8, 1375.0, "+ NVLS reductions"),
        _bench_line("bert-large", "native", 8, 1557.0, "+ pushed all-gather")]) + "\n")
    out = _run("ablation.py", str(src), str(tmp_path / "ab.svg"))
    assert "+ pushed all-gather: 1557.0 samples/s (1.25 x)" in out
    _check_svg(tmp_path / "ab.svg")


def test_autotune_and_search_space(tmp_path):
    db = {"(batch_size: 256, ckpt_ratio: 1.0)": {"error_code": 1, "thrpt": 0.0},
          "(batch_size: 128, ckpt_ratio: 1.0)": {"error_code": 0, "thrpt": 410.5},
          "(batch_size: 128, ckpt_ratio: 0.5)": {"error_code": 0, "thrpt": 455.0}}
    src = tmp_path / "db.json"
    src.write_text(json.dumps(db))
    out = _run("autotune.py", str(src), str(tmp_path / "at.svg"))
    assert "failed" in out and "455.0 samples/s" in out
    assert len(_check_svg(tmp_path / "at.svg").getElementsByTagName("circle")) == 2
    out = _run("search_space.py", os.path.join(ROOT, "examples", "bert", "tune_cfg.py"),
               str(tmp_path / "poly.svg"), "gpus=8", "tp=8")
    assert "points" in out
    assert len(_check_svg(tmp_path / "poly.svg").getElementsByTagName("polygon")) == 1
