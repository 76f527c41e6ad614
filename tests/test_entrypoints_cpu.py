"""Entry points on CPU: the general training script on 4 gloo ranks (TP 2 x PP 2,
save then resume), the benchmark config parser and FLOP model, the examples."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "benchmark"))

TINY = ["--layers", "4", "--hidden", "64", "--heads", "4", "--vocab", "512", "--batch-size", "2",
        "--seq-len", "32", "--steps", "2", "--warmup", "1", "--dtype", "fp32", "--attn-op",
        "reference"]


def _run(cmd, **kw):
    env = dict(os.environ, PYTHONPATH=ROOT, OMP_NUM_THREADS="2")
    proc = subprocess.run(cmd, cwd=ROOT, env=env, text=True, capture_output=True, timeout=600, **kw)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-4000:]
    recs = [json.loads(l) for l in proc.stdout.splitlines() if l.startswith("{")]
    return recs


def test_train_entry_tp2_pp2_save_and_resume(tmp_path):
    import bench_single_node as B
    ck = str(tmp_path / "ck")
    args = ["--tp", "2", "--pp", "2", "--micro-batches", "4"] + TINY
    rec, text = B.launch("opt-350m", 4, args + ["--save", ck], port=29561, timeout=600)
    assert rec is not None, text[-3000:]
    assert rec["tp"] == 2 and rec["pp"] == 2 and rec["dp"] == 1 and rec["samples_per_sec"] > 0
    assert os.path.exists(os.path.join(ck, "manifest.json"))
    assert os.path.exists(os.path.join(ck, "model_pp1_tp1.pt"))
    rec2, text = B.launch("opt-350m", 4, args + ["--resume", ck], port=29562, timeout=600)
    assert rec2 is not None, text[-3000:]
    assert rec2["start_step"] == 3


def test_train_entry_tp2_pp2_paired_transfers_match_overlapped_ones():
    """The paired p2p schedule (the default next to the fused tensor-parallel kernels on GPUs)
    and the side-stream schedule compute the same step."""
    import bench_single_node as B
    args = ["--tp", "2", "--pp", "2", "--micro-batches", "4", "--sequence-parallel"] + TINY
    a, text = B.launch("opt-350m", 4, args + ["--p2p-mode", "paired"], port=29566, timeout=600)
    assert a is not None, text[-3000:]
    b, text = B.launch("opt-350m", 4, args + ["--p2p-mode", "overlap"], port=29567, timeout=600)
    assert b is not None, text[-3000:]
    assert abs(a["loss"] - b["loss"]) < 1e-5, (a["loss"], b["loss"])


def test_train_entry_dp2_sequence_parallel_tp():
    import bench_single_node as B
    rec, text = B.launch("bert-base", 4, ["--tp", "2", "--sequence-parallel"] + TINY, port=29563)
    assert rec is not None, text[-3000:]
    assert rec["dp"] == 2 and rec["sequence_parallel"] is True


def test_train_entry_without_tensor_parallelism_never_shards_over_other_axes():
    """tp == 1 with several ranks (pure pipeline, pure data parallel): the schedule must not
    treat the whole job as a tensor-parallel group."""
    import bench_single_node as B
    rec, text = B.launch("gpt-neo-125m", 2, ["--pp", "2", "--micro-batches", "2"] + TINY,
                         port=29564)
    assert rec is not None, text[-3000:]
    assert (rec["tp"], rec["pp"], rec["dp"]) == (1, 2, 1)
    assert rec["param_per_gpu_m"] > 0
    rec2, text = B.launch("gpt-neo-125m", 2, TINY, port=29565)       # dp = 2
    assert rec2 is not None, text[-3000:]
    assert (rec2["tp"], rec2["pp"], rec2["dp"]) == (1, 1, 2)
    # unsharded: each rank holds the full model (a pipeline stage holds about half of it)
    assert rec2["param_per_gpu_m"] > rec["param_per_gpu_m"]


def test_benchmark_config_and_flops():
    import bench_single_node as B
    runs = B.parse_config(os.path.join(ROOT, "benchmark", "configs", "single_node_b200.cfg"))
    bert8 = [r for r in runs if r["model"] == "bert-large" and r["gpus"] == 8][0]
    assert bert8["batch"] == 256 and bert8["tp"] == 8 and bert8["sp"]
    opt = [r for r in runs if r["model"] == "opt-2.7b"][0]
    assert (opt["tp"], opt["pp"], opt["micro"]) == (4, 2, 16)
    args = B.train_args_for(opt, 5, 3)
    assert args[args.index("--batch-size") + 1] == "4"      # 64 / dp 1 / 16 micro-batches
    # BERT-large at seq 512: about 6 * 335e6 * 512 = 1.03 TFLOP plus attention
    tf = B.model_tflop_per_sample("bert-large", 512)
    assert 1.0 < tf < 1.4
    assert B.model_tflop_per_sample("t5-large", 1024, 512) > 2.0


def test_example_launcher_and_walkthrough():
    recs = _run([sys.executable, "examples/gpt2/train.py"] + TINY)
    assert recs and recs[-1]["model"] == "gpt2-medium" and recs[-1]["seq_len"] == 32
    out = subprocess.run([sys.executable, "examples/schedule_walkthrough.py"], cwd=ROOT,
                         text=True, capture_output=True, timeout=300)
    assert out.returncode == 0 and "matches the original" in out.stdout, out.stderr[-2000:]


@pytest.mark.parametrize("family", ["bert", "roberta", "albert", "gpt2", "gpt_neo", "opt", "t5",
                                    "wideresnet"])
def test_tune_configs_load(family):
    from slapo_b200.autotune.tune import load_config
    cfg = load_config(os.path.join(ROOT, "examples", family, "tune_cfg.py"))
    lo, hi, step = cfg.get_bs_range({"gpus": 8, "tp": 8})
    assert 1 <= lo <= hi and step >= 1


def test_train_entry_albert_on_two_stages():
    """The shared layer of ALBERT on both stages of a pipeline, through the training script."""
    import bench_single_node as B
    rec, text = B.launch("albert-large", 2, ["--pp", "2", "--micro-batches", "2"] + TINY,
                         port=29581, timeout=600)
    assert rec is not None, text[-3000:]
    assert rec["pp"] == 2 and rec["samples_per_sec"] > 0 and 0 < rec["loss"] < 12
