"""The written-out training example runs end to end on CPU: one process (train, save, resume)
and two gloo ranks with tensor parallelism."""
import os
import re
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SCRIPT = os.path.join(ROOT, "examples", "train_text.py")
SMALL = ["--text", os.path.join(ROOT, "README.md"), "--layers", "2", "--hidden", "64", "--heads", "2",
         "--seq-len", "64", "--batch-size", "4", "--eval-every", "2"]


def _steps(out):
    return [(int(m.group(1)), float(m.group(2)), float(m.group(3)))
            for m in re.finditer(r"step (\d+): loss ([\d.]+)  validation ([\d.naN]+)", out)]


def _run(cmd):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="1")
    res = subprocess.run(cmd, capture_output=True, text=True, cwd=ROOT, env=env, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    return res.stdout + res.stderr


def test_train_save_resume(tmp_path):
    out = _run([sys.executable, SCRIPT, *SMALL, "--family", "bert", "--steps", "4",
                "--save", str(tmp_path / "ck")])
    steps = _steps(out)
    assert [s for s, _, _ in steps] == [2, 4] and all(v == v for _, _, v in steps)
    out = _run([sys.executable, SCRIPT, *SMALL, "--family", "bert", "--steps", "2",
                "--resume", str(tmp_path / "ck")])
    assert [s for s, _, _ in _steps(out)] == [6]


def test_two_ranks_tensor_parallel():
    out = _run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                "--master-addr", "127.0.0.1", "--master-port", "29581", SCRIPT, *SMALL, "--tp", "2",
                "--steps", "4"])
    steps = _steps(out)
    assert [s for s, _, _ in steps] == [2, 4]
    assert all(loss == loss and val == val for _, loss, val in steps)


def test_data_util_chunks(tmp_path):
    sys.path.insert(0, os.path.join(ROOT, "examples"))
    import data_util

    text = tmp_path / "t.txt"
    text.write_bytes(b"first paragraph of text\n\nsecond one, a little longer than the first\n\n" * 8)
    docs = data_util.read_documents(str(text))
    assert len(docs) == 16 and docs[0] == list(b"first paragraph of text")
    train, val, sampler = data_util.get_dataloaders(str(text), 16, 2, kind="mlm", seed=3)
    ids, labels = next(iter(train))
    assert ids.shape == (2, 16) and labels.shape == (2, 16)
    kept = labels != -100
    assert bool((labels[kept] == ids[kept]).all()) and int(ids.max()) <= data_util.EOS
    assert len(val) >= 1
    sampler.set_epoch(1)
