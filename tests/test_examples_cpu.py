"""The written-out training example runs end to end on CPU: one process (train, save, resume)
and two gloo ranks with tensor parallelism."""
import os
import re
import subprocess
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from dist_utils import run_distributed  # noqa: E402

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


def test_example_helpers():
    sys.path.insert(0, os.path.join(ROOT, "examples"))
    import copy

    import torch

    import utils as ex_utils

    import slapo_b200 as slapo
    from slapo_b200.models import BertConfig, BertForMaskedLM, mlm_loss

    cfg = ex_utils.get_ds_config(16, 4, fp16=False, zero_stage=1)
    assert cfg["train_micro_batch_size_per_gpu"] == 4 and cfg["zero_optimization"]["stage"] == 1
    assert ex_utils.generate_pipeline_cuts(24, 4) == [5, 11, 17]
    bcfg = BertConfig(vocab_size=128, hidden_size=32, num_hidden_layers=2, num_attention_heads=2,
                      intermediate_size=64, hidden_dropout_prob=0.0,
                      attention_probs_dropout_prob=0.0)
    torch.manual_seed(0)
    model = BertForMaskedLM(bcfg).init_weights()
    ids = torch.randint(0, 128, (4, 16))
    batches = [((ids,), ids.clone()) for _ in range(6)]
    opt = torch.optim.AdamW(model.parameters(), lr=1e-2)
    losses = ex_utils.train_with_torch(copy.deepcopy(model), batches, opt, steps=3)
    assert len(losses) == 3
    sch = slapo.model_schedule.apply_schedule(model, "bert", model_config=bcfg, group=False,
                                              attn_op_name="reference")
    engine, _ = slapo.build(sch, target="deepspeed", config=ex_utils.get_ds_config(4, 4, fp16=False),
                            init_weights=False, loss_fn=lambda o, l: mlm_loss(o["logits"], l))
    losses = ex_utils.train_with_deepspeed_engine(engine, batches, steps=6)
    assert len(losses) == 6 and losses[-1] < losses[0]


def _hf_example_worker(rank, world, argv, out):
    import deepspeed_hf as example

    losses = example.train(example.parse_args(argv))
    if rank == 0:
        torch.save(losses, out)


@pytest.mark.parametrize("family,pmp,tmp,world", [("opt", 2, 2, 4), ("gpt2", 1, 2, 4),
                                                  ("t5", 2, 1, 2)])
def test_hugging_face_example_script(family, pmp, tmp, world, tmp_path):
    """``examples/deepspeed_hf.py``: a ``transformers`` model built on the meta device, the
    family's recipe (pipeline cuts, sequence parallelism, recomputation), the ``"deepspeed"``
    target with a DeepSpeed-layout configuration - on gloo ranks, OPT as 2 stages x TP 2 and
    GPT-2 as TP 2 x DP 2."""
    pytest.importorskip("transformers")
    sys.path.insert(0, os.path.join(ROOT, "examples"))
    out = str(tmp_path / "losses.pt")
    argv = ["--family", family, "--hidden", "64", "--layers", "4", "--heads", "4", "--vocab", "512",
            "--seq-len", "32", "--dec-seq-len", "16", "--batch-size", "4",
            "--micro-batch-size", "2", "--pmp", str(pmp),
            "--tmp", str(tmp), "--sequence-parallel", "--checkpoint", "0.5", "--iter-nums", "3",
            "--device", "cpu", "--dtype", "fp32"]
    run_distributed(_hf_example_worker, world, argv, out)
    losses = torch.load(out)
    # random tokens: ln(512) = 6.24; T5 starts lower (tied head, labels = decoder inputs)
    assert len(losses) == 3 and all(0.0 < v < 7.0 for v in losses)
    if family != "t5":
        assert all(v > 5.5 for v in losses)


def test_reference_named_data_helpers():
    """``get_dataloader`` / ``LossTestDataset`` / ``train_with_deepspeed_engine`` exist under the
    names the reference's example scripts import, on local data."""
    sys.path.insert(0, os.path.join(ROOT, "examples"))
    import data_util
    import utils

    train, val = data_util.get_dataloader("bert-large-uncased", os.path.join(ROOT, "README.md"), 2,
                                          max_seq_length=64)
    ids, labels = next(iter(train))
    assert ids.shape == labels.shape == (2, 64) and (labels != -100).any()
    ids, labels = next(iter(data_util.get_dataloader("gpt2", os.path.join(ROOT, "README.md"), 2,
                                                     max_seq_length=64)[1]))
    assert torch.equal(ids, labels)
    doubled = data_util.LossTestDataset([1, 2, 3], lambda e: 2 * e)
    assert len(doubled) == 3 and doubled[1] == 4
    assert utils.train_with_deepspeed_engine is utils.train_with_engine
