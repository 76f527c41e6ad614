"""Engine (DP / ZeRO over gloo) and sharded checkpoints: resume gives the same
losses, a ZeRO dp2 checkpoint resumes on one rank, TP shards consolidate and
re-split (weights and optimizer moments)."""
import copy
import os
import tempfile

import pytest
import torch
from torch import nn

import slapo_b200 as slapo
from slapo_b200 import ckpt
from slapo_b200.parallel.mesh import DeviceMesh
from slapo_b200.runtime.engine import TrainEngine

from dist_utils import run_distributed


class MLP(nn.Module):
    def __init__(self):
        super().__init__()
        self.fc1 = nn.Linear(16, 64)
        self.drop = nn.Dropout(0.1)
        self.fc2 = nn.Linear(64, 16)
        self.norm = nn.LayerNorm(16)

    def forward(self, x, y):
        out = self.norm(self.fc2(self.drop(torch.relu(self.fc1(x)))))
        return {"loss": (out - y).pow(2).mean()}


def _data(step, rank=0):
    g = torch.Generator().manual_seed(1000 + 10 * step + rank)
    return torch.randn(8, 16, generator=g), torch.randn(8, 16, generator=g)


def _cfg(zero=True):
    return {"lr": 1e-2, "zero": zero, "bucket_mb": 0.001, "clip_grad": 1.0}


def _tp_model(rank):
    torch.manual_seed(0)
    sch = slapo.create_schedule(MLP())
    if sch.world_size > 1:
        sch["fc1"].shard("weight", axis=0)
        sch["fc1"].shard("bias", axis=0)
        sch["fc1"].sync("bwd_post", "all_reduce")
        sch["fc2"].shard("weight", axis=1)
        sch["fc2"].sync("fwd_post", "all_reduce")
    model, _ = slapo.build(sch, init_weights=False)
    return model


def _dp_worker(rank, world, tmp, zero):
    """DP=2: both ranks end with identical weights equal to a single-rank run
    on the concatenated batch; save / resume reproduces the loss sequence."""
    mesh = DeviceMesh(pp=1, dp=world, tp=1)
    slapo.set_random_seed(5, dp_rank=mesh.dp_rank)
    torch.manual_seed(0)
    model = MLP()
    model.drop.p = 0.0
    engine = TrainEngine(model, _cfg(zero), mesh=mesh)
    ref = copy.deepcopy(model)
    ref_opt = torch.optim.AdamW(   # like the engine: no weight decay on 1-D tensors
        [{"params": [p for p in ref.parameters() if p.dim() > 1], "weight_decay": 0.01},
         {"params": [p for p in ref.parameters() if p.dim() <= 1], "weight_decay": 0.0}], lr=1e-2)
    for step in range(3):
        x, y = _data(step, rank)
        engine.train_batch(x, y)
        xs = torch.cat([_data(step, r)[0] for r in range(world)])
        ys = torch.cat([_data(step, r)[1] for r in range(world)])
        ref_opt.zero_grad()
        ref(xs, ys)["loss"].backward()
        torch.nn.utils.clip_grad_norm_(ref.parameters(), 1.0)
        ref_opt.step()
    for (n, p), q in zip(model.named_parameters(), ref.parameters()):
        torch.testing.assert_close(p, q, rtol=2e-4, atol=2e-5, msg=n)
    ckpt.save_checkpoint(tmp, model, engine, mesh=mesh, extra={"note": "hi"})
    after = [float(engine.train_batch(*_data(s, rank))) for s in range(3, 6)]

    torch.manual_seed(123)
    model2 = MLP()
    model2.drop.p = 0.0
    engine2 = TrainEngine(model2, _cfg(zero), mesh=mesh)
    info = ckpt.load_checkpoint(tmp, model2, engine2, mesh=mesh)
    assert info["step"] == 3 and info["extra"] == {"note": "hi"} and engine2.step_count == 3
    again = [float(engine2.train_batch(*_data(s, rank))) for s in range(3, 6)]
    assert after == pytest.approx(again, rel=1e-6)


@pytest.mark.parametrize("zero", [True, False])
def test_dp_engine_matches_single_rank_and_resumes(zero):
    with tempfile.TemporaryDirectory() as tmp:
        run_distributed(_dp_worker, 2, tmp, zero)
        # the ZeRO dp2 checkpoint resumes on a single rank (other DP size, no ZeRO)
        torch.manual_seed(7)
        model = MLP()
        engine = TrainEngine(model, _cfg(False))
        info = ckpt.load_checkpoint(tmp, model, engine, load_rng=False)
        assert info["step"] == 3
        man = ckpt.read_manifest(tmp)
        assert man["mesh"] == {"pp": 1, "dp": 2, "tp": 1}
        full, opt = ckpt.consolidate_checkpoint(tmp, with_optimizer=True)
        torch.testing.assert_close(model.fc1.weight, full["fc1.weight"])
        assert opt["state"]["fc1.weight"]["exp_avg"].abs().sum() > 0
        assert float(engine.exp_avg.abs().sum()) > 0


def _tp_worker(rank, world, tmp):
    mesh = DeviceMesh(pp=1, dp=1, tp=world)
    slapo.set_random_seed(5, tp_rank=rank)
    model = _tp_model(rank)
    engine = TrainEngine(model, _cfg(), mesh=mesh)
    for step in range(2):
        engine.train_batch(*_data(step))
    ckpt.save_checkpoint(tmp, model, engine, mesh=mesh)
    # dropout is active: resuming must also restore the RNG streams
    after = [float(engine.train_batch(*_data(s))) for s in range(2, 4)]
    model2 = _tp_model(rank)
    engine2 = TrainEngine(model2, _cfg(), mesh=mesh)
    ckpt.load_checkpoint(tmp, model2, engine2, mesh=mesh)
    again = [float(engine2.train_batch(*_data(s))) for s in range(2, 4)]
    assert after == pytest.approx(again, rel=1e-6)


def test_tp_checkpoint_resume_consolidate_and_reshard():
    with tempfile.TemporaryDirectory() as tmp, tempfile.TemporaryDirectory() as tmp1:
        run_distributed(_tp_worker, 2, tmp)
        man = ckpt.read_manifest(tmp)
        assert man["params"]["fc1.weight"]["axis"] == 0
        assert man["params"]["fc2.weight"]["axis"] == 1
        assert man["params"]["norm.weight"]["axis"] is None
        full, opt = ckpt.consolidate_checkpoint(tmp, with_optimizer=True)
        assert full["fc1.weight"].shape == (64, 16) and full["fc2.weight"].shape == (16, 64)
        assert opt["state"]["fc2.weight"]["exp_avg_sq"].shape == (16, 64)
        # TP2 -> TP1: a plain single-rank model loads it (weights + optimizer) and trains on
        ckpt.reshard_checkpoint(tmp, tmp1, tp_size=1)
        model = MLP()
        engine = TrainEngine(model, _cfg(False))
        info = ckpt.load_checkpoint(tmp1, model, engine)
        assert info["step"] == 2
        torch.testing.assert_close(model.fc2.weight, full["fc2.weight"])
        assert torch.isfinite(engine.train_batch(*_data(9)))
        # loading the TP2 checkpoint directly into the TP1 model consolidates on the fly
        model_b = MLP()
        ckpt.load_checkpoint(tmp, model_b, load_rng=False)
        torch.testing.assert_close(model_b.fc1.weight, full["fc1.weight"])
        # TP1 -> TP4 keeps every axis and splits the moments the same way
        with tempfile.TemporaryDirectory() as tmp4:
            ckpt.reshard_checkpoint(tmp1, tmp4, tp_size=4)
            shard = torch.load(os.path.join(tmp4, "model_pp0_tp3.pt"))
            torch.testing.assert_close(shard["fc1.weight"], full["fc1.weight"].chunk(4, 0)[3])
            o = torch.load(os.path.join(tmp4, "optim_pp0_tp3.pt"))
            torch.testing.assert_close(o["state"]["fc2.weight"]["exp_avg"],
                                       opt["state"]["fc2.weight"]["exp_avg"].chunk(4, 1)[3])
            assert ckpt.read_manifest(tmp4)["mesh"]["tp"] == 4


def test_strict_mismatch_raises():
    with tempfile.TemporaryDirectory() as tmp:
        ckpt.save_checkpoint(tmp, MLP())
        with pytest.raises(KeyError):
            ckpt.load_checkpoint(tmp, nn.Linear(3, 3))
        ckpt.load_checkpoint(tmp, nn.Linear(3, 3), strict=False)


def _tp_no_mesh_worker(rank, world, tmp):
    # sharded over the WORLD group, saved and loaded without a mesh: every rank must write its
    # own shard file and the manifest must say tp = world
    model = _tp_model(rank)
    ckpt.save_checkpoint(tmp, model)
    model2 = _tp_model(rank)
    with torch.no_grad():
        for p in model2.parameters():
            p.zero_()
    ckpt.load_checkpoint(tmp, model2)
    for (n, a), (_, b) in zip(model.named_parameters(), model2.named_parameters()):
        torch.testing.assert_close(a, b, msg=lambda s: f"{n}: {s}")


def test_sharded_model_without_a_mesh_is_saved_as_one_tp_group():
    with tempfile.TemporaryDirectory() as tmp:
        run_distributed(_tp_no_mesh_worker, 2, tmp)
        man = ckpt.read_manifest(tmp)
        assert man["mesh"] == {"pp": 1, "dp": 1, "tp": 2}
        assert os.path.exists(os.path.join(tmp, "model_pp0_tp1.pt"))
        full = ckpt.consolidate_checkpoint(tmp)
        assert tuple(full["fc1.weight"].shape) == (64, 16)
        assert tuple(full["fc2.weight"].shape) == (16, 64)
        # shard files that do not add up to the recorded shape are refused
        shard = torch.load(os.path.join(tmp, "model_pp0_tp1.pt"), weights_only=False)
        shard["fc1.weight"] = shard["fc1.weight"][:8]
        torch.save(shard, os.path.join(tmp, "model_pp0_tp1.pt"))
        with pytest.raises(ValueError, match="do not belong to one tensor-parallel layout"):
            ckpt.consolidate_checkpoint(tmp)


# ---- checkpoints across pipeline layouts -------------------------------------------------- #
def _zoo_engine(name, pp, tp, seed):
    from test_train_equivalence_cpu import _tiny_spec

    torch.manual_seed(seed)
    spec = _tiny_spec(name)
    model = spec.build().init_weights()
    mesh = DeviceMesh(pp=pp, dp=1, tp=tp)
    slapo.set_random_seed(1, tp_rank=mesh.tp_rank, pp_rank=mesh.pp_rank)
    kwargs = dict(model_config=spec.config, group=mesh.schedule_group, attn_op_name="reference")
    if pp > 1:
        kwargs["pipeline_cuts"] = [[], []] if spec.kind == "seq2seq" else [1]
    sch = slapo.model_schedule.apply_schedule(model, spec.schedule_key, **kwargs)
    extra = dict(num_micro_batches=2) if pp > 1 else {}
    engine, _ = slapo.build(sch, target="native", mesh=mesh, init_weights=False,
                            loss_fn=spec.loss_fn(mesh.tp_group, tp > 1),
                            config={"lr": 1e-2, "clip_grad": 1.0, "weight_decay": 0.01}, **extra)
    return spec, engine


def _layout_worker(rank, world, name, tmp, pp, tp, phase):
    """``save``: train two steps, save, train two more and record their losses.  ``load``: a
    differently initialised model in another layout loads the checkpoint (weights and
    optimizer state) and must reproduce those losses."""
    spec, engine = _zoo_engine(name, pp, tp, seed=21 if phase == "save" else 99)
    inputs, labels = spec.make_batch(4, seq=32, seq_dec=16, seed=3)
    if phase == "save":
        for _ in range(2):
            engine.train_batch(*inputs, labels=labels)
        ckpt.save_checkpoint(tmp, None, engine)       # a pipeline engine stands for its stage
        after = [float(engine.train_batch(*inputs, labels=labels)) for _ in range(2)]
        if rank == 0:
            torch.save(after, os.path.join(tmp, "after.pt"))
        return
    info = ckpt.load_checkpoint(tmp, None, engine, load_rng=False)
    assert info["step"] == 2
    again = [float(engine.train_batch(*inputs, labels=labels)) for _ in range(2)]
    assert again == pytest.approx(torch.load(os.path.join(tmp, "after.pt")), rel=2e-5)


@pytest.mark.parametrize("name,saved,loaded", [
    ("gpt-neo-125m", (2, 2), [(2, 2), (1, 2), (1, 1)]),   # pipeline -> same, TP only, one rank
    ("t5-base", (1, 2), [(2, 2)]),      # into stages that know the tied table by other names
])
def test_checkpoint_moves_between_pipeline_layouts(name, saved, loaded):
    with tempfile.TemporaryDirectory() as tmp:
        run_distributed(_layout_worker, saved[0] * saved[1], name, tmp, *saved, "save")
        man = ckpt.read_manifest(tmp)
        assert man["mesh"]["pp"] == saved[0] and man["mesh"]["tp"] == saved[1]
        # tensors are stored under the unpartitioned model's names, whatever the layout
        assert not [n for n in man["params"] if "submod_" in n or n.startswith("module.")]
        if saved[0] == 1:        # an unpartitioned model knows its tied tables by all names
            assert any(e.get("aliases") for e in man["params"].values())
        for pp, tp in loaded:
            run_distributed(_layout_worker, pp * tp, name, tmp, pp, tp, "load")


def test_traced_modules_keep_buffers_out_of_the_state_dict():
    """A buffer registered with ``persistent=False`` stays non-persistent when its module is
    re-created as a graph module (fx registers copied buffers as persistent)."""
    from slapo_b200.models.albert import AlbertConfig, AlbertForMaskedLM

    cfg = AlbertConfig(vocab_size=128, embedding_size=16, hidden_size=32, num_hidden_layers=2,
                       intermediate_size=64, num_attention_heads=4, max_position_embeddings=32)
    model = AlbertForMaskedLM(cfg)
    assert "albert.embeddings.position_ids" not in model.state_dict()
    sch = slapo.create_schedule(model)
    sch.trace_until("albert.encoder")
    assert sch["albert.embeddings"].mod is not model.albert.embeddings       # re-created
    assert "albert.embeddings.position_ids" not in sch.mod.state_dict()
    assert "position_ids" in dict(sch["albert.embeddings"].mod.named_buffers())
