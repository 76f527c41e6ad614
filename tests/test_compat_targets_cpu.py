"""Code written against the reference passes ``target="deepspeed"`` with a DeepSpeed
configuration and topology; here that resolves to the native engines."""
import copy

import pytest
import torch

import slapo_b200 as slapo
from slapo_b200.framework_dialect import compat, get_all_dialects
from slapo_b200.models import BertConfig, BertForMaskedLM, mlm_loss


def _ds_config(batch, micro, zero_stage=0):
    cfg = {"steps_per_print": 10, "optimizer": {"type": "AdamW", "params": {"lr": 0.01}},
           "fp16": {"enabled": False, "initial_scale_power": 12}, "bf16": {"enabled": False},
           "gradient_clipping": 0.5, "train_batch_size": batch,
           "train_micro_batch_size_per_gpu": micro, "pipeline": {"sequence_parallel": False},
           "wall_clock_breakdown": False}
    if zero_stage:
        cfg["zero_optimization"] = {"stage": zero_stage, "overlap_comm": True,
                                    "reduce_scatter": True}
    return cfg


def test_config_translation():
    out = compat.translate_ds_config(_ds_config(32, 4, zero_stage=3), dp_size=2)
    assert out["lr"] == 0.01 and out["clip_grad"] == 0.5 and out["grad_accum_steps"] == 4
    assert out["zero"] is True and out["overlap_comm"] is True
    assert out["steps_per_print"] == 10                      # unknown keys are carried along
    assert compat.translate_ds_config(_ds_config(8, 8))["zero"] is False
    assert compat.translate_ds_config(None) is None


def test_topology_translation():
    class Topo:                       # the shape of deepspeed's PipeModelDataParallelTopology
        def get_dim(self, axis):
            return {"pipe": 1, "data": 1, "model": 1}[axis]

    assert compat.mesh_from_topology(None) is None
    assert compat.mesh_from_topology(Topo()) is None          # one process: no mesh needed
    assert compat.mesh_from_topology({"pp": 1, "dp": 1, "tp": 1}) is None
    with pytest.raises(TypeError):
        compat.mesh_from_topology(object())
    for kind in ("runtime_engine", "pipeline_stage", "pipeline_engine"):
        table = get_all_dialects(kind)
        assert "deepspeed" in table and "megatron" in table


def test_build_with_the_deepspeed_target_trains():
    cfg = BertConfig(vocab_size=128, hidden_size=32, num_hidden_layers=2, num_attention_heads=2,
                     intermediate_size=64, hidden_dropout_prob=0.0,
                     attention_probs_dropout_prob=0.0)
    torch.manual_seed(0)
    model = BertForMaskedLM(cfg).init_weights()
    sch = slapo.model_schedule.apply_schedule(copy.deepcopy(model), "bert", model_config=cfg,
                                              attn_op_name="reference", group=False)
    engine, opt = slapo.build(sch, target="deepspeed", config=_ds_config(4, 4), topology=None,
                              loss_fn=lambda out, lab: mlm_loss(out["logits"], lab),
                              init_weights=False)
    assert engine is opt and engine.cfg.lr == 0.01 and engine.cfg.clip_grad == 0.5
    ids = torch.randint(0, 128, (4, 16))
    losses = [float(engine.train_batch(ids, labels=ids.clone())) for _ in range(5)]
    assert losses[-1] < losses[0]


def _ds_dp_worker(rank, world):
    class Topo:
        def get_dim(self, axis):
            return {"pipe": 1, "data": world, "model": 1}[axis]

    cfg = BertConfig(vocab_size=128, hidden_size=32, num_hidden_layers=2, num_attention_heads=2,
                     intermediate_size=64, hidden_dropout_prob=0.0,
                     attention_probs_dropout_prob=0.0)
    torch.manual_seed(0)
    model = BertForMaskedLM(cfg).init_weights()
    sch = slapo.model_schedule.apply_schedule(copy.deepcopy(model), "bert", model_config=cfg,
                                              attn_op_name="reference", group=False)
    engine, _ = slapo.build(sch, target="deepspeed", config=_ds_config(8, 4, zero_stage=1),
                            topology=Topo(), init_weights=False,
                            loss_fn=lambda out, lab: mlm_loss(out["logits"], lab))
    assert engine.mesh.dp_size == world and engine.cfg.zero and engine.cfg.grad_accum_steps == 1
    g = torch.Generator().manual_seed(rank)
    ids = torch.randint(0, 128, (4, 16), generator=g)
    losses = [float(engine.train_batch(ids, labels=ids.clone())) for _ in range(4)]
    assert losses[-1] < losses[0]
    # the replicas hold identical parameters after the sharded optimizer steps
    import torch.distributed as dist

    flat = torch.cat([p.detach().flatten() for p in engine.model.parameters()])
    other = flat.clone()
    dist.broadcast(other, src=0)
    torch.testing.assert_close(flat, other)


def test_deepspeed_target_with_a_data_parallel_topology():
    from dist_utils import run_distributed

    run_distributed(_ds_dp_worker, 2)
