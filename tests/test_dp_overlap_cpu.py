"""Data-parallel gradient reduction launched from backward hooks, on gloo ranks.

The hook logic (calibrated firing counts, the last-backward gate, deferred buckets) is the
same on GPUs; ``overlap_on_cpu`` lets it run where the reduction is synchronous.  Covered:
a module called several times under re-entrant checkpointing (ALBERT's shared layer), and a
pipeline x data-parallel mesh with embeddings tied across stages and gradient clipping."""
import copy

import pytest
import torch
import torch.distributed as dist
from torch import nn
from torch.nn import functional as F

import slapo_b200 as slapo
from slapo_b200.models import (AlbertConfig, AlbertForMaskedLM, BertConfig, BertForMaskedLM,
                               mlm_loss)
from slapo_b200.parallel.mesh import DeviceMesh
from slapo_b200.runtime.engine import TrainEngine

from dist_utils import run_distributed


def _albert_worker(rank, world, zero):
    torch.manual_seed(6)
    cfg = AlbertConfig(vocab_size=128, embedding_size=16, hidden_size=32, num_hidden_layers=3,
                       num_attention_heads=2, intermediate_size=64, max_position_embeddings=32,
                       hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    ref = AlbertForMaskedLM(cfg).init_weights()
    engines = []
    for overlap in (False, True):
        sch = slapo.model_schedule.apply_schedule(copy.deepcopy(ref), "albert", model_config=cfg,
                                                  group=False, ckpt_ratio=1.0)
        model, _ = slapo.build(sch, init_weights=False)
        mesh = DeviceMesh(pp=1, dp=world, tp=1, create_groups=False)
        mesh.groups["dp"] = torch.distributed.group.WORLD
        engines.append(TrainEngine(
            model, mesh=mesh,
            config={"lr": 1e-2, "clip_grad": 0.5, "bucket_mb": 0.004, "zero": zero,
                    "overlap_comm": overlap, "overlap_on_cpu": True},
            loss_fn=lambda out, lab: mlm_loss(out["logits"], lab)))
    plain, hooked = engines
    assert hooked._overlap and not plain._overlap and len(hooked.buckets) > 2
    for step in range(3):
        torch.manual_seed(100 + step * world + rank)
        ids = torch.randint(0, 128, (2, 16))
        l0 = plain.train_batch(ids, labels=ids)
        l1 = hooked.train_batch(ids, labels=ids)
        torch.testing.assert_close(l0, l1)
        torch.testing.assert_close(plain.last_grad_norm, hooked.last_grad_norm)
    # the shared layer runs three times per forward: every one of its parameters accumulates
    # three times per backward, and the calibrated counts say so
    assert any(b.expected is not None and b.expected > b.n_params for b in hooked.buckets)
    torch.testing.assert_close(plain.flat_param, hooked.flat_param)


@pytest.mark.parametrize("zero", [True, False])
def test_overlap_with_module_called_several_times_under_checkpoint(zero):
    run_distributed(_albert_worker, 2, zero)


def _pp_dp_worker(rank, world, p2p_mode="overlap"):
    cfg = BertConfig(vocab_size=128, hidden_size=32, num_hidden_layers=4, num_attention_heads=2,
                     intermediate_size=64, hidden_dropout_prob=0.0,
                     attention_probs_dropout_prob=0.0)
    torch.manual_seed(5)
    ref = BertForMaskedLM(cfg).init_weights()
    mesh = DeviceMesh(pp=2, dp=2, tp=1)
    m, lr, clip = 2, 1e-2, 0.05
    sch = slapo.model_schedule.apply_schedule(
        copy.deepcopy(ref), "bert", model_config=cfg, group=False, attn_op_name="reference",
        pipeline_cuts=[1])
    engine, _ = slapo.build(
        sch, target="native", init_weights=False, mesh=mesh, num_micro_batches=m,
        config={"lr": lr, "clip_grad": clip, "weight_decay": 0.0, "bucket_mb": 0.004,
                "overlap_on_cpu": True, "p2p_mode": p2p_mode},
        loss_fn=lambda out, lab: mlm_loss(out["logits"], lab))
    assert engine.inner._overlap and engine._tied and engine._p2p_mode == p2p_mode
    # which reference parameter is which stage parameter (identical initial values)
    names = {}
    for p in engine.stage.parameters():
        hits = [n for n, q in ref.named_parameters()
                if q.shape == p.shape and torch.equal(q.data, p.data)]
        if len(hits) == 1 and p.dim() > 1:
            names[hits[0]] = p
    assert len(names) >= 6
    # every data-parallel replica gets its own batch; the reference sees all of them
    batches = []
    for r in range(mesh.dp_size):
        torch.manual_seed(40 + r)
        ids = torch.randint(0, 128, (4, 16))
        labels = ids.clone()
        labels[:, ::2] = -100
        batches.append((ids, labels))
    ref_opt = torch.optim.AdamW(ref.parameters(), lr=lr, weight_decay=0.0, eps=1e-8)
    for step in range(2):    # the second step runs with calibrated hooks
        ids, labels = batches[mesh.dp_rank]
        loss = engine.train_batch(ids, labels=labels)
        with torch.no_grad():   # this replica's loss, before the reference model moves
            mine = torch.stack([mlm_loss(ref(i)["logits"], l) for i, l in
                                zip(ids.chunk(m), labels.chunk(m))]).mean()
        torch.testing.assert_close(loss, mine, rtol=1e-4, atol=1e-5)
        ref_opt.zero_grad()
        losses = [mlm_loss(ref(i)["logits"], l) for ids_r, lab_r in batches
                  for i, l in zip(ids_r.chunk(m), lab_r.chunk(m))]
        ref_loss = torch.stack(losses).mean()
        ref_loss.backward()
        norm = torch.nn.utils.clip_grad_norm_(ref.parameters(), clip)
        ref_opt.step()
        torch.testing.assert_close(engine.inner.last_grad_norm, norm.detach(), rtol=1e-4,
                                   atol=1e-6)
        for name, p in names.items():
            torch.testing.assert_close(p.data, dict(ref.named_parameters())[name].data,
                                       rtol=1e-3, atol=1e-5, msg=lambda s: f"{name}: {s}")


@pytest.mark.parametrize("p2p_mode", ["overlap", "paired"])
def test_pipeline_times_data_parallel_with_tied_embeddings_and_clipping(p2p_mode):
    run_distributed(_pp_dp_worker, 4, p2p_mode)


def _replica_init_worker(rank, world, zero):
    """Replicas built from different seeds (a meta-device build seeds every data-parallel rank
    on its own) train as one model: the engine starts them from the first replica's values."""
    from slapo_b200.parallel.mesh import DeviceMesh
    from slapo_b200.runtime.engine import TrainEngine

    mesh = DeviceMesh(pp=1, dp=world, tp=1)
    torch.manual_seed(100 + rank)
    model = nn.Sequential(nn.Linear(8, 16), nn.GELU(), nn.Linear(16, 4))
    engine = TrainEngine(model, {"lr": 1e-2, "zero": zero}, mesh=mesh,
                         loss_fn=lambda out, lab: F.mse_loss(out, lab))
    flat = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    both = [torch.empty_like(flat) for _ in range(world)]
    dist.all_gather(both, flat)
    torch.testing.assert_close(both[0], both[1], rtol=0, atol=0)
    gen = torch.Generator().manual_seed(5 + rank)
    for _ in range(2):
        engine.train_batch(torch.randn(4, 8, generator=gen), labels=torch.randn(4, 4, generator=gen))
    flat = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    dist.all_gather(both, flat)
    torch.testing.assert_close(both[0], both[1], rtol=0, atol=0)


@pytest.mark.parametrize("zero", [True, False])
def test_replicas_start_from_the_first_replicas_parameters(zero):
    run_distributed(_replica_init_worker, 2, zero)
