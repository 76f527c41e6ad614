"""Training equivalence: three optimizer steps of the native engines on a scheduled model against
``torch.optim.AdamW`` on the unscheduled one, for every transformer family of the zoo and the
parallel layouts that combine the most machinery:

* 2 pipeline stages x 2-way tensor parallelism with sequence-parallel regions and activation
  checkpointing (4 gloo ranks; ALBERT's stages share their one layer);
* 2-way tensor parallelism (sequence parallel) x 2-way sharded data parallelism.

The first step's loss checks the forward pass; the second and third only match when every
gradient - sharded, replicated over the tensor-parallel group, tied across stages, reduced over
the data-parallel group -, the global gradient norm that clipping divides by, the weight-decay
mask and the optimizer state are right.  (The reference library has no such
test: its models are trained by DeepSpeed / Megatron-LM, outside its test suite.)"""
import copy
import dataclasses

import pytest
import torch

import slapo_b200 as slapo
from dist_utils import run_distributed

_TRANSFORMER = dict(vocab_size=512, hidden_size=64, intermediate_size=128, ffn_dim=128,
                    num_attention_heads=4, num_heads=4, num_hidden_layers=4, num_layers=4,
                    num_decoder_layers=4, embedding_size=32, d_model=64, d_kv=16, d_ff=128,
                    hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0, dropout=0.0,
                    dropout_rate=0.0, resid_dropout=0.0, embed_dropout=0.0, attention_dropout=0.0)
_CLIP, _DECAY = 0.05, 0.1                # a limit far below the gradient norms: always clipping
_POSITIONS = {"roberta-large": 66}      # RoBERTa's table starts after the padding index
_SP_FAMILIES = ("bert", "roberta", "gpt2", "gpt_neo", "opt")


def _tiny_spec(name):
    from slapo_b200.models.zoo import get_model_spec

    spec = get_model_spec(name)
    fields = {f.name for f in dataclasses.fields(spec.config)}
    for key, value in _TRANSFORMER.items():
        if key in fields:
            setattr(spec.config, key, value)
    for key in ("max_position_embeddings", "n_positions"):
        if key in fields:
            setattr(spec.config, key, _POSITIONS.get(name, 64))
    spec.num_layers = 4
    return spec


def _worker(rank, world, name, pp, tp, dp, ckpt, bcast=False):
    from slapo_b200.parallel.mesh import DeviceMesh

    torch.manual_seed(21)
    spec = _tiny_spec(name)
    ref = spec.build()
    ref.init_weights()
    ref.train()
    mesh = DeviceMesh(pp=pp, dp=dp, tp=tp)
    slapo.set_random_seed(1, tp_rank=mesh.tp_rank, pp_rank=mesh.pp_rank, dp_rank=mesh.dp_rank,
                          always_enable_tp_seed=True)
    kwargs = dict(model_config=spec.config, group=mesh.schedule_group, attn_op_name="reference",
                  ckpt_ratio=ckpt, bcast_input=bcast)
    if spec.schedule_key in _SP_FAMILIES:
        kwargs.update(sequence_parallel=True, sequence_parallel_axis=0)
    if pp > 1:
        kwargs["pipeline_cuts"] = [[], []] if spec.kind == "seq2seq" else [1]
    sch = slapo.model_schedule.apply_schedule(copy.deepcopy(ref), spec.schedule_key, **kwargs)
    micro = 2
    extra = dict(num_micro_batches=micro) if pp > 1 else {}
    engine, _ = slapo.build(
        sch, target="native", mesh=mesh, init_weights=False,
        loss_fn=spec.loss_fn(mesh.tp_group, tp > 1),
        config={"lr": 1e-2, "clip_grad": _CLIP, "weight_decay": _DECAY,
                "grad_accum_steps": 1 if pp > 1 else micro}, **extra)
    ref_loss = spec.loss_fn(None, False)
    # the engines decay matrices only (no biases, no norm weights); tied tensors count once
    unique = list({id(p): p for p in ref.parameters()}.values())
    ref_opt = torch.optim.AdamW(
        [{"params": [p for p in unique if p.dim() > 1], "weight_decay": _DECAY},
         {"params": [p for p in unique if p.dim() <= 1], "weight_decay": 0.0}], lr=1e-2, eps=1e-8)
    # every data-parallel rank trains on its own batch; the reference sees all of them
    batches = [spec.make_batch(4, seq=32, seq_dec=16, seed=3 + r) for r in range(dp)]
    inputs, labels = batches[mesh.dp_rank]
    if bcast and mesh.tp_rank > 0:
        # only the first rank of a tensor-parallel group holds the batch; the recipe's
        # input hook hands it to the others
        inputs = tuple(torch.zeros_like(t) for t in inputs)
    for step in range(3):
        if pp > 1:
            loss = engine.train_batch(*inputs, labels=labels)
        else:
            parts = [engine.train_batch(*(t.chunk(micro)[m] for t in inputs),
                                        labels=labels.chunk(micro)[m]) for m in range(micro)]
            loss = torch.stack([p.detach() for p in parts]).mean()
        ref_opt.zero_grad()
        wants = [ref_loss(ref(*(t.chunk(micro)[m] for t in ins)), lab.chunk(micro)[m])
                 for ins, lab in batches for m in range(micro)]
        torch.stack(wants).mean().backward()
        torch.nn.utils.clip_grad_norm_(unique, _CLIP)
        ref_opt.step()
        want = torch.stack(wants[mesh.dp_rank * micro:(mesh.dp_rank + 1) * micro]).mean().detach()
        if pp == 1 or mesh.pp_rank == pp - 1:
            torch.testing.assert_close(loss.detach().float().cpu(), want, rtol=2e-4, atol=2e-4,
                                       msg=lambda m: f"{name} step {step}: {m}")


_MODELS = ["bert-base", "roberta-large", "albert-large", "gpt2-medium", "gpt-neo-125m", "opt-350m",
           "t5-base"]


@pytest.mark.parametrize("name", _MODELS)
def test_pipeline_x_tensor_parallel_training_matches_adamw(name):
    run_distributed(_worker, 4, name, 2, 2, 1, 0.5)


@pytest.mark.parametrize("name", _MODELS)
def test_tensor_x_data_parallel_training_matches_adamw(name):
    run_distributed(_worker, 4, name, 1, 2, 2, 0.0)


@pytest.mark.parametrize("name", ["bert-base", "t5-base"])
def test_broadcast_input_hook_under_pipeline_stages(name):
    """``bcast_input=True``: the hook on the whole model survives the partition and runs where
    the inputs enter the pipeline - for T5 also over the decoder ids, which only the second
    stage reads."""
    run_distributed(_worker, 4, name, 2, 2, 1, 0.0, True)


def test_pipeline_mesh_without_cuts_is_refused():
    """A mesh with pipeline stages and a schedule without cuts would train one whole model
    per pipeline rank without anyone noticing."""
    from types import SimpleNamespace

    sch = slapo.create_schedule(torch.nn.Linear(4, 4))
    with pytest.raises(ValueError, match="pipeline stages"):
        slapo.build(sch, target="native", init_weights=False,
                    mesh=SimpleNamespace(pp_size=2))


def test_cut_after_a_given_call_of_a_shared_module():
    """``cut_pipeline_stage(call_index=k)`` on a module that its parent calls several times."""

    class Body(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.shared = torch.nn.Linear(4, 4)

        def forward(self, x):
            for _ in range(3):
                x = self.shared(x)
            return x

    class Top(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.body = Body()

        def forward(self, x):
            return self.body(x)

    sch = slapo.create_schedule(Top())
    sch.trace_until("body")
    sch["body.shared"].cut_pipeline_stage(call_index=1)
    calls = [n for n in sch["body"].mod.graph.nodes if n.op == "call_module"]
    assert [bool(n.meta.get("partition")) for n in calls] == [False, True, False]
    with pytest.raises(IndexError):
        sch["body.shared"].cut_pipeline_stage(call_index=3)


_WRN = {"_name_or_path": "wideresnet-tiny", "block_size": (32, [1, 2, 1, 1])}


def _wrn_worker(rank, world):
    """Two pipeline stages of a Wide ResNet (cut inside the second residual group): BatchNorm
    statistics per micro-batch, the wrapper's ``labels`` input frozen out of the stages."""
    from slapo_b200.models import get_wideresnet
    from slapo_b200.parallel.mesh import DeviceMesh

    torch.manual_seed(3)
    ref = get_wideresnet(_WRN, num_classes=10)
    ref.train()
    mesh = DeviceMesh(pp=2, dp=1, tp=1)
    slapo.set_random_seed(1, pp_rank=mesh.pp_rank)
    sch = slapo.model_schedule.apply_schedule(copy.deepcopy(ref), "wideresnet", model_config=_WRN,
                                              group=mesh.schedule_group,
                                              pipeline_cuts=[[], [0], [], []])

    def loss_fn(out, labels):
        return torch.nn.functional.cross_entropy(out["output"].float(), labels.reshape(-1))

    engine, _ = slapo.build(sch, target="native", mesh=mesh, init_weights=False, loss_fn=loss_fn,
                            num_micro_batches=2,
                            config={"lr": 1e-3, "clip_grad": 0.5, "weight_decay": 0.0})
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-3, weight_decay=0.0, eps=1e-8)
    gen = torch.Generator().manual_seed(5)
    x = torch.randn(4, 3, 64, 64, generator=gen)
    y = torch.randint(0, 10, (4,), generator=gen)
    for step in range(3):
        loss = engine.train_batch(x, labels=y)
        opt.zero_grad()
        want = torch.stack([loss_fn(ref(x.chunk(2)[m]), y.chunk(2)[m]) for m in range(2)]).mean()
        want.backward()
        torch.nn.utils.clip_grad_norm_(ref.parameters(), 0.5)
        opt.step()
        torch.testing.assert_close(loss.detach().float(), want.detach(), rtol=1e-3, atol=1e-4,
                                   msg=lambda m: f"step {step}: {m}")


def test_wideresnet_pipeline_training_matches_adamw():
    run_distributed(_wrn_worker, 2)


def _meta_pipeline_worker(rank, world, name):
    """A model built on the meta device, cut into stages, initialised by ``build``: every norm
    weight is one and every matrix is filled, on every stage.  (Dissolved into graphs by the
    trace, the package's fused blocks used to leave their norm weights on bare containers that
    the model's initialiser did not recognise: they stayed zero and the model was dead.)"""
    from slapo_b200.parallel.mesh import DeviceMesh

    spec = _tiny_spec(name)
    mesh = DeviceMesh(pp=2, dp=1, tp=world // 2)
    slapo.set_random_seed(7, pp_rank=mesh.pp_rank, tp_rank=mesh.tp_rank)
    with slapo.init_empty_weights():
        model = spec.build()
    kwargs = dict(model_config=spec.config, group=mesh.schedule_group, attn_op_name="reference",
                  pipeline_cuts=[[], []] if spec.kind == "seq2seq" else [1])
    sch = slapo.model_schedule.apply_schedule(model, spec.schedule_key, **kwargs)
    engine, _ = slapo.build(sch, target="native", mesh=mesh, init_weights=model._init_weights,
                            device="cpu", num_micro_batches=2,
                            loss_fn=spec.loss_fn(mesh.tp_group, mesh.tp_size > 1),
                            config={"lr": 1e-2, "clip_grad": 1.0})
    stage = engine.inner.model
    assert not any(p.is_meta for p in stage.parameters())
    # the word embedding and the head stay tied across the stages: each rank materialised only
    # its own copy, yet the engine knows the tie and both copies hold the first stage's values
    import torch.distributed as dist

    assert engine._tied, "the tie between the stages was lost"
    mine = [float(p.detach().double().sum()) for p, _ in engine._tied]
    sums = [None] * world
    dist.all_gather_object(sums, mine)
    tp = mesh.tp_size
    assert sums[mesh.tp_rank] == sums[tp + mesh.tp_rank], sums
    for pname, p in stage.named_parameters():
        if p.dim() > 1:
            assert float(p.abs().sum()) > 0, f"{pname} was left at zero"
        elif pname.endswith("weight") and ("orm" in pname or "ln_" in pname):
            torch.testing.assert_close(p.data, torch.ones_like(p), msg=f"{pname} is not one")
    inputs, labels = spec.make_batch(4, seq=32, seq_dec=16, seed=3)
    first = float(engine.train_batch(*inputs, labels=labels))
    for _ in range(3):
        last = float(engine.train_batch(*inputs, labels=labels))
    assert last < first - 0.05          # it learns the batch


@pytest.mark.parametrize("name", ["bert-base", "opt-350m", "t5-base"])
def test_meta_device_model_under_pipeline_stages_is_initialised(name):
    run_distributed(_meta_pipeline_worker, 4, name)


def _tie_worker(rank, world, name):
    spec = _tiny_spec(name)
    with slapo.init_empty_weights():
        model = spec.build()

    def groups(mod):
        by_id = {}
        for pname, p in mod.named_parameters(remove_duplicate=False):
            by_id.setdefault(id(p), []).append(pname)
        return sorted(sorted(v) for v in by_id.values() if len(v) > 1)

    want = groups(model)
    assert want, "the family ties its word embedding to the head"
    sch = slapo.model_schedule.apply_schedule(model, spec.schedule_key, model_config=spec.config,
                                              attn_op_name="reference")
    built, _ = slapo.build(sch, init_weights=model._init_weights, device="cpu")
    assert groups(built) == want


@pytest.mark.parametrize("name", ["bert-base", "albert-large", "gpt2-medium", "opt-350m", "t5-base"])
def test_meta_device_build_keeps_tied_tensors_tied(name):
    """Two tensor-parallel ranks, model on the meta device: after ``build`` the head still
    shares the (sharded) word embedding - also for T5, whose embedding module sits under three
    paths of the model."""
    run_distributed(_tie_worker, 2, name)
