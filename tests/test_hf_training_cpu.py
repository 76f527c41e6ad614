"""Unmodified Hugging Face models through the recipes and the native engines: three optimizer
steps on 2 pipeline stages x 2-way tensor parallelism (sequence-parallel regions where the
recipe has them, half of the layers recomputed) against ``torch.optim.AdamW`` on the same
Hugging Face model, untouched.

This is the workflow of the reference's example scripts (a ``transformers`` model, the family's
recipe with ``pipeline_cuts``, a pipeline runtime: examples/bert/deepspeed_hf.py:60-140 of the
reference), with the native runtime in place of DeepSpeed.  What it pins beyond the zoo-model
tests: the ``"huggingface"`` tracer inside the recipes, ``ModelOutput`` / tuple values crossing
stage boundaries, collectives on modules that return structured outputs, shape propagation
through the scatter / gather hooks, Hugging Face's per-stack T5 embedding modules."""
import copy

import pytest
import torch

import slapo_b200 as slapo
from dist_utils import run_distributed

transformers = pytest.importorskip("transformers")

_SP = ("bert", "roberta", "gpt2", "gpt_neo", "opt")


def _make(family):
    tr = transformers
    common = dict(vocab_size=512)
    if family in ("bert", "roberta", "albert"):
        kw = dict(hidden_size=64, num_hidden_layers=4, num_attention_heads=4, intermediate_size=128,
                  max_position_embeddings=66, hidden_dropout_prob=0.0,
                  attention_probs_dropout_prob=0.0, **common)
        if family == "albert":
            return tr.AlbertForMaskedLM(tr.AlbertConfig(embedding_size=32, **kw)), "mlm"
        cls = {"bert": (tr.BertConfig, tr.BertForMaskedLM),
               "roberta": (tr.RobertaConfig, tr.RobertaForMaskedLM)}[family]
        return cls[1](cls[0](**kw)), "mlm"
    if family == "gpt2":
        cfg = tr.GPT2Config(n_embd=64, n_layer=4, n_head=4, n_positions=64, resid_pdrop=0.0,
                            embd_pdrop=0.0, attn_pdrop=0.0, **common)
        return tr.GPT2LMHeadModel(cfg), "causal"
    if family == "gpt_neo":
        cfg = tr.GPTNeoConfig(hidden_size=64, num_layers=4, num_heads=4,
                              attention_types=[[["global"], 4]], max_position_embeddings=64,
                              resid_dropout=0.0, embed_dropout=0.0, attention_dropout=0.0, **common)
        return tr.GPTNeoForCausalLM(cfg), "causal"
    if family == "opt":
        cfg = tr.OPTConfig(hidden_size=64, num_hidden_layers=4, ffn_dim=128, num_attention_heads=4,
                           max_position_embeddings=64, dropout=0.0, attention_dropout=0.0,
                           word_embed_proj_dim=64, **common)
        return tr.OPTForCausalLM(cfg), "causal"
    cfg = tr.T5Config(d_model=64, d_kv=16, d_ff=128, num_layers=2, num_decoder_layers=2,
                      num_heads=4, dropout_rate=0.0, **common)
    return tr.T5ForConditionalGeneration(cfg), "seq2seq"


def _logits(out):
    return out["logits"] if isinstance(out, dict) else out.logits


def _worker(rank, world, family, pp, tp, sp_axis=0):
    from slapo_b200.models import causal_lm_loss, mlm_loss, seq2seq_loss
    from slapo_b200.parallel.mesh import DeviceMesh

    torch.manual_seed(21)
    ref, kind = _make(family)
    ref.train()
    mesh = DeviceMesh(pp=pp, dp=1, tp=tp)
    sp = family in _SP and tp > 1
    slapo.set_random_seed(1, tp_rank=mesh.tp_rank, pp_rank=mesh.pp_rank, always_enable_tp_seed=sp)
    kwargs = dict(model_config=ref.config, group=mesh.schedule_group, attn_op_name="reference",
                  ckpt_ratio=0.5)
    if family in _SP:
        kwargs.update(sequence_parallel=sp, sequence_parallel_axis=sp_axis)
    if pp > 1:
        # the graphs of a Hugging Face model are specialised on the micro-batch's shapes
        if kind == "seq2seq":
            kwargs.update(pipeline_cuts=[[], []] if pp == 2 else [[0], [0]], trace_config={
                "input_shapes": {"input_ids": (2, 32), "decoder_input_ids": (2, 16)}})
        else:
            kwargs.update(pipeline_cuts=[1] if pp == 2 else [0, 1, 2],
                          trace_config={"batch_size": 2, "seq_len": 32})
    sch = slapo.model_schedule.apply_schedule(copy.deepcopy(ref), family, **kwargs)
    loss_of = {"mlm": mlm_loss, "causal": causal_lm_loss, "seq2seq": seq2seq_loss}[kind]
    extra = dict(num_micro_batches=2) if pp > 1 else {}
    engine, _ = slapo.build(
        sch, target="native", mesh=mesh, init_weights=False,
        loss_fn=lambda out, lab: loss_of(_logits(out), lab, mesh.tp_group, tp > 1),
        config={"lr": 1e-2, "clip_grad": 0.05, "weight_decay": 0.0,
                "grad_accum_steps": 1 if pp > 1 else 2}, **extra)
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-2, weight_decay=0.0, eps=1e-8)
    gen = torch.Generator().manual_seed(5)
    ids = torch.randint(0, 512, (4, 32), generator=gen)
    if kind == "mlm":
        labels = torch.full_like(ids, -100)
        pick = torch.rand(4, 32, generator=gen) < 0.3
        labels[pick] = ids[pick]
        inputs = {"input_ids": ids}
    elif kind == "causal":
        labels, inputs = ids.clone(), {"input_ids": ids}
    else:
        dec = torch.randint(0, 512, (4, 16), generator=gen)
        labels, inputs = dec.clone(), {"input_ids": ids, "decoder_input_ids": dec}

    def part(m):
        return {k: v.chunk(2)[m] for k, v in inputs.items()}

    for step in range(3):
        if pp > 1:
            loss = engine.train_batch(**inputs, labels=labels)
        else:
            loss = torch.stack([engine.train_batch(**part(m), labels=labels.chunk(2)[m]).detach()
                                for m in range(2)]).mean()
        opt.zero_grad()
        want = torch.stack([loss_of(_logits(ref(**part(m))), labels.chunk(2)[m])
                            for m in range(2)]).mean()
        want.backward()
        torch.nn.utils.clip_grad_norm_(ref.parameters(), 0.05)
        opt.step()
        torch.testing.assert_close(loss.detach().float(), want.detach(), rtol=3e-4, atol=3e-4,
                                   msg=lambda m: f"{family} step {step}: {m}")


@pytest.mark.parametrize("family", ["bert", "roberta", "albert", "gpt2", "gpt_neo", "opt", "t5"])
def test_hugging_face_model_trains_on_two_stages_x_two_way_tensor_parallel(family):
    run_distributed(_worker, 4, family, 2, 2)


def test_hugging_face_t5_keeps_its_embedding_tied_under_tensor_parallelism():
    """Every T5 stack of recent ``transformers`` has an embedding module of its own on the
    shared weight: without vocabulary-parallel hooks on each, training would quietly split
    the encoder's table from the head's (two steps are enough to see it)."""
    run_distributed(_worker, 2, "t5", 1, 2)


@pytest.mark.parametrize("family", ["bert", "gpt2", "gpt_neo"])
def test_hugging_face_model_with_the_sequence_axis_split(family):
    """``sequence_parallel_axis=1`` (the reference's layout).  The decoders of recent
    ``transformers`` number positions from the embedded tokens' length, so their embeddings
    stay whole and the split happens in front of the first block."""
    run_distributed(_worker, 4, family, 2, 2, 1)


def test_hugging_face_opt_refuses_the_sequence_axis_split():
    with pytest.raises(Exception, match="sequence_parallel_axis=0"):
        run_distributed(_worker, 2, "opt", 1, 2, 1)


@pytest.mark.parametrize("family", ["t5", "gpt2"])
def test_hugging_face_model_on_four_stages(family):
    """More stages than micro-batches; for T5 the relative-position biases (permuted views,
    with gradients) cross the stage boundaries next to the hidden states."""
    run_distributed(_worker, 4, family, 4, 1)
