"""GPT-2 / GPT-Neo / OPT recipes: the scheduled model (flash-attention module,
fused MLP, fused LayerNorm) must reproduce the original, alone and under
tensor (+ sequence) parallelism on two gloo ranks."""
import copy

import pytest
import torch

import slapo_b200 as slapo
from slapo_b200.models import (GPT2LMHeadModel, GPTConfig, GPTNeoForCausalLM, OPTConfig,
                               OPTForCausalLM, causal_lm_loss)

from dist_utils import run_distributed


def _make(family):
    torch.manual_seed(3)
    if family == "opt":
        cfg = OPTConfig(vocab_size=512, hidden_size=64, num_hidden_layers=2,
                        num_attention_heads=4, ffn_dim=128, max_position_embeddings=64,
                        dropout=0.0, attention_dropout=0.0)
        return cfg, OPTForCausalLM(cfg).init_weights()
    cfg = GPTConfig(vocab_size=512, n_positions=64, hidden_size=64, num_layers=2, num_heads=4,
                    resid_dropout=0.0, embed_dropout=0.0, attention_dropout=0.0,
                    model_type=family)
    cls = GPT2LMHeadModel if family == "gpt2" else GPTNeoForCausalLM
    return cfg, cls(cfg).init_weights()


@pytest.mark.parametrize("family", ["gpt2", "gpt_neo", "opt"])
def test_decoder_recipe_single(family):
    cfg, ref = _make(family)
    ids = torch.randint(0, 512, (2, 32))
    out_ref = ref(ids)["logits"]
    sch = slapo.model_schedule.apply_schedule(copy.deepcopy(ref), family, model_config=cfg,
                                              attn_op_name="reference")
    model, _ = slapo.build(sch, init_weights=False)
    torch.testing.assert_close(model(ids)["logits"], out_ref, rtol=1e-4, atol=1e-4)


def _tp_worker(rank, world, family, sp):
    cfg, ref = _make(family)
    slapo.set_random_seed(17, tp_rank=rank, always_enable_tp_seed=sp)
    torch.manual_seed(99)
    ids = torch.randint(0, 512, (4, 32))
    loss_ref = ref(ids, labels=ids)["loss"]
    loss_ref.backward()
    sch = slapo.model_schedule.apply_schedule(
        copy.deepcopy(ref), family, model_config=cfg, attn_op_name="reference",
        sequence_parallel=sp, sequence_parallel_axis=1)
    model, _ = slapo.build(sch, init_weights=False)
    logits = model(ids)["logits"]
    assert logits.shape[-1] == cfg.vocab_size // world
    loss = causal_lm_loss(logits, ids, None, vocab_parallel=True)
    torch.testing.assert_close(loss, loss_ref.detach(), rtol=1e-4, atol=1e-4)
    loss.backward()
    # a row-parallel weight gradient equals the matching slice of the full one
    if family == "opt":
        g_ref = ref.model.decoder.layers[0].fc2.weight.grad
        g_tp = model.model.decoder.layers[0].fc2.weight.grad
    else:
        ref_w = ref.transformer.h[0].mlp.c_proj.weight.grad
        g_ref = ref_w.t() if family == "gpt2" else ref_w
        g_tp = model.transformer.h[0].mlp.fc_out.weight.grad
    torch.testing.assert_close(g_tp, g_ref.chunk(world, dim=1)[rank], rtol=1e-3, atol=1e-5)


@pytest.mark.parametrize("family,sp", [("gpt2", False), ("gpt2", True), ("gpt_neo", False),
                                       ("opt", False), ("opt", True)])
def test_decoder_recipe_tp2(family, sp):
    run_distributed(_tp_worker, 2, family, sp)


def _sp_replicated_grad_worker(rank, world, family, axis):
    """Every parameter that stays whole on each rank (LayerNorms, row-parallel biases, position
    tables) must end with the full model's gradient once the tagged ones are summed over the
    group, whichever activation axis the sequence-parallel regions split."""
    import torch.distributed as dist

    cfg, ref = _make(family)
    slapo.set_random_seed(17, tp_rank=rank, always_enable_tp_seed=True)
    torch.manual_seed(99)
    ids = torch.randint(0, 512, (4, 32))
    ref(ids, labels=ids)["loss"].backward()
    sch = slapo.model_schedule.apply_schedule(
        copy.deepcopy(ref), family, model_config=cfg, attn_op_name="reference",
        sequence_parallel=True, sequence_parallel_axis=axis)
    model, _ = slapo.build(sch, init_weights=False)
    causal_lm_loss(model(ids)["logits"], ids, None, vocab_parallel=True).backward()
    want = {n: p.grad for n, p in ref.named_parameters()}
    checked = 0
    for name, p in model.named_parameters():
        if name not in want or p.shape != want[name].shape:
            continue            # sharded or re-laid-out by the recipe
        grad = p.grad.clone()
        if getattr(p, "replicated_param", False):
            dist.all_reduce(grad)
        torch.testing.assert_close(grad, want[name], rtol=1e-3, atol=1e-5, msg=name)
        checked += 1
    assert checked >= 5


@pytest.mark.parametrize("family,axis", [("opt", 0), ("opt", 1), ("gpt2", 0), ("gpt_neo", 0)])
def test_sequence_parallel_replicated_gradients(family, axis):
    run_distributed(_sp_replicated_grad_worker, 2, family, axis)
