"""BERT-base-shaped 2-layer encoder, fp32, gloo world_size=2: the tensor-
parallel schedule (QKV / FC1 columns, out-proj / FC2 rows + sync) must
reproduce the unsharded model's output and gradients."""
import copy

import torch

import slapo_b200 as slapo
from slapo_b200.models import BertConfig, BertForMaskedLM, BertModel, mlm_loss

from dist_utils import run_distributed


def _make_batch(vocab, batch=8, seq=128, seed=0):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, vocab, (batch, seq), generator=g)
    labels = torch.full_like(ids, -100)
    pick = torch.rand(batch, seq, generator=g) < 0.15
    labels[pick] = ids[pick]
    return ids, labels


def _tp_worker(rank, world, sequence_parallel, via_verify, sp_axis=0):
    cfg = BertConfig(vocab_size=30522, hidden_size=768, num_hidden_layers=2,
                     num_attention_heads=12, intermediate_size=3072,
                     hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    torch.manual_seed(1234)
    ref = BertModel(cfg, add_pooling_layer=False).init_weights()
    ids, _ = _make_batch(cfg.vocab_size)
    if via_verify:
        sch = slapo.create_schedule(copy.deepcopy(ref))
        with slapo.Verify(sch, [ids], device="cpu", eval_mode=True):
            for i in range(cfg.num_hidden_layers):
                attn = sch[f"encoder.layer.{i}.attention"]
                for name in ("query", "key", "value"):
                    attn[f"self.{name}"].shard("weight", axis=0)
                    attn[f"self.{name}"].shard("bias", axis=0)
                    attn[f"self.{name}"].sync("bwd_post", "all_reduce")
                attn["output.dense"].shard("weight", axis=1)
                attn["output.dense"].sync("fwd_post", "all_reduce")
                sch[f"encoder.layer.{i}.intermediate.dense"].shard("weight", axis=0)
                sch[f"encoder.layer.{i}.intermediate.dense"].shard("bias", axis=0)
                sch[f"encoder.layer.{i}.intermediate.dense"].sync("bwd_post", "all_reduce")
                sch[f"encoder.layer.{i}.output.dense"].shard("weight", axis=1)
                sch[f"encoder.layer.{i}.output.dense"].sync("fwd_post", "all_reduce")
        return
    # recipe path: compare explicitly, including gradients
    model = copy.deepcopy(ref)
    sch = slapo.model_schedule.apply_schedule(
        model, "bert", model_config=cfg, prefix="", sequence_parallel=sequence_parallel,
        sequence_parallel_axis=sp_axis, attn_op_name="reference")
    tp_model, _ = slapo.build(sch, init_weights=False)
    out_ref = ref(ids)["last_hidden_state"]
    out_ref.pow(2).mean().backward()
    out_tp = tp_model(ids)["last_hidden_state"]
    out_tp.pow(2).mean().backward()
    torch.testing.assert_close(out_tp, out_ref, rtol=1e-4, atol=1e-4)
    # row-parallel weight gradient = column slice of the full gradient
    g_ref = ref.encoder.layer[0].output.dense.weight.grad
    g_tp = tp_model.encoder.layer[0].output.dense.weight.grad
    torch.testing.assert_close(g_tp, g_ref.chunk(world, dim=1)[rank], rtol=1e-4, atol=1e-5)
    g_ref = ref.encoder.layer[1].intermediate.dense.weight.grad
    g_tp = tp_model.encoder.layer[1].intermediate.dense.weight.grad
    torch.testing.assert_close(g_tp, g_ref.chunk(world, dim=0)[rank], rtol=1e-4, atol=1e-5)
    # replicated LayerNorm: full gradient without SP, partial (summing to the
    # full one over ranks) with SP
    g_ref = ref.encoder.layer[0].output.LayerNorm.weight.grad
    g_tp = tp_model.encoder.layer[0].output.LayerNorm.weight.grad.clone()
    if sequence_parallel:
        assert tp_model.encoder.layer[0].output.LayerNorm.weight.replicated_param
        torch.distributed.all_reduce(g_tp)
    torch.testing.assert_close(g_tp, g_ref, rtol=1e-4, atol=1e-5)
    # vocabulary-parallel embedding
    g_ref = ref.embeddings.word_embeddings.weight.grad
    g_tp = tp_model.embeddings.word_embeddings.weight.grad
    torch.testing.assert_close(g_tp, g_ref.chunk(world, dim=0)[rank], rtol=1e-4, atol=1e-5)


def test_bert_tp2_verify_output_and_grads():
    run_distributed(_tp_worker, 2, False, True)


def test_bert_tp2_recipe_matches_unsharded():
    run_distributed(_tp_worker, 2, False, False)


def test_bert_tp2_sequence_parallel_matches_unsharded():
    run_distributed(_tp_worker, 2, True, False, 0)


def test_bert_tp2_sequence_parallel_axis1_matches_unsharded():
    run_distributed(_tp_worker, 2, True, False, 1)


def _mlm_worker(rank, world):
    cfg = BertConfig(vocab_size=512, hidden_size=64, num_hidden_layers=2,
                     num_attention_heads=4, intermediate_size=128,
                     hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    torch.manual_seed(7)
    ref = BertForMaskedLM(cfg).init_weights()
    ids, labels = _make_batch(cfg.vocab_size, 4, 32)
    model = copy.deepcopy(ref)
    sch = slapo.model_schedule.apply_schedule(model, "bert", model_config=cfg,
                                              attn_op_name="reference")
    tp_model, _ = slapo.build(sch, init_weights=False)
    # tied weights stay tied after sharding
    assert tp_model.cls.predictions.decoder.weight is tp_model.bert.embeddings.word_embeddings.weight
    loss_ref = ref(ids, labels=labels)["loss"]
    logits = tp_model(ids)["logits"]
    assert logits.shape[-1] == cfg.vocab_size // world
    loss_tp = mlm_loss(logits, labels, vocab_parallel=True)
    torch.testing.assert_close(loss_tp, loss_ref, rtol=1e-4, atol=1e-5)
    loss_ref.backward()
    loss_tp.backward()
    g_ref = ref.bert.embeddings.word_embeddings.weight.grad
    g_tp = tp_model.bert.embeddings.word_embeddings.weight.grad
    torch.testing.assert_close(g_tp, g_ref.chunk(world, dim=0)[rank], rtol=1e-3, atol=1e-5)


def test_bert_mlm_vocab_parallel_loss():
    run_distributed(_mlm_worker, 2)


def _roberta_mlm_worker(rank, world):
    """RoBERTa keeps its head under ``lm_head`` and its trunk under ``roberta``: the recipe must
    shard both like BERT's, tied weight included, and padding-aware position ids must survive."""
    from slapo_b200.models import RobertaForMaskedLM, roberta_config

    cfg = roberta_config(vocab_size=512, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                         intermediate_size=128, hidden_dropout_prob=0.0,
                         attention_probs_dropout_prob=0.0, max_position_embeddings=64)
    torch.manual_seed(8)
    ref = RobertaForMaskedLM(cfg).init_weights()
    ids, labels = _make_batch(cfg.vocab_size, 4, 32)
    ids = ids.clamp(min=2)
    ids[1, 24:] = cfg.pad_token_id
    model = copy.deepcopy(ref)
    sch = slapo.model_schedule.apply_schedule(model, "roberta", model_config=cfg,
                                              attn_op_name="reference")
    tp_model, _ = slapo.build(sch, init_weights=False)
    assert tp_model.lm_head.decoder.weight is tp_model.roberta.embeddings.word_embeddings.weight
    assert tp_model.lm_head.decoder.weight.shape[0] == cfg.vocab_size // world
    loss_ref = ref(ids, labels=labels)["loss"]
    logits = tp_model(ids)["logits"]
    assert logits.shape[-1] == cfg.vocab_size // world
    loss_tp = mlm_loss(logits, labels, vocab_parallel=True)
    torch.testing.assert_close(loss_tp, loss_ref, rtol=1e-4, atol=1e-5)
    loss_ref.backward()
    loss_tp.backward()
    g_ref = ref.roberta.embeddings.word_embeddings.weight.grad
    g_tp = tp_model.roberta.embeddings.word_embeddings.weight.grad
    torch.testing.assert_close(g_tp, g_ref.chunk(world, dim=0)[rank], rtol=1e-3, atol=1e-5)


def test_roberta_mlm_vocab_parallel_loss():
    run_distributed(_roberta_mlm_worker, 2)
