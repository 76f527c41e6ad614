"""T5, ALBERT and Wide ResNet recipes: the scheduled model reproduces the
original alone, and under tensor parallelism on two gloo ranks (loss and a
sharded weight gradient)."""
import copy

import pytest
import torch

import slapo_b200 as slapo
from slapo_b200.models import (AlbertConfig, AlbertForMaskedLM, T5Config,
                               T5ForConditionalGeneration, get_wideresnet, mlm_loss, seq2seq_loss)

from dist_utils import run_distributed


def _t5(gated):
    torch.manual_seed(5)
    cfg = T5Config(vocab_size=256, d_model=64, d_kv=16, d_ff=128, num_layers=2, num_heads=4,
                   dropout_rate=0.0, attn_op_name="reference",
                   feed_forward_proj="gated-gelu" if gated else "relu")
    return cfg, T5ForConditionalGeneration(cfg).init_weights()


def _t5_batch():
    g = torch.Generator().manual_seed(1)
    return (torch.randint(0, 256, (2, 24), generator=g), torch.randint(0, 256, (2, 16), generator=g))


@pytest.mark.parametrize("gated", [False, True])
def test_t5_recipe_single(gated):
    cfg, ref = _t5(gated)
    src, tgt = _t5_batch()
    out_ref = ref(src, tgt)["logits"]
    sch = slapo.model_schedule.apply_schedule(copy.deepcopy(ref), "t5", model_config=cfg,
                                              ckpt_ratio=0.5)
    model, _ = slapo.build(sch, init_weights=False)
    torch.testing.assert_close(model(src, tgt)["logits"], out_ref, rtol=1e-4, atol=1e-4)


def _t5_tp_worker(rank, world, gated):
    cfg, ref = _t5(gated)
    src, tgt = _t5_batch()
    loss_ref = ref(src, tgt, labels=tgt)["loss"]
    loss_ref.backward()
    sch = slapo.model_schedule.apply_schedule(copy.deepcopy(ref), "t5", model_config=cfg)
    model, _ = slapo.build(sch, init_weights=False)
    logits = model(src, tgt)["logits"]
    assert logits.shape[-1] == cfg.vocab_size // world
    loss = seq2seq_loss(logits, tgt, None, vocab_parallel=True)
    torch.testing.assert_close(loss, loss_ref.detach(), rtol=1e-4, atol=1e-4)
    loss.backward()
    ffn = lambda m: m.decoder.block[1].layer[2].DenseReluDense.wo.weight.grad  # noqa: E731
    torch.testing.assert_close(ffn(model), ffn(ref).chunk(world, dim=1)[rank], rtol=1e-3, atol=1e-5)
    tab = lambda m: (m.encoder.block[0].layer[0].SelfAttention  # noqa: E731
                     .relative_attention_bias.weight.grad)
    torch.testing.assert_close(tab(model), tab(ref).chunk(world, dim=1)[rank], rtol=1e-3, atol=1e-5)


@pytest.mark.parametrize("gated", [False, True])
def test_t5_recipe_tp2(gated):
    run_distributed(_t5_tp_worker, 2, gated)


# ---------------------------------------------------------------------- #
def _albert():
    torch.manual_seed(6)
    cfg = AlbertConfig(vocab_size=256, embedding_size=32, hidden_size=64, num_hidden_layers=3,
                       num_attention_heads=4, intermediate_size=128, max_position_embeddings=64)
    return cfg, AlbertForMaskedLM(cfg).init_weights()


def test_albert_recipe_single():
    cfg, ref = _albert()
    ids = torch.randint(0, 256, (2, 32))
    out_ref = ref(ids)["logits"]
    sch = slapo.model_schedule.apply_schedule(copy.deepcopy(ref), "albert", model_config=cfg,
                                              ckpt_ratio=1.0)
    model, _ = slapo.build(sch, init_weights=False)
    torch.testing.assert_close(model(ids)["logits"], out_ref, rtol=1e-4, atol=1e-4)


def _albert_tp_worker(rank, world):
    cfg, ref = _albert()
    torch.manual_seed(11)
    ids = torch.randint(0, 256, (2, 32))
    loss_ref = ref(ids, labels=ids)["loss"]
    loss_ref.backward()
    sch = slapo.model_schedule.apply_schedule(copy.deepcopy(ref), "albert", model_config=cfg)
    model, _ = slapo.build(sch, init_weights=False)
    logits = model(ids)["logits"]
    assert logits.shape[-1] == cfg.vocab_size // world
    loss = mlm_loss(logits, ids, None, vocab_parallel=True)
    torch.testing.assert_close(loss, loss_ref.detach(), rtol=1e-4, atol=1e-4)
    loss.backward()
    lay = lambda m: m.albert.encoder.albert_layer_groups[0].albert_layers[0]  # noqa: E731
    torch.testing.assert_close(lay(model).ffn_output.weight.grad,
                               lay(ref).ffn_output.weight.grad.chunk(world, dim=1)[rank],
                               rtol=1e-3, atol=1e-5)


def test_albert_recipe_tp2():
    run_distributed(_albert_tp_worker, 2)


# ---------------------------------------------------------------------- #
_WRN_CFG = {"_name_or_path": "wideresnet-tiny", "block_size": (32, [1, 2, 1, 1])}


def _wrn():
    torch.manual_seed(8)
    return get_wideresnet(_WRN_CFG, num_classes=10)


def test_wideresnet_recipe_single():
    ref = _wrn().eval()
    x = torch.randn(2, 3, 64, 64)
    out_ref = ref(x)["output"]
    sch = slapo.model_schedule.apply_schedule(copy.deepcopy(ref), "wideresnet",
                                              model_config=_WRN_CFG, ckpt_ratio=1.0)
    model, _ = slapo.build(sch, init_weights=False)
    torch.testing.assert_close(model.eval()(x)["output"], out_ref, rtol=1e-4, atol=1e-4)


def _wrn_tp_worker(rank, world):
    ref = _wrn()
    torch.manual_seed(21)
    x = torch.randn(4, 3, 64, 64)
    y = torch.randint(0, 10, (4,))
    loss_ref = ref(x, y)["loss"]
    loss_ref.backward()
    sch = slapo.model_schedule.apply_schedule(copy.deepcopy(ref), "wideresnet",
                                              model_config=_WRN_CFG)
    model, _ = slapo.build(sch, init_weights=False)
    loss = model(x, y)["loss"]
    torch.testing.assert_close(loss, loss_ref.detach(), rtol=1e-4, atol=1e-4)
    loss.backward()
    g = model.model.layer2[1].conv2.weight.grad
    g_ref = ref.model.layer2[1].conv2.weight.grad.chunk(world, dim=1)[rank]
    torch.testing.assert_close(g, g_ref, rtol=1e-3, atol=1e-5)
    g = model.model.layer2[1].bn1.weight.grad
    torch.testing.assert_close(g, ref.model.layer2[1].bn1.weight.grad.chunk(world)[rank],
                               rtol=1e-3, atol=1e-5)


def test_wideresnet_recipe_tp2():
    run_distributed(_wrn_tp_worker, 2)


def test_wideresnet_pipeline_cuts():
    ref = _wrn()
    sch = slapo.model_schedule.apply_schedule(copy.deepcopy(ref), "wideresnet",
                                              model_config=_WRN_CFG,
                                              pipeline_cuts=[[], [0], [], []])
    from slapo_b200.parallel.pipeline_partition import generate_pipeline_partition
    pipe = generate_pipeline_partition(sch)
    stages = [n for n in pipe.mod.graph.nodes if n.op == "call_module"]
    assert len(stages) == 2
    x = torch.randn(2, 3, 64, 64)
    ref.eval()
    # the stages end at the logits: the wrapper's optional ``labels`` is frozen at None for the
    # trace, the loss belongs to the engine's loss function
    out = pipe.mod.eval()(x)
    torch.testing.assert_close(out["output"], ref(x)["output"], rtol=1e-4, atol=1e-4)


def test_decoder_vocab_shards_stay_16_byte_aligned():
    """A vocabulary shard of the GPT family is a multiple of 8 rows for every group size up to 8
    (rows of 16-bit logits / gradients must be multiples of 16 bytes for the fused kernels)."""
    from slapo_b200.models import zoo

    for name in ("gpt2-medium", "gpt-neo-125m", "gpt-neo-2.7b"):
        vocab = zoo.get_model_spec(name).config.vocab_size
        assert vocab >= 50257
        for tp in (2, 4, 8):
            assert vocab % tp == 0 and (vocab // tp) % 8 == 0, (name, vocab, tp)


def test_t5_fused_projections_structure():
    """Self-attention gets one ``qkv`` projection, cross-attention ``q`` + one ``kv``; the
    fused weights are the head-interleaved stack of the separate ones."""
    from slapo_b200.models.t5 import T5FusedAttention

    cfg, ref = _t5(False)
    sch = slapo.model_schedule.apply_schedule(copy.deepcopy(ref), "t5", model_config=cfg)
    model, _ = slapo.build(sch, init_weights=False)
    sa = model.decoder.block[0].layer[0].SelfAttention
    ca = model.decoder.block[0].layer[1].EncDecAttention
    assert isinstance(sa, T5FusedAttention) and isinstance(ca, T5FusedAttention)
    assert not hasattr(sa, "q") and sa.qkv.weight.shape[0] == 3 * cfg.num_heads * cfg.d_kv
    assert hasattr(ca, "q") and ca.kv.weight.shape[0] == 2 * cfg.num_heads * cfg.d_kv
    old = ref.decoder.block[0].layer[0].SelfAttention
    w = sa.qkv.weight.view(cfg.num_heads, 3, cfg.d_kv, -1)
    torch.testing.assert_close(w[:, 1].reshape(-1, w.shape[-1]), old.k.weight)
    # and the unfused recipe is still available
    sch2 = slapo.model_schedule.apply_schedule(copy.deepcopy(ref), "t5", model_config=cfg,
                                               fuse_qkv=False)
    assert hasattr(sch2.mod.decoder.block[0].layer[0].SelfAttention, "k")
