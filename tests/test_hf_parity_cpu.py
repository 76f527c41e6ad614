"""The model zoo against Hugging Face transformers: a randomly initialised Hugging Face model's
``state_dict`` loads into the zoo model with no missing and no unexpected key, and both compute
the same logits (fp32, dropout off).  This pins the parameter names (checkpoints of either side
load into the other) and the architectures."""
import pytest
import torch

tf = pytest.importorskip("transformers")

from slapo_b200 import models as M  # noqa: E402

SMALL = dict(vocab_size=128, hidden_size=32, num_hidden_layers=2, num_attention_heads=2,
             intermediate_size=64, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)


def _compare(hf, zoo, call_hf, call_zoo, atol=2e-5):
    hf.eval()
    zoo.eval()
    res = zoo.load_state_dict(hf.state_dict(), strict=False)
    assert not res.missing_keys, res.missing_keys
    assert not res.unexpected_keys, res.unexpected_keys
    with torch.no_grad():
        want, got = call_hf(hf), call_zoo(zoo)
    torch.testing.assert_close(got, want, rtol=1e-4, atol=atol)
    # and the other way round: the zoo's names are the Hugging Face names
    assert set(zoo.state_dict()) == set(hf.state_dict())


def _ids(batch=2, seq=16, lo=2, hi=120, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(lo, hi, (batch, seq), generator=g)


def test_bert_with_padding_mask():
    torch.manual_seed(0)
    hf = tf.BertForMaskedLM(tf.BertConfig(max_position_embeddings=64, **SMALL))
    zoo = M.BertForMaskedLM(M.BertConfig(max_position_embeddings=64, **SMALL))
    ids = _ids()
    mask = torch.ones_like(ids)
    mask[1, 10:] = 0
    types = torch.zeros_like(ids)
    types[:, 8:] = 1
    _compare(hf, zoo,
             lambda m: m(input_ids=ids, attention_mask=mask, token_type_ids=types).logits,
             lambda m: m(ids, attention_mask=mask, token_type_ids=types)["logits"])


def test_roberta_position_ids_skip_padding():
    torch.manual_seed(1)
    # Hugging Face counts the two reserved positions in max_position_embeddings, the zoo adds them
    hf = tf.RobertaForMaskedLM(tf.RobertaConfig(max_position_embeddings=66, pad_token_id=1,
                                                type_vocab_size=1, layer_norm_eps=1e-5, **SMALL))
    zoo = M.RobertaForMaskedLM(M.roberta_config(max_position_embeddings=64, **SMALL))
    ids = _ids()
    ids[1, 12:] = 1                      # padding at the end of the second sequence
    mask = (ids != 1).long()
    _compare(hf, zoo, lambda m: m(input_ids=ids, attention_mask=mask).logits,
             lambda m: m(ids, attention_mask=mask)["logits"])


def test_albert():
    torch.manual_seed(2)
    kw = dict(SMALL, embedding_size=16, max_position_embeddings=64)
    hf = tf.AlbertForMaskedLM(tf.AlbertConfig(classifier_dropout_prob=0.0, **kw))
    zoo = M.AlbertForMaskedLM(M.AlbertConfig(**kw))
    ids = _ids()
    _compare(hf, zoo, lambda m: m(input_ids=ids).logits, lambda m: m(ids)["logits"])


def test_gpt2_and_gpt_neo():
    torch.manual_seed(3)
    ids = _ids()
    hf = tf.GPT2LMHeadModel(tf.GPT2Config(vocab_size=128, n_positions=64, n_embd=32, n_layer=2,
                                          n_head=2, resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0))
    kw = dict(vocab_size=128, n_positions=64, hidden_size=32, num_layers=2, num_heads=2,
              resid_dropout=0.0, embed_dropout=0.0, attention_dropout=0.0)
    zoo = M.GPT2LMHeadModel(M.GPTConfig(**kw))
    _compare(hf, zoo, lambda m: m(input_ids=ids).logits, lambda m: m(ids)["logits"])
    hf = tf.GPTNeoForCausalLM(tf.GPTNeoConfig(
        vocab_size=128, max_position_embeddings=64, hidden_size=32, num_layers=2, num_heads=2,
        attention_types=[[["global"], 2]], resid_dropout=0.0, embed_dropout=0.0,
        attention_dropout=0.0))
    zoo = M.GPTNeoForCausalLM(M.GPTConfig(model_type="gpt_neo", **kw))
    _compare(hf, zoo, lambda m: m(input_ids=ids).logits, lambda m: m(ids)["logits"])


def test_opt():
    torch.manual_seed(4)
    kw = dict(vocab_size=128, hidden_size=32, num_hidden_layers=2, ffn_dim=64, num_attention_heads=2,
              max_position_embeddings=64, dropout=0.0, attention_dropout=0.0)
    hf = tf.OPTForCausalLM(tf.OPTConfig(word_embed_proj_dim=32, **kw))
    zoo = M.OPTForCausalLM(M.OPTConfig(**kw))
    ids = _ids()
    _compare(hf, zoo, lambda m: m(input_ids=ids).logits, lambda m: m(ids)["logits"])


@pytest.mark.parametrize("gated", [False, True])
def test_t5(gated):
    torch.manual_seed(5)
    kw = dict(vocab_size=128, d_model=32, d_kv=8, d_ff=64, num_layers=2, num_decoder_layers=2,
              num_heads=4, relative_attention_num_buckets=8, relative_attention_max_distance=16,
              dropout_rate=0.0, feed_forward_proj="gated-gelu" if gated else "relu",
              tie_word_embeddings=not gated)
    hf = tf.T5ForConditionalGeneration(tf.T5Config(**kw))
    zoo = M.T5ForConditionalGeneration(M.T5Config(**kw))
    ids, dec = _ids(), _ids(seq=8, seed=9)
    _compare(hf, zoo, lambda m: m(input_ids=ids, decoder_input_ids=dec).logits,
             lambda m: m(ids, decoder_input_ids=dec)["logits"], atol=5e-5)


def _hf_cases():
    small = dict(vocab_size=128, hidden_size=32, num_hidden_layers=2, num_attention_heads=2,
                 intermediate_size=64, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    return {
        "bert": lambda: tf.BertForMaskedLM(tf.BertConfig(max_position_embeddings=64, **small)),
        "roberta": lambda: tf.RobertaForMaskedLM(tf.RobertaConfig(
            max_position_embeddings=66, pad_token_id=1, type_vocab_size=1, **small)),
        "albert": lambda: tf.AlbertForMaskedLM(tf.AlbertConfig(
            embedding_size=16, max_position_embeddings=64, classifier_dropout_prob=0.0, **small)),
        "gpt2": lambda: tf.GPT2LMHeadModel(tf.GPT2Config(
            vocab_size=128, n_positions=64, n_embd=32, n_layer=2, n_head=2, resid_pdrop=0.0,
            embd_pdrop=0.0, attn_pdrop=0.0)),
        "gpt_neo": lambda: tf.GPTNeoForCausalLM(tf.GPTNeoConfig(
            vocab_size=128, max_position_embeddings=64, hidden_size=32, num_layers=2, num_heads=2,
            attention_types=[[["global"], 2]], resid_dropout=0.0, embed_dropout=0.0,
            attention_dropout=0.0)),
        "opt": lambda: tf.OPTForCausalLM(tf.OPTConfig(
            vocab_size=128, hidden_size=32, num_hidden_layers=2, ffn_dim=64, num_attention_heads=2,
            max_position_embeddings=64, dropout=0.0, attention_dropout=0.0, word_embed_proj_dim=32)),
        "t5": lambda: tf.T5ForConditionalGeneration(tf.T5Config(
            vocab_size=128, d_model=32, d_kv=8, d_ff=64, num_layers=2, num_decoder_layers=2,
            num_heads=4, relative_attention_num_buckets=8, relative_attention_max_distance=16,
            dropout_rate=0.0)),
    }


@pytest.mark.parametrize("family", ["bert", "roberta", "albert", "gpt2", "gpt_neo", "opt", "t5"])
def test_recipe_on_an_unmodified_hugging_face_model(family):
    """The scheduling recipes take a Hugging Face model as it is (module paths and configuration
    field names of either side): attention and fused blocks are replaced, the logits stay."""
    import copy

    import slapo_b200 as slapo

    torch.manual_seed(6)
    hf = _hf_cases()[family]().eval()
    ids = _ids()
    extra = {"decoder_input_ids": _ids(seq=8, seed=4)} if family == "t5" else {}
    with torch.no_grad():
        want = hf(input_ids=ids, **extra).logits
    sch = slapo.model_schedule.apply_schedule(copy.deepcopy(hf), family, model_config=hf.config,
                                              attn_op_name="reference")
    model, _ = slapo.build(sch, init_weights=False)
    with torch.no_grad():
        out = model(ids, **extra)
    got = out["logits"] if isinstance(out, dict) else out.logits
    torch.testing.assert_close(got, want, rtol=1e-4, atol=2e-5)
    replaced = [type(m).__name__ for m in model.modules()]
    if family != "t5":
        # (Hugging Face's T5 attention has its own call convention: the recipe fuses the
        # projections of the zoo's T5 only and leaves a Hugging Face T5 as it is at TP = 1)
        marks = ("FlashAttention", "Fused", "LinearWithAct")             # something was scheduled
        assert any(any(m in n for m in marks) for n in replaced), sorted(set(replaced))


def test_causal_plus_padding_mask_reduces_to_the_key_padding_row():
    from slapo_b200.ops.attention import FlashAttentionOp

    op = FlashAttentionOp(attn_op_name="reference", apply_causal_mask=True)
    b, s = 2, 6
    pad = torch.zeros(b, s)
    pad[1, 4:] = -10000.0
    causal = torch.full((s, s), -10000.0).triu(1)
    full = (causal[None, None] + pad[:, None, None, :]).clamp(min=-10000.0)
    torch.testing.assert_close(op._key_bias(full, b, s), pad)
    torch.testing.assert_close(op._key_bias(pad[:, None, None, :], b, s), pad)
    keep = full > -1.0                                  # boolean form: True = attend
    torch.testing.assert_close(op._key_bias(keep, b, s), pad)
    with pytest.raises(NotImplementedError):
        FlashAttentionOp(attn_op_name="reference")._key_bias(full, b, s)


def test_bias_per_head_and_query_runs_the_reference_attention():
    """A ``[B, H, Sq, Sk]`` additive bias (ALiBi-like, or a relative bias computed outside)
    is honoured: the op takes the PyTorch path for it, whichever kernel name it carries."""
    from slapo_b200.ops.attention import FlashAttentionOp

    torch.manual_seed(3)
    b, s, h, d = 2, 6, 3, 8
    q, k, v = (torch.randn(b, s, h, d) for _ in range(3))
    bias = torch.randn(b, h, s, s)
    for causal in (False, True):
        op = FlashAttentionOp(attn_op_name="auto", apply_causal_mask=causal).eval()
        scores = torch.einsum("bqhd,bkhd->bhqk", q, k) / d ** 0.5 + bias
        if causal:
            scores = scores.masked_fill(torch.ones(s, s).triu(1).bool(), float("-inf"))
        want = torch.einsum("bhqk,bkhd->bqhd", scores.softmax(-1), v)
        torch.testing.assert_close(op(q, k, v, bias), want, rtol=1e-5, atol=1e-5)
    # a boolean mask per (query, key) pair, shared by the heads, without causal masking
    keep = torch.rand(b, 1, s, s) > 0.3
    keep[..., 0] = True
    op = FlashAttentionOp(attn_op_name="auto").eval()
    scores = torch.einsum("bqhd,bkhd->bhqk", q, k) / d ** 0.5
    want = torch.einsum("bhqk,bkhd->bqhd",
                        (scores + (~keep).float() * -10000.0).softmax(-1), v)
    torch.testing.assert_close(op(q, k, v, keep), want, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("family,min_graph_modules", [("bert", 10), ("roberta", 10), ("albert", 5),
                                                      ("gpt2", 10), ("gpt_neo", 8), ("t5", 8),
                                                      ("opt", 5)])
def test_hierarchical_trace_of_a_hugging_face_model(family, min_graph_modules):
    """``trace(tracer="huggingface")`` on an unmodified Hugging Face model: catch-all ``**kwargs``
    are dropped for the trace, ``ModelOutput`` reads (by position or attribute) become dict
    reads, lower levels are traced on the shapes that the parent's meta-tensor trace recorded,
    levels whose Python control flow still depends on tensor values stay eager modules - and
    the traced tree computes what the model computed."""
    import copy

    import torch.fx as fx

    import slapo_b200 as slapo

    torch.manual_seed(7)
    hf = _hf_cases()[family]().eval()
    ids = _ids()
    extra = {"decoder_input_ids": _ids(seq=8, seed=4)} if family == "t5" else {}
    with torch.no_grad():
        want = hf(input_ids=ids, **extra).logits
    sch = slapo.create_schedule(copy.deepcopy(hf))
    config = hf.config
    if family == "t5":
        # the meta-tensor engine specialises the graph on the example shapes: inputs of
        # different lengths are described explicitly
        config = {"input_shapes": {"input_ids": (tuple(ids.shape), torch.long),
                                   "decoder_input_ids": ((2, 8), torch.long)}}
    sch.trace(tracer="huggingface", config=config)
    n_traced = sum(isinstance(m, fx.GraphModule) for m in sch.mod.modules())
    assert n_traced >= min_graph_modules, n_traced
    with torch.no_grad():
        out = sch.mod(ids, **extra)
    got = out["logits"] if isinstance(out, dict) else out.logits
    torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-6)


def test_static_graph_primitives_on_a_traced_hugging_face_attention():
    """trace -> find -> horizontal replace on Hugging Face's own BertSelfAttention: the three
    projection chains (linear, view, transpose) are found as three matches and replaced by one
    fused module whose outputs are picked apart by ``getitem`` nodes."""
    import copy

    from torch import nn

    import slapo_b200 as slapo
    from slapo_b200.pattern import call_module

    torch.manual_seed(8)
    hf = _hf_cases()["bert"]().eval()
    ids = _ids()
    with torch.no_grad():
        want = hf(input_ids=ids).logits
    sch = slapo.create_schedule(copy.deepcopy(hf))
    sch.trace(tracer="huggingface", config=hf.config)       # meta shapes: batch 2, 16 tokens
    att = sch["bert.encoder.layer.0.attention.self"]

    def pattern(x):
        x = call_module("query|key|value", x)
        x = x.view(2, 16, -1, 16)
        return x.transpose(1, 2)

    groups = att.find(pattern)
    assert len(groups) == 3 and all(len(g) == 3 for g in groups)

    class FusedProjections(nn.Module):
        def __init__(self, q, k, v, heads):
            super().__init__()
            self.fused = nn.Linear(q.in_features, 3 * q.out_features)
            self.fused.weight.data = torch.cat([q.weight, k.weight, v.weight], 0).data
            self.fused.bias.data = torch.cat([q.bias, k.bias, v.bias], 0).data
            self.heads = heads

        def forward(self, x):
            b, s, _ = x.shape
            return tuple(t.view(b, s, self.heads, -1).transpose(1, 2)
                         for t in self.fused(x).chunk(3, -1))

    old = att.mod
    att.replace(FusedProjections(old.query, old.key, old.value, 2), groups)
    calls = [n for n in att.mod.graph.nodes if n.op == "call_module"]
    assert len(calls) == 1 and "FusedProjections" in str(calls[0].target)
    with torch.no_grad():
        out = sch.mod(ids)
    got = out["logits"] if isinstance(out, dict) else out.logits
    torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-6)


def _hf_tp_worker(rank, world, family):
    import copy

    import torch.distributed as dist

    import slapo_b200 as slapo

    torch.manual_seed(0)
    hf = _hf_cases()[family]().eval()
    slapo.set_random_seed(3, tp_rank=rank)
    ids = _ids(seed=1)
    extra = {"decoder_input_ids": _ids(seq=8, seed=2)} if family == "t5" else {}
    with torch.no_grad():
        want = hf(input_ids=ids, **extra).logits
    sch = slapo.model_schedule.apply_schedule(copy.deepcopy(hf), family, model_config=hf.config,
                                              attn_op_name="reference")
    model, _ = slapo.build(sch, init_weights=False)
    with torch.no_grad():
        out = model(ids, **extra)
    got = out["logits"] if isinstance(out, dict) else out.logits
    assert got.shape[-1] == want.shape[-1] // world         # vocabulary-parallel logits
    parts = [torch.empty_like(got) for _ in range(world)]
    dist.all_gather(parts, got.contiguous())
    torch.testing.assert_close(torch.cat(parts, -1), want, rtol=1e-4, atol=2e-5)


@pytest.mark.parametrize("family", ["bert", "gpt2", "opt", "t5"])
def test_tensor_parallel_recipe_on_a_hugging_face_model(family):
    """Two gloo ranks: the recipe shards an unmodified Hugging Face model (attention, MLP,
    vocabulary-parallel embedding and head) and the gathered logits equal the model's."""
    from dist_utils import run_distributed

    run_distributed(_hf_tp_worker, 2, family)
