"""Named model configurations used by the examples, the benchmark sweeps and
the auto-tuner: ``get_model_spec("opt-2.7b")`` returns how to build the model,
which scheduling recipe applies, how to make a synthetic batch of the
benchmark shape and how to compute the (vocabulary-parallel) loss.

The names follow the Hugging Face checkpoints the reference benchmarks
(benchmark/bench_single_node.py:222-330 and examples/*/deepspeed_hf.py of the
reference); weights are always random-initialised.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch

from .albert import AlbertConfig, AlbertForMaskedLM
from .bert import BertConfig, BertForMaskedLM, RobertaForMaskedLM, mlm_loss, roberta_config
from .gpt import GPT2LMHeadModel, GPTConfig, GPTNeoForCausalLM, causal_lm_loss
from .opt import OPTConfig, OPTForCausalLM
from .t5 import T5Config, T5ForConditionalGeneration, seq2seq_loss
from .wideresnet import get_wideresnet, wideresnet_config


@dataclass
class ModelSpec:
    name: str
    schedule_key: str
    config: object
    build: Callable[[], torch.nn.Module]
    kind: str                    # "mlm" | "causal" | "seq2seq" | "image"
    num_layers: int
    default_seq: int = 512
    default_seq_dec: int = 0

    # ------------------------------------------------------------------ #
    def make_batch(self, batch, seq=None, seq_dec=None, seed=0, device="cpu", pin=False):
        """Synthetic inputs of the benchmark shape: ``(inputs tuple, labels)``."""
        g = torch.Generator().manual_seed(seed)
        seq = seq or self.default_seq
        if self.kind == "image":
            x = torch.randn(batch, 3, 224, 224, generator=g)
            y = torch.randint(0, 1000, (batch,), generator=g)
            tensors = [x, y]
        else:
            vocab = self.config.vocab_size
            ids = torch.randint(0, vocab, (batch, seq), generator=g)
            if self.kind == "mlm":
                labels = torch.full_like(ids, -100)
                pick = torch.rand(batch, seq, generator=g) < 0.15
                labels[pick] = ids[pick]
                tensors = [ids, labels]
            elif self.kind == "causal":
                tensors = [ids, ids.clone()]
            else:
                dec = torch.randint(0, vocab, (batch, seq_dec or self.default_seq_dec), generator=g)
                tensors = [ids, dec, dec.clone()]
        if pin:
            tensors = [t.pin_memory() for t in tensors]
        tensors = [t.to(device, non_blocking=pin) for t in tensors]
        return tuple(tensors[:-1]), tensors[-1]

    def loss_fn(self, tp_group=None, vocab_parallel=False):
        """``loss_fn(model_output, labels)`` for the engines."""
        if self.kind == "mlm":
            return lambda out, lab: mlm_loss(out["logits"], lab, tp_group, vocab_parallel)
        if self.kind == "causal":
            return lambda out, lab: causal_lm_loss(out["logits"], lab, tp_group, vocab_parallel)
        if self.kind == "seq2seq":
            return lambda out, lab: seq2seq_loss(out["logits"], lab, tp_group, vocab_parallel)
        return lambda out, lab: torch.nn.functional.cross_entropy(out["output"].float(),
                                                                  lab.reshape(-1))

    def samples_flops(self, seq=None):
        """Training FLOPs per sample (6 * params * tokens, attention excluded)."""
        seq = seq or self.default_seq
        model = None
        try:
            with torch.device("meta"):
                model = self.build()
            n = sum(p.numel() for p in model.parameters())
        except Exception:
            n = 0
        return 6.0 * n * seq


def _pad_vocab(v, multiple=8):
    return (v + multiple - 1) // multiple * multiple


def _bert(name, **kw):
    cfg = BertConfig(**kw)
    return ModelSpec(name, "bert", cfg, lambda: BertForMaskedLM(cfg), "mlm", cfg.num_hidden_layers)


def _roberta(name, **kw):
    cfg = roberta_config(**kw)
    return ModelSpec(name, "roberta", cfg, lambda: RobertaForMaskedLM(cfg), "mlm",
                     cfg.num_hidden_layers)


def _albert(name, **kw):
    cfg = AlbertConfig(**kw)
    return ModelSpec(name, "albert", cfg, lambda: AlbertForMaskedLM(cfg), "mlm",
                     cfg.num_hidden_layers)


def _gpt(name, family, **kw):
    cfg = GPTConfig(model_type=family, **kw)
    cls = GPT2LMHeadModel if family == "gpt2" else GPTNeoForCausalLM
    return ModelSpec(name, family, cfg, lambda: cls(cfg), "causal", cfg.num_layers,
                     default_seq=1024)


def _opt(name, **kw):
    cfg = OPTConfig(**kw)
    return ModelSpec(name, "opt", cfg, lambda: OPTForCausalLM(cfg), "causal",
                     cfg.num_hidden_layers, default_seq=1024)


def _t5(name, **kw):
    cfg = T5Config(**kw)
    return ModelSpec(name, "t5", cfg, lambda: T5ForConditionalGeneration(cfg), "seq2seq",
                     cfg.num_layers, default_seq=1024, default_seq_dec=512)


def _wrn(name):
    cfg = wideresnet_config(name)
    return ModelSpec(name, "wideresnet", cfg, lambda: get_wideresnet(cfg), "image",
                     sum(cfg["block_size"][1]))


# GPT-2 / GPT-Neo: 50257 -> 50304, a multiple of 128, so that a vocabulary shard stays a multiple of
# 8 elements (16 bytes, what TMA and the vector kernels need) for every group size up to 8
_V_BERT, _V_GPT, _V_OPT = _pad_vocab(30522), _pad_vocab(50257, 128), 50272

MODEL_BUILDERS = {
    "bert-base": lambda: _bert("bert-base", vocab_size=_V_BERT, hidden_size=768,
                               num_hidden_layers=12, num_attention_heads=12,
                               intermediate_size=3072),
    "bert-large": lambda: _bert("bert-large", vocab_size=_V_BERT, hidden_size=1024,
                                num_hidden_layers=24, num_attention_heads=16,
                                intermediate_size=4096),
    "roberta-large": lambda: _roberta("roberta-large", vocab_size=_pad_vocab(50265),
                                      hidden_size=1024, num_hidden_layers=24,
                                      num_attention_heads=16, intermediate_size=4096),
    "albert-large": lambda: _albert("albert-large", vocab_size=30000, embedding_size=128,
                                    hidden_size=1024, num_hidden_layers=24,
                                    num_attention_heads=16, intermediate_size=4096),
    "albert-xxlarge": lambda: _albert("albert-xxlarge", vocab_size=30000, embedding_size=128,
                                      hidden_size=4096, num_hidden_layers=12,
                                      num_attention_heads=64, intermediate_size=16384),
    "gpt2-medium": lambda: _gpt("gpt2-medium", "gpt2", vocab_size=_V_GPT, hidden_size=1024,
                                num_layers=24, num_heads=16),
    "gpt2-xl": lambda: _gpt("gpt2-xl", "gpt2", vocab_size=_V_GPT, hidden_size=1600,
                            num_layers=48, num_heads=25),
    "gpt-neo-125m": lambda: _gpt("gpt-neo-125m", "gpt_neo", vocab_size=_V_GPT, hidden_size=768,
                                 num_layers=12, num_heads=12, n_positions=2048),
    "gpt-neo-1.3b": lambda: _gpt("gpt-neo-1.3b", "gpt_neo", vocab_size=_V_GPT, hidden_size=2048,
                                 num_layers=24, num_heads=16, n_positions=2048),
    # 20 heads: tensor parallelism over whole heads allows TP in {1, 2, 4, 5, 10, 20}
    "gpt-neo-2.7b": lambda: _gpt("gpt-neo-2.7b", "gpt_neo", vocab_size=_V_GPT, hidden_size=2560,
                                 num_layers=32, num_heads=20, n_positions=2048),
    "opt-350m": lambda: _opt("opt-350m", vocab_size=_V_OPT, hidden_size=1024,
                             num_hidden_layers=24, num_attention_heads=16, ffn_dim=4096),
    "opt-1.3b": lambda: _opt("opt-1.3b", vocab_size=_V_OPT, hidden_size=2048,
                             num_hidden_layers=24, num_attention_heads=32, ffn_dim=8192),
    "opt-2.7b": lambda: _opt("opt-2.7b", vocab_size=_V_OPT, hidden_size=2560,
                             num_hidden_layers=32, num_attention_heads=32, ffn_dim=10240),
    "t5-base": lambda: _t5("t5-base", d_model=768, d_kv=64, d_ff=3072, num_layers=12,
                           num_heads=12),
    "t5-large": lambda: _t5("t5-large", d_model=1024, d_kv=64, d_ff=2816, num_layers=24,
                            num_heads=16, feed_forward_proj="gated-gelu"),
    "wideresnet-250M": lambda: _wrn("wideresnet-250M"),
    "wideresnet-1.3B": lambda: _wrn("wideresnet-1.3B"),
    "wideresnet-2.4B": lambda: _wrn("wideresnet-2.4B"),
}


def list_models():
    return sorted(MODEL_BUILDERS)


def get_model_spec(name, **overrides) -> ModelSpec:
    """Spec for ``name``; ``overrides`` replace config attributes (for example
    ``num_hidden_layers=2`` for a smoke run)."""
    if name not in MODEL_BUILDERS:
        raise KeyError(f"unknown model '{name}'; known: {list_models()}")
    spec = MODEL_BUILDERS[name]()
    for key, val in overrides.items():
        if isinstance(spec.config, dict):
            spec.config[key] = val
        else:
            setattr(spec.config, key, val)
    if overrides and not isinstance(spec.config, dict):
        for attr in ("num_hidden_layers", "num_layers"):
            if hasattr(spec.config, attr):
                spec.num_layers = getattr(spec.config, attr)
                break
    return spec
