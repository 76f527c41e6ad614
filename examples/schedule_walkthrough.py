"""The schedule language on a small BERT, step by step (runs on CPU in seconds).

    python examples/schedule_walkthrough.py
"""
import os
import sys

import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

import slapo_b200 as slapo  # noqa: E402
from slapo_b200.models import BertConfig, BertForMaskedLM  # noqa: E402
from slapo_b200.models.schedules.bert import replace_attention  # noqa: E402


def main():
    cfg = BertConfig(vocab_size=512, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                     intermediate_size=256, hidden_dropout_prob=0.0,
                     attention_probs_dropout_prob=0.0)
    model = BertForMaskedLM(cfg).init_weights().eval()
    ids = torch.randint(0, 512, (2, 16))
    want = model(ids)["logits"]

    sch = slapo.create_schedule(model)
    print("primitives:", slapo.list_primitives())
    # 1. replace every self-attention by the fused-QKV flash-attention module (the recipe's
    #    helper converts the three projection weights to the head-interleaved layout)
    replace_attention(sch, cfg, "bert", attn_op_name="reference")
    with slapo.Verify(sch, [ids], device="cpu"):
        for i in range(cfg.num_hidden_layers):
            layer = sch[f"bert.encoder.layer.{i}"]
            # 2. expose the bias add of the FFN's first Linear, trace, find bias+GeLU, fuse it
            ffn = layer["intermediate"]
            ffn["dense"].decompose()
            ffn.trace(flatten=True)
            matches = ffn.find(lambda x, b: F.gelu(x + b))
            if matches:
                ffn.fuse(matches, compiler="native", name="BiasGeLU")
            # 3. recompute this layer in backward
            layer.checkpoint()
    built, _ = slapo.build(sch, init_weights=False)
    torch.testing.assert_close(built(ids)["logits"], want, rtol=1e-4, atol=1e-4)
    print(built.bert.encoder.layer[0])
    print("scheduled model matches the original")


if __name__ == "__main__":
    main()
