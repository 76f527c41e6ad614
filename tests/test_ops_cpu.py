"""Op modules on CPU: fused-QKV layout, attention module with past keys, FusedMLP activation
handling, matmul -> sync -> bias ordering, vocabulary-parallel cross entropy on two ranks,
Print inside traced graphs."""
import io
from contextlib import redirect_stdout

import pytest
import torch
import torch.nn.functional as F
from torch import nn

import slapo_b200 as slapo
from slapo_b200 import op

from dist_utils import run_distributed


def test_fused_qkv_layout_matches_separate_projections():
    torch.manual_seed(0)
    h, heads = 32, 4
    q, k, v = (nn.Linear(h, h) for _ in range(3))
    attn = op.FlashAttention(h, heads, attn_op_name="reference", fused_qkv=True, output_proj=False,
                             causal=False)
    with torch.no_grad():
        attn.qkv.weight.copy_(op.FlashAttention.layout_qkv_from_separate(
            q.weight, k.weight, v.weight, heads))
        attn.qkv.bias.copy_(op.FlashAttention.layout_qkv_from_separate(q.bias, k.bias, v.bias, heads))
    x = torch.randn(2, 6, h)
    out, _ = attn(x)
    sp = lambda t: t.view(2, 6, heads, h // heads).transpose(1, 2)   # noqa: E731
    ref = F.scaled_dot_product_attention(sp(q(x)), sp(k(x)), sp(v(x))).transpose(1, 2).reshape(2, 6, h)
    torch.testing.assert_close(out, ref, rtol=1e-4, atol=1e-5)
    # sharding the fused weight along axis 0 keeps whole heads: the first half of the rows
    # is exactly heads 0..1 of q, k and v
    half = attn.qkv.weight[: 3 * h // 2]
    want = op.FlashAttention.layout_qkv_from_separate(q.weight[: h // 2], k.weight[: h // 2],
                                                      v.weight[: h // 2], heads // 2)
    torch.testing.assert_close(half, want)


def test_attention_module_causal_flag_and_kv_cache():
    torch.manual_seed(1)
    attn = op.FlashAttention(32, 4, attn_op_name="reference", fused_qkv=False, output_proj=True,
                             causal=True).eval()
    x = torch.randn(1, 5, 32)
    full, _ = attn(x)
    # decoding the last token with the cached keys / values of the first four gives the same row
    _, present = attn(x[:, :4], use_cache=True)
    last, _ = attn(x[:, 4:], layer_past=present)
    torch.testing.assert_close(last[:, 0], full[:, 4], rtol=1e-4, atol=1e-5)
    # the reference derives causality from output_proj; an explicit flag overrides it
    assert op.FlashAttention(32, 4, attn_op_name="reference", output_proj=True).attn_op.apply_causal_mask
    assert not op.FlashAttention(32, 4, attn_op_name="reference", output_proj=True,
                                 causal=False).attn_op.apply_causal_mask


@pytest.mark.parametrize("act", ["gelu", "gelu_new", "relu"])
def test_fused_mlp_uses_the_requested_activation(act):
    torch.manual_seed(2)
    mlp = op.FusedMLP(16, 32, act, resid_pdrop=0.0).eval()
    x = torch.randn(3, 16)
    ref_act = {"gelu": F.gelu, "gelu_new": lambda t: F.gelu(t, approximate="tanh"), "relu": F.relu}[act]
    h = ref_act(F.linear(x, mlp.fc_in.weight, mlp.fc_in.bias))
    ref = F.linear(h, mlp.fc_out.weight, mlp.fc_out.bias)
    torch.testing.assert_close(mlp(x), ref, rtol=1e-4, atol=1e-5)


def test_linear_with_sync_func_adds_bias_after_the_sync():
    lin = op.LinearWithSyncFunc(8, 4, bias=True, sync_fn=lambda t: t * 2.0)   # stands for a 2-rank sum
    x = torch.randn(5, 8)
    want = F.linear(x, lin.weight) * 2.0 + lin.bias
    torch.testing.assert_close(lin(x), want)
    assert "sync_fn" in repr(lin)
    sep = op.LinearWithSeparateBias(8, 4)
    torch.testing.assert_close(sep(x), F.linear(x, sep.weight, sep.bias))


def _ce_worker(rank, world):
    torch.manual_seed(3)
    logits = torch.randn(6, 10, 32)
    labels = torch.randint(0, 32, (6, 10))
    labels[0, :3] = -100
    full = logits.clone().requires_grad_(True)
    ref = F.cross_entropy(full.view(-1, 32), labels.view(-1), reduction="none", ignore_index=-100)
    ref.sum().backward()
    local = logits.chunk(world, dim=-1)[rank].clone().requires_grad_(True)
    loss = op.ParallelCrossEntropy()(local, labels)
    torch.testing.assert_close(loss.view(-1), ref.detach(), rtol=1e-5, atol=1e-5)
    loss.sum().backward()
    torch.testing.assert_close(local.grad, full.grad.chunk(world, dim=-1)[rank], rtol=1e-5, atol=1e-6)
    # label smoothing agrees with PyTorch's definition too
    sm = op.ParallelCrossEntropy(label_smoothing=0.1)(local.detach(), labels)
    ref_sm = F.cross_entropy(logits.view(-1, 32), labels.view(-1), reduction="none",
                             ignore_index=-100, label_smoothing=0.1)
    torch.testing.assert_close(sm.view(-1), ref_sm, rtol=1e-4, atol=1e-5)


def test_vocab_parallel_cross_entropy_two_ranks():
    run_distributed(_ce_worker, 2)


def test_print_survives_tracing_and_prints_runtime_values():
    class M(nn.Module):
        def __init__(self):
            super().__init__()
            self.lin = nn.Linear(4, 4)
            self.print = op.Print()

        def forward(self, x):
            y = self.lin(x) + 1
            y = self.print(y, "y has shape", y.shape)          # values passed lazily
            self.print(x, f"eager text {x}")                    # result unused: dropped by DCE
            return y * 2

    model = M()
    sch = slapo.create_schedule(model)
    sch.trace()
    targets = [n.target for n in sch.mod.graph.nodes if n.op == "call_module"]
    assert "print" in targets
    sch.mod.graph.eliminate_dead_code()
    sch.mod.recompile()
    assert [n.target for n in sch.mod.graph.nodes if n.op == "call_module"].count("print") == 1
    buf = io.StringIO()
    with redirect_stdout(buf):
        out = sch.mod(torch.zeros(2, 4))
    assert "y has shape torch.Size([2, 4])" in buf.getvalue()
    torch.testing.assert_close(out, (model.lin(torch.zeros(2, 4)) + 1) * 2)
