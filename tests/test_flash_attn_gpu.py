"""tcgen05 flash attention (forward + backward) against the fp32 PyTorch
reference of the same attention."""
import pytest
import torch

from slapo_b200.ops import functional as NF
from slapo_b200.ops import native
from slapo_b200.ops.flash_attn import dropout_keep_mask, effective_dropout_p

pytestmark = pytest.mark.gpu


def _mk(b, s, h, d, dtype, fused_layout=False):
    if fused_layout:  # q/k/v as strided slices of one projection output
        qkv = torch.randn(b, s, h, 3, d, device="cuda", dtype=dtype)
        return [qkv[..., i, :].detach().requires_grad_(True) for i in range(3)]
    return [torch.randn(b, s, h, d, device="cuda", dtype=dtype, requires_grad=True) for _ in range(3)]


def _compare(q, k, v, out_fn, ref_fn, tol=3e-2):
    out = out_fn(q, k, v)
    assert native.ops().device_status() == 0, "a bounded wait inside the kernel ran out"
    g = torch.randn_like(out)
    out.backward(g)
    got = [out] + [t.grad.clone() for t in (q, k, v)]
    qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ref = ref_fn(qr, kr, vr)
    ref.backward(g.float())
    want = [ref, qr.grad, kr.grad, vr.grad]
    for name, a, b in zip(("out", "dq", "dk", "dv"), got, want):
        scale = b.abs().max().clamp(min=1e-3)
        err = ((a.float() - b).abs().max() / scale).item()
        assert err < tol, f"{name}: relative max error {err:.4f}"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", [(2, 128, 2, 64), (2, 512, 4, 64), (1, 384, 2, 128),
                                   (2, 200, 3, 64), (1, 1024, 2, 128)])
def test_flash_attention_matches_reference(shape, causal, dtype):
    b, s, h, d = shape
    q, k, v = _mk(b, s, h, d, dtype, fused_layout=(s == 512))
    _compare(q, k, v,
             lambda q, k, v: NF.flash_attention(q, k, v, causal=causal),
             lambda q, k, v: NF.attention_reference(q, k, v, causal=causal))


def test_flash_attention_key_padding_bias():
    b, s, h, d = 3, 320, 2, 64
    q, k, v = _mk(b, s, h, d, torch.bfloat16)
    lens = torch.tensor([320, 200, 77], device="cuda")
    bias = torch.where(torch.arange(s, device="cuda")[None] < lens[:, None], 0.0, -10000.0)
    _compare(q, k, v,
             lambda q, k, v: NF.flash_attention(q, k, v, key_padding_bias=bias),
             lambda q, k, v: NF.attention_reference(q, k, v, key_padding_bias=bias))


def test_flash_attention_cross_lengths():
    b, h, d = 2, 2, 64
    q = torch.randn(b, 256, h, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(b, 640, h, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(b, 640, h, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    _compare(q, k, v, lambda q, k, v: NF.flash_attention(q, k, v),
             lambda q, k, v: NF.attention_reference(q, k, v))


@pytest.mark.parametrize("bidirectional", [True, False])
def test_flash_attention_t5_relative_bias(bidirectional):
    b, s, h, d = 2, 256, 4, 64
    q, k, v = _mk(b, s, h, d, torch.bfloat16)
    table = (torch.randn(32, h, device="cuda") * 0.5).requires_grad_(True)
    table_ref = table.detach().clone().requires_grad_(True)
    kw = dict(causal=not bidirectional, scale=1.0, rel_bidirectional=bidirectional,
              rel_max_distance=128)
    q.data *= 0.2
    k.data *= 0.2
    _compare(q, k, v,
             lambda q, k, v: NF.flash_attention(q, k, v, rel_bias_table=table, **kw),
             lambda q, k, v: NF.attention_reference(q, k, v, rel_bias_table=table_ref, **kw))
    scale = table_ref.grad.abs().max().clamp(min=1e-3)
    err = ((table.grad - table_ref.grad).abs().max() / scale).item()
    assert err < 3e-2, f"relative-position table grad: {err}"


@pytest.mark.parametrize("shape,causal", [((2, 200, 3, 64), False), ((2, 384, 2, 64), True),
                                          ((1, 256, 2, 128), False), ((1, 300, 2, 128), True)])
def test_flash_attention_dropout_masked_paths(shape, causal):
    """Dropout on the general path (causal, ragged sequence lengths, head dim 128)."""
    b, s, h, d = shape
    p = 0.2
    q, k, v = _mk(b, s, h, d, torch.bfloat16)
    torch.cuda.manual_seed(7)
    mask = dropout_keep_mask(b, h, s, s, p)
    _compare(q, k, v,
             lambda q, k, v: NF.flash_attention(q, k, v, causal=causal, dropout_p=p, training=True),
             lambda q, k, v: NF.attention_reference(q, k, v, causal=causal,
                                                    dropout_p=effective_dropout_p(p),
                                                    dropout_mask=mask.float()))


def test_effective_dropout_probability():
    assert effective_dropout_p(0.0) == 0.0 and effective_dropout_p(0.5) == 0.5
    assert abs(effective_dropout_p(0.1) - 13 / 128) < 1e-9
    mask = dropout_keep_mask(2, 4, 512, 512, 0.1)
    assert abs(mask.float().mean().item() - (1 - 13 / 128)) < 2e-3


@pytest.mark.parametrize("p", [0.1, 0.3])
def test_flash_attention_dropout_replay(p):
    b, s, h, d = 2, 256, 2, 64
    q, k, v = _mk(b, s, h, d, torch.bfloat16)
    torch.cuda.manual_seed(123)
    mask = dropout_keep_mask(b, h, s, s, p)
    keep = mask.float().mean().item()
    assert abs(keep - (1 - p)) < 0.01, keep
    _compare(q, k, v,
             lambda q, k, v: NF.flash_attention(q, k, v, dropout_p=p, training=True),
             lambda q, k, v: NF.attention_reference(q, k, v, dropout_p=effective_dropout_p(p),
                                                    dropout_mask=mask.float()))
