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


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape,fused", [((2, 256, 4, 80), False), ((2, 200, 3, 80), False),
                                         ((1, 1024, 2, 80), True), ((2, 384, 2, 96), True),
                                         ((2, 130, 2, 40), False), ((1, 256, 2, 120), False)])
def test_flash_attention_padded_head_dims(shape, fused, causal):
    """Head dimensions between the tile widths (OPT-2.7B: 80): the tile loads zero-fill the
    columns beyond D, outputs and gradients have exactly D columns; ragged sequence lengths,
    separate and packed q/k/v layouts."""
    b, s, h, d = shape
    q, k, v = _mk(b, s, h, d, torch.bfloat16, fused_layout=fused)
    from slapo_b200.ops.flash_attn import native_supported
    assert native_supported(q, k, v)
    _compare(q, k, v,
             lambda q, k, v: NF.flash_attention(q, k, v, causal=causal),
             lambda q, k, v: NF.attention_reference(q, k, v, causal=causal))


def test_flash_attention_head_dim_80_packed_with_dropout():
    from slapo_b200.ops.flash_attn import flash_attention_qkvpacked, packed_supported

    b, s, h, d, p = 2, 256, 4, 80, 0.1
    qkv = torch.randn(b, s, h, 3, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    assert packed_supported(qkv)
    torch.cuda.manual_seed(11)
    mask = dropout_keep_mask(b, h, s, s, p)
    out = flash_attention_qkvpacked(qkv, causal=True, p=p)
    g = torch.randn_like(out)
    out.backward(g)
    ref_in = qkv.detach().float().requires_grad_(True)
    ref = NF.attention_reference(ref_in[..., 0, :], ref_in[..., 1, :], ref_in[..., 2, :],
                                 causal=True, dropout_p=effective_dropout_p(p),
                                 dropout_mask=mask.float())
    ref.backward(g.float())
    for name, a, b_ in (("out", out, ref), ("dqkv", qkv.grad, ref_in.grad)):
        scale = b_.abs().max().clamp(min=1e-3)
        err = ((a.float() - b_).abs().max() / scale).item()
        assert err < 3e-2, f"{name}: relative max error {err:.4f}"
    assert native.ops().device_status() == 0


def test_attention_fallback_is_announced(caplog):
    """Shapes the kernels do not take (head dim not a multiple of 8) run the PyTorch
    reference - and say so once, instead of silently materialising the score matrix."""
    import logging

    q = torch.randn(1, 64, 2, 36, device="cuda", dtype=torch.bfloat16)
    with caplog.at_level(logging.WARNING):
        NF.flash_attention(q, q, q)
        NF.flash_attention(q, q, q)
    hits = [r for r in caplog.records if "falls back" in r.getMessage()]
    assert len(hits) == 1 and "36" in hits[0].getMessage()
