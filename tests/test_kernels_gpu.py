"""Numerics of the hand-written sm_100a element-wise / normalisation kernels
against plain PyTorch fp32 references of the same ops."""
import pytest
import torch
import torch.nn.functional as F

from slapo_b200.ops import functional as NF
from slapo_b200.ops import native

pytestmark = pytest.mark.gpu

DTYPES = [torch.bfloat16, torch.float16, torch.float32]


def _tol(dtype):
    return {torch.bfloat16: (2e-2, 2e-2), torch.float16: (4e-3, 4e-3),
            torch.float32: (2e-4, 2e-4)}[dtype]  # kernels use fast-math intrinsics


@pytest.fixture(autouse=True)
def _need_native():
    assert native.available(), f"native extension missing: {native.load_error()}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("act", ["gelu", "gelu_new", "relu"])
@pytest.mark.parametrize("shape", [(4, 37, 1024), (3, 5, 520), (2048, 4096)])
def test_bias_act(dtype, act, shape):
    x = torch.randn(*shape, device="cuda", dtype=dtype, requires_grad=True)
    b = torch.randn(shape[-1], device="cuda", dtype=dtype, requires_grad=True)
    before = native.launch_count()
    y = NF.bias_act(x, b, act)
    g = torch.randn_like(y)
    y.backward(g)
    assert native.launch_count() > before
    xr = x.detach().float().requires_grad_(True)
    br = b.detach().float().requires_grad_(True)
    yr = NF._act_ref(xr + br, act)
    yr.backward(g.float())
    rtol, atol = _tol(dtype)
    torch.testing.assert_close(y.float(), yr, rtol=rtol, atol=atol)
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=rtol, atol=atol)
    # the bias gradient sums thousands of rows: compare relative to its scale
    scale = br.grad.abs().max().clamp(min=1.0)
    torch.testing.assert_close(b.grad.float() / scale, br.grad / scale, rtol=rtol, atol=atol)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("cols", [256, 1024, 2560, 4096, 8192])
@pytest.mark.parametrize("rms", [False, True])
def test_layer_norm(dtype, cols, rms):
    rows = 777
    x = torch.randn(rows, cols, device="cuda", dtype=dtype) * 2 + 0.5
    x.requires_grad_(True)
    w = (torch.randn(cols, device="cuda", dtype=dtype) * 0.1 + 1).requires_grad_(True)
    b = (torch.randn(cols, device="cuda", dtype=dtype) * 0.1).requires_grad_(True)
    if rms:
        y = NF.rms_norm(x, w, 1e-6)
    else:
        y = NF.layer_norm(x, w, b, 1e-5)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    br = b.detach().float().requires_grad_(True)
    if rms:
        yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-6) * wr
    else:
        yr = F.layer_norm(xr, (cols,), wr, br, 1e-5)
    yr.backward(g.float())
    rtol, atol = _tol(dtype)
    torch.testing.assert_close(y.float(), yr, rtol=rtol, atol=atol)
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=rtol, atol=atol * 2)
    s = wr.grad.abs().max().clamp(min=1.0)
    torch.testing.assert_close(w.grad.float() / s, wr.grad / s, rtol=rtol, atol=atol)
    if not rms:
        s = br.grad.abs().max().clamp(min=1.0)
        torch.testing.assert_close(b.grad.float() / s, br.grad / s, rtol=rtol, atol=atol)


def _recover_mask(shape, dtype, p, seed):
    torch.cuda.manual_seed(seed)
    ones = torch.ones(*shape, device="cuda", dtype=dtype)
    y = NF.bias_dropout_add(ones, None, None, p, True)
    return (y != 0)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("p", [0.1, 0.5])
def test_bias_dropout_add(dtype, p):
    shape = (6, 100, 1024)
    mask = _recover_mask(shape, dtype, p, 11)
    keep = mask.float().mean().item()
    assert abs(keep - (1 - p)) < 0.01, keep
    # a different seed gives a different mask, the same seed the same one
    assert not torch.equal(mask, _recover_mask(shape, dtype, p, 12))
    assert torch.equal(mask, _recover_mask(shape, dtype, p, 11))
    x = torch.randn(*shape, device="cuda", dtype=dtype, requires_grad=True)
    b = torch.randn(shape[-1], device="cuda", dtype=dtype, requires_grad=True)
    r = torch.randn(*shape, device="cuda", dtype=dtype, requires_grad=True)
    torch.cuda.manual_seed(11)
    y = NF.bias_dropout_add(x, b, r, p, True)
    g = torch.randn_like(y)
    y.backward(g)
    xr, br, rr = (t.detach().float().requires_grad_(True) for t in (x, b, r))
    yr = (xr + br) * mask / (1 - NF.effective_dropout_p(p)) + rr
    yr.backward(g.float())
    rtol, atol = _tol(dtype)
    torch.testing.assert_close(y.float(), yr, rtol=rtol, atol=atol)
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=rtol, atol=atol)
    torch.testing.assert_close(r.grad.float(), rr.grad, rtol=rtol, atol=atol)
    s = br.grad.abs().max().clamp(min=1.0)
    torch.testing.assert_close(b.grad.float() / s, br.grad / s, rtol=rtol, atol=atol)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("p", [0.0, 0.1])
@pytest.mark.parametrize("cols", [1024, 2560])
def test_dropout_add_layer_norm(dtype, p, cols):
    shape = (3, 129, cols)
    mask = _recover_mask(shape, dtype, p, 21) if p > 0 else torch.ones(shape, device="cuda", dtype=torch.bool)
    x = torch.randn(*shape, device="cuda", dtype=dtype, requires_grad=True)
    b = torch.randn(cols, device="cuda", dtype=dtype, requires_grad=True)
    r = torch.randn(*shape, device="cuda", dtype=dtype, requires_grad=True)
    w = (torch.randn(cols, device="cuda", dtype=dtype) * 0.1 + 1).requires_grad_(True)
    lb = (torch.randn(cols, device="cuda", dtype=dtype) * 0.1).requires_grad_(True)
    torch.cuda.manual_seed(21)
    y, z = NF.dropout_add_layer_norm(x, b, r, w, lb, p, 1e-5, True)
    gy, gz = torch.randn_like(y), torch.randn_like(z)
    torch.autograd.backward([y, z], [gy, gz])
    xr, br, rr, wr, lbr = (t.detach().float().requires_grad_(True) for t in (x, b, r, w, lb))
    zr = (xr + br) * mask / (1 - NF.effective_dropout_p(p)) + rr
    yr = F.layer_norm(zr, (cols,), wr, lbr, 1e-5)
    torch.autograd.backward([yr, zr], [gy.float(), gz.float()])
    rtol, atol = _tol(dtype)
    torch.testing.assert_close(z.float(), zr, rtol=rtol, atol=atol)
    torch.testing.assert_close(y.float(), yr, rtol=rtol, atol=atol * 2)
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=rtol, atol=atol * 4)
    torch.testing.assert_close(r.grad.float(), rr.grad, rtol=rtol, atol=atol * 4)
    for got, ref in ((w.grad, wr.grad), (lb.grad, lbr.grad), (b.grad, br.grad)):
        s = ref.abs().max().clamp(min=1.0)
        torch.testing.assert_close(got.float() / s, ref / s, rtol=rtol, atol=atol)


def test_fused_adamw_matches_torch():
    n = 8 * 1000
    torch.manual_seed(0)
    w0 = torch.randn(n, device="cuda")
    p = w0.to(torch.bfloat16)
    master = p.float().clone()
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    decay = torch.ones(n, device="cuda", dtype=torch.uint8)
    ref = torch.nn.Parameter(master.clone())
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    scale = torch.ones(1, device="cuda")
    for step in range(1, 4):
        g = torch.randn(n, device="cuda").to(torch.bfloat16)
        native.ops().fused_adamw(p, g, master, m, v, decay, scale, 1e-2, 0.9, 0.95, 1e-8, 0.1,
                                 1 - 0.9 ** step, 1 - 0.95 ** step)
        ref.grad = g.float()
        opt.step()
        torch.testing.assert_close(master, ref.data, rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(p.float(), ref.data, rtol=1e-2, atol=1e-2)
