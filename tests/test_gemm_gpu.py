"""tcgen05 GEMM against an fp32 PyTorch matmul of the same operands."""
import pytest
import torch

from slapo_b200.ops import native
from slapo_b200.ops.functional import _act_ref

pytestmark = pytest.mark.gpu


def _ops():
    assert native.available(), native.load_error()
    return native.ops()


def _run(M, N, K, a_mn, b_mn, dtype=torch.bfloat16, bias=False, act=-1):
    torch.manual_seed(M * 7 + N * 3 + K)
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda", dtype=dtype)
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda", dtype=dtype)
    bias_t = torch.randn(N, device="cuda", dtype=dtype) if bias else None
    c = _ops().gemm(a, b, bias_t, act, a_mn, b_mn)
    assert _ops().device_status() == 0, "a bounded wait inside the kernel ran out"
    af = a.float().t() if a_mn else a.float()
    bf = b.float() if b_mn else b.float().t()
    ref = af @ bf
    if bias:
        ref = ref + bias_t.float()
    if act >= 0:
        ref = _act_ref(ref, {0: "gelu", 1: "gelu_new", 2: "relu"}[act])
    scale = max(1.0, K ** 0.5)
    torch.testing.assert_close(c.float() / scale, ref / scale, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 192), (384, 128, 1024),
                                   (200, 72, 136), (1000, 1000, 520)])
def test_gemm_layouts(shape, a_mn, b_mn):
    M, N, K = shape
    if a_mn and M % 8:
        pytest.skip("M-major A needs M % 8 == 0")
    _run(M, N, K, a_mn, b_mn)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("act", [-1, 0, 1, 2])
def test_gemm_epilogue(dtype, act):
    _run(512, 1024, 256, False, False, dtype, bias=True, act=act)


def test_gemm_large_persistent():
    # more tiles than SMs: exercises the persistent loop and both accumulators
    _run(4096, 4096, 1024, False, False)
    _run(2048, 3072, 2048, False, True)
    _run(4096, 1024, 4096, True, True)


# ---------------------------------------------------------------------- #
# CTA-pair kernel (cta_group::2), split-K, second output, and the linear layer built on them
def _run_pair(M, N, K, a_mn, b_mn, split=False, bias=False, act=-1, pre=False,
              dtype=torch.bfloat16):
    torch.manual_seed(M + 3 * N + 7 * K)
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda", dtype=dtype)
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda", dtype=dtype)
    bias_t = torch.randn(N, device="cuda", dtype=dtype) if bias else None
    pre_t = torch.empty(M, N, device="cuda", dtype=dtype) if pre else None
    c = _ops().gemm_out(a, b, bias_t, act, a_mn, b_mn, None, pre_t, 2, split)
    assert _ops().device_status() == 0, "a bounded wait inside the kernel ran out"
    ref = (a.float().t() if a_mn else a.float()) @ (b.float() if b_mn else b.float().t())
    if bias:
        ref = ref + bias_t.float()
    scale = max(1.0, K ** 0.5)
    if pre:
        torch.testing.assert_close(pre_t.float() / scale, ref / scale, rtol=2e-2, atol=2e-2)
    if act >= 0:
        ref = _act_ref(ref, {0: "gelu", 1: "gelu_new", 2: "relu"}[act])
    torch.testing.assert_close(c.float() / scale, ref / scale, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("shape", [(256, 256, 64), (512, 128, 1024), (384, 136, 136),
                                   (1000, 1000, 520), (264, 72, 64), (4096, 384, 1024)])
def test_pair_gemm_layouts_and_edges(shape, a_mn, b_mn):
    M, N, K = shape
    _run_pair(M, N, K, a_mn, b_mn)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("act", [-1, 0, 1, 2])
def test_pair_gemm_epilogue_and_second_output(dtype, act):
    _run_pair(512, 1024, 256, False, False, bias=True, act=act, pre=True, dtype=dtype)
    _run_pair(520, 264, 256, False, False, bias=True, act=act, pre=True, dtype=dtype)  # edge tiles


def test_pair_gemm_split_k_leaves_its_scratch_clean():
    # weight-gradient shapes: few tiles, long contraction; twice, so that a dirty workspace or
    # counter of the first launch would show in the second
    for _ in range(2):
        _run_pair(1024, 512, 16384, True, True, split=True)
        _run_pair(520, 264, 8192, True, True, split=True, bias=True)
    assert _ops().gemm2_splits(1024, 512, 16384) > 1


@pytest.mark.parametrize("act", [None, "gelu", "relu"])
@pytest.mark.parametrize("bias", [True, False])
def test_linear_forward_and_backward(act, bias):
    from slapo_b200.ops import functional as NF

    torch.manual_seed(3)
    x = torch.randn(4, 160, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(512, 256, device="cuda", dtype=torch.bfloat16) * 0.05).requires_grad_(True)
    b = torch.randn(512, device="cuda", dtype=torch.bfloat16).requires_grad_(True) if bias else None
    g = torch.randn(4, 160, 512, device="cuda", dtype=torch.bfloat16)
    y = NF.linear(x, w, b, act)
    y.backward(g)
    xf, wf = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    bf = b.detach().float().requires_grad_(True) if bias else None
    ref = torch.nn.functional.linear(xf, wf, bf)
    if act is not None:
        ref = _act_ref(ref, act)
    ref.backward(g.float())
    torch.testing.assert_close(y.float(), ref, rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(x.grad.float(), xf.grad, rtol=3e-2, atol=5e-2)
    torch.testing.assert_close(w.grad.float() / 8, wf.grad / 8, rtol=3e-2, atol=5e-2)
    if bias:
        torch.testing.assert_close(b.grad.float() / 8, bf.grad / 8, rtol=3e-2, atol=5e-2)
    assert _ops().device_status() == 0


def test_adopted_linear_modules_run_the_native_gemm():
    from torch import nn

    from slapo_b200.ops.linear import Linear, adopt_native_linears

    torch.manual_seed(4)
    model = nn.Sequential(nn.Linear(256, 512), nn.GELU(), nn.Linear(512, 256)).cuda().bfloat16()
    assert adopt_native_linears(model) == 2 and isinstance(model[0], Linear)
    x = torch.randn(384, 256, device="cuda", dtype=torch.bfloat16)
    before = native.launch_count()
    model(x).float().sum().backward()
    # 2 forward GEMMs + 2 weight gradients + 1 input gradient (+ bias column sums)
    assert native.launch_count() - before >= 5
    assert model[0].weight.grad is not None and _ops().device_status() == 0


def test_colsum_matches_fp32():
    x = torch.randn(3000, 1024, device="cuda", dtype=torch.bfloat16)
    torch.testing.assert_close(_ops().colsum(x).float(), x.float().sum(0), rtol=2e-2, atol=0.5)
    view = x[:, :512]            # row stride larger than the width
    torch.testing.assert_close(_ops().colsum(view).float(), view.float().sum(0), rtol=2e-2, atol=0.5)


def test_linear_with_in_out_weight_layout():
    """GPT-2's Conv1D layout (weight [in, out]): forward and both gradients on the native GEMM."""
    from slapo_b200.ops import functional as NF

    torch.manual_seed(5)
    x = torch.randn(3, 128, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(256, 768, device="cuda", dtype=torch.bfloat16) * 0.05).requires_grad_(True)
    b = torch.randn(768, device="cuda", dtype=torch.bfloat16).requires_grad_(True)
    g = torch.randn(3, 128, 768, device="cuda", dtype=torch.bfloat16)
    before = native.launch_count()
    y = NF.linear_t(x, w, b)
    y.backward(g)
    assert native.launch_count() - before >= 4
    xf, wf, bf = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    ref = xf @ wf + bf
    ref.backward(g.float())
    torch.testing.assert_close(y.float(), ref, rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(x.grad.float(), xf.grad, rtol=3e-2, atol=5e-2)
    torch.testing.assert_close(w.grad.float() / 8, wf.grad / 8, rtol=3e-2, atol=5e-2)
    torch.testing.assert_close(b.grad.float() / 8, bf.grad / 8, rtol=3e-2, atol=5e-2)
    assert _ops().device_status() == 0
