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
