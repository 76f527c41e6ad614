"""The allocation-free C entry point ``slapo_bias_act_bwd_noalloc`` gives the
same result as the torch op ``bias_act_bwd`` on two calls in a row, and
refuses shapes beyond its static scratch.  Collected last on purpose: it must
pass alone and after every other GPU test has used the device."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

_DT = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


def _lib():
    from slapo_b200.ops import native
    native.ops()  # loads the extension (and fails loudly if it is missing)
    lib = ctypes.CDLL(native.lib_path())
    fn = lib.slapo_bias_act_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int] * 4 + [ctypes.c_void_p, ctypes.c_char_p,
                                                                 ctypes.c_int]
    return fn


def _call(fn, dy, x, bias, dx, dbias, act):
    cols = x.size(-1)
    rows = x.numel() // cols
    err = ctypes.create_string_buffer(256)
    rc = fn(dy.data_ptr(), x.data_ptr(), bias.data_ptr() if bias is not None else None,
            dx.data_ptr(), dbias.data_ptr() if dbias is not None else None, rows, cols, act,
            _DT[x.dtype], torch.cuda.current_stream().cuda_stream, err, 256)
    return rc, err.value.decode()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,cols,act", [(4096, 4096, 1), (1000, 1024, 0), (37, 264, 2)])
def test_noalloc_matches_torch_op(dtype, rows, cols, act):
    from slapo_b200.ops import native
    fn = _lib()
    torch.manual_seed(0)
    for call in range(2):  # two calls in a row reuse the same static scratch
        x = torch.randn(rows, cols, device="cuda", dtype=dtype)
        dy = torch.randn(rows, cols, device="cuda", dtype=dtype)
        bias = torch.randn(cols, device="cuda", dtype=dtype)
        dx_ref, db_ref = native.ops().bias_act_bwd(dy, x, bias, act)
        dx = torch.empty_like(x)
        db = torch.empty_like(bias)
        rc, msg = _call(fn, dy, x, bias, dx, db, act)
        assert rc == 0, msg
        torch.cuda.synchronize()
        # same kernels, same launch geometry: bitwise equal
        assert torch.equal(dx, dx_ref), f"dx differs on call {call}"
        assert torch.equal(db, db_ref), f"dbias differs on call {call}"
        # and both agree with plain fp32 PyTorch
        xf = (x.float() + bias.float()).requires_grad_(True)
        ref = {0: lambda t: torch.nn.functional.gelu(t),
               1: lambda t: torch.nn.functional.gelu(t, approximate="tanh"),
               2: torch.relu}[act](xf)
        ref.backward(dy.float())
        tol = dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=2e-4, atol=2e-4)
        torch.testing.assert_close(dx.float(), xf.grad, **tol)
        # the bias gradient is the column sum of dx (fp32 oracle; sums of `rows` terms)
        scale = max(1.0, rows ** 0.5)
        torch.testing.assert_close(db.float() / scale, xf.grad.sum(0) / scale, **tol)


def test_noalloc_without_bias_grad():
    from slapo_b200.ops import native
    fn = _lib()
    x = torch.randn(512, 512, device="cuda", dtype=torch.bfloat16)
    dy = torch.randn_like(x)
    dx_ref, _ = native.ops().bias_act_bwd(dy, x, None, 1)
    dx = torch.empty_like(x)
    rc, msg = _call(fn, dy, x, None, dx, None, 1)
    assert rc == 0, msg
    torch.cuda.synchronize()
    assert torch.equal(dx, dx_ref)


def test_noalloc_rejects_oversize_and_bad_arguments():
    fn = _lib()
    t = torch.empty(8, device="cuda", dtype=torch.bfloat16)  # never touched: the call is refused
    err = ctypes.create_string_buffer(256)
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(t.data_ptr(), t.data_ptr(), None, t.data_ptr(), t.data_ptr(), 64, 16384 + 8, 1, 0,
            stream, err, 256)
    assert rc == 2 and b"exceeds the maximum" in err.value
    rc = fn(t.data_ptr(), t.data_ptr(), None, t.data_ptr(), None, 64, 12, 1, 0, stream, err, 256)
    assert rc == 1 and b"multiple of 8" in err.value
    rc = fn(None, t.data_ptr(), None, t.data_ptr(), None, 64, 16, 1, 0, stream, err, 256)
    assert rc == 1
    torch.cuda.synchronize()
