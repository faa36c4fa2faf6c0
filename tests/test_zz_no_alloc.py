"""The allocation-free RMSNorm-backward entry point, called through its exported C symbol.

Some users of this library run where device allocation is not allowed (a pre-planned arena, a
loop that must not synchronise the device).  For them the library exports one plain C function
whose workspace is a fixed array inside the library.  This test calls that symbol with ctypes
and checks it against the regular entry point and against the fp32 statement of the op, on
calls in a row with different data and widths, so that a result depending on what the previous
call left in the shared workspace would show.
"""
import ctypes
import gc

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from odc_b200 import _ext
    _ext.load()
    lib = ctypes.CDLL(_ext.so_path())
    fn = lib.odc_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int]
    return fn


def _call(fn, dy, x, w, rstd, dx, dw, rows, cols):
    err = ctypes.create_string_buffer(256)
    rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(), rows, cols,
            torch.cuda.current_stream().cuda_stream, err, 256)
    return rc, err.value.decode()


def _fp32_reference(dy, x, w, eps):
    xf = x.float().requires_grad_(True)
    wf = w.float().requires_grad_(True)
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * wf
    y.backward(dy.float())
    return xf.grad, wf.grad


def test_no_alloc_rmsnorm_bwd_matches_regular_entry_point():
    from odc_b200 import _ext
    ext = _ext.load()
    fn = _lib()
    torch.cuda.set_device(0)
    # (300, 8192) is the widest row accepted: every thread then holds its fourth register slice
    for call, (rows, cols) in enumerate([(777, 2048), (300, 5120), (300, 8192), (5, 2048)]):
        g = torch.Generator(device="cuda").manual_seed(100 + call)
        x = torch.randn(rows, cols, device="cuda", generator=g).bfloat16()
        w = (1 + 0.1 * torch.randn(cols, device="cuda", generator=g)).bfloat16()
        dy = torch.randn(rows, cols, device="cuda", generator=g).bfloat16()
        _, rstd = ext.rmsnorm_fwd(x, w, 1e-5)
        dx_ref, dw_ref = ext.rmsnorm_bwd(dy, x, w, rstd)
        dx32, dw32 = _fp32_reference(dy, x, w, 1e-5)
        dx = torch.empty_like(x)           # outputs are the caller's
        dw = torch.full((cols,), float("nan"), device="cuda")
        gc.collect()                       # nothing of the reference computation is freed between the two readings
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before, _ = torch.cuda.mem_get_info()
        rc, msg = _call(fn, dy, x, w, rstd, dx, dw, rows, cols)
        torch.cuda.synchronize()
        assert rc == 0, msg
        assert torch.cuda.memory_allocated() <= before
        if call > 0:  # the first launch in a process may make the CUDA runtime load the library's GPU code
            free_after, _ = torch.cuda.mem_get_info()
            assert free_after >= free_before, "the device's free memory shrank across an allocation-free call"
        torch.testing.assert_close(dx.float(), dx_ref.float(), rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(dw, dw_ref.float(), rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(dx.float(), dx32, rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(dw, dw32, rtol=2e-2, atol=rows ** 0.5 * 2e-2)


def test_no_alloc_zero_rows_writes_zero_dw():
    fn = _lib()
    cols = 2048
    x = torch.empty(0, cols, device="cuda", dtype=torch.bfloat16)
    pad = torch.zeros(8, device="cuda", dtype=torch.bfloat16)  # valid addresses for the empty operands
    w = torch.ones(cols, device="cuda", dtype=torch.bfloat16)
    rstd = torch.zeros(1, device="cuda")
    dw = torch.full((cols,), float("nan"), device="cuda")
    rc, msg = _call(fn, pad, pad, w, rstd, pad, dw, 0, cols)
    torch.cuda.synchronize()
    assert rc == 0, msg
    assert x.numel() == 0 and torch.count_nonzero(dw).item() == 0


def test_no_alloc_rejects_oversized_rows():
    fn = _lib()
    t = torch.zeros(8, device="cuda")
    rc, msg = _call(fn, t, t, t, t, t, t, 1, 8192 + 8)
    assert rc != 0 and "exceeds" in msg
    rc, msg = _call(fn, t, t, t, t, t, t, 1, 12)
    assert rc != 0 and "multiple of 8" in msg


def test_no_alloc_refuses_misaligned_pointers():
    """A sliced tensor starts 2 bytes off a 16-byte boundary: refused with an error code, nothing is launched."""
    fn = _lib()
    cols = 2048
    buf = torch.zeros(4 * cols + 8, device="cuda", dtype=torch.bfloat16)
    ok = buf[: 2 * cols].view(2, cols)
    off = buf[1: 1 + 2 * cols].view(2, cols)   # data_ptr is 2 bytes past an aligned address
    w = torch.ones(cols, device="cuda", dtype=torch.bfloat16)
    rstd = torch.ones(2, device="cuda")
    dw = torch.zeros(cols, device="cuda")
    for args in ((off, ok, w, rstd, ok, dw), (ok, off, w, rstd, ok, dw), (ok, ok, w, rstd, off, dw)):
        rc, msg = _call(fn, *args, 2, cols)
        assert rc != 0 and "aligned" in msg
    torch.cuda.synchronize()
