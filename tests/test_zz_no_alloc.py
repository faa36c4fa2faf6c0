"""The allocation-free RMSNorm-backward entry point, called through its exported C symbol.

Some users of this library run where device allocation is not allowed (a pre-planned arena, a
loop that must not synchronise the device).  For them the library exports one plain C function
whose workspace is a fixed array inside the library.  This test calls that symbol with ctypes
and checks it against the regular entry point, twice in a row with different data, so that a
result depending on what the previous call left in the shared workspace would show.
"""
import ctypes

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


def test_no_alloc_rmsnorm_bwd_matches_regular_entry_point():
    from odc_b200 import _ext
    ext = _ext.load()
    fn = _lib()
    torch.cuda.set_device(0)
    for call, (rows, cols) in enumerate([(777, 2048), (300, 5120)]):
        g = torch.Generator(device="cuda").manual_seed(100 + call)
        x = torch.randn(rows, cols, device="cuda", generator=g).bfloat16()
        w = (1 + 0.1 * torch.randn(cols, device="cuda", generator=g)).bfloat16()
        dy = torch.randn(rows, cols, device="cuda", generator=g).bfloat16()
        _, rstd = ext.rmsnorm_fwd(x, w, 1e-5)
        dx_ref, dw_ref = ext.rmsnorm_bwd(dy, x, w, rstd)
        dx = torch.empty_like(x)           # outputs are the caller's
        dw = torch.full((cols,), float("nan"), device="cuda")
        before = torch.cuda.memory_allocated()
        rc, msg = _call(fn, dy, x, w, rstd, dx, dw, rows, cols)
        torch.cuda.synchronize()
        assert rc == 0, msg
        assert torch.cuda.memory_allocated() == before
        torch.testing.assert_close(dx.float(), dx_ref.float(), rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(dw, dw_ref, rtol=2e-2, atol=2e-2)


def test_no_alloc_rejects_oversized_rows():
    fn = _lib()
    t = torch.zeros(8, device="cuda")
    rc, msg = _call(fn, t, t, t, t, t, t, 1, 8192 + 8)
    assert rc != 0 and "exceeds" in msg
    rc, msg = _call(fn, t, t, t, t, t, t, 1, 12)
    assert rc != 0 and "multiple of 8" in msg
