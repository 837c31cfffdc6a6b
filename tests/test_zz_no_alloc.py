"""The allocation-free column sum, called through its exported C symbol.

Some users of the library cannot allocate device memory where they call it (a fixed arena owned by
a serving process, a real-time loop, a host application that forbids allocation after start-up).
For them ``wx_column_sum_bf16_noalloc`` keeps its fp32 scratch in a device array inside the
library. This test calls it twice in a row (the second call must not see the first call's sums in
the shared scratch) and compares with the regular, allocating entry point. It is collected last so
that a failure here cannot hide any other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, x, out):
    stream = torch.cuda.current_stream().cuda_stream
    return lib.wx_column_sum_bf16_noalloc(ctypes.c_void_p(x.data_ptr()), x.stride(0), ctypes.c_void_p(out.data_ptr()),
                                          x.shape[0], x.shape[1], ctypes.c_void_p(stream))


def test_no_alloc_column_sum_matches_regular_entry_point_twice():
    from wallx_b200.ops import _ext, no_alloc

    lib = no_alloc.load()
    C = _ext.get()
    torch.manual_seed(0)
    for rows, cols in [(1000, 2048), (777, 3456)]:  # two calls in a row, the second wider than the first
        x = torch.randn(rows, cols, device="cuda").to(torch.bfloat16)
        out = torch.full((cols,), 7.0, device="cuda", dtype=torch.bfloat16)
        rc = _call(lib, x, out)
        assert rc == 0, lib.wx_noalloc_strerror(rc).decode()
        expect = C.column_sum(x)
        torch.cuda.synchronize()
        fp32 = x.float().sum(0)
        assert torch.allclose(out.float(), expect.float(), atol=0.3, rtol=2e-2)
        assert torch.allclose(out.float(), fp32, atol=0.3, rtol=2e-2)
    # same input again: the scratch kept the last sums and must have been cleared
    out2 = torch.empty_like(out)
    assert _call(lib, x, out2) == 0
    torch.cuda.synchronize()
    assert torch.equal(out2, out) or torch.allclose(out2.float(), out.float(), atol=0.3, rtol=2e-2)


def test_no_alloc_odd_shapes_pitched_rows_and_empty_input():
    """The scalar path (odd width, odd pitch), a pitched view (row pitch larger than the width) and zero rows."""
    from wallx_b200.ops import no_alloc

    lib = no_alloc.load()
    torch.manual_seed(1)
    base = torch.randn(5, 9, device="cuda").to(torch.bfloat16)
    x = base[:, :7]  # 5 x 7, pitch 9: odd width and odd pitch
    out = torch.full((7,), 3.0, device="cuda", dtype=torch.bfloat16)
    assert _call(lib, x, out) == 0
    torch.cuda.synchronize()
    assert torch.allclose(out.float(), x.float().sum(0), atol=2e-2, rtol=2e-2)
    wide = torch.randn(300, 64, device="cuda").to(torch.bfloat16)
    v = wide[:, 8:40]  # 300 x 32 view with pitch 64 (paired loads, pitch > width)
    out = torch.empty(32, device="cuda", dtype=torch.bfloat16)
    assert _call(lib, v, out) == 0
    torch.cuda.synchronize()
    assert torch.allclose(out.float(), v.float().sum(0), atol=0.2, rtol=2e-2)
    empty = torch.empty(0, 8, device="cuda", dtype=torch.bfloat16)
    out = torch.full((8,), 5.0, device="cuda", dtype=torch.bfloat16)
    assert lib.wx_column_sum_bf16_noalloc(ctypes.c_void_p(wide.data_ptr()), 8, ctypes.c_void_p(out.data_ptr()), 0, 8,
                                          ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)) == 0
    torch.cuda.synchronize()
    assert empty.shape[0] == 0 and torch.equal(out.float(), torch.zeros(8, device="cuda"))  # a sum over no rows is zero


def test_no_alloc_rejects_too_wide_and_bad_arguments():
    from wallx_b200.ops import no_alloc

    lib = no_alloc.load()
    x = torch.zeros(2, 8, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(8, device="cuda", dtype=torch.bfloat16)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.wx_column_sum_bf16_noalloc(ctypes.c_void_p(x.data_ptr()), no_alloc.MAX_COLS + 8, ctypes.c_void_p(out.data_ptr()),
                                        2, no_alloc.MAX_COLS + 8, stream)
    assert rc == -2 and b"65536" in lib.wx_noalloc_strerror(rc)
    assert lib.wx_column_sum_bf16_noalloc(None, 8, ctypes.c_void_p(out.data_ptr()), 2, 8, stream) == -1
