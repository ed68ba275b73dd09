"""The allocation-free per-column reduction, called through its exported C symbol, against
the existing entry point that takes a caller-provided zero-filled workspace."""
import ctypes

import pytest
import torch

from lbann_b200.ops import native

pytestmark = pytest.mark.gpu

c_void_p, c_int, c_ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong


def _symbols():
    lib = native.cuda_lib()
    fn = lib.lb_column_sums_noalloc
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_void_p, c_ll, c_int, c_int, c_void_p]
    ref = lib.lb_bn_partial_sums
    ref.restype = c_int
    ref.argtypes = [c_void_p, c_void_p, c_ll, c_int, c_int, c_int, c_int, c_void_p]
    return fn, ref


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_two_calls_in_a_row_match_existing_entry_point(dtype):
    fn, ref = _symbols()
    torch.manual_seed(0)
    stream = native.stream_ptr()
    code = native.dtype_code(dtype)
    # the second call has fewer columns and other data: stale workspace contents would show
    for rows, cols in ((3001, 256), (777, 64)):
        x = torch.randn(rows, cols, device="cuda").to(dtype)
        out = torch.full((2 * cols,), float("nan"), dtype=torch.float32, device="cuda")
        assert fn(x.data_ptr(), out.data_ptr(), rows, cols, code, stream) == 0
        want = torch.zeros(2 * cols, dtype=torch.float32, device="cuda")
        assert ref(x.data_ptr(), want.data_ptr(), rows, cols, 1, code, 1, stream) == 0
        torch.cuda.synchronize()
        torch.testing.assert_close(out, want, rtol=1e-4, atol=1e-2)
        xf = x.float()
        torch.testing.assert_close(out[:cols], xf.sum(0), rtol=1e-4, atol=1e-2)
        torch.testing.assert_close(out[cols:], (xf * xf).sum(0), rtol=1e-4, atol=1e-2)
    assert native.consume_status() == 0


@pytest.mark.parametrize("rows,cols", [(130, 264), (5, 4096), (0, 64), (1, 8), (63, 520)])
def test_edge_shapes_against_fp32_sums(rows, cols):
    """Several vector blocks along the columns with a partly filled last one (264 and 520
    columns), the widest matrix the workspace serves, no rows at all, a single row, fewer
    rows than one block takes."""
    fn, _ = _symbols()
    torch.manual_seed(rows * 131 + cols)
    x = torch.randn(rows, cols, device="cuda").to(torch.bfloat16)
    out = torch.full((2 * cols,), float("nan"), dtype=torch.float32, device="cuda")
    assert fn(x.data_ptr() if rows else out.data_ptr(), out.data_ptr(), rows, cols, native.DT_BF16,
              native.stream_ptr()) == 0
    torch.cuda.synchronize()
    xf = x.float()
    torch.testing.assert_close(out[:cols], xf.sum(0), rtol=1e-4, atol=1e-2)
    torch.testing.assert_close(out[cols:], (xf * xf).sum(0), rtol=1e-4, atol=1e-2)


def test_rejects_sizes_beyond_the_workspace():
    fn, _ = _symbols()
    x = torch.zeros(2, 8192, device="cuda", dtype=torch.float16)
    out = torch.zeros(2 * 8192, dtype=torch.float32, device="cuda")
    assert fn(x.data_ptr(), out.data_ptr(), 2, 8192, native.DT_F16, native.stream_ptr()) == -2
    assert fn(x.data_ptr(), out.data_ptr(), 2, 12, native.DT_F16, native.stream_ptr()) == -1
    assert fn(x.data_ptr(), out.data_ptr(), -1, 64, native.DT_F16, native.stream_ptr()) == -1
    assert fn(x.data_ptr() + 2, out.data_ptr(), 2, 64, native.DT_F16, native.stream_ptr()) == -1
