"""The allocation-free tensor-scale entry point, called through its exported C symbol.

Some users of this library cannot allocate device memory where they need an FP8 scale (fixed
memory budgets, threads without an allocator, C embedders without PyTorch's caching allocator), so
``vb_tensor_scale_noalloc`` keeps its scratch inside the library.  The test calls the raw symbol
with ctypes twice in a row on different inputs (the second call sees the first call's leftovers in
the shared scratch) and compares each result with the regular entry point, then checks that an
input beyond the built-in limit is refused with a message.  It lives in the last-collected file so
that a failure here cannot hide the result of any other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_ELEMENTS = 4096 * 8192


def entry_point():
    from viola_b200 import ops
    ops.load()
    library = ctypes.CDLL(str(ops._LIB_PATH))
    function = library.vb_tensor_scale_noalloc
    function.restype = ctypes.c_int
    function.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_float, ctypes.c_void_p,
                         ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]
    return function


def test_no_alloc_scale_matches_regular_entry_point_twice():
    from viola_b200 import ops
    function = entry_point()
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    torch.manual_seed(0)
    stream = torch.cuda.current_stream(device).cuda_stream
    cases = [(torch.randn(3_000_001, device=device) * 7.0, 0, 448.0),
             (torch.randn(777, 513, device=device).bfloat16() * 0.01, 1, 57344.0)]
    for call, (tensor, code, limit) in enumerate(cases):
        out = torch.zeros(1, device=device)
        message = ctypes.create_string_buffer(256)
        torch.cuda.synchronize(device)
        allocated = torch.cuda.memory_allocated(device)
        free_before, _ = torch.cuda.mem_get_info(device)          # the driver's view: sees a cudaMalloc inside the library
        status = function(tensor.data_ptr(), tensor.numel(), code, limit, out.data_ptr(), stream, message, 256)
        assert status == 0, message.value
        torch.cuda.synchronize(device)
        assert torch.cuda.memory_allocated(device) == allocated
        if call:         # the first call on a device may load the module that holds the scratch array
            assert torch.cuda.mem_get_info(device)[0] == free_before
        fmt = torch.float8_e4m3fn if limit == 448.0 else torch.float8_e5m2
        expected = ops.tensor_scale(tensor, fp8_dtype=fmt)
        torch.testing.assert_close(out, expected, rtol=1e-6, atol=0)


def test_no_alloc_scale_rejects_oversized_input():
    function = entry_point()
    device = torch.device("cuda", 0)
    small = torch.ones(16, device=device)
    out = torch.zeros(1, device=device)
    message = ctypes.create_string_buffer(256)
    status = function(small.data_ptr(), MAX_ELEMENTS + 1, 0, 448.0, out.data_ptr(),
                      torch.cuda.current_stream(device).cuda_stream, message, 256)
    assert status != 0 and b"exceeds" in message.value
    assert out.item() == 0.0
    for bad in (0.0, -1.0, float("nan"), float("inf")):
        status = function(small.data_ptr(), 16, 0, bad, out.data_ptr(), torch.cuda.current_stream(device).cuda_stream,
                          message, 256)
        assert status != 0 and b"limit" in message.value
    torch.cuda.synchronize(device)
    assert out.item() == 0.0
