"""Allocation-free column sum: same result as the workspace-taking entry point, twice in a row."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _fn():
    from fairscale_b200 import _native

    lib = _native.lib()
    f = lib.fsb_colsum_static
    f.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    f.restype = ctypes.c_int
    err = lib.fsb_colsum_static_strerror
    err.argtypes = [ctypes.c_int]
    err.restype = ctypes.c_char_p
    return lib, f, err


def test_colsum_static_matches_workspace_variant_twice():
    from fairscale_b200.ops.reduce import column_sum

    lib, f, err = _fn()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    torch.manual_seed(0)
    assert lib.fsb_colsum_static_max_h() == 8192
    # the second call is smaller than the first, so stale partials of the first stay in the shared array
    for rows, H in [(4096, 4096), (333, 1024)]:
        x = torch.randn(rows, H, device=dev, dtype=torch.bfloat16)
        want = column_sum(x)
        got = torch.empty(H, device=dev, dtype=torch.bfloat16)
        stream = torch.cuda.current_stream(dev).cuda_stream
        code = f(x.data_ptr(), rows, H, got.data_ptr(), stream)
        assert code == 0, err(code).decode()
        torch.cuda.synchronize(dev)
        torch.testing.assert_close(got.float(), want.float(), atol=0, rtol=0)  # same kernels, same order of sums
        oracle = x.float().sum(0)
        torch.testing.assert_close(got.float(), oracle, atol=0.5, rtol=2e-2)


def test_colsum_static_rejects_sizes_beyond_the_limit():
    lib, f, err = _fn()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    x = torch.zeros(8, 8200, device=dev, dtype=torch.bfloat16)
    out = torch.zeros(8200, device=dev, dtype=torch.bfloat16)
    code = f(x.data_ptr(), 8, 8200, out.data_ptr(), torch.cuda.current_stream(dev).cuda_stream)
    assert code == -2 and b"8192" in err(code)
    assert f(x.data_ptr(), 8, 12, out.data_ptr(), torch.cuda.current_stream(dev).cuda_stream) == -1
