"""dyninfer_cuda_argmax_static: the argmax entry point that allocates nothing.

Collected last (file name) so that it also runs after every other GPU test has used the library;
it must pass alone as well. Every call goes through the C ABI and is compared with the existing
dyninfer_cuda_argmax on the same device vector, for two calls in a row.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptr(t):
    return C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _both(lib, v):
    """(existing entry point, no-alloc entry point) on one device vector."""
    n = v.numel()
    out_a = torch.full((1,), -1, dtype=torch.int64, device=v.device)
    out_b = torch.full((1,), -1, dtype=torch.int64, device=v.device)
    scratch = torch.empty(lib.dyninfer_cuda_argmax_scratch_bytes(n), dtype=torch.uint8, device=v.device)
    rc = lib.dyninfer_cuda_argmax(_ptr(v), n, _ptr(out_a), _ptr(scratch), _stream())
    assert rc == 0, lib.dyninfer_cuda_last_error().decode()
    rc = lib.dyninfer_cuda_argmax_static(_ptr(v), n, _ptr(out_b), _stream())
    assert rc == 0, lib.dyninfer_cuda_last_error().decode()
    torch.cuda.synchronize()
    return int(out_a.item()), int(out_b.item())


def test_matches_existing_entry_point_twice_in_a_row(native_lib):
    lib = native_lib
    rng = np.random.default_rng(11)
    # two calls in a row with different lengths: the second must not see the first one's partials
    first = rng.normal(size=151936).astype(np.float32)
    second = rng.normal(size=5000).astype(np.float32)
    second[4097] = 9.0
    for host in (first, second):
        a, b = _both(lib, torch.from_numpy(host).cuda())
        assert a == b == int(np.argmax(host))


@pytest.mark.parametrize("n", [1, 255, 4096, 4097, 151936, 1 << 20])
def test_sizes_ties_and_non_finite(native_lib, n):
    lib = native_lib
    rng = np.random.default_rng(n)
    v = rng.normal(size=n).astype(np.float32)
    a, b = _both(lib, torch.from_numpy(v).cuda())
    assert a == b == int(np.argmax(v))
    if n >= 255:
        v[[n // 3, n // 2, n - 1]] = 60.0            # ties: the lowest index wins
        v[5] = np.nan                                # NaN never wins
        a, b = _both(lib, torch.from_numpy(v).cuda())
        assert a == b == n // 3
    v[:] = -np.inf                                   # nothing finite: index 0
    a, b = _both(lib, torch.from_numpy(v).cuda())
    assert a == b == 0


def test_largest_supported_and_rejection(native_lib):
    lib = native_lib
    max_n = lib.dyninfer_cuda_argmax_static_max_n()
    assert max_n == 1024 * 4096
    v = torch.zeros(max_n + 1, dtype=torch.float32, device="cuda")
    v[max_n - 1] = 1.0
    out = torch.full((1,), -1, dtype=torch.int64, device="cuda")
    assert lib.dyninfer_cuda_argmax_static(_ptr(v), max_n, _ptr(out), _stream()) == 0
    torch.cuda.synchronize()
    assert int(out.item()) == max_n - 1
    rc = lib.dyninfer_cuda_argmax_static(_ptr(v), max_n + 1, _ptr(out), _stream())
    assert rc != 0
    msg = lib.dyninfer_cuda_last_error().decode()
    assert "exceeds" in msg and str(max_n) in msg
    assert lib.dyninfer_cuda_argmax_static(_ptr(v), 0, _ptr(out), _stream()) != 0
