"""The give-up path of the bounded device-side waits, driven without faulting the GPU: a self-test kernel waits on an
mbarrier nobody arrives on, with the wait limit shortened to about a millisecond.  The kernel must return, the host
must see the flag as an exception, a kernel launched while the flag is set must skip its work, and after the flag
has been read the real kernels must work as before."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_returns_and_raises_on_the_host():
    from protenix_b200 import _lib, ops

    lib = _lib.load()
    assert ops.device_error_flags() == 0
    st = torch.cuda.current_stream().cuda_stream
    out = torch.zeros(2, dtype=torch.int32, device="cuda")
    assert lib.px_set_wait_limit_cycles(2_000_000) == 0
    try:
        assert lib.px_selftest_wait_timeout(ctypes.c_void_p(out.data_ptr()), st) == 0
        assert lib.px_selftest_wait_timeout(ctypes.c_void_p(out.data_ptr() + 4), st) == 0
        with pytest.raises(RuntimeError, match="selftest"):
            ops.device_error_flags()
        assert out.tolist() == [1, 2]          # first launch gave up after the limit, second one skipped its work
        assert ops.device_error_flags() == 0   # reading clears the record
        assert lib.px_selftest_wait_timeout(ctypes.c_void_p(out.data_ptr()), st) == 0
        assert ops.device_error_flags(raise_on_error=False) == 1 << ops.KERNEL_FAMILIES.index("selftest")
    finally:
        assert lib.px_set_wait_limit_cycles(0) == 0
    # the context is intact: a tensor-core kernel runs and agrees with torch
    a = torch.randn(128, 64, 64, device="cuda").to(torch.float16)
    b = torch.randn(128, 64, 64, device="cuda").to(torch.float16)
    x = ops.trimul_contract(a, b)
    ref = torch.einsum("cik,cjk->cij", a.float(), b.float()) * ops.X_SCALE
    assert float((x.float() - ref).norm() / ref.norm()) < 1e-3
    assert ops.device_error_flags() == 0
