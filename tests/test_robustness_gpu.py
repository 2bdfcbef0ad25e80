"""Bounded device-side waits: a wait that runs out ends as a status code on the host, and the library keeps working."""
import ctypes

import numpy as np
import pytest

from conftest import TOL_BF16, bf16_round, rel_err

pytestmark = pytest.mark.gpu


def test_wait_that_runs_out_sets_status_and_library_stays_usable(cuda, oracle):
    import torch
    from mograd_b200 import _lib
    from mograd_b200 import dispatch as K

    assert _lib.device_status() == (0, 0)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _lib.call("mograd_b200_selftest_wait_expiry", 1000, stream)  # nothing ever completes the barrier: 1 ms, then out
    torch.cuda.synchronize()
    code, detail = _lib.device_status()
    assert code == 901
    assert 1000 <= detail < 100000  # microseconds the wait lasted before it gave up
    assert _lib.device_status() == (0, 0)  # the read cleared it
    # the host-facing check turns the same condition into an exception
    _lib.call("mograd_b200_selftest_wait_expiry", 500, stream)
    with pytest.raises(_lib.KernelError):
        _lib.check_device_status("test")
    # and the context is intact: a tensor-core GEMM right after gives the oracle's result
    rng = np.random.default_rng(0)
    a = bf16_round(rng.standard_normal((256, 512)).astype(np.float32))
    w = bf16_round((rng.standard_normal((384, 512)) / 22).astype(np.float32))
    y = K.matmul_bias_strided(torch.from_numpy(a).to(cuda).bfloat16(), torch.from_numpy(w).to(cuda).bfloat16())
    assert rel_err(y.float().cpu().numpy(), oracle.matmul_bias_bt(a, w)) <= TOL_BF16
    assert _lib.device_status() == (0, 0)


def test_selftest_rejects_limits_out_of_range():
    from mograd_b200 import _lib

    lib = _lib.load()
    assert lib.mograd_b200_selftest_wait_expiry(0, None) == _lib.EINVAL
    assert lib.mograd_b200_selftest_wait_expiry(10_000_000, None) == _lib.EINVAL
