import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def rel_err(got, want):
    """max |got - want| / max |want| (NaN anywhere -> inf), the metric every parity test uses."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    if got.shape != want.shape:
        raise AssertionError(f"shape mismatch {got.shape} vs {want.shape}")
    if not np.all(np.isfinite(got)):
        return float("inf")
    denom = max(float(np.max(np.abs(want))), 1e-30)
    return float(np.max(np.abs(got - want))) / denom


# Tolerances: fp32 paths rel <= 1e-4; bf16 paths
# max-abs-err / max-abs-ref <= 2e-2 against the fp32/f64 CPU result.
TOL_F32 = 1e-4
TOL_BF16 = 2e-2
# float16 storage: the reference's own gate for its half-precision tensor-core kernels
# (tests/kernels/attention/mma.mojo:423-424, f16 backward 8e-3)
TOL_F16 = 8e-3


def tol_of(dt):
    return {"f32": TOL_F32, "bf16": TOL_BF16, "f16": TOL_F16}[dt]


def torch_dtype(dt):
    import torch

    return {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[dt]


def round_to(dt, x):
    """float32 numpy array rounded through the storage type dt (identity for f32)."""
    x = np.asarray(x, dtype=np.float32)
    if dt == "bf16":
        return bf16_round(x)
    if dt == "f16":
        return x.astype(np.float16).astype(np.float32)
    return x


@pytest.fixture(scope="session")
def oracle():
    import oracle as orc

    orc.build()
    return orc


@pytest.fixture(scope="session")
def cuda():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import mograd_b200

    mograd_b200.load()  # fail loudly if the kernel library is missing
    return torch.device("cuda:0")


def bf16_round(x):
    """numpy float32 -> bf16 (nearest even) -> float32."""
    import oracle as orc

    return orc.round_bf16(np.asarray(x, dtype=np.float32))
