"""matmul_bias_bt forward and backward (tcgen05 path and CUDA-core path) vs the CPU oracle."""
import numpy as np
import pytest

from conftest import TOL_BF16, TOL_F32, bf16_round, rel_err, round_to, tol_of, torch_dtype

pytestmark = pytest.mark.gpu

# (M, N, K): aligned shapes run on tensor cores; N=10 / 65 and K=100 exercise ragged tiles and the fallback
SHAPES = [(128, 256, 64), (128, 128, 128), (256, 512, 256), (100, 72, 136), (384, 384, 784), (130, 10, 256),
          (257, 65, 384), (64, 1000, 100), (512, 768, 768), (1024, 3072, 768), (3, 8, 8)]


def _mk(M, N, K, dt, seed):
    rng = np.random.default_rng(seed)
    a = rng.standard_normal((M, K)).astype(np.float32)
    w = (rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32)
    b = rng.standard_normal(N).astype(np.float32)
    dy = rng.standard_normal((M, N)).astype(np.float32)
    a, w, b, dy = (round_to(dt, t) for t in (a, w, b, dy))
    return a, w, b, dy


def _dev(t, cuda, dt):
    import torch

    return torch.from_numpy(t).to(cuda).to(torch_dtype(dt))


def _status():
    import ctypes
    from mograd_b200 import _lib

    code, detail = ctypes.c_int(0), ctypes.c_int(0)
    assert _lib.load().mograd_b200_device_status(ctypes.byref(code), ctypes.byref(detail)) == 0
    return code.value


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("dt", ["bf16", "f32", "f16"])
def test_forward(cuda, oracle, M, N, K, dt):
    from mograd_b200 import dispatch as Kx

    a, w, b, _ = _mk(M, N, K, dt, M + N + K)
    want = oracle.matmul_bias_bt(a, w, b)
    y = Kx.matmul_bias_strided(_dev(a, cuda, dt), _dev(w, cuda, dt), _dev(b, cuda, dt))
    assert _status() == 0
    assert rel_err(y.float().cpu().numpy(), want) <= tol_of(dt)
    # no bias + fused ReLU
    y2 = Kx.matmul_bias_strided(_dev(a, cuda, dt), _dev(w, cuda, dt), None, act=1)
    want2 = np.maximum(oracle.matmul_bias_bt(a, w), 0)
    assert rel_err(y2.float().cpu().numpy(), want2) <= tol_of(dt)


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("dt", ["bf16", "f32", "f16"])
def test_backward(cuda, oracle, M, N, K, dt):
    from mograd_b200 import dispatch as Kx

    x, w, _, dy = _mk(M, N, K, dt, 3 * M + N + K)
    wdx, wdw, wdb = oracle.matmul_bias_bt_bwd(dy, x, w)
    dx, dw, db = Kx.matmul_bias_bt_bwd(_dev(dy, cuda, dt), _dev(x, cuda, dt), _dev(w, cuda, dt))
    assert _status() == 0
    tol = tol_of(dt)
    assert rel_err(dx.float().cpu().numpy(), wdx) <= tol
    assert rel_err(dw.float().cpu().numpy(), wdw) <= tol
    assert rel_err(db.float().cpu().numpy(), wdb) <= tol


def test_identity_and_known_values(cuda):
    """tests/test_ops.mojo:27-94 style identity / known-value products."""
    import torch
    from mograd_b200 import dispatch as Kx

    a = torch.arange(12, dtype=torch.float32, device=cuda).reshape(3, 4)
    y = Kx.matmul_bias_strided(a, torch.eye(4, device=cuda))
    assert torch.equal(y, a)
    y = Kx.matmul_bias_strided(torch.tensor([[1.0, 2], [3, 4]], device=cuda), torch.tensor([[5.0, 6], [7, 8]], device=cuda))
    assert torch.equal(y.cpu(), torch.tensor([[17.0, 23], [39, 53]]))
    ab = torch.eye(256, device=cuda).bfloat16()
    xb = torch.randn((128, 256), device=cuda).bfloat16()
    assert torch.equal(Kx.matmul_bias_strided(xb, ab), xb)  # X @ I^T on the tensor-core path is exact


def test_split_contraction_dw(cuda, oracle):
    """dW of a tall batch (contraction 8192) takes the split-contraction path; deterministic."""
    import torch
    from mograd_b200 import dispatch as Kx

    x, w, _, dy = _mk(8192, 256, 384, "bf16", 5)
    _, wdw, wdb = oracle.matmul_bias_bt_bwd(dy, x, w)
    args = (_dev(dy, cuda, "bf16"), _dev(x, cuda, "bf16"), _dev(w, cuda, "bf16"))
    _, dw1, db1 = Kx.matmul_bias_bt_bwd(*args, need_dx=False)
    _, dw2, _ = Kx.matmul_bias_bt_bwd(*args, need_dx=False)
    assert _status() == 0
    assert rel_err(dw1.float().cpu().numpy(), wdw) <= TOL_BF16
    assert rel_err(db1.float().cpu().numpy(), wdb) <= TOL_BF16
    assert torch.equal(dw1, dw2)


def test_batch_dims_collapse(cuda, oracle):
    import torch
    from mograd_b200 import dispatch as Kx

    a, w, b, _ = _mk(6 * 64, 128, 64, "bf16", 8)
    y = Kx.matmul_bias_strided(_dev(a, cuda, "bf16").view(6, 64, 64), _dev(w, cuda, "bf16"), _dev(b, cuda, "bf16"))
    assert y.shape == (6, 64, 128)
    assert rel_err(y.float().cpu().numpy().reshape(-1, 128), oracle.matmul_bias_bt(a, w, b)) <= TOL_BF16


def test_large_linearity(cuda):
    """Full-size product (16384 x 768 x 3072): linear in A, checked without a CPU GEMM."""
    import torch
    from mograd_b200 import dispatch as Kx

    g = torch.Generator(device=cuda).manual_seed(2)
    a1 = torch.randn((16384, 768), generator=g, device=cuda).bfloat16()
    w = (torch.randn((3072, 768), generator=g, device=cuda) / 28).bfloat16()
    y1 = Kx.matmul_bias_strided(a1, w).float()
    y2 = Kx.matmul_bias_strided((a1.float() * 2).bfloat16(), w).float()  # exact doubling in bf16
    assert _status() == 0
    assert torch.equal(y2, y1 * 2)
    ref = (a1[:256].float() @ w.float().T)
    assert rel_err(y1[:256].cpu().numpy(), ref.cpu().numpy()) <= TOL_BF16


@pytest.mark.parametrize("dt", ["bf16", "f32", "f16"])
@pytest.mark.parametrize("M,N,K", [(256, 384, 128), (130, 72, 200), (64, 10, 32)])
def test_extended_epilogues(cuda, oracle, M, N, K, dt):
    """Fused residual add (forward), ReLU-backward mask and gradient accumulation (dX), db inside the dW GEMM."""
    from mograd_b200 import dispatch as Kx

    rng = np.random.default_rng(M + N)
    x, w, b, dy = _mk(M, N, K, dt, 11)
    res = rng.standard_normal((M, N)).astype(np.float32)
    relu_y = np.maximum(rng.standard_normal((M, K)), 0).astype(np.float32)
    dres = rng.standard_normal((M, K)).astype(np.float32)
    res, relu_y, dres = round_to(dt, res), round_to(dt, relu_y), round_to(dt, dres)
    tol = tol_of(dt)
    y = Kx.matmul_bias_strided(_dev(x, cuda, dt), _dev(w, cuda, dt), _dev(b, cuda, dt), act=1, residual=_dev(res, cuda, dt))
    want = np.maximum(oracle.matmul_bias_bt(x, w, b), 0) + res
    assert rel_err(y.float().cpu().numpy(), want) <= tol
    wdx, wdw, wdb = oracle.matmul_bias_bt_bwd(dy, x, w)
    wdx = oracle.relu_grad(relu_y, wdx) + dres
    dx, dw, db = Kx.matmul_bias_bt_bwd(_dev(dy, cuda, dt), _dev(x, cuda, dt), _dev(w, cuda, dt),
                                       relu_y=_dev(relu_y, cuda, dt), dx_residual=_dev(dres, cuda, dt))
    assert _status() == 0
    assert rel_err(dx.float().cpu().numpy(), wdx) <= tol
    assert rel_err(dw.float().cpu().numpy(), wdw) <= tol
    assert rel_err(db.float().cpu().numpy(), wdb) <= tol


def test_db_inside_dw_gemm_tall(cuda, oracle):
    """Bias gradient accumulated from the dY tiles of the split dW GEMM (contraction 16384)."""
    from mograd_b200 import dispatch as Kx

    x, w, _, dy = _mk(16384, 384, 256, "bf16", 21)
    _, wdw, wdb = oracle.matmul_bias_bt_bwd(dy, x, w)
    args = (_dev(dy, cuda, "bf16"), _dev(x, cuda, "bf16"), _dev(w, cuda, "bf16"))
    _, dw, db = Kx.matmul_bias_bt_bwd(*args, need_dx=False)
    _, dw2, db2 = Kx.matmul_bias_bt_bwd(*args, need_dx=False)
    assert _status() == 0
    assert rel_err(dw.float().cpu().numpy(), wdw) <= TOL_BF16
    assert rel_err(db.float().cpu().numpy(), wdb) <= TOL_BF16
    import torch

    assert torch.equal(db, db2) and torch.equal(dw, dw2)


@pytest.mark.parametrize("M,N,K", [(1024, 2560, 2048), (4096, 2048, 1024), (2048, 4096, 1024), (2200, 2312, 2056)])
def test_cta_pair_kernel(cuda, oracle, M, N, K):
    """Shapes large enough for the two-CTA (256 x 256 tile) kernel, in all three operand-major combinations,
    including ragged edges where the second CTA's rows fall partly or wholly outside the matrix."""
    from mograd_b200 import dispatch as Kx

    x, w, b, dy = _mk(M, N, K, "bf16", M + K)
    res = bf16_round(np.random.default_rng(1).standard_normal((M, N)).astype(np.float32))
    y = Kx.matmul_bias_strided(_dev(x, cuda, "bf16"), _dev(w, cuda, "bf16"), _dev(b, cuda, "bf16"), act=1,
                               residual=_dev(res, cuda, "bf16"))
    assert _status() == 0
    assert rel_err(y.float().cpu().numpy(), np.maximum(oracle.matmul_bias_bt(x, w, b), 0) + res) <= TOL_BF16
    wdx, wdw, _ = oracle.matmul_bias_bt_bwd(dy, x, w, need_db=False)
    dx, dw, _ = Kx.matmul_bias_bt_bwd(_dev(dy, cuda, "bf16"), _dev(x, cuda, "bf16"), _dev(w, cuda, "bf16"), need_db=False)
    assert _status() == 0
    assert rel_err(dx.float().cpu().numpy(), wdx) <= TOL_BF16
    assert rel_err(dw.float().cpu().numpy(), wdw) <= TOL_BF16


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(256, 384, 128), (300, 1000, 72), (128, 64, 64), (1000, 3072, 256)])
def test_relu_bit_mask_pair(cuda, oracle, M, N, K):
    """Forward emits one bit per output (Y > 0); backward masked by the bits equals backward masked by Y itself."""
    import torch
    from mograd_b200 import dispatch as Kd

    rng = np.random.default_rng(M + N + K)
    a = bf16_round(rng.standard_normal((M, K)).astype(np.float32))
    w = bf16_round((rng.standard_normal((N, K)) / np.sqrt(K)).astype(np.float32))
    b = bf16_round(rng.standard_normal(N).astype(np.float32) * 0.1)
    dev = lambda t: torch.from_numpy(t).to(cuda).bfloat16()
    bits = torch.full((M, (N + 31) // 32), -1, dtype=torch.int32, device=cuda)
    y = Kd.matmul_bias_strided(dev(a), dev(w), dev(b), act=1, relu_bits=bits)
    y_ref = Kd.matmul_bias_strided(dev(a), dev(w), dev(b), act=1)
    assert torch.equal(y, y_ref)
    # the bits are exactly (y > 0), padding bits of the last word are clear
    yy = (y.float().cpu().numpy() > 0)
    pad = np.zeros((M, bits.shape[1] * 32), dtype=bool)
    pad[:, :N] = yy
    want_words = np.packbits(pad.reshape(M, -1, 32), axis=-1, bitorder="little").view(np.uint32).reshape(M, -1)
    assert np.array_equal(bits.cpu().numpy().view(np.uint32), want_words)
    # backward of the next layer (contraction over its outputs), masked either way
    N2 = 96
    w2 = bf16_round((rng.standard_normal((N2, N)) / np.sqrt(N)).astype(np.float32))
    dy = bf16_round(rng.standard_normal((M, N2)).astype(np.float32))
    res = bf16_round(rng.standard_normal((M, N)).astype(np.float32))
    dx1, _, _ = Kd.matmul_bias_bt_bwd(dev(dy), y, dev(w2), need_dw=False, need_db=False, relu_y=y, dx_residual=dev(res))
    dx2, _, _ = Kd.matmul_bias_bt_bwd(dev(dy), y, dev(w2), need_dw=False, need_db=False, relu_bits=bits,
                                      dx_residual=dev(res))
    assert torch.equal(dx1, dx2)
    want = (dy.astype(np.float64) @ w2.astype(np.float64)) * yy + res
    assert rel_err(dx2.float().cpu().numpy(), want) <= TOL_BF16


@pytest.mark.gpu
def test_relu_bit_mask_rejected_off_the_tensor_core_path(cuda):
    import torch
    from mograd_b200 import dispatch as Kd
    from mograd_b200._lib import KernelError

    a = torch.zeros((8, 16), device=cuda)
    w = torch.zeros((40, 16), device=cuda)
    bits = torch.zeros((8, 2), dtype=torch.int32, device=cuda)
    with pytest.raises(KernelError):
        Kd.matmul_bias_strided(a, w, None, act=1, relu_bits=bits)  # fp32 has no bit-mask path
