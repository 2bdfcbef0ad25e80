"""Attention forward / backward (tcgen05 path and CUDA-core path) vs the f64 CPU oracle."""
import ctypes
import math

import numpy as np
import pytest

from conftest import TOL_BF16, TOL_F32, bf16_round, rel_err, round_to, tol_of, torch_dtype

pytestmark = pytest.mark.gpu


def _status():
    from mograd_b200 import _lib

    code, detail = ctypes.c_int(0), ctypes.c_int(0)
    assert _lib.load().mograd_b200_device_status(ctypes.byref(code), ctypes.byref(detail)) == 0
    return code.value


def _mk(B, S, H, D, dt, seed):
    rng = np.random.default_rng(seed)
    q, k, v = (rng.standard_normal((B, S, H, D)).astype(np.float32) for _ in range(3))
    dy = rng.standard_normal((B, H, S, D)).astype(np.float32)
    q, k, v, dy = (round_to(dt, t) for t in (q, k, v, dy))
    return q, k, v, dy


def _run(cuda, q, k, v, dy, dt, causal, mask=None):
    import torch
    from mograd_b200 import dispatch as K

    tdt = torch_dtype(dt)
    dev = lambda t: None if t is None else torch.from_numpy(t).to(cuda).to(tdt)
    qd, kd, vd, dyd, md = dev(q), dev(k), dev(v), dev(dy), dev(mask)
    o, lse = K.flash_attn_fwd_dispatch(qd, kd, vd, md, None, causal, mask is not None)
    dq, dk, dv = K.flash_attn_bwd_dispatch(dyd, o, qd, kd, vd, md, lse, None, causal, mask is not None)
    assert _status() == 0
    f = lambda t: t.float().cpu().numpy()
    return f(o), f(lse), f(dq), f(dk), f(dv)


# (B, S, H, D): tensor-core shapes (D 64 / 128; S multiple of 128, ragged, single tile, many tiles)
TC_SHAPES = [(1, 128, 1, 64), (1, 128, 1, 128), (2, 256, 3, 64), (1, 384, 2, 128), (1, 200, 2, 64), (1, 80, 1, 128),
             (2, 1024, 2, 64), (1, 1024, 1, 128), (1, 300, 2, 128), (1, 600, 1, 128), (1, 520, 1, 64)]


@pytest.mark.parametrize("B,S,H,D", TC_SHAPES)
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("dt", ["bf16", "f16"])
def test_tensor_core_path(cuda, oracle, B, S, H, D, causal, dt):
    """bf16 gate 2e-2; float16 gate 8e-3, the reference's own for its half tensor-core kernels
    (tests/kernels/attention/mma.mojo:423-424)."""
    q, k, v, dy = _mk(B, S, H, D, dt, S + D + B)
    scale = 1 / math.sqrt(D)
    wo, wlse = oracle.sdpa_fwd(q, k, v, scale, causal)
    wdq, wdk, wdv = oracle.sdpa_bwd(q, k, v, dy, scale, causal)
    o, lse, dq, dk, dv = _run(cuda, q, k, v, dy, dt, causal)
    assert rel_err(o, wo) <= tol_of(dt)
    assert rel_err(lse, wlse) <= 2e-3
    assert rel_err(dq, wdq) <= tol_of(dt)
    assert rel_err(dk, wdk) <= tol_of(dt)
    assert rel_err(dv, wdv) <= tol_of(dt)


# CUDA-core path: fp32, odd head dims, tiny and ragged sequences (the reference tests S=80/96, D=8, T=2/Dh=1)
GEN_SHAPES = [(1, 2, 1, 1), (1, 4, 1, 8), (2, 80, 2, 16), (1, 96, 3, 40), (1, 128, 1, 8), (1, 65, 2, 72)]


@pytest.mark.parametrize("B,S,H,D", GEN_SHAPES)
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
def test_cuda_core_path(cuda, oracle, B, S, H, D, causal, dt):
    q, k, v, dy = _mk(B, S, H, D, dt, 7 * S + D)
    scale = 1 / math.sqrt(D)
    wo, wlse = oracle.sdpa_fwd(q, k, v, scale, causal)
    o, lse, dq, dk, dv = _run(cuda, q, k, v, dy, dt, causal)
    # 16-bit storage: delta = rowsum(O * dO) comes from the stored (rounded) O, as in the reference's GPU kernels;
    # at these tiny shapes dS = P * (dP - delta) cancels heavily, so the oracle is given the same O
    wdq, wdk, wdv = oracle.sdpa_bwd(q, k, v, dy, scale, causal, o_saved=None if dt == "f32" else o)
    tol = tol_of(dt)
    assert rel_err(o, wo) <= tol
    assert rel_err(lse, wlse) <= (1e-4 if dt == "f32" else 2e-3)
    assert rel_err(dq, wdq) <= tol and rel_err(dk, wdk) <= tol and rel_err(dv, wdv) <= tol


def test_additive_bias_path(cuda, oracle):
    B, S, H, D = 1, 48, 2, 16
    q, k, v, dy = _mk(B, S, H, D, "f32", 3)
    mask = np.random.default_rng(4).standard_normal((B, H, S, S)).astype(np.float32)
    scale = 0.25
    import torch
    from mograd_b200 import dispatch as K

    dev = lambda t: torch.from_numpy(t).to(cuda)
    o, lse = K.flash_attn_fwd_dispatch(dev(q), dev(k), dev(v), dev(mask), scale, False, True)
    dq, dk, dv = K.flash_attn_bwd_dispatch(dev(dy), o, dev(q), dev(k), dev(v), dev(mask), lse, scale, False, True)
    wo, _ = oracle.sdpa_fwd(q, k, v, scale, False, mask=mask)
    wdq, wdk, wdv = oracle.sdpa_bwd(q, k, v, dy, scale, False, mask=mask)
    f = lambda t: t.cpu().numpy()
    assert rel_err(f(o), wo) <= TOL_F32 and rel_err(f(dq), wdq) <= TOL_F32
    assert rel_err(f(dk), wdk) <= TOL_F32 and rel_err(f(dv), wdv) <= TOL_F32


@pytest.mark.parametrize("B,S,H,D", [(1, 256, 2, 64), (2, 200, 1, 128), (1, 203, 2, 64), (1, 384, 1, 128)])
@pytest.mark.parametrize("dt", ["bf16", "f16"])
def test_additive_bias_on_tensor_cores(cuda, oracle, B, S, H, D, dt):
    """A dense (B, H, S, S) additive mask with 16-bit storage and D in {64, 128} runs on the tcgen05 kernels
    (forward and backward); S = 203 takes the unaligned mask loads."""
    q, k, v, dy = _mk(B, S, H, D, dt, 11 + S)
    mask = round_to(dt, 2.0 * np.random.default_rng(S).standard_normal((B, H, S, S)).astype(np.float32))
    scale = 1 / math.sqrt(D)
    wo, wlse = oracle.sdpa_fwd(q, k, v, scale, False, mask=mask)
    wdq, wdk, wdv = oracle.sdpa_bwd(q, k, v, dy, scale, False, mask=mask)
    o, lse, dq, dk, dv = _run(cuda, q, k, v, dy, dt, False, mask=mask)
    tol = tol_of(dt)
    assert rel_err(o, wo) <= tol and rel_err(lse, wlse) <= 2e-3
    assert rel_err(dq, wdq) <= tol and rel_err(dk, wdk) <= tol and rel_err(dv, wdv) <= tol


def test_causal_and_bias_together_rejected(cuda):
    import torch
    from mograd_b200 import _lib
    from mograd_b200 import dispatch as K

    q = torch.zeros((1, 4, 1, 8), device=cuda)
    with pytest.raises(_lib.KernelError) as e:
        K.flash_attn_fwd_dispatch(q, q, q, torch.zeros((1, 1, 4, 4), device=cuda), None, True, True)
    assert e.value.code == _lib.EINVAL


def test_reference_analytic_cases_on_gpu(cuda):
    """tests/test_ops.mojo:903-946, 1091-1111 and tests/test_grad.mojo:1001-1023 through the CUDA path."""
    import torch
    from mograd_b200 import dispatch as K

    # T = 2, Dh = 1 known values
    one = torch.ones((1, 2, 1, 1), device=cuda)
    vv = torch.tensor([1.0, -1.0], device=cuda).view(1, 2, 1, 1)
    o, _ = K.flash_attn_fwd_dispatch(one, one, vv, None, 1.0, True, False)
    np.testing.assert_allclose(o.cpu().numpy().ravel(), [1, 0], atol=1e-3)
    # Q = K = 0, causal: prefix mean, S = 128 spans two 64-row tiles of the reference kernels
    S, D = 128, 8
    g = torch.Generator().manual_seed(150)
    v = torch.randn((1, S, 1, D), generator=g).to(cuda)
    z = torch.zeros_like(v)
    o, lse = K.flash_attn_fwd_dispatch(z, z, v, None, None, True, False)
    want = torch.cumsum(v[0, :, 0, :].double(), 0) / torch.arange(1, S + 1, device=cuda).double()[:, None]
    np.testing.assert_allclose(o[0, 0].cpu().numpy(), want.cpu().numpy(), atol=2e-2)
    # same in bf16 at D = 64 on the tensor-core path
    v64 = torch.randn((1, S, 1, 64), generator=g).to(cuda).bfloat16()
    z64 = torch.zeros_like(v64)
    o64, lse64 = K.flash_attn_fwd_dispatch(z64, z64, v64, None, None, True, False)
    want64 = torch.cumsum(v64[0, :, 0, :].double(), 0) / torch.arange(1, S + 1, device=cuda).double()[:, None]
    np.testing.assert_allclose(o64[0, 0].float().cpu().numpy(), want64.cpu().numpy(), atol=2e-2)
    # loss = sum(O): dV[j] = sum_{i >= j} 1 / (i + 1)
    do = torch.ones((1, 1, S, 64), device=cuda).bfloat16()
    dq, dk, dv = K.flash_attn_bwd_dispatch(do, o64, z64, z64, v64, None, lse64, None, True, False)
    tail = np.array([sum(1.0 / (i + 1) for i in range(j, S)) for j in range(S)])
    np.testing.assert_allclose(dv[0, :, 0, :].float().cpu().numpy(), np.repeat(tail[:, None], 64, 1), rtol=2e-2, atol=2e-2)
    assert dk.float().abs().max().item() < 1e-6 and _status() == 0


def test_determinism(cuda):
    """Forward, dK and dV bitwise reproducible; dQ (fp32 reductions in arbitrary order) within a small spread
    (the reference checks the same: tests/kernels/attention/mma.mojo:291-324, 616-685)."""
    import torch
    from mograd_b200 import dispatch as K

    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn((2, 512, 4, 64), generator=g).to(cuda).bfloat16() for _ in range(3))
    do = torch.randn((2, 4, 512, 64), generator=g).to(cuda).bfloat16()
    o1, l1 = K.flash_attn_fwd_dispatch(q, k, v, None, None, True, False)
    o2, l2 = K.flash_attn_fwd_dispatch(q, k, v, None, None, True, False)
    assert torch.equal(o1, o2) and torch.equal(l1, l2)
    a = K.flash_attn_bwd_dispatch(do, o1, q, k, v, None, l1, None, True, False)
    b = K.flash_attn_bwd_dispatch(do, o1, q, k, v, None, l1, None, True, False)
    assert torch.equal(a[1], b[1]) and torch.equal(a[2], b[2])
    assert (a[0].float() - b[0].float()).abs().max().item() < 1e-2


def test_full_size_properties(cuda, oracle):
    """B=4 H=16 S=4096 D=128 causal bf16: first query row copies V0, dV of the last key row, one sampled head vs
    the oracle at reduced length is covered above; here linearity in dO and finiteness at full size."""
    import torch
    from mograd_b200 import dispatch as K

    B, S, H, D = 4, 4096, 16, 128
    g = torch.Generator(device=cuda).manual_seed(6)
    q, k, v = (torch.randn((B, S, H, D), generator=g, device=cuda).bfloat16() for _ in range(3))
    do = torch.randn((B, H, S, D), generator=g, device=cuda).bfloat16()
    o, lse = K.flash_attn_fwd_dispatch(q, k, v, None, None, True, False)
    assert torch.equal(o[:, :, 0, :], v[:, 0, :, :])  # causal: row 0 attends to itself only
    dq, dk, dv = K.flash_attn_bwd_dispatch(do, o, q, k, v, None, lse, None, True, False)
    dq2, dk2, dv2 = K.flash_attn_bwd_dispatch((do.float() * 2).bfloat16(), o, q, k, v, None, lse, None, True, False)
    assert _status() == 0
    for a, b in ((dq, dq2), (dk, dk2), (dv, dv2)):
        assert torch.isfinite(a.float()).all()
        err = ((b.float() - 2 * a.float()).abs().max() / b.float().abs().max()).item()
        assert err < 2e-2  # gradients are linear in dO (up to bf16 rounding)
    # last key row receives gradient from the last query row only: dV[S-1] = P[S-1,S-1] * dO[S-1]
    bsel, hsel = 1, 3
    qs = q[bsel, :, hsel].float().cpu().numpy()[None, :, None, :]
    ks = k[bsel, :, hsel].float().cpu().numpy()[None, :, None, :]
    vs = v[bsel, :, hsel].float().cpu().numpy()[None, :, None, :]
    wo, wlse = oracle.sdpa_fwd(qs[:, :512], ks[:, :512], vs[:, :512], 1 / math.sqrt(D), True)
    assert rel_err(o[bsel, hsel, :512].float().cpu().numpy(), wo[0, 0]) <= TOL_BF16


@pytest.mark.parametrize("B,S,H,D,dt", [(2, 256, 3, 64, "bf16"), (1, 200, 2, 128, "bf16"), (2, 40, 2, 16, "f32"),
                                         (2, 256, 3, 64, "f16")])
def test_fused_projection_layout(cuda, oracle, B, S, H, D, dt):
    """Q, K, V as column blocks of one (tokens, 3*H*D) buffer, O / dO token-major (BSHD), dQ/dK/dV into one buffer."""
    import torch
    from mograd_b200 import dispatch as K

    q, k, v, dy = _mk(B, S, H, D, dt, 31)
    scale = 1 / math.sqrt(D)
    wo, _ = oracle.sdpa_fwd(q, k, v, scale, True)
    wdq, wdk, wdv = oracle.sdpa_bwd(q, k, v, dy, scale, True)
    tdt = torch_dtype(dt)
    qkv = torch.from_numpy(np.stack([q, k, v], axis=2)).to(cuda).to(tdt)  # (B, S, 3, H, D)
    q4, k4, v4 = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    o, lse = K.flash_attn_fwd_dispatch(q4, k4, v4, None, None, True, False, o_bshd=True)
    assert o.shape == (B, S, H, D)
    tol = tol_of(dt)
    assert rel_err(o.float().cpu().numpy(), wo.transpose(0, 2, 1, 3)) <= tol
    dqkv = torch.full_like(qkv, float("nan"))
    do = torch.from_numpy(np.ascontiguousarray(dy.transpose(0, 2, 1, 3))).to(cuda).to(tdt)  # BSHD
    K.flash_attn_bwd_dispatch(do, o, q4, k4, v4, None, lse, None, True, False,
                              out=(dqkv[:, :, 0], dqkv[:, :, 1], dqkv[:, :, 2]), o_bshd=True)
    assert _status() == 0
    got = dqkv.float().cpu().numpy()
    assert rel_err(got[:, :, 0], wdq) <= tol and rel_err(got[:, :, 1], wdk) <= tol and rel_err(got[:, :, 2], wdv) <= tol
