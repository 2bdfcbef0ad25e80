"""LayerNorm forward / backward kernels vs the CPU oracle, through the C ABI."""
import numpy as np
import pytest

from conftest import TOL_BF16, TOL_F32, bf16_round, rel_err, round_to, tol_of, torch_dtype

pytestmark = pytest.mark.gpu

SHAPES = [(1, 4), (2, 4), (128, 256), (300, 384), (257, 768), (64, 1000), (33, 4096), (7, 5000), (5, 16384), (3, 37)]


@pytest.mark.parametrize("rows,cols", SHAPES)
@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
def test_bwd_matches_oracle(cuda, oracle, rows, cols, dt):
    import torch
    from mograd_b200 import dispatch as K

    rng = np.random.default_rng(rows * 131 + cols)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    dy = rng.standard_normal((rows, cols)).astype(np.float32)
    g = (1.0 + 0.1 * rng.standard_normal(cols)).astype(np.float32)
    tdt = torch_dtype(dt)
    x, dy, g = round_to(dt, x), round_to(dt, dy), round_to(dt, g)
    wdx, wdg, wdb = oracle.layer_norm_bwd(dy, x, g)
    dx, dg, db = K.layer_norm_bwd_dispatch(torch.from_numpy(dy).to(cuda).to(tdt), torch.from_numpy(x).to(cuda).to(tdt),
                                           torch.from_numpy(g).to(cuda).to(tdt))
    tol = tol_of(dt)
    assert rel_err(dx.float().cpu().numpy(), wdx) <= tol
    assert rel_err(dg.float().cpu().numpy(), wdg) <= tol
    assert rel_err(db.float().cpu().numpy(), wdb) <= tol


@pytest.mark.parametrize("rows,cols", SHAPES)
@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
def test_fwd_matches_oracle(cuda, oracle, rows, cols, dt):
    import torch
    from mograd_b200 import dispatch as K

    rng = np.random.default_rng(rows * 17 + cols)
    x = (rng.standard_normal((rows, cols)) * 1.5 + 0.3).astype(np.float32)
    g = (1.0 + 0.1 * rng.standard_normal(cols)).astype(np.float32)
    b = (0.1 * rng.standard_normal(cols)).astype(np.float32)
    tdt = torch_dtype(dt)
    x, g, b = round_to(dt, x), round_to(dt, g), round_to(dt, b)
    wy, wmean, wrstd = oracle.layer_norm_fwd(x, g, b)
    y, mean, rstd = K.layer_norm_fwd_dispatch(torch.from_numpy(x).to(cuda).to(tdt), torch.from_numpy(g).to(cuda).to(tdt),
                                              torch.from_numpy(b).to(cuda).to(tdt), save_stats=True)
    tol = tol_of(dt)
    assert rel_err(y.float().cpu().numpy(), wy) <= tol
    assert rel_err(mean.cpu().numpy(), wmean) <= 1e-4 + (0 if dt == "f32" else 1e-3)
    assert rel_err(rstd.cpu().numpy(), wrstd) <= 1e-4


def test_reference_known_answers_on_gpu(cuda):
    """tests/test_nn.mojo:283-324 and tests/test_grad.mojo:776-856 through the CUDA path."""
    import torch
    from mograd_b200 import dispatch as K

    t = lambda v: torch.tensor(v, dtype=torch.float32, device=cuda)
    y = K.layer_norm_fwd_dispatch(t([[1, 2, 3, 4]]), t([1, 2, 1, 2]), t([0.1, 0.2, 0.1, 0.2]))
    np.testing.assert_allclose(y.cpu().numpy().ravel(), [-1.241641, -0.694427, 0.547214, 2.883282], atol=1e-4)
    y = K.layer_norm_fwd_dispatch(t([[3, 3, 3, 3]]), t([1, 1, 1, 1]), t([0.5] * 4))
    np.testing.assert_allclose(y.cpu().numpy().ravel(), [0.5] * 4, atol=1e-4)
    dx, dg, db = K.layer_norm_bwd_dispatch(t([[0.1, 0.2, 0.3, 0.4]]), t([[1, 2, 3, 4]]), t([1, 2, 1, 2]))
    np.testing.assert_allclose(dx.cpu().numpy().ravel(), [0.0, 0.089443, -0.178886, 0.089443], atol=2e-4)
    np.testing.assert_allclose(dg.cpu().numpy(), [-0.134164, -0.089443, 0.134164, 0.536656], atol=2e-4)
    np.testing.assert_allclose(db.cpu().numpy(), [0.1, 0.2, 0.3, 0.4], atol=1e-5)
    _, _, db = K.layer_norm_bwd_dispatch(t([[0.1, 0.2, 0.3, 0.4]] * 2), t([[1, 2, 3, 4]] * 2), t([1, 1, 1, 1]))
    np.testing.assert_allclose(db.cpu().numpy(), [0.2, 0.4, 0.6, 0.8], atol=1e-5)
    dx, _, _ = K.layer_norm_bwd_dispatch(t([[1, 1, 1, 1]]), t([[1, 2, 3, 4]]), t([1, 1, 1, 1]))
    np.testing.assert_allclose(dx.cpu().numpy().ravel(), [0, 0, 0, 0], atol=1e-5)


def test_bwd_deterministic_and_poison_free(cuda):
    import torch
    from mograd_b200 import dispatch as K

    g = torch.Generator(device="cpu").manual_seed(0)
    x = torch.randn((4099, 768), generator=g).to(cuda).bfloat16()
    dy = torch.randn((4099, 768), generator=g).to(cuda).bfloat16()
    gamma = torch.ones(768, device=cuda).bfloat16()
    a = K.layer_norm_bwd_dispatch(dy, x, gamma)
    b = K.layer_norm_bwd_dispatch(dy, x, gamma)
    for u, v in zip(a, b):
        assert torch.equal(u, v) and torch.isfinite(u.float()).all()


def test_full_size_properties(cuda, oracle):
    """(65536 x 4096) bf16: dbeta = column sums of dy, sampled rows of dx vs the oracle."""
    import torch
    from mograd_b200 import dispatch as K

    rows, cols = 65536, 4096
    g = torch.Generator(device=cuda).manual_seed(9)
    x = torch.randn((rows, cols), generator=g, device=cuda).bfloat16()
    dy = torch.randn((rows, cols), generator=g, device=cuda).bfloat16()
    gamma = (1 + 0.1 * torch.randn(cols, generator=g, device=cuda)).bfloat16()
    dx, dg, db = K.layer_norm_bwd_dispatch(dy, x, gamma)
    want_db = dy.double().sum(dim=0).cpu().numpy()
    assert rel_err(db.float().cpu().numpy(), want_db) <= TOL_BF16
    sel = [0, 1, 4097, 65535]
    wdx, _, _ = oracle.layer_norm_bwd(dy[sel].float().cpu().numpy(), x[sel].float().cpu().numpy(), gamma.float().cpu().numpy())
    assert rel_err(dx[sel].float().cpu().numpy(), wdx) <= TOL_BF16
    # dx of every row is orthogonal to the all-ones vector when gamma-weighted terms are removed: sum_c dx = 0
    assert dx.float().sum(dim=1).abs().max().item() < 0.5


@pytest.mark.parametrize("rows,cols", [(300, 768), (65, 4096), (9, 37)])
@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
def test_bwd_with_residual_gradient(cuda, oracle, rows, cols, dt):
    """dx = layer_norm_bwd(...) + dx_residual, in place on the residual buffer."""
    import torch
    from mograd_b200 import dispatch as K

    rng = np.random.default_rng(rows + cols)
    x, dy, res = (rng.standard_normal((rows, cols)).astype(np.float32) for _ in range(3))
    g = (1.0 + 0.1 * rng.standard_normal(cols)).astype(np.float32)
    tdt = torch_dtype(dt)
    x, dy, res, g = (round_to(dt, t) for t in (x, dy, res, g))
    wdx, wdg, wdb = oracle.layer_norm_bwd(dy, x, g)
    dev = lambda t: torch.from_numpy(t).to(cuda).to(tdt)
    rbuf = dev(res)
    dx, dg, db = K.layer_norm_bwd_dispatch(dev(dy), dev(x), dev(g), dx_out=rbuf, dx_residual=rbuf)
    tol = tol_of(dt)
    assert dx.data_ptr() == rbuf.data_ptr()
    assert rel_err(dx.float().cpu().numpy(), wdx + res) <= tol
    assert rel_err(dg.float().cpu().numpy(), wdg) <= tol and rel_err(db.float().cpu().numpy(), wdb) <= tol


@pytest.mark.parametrize("rows,cols", [(300, 768), (65, 4096), (9, 37), (40, 16384)])
@pytest.mark.parametrize("dt", ["f32", "bf16", "f16"])
def test_bwd_in_place_on_dy(cuda, oracle, rows, cols, dt):
    """dx may be written over dy (the train-step runner does so): a row's dy is read before its dx is stored."""
    import torch
    from mograd_b200 import dispatch as K

    rng = np.random.default_rng(rows * 7 + cols)
    x, dy = (rng.standard_normal((rows, cols)).astype(np.float32) for _ in range(2))
    g = (1.0 + 0.1 * rng.standard_normal(cols)).astype(np.float32)
    tdt = torch_dtype(dt)
    x, dy, g = (round_to(dt, t) for t in (x, dy, g))
    wdx, wdg, wdb = oracle.layer_norm_bwd(dy, x, g)
    dev = lambda t: torch.from_numpy(t).to(cuda).to(tdt)
    buf = dev(dy)
    dx, dg, db = K.layer_norm_bwd_dispatch(buf, dev(x), dev(g), dx_out=buf)
    tol = tol_of(dt)
    assert dx.data_ptr() == buf.data_ptr()
    assert rel_err(dx.float().cpu().numpy(), wdx) <= tol
    assert rel_err(dg.float().cpu().numpy(), wdg) <= tol and rel_err(db.float().cpu().numpy(), wdb) <= tol


def test_bwd_many_launches_alternating_shapes(cuda, oracle):
    """Eighty back-to-back launches of alternating shapes share one workspace in stream order: the first of each
    shape matches the oracle and every repeat is bit-identical to it."""
    import torch
    from mograd_b200 import dispatch as K

    cases = []
    for i, (rows, cols) in enumerate([(5000, 768), (777, 1024), (64, 8192), (3000, 384)]):
        rng = np.random.default_rng(100 + i)
        x, dy = (bf16_round(rng.standard_normal((rows, cols)).astype(np.float32)) for _ in range(2))
        g = bf16_round((1.0 + 0.1 * rng.standard_normal(cols)).astype(np.float32))
        dev = lambda t: torch.from_numpy(t).to(cuda).bfloat16()
        cases.append((dev(dy), dev(x), dev(g), oracle.layer_norm_bwd(dy, x, g)))
    first = {}
    for it in range(80):
        dyd, xd, gd, want = cases[it % len(cases)]
        dx, dg, db = K.layer_norm_bwd_dispatch(dyd, xd, gd)
        if it % len(cases) not in first:
            first[it % len(cases)] = (dx.clone(), dg.clone(), db.clone())
            assert rel_err(dx.float().cpu().numpy(), want[0]) <= TOL_BF16
            assert rel_err(dg.float().cpu().numpy(), want[1]) <= TOL_BF16
            assert rel_err(db.float().cpu().numpy(), want[2]) <= TOL_BF16
        else:
            f = first[it % len(cases)]
            assert torch.equal(dx, f[0]) and torch.equal(dg, f[1]) and torch.equal(db, f[2])
