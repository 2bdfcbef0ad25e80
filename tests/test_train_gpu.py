"""Whole train steps on the GPU vs the CPU restatement of the reference's example models."""
import numpy as np
import pytest

from conftest import TOL_BF16, TOL_F32, bf16_round, rel_err

pytestmark = pytest.mark.gpu


def _params_np(model):
    return {n: model.store.master[a:b].view(shape).cpu().numpy().copy()
            for n, shape, _ in model.store.specs for a, b in [model.store.range[n]]}


def test_mlp_c1_fp32_step_matches_oracle(cuda, oracle):
    """BASELINE config 1: 784 -> 256 (ReLU) -> LayerNorm(256) -> 10, batch 128, fp32, seed 0."""
    import torch
    from mograd_b200.train import MLP, AdamWConfig
    from oracle import ref_model

    m = MLP([784, 256, 10], 128, dtype=torch.float32, device=cuda, seed=0, opt=AdamWConfig(lr=1e-3, weight_decay=0.1))
    rng = np.random.default_rng(0)
    x = rng.random((128, 784), dtype=np.float32)
    y = rng.integers(0, 10, 128).astype(np.int64)
    p0 = _params_np(m)
    want_loss, want_g = ref_model.mlp_step(p0, x, y)
    loss = m.step(torch.from_numpy(x).pin_memory(), torch.from_numpy(y).pin_memory())
    assert abs(loss - want_loss) <= 1e-4 * abs(want_loss)
    for name in want_g:
        got = m.store.G[name].float().cpu().numpy()
        assert rel_err(got, want_g[name]) <= TOL_F32, name
    # optimiser: first AdamW step
    p1 = _params_np(m)
    for name in want_g:
        w, _, _ = ref_model.adamw(p0[name], want_g[name], 0.0, 0.0, 1, 1e-3, 0.9, 0.999, 1e-8, 0.1)
        assert rel_err(p1[name], w) <= 1e-4, name


def test_mlp_c2_shape_bf16_step_matches_oracle(cuda, oracle):
    """README MLP structure (Linear-ReLU-LN-Linear-ReLU-Linear) at reduced width, bf16."""
    import torch
    from mograd_b200.train import MLP
    from oracle import ref_model

    m = MLP([512, 512, 512, 10], 256, dtype=torch.bfloat16, device=cuda, seed=1)
    rng = np.random.default_rng(1)
    x = bf16_round(rng.standard_normal((256, 512)).astype(np.float32))
    y = rng.integers(0, 10, 256).astype(np.int64)
    p0 = _params_np(m)
    want_loss, want_g = ref_model.mlp_step(p0, x, y, round_fn=bf16_round)
    loss = m.step(torch.from_numpy(x).to(torch.bfloat16).pin_memory(), torch.from_numpy(y).pin_memory())
    assert abs(loss - want_loss) <= 2e-2 * abs(want_loss)
    for name in want_g:
        got = m.store.G[name].float().cpu().numpy()
        assert rel_err(got, want_g[name]) <= 3e-2, name  # bf16 chain of 3 GEMMs: 2e-2 per op, compounding
