"""Whole train steps on the GPU vs the CPU restatement of the reference's example models."""
import numpy as np
import pytest

from conftest import TOL_BF16, TOL_F16, TOL_F32, bf16_round, rel_err, round_to

pytestmark = pytest.mark.gpu


def _params_np(model):
    """Parameters (fp32 master copy) under the reference model's names."""
    return {n: model.store.master[a:b].view(shape).cpu().numpy().copy()
            for n, shape in model.store.reference_names() for a, b in [model.store.range[n]]}


def test_mlp_c1_fp32_step_matches_oracle(cuda, oracle):
    """The reference's MNIST MLP: 784 -> 256 (ReLU) -> LayerNorm(256) -> 10, batch 128, fp32, seed 0."""
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


def _tf_check(cuda, cfg, dtype_name, tol, loss_tol):
    import torch
    from mograd_b200.train import TinyTransformer, AdamWConfig
    from oracle import ref_model

    dt = torch.float32 if dtype_name == "f32" else torch.bfloat16
    m = TinyTransformer(cfg["vocab"], cfg["d"], cfg["dff"], cfg["L"], cfg["H"], cfg["B"], cfg["S"], dtype=dt, device=cuda,
                        seed=3, init_std=cfg.get("std", 0.02), opt=AdamWConfig(lr=1e-3, weight_decay=0.1))
    rng = np.random.default_rng(5)
    tok = rng.integers(0, cfg["vocab"], (cfg["B"], cfg["S"])).astype(np.int64)
    tgt = rng.integers(0, cfg["vocab"], (cfg["B"], cfg["S"])).astype(np.int64)
    p0 = _params_np(m)
    rf = (lambda x: x) if dtype_name == "f32" else bf16_round
    want_loss, want_g = ref_model.transformer_step(p0, tok, tgt, cfg["L"], cfg["H"], round_fn=rf)
    loss = m.step(torch.from_numpy(tok).pin_memory(), torch.from_numpy(tgt).pin_memory())
    assert abs(loss - want_loss) <= loss_tol * abs(want_loss)
    worst = {}
    for name in want_g:
        got = m.store.G[name].float().cpu().numpy()
        worst[name] = rel_err(got, want_g[name])
    bad = {k: v for k, v in worst.items() if v > tol}
    assert not bad, bad
    return m, p0, want_g


def test_transformer_fp32_step_matches_oracle(cuda, oracle):
    """Reference transformer structure at toy size, fp32 (CUDA-core attention and GEMM paths)."""
    cfg = dict(vocab=65, d=32, dff=128, L=2, H=4, B=2, S=24, std=0.2)
    m, p0, want_g = _tf_check(cuda, cfg, "f32", 2e-4, 1e-4)
    from oracle import ref_model

    p1 = _params_np(m)
    for name in ("Wq0", "lm_head", "b1_1", "g2_0", "embed"):
        w, _, _ = ref_model.adamw(p0[name], want_g[name], 0.0, 0.0, 1, 1e-3, 0.9, 0.999, 1e-8, 0.1)
        assert rel_err(p1[name], w) <= 1e-3, name


def test_transformer_bf16_step_matches_oracle(cuda, oracle):
    """Char-transformer shape at reduced depth/width (head dim 64: tensor-core attention and GEMMs), bf16.

    Two stacked blocks of bf16-stored activations perturb some gradients by several percent of their largest
    entry even when every operator is computed exactly, so the check is the reference harness's relative gate
    (tests/kernels/attention/harness.mojo:192-194): error against the f64 result <= factor * baseline + floor,
    where the baseline is the error of the f64 oracle run with bf16 storage (the same rounding points)."""
    import torch
    from mograd_b200.train import TinyTransformer
    from oracle import ref_model

    cfg = dict(vocab=65, d=128, dff=512, L=2, H=2, B=2, S=256)
    m = TinyTransformer(cfg["vocab"], cfg["d"], cfg["dff"], cfg["L"], cfg["H"], cfg["B"], cfg["S"], dtype=torch.bfloat16,
                        device=cuda, seed=3, init_std=0.05)
    rng = np.random.default_rng(5)
    tok = rng.integers(0, cfg["vocab"], (cfg["B"], cfg["S"])).astype(np.int64)
    tgt = rng.integers(0, cfg["vocab"], (cfg["B"], cfg["S"])).astype(np.int64)
    p0 = _params_np(m)
    loss64, g64 = ref_model.transformer_step(p0, tok, tgt, cfg["L"], cfg["H"])
    loss16, g16 = ref_model.transformer_step(p0, tok, tgt, cfg["L"], cfg["H"], round_fn=bf16_round)
    loss = m.step(torch.from_numpy(tok).pin_memory(), torch.from_numpy(tgt).pin_memory())
    assert abs(loss - loss64) <= 2e-2 * abs(loss64)
    bad = {}
    for name in g64:
        got = m.store.G[name].float().cpu().numpy()
        err = rel_err(got, g64[name])
        baseline = rel_err(g16[name], g64[name])
        if err > 2.0 * baseline + TOL_BF16:
            bad[name] = (err, baseline)
    assert not bad, bad


def test_transformer_f16_step_matches_oracle(cuda, oracle):
    """The same reduced char-transformer in float16 storage (the half type mograd's buffers carry today): tensor-core
    GEMMs and attention with fp16 operands.  Same relative gate, with the float16 floor of 8e-3."""
    import torch
    from mograd_b200.train import TinyTransformer
    from oracle import ref_model

    cfg = dict(vocab=65, d=128, dff=512, L=2, H=2, B=2, S=256)
    m = TinyTransformer(cfg["vocab"], cfg["d"], cfg["dff"], cfg["L"], cfg["H"], cfg["B"], cfg["S"], dtype=torch.float16,
                        device=cuda, seed=3, init_std=0.05)
    rng = np.random.default_rng(5)
    tok = rng.integers(0, cfg["vocab"], (cfg["B"], cfg["S"])).astype(np.int64)
    tgt = rng.integers(0, cfg["vocab"], (cfg["B"], cfg["S"])).astype(np.int64)
    p0 = _params_np(m)
    rf = lambda x: round_to("f16", x)
    loss64, g64 = ref_model.transformer_step(p0, tok, tgt, cfg["L"], cfg["H"])
    loss16, g16 = ref_model.transformer_step(p0, tok, tgt, cfg["L"], cfg["H"], round_fn=rf)
    loss = m.step(torch.from_numpy(tok).pin_memory(), torch.from_numpy(tgt).pin_memory())
    assert abs(loss - loss64) <= TOL_F16 * abs(loss64)
    bad = {}
    for name in g64:
        got = m.store.G[name].float().cpu().numpy()
        err = rel_err(got, g64[name])
        baseline = rel_err(g16[name], g64[name])
        if err > 2.0 * baseline + TOL_F16:
            bad[name] = (err, baseline)
    assert not bad, bad


def test_graph_replay_of_the_step_matches_eager_launches(cuda, oracle):
    """Model.step() replays a captured CUDA graph of the whole step from its third call on.  Six steps with the
    replay against six steps launched kernel by kernel, same seeds, two alternating batches with prefetch: the MLP
    (no atomics anywhere on its path) must end with bit-identical parameters and losses; the transformer, whose dQ
    and embedding gradients are accumulated by fp32 atomics in an order that is not fixed, with losses that agree
    to 1e-3."""
    import torch
    from mograd_b200.train import MLP, AdamWConfig, TinyTransformer

    def run(make, batches, graph, ahead=False):
        m = make()
        m.use_graph = graph
        losses = [m.step(*batches[i & 1], prefetch=batches[(i + 1) & 1], launch_next=ahead and i < 5)
                  for i in range(6)]
        torch.cuda.synchronize()
        assert (m._graphs[0] is not None and m._graphs[1] is not None) == graph
        assert m._inflight is None
        return losses, m.store.master.clone(), m.store.w.clone(), int(m.d_step.item())

    rng = np.random.default_rng(21)
    mk = lambda: MLP([256, 512, 512, 10], 64, dtype=torch.bfloat16, device=cuda, seed=4,
                     opt=AdamWConfig(lr=1e-2, weight_decay=0.1))
    b = [(torch.from_numpy(rng.standard_normal((64, 256)).astype(np.float32)).to(torch.bfloat16).pin_memory(),
          torch.from_numpy(rng.integers(0, 10, 64).astype(np.int64)).pin_memory()) for _ in range(2)]
    le, me, we, se = run(mk, b, False)
    lg, mg, wg, sg = run(mk, b, True)
    assert se == sg == 6
    assert le == lg, (le, lg)
    assert torch.equal(me, mg) and torch.equal(we, wg)
    assert le[-1] < le[0]  # and the optimiser does make progress
    # with each step's successor queued before the step's own loss is read (launch_next): same losses, same state
    la, ma, wa, sa = run(mk, b, True, ahead=True)
    assert sa == 6 and la == le and torch.equal(ma, me) and torch.equal(wa, we)
    # ... and the same without graphs (the successor's kernels are launched one by one before the loss is read)
    la, ma, wa, sa = run(mk, b, False, ahead=True)
    assert sa == 6 and la == le and torch.equal(ma, me) and torch.equal(wa, we)
    # a call that committed to its successor refuses any other batch next
    m = mk()
    for i in range(5):
        m.step(*b[i & 1], prefetch=b[(i + 1) & 1], launch_next=i == 4)
    assert m._inflight is not None
    other = (b[1][0].clone().pin_memory(), b[1][1])
    with pytest.raises(ValueError):
        m.step(*other)
    torch.cuda.synchronize()

    mk = lambda: TinyTransformer(65, 128, 512, 2, 2, 2, 256, dtype=torch.bfloat16, device=cuda, seed=3, init_std=0.05,
                                 opt=AdamWConfig(lr=1e-3, weight_decay=0.1))
    b = [(torch.from_numpy(rng.integers(0, 65, (2, 256)).astype(np.int64)).pin_memory(),
          torch.from_numpy(rng.integers(0, 65, (2, 256)).astype(np.int64)).pin_memory()) for _ in range(2)]
    le, _, _, se = run(mk, b, False)
    lg, _, _, sg = run(mk, b, True)
    la, _, _, sa = run(mk, b, True, ahead=True)
    assert se == sg == sa == 6
    assert all(abs(a - c) <= 1e-3 * abs(a) for a, c in zip(le, lg)), (le, lg)
    assert all(abs(a - c) <= 1e-3 * abs(a) for a, c in zip(le, la)), (le, la)


def test_dw_products_on_their_own_stream_give_the_same_gradients(cuda, oracle):
    """The transformer's backward pass issues every dW product on a second stream that only waits for dY.  One
    forward + backward from the same state with and without it: gradients that no attention backward feeds (the
    vocabulary projection and the last block's W2, W1, b1, Wo) must be bit-identical, the rest equal up to the
    order of the dQ atomics."""
    import torch
    from mograd_b200.train import TinyTransformer

    rng = np.random.default_rng(31)
    tok = torch.from_numpy(rng.integers(0, 97, (4, 256)).astype(np.int64))
    tgt = torch.from_numpy(rng.integers(0, 97, (4, 256)).astype(np.int64))
    grads = []
    for overlap in (False, True):
        m = TinyTransformer(97, 256, 1024, 3, 4, 4, 256, dtype=torch.bfloat16, device=cuda, seed=8, init_std=0.05)
        m.dw_overlap = overlap
        if overlap and m.dw_stream is None:
            m.dw_stream = torch.cuda.Stream(device=m.device)
        m.d_inputs.copy_(tok)
        m.d_targets.copy_(tgt)
        for _ in range(3):  # the streams drift apart differently from call to call
            m.forward_backward()
        torch.cuda.synchronize()
        grads.append({n: m.store.G[n].float().cpu().numpy().copy() for n in m.store.G})
    a, b = grads
    exact = ["lm_head", "W2_2", "W1_2", "b1_2", "Wo2"]
    for n in exact:
        assert np.array_equal(a[n], b[n]), n
    worst = max((rel_err(b[n], a[n]), n) for n in a)
    assert worst[0] <= 1e-2, worst


@pytest.mark.parametrize("dt", ["f32", "bf16"])
def test_adamw_against_oracle_host_step_and_device_step(cuda, oracle, dt):
    """Five AdamW updates of an odd-sized vector against the oracle's float64 arithmetic
    (mograd/nn/optim/adam.mojo:6-58), once with the step number passed by value and once with it kept in device
    memory (the entry point captured steps use); the two kernels' results agree to float32 rounding."""
    import torch
    from conftest import torch_dtype
    from mograd_b200 import dispatch as K
    from oracle import ref_model

    n = 100003
    rng = np.random.default_rng(77)
    w0 = rng.standard_normal(n).astype(np.float32)
    grads = [round_to(dt, (rng.standard_normal(n) * 0.1).astype(np.float32)) for _ in range(5)]
    td = torch_dtype(dt)
    lr, b1, b2, eps, wd = 1e-2, 0.9, 0.999, 1e-8, 0.1
    state = []
    for dev_step in (False, True):
        master = torch.from_numpy(w0).to(cuda)
        w = master.to(td)
        m, v = torch.zeros(n, device=cuda), torch.zeros(n, device=cuda)
        d_step = torch.zeros(1, dtype=torch.int32, device=cuda)
        for t, g in enumerate(grads, start=1):
            gt = torch.from_numpy(g).to(cuda).to(td)
            if dev_step:
                K.adamw_step_dev(w, gt, m, v, master, lr, b1, b2, eps, wd, d_step, True)
            else:
                K.adamw_step(w, gt, m, v, master, lr, b1, b2, eps, wd, t)
        assert not dev_step or int(d_step.item()) == 5
        state.append((master.cpu().numpy(), m.cpu().numpy(), v.cpu().numpy(), w.float().cpu().numpy()))
    ww, wm, wv = w0.astype(np.float64), np.zeros(n), np.zeros(n)
    for t, g in enumerate(grads, start=1):
        ww, wm, wv = ref_model.adamw(ww, g, wm, wv, t, lr, b1, b2, eps, wd)
    for master, m, v, w in state:
        # (1 - beta2 is formed in float32, as the hyper-parameters arrive: 1.3e-5 off the float64 value)
        assert rel_err(master, ww) <= TOL_F32 and rel_err(m, wm) <= TOL_F32 and rel_err(v, wv) <= TOL_F32
        assert rel_err(w, ww) <= (TOL_F32 if dt == "f32" else 4e-3)  # the storage copy is the rounded master copy
    assert rel_err(state[1][0], state[0][0]) <= 1e-6
