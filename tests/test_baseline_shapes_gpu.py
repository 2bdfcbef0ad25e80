"""Parity against the CPU oracle at the benchmark configurations' own sizes.

The per-kernel test files compare whole tensors at sizes the oracle finishes in
a blink; this file runs the kernels at the sizes the throughput figures are
quoted on and compares with the oracle on sampled heads / rows / columns (or
on everything, in chunks, where the oracle is fast enough):

  * flash-attention backward, B=4 H=16 S=4096 D=128 causal bf16
  * the vocabulary projection 16384 x 50304 x 768 with a padded output row
    stride: forward, dX and dW
  * LayerNorm backward 65536 x 4096: every row of dx, all of dgamma / dbeta
  * whole train steps: the char transformer at its full size, the
    GPT-2-small-shaped decoder at full width / depth / vocabulary with two
    sequences, the README MLP at full width with 256 samples
"""
import ctypes
import math

import numpy as np
import pytest

from conftest import TOL_BF16, bf16_round, rel_err

pytestmark = pytest.mark.gpu


def _status():
    from mograd_b200 import _lib

    code, detail = ctypes.c_int(0), ctypes.c_int(0)
    assert _lib.load().mograd_b200_device_status(ctypes.byref(code), ctypes.byref(detail)) == 0
    return code.value


def _np(t):
    return t.float().cpu().numpy()


# --------------------------------------------------------------------------- attention backward at S = 4096
def test_flash_attn_bwd_B4_H16_S4096_D128_causal(cuda, oracle):
    """dQ / dK / dV of sampled (batch, head) pairs against orc_sdpa_bwd with delta taken from the stored
    forward output, gate 2e-2; dK / dV bitwise equal between two runs and dQ within the reference's bound on
    its reduction spread (tests/kernels/attention/mma.mojo:616-685)."""
    import torch
    from mograd_b200 import dispatch as K

    B, S, H, D = 4, 4096, 16, 128
    g = torch.Generator(device=cuda).manual_seed(40)
    q, k, v = (torch.randn((B, S, H, D), generator=g, device=cuda).bfloat16() for _ in range(3))
    do = torch.randn((B, H, S, D), generator=g, device=cuda).bfloat16()
    o, lse = K.flash_attn_fwd_dispatch(q, k, v, None, None, True, False)
    dq, dk, dv = K.flash_attn_bwd_dispatch(do, o, q, k, v, None, lse, None, True, False)
    dq2, dk2, dv2 = K.flash_attn_bwd_dispatch(do, o, q, k, v, None, lse, None, True, False)
    assert _status() == 0
    assert torch.equal(dk, dk2) and torch.equal(dv, dv2)
    assert (dq.float() - dq2.float()).abs().max().item() < 1e-2
    scale = 1 / math.sqrt(D)
    picks = [(0, 0), (3, 15), (1, 6)]
    # one oracle call over the sampled heads (they become the H axis of a batch of one)
    qs = np.stack([_np(q[b, :, h]) for b, h in picks], axis=1)[None]  # (1, S, n, D)
    ks = np.stack([_np(k[b, :, h]) for b, h in picks], axis=1)[None]
    vs = np.stack([_np(v[b, :, h]) for b, h in picks], axis=1)[None]
    dos = np.stack([_np(do[b, h]) for b, h in picks], axis=0)[None]  # (1, n, S, D)
    osv = np.stack([_np(o[b, h]) for b, h in picks], axis=0)[None]
    wo, wlse = oracle.sdpa_fwd(qs, ks, vs, scale, True)
    wdq, wdk, wdv = oracle.sdpa_bwd(qs, ks, vs, dos, scale, True, o_saved=osv)
    errs = {}
    for n, (b, h) in enumerate(picks):
        errs[f"o[{b},{h}]"] = rel_err(_np(o[b, h]), wo[0, n])
        errs[f"lse[{b},{h}]"] = rel_err(_np(lse[b, h]), wlse[0, n])
        errs[f"dq[{b},{h}]"] = rel_err(_np(dq[b, :, h]), wdq[0, :, n])
        errs[f"dk[{b},{h}]"] = rel_err(_np(dk[b, :, h]), wdk[0, :, n])
        errs[f"dv[{b},{h}]"] = rel_err(_np(dv[b, :, h]), wdv[0, :, n])
    print("flash_attn S=4096 errors:", {k_: f"{e:.2e}" for k_, e in errs.items()})
    bad = {k_: e for k_, e in errs.items() if e > (2e-3 if k_.startswith("lse") else TOL_BF16)}
    assert not bad, bad


# --------------------------------------------------------------------------- vocabulary projection
def test_vocabulary_projection_16384x50304x768(cuda, oracle):
    """Y = X W^T with the logits' padded row stride, dX = dY W and dW = dY^T X at M=16384 N=50304 K=768:
    128 sampled rows of Y and dX, 64 sampled vocabulary rows of dW over the whole batch."""
    import torch
    from mograd_b200 import dispatch as Kx

    M, N, Kd = 16384, 50304, 768
    g = torch.Generator(device=cuda).manual_seed(41)
    x = torch.randn((M, Kd), generator=g, device=cuda).bfloat16()
    w = (torch.randn((N, Kd), generator=g, device=cuda) / math.sqrt(Kd)).bfloat16()
    ldy = N + 64  # padded rows, as the train step's logits buffer when the vocabulary is not a multiple of 8
    ybuf = torch.full((M, ldy), float("nan"), dtype=torch.bfloat16, device=cuda)
    y = ybuf[:, :N]
    Kx.matmul_bias_strided(x, w, None, out=y)
    assert _status() == 0
    assert torch.isnan(ybuf[:, N:].float()).all()  # the padding is not written
    rng = np.random.default_rng(41)
    rows = np.sort(rng.choice(M, 128, replace=False))
    rows[0], rows[-1] = 0, M - 1
    vrows = np.sort(rng.choice(N, 64, replace=False))
    vrows[0], vrows[-1] = 0, N - 1
    rt, vt = torch.from_numpy(rows).to(cuda), torch.from_numpy(vrows).to(cuda)
    wf = _np(w)
    want_y = oracle.matmul_bias_bt(_np(x[rt]), wf)
    e_y = rel_err(_np(y[rt]), want_y)
    # backward: dY overwrites the logits in place, as in the train step
    dyt = torch.randn((M, N), generator=g, device=cuda).bfloat16()
    y.copy_(dyt)
    del dyt
    dx, dw, _ = Kx.matmul_bias_bt_bwd(y, x, w, need_db=False)
    assert _status() == 0
    want_dx, _, _ = oracle.matmul_bias_bt_bwd(_np(y[rt]), _np(x[rt]), wf, need_db=False)
    e_dx = rel_err(_np(dx[rt]), want_dx)
    _, want_dw, _ = oracle.matmul_bias_bt_bwd(_np(y[:, vt]), _np(x), wf[vrows], need_db=False)
    e_dw = rel_err(_np(dw[vt]), want_dw)
    print(f"vocabulary projection errors: y {e_y:.2e} dx {e_dx:.2e} dw {e_dw:.2e}")
    assert e_y <= TOL_BF16 and e_dx <= TOL_BF16 and e_dw <= TOL_BF16


# --------------------------------------------------------------------------- LayerNorm backward 65536 x 4096
def test_layer_norm_bwd_65536x4096_all_outputs(cuda, oracle):
    """Every row of dx and the complete dgamma / dbeta against the oracle, which runs chunk by chunk (its
    column sums are added up here in float64)."""
    import torch
    from mograd_b200 import dispatch as K

    rows, cols = 65536, 4096
    g = torch.Generator(device=cuda).manual_seed(42)
    x = torch.randn((rows, cols), generator=g, device=cuda).bfloat16()
    dy = torch.randn((rows, cols), generator=g, device=cuda).bfloat16()
    gamma = (1 + 0.1 * torch.randn(cols, generator=g, device=cuda)).bfloat16()
    dx, dg, db = K.layer_norm_bwd_dispatch(dy, x, gamma)
    gm = _np(gamma)
    wdg, wdb = np.zeros(cols), np.zeros(cols)
    worst_dx, chunk = 0.0, 8192
    for r0 in range(0, rows, chunk):
        cdx, cdg, cdb = oracle.layer_norm_bwd(_np(dy[r0:r0 + chunk]), _np(x[r0:r0 + chunk]), gm)
        wdg += cdg.astype(np.float64)
        wdb += cdb.astype(np.float64)
        worst_dx = max(worst_dx, rel_err(_np(dx[r0:r0 + chunk]), cdx))
    e_g, e_b = rel_err(_np(dg), wdg), rel_err(_np(db), wdb)
    print(f"layer_norm_bwd 65536x4096 errors: dx {worst_dx:.2e} dgamma {e_g:.2e} dbeta {e_b:.2e}")
    assert worst_dx <= TOL_BF16 and e_g <= TOL_BF16 and e_b <= TOL_BF16


# --------------------------------------------------------------------------- whole steps at the configs' sizes
def _params_np(model):
    return {n: model.store.master[a:b].view(shape).cpu().numpy().copy()
            for n, shape in model.store.reference_names() for a, b in [model.store.range[n]]}


def _l2_err(got, want):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    if not np.all(np.isfinite(got)):
        return float("inf")
    return float(np.linalg.norm(got - want)) / max(float(np.linalg.norm(want)), 1e-30)


def _gate(model, g64, g16, label):
    """The reference harness's relative gate (tests/kernels/attention/harness.mojo:192-194): the error against
    the f64 result may be at most 2 x the error of the oracle run with bf16 storage + 2e-2.  A tensor passes on
    the max-norm form of that gate, or, for the run-to-run spread of a whole train step, on its l2 form together
    with a 3 x bound on the max norm: dQ is accumulated by fp32 atomics whose order differs between runs, and one
    flipped bf16 rounding twelve layers deep moves the single worst element of a small gradient (the query
    projections at initialisation) by about 1e-2 of its maximum, while the l2 error does not move.  The raw
    errors are printed so the slack the gate allows is visible."""
    bad, table = {}, []
    for name in g64:
        got = model.store.G[name].float().cpu().numpy()
        err, base = rel_err(got, g64[name]), rel_err(g16[name], g64[name])
        table.append((err, base, name))
        if err <= 2.0 * base + TOL_BF16:
            continue
        e2, b2 = _l2_err(got, g64[name]), _l2_err(g16[name], g64[name])
        if not (e2 <= 2.0 * b2 + TOL_BF16 and err <= 3.0 * base + TOL_BF16):
            bad[name] = dict(max_err=err, max_base=base, l2_err=e2, l2_base=b2)
    table.sort(reverse=True)
    print(f"{label}: worst gradient errors vs f64 (error, bf16-storage oracle error, tensor): " +
          ", ".join(f"({e:.3f}, {b:.3f}, {n})" for e, b, n in table[:6]) +
          f"; tensors within 2e-2 outright: {sum(1 for e, _, _ in table if e <= TOL_BF16)} of {len(table)}")
    assert not bad, bad


def _transformer_case(cuda, vocab, d, dff, L, H, B, S, label):
    import torch
    from mograd_b200.train import TinyTransformer
    from oracle import ref_model

    m = TinyTransformer(vocab, d, dff, L, H, B, S, dtype=torch.bfloat16, device=cuda, seed=11, init_std=0.02)
    rng = np.random.default_rng(12)
    tok = rng.integers(0, vocab, (B, S)).astype(np.int64)
    tgt = rng.integers(0, vocab, (B, S)).astype(np.int64)
    p0 = _params_np(m)
    loss64, g64 = ref_model.transformer_step(p0, tok, tgt, L, H)
    loss16, g16 = ref_model.transformer_step(p0, tok, tgt, L, H, round_fn=bf16_round)
    loss = m.step(torch.from_numpy(tok).pin_memory(), torch.from_numpy(tgt).pin_memory())
    assert _status() == 0
    print(f"{label}: loss {loss:.5f}, oracle f64 {loss64:.5f}, oracle with bf16 storage {loss16:.5f}")
    assert abs(loss - loss64) <= 2e-2 * abs(loss64)
    _gate(m, g64, g16, label)


def test_char_transformer_full_size_step(cuda, oracle):
    """vocab 65, context 256, 6 layers, 6 heads, d 384, batch 64 (the reference's tinyshakespear example)."""
    _transformer_case(cuda, 65, 384, 1536, 6, 6, 64, 256, "char transformer 64x256")


def test_gpt2_small_shape_step_batch2(cuda, oracle):
    """12 layers, 12 heads, d 768, d_ff 3072, context 1024, vocabulary 50304; two sequences."""
    _transformer_case(cuda, 50304, 768, 3072, 12, 12, 2, 1024, "gpt2-small shape 2x1024")


def test_readme_mlp_full_width_step(cuda, oracle):
    """4096 -> 4096 (ReLU) -> LayerNorm -> 4096 (ReLU) -> 10 at full width, 256 samples."""
    import torch
    from mograd_b200.train import MLP
    from oracle import ref_model

    m = MLP([4096, 4096, 4096, 10], 256, dtype=torch.bfloat16, device=cuda, seed=13)
    rng = np.random.default_rng(14)
    x = bf16_round(rng.standard_normal((256, 4096)).astype(np.float32))
    y = rng.integers(0, 10, 256).astype(np.int64)
    p0 = _params_np(m)
    loss64, g64 = ref_model.mlp_step(p0, x, y)
    loss16, g16 = ref_model.mlp_step(p0, x, y, round_fn=bf16_round)
    loss = m.step(torch.from_numpy(x).to(torch.bfloat16).pin_memory(), torch.from_numpy(y).pin_memory())
    assert _status() == 0
    print(f"README MLP 256x4096: loss {loss:.5f}, oracle f64 {loss64:.5f}, oracle with bf16 storage {loss16:.5f}")
    assert abs(loss - loss64) <= 2e-2 * abs(loss64)
    _gate(m, g64, g16, "README MLP 256x4096")
