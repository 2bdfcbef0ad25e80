"""CPU restatement of the reference's example models' train step (test infrastructure).

Forward and backward are composed from the oracle's operator restatements in
the order mograd's gradient rules would visit them: MLP (examples/mnist) and
the decoder-only transformer of examples/tinyshakespear/model.mojo:10-130.
Everything is float32 numpy with float64 arithmetic inside the operators.
`round_fn` (identity or bf16 rounding) is applied to every stored activation
and gradient so the comparison with a bf16 GPU run sees the same storage
precision.
"""
from __future__ import annotations

import math

import numpy as np

import oracle as O


def _id(x):
    return x


def mlp_step(params, x, labels, round_fn=_id):
    """params: W0,b0,ln_g,ln_b,W1,b1,... ; returns (loss, grads dict)."""
    nl = sum(1 for k in params if k.startswith("W"))
    acts = []
    h = round_fn(O.relu(O.matmul_bias_bt(x, params["W0"], params["b0"])))
    acts.append(h)
    ln, _, _ = O.layer_norm_fwd(h, params["ln_g"], params["ln_b"])
    ln = round_fn(ln)
    cur = ln
    for i in range(1, nl - 1):
        cur = round_fn(O.relu(O.matmul_bias_bt(cur, params[f"W{i}"], params[f"b{i}"])))
        acts.append(cur)
    logits = round_fn(O.matmul_bias_bt(cur, params[f"W{nl - 1}"], params[f"b{nl - 1}"]))
    loss, dl, _ = O.cross_entropy_index(logits, labels)
    dy = round_fn(dl)
    grads = {}
    for i in range(nl - 1, 0, -1):
        inp = acts[i - 1] if i > 1 else ln
        dx, dw, db = O.matmul_bias_bt_bwd(dy, inp, params[f"W{i}"])
        grads[f"W{i}"], grads[f"b{i}"] = dw, db
        dx = round_fn(dx)
        if i > 1:
            dx = O.relu_grad(acts[i - 1], dx)
        dy = dx
    dx, dg, db = O.layer_norm_bwd(dy, acts[0], params["ln_g"])
    grads["ln_g"], grads["ln_b"] = dg, db
    dx = O.relu_grad(acts[0], round_fn(dx))
    _, dw, db = O.matmul_bias_bt_bwd(dx, x, params["W0"])
    grads["W0"], grads["b0"] = dw, db
    return loss, grads


def transformer_step(params, tokens, targets, n_layers, n_heads, round_fn=_id):
    """tokens/targets (B, S) int64; returns (loss, grads dict)."""
    B, S = tokens.shape
    V, d = params["embed"].shape
    H, Dh = n_heads, d // n_heads
    T = B * S
    tok = tokens.reshape(-1)
    r = round_fn
    x = [O.embedding_fwd(params["embed"], tok)]
    saved = []
    for l in range(n_layers):
        xin = x[l]
        ln1 = r(O.layer_norm_fwd(xin, params[f"g1_{l}"], params[f"be1_{l}"])[0])
        q = r(O.matmul_bias_bt(ln1, params[f"Wq{l}"]))
        k = r(O.matmul_bias_bt(ln1, params[f"Wk{l}"]))
        v = r(O.matmul_bias_bt(ln1, params[f"Wv{l}"]))
        o, _ = O.sdpa_fwd(q.reshape(B, S, H, Dh), k.reshape(B, S, H, Dh), v.reshape(B, S, H, Dh), 1 / math.sqrt(Dh), True)
        o = r(o)
        ctx = np.ascontiguousarray(o.transpose(0, 2, 1, 3)).reshape(T, d)
        h = r(xin + r(O.matmul_bias_bt(ctx, params[f"Wo{l}"])))
        ln2 = r(O.layer_norm_fwd(h, params[f"g2_{l}"], params[f"be2_{l}"])[0])
        f1 = r(O.relu(O.matmul_bias_bt(ln2, params[f"W1_{l}"], params[f"b1_{l}"])))
        out = r(h + r(O.matmul_bias_bt(f1, params[f"W2_{l}"])))
        saved.append(dict(ln1=ln1, q=q, k=k, v=v, o=o, ctx=ctx, h=h, ln2=ln2, f1=f1))
        x.append(out)
    logits = r(O.matmul_bias_bt(x[-1], params["lm_head"]))
    loss, dl, _ = O.cross_entropy_index(logits, targets.reshape(-1))
    dl = r(dl)
    grads = {}
    dx, grads["lm_head"], _ = O.matmul_bias_bt_bwd(dl, x[-1], params["lm_head"], need_db=False)
    dx = r(dx)
    for l in range(n_layers - 1, -1, -1):
        sv, xin = saved[l], x[l]
        dff, grads[f"W2_{l}"], _ = O.matmul_bias_bt_bwd(dx, sv["f1"], params[f"W2_{l}"], need_db=False)
        dff = O.relu_grad(sv["f1"], r(dff))
        dln2, grads[f"W1_{l}"], grads[f"b1_{l}"] = O.matmul_bias_bt_bwd(dff, sv["ln2"], params[f"W1_{l}"])
        dh_ln, grads[f"g2_{l}"], grads[f"be2_{l}"] = O.layer_norm_bwd(r(dln2), sv["h"], params[f"g2_{l}"])
        dh = r(dx + r(dh_ln))
        dctx, grads[f"Wo{l}"], _ = O.matmul_bias_bt_bwd(dh, sv["ctx"], params[f"Wo{l}"], need_db=False)
        dO = np.ascontiguousarray(r(dctx).reshape(B, S, H, Dh).transpose(0, 2, 1, 3))
        dq, dk, dv = O.sdpa_bwd(sv["q"].reshape(B, S, H, Dh), sv["k"].reshape(B, S, H, Dh), sv["v"].reshape(B, S, H, Dh),
                                dO, 1 / math.sqrt(Dh), True, o_saved=None if round_fn is _id else sv["o"])
        dq, dk, dv = (r(t).reshape(T, d) for t in (dq, dk, dv))
        d1, grads[f"Wq{l}"], _ = O.matmul_bias_bt_bwd(dq, sv["ln1"], params[f"Wq{l}"], need_db=False)
        d2, grads[f"Wk{l}"], _ = O.matmul_bias_bt_bwd(dk, sv["ln1"], params[f"Wk{l}"], need_db=False)
        d3, grads[f"Wv{l}"], _ = O.matmul_bias_bt_bwd(dv, sv["ln1"], params[f"Wv{l}"], need_db=False)
        dln1 = r(r(r(d1) + r(d2)) + r(d3))
        dx_ln, grads[f"g1_{l}"], grads[f"be1_{l}"] = O.layer_norm_bwd(dln1, xin, params[f"g1_{l}"])
        dx = r(dh + r(dx_ln))
    grads["embed"] = O.embedding_bwd(dx, tok, V)
    return loss, grads


def adamw(w, g, m, v, step, lr, beta1, beta2, eps, wd):
    """mograd/nn/optim/adam.mojo:6-58 with decoupled weight decay; returns (w, m, v) in float64."""
    g = g.astype(np.float64)
    m = beta1 * m + (1 - beta1) * g
    v = beta2 * v + (1 - beta2) * g * g
    mh = m / (1 - beta1 ** step)
    vh = v / (1 - beta2 ** step)
    w = w.astype(np.float64)
    if wd > 0:
        w = w * (1 - lr * wd)
    return w - lr * mh / (np.sqrt(vh) + eps), m, v
