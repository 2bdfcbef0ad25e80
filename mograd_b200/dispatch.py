"""Host-side mirror of mograd's kernel dispatch for the training hot path.

Each function here plays the part of one exec rule / dispatch helper of the
reference (mograd/runtime/gpu/kernels/dispatch.mojo): it reads the shapes,
allocates the outputs (torch.empty stands in for AnyBuffer.create and the
caching pool of mograd/memory.mojo), takes kernel scratch from a per-stream
workspace (scratch_take, memory.mojo:340-345), and calls the C ABI with raw
device pointers and the current CUDA stream.  Tensors are torch CUDA tensors
used purely as device buffers; no arithmetic happens in PyTorch.
"""
from __future__ import annotations

import ctypes
import math

import torch

from . import _lib
from ._lib import KernelError, call, query

_DT = {torch.bfloat16: _lib.BF16, torch.float32: _lib.F32, torch.float16: _lib.F16}
_workspaces: dict = {}


def dtype_code(t: torch.Tensor) -> int:
    """Erase a tensor dtype into the ABI's dtype code (dispatch.mojo:564-576)."""
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError("dispatch_dtype", _lib.EDTYPE, f"unsupported dtype {t.dtype}") from None


def _ptr(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _require_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise KernelError("dispatch", _lib.EINVAL, "mograd_b200 kernels take device buffers; got a host tensor")


def scratch_take(nbytes: int, device) -> torch.Tensor:
    """Per-(device, stream) scratch buffer, reused across calls in stream order."""
    key = (torch.device(device).index, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(int(nbytes), 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def _rows2d(t: torch.Tensor) -> tuple[int, int, int]:
    """(rows, cols, row stride) of a tensor whose leading dims collapse into rows."""
    cols = t.shape[-1]
    rows = t.numel() // cols
    if t.stride(-1) != 1:
        raise KernelError("dispatch", _lib.EINVAL, "last axis must be contiguous")
    if t.dim() == 1:
        return 1, cols, cols
    ld = t.stride(-2)
    expect = ld
    for d in range(t.dim() - 2, -1, -1):
        if t.shape[d] != 1 and t.stride(d) != expect:
            raise KernelError("dispatch", _lib.EINVAL, "batch dims are not collapsible")
        expect = t.stride(d) * t.shape[d]
    return rows, cols, ld


def _packed_rows(t, rows, cols, who, name):
    """A (rows, cols) operand the kernels index as packed rows: shape and contiguity are checked here because the
    C ABI takes a bare pointer for it."""
    if t is None:
        return
    if t.numel() != rows * cols or t.shape[-1] != cols or not t.is_contiguous():
        raise KernelError(who, _lib.EINVAL, f"{name}: expected a contiguous ({rows}, {cols}) buffer, got shape "
                                            f"{tuple(t.shape)} strides {tuple(t.stride())}")


def _packed_vec(t, n, who, name):
    if t is not None and (t.numel() != n or not t.is_contiguous()):
        raise KernelError(who, _lib.EINVAL, f"{name}: expected a contiguous vector of {n} elements, got shape "
                                            f"{tuple(t.shape)} strides {tuple(t.stride())}")


# ----------------------------------------------------------------------------
# matmul_bias_bt (dispatch.mojo:247-278)
# ----------------------------------------------------------------------------
def matmul_bias_strided(a, w, bias=None, act: int = 0, out=None, residual=None, relu_bits=None):
    """Y = A @ W.T (+ bias) (, ReLU) (+ residual): exec rule `matmul_bias_bt` / `matmul_bt`.
    relu_bits (int32 (M, ceil(N/32)), with act=1 and no residual): receives one bit per output, set where Y > 0."""
    _require_cuda(a, w, bias, residual, relu_bits)
    M, K, lda = _rows2d(a)
    N, K2, ldw = _rows2d(w)
    if K2 != K:
        raise KernelError("matmul_bias_bt", _lib.EINVAL, f"inner dims differ: {K} vs {K2}")
    _packed_vec(bias, N, "matmul_bias_bt", "bias")
    if out is None:
        out = torch.empty(a.shape[:-1] + (N,), dtype=a.dtype, device=a.device)
    Mo, No, ldy = _rows2d(out)
    if (Mo, No) != (M, N):
        raise KernelError("matmul_bias_bt", _lib.EINVAL, f"out is {Mo}x{No}, expected {M}x{N}")
    if residual is not None and _rows2d(residual)[:2] != (M, N):
        raise KernelError("matmul_bias_bt", _lib.EINVAL, f"residual must be {M}x{N}")
    if relu_bits is not None:
        if act != 1 or residual is not None:
            raise KernelError("matmul_bias_bt", _lib.EINVAL, "relu_bits goes with act=1 and no residual")
        call("mograd_b200_matmul_bias_bt_relu_bits", _ptr(a), _ptr(w), _ptr(bias), _ptr(out), _ptr(relu_bits), M, N, K,
             lda, ldw, ldy, relu_bits.stride(0), dtype_code(a), _stream())
        return out
    ldr = _rows2d(residual)[2] if residual is not None else 0
    call("mograd_b200_matmul_bias_bt_ex", _ptr(a), _ptr(w), _ptr(bias), _ptr(residual), _ptr(out), M, N, K, lda, ldw,
         ldr, ldy, int(act), dtype_code(a), _stream())
    return out


def matmul_bias_bt_bwd(dy, x, w, need_dx=True, need_dw=True, need_db=True, dx_out=None, dw_out=None, db_out=None,
                       relu_y=None, dx_residual=None, relu_bits=None):
    """(dX, dW, db) of Y = X @ W.T + b in one call; outputs not needed are None.
    relu_y: ReLU output that produced X (dX is masked by relu_y > 0), or relu_bits: the same mask as one bit per
    element (from matmul_bias_strided(..., relu_bits=)); dx_residual: added to dX."""
    _require_cuda(dy, x, w, relu_y, dx_residual, relu_bits)
    M, N, lddy = _rows2d(dy)
    M2, K, ldx = _rows2d(x)
    N2, K2, ldw = _rows2d(w)
    if M2 != M or N2 != N or K2 != K:
        raise KernelError("matmul_bias_bt_bwd", _lib.EINVAL, "shape mismatch between dY, X and W")
    dx = dx_out if dx_out is not None else (torch.empty_like(x) if need_dx else None)
    dw = dw_out if dw_out is not None else (torch.empty((N, K), dtype=w.dtype, device=w.device) if need_dw else None)
    db = db_out if db_out is not None else (torch.empty((N,), dtype=w.dtype, device=w.device) if need_db else None)
    code = dtype_code(dy)
    nbytes = query("mograd_b200_matmul_bias_bt_bwd_workspace_bytes", M, N, K, code)
    ws = scratch_take(nbytes, dy.device)
    lddx = _rows2d(dx)[2] if dx is not None else K
    lddw = dw.stride(0) if dw is not None else K
    ldm = _rows2d(relu_y)[2] if relu_y is not None else 0
    ldr = _rows2d(dx_residual)[2] if dx_residual is not None else 0
    if relu_bits is not None:
        call("mograd_b200_matmul_bias_bt_bwd_relu_bits", _ptr(dy), _ptr(x), _ptr(w), _ptr(relu_bits), _ptr(dx_residual),
             _ptr(dx), _ptr(dw), _ptr(db), M, N, K, lddy, ldx, ldw, relu_bits.stride(0), ldr, lddx, lddw, code, _ptr(ws),
             ws.numel(), _stream())
        return dx, dw, db
    call("mograd_b200_matmul_bias_bt_bwd_ex", _ptr(dy), _ptr(x), _ptr(w), _ptr(relu_y), _ptr(dx_residual), _ptr(dx),
         _ptr(dw), _ptr(db), M, N, K, lddy, ldx, ldw, ldm, ldr, lddx, lddw, code, _ptr(ws), ws.numel(), _stream())
    return dx, dw, db


# ----------------------------------------------------------------------------
# LayerNorm (dispatch.mojo:281-358)
# ----------------------------------------------------------------------------
def layer_norm_fwd_dispatch(x, gamma, beta, eps: float = 1e-5, save_stats: bool = False, out=None):
    _require_cuda(x, gamma, beta)
    x = x if x.is_contiguous() else x.contiguous()
    cols = x.shape[-1]
    rows = x.numel() // cols
    out = torch.empty_like(x) if out is None else out
    _packed_rows(out, rows, cols, "layer_norm_fwd", "out")
    _packed_vec(gamma, cols, "layer_norm_fwd", "gamma")
    _packed_vec(beta, cols, "layer_norm_fwd", "beta")
    mean = rstd = None
    if save_stats:
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    call("mograd_b200_layer_norm_fwd", _ptr(x), _ptr(gamma), _ptr(beta), _ptr(out), _ptr(mean), _ptr(rstd), rows,
         cols, float(eps), dtype_code(x), _stream())
    return (out, mean, rstd) if save_stats else out


def layer_norm_bwd_dispatch(dy, x, gamma, eps: float = 1e-5, dx_out=None, dgamma_out=None, dbeta_out=None,
                            dx_residual=None):
    """inputs [dy, x, gamma] -> [dx (+ dx_residual), dgamma, dbeta] (dispatch.mojo:332-358)."""
    _require_cuda(dy, x, gamma, dx_residual)
    x = x if x.is_contiguous() else x.contiguous()
    dy = dy if dy.is_contiguous() else dy.contiguous()
    cols = x.shape[-1]
    rows = x.numel() // cols
    dx = torch.empty_like(x) if dx_out is None else dx_out
    dgamma = torch.empty_like(gamma) if dgamma_out is None else dgamma_out
    dbeta = torch.empty_like(gamma) if dbeta_out is None else dbeta_out
    who = "layer_norm_bwd"
    _packed_rows(dy, rows, cols, who, "dy")
    _packed_rows(dx, rows, cols, who, "dx")
    _packed_rows(dx_residual, rows, cols, who, "dx_residual")
    for name, t in (("gamma", gamma), ("dgamma", dgamma), ("dbeta", dbeta)):
        _packed_vec(t, cols, who, name)
    code = dtype_code(x)
    nbytes = query("mograd_b200_layer_norm_bwd_workspace_bytes", rows, cols, code)
    ws = scratch_take(nbytes, x.device)
    call("mograd_b200_layer_norm_bwd_ex", _ptr(dy), _ptr(x), _ptr(gamma), _ptr(dx_residual), _ptr(dx), _ptr(dgamma),
         _ptr(dbeta), rows, cols, float(eps), code, _ptr(ws), ws.numel(), _stream())
    return [dx, dgamma, dbeta]


# ----------------------------------------------------------------------------
# Cross-entropy (runtime/__init__.mojo:530-533, 563-580)
# ----------------------------------------------------------------------------
def cross_entropy(logits, labels):
    """Mean cross-entropy with dense float labels -> one-element tensor of the logits' dtype."""
    _require_cuda(logits, labels)
    N, C, ldx = _rows2d(logits)
    N2, C2, ldl = _rows2d(labels)
    if (N2, C2) != (N, C) or labels.dtype != logits.dtype:
        raise KernelError("cross_entropy", _lib.EINVAL, "labels must have the logits' shape and dtype")
    loss = torch.empty(1, dtype=logits.dtype, device=logits.device)
    code = dtype_code(logits)
    ws = scratch_take(query("mograd_b200_cross_entropy_workspace_bytes", N, C, code), logits.device)
    call("mograd_b200_cross_entropy", _ptr(logits), _ptr(labels), _ptr(loss), N, C, ldx, ldl, code, _ptr(ws),
         ws.numel(), _stream())
    return loss


def cross_entropy_grad(upstream, logits, labels):
    """(softmax(logits) - labels) * upstream / N."""
    _require_cuda(upstream, logits, labels)
    N, C, ldx = _rows2d(logits)
    _, _, ldl = _rows2d(labels)
    dst = torch.empty((N, C), dtype=logits.dtype, device=logits.device)
    call("mograd_b200_cross_entropy_grad", _ptr(upstream), _ptr(logits), _ptr(labels), _ptr(dst), N, C, ldx, ldl, C,
         dtype_code(logits), _stream())
    return dst.view(logits.shape)


def softmax_xent_fwd_bwd(logits, index, upstream: float = 1.0, want_loss=True, want_grad=True, inplace=False):
    """Fused loss + dlogits for one class index per row. Returns (loss fp32 scalar tensor, dlogits)."""
    _require_cuda(logits, index)
    if index.dtype != torch.int64:
        raise KernelError("softmax_xent_fwd_bwd", _lib.EDTYPE, "class indices must be int64")
    N, C, ldx = _rows2d(logits)
    loss = torch.empty((), dtype=torch.float32, device=logits.device) if want_loss else None
    dl = None
    lddx = ldx
    if want_grad:
        dl = logits if inplace else torch.empty_like(logits)
        lddx = _rows2d(dl)[2]
    code = dtype_code(logits)
    ws = scratch_take(query("mograd_b200_softmax_xent_workspace_bytes", N, C, code), logits.device)
    call("mograd_b200_softmax_xent_fwd_bwd", _ptr(logits), _ptr(index), _ptr(loss), _ptr(dl), N, C, ldx, lddx,
         float(upstream), code, _ptr(ws), ws.numel(), _stream())
    return loss, dl


# ----------------------------------------------------------------------------
# Attention (dispatch.mojo:380-481)
# ----------------------------------------------------------------------------
def _token_stride(t, name):
    """Elements between consecutive tokens of a (B,S,H,D) tensor whose heads are packed inside a token row."""
    B, S, H, D = t.shape
    if t.stride(3) != 1 or t.stride(2) != D or (B > 1 and t.stride(0) != S * t.stride(1)):
        raise KernelError("flash_attn", _lib.EINVAL, f"{name}: heads must be packed inside each token row")
    return t.stride(1)


def _attn_layout_checks(who, B, S, H, D, oshape, mask, has_bias, lse, **packed):
    """O / dO are packed tensors of the agreed layout, LSE is packed (B, H, S) float32, the mask packed (B, H, S, S)."""
    for name, t in packed.items():
        if tuple(t.shape) != tuple(oshape) or not t.is_contiguous():
            raise KernelError(who, _lib.EINVAL, f"{name}: expected a contiguous {tuple(oshape)} tensor, got shape "
                                                f"{tuple(t.shape)} strides {tuple(t.stride())}")
    if tuple(lse.shape) != (B, H, S) or lse.dtype != torch.float32 or not lse.is_contiguous():
        raise KernelError(who, _lib.EINVAL, "lse must be a contiguous float32 (B, H, S) tensor")
    if has_bias and (mask is None or tuple(mask.shape) != (B, H, S, S) or not mask.is_contiguous()):
        raise KernelError(who, _lib.EINVAL, "has_bias needs a contiguous (B, H, S, S) mask")


def flash_attn_fwd_dispatch(q, k, v, mask=None, scale=None, is_causal=True, has_bias=None, out=None, lse_out=None,
                            o_bshd=False):
    """srcs [Q, K, V, mask] all BSHD -> [O (BHSD, or BSHD when o_bshd), LSE (B,H,S) float32].
    Q, K, V may be column blocks of one fused projection output (equal token strides)."""
    _require_cuda(q, k, v, mask)
    B, S, H, D = q.shape
    if has_bias is None:
        has_bias = mask is not None and not is_causal
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    ld = _token_stride(q, "q")
    if _token_stride(k, "k") != ld or _token_stride(v, "v") != ld:
        raise KernelError("flash_attn_fwd", _lib.EINVAL, "q, k and v must share one token stride")
    oshape = (B, S, H, D) if o_bshd else (B, H, S, D)
    dst = torch.empty(oshape, dtype=q.dtype, device=q.device) if out is None else out
    lse = torch.empty((B, H, S), dtype=torch.float32, device=q.device) if lse_out is None else lse_out
    _attn_layout_checks("flash_attn_fwd", B, S, H, D, oshape, mask, has_bias, lse, out=dst)
    call("mograd_b200_flash_attn_fwd_ex", _ptr(q), _ptr(k), _ptr(v), _ptr(mask), _ptr(dst), _ptr(lse), B, S, H, D,
         float(scale), int(bool(is_causal)), int(bool(has_bias)), ld, int(bool(o_bshd)), dtype_code(q), _stream())
    return [dst, lse]


def flash_attn_bwd_dispatch(dy, o, q, k, v, mask, lse, scale=None, is_causal=True, has_bias=None, out=None,
                            o_bshd=False):
    """srcs [dO, O, Q, K, V, mask, LSE] -> [dQ, dK, dV] (BSHD); dO and O are BHSD, or BSHD when o_bshd."""
    _require_cuda(dy, o, q, k, v, mask, lse)
    B, S, H, D = q.shape
    if has_bias is None:
        has_bias = mask is not None and not is_causal
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    dy = dy if dy.is_contiguous() else dy.contiguous()  # the rule makes dO contiguous (grad.mojo:336-339)
    oshape = (B, S, H, D) if o_bshd else (B, H, S, D)
    _attn_layout_checks("flash_attn_bwd", B, S, H, D, oshape, mask, has_bias, lse, dy=dy, o=o)
    ld = _token_stride(q, "q")
    if _token_stride(k, "k") != ld or _token_stride(v, "v") != ld:
        raise KernelError("flash_attn_bwd", _lib.EINVAL, "q, k and v must share one token stride")
    if out is not None:
        dq, dk, dv = out
    else:
        dq, dk, dv = (torch.empty((B, S, H, D), dtype=q.dtype, device=q.device) for _ in range(3))
    ldd = _token_stride(dq, "dq")
    if _token_stride(dk, "dk") != ldd or _token_stride(dv, "dv") != ldd:
        raise KernelError("flash_attn_bwd", _lib.EINVAL, "dq, dk and dv must share one token stride")
    code = dtype_code(q)
    ws = scratch_take(query("mograd_b200_flash_attn_bwd_workspace_bytes", B, S, H, D, code), q.device)
    call("mograd_b200_flash_attn_bwd_ex", _ptr(dy), _ptr(o), _ptr(q), _ptr(k), _ptr(v), _ptr(mask), _ptr(lse), _ptr(dq),
         _ptr(dk), _ptr(dv), B, S, H, D, float(scale), int(bool(is_causal)), int(bool(has_bias)), ld, ldd,
         int(bool(o_bshd)), code, _ptr(ws), ws.numel(), _stream())
    return [dq, dk, dv]


# ----------------------------------------------------------------------------
# Callers of the hot path inside a train step
# ----------------------------------------------------------------------------
def relu_grad(y, dy, out=None):
    """RELU_GRAD(node=relu output, upstream) (runtime/__init__.mojo:351-352)."""
    _require_cuda(y, dy)
    out = dy if out is None else out
    call("mograd_b200_relu_grad", _ptr(y), _ptr(dy), _ptr(out), y.numel(), dtype_code(y), _stream())
    return out


def add(a, b, out=None):
    _require_cuda(a, b)
    out = torch.empty_like(a) if out is None else out
    call("mograd_b200_add", _ptr(a), _ptr(b), _ptr(out), a.numel(), dtype_code(a), _stream())
    return out


def gather_rows(table, idx, out=None):
    """Embedding forward: out[t] = table[idx[t]]."""
    _require_cuda(table, idx)
    V, d = table.shape
    T = idx.numel()
    out = torch.empty((T, d), dtype=table.dtype, device=table.device) if out is None else out
    call("mograd_b200_gather_rows", _ptr(table), _ptr(idx), _ptr(out), T, V, d, dtype_code(table), _stream())
    return out


def scatter_add_rows(dout, idx, vocab, out=None):
    """Embedding backward: dtable[v] = sum of dout rows whose index is v."""
    _require_cuda(dout, idx)
    T, d = dout.shape
    out = torch.empty((vocab, d), dtype=dout.dtype, device=dout.device) if out is None else out
    code = dtype_code(dout)
    ws = scratch_take(query("mograd_b200_scatter_add_rows_workspace_bytes", vocab, d, code), dout.device)
    call("mograd_b200_scatter_add_rows", _ptr(dout), _ptr(idx), _ptr(out), T, vocab, d, code, _ptr(ws), ws.numel(),
         _stream())
    return out


def adamw_step(w, g, m, v, master, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0):
    _require_cuda(w, g, m, v, master)
    call("mograd_b200_adamw_step", _ptr(w), _ptr(g), _ptr(m), _ptr(v), _ptr(master), w.numel(), float(lr), float(beta1),
         float(beta2), float(eps), float(weight_decay), int(step), float(grad_scale), dtype_code(w), _stream())


def adamw_step_dev(w, g, m, v, master, lr, beta1, beta2, eps, weight_decay, step_dev, advance, grad_scale=1.0):
    """AdamW with the 1-based step number in the device int32 tensor step_dev (for captured / replayed streams);
    advance=True adds 1 to it on the stream first."""
    _require_cuda(w, g, m, v, master, step_dev)
    call("mograd_b200_adamw_step_dev", _ptr(w), _ptr(g), _ptr(m), _ptr(v), _ptr(master), w.numel(), float(lr),
         float(beta1), float(beta2), float(eps), float(weight_decay), _ptr(step_dev), int(bool(advance)),
         float(grad_scale), dtype_code(w), _stream())