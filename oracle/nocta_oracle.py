"""CPU restatement of the reference's training-path arithmetic (TEST INFRASTRUCTURE ONLY).

Nothing under nocta_b200/ imports this module: it is the checker used by tests/, by
__graft_entry__.smoke() and by bench.py's cpu_baseline leg, never a product code path.

Each function restates one reference routine in numpy, with the accumulation precision the
reference's CPU path uses (float64 where it accumulates in `double`, float32 where it works in
`float`), and cites the file:line it follows (paths relative to the reference project root).
Pinned against the compiled reference itself (oracle/_ref/libnocta_ref.so) by
tests/test_oracle_pinning.py and against the committed fixtures in tests/golden/.

PARITY UNPINNED for gelu_backward only: the reference has no GELU backward (src/ops/activation.c
289-310 registers no autograd node); the formula here is the analytic derivative of its forward.
"""
from __future__ import annotations

import numpy as np

F32 = np.float32
F64 = np.float64


# --------------------------------------------------------------------------------------------
# conv2d — forward src/nn/conv.c:381-586 (im2col + f32 GEMM + bias), backward src/nn/conv.c:118-375
# --------------------------------------------------------------------------------------------
def _windows(xp: np.ndarray, kH: int, kW: int, stride: int) -> np.ndarray:
    """(N,C,Hp,Wp) -> view (N,C,Ho,Wo,kH,kW)."""
    N, C, Hp, Wp = xp.shape
    Ho = (Hp - kH) // stride + 1
    Wo = (Wp - kW) // stride + 1
    s = xp.strides
    return np.lib.stride_tricks.as_strided(
        xp, (N, C, Ho, Wo, kH, kW), (s[0], s[1], s[2] * stride, s[3] * stride, s[2], s[3]), writeable=False)


def conv2d_forward(x, w, b=None, stride=1, padding=0, acc=F64):
    """y[n,co,ho,wo] = sum_{ci,kh,kw} x[n,ci,ho*s+kh-p,wo*s+kw-p] * w[co,ci,kh,kw] + b[co].

    The reference accumulates this GEMM in f32 (src/ops/matmul.c:226-235); `acc` selects the
    accumulator used here (float64 gives the exact value both sides are compared against)."""
    x = np.asarray(x, F32)
    w = np.asarray(w, F32)
    N, C, H, W = x.shape
    Co, Ci, kH, kW = w.shape
    assert Ci == C
    xp = np.pad(x.astype(acc), ((0, 0), (0, 0), (padding, padding), (padding, padding)))
    win = _windows(xp, kH, kW, stride)  # N,C,Ho,Wo,kH,kW
    y = np.tensordot(win, w.astype(acc), axes=([1, 4, 5], [1, 2, 3]))  # N,Ho,Wo,Co
    y = np.transpose(y, (0, 3, 1, 2))
    if b is not None:
        y = y + np.asarray(b, acc).reshape(1, -1, 1, 1)
    return np.ascontiguousarray(y).astype(F32)


def conv2d_backward(x, w, grad_out, stride=1, padding=0, has_bias=True):
    """dX (scatter form, src/nn/conv.c:233-259), dW (double accumulation over (n,ho,wo),
    src/nn/conv.c:269-299) and db (double sum, src/nn/conv.c:200-210).  Computed in float64."""
    x = np.asarray(x, F32)
    w = np.asarray(w, F32)
    g = np.asarray(grad_out, F32).astype(F64)
    N, C, H, W = x.shape
    Co, Ci, kH, kW = w.shape
    xp = np.pad(x.astype(F64), ((0, 0), (0, 0), (padding, padding), (padding, padding)))
    win = _windows(xp, kH, kW, stride)  # N,C,Ho,Wo,kH,kW
    dW = np.tensordot(g, win, axes=([0, 2, 3], [0, 2, 3]))  # Co,C,kH,kW
    db = g.sum(axis=(0, 2, 3)) if has_bias else None
    Ho, Wo = g.shape[2], g.shape[3]
    dxp = np.zeros_like(xp)
    w64 = w.astype(F64)
    for kh in range(kH):
        for kw in range(kW):
            # contribution of tap (kh,kw): dxp[n,ci,ho*s+kh,wo*s+kw] += sum_co g[n,co,ho,wo]*w[co,ci,kh,kw]
            t = np.tensordot(g, w64[:, :, kh, kw], axes=([1], [0]))  # N,Ho,Wo,Ci
            dxp[:, :, kh:kh + Ho * stride:stride, kw:kw + Wo * stride:stride] += np.transpose(t, (0, 3, 1, 2))
    dx = dxp[:, :, padding:padding + H, padding:padding + W]
    return (np.ascontiguousarray(dx).astype(F32), dW.astype(F32), None if db is None else db.astype(F32))


# --------------------------------------------------------------------------------------------
# max pooling — src/nn/conv.c:756-849 (forward), :672-745 (backward recomputes the argmax)
# start value -1e30, strict '>', window scanned (kh, kw) row-major: the FIRST maximum wins.
# --------------------------------------------------------------------------------------------
def maxpool2d_forward(x, k, stride):
    x = np.asarray(x, F32)
    win = _windows(x, k, k, stride)  # N,C,Ho,Wo,k,k
    flat = win.reshape(*win.shape[:4], k * k).astype(F64)
    best = np.full(flat.shape[:4], -1e30, F64)
    arg = np.zeros(flat.shape[:4], np.uint8)
    for t in range(k * k):
        v = flat[..., t]
        m = v > best
        best = np.where(m, v, best)
        arg = np.where(m, np.uint8(t), arg)
    return best.astype(F32), arg


def maxpool2d_backward(x, grad_out, k, stride):
    x = np.asarray(x, F32)
    g = np.asarray(grad_out, F32)
    _, arg = maxpool2d_forward(x, k, stride)
    N, C, Ho, Wo = g.shape
    dx = np.zeros(x.shape, F64)
    n, c, ho, wo = np.meshgrid(np.arange(N), np.arange(C), np.arange(Ho), np.arange(Wo), indexing="ij")
    h = ho * stride + arg // k
    w = wo * stride + arg % k
    np.add.at(dx, (n, c, h, w), g.astype(F64))
    return dx.astype(F32)


# --------------------------------------------------------------------------------------------
# BatchNorm2d — src/nn/batchnorm.c:171-371 (forward), :43-165 (backward); double inside
# --------------------------------------------------------------------------------------------
def batchnorm2d_forward(x, gamma, beta, running_mean, running_var, training=True, momentum=0.1, eps=1e-5):
    """Returns y, batch_mean(f32), batch_var(f32, biased), new_running_mean, new_running_var."""
    x64 = np.asarray(x, F32).astype(F64)
    N, C, H, W = x64.shape
    M = N * H * W
    if training:
        mean = x64.sum(axis=(0, 2, 3)) / M
        var_sum = ((x64 - mean.reshape(1, C, 1, 1)) ** 2).sum(axis=(0, 2, 3))
        var = var_sum / M
        rm, rv = running_mean, running_var
        if rm is not None and rv is not None:
            unbiased = var_sum / (M - 1) if M > 1 else var  # src/nn/batchnorm.c:312-313
            rm = ((1.0 - momentum) * np.asarray(rm, F32).astype(F64) + momentum * mean).astype(F32)
            rv = ((1.0 - momentum) * np.asarray(rv, F32).astype(F64) + momentum * unbiased).astype(F32)
    else:
        mean = np.zeros(C) if running_mean is None else np.asarray(running_mean, F32).astype(F64)
        var = np.ones(C) if running_var is None else np.asarray(running_var, F32).astype(F64)
        rm, rv = running_mean, running_var
    inv = 1.0 / np.sqrt(var + eps)
    g = np.ones(C) if gamma is None else np.asarray(gamma, F32).astype(F64)
    b = np.zeros(C) if beta is None else np.asarray(beta, F32).astype(F64)
    y = g.reshape(1, C, 1, 1) * ((x64 - mean.reshape(1, C, 1, 1)) * inv.reshape(1, C, 1, 1)) + b.reshape(1, C, 1, 1)
    return y.astype(F32), mean.astype(F32), var.astype(F32), rm, rv


def batchnorm2d_backward(grad_out, x, gamma, save_mean, save_var, eps=1e-5):
    """dx, dgamma, dbeta using the saved f32 batch statistics (src/nn/batchnorm.c:113-162)."""
    g = np.asarray(grad_out, F32).astype(F64)
    x64 = np.asarray(x, F32).astype(F64)
    N, C, H, W = x64.shape
    M = N * H * W
    mu = np.asarray(save_mean, F32).astype(F64).reshape(1, C, 1, 1)
    inv = 1.0 / np.sqrt(np.asarray(save_var, F32).astype(F64) + eps)
    xh = (x64 - mu) * inv.reshape(1, C, 1, 1)
    sg = g.sum(axis=(0, 2, 3))
    sgx = (g * xh).sum(axis=(0, 2, 3))
    gam = np.ones(C) if gamma is None else np.asarray(gamma, F32).astype(F64)
    coeff = (gam * inv / M).reshape(1, C, 1, 1)
    dx = coeff * (M * g - sg.reshape(1, C, 1, 1) - xh * sgx.reshape(1, C, 1, 1))
    return dx.astype(F32), sgx.astype(F32), sg.astype(F32)


# --------------------------------------------------------------------------------------------
# LayerNorm over the last dimension — src/nn/batchnorm.c:946-1026 (forward), :600-702 (backward)
# --------------------------------------------------------------------------------------------
def layernorm_forward(x, gamma, beta, eps=1e-5):
    x64 = np.asarray(x, F32).astype(F64)
    D = x64.shape[-1]
    mean = x64.sum(-1, keepdims=True) / D
    var = ((x64 - mean) ** 2).sum(-1, keepdims=True) / D
    inv = 1.0 / np.sqrt(var + eps)
    g = np.ones(D) if gamma is None else np.asarray(gamma, F32).astype(F64)
    b = np.zeros(D) if beta is None else np.asarray(beta, F32).astype(F64)
    return (g * ((x64 - mean) * inv) + b).astype(F32)


def layernorm_backward(grad_out, x, gamma, eps=1e-5):
    """dx, dgamma, dbeta.  The reference adds dgamma/dbeta in f32 with `omp atomic` in a
    thread-dependent order (src/nn/batchnorm.c:662-670); the float64 sums here are the value
    those orderings scatter around."""
    g = np.asarray(grad_out, F32).astype(F64)
    x64 = np.asarray(x, F32).astype(F64)
    D = x64.shape[-1]
    mean = x64.sum(-1, keepdims=True) / D
    var = ((x64 - mean) ** 2).sum(-1, keepdims=True) / D
    inv = 1.0 / np.sqrt(var + eps)
    xh = (x64 - mean) * inv
    gam = np.ones(D) if gamma is None else np.asarray(gamma, F32).astype(F64)
    gg = g * gam
    sg = gg.sum(-1, keepdims=True)
    sgx = (gg * xh).sum(-1, keepdims=True)
    dx = inv / D * (D * gg - sg - xh * sgx)
    red = tuple(range(g.ndim - 1))
    return dx.astype(F32), (g * xh).sum(axis=red).astype(F32), g.sum(axis=red).astype(F32)


# --------------------------------------------------------------------------------------------
# activations — src/ops/activation.c:195-225 / :33-70 (ReLU), :289-310 (GELU forward)
# --------------------------------------------------------------------------------------------
def relu_forward(x):
    x = np.asarray(x, F32)
    return np.where(x > 0, x, F32(0)).astype(F32)


def relu_backward(grad_out, x):
    """dx = x > 0 ? dy : 0, tested on the saved INPUT (src/ops/activation.c:63-67)."""
    return np.where(np.asarray(x, F32) > 0, np.asarray(grad_out, F32), F32(0)).astype(F32)


_GELU_C = np.sqrt(2.0 / np.pi)
_GELU_A = 0.044715


def gelu_forward(x):
    v = np.asarray(x, F32).astype(F64)
    return (0.5 * v * (1.0 + np.tanh(_GELU_C * (v + _GELU_A * v ** 3)))).astype(F32)


def gelu_backward(grad_out, x):
    v = np.asarray(x, F32).astype(F64)
    u = _GELU_C * (v + _GELU_A * v ** 3)
    th = np.tanh(u)
    d = 0.5 * (1.0 + th) + 0.5 * v * (1.0 - th * th) * _GELU_C * (1.0 + 3.0 * _GELU_A * v * v)
    return (np.asarray(grad_out, F32).astype(F64) * d).astype(F32)


def softmax(x):
    """src/ops/activation.c:373-430 over the last dim, double."""
    v = np.asarray(x, F32).astype(F64)
    e = np.exp(v - v.max(-1, keepdims=True))
    return (e / e.sum(-1, keepdims=True)).astype(F32)


# --------------------------------------------------------------------------------------------
# losses — src/ops/loss.c:176-317 / :33-106 (cross entropy, mean), :319-351 / :112-137 (MSE)
# --------------------------------------------------------------------------------------------
def cross_entropy(logits, targets, upstream=1.0):
    """Returns (loss f32, grad_logits f32).  Labels go through (int); out-of-range labels are
    skipped in the loss and get no '-1' in the gradient (src/ops/loss.c:278-281, 86-91)."""
    v = np.asarray(logits, F32).astype(F64)
    B, C = v.shape
    lab = np.asarray(targets).astype(np.int64).astype(np.int32)
    m = v.max(-1, keepdims=True)
    lse = np.log(np.exp(v - m).sum(-1, keepdims=True)) + m
    logp = v - lse
    valid = (lab >= 0) & (lab < C)
    rows = np.arange(B)
    loss = -(logp[rows[valid], lab[valid]]).sum() / B
    p = np.asarray(softmax(logits), F32).astype(F64)  # the reference clones the f32 softmax
    p[rows[valid], lab[valid]] -= 1.0
    grad = p * (upstream / B)
    return F32(loss), grad.astype(F32)


def mse(pred, target, upstream=1.0):
    p = np.asarray(pred, F32).astype(F64)
    t = np.asarray(target, F32).astype(F64)
    d = p - t
    loss = (d * d).sum() / d.size
    scale = 2.0 * upstream / d.size
    return F32(loss), (scale * d).astype(F32), (-scale * d).astype(F32)


# --------------------------------------------------------------------------------------------
# linear — src/nn/linear.c:78-152 (forward), :45-75 (backward); sums over batch in double
# (src/ops/reduction.c:158-198), GEMMs in f32 on the reference, float64 here
# --------------------------------------------------------------------------------------------
def linear_forward(x, W, b=None):
    y = np.asarray(x, F32).astype(F64) @ np.asarray(W, F32).astype(F64).T
    if b is not None:
        y = y + np.asarray(b, F32).astype(F64)
    return y.astype(F32)


def linear_backward(grad_out, x, W, need_dx=True):
    g = np.asarray(grad_out, F32).astype(F64)
    dx = (g @ np.asarray(W, F32).astype(F64)).astype(F32) if need_dx else None
    dW = (g.T @ np.asarray(x, F32).astype(F64)).astype(F32)
    db = g.sum(0).astype(F32)
    return dx, dW, db


# --------------------------------------------------------------------------------------------
# optimizers — src/optim/sgd.c:13-115, src/optim/adam.c:11-75: double math, f32 storage
# --------------------------------------------------------------------------------------------
def sgd_step(p, g, v, lr, momentum=0.0, dampening=0.0, weight_decay=0.0, nesterov=False, first_step=False):
    """Returns (new_p, new_v, new_g).  First step: v = g (src/optim/sgd.c:74-78)."""
    p64 = np.asarray(p, F32).astype(F64)
    g64 = np.asarray(g, F32).astype(F64)
    if weight_decay != 0.0:
        g64 = (g64 + weight_decay * p64).astype(F32).astype(F64)  # stored back as f32 (sgd.c:24-30)
    new_v = v
    if momentum != 0.0:
        v64 = np.zeros_like(p64) if v is None else np.asarray(v, F32).astype(F64)
        v64 = g64.copy() if first_step else momentum * v64 + (1.0 - dampening) * g64
        new_v = v64.astype(F32)
        v64 = new_v.astype(F64)
        upd = g64 + momentum * v64 if nesterov else v64
    else:
        upd = g64
    return (p64 - lr * upd).astype(F32), new_v, g64.astype(F32)


def adam_step(p, g, m, v, t, lr, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, v_max=None):
    """One Adam/AdamW step with step counter t (already incremented, src/optim/adam.c:15).
    m_hat / v_hat use the double moments before they are rounded to f32 (adam.c:49-62)."""
    bc1 = 1.0 - beta1 ** t
    bc2 = 1.0 - beta2 ** t
    p64 = np.asarray(p, F32).astype(F64)
    g64 = np.asarray(g, F32).astype(F64)
    if weight_decay != 0.0:
        p64 = p64 - lr * weight_decay * p64
    m64 = beta1 * np.asarray(m, F32).astype(F64) + (1.0 - beta1) * g64
    v64 = beta2 * np.asarray(v, F32).astype(F64) + (1.0 - beta2) * g64 * g64
    mh = m64 / bc1
    vh = v64 / bc2
    new_vmax = None
    if v_max is not None:
        new_vmax = np.maximum(np.asarray(v_max, F32).astype(F64), vh).astype(F32)
        vh = new_vmax.astype(F64)
    p64 = p64 - lr * mh / (np.sqrt(vh) + eps)
    return p64.astype(F32), m64.astype(F32), v64.astype(F32), new_vmax


# --------------------------------------------------------------------------------------------
# tolerance helper shared by the tests: max-abs error relative to the largest reference
# magnitude, and relative L2 error
# --------------------------------------------------------------------------------------------
def rel_errors(got, ref):
    a = np.asarray(got, F64).ravel()
    b = np.asarray(ref, F64).ravel()
    if a.size == 0:
        return 0.0, 0.0
    denom = max(np.abs(b).max(), 1e-30)
    e_max = np.abs(a - b).max() / denom
    e_l2 = np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30)
    return float(e_max), float(e_l2)
