"""Pins the numpy restatement (oracle/nocta_oracle.py) against the compiled reference CPU library,
op by op, on seeded inputs, and against the known-answer values of the reference's own unit tests
(tests/test_nn.c:7-66, tests/test_ops.c:21-56, tests/test_optim.c:6-64 in the reference tree)."""
import ctypes as C

import numpy as np
import pytest

from nocta_b200 import capi
from oracle import nocta_oracle as O

TOL = 2e-6  # f32 storage rounding + f32 GEMM accumulation in the reference forward


def close(a, b, tol=TOL):
    emax, el2 = O.rel_errors(a, b)
    assert emax <= tol and el2 <= tol, (emax, el2)


@pytest.mark.parametrize("shape", [(2, 3, 7, 7, 4, 3, 1, 1), (3, 1, 12, 12, 6, 5, 1, 0), (2, 4, 9, 8, 5, 3, 2, 1)])
def test_conv2d_forward_backward(ref, shape):
    N, Ci, H, W, Co, k, s, p = shape
    rng = np.random.default_rng(10)
    x = rng.standard_normal((N, Ci, H, W)).astype(np.float32)
    w = rng.standard_normal((Co, Ci, k, k)).astype(np.float32)
    b = rng.standard_normal(Co).astype(np.float32)
    tx, tw, tb = ref.from_numpy(x, True), ref.from_numpy(w, True), ref.from_numpy(b, True)
    y = ref.nc_conv2d_forward(tx, tw, tb, s, p)
    yn = ref.to_numpy(y)
    close(O.conv2d_forward(x, w, b, s, p), yn)
    g = rng.standard_normal(yn.shape).astype(np.float32)
    tg = ref.from_numpy(g)
    assert ref.nc_backward(y, tg) == 0
    dx, dw, db = O.conv2d_backward(x, w, g, s, p)
    close(dx, ref.grad_numpy(tx))
    close(dw, ref.grad_numpy(tw))
    close(db, ref.grad_numpy(tb))


def test_conv_known_answer():
    # reference tests/test_nn.c:38-66: 2x2 ones kernel on a 3x3 ones image -> 2x2 of 4.0
    y = O.conv2d_forward(np.ones((1, 1, 3, 3), np.float32), np.ones((1, 1, 2, 2), np.float32))
    assert y.shape == (1, 1, 2, 2) and np.all(y == 4.0)


def test_linear_known_answer(ref):
    # reference tests/test_nn.c:7-36: ones(1,3) through W=ones(2,3), b=3 ... -> 6.0 ; restated with explicit values
    x = np.ones((1, 3), np.float32)
    W = np.ones((2, 3), np.float32)
    b = np.full(2, 3.0, np.float32)
    assert np.all(O.linear_forward(x, W, b) == 6.0)
    y = ref.nc_linear_forward(ref.from_numpy(x), ref.from_numpy(W), ref.from_numpy(b))
    assert np.all(ref.to_numpy(y) == 6.0)


@pytest.mark.parametrize("k,s,H", [(2, 2, 8), (3, 2, 9), (2, 1, 5)])
def test_maxpool(ref, k, s, H):
    rng = np.random.default_rng(11)
    x = rng.standard_normal((2, 3, H, H)).astype(np.float32)
    x[x < 0] = 0.0  # post-ReLU style input: ties are common and the first maximum must win
    tx = ref.from_numpy(x, True)
    y = ref.nc_maxpool2d_forward(tx, k, s)
    yo, _ = O.maxpool2d_forward(x, k, s)
    assert np.array_equal(yo, ref.to_numpy(y))
    g = rng.standard_normal(yo.shape).astype(np.float32)
    assert ref.nc_backward(y, ref.from_numpy(g)) == 0
    close(O.maxpool2d_backward(x, g, k, s), ref.grad_numpy(tx), 1e-7)


def test_batchnorm2d(ref):
    rng = np.random.default_rng(12)
    N, Cc, H, W = 4, 5, 6, 7
    x = (rng.standard_normal((N, Cc, H, W)) * 2 + 3).astype(np.float32)
    gam = rng.standard_normal(Cc).astype(np.float32)
    bet = rng.standard_normal(Cc).astype(np.float32)
    rm = rng.standard_normal(Cc).astype(np.float32)
    rv = (rng.random(Cc) + 0.5).astype(np.float32)
    tx, tg_, tb = ref.from_numpy(x, True), ref.from_numpy(gam, True), ref.from_numpy(bet, True)
    trm, trv = ref.from_numpy(rm), ref.from_numpy(rv)
    y = ref.nc_batchnorm2d_forward_fn(tx, trm, trv, tg_, tb, True, 0.1, 1e-5)
    yo, mean, var, nrm, nrv = O.batchnorm2d_forward(x, gam, bet, rm, rv, True, 0.1, 1e-5)
    close(yo, ref.to_numpy(y))
    close(nrm, ref.to_numpy(trm), 1e-7)
    close(nrv, ref.to_numpy(trv), 1e-7)
    g = rng.standard_normal(x.shape).astype(np.float32)
    assert ref.nc_backward(y, ref.from_numpy(g)) == 0
    dx, dg, dbeta = O.batchnorm2d_backward(g, x, gam, mean, var, 1e-5)
    close(dx, ref.grad_numpy(tx))
    close(dg, ref.grad_numpy(tg_))
    close(dbeta, ref.grad_numpy(tb))
    # eval mode uses the running statistics
    ye = ref.nc_batchnorm2d_forward_fn(tx, trm, trv, tg_, tb, False, 0.1, 1e-5)
    yeo = O.batchnorm2d_forward(x, gam, bet, nrm, nrv, False)[0]
    close(yeo, ref.to_numpy(ye))


def test_layernorm(ref):
    rng = np.random.default_rng(13)
    x = (rng.standard_normal((9, 24)) + 1).astype(np.float32)
    gam = rng.standard_normal(24).astype(np.float32)
    bet = rng.standard_normal(24).astype(np.float32)
    tx, tg_, tb = ref.from_numpy(x, True), ref.from_numpy(gam, True), ref.from_numpy(bet, True)
    y = ref.nc_layernorm_forward_fn(tx, capi.shape_arr([24]), 1, tg_, tb, 1e-5)
    close(O.layernorm_forward(x, gam, bet), ref.to_numpy(y))
    g = rng.standard_normal(x.shape).astype(np.float32)
    assert ref.nc_backward(y, ref.from_numpy(g)) == 0
    dx, dg, db = O.layernorm_backward(g, x, gam)
    close(dx, ref.grad_numpy(tx))
    close(dg, ref.grad_numpy(tg_))
    close(db, ref.grad_numpy(tb))


def test_relu_gelu(ref):
    rng = np.random.default_rng(14)
    x = rng.standard_normal((5, 17)).astype(np.float32)
    x[0, :4] = 0.0
    tx = ref.from_numpy(x, True)
    y = ref.nc_relu(tx)
    assert np.array_equal(O.relu_forward(x), ref.to_numpy(y))
    g = rng.standard_normal(x.shape).astype(np.float32)
    assert ref.nc_backward(y, ref.from_numpy(g)) == 0
    assert np.array_equal(O.relu_backward(g, x), ref.grad_numpy(tx))
    close(O.gelu_forward(x), ref.to_numpy(ref.nc_gelu(ref.from_numpy(x))), 1e-7)
    # the reference has no GELU backward; the shim (oracle/ref_shims.c) and the numpy form agree
    tx2 = ref.from_numpy(x, True)
    y2 = ref.shim_gelu(tx2)
    assert ref.nc_backward(y2, ref.from_numpy(g)) == 0
    close(O.gelu_backward(g, x), ref.grad_numpy(tx2), 1e-7)


def test_losses(ref):
    rng = np.random.default_rng(15)
    logits = (rng.standard_normal((16, 10)) * 3).astype(np.float32)
    labels = rng.integers(0, 10, 16).astype(np.int64)
    tl = ref.from_numpy(logits, True)
    loss = ref.nc_cross_entropy_loss(tl, ref.from_numpy(labels))
    lo, go = O.cross_entropy(logits, labels)
    close(lo, ref.to_numpy(loss), 1e-6)
    assert ref.nc_backward_scalar(loss) == 0
    close(go, ref.grad_numpy(tl), 1e-6)
    p = rng.standard_normal((8, 12)).astype(np.float32)
    t = rng.standard_normal((8, 12)).astype(np.float32)
    tp = ref.from_numpy(p, True)
    ml = ref.nc_mse_loss(tp, ref.from_numpy(t))
    mo, gp, _ = O.mse(p, t)
    close(mo, ref.to_numpy(ml), 1e-6)
    assert ref.nc_backward_scalar(ml) == 0
    close(gp, ref.grad_numpy(tp), 1e-6)


def test_linear(ref):
    rng = np.random.default_rng(16)
    x = rng.standard_normal((6, 20)).astype(np.float32)
    W = rng.standard_normal((7, 20)).astype(np.float32)
    b = rng.standard_normal(7).astype(np.float32)
    tx, tw, tb = ref.from_numpy(x, True), ref.from_numpy(W, True), ref.from_numpy(b, True)
    y = ref.nc_linear_forward(tx, tw, tb)
    close(O.linear_forward(x, W, b), ref.to_numpy(y))
    g = rng.standard_normal((6, 7)).astype(np.float32)
    assert ref.nc_backward(y, ref.from_numpy(g)) == 0
    dx, dW, db = O.linear_backward(g, x, W)
    close(dx, ref.grad_numpy(tx))
    close(dW, ref.grad_numpy(tw))
    close(db, ref.grad_numpy(tb))


def test_sgd_momentum(ref):
    # also the reference's known answers (tests/test_optim.c:6-64): 1 -> 0.95 ; momentum -0.1 then -0.29
    p = np.array([1.0], np.float32)
    assert np.allclose(O.sgd_step(p, np.array([0.5], np.float32), None, 0.1)[0], 0.95)
    p1, v1, _ = O.sgd_step(np.zeros(1, np.float32), np.ones(1, np.float32), None, 0.1, momentum=0.9, first_step=True)
    assert np.allclose(p1, -0.1)
    p2, v2, _ = O.sgd_step(p1, np.ones(1, np.float32), v1, 0.1, momentum=0.9)
    assert np.allclose(p2, -0.29)
    rng = np.random.default_rng(17)
    w = rng.standard_normal((4, 5)).astype(np.float32)
    lin = ref.nc_linear(5, 4, False)
    tw = ref.nc_module_get_param(lin, b"weight")
    ref.set_data(tw, w)
    opt = ref.nc_sgd_momentum(lin, 0.05, 0.9)
    cur, vel = w.copy(), None
    for step in range(3):
        g = rng.standard_normal((4, 5)).astype(np.float32)
        ref.nc_optimizer_zero_grad(opt)
        ref.set_data(tw.contents.grad, g)
        ref.nc_optimizer_step(opt)
        cur, vel, _ = O.sgd_step(cur, g, vel, 0.05, momentum=0.9, first_step=(step == 0))
        close(cur, ref.to_numpy(tw), 1e-7)
    assert opt.contents.t == 3


def test_adamw(ref):
    rng = np.random.default_rng(18)
    w = rng.standard_normal((3, 6)).astype(np.float32)
    lin = ref.nc_linear(6, 3, False)
    tw = ref.nc_module_get_param(lin, b"weight")
    ref.set_data(tw, w)
    opt = ref.nc_adamw(lin, 1e-2, 0.01)
    cur, m, v = w.copy(), np.zeros_like(w), np.zeros_like(w)
    for step in range(1, 4):
        g = rng.standard_normal((3, 6)).astype(np.float32)
        ref.nc_optimizer_zero_grad(opt)
        ref.set_data(tw.contents.grad, g)
        ref.nc_optimizer_step(opt)
        cur, m, v, _ = O.adam_step(cur, g, m, v, step, 1e-2, weight_decay=0.01)
        close(cur, ref.to_numpy(tw), 1e-7)
    assert opt.contents.t == 3
