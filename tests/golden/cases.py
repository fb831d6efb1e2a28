"""Seeded op-level and step-level cases driven through the nc_* C API.

`run_all(runner)` executes every case on whatever library the runner is bound to (the compiled
reference on the CPU, or this repository's CUDA library) and returns {name: ndarray}.  The generator
(make_golden.py) stores the reference's results; the tests compare the numpy oracle (CPU suite) and the
CUDA library (GPU suite) with them.  Reference entry points exercised: src/nn/conv.c, src/nn/pooling.c,
src/nn/batchnorm.c, src/ops/activation.c, src/ops/loss.c, src/nn/linear.c, src/optim/sgd.c, src/optim/adam.c.
"""
from __future__ import annotations

import numpy as np

from nocta_b200 import capi, configs

CONV_SHAPES = [(2, 3, 7, 7, 4, 3, 1, 1), (3, 1, 12, 12, 6, 5, 1, 0), (2, 4, 9, 8, 5, 3, 2, 1)]
POOL_SHAPES = [(2, 2, 8), (3, 2, 9), (2, 1, 5)]


def inputs():
    """All seeded inputs, independent of any library (also used by the oracle test)."""
    d = {}
    for i, (N, Ci, H, W, Co, k, s, p) in enumerate(CONV_SHAPES):
        rng = np.random.default_rng(100 + i)
        d[f"conv{i}.x"] = rng.standard_normal((N, Ci, H, W)).astype(np.float32)
        d[f"conv{i}.w"] = rng.standard_normal((Co, Ci, k, k)).astype(np.float32)
        d[f"conv{i}.b"] = rng.standard_normal(Co).astype(np.float32)
        Ho, Wo = (H + 2 * p - k) // s + 1, (W + 2 * p - k) // s + 1
        d[f"conv{i}.g"] = rng.standard_normal((N, Co, Ho, Wo)).astype(np.float32)
    for i, (k, s, H) in enumerate(POOL_SHAPES):
        rng = np.random.default_rng(110 + i)
        x = rng.standard_normal((2, 3, H, H)).astype(np.float32)
        x[x < 0] = 0.0  # ties: the first maximum must win
        Ho = (H - k) // s + 1
        d[f"pool{i}.x"] = x
        d[f"pool{i}.g"] = rng.standard_normal((2, 3, Ho, Ho)).astype(np.float32)
    rng = np.random.default_rng(120)
    d["bn.x"] = (rng.standard_normal((4, 5, 6, 7)) * 2 + 3).astype(np.float32)
    d["bn.gamma"] = rng.standard_normal(5).astype(np.float32)
    d["bn.beta"] = rng.standard_normal(5).astype(np.float32)
    d["bn.rm"] = rng.standard_normal(5).astype(np.float32)
    d["bn.rv"] = (rng.random(5) + 0.5).astype(np.float32)
    d["bn.g"] = rng.standard_normal((4, 5, 6, 7)).astype(np.float32)
    rng = np.random.default_rng(121)
    d["ln.x"] = (rng.standard_normal((9, 24)) + 1).astype(np.float32)
    d["ln.gamma"] = rng.standard_normal(24).astype(np.float32)
    d["ln.beta"] = rng.standard_normal(24).astype(np.float32)
    d["ln.g"] = rng.standard_normal((9, 24)).astype(np.float32)
    rng = np.random.default_rng(122)
    x = rng.standard_normal((5, 17)).astype(np.float32)
    x[0, :4] = 0.0
    d["act.x"] = x
    d["act.g"] = rng.standard_normal((5, 17)).astype(np.float32)
    rng = np.random.default_rng(123)
    d["ce.logits"] = (rng.standard_normal((16, 10)) * 3).astype(np.float32)
    d["ce.labels"] = rng.integers(0, 10, 16).astype(np.int64)
    d["mse.p"] = rng.standard_normal((8, 12)).astype(np.float32)
    d["mse.t"] = rng.standard_normal((8, 12)).astype(np.float32)
    rng = np.random.default_rng(124)
    d["lin.x"] = rng.standard_normal((6, 20)).astype(np.float32)
    d["lin.w"] = rng.standard_normal((7, 20)).astype(np.float32)
    d["lin.b"] = rng.standard_normal(7).astype(np.float32)
    d["lin.g"] = rng.standard_normal((6, 7)).astype(np.float32)
    rng = np.random.default_rng(125)
    d["sgd.w"] = rng.standard_normal((4, 5)).astype(np.float32)
    d["sgd.g"] = rng.standard_normal((3, 4, 5)).astype(np.float32)
    d["adamw.w"] = rng.standard_normal((3, 6)).astype(np.float32)
    d["adamw.g"] = rng.standard_normal((3, 3, 6)).astype(np.float32)
    return d


def _set_grad(r, t, g):
    """Write `g` into t->grad wherever it lives (the optimizer cases feed known gradients)."""
    r.load(t.contents.grad, g)


def run_all(r: configs.Runner) -> dict:
    a = r.api
    d = inputs()
    out = {}
    for i, (N, Ci, H, W, Co, k, s, p) in enumerate(CONV_SHAPES):
        tx, tw, tb = (r.tensor(d[f"conv{i}.{n}"], True) for n in ("x", "w", "b"))
        y = a.nc_conv2d_forward(tx, tw, tb, s, p)
        out[f"conv{i}.y"] = a.to_numpy(y)
        assert a.nc_backward(y, r.tensor(d[f"conv{i}.g"])) == 0
        out[f"conv{i}.dx"], out[f"conv{i}.dw"], out[f"conv{i}.db"] = a.grad_numpy(tx), a.grad_numpy(tw), a.grad_numpy(tb)
    for i, (k, s, H) in enumerate(POOL_SHAPES):
        tx = r.tensor(d[f"pool{i}.x"], True)
        y = a.nc_maxpool2d_forward(tx, k, s)
        out[f"pool{i}.y"] = a.to_numpy(y)
        assert a.nc_backward(y, r.tensor(d[f"pool{i}.g"])) == 0
        out[f"pool{i}.dx"] = a.grad_numpy(tx)
    tx, tg, tb = r.tensor(d["bn.x"], True), r.tensor(d["bn.gamma"], True), r.tensor(d["bn.beta"], True)
    trm, trv = r.tensor(d["bn.rm"]), r.tensor(d["bn.rv"])
    y = a.nc_batchnorm2d_forward_fn(tx, trm, trv, tg, tb, True, 0.1, 1e-5)
    out["bn.y"], out["bn.rm"], out["bn.rv"] = a.to_numpy(y), a.to_numpy(trm), a.to_numpy(trv)
    assert a.nc_backward(y, r.tensor(d["bn.g"])) == 0
    out["bn.dx"], out["bn.dgamma"], out["bn.dbeta"] = a.grad_numpy(tx), a.grad_numpy(tg), a.grad_numpy(tb)
    out["bn.y_eval"] = a.to_numpy(a.nc_batchnorm2d_forward_fn(tx, trm, trv, tg, tb, False, 0.1, 1e-5))
    tx, tg, tb = r.tensor(d["ln.x"], True), r.tensor(d["ln.gamma"], True), r.tensor(d["ln.beta"], True)
    y = a.nc_layernorm_forward_fn(tx, capi.shape_arr([24]), 1, tg, tb, 1e-5)
    out["ln.y"] = a.to_numpy(y)
    assert a.nc_backward(y, r.tensor(d["ln.g"])) == 0
    out["ln.dx"], out["ln.dgamma"], out["ln.dbeta"] = a.grad_numpy(tx), a.grad_numpy(tg), a.grad_numpy(tb)
    tx = r.tensor(d["act.x"], True)
    y = a.nc_relu(tx)
    out["relu.y"] = a.to_numpy(y)
    assert a.nc_backward(y, r.tensor(d["act.g"])) == 0
    out["relu.dx"] = a.grad_numpy(tx)
    tx = r.tensor(d["act.x"], True)
    y = r.gelu(tx)
    out["gelu.y"] = a.to_numpy(y)
    assert a.nc_backward(y, r.tensor(d["act.g"])) == 0
    out["gelu.dx"] = a.grad_numpy(tx)
    tl = r.tensor(d["ce.logits"], True)
    loss = a.nc_cross_entropy_loss(tl, r.tensor(d["ce.labels"]))
    out["ce.loss"] = a.to_numpy(loss).reshape(1)
    assert a.nc_backward_scalar(loss) == 0
    out["ce.dlogits"] = a.grad_numpy(tl)
    tp = r.tensor(d["mse.p"], True)
    loss = a.nc_mse_loss(tp, r.tensor(d["mse.t"]))
    out["mse.loss"] = a.to_numpy(loss).reshape(1)
    assert a.nc_backward_scalar(loss) == 0
    out["mse.dp"] = a.grad_numpy(tp)
    tx, tw, tb = r.tensor(d["lin.x"], True), r.tensor(d["lin.w"], True), r.tensor(d["lin.b"], True)
    y = a.nc_linear_forward(tx, tw, tb)
    out["lin.y"] = a.to_numpy(y)
    assert a.nc_backward(y, r.tensor(d["lin.g"])) == 0
    out["lin.dx"], out["lin.dw"], out["lin.db"] = a.grad_numpy(tx), a.grad_numpy(tw), a.grad_numpy(tb)
    # optimizers on known gradients, three steps each
    for name, make in (("sgd", lambda m: a.nc_sgd_momentum(m, 0.05, 0.9)), ("adamw", lambda m: a.nc_adamw(m, 1e-2, 0.01))):
        w = d[f"{name}.w"]
        lin = a.nc_linear(w.shape[1], w.shape[0], False)
        tw = a.nc_module_get_param(lin, b"weight")
        r.load(tw, w)
        opt = make(lin)
        steps = []
        for g in d[f"{name}.g"]:
            a.nc_optimizer_zero_grad(opt)
            if not tw.contents.grad:  # the gradient buffer appears on the first backward
                y = a.nc_linear_forward(r.tensor(np.zeros((1, w.shape[1]), np.float32)), tw, None)
                assert a.nc_backward(y, r.tensor(np.zeros((1, w.shape[0]), np.float32))) == 0
            _set_grad(r, tw, g)
            a.nc_optimizer_step(opt)
            steps.append(a.to_numpy(tw))
        out[f"{name}.params"] = np.stack(steps)
        out[f"{name}.t"] = np.array([opt.contents.t], np.int64)
    # one LeNet-style training step: loss, the gradients of the small layers, checksums of all
    net, forward, kind, data = configs.build_lenet(r)
    tensors = configs.upload(r, kind, data)
    loss = configs.train_step(r, net, forward, kind, tensors)
    out["lenet.loss"] = a.to_numpy(loss).reshape(1)
    sums = []
    for n, p in net.named_params():
        g = a.grad_numpy(p)
        if g.size <= 2500:
            out[f"lenet.grad.{n}"] = g
        sums.append([g.astype(np.float64).sum(), np.sqrt((g.astype(np.float64) ** 2).sum())])
    out["lenet.grad_sums"] = np.array(sums)
    net.free_step_tensors()
    configs.free_inputs(r, kind, tensors)
    return out
