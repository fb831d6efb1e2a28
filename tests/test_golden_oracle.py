"""The numpy oracle against the committed golden vectors (tests/golden/reference_cpu.npz: outputs of the
compiled reference CPU library on the seeded cases of tests/golden/cases.py).  Needs neither the
reference sources nor a GPU, so the oracle stays pinned wherever the suite runs."""
import sys
from pathlib import Path

import numpy as np
import pytest

sys.path.insert(0, str(Path(__file__).resolve().parent / "golden"))
import cases  # noqa: E402
from oracle import nocta_oracle as O  # noqa: E402

GOLD = np.load(Path(__file__).resolve().parent / "golden" / "reference_cpu.npz")
IN = cases.inputs()
TOL = 2e-6


def close(a, b, tol=TOL):
    emax, el2 = O.rel_errors(a, b)
    assert emax <= tol and el2 <= tol, (emax, el2)


@pytest.mark.parametrize("i", range(len(cases.CONV_SHAPES)))
def test_conv(i):
    N, Ci, H, W, Co, k, s, p = cases.CONV_SHAPES[i]
    x, w, b, g = (IN[f"conv{i}.{n}"] for n in ("x", "w", "b", "g"))
    close(O.conv2d_forward(x, w, b, s, p), GOLD[f"conv{i}.y"])
    dx, dw, db = O.conv2d_backward(x, w, g, s, p)
    close(dx, GOLD[f"conv{i}.dx"])
    close(dw, GOLD[f"conv{i}.dw"])
    close(db, GOLD[f"conv{i}.db"])


@pytest.mark.parametrize("i", range(len(cases.POOL_SHAPES)))
def test_maxpool(i):
    k, s, H = cases.POOL_SHAPES[i]
    y, _ = O.maxpool2d_forward(IN[f"pool{i}.x"], k, s)
    assert np.array_equal(y, GOLD[f"pool{i}.y"])
    close(O.maxpool2d_backward(IN[f"pool{i}.x"], IN[f"pool{i}.g"], k, s), GOLD[f"pool{i}.dx"], 1e-7)


def test_batchnorm():
    y, mean, var, rm, rv = O.batchnorm2d_forward(IN["bn.x"], IN["bn.gamma"], IN["bn.beta"], IN["bn.rm"], IN["bn.rv"], True, 0.1, 1e-5)
    close(y, GOLD["bn.y"])
    close(rm, GOLD["bn.rm"], 1e-7)
    close(rv, GOLD["bn.rv"], 1e-7)
    dx, dg, db = O.batchnorm2d_backward(IN["bn.g"], IN["bn.x"], IN["bn.gamma"], mean, var, 1e-5)
    close(dx, GOLD["bn.dx"])
    close(dg, GOLD["bn.dgamma"])
    close(db, GOLD["bn.dbeta"])
    close(O.batchnorm2d_forward(IN["bn.x"], IN["bn.gamma"], IN["bn.beta"], rm, rv, False)[0], GOLD["bn.y_eval"])


def test_layernorm():
    close(O.layernorm_forward(IN["ln.x"], IN["ln.gamma"], IN["ln.beta"]), GOLD["ln.y"])
    dx, dg, db = O.layernorm_backward(IN["ln.g"], IN["ln.x"], IN["ln.gamma"])
    close(dx, GOLD["ln.dx"])
    close(dg, GOLD["ln.dgamma"])
    close(db, GOLD["ln.dbeta"])


def test_activations():
    assert np.array_equal(O.relu_forward(IN["act.x"]), GOLD["relu.y"])
    assert np.array_equal(O.relu_backward(IN["act.g"], IN["act.x"]), GOLD["relu.dx"])
    close(O.gelu_forward(IN["act.x"]), GOLD["gelu.y"], 1e-7)
    close(O.gelu_backward(IN["act.g"], IN["act.x"]), GOLD["gelu.dx"], 1e-7)


def test_losses():
    lo, go = O.cross_entropy(IN["ce.logits"], IN["ce.labels"])
    close(lo, GOLD["ce.loss"], 1e-6)
    close(go, GOLD["ce.dlogits"], 1e-6)
    mo, gp, _ = O.mse(IN["mse.p"], IN["mse.t"])
    close(mo, GOLD["mse.loss"], 1e-6)
    close(gp, GOLD["mse.dp"], 1e-6)


def test_linear():
    close(O.linear_forward(IN["lin.x"], IN["lin.w"], IN["lin.b"]), GOLD["lin.y"])
    dx, dw, db = O.linear_backward(IN["lin.g"], IN["lin.x"], IN["lin.w"])
    close(dx, GOLD["lin.dx"])
    close(dw, GOLD["lin.dw"])
    close(db, GOLD["lin.db"])


def test_optimizers():
    cur, vel = IN["sgd.w"].copy(), None
    for step, g in enumerate(IN["sgd.g"]):
        cur, vel, _ = O.sgd_step(cur, g, vel, 0.05, momentum=0.9, first_step=(step == 0))
        close(cur, GOLD["sgd.params"][step], 1e-7)
    assert int(GOLD["sgd.t"][0]) == 3
    cur, m, v = IN["adamw.w"].copy(), np.zeros_like(IN["adamw.w"]), np.zeros_like(IN["adamw.w"])
    for step, g in enumerate(IN["adamw.g"], start=1):
        cur, m, v, _ = O.adam_step(cur, g, m, v, step, 1e-2, weight_decay=0.01)
        close(cur, GOLD["adamw.params"][step - 1], 1e-6)
    assert int(GOLD["adamw.t"][0]) == 3
