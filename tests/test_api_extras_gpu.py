"""The rest of the reference's public API that its own example programs use (sigmoid, BatchNorm1d, dropout, row
broadcasts of (1, C) operands), against the compiled reference through the same C API calls; and the reference's
example programs themselves, compiled unmodified against this repository's headers and libraries
(oracle/Makefile, target `apps`), run as a second caller of the API.
Reference: src/ops/activation.c:72-105,312-340, src/nn/batchnorm.c:705-860, src/nn/dropout.c:52-97."""
import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np
import pytest

from oracle import nocta_oracle as O

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parents[1]
APPS = ROOT / "oracle" / "_ref" / "apps"
TOL = 2e-5


def bind(api):
    from nocta_b200 import capi
    lib, T = api.lib, capi.TensorP
    lib.nc_sigmoid.restype, lib.nc_sigmoid.argtypes = T, [T]
    lib.nc_sub.restype, lib.nc_sub.argtypes = T, [T, T]
    lib.nc_mean_all.restype, lib.nc_mean_all.argtypes = T, [T]
    lib.nc_dropout_fn.restype, lib.nc_dropout_fn.argtypes = T, [T, C.c_double, C.c_bool]
    lib.nc_batchnorm1d_forward_fn.restype = T
    lib.nc_batchnorm1d_forward_fn.argtypes = [T, T, T, T, T, C.c_bool, C.c_double, C.c_double]
    return lib


@pytest.fixture(scope="module")
def both(ref):
    from nocta_b200 import configs
    ours = configs.Runner(configs.load_library(), on_device=True)
    theirs = configs.Runner(ref, on_device=False)
    ours.api.lib.nc_cuda_set_math_mode.argtypes = [C.c_int]
    ours.api.lib.nc_cuda_set_math_mode(3)
    bind(ours.api), bind(theirs.api)
    yield ours, theirs
    ours.api.lib.nc_cuda_set_math_mode(0)


def close(a, b, tol=TOL):
    emax, el2 = O.rel_errors(a, b)
    assert emax <= tol and el2 <= tol, (emax, el2)


def test_sigmoid_forward_backward(both):
    rng = np.random.default_rng(31)
    x = (rng.standard_normal((7, 33)) * 3).astype(np.float32)
    g = rng.standard_normal((7, 33)).astype(np.float32)
    res = []
    for r in both:
        tx = r.tensor(x, True)
        y = r.api.lib.nc_sigmoid(tx)
        assert r.api.nc_backward(y, r.tensor(g)) == 0
        res.append((r.api.to_numpy(y), r.api.grad_numpy(tx)))
    close(res[0][0], res[1][0])
    close(res[0][1], res[1][1])
    close(res[0][0], 1.0 / (1.0 + np.exp(-x.astype(np.float64))), 1e-6)


@pytest.mark.parametrize("shape", [(16, 10), (6, 5, 9)])
def test_batchnorm1d(both, shape):
    rng = np.random.default_rng(32)
    Cc = shape[1]
    x = (rng.standard_normal(shape) * 2 + 1).astype(np.float32)
    gamma, beta = rng.standard_normal(Cc).astype(np.float32), rng.standard_normal(Cc).astype(np.float32)
    rm, rv = rng.standard_normal(Cc).astype(np.float32), (rng.random(Cc) + 0.5).astype(np.float32)
    g = rng.standard_normal(shape).astype(np.float32)
    res = []
    for r in both:
        a = r.api
        tx, tg, tb = r.tensor(x, True), r.tensor(gamma, True), r.tensor(beta, True)
        trm, trv = r.tensor(rm), r.tensor(rv)
        y = a.lib.nc_batchnorm1d_forward_fn(tx, trm, trv, tg, tb, True, 0.1, 1e-5)
        out = [a.to_numpy(y), a.to_numpy(trm), a.to_numpy(trv)]
        assert a.nc_backward(y, r.tensor(g)) == 0
        out += [a.grad_numpy(tx), a.grad_numpy(tg), a.grad_numpy(tb)]
        out.append(a.to_numpy(a.lib.nc_batchnorm1d_forward_fn(tx, trm, trv, tg, tb, False, 0.1, 1e-5)))
        res.append(out)
    for got, exp in zip(*res):
        close(got, exp)


def test_dropout_draws_the_reference_mask(both):
    libc = C.CDLL(None)
    rng = np.random.default_rng(33)
    x = rng.standard_normal((5, 3, 4, 6)).astype(np.float32)
    g = rng.standard_normal(x.shape).astype(np.float32)
    res = []
    for r in both:
        libc.srand(1234)                       # both libraries draw from the C library generator of this process
        tx = r.tensor(x, True)
        y = r.api.lib.nc_dropout_fn(tx, 0.3, True)
        assert r.api.nc_backward(y, r.tensor(g)) == 0
        res.append((r.api.to_numpy(y), r.api.grad_numpy(tx), r.api.to_numpy(r.api.lib.nc_dropout_fn(tx, 0.3, False))))
    ours, theirs = res
    assert np.array_equal(ours[0] == 0, theirs[0] == 0)          # the same elements are dropped
    assert 0.15 < float((theirs[0] == 0).mean()) < 0.45
    close(ours[0], theirs[0], 1e-6)
    close(ours[1], theirs[1], 1e-6)
    assert np.array_equal(ours[2], x) and np.array_equal(theirs[2], x)   # evaluation mode: a copy


def test_row_broadcast_of_2d_bias_and_host_operands(both):
    """(4, 8) + (1, 8) and (4, 1) + (1, 1) as the reference's xor example writes them; gradients reach the bias."""
    from nocta_b200 import capi
    rng = np.random.default_rng(34)
    a_ = rng.standard_normal((4, 8)).astype(np.float32)
    b_ = rng.standard_normal((1, 8)).astype(np.float32)
    g = rng.standard_normal((4, 8)).astype(np.float32)
    res = []
    for r in both:
        ta, tb = r.tensor(a_, True), r.tensor(b_, True)
        y = r.api.nc_add(ta, tb)
        assert r.api.nc_backward(y, r.tensor(g)) == 0
        res.append((r.api.to_numpy(y), r.api.grad_numpy(ta), r.api.grad_numpy(tb)))
    for got, exp in zip(*res):
        close(got, exp)
    # an operand that still lives on the host is moved to the device by the op that needs it
    ours = both[0]
    th = ours.api.from_numpy(a_)               # from_numpy after nc_init is already on the device: force a host tensor
    ours.api.nc_tensor_to_device(th, capi.NC_DEVICE_CPU)
    assert th.contents.storage.contents.device == capi.NC_DEVICE_CPU
    y = ours.api.nc_relu(th)
    assert y and th.contents.storage.contents.device == capi.NC_DEVICE_CUDA
    assert np.array_equal(ours.api.to_numpy(y), np.maximum(a_, 0))


def run_app(name, timeout=300):
    exe = APPS / name
    if not exe.exists():
        pytest.skip(f"{exe} has not been built (make -C oracle apps needs the reference sources)")
    # FP32 arithmetic like the reference's CPU path these programs were written for (the default TF32 mode rounds
    # activations to 10 mantissa bits, which a 5000-step toy optimisation at learning rate 1 does notice)
    env = dict(os.environ, NOCTA_CUDA_MATH_MODE="3")
    p = subprocess.run([str(exe)], cwd=str(APPS), capture_output=True, text=True, timeout=timeout, env=env)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    return p.stdout


def test_reference_example_xor_trains():
    """The program seeds its weights from the clock, and the optimisation (a ReLU network at learning rate 1) stops on
    a plateau for some seeds on either library: test_xor_trajectory_matches_reference follows both from identical
    weights and sees the same plateau on both.  So the test asks for convergence within three attempts (three clock
    seconds) and for a falling loss every time."""
    import time
    best = None
    for attempt in range(3):
        out = run_app("xor")
        losses = [float(line.split("Loss:")[1].split("|")[0]) for line in out.splitlines() if "Loss:" in line]
        assert len(losses) >= 5 and losses[-1] < losses[0] and all(np.isfinite(losses)), out[-1500:]
        preds = [float(line.split("pred:")[1].strip(" )\n")) for line in out.splitlines() if "pred:" in line]
        assert len(preds) == 4, out[-1500:]
        best = preds
        if preds[0] < 0.2 and preds[1] > 0.8 and preds[2] > 0.8 and preds[3] < 0.2:
            return
        time.sleep(1.1)  # next clock second, next seed
    raise AssertionError(f"xor did not converge in three attempts, last predictions {best}")


def test_reference_example_batchnorm():
    out = run_app("batchnorm")
    assert "All tests completed!" in out
    # its own printed checks: normalised outputs have mean ~0 and std ~1
    stats = [line for line in out.splitlines() if "expected: ~0, ~1" in line]
    assert len(stats) >= 3
    for line in stats:
        mean = float(line.split("mean=")[1].split(",")[0])
        std = float(line.split("std=")[1].split(" ")[0])
        assert abs(mean) < 1e-3 and abs(std - 1.0) < 1e-2, line


def test_reference_example_dropout():
    out = run_app("dropout_test")
    assert "FAILED" not in out, out[-1500:]
    assert out.count("PASSED") >= 2


def test_reference_example_save_load():
    out = run_app("save_load")
    assert "Done!" in out and "FAILED" not in out and "mismatch" not in out.lower(), out[-1500:]


def test_xor_graph_matches_reference(both):
    """The graph of the reference's xor example (matmul, (1, C) bias adds, relu, sigmoid, sub, mul of a tensor with
    itself, mean_all), one forward + backward on identical weights: loss and all four gradients."""
    rng = np.random.default_rng(35)
    X = np.array([[0, 0], [0, 1], [1, 0], [1, 1]], np.float32)
    Y = np.array([[0], [1], [1], [0]], np.float32)
    W1, b1 = (rng.standard_normal((2, 8)) * 0.5).astype(np.float32), (rng.standard_normal((1, 8)) * 0.1).astype(np.float32)
    W2, b2 = (rng.standard_normal((8, 1)) * 0.5).astype(np.float32), (rng.standard_normal((1, 1)) * 0.1).astype(np.float32)
    res = []
    for r in both:
        a = r.api
        tX, tY = r.tensor(X), r.tensor(Y)
        p = [r.tensor(v, True) for v in (W1, b1, W2, b2)]
        h = a.nc_relu(a.nc_add(a.nc_matmul(tX, p[0]), p[1]))
        pred = a.lib.nc_sigmoid(a.nc_add(a.nc_matmul(h, p[2]), p[3]))
        diff = a.lib.nc_sub(pred, tY)
        loss = a.lib.nc_mean_all(a.nc_mul(diff, diff))
        assert a.nc_backward_scalar(loss) == 0
        res.append([a.to_numpy(loss).reshape(1)] + [a.grad_numpy(t) for t in p])
    names = ["loss", "dW1", "db1", "dW2", "db2"]
    bad = []
    for n, got, exp in zip(names, *res):
        emax, el2 = O.rel_errors(got, exp)
        if max(emax, el2) > TOL:
            bad.append((n, emax, el2, got.ravel()[:8], exp.ravel()[:8]))
    assert not bad, bad


def test_xor_trajectory_matches_reference(both):
    """The xor example's whole loop (zero_grad, forward, backward, w -= grad through get_flat/set_flat, biases starting
    at exactly 0 so that row 0 sits on the ReLU boundary) from identical weights on both libraries.  The loss follows
    the reference's for hundreds of steps; a pre-activation within rounding of 0 may flip a ReLU on one side only, so
    the bound on the loss is loose (1 %) where the single-step test is tight.  Seed 7 stops on the plateau at 0.25 on
    both libraries."""
    from nocta_b200 import capi
    X = np.array([[0, 0], [0, 1], [1, 0], [1, 1]], np.float32)
    Y = np.array([[0], [1], [1], [0]], np.float32)
    for r in both:
        r.api.lib.nc_tensor_set_flat.restype = None
        r.api.lib.nc_tensor_set_flat.argtypes = [capi.TensorP, C.c_size_t, C.c_double]
    for seed, steps in ((0, 300), (3, 300), (7, 300)):
        rng = np.random.default_rng(seed)
        init = [(rng.standard_normal((2, 8)) * 0.5).astype(np.float32), np.zeros((1, 8), np.float32),
                (rng.standard_normal((8, 1)) * 0.5).astype(np.float32), np.zeros((1, 1), np.float32)]
        curves = []
        for r in both:
            a = r.api
            tX, tY = r.tensor(X), r.tensor(Y)
            p = [r.tensor(v, True) for v in init]
            curve = []
            for _ in range(steps):
                for t in p:
                    a.nc_tensor_zero_grad_(t)
                h = a.nc_relu(a.nc_add(a.nc_matmul(tX, p[0]), p[1]))
                pred = a.lib.nc_sigmoid(a.nc_add(a.nc_matmul(h, p[2]), p[3]))
                diff = a.lib.nc_sub(pred, tY)
                loss = a.lib.nc_mean_all(a.nc_mul(diff, diff))
                assert a.nc_backward_scalar(loss) == 0
                curve.append(a.nc_tensor_get_flat(loss, 0))
                for t in p:
                    g = a.grad_numpy(t).ravel()
                    for i in range(g.size):
                        a.lib.nc_tensor_set_flat(t, i, a.nc_tensor_get_flat(t, i) - float(g[i]))
            curves.append(np.array(curve))
        ours, theirs = curves
        assert np.all(np.isfinite(ours))
        assert np.abs(ours[:50] - theirs[:50]).max() <= 1e-5, (seed, np.abs(ours[:50] - theirs[:50]).max())
        assert np.abs(ours - theirs).max() <= 1e-2 * max(theirs.max(), 1e-3), (seed, ours[-1], theirs[-1])
        if seed == 7:
            assert abs(ours[-1] - 0.25) < 1e-3 and abs(theirs[-1] - 0.25) < 1e-3


def _vm_lines(binary, script, env_extra):
    env = dict(os.environ, **env_extra)
    out = subprocess.run([str(binary), str(script)], capture_output=True, text=True, timeout=300, env=env)
    assert out.returncode == 0, out.stderr[-2000:]
    return [l for l in out.stdout.splitlines() if l.startswith("step ") or l.startswith("w0 ")], out.stderr


@pytest.mark.parametrize("mode,tol", [("2", 2e-4), ("0", 2e-2)])
def test_script_interpreter_trains_on_the_cuda_library(mode, tol):
    """The reference's script interpreter (src/lang/*.c + src/main.c), compiled UNMODIFIED against this repository's
    headers and libraries (oracle/Makefile, target `vm`), runs a four-step training script (tests/golden/vm/train_cnn.noc:
    conv2d, batch_norm2d, relu, max_pool2d, reshape, matmul + bias, cross_entropy, backward, apply_sgd_momentum — the
    natives of src/lang/vm.c:924-1112) and prints the same losses and final weights as the same interpreter linked against
    the compiled reference.  apply_sgd_momentum updates the parameters through raw nc_tensor_data pointers
    (vm.c:1090-1112): the library hands out host memory for that and moves the tensors back on their next use.
    Printed numbers carry six digits; 3xTF32 mode is held to 2e-4 over the four steps, plain TF32 to 2e-2."""
    vm, vm_ref = APPS / "noc_vm", APPS / "noc_vm_ref"
    if not vm.exists() or not vm_ref.exists():
        pytest.skip("oracle/_ref/apps/noc_vm(_ref) not built (reference sources were absent at build time)")
    script = ROOT / "tests" / "golden" / "vm" / "train_cnn.noc"
    want, _ = _vm_lines(vm_ref, script, {"OMP_NUM_THREADS": "1"})
    got, err = _vm_lines(vm, script, {"NOCTA_CUDA_MATH_MODE": mode})
    assert len(want) == 5 and len(got) == 5, (want, got, err[-1000:])
    import re
    num = re.compile(r"-?\d+\.?\d*(?:e-?\d+)?")
    for lw, lg in zip(want, got):
        vw, vg = [float(v) for v in num.findall(lw)], [float(v) for v in num.findall(lg)]
        assert len(vw) == len(vg)
        for a, b in zip(vw, vg):
            assert abs(a - b) <= tol * max(abs(a), 1e-2), (lw, lg)
    assert "not on the training path" not in err
