"""The CUDA library, driven through the nc_* C API by the same case code that produced the golden
vectors (tests/golden/cases.py), against those vectors.  FP32 SIMT and 3xTF32 math modes, tolerance
2e-5 (max-abs over max-abs reference and relative L2); ReLU, max-pool values and the optimizer step
counter are compared exactly."""
import ctypes as C
import sys
from pathlib import Path

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

sys.path.insert(0, str(Path(__file__).resolve().parent / "golden"))
import cases  # noqa: E402
from oracle import nocta_oracle as O  # noqa: E402

GOLD = np.load(Path(__file__).resolve().parent / "golden" / "reference_cpu.npz")
EXACT = {"relu.y", "relu.dx", "pool0.y", "pool1.y", "pool2.y", "sgd.t", "adamw.t"}
TOL = 2e-5


@pytest.fixture(scope="module")
def ours():
    from nocta_b200 import configs
    api = configs.load_library()
    r = configs.Runner(api, on_device=True)
    api.lib.nc_cuda_set_math_mode.argtypes = [C.c_int]
    return r


@pytest.mark.parametrize("mode", [3, 2])
def test_all_cases_match_the_reference_outputs(ours, mode):
    ours.api.lib.nc_cuda_set_math_mode(mode)
    try:
        got = cases.run_all(ours)
    finally:
        ours.api.lib.nc_cuda_set_math_mode(0)
    assert set(got) == set(GOLD.files)
    bad = []
    for name in GOLD.files:
        g, e = got[name], GOLD[name]
        assert g.shape == e.shape, (name, g.shape, e.shape)
        if name in EXACT:
            if not np.array_equal(g, e):
                bad.append((name, "not bit-equal"))
            continue
        tol = 1e-4 if name.startswith("adamw") else TOL  # Adam's update is ~lr * sign(g): see test_configs_gpu
        emax, el2 = O.rel_errors(g, e)
        if not (emax <= tol and el2 <= tol):
            bad.append((name, emax, el2))
    assert not bad, bad
