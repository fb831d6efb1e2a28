"""The .ncta path with the tensors on the CUDA device: files byte-identical to the golden files the compiled
reference wrote, loads land on the device, and a training run resumed from a checkpoint (model +
optimizer state + step counter) continues bit for bit like the uninterrupted run."""
import ctypes as C
import sys
from pathlib import Path

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

sys.path.insert(0, str(Path(__file__).resolve().parent / "golden"))
import ncta_cases as N  # noqa: E402

GOLD = Path(__file__).resolve().parent / "golden" / "ncta"


@pytest.fixture(scope="module")
def dev():
    from nocta_b200 import capi, configs
    r = configs.Runner(configs.load_library(), on_device=True)
    lib = N.bind(r.api.lib)
    lib.nc_cuda_set_math_mode.argtypes = [C.c_int]
    SDP = C.POINTER(N.StateDict)
    lib.nc_optimizer_state_dict.restype = SDP
    lib.nc_optimizer_state_dict.argtypes = [capi.OptimizerP]
    lib.nc_optimizer_load_state_dict.restype = C.c_int
    lib.nc_optimizer_load_state_dict.argtypes = [capi.OptimizerP, SDP]
    return r


def test_device_tensors_write_the_reference_bytes(dev, tmp_path):
    from nocta_b200 import capi
    for name, path in N.write_all(dev, tmp_path).items():
        assert path.read_bytes() == (GOLD / name).read_bytes(), name
    root, mods = N.build_model(dev)
    assert dev.api.lib.nc_module_load(root, str(GOLD / "module.ncta").encode()) == 0
    for name, w in N.weights().items():
        mod, pname = name.rsplit(".", 1)
        p = dev.api.nc_module_get_param(mods[mod], pname.encode())
        assert p.contents.storage.contents.device == capi.NC_DEVICE_CUDA
        assert np.array_equal(dev.api.to_numpy(p), w), name
    t = dev.api.lib.nc_tensor_load(str(GOLD / "tensor.ncta").encode())
    assert t.contents.storage.contents.device == capi.NC_DEVICE_CUDA


@pytest.mark.parametrize("name", ["lenet", "convbn"])
def test_resume_from_checkpoint_is_bit_exact(dev, tmp_path, name):
    """3 steps straight == 2 steps, checkpoint, fresh process state, load, 1 step (SGD momentum / AdamW)."""
    from nocta_b200 import configs
    a, lib = dev.api, dev.api.lib
    kw = dict(batch=16) if name == "convbn" else {}
    path = str(tmp_path / f"{name}.ncta").encode()
    lib.nc_cuda_set_math_mode(3)
    try:
        def steps(net, forward, kind, tensors, n):
            for _ in range(n):
                configs.train_step(dev, net, forward, kind, tensors)
                net.free_step_tensors()

        net, forward, kind, data = configs.BUILDERS[name](dev, **kw)
        tensors = configs.upload(dev, kind, data)
        steps(net, forward, kind, tensors, 3)
        straight = {n: a.to_numpy(p) for n, p in net.named_params()}

        net1, forward1, _, _ = configs.BUILDERS[name](dev, **kw)
        steps(net1, forward1, kind, tensors, 2)
        ck = N.Checkpoint()
        ck.model_state = lib.nc_state_dict_create()
        for n, p in net1.named_params():
            lib.nc_state_dict_add(ck.model_state, n.encode(), a.nc_tensor_clone(p))
        ck.optimizer_state = lib.nc_optimizer_state_dict(net1.optimizer)
        ck.epoch, ck.loss = 2, 1.5
        assert lib.nc_checkpoint_save(C.byref(ck), path) == 0
        assert lib.nc_file_verify(path)

        net2, forward2, _, _ = configs.BUILDERS[name](dev, seed=99, **kw)  # different initial weights on purpose
        loaded = lib.nc_checkpoint_load(path)
        assert loaded and loaded.contents.epoch == 2 and loaded.contents.loss == 1.5
        state = N.read_state_dict(dev, loaded.contents.model_state)
        for n, p in net2.named_params():
            dev.load(p, state[n])
        assert lib.nc_optimizer_load_state_dict(net2.optimizer, loaded.contents.optimizer_state) == 0
        assert net2.optimizer.contents.t == 2
        steps(net2, forward2, kind, tensors, 1)
        resumed = {n: a.to_numpy(p) for n, p in net2.named_params()}
        for n in straight:
            assert np.array_equal(straight[n], resumed[n]), n
        lib.nc_checkpoint_free(loaded)
    finally:
        lib.nc_cuda_set_math_mode(0)
