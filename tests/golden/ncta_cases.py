"""Writers of .ncta files driven through the C API of whichever library the runner is bound to (the
compiled reference on the host, or this repository's library with the tensors on the CUDA device).
The same code produced the committed golden files (make_golden.py) and runs in the tests, so the files
must be byte-identical.  Reference: src/core/serialize.c:32-101, 223-306, 385-490; the single-tensor case
repeats the reference's own tests/test_io.c:5-28."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

from nocta_b200 import capi


class StateDict(C.Structure):
    _fields_ = [("names", C.POINTER(C.c_char_p)), ("tensors", C.POINTER(capi.TensorP)), ("n_tensors", C.c_size_t), ("capacity", C.c_size_t)]


class Checkpoint(C.Structure):
    _fields_ = [("model_state", C.POINTER(StateDict)), ("optimizer_state", C.POINTER(StateDict)), ("epoch", C.c_size_t), ("loss", C.c_double)]


def bind(lib):
    SDP, CKP = C.POINTER(StateDict), C.POINTER(Checkpoint)
    sig = {
        "nc_tensor_save": (C.c_int, [capi.TensorP, C.c_char_p]), "nc_tensor_load": (capi.TensorP, [C.c_char_p]),
        "nc_state_dict_create": (SDP, []), "nc_state_dict_free": (None, [SDP]),
        "nc_state_dict_add": (None, [SDP, C.c_char_p, capi.TensorP]), "nc_state_dict_get": (capi.TensorP, [SDP, C.c_char_p]),
        "nc_state_dict_save": (C.c_int, [SDP, C.c_char_p]), "nc_state_dict_load": (SDP, [C.c_char_p]),
        "nc_module_state_dict": (SDP, [capi.ModuleP]), "nc_module_load_state_dict": (C.c_int, [capi.ModuleP, SDP]),
        "nc_module_save": (C.c_int, [capi.ModuleP, C.c_char_p]), "nc_module_load": (C.c_int, [capi.ModuleP, C.c_char_p]),
        "nc_module_save_desc": (C.c_int, [capi.ModuleP, C.c_char_p, C.c_char_p]),
        "nc_checkpoint_save": (C.c_int, [CKP, C.c_char_p]), "nc_checkpoint_load": (CKP, [C.c_char_p]), "nc_checkpoint_free": (None, [CKP]),
        "nc_file_verify": (C.c_bool, [C.c_char_p]),
        "nc_module_create": (capi.ModuleP, [C.c_char_p]), "nc_module_add_submodule": (None, [capi.ModuleP, C.c_char_p, capi.ModuleP]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    return lib


def weights():
    rng = np.random.default_rng(4242)
    return {
        "features.conv.weight": rng.standard_normal((3, 2, 3, 3)).astype(np.float32),
        "features.conv.bias": rng.standard_normal(3).astype(np.float32),
        "features.bn.weight": rng.standard_normal(3).astype(np.float32),
        "features.bn.bias": rng.standard_normal(3).astype(np.float32),
        "features.bn.running_mean": rng.standard_normal(3).astype(np.float32),
        "features.bn.running_var": (rng.random(3) + 0.5).astype(np.float32),
        "head.weight": rng.standard_normal((4, 5)).astype(np.float32),
        "head.bias": rng.standard_normal(4).astype(np.float32),
    }


def build_model(r, values=None):
    """root { features { conv, bn }, head }: nested names exercise the dotted-name walk."""
    a, lib = r.api, r.api.lib
    root, features = lib.nc_module_create(b"net"), lib.nc_module_create(b"features")
    conv, bn, head = a.nc_conv2d(2, 3, 3, 1, 1, True), a.nc_batchnorm2d(3), a.nc_linear(5, 4, True)
    lib.nc_module_add_submodule(features, b"conv", conv)
    lib.nc_module_add_submodule(features, b"bn", bn)
    lib.nc_module_add_submodule(root, b"features", features)
    lib.nc_module_add_submodule(root, b"head", head)
    mods = {"features.conv": conv, "features.bn": bn, "head": head}
    if values is not None:
        for name, v in values.items():
            mod, pname = name.rsplit(".", 1)
            r.load(a.nc_module_get_param(mods[mod], pname.encode()), v)
    return root, mods


def optimizer_arrays():
    rng = np.random.default_rng(777)
    return {"step": np.array([12], np.int64), "velocity.0": rng.standard_normal((3, 2, 3, 3)).astype(np.float32),
            "velocity.6": rng.standard_normal((4, 5)).astype(np.float32)}


def write_all(r, outdir: Path) -> dict:
    """Writes tensor.ncta, module.ncta, checkpoint.ncta into outdir; returns {file name: path}."""
    a, lib = r.api, bind(r.api.lib)
    outdir.mkdir(parents=True, exist_ok=True)
    paths = {n: outdir / n for n in ("tensor.ncta", "module.ncta", "checkpoint.ncta")}
    t = np.zeros((2, 2), np.float32)
    t[0, 0], t[1, 1] = 1.23, 4.56
    assert lib.nc_tensor_save(r.tensor(t), str(paths["tensor.ncta"]).encode()) == 0
    root, _ = build_model(r, weights())
    assert lib.nc_module_save_desc(root, str(paths["module.ncta"]).encode(), b"golden module") == 0
    ck = Checkpoint()
    ck.model_state = lib.nc_module_state_dict(root)
    ck.optimizer_state = lib.nc_state_dict_create()
    for name, v in optimizer_arrays().items():
        lib.nc_state_dict_add(ck.optimizer_state, name.encode(), r.tensor(v))
    ck.epoch, ck.loss = 7, 0.123456
    assert lib.nc_checkpoint_save(C.byref(ck), str(paths["checkpoint.ncta"]).encode()) == 0
    lib.nc_state_dict_free(ck.model_state)
    lib.nc_state_dict_free(ck.optimizer_state)
    return paths


def read_state_dict(r, sd) -> dict:
    out = {}
    for i in range(sd.contents.n_tensors):
        out[sd.contents.names[i].decode()] = r.api.to_numpy(sd.contents.tensors[i])
    return out
