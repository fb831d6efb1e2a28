"""ctypes binding of the nc_* C API (tensors, autograd, nn modules, optimizers).

The same declarations serve two shared objects, because the API is the drop-in boundary:
  - nocta_b200/lib/libnocta.so : this repository's host library (CUDA device storage)
  - a CPU build of the reference library (test oracle), loaded by oracle/ref_lib.py

The struct layouts mirror the public C structs (include/nocta/nocta.h here; in the reference
include/nocta/core/tensor.h:16-39, core/memory.h:64-70, nn/module.h:20-44, optim/optimizer.h:16-33).
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

NC_MAX_DIMS = 8
NC_F32, NC_F64, NC_I32, NC_I64, NC_U8, NC_BOOL = range(6)
NC_DEVICE_CPU, NC_DEVICE_CUDA = 0, 1
_NP_DTYPES = {NC_F32: np.float32, NC_F64: np.float64, NC_I32: np.int32, NC_I64: np.int64, NC_U8: np.uint8,
              NC_BOOL: np.uint8}
_NC_OF_NP = {np.dtype(np.float32): NC_F32, np.dtype(np.float64): NC_F64, np.dtype(np.int32): NC_I32,
             np.dtype(np.int64): NC_I64, np.dtype(np.uint8): NC_U8}


class Storage(C.Structure):
    _fields_ = [("data", C.c_void_p), ("cuda_data", C.c_void_p), ("size", C.c_size_t), ("refcount", C.c_int),
                ("device", C.c_int)]


class Tensor(C.Structure):
    pass


Tensor._fields_ = [
    ("storage", C.POINTER(Storage)), ("offset", C.c_size_t), ("ndim", C.c_size_t),
    ("shape", C.c_size_t * NC_MAX_DIMS), ("strides", C.c_size_t * NC_MAX_DIMS), ("numel", C.c_size_t),
    ("dtype", C.c_int), ("requires_grad", C.c_bool), ("grad", C.POINTER(Tensor)), ("grad_fn", C.c_void_p),
    ("is_leaf", C.c_bool), ("is_contiguous", C.c_bool), ("is_reachable", C.c_bool),
]
TensorP = C.POINTER(Tensor)


class Module(C.Structure):
    _fields_ = [
        ("name", C.c_char * 64), ("params", TensorP * 64), ("param_names", C.c_char_p * 64), ("n_params", C.c_size_t),
        ("submodules", C.c_void_p * 32), ("submodule_names", C.c_char_p * 32), ("n_submodules", C.c_size_t),
        ("forward", C.c_void_p), ("training", C.c_bool), ("extra", C.c_void_p), ("free_extra", C.c_void_p),
    ]


ModuleP = C.POINTER(Module)


class Optimizer(C.Structure):
    _fields_ = [("params", TensorP * 256), ("n_params", C.c_size_t), ("lr", C.c_double), ("step", C.c_void_p),
                ("state", C.c_void_p), ("free_state", C.c_void_p), ("t", C.c_size_t)]


OptimizerP = C.POINTER(Optimizer)


class SgdConfig(C.Structure):
    _fields_ = [("momentum", C.c_double), ("dampening", C.c_double), ("weight_decay", C.c_double),
                ("nesterov", C.c_bool)]


class AdamConfig(C.Structure):
    _fields_ = [("beta1", C.c_double), ("beta2", C.c_double), ("eps", C.c_double), ("weight_decay", C.c_double),
                ("amsgrad", C.c_bool)]


_sz = C.c_size_t
_szp = C.POINTER(C.c_size_t)
_SIGS = {
    # tensors
    "nc_tensor_empty": (TensorP, [_szp, _sz, C.c_int]),
    "nc_tensor_zeros": (TensorP, [_szp, _sz, C.c_int]),
    "nc_tensor_from_data": (TensorP, [C.c_void_p, _szp, _sz, C.c_int]),
    "nc_tensor_scalar": (TensorP, [C.c_double, C.c_int]),
    "nc_tensor_clone": (TensorP, [TensorP]),
    "nc_tensor_free": (None, [TensorP]),
    "nc_tensor_reshape": (TensorP, [TensorP, _szp, _sz]),
    "nc_tensor_contiguous": (TensorP, [TensorP]),
    "nc_tensor_transpose": (TensorP, [TensorP, _sz, _sz]),
    "nc_tensor_requires_grad_": (None, [TensorP, C.c_bool]),
    "nc_tensor_zero_grad_": (None, [TensorP]),
    "nc_tensor_fill_": (None, [TensorP, C.c_double]),
    "nc_tensor_get_flat": (C.c_double, [TensorP, _sz]),
    "nc_tensor_to_device": (None, [TensorP, C.c_int]),
    # autograd
    "nc_backward": (C.c_int, [TensorP, TensorP]),
    "nc_backward_scalar": (C.c_int, [TensorP]),
    "nc_set_grad_enabled": (None, [C.c_int]),
    # ops
    "nc_add": (TensorP, [TensorP, TensorP]),
    "nc_mul": (TensorP, [TensorP, TensorP]),
    "nc_add_": (None, [TensorP, TensorP]),
    "nc_matmul": (TensorP, [TensorP, TensorP]),
    "nc_relu": (TensorP, [TensorP]),
    "nc_gelu": (TensorP, [TensorP]),
    "nc_softmax": (TensorP, [TensorP, C.c_int]),
    "nc_sum": (TensorP, [TensorP, C.c_int, C.c_bool]),
    "nc_argmax": (TensorP, [TensorP, C.c_int, C.c_bool]),
    "nc_cross_entropy_loss": (TensorP, [TensorP, TensorP]),
    "nc_mse_loss": (TensorP, [TensorP, TensorP]),
    # nn
    "nc_module_forward": (TensorP, [ModuleP, TensorP]),
    "nc_module_free": (None, [ModuleP]),
    "nc_module_get_param": (TensorP, [ModuleP, C.c_char_p]),
    "nc_module_zero_grad": (None, [ModuleP]),
    "nc_module_train": (None, [ModuleP, C.c_bool]),
    "nc_module_num_parameters": (_sz, [ModuleP]),
    "nc_linear": (ModuleP, [_sz, _sz, C.c_bool]),
    "nc_linear_forward": (TensorP, [TensorP, TensorP, TensorP]),
    "nc_conv2d": (ModuleP, [_sz, _sz, _sz, _sz, _sz, C.c_bool]),
    "nc_conv2d_forward": (TensorP, [TensorP, TensorP, TensorP, _sz, _sz]),
    "nc_maxpool2d": (ModuleP, [_sz, _sz]),
    "nc_maxpool2d_forward": (TensorP, [TensorP, _sz, _sz]),
    "nc_flatten": (ModuleP, []),
    "nc_batchnorm2d": (ModuleP, [_sz]),
    "nc_batchnorm2d_forward_fn": (TensorP, [TensorP, TensorP, TensorP, TensorP, TensorP, C.c_bool, C.c_double,
                                            C.c_double]),
    "nc_layernorm": (ModuleP, [_szp, _sz]),
    "nc_layernorm_forward_fn": (TensorP, [TensorP, _szp, _sz, TensorP, TensorP, C.c_double]),
    # optim
    "nc_sgd": (OptimizerP, [C.c_double, SgdConfig]),
    "nc_sgd_momentum": (OptimizerP, [ModuleP, C.c_double, C.c_double]),
    "nc_adam": (OptimizerP, [C.c_double, AdamConfig]),
    "nc_adamw": (OptimizerP, [ModuleP, C.c_double, C.c_double]),
    "nc_optimizer_add_param": (None, [OptimizerP, TensorP]),
    "nc_optimizer_add_module": (None, [OptimizerP, ModuleP]),
    "nc_optimizer_step": (None, [OptimizerP]),
    "nc_optimizer_zero_grad": (None, [OptimizerP]),
    "nc_optimizer_free": (None, [OptimizerP]),
}


def shape_arr(shape):
    return (C.c_size_t * len(shape))(*[int(s) for s in shape])


class NoctaAPI:
    """A loaded library exporting the nc_* API, plus numpy conveniences for the harness."""

    def __init__(self, path: Path | str, optional=()):
        path = Path(path)
        if not path.exists():
            raise RuntimeError(f"{path} is missing")
        self.path = path
        self.lib = C.CDLL(str(path), mode=C.RTLD_LOCAL)
        for name, (res, args) in _SIGS.items():
            try:
                fn = getattr(self.lib, name)
            except AttributeError:
                if name in optional:
                    continue
                raise
            fn.restype = res
            fn.argtypes = args
            setattr(self, name, fn)

    # ---- numpy <-> tensor ----
    def from_numpy(self, a: np.ndarray, requires_grad: bool = False, device: int = NC_DEVICE_CPU):
        a = np.ascontiguousarray(a)
        t = self.nc_tensor_from_data(a.ctypes.data_as(C.c_void_p), shape_arr(a.shape), a.ndim, _NC_OF_NP[a.dtype])
        if not t:
            raise RuntimeError("nc_tensor_from_data failed")
        if device != NC_DEVICE_CPU:
            self.nc_tensor_to_device(t, device)
        if requires_grad:
            self.nc_tensor_requires_grad_(t, True)
        return t

    def to_numpy(self, t) -> np.ndarray:
        """Dense copy of the tensor's logical contents (honours strides; pulls device data back)."""
        if not t:
            raise RuntimeError("null tensor")
        tt = t.contents
        if tt.storage.contents.device != NC_DEVICE_CPU:
            c = self.nc_tensor_clone(t)
            self.nc_tensor_to_device(c, NC_DEVICE_CPU)
            out = self.to_numpy(c)
            self.nc_tensor_free(c)
            return out
        dt = np.dtype(_NP_DTYPES[tt.dtype])
        shape = tuple(tt.shape[i] for i in range(tt.ndim))
        strides = tuple(tt.strides[i] * dt.itemsize for i in range(tt.ndim))
        base = tt.storage.contents.data + tt.offset * dt.itemsize
        if tt.numel == 0:
            return np.zeros(shape, dt)
        span = 1 + sum((s - 1) * st for s, st in zip(shape, (tt.strides[i] for i in range(tt.ndim))))
        buf = (C.c_char * (span * dt.itemsize)).from_address(base)
        flat = np.frombuffer(buf, dtype=dt, count=span)
        view = np.lib.stride_tricks.as_strided(flat, shape, strides, writeable=False)
        return np.array(view, copy=True)

    def grad_numpy(self, t):
        g = t.contents.grad
        return self.to_numpy(g) if g else None

    def set_data(self, t, a: np.ndarray) -> None:
        """Overwrite a (CPU-resident, contiguous) tensor's contents."""
        tt = t.contents
        a = np.ascontiguousarray(a, dtype=_NP_DTYPES[tt.dtype])
        assert a.size == tt.numel, (a.size, tt.numel)
        assert tt.storage.contents.device == NC_DEVICE_CPU and tt.is_contiguous
        C.memmove(tt.storage.contents.data + tt.offset * a.itemsize, a.ctypes.data, a.nbytes)

    def module_params(self, m):
        mm = m.contents
        return [(mm.param_names[i].decode(), mm.params[i]) for i in range(mm.n_params)]
