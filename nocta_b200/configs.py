"""The five training configurations, written once against the nc_* C API.

The same driver code runs on any library that exports that API: this repository's libnocta.so
(device tensors, CUDA kernels) and — in the tests and the CPU-baseline leg of the bench — a CPU
build of the reference.  Two operations are looked up by capability because the reference lacks
their autograd: `flatten` (nc_flatten_forward here, a test shim there) and `gelu`.

Every tensor value comes from numpy `default_rng(seed)` so both sides see identical inputs,
labels, masks and initial weights (the reference cannot be seeded: src/core/tensor.c:23-28).
Synthetic data only: the shapes are MNIST-/CIFAR-like, no dataset items are used.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import numpy as np

from . import capi


def _kaiming(rng, shape):
    fan_in = int(np.prod(shape[1:]))
    return (rng.standard_normal(shape) * np.sqrt(2.0 / fan_in)).astype(np.float32)


def _uniform_fan(rng, shape, fan_in):
    b = 1.0 / np.sqrt(fan_in)
    return rng.uniform(-b, b, shape).astype(np.float32)


@dataclass
class Net:
    """A model built from nc_* modules plus the numpy copies of what was loaded into them."""
    api: object
    modules: dict = field(default_factory=dict)      # name -> nc_module*
    order: list = field(default_factory=list)        # parameter order: (module name, param name)
    optimizer: object = None
    keep: list = field(default_factory=list)         # tensors that must outlive backward

    def param(self, mod: str, name: str):
        return self.api.nc_module_get_param(self.modules[mod], name.encode())

    def named_params(self):
        return [(f"{m}.{p}", self.param(m, p)) for m, p in self.order]

    def free_step_tensors(self):
        for t in reversed(self.keep):
            self.api.nc_tensor_free(t)
        self.keep.clear()


class Runner:
    """Binds a loaded library: uploads numpy data, knows which flatten / gelu to call."""

    def __init__(self, api, on_device: bool):
        self.api = api
        self.on_device = on_device
        lib = api.lib
        if hasattr(lib, "nc_flatten_forward"):
            self.flatten = self._bind(lib.nc_flatten_forward)
            self.gelu = api.nc_gelu
            lib.nc_batchnorm2d_relu.restype = capi.TensorP
            lib.nc_batchnorm2d_relu.argtypes = [capi.ModuleP, capi.TensorP]
            self._bn_relu = lib.nc_batchnorm2d_relu
            lib.nc_batchnorm2d_relu_maxpool2.restype = capi.TensorP
            lib.nc_batchnorm2d_relu_maxpool2.argtypes = [capi.ModuleP, capi.TensorP]
            self._bn_relu_pool = lib.nc_batchnorm2d_relu_maxpool2
        else:  # reference build: differentiable shims compiled next to it
            self.flatten = api.shim_flatten
            self.gelu = api.shim_gelu
            self._bn_relu = None
        if on_device:
            lib.nc_init.restype = None
            lib.nc_init()
            self._h2d = lib.nc_cuda_memcpy_h2d
            self._h2d.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
            self._h2d.restype = None

    @staticmethod
    def _bind(fn):
        fn.restype = capi.TensorP
        fn.argtypes = [capi.TensorP]
        return fn

    def bn_relu(self, keep, module, x):
        """BatchNorm2d + ReLU: one fused call where the library has it, else the two reference calls."""
        if self._bn_relu is not None:
            return _k(keep, self._bn_relu(module, x))
        h = _k(keep, self.api.nc_module_forward(module, x))
        return _k(keep, self.api.nc_relu(h))

    def bn_relu_pool(self, keep, module, x):
        """BatchNorm2d + ReLU + MaxPool(2, 2): one fused call where the library has it, else the reference calls."""
        fused = getattr(self, "_bn_relu_pool", None)
        if fused is not None:
            return _k(keep, fused(module, x))
        return _k(keep, self.api.nc_maxpool2d_forward(self.bn_relu(keep, module, x), 2, 2))

    def tensor(self, a: np.ndarray, requires_grad=False):
        # after nc_init the default device is CUDA, so from_data uploads
        return self.api.from_numpy(a, requires_grad=requires_grad)

    def load(self, t, a: np.ndarray):
        """Overwrite a parameter tensor with `a` wherever it lives."""
        tt = t.contents
        a = np.ascontiguousarray(a, dtype=np.float32)
        assert a.size == tt.numel, (a.size, tt.numel)
        if tt.storage.contents.device == capi.NC_DEVICE_CUDA:
            self._h2d(tt.storage.contents.cuda_data + tt.offset * 4, a.ctypes.data, a.nbytes)
        else:
            self.api.set_data(t, a)


# ----------------------------------------------------------------------------------------------
# model definitions
# ----------------------------------------------------------------------------------------------
def _add(net: Net, r: Runner, name: str, module, weights: dict):
    net.modules[name] = module
    for pname, value in weights.items():
        r.load(net.param(name, pname), value)
        net.order.append((name, pname))


def build_lenet(r: Runner, seed=1235):
    """Config 1: LeNet-style CNN, batch 64, SGD lr 0.01 momentum 0.9, all weights N(0, 0.1^2)."""
    api, rng = r.api, np.random.default_rng(seed)
    net = Net(api)
    n = lambda *s: (rng.standard_normal(s) * 0.1).astype(np.float32)
    _add(net, r, "conv1", api.nc_conv2d(1, 6, 5, 1, 0, True), {"weight": n(6, 1, 5, 5), "bias": n(6)})
    _add(net, r, "conv2", api.nc_conv2d(6, 16, 5, 1, 0, True), {"weight": n(16, 6, 5, 5), "bias": n(16)})
    _add(net, r, "fc1", api.nc_linear(256, 120, True), {"weight": n(120, 256), "bias": n(120)})
    _add(net, r, "fc2", api.nc_linear(120, 84, True), {"weight": n(84, 120), "bias": n(84)})
    _add(net, r, "fc3", api.nc_linear(84, 10, True), {"weight": n(10, 84), "bias": n(10)})
    net.optimizer = _sgd(api, net, 0.01, 0.9)
    x = rng.random((64, 1, 28, 28), dtype=np.float32)
    y = rng.integers(0, 10, 64).astype(np.int64)

    def forward(net, xt):
        a, k, m = net.api, net.keep, net.modules
        h = _k(k, a.nc_module_forward(m["conv1"], xt))
        h = _k(k, a.nc_relu(h))
        h = _k(k, a.nc_maxpool2d_forward(h, 2, 2))
        h = _k(k, a.nc_module_forward(m["conv2"], h))
        h = _k(k, a.nc_relu(h))
        h = _k(k, a.nc_maxpool2d_forward(h, 2, 2))
        h = _k(k, r.flatten(h))
        h = _k(k, a.nc_relu(_k(k, a.nc_module_forward(m["fc1"], h))))
        h = _k(k, a.nc_relu(_k(k, a.nc_module_forward(m["fc2"], h))))
        return _k(k, a.nc_module_forward(m["fc3"], h))

    return net, forward, "ce", (x, y)


def build_convbn(r: Runner, seed=1236, batch=128):
    """Config 2: conv-BN CNN, batch 128, AdamW lr 1e-3 wd 0.01, Kaiming-normal convs, no conv bias."""
    api, rng = r.api, np.random.default_rng(seed)
    net = Net(api)
    _add(net, r, "conv1", api.nc_conv2d(3, 64, 3, 1, 1, False), {"weight": _kaiming(rng, (64, 3, 3, 3))})
    _add(net, r, "bn1", api.nc_batchnorm2d(64), {})
    _add(net, r, "conv2", api.nc_conv2d(64, 128, 3, 1, 1, False), {"weight": _kaiming(rng, (128, 64, 3, 3))})
    _add(net, r, "bn2", api.nc_batchnorm2d(128), {})
    _add(net, r, "fc", api.nc_linear(8192, 10, True),
         {"weight": _uniform_fan(rng, (10, 8192), 8192), "bias": _uniform_fan(rng, (10,), 8192)})
    for bn in ("bn1", "bn2"):
        net.order += [(bn, p) for p in ("weight", "bias", "running_mean", "running_var")]
    # nc_adamw(module, ...) takes one module; the networks here are several, so the optimizer is filled
    # module by module, BN running statistics included (they are registered parameters and get decayed)
    net.optimizer = _adam(api, net, 1e-3, 0.01)
    x = rng.standard_normal((batch, 3, 32, 32)).astype(np.float32)
    y = rng.integers(0, 10, batch).astype(np.int64)

    def forward(net, xt):
        a, k, m = net.api, net.keep, net.modules
        h = xt
        for c, b in (("conv1", "bn1"), ("conv2", "bn2")):
            h = _k(k, a.nc_module_forward(m[c], h))
            h = r.bn_relu(k, m[b], h)
            h = _k(k, a.nc_maxpool2d_forward(h, 2, 2))
        h = _k(k, r.flatten(h))
        return _k(k, a.nc_module_forward(m["fc"], h))

    return net, forward, "ce", (x, y)


def build_mlp(r: Runner, seed=1238, batch=4096, width=1024, hidden=4096, blocks=4):
    """Config 4: x + LayerNorm(mask * fc2(gelu(fc1(x)))) four times, MSE, Adam lr 1e-4."""
    api, rng = r.api, np.random.default_rng(seed)
    net = Net(api)
    for b in range(blocks):
        _add(net, r, f"fc1_{b}", api.nc_linear(width, hidden, True),
             {"weight": _uniform_fan(rng, (hidden, width), width), "bias": _uniform_fan(rng, (hidden,), width)})
        _add(net, r, f"fc2_{b}", api.nc_linear(hidden, width, True),
             {"weight": _uniform_fan(rng, (width, hidden), hidden), "bias": _uniform_fan(rng, (width,), hidden)})
        _add(net, r, f"ln_{b}", api.nc_layernorm(capi.shape_arr([width]), 1), {})
        net.order += [(f"ln_{b}", "weight"), (f"ln_{b}", "bias")]
    net.optimizer = _adam(api, net, 1e-4, 0.0)
    x = rng.standard_normal((batch, width)).astype(np.float32)
    target = rng.standard_normal((batch, width)).astype(np.float32)
    masks = [(rng.random((batch, width)) >= 0.1).astype(np.float32) / np.float32(0.9) for _ in range(blocks)]

    def forward(net, xt, mask_tensors):
        a, k, m = net.api, net.keep, net.modules
        h = xt
        for b in range(blocks):
            u = _k(k, a.nc_module_forward(m[f"fc1_{b}"], h))
            u = _k(k, r.gelu(u))
            u = _k(k, a.nc_module_forward(m[f"fc2_{b}"], u))
            u = _k(k, a.nc_mul(u, mask_tensors[b]))
            u = _k(k, a.nc_module_forward(m[f"ln_{b}"], u))
            h = _k(k, a.nc_add(h, u))
        return h

    return net, forward, "mse", (x, target, masks)


def build_vgg(r: Runner, seed=1239, batch=256, classes=100, rank=0, size=64, widths=(64, 128, 256)):
    """Config 5: conv(3->64->64) pool conv(->128->128) pool conv(->256->256) pool, each conv 3x3 p1 +
    BN + ReLU, then linear -> classes; SGD lr 0.01 momentum 0.9.  Weights depend on `seed` only
    (every rank holds the same replica); the data shard depends on seed + rank."""
    api = r.api
    wrng = np.random.default_rng(seed)
    net = Net(api)
    cin, idx = 3, 0
    stages = []
    for w in widths:
        names = []
        for _ in range(2):
            _add(net, r, f"conv{idx}", api.nc_conv2d(cin, w, 3, 1, 1, False), {"weight": _kaiming(wrng, (w, cin, 3, 3))})
            _add(net, r, f"bn{idx}", api.nc_batchnorm2d(w), {})
            net.order += [(f"bn{idx}", p) for p in ("weight", "bias")]
            names.append((f"conv{idx}", f"bn{idx}"))
            cin = w
            idx += 1
        stages.append(names)
    feat = widths[-1] * (size // 8) ** 2
    _add(net, r, "fc", api.nc_linear(feat, classes, True),
         {"weight": _uniform_fan(wrng, (classes, feat), feat), "bias": _uniform_fan(wrng, (classes,), feat)})
    net.optimizer = _sgd(api, net, 0.01, 0.9, skip=("running_mean", "running_var"))
    drng = np.random.default_rng(seed + 1000 + rank)
    x = drng.standard_normal((batch, 3, size, size)).astype(np.float32)
    y = drng.integers(0, classes, batch).astype(np.int64)

    def forward(net, xt):
        a, k, m = net.api, net.keep, net.modules
        h = xt
        for names in stages:
            for i, (c, b) in enumerate(names):
                h = _k(k, a.nc_module_forward(m[c], h))
                h = r.bn_relu_pool(k, m[b], h) if i == len(names) - 1 else r.bn_relu(k, m[b], h)
        h = _k(k, r.flatten(h))
        return _k(k, a.nc_module_forward(m["fc"], h))

    return net, forward, "ce", (x, y)


def _k(keep, t):
    if not t:
        raise RuntimeError("an nc_* call returned NULL")
    keep.append(t)
    return t


def _sgd(api, net, lr, momentum, skip=()):
    cfg = capi.SgdConfig(momentum, 0.0, 0.0, False)
    opt = api.nc_sgd(lr, cfg)
    for mname, mod in net.modules.items():
        for pname, p in api.module_params(mod):
            if pname not in skip:
                api.nc_optimizer_add_param(opt, p)
    return opt


def _adam(api, net, lr, wd):
    cfg = capi.AdamConfig(0.9, 0.999, 1e-8, wd, False)
    opt = api.nc_adam(lr, cfg)
    for mod in net.modules.values():
        api.nc_optimizer_add_module(opt, mod)
    return opt


# ----------------------------------------------------------------------------------------------
# one training step
# ----------------------------------------------------------------------------------------------
def train_step(r: Runner, net: Net, forward, loss_kind, tensors, after_backward=None):
    """zero_grad -> forward -> loss -> backward -> [after_backward()] -> optimizer step.  Returns the
    loss tensor (kept alive in net.keep until free_step_tensors).  `after_backward` is where a
    data-parallel caller sums the gradients across ranks."""
    api = r.api
    api.nc_optimizer_zero_grad(net.optimizer)
    if loss_kind == "ce":
        xt, yt = tensors
        out = forward(net, xt)
        loss = _k(net.keep, api.nc_cross_entropy_loss(out, yt))
    else:
        xt, tt, masks = tensors
        out = forward(net, xt, masks)
        loss = _k(net.keep, api.nc_mse_loss(out, tt))
    rc = api.nc_backward_scalar(loss)
    if rc != 0:
        raise RuntimeError(f"nc_backward_scalar failed with {rc}")
    if after_backward is not None:
        after_backward()
    api.nc_optimizer_step(net.optimizer)
    return loss


def eval_accuracy(r: Runner, net: Net, forward, x: np.ndarray, labels: np.ndarray):
    """The inference half of the reference's training loop (examples/mnist.c:359-381): every module in
    eval mode (BatchNorm normalises with its running statistics, src/nn/batchnorm.c:315-319), one forward,
    row argmax (src/ops/reduction.c:473-513), count of correct predictions.  Returns (logits, predictions,
    correct); the modules are put back into training mode."""
    api = r.api
    for m in net.modules.values():
        api.nc_module_train(m, False)
    xt = r.tensor(x)
    try:
        out = forward(net, xt)
        pred_t = _k(net.keep, api.nc_argmax(out, 1, False))
        logits = api.to_numpy(out)
        pred = api.to_numpy(pred_t).astype(np.int64).reshape(-1)
    finally:
        net.free_step_tensors()
        api.nc_tensor_free(xt)
        for m in net.modules.values():
            api.nc_module_train(m, True)
    return logits, pred, int((pred == labels.reshape(-1)).sum())


def upload(r: Runner, loss_kind, data):
    if loss_kind == "ce":
        x, y = data
        return r.tensor(x), r.tensor(y)
    x, t, masks = data
    return r.tensor(x), r.tensor(t), [r.tensor(m) for m in masks]


def free_inputs(r: Runner, loss_kind, tensors):
    if loss_kind == "ce":
        for t in tensors:
            r.api.nc_tensor_free(t)
    else:
        x, t, masks = tensors
        for u in [x, t, *masks]:
            r.api.nc_tensor_free(u)


BUILDERS = {"lenet": build_lenet, "convbn": build_convbn, "mlp": build_mlp, "vgg": build_vgg}


def load_library():
    """This repository's host library (fails loudly when it has not been built)."""
    from pathlib import Path
    path = Path(__file__).resolve().parent / "lib" / "libnocta.so"
    if not path.exists():
        raise RuntimeError(f"{path} is missing: run `python -m nocta_b200.build`")
    return capi.NoctaAPI(path)
