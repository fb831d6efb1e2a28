"""The double-buffered input feeder: batches uploaded on the copy stream must arrive intact and in order.
Each step's loss through the feeder is compared bit for bit with the loss of the same step fed by plain
nc_tensor_from_data uploads (same library, same kernels, FP32 SIMT mode)."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def test_feeder_delivers_each_batch_in_order():
    from nocta_b200 import capi, configs
    api = configs.load_library()
    r = configs.Runner(api, on_device=True)
    lib = api.lib
    lib.nc_cuda_set_math_mode.argtypes = [C.c_int]
    lib.nc_cuda_host_alloc.restype = C.c_void_p
    lib.nc_cuda_host_alloc.argtypes = [C.c_size_t]
    lib.nc_cuda_host_free.argtypes = [C.c_void_p]
    TP = C.POINTER(capi.Tensor)
    lib.nc_feeder_create.restype = C.c_void_p
    lib.nc_feeder_create.argtypes = [C.c_int, C.POINTER(C.c_size_t), C.c_size_t, C.c_int, C.POINTER(C.c_size_t), C.c_size_t, C.c_int]
    lib.nc_feeder_submit.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
    lib.nc_feeder_acquire.argtypes = [C.c_void_p, C.c_int, C.POINTER(TP), C.POINTER(TP)]
    lib.nc_feeder_release.argtypes = [C.c_void_p, C.c_int]
    lib.nc_feeder_wait.argtypes = [C.c_void_p, C.c_int]
    lib.nc_feeder_free.argtypes = [C.c_void_p]
    lib.nc_feeder_free.restype = None
    lib.nc_cuda_set_math_mode(3)
    try:
        steps = 5
        rng = np.random.default_rng(5)

        def batches(shape_x, n):
            return [(rng.standard_normal(shape_x).astype(np.float32), rng.integers(0, 10, shape_x[0]).astype(np.int64)) for _ in range(n)]

        def losses(feed):
            net, forward, kind, data = configs.build_lenet(r)
            out = feed(net, forward, kind, data)
            return out

        data_batches = None

        def plain(net, forward, kind, data):
            nonlocal data_batches
            data_batches = batches(data[0].shape, steps)
            res = []
            for x, y in data_batches:
                ts = (r.tensor(x), r.tensor(y))
                loss = configs.train_step(r, net, forward, kind, ts)
                res.append(float(api.to_numpy(loss).ravel()[0]))
                net.free_step_tensors()
                configs.free_inputs(r, kind, ts)
            return res

        def fed(net, forward, kind, data):
            xs, ys = data_batches[0]
            pinned = []
            for x, y in data_batches:  # every batch in its own pinned buffer
                px, py = lib.nc_cuda_host_alloc(x.nbytes), lib.nc_cuda_host_alloc(y.nbytes)
                C.memmove(px, x.ctypes.data, x.nbytes)
                C.memmove(py, y.ctypes.data, y.nbytes)
                pinned.append((px, py))
            f = lib.nc_feeder_create(2, capi.shape_arr(xs.shape), xs.ndim, capi.NC_F32, capi.shape_arr(ys.shape), ys.ndim, capi.NC_I64)
            assert f
            # misuse is reported, not executed
            assert lib.nc_feeder_acquire(f, 0, None, None) != 0      # nothing submitted
            assert lib.nc_feeder_submit(f, 5, pinned[0][0], pinned[0][1]) != 0  # no such slot
            res = []
            assert lib.nc_feeder_submit(f, 0, *pinned[0]) == 0
            assert lib.nc_feeder_submit(f, 0, *pinned[0]) != 0       # already in flight
            for i in range(steps):
                slot = i & 1
                xt, yt = TP(), TP()
                assert lib.nc_feeder_acquire(f, slot, C.byref(xt), C.byref(yt)) == 0
                if i + 1 < steps:
                    assert lib.nc_feeder_submit(f, slot ^ 1, *pinned[i + 1]) == 0
                loss = configs.train_step(r, net, forward, kind, (xt, yt))
                res.append(float(api.to_numpy(loss).ravel()[0]))
                net.free_step_tensors()
                assert lib.nc_feeder_release(f, slot) == 0
            assert lib.nc_feeder_wait(f, (steps - 1) & 1) == 0
            lib.nc_feeder_free(f)
            for px, py in pinned:
                lib.nc_cuda_host_free(px)
                lib.nc_cuda_host_free(py)
            return res

        a = losses(plain)
        b = losses(fed)
        assert a == b, (a, b)
        assert len(set(a)) == steps  # different batches give different losses, so order matters
    finally:
        lib.nc_cuda_set_math_mode(0)
