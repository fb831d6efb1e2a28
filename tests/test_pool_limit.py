"""Device-pool allocation failure, injected on the host through nc_device_pool_set_limit: the call that needed the memory
returns the reference's error shape (NULL / unchanged tensor + NC_ERR_ALLOC in nc_last_error), the pool's accounting stays
consistent, and work resumes once the cap is lifted.  The CPU case needs no GPU (the cap refuses before the driver is asked);
the GPU case interrupts a training step in the middle of its forward pass."""
import ctypes as C

import numpy as np
import pytest

NC_ERR_ALLOC = 2


class PoolStats(C.Structure):
    _fields_ = [(n, C.c_size_t) for n in ("bytes_reserved", "bytes_in_use", "peak_in_use", "cuda_mallocs", "pool_hits")]


def bind(lib):
    lib.nc_device_pool_set_limit.argtypes = [C.c_size_t]
    lib.nc_device_pool_set_limit.restype = None
    lib.nc_device_pool_get_limit.restype = C.c_size_t
    lib.nc_device_pool_get_stats.restype = PoolStats
    lib.nc_device_pool_release.restype = None
    return lib


def last_error(lib):
    return C.c_int.in_dll(lib, "nc_last_error").value


def clear_error(lib):
    C.c_int.in_dll(lib, "nc_last_error").value = 0


def test_refused_allocation_leaves_the_tensor_on_the_host_and_sets_the_error():
    from nocta_b200 import capi, configs
    api = configs.load_library()
    lib = bind(api.lib)
    t = api.from_numpy(np.arange(4096, dtype=np.float32))
    before = lib.nc_device_pool_get_stats()
    lib.nc_device_pool_set_limit(before.bytes_reserved + 512)      # room for 512 bytes more, 16 KB asked
    try:
        assert lib.nc_device_pool_get_limit() == before.bytes_reserved + 512
        clear_error(lib)
        api.nc_tensor_to_device(t, capi.NC_DEVICE_CUDA)
        assert last_error(lib) == NC_ERR_ALLOC
        st = t.contents.storage.contents
        assert st.device == capi.NC_DEVICE_CPU and st.data and not st.cuda_data      # unchanged, still readable
        np.testing.assert_array_equal(api.to_numpy(t), np.arange(4096, dtype=np.float32))
        after = lib.nc_device_pool_get_stats()
        assert (after.bytes_reserved, after.bytes_in_use, after.cuda_mallocs) == (before.bytes_reserved, before.bytes_in_use, before.cuda_mallocs)
    finally:
        lib.nc_device_pool_set_limit(0)
        clear_error(lib)
        api.nc_tensor_free(t)


@pytest.mark.gpu
def test_training_step_interrupted_by_the_cap_fails_cleanly_and_resumes():
    pytest.importorskip("torch")
    from nocta_b200 import configs
    api = configs.load_library()
    lib = bind(api.lib)
    r = configs.Runner(api, on_device=True)
    kw = dict(batch=8, size=16, widths=(32, 64, 128), classes=10)
    net, forward, kind, data = configs.BUILDERS["vgg"](r, **kw)
    tensors = configs.upload(r, kind, data)
    loss0 = float(api.to_numpy(configs.train_step(r, net, forward, kind, tensors)).ravel()[0])   # warm: the pool now holds a step's blocks
    net.free_step_tensors()
    api.nc_optimizer_zero_grad(net.optimizer)     # releases the gradients now, so that the step below starts from `base`
    lib.nc_device_pool_release()
    base = lib.nc_device_pool_get_stats()
    assert base.bytes_reserved == base.bytes_in_use
    # room for one activation of 8 x 32 x 16 x 16 floats (256 KB), not for two
    room = 300 << 10
    lib.nc_device_pool_set_limit(base.bytes_reserved + room)
    try:
        clear_error(lib)
        with pytest.raises(RuntimeError):
            configs.train_step(r, net, forward, kind, tensors)
        assert last_error(lib) == NC_ERR_ALLOC
        net.free_step_tensors()
        mid = lib.nc_device_pool_get_stats()
        assert mid.bytes_reserved <= base.bytes_reserved + room
        assert mid.bytes_in_use == base.bytes_in_use                 # everything the broken step took was given back
    finally:
        lib.nc_device_pool_set_limit(0)
        clear_error(lib)
    loss1 = float(api.to_numpy(configs.train_step(r, net, forward, kind, tensors)).ravel()[0])
    assert np.isfinite(loss1) and loss1 < loss0 * 1.5                # the same network keeps training
    assert last_error(lib) == 0
    net.free_step_tensors()
    configs.free_inputs(r, kind, tensors)
    assert lib.nc_cuda_device_error_word() == 0
