"""ctypes binding of the nc_cuda_* C ABI (include/nocta_cuda.h) exported by libnocta_cuda.so.

The library is the product; this module only declares argument types so that tests and the
bench can call the entry points with device pointers (e.g. torch.Tensor.data_ptr()).
Loading fails loudly when the shared object is missing: there is no other implementation.
"""
from __future__ import annotations

import ctypes as C
import re
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "lib" / "libnocta_cuda.so"
HEADER = PKG.parent / "include" / "nocta_cuda.h"

_f = C.c_float
_d = C.c_double
_i = C.c_int
_z = C.c_size_t
_p = C.c_void_p
_b = C.c_bool

# name -> (restype, argtypes)
SIGNATURES = {
    "nc_cuda_available": (_b, []),
    "nc_cuda_device_count": (_i, []),
    "nc_cuda_set_device": (None, [_i]),
    "nc_cuda_synchronize": (None, []),
    "nc_cuda_init": (None, []),
    "nc_cuda_cleanup": (None, []),
    "nc_cuda_malloc": (_p, [_z]),
    "nc_cuda_free": (None, [_p]),
    "nc_cuda_memcpy_h2d": (None, [_p, _p, _z]),
    "nc_cuda_memcpy_d2h": (None, [_p, _p, _z]),
    "nc_cuda_memcpy_d2d": (None, [_p, _p, _z]),
    "nc_cuda_memset": (None, [_p, _i, _z]),
    "nc_cuda_device_props": (_i, [_i, C.c_char_p, C.POINTER(_z), C.POINTER(_z), C.POINTER(_i)]),
    "nc_cuda_set_stream": (None, [_p]),
    "nc_cuda_get_stream": (_p, []),
    "nc_cuda_memcpy_h2d_async": (_i, [_p, _p, _z, _p]),
    "nc_cuda_memcpy_d2h_async": (_i, [_p, _p, _z, _p]),
    "nc_cuda_memset_async": (_i, [_p, _i, _z, _p]),
    "nc_cuda_host_alloc": (_p, [_z]),
    "nc_cuda_host_free": (None, [_p]),
    "nc_cuda_stream_synchronize": (_i, [_p]),
    "nc_cuda_stream_create": (_p, []),
    "nc_cuda_stream_destroy": (None, [_p]),
    "nc_cuda_event_create": (_p, []),
    "nc_cuda_event_destroy": (None, [_p]),
    "nc_cuda_event_record": (_i, [_p, _p]),
    "nc_cuda_stream_wait_event": (_i, [_p, _p]),
    "nc_cuda_event_synchronize": (_i, [_p]),
    "nc_cuda_event_create_timed": (_p, []),
    "nc_cuda_event_elapsed_ms": (_i, [_p, _p, C.POINTER(_f)]),
    "nc_cuda_last_status": (_i, []),
    "nc_cuda_last_message": (C.c_char_p, []),
    "nc_cuda_clear_status": (None, []),
    "nc_cuda_set_math_mode": (_i, [_i]),
    "nc_cuda_get_math_mode": (_i, []),
    "nc_cuda_set_round_outputs": (_i, [_i]),
    "nc_cuda_set_conv_stats": (_i, [_i]),
    "nc_cuda_offer_batchnorm_backward_sums_f32": (_i, [_p, _p, _p, _p, _p, _d, _i, C.c_longlong]),
    "nc_cuda_batchnorm_backward_fold_count": (C.c_ulonglong, []),
    "nc_cuda_set_batchnorm_backward_fold": (_i, [_i]),
    "nc_cuda_device_error_word": (C.c_uint, []),
    "nc_cuda_launch_count": (C.c_ulonglong, []),
    "nc_cuda_reset_launch_count": (None, []),
    "nc_cuda_profile_begin": (_i, []),
    "nc_cuda_profile_end": (_i, []),
    "nc_cuda_profile_categories": (_i, []),
    "nc_cuda_profile_category_name": (C.c_char_p, [_i]),
    "nc_cuda_profile_read": (_i, [_i, C.POINTER(_d), C.POINTER(C.c_ulonglong), C.POINTER(_d)]),
    # elementwise
    "nc_cuda_fill_f32": (None, [_p, _f, _z]),
    "nc_cuda_copy_f32": (None, [_p, _p, _z]),
    "nc_cuda_add_f32": (None, [_p, _p, _p, _z]),
    "nc_cuda_sub_f32": (None, [_p, _p, _p, _z]),
    "nc_cuda_mul_f32": (None, [_p, _p, _p, _z]),
    "nc_cuda_div_f32": (None, [_p, _p, _p, _z]),
    "nc_cuda_add_scalar_f32": (None, [_p, _p, _f, _z]),
    "nc_cuda_mul_scalar_f32": (None, [_p, _p, _f, _z]),
    "nc_cuda_add_broadcast_batch_f32": (None, [_p, _p, _p, _z, _i]),
    "nc_cuda_fill_f32_ex": (_i, [_p, _f, _z, _p]),
    "nc_cuda_copy_f32_ex": (_i, [_p, _p, _z, _p]),
    "nc_cuda_binary_f32_ex": (_i, [_i, _p, _p, _p, _z, _p]),
    "nc_cuda_scalar_f32_ex": (_i, [_i, _p, _p, _f, _z, _p]),
    "nc_cuda_add_broadcast_batch_f32_ex": (_i, [_p, _p, _p, _z, _i, _p]),
    "nc_cuda_strided_copy_f32_ex": (_i, [_p, _p, C.POINTER(_z), C.POINTER(_z), _p]),
    "nc_cuda_nchw_to_nhwc_f32_ex": (_i, [_p, _p, _i, _i, _i, _i, _p]),
    "nc_cuda_nhwc_to_nchw_f32_ex": (_i, [_p, _p, _i, _i, _i, _p]),
    "nc_cuda_round_tf32_f32_ex": (_i, [_p, _p, _z, _p]),
    # activations
    "nc_cuda_relu_f32": (None, [_p, _p, _z]),
    "nc_cuda_relu_backward_f32": (None, [_p, _p, _p, _z]),
    "nc_cuda_softmax_f32": (None, [_p, _p, _z, _z]),
    "nc_cuda_relu_f32_ex": (_i, [_p, _p, _z, _p]),
    "nc_cuda_relu_backward_f32_ex": (_i, [_p, _p, _p, _z, _p]),
    "nc_cuda_sigmoid_f32": (None, [_p, _p, _z]),
    "nc_cuda_sigmoid_f32_ex": (_i, [_p, _p, _z, _p]),
    "nc_cuda_sigmoid_backward_f32_ex": (_i, [_p, _p, _p, _z, _p]),
    "nc_cuda_softmax_f32_ex": (_i, [_p, _p, _z, _z, _p]),
    "nc_cuda_gelu_f32_ex": (_i, [_p, _p, _z, _p]),
    "nc_cuda_gelu_backward_f32_ex": (_i, [_p, _p, _p, _z, _p]),
    # matmul / linear
    "nc_cuda_matmul_f32": (None, [_p, _p, _p, _i, _i, _i, _f, _f, _i, _i]),
    "nc_cuda_matmul_f32_ex": (_i, [_p, _i, _p, _i, _p, _i, _i, _i, _i, _f, _f, _i, _i, _p, _p]),
    "nc_cuda_linear_forward_f32_ex": (_i, [_p, _p, _p, _p, _i, _i, _i, _p]),
    "nc_cuda_linear_backward_f32_ex": (_i, [_p, _p, _p, _p, _p, _p, _i, _i, _i, _p]),
    # reductions
    "nc_cuda_sum_f32": (_f, [_p, _z]),
    "nc_cuda_argmax_f32": (_z, [_p, _z]),
    "nc_cuda_sum_axis_f32": (None, [_p, _p, _z, _z, _z]),
    "nc_cuda_sum_axis_f32_ex": (_i, [_p, _p, _z, _z, _z, _p]),
    "nc_cuda_argmax_rows_f32_ex": (_i, [_p, _p, _z, _z, _p]),
    # conv
    "nc_cuda_conv2d_forward_f32": (None, [_p, _p, _p, _p] + [_i] * 9),
    "nc_cuda_conv2d_backward_input_f32": (None, [_p, _p, _p] + [_i] * 9),
    "nc_cuda_conv2d_backward_weight_f32": (None, [_p, _p, _p] + [_i] * 9),
    "nc_cuda_conv2d_backward_bias_f32": (None, [_p, _p, _i, _i, _i, _i]),
    "nc_cuda_conv2d_forward_f32_ex": (_i, [_p, C.POINTER(_z), _p, C.POINTER(_z), _p, _p] + [_i] * 9 + [_p]),
    "nc_cuda_conv2d_backward_input_f32_ex": (_i, [_p, C.POINTER(_z), _p, C.POINTER(_z), _p] + [_i] * 9 + [_p]),
    "nc_cuda_conv2d_backward_weight_f32_ex": (_i, [_p, _p, _p, C.POINTER(_z), _p, C.POINTER(_z)] + [_i] * 9 + [_p]),
    "nc_cuda_conv2d_backward_f32_ex": (_i, [_p, _p, _p, _p, _p, _p] + [_i] * 9 + [_p]),
    # pooling
    "nc_cuda_maxpool2d_forward_f32": (None, [_p, _p] + [_i] * 7),
    "nc_cuda_maxpool2d_backward_f32": (None, [_p, _p, _p, _p] + [_i] * 7),
    "nc_cuda_maxpool2d_forward_idx_f32_ex": (_i, [_p, _p, _p] + [_i] * 7 + [_p]),
    "nc_cuda_maxpool2d_backward_idx_f32_ex": (_i, [_p, _p, _p] + [_i] * 7 + [_p]),
    # norms
    "nc_cuda_batchnorm_forward_f32": (None, [_p] * 8 + [_i, _i, _i, _f, _f, _b]),
    "nc_cuda_batchnorm_backward_f32": (None, [_p] * 8 + [_i, _i, _i, _f]),
    "nc_cuda_batchnorm_forward_f32_ex": (_i, [_p] * 8 + [_i, _i, _i, _d, _d, _i, _i, _i, _p]),
    "nc_cuda_batchnorm_backward_f32_ex": (_i, [_p] * 10 + [_i, _i, _i, _i, _d, _i, _p]),
    "nc_cuda_batchnorm_relu_maxpool2_forward_f32_ex": (_i, [_p] * 9 + [_i] * 4 + [_d, _d, _i, _p]),
    "nc_cuda_batchnorm_relu_maxpool2_backward_f32_ex": (_i, [_p] * 10 + [_i] * 4 + [_d, _p]),
    "nc_cuda_layernorm_forward_f32_ex": (_i, [_p, _p, _p, _p, _z, _z, _d, _p]),
    "nc_cuda_layernorm_backward_f32_ex": (_i, [_p, _p, _p, _p, _p, _p, _z, _z, _d, _p]),
    # losses
    "nc_cuda_cross_entropy_forward_f32": (None, [_p, _p, _p, _i, _i]),
    "nc_cuda_cross_entropy_backward_f32": (None, [_p, _p, _p, _i, _i]),
    "nc_cuda_cross_entropy_fused_f32_ex": (_i, [_p, _p, _p, _p, _i, _i, _f, _p]),
    "nc_cuda_cross_entropy_fused_static_f32_ex": (_i, [_p, _p, _p, _p, _i, _i, _f, _p]),
    "nc_cuda_mse_fused_f32_ex": (_i, [_p, _p, _p, _p, _p, _z, _f, _p]),
    # optimizers
    "nc_cuda_sgd_step_f32": (None, [_p, _p, _f, _z]),
    "nc_cuda_sgd_momentum_f32": (None, [_p, _p, _p, _f, _f, _f, _i, _z]),
    "nc_cuda_sgd_update_f32_ex": (_i, [_p, _p, _p, _d, _d, _d, _d, _i, _i, _d, _z, _p]),
    "nc_cuda_adam_update_f32_ex": (_i, [_p] * 5 + [_d] * 8 + [_z, _p]),
    "nc_cuda_sgd_update_multi_f32_ex": (_i, [_i, _p, _p, _p, _p, _d, _d, _d, _d, _i, _i, _d, _p]),
    "nc_cuda_adam_update_multi_f32_ex": (_i, [_i, _p, _p, _p, _p, _p, _p] + [_d] * 8 + [_p]),
}


def header_symbols() -> list[str]:
    """Every nc_cuda_* function name declared in include/nocta_cuda.h."""
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(nc_cuda_[a-z0-9_]+)\s*\(", text)))


class CudaABI:
    """Loaded libnocta_cuda.so with typed entry points as attributes."""

    def __init__(self, path: Path | str = LIB_PATH):
        path = Path(path)
        if not path.exists():
            raise RuntimeError(
                f"{path} is missing: build it with `python -m nocta_b200.build` "
                "(the CUDA kernel library has no substitute)")
        self.path = path
        self.lib = C.CDLL(str(path), mode=C.RTLD_LOCAL)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(self.lib, name)
            fn.restype = res
            fn.argtypes = args
            setattr(self, name, fn)

    def check(self, status: int, what: str = "") -> None:
        if status != 0:
            msg = self.nc_cuda_last_message()
            raise RuntimeError(f"nc_cuda status {status} {what}: {msg.decode() if msg else ''}")


_abi: CudaABI | None = None


def load() -> CudaABI:
    global _abi
    if _abi is None:
        _abi = CudaABI()
    return _abi


def size4(values) -> "C.Array":
    return (C.c_size_t * 4)(*[int(v) for v in values])
