"""ctypes binding of libpetb200.so — the C ABI declared in include/petb200.h.

The library is the product: importing this module fails loudly when it has not been built
(`python -m pet_b200.build`), there is no CPU fallback.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libpetb200.so")

OK, ERR_INVALID, ERR_UNSUPPORTED, ERR_CUDA, ERR_NOMEM, ERR_DEVICE = range(6)
ACT = {"none": 0, None: 0, "relu": 1, "sigmoid": 2, "tanh": 3, "gelu": 4}
ALGO = {"auto": 0, "tc_3xtf32": 1, "simt_fp32": 2, "tc_1xtf32": 3, "tc_bf16x3": 4}

# every symbol include/petb200.h declares, with (restype, argtypes)
_vp, _i, _sz, _fp = C.c_void_p, C.c_int, C.c_size_t, C.c_float
_ip = C.POINTER(C.c_int)


class TransposeDesc(C.Structure):
    _fields_ = [("split", _i), ("factor", _i), ("ngroups", _i), ("group_sizes", _i * 8), ("flat", _i * 8)]


SYMBOLS = {
    "petb200_ctx_create": (_i, [_i, C.POINTER(_vp)]),
    "petb200_ctx_destroy": (_i, [_vp]),
    "petb200_last_error": (C.c_char_p, [_vp]),
    "petb200_status_string": (C.c_char_p, [_i]),
    "petb200_launch_count": (C.c_uint64, [_vp]),
    "petb200_check_device_status": (_i, [_vp, _vp]),
    "petb200_plan_destroy": (None, [_vp]),
    "petb200_plan_device_bytes": (_sz, [_vp]),
    "petb200_plan_kernel": (C.c_char_p, [_vp]),
    "petb200_conv2d_plan": (_i, [_vp, _ip, _i, C.POINTER(_vp)]),
    "petb200_conv2d_set_weights": (_i, [_vp, _vp, _vp]),
    "petb200_conv2d_run": (_i, [_vp, _vp, _vp, _vp, _vp]),
    "petb200_conv2d_out_dims": (_i, [_vp, _ip]),
    "petb200_conv2d_correct": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "petb200_conv3d_plan": (_i, [_vp, _ip, _i, C.POINTER(_vp)]),
    "petb200_conv3d_set_weights": (_i, [_vp, _vp, _vp]),
    "petb200_conv3d_run": (_i, [_vp, _vp, _vp, _vp, _vp]),
    "petb200_convtrans_plan": (_i, [_vp, _ip, _i, C.POINTER(_vp)]),
    "petb200_convtrans_set_weights": (_i, [_vp, _vp, _vp]),
    "petb200_convtrans_run": (_i, [_vp, _vp, _vp, _vp, _vp]),
    "petb200_convtrans_out_dims": (_i, [_vp, _ip]),
    "petb200_g2bmm_run": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "petb200_gbmml_run": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "petb200_banded_time": (_i, [_vp, _i, _i, _i, _i, _i, _i, _i, _i, C.POINTER(_fp), _vp]),
    "petb200_conv_run_residual": (_i, [_vp, _vp, _vp, _vp, _vp, _vp]),
    "petb200_matmul_plan": (_i, [_vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, C.POINTER(_vp)]),
    "petb200_matmul_plan_strided": (_i, [_vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, C.POINTER(C.c_longlong), C.POINTER(_vp)]),
    "petb200_matmul_set_weights": (_i, [_vp, _vp, _vp]),
    "petb200_matmul_run": (_i, [_vp, _vp, _vp, _vp, _vp, _vp]),
    "petb200_matmul_run_residual": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "petb200_transpose_plan": (_i, [_vp, _i, _ip, _i, C.POINTER(TransposeDesc), C.POINTER(_vp)]),
    "petb200_transpose_halo_plan": (_i, [_vp, _i, _ip, C.POINTER(TransposeDesc), _i, _i, _i, _i, C.POINTER(_vp)]),
    "petb200_pad_plan": (_i, [_vp, _i, _ip, _ip, _ip, C.POINTER(_vp)]),
    "petb200_slice_plan": (_i, [_vp, _i, _ip, _ip, _ip, C.POINTER(_vp)]),
    "petb200_extend_plan": (_i, [_vp, _i, _ip, _i, _i, C.POINTER(_vp)]),
    "petb200_layout_out_dims": (_i, [_vp, _ip]),
    "petb200_layout_run": (_i, [_vp, _vp, _vp, _vp]),
    "petb200_concat_run": (_i, [_vp, _i, _ip, _i, _i, _ip, C.POINTER(_vp), _vp, _vp]),
    "petb200_split_run": (_i, [_vp, _i, _ip, _i, _i, _ip, _vp, C.POINTER(_vp), _vp]),
    "petb200_eltwise_run": (_i, [_vp, _i, _i, C.POINTER(_vp), C.POINTER(_sz), _vp, _sz, _i, _vp]),
    "petb200_activation_run": (_i, [_vp, _vp, _vp, _sz, _i, _vp]),
    "petb200_batchnorm_run": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _i, _sz, _fp, _vp]),
    "petb200_pool2d_run": (_i, [_vp, _i, _vp, _vp] + [_i] * 10 + [_vp]),
    "petb200_div_run": (_i, [_vp, _vp, _sz, _vp, _sz, _vp, _sz, _vp]),
    "petb200_pow_run": (_i, [_vp, _vp, _vp, _sz, _i, _vp]),
    "petb200_reducemean_run": (_i, [_vp, _vp, _vp, _sz, _i, _sz, _vp]),
    "petb200_gather_run": (_i, [_vp, _vp, _vp, _vp, _sz, _sz, _i, _sz, _vp]),
    "petb200_rowmean_run": (_i, [_vp, _vp, _vp, _sz, _i, _vp]),
    "petb200_softmax_run": (_i, [_vp, _vp, _vp, _sz, _i, _vp]),
    "petb200_softmax_axis_run": (_i, [_vp, _vp, _vp, _sz, _i, _sz, _vp]),
    "petb200_layernorm_run": (_i, [_vp, _vp, _vp, _vp, _vp, _sz, _i, _fp, _vp]),
    "petb200_attention_supported": (_i, [_i, _i, _i, _i]),
    "petb200_attention_run": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp]),
    "petb200_matmul_splitk_noalloc": (_i, [_i] * 7 + [_vp, _vp, _vp, _vp, _i, _vp, C.c_char_p, _sz]),
    "petb200_plan_time": (_i, [_vp, _i, _i, C.POINTER(_fp), _vp]),
}

_lib = None


def load():
    """Returns the loaded library with prototypes set; raises if it is missing or lacks a declared symbol."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m pet_b200.build` "
                               "(nvcc, sm_100a). There is no CPU fallback.")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(lib, name)  # AttributeError = the header and the library disagree
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


class PetError(RuntimeError):
    def __init__(self, status, text):
        super().__init__(f"petb200 status {status}: {text}")
        self.status = status


def ints(v):
    return (C.c_int * len(v))(*[int(x) for x in v])
