"""Loads the CUDA backend (libphoenix_core_b200.so) and declares its C ABI for ctypes.

There is no CPU fallback: if the library is missing, import of the compute entry points fails loudly.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "csrc", "libphoenix_core_b200.so")

# status codes of include/phoenix_core_b200.h
PCB_OK = 0
PCB_ERR_INVALID_ARGUMENT = -1
PCB_ERR_UNSUPPORTED = -2
PCB_ERR_WORKSPACE = -3
PCB_ERR_CUDA = -4
PCB_ERR_DEVICE_TIMEOUT = -5
PCB_ERR_TOO_LARGE = -6

PCB_F32, PCB_F16, PCB_BF16 = 0, 1, 2
VARIANT_16_PRODUCT, VARIANT_8_PRODUCT = 0, 1
FP16_POLICY_FULL32, FP16_POLICY_FULL16, FP16_POLICY_BACKWARD32 = 0, 1, 2
ENGINE_AUTO, ENGINE_SIMT, ENGINE_TENSOR = 0, 1, 2


class ConvDesc(ctypes.Structure):
    """pcb_conv2d_desc"""
    _fields_ = [(k, ctypes.c_int32) for k in (
        "dtype", "n", "ci", "co", "h", "w", "kh", "kw", "stride_h", "stride_w", "dilation_h", "dilation_w",
        "pad_top", "pad_left", "pad_bottom", "pad_right", "groups", "has_bias", "require_input_grad",
        "real_valued_input", "variant", "fp16_policy", "engine", "algebra", "data_format", "filter_layout")]


class DenseDesc(ctypes.Structure):
    """pcb_dense_desc"""
    _fields_ = [(k, ctypes.c_int32) for k in (
        "dtype", "batch", "in_features", "out_features", "filter_oi", "has_bias", "require_input_grad", "variant",
        "engine", "algebra")]


# name -> (restype, argtypes); this is every symbol include/phoenix_core_b200.h declares
_vp, _sz, _i = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
_cd, _dd = ctypes.POINTER(ConvDesc), ctypes.POINTER(DenseDesc)
SYMBOLS = {
    "pcb_version": (ctypes.c_char_p, []),
    "pcb_status_string": (ctypes.c_char_p, [_i]),
    "pcb_last_error_message": (ctypes.c_char_p, []),
    "pcb_conv2d_output_size": (_i, [_cd, ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int32)]),
    "pcb_qconv2d_fwd_workspace_size": (_sz, [_cd]),
    "pcb_qconv2d_bwd_workspace_size": (_sz, [_cd]),
    "pcb_qdense_fwd_workspace_size": (_sz, [_dd]),
    "pcb_qdense_bwd_workspace_size": (_sz, [_dd]),
    "pcb_qconv2d_fwd": (_i, [_cd, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "pcb_qconv2d_bwd": (_i, [_cd, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "pcb_qconv2d_fwd_keeps_input": (_i, [_cd]),
    "pcb_qconv2d_bwd_kept": (_i, [_cd, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp, _sz, _vp]),
    "pcb_qconv2d_bwd_data": (_i, [_cd, _vp, _vp, _vp, _vp, _sz, _vp]),
    "pcb_qconv2d_bwd_filter": (_i, [_cd, _vp, _vp, _vp, _vp, _sz, _vp]),
    "pcb_qconv2d_bwd_filter_noalloc": (_i, [_cd, _vp, _vp, _vp, _vp]),
    "pcb_qdense_fwd": (_i, [_dd, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "pcb_qdense_bwd": (_i, [_dd, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp]),
    "pcb_qconv2d_engine_for": (_i, [_cd, _i]),
    "pcb_qdense_engine_for": (_i, [_dd, _i]),
    "pcb_check_device_status": (_i, [_vp, _sz, _vp]),
    "pcb_selftest_wait_expiry": (_i, [_cd, _vp, _vp, _vp, _vp, _sz, ctypes.c_longlong, _vp]),
    "pcb_aux_bn_relu_fwd": (_i, [_i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, ctypes.c_float, _i, _vp]),
    "pcb_aux_bn_relu_bwd": (_i, [_i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "pcb_aux_bn_relu_bwd_from_input": (_i, [_i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "pcb_aux_bn_relu_maxpool_fwd": (_i, [_i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, ctypes.c_float, _vp]),
    "pcb_aux_bn_relu_maxpool_bwd": (_i, [_i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "pcb_aux_bn_add_relu_fwd": (_i, [_i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, ctypes.c_float, _vp]),
    "pcb_aux_bn_add_relu_bwd": (_i, [_i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "pcb_aux_maxpool3x3s2_fwd": (_i, [_i, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "pcb_aux_maxpool3x3s2_bwd": (_i, [_i, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "pcb_aux_clock_probe": (_i, [ctypes.c_longlong, _vp, _vp]),
    "pcb_set_sm_margin": (_i, [_i]),
    "pcb_get_sm_margin": (_i, []),
}

_lib = None


class BackendError(RuntimeError):
    def __init__(self, status, message):
        super().__init__("phoenix_core_b200: %s (status %d)" % (message, status))
        self.status = status


def lib():
    """Returns the loaded library; raises if it has not been built (python -m phoenix_core_b200.csrc.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("CUDA backend not built: %s is missing. Run `python -m phoenix_core_b200.csrc.build`. "
                              "There is no CPU fallback." % LIB_PATH)
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(handle, name)     # AttributeError if a declared symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(status):
    """Maps a C-ABI status to the exception classes of the reference (std::invalid_argument ->
    ValueError, std::runtime_error -> RuntimeError)."""
    if status == PCB_OK:
        return
    msg = lib().pcb_last_error_message().decode() or lib().pcb_status_string(status).decode()
    if status == PCB_ERR_INVALID_ARGUMENT:
        raise ValueError("phoenix_core_b200: " + msg)
    raise BackendError(status, msg)
