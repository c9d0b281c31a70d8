"""ctypes binding of libntb200.so (the C ABI declared in include/ntb200.h).

The library is built in-tree by `python -m neurotensor_b200.build`; importing this module fails loudly
when it is missing -- there is no CPU or PyTorch fallback behind any call.
"""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libntb200.so")

F32, F16, BF16, I8, I16, I32, I64, F64, U8, U16, U32, C64, C128, C32 = range(14)
ROUTE_AUTO, ROUTE_TENSOR, ROUTE_SIMT = 0, 1, 2
F16_ROUND_ONCE, F16_ROUND_PER_KTILE = 0, 1
OK, ERR_INVALID_ARG, ERR_UNSUPPORTED, ERR_ALLOC, ERR_CUDA, ERR_TIMEOUT, ERR_NO_DEVICE = range(7)
CONV2D_STATIC_SCRATCH_BYTES = 32 * 1024 * 1024

_i64, _vp, _ci, _sz = ctypes.c_int64, ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t


class GemmDesc(ctypes.Structure):
    _fields_ = [
        ("dtype", ctypes.c_int32), ("route", ctypes.c_int32), ("accumulate", ctypes.c_int32),
        ("f16_rounding", ctypes.c_int32),
        ("m", _i64), ("n", _i64), ("k", _i64), ("batch", _i64),
        ("a", _vp), ("a_row_stride", _i64), ("a_col_stride", _i64), ("a_batch_stride", _i64),
        ("b", _vp), ("b_row_stride", _i64), ("b_col_stride", _i64), ("b_batch_stride", _i64),
        ("c", _vp), ("c_row_stride", _i64), ("c_batch_stride", _i64),
        ("bias", _vp), ("bias_row_stride", _i64), ("bias_col_stride", _i64), ("bias_batch_stride", _i64),
    ]


class Conv3dGeom(ctypes.Structure):
    """ntb200_conv3d_geom: three-element arrays are (depth, height, width)."""
    _fields_ = [(n, ctypes.c_int64) for n in ("batch", "channels", "depth", "height", "width", "cout", "groups")] + \
               [(n, ctypes.c_int64 * 3) for n in ("kernel", "stride", "padding", "dilation")]


class ConvNdGeom(ctypes.Structure):
    """ntb200_convnd_geom: arrays hold one entry per spatial dimension, outermost first."""
    MAX_DIMS = 8
    _fields_ = [(n, ctypes.c_int64) for n in ("dims", "batch", "channels", "cout", "groups")] + \
               [(n, ctypes.c_int64 * 8) for n in ("size", "kernel", "stride", "padding", "dilation")]


class GemmEpilogue(ctypes.Structure):
    _fields_ = [("relu_out", _vp), ("relu_mask_src", _vp)]


ALLGATHER_FN = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t)

# name -> (restype, argtypes); every symbol include/ntb200.h declares
SIGNATURES = {
    "ntb200_version": (ctypes.c_char_p, []),
    "ntb200_last_error_string": (ctypes.c_char_p, []),
    "ntb200_device_count": (_ci, [ctypes.POINTER(_ci)]),
    "ntb200_set_device": (_ci, [_ci]),
    "ntb200_get_device": (_ci, [ctypes.POINTER(_ci)]),
    "ntb200_kernel_launch_count": (ctypes.c_uint64, []),
    "ntb200_last_gemm_route": (ctypes.c_char_p, []),
    "ntb200_check_device_status": (_ci, [_vp]),
    "ntb200_selftest_wait_timeout": (_ci, [ctypes.c_uint, _vp]),
    "ntb200_malloc_async": (_ci, [ctypes.POINTER(_vp), _sz, _vp]),
    "ntb200_free_async": (_ci, [_vp, _vp]),
    "ntb200_memset_async": (_ci, [_vp, _ci, _sz, _vp]),
    "ntb200_memcpy_h2d_async": (_ci, [_vp, _vp, _sz, _vp]),
    "ntb200_memcpy_d2h_async": (_ci, [_vp, _vp, _sz, _vp]),
    "ntb200_memcpy_d2d_async": (_ci, [_vp, _vp, _sz, _vp]),
    "ntb200_stream_synchronize": (_ci, [_vp]),
    "ntb200_host_alloc": (_ci, [ctypes.POINTER(_vp), _sz]),
    "ntb200_host_free": (_ci, [_vp]),
    "ntb200_host_register": (_ci, [_vp, _sz]),
    "ntb200_host_unregister": (_ci, [_vp]),
    "ntb200_pool_stats": (_ci, [ctypes.POINTER(ctypes.c_uint64), ctypes.POINTER(ctypes.c_uint64)]),
    "ntb200_scratch_stats": (_ci, [ctypes.POINTER(ctypes.c_uint64)] * 3),
    "ntb200_scratch_release_all": (_ci, []),
    "ntb200_device_pool_usage": (_ci, [ctypes.POINTER(ctypes.c_uint64)] * 3 + [_ci]),
    "ntb200_gemm": (_ci, [ctypes.POINTER(GemmDesc), _vp]),
    "ntb200_gemm_fused": (_ci, [ctypes.POINTER(GemmDesc), ctypes.POINTER(GemmEpilogue), _vp]),
    "ntb200_gemm_push": (_ci, [ctypes.POINTER(GemmDesc), ctypes.POINTER(_vp), _ci, _vp]),
    "ntb200_gemm_push_relu": (_ci, [ctypes.POINTER(GemmDesc), _vp, _i64, ctypes.POINTER(_vp), _ci, _vp]),
    "ntb200_peer_alloc": (_ci, [ctypes.POINTER(_vp), _sz]),
    "ntb200_peer_free": (_ci, [_vp]),
    "ntb200_peer_export": (_ci, [_vp, ctypes.c_char_p]),
    "ntb200_peer_import": (_ci, [ctypes.c_char_p, ctypes.POINTER(_vp)]),
    "ntb200_peer_release": (_ci, [_vp]),
    "ntb200_dist_shard": (_ci, [_i64, _ci, _ci, _i64, ctypes.POINTER(_i64), ctypes.POINTER(_i64)]),
    "ntb200_dist_init": (_ci, [ctypes.POINTER(_vp), _ci, _ci, ALLGATHER_FN, _vp]),
    "ntb200_dist_destroy": (_ci, [_vp]),
    "ntb200_dist_rank": (_ci, [_vp]),
    "ntb200_dist_world": (_ci, [_vp]),
    "ntb200_dist_buffer_create": (_ci, [_vp, _sz, ctypes.POINTER(_vp)]),
    "ntb200_dist_buffer_destroy": (_ci, [_vp]),
    "ntb200_dist_buffer_ptr": (_vp, [_vp]),
    "ntb200_dist_barrier": (_ci, [_vp, _vp]),
    "ntb200_dist_set_barrier_limit_ms": (_ci, [_vp, ctypes.c_uint]),
    "ntb200_dist_gemm_allgather": (_ci, [_vp, ctypes.POINTER(GemmDesc), _vp, _i64, _i64, _ci, _vp]),
    "ntb200_dist_gemm_allgather_at": (_ci, [_vp, ctypes.POINTER(GemmDesc), _vp, _i64, _i64, _i64, _ci, _vp]),
    "ntb200_dist_gemm_push_at": (_ci, [_vp, ctypes.POINTER(GemmDesc), _vp, _i64, _i64, _i64, _ci, _vp]),
    "ntb200_mse_grad_block": (_ci, [_ci, _vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64, _vp]),
    "ntb200_dist_allgather_columns": (_ci, [_vp, _ci, _vp, _i64, _i64, _i64, _vp, _i64, _i64, _vp]),
    "ntb200_matmult": (_ci, [_ci, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _ci, _ci, _vp]),
    "ntb200_matmult_batch": (_ci, [_ci, ctypes.POINTER(_vp), ctypes.POINTER(_vp), ctypes.POINTER(_vp), _i64, _i64,
                                   _i64, _i64, _i64, _ci, _ci, _vp]),
    "ntb200_matmult_host": (_ci, [_ci, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _ci, _ci, _ci]),
    "ntb200_im2col": (_ci, [_ci, _vp, _vp] + [_i64] * 12 + [_vp]),
    "ntb200_col2im": (_ci, [_ci, _vp, _vp] + [_i64] * 12 + [_vp]),
    "ntb200_conv2d_workspace_bytes": (_sz, [_ci] + [_i64] * 12),
    "ntb200_conv2d": (_ci, [_ci, _vp, _vp, _vp, _vp] + [_i64] * 13 + [_vp]),
    "ntb200_conv2d_backward_workspace_bytes": (_sz, [_ci] + [_i64] * 13),
    "ntb200_conv2d_backward_image": (_ci, [_ci, _vp, _vp, _vp, _vp] + [_i64] * 13 + [_vp]),
    "ntb200_conv2d_backward_kernel": (_ci, [_ci, _vp, _vp, _vp, _vp, _ci] + [_i64] * 13 + [_vp]),
    "ntb200_conv2d_grouped_workspace_bytes": (_sz, [_ci] + [_i64] * 14),
    "ntb200_conv2d_grouped": (_ci, [_ci, _vp, _vp, _vp, _vp] + [_i64] * 14 + [_vp]),
    "ntb200_conv2d_grouped_backward_image": (_ci, [_ci, _vp, _vp, _vp, _vp] + [_i64] * 14 + [_vp]),
    "ntb200_conv2d_grouped_backward_kernel": (_ci, [_ci, _vp, _vp, _vp, _vp, _ci] + [_i64] * 14 + [_vp]),
    "ntb200_im2col3d": (_ci, [_ci, _vp, _vp, ctypes.POINTER(Conv3dGeom), _vp]),
    "ntb200_col2im3d": (_ci, [_ci, _vp, _vp, ctypes.POINTER(Conv3dGeom), _vp]),
    "ntb200_im2colnd": (_ci, [_ci, _vp, _vp, ctypes.POINTER(ConvNdGeom), _vp]),
    "ntb200_col2imnd": (_ci, [_ci, _vp, _vp, ctypes.POINTER(ConvNdGeom), _vp]),
    "ntb200_convnd_workspace_bytes": (_sz, [_ci, ctypes.POINTER(ConvNdGeom)]),
    "ntb200_convnd": (_ci, [_ci, _vp, _vp, _vp, _vp, ctypes.POINTER(ConvNdGeom), _vp]),
    "ntb200_convnd_backward_image": (_ci, [_ci, _vp, _vp, _vp, _vp, ctypes.POINTER(ConvNdGeom), _vp]),
    "ntb200_convnd_backward_kernel": (_ci, [_ci, _vp, _vp, _vp, _vp, _ci, ctypes.POINTER(ConvNdGeom), _vp]),
    "ntb200_conv3d_workspace_bytes": (_sz, [_ci, ctypes.POINTER(Conv3dGeom)]),
    "ntb200_conv3d": (_ci, [_ci, _vp, _vp, _vp, _vp, ctypes.POINTER(Conv3dGeom), _vp]),
    "ntb200_conv3d_backward_image": (_ci, [_ci, _vp, _vp, _vp, _vp, ctypes.POINTER(Conv3dGeom), _vp]),
    "ntb200_conv3d_backward_kernel": (_ci, [_ci, _vp, _vp, _vp, _vp, _ci, ctypes.POINTER(Conv3dGeom), _vp]),
    "ntb200_conv2d_static_scratch": (_ci, [_ci, _vp, _vp, _vp] + [_i64] * 13 + [_vp]),
    "ntb200_relu": (_ci, [_ci, _vp, _vp, _i64, _vp]),
    "ntb200_relu_backward": (_ci, [_ci, _vp, _vp, _vp, _i64, _vp]),
    "ntb200_mse": (_ci, [_ci, _vp, _vp, _vp, _vp, _i64, _vp]),
    "ntb200_column_sum": (_ci, [_ci, _vp, _vp, _i64, _i64, _vp]),
    "ntb200_add_inplace": (_ci, [_ci, _vp, _vp, _i64, _vp]),
    "ntb200_bias_add_channels": (_ci, [_ci, _vp, _vp, _i64, _i64, _i64, _vp]),
    "ntb200_sum_channels": (_ci, [_ci, _vp, _vp, _i64, _i64, _i64, _vp]),
    "ntb200_sgd_step": (_ci, [_ci, _vp, _vp, _i64, ctypes.c_double, _vp]),
    "ntb200_adam_step": (_ci, [_ci, _vp, _vp, _vp, _vp, _i64] + [ctypes.c_double] * 4 + [_i64, _vp]),
    "ntb200_copy_strided_2d": (_ci, [_ci, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _vp]),
    "ntb200_convert": (_ci, [_ci, _vp, _ci, _vp, _i64, _vp]),
}


class Ntb200Error(RuntimeError):
    def __init__(self, code, message):
        super().__init__("ntb200 error %d: %s" % (code, message))
        self.code = code


_lib = None


def lib():
    """The loaded library.  Raises if libntb200.so has not been built: nothing here degrades to a CPU path."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("libntb200.so is missing at %s; build it with `python -m neurotensor_b200.build`"
                              % LIB_PATH)
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError if the library lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(rc):
    if rc != OK:
        raise Ntb200Error(rc, lib().ntb200_last_error_string().decode())
    return rc


def launch_count():
    return int(lib().ntb200_kernel_launch_count())


def last_route():
    return lib().ntb200_last_gemm_route().decode()
