"""ctypes binding of libdistconv_b200.so (the C ABI declared in include/dcb.h).

The library is mandatory: importing this module on a machine without the built
shared object raises, there is no CPU fallback.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_double, c_float, c_int32, c_int64, c_uint32, c_void_p

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libdistconv_b200.so")

DCB_MAX_DIMS = 5
DCB_MAX_SPATIAL = 3
HALO_BLOB_BYTES = 256
COMM_BLOB_BYTES = 128
NCCL_ID_BYTES = 128

OK, BAD_ARG, UNSUPPORTED, CUDA_ERROR, PEER_TIMEOUT, NCCL_ERROR, NOT_CONNECTED = range(7)

HALO_REVERSE = 0x1
HALO_SKIP_UNPACK = 0x2
HALO_CLEAR_BOUNDARY = 0x4
HALO_OPS = {"ID": 0 << 4, "SUM": 1 << 4, "MAX": 2 << 4, "MIN": 3 << 4}

MATH_FP32, MATH_TF32, MATH_FP32_SIMT, MATH_BF16 = 0, 1, 2, 3


class TensorDesc(ctypes.Structure):
    _fields_ = [
        ("ndims", c_int32),
        ("dtype", c_int32),
        ("local_shape", c_int64 * DCB_MAX_DIMS),
        ("real_shape", c_int64 * DCB_MAX_DIMS),
        ("overlap", c_int32 * DCB_MAX_DIMS),
        ("pitch", c_int64),
    ]


class NdDesc(ctypes.Structure):
    _fields_ = [
        ("nsd", c_int32),
        ("n", c_int64),
        ("c", c_int64),
        ("dims", c_int64 * DCB_MAX_SPATIAL),
        ("sn", c_int64),
        ("sc", c_int64),
        ("strides", c_int64 * DCB_MAX_SPATIAL),
    ]


class Box(ctypes.Structure):
    _fields_ = [("off", c_int64 * DCB_MAX_DIMS), ("ext", c_int64 * DCB_MAX_DIMS)]


SHUFFLE_BLOB_BYTES = 128


class PoolDesc(ctypes.Structure):
    _fields_ = [
        ("nsd", c_int32),
        ("window", c_int32 * DCB_MAX_SPATIAL),
        ("pads", c_int32 * DCB_MAX_SPATIAL),
        ("strides", c_int32 * DCB_MAX_SPATIAL),
        ("mode", c_int32),
        ("outside_lo", c_int32 * DCB_MAX_SPATIAL),
        ("outside_hi", c_int32 * DCB_MAX_SPATIAL),
    ]


POOL_MODES = {"MAX": 0, "AVERAGE": 1, "AVERAGE_NO_PAD": 2}


class ConvDesc(ctypes.Structure):
    _fields_ = [
        ("nsd", c_int32),
        ("k", c_int32),
        ("c", c_int32),
        ("filter", c_int32 * DCB_MAX_SPATIAL),
        ("pads", c_int32 * DCB_MAX_SPATIAL),
        ("strides", c_int32 * DCB_MAX_SPATIAL),
        ("dilations", c_int32 * DCB_MAX_SPATIAL),
        ("groups", c_int32),
        ("math_mode", c_int32),
    ]


class DcbError(RuntimeError):
    def __init__(self, status: int, where: str, detail: str):
        self.status = status
        super().__init__(f"{where}: {lib().dcb_status_string(status).decode()} ({detail})")


_LIB = None

_P = c_void_p
_SIGS = {
    "dcb_status_string": (c_char_p, [c_int32]),
    "dcb_last_error": (c_char_p, []),
    "dcb_version": (c_int32, []),
    "dcb_set_wait_budget_ns": (c_int32, [c_int64]),
    "dcb_halo_plan_create": (c_int32, [POINTER(TensorDesc), POINTER(c_int32), c_int32, POINTER(_P)]),
    "dcb_halo_plan_destroy": (c_int32, [_P]),
    "dcb_halo_plan_export": (c_int32, [_P, _P]),
    "dcb_halo_plan_connect": (c_int32, [_P, _P, c_int32]),
    "dcb_halo_pack_put": (c_int32, [_P, _P, c_int32, c_uint32, _P]),
    "dcb_halo_wait_unpack": (c_int32, [_P, _P, c_int32, c_uint32, _P]),
    "dcb_halo_exchange": (c_int32, [_P, _P, c_uint32, _P]),
    "dcb_halo_unpack": (c_int32, [_P, _P, c_uint32, _P]),
    "dcb_halo_plan_status": (c_int32, [_P, _P]),
    "dcb_clear_halo": (c_int32, [POINTER(TensorDesc), _P, c_int32, _P]),
    "dcb_halo_pack": (c_int32, [POINTER(TensorDesc), _P, c_int32, c_int32, c_int32, c_int32, _P, _P]),
    "dcb_halo_unpack_slab": (c_int32, [POINTER(TensorDesc), _P, c_int32, c_int32, c_int32, c_int32, _P, c_uint32, _P]),
    "dcb_conv_plan_create": (c_int32, [POINTER(ConvDesc), POINTER(NdDesc), POINTER(NdDesc), POINTER(_P)]),
    "dcb_conv_plan_destroy": (c_int32, [_P]),
    "dcb_conv_fwd": (c_int32, [_P, c_double, _P, _P, c_double, _P, _P]),
    "dcb_conv_fwd_stats": (c_int32, [_P, c_double, _P, _P, _P, _P, _P, _P]),
    "dcb_conv_bwd_data": (c_int32, [_P, c_double, _P, _P, c_double, _P, _P]),
    "dcb_conv_bwd_filter": (c_int32, [_P, c_double, _P, _P, c_double, _P, _P]),
    "dcb_conv_plan_kernel_kind": (c_int32, [_P, c_int32]),
    "dcb_conv_plan_kernel_variant": (c_int32, [_P, c_int32]),
    "dcb_conv_plan_status": (c_int32, [_P, _P]),
    "dcb_bias_fwd": (c_int32, [c_double, _P, c_double, POINTER(NdDesc), _P, _P]),
    "dcb_bias_bwd": (c_int32, [c_double, POINTER(NdDesc), _P, c_double, _P, _P]),
    "dcb_bn_plan_create": (c_int32, [POINTER(NdDesc), POINTER(_P)]),
    "dcb_bn_plan_destroy": (c_int32, [_P]),
    "dcb_bn_stats": (c_int32, [_P, _P, _P, _P, _P]),
    "dcb_bn_stats_noalloc": (c_int32, [POINTER(NdDesc), _P, _P, _P, _P]),
    "dcb_bn_finalize": (c_int32, [c_int32, c_int64, c_float, _P, _P, _P, _P, _P]),
    "dcb_bn_apply": (c_int32, [POINTER(NdDesc), _P, _P, _P, _P, _P, c_float, POINTER(NdDesc), _P, _P]),
    "dcb_bn_apply_leaky_relu": (c_int32, [POINTER(NdDesc), _P, _P, _P, _P, _P, c_float, c_float, POINTER(NdDesc), _P,
                                          _P]),
    "dcb_bn_bwd_reduce": (c_int32, [_P, _P, POINTER(NdDesc), _P, _P, _P, _P, c_float, _P, _P, _P, _P, _P]),
    "dcb_bn_bwd_apply": (c_int32, [POINTER(NdDesc), _P, POINTER(NdDesc), _P, _P, _P, _P, _P, _P, c_float, c_int64,
                                   POINTER(NdDesc), _P, _P]),
    "dcb_leaky_relu_fwd": (c_int32, [POINTER(NdDesc), _P, c_float, POINTER(NdDesc), _P, _P]),
    "dcb_leaky_relu_bwd": (c_int32, [POINTER(NdDesc), _P, POINTER(NdDesc), _P, c_float, POINTER(NdDesc), _P, _P]),
    "dcb_pool_fwd": (c_int32, [POINTER(PoolDesc), POINTER(NdDesc), POINTER(NdDesc), c_double, _P, c_double, _P, _P]),
    "dcb_pool_bwd": (c_int32, [POINTER(PoolDesc), POINTER(NdDesc), POINTER(NdDesc), c_double, _P, _P, _P, c_double,
                               _P, _P, c_int64, _P]),
    "dcb_pool_bwd_workspace_bytes": (c_int64, [POINTER(PoolDesc), POINTER(NdDesc), POINTER(NdDesc)]),
    "dcb_shuffle_plan_create": (c_int32, [POINTER(TensorDesc), POINTER(TensorDesc), POINTER(Box), POINTER(Box),
                                          c_int32, c_int32, POINTER(_P)]),
    "dcb_shuffle_plan_destroy": (c_int32, [_P]),
    "dcb_shuffle_plan_export": (c_int32, [_P, _P]),
    "dcb_shuffle_plan_connect": (c_int32, [_P, _P, c_int32]),
    "dcb_shuffle_put": (c_int32, [_P, _P, _P]),
    "dcb_shuffle_wait_unpack": (c_int32, [_P, _P, _P]),
    "dcb_shuffle": (c_int32, [_P, _P, _P, _P]),
    "dcb_shuffle_plan_status": (c_int32, [_P, _P]),
    "dcb_nccl_unique_id": (c_int32, [_P]),
    "dcb_comm_create_nccl": (c_int32, [_P, c_int32, c_int32, POINTER(_P)]),
    "dcb_comm_create_peer": (c_int32, [c_int32, c_int32, c_int32, POINTER(_P)]),
    "dcb_comm_export": (c_int32, [_P, _P]),
    "dcb_comm_connect": (c_int32, [_P, _P, c_int32]),
    "dcb_comm_destroy": (c_int32, [_P]),
    "dcb_allreduce_sum": (c_int32, [_P, _P, c_int64, _P]),
    "dcb_allreduce_push": (c_int32, [_P, _P, c_int64, _P]),
    "dcb_allreduce_pull": (c_int32, [_P, _P, c_int64, _P]),
    "dcb_comm_status": (c_int32, [_P, _P]),
}

EXPORTED_SYMBOLS = tuple(_SIGS)


def lib():
    """Loads the shared library (once).  Raises if it has not been built."""
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m dihydrogen_b200.build` "
                "(there is no CPU fallback)")
        L = ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)
        for name, (res, args) in _SIGS.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _LIB = L
    return _LIB


def check(status: int, where: str):
    if status != OK:
        raise DcbError(status, where, lib().dcb_last_error().decode())


def call(name: str, *args):
    check(getattr(lib(), name)(*args), name)
