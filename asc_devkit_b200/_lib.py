"""ctypes binding of ``libascq.so`` -- the same C ABI a C or C++ host program links against
(``include/ascq.h``).  Loading fails loudly when the library has not been built; nothing here
falls back to another implementation."""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libascq.so")

# ascq_status
OK, ERR_INVALID_ARG, ERR_UNSUPPORTED, ERR_ALIGNMENT, ERR_CUDA, ERR_NCCL, ERR_TIMEOUT = range(7)
# ascq_dtype
(DT_F16, DT_BF16, DT_F32, DT_I8, DT_I32, DT_U64, DT_FP4X2_E2M1, DT_E8M0, DT_FP8_E4M3, DT_FP8_E5M2, DT_HIF8,
 DT_FP4X2_E1M2, DT_I4X2) = range(13)
# ascq_policy
PER_TENSOR, PER_CHANNEL, PER_TOKEN, PER_GROUP, PER_CHANNEL_PER_GROUP, PER_TOKEN_PER_GROUP = range(6)
# ascq_round
CAST_NONE, CAST_RINT, CAST_FLOOR, CAST_CEIL, CAST_ROUND, CAST_TRUNC = range(6)


class QuantParam(C.Structure):
    _fields_ = [("m", C.c_uint32), ("n", C.c_uint32), ("calCount", C.c_uint32), ("groupSize", C.c_uint32),
                ("hasOffset", C.c_int32), ("kDim", C.c_int32), ("roundMode", C.c_int)]


class DequantParam(C.Structure):
    _fields_ = [("m", C.c_uint32), ("n", C.c_uint32), ("calCount", C.c_uint32), ("groupSize", C.c_uint32),
                ("kDim", C.c_int32)]


class AntiQuantParam(C.Structure):
    _fields_ = [("m", C.c_uint32), ("n", C.c_uint32), ("calCount", C.c_uint32), ("groupSize", C.c_uint32),
                ("hasOffset", C.c_int32), ("isTranspose", C.c_int32), ("kDim", C.c_int32)]


class QuantizeParam(C.Structure):
    """ascq_quantize_param: QuantizeConfig + QuantizeParams of the unified interface."""
    _fields_ = [("m", C.c_uint32), ("n", C.c_uint32), ("groupSize", C.c_uint32), ("hasOffset", C.c_int32),
                ("kDim", C.c_int32), ("roundMode", C.c_int)]


class AscqError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"{status_string(status)}: {message}")
        self.status = status
        self.message = message


_vp, _i, _u32, _f = C.c_void_p, C.c_int, C.c_uint32, C.c_float
_P64, _PU32 = C.POINTER(C.c_int64), C.POINTER(C.c_uint32)

# name -> (restype, argtypes); every symbol include/ascq.h declares
SIGNATURES = {
    "ascq_status_string": (C.c_char_p, [_i]),
    "ascq_last_error": (C.c_char_p, []),
    "ascq_version": (_i, []),
    "ascq_quant": (_i, [_vp, _i, _vp, _i, _vp, _vp, _i, _f, _f, _i, C.POINTER(QuantParam), _vp]),
    "ascq_dynamic_quant_per_token": (_i, [_vp, _vp, _vp, _vp, _i, _u32, _u32, _vp]),
    "ascq_dynamic_quant_mxfp4": (_i, [_vp, _vp, _vp, _i, _u32, _u32, _vp]),
    "ascq_dequant": (_i, [_vp, _i, _vp, _i, _vp, _vp, _i, _f, _i, C.POINTER(DequantParam), _vp]),
    "ascq_antiquant": (_i, [_vp, _i, _vp, _i, _vp, _vp, _i, _f, _f, _i, C.POINTER(AntiQuantParam), _vp]),
   "ascq_quantize": (_i, [_vp, _i, _vp, _i, _vp, _vp, _i, _f, _f, _i, C.POINTER(QuantizeParam), _vp]),
    "ascq_dequantize": (_i, [_vp, _i, _vp, _i, _vp, _i, _f, _i, C.POINTER(QuantizeParam), _vp]),
    "ascq_antiquantize": (_i, [_vp, _i, _vp, _i, _vp, _vp, _i, _f, _f, _i, C.POINTER(QuantizeParam), _vp]),
    "ascq_matmul_w8a8": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp]),
    "ascq_group_matmul_w8a8": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _vp, _P64, _i, _i, _i, _i, _vp]),
    "ascq_matmul_w8a8_scatter": (_i, [C.POINTER(_vp), _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "ascq_matmul_i8_quant": (_i, [_vp, _vp, _vp, _vp, _vp, _f, _i, _i, _i, _i, _vp]),
    "ascq_matmul_i8_requant": (_i, [_vp, _vp, _vp, _vp, _vp, C.c_uint64, _i, _i, _i, _i, _vp]),
    "ascq_transpose_i8_kn_to_nk": (_i, [_vp, _vp, _i, _i, _vp]),
    "ascq_matmul_f16_quant": (_i, [_vp, _vp, _vp, _i, _vp, C.c_uint64, _i, _i, _i, _i, _vp]),
    "ascq_matmul_f16": (_i, [_vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "ascq_matmul_w8a16": (_i, [_vp, _i, _vp, _i, _vp, _vp, _vp, _f, _f, _i, _i, _i, _i, _vp, C.c_size_t, _vp]),
    "ascq_matmul_w8a16_workspace_size": (C.c_size_t, [_i, _i]),
    "ascq_matmul_w4a16": (_i, [_vp, _i, _vp, _i, _vp, _vp, _vp, _f, _f, _i, _i, _i, _i, _vp, C.c_size_t, _vp]),
    "ascq_matmul_status": (_i, [_vp]),
    "ascq_comm_flag_bytes": (C.c_size_t, []),
    "ascq_comm_create": (_i, [C.POINTER(_vp), _i, _i, C.POINTER(_vp)]),
    "ascq_comm_destroy": (_i, [_vp]),
    "ascq_comm_rank": (_i, [_vp, C.POINTER(_i), C.POINTER(_i)]),
    "ascq_comm_ipc_handle_bytes": (C.c_size_t, []),
    "ascq_comm_ipc_export": (_i, [_vp, _vp]),
    "ascq_comm_ipc_open": (_i, [C.POINTER(_vp), _vp]),
    "ascq_comm_ipc_close": (_i, [_vp]),
    "ascq_comm_barrier": (_i, [_vp, _vp]),
    "ascq_shard_columns": (_i, [_i, _i, _i, C.POINTER(_i), C.POINTER(_i)]),
    "ascq_shard_groups_lpt": (_i, [_P64, _i, _i, C.POINTER(_i)]),
    "ascq_matmul_w8a8_sharded": (_i, [_vp, C.POINTER(_vp), _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "ascq_group_matmul_mxfp4_sharded": (_i, [_vp, C.POINTER(_vp), _vp, _vp, _vp, _vp, _P64, _i, _i, _i, _vp, C.c_size_t, _vp]),
    "ascq_set_wait_limit_cycles": (_i, [C.c_longlong]),
    "ascq_test_withhold_after": (_i, [_i]),
    "ascq_measure_tensor_rate": (_i, [_i, _i, C.POINTER(C.c_double), _vp]),
    "ascq_group_matmul_mxfp4": (_i, [_vp, _vp, _vp, _vp, _vp, _P64, _i, _i, _i, _vp, C.c_size_t, _vp]),
    "ascq_group_matmul_mxfp4_scatter": (_i, [C.POINTER(_vp), _i, _i, _P64, _vp, _vp, _vp, _vp, _P64, _i, _i, _i, _vp, C.c_size_t, _vp]),
    "ascq_group_matmul_mxfp8": (_i, [_vp, _i, _vp, _i, _vp, _vp, _i, _vp, _P64, _i, _i, _i, _vp, C.c_size_t, _vp]),
    "ascq_group_matmul_mxfp8_workspace_size": (C.c_size_t, [C.c_int64, _i, _i, _i]),
    "ascq_group_matmul_mxfp4_packed_scale_b_size": (C.c_size_t, [_i, _i, _i]),
    "ascq_group_matmul_mxfp4_pack_scale_b": (_i, [_vp, _vp, _i, _i, _i, _vp]),
    "ascq_group_matmul_mxfp4_prepacked": (_i, [_vp, _vp, _vp, _vp, _vp, _P64, _i, _i, _i, _vp, C.c_size_t, _vp]),
    "ascq_group_matmul_mxfp4_workspace_size": (C.c_size_t, [C.c_int64, _i, _i, _i]),
    "ascq_group_matmul_mxfp4_noalloc": (_i, [_vp, _vp, _vp, _vp, _vp, _P64, _i, _i, _i, _vp]),
    "ascq_group_matmul_mxfp4_noalloc_max_scratch": (C.c_size_t, []),
    "ascq_mx_repack_b_kn_to_nk": (_i, [_vp, _vp, _i, _i, _vp]),
    "ascq_mx_repack_scale_b": (_i, [_vp, _vp, _i, _i, _vp]),
    "ascq_get_ascend_quant_max_min_tmp_size": (_i, [_P64, _i, _u32, _PU32, _PU32]),
    "ascq_get_ascend_quant_tmp_buffer_factor_size": (None, [_PU32, _PU32]),
    "ascq_get_ascend_dequant_max_min_tmp_size": (_i, [_P64, _i, _u32, _PU32, _PU32]),
    "ascq_get_ascend_dequant_tmp_buffer_factor_size": (None, [_P64, _i, _PU32, _PU32]),
    "ascq_get_ascend_antiquant_max_min_tmp_size": (_i, [_P64, _i, _P64, _i, _i, _i, _i, _PU32, _PU32]),
    "ascq_get_ascend_antiquant_tmp_buffer_factor_size": (None, [_P64, _i, _P64, _i, _i, _i, _i, _PU32, _PU32]),
}

_lib = None


def lib() -> C.CDLL:
    """The loaded library.  Raises if ``libascq.so`` is missing: build it with
    ``python -m asc_devkit_b200.build`` (needs nvcc)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: run `python -m asc_devkit_b200.build` (nvcc, sm_100a); "
                               "there is no fallback implementation")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def status_string(status: int) -> str:
    return lib().ascq_status_string(int(status)).decode()


def check(status: int) -> None:
    if status != OK:
        raise AscqError(status, lib().ascq_last_error().decode())
