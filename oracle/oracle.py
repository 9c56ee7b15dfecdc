"""ctypes front end of the CPU oracle (``oracle/ascq_oracle.c``).

Test infrastructure only: imported by ``tests/``, by ``__graft_entry__.smoke()`` and by the
CPU-baseline / reference legs of ``bench.py``.  The product package never imports it.

Arrays are numpy; bf16 tensors travel as ``uint16`` bit patterns, fp4x2 and e8m0 as ``uint8``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libascq_oracle.so")

# dtype / policy / round codes (identical to include/ascq.h)
F16, BF16, F32, I8, I32, U64, FP4X2_E2M1, E8M0 = range(8)
I4X2 = 12   # int4b_t, two per byte
PER_TENSOR, PER_CHANNEL, PER_TOKEN, PER_GROUP, PER_CHANNEL_PER_GROUP, PER_TOKEN_PER_GROUP = range(6)
CAST_NONE, CAST_RINT, CAST_FLOOR, CAST_CEIL, CAST_ROUND, CAST_TRUNC = range(6)

DT_SIZE = {F16: 2, BF16: 2, F32: 4, I8: 1, I32: 4, U64: 8, FP4X2_E2M1: 1, E8M0: 1}
NP_DTYPE = {F16: np.float16, BF16: np.uint16, F32: np.float32, I8: np.int8, I32: np.int32, U64: np.uint64,
            FP4X2_E2M1: np.uint8, E8M0: np.uint8}


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside it (gcc, a second or two)."""
    src = os.path.join(_HERE, "ascq_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-s"], check=True)
    return _SO


class _QuantParam(C.Structure):
    _fields_ = [("m", C.c_uint32), ("n", C.c_uint32), ("calCount", C.c_uint32), ("groupSize", C.c_uint32),
                ("hasOffset", C.c_int32), ("kDim", C.c_int32), ("roundMode", C.c_int32)]


class _DequantParam(C.Structure):
    _fields_ = [("m", C.c_uint32), ("n", C.c_uint32), ("calCount", C.c_uint32), ("groupSize", C.c_uint32),
                ("kDim", C.c_int32)]


class _AntiQuantParam(C.Structure):
    _fields_ = [("m", C.c_uint32), ("n", C.c_uint32), ("calCount", C.c_uint32), ("groupSize", C.c_uint32),
                ("hasOffset", C.c_int32), ("isTranspose", C.c_int32), ("kDim", C.c_int32)]


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        _lib.orc_f16_to_f32.restype = C.c_float
        _lib.orc_f16_to_f32.argtypes = [C.c_uint16]
        _lib.orc_bf16_to_f32.restype = C.c_float
        _lib.orc_bf16_to_f32.argtypes = [C.c_uint16]
        _lib.orc_f32_to_f16_sat.restype = C.c_uint16
        _lib.orc_f32_to_f16_sat.argtypes = [C.c_float]
        _lib.orc_f32_to_bf16_sat.restype = C.c_uint16
        _lib.orc_f32_to_bf16_sat.argtypes = [C.c_float]
        _lib.orc_f16_to_i8.restype = C.c_int8
        _lib.orc_f16_to_i8.argtypes = [C.c_uint16, C.c_int]
        _lib.orc_f32_to_i16.restype = C.c_int16
        _lib.orc_f32_to_i16.argtypes = [C.c_float, C.c_int]
        _lib.orc_i32_to_f32.restype = C.c_float
        _lib.orc_i32_to_f32.argtypes = [C.c_int32]
        _lib.orc_f16_mul.restype = C.c_uint16
        _lib.orc_f16_mul.argtypes = [C.c_uint16, C.c_uint16]
        _lib.orc_f16_add.restype = C.c_uint16
        _lib.orc_f16_add.argtypes = [C.c_uint16, C.c_uint16]
        _lib.orc_bf16_mul.restype = C.c_uint16
        _lib.orc_bf16_mul.argtypes = [C.c_uint16, C.c_uint16]
        _lib.orc_bf16_add.restype = C.c_uint16
        _lib.orc_bf16_add.argtypes = [C.c_uint16, C.c_uint16]
        _lib.orc_e2m1_to_f32.restype = C.c_float
        _lib.orc_e2m1_to_f32.argtypes = [C.c_uint8]
        _lib.orc_e8m0_to_bf16.restype = C.c_uint16
        _lib.orc_e8m0_to_bf16.argtypes = [C.c_uint8]
        _lib.orc_f32_to_e2m1.restype = C.c_uint8
        _lib.orc_f32_to_e2m1.argtypes = [C.c_float, C.c_int]
        _lib.ascq_oracle_dequant_dst_stride.restype = C.c_uint32
        _lib.ascq_oracle_dequant_dst_stride.argtypes = [C.c_uint32, C.c_int]
        for name in ("ascq_oracle_quant", "ascq_oracle_dequant", "ascq_oracle_antiquant", "ascq_oracle_matmul_w8a8",
                     "ascq_oracle_group_matmul_mxfp4", "ascq_oracle_dynamic_quant_per_token",
                     "ascq_oracle_quant_tmp_size", "ascq_oracle_dequant_tmp_size", "ascq_oracle_antiquant_tmp_size"):
            getattr(_lib, name).restype = C.c_int
    return _lib


def _p(a):
    if a is None:
        return None
    assert isinstance(a, np.ndarray) and a.flags["C_CONTIGUOUS"], "oracle wants contiguous numpy arrays"
    return a.ctypes.data_as(C.c_void_p)


class OracleError(RuntimeError):
    def __init__(self, code):
        super().__init__({1: "invalid argument", 2: "unsupported"}.get(code, f"code {code}"))
        self.code = code


def _check(rc):
    if rc != 0:
        raise OracleError(rc)


def num_threads() -> int:
    return lib().ascq_oracle_num_threads()


def ascend_quant(src, srcT, *, policy, m=0, n=0, calCount=None, scale=None, offset=None, scaleT=F16,
                 scaleScalar=0.0, offsetScalar=0.0, groupSize=0, hasOffset=False, kDim=1, roundMode=CAST_RINT,
                 dstT=I8):
    """AscendQuant; returns int8 array (or uint8 packed fp4x2) shaped like src (flattened count for fp4)."""
    cal = int(src.size if calCount is None else calCount)
    if dstT == I8:
        dst = np.zeros(src.shape, np.int8)
    else:
        dst = np.zeros(src.size // 2, np.uint8)
    p = _QuantParam(m, n, cal, groupSize, int(hasOffset), kDim, roundMode)
    _check(lib().ascq_oracle_quant(_p(dst), dstT, _p(src), srcT, _p(scale), _p(offset), scaleT,
                                   C.c_float(scaleScalar), C.c_float(offsetScalar), policy, C.byref(p)))
    return dst


def dynamic_quant_per_token(src, srcT, m, n):
    dst = np.zeros((m, n), np.int8)
    sc = np.zeros(m, np.float32)
    dq = np.zeros(m, np.float32)
    _check(lib().ascq_oracle_dynamic_quant_per_token(_p(dst), _p(sc), _p(dq), _p(src), srcT, C.c_uint32(m),
                                                     C.c_uint32(n)))
    return dst, sc, dq


def dynamic_quant_mxfp4(src, srcT, m, n):
    """Returns (codes uint8 [m, n/2], scale bytes uint8 [m, n/32])."""
    dst = np.zeros((m, n // 2), np.uint8)
    sc = np.zeros((m, n // 32), np.uint8)
    _check(lib().ascq_oracle_dynamic_quant_mxfp4(_p(dst), _p(sc), _p(src), srcT, C.c_uint32(m), C.c_uint32(n)))
    return dst, sc


def dequant_dst_stride(n, dstT):
    return int(lib().ascq_oracle_dequant_dst_stride(n, dstT))


def ascend_dequant(src, srcT, dstT, *, policy, m, n, calCount, scale=None, tokScale=None, scaleT=F32,
                   scaleScalar=0.0, groupSize=0, kDim=1, fill=0):
    """AscendDequant; returns [rows, dstStride] array of dstT (uint16 bits for bf16)."""
    if policy in (PER_TENSOR, PER_CHANNEL):
        rows, stride = m, dequant_dst_stride(n, dstT)
    else:
        rows, stride = calCount // n, n
    dst = np.empty((rows, stride), NP_DTYPE[dstT])
    dst.view(np.uint16 if DT_SIZE[dstT] == 2 else np.uint32).fill(fill)  # `fill` is a bit pattern
    p = _DequantParam(m, n, calCount, groupSize, kDim)
    _check(lib().ascq_oracle_dequant(_p(dst), dstT, _p(src), srcT, _p(scale), _p(tokScale), scaleT,
                                     C.c_float(scaleScalar), policy, C.byref(p)))
    return dst


def ascend_antiquant(src, srcT, dstT, *, policy, m, n, calCount=0, scale=None, offset=None, scaleT=BF16,
                     scaleScalar=0.0, offsetScalar=0.0, groupSize=0, hasOffset=True, isTranspose=False, kDim=1):
    total = calCount if calCount else m * n
    dst = np.zeros((total // n, n), NP_DTYPE[dstT])
    p = _AntiQuantParam(m, n, calCount, groupSize, int(hasOffset), int(isTranspose), kDim)
    _check(lib().ascq_oracle_antiquant(_p(dst), dstT, _p(src), srcT, _p(offset), _p(scale), scaleT,
                                       C.c_float(offsetScalar), C.c_float(scaleScalar), policy, C.byref(p)))
    return dst


class _QuantizeParam(C.Structure):
    _fields_ = [("m", C.c_uint32), ("n", C.c_uint32), ("groupSize", C.c_uint32), ("hasOffset", C.c_int32),
                ("kDim", C.c_int32), ("roundMode", C.c_int32)]


def quantize(src, srcT, *, policy, m, n, scale=None, offset=None, scaleT=F32, scaleScalar=0.0, offsetScalar=0.0,
             groupSize=0, hasOffset=False, kDim=1, roundMode=CAST_RINT, dstT=I8):
    """The unified Quantize interface (fp32 arithmetic for every policy); returns int8 [m, n] (or packed fp4x2)."""
    dst = np.zeros((m, n), np.int8) if dstT == I8 else np.zeros(m * n // 2, np.uint8)
    p = _QuantizeParam(m, n, groupSize, int(hasOffset), kDim, roundMode)
    _check(lib().ascq_oracle_quantize(_p(dst), dstT, _p(src), srcT, _p(scale), _p(offset), scaleT, C.c_float(scaleScalar),
                                      C.c_float(offsetScalar), policy, C.byref(p)))
    return dst


def dequantize(src, srcT, dstT, *, policy, m, n, scale=None, scaleT=F32, scaleScalar=0.0, groupSize=0, kDim=1, fill=0):
    """The unified Dequantize interface: AscendDequant on whole rows (dequantize_impl.h:100-215)."""
    cal = n if policy in (PER_TENSOR, PER_CHANNEL) else m * n
    return ascend_dequant(src, srcT, dstT, policy=policy, m=m, n=n, calCount=cal, scale=scale, scaleT=scaleT,
                          scaleScalar=scaleScalar, groupSize=groupSize, kDim=kDim, fill=fill)


def antiquantize(src, srcT, dstT, *, policy, m, n, scale=None, offset=None, scaleT=BF16, scaleScalar=0.0,
                 offsetScalar=0.0, groupSize=0, hasOffset=False, kDim=1):
    """The unified AntiQuantize interface (fp32 arithmetic for every policy); returns [m, n] of dstT."""
    dst = np.zeros((m, n), NP_DTYPE[dstT])
    p = _QuantizeParam(m, n, groupSize, int(hasOffset), kDim, CAST_RINT)
    _check(lib().ascq_oracle_antiquantize(_p(dst), dstT, _p(src), srcT, _p(offset), _p(scale), scaleT,
                                          C.c_float(offsetScalar), C.c_float(scaleScalar), policy, C.byref(p)))
    return dst


def matmul_w8a8(A, B_nk, sA=None, sB=None, bias_bf16=None, want_acc=False, ldc=None):
    M, K = A.shape
    N = B_nk.shape[0]
    ldc = N if ldc is None else ldc
    Cb = np.zeros((M, ldc), np.uint16)
    acc = np.zeros((M, N), np.int32) if want_acc else None
    _check(lib().ascq_oracle_matmul_w8a8(_p(Cb), _p(A), _p(B_nk), _p(sA), _p(sB), _p(bias_bf16), M, N, K, ldc,
                                         _p(acc)))
    return (Cb, acc) if want_acc else Cb


def group_matmul_w8a8(A, B_gnk, sA, sB_gn, groupList, bias_bf16=None, out=F16, act=False, want_acc=False):
    """Grouped W8A8 matmul with per-group channel scales and per-token scales (quant_group_matmul_custom.asc);
    returns [sumM, N] float16, or bf16 bit patterns (uint16) with ``out=BF16``."""
    sumM, K = A.shape
    G, N = B_gnk.shape[0], B_gnk.shape[1]
    gl = np.ascontiguousarray(groupList, np.int64)
    Cq = np.zeros((sumM, N), np.uint16)
    acc = np.zeros((sumM, N), np.int32) if want_acc else None
    _check(lib().ascq_oracle_group_matmul_w8a8(_p(Cq), _p(A), _p(B_gnk), _p(sA), _p(sB_gn), _p(bias_bf16), _p(gl), G, N, K,
                                               1 if out == BF16 else 0, 1 if act else 0, _p(acc)))
    res = Cq if out == BF16 else Cq.view(np.float16)
    return (res, acc) if want_acc else res


def matmul_i8_quant(A, B_nk, bias=None, quantVector=None, quantScalar=1.0):
    """int8 matmul + int32 bias, result quantised as the fixpipe does (fp16); returns [M, N] float16."""
    M, K = A.shape
    N = B_nk.shape[0]
    Cq = np.zeros((M, N), np.float16)
    _check(lib().ascq_oracle_matmul_i8_quant(_p(Cq), _p(A), _p(B_nk), _p(bias), _p(quantVector), C.c_float(quantScalar),
                                             M, N, K, N))
    return Cq


def req8(data, q):
    """One value through the fixpipe requantisation: int32 ``data``, 64-bit parameter ``q`` -> int in [-128, 255]."""
    f = lib().ascq_oracle_req8
    f.restype = C.c_int
    f.argtypes = [C.c_int32, C.c_uint64]
    return int(f(int(data), int(q) & 0xFFFFFFFFFFFFFFFF))


def matmul_i8_requant(A, B_nk, bias=None, quantVector=None, quantScalar=0):
    """int8 matmul + int32 bias, result requantised to bytes as the fixpipe does ((V)REQ8); returns [M, N] uint8."""
    M, K = A.shape
    N = B_nk.shape[0]
    Cq = np.zeros((M, N), np.uint8)
    f = lib().ascq_oracle_matmul_i8_requant
    f.restype = C.c_int
    f.argtypes = [C.c_void_p] * 5 + [C.c_uint64] + [C.c_int] * 4
    _check(f(_p(Cq), _p(A), _p(B_nk), _p(bias), _p(quantVector), int(quantScalar) & 0xFFFFFFFFFFFFFFFF, M, N, K, N))
    return Cq


def group_matmul_mxfp4(A, sA, B, sB, groupList, K, N, want_f32=False):
    """A [sumM, K/2] u8, sA [sumM, K/32] u8, B [G, N, K/2] u8, sB [G, N, K/32] u8, groupList int64 [G]."""
    G = int(len(groupList))
    sumM = int(np.sum(groupList))
    Cb = np.zeros((sumM, N), np.uint16)
    Cf = np.zeros((sumM, N), np.float32) if want_f32 else None
    gl = np.ascontiguousarray(groupList, np.int64)
    _check(lib().ascq_oracle_group_matmul_mxfp4(_p(Cb), _p(Cf), _p(A), _p(sA), _p(B), _p(sB), _p(gl), G, K, N))
    return (Cb, Cf) if want_f32 else Cb


def matmul_f16(A, B_nk, abT, cT=F32):
    """A [M, K], B_nk [N, K] as float16 arrays or bf16 bit patterns (uint16); returns (cT cast as uint16 bits or None, fp32)."""
    M, K = A.shape
    N = B_nk.shape[0]
    Cf = np.zeros((M, N), np.float32)
    C16 = np.zeros((M, N), np.uint16) if cT != F32 else None
    _check(lib().ascq_oracle_matmul_f16(_p(C16), _p(Cf), cT, _p(np.ascontiguousarray(A).view(np.uint16)),
                                        _p(np.ascontiguousarray(B_nk).view(np.uint16)), abT, M, N, K))
    return C16, Cf


def matmul_w8a16(A, abT, B_nk, offset, scale, cT=F32):
    """Weight-only-quantised matmul: AscendAntiQuant<int8, abT, isTranspose=true> on B_nk [N, K] (per-channel tensors
    [N] or two floats), then the half / bfloat16 matmul."""
    N, K = B_nk.shape
    if isinstance(scale, np.ndarray):
        W = ascend_antiquant(B_nk, I8, abT, policy=PER_CHANNEL, m=N, n=K, scale=scale, offset=offset, scaleT=abT,
                             isTranspose=True)
    else:
        W = ascend_antiquant(B_nk, I8, abT, policy=PER_TENSOR, m=N, n=K, scaleScalar=float(scale), offsetScalar=float(offset),
                             scaleT=abT, isTranspose=True, hasOffset=True)
    return matmul_f16(A, W, abT, cT), W


def qf322b8(data, q):
    """One fp32 value through the fixpipe quantisation to int8 / uint8: -> int in [-128, 255]."""
    f = lib().ascq_oracle_qf322b8
    f.restype = C.c_int
    f.argtypes = [C.c_float, C.c_uint64]
    return int(f(float(data), int(q) & 0xFFFFFFFFFFFFFFFF))


def matmul_f16_quant(A, B_nk, abT, quantVector=None, quantScalar=0):
    """half / bfloat16 matmul whose fp32 result is quantised to bytes as the fixpipe does ((V)QF322B8_PRE); [M, N] uint8."""
    M, K = A.shape
    N = B_nk.shape[0]
    Cq = np.zeros((M, N), np.uint8)
    f = lib().ascq_oracle_matmul_f16_quant
    f.restype = C.c_int
    f.argtypes = [C.c_void_p] * 3 + [C.c_int, C.c_void_p, C.c_uint64] + [C.c_int] * 4
    _check(f(_p(Cq), _p(np.ascontiguousarray(A).view(np.uint16)), _p(np.ascontiguousarray(B_nk).view(np.uint16)), abT,
             _p(quantVector), int(quantScalar) & 0xFFFFFFFFFFFFFFFF, M, N, K, N))
    return Cq


def group_matmul_mxfp8(A, aFmt, sA, B, bFmt, sB, groupList, K, N):
    """A [sumM, K] u8 (fp8 codes), sA [sumM, K/32] u8, B [G, N, K] u8, sB [G, N, K/32] u8; aFmt/bFmt 0 = e4m3fn, 1 = e5m2.
    Returns (bf16 bits, fp32)."""
    G = int(len(groupList))
    sumM = int(np.sum(groupList))
    Cb = np.zeros((sumM, N), np.uint16)
    Cf = np.zeros((sumM, N), np.float32)
    gl = np.ascontiguousarray(groupList, np.int64)
    _check(lib().ascq_oracle_group_matmul_mxfp8(_p(Cb), _p(Cf), _p(A), aFmt, _p(sA), _p(B), bFmt, _p(sB), _p(gl), G, K, N))
    return Cb, Cf


def _dims(d):
    arr = (C.c_int64 * len(d))(*d)
    return arr, len(d)


def quant_tmp_size(dims, typeSize):
    a, r = _dims(dims)
    mx, mn = C.c_uint32(), C.c_uint32()
    _check(lib().ascq_oracle_quant_tmp_size(a, r, C.c_uint32(typeSize), C.byref(mx), C.byref(mn)))
    return mx.value, mn.value


def quant_factor():
    a, b = C.c_uint32(), C.c_uint32(7)
    lib().ascq_oracle_quant_factor(C.byref(a), C.byref(b))
    return a.value, b.value


def dequant_tmp_size(dims, typeSize):
    a, r = _dims(dims)
    mx, mn = C.c_uint32(), C.c_uint32()
    _check(lib().ascq_oracle_dequant_tmp_size(a, r, C.c_uint32(typeSize), C.byref(mx), C.byref(mn)))
    return mx.value, mn.value


def dequant_factor(dims):
    a, r = _dims(dims)
    x, y = C.c_uint32(), C.c_uint32()
    lib().ascq_oracle_dequant_factor(a, r, C.byref(x), C.byref(y))
    return x.value, y.value


def antiquant_tmp_size(srcDims, scaleDims, isTranspose, inT, outT):
    a, r = _dims(srcDims)
    b, s = _dims(scaleDims)
    mx, mn = C.c_uint32(), C.c_uint32()
    _check(lib().ascq_oracle_antiquant_tmp_size(a, r, b, s, int(isTranspose), inT, outT, C.byref(mx), C.byref(mn)))
    return mx.value, mn.value


def antiquant_factor(srcDims, scaleDims, isTranspose, inT, outT):
    a, r = _dims(srcDims)
    b, s = _dims(scaleDims)
    x, y = C.c_uint32(), C.c_uint32()
    lib().ascq_oracle_antiquant_factor(a, r, b, s, int(isTranspose), inT, outT, C.byref(x), C.byref(y))
    return x.value, y.value


# ---- small numpy helpers shared by tests and bench (bit-level, no ml_dtypes needed) -------------
def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-half-to-even fp32 -> bf16 bit patterns (finite inputs)."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    r = u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))
    return (r >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


@dataclass
class UlpReport:
    max_ulp: int
    mismatches: int
    total: int


def bf16_ulp_diff(a_bits: np.ndarray, b_bits: np.ndarray) -> UlpReport:
    """Distance in bf16 ULPs between two bit-pattern arrays (sign-magnitude -> ordered ints)."""
    def order(v):
        v = v.astype(np.int32)
        return np.where(v & 0x8000, -(v & 0x7FFF), v & 0x7FFF)
    d = np.abs(order(a_bits) - order(b_bits))
    return UlpReport(int(d.max(initial=0)), int(np.count_nonzero(d)), int(d.size))
