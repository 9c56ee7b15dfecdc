"""Python mirror of the Ascend C quantization operator interface, on CUDA tensors.

The names, argument order and argument meaning follow ``include/adv_api/quantization/ascend_quant.h``,
``ascend_dequant.h`` and ``ascend_antiquant.h`` of asc-devkit; compile-time config structs become keyword
arguments.  Each function forwards device pointers to the C ABI (``include/ascq.h``) and raises
:class:`AscqError` where the reference would assert.  torch is used only to own device memory and streams.
"""
from __future__ import annotations

import ctypes as C
from ctypes import c_int64 as C_int64
from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib as L
from ._lib import (AscqError, CAST_CEIL, CAST_FLOOR, CAST_NONE, CAST_RINT, CAST_ROUND, CAST_TRUNC,  # noqa: F401
                   PER_CHANNEL, PER_CHANNEL_PER_GROUP, PER_GROUP, PER_TENSOR, PER_TOKEN, PER_TOKEN_PER_GROUP)

_TORCH_DT = {torch.float16: L.DT_F16, torch.bfloat16: L.DT_BF16, torch.float32: L.DT_F32, torch.int8: L.DT_I8,
             torch.int32: L.DT_I32}


def dtype_code(t: torch.Tensor, override: Optional[int] = None) -> int:
    """ascq_dtype of a tensor; uint8/int64 carriers of fp4x2 / e8m0 / uint64 scales need ``override``."""
    if override is not None:
        return override
    if t.dtype not in _TORCH_DT:
        raise TypeError(f"no ascq dtype for {t.dtype}; pass the dtype code explicitly")
    return _TORCH_DT[t.dtype]


def _ptr(t: Optional[torch.Tensor]):
    if t is None:
        return None
    if not t.is_cuda:
        raise ValueError("ascq operators take CUDA tensors (there is no CPU path)")
    if not t.is_contiguous():
        raise ValueError("ascq operators take contiguous tensors")
    return C.c_void_p(t.data_ptr())


def _ptr_pitched(t: torch.Tensor):
    """Pointer of a 2-D output whose rows are contiguous but may be spaced by a pitch (``t.stride(0)`` goes in as ldc)."""
    if not t.is_cuda:
        raise ValueError("ascq operators take CUDA tensors (there is no CPU path)")
    if t.dim() != 2 or t.stride(1) != 1 or t.stride(0) < t.shape[1]:
        raise ValueError("a matmul output must be 2-D with contiguous rows")
    return C.c_void_p(t.data_ptr())


def _workspace(need: int, device, stream: Optional[torch.cuda.Stream]) -> torch.Tensor:
    """A temporary workspace for a call that returns while its kernels still run.  The caching allocator hands a freed
    block back to torch's current stream; when the kernels run on another stream the block is tied to that one too."""
    ws = torch.empty(max(int(need), 256), dtype=torch.uint8, device=device)
    if stream is not None and stream != torch.cuda.current_stream(ws.device):
        ws.record_stream(stream)
    return ws


def _stream(stream: Optional[torch.cuda.Stream]):
    """Raw cudaStream_t of ``stream`` or of torch's current stream (the raw-handle getter skips building a Stream
    object: a few microseconds per call, which matters next to a 10 us kernel)."""
    if stream is None:
        return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())
    return stream.cuda_stream


@dataclass
class AscendQuantParam:
    """include/adv_api/quantization/ascend_quant_utils.h:82-87"""
    m: int
    n: int
    calCount: int
    groupSize: int = 0


def AscendQuant(dstTensor: torch.Tensor, srcTensor: torch.Tensor, scale, offset, calCount: Optional[int] = None, *,
                policy: int = PER_TENSOR, para: Optional[AscendQuantParam] = None, scaleCount: Optional[int] = None,
                hasOffset: Optional[bool] = None, kDim: int = 1, roundMode: int = CAST_RINT, dst_dtype: int = L.DT_I8,
                stream=None) -> torch.Tensor:
    """AscendQuant (include/adv_api/quantization/ascend_quant.h).

    * per tensor  : ``scale`` and ``offset`` are Python floats (ascend_quant.h:63-97).
    * per channel : ``scale`` is a tensor of ``scaleCount`` elements, ``offset`` a float or a tensor
      (ascend_quant.h:159-347); ``calCount`` must be a multiple of ``scaleCount``.
    * PER_TOKEN / PER_GROUP : ``scale``/``offset`` tensors and ``para`` (ascend_quant.h:667-762).
    """
    scale_is_t = isinstance(scale, torch.Tensor)
    offset_is_t = isinstance(offset, torch.Tensor)
    if policy == PER_TENSOR and scale_is_t:
        policy = PER_CHANNEL
    cal = srcTensor.numel() if calCount is None else int(calCount)
    if para is not None:
        m, n, cal, gs = para.m, para.n, para.calCount, para.groupSize
    elif policy == PER_CHANNEL:
        n = int(scaleCount if scaleCount is not None else scale.numel())
        m, gs = (cal // n if n else 0), 0
    else:
        m, n, gs = 1, cal, 0
    if hasOffset is None:
        hasOffset = offset is not None
    p = L.QuantParam(m, n, cal, gs, int(bool(hasOffset)), kDim, roundMode)
    scaleT = dtype_code(scale) if scale_is_t else L.DT_F32
    L.check(L.lib().ascq_quant(_ptr(dstTensor), dst_dtype, _ptr(srcTensor), dtype_code(srcTensor),
                               _ptr(scale) if scale_is_t else None, _ptr(offset) if offset_is_t else None, scaleT,
                               float(scale) if not scale_is_t else 0.0,
                               float(offset) if (offset is not None and not offset_is_t) else 0.0,
                               policy, C.byref(p), _stream(stream)))
    return dstTensor


def DynamicQuantPerToken(dstTensor, scaleOut, srcTensor, deqScaleOut=None, stream=None):
    """Per-token absmax -> scale -> int8 in one launch (``ascq_dynamic_quant_per_token``)."""
    m, n = srcTensor.shape
    L.check(L.lib().ascq_dynamic_quant_per_token(_ptr(dstTensor), _ptr(scaleOut), _ptr(deqScaleOut), _ptr(srcTensor),
                                                 dtype_code(srcTensor), m, n, _stream(stream)))
    return dstTensor, scaleOut


def DynamicQuantMxfp4(dstTensor: torch.Tensor, scaleOut: torch.Tensor, srcTensor: torch.Tensor, stream=None):
    """Blocks of 32 elements -> E8M0 scale byte + 32 E2M1 codes (``ascq_dynamic_quant_mxfp4``): dst uint8 [m, n/2],
    scale uint8 [m, n/32]."""
    m, n = srcTensor.shape
    L.check(L.lib().ascq_dynamic_quant_mxfp4(_ptr(dstTensor), _ptr(scaleOut), _ptr(srcTensor), dtype_code(srcTensor), m, n,
                                             _stream(stream)))
    return dstTensor, scaleOut


@dataclass
class DequantParams:
    """include/adv_api/quantization/ascend_dequant_utils.h:26-30"""
    m: int
    n: int
    calCount: int
    groupSize: int = 0


def dequant_dst_stride(n: int, dst: torch.dtype) -> int:
    """Row stride of AscendDequant's destination: n rounded up to 32 bytes."""
    per_blk = 32 // torch.empty((), dtype=dst).element_size()
    return (n + per_blk - 1) // per_blk * per_blk


def AscendDequant(dstTensor: torch.Tensor, srcTensor: torch.Tensor, deqScale, params: DequantParams, *,
                  policy: Optional[int] = None, tokScale: Optional[torch.Tensor] = None, kDim: int = 1,
                  scale_dtype: Optional[int] = None, stream=None) -> torch.Tensor:
    """AscendDequant (include/adv_api/quantization/ascend_dequant.h).

    ``deqScale`` float -> scalar overload; tensor -> per channel (default) or PER_TOKEN / PER_GROUP when
    ``policy`` says so.  ``tokScale`` (fp32 [m]) fuses the per-token multiply of the grouped-matmul epilogue.
    A uint64 scale tensor is passed as int64 storage with ``scale_dtype=DT_U64``."""
    is_t = isinstance(deqScale, torch.Tensor)
    if policy is None:
        policy = PER_CHANNEL if is_t else PER_TENSOR
    p = L.DequantParam(params.m, params.n, params.calCount, params.groupSize, kDim)
    scaleT = dtype_code(deqScale, scale_dtype) if is_t else L.DT_F32
    L.check(L.lib().ascq_dequant(_ptr(dstTensor), dtype_code(dstTensor), _ptr(srcTensor), dtype_code(srcTensor),
                                 _ptr(deqScale) if is_t else None, _ptr(tokScale), scaleT,
                                 0.0 if is_t else float(deqScale), policy, C.byref(p), _stream(stream)))
    return dstTensor


@dataclass
class AscendAntiQuantParam:
    m: int
    n: int
    calCount: int = 0
    groupSize: int = 0


def AscendAntiQuant(dstTensor: torch.Tensor, srcTensor: torch.Tensor, offset, scale, para: AscendAntiQuantParam, *,
                    isTranspose: bool = False, policy: Optional[int] = None, hasOffset: Optional[bool] = None,
                    kDim: int = 1, src_dtype: Optional[int] = None, scale_dtype: Optional[int] = None,
                    stream=None) -> torch.Tensor:
    """AscendAntiQuant (include/adv_api/quantization/ascend_antiquant.h): dst = scale * (src + offset).

    ``para.m, para.n`` is the shape of ``srcTensor`` as stored ([K,N], or [N,K] with ``isTranspose``).
    fp4 sources are uint8 tensors with ``src_dtype=DT_FP4X2_E2M1`` and an e8m0 scale (``scale_dtype=DT_E8M0``)."""
    is_t = isinstance(scale, torch.Tensor)
    off_t = isinstance(offset, torch.Tensor)
    if policy is None:
        policy = PER_CHANNEL if is_t else PER_TENSOR
    if hasOffset is None:
        hasOffset = offset is not None
    p = L.AntiQuantParam(para.m, para.n, para.calCount, para.groupSize, int(bool(hasOffset)), int(isTranspose), kDim)
    scaleT = dtype_code(scale, scale_dtype) if is_t else dtype_code(dstTensor)
    L.check(L.lib().ascq_antiquant(_ptr(dstTensor), dtype_code(dstTensor), _ptr(srcTensor),
                                   dtype_code(srcTensor, src_dtype), _ptr(offset) if off_t else None,
                                   _ptr(scale) if is_t else None, scaleT,
                                   float(offset) if (offset is not None and not off_t) else 0.0,
                                   0.0 if is_t else float(scale), policy, C.byref(p), _stream(stream)))
    return dstTensor


# ---- the unified interface (include/adv_api/quantization/quantize.h, dequantize.h, antiquantize.h) ---------------
@dataclass
class QuantizeParams:
    """QuantizeParams / DequantizeParams / AntiQuantizeParams (quantize_utils.h:43-47)"""
    m: int
    n: int
    groupSize: int = 0


def _scalar_code(dstTensor, scale, override):
    return dtype_code(scale, override) if isinstance(scale, torch.Tensor) else L.DT_F32


def Quantize(dstTensor: torch.Tensor, srcTensor: torch.Tensor, scale, offset, params: QuantizeParams, *, policy: int,
             hasOffset: bool = False, roundMode: int = CAST_RINT, kDim: int = 1, dst_dtype: int = L.DT_I8, stream=None):
    """Quantize<config>(dst, src, scale, offset, params) (quantize.h:41-62): fp32 arithmetic for every policy.
    PER_TENSOR takes Python floats, the other policies tensors (PER_CHANNEL also a float offset)."""
    st, ot = isinstance(scale, torch.Tensor), isinstance(offset, torch.Tensor)
    p = L.QuantizeParam(params.m, params.n, params.groupSize, int(bool(hasOffset)), kDim, roundMode)
    L.check(L.lib().ascq_quantize(_ptr(dstTensor), dst_dtype, _ptr(srcTensor), dtype_code(srcTensor),
                                  _ptr(scale) if st else None, _ptr(offset) if ot else None,
                                  dtype_code(scale) if st else L.DT_F32, 0.0 if st else float(scale),
                                  float(offset) if (offset is not None and not ot) else 0.0, policy, C.byref(p),
                                  _stream(stream)))
    return dstTensor


def Dequantize(dstTensor: torch.Tensor, srcTensor: torch.Tensor, scale, offset, params: QuantizeParams, *, policy: int,
               hasOffset: bool = False, kDim: int = 1, scale_dtype: Optional[int] = None, stream=None):
    """Dequantize<config>(dst, src, scale, offset, params) (dequantize.h): forwards to the AscendDequant kernels on
    whole rows; the reference accepts no offset yet (``offset`` is ignored, ``hasOffset`` must be False)."""
    st = isinstance(scale, torch.Tensor)
    p = L.QuantizeParam(params.m, params.n, params.groupSize, int(bool(hasOffset)), kDim, CAST_RINT)
    L.check(L.lib().ascq_dequantize(_ptr(dstTensor), dtype_code(dstTensor), _ptr(srcTensor), dtype_code(srcTensor),
                                    _ptr(scale) if st else None, dtype_code(scale, scale_dtype) if st else L.DT_F32,
                                    0.0 if st else float(scale), policy, C.byref(p), _stream(stream)))
    return dstTensor


def AntiQuantize(dstTensor: torch.Tensor, srcTensor: torch.Tensor, scale, offset, params: QuantizeParams, *, policy: int,
                 hasOffset: bool = False, kDim: int = 1, stream=None):
    """AntiQuantize<config>(dst, src, scale, offset, params) (antiquantize.h): dst = (src + offset) * scale in fp32."""
    st, ot = isinstance(scale, torch.Tensor), isinstance(offset, torch.Tensor)
    p = L.QuantizeParam(params.m, params.n, params.groupSize, int(bool(hasOffset)), kDim, CAST_RINT)
    L.check(L.lib().ascq_antiquantize(_ptr(dstTensor), dtype_code(dstTensor), _ptr(srcTensor), dtype_code(srcTensor),
                                      _ptr(offset) if ot else None, _ptr(scale) if st else None,
                                      dtype_code(scale) if st else dtype_code(dstTensor),
                                      float(offset) if (offset is not None and not ot) else 0.0,
                                      0.0 if st else float(scale), policy, C.byref(p), _stream(stream)))
    return dstTensor


def MatmulW8A8(C: Optional[torch.Tensor], A: torch.Tensor, B_nk: torch.Tensor, scaleA: Optional[torch.Tensor] = None,
               scaleB: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
               accDump: Optional[torch.Tensor] = None, stream=None):
    """int8 x int8 -> int32 matmul with the per-channel x per-token dequant, bias and bf16 cast fused
    (``ascq_matmul_w8a8``).  A [M,K], B_nk [N,K] (K-major, the reference's SetTensorB(..., isTransposeB=true)),
    C bf16 [M, ldc>=N] (row stride taken from C.stride(0))."""
    M, K = A.shape
    N = B_nk.shape[0]
    if C is not None and C.stride(1) != 1:
        raise ValueError("C must have unit column stride")
    ldc = C.stride(0) if C is not None else N
    cptr = C.data_ptr() if C is not None else None
    L.check(L.lib().ascq_matmul_w8a8(cptr, _ptr(A), _ptr(B_nk), _ptr(scaleA), _ptr(scaleB), _ptr(bias), M, N, K, ldc,
                                     _ptr(accDump), _stream(stream)))
    return C


def MatmulI8Quant(C: torch.Tensor, A: torch.Tensor, B_nk: torch.Tensor, bias: Optional[torch.Tensor] = None,
                  quantVector: Optional[torch.Tensor] = None, quantScalar: float = 1.0, stream=None):
    """int8 matmul whose result leaves through the fixpipe quantisation of the reference (SetQuantScalar /
    SetQuantVector, fp16 output): ``ascq_matmul_i8_quant``.  ``quantVector`` is an int64 tensor holding the uint64
    words (fp32 bits in the low half), ``bias`` int32 [N]."""
    M, K = A.shape
    N = B_nk.shape[0]
    L.check(L.lib().ascq_matmul_i8_quant(_ptr(C), _ptr(A), _ptr(B_nk), _ptr(bias), _ptr(quantVector), float(quantScalar),
                                         M, N, K, C.stride(0), _stream(stream)))
    return C


def MatmulI8Requant(C: torch.Tensor, A: torch.Tensor, B_nk: torch.Tensor, bias: Optional[torch.Tensor] = None,
                    quantVector: Optional[torch.Tensor] = None, quantScalar: int = 0, stream=None):
    """int8 matmul whose result is requantised to int8 / uint8 by the fixpipe rule ((V)REQ8): ``ascq_matmul_i8_requant``.
    ``C`` is an int8 or uint8 [M, N] tensor, ``quantVector`` an int64 tensor holding the 64-bit parameter words,
    ``quantScalar`` the same word as a Python int (used when ``quantVector`` is None)."""
    M, K = A.shape
    N = B_nk.shape[0]
    L.check(L.lib().ascq_matmul_i8_requant(_ptr(C), _ptr(A), _ptr(B_nk), _ptr(bias), _ptr(quantVector),
                                           int(quantScalar) & 0xFFFFFFFFFFFFFFFF, M, N, K, C.stride(0), _stream(stream)))
    return C


def TransposeI8KnToNk(B_nk: torch.Tensor, B_kn: torch.Tensor, stream=None):
    K, N = B_kn.shape
    L.check(L.lib().ascq_transpose_i8_kn_to_nk(_ptr(B_nk), _ptr(B_kn), K, N, _stream(stream)))
    return B_nk


def MatmulF16(C: torch.Tensor, A: torch.Tensor, B_nk: torch.Tensor, stream=None):
    """half / bfloat16 matmul with fp32 accumulation (``ascq_matmul_f16``): C [M, N] = A [M, K] . B_nk [N, K]^T."""
    M, K = A.shape
    N = B_nk.shape[0]
    L.check(L.lib().ascq_matmul_f16(_ptr(C), dtype_code(C), _ptr(A), _ptr(B_nk), dtype_code(A), M, N, K, C.stride(0),
                                    _stream(stream)))
    return C


def MatmulF16Quant(C: torch.Tensor, A: torch.Tensor, B_nk: torch.Tensor, quantVector: Optional[torch.Tensor] = None,
                   quantScalar: int = 0, stream=None):
    """half / bfloat16 matmul whose fp32 result is quantised to int8 / uint8 by the fixpipe rule ((V)QF322B8_PRE):
    ``ascq_matmul_f16_quant``.  Parameter words as for ``MatmulI8Requant``."""
    M, K = A.shape
    N = B_nk.shape[0]
    L.check(L.lib().ascq_matmul_f16_quant(_ptr(C), _ptr(A), _ptr(B_nk), dtype_code(A), _ptr(quantVector),
                                          int(quantScalar) & 0xFFFFFFFFFFFFFFFF, M, N, K, C.stride(0), _stream(stream)))
    return C


def MatmulW8A16(C: torch.Tensor, A: torch.Tensor, B_nk: torch.Tensor, offset, scale, workspace: Optional[torch.Tensor] = None,
                stream=None):
    """Weight-only-quantised matmul (``ascq_matmul_w8a16``): B_nk int8 [N, K] goes through AscendAntiQuant (per-channel
    ``offset`` / ``scale`` tensors of A's dtype, or two Python floats: SetAntiQuantVector / SetAntiQuantScalar) and then
    through the half / bfloat16 matmul."""
    M, K = A.shape
    N = B_nk.shape[0]
    if workspace is None:
        workspace = _workspace(N * K * 2, A.device, stream)
    st = isinstance(scale, torch.Tensor)
    L.check(L.lib().ascq_matmul_w8a16(_ptr_pitched(C), dtype_code(C), _ptr(A), dtype_code(A), _ptr(B_nk),
                                      _ptr(offset) if isinstance(offset, torch.Tensor) else None, _ptr(scale) if st else None,
                                      0.0 if st else float(offset), 0.0 if st else float(scale), M, N, K, C.stride(0),
                                      _ptr(workspace), workspace.numel(), _stream(stream)))
    return C


def MatmulW4A16(C: torch.Tensor, A: torch.Tensor, B_nk_int4: torch.Tensor, offset, scale,
                workspace: Optional[torch.Tensor] = None, stream=None):
    """``MatmulW8A16`` with int4b_t weights: ``B_nk_int4`` is a uint8 tensor [N, K/2] (two signed nibbles per byte)."""
    M, K = A.shape
    N = B_nk_int4.shape[0]
    if workspace is None:
        workspace = _workspace(N * K * 2, A.device, stream)
    st = isinstance(scale, torch.Tensor)
    L.check(L.lib().ascq_matmul_w4a16(_ptr_pitched(C), dtype_code(C), _ptr(A), dtype_code(A), _ptr(B_nk_int4),
                                      _ptr(offset) if isinstance(offset, torch.Tensor) else None, _ptr(scale) if st else None,
                                      0.0 if st else float(offset), 0.0 if st else float(scale), M, N, K, C.stride(0),
                                      _ptr(workspace), workspace.numel(), _stream(stream)))
    return C


def GroupMatmulMxfp4Workspace(sumM: int, G: int, K: int, N: int) -> int:
    return int(L.lib().ascq_group_matmul_mxfp4_workspace_size(sumM, G, K, N))


def GroupMatmulMxfp4(C: torch.Tensor, A: torch.Tensor, scaleA: torch.Tensor, B: torch.Tensor, scaleB: torch.Tensor,
                     groupList, K: int, N: int, workspace: Optional[torch.Tensor] = None, stream=None):
    """MX-FP4 grouped matmul (``ascq_group_matmul_mxfp4``).  A [sumM, K/2] uint8, scaleA [sumM, K/32] uint8 (e8m0),
    B [G, N, K/2] uint8, scaleB [G, N, K/32] uint8, groupList = rows per group (host sequence), C [sumM, N] bf16.
    ``workspace`` (uint8, CUDA) is allocated here when not given; the C entry point itself never allocates."""
    gl = (C_int64 * len(groupList))(*[int(v) for v in groupList])
    G = len(groupList)
    need = GroupMatmulMxfp4Workspace(int(sum(int(v) for v in groupList)), G, K, N)
    if workspace is None:
        workspace = _workspace(need, C.device, stream)
    L.check(L.lib().ascq_group_matmul_mxfp4(_ptr(C), _ptr(A), _ptr(scaleA), _ptr(B), _ptr(scaleB), gl, G, K, N,
                                            _ptr(workspace), workspace.numel(), _stream(stream)))
    return C


def GroupMatmulMxfp4PackScaleB(scaleB: torch.Tensor, K: int, N: int, stream=None) -> torch.Tensor:
    """Packs the scales of static weights once (``ascq_group_matmul_mxfp4_pack_scale_b``); returns the packed buffer."""
    G = scaleB.shape[0]
    out = torch.empty(int(L.lib().ascq_group_matmul_mxfp4_packed_scale_b_size(G, K, N)), dtype=torch.uint8, device=scaleB.device)
    L.check(L.lib().ascq_group_matmul_mxfp4_pack_scale_b(_ptr(out), _ptr(scaleB), G, K, N, _stream(stream)))
    return out


def GroupMatmulMxfp4Prepacked(C: torch.Tensor, A: torch.Tensor, scaleA: torch.Tensor, B: torch.Tensor, scaleB_packed: torch.Tensor,
                              groupList, K: int, N: int, workspace: Optional[torch.Tensor] = None, stream=None):
    """``GroupMatmulMxfp4`` with the scales of B already packed by ``GroupMatmulMxfp4PackScaleB``."""
    gl = (C_int64 * len(groupList))(*[int(v) for v in groupList])
    G = len(groupList)
    need = GroupMatmulMxfp4Workspace(int(sum(int(v) for v in groupList)), G, K, N)
    if workspace is None:
        workspace = _workspace(need, C.device, stream)
    L.check(L.lib().ascq_group_matmul_mxfp4_prepacked(_ptr(C), _ptr(A), _ptr(scaleA), _ptr(B), _ptr(scaleB_packed), gl, G, K, N,
                                                      _ptr(workspace), workspace.numel(), _stream(stream)))
    return C


def GroupMatmulMxfp8(C: torch.Tensor, A: torch.Tensor, a_dtype: int, scaleA: torch.Tensor, B: torch.Tensor, b_dtype: int,
                     scaleB: torch.Tensor, groupList, K: int, N: int, workspace: Optional[torch.Tensor] = None, stream=None):
    """MX matmul with fp8 operands (``ascq_group_matmul_mxfp8``).  A [sumM, K] uint8 (fp8 codes), B [G, N, K] uint8,
    scales [rows, K/32] uint8 (e8m0), ``a_dtype`` / ``b_dtype`` = DT_FP8_E4M3 or DT_FP8_E5M2, C bf16 or fp32 [sumM, N]."""
    G = len(groupList)
    gl = (C_int64 * G)(*[int(v) for v in groupList])
    need = int(L.lib().ascq_group_matmul_mxfp8_workspace_size(int(sum(int(v) for v in groupList)), G, K, N))
    if workspace is None:
        workspace = _workspace(need, C.device, stream)
    L.check(L.lib().ascq_group_matmul_mxfp8(_ptr(C), dtype_code(C), _ptr(A), a_dtype, _ptr(scaleA), _ptr(B), b_dtype,
                                            _ptr(scaleB), gl, G, K, N, _ptr(workspace), workspace.numel(), _stream(stream)))
    return C


def GroupMatmulMxfp4Scatter(buffer_ptrs, first_buf: int, out_row_start, A: torch.Tensor, scaleA: torch.Tensor, B: torch.Tensor,
                            scaleB: torch.Tensor, groupList, K: int, N: int, workspace: Optional[torch.Tensor] = None,
                            stream=None):
    """Grouped MX-FP4 matmul whose epilogue writes group g's rows to rows ``out_row_start[g]``.. of every bf16 [*, N]
    buffer in ``buffer_ptrs`` (device addresses; this GPU's buffer and peer-mapped ones):
    ``ascq_group_matmul_mxfp4_scatter``."""
    G = len(groupList)
    gl = (C_int64 * G)(*[int(v) for v in groupList])
    rs = (C_int64 * G)(*[int(v) for v in out_row_start]) if out_row_start is not None else None
    need = GroupMatmulMxfp4Workspace(int(sum(int(v) for v in groupList)), G, K, N)
    if workspace is None:
        workspace = _workspace(need, A.device, stream)
    arr = (C.c_void_p * len(buffer_ptrs))(*[C.c_void_p(int(v)) for v in buffer_ptrs])
    L.check(L.lib().ascq_group_matmul_mxfp4_scatter(arr, len(buffer_ptrs), first_buf, rs, _ptr(A), _ptr(scaleA), _ptr(B),
                                                    _ptr(scaleB), gl, G, K, N, _ptr(workspace), workspace.numel(),
                                                    _stream(stream)))


def MxRepackBKnToNk(B_nk: torch.Tensor, B_kn: torch.Tensor, K: int, N: int, stream=None):
    L.check(L.lib().ascq_mx_repack_b_kn_to_nk(_ptr(B_nk), _ptr(B_kn), K, N, _stream(stream)))
    return B_nk


def MxRepackScaleB(sB_nk: torch.Tensor, sB_ref: torch.Tensor, sK: int, N: int, stream=None):
    L.check(L.lib().ascq_mx_repack_scale_b(_ptr(sB_nk), _ptr(sB_ref), sK, N, _stream(stream)))
    return sB_nk


def GroupMatmulW8A8(C: torch.Tensor, A: torch.Tensor, B_gnk: torch.Tensor, scaleA, scaleB_gn, groupList, bias_gn=None,
                    activation: int = 0, stream=None):
    """Grouped W8A8 matmul (``ascq_group_matmul_w8a8``): A int8 [sumM, K], B int8 [G, N, K], scaleA fp32 [sumM], scaleB fp32
    [G, N], groupList = rows per group (host sequence), C half or bf16 [sumM, N]; ``activation=1`` applies FasterGelu."""
    G, N, K = B_gnk.shape
    gl = (C_int64 * len(groupList))(*[int(v) for v in groupList])
    L.check(L.lib().ascq_group_matmul_w8a8(_ptr(C), dtype_code(C), _ptr(A), _ptr(B_gnk), _ptr(scaleA), _ptr(scaleB_gn),
                                           _ptr(bias_gn), gl, len(groupList), N, K, int(activation), _stream(stream)))
    return C


def MatmulW8A8Scatter(buffer_ptrs, first_buf: int, col_offset: int, ldc: int, A: torch.Tensor, B_nk: torch.Tensor,
                      scaleA=None, scaleB=None, bias=None, stream=None):
    """W8A8 matmul whose epilogue writes the [M, N_local] block into columns [col_offset, col_offset + N_local) of every
    bf16 [M, ldc] buffer in ``buffer_ptrs`` (device addresses; this GPU's buffer and peer-mapped ones):
    ``ascq_matmul_w8a8_scatter``."""
    M, K = A.shape
    N = B_nk.shape[0]
    arr = (C.c_void_p * len(buffer_ptrs))(*[C.c_void_p(int(v)) for v in buffer_ptrs])
    L.check(L.lib().ascq_matmul_w8a8_scatter(arr, len(buffer_ptrs), first_buf, col_offset, ldc, _ptr(A), _ptr(B_nk),
                                             _ptr(scaleA), _ptr(scaleB), _ptr(bias), M, N, K, _stream(stream)))


class Comm:
    """The communicator of the sharded matmuls (``ascq_comm_create``): this rank's position among the GPUs of one box and
    every rank's flag block as mapped into this process.  ``flag_block_ptrs[r]`` is the device address of rank r's block
    (``Comm.flag_bytes()`` bytes, zeroed, 128-byte aligned; ``flag_block_ptrs[rank]`` the local one).  The caller maps
    the blocks (CUDA IPC through ``IpcExport`` / ``IpcOpen``, or a symmetric-memory allocator) and makes sure every rank
    has zeroed its block before any rank launches."""

    def __init__(self, rank: int, nranks: int, flag_block_ptrs):
        if len(flag_block_ptrs) != nranks:
            raise ValueError("one flag block per rank is needed")
        arr = (C.c_void_p * nranks)(*[C.c_void_p(int(v)) for v in flag_block_ptrs])
        h = C.c_void_p()
        L.check(L.lib().ascq_comm_create(C.byref(h), rank, nranks, arr))
        self.handle, self.rank, self.nranks = h, rank, nranks

    @staticmethod
    def flag_bytes() -> int:
        return int(L.lib().ascq_comm_flag_bytes())

    def barrier(self, stream=None):
        """The end-of-step exchange as a launch of its own (``ascq_comm_barrier``)."""
        L.check(L.lib().ascq_comm_barrier(self.handle, _stream(stream)))

    def destroy(self):
        if self.handle:
            L.check(L.lib().ascq_comm_destroy(self.handle))
            self.handle = C.c_void_p()


def IpcExport(t: torch.Tensor) -> bytes:
    """CUDA IPC handle of a cudaMalloc'ed buffer of this process (``ascq_comm_ipc_export``)."""
    buf = C.create_string_buffer(int(L.lib().ascq_comm_ipc_handle_bytes()))
    L.check(L.lib().ascq_comm_ipc_export(buf, C.c_void_p(t.data_ptr())))
    return buf.raw


def IpcOpen(handle: bytes) -> int:
    """Maps a peer's buffer into this process; returns its device address (``ascq_comm_ipc_open``)."""
    p = C.c_void_p()
    L.check(L.lib().ascq_comm_ipc_open(C.byref(p), C.create_string_buffer(handle, len(handle))))
    return int(p.value)


def ShardColumns(N: int, nranks: int, rank: int):
    a, b = C.c_int(), C.c_int()
    L.check(L.lib().ascq_shard_columns(N, nranks, rank, C.byref(a), C.byref(b)))
    return a.value, b.value


def ShardGroupsLpt(groupList, nranks: int):
    """owner[g] = rank of group g (``ascq_shard_groups_lpt``)."""
    G = len(groupList)
    gl = (C_int64 * G)(*[int(v) for v in groupList])
    own = (C.c_int * G)()
    L.check(L.lib().ascq_shard_groups_lpt(gl, G, nranks, own))
    return list(own)


def MatmulW8A8Sharded(comm: Comm, C_buf_ptrs, A: torch.Tensor, B_local: torch.Tensor, scaleA=None, scaleB_local=None,
                      bias_local=None, N: Optional[int] = None, multicast_ptr: int = 0, stream=None):
    """Column-parallel W8A8 matmul of one rank (``ascq_matmul_w8a8_sharded``): ``C_buf_ptrs[r]`` = device address of rank
    r's bf16 [M, N] matrix; ``B_local`` [N / nranks, K].  The all-gather and the end-of-step exchange are part of the
    launch."""
    M, K = A.shape
    N = int(N if N is not None else B_local.shape[0] * comm.nranks)
    arr = (C.c_void_p * len(C_buf_ptrs))(*[C.c_void_p(int(v)) for v in C_buf_ptrs])
    L.check(L.lib().ascq_matmul_w8a8_sharded(comm.handle, arr, C.c_void_p(int(multicast_ptr)) if multicast_ptr else None,
                                             _ptr(A), _ptr(B_local), _ptr(scaleA), _ptr(scaleB_local), _ptr(bias_local), M, N, K,
                                             _stream(stream)))


def GroupMatmulMxfp4Sharded(comm: Comm, C_buf_ptrs, A_local: torch.Tensor, scaleA_local: torch.Tensor, B_local: torch.Tensor,
                            scaleB_local: torch.Tensor, groupList, K: int, N: int, workspace: torch.Tensor, stream=None):
    """Group-parallel MX-FP4 matmul of one rank (``ascq_group_matmul_mxfp4_sharded``): ``groupList`` holds all groups,
    the ``*_local`` tensors this rank's groups (``ShardGroupsLpt``) back to back in ascending group order."""
    G = len(groupList)
    gl = (C_int64 * G)(*[int(v) for v in groupList])
    arr = (C.c_void_p * len(C_buf_ptrs))(*[C.c_void_p(int(v)) for v in C_buf_ptrs])
    L.check(L.lib().ascq_group_matmul_mxfp4_sharded(comm.handle, arr, _ptr(A_local), _ptr(scaleA_local), _ptr(B_local),
                                                    _ptr(scaleB_local), gl, G, K, N, _ptr(workspace), workspace.numel(),
                                                    _stream(stream)))


def MeasureTensorRate(operand_dtype: int, k_blocks: int, stream=None) -> float:
    """Enqueues the MMA-only kernel (``ascq_measure_tensor_rate``) and returns the operations it performs; time the call
    with CUDA events to get the tensor cores' rate for int8 (``DT_I8``) or MX-FP4 (``DT_FP4X2_E2M1``) operands."""
    n = C.c_double()
    L.check(L.lib().ascq_measure_tensor_rate(operand_dtype, k_blocks, C.byref(n), _stream(stream)))
    return float(n.value)


def SetWaitLimitCycles(cycles: int):
    """Limit of the bounded device-side waits in SM cycles on the current device; <= 0 restores the default."""
    L.check(L.lib().ascq_set_wait_limit_cycles(int(cycles)))


def MatmulStatus(stream=None):
    """Synchronise and raise AscqError(ERR_TIMEOUT) if a matmul kernel gave up a bounded wait."""
    L.check(L.lib().ascq_matmul_status(_stream(stream)))


# ---- host tiling helpers (include/adv_api/quantization/ascend_*_tiling.h) ------------------------
def _dims(d):
    return (C.c_int64 * len(d))(*d), len(d)


def GetAscendQuantMaxMinTmpSize(srcShape, typeSize):
    a, r = _dims(srcShape)
    mx, mn = C.c_uint32(), C.c_uint32()
    L.check(L.lib().ascq_get_ascend_quant_max_min_tmp_size(a, r, typeSize, C.byref(mx), C.byref(mn)))
    return mx.value, mn.value


def GetAscendQuantTmpBufferFactorSize():
    a, b = C.c_uint32(), C.c_uint32(1)
    L.lib().ascq_get_ascend_quant_tmp_buffer_factor_size(C.byref(a), C.byref(b))
    return a.value, b.value


def GetAscendDequantMaxMinTmpSize(srcShape, typeSize):
    a, r = _dims(srcShape)
    mx, mn = C.c_uint32(), C.c_uint32()
    L.check(L.lib().ascq_get_ascend_dequant_max_min_tmp_size(a, r, typeSize, C.byref(mx), C.byref(mn)))
    return mx.value, mn.value


def GetAscendDequantTmpBufferFactorSize(srcShape):
    a, r = _dims(srcShape)
    x, y = C.c_uint32(), C.c_uint32()
    L.lib().ascq_get_ascend_dequant_tmp_buffer_factor_size(a, r, C.byref(x), C.byref(y))
    return x.value, y.value


def GetAscendAntiQuantMaxMinTmpSize(srcShape, scaleShape, isTranspose, inputDataType, outputDataType):
    a, r = _dims(srcShape)
    b, s = _dims(scaleShape)
    mx, mn = C.c_uint32(), C.c_uint32()
    L.check(L.lib().ascq_get_ascend_antiquant_max_min_tmp_size(a, r, b, s, int(isTranspose), inputDataType,
                                                               outputDataType, C.byref(mx), C.byref(mn)))
    return mx.value, mn.value


def GetAscendAntiQuantTmpBufferFactorSize(srcShape, scaleShape, isTranspose, inputDataType, outputDataType):
    a, r = _dims(srcShape)
    b, s = _dims(scaleShape)
    x, y = C.c_uint32(), C.c_uint32()
    L.lib().ascq_get_ascend_antiquant_tmp_buffer_factor_size(a, r, b, s, int(isTranspose), inputDataType,
                                                             outputDataType, C.byref(x), C.byref(y))
    return x.value, y.value
