"""Host-side mirror of the reference's linear operator over packed weights.

``QuantLinear.forward`` has the call shape of ``QatLinear::forward``
(crates/aarambh-studio-quant/src/qat.rs:315-348): any leading dimensions are
flattened into tokens, the last dimension is ``in_features``, there is no bias.
The weight stays packed on the GPU; dequantisation is fused into the product.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import _lib
from ._lib import check, lib

_TORCH_DTYPES = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _TORCH_DTYPES[dtype]
    except KeyError:
        raise _lib.Ab2Error(-3, f"unsupported dtype {dtype}") from None


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(a) -> int:
    """Address of a contiguous numpy array (host) or torch tensor (device/host)."""
    if isinstance(a, torch.Tensor):
        if not a.is_contiguous():
            raise _lib.Ab2Error(-1, "tensor must be contiguous")
        return a.data_ptr()
    a = np.ascontiguousarray(a)
    return a.ctypes.data


class QuantLinear:
    """A packed [out_features, in_features] weight living in GPU memory."""

    def __init__(self, handle: int, keepalive=None):
        self._h = C.c_void_p(handle)
        self._keep = keepalive
        n, k, g, f = C.c_int(), C.c_int(), C.c_int(), C.c_int()
        check(lib.ab2_qweight_shape(self._h, n, k, g, f))
        self.out_features, self.in_features, self.group, self.format = n.value, k.value, g.value, f.value

    # -- constructors from the reference's serialised layouts -----------------
    @classmethod
    def _make(cls, fn, *args):
        h = C.c_void_p()
        check(fn(C.byref(h), *args))
        return cls(h.value)

    @classmethod
    def from_i8_tensor(cls, codes, scale: float, N: int, K: int):
        codes = _contig(codes, np.int8)
        return cls._make(lib.ab2_qweight_from_i8_tensor, _ptr(codes), float(scale), N, K)

    @classmethod
    def from_i8_channel(cls, codes, scales, N: int, K: int):
        codes = _contig(codes, np.int8); scales = _contig(scales, np.float32)
        return cls._make(lib.ab2_qweight_from_i8_channel, _ptr(codes), _ptr(scales), N, K)

    @classmethod
    def from_i4_affine(cls, packed, scales, zeros, N: int, K: int, group: int):
        packed = _contig(packed, np.uint8); scales = _contig(scales, np.float32)
        zeros = _contig(zeros, np.float32)
        return cls._make(lib.ab2_qweight_from_i4_affine, _ptr(packed), _ptr(scales), _ptr(zeros), N, K, group)

    @classmethod
    def from_q4km_blocks(cls, blocks, N: int, K: int):
        blocks = _contig(blocks, np.uint8)
        return cls._make(lib.ab2_qweight_from_q4km_blocks, _ptr(blocks), N, K)

    @classmethod
    def from_w4a16_gptq(cls, qweight, scales_bf16, qzeros, N: int, K: int, group: int):
        return cls._make(lib.ab2_qweight_from_w4a16_gptq, _ptr(_contig(qweight, np.uint32)),
                         _ptr(_contig(scales_bf16, np.uint16)), _ptr(_contig(qzeros, np.uint32)), N, K, group)

    @classmethod
    def from_w4a16_awq(cls, qweight, scales_bf16, qzeros, N: int, K: int, group: int):
        return cls._make(lib.ab2_qweight_from_w4a16_awq, _ptr(_contig(qweight, np.uint32)),
                         _ptr(_contig(scales_bf16, np.uint16)), _ptr(_contig(qzeros, np.uint32)), N, K, group)

    # -- device-side quantisers ----------------------------------------------
    @classmethod
    def quantise(cls, weight: torch.Tensor, method: str, group: int = 128):
        """Quantise a dense f32 CUDA weight with the reference arithmetic.

        ``method``: ``int8`` (per tensor), ``int8_channel``, ``int4`` (affine f32
        parameters), ``q4_k_m`` (256-blocks), ``w4a16`` (bf16 scale, u4 zero).
        """
        if weight.dtype != torch.float32 or not weight.is_cuda or weight.dim() != 2:
            raise _lib.Ab2Error(-3, "quantise expects a 2-D float32 CUDA tensor")
        w = weight.contiguous()
        N, K = w.shape
        s = stream_ptr()
        if method == "int8":
            return cls._make(lib.ab2_qweight_quantise_i8, w.data_ptr(), N, K, 0, s)
        if method == "int8_channel":
            return cls._make(lib.ab2_qweight_quantise_i8, w.data_ptr(), N, K, 1, s)
        if method == "int4":
            return cls._make(lib.ab2_qweight_quantise_i4_affine, w.data_ptr(), N, K, group, s)
        if method == "q4_k_m":
            return cls._make(lib.ab2_qweight_quantise_q4km, w.data_ptr(), N, K, s)
        if method == "w4a16":
            return cls._make(lib.ab2_qweight_quantise_w4a16, w.data_ptr(), N, K, group, s)
        raise _lib.Ab2Error(-7, f"unsupported quantisation method '{method}'")

    # -- operator -------------------------------------------------------------
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.shape[-1] != self.in_features:
            raise _lib.Ab2Error(-1, f"input has {x.shape[-1]} features, weight expects {self.in_features}")
        x2 = x.contiguous().view(-1, self.in_features)
        y = torch.empty((x2.shape[0], self.out_features), dtype=x.dtype, device=x.device)
        check(lib.ab2_qlinear_forward(self._h, x2.data_ptr(), x2.shape[0], dtype_code(x.dtype),
                                      y.data_ptr(), stream_ptr()))
        return y.view(*x.shape[:-1], self.out_features)

    __call__ = forward

    def dequantise(self, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        out = torch.empty((self.out_features, self.in_features), dtype=dtype, device="cuda")
        check(lib.ab2_qweight_dequant(self._h, out.data_ptr(), dtype_code(dtype), stream_ptr()))
        return out

    def nbytes(self) -> int:
        n = C.c_size_t()
        check(lib.ab2_qweight_nbytes(self._h, C.byref(n)))
        return n.value

    def export(self):
        """Packed codes and parameters as numpy arrays (constructor layout)."""
        N, K, g = self.out_features, self.in_features, self.group
        n = N * K
        if self.format == _lib.FMT_I8:
            codes = np.empty((N, K), np.int8); scales = np.empty(N, np.float32)
            check(lib.ab2_qweight_export(self._h, codes.ctypes.data, scales.ctypes.data, None))
            return codes, scales, None
        if self.format == _lib.FMT_I4_AFFINE:
            ng = -(-n // g)
            codes = np.empty(-(-n // 2), np.uint8)
            scales = np.empty(ng, np.float32); zeros = np.empty(ng, np.float32)
            check(lib.ab2_qweight_export(self._h, codes.ctypes.data, scales.ctypes.data, zeros.ctypes.data))
            return codes, scales, zeros
        if self.format == _lib.FMT_Q4KM:
            blocks = np.empty(-(-n // 256) * 132, np.uint8)
            check(lib.ab2_qweight_export(self._h, blocks.ctypes.data, None, None))
            return blocks, None, None
        G = K // g
        codes = np.empty((N, K // 8), np.uint32)
        scales = np.empty((N, G), np.uint16); zeros = np.empty((N, -(-G // 8)), np.uint32)
        check(lib.ab2_qweight_export(self._h, codes.ctypes.data, scales.ctypes.data, zeros.ctypes.data))
        return codes, scales, zeros

    def __del__(self):
        try:
            if self._h:
                lib.ab2_qweight_destroy(self._h)
                self._h = None
        except Exception:
            pass


def _contig(a, dtype):
    if isinstance(a, torch.Tensor):
        return a.contiguous()
    return np.ascontiguousarray(a, dtype=dtype)
