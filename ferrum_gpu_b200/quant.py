"""Quantised weights and their products: the host-side mirror of `ferrum_wgpu::ops::quant`
(ferrum_wgpu/src/ops/quant.rs). Same names and argument meaning; the arithmetic runs in the CUDA
library."""
from __future__ import annotations

import ctypes as C
from enum import IntEnum

import numpy as np

from . import _ffi
from .device import CudaError, Device


class QKind(IntEnum):
    """`QKind` restricted to the formats on this path, plus F32 for ineligible matrices."""
    F32 = _ffi.FC_F32
    Q8_0 = _ffi.FC_Q8_0
    Q4_0 = _ffi.FC_Q4_0
    F16 = _ffi.FC_F16
    FP8_E4M3 = _ffi.FC_FP8_E4M3
    FP8_E5M2 = _ffi.FC_FP8_E5M2
    MXFP4 = _ffi.FC_MXFP4
    Q2_K = _ffi.FC_Q2_K

    def label(self) -> str:
        """`QKind::label` (ops/quant.rs:L60-L70)."""
        return {0: "F32", 1: "Q8_0", 2: "Q4_0", 3: "F16", 4: "FP8 E4M3", 5: "FP8 E5M2", 6: "MXFP4", 7: "Q2_K"}[int(self)]


class Mode(IntEnum):
    EXACT_F32 = _ffi.FC_EXACT_F32
    TENSOR_F16 = _ffi.FC_TENSOR_F16


def eligible(k: int) -> bool:
    """ops/quant.rs:L125-L128"""
    return k > 0 and k % 32 == 0


def block_bytes(kind: QKind, n_elems: int) -> int:
    return _ffi.load().fc_block_bytes(int(kind), n_elems)


class QWeight:
    """A quantised weight resident on the device: `n` output columns of `k` inputs (ops/quant.rs:L150-L183)."""

    def __init__(self, dev: Device, handle):
        self.dev, self._h, self._lib = dev, handle, _ffi.load()
        kind, k, n, b = C.c_int(), C.c_uint32(), C.c_uint32(), C.c_uint64()
        dev.check(self._lib.fc_qweight_info(handle, C.byref(kind), C.byref(k), C.byref(n), C.byref(b)))
        self._kind, self._k, self._n, self._bytes = QKind(kind.value), k.value, n.value, b.value
        dev.adopt(self)

    def kind(self) -> QKind:
        return self._kind

    def k(self) -> int:
        return self._k

    def n(self) -> int:
        return self._n

    def device_bytes(self) -> int:
        return self._bytes

    @property
    def handle(self):
        return self._h

    def close(self):
        if self._h:
            self._lib.fc_qweight_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def blocks(self) -> np.ndarray:
        """The GGUF block bytes the device holds (inverse of the upload repack)."""
        out = np.empty(block_bytes(self._kind, self._k * self._n), dtype=np.uint8)
        self.dev.check(self._lib.fc_qweight_blocks(self._h, out.ctypes.data, out.size))
        return out

    def dequantised(self) -> np.ndarray:
        """`[n, k]` f32 values the kernels compute with, decoded on the device."""
        out = np.empty(self._k * self._n, dtype=np.float32)
        self.dev.check(self._lib.fc_dequant(self._h, out.ctypes.data, out.size))
        return out.reshape(self._n, self._k)


def upload_quantised(dev: Device, kind: QKind, w, k: int, n: int) -> QWeight:
    """Quantise an `[in, out]` f32 weight and upload it (ops/quant.rs:L279-L288)."""
    w = np.ascontiguousarray(w, dtype=np.float32).reshape(-1)
    if w.size != k * n:
        raise CudaError(_ffi.FC_ERR_SHAPE,
                        f"cannot quantise {w.size} elements as a {k} x {n} weight in whole 32-blocks")
    h = C.c_void_p()
    dev.check(_ffi.load().fc_qweight_create(dev.handle, int(kind), w.ctypes.data, k, n, C.byref(h)))
    return QWeight(dev, h)


def upload_qweight(dev: Device, kind: QKind, data, k: int, n: int) -> QWeight:
    """Upload GGUF block bytes (`n` rows of `k/32` blocks) as a resident weight (ops/quant.rs:L266-L277)."""
    b = np.ascontiguousarray(data, dtype=np.uint8).reshape(-1)
    h = C.c_void_p()
    dev.check(_ffi.load().fc_qweight_create_from_blocks(dev.handle, int(kind), b.ctypes.data, b.size, k, n,
                                                        C.byref(h)))
    return QWeight(dev, h)


def linear_q(dev: Device, x, w: QWeight, rows: int, mode: Mode = Mode.EXACT_F32) -> np.ndarray:
    """`y[rows, n] = x[rows, k] * W` (ops/quant.rs:L326-L335); host buffers in and out."""
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    if x.size != rows * w.k():
        raise CudaError(_ffi.FC_ERR_SHAPE, f"linear_q x has {x.size} elements, needs {rows * w.k()}")
    y = np.empty(rows * w.n(), dtype=np.float32)
    dev.check(_ffi.load().fc_qmatmul(w.handle, x.ctypes.data, rows, y.ctypes.data, int(mode)))
    return y.reshape(rows, w.n())
