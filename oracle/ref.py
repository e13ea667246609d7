"""ctypes face of oracle/_ref/libgarnet_ref.so: the reference's own int4 CPU
sources (weight quantizer and Q4Q8Linear) compiled unchanged behind
oracle/ref_shim.cpp.  TEST INFRASTRUCTURE ONLY; used to pin the oracle, to
generate golden vectors and as the timed CPU reference arm of the benchmark."""
from __future__ import annotations

import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libgarnet_ref.so")
_lib = None


def available() -> bool:
    return os.path.exists(LIB_PATH)


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        L = ctypes.CDLL(LIB_PATH)
        L.ref_last_error.restype = ctypes.c_char_p
        L.ref_quantize_int4.restype = ctypes.c_int
        L.ref_quantize_int4.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_longlong,
                                        ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                                        ctypes.POINTER(ctypes.c_double)]
        L.ref_q4q8_create.restype = ctypes.c_void_p
        L.ref_q4q8_create.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int]
        L.ref_q4q8_forward.restype = ctypes.c_int
        L.ref_q4q8_forward.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int]
        L.ref_q4q8_destroy.restype = None
        L.ref_q4q8_destroy.argtypes = [ctypes.c_void_p]
        _lib = L
    return _lib


def quantize_int4(w: np.ndarray, block: int):
    """Garnet::QuantizeSymmetricINT4 on an fp32 matrix -> (nibbles, fp16 scale bits, max error)."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    rows, cols = w.shape
    packed = np.zeros(rows * cols // 2, dtype=np.uint8)
    scales = np.zeros(rows * (cols // block), dtype=np.uint16)
    err = ctypes.c_double(0)
    rc = lib().ref_quantize_int4(w.ctypes.data, rows, cols, block, packed.ctypes.data,
                                 scales.ctypes.data, ctypes.byref(err))
    if rc:
        raise RuntimeError(lib().ref_last_error().decode())
    return packed, scales.reshape(rows, cols // block), err.value


class Q4Q8Linear:
    """Garnet::Q4Q8Linear over canonical nibbles and fp32 scales."""

    def __init__(self, packed: np.ndarray, scales_f32: np.ndarray, rows: int, cols: int, block: int):
        self._packed = np.ascontiguousarray(packed, dtype=np.uint8)
        self._scales = np.ascontiguousarray(scales_f32, dtype=np.float32)
        self.rows, self.cols = rows, cols
        self._h = lib().ref_q4q8_create(self._packed.ctypes.data, self._scales.ctypes.data, rows, cols, block)
        if not self._h:
            raise RuntimeError(lib().ref_last_error().decode())

    def forward(self, x: np.ndarray, threads: int = 1, out: np.ndarray | None = None) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(self.cols)
        y = np.empty(self.rows, dtype=np.float32) if out is None else out
        if lib().ref_q4q8_forward(self._h, x.ctypes.data, y.ctypes.data, threads):
            raise RuntimeError(lib().ref_last_error().decode())
        return y

    def __del__(self):
        if getattr(self, "_h", None):
            lib().ref_q4q8_destroy(self._h)
            self._h = None
