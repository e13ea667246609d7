"""CPU oracle for the quantized-matmul path.  TEST INFRASTRUCTURE ONLY.

Python face of ``oracle/oracle.c`` (a plain-C restatement of the reference's
int4 linear and MXFP4 MoE arithmetic, each C function citing the reference
file:line it follows) plus small numpy helpers.  Only ``tests/``,
``__graft_entry__.smoke()`` and the CPU-baseline / reference legs of ``bench.py``
may import this package; the product (``garnet_b200``) never does.

Pinning: ``tests/test_oracle_golden.py`` checks these functions against the
committed golden vectors in ``tests/golden/`` (generated from the reference's own
compiled int4 sources and from its pure-Python MoE) and, when
``oracle/_ref/libgarnet_ref.so`` is present, bit-for-bit against the reference
itself.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "liboracle.so")
_lib = None

_u8p = ctypes.POINTER(ctypes.c_uint8)
_u16p = ctypes.POINTER(ctypes.c_uint16)
_i32p = ctypes.POINTER(ctypes.c_int32)
_f32p = ctypes.POINTER(ctypes.c_float)
_f64p = ctypes.POINTER(ctypes.c_double)


def build(force: bool = False) -> str:
    """Compiles oracle.c with gcc (via oracle/Makefile) if the library is stale."""
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "--no-print-directory"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_LIB_PATH)
        L.orc_bf16_round.restype = ctypes.c_float
        L.orc_bf16_round.argtypes = [ctypes.c_float]
        L.orc_threads.restype = ctypes.c_int
        L.orc_float_to_fp16.restype = ctypes.c_uint16
        L.orc_float_to_fp16.argtypes = [ctypes.c_float]
        L.orc_fp16_to_float.restype = ctypes.c_float
        L.orc_fp16_to_float.argtypes = [ctypes.c_uint16]
        L.orc_int4_quantize.restype = ctypes.c_double
        L.orc_int4_quantize.argtypes = [_f32p, ctypes.c_long, ctypes.c_long, ctypes.c_int,
                                        ctypes.c_int, _u8p, _u16p]
        L.orc_int4_dequant.restype = None
        L.orc_int4_dequant.argtypes = [_u8p, _f32p, ctypes.c_long, ctypes.c_long, ctypes.c_int, _f32p]
        L.orc_w4a16_exact.restype = None
        L.orc_w4a16_exact.argtypes = [_u8p, _f32p, ctypes.c_long, ctypes.c_long, ctypes.c_int,
                                      _f32p, ctypes.c_long, _f32p, _f64p]
        L.orc_q4q8_forward.restype = None
        L.orc_q4q8_forward.argtypes = [_u8p, _f32p, ctypes.c_long, ctypes.c_long, ctypes.c_int,
                                       _f32p, _f32p, ctypes.c_int]
        L.orc_mxfp4_value.restype = ctypes.c_float
        L.orc_mxfp4_value.argtypes = [ctypes.c_int, ctypes.c_int]
        L.orc_mxfp4_value_ldexp.restype = ctypes.c_float
        L.orc_mxfp4_value_ldexp.argtypes = [ctypes.c_int, ctypes.c_int]
        L.orc_mxfp4_dequant.restype = None
        L.orc_mxfp4_dequant.argtypes = [_u8p, _u8p, ctypes.c_long, ctypes.c_long, _f32p]
        L.orc_moe_route.restype = None
        L.orc_moe_route.argtypes = [_f32p, _f32p, _f32p, ctypes.c_long, ctypes.c_int, ctypes.c_int,
                                    ctypes.c_int, _f32p, _i32p, _f32p]
        L.orc_moe_experts.restype = None
        L.orc_moe_experts.argtypes = [_f32p, _i32p, _f32p, _u8p, _u8p, _f32p, _u8p, _u8p, _f32p,
                                      ctypes.c_long, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                      ctypes.c_int, ctypes.c_float, ctypes.c_int, ctypes.c_int,
                                      ctypes.c_int, ctypes.c_int, ctypes.c_int, _f32p, _f32p]
        _lib = L
    return _lib


def _c(a: np.ndarray, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


def _p(a: np.ndarray, ptype):
    return a.ctypes.data_as(ptype)


# --------------------------------------------------------------- bf16 helpers

def bf16_round(x) -> np.ndarray:
    """fp32 -> nearest-even bf16 -> fp32 (kernel_parity.cpp:20)."""
    a = np.ascontiguousarray(x, dtype=np.float32)
    v = a.view(np.uint32).astype(np.uint64)
    nan = (v & 0x7FFFFFFF) > 0x7F800000
    r = ((v + 0x7FFF + ((v >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    r = np.where(nan, (v.astype(np.uint32) | 0x00400000) & 0xFFFF0000, r).astype(np.uint32)
    return r.view(np.float32).reshape(a.shape)


def bf16_bits(x) -> np.ndarray:
    """fp32 -> bf16 bit patterns (uint16), round-to-nearest-even."""
    return (bf16_round(x).view(np.uint32) >> 16).astype(np.uint16)


def bf16_from_bits(b) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# ----------------------------------------------------------------- int4 path

def int4_unpack(packed: np.ndarray, rows: int, cols: int) -> np.ndarray:
    """Canonical nibbles -> int8 [rows, cols] (weight_quantization_test.cpp:47-53)."""
    p = _c(packed, np.uint8).reshape(-1)
    lo = (p & 15).astype(np.int8)
    hi = (p >> 4).astype(np.int8)
    q = np.empty(p.size * 2, dtype=np.int8)
    q[0::2] = lo
    q[1::2] = hi
    q = np.where(q >= 8, q - 16, q).astype(np.int8)
    return q[: rows * cols].reshape(rows, cols)


def int4_pack(q: np.ndarray) -> np.ndarray:
    """int8 values in [-8,7] -> canonical nibbles (weight_quantization.cpp:253-259)."""
    flat = (np.ascontiguousarray(q, dtype=np.int8).reshape(-1) & 15).astype(np.uint8)
    return (flat[0::2] | (flat[1::2] << 4)).astype(np.uint8)


def int4_quantize(w: np.ndarray, block: int, scale_kind: str = "fp16"):
    """Reference quantizer restatement; returns (packed u8, scale bits u16, max error)."""
    w = _c(w, np.float32)
    rows, cols = w.shape
    packed = np.zeros((rows * cols + 1) // 2, dtype=np.uint8)
    scales = np.zeros(rows * (cols // block), dtype=np.uint16)
    err = lib().orc_int4_quantize(_p(w, _f32p), rows, cols, block, 0 if scale_kind == "fp16" else 1,
                                  _p(packed, _u8p), _p(scales, _u16p))
    return packed, scales.reshape(rows, cols // block), err


def int4_dequant(packed, scales_f32, rows, cols, block) -> np.ndarray:
    packed = _c(packed, np.uint8)
    s = _c(scales_f32, np.float32)
    out = np.empty((rows, cols), dtype=np.float32)
    lib().orc_int4_dequant(_p(packed, _u8p), _p(s, _f32p), rows, cols, block, _p(out, _f32p))
    return out


def w4a16_exact(packed, scales_f32, N, K, block, x, want_f64=True):
    """Exact W4A16 product; returns (y32 [M,N], y64 [M,N] or None), unrounded."""
    packed = _c(packed, np.uint8)
    s = _c(scales_f32, np.float32)
    x = _c(x, np.float32).reshape(-1, K)
    M = x.shape[0]
    y32 = np.empty((M, N), dtype=np.float32)
    y64 = np.empty((M, N), dtype=np.float64) if want_f64 else None
    lib().orc_w4a16_exact(_p(packed, _u8p), _p(s, _f32p), N, K, block, _p(x, _f32p), M,
                          _p(y32, _f32p), _p(y64, _f64p) if want_f64 else None)
    return y32, y64


def w4a16_blas(packed, scales_f32, N, K, block, x) -> np.ndarray:
    """Same product through a float64 BLAS matmul, for shapes too large for the
    scalar loop.  Dequantisation is the exact q*s; only the summation order differs."""
    w = int4_dequant(packed, scales_f32, N, K, block).astype(np.float64)
    return np.asarray(x, dtype=np.float64).reshape(-1, K) @ w.T


def q4q8_forward(packed, scales_f32, N, K, block, x, threads=1) -> np.ndarray:
    """Restatement of the reference CPU operator Q4Q8Linear::Forward (W4A8)."""
    packed = _c(packed, np.uint8)
    s = _c(scales_f32, np.float32)
    x = _c(x, np.float32).reshape(K)
    y = np.empty(N, dtype=np.float32)
    lib().orc_q4q8_forward(_p(packed, _u8p), _p(s, _f32p), N, K, block, _p(x, _f32p), _p(y, _f32p), threads)
    return y


# ---------------------------------------------------------------- MXFP4 / MoE

def mxfp4_table() -> np.ndarray:
    """[256 scales, 16 codes] fp32 values built by the bit constructor."""
    L = lib()
    return np.array([[L.orc_mxfp4_value(c, e) for c in range(16)] for e in range(256)], dtype=np.float32)


def mxfp4_table_ldexp() -> np.ndarray:
    L = lib()
    return np.array([[L.orc_mxfp4_value_ldexp(c, e) for c in range(16)] for e in range(256)], dtype=np.float32)


def mxfp4_dequant(blocks, scales, rows, width) -> np.ndarray:
    b = _c(blocks, np.uint8)
    s = _c(scales, np.uint8)
    out = np.empty((rows, width), dtype=np.float32)
    lib().orc_mxfp4_dequant(_p(b, _u8p), _p(s, _u8p), rows, width, _p(out, _f32p))
    return out


def moe_route(x, router_w, router_b, experts, topk):
    """Returns (bf16-rounded logits [T,E], selected [T,k] int32, probs [T,k])."""
    x = _c(x, np.float32)
    T, H = x.shape
    w = _c(router_w, np.float32)
    b = _c(router_b, np.float32)
    logits = np.empty((T, experts), dtype=np.float32)
    sel = np.empty((T, topk), dtype=np.int32)
    pr = np.empty((T, topk), dtype=np.float32)
    lib().orc_moe_route(_p(x, _f32p), _p(w, _f32p), _p(b, _f32p), T, H, experts, topk,
                        _p(logits, _f32p), _p(sel, _i32p), _p(pr, _f32p))
    return logits, sel, pr


def moe_experts(x, selected, probs, gu_blocks, gu_scales, gu_bias, dn_blocks, dn_scales, dn_bias,
                hidden, inter, experts, topk, limit=7.0, expert_lo=0, expert_hi=None,
                modulo=0, residue=0, round_output=True, want_mass=False):
    """Experts for a given routing.  With want_mass, also returns
    sum_j |per-slot value| * p_j, the scale of the summands of each output."""
    x = _c(x, np.float32).reshape(-1, hidden)
    T = x.shape[0]
    sel = _c(selected, np.int32)
    pr = _c(probs, np.float32)
    gb, gs, gbi = _c(gu_blocks, np.uint8), _c(gu_scales, np.uint8), _c(gu_bias, np.float32)
    db, ds, dbi = _c(dn_blocks, np.uint8), _c(dn_scales, np.uint8), _c(dn_bias, np.float32)
    y = np.empty((T, hidden), dtype=np.float32)
    mass = np.empty((T, hidden), dtype=np.float32) if want_mass else None
    lib().orc_moe_experts(_p(x, _f32p), _p(sel, _i32p), _p(pr, _f32p), _p(gb, _u8p), _p(gs, _u8p),
                          _p(gbi, _f32p), _p(db, _u8p), _p(ds, _u8p), _p(dbi, _f32p), T, hidden,
                          inter, experts, topk, limit, expert_lo,
                          experts if expert_hi is None else expert_hi, modulo, residue,
                          1 if round_output else 0, _p(y, _f32p), _p(mass, _f32p) if want_mass else None)
    return (y, mass) if want_mass else y


def moe_rows_hidden(x_rows, row_expert, gu_blocks, gu_scales, gu_bias, hidden, inter, limit=7.0):
    """SwiGLU activations [rows, inter] of already routed rows (one expert per row)."""
    x = _c(x_rows, np.float32).reshape(-1, hidden)
    ex = _c(row_expert, np.int32).reshape(-1)
    gb, gs, gbi = _c(gu_blocks, np.uint8), _c(gu_scales, np.uint8), _c(gu_bias, np.float32)
    out = np.empty((x.shape[0], inter), dtype=np.float32)
    L = lib()
    L.orc_moe_rows_hidden.restype = None
    L.orc_moe_rows_hidden.argtypes = [_f32p, _i32p, _u8p, _u8p, _f32p, ctypes.c_long, ctypes.c_int, ctypes.c_int,
                                      ctypes.c_float, _f32p]
    L.orc_moe_rows_hidden(_p(x, _f32p), _p(ex, _i32p), _p(gb, _u8p), _p(gs, _u8p), _p(gbi, _f32p), x.shape[0], hidden,
                          inter, limit, _p(out, _f32p))
    return out


def moe_rows_down(h_rows, row_expert, dn_blocks, dn_scales, dn_bias, hidden, inter):
    """Per-row values bf(bf(h . w_down) + b) [rows, hidden] for given activations."""
    h = _c(h_rows, np.float32).reshape(-1, inter)
    ex = _c(row_expert, np.int32).reshape(-1)
    db, ds, dbi = _c(dn_blocks, np.uint8), _c(dn_scales, np.uint8), _c(dn_bias, np.float32)
    out = np.empty((h.shape[0], hidden), dtype=np.float32)
    L = lib()
    L.orc_moe_rows_down.restype = None
    L.orc_moe_rows_down.argtypes = [_f32p, _i32p, _u8p, _u8p, _f32p, ctypes.c_long, ctypes.c_int, ctypes.c_int, _f32p]
    L.orc_moe_rows_down(_p(h, _f32p), _p(ex, _i32p), _p(db, _u8p), _p(ds, _u8p), _p(dbi, _f32p), h.shape[0], hidden,
                        inter, _p(out, _f32p))
    return out


def moe_forward(x, router_w, router_b, gu_blocks, gu_scales, gu_bias, dn_blocks, dn_scales, dn_bias,
                hidden, inter, experts, topk, limit=7.0):
    """Route + experts; returns (y, logits, selected, probs)."""
    logits, sel, pr = moe_route(np.asarray(x, np.float32).reshape(-1, hidden), router_w, router_b, experts, topk)
    y = moe_experts(x, sel, pr, gu_blocks, gu_scales, gu_bias, dn_blocks, dn_scales, dn_bias,
                    hidden, inter, experts, topk, limit)
    return y, logits, sel, pr
