"""ctypes face of oracle/_ref/libgarnet_ref_gpu.so: the reference's own GPU MoE (its scalar and
grouped WMMA paths behind RunGptOssMoe, and the production GptOssMarlin GEMM), compiled unchanged
from the reference's sources behind oracle/ref_gpu_shim.cu.  TEST AND MEASUREMENT INFRASTRUCTURE
ONLY: GPU parity tests compare the product with it on the same inputs, and the reference arm of
bench.py times it on the same box.  Operands are torch CUDA tensors in the reference's own
operand order (src/backends/tensorrt/gpt_oss_lowering.cpp:309-312), x and y in its fp32 carrier."""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libgarnet_ref_gpu.so")
_lib = None


def available() -> bool:
    return os.path.exists(LIB_PATH)


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        L = ctypes.CDLL(LIB_PATH)
        i, vp, f = ctypes.c_int, ctypes.c_void_p, ctypes.c_float
        L.ref_gpu_moe_workspace.restype = ctypes.c_size_t
        L.ref_gpu_moe_workspace.argtypes = [i, i, i, i, i, i, f, i]
        L.ref_gpu_moe_run.argtypes = [vp, vp, vp, i, i, i, i, i, f, i, vp]
        L.ref_gpu_marlin_create.restype = vp
        L.ref_gpu_marlin_create.argtypes = [i, i, i, i, f, i]
        L.ref_gpu_marlin_run.argtypes = [vp, vp, vp, vp, i, vp]
        L.ref_gpu_marlin_destroy.restype = None
        L.ref_gpu_marlin_destroy.argtypes = [vp]
        L.ref_gpu_rms_norm.argtypes = [vp, vp, vp, i, i, f, i, vp]
        L.ref_gpu_rope.argtypes = [vp, vp, vp, i, i, i, i, f, f, f, f, f, vp]
        L.ref_gpu_attention.argtypes = [vp, vp, vp, i, i, i, i, i, i, i, i, i, i, i, vp]
        L.ref_gpu_vocab_top1.argtypes = [vp, vp, i, i, i, vp]
        L.ref_gpu_decode_gemv.argtypes = [vp, vp, vp, i, i, i, i, i, i, i, i, vp]
        _lib = L
    return _lib


class RefMoe:
    """One layer's operands and the reference's two entry points over them.
    `operands` = [router W, router b, gate_up blocks, scales, bias, down blocks, scales, bias] as
    contiguous CUDA tensors (fp32 for weights of the router and biases, uint8 for blocks and scales)."""

    def __init__(self, hidden, intermediate, experts, top_k, operands, limit=7.0, prefill=0):
        import torch
        self.torch = torch
        self.shape = (hidden, intermediate, experts, top_k)
        self.limit, self.prefill = float(limit), int(prefill)
        self.operands = [t.contiguous() for t in operands]
        self._marlin = None
        self._ws = {}

    def _in(self, x):
        ptrs = [x.data_ptr()] + [t.data_ptr() for t in self.operands]
        return (ctypes.c_void_p * 9)(*ptrs)

    def _workspace(self, which, tokens):
        key = (which, tokens)
        if key not in self._ws:
            n = lib().ref_gpu_moe_workspace(which, tokens, *self.shape, self.limit, self.prefill)
            self._ws[key] = self.torch.zeros(max(n, 256), dtype=self.torch.uint8, device="cuda")
        return self._ws[key]

    def run(self, x, out=None):
        """RunGptOssMoe: x [tokens, hidden] fp32 (bf16-valued) -> y fp32.  Returns (cudaError_t, y)."""
        x = x.contiguous()
        y = out if out is not None else self.torch.empty_like(x)
        ws = self._workspace(0, x.shape[0])
        rc = lib().ref_gpu_moe_run(self._in(x), y.data_ptr(), ws.data_ptr(), x.shape[0], *self.shape, self.limit, self.prefill,
                                   self.torch.cuda.current_stream().cuda_stream)
        return rc, y

    def run_marlin(self, x, out=None):
        """GptOssMarlin::Run.  cudaErrorNotSupported (801) = the reference itself would fall back."""
        x = x.contiguous()
        y = out if out is not None else self.torch.empty_like(x)
        if self._marlin is None:
            self._marlin = lib().ref_gpu_marlin_create(*self.shape, self.limit, self.prefill)
        ws = self._workspace(1, x.shape[0])
        rc = lib().ref_gpu_marlin_run(self._marlin, self._in(x), y.data_ptr(), ws.data_ptr(), x.shape[0],
                                      self.torch.cuda.current_stream().cuda_stream)
        return rc, y

    def close(self):
        if self._marlin:
            lib().ref_gpu_marlin_destroy(self._marlin)
            self._marlin = None
