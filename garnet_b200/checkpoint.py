"""Host-side caller of the checkpoint entry points of libgarnet_b200.so: the .safetensors reader and
writer, the host int4 quantizer, derived-constant names and the packed-constant cache
(garnet_b200_safetensors_*, garnet_b200_int4_quantize_host, garnet_b200_packed_tensor_name,
garnet_b200_checkpoint_build_cache).  Mirrors Garnet::SafeTensorsIndex
(src/model/safetensors_index.h:42-60)."""
from __future__ import annotations

import ctypes

import numpy as np

from ._lib import BF16, FP16, FP32, check, lib

_NP = {"F32": np.float32, "F16": np.float16, "BF16": np.uint16, "U8": np.uint8, "I8": np.int8, "I32": np.int32,
       "I64": np.int64, "U16": np.uint16, "I16": np.int16, "F64": np.float64, "U32": np.uint32, "BOOL": np.uint8}


class SafeTensors:
    """A checkpoint opened for reading: a file, a Hugging Face shard index or a directory with either."""

    def __init__(self, path: str):
        self._h = ctypes.c_void_p(None)
        check(lib().garnet_b200_safetensors_open(str(path).encode(), ctypes.byref(self._h)))

    def __len__(self) -> int:
        return lib().garnet_b200_safetensors_count(self._h)

    def _entry(self, index: int, name):
        nm, dt = ctypes.c_char_p(), ctypes.c_char_p()
        rank, shape = ctypes.c_int(0), (ctypes.c_longlong * 8)()
        data, nbytes = ctypes.c_void_p(None), ctypes.c_size_t(0)
        check(lib().garnet_b200_safetensors_entry(self._h, index, name.encode() if name is not None else None, ctypes.byref(nm),
                                                  ctypes.byref(dt), ctypes.byref(rank), shape, ctypes.byref(data),
                                                  ctypes.byref(nbytes)))
        return nm.value.decode(), dt.value.decode(), tuple(shape[:rank.value]), data.value, nbytes.value

    def names(self):
        return [self._entry(i, None)[0] for i in range(len(self))]

    def info(self, name: str):
        _, dtype, shape, _, nbytes = self._entry(-1, name)
        return dtype, shape, nbytes

    def tensor(self, name: str) -> np.ndarray:
        """A copy of the tensor (bf16 as its uint16 bit patterns)."""
        _, dtype, shape, ptr, nbytes = self._entry(-1, name)
        raw = np.ctypeslib.as_array((ctypes.c_ubyte * nbytes).from_address(ptr)).copy() if nbytes else np.zeros(0, np.uint8)
        return raw.view(_NP[dtype]).reshape(shape)

    def build_cache(self, out_path: str, group: int = 128, scale_dtype: int = BF16, moe_layouts: int = 0, tp_rank: int = 0,
                    tp_world: int = 1) -> None:
        check(lib().garnet_b200_checkpoint_build_cache(self._h, str(out_path).encode(), group, scale_dtype, moe_layouts, tp_rank,
                                                       tp_world))

    def close(self) -> None:
        if self._h:
            lib().garnet_b200_safetensors_close(self._h)
            self._h = ctypes.c_void_p(None)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def write_safetensors(path: str, tensors: dict, dtypes: dict | None = None) -> None:
    """tensors: name -> numpy array; dtypes: name -> safetensors dtype string where numpy cannot say (BF16 bits in uint16)."""
    names = list(tensors)
    arrays = [np.ascontiguousarray(tensors[n]) for n in names]
    back = {np.dtype(v): k for k, v in _NP.items() if k not in ("BF16", "BOOL", "U16")}
    back[np.dtype(np.uint16)] = "U16"
    dts = [(dtypes or {}).get(n) or back[a.dtype] for n, a in zip(names, arrays)]
    n = len(names)
    c_names = (ctypes.c_char_p * n)(*[s.encode() for s in names])
    c_dtypes = (ctypes.c_char_p * n)(*[s.encode() for s in dts])
    c_ranks = (ctypes.c_int * n)(*[a.ndim for a in arrays])
    shapes = [(ctypes.c_longlong * max(1, a.ndim))(*a.shape) for a in arrays]
    c_shapes = (ctypes.c_void_p * n)(*[ctypes.addressof(s) for s in shapes])
    c_datas = (ctypes.c_void_p * n)(*[a.ctypes.data for a in arrays])
    c_bytes = (ctypes.c_size_t * n)(*[a.nbytes for a in arrays])
    check(lib().garnet_b200_safetensors_write(str(path).encode(), c_names, c_dtypes, c_ranks, c_shapes, c_datas, c_bytes, n))


def quantize_int4_host(w: np.ndarray, group: int = 128, scale_dtype: int = BF16, w_dtype: int | None = None):
    """QuantizeSymmetricINT4 on the host; w is fp32, fp16, or uint16 bf16 bits (w_dtype = BF16)."""
    w = np.ascontiguousarray(w)
    code = w_dtype if w_dtype is not None else {np.dtype(np.float32): FP32, np.dtype(np.float16): FP16}[w.dtype]
    n, k = w.shape
    nib = np.empty(n * k // 2, np.uint8)
    sc = np.empty((n, k // group), np.uint16)
    err = ctypes.c_double(0)
    check(lib().garnet_b200_int4_quantize_host(w.ctypes.data, code, n, k, group, scale_dtype, nib.ctypes.data, sc.ctypes.data,
                                               ctypes.byref(err)))
    return nib, sc, err.value


def packed_name(source: str, kind: int, a: int, b: int, c: int = 0) -> str:
    out = ctypes.create_string_buffer(1024)
    check(lib().garnet_b200_packed_tensor_name(source.encode(), kind, a, b, c, out, 1024))
    return out.value.decode()


def parse_packed_name(name: str):
    kind, a, b, c = ctypes.c_int(), ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    src = ctypes.c_char_p()
    check(lib().garnet_b200_packed_tensor_name_parse(name.encode(), ctypes.byref(kind), ctypes.byref(a), ctypes.byref(b),
                                                     ctypes.byref(c), ctypes.byref(src)))
    return kind.value, a.value, b.value, c.value, src.value.decode()
