"""ctypes binding of libgarnet_b200.so (the C ABI declared in include/garnet_b200.h).

There is no fallback: if the library is missing or a call fails, an exception
is raised."""
from __future__ import annotations

import ctypes
import os

from . import _build

OK, INVALID_VALUE, NOT_SUPPORTED, CUDA_ERROR, DEVICE_FAULT, OUT_OF_MEMORY = range(6)
FP16, BF16, FP32 = 0, 1, 2

_lib = None


class GarnetB200Error(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"garnet_b200 status {code}: {message}")
        self.code = code


def _declare(L: ctypes.CDLL) -> None:
    c = ctypes
    vp, i, u, sz = c.c_void_p, c.c_int, c.c_uint, c.c_size_t
    L.garnet_b200_last_error.restype = c.c_char_p
    L.garnet_b200_abi_version.restype = i
    L.garnet_b200_manifest_json.restype = c.c_char_p
    L.garnet_b200_resolve.restype = vp
    L.garnet_b200_resolve.argtypes = [c.c_char_p]
    L.garnet_b200_binary_path.restype = c.c_char_p
    L.garnet_b200_is_int4_linear_weight.argtypes = [c.c_char_p, c.c_char_p, i, c.POINTER(c.c_int64), i]
    L.garnet_b200_selftest_bounded_wait.argtypes = [i, vp]
    L.garnet_b200_int4_quantize.argtypes = [vp, i, c.c_int64, c.c_int64, i, i, vp, vp, vp]
    L.garnet_b200_w4a16_packed_bytes.argtypes = [i, i, i, c.POINTER(sz)]
    L.garnet_b200_w4a16_pack_host.argtypes = [vp, vp, i, i, i, i, vp]
    L.garnet_b200_w4a16_create.argtypes = [vp, vp, i, i, i, i, i, i, vp, c.POINTER(vp)]
    L.garnet_b200_w4a16_create_k_shard.argtypes = [vp, vp, i, i, i, i, i, i, vp, c.POINTER(vp)]
    L.garnet_b200_w4a16_create_prepacked.argtypes = [vp, i, i, i, i, c.POINTER(vp)]
    L.garnet_b200_w4a16_shape.argtypes = [vp, c.POINTER(i), c.POINTER(i)]
    L.garnet_b200_w4a16_workspace.argtypes = [vp, i, c.POINTER(sz)]
    L.garnet_b200_w4a16_run.argtypes = [vp, vp, vp, i, vp, sz, u, vp]
    L.garnet_b200_w4a16_run_group.argtypes = [vp, i, vp, vp, i, u, vp]
    L.garnet_b200_w4a16_reserve_host.argtypes = [vp, i]
    L.garnet_b200_w4a16_run_host.argtypes = [vp, vp, vp, i, vp]
    L.garnet_b200_w4a16_run_host_async.argtypes = [vp, vp, vp, i, vp]
    L.garnet_b200_w4a16_batch_create.argtypes = [vp, vp, vp, vp, i, vp]
    L.garnet_b200_w4a16_batch_run.argtypes = [vp, vp]
    L.garnet_b200_w4a16_batch_destroy.argtypes = [vp]
    L.garnet_b200_w4a16_batch_destroy.restype = None
    L.garnet_b200_w4a16_list_create.argtypes = [vp, vp, vp, vp, i, i, vp]
    L.garnet_b200_w4a16_list_run.argtypes = [vp, u, vp]
    L.garnet_b200_w4a16_list_fault.argtypes = [vp]
    L.garnet_b200_w4a16_list_destroy.argtypes = [vp]
    L.garnet_b200_w4a16_list_destroy.restype = None
    L.garnet_b200_w4a16_dequant.argtypes = [vp, vp, vp]
    L.garnet_b200_w4a16_fault.argtypes = [vp]
    L.garnet_b200_w4a16_destroy.argtypes = [vp]
    L.garnet_b200_w4a16_destroy.restype = None
    L.garnet_b200_w4a16_list_create_ex.argtypes = [vp, i, i, c.POINTER(vp)]
    L.garnet_b200_attention_decode_workspace.argtypes = [vp, i, c.POINTER(sz)]
    L.garnet_b200_attention_decode.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, sz, i, c.c_uint, vp]
    L.garnet_b200_embedding_gather.argtypes = [vp, vp, vp, i, i, i, c.c_uint, vp]
    L.garnet_b200_argmax_bf16.argtypes = [vp, vp, i, i, c.c_uint, vp]
    L.garnet_b200_safetensors_open.argtypes = [c.c_char_p, c.POINTER(vp)]
    L.garnet_b200_safetensors_count.argtypes = [vp]
    L.garnet_b200_safetensors_entry.argtypes = [vp, i, c.c_char_p, c.POINTER(c.c_char_p), c.POINTER(c.c_char_p), c.POINTER(i),
                                                c.POINTER(c.c_longlong), c.POINTER(vp), c.POINTER(sz)]
    L.garnet_b200_safetensors_close.argtypes = [vp]
    L.garnet_b200_safetensors_close.restype = None
    L.garnet_b200_safetensors_write.argtypes = [c.c_char_p, vp, vp, vp, vp, vp, vp, i]
    L.garnet_b200_int4_quantize_host.argtypes = [vp, i, i, i, i, i, vp, vp, c.POINTER(c.c_double)]
    L.garnet_b200_packed_tensor_name.argtypes = [c.c_char_p, i, i, i, i, c.c_char_p, sz]
    L.garnet_b200_packed_tensor_name_parse.argtypes = [c.c_char_p, c.POINTER(i), c.POINTER(i), c.POINTER(i), c.POINTER(i),
                                                       c.POINTER(c.c_char_p)]
    L.garnet_b200_checkpoint_build_cache.argtypes = [vp, c.c_char_p, i, i, i, i, i]
    L.garnet_b200_gpt_oss_rms_norm.argtypes = [vp, vp, vp, i, i, c.c_float, vp]
    L.garnet_b200_gpt_oss_rope.argtypes = [vp, vp, vp, vp, i, vp]
    L.garnet_b200_gpt_oss_attention_workspace.argtypes = [vp, i, i, c.POINTER(sz)]
    L.garnet_b200_gpt_oss_attention.argtypes = [vp, vp, vp, vp, sz, i, i, i, i, vp]
    L.garnet_b200_gpt_oss_vocab_top1.argtypes = [vp, vp, i, i, i, vp]
    L.garnet_b200_gpt_oss_decode_gemv.argtypes = [vp, vp, vp, i, i, i, i, i, i, i, i, vp]
    L.garnet_b200_moe_workspace.argtypes = [vp, i, c.POINTER(sz)]
    L.garnet_b200_moe_create.argtypes = [vp, vp, vp, c.POINTER(vp)]
    L.garnet_b200_moe_run.argtypes = [vp, vp, vp, vp, sz, i, vp]
    L.garnet_b200_moe_run_static.argtypes = [vp, vp, vp, i, vp]
    L.garnet_b200_moe_rows_workspace.argtypes = [vp, i, c.POINTER(sz)]
    L.garnet_b200_moe_run_rows.argtypes = [vp, vp, vp, i, vp, vp, sz, vp]
    L.garnet_b200_moe_run_rows_stage.argtypes = [vp, i, vp, vp, i, vp, vp, vp, sz, vp]
    L.garnet_b200_moe_combine.argtypes = [vp, vp, vp, vp, i, vp]
    L.garnet_b200_moe_route.argtypes = [vp, vp, vp, vp, vp, i, vp]
    L.garnet_b200_moe_route_workspace.argtypes = [vp, i, c.POINTER(sz)]
    L.garnet_b200_moe_route_ws.argtypes = [vp, vp, vp, vp, vp, i, vp, sz, vp]
    L.garnet_b200_mxfp4_decode.argtypes = [vp, vp, vp, i, vp]
    L.garnet_b200_moe_dequant.argtypes = [vp, i, i, vp, vp]
    L.garnet_b200_mx_split_rows.argtypes = [vp, i, i, vp, vp, vp, vp]
    L.garnet_b200_moe_packed_bytes.argtypes = [vp, i, i, i, c.POINTER(sz)]
    L.garnet_b200_moe_pack_host.argtypes = [vp, i, i, vp, vp, i, vp]
    L.garnet_b200_moe_packed_view.argtypes = [vp, i, i, c.POINTER(vp), c.POINTER(sz)]
    L.garnet_b200_moe_create_prepacked.argtypes = [vp, vp, vp, vp, c.POINTER(vp)]
    L.garnet_b200_moe_gather_intermediate_shard.argtypes = [vp, sz, c.POINTER(c.c_longlong), i, sz, i, i, i, vp]
    L.garnet_b200_comm_create.argtypes = [i, i, sz, c.POINTER(vp)]
    L.garnet_b200_comm_export.argtypes = [vp, vp, sz]
    L.garnet_b200_comm_connect.argtypes = [vp, vp]
    L.garnet_b200_comm_fault.argtypes = [vp]
    L.garnet_b200_comm_destroy.argtypes = [vp]
    L.garnet_b200_comm_destroy.restype = None
    L.garnet_b200_comm_channel_create.argtypes = [vp, sz, c.POINTER(vp)]
    L.garnet_b200_comm_channel_destroy.argtypes = [vp]
    L.garnet_b200_comm_channel_destroy.restype = None
    L.garnet_b200_comm_all_gather.argtypes = [vp, vp, sz, vp, vp]
    L.garnet_b200_comm_all_reduce.argtypes = [vp, vp, vp, sz, i, vp]
    L.garnet_b200_comm_all_reduce_bf16.argtypes = [vp, vp, vp, sz, vp]
    L.garnet_b200_comm_selftest_wait.argtypes = [vp, i, vp]
    L.garnet_b200_moe_ep_arena_bytes.argtypes = [vp, i, i, c.POINTER(sz)]
    L.garnet_b200_moe_ep_create.argtypes = [vp, vp, i, c.POINTER(vp)]
    L.garnet_b200_moe_ep_run.argtypes = [vp, vp, vp, i, vp]
    L.garnet_b200_moe_ep_rows_received.argtypes = [vp]
    L.garnet_b200_moe_ep_destroy.argtypes = [vp]
    L.garnet_b200_moe_ep_destroy.restype = None
    L.garnet_b200_moe_ep_plan_host.argtypes = [vp, i, i, i, vp, vp]
    L.garnet_b200_moe_fault.argtypes = [vp]
    L.garnet_b200_moe_destroy.argtypes = [vp]
    L.garnet_b200_moe_destroy.restype = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path = _build.build()      # does nothing when the binary is newer than its sources
        L = ctypes.CDLL(path)
        _declare(L)
        if L.garnet_b200_abi_version() != 1:
            raise RuntimeError("libgarnet_b200.so reports an unexpected ABI version")
        _lib = L
    return _lib


def check(code: int) -> None:
    if code != OK:
        raise GarnetB200Error(code, lib().garnet_b200_last_error().decode())
