"""ctypes callers of the gpt-oss layer operators around the MoE (garnet_b200_gpt_oss_*): RMS norm,
YaRN RoPE, paged attention with sinks and a sliding window, decode GEMV, vocabulary top-1.  They
mirror the reference's RunGptOssRmsNorm / Rope / Attention / DecodeGemv / VocabTop1
(plugins/gpt_oss/include/gpt_oss_kernels.h:24-40)."""
from __future__ import annotations

import ctypes

import torch

from ._lib import check, lib


class GptOssOptions(ctypes.Structure):
    _fields_ = [("abi", ctypes.c_int), ("struct_size", ctypes.c_int), ("q_heads", ctypes.c_int), ("kv_heads", ctypes.c_int),
                ("head_dim", ctypes.c_int), ("layer", ctypes.c_int), ("page_size", ctypes.c_int), ("window", ctypes.c_int),
                ("prefill", ctypes.c_int), ("theta", ctypes.c_float), ("factor", ctypes.c_float),
                ("initial_context", ctypes.c_float), ("beta_fast", ctypes.c_float), ("beta_slow", ctypes.c_float)]


def options(q_heads=64, kv_heads=8, head_dim=64, layer=0, page_size=16, window=0, prefill=0, theta=150000.0, factor=32.0,
            initial_context=4096.0, beta_fast=32.0, beta_slow=1.0) -> GptOssOptions:
    return GptOssOptions(abi=1, struct_size=ctypes.sizeof(GptOssOptions), q_heads=q_heads, kv_heads=kv_heads, head_dim=head_dim,
                         layer=layer, page_size=page_size, window=window, prefill=prefill, theta=theta, factor=factor,
                         initial_context=initial_context, beta_fast=beta_fast, beta_slow=beta_slow)


def _s() -> int:
    return torch.cuda.current_stream().cuda_stream


def rms_norm(x, weight, eps=1e-5):
    y = torch.empty_like(x)
    check(lib().garnet_b200_gpt_oss_rms_norm(x.data_ptr(), weight.data_ptr(), y.data_ptr(), x.shape[0], x.shape[1], eps, _s()))
    return y


def rope(opt, x, positions):
    y = torch.empty_like(x)
    check(lib().garnet_b200_gpt_oss_rope(ctypes.byref(opt), x.data_ptr(), positions.data_ptr(), y.data_ptr(), x.shape[0], _s()))
    return y


def attention(opt, qkv, keys, values, table, lengths, starts, active, sinks, batch, tokens, physical_pages, workspace=None):
    logical_pages = table.shape[1]
    y = torch.empty(batch * tokens, opt.q_heads * opt.head_dim, dtype=torch.float32, device=qkv.device)
    need = ctypes.c_size_t(0)
    check(lib().garnet_b200_gpt_oss_attention_workspace(ctypes.byref(opt), batch, logical_pages, ctypes.byref(need)))
    ws = workspace if workspace is not None else torch.zeros(need.value, dtype=torch.uint8, device=qkv.device)
    ops = (ctypes.c_void_p * 8)(*[t.data_ptr() for t in (qkv, keys, values, table, lengths, starts, active, sinks)])
    check(lib().garnet_b200_gpt_oss_attention(ctypes.byref(opt), ops, y.data_ptr(), ws.data_ptr(), ws.numel(), batch, tokens,
                                              logical_pages, physical_pages, _s()))
    return y


def vocab_top1(logits, rank=0):
    pairs = torch.empty(logits.shape[0], 2, dtype=torch.float32, device=logits.device)
    check(lib().garnet_b200_gpt_oss_vocab_top1(logits.data_ptr(), pairs.data_ptr(), logits.shape[0], logits.shape[1], rank, _s()))
    return pairs


def decode_gemv(x, weight, rows, columns, column_offset=0, q_heads=0, kv_heads=0, head_dim=0, rank=0):
    y = torch.empty(rows, dtype=torch.bfloat16, device=x.device)
    check(lib().garnet_b200_gpt_oss_decode_gemv(x.data_ptr(), weight.data_ptr(), y.data_ptr(), rows, columns, weight.shape[1],
                                                column_offset, q_heads, kv_heads, head_dim, rank, _s()))
    return y
