"""One decode step of a Qwen3-style dense decoder (the model of BASELINE's config 3) on the
CUDA path: every int4 linear of the step runs in garnet_b200_w4a16_list launches with the
layer's glue folded in, attention runs in garnet_b200_attention_decode, and the whole step
is one CUDA graph of 2 launches per layer.

Structure of a step (reference: the per-layer operator sequence that
src/backends/tensorrt/trt_builder.cpp lowers - packed q/k/v with head norms and RoPE
:7565-7726, the isLinear projections :7268-7423, packed gate/up with SiLU and multiply
:7727-7800 - and the paged KV decode attention of src/cuda/text_kv_attention_kernel.cu):

    x = embedding[token]
    list 0:     qkv_0 = W_qkv0 . norm_in0(x)
    per layer L:
      attention: a = attn(rope(headnorm(q)), cache + rope(headnorm(k)), v)      1 launch
      list L+1:  x1 = x + W_o a;  gu = W_gu . norm_post(x1);                    1 launch
                 x = x1 + W_d (silu(gate) * up);  qkv_{L+1} = W_qkv . norm_in(x)
                 (after the last layer: logits = W_lm . norm_final(x) instead)
    token = argmax(logits)

Weights arrive in the canonical int4 form (nibbles + bf16 group scales); q/k/v and gate/up
are concatenated along N before they are packed, as the reference's packed operators do."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import numpy as np
import torch

from ._lib import check, lib
from .linear import GlueList, W4A16Linear


@dataclass
class DecoderConfig:
    hidden: int = 2048
    q_heads: int = 16
    kv_heads: int = 8
    head_dim: int = 128
    intermediate: int = 6144
    vocab: int = 151936
    layers: int = 28
    eps: float = 1e-6
    rope_theta: float = 1e6
    page_size: int = 16
    group: int = 128

    @property
    def qkv_width(self) -> int:
        return (self.q_heads + 2 * self.kv_heads) * self.head_dim


class AttentionOptions(ctypes.Structure):
    _fields_ = [("abi", ctypes.c_int), ("struct_size", ctypes.c_int), ("q_heads", ctypes.c_int), ("kv_heads", ctypes.c_int),
                ("head_dim", ctypes.c_int), ("page_size", ctypes.c_int), ("max_logical_pages", ctypes.c_int),
                ("max_context", ctypes.c_int), ("rope_positions", ctypes.c_int), ("norm_eps", ctypes.c_float)]


def rope_tables(positions: int, head_dim: int, theta: float):
    """cos / sin [positions, head_dim / 2] in fp32: angle = position * theta^(-2 i / head_dim),
    evaluated in float64 and rounded once."""
    inv = theta ** (-np.arange(0, head_dim, 2, dtype=np.float64) / head_dim)
    ang = np.arange(positions, dtype=np.float64)[:, None] * inv[None, :]
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


def _stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


class PagedAttention:
    """garnet_b200_attention_decode with its workspace."""

    def __init__(self, cfg: DecoderConfig, batch: int, max_context: int, max_logical_pages: int, rope_positions: int):
        self.opt = AttentionOptions(abi=1, struct_size=ctypes.sizeof(AttentionOptions), q_heads=cfg.q_heads,
                                    kv_heads=cfg.kv_heads, head_dim=cfg.head_dim, page_size=cfg.page_size,
                                    max_logical_pages=max_logical_pages, max_context=max_context,
                                    rope_positions=rope_positions, norm_eps=cfg.eps)
        need = ctypes.c_size_t(0)
        check(lib().garnet_b200_attention_decode_workspace(ctypes.byref(self.opt), batch, ctypes.byref(need)))
        self.ws = torch.zeros(need.value, dtype=torch.uint8, device="cuda")
        self.batch = batch

    def run(self, qkv, q_norm_w, k_norm_w, cos, sin, key_pages, value_pages, page_tables, positions, out, pdl: bool = False):
        check(lib().garnet_b200_attention_decode(ctypes.byref(self.opt), qkv.data_ptr(), q_norm_w.data_ptr(), k_norm_w.data_ptr(),
                                                 cos.data_ptr(), sin.data_ptr(), key_pages.data_ptr(), value_pages.data_ptr(),
                                                 page_tables.data_ptr(), positions.data_ptr(), out.data_ptr(), self.ws.data_ptr(),
                                                 self.ws.numel(), self.batch, 1 if pdl else 0, _stream_ptr()))
        return out


def embedding_gather(table, ids, out, pdl: bool = False):
    check(lib().garnet_b200_embedding_gather(table.data_ptr(), ids.data_ptr(), out.data_ptr(), ids.numel(), table.shape[1],
                                             table.shape[0], 1 if pdl else 0, _stream_ptr()))
    return out


def argmax_bf16(logits, out, pdl: bool = False):
    check(lib().garnet_b200_argmax_bf16(logits.data_ptr(), out.data_ptr(), logits.shape[0], logits.shape[1], 1 if pdl else 0,
                                        _stream_ptr()))
    return out


class DecodeStep:
    """The decode step of a model given as a dict of device tensors:
      embedding [V, H] bf16, final_norm [H] bf16, lm_head = (nibbles, scales),
      layers[L] = dict(in_norm, post_norm [H], q_norm, k_norm [128] bf16,
                       qkv, o, gate_up, down = (nibbles uint8, scales bf16 [N, K/128])).
    The KV cache (key_pages / value_pages [pages, page_size, kv_heads, 128] bf16 per layer) and the
    page tables [batch, max_logical_pages] int32 belong to the caller, as in the reference."""

    def __init__(self, cfg: DecoderConfig, weights: dict, batch: int, max_context: int, key_pages, value_pages, page_tables):
        self.cfg, self.batch = cfg, batch
        H, I, V = cfg.hidden, cfg.intermediate, cfg.vocab
        qw = cfg.q_heads * cfg.head_dim
        dev = "cuda"
        bf = dict(dtype=torch.bfloat16, device=dev)
        self.w = weights
        self.key_pages, self.value_pages, self.page_tables = key_pages, value_pages, page_tables
        mk = lambda pair, n, k: W4A16Linear().prepare(pair[0], pair[1], n, k, cfg.group)   # noqa: E731
        self.lin = [dict(qkv=mk(l["qkv"], cfg.qkv_width, H), o=mk(l["o"], H, qw), gate_up=mk(l["gate_up"], 2 * I, H),
                         down=mk(l["down"], H, I)) for l in weights["layers"]]
        self.lm_head = mk(weights["lm_head"], V, H)
        self.token_in = torch.zeros(batch, dtype=torch.int32, device=dev)
        self.positions = torch.zeros(batch, dtype=torch.int32, device=dev)
        self.x = [torch.zeros(batch, H, **bf) for _ in range(2)]      # residual stream after a layer, alternating
        self.x_mid = torch.zeros(batch, H, **bf)                      # residual stream after attention
        self.qkv = torch.zeros(batch, cfg.qkv_width, **bf)
        self.attn_out = torch.zeros(batch, qw, **bf)
        self.gu = torch.zeros(batch, 2 * I, **bf)
        self.logits = torch.zeros(batch, V, **bf)
        self.token_out = torch.zeros(batch, dtype=torch.int32, device=dev)
        rope_positions = page_tables.shape[1] * cfg.page_size
        cos, sin = rope_tables(rope_positions, cfg.head_dim, cfg.rope_theta)
        self.cos, self.sin = torch.from_numpy(cos).to(dev), torch.from_numpy(sin).to(dev)
        self.attn = PagedAttention(cfg, batch, max_context, page_tables.shape[1], rope_positions)
        L = weights["layers"]
        self.lists = [GlueList([dict(linear=self.lin[0]["qkv"], x=self.x[0], y=self.qkv, norm_weight=L[0]["in_norm"],
                                     norm_eps=cfg.eps)], m=batch)]
        for i in range(cfg.layers):
            x_in, x_out = self.x[i & 1], self.x[(i + 1) & 1]
            last = i == cfg.layers - 1
            tail = (dict(linear=self.lm_head, x=x_out, y=self.logits, dep=2, norm_weight=weights["final_norm"], norm_eps=cfg.eps)
                    if last else
                    dict(linear=self.lin[i + 1]["qkv"], x=x_out, y=self.qkv, dep=2, norm_weight=L[i + 1]["in_norm"],
                         norm_eps=cfg.eps))
            self.lists.append(GlueList([
                dict(linear=self.lin[i]["o"], x=self.attn_out, y=self.x_mid, residual=x_in),
                dict(linear=self.lin[i]["gate_up"], x=self.x_mid, y=self.gu, dep=0, norm_weight=L[i]["post_norm"],
                     norm_eps=cfg.eps),
                dict(linear=self.lin[i]["down"], x=self.gu, y=x_out, dep=1, activation=1, residual_dep=0),
                tail], m=batch))
        self.launches = 2 + 2 * cfg.layers + 1
        self._graph = None

    def enqueue(self) -> None:
        L = self.w["layers"]
        embedding_gather(self.w["embedding"], self.token_in, self.x[0])
        self.lists[0].run(pdl=True)
        for i in range(self.cfg.layers):
            self.attn.run(self.qkv, L[i]["q_norm"], L[i]["k_norm"], self.cos, self.sin, self.key_pages[i], self.value_pages[i],
                          self.page_tables, self.positions, self.attn_out, pdl=True)
            self.lists[i + 1].run(pdl=True)
        argmax_bf16(self.logits, self.token_out, pdl=True)

    def capture(self) -> None:
        """Records the step as one CUDA graph (after one eager run to settle allocations)."""
        self.enqueue()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.enqueue()
        self._graph = g

    def run(self) -> None:
        """One step on the tokens in `token_in` at the slots in `positions` (device tensors the
        caller fills); afterwards `token_out` holds the greedy tokens and `logits` the logits."""
        if self._graph is not None:
            self._graph.replay()
        else:
            self.enqueue()

    def fault(self) -> int:
        return max(l.fault() for l in self.lists)


def synthetic_decoder(cfg: DecoderConfig, seed: int = 0, device: str = "cuda") -> dict:
    """Random weights of the architecture in the canonical int4 form: codes uniform in -8..7,
    scales bf16(|N(0, 0.02)| / 7) per (row, 128 columns), norm weights near 1, embedding N(0, 1)."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)

    def int4(n, k):
        nib = torch.randint(0, 256, (n * k // 2,), dtype=torch.uint8, device=device, generator=gen)
        sc = (torch.randn(n, k // cfg.group, device=device, generator=gen).abs() * (0.02 / 7.0)).to(torch.bfloat16)
        return nib, sc

    def norm(n):
        return (1.0 + 0.1 * torch.randn(n, device=device, generator=gen)).to(torch.bfloat16)

    H, I, qw = cfg.hidden, cfg.intermediate, cfg.q_heads * cfg.head_dim
    layers = [dict(in_norm=norm(H), post_norm=norm(H), q_norm=norm(cfg.head_dim), k_norm=norm(cfg.head_dim),
                   qkv=int4(cfg.qkv_width, H), o=int4(H, qw), gate_up=int4(2 * I, H), down=int4(H, I)) for _ in range(cfg.layers)]
    return dict(embedding=torch.randn(cfg.vocab, H, device=device, generator=gen).to(torch.bfloat16), final_norm=norm(H),
                lm_head=int4(cfg.vocab, H), layers=layers)
