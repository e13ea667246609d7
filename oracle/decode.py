"""CPU oracle of one Qwen3-style decode step.  TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

A numpy restatement, in float64 with a bf16 rounding wherever a bf16 network stores a tensor,
of the operator sequence the reference lowers for a dense Qwen3 decoder layer:
  * RMS norm: x / sqrt(mean(x^2) + eps) * w (Qwen3 norms; the fused-norm inputs of the packed
    operators, src/backends/tensorrt/trt_builder.cpp:7565-7726);
  * packed q/k/v, per-head RMS norm of q and k, rotate-half RoPE with cos/sin tables
    (:7565-7726, :1815-1870: out = x cos + rotate_half(x) sin, rotate_half(x) = [-x2, x1]);
  * paged KV cache, row ((page * page_size + offset) * kv_heads + kv_head) * head_dim, and the
    decode attention softmax(q K^T / sqrt(head_dim)) V over the sequence's context
    (src/cuda/text_kv_attention_kernel.cu:640-840);
  * packed gate/up, SiLU(gate) * up (:7727-7800), down projection, the two residual additions;
  * greedy token: the largest logit, the lowest index among equals.
The int4 linears are the exact target of the W4A16 operator: y = bf16(sum_k x_k q_k s) with the
residual, where there is one, added before the single rounding (the CUDA path fuses it).

Parity unpinned: the reference evaluates these layers inside TensorRT, which is not available,
and holds no golden vectors for a Qwen3 decode step; the tests compare the CUDA path with this
restatement within a stated tolerance."""
from __future__ import annotations

import numpy as np

from . import bf16_round, int4_unpack


def _bf(a):
    return bf16_round(np.asarray(a, np.float32)).astype(np.float64)


def dequant(nibbles: np.ndarray, scales_f32: np.ndarray, n: int, k: int, group: int = 128) -> np.ndarray:
    q = int4_unpack(np.ascontiguousarray(nibbles, np.uint8), n, k).astype(np.float64)
    return q * np.repeat(scales_f32.astype(np.float64).reshape(n, k // group), group, axis=1)


def rms_norm(x, w, eps):
    x = np.asarray(x, np.float64)
    return _bf(x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps) * np.asarray(w, np.float64))


def rope(x, cos, sin):
    """x [..., 128]; cos, sin [64] of the position."""
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    return _bf(np.concatenate([x1 * cos - x2 * sin, x2 * cos + x1 * sin], axis=-1))


def silu_mul(gu, inter):
    g, u = gu[..., :inter], gu[..., inter:]
    return _bf(g / (1.0 + np.exp(-g)) * u)


class Decoder:
    """Weights as float64 matrices (dequantised once); caches and page tables as numpy arrays
    with the CUDA path's shapes: key_pages / value_pages [layers][pages, page_size, kv_heads, 128]."""

    def __init__(self, cfg, weights: dict, key_pages, value_pages, page_tables, cos, sin):
        self.cfg, self.w = cfg, weights
        self.key_pages, self.value_pages, self.page_tables = key_pages, value_pages, page_tables
        self.cos, self.sin = cos.astype(np.float64), sin.astype(np.float64)

    def attention(self, layer: int, qkv, positions):
        cfg = self.cfg
        qh, kvh, d = cfg.q_heads, cfg.kv_heads, cfg.head_dim
        lw = self.w["layers"][layer]
        out = np.zeros((qkv.shape[0], qh * d))
        for b in range(qkv.shape[0]):
            slot = int(positions[b])
            q = qkv[b, :qh * d].reshape(qh, d)
            k = qkv[b, qh * d:(qh + kvh) * d].reshape(kvh, d)
            v = qkv[b, (qh + kvh) * d:].reshape(kvh, d)
            cs, sn = self.cos[slot], self.sin[slot]
            qn = rope(rms_norm(q, lw["q_norm"], cfg.eps), cs, sn)
            kn = rope(rms_norm(k, lw["k_norm"], cfg.eps), cs, sn)
            table = self.page_tables[b]
            page, off = int(table[slot // cfg.page_size]), slot % cfg.page_size
            self.key_pages[layer][page, off] = kn
            self.value_pages[layer][page, off] = v
            rows = [(int(table[p // cfg.page_size]), p % cfg.page_size) for p in range(slot + 1)]
            K = np.stack([self.key_pages[layer][pg, of] for pg, of in rows])      # [ctx, kvh, d]
            V = np.stack([self.value_pages[layer][pg, of] for pg, of in rows])
            for h in range(qh):
                g = h // (qh // kvh)
                s = K[:, g] @ qn[h] / np.sqrt(float(d))
                p = np.exp(s - s.max())
                out[b, h * d:(h + 1) * d] = (p / p.sum()) @ V[:, g]
        return _bf(out)

    def step(self, tokens, positions):
        """Returns (greedy tokens, logits, per-layer residual streams) and appends to the caches."""
        cfg, w = self.cfg, self.w
        x = w["embedding"][np.asarray(tokens)].astype(np.float64)
        trace = []
        for i, lw in enumerate(w["layers"]):
            qkv = _bf(rms_norm(x, lw["in_norm"], cfg.eps) @ lw["qkv"].T)
            a = self.attention(i, qkv, positions)
            x1 = _bf(a @ lw["o"].T + x)
            gu = _bf(rms_norm(x1, lw["post_norm"], cfg.eps) @ lw["gate_up"].T)
            x = _bf(silu_mul(gu, cfg.intermediate) @ lw["down"].T + x1)
            trace.append(x.copy())
        logits = _bf(rms_norm(x, w["final_norm"], cfg.eps) @ w["lm_head"].T)
        return logits.argmax(axis=1).astype(np.int32), logits, trace
