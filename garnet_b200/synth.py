"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations (no checkpoint or dataset is involved).

int4 linear: codes uniform in [-8, 7]; one bf16 scale |N(0, 0.02)| / 7 per
(row, 128 columns); activations bf16 ~ N(0, 1).
MXFP4 MoE (gpt-oss-120b layer): e2m1 codes uniform over the 16 values; e8m0
scale exponent uniform in [-10, -4] (bytes 117..123); router weights
N(0, 1/sqrt(hidden)) so that logits are ~ N(0, 1); top-4 of 128 experts."""
from __future__ import annotations

import numpy as np

QWEN3_1P7B_PROJECTIONS = [
    # name, K (in), N (out)
    ("q_proj", 2048, 2048),
    ("k_proj", 2048, 1024),
    ("v_proj", 2048, 1024),
    ("o_proj", 2048, 2048),
    ("gate_proj", 2048, 6144),
    ("up_proj", 2048, 6144),
    ("down_proj", 6144, 2048),
]
QWEN3_1P7B_LM_HEAD = ("lm_head", 2048, 151936)
QWEN3_1P7B_LAYERS = 28


def bf16_round_np(x: np.ndarray) -> np.ndarray:
    v = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    return ((v + 0x7FFF + ((v >> 16) & 1)) & 0xFFFF0000).astype(np.uint32).view(np.float32).reshape(np.shape(x))


def bf16_bits_np(x: np.ndarray) -> np.ndarray:
    return (bf16_round_np(x).view(np.uint32) >> 16).astype(np.uint16)


def int4_linear(n: int, k: int, m: int, group: int = 128, seed: int = 0):
    """Returns dict(nibbles u8 [n*k/2], scales_bits u16 [n, k/group] (bf16 bits),
    scales_f32, x_f32 [m, k] bf16-valued, x_bits u16)."""
    rng = np.random.default_rng(seed)
    codes = rng.integers(-8, 8, size=(n, k), dtype=np.int8)
    flat = (codes.reshape(-1) & 15).astype(np.uint8)
    nibbles = (flat[0::2] | (flat[1::2] << 4)).astype(np.uint8)
    scales = bf16_round_np(np.abs(rng.normal(0.0, 0.02, size=(n, k // group))).astype(np.float32) / np.float32(7.0))
    x = bf16_round_np(rng.normal(0.0, 1.0, size=(m, k)).astype(np.float32))
    return dict(nibbles=nibbles, scales_bits=bf16_bits_np(scales), scales_f32=scales, x_f32=x,
                x_bits=bf16_bits_np(x), codes=codes)


def moe_layer(tokens: int, hidden: int = 2880, inter: int = 2880, experts: int = 128, topk: int = 4,
              seed: int = 0, zipf_s: float | None = None, bias_scale: float = 0.0):
    """gpt-oss style MoE layer tensors in the reference's original layout:
    gate_up blocks [E, 2I, H/32, 16] u8, scales [E, 2I, H/32] u8, bias [E, 2I];
    down blocks [E, H, I/32, 16], scales [E, H, I/32], bias [E, H]."""
    rng = np.random.default_rng(seed)
    x = bf16_round_np(rng.normal(0, 1, size=(tokens, hidden)).astype(np.float32))
    router_w = bf16_round_np(rng.normal(0, 1.0 / np.sqrt(hidden), size=(experts, hidden)).astype(np.float32))
    router_b = np.zeros(experts, np.float32)
    if zipf_s is not None:
        ranks = rng.permutation(experts) + 1
        pop = ranks.astype(np.float64) ** (-zipf_s)
        router_b = bf16_round_np(np.log(pop / pop.sum() * experts).astype(np.float32))
    gu_blocks = rng.integers(0, 256, size=(experts, 2 * inter, hidden // 32, 16), dtype=np.uint8)
    gu_scales = rng.integers(117, 124, size=(experts, 2 * inter, hidden // 32), dtype=np.uint8)
    dn_blocks = rng.integers(0, 256, size=(experts, hidden, inter // 32, 16), dtype=np.uint8)
    dn_scales = rng.integers(117, 124, size=(experts, hidden, inter // 32), dtype=np.uint8)
    gu_bias = bf16_round_np((rng.normal(0, 1, size=(experts, 2 * inter)) * bias_scale).astype(np.float32))
    dn_bias = bf16_round_np((rng.normal(0, 1, size=(experts, hidden)) * bias_scale).astype(np.float32))
    return dict(x=x, router_w=router_w, router_b=router_b, gu_blocks=gu_blocks, gu_scales=gu_scales,
                gu_bias=gu_bias, dn_blocks=dn_blocks, dn_scales=dn_scales, dn_bias=dn_bias,
                hidden=hidden, inter=inter, experts=experts, topk=topk)
