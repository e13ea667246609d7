"""CPU-side checks of the C ABI: the library loads, exports every symbol the
header declares, validates arguments before touching pointers, and its host
repacker writes the documented layout (checked by an independent
inverse-coordinate restatement, in the manner of the reference's
test2026/gpt_oss/marlin_weight_pack.cpp:54-78)."""
import ctypes
import json
import os
import re

import numpy as np
import pytest
import torch

import garnet_b200
from garnet_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "garnet_b200.h")).read()
    return sorted(set(re.findall(r"\b(garnet_b200_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported():
    L = garnet_b200.lib()
    names = declared_symbols()
    assert len(names) >= 15
    for name in names:
        assert hasattr(L, name), name
        assert L.garnet_b200_resolve(name.encode()), name
    assert L.garnet_b200_resolve(b"printf") is None


def test_manifest_keys_match_reference_contract():
    L = garnet_b200.lib()
    m = json.loads(L.garnet_b200_manifest_json().decode())
    for key in ("id", "module", "abi", "version", "backend", "operators"):
        assert key in m
    assert m["abi"] == L.garnet_b200_abi_version() == 1
    assert "gpt_oss_moe_mxfp4" in m["operators"] and "lm_head" in m["operators"]
    assert os.path.exists(L.garnet_b200_binary_path().decode())
    reg = json.load(open(os.path.join(ROOT, "garnet_b200", "registry.json")))
    assert reg["plugins"][m["id"]]["module"] == m["module"]


def test_invalid_arguments_are_rejected_before_pointer_access():
    L = garnet_b200.lib()
    out = ctypes.c_void_p(None)
    sz = ctypes.c_size_t(0)
    assert L.garnet_b200_w4a16_create(None, None, 1, 128, 128, 128, 0, 1, None, ctypes.byref(out)) == _lib.INVALID_VALUE
    assert b"null" in L.garnet_b200_last_error()
    assert L.garnet_b200_w4a16_packed_bytes(128, 100, 128, ctypes.byref(sz)) == _lib.INVALID_VALUE
    assert L.garnet_b200_w4a16_packed_bytes(128, 128, 64, ctypes.byref(sz)) == _lib.NOT_SUPPORTED
    assert L.garnet_b200_w4a16_run(None, None, None, 1, None, 0, 0, None) == _lib.INVALID_VALUE
    assert L.garnet_b200_w4a16_workspace(None, 1, ctypes.byref(sz)) == _lib.INVALID_VALUE
    assert L.garnet_b200_int4_quantize(None, 2, 1, 128, 128, 1, None, None, None) == _lib.INVALID_VALUE


def row_of_g(g):
    return (g >> 1) + 4 * (g & 1)


def expected_position(n, k, chunks):
    """Independent statement of the packed int4 layout: byte offset of the word
    and nibble index that hold element (n, k).  Strips of 16 rows, chunks of 128
    columns (1024 code bytes + 32 scale bytes), 512-byte tiles of 64 columns,
    16-byte units 4*g + t, words h + 2*j."""
    strip, r16 = divmod(n, 16)
    chunk, kl = divmod(k, 128)
    tile, kk = divmod(kl, 64)
    h, r8 = divmod(r16, 8)
    g = next(g for g in range(8) if row_of_g(g) == r8)
    octet, e = divmod(kk, 8)
    j, t = divmod(octet, 4)
    byte = (strip * chunks + chunk) * 1056 + tile * 512 + (4 * g + t) * 16 + (h + 2 * j) * 4
    return byte, (e >> 1) + 4 * (e & 1)


@pytest.mark.parametrize("n,k,group", [(128, 128, 128), (200, 256, 128), (384, 512, 256), (16, 384, 128)])
def test_host_packer_layout(n, k, group):
    rng = np.random.default_rng(n + k)
    codes = rng.integers(-8, 8, size=(n, k)).astype(np.int8)
    flat = (codes.reshape(-1) & 15).astype(np.uint8)
    nibbles = (flat[0::2] | (flat[1::2] << 4)).astype(np.uint8)
    scales = rng.integers(0, 65536, size=(n, k // group)).astype(np.uint16)
    packed = garnet_b200.pack_host(torch.from_numpy(nibbles), torch.from_numpy(scales.view(np.int16)).view(torch.bfloat16),
                                   n, k, group).numpy()
    chunks = k // 128
    strips_padded = ((n + 15) // 16 + 7) // 8 * 8
    assert packed.size == strips_padded * chunks * 1056 == garnet_b200.packed_bytes(n, k, group)
    words = packed.view(np.uint32)
    for nn in range(0, n, 7):
        for kk in range(0, k, 5):
            byte, nib = expected_position(nn, kk, chunks)
            got = (int(words[byte // 4]) >> (4 * nib)) & 15
            assert got == (int(codes[nn, kk]) & 15), (nn, kk)
    # scales: [g][h] 16-bit words after the 1024 code bytes of each strip-chunk
    for nn in range(0, n, 3):
        for c in range(chunks):
            strip, r16 = divmod(nn, 16)
            h, r8 = divmod(r16, 8)
            g = next(g for g in range(8) if row_of_g(g) == r8)
            off = (strip * chunks + c) * 1056 + 1024 + g * 4 + h * 2
            assert packed[off:off + 2].view(np.uint16)[0] == scales[nn, (c * 128) // group]
    # padding rows hold zero codes
    if n % 128:
        byte, _ = expected_position(strips_padded * 16 - 1, 0, chunks)
        assert words[byte // 4] == 0


def test_int4_weight_predicate_follows_the_reference_rule():
    """Garnet::IsQwenLinearWeightForINT4 (src/model/weight_quantization.cpp:146-186): rank 2,
    K a multiple of the block, a float dtype and one of the Qwen projection endings."""
    L = garnet_b200.lib()

    def ok(name, dtype="BF16", shape=(2048, 2048), block=128):
        arr = (ctypes.c_int64 * len(shape))(*shape)
        return L.garnet_b200_is_int4_linear_weight(name.encode(), dtype.encode(), len(shape), arr, block)

    for ending in ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj", "mlp.gate_proj",
                   "mlp.up_proj", "mlp.down_proj", "linear_attn.in_proj_qkv", "linear_attn.in_proj_z",
                   "linear_attn.in_proj_b", "linear_attn.in_proj_a", "linear_attn.out_proj"):
        assert ok(f"model.layers.3.{ending}.weight") == 1
    assert ok("lm_head.weight", shape=(151936, 2048)) == 1
    assert ok("model.lm_head.weight") == 1                       # ending match, as in the reference
    assert ok("model.layers.0.self_attn.q_proj.weight", dtype="F16") == 1
    assert ok("model.layers.0.self_attn.q_proj.weight", dtype="F32") == 1
    assert ok("model.layers.0.self_attn.q_proj.weight", dtype="I8") == 0
    assert ok("model.layers.0.self_attn.q_proj.bias") == 0
    assert ok("model.embed_tokens.weight") == 0
    assert ok("model.layers.0.input_layernorm.weight", shape=(2048,)) == 0
    assert ok("model.layers.0.self_attn.q_norm.weight", shape=(128,)) == 0
    assert ok("model.layers.0.mlp.down_proj.weight", shape=(2048, 6100)) == 0    # K not a multiple of the block
    assert ok("model.layers.0.mlp.down_proj.weight", shape=(2048, 6144), block=0) == 0
    assert ok("model.layers.0.mlp.down_proj.weight", shape=(0, 6144)) == 0
    assert ok("model.layers.0.mlp.experts.0.down_proj.weight") == 0              # not the dense MLP ending
