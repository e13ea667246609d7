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


# ------------------------------------------------------------- MoE packed constants

def _mx_case(experts, rows, k, seed):
    rng = np.random.default_rng(seed)
    blocks = rng.integers(0, 256, size=(experts, rows, k // 32, 16), dtype=np.uint8)
    scales = rng.integers(100, 140, size=(experts, rows, k // 32), dtype=np.uint8)
    return blocks, scales


def _code(blocks, e, row, col):
    byte = blocks[e, row, col // 32, (col % 32) // 2]
    return (int(byte) >> (4 * (col & 1))) & 15


@pytest.mark.parametrize("hidden,inter", [(64, 32), (96, 64), (160, 288)])
def test_moe_host_packer_streaming_layout(hidden, inter):
    """Inverse-coordinate restatement of the streaming layout (strips of 16 rows, 544-byte
    chunks of 64 columns, MMA-lane order inside a 512-byte tile, gate_i / up_i eight
    strip rows apart), in the manner of marlin_weight_pack.cpp:54-78."""
    from garnet_b200 import moe as moe_mod
    experts = 3
    moe = garnet_b200.GptOssMoe(hidden, inter, experts, 2)
    for which, (rows, k) in enumerate(((2 * inter, hidden), (hidden, inter))):
        blocks, scales = _mx_case(experts, rows, k, 10 * hidden + inter + which)
        blob = moe.pack_host(which, moe_mod.LAYOUT_STREAM, blocks, scales)
        chunks = (k + 63) // 64
        strips_padded = ((rows + 15) // 16 + 7) // 8 * 8
        matrix = strips_padded * chunks * 544
        assert blob.size == experts * matrix == moe.packed_bytes(which, moe_mod.LAYOUT_STREAM, experts)
        for e in range(experts):
            for prow in range(0, strips_padded * 16, 3):      # packed row
                strip, r16 = divmod(prow, 16)
                # which source row sits at this packed row
                src = 2 * (strip * 8 + (r16 & 7)) + (r16 >> 3) if which == 0 else prow
                h, r8 = divmod(r16, 8)
                g = next(g for g in range(8) if row_of_g(g) == r8)
                for col in range(0, chunks * 64, 5):
                    chunk, kl = divmod(col, 64)
                    octet, el = divmod(kl, 8)
                    t, j = octet & 3, octet >> 2
                    byte = e * matrix + (strip * chunks + chunk) * 544 + (4 * g + t) * 16 + (h + 2 * j) * 4 + el // 2
                    got = (int(blob[byte]) >> (4 * (el & 1))) & 15
                    want = _code(blocks, e, src, col) if (src < rows and prow < rows and col < k) else 0
                    assert got == want, (which, e, prow, col)
                for grp in range(chunks * 2):
                    off = e * matrix + (strip * chunks + grp // 2) * 544 + 512 + g * 4 + h + 2 * (grp & 1)
                    want = scales[e, src, grp] if (prow < rows and grp * 32 < k) else 127
                    assert blob[off] == want, (which, e, prow, grp)


@pytest.mark.parametrize("hidden,inter", [(64, 32), (160, 288)])
def test_moe_host_packer_block_layout(hidden, inter):
    """The block-scaled layout by reshapes: blocks [tile][slab][240 rows][64 bytes] in the
    checkpoint's row order, zero padded; then scale atoms [tile][slab][2][512] with byte
    (r % 32) * 16 + (r // 32) * 4 + group for row r of a 128-row atom, padded with 127."""
    from garnet_b200 import moe as moe_mod
    experts = 2
    moe = garnet_b200.GptOssMoe(hidden, inter, experts, 2)
    for which, (rows, k) in enumerate(((2 * inter, hidden), (hidden, inter))):
        blocks, scales = _mx_case(experts, rows, k, hidden + inter + which)
        blob = moe.pack_host(which, moe_mod.LAYOUT_BLOCK, blocks, scales)
        nt, ks = (rows + 239) // 240, (k + 127) // 128
        code_bytes = experts * nt * ks * 15360
        assert blob.size == code_bytes + experts * nt * ks * 1024 == moe.packed_bytes(which, moe_mod.LAYOUT_BLOCK, experts)
        padded = np.zeros((experts, nt * 240, ks * 64), np.uint8)
        padded[:, :rows, :k // 2] = blocks.reshape(experts, rows, k // 2)
        want = padded.reshape(experts, nt, 240, ks, 64).transpose(0, 1, 3, 2, 4)
        assert np.array_equal(blob[:code_bytes].reshape(want.shape), want)
        sc = np.full((experts, nt, 256, ks * 4), 127, np.uint8)     # 2 atoms of 128 rows per tile; rows 240..255 unused
        for tile in range(nt):
            r = min(240, rows - tile * 240)
            sc[:, tile, :r, :k // 32] = scales[:, tile * 240:tile * 240 + r]
        # [e][tile][atom][r // 32][r % 32][slab][group] -> [e][tile][slab][atom][r % 32][r // 32][group]
        want = sc.reshape(experts, nt, 2, 4, 32, ks, 4).transpose(0, 1, 5, 2, 4, 3, 6)
        assert np.array_equal(blob[code_bytes:].reshape(want.shape), want)


def test_intermediate_shard_gather_follows_the_reference_rule():
    """GatherGptOssIntermediateShard (gpt_oss_weight_shard.h:25-60; its test
    test2026/gpt_oss/expert_weight_shard.cpp): mode 1 slices axis 1, mode 2 axis 2, mode 3
    keeps the tensor on rank 0 and zeros it elsewhere; bad descriptors are refused."""
    from garnet_b200 import moe as moe_mod
    rng = np.random.default_rng(3)
    for dtype in (np.uint8, np.uint16, np.float32):
        for shape in ((3, 8), (3, 8, 6), (2, 8, 6, 16)):
            a = (rng.integers(0, 200, size=shape)).astype(dtype)
            for world in (2, 4):
                for rank in range(world):
                    part = shape[1] // world
                    assert np.array_equal(moe_mod.gather_intermediate_shard(a, rank, world, 1), a[:, rank * part:(rank + 1) * part])
                    if len(shape) >= 3 and shape[2] % world == 0:
                        p2 = shape[2] // world
                        assert np.array_equal(moe_mod.gather_intermediate_shard(a, rank, world, 2), a[:, :, rank * p2:(rank + 1) * p2])
                    if len(shape) == 2:
                        got = moe_mod.gather_intermediate_shard(a, rank, world, 3)
                        assert np.array_equal(got, a if rank == 0 else np.zeros_like(a))
    L = garnet_b200.lib()
    a = np.zeros((3, 7), np.uint8)
    out = np.zeros(64, np.uint8)
    shape = (ctypes.c_longlong * 2)(3, 7)
    call = L.garnet_b200_moe_gather_intermediate_shard
    assert call(a.ctypes.data, a.nbytes, shape, 2, 1, 0, 2, 1, out.ctypes.data) == 1      # 7 does not divide
    assert call(a.ctypes.data, a.nbytes + 1, shape, 2, 1, 0, 2, 3, out.ctypes.data) == 1  # byte count mismatch
    assert call(a.ctypes.data, a.nbytes, shape, 2, 1, 0, 2, 2, out.ctypes.data) == 1      # mode 2 needs 3 axes
    assert call(a.ctypes.data, a.nbytes, shape, 2, 1, 2, 2, 3, out.ctypes.data) == 1      # rank outside the world
    assert call(a.ctypes.data, a.nbytes, shape, 2, 3, 0, 2, 3, out.ctypes.data) == 1      # element size
    assert call(None, a.nbytes, shape, 2, 1, 0, 2, 3, out.ctypes.data) == 1


def test_moe_options_of_the_first_struct_version_are_accepted():
    """A caller compiled against the struct that ends after `limit` passes the smaller
    struct_size and gets the defaults of the later fields."""
    from garnet_b200.moe import MoeOptions
    first = MoeOptions.layouts.offset
    opt = MoeOptions(abi=1, struct_size=first, hidden=64, intermediate=64, experts=4, top_k=2, io_dtype=_lib.FP32, limit=7.0,
                     layouts=99, tp_world=5)      # garbage behind the old end is not read
    n_old, n_new = ctypes.c_size_t(0), ctypes.c_size_t(0)
    L = garnet_b200.lib()
    assert L.garnet_b200_moe_workspace(ctypes.byref(opt), 8, ctypes.byref(n_old)) == 0
    opt2 = MoeOptions(abi=1, struct_size=ctypes.sizeof(MoeOptions), hidden=64, intermediate=64, experts=4, top_k=2,
                      io_dtype=_lib.FP32, limit=7.0)
    assert L.garnet_b200_moe_workspace(ctypes.byref(opt2), 8, ctypes.byref(n_new)) == 0
    assert n_old.value == n_new.value > 0
    opt2.struct_size = first + 4
    assert L.garnet_b200_moe_workspace(ctypes.byref(opt2), 8, ctypes.byref(n_new)) == 1
    opt2.struct_size = ctypes.sizeof(MoeOptions)
    opt2.tp_world, opt2.tp_rank = 2, 2
    assert L.garnet_b200_moe_workspace(ctypes.byref(opt2), 8, ctypes.byref(n_new)) == 1
    opt2.tp_rank, opt2.intermediate = 0, 96       # 96 / 2 is not a whole number of 32-column groups
    assert L.garnet_b200_moe_workspace(ctypes.byref(opt2), 8, ctypes.byref(n_new)) == 1


def test_moe_workspace_sizes_never_shrink_with_the_token_count():
    """A caller sizes its workspaces once for its largest batch (garnet_b200_moe_ep_create does): a smaller batch
    must fit in them, also across the token counts where the router changes its number of K ranges."""
    from garnet_b200.moe import MoeOptions
    opt = MoeOptions(abi=1, struct_size=ctypes.sizeof(MoeOptions), hidden=2880, intermediate=2880, experts=128, top_k=4,
                     io_dtype=_lib.BF16, limit=7.0)
    L = garnet_b200.lib()
    n = ctypes.c_size_t(0)
    last_route = last_run = 0
    for tokens in list(range(1, 40)) + list(range(480, 560)) + [1000, 1024, 4096, 8192]:
        assert L.garnet_b200_moe_route_workspace(ctypes.byref(opt), tokens, ctypes.byref(n)) == 0
        assert n.value >= last_route, tokens
        last_route = n.value
        assert L.garnet_b200_moe_workspace(ctypes.byref(opt), tokens, ctypes.byref(n)) == 0
        assert n.value >= last_run, tokens
        last_run = n.value
