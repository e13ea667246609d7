"""The checkpoint side on the CPU: the .safetensors reader (single file, shard index, directory)
and writer round trip; the host int4 quantizer bit for bit against the oracle (itself bit-identical
to the reference's QuantizeSymmetricINT4); derived-constant names; and the packed-constant cache of a
small checkpoint: every Qwen linear arrives as exactly the bytes quantize + pack give, every gpt-oss
expert pair as exactly the bytes of the host packer, everything else unchanged."""
import json
import os
import struct

import numpy as np
import pytest

import garnet_b200
import oracle
from garnet_b200 import _lib, checkpoint as ck
from garnet_b200 import moe as moe_mod


def bf16_bits(a):
    return oracle.bf16_bits(np.asarray(a, np.float32))


def test_reader_and_writer_round_trip(tmp_path):
    rng = np.random.default_rng(0)
    tensors = {"a.weight": rng.normal(size=(3, 5)).astype(np.float32), "b": rng.integers(0, 255, size=(7,)).astype(np.uint8),
               'odd "name"\\x': rng.normal(size=(2, 2, 2)).astype(np.float16), "empty": np.zeros((0, 4), np.float32),
               "bits": bf16_bits(rng.normal(size=(4, 8)))}
    path = tmp_path / "one.safetensors"
    ck.write_safetensors(path, tensors, {"bits": "BF16"})
    # the file is what any safetensors reader expects: 8-byte header length, JSON, data
    raw = path.read_bytes()
    n = struct.unpack("<Q", raw[:8])[0]
    header = json.loads(raw[8:8 + n])
    assert header["bits"]["dtype"] == "BF16" and header["a.weight"]["shape"] == [3, 5] and (8 + n) % 256 == 0
    st = ck.SafeTensors(path)
    assert sorted(st.names()) == sorted(tensors)
    for name, a in tensors.items():
        got = st.tensor(name)
        assert got.shape == a.shape and np.array_equal(got, a)
    assert st.info("bits") == ("BF16", (4, 8), 64)
    with pytest.raises(garnet_b200.GarnetB200Error):
        st.tensor("missing")
    st.close()


def test_shard_index_and_directory(tmp_path):
    rng = np.random.default_rng(1)
    a, b, c = [rng.normal(size=(4, 4)).astype(np.float32) for _ in range(3)]
    ck.write_safetensors(tmp_path / "model-00001-of-00002.safetensors", {"x": a, "y": b})
    ck.write_safetensors(tmp_path / "model-00002-of-00002.safetensors", {"z": c})
    index = {"metadata": {"total_size": 192}, "weight_map": {"x": "model-00001-of-00002.safetensors",
                                                               "y": "model-00001-of-00002.safetensors",
                                                               "z": "model-00002-of-00002.safetensors"}}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index, indent=2))
    for path in (tmp_path, tmp_path / "model.safetensors.index.json"):
        st = ck.SafeTensors(path)
        assert len(st) == 3 and np.array_equal(st.tensor("z"), c) and np.array_equal(st.tensor("x"), a)
        st.close()
    index["weight_map"]["ghost"] = "model-00002-of-00002.safetensors"
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    with pytest.raises(garnet_b200.GarnetB200Error):
        ck.SafeTensors(tmp_path)


def test_malformed_files_are_refused(tmp_path):
    bad = tmp_path / "bad.safetensors"
    bad.write_bytes(b"\x05\x00")
    with pytest.raises(garnet_b200.GarnetB200Error):
        ck.SafeTensors(bad)
    bad.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")                       # header longer than the file
    with pytest.raises(garnet_b200.GarnetB200Error):
        ck.SafeTensors(bad)
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 64]}}).encode()   # data beyond the file
    bad.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 16)
    with pytest.raises(garnet_b200.GarnetB200Error):
        ck.SafeTensors(bad)
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [3], "data_offsets": [0, 16]}}).encode()   # 3 floats are not 16 bytes
    bad.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 16)
    with pytest.raises(garnet_b200.GarnetB200Error):
        ck.SafeTensors(bad)
    with pytest.raises(garnet_b200.GarnetB200Error):
        ck.SafeTensors(tmp_path / "nowhere.safetensors")


@pytest.mark.parametrize("scale_kind,code", [("fp16", _lib.FP16), ("bf16", _lib.BF16)])
def test_host_quantizer_is_the_oracle_bit_for_bit(scale_kind, code):
    rng = np.random.default_rng(5)
    w = (rng.normal(size=(24, 512)) * 0.05).astype(np.float32)
    w[3, :128] = 0.0                       # an all-zero group: scale 1
    w[5, 7] = 3.0e4                        # a large value
    w[6, :128] *= 1e-7                     # scales that are fp16 subnormals
    for src, src_code in ((w, None), (w.astype(np.float16), None), (bf16_bits(w), _lib.BF16)):
        as_f32 = src.astype(np.float32) if src_code is None else oracle.bf16_from_bits(src)
        nib, sc, err = ck.quantize_int4_host(src, 128, code, src_code)
        o_nib, o_sc, o_err = oracle.int4_quantize(as_f32, 128, scale_kind)
        assert np.array_equal(nib, o_nib) and np.array_equal(sc.reshape(-1), np.asarray(o_sc).reshape(-1))
        assert err == pytest.approx(o_err, rel=0, abs=0)


def test_derived_names_round_trip():
    n = ck.packed_name("model.layers.3.mlp.down_proj.weight", 0, 128, _lib.BF16)
    assert n == "__garnet_b200_w4a16_v1_g128_s1__:model.layers.3.mlp.down_proj.weight"
    assert ck.parse_packed_name(n) == (0, 128, _lib.BF16, 0, "model.layers.3.mlp.down_proj.weight")
    m = ck.packed_name("block.7.mlp.mlp1_weight", 2, 0, 1, 2)
    assert m == "__garnet_b200_mxb_v1_u0_t1of2__:block.7.mlp.mlp1_weight"
    assert ck.parse_packed_name(m) == (2, 0, 1, 2, "block.7.mlp.mlp1_weight")
    for bad in ("model.weight", "__garnet_b200_w4a16_v1_g128_s1__:", "__garnet_b200_mxq_v1_u0_t0of1__:x"):
        with pytest.raises(garnet_b200.GarnetB200Error):
            ck.parse_packed_name(bad)


def test_packed_constant_cache_of_a_small_checkpoint(tmp_path):
    rng = np.random.default_rng(9)
    H, I, E = 64, 64, 3
    qw = (rng.normal(size=(256, 128)) * 0.03).astype(np.float32)
    tensors = {
        "model.layers.0.self_attn.q_proj.weight": bf16_bits(qw),
        "model.layers.0.input_layernorm.weight": bf16_bits(1 + 0.1 * rng.normal(size=128)),
        "model.layers.0.mlp.odd.weight": bf16_bits(rng.normal(size=(8, 100))),            # K is not a multiple of the group: copied
        "block.0.mlp.mlp1_weight.blocks": rng.integers(0, 256, size=(E, 2 * I, H // 32, 16), dtype=np.uint8),
        "block.0.mlp.mlp1_weight.scales": rng.integers(110, 130, size=(E, 2 * I, H // 32), dtype=np.uint8),
        "block.0.mlp.mlp2_weight.blocks": rng.integers(0, 256, size=(E, H, I // 32, 16), dtype=np.uint8),
        "block.0.mlp.mlp2_weight.scales": rng.integers(110, 130, size=(E, H, I // 32), dtype=np.uint8),
        "block.0.mlp.mlp1_bias": bf16_bits(rng.normal(size=(E, 2 * I))),
    }
    dts = {k: "BF16" for k, v in tensors.items() if v.dtype == np.uint16}
    ck.write_safetensors(tmp_path / "model.safetensors", tensors, dts)
    st = ck.SafeTensors(tmp_path)
    st.build_cache(tmp_path / "cache.safetensors", 128, _lib.BF16)
    cache = ck.SafeTensors(tmp_path / "cache.safetensors")
    names = set(cache.names())
    # the linear: quantized and packed, under its derived name, and gone under its own
    lin = ck.packed_name("model.layers.0.self_attn.q_proj.weight", 0, 128, _lib.BF16)
    assert lin in names and "model.layers.0.self_attn.q_proj.weight" not in names
    nib, sc, _ = ck.quantize_int4_host(tensors["model.layers.0.self_attn.q_proj.weight"], 128, _lib.BF16, _lib.BF16)
    import torch
    want = garnet_b200.pack_host(torch.from_numpy(nib), torch.from_numpy(sc.view(np.int16)).view(torch.bfloat16), 256, 128, 128).numpy()
    assert np.array_equal(cache.tensor(lin), want)
    # the expert pairs: both layouts, exactly the host packer's bytes; blocks and scales are consumed
    moe = garnet_b200.GptOssMoe(H, I, E, 1)
    for which, stem in ((0, "block.0.mlp.mlp1_weight"), (1, "block.0.mlp.mlp2_weight")):
        for kind, layout in ((1, moe_mod.LAYOUT_STREAM), (2, moe_mod.LAYOUT_BLOCK)):
            name = ck.packed_name(stem, kind, which, 0, 1)
            assert name in names
            assert np.array_equal(cache.tensor(name), moe.pack_host(which, layout, tensors[stem + ".blocks"], tensors[stem + ".scales"]))
        assert stem + ".blocks" not in names and stem + ".scales" not in names
    # everything else is copied as it is
    for keep in ("model.layers.0.input_layernorm.weight", "model.layers.0.mlp.odd.weight", "block.0.mlp.mlp1_bias"):
        assert cache.info(keep)[0] == "BF16" and np.array_equal(cache.tensor(keep), tensors[keep])
    # one layout only, and this rank's half of the intermediate axis
    st.build_cache(tmp_path / "cache_tp.safetensors", 128, _lib.BF16, moe_mod.LAYOUT_BLOCK, 1, 2)
    tp = ck.SafeTensors(tmp_path / "cache_tp.safetensors")
    moe_tp = garnet_b200.GptOssMoe(H, I, E, 1, tp_rank=1, tp_world=2)
    name = ck.packed_name("block.0.mlp.mlp2_weight", 2, 1, 1, 2)
    local_b = moe_mod.gather_intermediate_shard(tensors["block.0.mlp.mlp2_weight.blocks"], 1, 2, 2)
    local_s = moe_mod.gather_intermediate_shard(tensors["block.0.mlp.mlp2_weight.scales"], 1, 2, 2)
    assert np.array_equal(tp.tensor(name), moe_tp.pack_host(1, moe_mod.LAYOUT_BLOCK, local_b, local_s))
    assert ck.packed_name("block.0.mlp.mlp2_weight", 1, 1, 1, 2) not in set(tp.names())
