"""Generates the golden vectors in this directory from the reference itself.

Run in a container that has the reference checkout (pass its path as argv[1] or
set GARNET_REFERENCE_DIR) after `make -C oracle ref REF=<checkout>`:

    python tests/golden/make_golden.py <checkout>

int4_ref.npz      outputs of the reference's compiled int4 sources
                  (Garnet::QuantizeSymmetricINT4, Garnet::Q4Q8Linear) on the
                  closed-form inputs of test2026/native/q4q8_linear_test.cpp:33-43
                  and test2026/native/weight_quantization_test.cpp:57-64,100-110,152-158.
gpt_oss_tiny_moe.npz
                  every (input, output) pair that passes through the pure-Python
                  MoE of test2026/gpt_oss/make_fixture.py:117-135 while that
                  script builds its tiny checkpoint (5 experts, top-2, hidden 32),
                  together with the MoE tensors it wrote.  The pairs are captured
                  with a profile hook; the reference script is run unmodified.
"""
import json
import os
import struct
import sys
import tempfile
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
HERE = Path(__file__).resolve().parent


def bf16_bits_to_f32(b):
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_f32(x):
    v = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    return (((v + 0x7FFF + ((v >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)).view(np.float32)


def int4_golden():
    import oracle.ref as ref
    out = {}
    # q4q8_linear_test.cpp:33-43
    rows, cols, g = 7, 256, 128
    # the reference evaluates std::sin / std::cos on float arguments: use libm's float forms
    import ctypes
    m = ctypes.CDLL("libm.so.6")
    m.sinf.restype = ctypes.c_float; m.sinf.argtypes = [ctypes.c_float]
    m.cosf.restype = ctypes.c_float; m.cosf.argtypes = [ctypes.c_float]
    src = np.array([m.sinf(np.float32(i) * np.float32(0.019)) * np.float32(0.08)
                    for i in range(rows * cols)], dtype=np.float32).reshape(rows, cols)
    x = np.array([m.cosf(np.float32(i) * np.float32(0.031)) for i in range(cols)], dtype=np.float32)
    packed, scales, err = ref.quantize_int4(src, g)
    op = ref.Q4Q8Linear(packed, scales.view(np.float16).astype(np.float32), rows, cols, g)
    out.update(q4q8_src=src, q4q8_x=x, q4q8_packed=packed, q4q8_scales_fp16=scales,
               q4q8_y=op.forward(x, 4), q4q8_max_error=np.float64(err))
    # weight_quantization_test.cpp: three bf16 sources
    cases = [("blk64", 2, 64, 64, lambda i: m.sinf(np.float32(i) * np.float32(0.17)) * np.float32(0.75 if i < 64 else 2.5)),
             ("blk128", 2, 128, 128, lambda i: m.cosf(np.float32(i) * np.float32(0.11)) * np.float32(1.25 if i < 128 else 3.0)),
             ("chan256", 2, 256, 256, lambda i: m.sinf(np.float32(i) * np.float32(0.03)) * np.float32(2.0))]
    for name, r, c, blk, fn in cases:
        w = f32_to_bf16_f32(np.array([fn(i) for i in range(r * c)], dtype=np.float32)).reshape(r, c)
        p, s, e = ref.quantize_int4(w, blk)
        out[f"quant_{name}_src"] = w
        out[f"quant_{name}_packed"] = p
        out[f"quant_{name}_scales_fp16"] = s
        out[f"quant_{name}_max_error"] = np.float64(e)
    # a seeded random case through both reference entry points
    rng = np.random.default_rng(20240607)
    N, K, g = 48, 512, 128
    w = rng.normal(0, 0.02, (N, K)).astype(np.float32)
    p, s, e = ref.quantize_int4(w, g)
    sb = f32_to_bf16_f32(s.view(np.float16).astype(np.float32))
    xs = f32_to_bf16_f32(rng.normal(0, 1, K).astype(np.float32))
    op = ref.Q4Q8Linear(p, sb, N, K, g)
    out.update(rand_src=w, rand_packed=p, rand_scales_fp16=s, rand_scales_bf16_as_f32=sb,
               rand_x=xs, rand_y_q4q8=op.forward(xs, 2))
    np.savez_compressed(HERE / "int4_ref.npz", **out)
    print("int4_ref.npz:", {k: getattr(v, "shape", v) for k, v in out.items()})


def read_safetensors(path):
    raw = Path(path).read_bytes()
    n = struct.unpack("<Q", raw[:8])[0]
    header = json.loads(raw[8:8 + n])
    data = raw[8 + n:]
    tensors = {}
    for name, e in header.items():
        a, b = e["data_offsets"]
        buf = np.frombuffer(data[a:b], dtype=np.uint8)
        if e["dtype"] == "U8":
            tensors[name] = buf.reshape(e["shape"]).copy()
        else:
            tensors[name] = bf16_bits_to_f32(buf.view(np.uint16)).reshape(e["shape"]).copy()
    return tensors


def moe_golden(reference_dir):
    sys.path.insert(0, str(Path(reference_dir) / "test2026" / "gpt_oss"))
    import make_fixture
    out = {}
    for inter in (32, 64):
        calls = []

        def hook(frame, event, arg):
            if frame.f_code.co_name == "moe" and frame.f_code.co_filename == make_fixture.__file__:
                if event == "call":
                    frame.f_locals  # materialise
                    calls.append([list(frame.f_locals["x"]), frame.f_locals["p"], None])
                elif event == "return":
                    # returns come in LIFO order; moe() is not re-entrant
                    for c in reversed(calls):
                        if c[2] is None:
                            c[2] = list(arg)
                            break

        with tempfile.TemporaryDirectory() as tmp:
            sys.setprofile(hook)
            try:
                make_fixture.create(Path(tmp) / "fx", intermediate=inter)
            finally:
                sys.setprofile(None)
            tensors = read_safetensors(Path(tmp) / "fx" / "model.safetensors")
        tag = f"i{inter}"
        for layer in range(2):
            p = f"block.{layer}.mlp"
            out[f"{tag}_l{layer}_router_w"] = tensors[p + ".gate.weight"]
            out[f"{tag}_l{layer}_router_b"] = tensors[p + ".gate.bias"]
            out[f"{tag}_l{layer}_gu_blocks"] = tensors[p + ".mlp1_weight.blocks"]
            out[f"{tag}_l{layer}_gu_scales"] = tensors[p + ".mlp1_weight.scales"]
            out[f"{tag}_l{layer}_gu_bias"] = tensors[p + ".mlp1_bias"]
            out[f"{tag}_l{layer}_dn_blocks"] = tensors[p + ".mlp2_weight.blocks"]
            out[f"{tag}_l{layer}_dn_scales"] = tensors[p + ".mlp2_weight.scales"]
            out[f"{tag}_l{layer}_dn_bias"] = tensors[p + ".mlp2_bias"]
            xs = np.array([c[0] for c in calls if c[1] == p], dtype=np.float32)
            ys = np.array([c[2] for c in calls if c[1] == p], dtype=np.float32)
            # drop exact duplicates (the script re-evaluates prefixes)
            _, keep = np.unique(xs.view(np.uint32), axis=0, return_index=True)
            keep.sort()
            out[f"{tag}_l{layer}_x"] = xs[keep]
            out[f"{tag}_l{layer}_y"] = ys[keep]
    np.savez_compressed(HERE / "gpt_oss_tiny_moe.npz", **out)
    print("gpt_oss_tiny_moe.npz:", {k: v.shape for k, v in out.items() if k.endswith(("_x", "_y"))})


if __name__ == "__main__":
    ref_dir = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("GARNET_REFERENCE_DIR", "")
    if not ref_dir:
        sys.exit("usage: make_golden.py <reference checkout>")
    int4_golden()
    moe_golden(ref_dir)
