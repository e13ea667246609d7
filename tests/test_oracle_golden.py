"""Pins the CPU oracle: against the committed golden vectors produced by the
reference's own code, against the reference's test bounds, and (when the
compiled reference sources are present) bit-for-bit against the reference."""
import os

import numpy as np
import pytest

import oracle
import oracle.ref as ref

GOLD = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def int4():
    return np.load(os.path.join(GOLD, "int4_ref.npz"))


@pytest.fixture(scope="module")
def tiny_moe():
    return np.load(os.path.join(GOLD, "gpt_oss_tiny_moe.npz"))


def fp16_bits_to_f32(b):
    return np.asarray(b, np.uint16).view(np.float16).astype(np.float32)


@pytest.mark.parametrize("name,block", [("blk64", 64), ("blk128", 128), ("chan256", 256)])
def test_quantizer_matches_reference_bytes(int4, name, block):
    src = int4[f"quant_{name}_src"]
    packed, scales, err = oracle.int4_quantize(src, block, "fp16")
    assert np.array_equal(packed, int4[f"quant_{name}_packed"])
    assert np.array_equal(scales, int4[f"quant_{name}_scales_fp16"])
    assert err == float(int4[f"quant_{name}_max_error"])
    # weight_quantization_test.cpp:74-94: reconstruction within half a step
    s = fp16_bits_to_f32(scales)
    rec = oracle.int4_dequant(packed, s, src.shape[0], src.shape[1], block)
    bound = np.repeat(s, block, axis=1) * 0.501 + 1e-6
    assert (np.abs(rec - src) <= bound).all()
    assert scales.shape == (src.shape[0], src.shape[1] // block)


def test_q4q8_matches_reference_output(int4):
    rows, cols, g = 7, 256, 128
    s = fp16_bits_to_f32(int4["q4q8_scales_fp16"])
    y = oracle.q4q8_forward(int4["q4q8_packed"], s, rows, cols, g, int4["q4q8_x"])
    assert np.array_equal(y, int4["q4q8_y"])
    # q4q8_linear_test.cpp:84-120: the scalar int8 restatement agrees to 1e-5
    q = oracle.int4_unpack(int4["q4q8_packed"], rows, cols).astype(np.int64)
    x = int4["q4q8_x"]
    expect = np.zeros(rows, np.float32)
    for gi in range(cols // g):
        xs = x[gi * g:(gi + 1) * g]
        sx = np.float32(np.abs(xs).max() / np.float32(127.0))
        qx = np.clip(np.rint(xs / sx), -127, 127).astype(np.int64)
        dot = (q[:, gi * g:(gi + 1) * g] * qx).sum(axis=1)
        expect += dot.astype(np.float32) * sx * s[:, gi]
    assert np.abs(expect - y).max() <= 1e-5


def test_q4q8_random_case_and_exact_oracle(int4):
    N, K, g = 48, 512, 128
    s = int4["rand_scales_bf16_as_f32"]
    y = oracle.q4q8_forward(int4["rand_packed"], s, N, K, g, int4["rand_x"])
    assert np.array_equal(y, int4["rand_y_q4q8"])
    y32, y64 = oracle.w4a16_exact(int4["rand_packed"], s, N, K, g, int4["rand_x"])
    # the W4A8 operator differs from the exact W4A16 product only by its int8
    # activation rounding: well inside 1e-2 in the reference's error form
    assert (np.abs(y - y64[0]) <= 1e-2 * (1 + np.abs(y64[0]))).all()
    assert np.abs(y32 - y64).max() <= 1e-4
    assert np.allclose(oracle.w4a16_blas(int4["rand_packed"], s, N, K, g, int4["rand_x"]), y64, rtol=0, atol=1e-9)


def test_int4_pack_roundtrip():
    rng = np.random.default_rng(1)
    q = rng.integers(-8, 8, size=(5, 64)).astype(np.int8)
    assert np.array_equal(oracle.int4_unpack(oracle.int4_pack(q), 5, 64), q)


def test_mxfp4_all_codes_and_scales():
    """kernel_parity.cpp:537-559: every (e8m0, code) pair, including subnormal
    results, overflow, signed zero and the NaN scale."""
    bits = oracle.mxfp4_table()
    ldexp = oracle.mxfp4_table_ldexp()
    assert np.array_equal(bits[:255].view(np.uint32), ldexp[:255].view(np.uint32))
    assert np.isnan(bits[255]).all()
    assert np.signbit(bits[127][8]) and bits[127][8] == 0.0
    assert list(bits[127][:8]) == [0, .5, 1, 1.5, 2, 3, 4, 6]
    assert np.isinf(bits[254][4:8]).all() and bits[254][3] == np.float32(1.5) * np.float32(2.0) ** 127
    assert bits[0][1] == np.float32(2.0) ** -128


@pytest.mark.parametrize("inter", [32, 64])
@pytest.mark.parametrize("layer", [0, 1])
def test_moe_matches_reference_python(tiny_moe, inter, layer):
    g, t = tiny_moe, f"i{inter}_l{layer}_"
    y, logits, sel, pr = oracle.moe_forward(
        g[t + "x"], g[t + "router_w"], g[t + "router_b"], g[t + "gu_blocks"], g[t + "gu_scales"],
        g[t + "gu_bias"].reshape(-1), g[t + "dn_blocks"], g[t + "dn_scales"], g[t + "dn_bias"].reshape(-1),
        32, inter, 5, 2)
    # make_fixture.py accumulates in double; allow the reference's own bound
    # (compiled_parity.py tol .025) but expect far better
    assert np.abs(y - g[t + "y"]).max() <= 2.0 ** -8
    assert (y == g[t + "y"]).mean() > 0.98


def test_moe_sharded_partials_sum_to_full(tiny_moe):
    """kernel_parity.cpp:653-673: two expert-parallel partial sums, rounded after
    the add, reproduce the unsharded result."""
    g, t = tiny_moe, "i64_l0_"
    args = (g[t + "gu_blocks"], g[t + "gu_scales"], g[t + "gu_bias"].reshape(-1), g[t + "dn_blocks"],
            g[t + "dn_scales"], g[t + "dn_bias"].reshape(-1), 32, 64, 5, 2)
    x = g[t + "x"]
    _, sel, pr = oracle.moe_route(x, g[t + "router_w"], g[t + "router_b"], 5, 2)
    full = oracle.moe_experts(x, sel, pr, *args)
    parts = [oracle.moe_experts(x, sel, pr, *args, modulo=2, residue=r, round_output=False) for r in (0, 1)]
    assert np.abs(oracle.bf16_round(parts[0] + parts[1]) - full).max() <= 0.002 * (1 + np.abs(full).max())
    blocks = [oracle.moe_experts(x, sel, pr, *args, expert_lo=lo, expert_hi=hi, round_output=False)
              for lo, hi in ((0, 2), (2, 5))]
    assert np.abs(oracle.bf16_round(blocks[0] + blocks[1]) - full).max() <= 0.002 * (1 + np.abs(full).max())


def test_route_tie_break_lowest_index():
    x = np.ones((3, 32), np.float32)
    sel = oracle.moe_route(x, np.zeros((5, 32), np.float32), np.zeros(5, np.float32), 5, 2)[1]
    assert (sel == np.array([0, 1])).all()


@pytest.mark.skipif(not ref.available(), reason="compiled reference sources not present")
def test_oracle_bit_exact_with_compiled_reference():
    rng = np.random.default_rng(7)
    for (N, K, g) in [(64, 256, 64), (96, 1024, 128), (40, 512, 256)]:
        w = rng.normal(0, 0.05, (N, K)).astype(np.float32)
        a, b = ref.quantize_int4(w, g), oracle.int4_quantize(w, g, "fp16")
        assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1]) and a[2] == b[2]
        s = oracle.bf16_round(fp16_bits_to_f32(a[1]))
        op = ref.Q4Q8Linear(a[0], s, N, K, g)
        for i in range(3):
            x = oracle.bf16_round(rng.normal(0, 1, K).astype(np.float32))
            if i == 2:
                x[:g] = 0
            assert np.array_equal(op.forward(x, 2), oracle.q4q8_forward(a[0], s, N, K, g, x))
