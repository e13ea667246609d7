"""Parity of the MXFP4 MoE operator on the GPU, through the C ABI, against the
CPU oracle.  Cases and bounds follow test2026/gpt_oss/kernel_parity.cpp: the
exhaustive 256 x 16 decode table (:537-559, bit-exact), the closed-form MoE
fixtures of testMoe (:610-652; tolerance .002 in the form |a-e| <= tol (1+|e|)),
two-rank expert-parallel partial sums (:653-673), plus the gpt-oss-120b layer
shape with the synthetic distributions of the benchmark (tolerance 1e-2, the
specified bound)."""
import os

import numpy as np
import pytest
import torch

import garnet_b200
import oracle
from garnet_b200 import synth

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def reference_fixture(tokens, h=32, inter=32, tied=False):
    """Inputs of testMoe (kernel_parity.cpp:610-626), restated from their closed forms."""
    f32 = np.float32
    bf = oracle.bf16_round
    x = bf(np.cos(np.arange(tokens * h, dtype=f32) * f32(.17)).astype(f32)).reshape(tokens, h)
    router = bf((np.sin(np.arange(5 * h, dtype=f32) * f32(.37)) * f32(.1)).astype(f32)).reshape(5, h)
    rb = np.array([-.2, .4, -.1, .3, -.5], f32)
    if tied:
        router[:] = 0
        rb[:] = 0
    ub = bf(((np.arange(5 * 2 * inter) % 9 - 4).astype(f32) * f32(.125))).reshape(5, 2 * inter)
    db = bf(((np.arange(5 * h) % 7 - 3).astype(f32) * f32(.125))).reshape(5, h)
    up = ((np.arange(5 * 2 * inter * h // 2, dtype=np.int64) * 73 + 11) % 256).astype(np.uint8)
    down = ((np.arange(5 * h * inter // 2, dtype=np.int64) * 31 + 57) % 256).astype(np.uint8)
    us = np.full(5 * 2 * inter * h // 32, 123, np.uint8)
    ds = np.full(5 * h * inter // 32, 124, np.uint8)
    return dict(x=x, router_w=router, router_b=rb, gu_blocks=up.reshape(5, 2 * inter, h // 32, 16),
                gu_scales=us.reshape(5, 2 * inter, h // 32), gu_bias=ub, dn_blocks=down.reshape(5, h, inter // 32, 16),
                dn_scales=ds.reshape(5, h, inter // 32), dn_bias=db, hidden=h, inter=inter, experts=5, topk=2)


def build(case, **kw):
    moe = garnet_b200.GptOssMoe(case["hidden"], case["inter"], case["experts"], case["topk"], **kw)
    return moe.prepare(*[dev(case[k]) for k in ("router_w", "router_b", "gu_blocks", "gu_scales", "gu_bias",
                                                 "dn_blocks", "dn_scales", "dn_bias")])


def oracle_args(case):
    return (case["gu_blocks"], case["gu_scales"], case["gu_bias"].reshape(-1), case["dn_blocks"], case["dn_scales"],
            case["dn_bias"].reshape(-1), case["hidden"], case["inter"], case["experts"], case["topk"])


def assert_close(actual, expected, tol, what="", mass=None):
    """|a - e| <= tol * (1 + |e|) (kernel_parity.cpp:46-57).  With `mass`, the scale
    of the summands of each output, outputs that nearly cancel are judged against
    that scale instead: every per-slot value is rounded to bf16 before the
    weighted sum (in the reference as here), so one rounding step of a large
    summand legitimately moves a small sum by more than tol * (1 + |sum|)."""
    err = np.abs(actual.astype(np.float64) - expected.astype(np.float64))
    assert np.isfinite(actual).all(), what
    scale = 1 + np.abs(expected) if mass is None else 1 + np.maximum(np.abs(expected), mass)
    worst = (err / scale).max()
    assert worst <= tol, f"{what}: scaled error {worst}"
    if mass is not None:
        assert (err <= tol * (1 + np.abs(expected))).mean() >= 0.98, what


def check_routing(case, logits, sel, pr):
    """Router parity that does not depend on the fp32 summation order:
    - logits equal the oracle's bf16-rounded logits, except where a different
      summation order rounds the other way (at most one bf16 step, rarely);
    - the selection is exactly the top-k of the device's own logits under the
      reference's order (value descending, index ascending, kernel_parity.cpp:630);
    - probabilities are bf(softmax) of the selected device logits (one bf16 step
      allowed for the device's expf)."""
    E, k = case["experts"], case["topk"]
    o_logits, o_sel, o_pr = oracle.moe_route(case["x"], case["router_w"], case["router_b"], E, k)
    step = np.maximum(np.abs(o_logits), 2.0 ** -126) * 2.0 ** -7
    assert (np.abs(logits - o_logits) <= step).all()
    assert (logits == o_logits).mean() >= 0.97
    order = np.lexsort((np.broadcast_to(np.arange(E), logits.shape), -logits), axis=1)[:, :k]
    assert np.array_equal(sel, order.astype(np.int32))
    top = np.take_along_axis(logits, order, axis=1).astype(np.float32)
    ex = np.exp((top - top[:, :1]).astype(np.float32)).astype(np.float32)
    want = oracle.bf16_round((ex / ex.sum(axis=1, keepdims=True, dtype=np.float32)).astype(np.float32))
    assert (np.abs(pr - want) <= np.abs(want) * 2.0 ** -7 + 1e-30).all()
    assert (pr == want).mean() >= 0.97
    same = (logits == o_logits).all(axis=1)
    assert np.array_equal(sel[same], o_sel[same])


def run_and_compare(case, tol, use_mass=False, **kw):
    """Routing is checked on its own; expert outputs are compared with the oracle
    evaluated on the device's routing, so that a legitimate one-step difference
    in a router logit cannot change which experts are compared."""
    moe = build(case, **kw)
    x = dev(case["x"])
    y = moe.run(x).cpu().numpy()
    torch.cuda.synchronize()
    assert moe.fault() == 0
    logits, sel, pr = [t.cpu().numpy() for t in moe.route(x)]
    check_routing(case, logits, sel, pr)
    expect, mass = oracle.moe_experts(case["x"], sel, pr, *oracle_args(case), want_mass=True)
    assert_close(y, expect, tol, "moe output", mass if use_mass else None)
    return moe, y, sel, pr


def test_mxfp4_decode_all_codes_and_scales_bit_exact():
    blocks = np.zeros((256, 16), np.uint8)
    for byte in range(16):
        blocks[:, byte] = ((2 * byte) & 15) | (((2 * byte + 1) & 15) << 4)
    scales = np.arange(256, dtype=np.uint8)
    got = garnet_b200.mxfp4_decode(dev(blocks), dev(scales)).cpu().numpy()
    table = oracle.mxfp4_table()          # [scale, code]
    expect = np.stack([table[:, c & 15] for c in range(32)], axis=1)
    assert np.isnan(got[255]).all()
    assert np.array_equal(got[:255].view(np.uint32), expect[:255].view(np.uint32))


@pytest.mark.parametrize("h,inter", [(32, 32), (96, 64), (2880, 64), (64, 2880)])
def test_packed_expert_matrices_decode_bit_exact(h, inter):
    case = synth.moe_layer(1, h, inter, experts=3, topk=2, seed=h + inter)
    case["gu_scales"][0, :5, 0] = [0, 1, 254, 255, 2]       # subnormal, NaN and extreme scales
    moe = build(case)
    for e in range(3):
        up = moe.dequantized(0, e).cpu().numpy()
        dn = moe.dequantized(1, e).cpu().numpy()
        eu = oracle.mxfp4_dequant(case["gu_blocks"][e], case["gu_scales"][e], 2 * inter, h)
        ed = oracle.mxfp4_dequant(case["dn_blocks"][e], case["dn_scales"][e], h, inter)
        same = lambda a, b: np.array_equal(a.view(np.uint32)[~np.isnan(b)], b.view(np.uint32)[~np.isnan(b)]) and np.array_equal(np.isnan(a), np.isnan(b))
        assert same(up, eu) and same(dn, ed)


@pytest.mark.parametrize("tokens", [1, 3, 17, 65])
@pytest.mark.parametrize("h,inter", [(32, 32), (96, 64)])
def test_reference_fixtures(tokens, h, inter):
    run_and_compare(reference_fixture(tokens, h, inter), 0.002)


@pytest.mark.parametrize("tokens,h,inter,tied", [(65, 96, 64, True), (513, 32, 32, True), (128, 96, 64, False),
                                                 (3, 96, 2880, False), (513, 96, 64, True), (1024, 96, 256, False)])
def test_reference_fixtures_large(tokens, h, inter, tied):
    case = reference_fixture(tokens, h, inter, tied)
    moe, y, sel, pr = run_and_compare(case, 0.002)
    if tied:      # all logits equal: lowest indices win (kernel_parity.cpp:630)
        assert (sel == np.array([0, 1])).all()


@pytest.mark.parametrize("inter", [32, 64])
def test_golden_pairs_from_reference_python(inter):
    g = np.load(os.path.join(GOLD, "gpt_oss_tiny_moe.npz"))
    for layer in range(2):
        t = f"i{inter}_l{layer}_"
        case = dict(x=g[t + "x"], router_w=g[t + "router_w"], router_b=g[t + "router_b"], gu_blocks=g[t + "gu_blocks"],
                    gu_scales=g[t + "gu_scales"], gu_bias=g[t + "gu_bias"], dn_blocks=g[t + "dn_blocks"],
                    dn_scales=g[t + "dn_scales"], dn_bias=g[t + "dn_bias"], hidden=32, inter=inter, experts=5, topk=2)
        y = build(case).run(dev(case["x"])).cpu().numpy()
        assert_close(y, g[t + "y"], 0.004, "golden")


def test_bf16_io_matches_fp32_carrier():
    case = reference_fixture(17, 96, 64)
    y32 = build(case).run(dev(case["x"]))
    y16 = build(case, io_dtype=torch.bfloat16).run(dev(case["x"]).bfloat16())
    assert torch.equal(y32.bfloat16(), y16)


@pytest.mark.parametrize("tokens", [1, 32])
def test_gpt_oss_120b_layer_shape(tokens):
    case = synth.moe_layer(tokens, seed=tokens)
    run_and_compare(case, 1e-2, use_mass=True)


def test_gpt_oss_120b_layer_shape_sampled_tokens():
    tokens = 512
    case = synth.moe_layer(tokens, seed=7, bias_scale=0.05)
    moe = build(case)
    x = dev(case["x"])
    y = moe.run(x).cpu().numpy()
    _, sel, pr = [t.cpu().numpy() for t in moe.route(x)]
    pick = np.random.default_rng(0).choice(tokens, 24, replace=False)
    expect, mass = oracle.moe_experts(case["x"][pick], sel[pick], pr[pick], *oracle_args(case), want_mass=True)
    assert_close(y[pick], expect, 1e-2, "sampled tokens", mass)
    counts = np.bincount(sel.reshape(-1), minlength=128)
    assert counts.sum() == tokens * 4 and (np.sort(sel, axis=1)[:, 1:] != np.sort(sel, axis=1)[:, :-1]).all()


def test_expert_parallel_partials():
    """Interleaved 2-way split (the reference's rule) and contiguous 4-way blocks:
    unrounded per-rank partials, summed and rounded, reproduce the full result;
    rank-local expert tensors give the same partial exactly."""
    case = reference_fixture(65, 96, 64)
    case["experts"] = 5
    full = build(case).run(dev(case["x"])).cpu().numpy()
    parts = [build(case, ep_rank=r, ep_world=2, ep_interleaved=True).run(dev(case["x"])).cpu().numpy() for r in (0, 1)]
    assert_close(oracle.bf16_round(parts[0] + parts[1]), full, 0.002, "two-rank sum")
    for r in (0, 1):
        ids = np.arange(r, 5, 2)
        local = dict(case)
        for k in ("gu_blocks", "gu_scales", "gu_bias", "dn_blocks", "dn_scales", "dn_bias"):
            local[k] = case[k][ids]
        got = build(local, ep_rank=r, ep_world=2, ep_interleaved=True, expert_weights_sharded=True).run(dev(case["x"])).cpu().numpy()
        assert np.array_equal(got, parts[r])
    wide = synth.moe_layer(40, 64, 96, experts=8, topk=4, seed=3, bias_scale=0.1)
    full = build(wide).run(dev(wide["x"])).cpu().numpy()
    parts = [build(wide, ep_rank=r, ep_world=4).run(dev(wide["x"])).cpu().numpy() for r in range(4)]
    assert_close(oracle.bf16_round(sum(parts)), full, 0.002, "four-rank sum")
    _, sel, pr = oracle.moe_route(wide["x"], wide["router_w"], wide["router_b"], 8, 4)
    o = oracle.moe_experts(wide["x"], sel, pr, *oracle_args(wide), expert_lo=2, expert_hi=4, round_output=False)
    assert_close(parts[1], o, 0.002, "rank-1 partial vs oracle")


def test_rejects_bad_arguments():
    L = garnet_b200.lib()
    import ctypes
    sz = ctypes.c_size_t(0)
    opt = garnet_b200.MoeOptions(abi=1, struct_size=ctypes.sizeof(garnet_b200.MoeOptions), hidden=33, intermediate=32,
                                 experts=5, top_k=2, io_dtype=2, limit=7.0)
    assert L.garnet_b200_moe_workspace(ctypes.byref(opt), 1, ctypes.byref(sz)) == 1
    opt.hidden = 32
    opt.abi = 2
    assert L.garnet_b200_moe_workspace(ctypes.byref(opt), 1, ctypes.byref(sz)) == 1
    opt.abi = 1
    assert L.garnet_b200_moe_workspace(ctypes.byref(opt), 1, ctypes.byref(sz)) == 0 and sz.value > 0
    out = ctypes.c_void_p(None)
    assert L.garnet_b200_moe_create(ctypes.byref(opt), None, None, ctypes.byref(out)) == 1
    assert L.garnet_b200_moe_run(None, None, None, None, 0, 1, None) == 1


def test_rows_entry_point_and_combine_match_full_operator():
    """The expert-parallel building blocks (experts on already routed rows, then the
    weighted combine) give bit-for-bit what the one-call operator gives; with the
    experts split over two handles (contiguous blocks, as on two GPUs) as well."""
    case = synth.moe_layer(40, 96, 64, experts=8, topk=4, seed=5, bias_scale=0.1)
    x = dev(case["x"])
    full = build(case)
    y = full.run(x)
    _, sel, pr = full.route(x)
    slots = sel.reshape(-1)
    rows = x[torch.arange(slots.numel(), device="cuda") // 4]
    vals = full.run_rows(rows, slots)
    assert torch.equal(full.combine(vals, pr), y)
    # two owners: rank r holds experts [4r, 4r+4) and sees only its rows, in arrival order
    merged = torch.zeros_like(vals)
    for r in range(2):
        owner = build(case, ep_rank=r, ep_world=2)
        mine = torch.nonzero((slots // 4) == r).reshape(-1)
        perm = mine[torch.randperm(mine.numel(), device="cuda")]
        merged[perm] = owner.run_rows(rows[perm], slots[perm])
        assert owner.fault() == 0
    assert torch.equal(full.combine(merged, pr), y)
    # bf16 wire format is exact for the per-row values
    assert torch.equal(vals.bfloat16().float(), vals)


def test_block_scaled_path_at_every_size():
    """Small batches normally take the streaming kernel; GARNET_B200_MOE_MX=2 sends every
    size through the block-scaled tensor-core path.  The switch is read once per process,
    so the fixture and golden parity tests are re-run in a child process with it set."""
    import os
    import subprocess
    import sys
    if os.environ.get("GARNET_B200_MOE_MX") == "2":
        pytest.skip("already running with the block-scaled path forced")
    env = dict(os.environ, GARNET_B200_MOE_MX="2")
    here = os.path.dirname(os.path.abspath(__file__))
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.join(here, "test_moe_gpu.py"), "-m", "gpu", "-q", "-x",
                        "-k", "fixtures or golden or bf16_io or rows"], env=env, capture_output=True, text=True,
                       timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
