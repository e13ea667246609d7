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
from garnet_b200 import moe as moe_mod
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


@pytest.mark.parametrize("h,inter", [(32, 32), (96, 64), (2880, 64), (64, 2880), (480, 256)])
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
        # the second copy (15 KiB blocks of 240 rows + scale atoms of the block-scaled kernels)
        assert same(moe.dequantized(2, e).cpu().numpy(), eu) and same(moe.dequantized(3, e).cpu().numpy(), ed)


@pytest.mark.parametrize("tokens", [1, 3, 17, 65])
@pytest.mark.parametrize("h,inter", [(32, 32), (96, 64), (128, 64)])   # hidden 128: the tensor-core router's shapes
def test_reference_fixtures(tokens, h, inter):
    run_and_compare(reference_fixture(tokens, h, inter), 0.002)


@pytest.mark.parametrize("tokens", [9, 40, 200])
def test_tensor_core_router_on_synthetic_layers(tokens):
    """Above a decode batch the router runs on the tensor cores (hidden a multiple of 64) and one kernel adds its
    K ranges, picks the top k, counts the rows and writes the fp16 row copies: random layers, both io types,
    whole and expert-sharded."""
    case = synth.moe_layer(tokens, 128, 96, experts=16, topk=4, seed=tokens, bias_scale=0.1)
    tol = 0.002 if tokens * 4 <= 8 * 16 else 0.004   # more than 8 rows per expert: the block-scaled kernels' bound
    run_and_compare(case, tol)
    x = dev(case["x"])
    y32 = build(case).run(x)
    y16 = build(case, io_dtype=torch.bfloat16).run(x.bfloat16())
    assert torch.equal(y32.bfloat16(), y16)
    parts = [build(case, ep_rank=r, ep_world=4).run(x).cpu().numpy() for r in range(4)]
    assert_close(oracle.bf16_round(sum(parts)), y32.cpu().numpy(), tol, "four-rank sum")


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


@pytest.mark.parametrize("tokens", [1, 8, 32])
def test_gpt_oss_120b_layer_shape(tokens):
    case = synth.moe_layer(tokens, seed=tokens)
    run_and_compare(case, 1e-2, use_mass=True)


@pytest.mark.parametrize("tokens", [96, 200, 512])   # streaming kernel, near the crossover, block-scaled kernel
def test_gpt_oss_120b_layer_shape_sampled_tokens(tokens):
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
    # decode-sized batches take the router kernel's own bookkeeping (one token: a shortcut of its own)
    for tokens in (1, 2, 8):
        small = dict(wide)
        small["x"] = wide["x"][:tokens]
        full = build(small).run(dev(small["x"])).cpu().numpy()
        for world, inter in ((4, False), (2, True)):
            parts = [build(small, ep_rank=r, ep_world=world, ep_interleaved=inter).run(dev(small["x"])).cpu().numpy()
                     for r in range(world)]
            assert_close(oracle.bf16_round(sum(parts)), full, 0.002, f"{tokens} token(s), {world} ranks")
        _, sel, pr = oracle.moe_route(small["x"], small["router_w"], small["router_b"], 8, 4)
        o = oracle.moe_experts(small["x"], sel, pr, *oracle_args(small), expert_lo=2, expert_hi=4, round_output=False)
        assert_close(build(small, ep_rank=1, ep_world=4).run(dev(small["x"])).cpu().numpy(), o, 0.002, f"{tokens} token(s), rank-1 partial vs oracle")


def test_host_packer_bytes_equal_device_bytes_and_prepacked_handle_is_the_same_operator():
    """The reference checks that its host packer and its GPU repacker write the same bytes
    (kernel_parity.cpp:576-586, marlin_weight_pack.cpp:33-111).  Here: both layouts of both
    projections, then a handle that borrows the host-packed blobs gives bit-identical
    results, with few rows per expert and with many."""
    case = synth.moe_layer(96, hidden=160, inter=288, experts=6, topk=2, seed=5, bias_scale=0.1)   # 576 gate/up rows: 3 blocks of 240
    moe = build(case)
    blobs = []
    for layout in (moe_mod.LAYOUT_STREAM, moe_mod.LAYOUT_BLOCK):
        for which, (bk, sk) in enumerate((("gu_blocks", "gu_scales"), ("dn_blocks", "dn_scales"))):
            host = moe.pack_host(which, layout, case[bk], case[sk])
            device = moe.packed_view(which, layout).cpu().numpy()
            assert host.shape == device.shape and np.array_equal(host, device), (layout, which)
            blobs.append(dev(host))
    small = [dev(case[k]) for k in ("router_w", "router_b", "gu_bias", "dn_bias")]
    pre = garnet_b200.GptOssMoe(case["hidden"], case["inter"], case["experts"], case["topk"]).prepare_prepacked(*small, blobs)
    for tokens in (3, 96):
        x = dev(case["x"][:tokens])
        assert torch.equal(pre.run(x), moe.run(x))
    assert pre.fault() == 0
    for which in range(4):
        assert torch.equal(pre.dequantized(which, 5), moe.dequantized(which, 5))


def test_handles_that_hold_one_layout():
    """layouts = stream / block: one copy of the experts, every token count runs on it."""
    case = synth.moe_layer(80, hidden=128, inter=256, experts=4, topk=2, seed=6, bias_scale=0.1)
    for layout, missing in ((moe_mod.LAYOUT_STREAM, moe_mod.LAYOUT_BLOCK), (moe_mod.LAYOUT_BLOCK, moe_mod.LAYOUT_STREAM)):
        moe = build(case, layouts=layout)
        with pytest.raises(garnet_b200.GarnetB200Error):
            moe.packed_view(0, missing)
        for tokens in (2, 80):
            sub = dict(case, x=case["x"][:tokens])
            x = dev(sub["x"])
            y = moe.run(x).cpu().numpy()
            _, sel, pr = [t.cpu().numpy() for t in moe.route(x)]
            expect, mass = oracle.moe_experts(sub["x"], sel, pr, *oracle_args(sub), want_mass=True)
            # .004: the reference's bound for its tensor-core path (kernel_parity.cpp:714)
            assert_close(y, expect, 0.004, f"layout {layout}, {tokens} tokens", mass)
        assert moe.fault() == 0
    # the prepacked form with one layout takes only that layout's blobs
    moe = build(case, layouts=moe_mod.LAYOUT_BLOCK)
    blobs = [None, None] + [moe.packed_view(w, moe_mod.LAYOUT_BLOCK) for w in (0, 1)]
    small = [dev(case[k]) for k in ("router_w", "router_b", "gu_bias", "dn_bias")]
    pre = garnet_b200.GptOssMoe(case["hidden"], case["inter"], case["experts"], case["topk"],
                                layouts=moe_mod.LAYOUT_BLOCK).prepare_prepacked(*small, blobs)
    x = dev(case["x"])
    assert torch.equal(pre.run(x), moe.run(x))


@pytest.mark.parametrize("world", [2, 4])
def test_intermediate_axis_split(world):
    """The reference's inner tensor parallelism (gpt_oss_weight_shard.h:9-11; its test
    kernel_parity.cpp:674-709, tolerance .025): every rank keeps all experts and
    1/world of the intermediate channels, adds the down bias on rank 0 only and returns
    an unrounded partial sum.  A handle given the full tensors and one given the
    rank-local tensors (gathered on the host) are the same operator."""
    case = synth.moe_layer(70, hidden=96, inter=256, experts=5, topk=2, seed=9, bias_scale=0.1)
    x = dev(case["x"])
    full = build(case)
    y_full = full.run(x).cpu().numpy()
    _, sel, pr = [t.cpu().numpy() for t in full.route(x)]
    expect = oracle.moe_experts(case["x"], sel, pr, *oracle_args(case))
    for tokens in (2, 70):
        xs = x[:tokens]
        parts = []
        for r in range(world):
            moe = build(case, tp_rank=r, tp_world=world)
            parts.append(moe.run(xs).cpu().numpy())
            local = dict(case)
            for key, mode in (("gu_blocks", 1), ("gu_scales", 1), ("gu_bias", 1), ("dn_blocks", 2), ("dn_scales", 2), ("dn_bias", 3)):
                local[key] = moe_mod.gather_intermediate_shard(case[key], r, world, mode)
            pre = build(local, tp_rank=r, tp_world=world, tp_weights_sharded=True)
            assert np.array_equal(pre.run(xs).cpu().numpy(), parts[r])
            assert moe.fault() == 0
        total = oracle.bf16_round(np.sum(parts, axis=0, dtype=np.float32))
        assert_close(total, expect[:tokens], 0.025, f"sum of {world} partial sums, {tokens} tokens")
        assert_close(total, y_full[:tokens], 0.025, "against the unsplit operator")


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


def check_rows_in_two_halves(moe, case, rows, row_expert_dev, pick, what, expert_base=0):
    """Per-row values BEFORE the weighted sum, in the plain form |a - e| <= 1e-2 (1 + |e|), one
    projection at a time: the SwiGLU activations against the oracle's, then the down
    projection of the DEVICE's activations against the oracle's down projection of the
    same activations (so that a one-step difference in a bf16 rounding of an activation,
    which depends on the fp32 summation order, is not amplified 2880-fold); the two
    halves together are bit-for-bit what the one-call form returns."""
    hid = moe.run_rows_hidden(rows, row_expert_dev)
    vals = moe.run_rows(rows, row_expert_dev)
    torch.cuda.synchronize()
    assert moe.fault() == 0
    assert torch.equal(moe.run_rows_down(hid, row_expert_dev), vals)
    sel = torch.from_numpy(pick).cuda()
    experts = row_expert_dev[sel].cpu().numpy() - expert_base
    x_rows = rows[sel].float().cpu().numpy()
    h_dev = hid[sel].cpu().numpy()
    h_ref = oracle.moe_rows_hidden(x_rows, experts, case["gu_blocks"], case["gu_scales"], case["gu_bias"].reshape(-1),
                                   case["hidden"], case["inter"])
    # An activation is the end of a chain of six bf16 roundings (g, u, 1.702 g, the sigmoid,
    # the two products: gpt_oss_kernels.cu:786-789) fed by two 2880-term fp32 sums whose
    # order differs between any two implementations.  A sum that lands on the other side
    # of a rounding boundary moves g or u by one bf16 step (2^-8), and the chain can turn
    # that into a few steps of the result (d ln(g sigmoid(1.702 g)) / d ln g <= 1.3, plus one
    # step per later rounding that flips): the bound is 8 steps, nearly all values agree
    # to two steps, and most are identical.
    assert_close(h_dev, h_ref, 8 * 2.0 ** -8, what + ": activations")
    assert (np.abs(h_dev - h_ref) <= 2.0 ** -7 * np.abs(h_ref) + 1e-6).mean() >= 0.999
    assert (h_dev == h_ref).mean() >= 0.9
    v_ref = oracle.moe_rows_down(h_dev, experts, case["dn_blocks"], case["dn_scales"], case["dn_bias"].reshape(-1),
                                 case["hidden"], case["inter"])
    assert_close(vals[sel].cpu().numpy(), v_ref, 1e-2, what + ": per-row values")
    return vals


def positions_in_expert(slots_expert):
    """Position of every slot inside its expert's run of the stable slot order."""
    order = np.argsort(slots_expert, kind="stable")
    counts = np.bincount(slots_expert, minlength=slots_expert.max() + 1)
    starts = np.concatenate([[0], np.cumsum(counts)[:-1]])
    pos = np.empty_like(order)
    pos[order] = np.arange(order.size) - starts[slots_expert[order]]
    return pos, counts


def test_gpt_oss_120b_layer_at_4096_tokens_per_slot_values_and_output():
    """The configuration the MoE throughput is quoted on: 4096 tokens, 128 experts, top-4
    (128 +- 11 rows per expert: many experts own a full 128-row tile and a nearly empty
    second one).  Per-slot values BEFORE the weighted sum, in the plain form
    |a - e| <= 1e-2 (1 + |e|), on slots that include second-tile rows; every output column
    (hence every 240-row weight tile, the last one too) is compared.  Then sampled outputs."""
    tokens = 4096
    case = synth.moe_layer(tokens, seed=11, bias_scale=0.05)
    moe = build(case, io_dtype=torch.bfloat16)
    x = dev(case["x"]).bfloat16()
    _, sel_t, pr_t = moe.route(x)
    sel, pr = sel_t.cpu().numpy(), pr_t.cpu().numpy()
    slots = sel.reshape(-1)
    rows = x[torch.arange(slots.size, device="cuda") // 4]
    pos, counts = positions_in_expert(slots)
    assert counts.max() > 128 and counts.min() > 0
    rng = np.random.default_rng(1)
    second_tile = np.flatnonzero(pos >= 128)
    last_of_expert = np.flatnonzero(pos == counts[slots] - 1)
    pick = np.unique(np.concatenate([rng.choice(second_tile, min(32, second_tile.size), replace=False),
                                     rng.choice(last_of_expert, 16, replace=False),
                                     rng.choice(slots.size, 24, replace=False)]))
    assert (pos[pick] >= 128).sum() >= 16
    vals = check_rows_in_two_halves(moe, case, rows, sel_t.reshape(-1), pick, "4096 tokens")
    # the one-call operator gives the combine of exactly these values
    y = moe.run(x)
    assert torch.equal(moe.combine(vals, pr_t), y)
    tok = rng.choice(tokens, 16, replace=False)
    exp_y, mass = oracle.moe_experts(case["x"][tok], sel[tok], pr[tok], *oracle_args(case), want_mass=True)
    assert_close(y[torch.from_numpy(tok).cuda()].float().cpu().numpy(), exp_y, 1e-2, "outputs at 4096 tokens", mass)


def test_zipf_routed_rows_on_the_busiest_of_eight_ranks():
    """The expert-parallel configuration on one GPU: 8192 tokens routed with Zipf(1.1)
    popularity; the rank that owns the most popular block of 16 experts receives several
    times the mean load (experts with thousands of rows beside experts with none)."""
    tokens, world = 8192, 8
    case = synth.moe_layer(tokens, seed=12, zipf_s=1.1, bias_scale=0.05)
    _, sel, _ = oracle.moe_route(case["x"], case["router_w"], case["router_b"], 128, 4)
    slots = sel.reshape(-1)
    per = 128 // world
    load = np.bincount(slots // per, minlength=world)
    rank = int(load.argmax())
    assert load[rank] > 1.5 * load.mean()
    local = dict(case)
    for k in ("gu_blocks", "gu_scales", "gu_bias", "dn_blocks", "dn_scales", "dn_bias"):
        local[k] = case[k][rank * per:(rank + 1) * per]
    owner = build(local, ep_rank=rank, ep_world=world, expert_weights_sharded=True, io_dtype=torch.bfloat16)
    mine = np.flatnonzero(slots // per == rank)
    rng = np.random.default_rng(2)
    mine = mine[rng.permutation(mine.size)]                         # arrival order of an exchange
    rows = dev(case["x"][mine // 4]).bfloat16()
    counts = np.bincount(slots[mine] - rank * per, minlength=per)
    assert counts.max() > 1000
    pos, _ = positions_in_expert(slots[mine])
    pick = np.unique(np.concatenate([rng.choice(mine.size, 40, replace=False), np.flatnonzero(pos >= 1024)[:8],
                                     np.flatnonzero(pos == 0)]))
    check_rows_in_two_halves(owner, local, rows, dev(slots[mine].astype(np.int32)), pick, "zipf rows", expert_base=rank * per)


def e4m3_decode(codes):
    c = codes.astype(np.int32)
    sign = np.where(c & 0x80, -1.0, 1.0)
    e, m = (c >> 3) & 15, c & 7
    mag = np.where(e == 0, m / 8.0 * 2.0 ** -6, (1 + m / 8.0) * 2.0 ** (e - 7.0))
    return np.where((c & 0x7f) == 0x7f, np.nan, sign * mag)


def test_activation_split_into_two_e4m3_pieces():
    """x = (hi + lo) * 2^(s - 127): exact within 2^-9 of the block's largest magnitude, to
    2^-17 of it otherwise; adversarial blocks: one huge value among tiny ones, all zeros,
    bf16 subnormals, the largest finite bf16, signed zeros; an infinity or a NaN makes
    the block's scale NaN (the reference, which keeps activations in bf16, produces an
    infinity or a NaN from them as well)."""
    rng = np.random.default_rng(3)
    k = 32 * 12
    x = oracle.bf16_round(rng.normal(0, 1, size=(64, k)).astype(np.float32))
    x[0, :32] = 0.0
    x[1, :32] = np.float32(2.0) ** -20 * rng.normal(size=32); x[1, 5] = 3.0e4        # one huge, many tiny
    x[2, :32] = np.float32(2.0) ** -130 * np.arange(32)                               # bf16 subnormals
    x[3, :32] = np.float32(3.3895314e38)                                              # largest finite bf16
    x[4, :32] = -0.0
    x[5, :64] = rng.normal(size=64) * np.float32(2.0) ** 60
    x[6, 32:64] = rng.normal(size=32); x[6, 40] = np.inf
    x[7, 64:96] = rng.normal(size=32); x[7, 70] = np.nan
    x = oracle.bf16_round(x)
    rows = x.shape[0]
    xd = torch.from_numpy(oracle.bf16_bits(x).view(np.int16)).view(torch.bfloat16).reshape(rows, k).cuda()
    hi = torch.empty(rows, k, dtype=torch.uint8, device="cuda")
    lo = torch.empty_like(hi)
    sc = torch.empty(rows, k // 32, dtype=torch.uint8, device="cuda")
    from garnet_b200._lib import check
    check(garnet_b200.lib().garnet_b200_mx_split_rows(xd.data_ptr(), rows, k, hi.data_ptr(), lo.data_ptr(), sc.data_ptr(), None))
    torch.cuda.synchronize()
    h, l, s = e4m3_decode(hi.cpu().numpy()), e4m3_decode(lo.cpu().numpy()), sc.cpu().numpy().astype(np.int32)
    scale = np.repeat(np.where(s == 255, np.nan, 2.0 ** (s - 127.0)), 32, axis=1)
    back = (h + l) * scale
    blocks = x.astype(np.float64).reshape(rows, k // 32, 32)
    amax = np.repeat(np.abs(blocks).max(axis=2), 32, axis=1)
    finite = np.isfinite(amax)
    assert (s[6, 1] == 255) and (s[7, 2] == 255) and np.isnan(back[6, 32:64]).all() and np.isnan(back[7, 64:96]).all()
    assert np.isfinite(back[finite]).all()
    err = np.abs(back - x.astype(np.float64))
    # blocks whose scale byte was clamped at 1 (subnormal range) keep absolute accuracy 2^-126 * 2^-9
    floor = 2.0 ** -140
    assert (err[finite] <= amax[finite] * 2.0 ** -17 + floor).all()
    near = finite & (np.abs(x) >= amax * 2.0 ** -9) & (amax >= 2.0 ** -100)
    assert (back[near] == x[near]).all()
    assert (back[0, :32] == 0).all() and (back[4, :32] == 0).all()


def test_no_alloc_limit_and_argument_checks():
    """Largest token count the built-in scratch holds at the gpt-oss-120b widths, and
    misaligned pointers: rejected before any launch."""
    import ctypes
    case = synth.moe_layer(4, 64, 64, experts=8, topk=4, seed=1)
    moe = build(case, io_dtype=torch.bfloat16)
    L = garnet_b200.lib()
    x = torch.zeros(8, 64, dtype=torch.bfloat16, device="cuda")
    y = torch.empty_like(x)
    ws = torch.empty(moe.workspace_bytes(4), dtype=torch.uint8, device="cuda")
    assert L.garnet_b200_moe_run(moe._h, x.data_ptr() + 2, y.data_ptr(), ws.data_ptr(), ws.numel(), 4, None) == 1
    assert b"aligned" in L.garnet_b200_last_error()
    assert L.garnet_b200_moe_run(moe._h, x.data_ptr(), y.data_ptr() + 8, ws.data_ptr(), ws.numel(), 4, None) == 1
    assert L.garnet_b200_moe_run_static(moe._h, x.data_ptr() + 4, y.data_ptr(), 4, None) == 1
    assert L.garnet_b200_moe_run_static(moe._h, x.data_ptr(), y.data_ptr(), 2 ** 31 - 1, None) == 1   # returns at once
    vals = torch.empty(16, 64, dtype=torch.float32, device="cuda")
    ex = torch.zeros(16, dtype=torch.int32, device="cuda")
    assert L.garnet_b200_moe_run_rows(moe._h, x.data_ptr() + 2, ex.data_ptr(), 8, vals.data_ptr(), ws.data_ptr(), ws.numel(), None) == 1
    assert L.garnet_b200_moe_combine(moe._h, vals.data_ptr() + 4, vals.data_ptr(), y.data_ptr(), 2, None) == 1
    # the documented limit at the gpt-oss-120b layer widths
    sz = ctypes.c_size_t(0)
    opt = garnet_b200.MoeOptions(abi=1, struct_size=ctypes.sizeof(garnet_b200.MoeOptions), hidden=2880, intermediate=2880,
                                 experts=128, top_k=4, io_dtype=1, limit=7.0)
    fits = lambda t: L.garnet_b200_moe_workspace(ctypes.byref(opt), t, ctypes.byref(sz)) == 0 and sz.value <= (8 << 20)
    assert fits(NO_ALLOC_TOKENS_120B) and not fits(NO_ALLOC_TOKENS_120B + 1)


NO_ALLOC_TOKENS_120B = 111


def _rerun_with_switch(value, selection):
    import subprocess
    import sys
    if os.environ.get("GARNET_B200_MOE_MX") == value:
        pytest.skip("already running with this switch")
    env = dict(os.environ, GARNET_B200_MOE_MX=value)
    here = os.path.dirname(os.path.abspath(__file__))
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.join(here, "test_moe_gpu.py"), "-m", "gpu", "-q", "-x",
                        "-k", selection], env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]


def test_block_scaled_path_at_every_size():
    """Small batches normally take the streaming kernel; GARNET_B200_MOE_MX=2 sends every
    size through the block-scaled tensor-core path.  The switch is read once per process,
    so the fixture and golden parity tests are re-run in a child process with it set."""
    _rerun_with_switch("2", "fixtures or golden or bf16_io or rows_entry")


def test_streaming_path_at_every_size():
    """GARNET_B200_MOE_MX=0 keeps every size on the streaming kernel: the path a handle
    takes when the block-scaled copy cannot be built (no tensor-map encoder in the driver)."""
    _rerun_with_switch("0", "fixtures or golden or bf16_io or rows_entry")


# ---------------------------------------------------- against the reference's own GPU kernels

def _ref_gpu():
    from oracle import ref_gpu
    if not ref_gpu.available():
        pytest.skip("oracle/_ref/libgarnet_ref_gpu.so has not been built (make -C oracle ref_gpu REF=...)")
    return ref_gpu


@pytest.mark.parametrize("tokens", [1, 3, 17, 65])
def test_against_the_reference_gpu_moe_on_its_own_fixtures(tokens):
    """The reference's GPU kernels (compiled unchanged from its sources) on the closed-form inputs of
    its own parity test (kernel_parity.cpp:610-652): RunGptOssMoe - the scalar path below 16 tokens,
    the grouped WMMA path from 16 - against this operator and against the CPU oracle, each within the
    reference's bound .002; and the production Marlin GEMM (8 tokens at most by default) within its .004."""
    ref_gpu = _ref_gpu()
    case = reference_fixture(tokens, 96, 64)
    ops = [dev(case[k]) for k in ("router_w", "router_b", "gu_blocks", "gu_scales", "gu_bias", "dn_blocks", "dn_scales", "dn_bias")]
    ref = ref_gpu.RefMoe(case["hidden"], case["inter"], case["experts"], case["topk"], ops)
    x = dev(case["x"])
    rc, y_ref = ref.run(x)
    torch.cuda.synchronize()
    assert rc == 0
    mine = build(case).run(x).cpu().numpy()
    y_ref = y_ref.cpu().numpy()
    expect = oracle.moe_forward(case["x"], case["router_w"], case["router_b"], *oracle_args(case))[0]
    assert_close(y_ref, expect, 0.002, "reference GPU vs oracle")
    assert_close(mine, y_ref, 0.002, "this operator vs reference GPU")
    if tokens <= 8:
        rc, y_m = ref.run_marlin(x)
        torch.cuda.synchronize()
        assert rc == 0
        assert_close(mine, y_m.cpu().numpy(), 0.004, "this operator vs reference Marlin")
    ref.close()


def test_against_the_reference_gpu_moe_at_the_gpt_oss_120b_shape():
    """Decode-sized batches of the benchmark's layer (2880 x 2880, 128 experts, top-4): this operator
    against the reference's scalar kernels and its Marlin GEMM on the same synthetic tensors, for the
    tokens whose routing agrees (a router logit may round the other way on either side), at the
    benchmark's bound 1e-2 judged against the scale of the summands."""
    ref_gpu = _ref_gpu()
    case = synth.moe_layer(8, seed=41)
    ops = [dev(case[k]) for k in ("router_w", "router_b", "gu_blocks", "gu_scales", "gu_bias", "dn_blocks", "dn_scales", "dn_bias")]
    ref = ref_gpu.RefMoe(2880, 2880, 128, 4, ops)
    x = dev(case["x"])
    moe = build(case)
    mine = moe.run(x).cpu().numpy()
    _, sel, pr = [t.cpu().numpy() for t in moe.route(x)]
    expect, mass = oracle.moe_experts(case["x"], sel, pr, *oracle_args(case), want_mass=True)
    _, o_sel, _ = oracle.moe_route(case["x"], case["router_w"], case["router_b"], 128, 4)
    same = (sel == o_sel).all(axis=1)
    assert same.sum() >= 6
    for name, fn, tol in (("RunGptOssMoe", ref.run, 1e-2), ("GptOssMarlin", ref.run_marlin, 1e-2)):
        rc, y = fn(x)
        torch.cuda.synchronize()
        assert rc == 0, name
        y = y.cpu().numpy()
        assert_close(y[same], expect[same], tol, f"{name} vs oracle", mass[same])
        assert_close(mine[same], y[same], tol, f"this operator vs {name}", mass[same])
    ref.close()
