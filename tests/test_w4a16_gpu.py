"""Parity of the int4 linear on the GPU, through the C ABI, against the CPU
oracle: bit-exact repack and dequantisation, GEMM outputs within 1e-2 in the
reference's error form |a - e| <= tol * (1 + |e|) (test2026/gpt_oss/kernel_parity.cpp:46-57)
of the fp64-accumulated exact product (the tolerance the specification names),
and far tighter in practice (checked too)."""
import os

import numpy as np
import pytest
import torch

import garnet_b200
import oracle
from garnet_b200 import synth

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
TOL = 1e-2


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.view(dtype)


def bf16_tensor(bits):
    return dev(bits.view(np.int16), torch.bfloat16)


def make_linear(case, n, k, group=128, **kw):
    lin = garnet_b200.W4A16Linear()
    scales = bf16_tensor(case["scales_bits"]).reshape(n, k // group)
    return lin.prepare(dev(case["nibbles"]), scales, n, k, group, **kw)


def check_close(y_dev, y64, tol=TOL, rounded_weights=False):
    y = y_dev.float().cpu().numpy().astype(np.float64)
    err = np.abs(y - y64)
    assert np.isfinite(y).all()
    assert (err <= tol * (1 + np.abs(y64))).all(), float((err / (1 + np.abs(y64))).max())
    # in practice the result is the correctly rounded bf16 of the exact sum, give or
    # take one ulp, plus an absolute term far below the row's output scale (up to 16
    # rows the activations enter as 15-bit block fixed point per 128 columns: exact
    # for values within 2^-6 of the block's maximum, 2^-15 of that maximum otherwise)
    ref = oracle.bf16_round(y64.astype(np.float32)).astype(np.float64)
    ulp = np.maximum(np.abs(ref), 2.0 ** -120) * 2.0 ** -7
    rms = np.sqrt((y64 ** 2).mean(axis=1, keepdims=True))
    # Above 16 rows the tensor-core tile kernel multiplies by w = bf16(q * s): each
    # weight carries one bf16 rounding (up to 2^-9 relative), which shows as up to
    # ~1e-2 of the row's output scale on individual outputs (the kernel reproduces
    # x . bf16(q*s) to the last bit; checked below where that model is passed in).
    slack = 2.5e-2 if rounded_weights else 2e-4
    assert (np.abs(y - ref) <= 1.01 * ulp + slack * rms + 1e-30).all()


@pytest.mark.parametrize("n,k,group", [(128, 128, 128), (200, 256, 128), (1024, 2048, 128), (256, 512, 256)])
def test_device_repack_equals_host_packer_and_dequant_is_bit_exact(n, k, group):
    case = synth.int4_linear(n, k, 1, group, seed=n + k)
    lin = make_linear(case, n, k, group)
    deq = lin.dequantized().cpu().numpy()
    expect = oracle.int4_dequant(case["nibbles"], case["scales_f32"], n, k, group)
    assert np.array_equal(deq.view(np.uint32), expect.view(np.uint32))
    # host-packed bytes, bound without copying, decode to the same matrix
    packed = garnet_b200.pack_host(torch.from_numpy(case["nibbles"]),
                                   torch.from_numpy(case["scales_bits"].view(np.int16)).view(torch.bfloat16).reshape(n, -1),
                                   n, k, group).cuda()
    view = garnet_b200.W4A16Linear().bind_packed(packed, torch.bfloat16, n, k, group)
    assert torch.equal(view.dequantized(), lin.dequantized())
    x = bf16_tensor(case["x_bits"])
    assert torch.equal(view.forward(x), lin.forward(x))


@pytest.mark.parametrize("m", [1, 2, 3, 8, 9, 16, 17, 40])
@pytest.mark.parametrize("n,k", [(256, 256), (200, 512), (2048, 2048), (2048, 6144), (1024, 2048)])
def test_linear_matches_exact_oracle(n, k, m):
    case = synth.int4_linear(n, k, m, seed=17 * m + n)
    lin = make_linear(case, n, k)
    y = lin.forward(bf16_tensor(case["x_bits"]).reshape(m, k))
    torch.cuda.synchronize()
    assert lin.fault() == 0
    _, y64 = oracle.w4a16_exact(case["nibbles"], case["scales_f32"], n, k, 128, case["x_f32"])
    # the tile kernel (weights rounded once to bf16) takes more than 16 rows, and more than 8
    # rows of a K above 4096: that many quantised rows do not fit the streaming kernel's
    # shared memory beside its ring
    check_close(y, y64, rounded_weights=m > 16 or (m > 8 and k > 4096))


@pytest.mark.parametrize("m", [33, 64, 130, 256, 300])
@pytest.mark.parametrize("n,k", [(384, 256), (6144, 2048), (2048, 6144), (200, 512)])
def test_linear_tensor_core_tiles(n, k, m):
    """Batches above 16 rows: 128- and 256-row weight tiles, partial batch tiles,
    several batch tiles, rows that are not a multiple of 128."""
    case = synth.int4_linear(n, k, m, seed=m + n + k)
    lin = make_linear(case, n, k)
    y = lin.forward(bf16_tensor(case["x_bits"]).reshape(m, k))
    torch.cuda.synchronize()
    assert lin.fault() == 0
    y64 = oracle.w4a16_blas(case["nibbles"], case["scales_f32"], n, k, 128, case["x_f32"])
    check_close(y, y64, rounded_weights=True)
    # against the same product with weights rounded once to bf16, the result is the
    # correctly rounded bf16 value up to fp32 accumulation noise
    wq = oracle.bf16_round(oracle.int4_dequant(case["nibbles"], case["scales_f32"], n, k, 128)).astype(np.float64)
    check_close(y, case["x_f32"].astype(np.float64) @ wq.T)


def test_tile_kernel_with_and_without_k_slices():
    """More than 16 rows on a small matrix: with the workspace garnet_b200_w4a16_workspace asks
    for, K is cut into slices whose fp32 partial sums are added in slice order; without one K
    stays whole.  Both are the same product; repeated calls give the same bits."""
    n, k, m = 1024, 2048, 64
    case = synth.int4_linear(n, k, m, seed=91)
    lin = make_linear(case, n, k)
    assert lin.workspace_bytes(m) > 0 and lin.workspace_bytes(16) == 0
    x = bf16_tensor(case["x_bits"]).reshape(m, k)
    sliced = lin.forward(x)
    again = lin.forward(x)
    whole = torch.empty_like(sliced)
    from garnet_b200._lib import check
    check(garnet_b200.lib().garnet_b200_w4a16_run(lin._h, x.data_ptr(), whole.data_ptr(), m, None, 0, 0, None))
    torch.cuda.synchronize()
    assert lin.fault() == 0 and torch.equal(sliced, again)
    y64 = oracle.w4a16_blas(case["nibbles"], case["scales_f32"], n, k, 128, case["x_f32"])
    check_close(sliced, y64, rounded_weights=True)
    check_close(whole, y64, rounded_weights=True)


def test_baseline_config_gate_proj_m1():
    """x[1,2048] ~ N(0,1), W [6144,2048] codes U[-8,7], scales |N(0,.02)|/7, seed 0."""
    n, k = 6144, 2048
    case = synth.int4_linear(n, k, 1, seed=0)
    lin = make_linear(case, n, k)
    x = bf16_tensor(case["x_bits"]).reshape(1, k)
    y1 = lin.forward(x)
    y2 = lin.forward(x)
    assert torch.equal(y1, y2)          # deterministic: K slices are reduced in a fixed order
    _, y64 = oracle.w4a16_exact(case["nibbles"], case["scales_f32"], n, k, 128, case["x_f32"])
    check_close(y1, y64)
    # the reference CPU operator quantises activations to int8 per group, so it is
    # itself only an approximation of this product; it must still land close by
    q4q8 = oracle.q4q8_forward(case["nibbles"], case["scales_f32"], n, k, 128, case["x_f32"][0])
    assert (np.abs(q4q8 - y64[0]) <= 5e-2 * (1 + np.abs(y64[0]))).all()
    assert (np.abs(q4q8 - y1.float().cpu().numpy()[0]) <= 5e-2 * (1 + np.abs(q4q8))).all()


def test_lm_head_slice_and_n_sharding():
    n, k, m = 151936 // 8, 2048, 4    # one eighth of the vocabulary: 18992 rows, not a multiple of 128
    case = synth.int4_linear(n, k, m, seed=5)
    x = bf16_tensor(case["x_bits"]).reshape(m, k)
    full = make_linear(case, n, k).forward(x)
    y64 = oracle.w4a16_blas(case["nibbles"], case["scales_f32"], n, k, 128, case["x_f32"])
    check_close(full, y64)
    for world in (2, 4):
        parts = [make_linear(case, n, k, shard_rank=r, shard_world=world).forward(x) for r in range(world)]
        assert torch.equal(torch.cat(parts, dim=1), full)


def test_fp16_scales_are_used_unrounded():
    n, k = 256, 256
    case = synth.int4_linear(n, k, 2, seed=3)
    s16 = (case["scales_f32"] * np.float32(1.0009765625)).astype(np.float16)   # not bf16-representable
    lin = garnet_b200.W4A16Linear().prepare(dev(case["nibbles"]), dev(s16), n, k)
    expect = oracle.int4_dequant(case["nibbles"], s16.astype(np.float32), n, k, 128)
    assert np.array_equal(lin.dequantized().cpu().numpy(), expect)
    y = lin.forward(bf16_tensor(case["x_bits"]).reshape(2, k))
    _, y64 = oracle.w4a16_exact(case["nibbles"], s16.astype(np.float32), n, k, 128, case["x_f32"])
    check_close(y, y64)


def test_edge_values():
    n, k = 128, 256
    case = synth.int4_linear(n, k, 3, seed=9)
    x = case["x_f32"].copy()
    x[0] = 0.0                                   # all-zero row
    x[1, :] = np.float32(2.0) ** 100              # large magnitudes stay finite in fp32
    case["scales_f32"][:] = oracle.bf16_round(np.float32(2.0) ** -110 * np.ones_like(case["scales_f32"]))
    case["scales_bits"] = oracle.bf16_bits(case["scales_f32"])
    lin = make_linear(case, n, k)
    y = lin.forward(bf16_tensor(oracle.bf16_bits(x)).reshape(3, k))
    _, y64 = oracle.w4a16_exact(case["nibbles"], case["scales_f32"], n, k, 128, x)
    assert (y[0] == 0).all()
    check_close(y, y64)


@pytest.mark.parametrize("scale_dtype,kind", [(torch.bfloat16, "bf16"), (torch.float16, "fp16")])
@pytest.mark.parametrize("src_dtype", [torch.float32, torch.bfloat16])
def test_device_quantizer_matches_reference_arithmetic(scale_dtype, kind, src_dtype):
    rng = np.random.default_rng(11)
    w = oracle.bf16_round(rng.normal(0, 0.05, size=(96, 512)).astype(np.float32))
    w[3, :128] = 0.0                              # degenerate group -> scale 1
    nib, sc = garnet_b200.quantize_int4(dev(w).to(src_dtype), 128, scale_dtype)
    p, s, _ = oracle.int4_quantize(w, 128, kind)
    assert np.array_equal(nib.cpu().numpy(), p)
    assert np.array_equal(sc.cpu().view(torch.int16).numpy().view(np.uint16), s)


def test_golden_reference_artifact():
    """The reference's own quantized artifact and its CPU operator output
    (tests/golden/int4_ref.npz, produced by the compiled reference sources)."""
    g = np.load(os.path.join(GOLD, "int4_ref.npz"))
    n, k = 48, 512
    s16 = g["rand_scales_fp16"].view(np.float16)
    lin = garnet_b200.W4A16Linear().prepare(dev(g["rand_packed"]), dev(s16), n, k)
    x = g["rand_x"]
    y = lin.forward(bf16_tensor(oracle.bf16_bits(x)).reshape(1, k)).float().cpu().numpy()[0]
    _, y64 = oracle.w4a16_exact(g["rand_packed"], s16.astype(np.float32), n, k, 128, x)
    check_close(torch.from_numpy(y)[None], y64)
    ref_cpu = g["rand_y_q4q8"]                    # Q4Q8Linear with bf16-rounded scales
    assert (np.abs(y - ref_cpu) <= TOL * (1 + np.abs(ref_cpu))).all()


def test_host_buffer_entry_point():
    n, k, m = 2048, 2048, 5
    case = synth.int4_linear(n, k, m, seed=21)
    lin = make_linear(case, n, k)
    xh = torch.from_numpy(case["x_bits"].view(np.int16)).view(torch.bfloat16).reshape(m, k).pin_memory()
    yh = torch.empty(m, n, dtype=torch.bfloat16).pin_memory()
    lin.forward_host(xh, yh)
    expected = lin.forward(xh.cuda()).cpu()
    assert torch.equal(yh, expected)
    # pageable (not pinned) output: the staged-copy route
    y_pageable = torch.empty(m, n, dtype=torch.bfloat16)
    lin.forward_host(xh, y_pageable)
    assert torch.equal(y_pageable, expected)
    # asynchronous form: complete after the stream is synchronised; batch above 16 (tile kernel)
    m2 = 40
    case2 = synth.int4_linear(n, k, m2, seed=22)
    xh2 = torch.from_numpy(case2["x_bits"].view(np.int16)).view(torch.bfloat16).reshape(m2, k).pin_memory()
    yh2 = torch.zeros(m2, n, dtype=torch.bfloat16).pin_memory()
    lin.forward_host_async(xh2, yh2)
    torch.cuda.synchronize()
    assert torch.equal(yh2, lin.forward(xh2.cuda()).cpu())
    # batched form: two linears reading the same host buffer, then one reading another
    case3 = synth.int4_linear(1024, k, m, seed=23)
    lin3 = make_linear(case3, 1024, k)
    ya = torch.zeros(m, n, dtype=torch.bfloat16).pin_memory()
    yb = torch.zeros(m, 1024, dtype=torch.bfloat16).pin_memory()
    yc = torch.zeros(m2, n, dtype=torch.bfloat16).pin_memory()
    garnet_b200.HostBatch([(lin, xh, ya), (lin3, xh, yb), (lin, xh2, yc)]).run()
    torch.cuda.synchronize()
    assert torch.equal(ya, expected)
    assert torch.equal(yb, lin3.forward(xh.cuda()).cpu())
    assert torch.equal(yc, yh2)


def test_run_rejects_bad_arguments():
    case = synth.int4_linear(128, 128, 1, seed=1)
    lin = make_linear(case, 128, 128)
    x = bf16_tensor(case["x_bits"])
    with pytest.raises(garnet_b200.GarnetB200Error):
        lin.forward(x, workspace=torch.empty(0, dtype=torch.uint8, device="cuda")) if lin.workspace_bytes(1) else (_ for _ in ()).throw(garnet_b200.GarnetB200Error(1, "no workspace needed"))
    with pytest.raises(garnet_b200.GarnetB200Error):
        garnet_b200.W4A16Linear().prepare(dev(case["nibbles"]), bf16_tensor(case["scales_bits"]), 128, 128, 64)


@pytest.mark.parametrize("m", [1, 5, 16, 40])
def test_grouped_launch_equals_separate_launches(m):
    """q/k/v-style group: three linears of different N sharing one x in one launch."""
    k = 2048
    shapes = [2048, 1024, 1000]
    cases = [synth.int4_linear(n, k, m, seed=100 + i) for i, n in enumerate(shapes)]
    lins = [make_linear(c, n, k) for c, n in zip(cases, shapes)]
    x = bf16_tensor(cases[0]["x_bits"]).reshape(m, k)
    separate = [lin.forward(x) for lin in lins]
    grouped = garnet_b200.forward_group(lins, x)
    # Up to 16 rows the fp32 sum over K follows one fixed tree however the launch splits
    # K among warps, so a group gives the bits of the separate launches; above 16 rows
    # the group is separate launches of the tile kernel anyway.
    for a, b in zip(separate, grouped):
        if m <= 16:
            assert torch.equal(a, b)
        else:
            # the tile kernel cuts K into slices when it is given a workspace (the separate calls)
            # and keeps K whole when it is not (the group): the fp32 sums associate differently
            a32, b32 = a.float(), b.float()
            step = torch.maximum(a32.abs(), b32.abs()) * 2.0 ** -7 + 1e-4 * a32.pow(2).mean().sqrt()
            assert bool(((a32 - b32).abs() <= step).all())
    assert all(lin.fault() == 0 for lin in lins)


def test_linear_list_equals_separate_runs_and_honours_dependencies():
    """One persistent launch over a list: independent linears give the bits of their own
    runs; a chain in which each linear reads the previous output gives the bits of
    running them one after the other (garnet_b200_w4a16_list_*)."""
    k = 2048
    shapes = [2048, 1024, 1024, 2048]
    cases = [synth.int4_linear(n, k, 1, seed=300 + i) for i, n in enumerate(shapes)]
    lins = [make_linear(c, n, k) for c, n in zip(cases, shapes)]
    for m in (1, 3, 8, 16):
        x = bf16_tensor(synth.int4_linear(16, k, m, seed=41)["x_bits"]).reshape(m, k)
        outs = [torch.zeros(m, n, dtype=torch.bfloat16, device="cuda") for n in shapes]
        lst = garnet_b200.LinearList([(lin, x, y) for lin, y in zip(lins, outs)], m=m)
        for _ in range(2):
            for y in outs:
                y.zero_()
            lst.run()
            torch.cuda.synchronize()
            assert lst.fault() == 0
            for lin, y in zip(lins, outs):
                assert torch.equal(y, lin.forward(x))
    # a chain of square linears and a gate -> down pair: true data dependencies
    sq = [make_linear(synth.int4_linear(k, k, 1, seed=400 + i), k, k) for i in range(5)]
    gate = make_linear(synth.int4_linear(6144, k, 1, seed=410), 6144, k)
    down = make_linear(synth.int4_linear(k, 6144, 1, seed=411), k, 6144)
    chain = sq + [gate, down]
    for m in (1, 4):
        bufs = [bf16_tensor(synth.int4_linear(16, k, m, seed=42)["x_bits"]).reshape(m, k) * 8]
        for lin in chain:
            bufs.append(torch.zeros(m, lin.n, dtype=torch.bfloat16, device="cuda"))
        lst = garnet_b200.LinearList([(lin, bufs[i], bufs[i + 1], i - 1) for i, lin in enumerate(chain)], m=m)
        for rep in range(3):                  # the run tag changes from run to run
            for b in bufs[1:]:
                b.zero_()
            lst.run()
            torch.cuda.synchronize()
            assert lst.fault() == 0
            cur = bufs[0]
            for i, lin in enumerate(chain):
                cur = lin.forward(cur)
                assert torch.equal(cur, bufs[i + 1]), (m, rep, i)


def test_linear_list_rejects_bad_dependencies():
    k = 256
    a = make_linear(synth.int4_linear(256, k, 1, seed=1), 256, k)
    b = make_linear(synth.int4_linear(128, k, 1, seed=2), 128, k)
    x = torch.zeros(1, k, dtype=torch.bfloat16, device="cuda")
    y1 = torch.zeros(1, 256, dtype=torch.bfloat16, device="cuda")
    y2 = torch.zeros(1, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(garnet_b200.GarnetB200Error):       # depends on a later linear
        garnet_b200.LinearList([(a, x, y1, 1), (b, y1, y2, -1)])
    with pytest.raises(garnet_b200.GarnetB200Error):       # x is not the output it claims to depend on
        garnet_b200.LinearList([(a, x, y1, -1), (b, x, y2, 0)])
    with pytest.raises(garnet_b200.GarnetB200Error):       # batch too large for a list
        garnet_b200.LinearList([(a, x, y1, -1)], m=64)
    garnet_b200.LinearList([(a, x, y1, -1), (b, y1, y2, 0)]).run()
    torch.cuda.synchronize()


def test_bounded_device_wait_reports_a_fault_and_leaves_the_context_usable():
    """A wait whose partner never arrives ends after its limit with DEVICE_FAULT (no
    hang, no trap); the next ordinary call works."""
    from garnet_b200 import _lib
    L = garnet_b200.lib()
    rc = L.garnet_b200_selftest_bounded_wait(20, None)
    assert rc == _lib.DEVICE_FAULT
    assert b"gave up" in L.garnet_b200_last_error()
    case = synth.int4_linear(128, 128, 2, seed=77)
    lin = make_linear(case, 128, 128)
    y = lin.forward(bf16_tensor(case["x_bits"]).reshape(2, 128))
    _, y64 = oracle.w4a16_exact(case["nibbles"], case["scales_f32"], 128, 128, 128, case["x_f32"])
    check_close(y, y64)
    assert lin.fault() == 0


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("m", [1, 5, 40])
def test_k_sharded_linear_partial_sums(world, m):
    """Row-parallel split (the reference slices the weight along axis 1,
    trt_builder.cpp:7347-7359): every rank holds K / world columns and returns bf16 partial
    sums; each rank's weights are exactly its columns of the full matrix, and the partial sums,
    added in fp32 in rank order and rounded once (the wire rule of the all-reduce), meet the
    exact result within the operator's tolerance plus the roundings of the partial sums."""
    n, k = 384, 2048
    case = synth.int4_linear(n, k, m, seed=m + world)
    full = make_linear(case, n, k)
    deq = full.dequantized()
    x = bf16_tensor(case["x_bits"]).reshape(m, k)
    kl = k // world
    total = torch.zeros(m, n, device="cuda")
    for r in range(world):
        lin = garnet_b200.W4A16Linear().prepare(dev(case["nibbles"]), bf16_tensor(case["scales_bits"]).reshape(n, k // 128),
                                                n, k, 128, r, world, shard_axis=1)
        assert torch.equal(lin.dequantized(), deq[:, r * kl:(r + 1) * kl])
        part = lin.forward(x[:, r * kl:(r + 1) * kl].contiguous())
        assert lin.fault() == 0 and part.shape == (m, n)
        total += part.float()
    y = total.bfloat16()
    _, y64 = oracle.w4a16_exact(case["nibbles"], case["scales_f32"], n, k, 128, case["x_f32"])
    err = np.abs(y.float().cpu().numpy().astype(np.float64) - y64)
    rms = np.sqrt((y64 ** 2).mean(axis=1, keepdims=True))
    # every partial sum carries one bf16 rounding of a value of the size of the row's output scale
    assert (err <= TOL * (1 + np.abs(y64)) + world * 2.0 ** -8 * 4 * rms).all()
    with pytest.raises(garnet_b200.GarnetB200Error):
        garnet_b200.W4A16Linear().prepare(dev(case["nibbles"]), bf16_tensor(case["scales_bits"]).reshape(n, k // 128),
                                          n, k, 128, 0, 3, shard_axis=1)          # 2048 / 3 is not a whole number of groups


def test_full_lm_head_at_the_benchmark_batches():
    """The whole lm_head of BASELINE's config 2 (151936 x 2048: 9496 strips, a vocabulary that is
    not a multiple of 128) at M = 1, 64 and 256, i.e. through the list kernel, the tile kernel with
    one batch tile and with two: every output column of sampled batch rows against the exact oracle."""
    n, k = 151936, 2048
    case = synth.int4_linear(n, k, 256, seed=77)
    lin = make_linear(case, n, k)
    x_all = bf16_tensor(case["x_bits"]).reshape(256, k)
    for m, rows in ((1, [0]), (64, [0, 31, 63]), (256, [0, 127, 128, 255])):
        y = lin.forward(x_all[:m].contiguous())
        torch.cuda.synchronize()
        assert lin.fault() == 0 and y.shape == (m, n)
        _, y64 = oracle.w4a16_exact(case["nibbles"], case["scales_f32"], n, k, 128, case["x_f32"][rows])
        check_close(y[torch.tensor(rows, device="cuda")], y64, rounded_weights=m > 16)
