"""The gpt-oss layer operators around the MoE, through the C ABI, against the reference's own GPU
kernels (compiled unchanged from its sources into oracle/_ref/libgarnet_ref_gpu.so) on the same
inputs: RMS norm, YaRN RoPE, paged attention with sinks and sliding window (decode and prefill,
including the cache append), the decode GEMV and the vocabulary top-1 pair.

Bounds: the element-wise operators follow the reference's arithmetic step for step and must agree
bit for bit, except where a sum is formed in another order (RMS norm, GEMV, attention): there the
bf16-valued result may differ by one rounding step, and by 2e-3 of the row's scale for attention."""
import ctypes

import numpy as np
import pytest
import torch

import garnet_b200
from garnet_b200 import gpt_oss as go

pytestmark = pytest.mark.gpu


def ref():
    from oracle import ref_gpu
    if not ref_gpu.available():
        pytest.skip("oracle/_ref/libgarnet_ref_gpu.so has not been built (make -C oracle ref_gpu REF=...)")
    return ref_gpu.lib()


def bf(t):
    return t.to(torch.bfloat16).float()


def one_step(got, want, extra=0.0):
    step = want.abs().clamp_min(2.0 ** -120) * 2.0 ** -7
    rms = want.pow(2).mean(dim=-1, keepdim=True).sqrt()
    return bool(((got - want).abs() <= 1.01 * step + extra * rms).all())


def s():
    return torch.cuda.current_stream().cuda_stream


def test_rms_norm():
    R = ref()
    g = torch.Generator(device="cuda").manual_seed(0)
    x = bf(torch.randn(7, 2880, device="cuda", generator=g) * 3)
    w = bf(1 + 0.2 * torch.randn(2880, device="cuda", generator=g))
    want = torch.empty_like(x)
    assert R.ref_gpu_rms_norm(x.data_ptr(), w.data_ptr(), want.data_ptr(), 7, 2880, 1e-5, 256, s()) == 0
    got = go.rms_norm(x, w, 1e-5)
    torch.cuda.synchronize()
    assert one_step(got, want) and (got == want).float().mean() >= 0.99


def test_yarn_rope_bit_for_bit():
    R = ref()
    g = torch.Generator(device="cuda").manual_seed(1)
    opt = go.options()
    tokens = 6
    x = bf(torch.randn(tokens, (64 + 16) * 64, device="cuda", generator=g))
    pos = torch.tensor([0, 1, 17, 4095, 4096, 131071], dtype=torch.int64, device="cuda")
    want = torch.empty_like(x)
    assert R.ref_gpu_rope(x.data_ptr(), pos.data_ptr(), want.data_ptr(), tokens, 64, 8, 64, 150000.0, 32.0, 4096.0, 32.0, 1.0, s()) == 0
    got = go.rope(opt, x, pos)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    # without YaRN scaling (factor 1) and another geometry
    opt2 = go.options(q_heads=4, kv_heads=2, head_dim=128, factor=1.0, theta=10000.0)
    x2 = bf(torch.randn(3, 8 * 128, device="cuda", generator=g))
    pos2 = torch.tensor([5, 0, 999], dtype=torch.int64, device="cuda")
    want2 = torch.empty_like(x2)
    assert R.ref_gpu_rope(x2.data_ptr(), pos2.data_ptr(), want2.data_ptr(), 3, 4, 2, 128, 10000.0, 1.0, 4096.0, 32.0, 1.0, s()) == 0
    assert torch.equal(go.rope(opt2, x2, pos2), want2)


def attention_case(window, prefill, tokens, lengths, q_heads=64, kv_heads=8, d=64, layers=3, layer=1, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    batch, logical = len(lengths), 48
    physical = batch * logical
    table = torch.randperm(physical, generator=torch.Generator().manual_seed(seed)).reshape(batch, logical).to(torch.int32).cuda()
    keys = torch.randn(layers, physical, 16, kv_heads, d, device="cuda", generator=g).to(torch.bfloat16)
    values = torch.randn(layers, physical, 16, kv_heads, d, device="cuda", generator=g).to(torch.bfloat16)
    qkv = bf(torch.randn(batch * tokens, (q_heads + 2 * kv_heads) * d, device="cuda", generator=g))
    lens = torch.tensor(lengths, dtype=torch.int32, device="cuda")
    starts = torch.tensor([max(0, n - tokens) for n in lengths], dtype=torch.int32, device="cuda")
    active = torch.tensor([1] * (batch - 1) + [0], dtype=torch.int32, device="cuda")
    sinks = torch.randn(q_heads, device="cuda", generator=g)
    opt = go.options(q_heads=q_heads, kv_heads=kv_heads, head_dim=d, layer=layer, window=window, prefill=prefill)
    return opt, qkv, keys, values, table, lens, starts, active, sinks, batch, physical


@pytest.mark.parametrize("window", [0, 128])
def test_decode_attention_with_sinks_and_window(window):
    R = ref()
    lengths = [1, 17, 130, 700, 64]                     # the last sequence is inactive
    opt, qkv, keys, values, table, lens, starts, active, sinks, batch, physical = attention_case(window, 0, 1, lengths)
    k_ref, v_ref = keys.clone(), values.clone()
    want = torch.empty(batch, 64 * 64, device="cuda")
    ws = torch.zeros(batch * 64 * 64 * 66 * 4, dtype=torch.uint8, device="cuda")
    ops = (ctypes.c_void_p * 8)(*[t.data_ptr() for t in (qkv, k_ref, v_ref, table, lens, starts, active, sinks)])
    assert R.ref_gpu_attention(ops, want.data_ptr(), ws.data_ptr(), batch, 1, table.shape[1], physical, 64, 8, 64, 1, 16, window, 0, s()) == 0
    for _ in range(2):                                   # second call: the counters are back at zero, the rows already appended
        got = go.attention(opt, qkv, keys, values, table, lens, starts, active, sinks, batch, 1, physical)
        torch.cuda.synchronize()
        assert one_step(got, want, 2e-3), float((got - want).abs().max())
    assert torch.equal(keys, k_ref) and torch.equal(values, v_ref)      # the cache append, bit for bit
    assert (got[-1] == 0).all()                                          # the inactive sequence


def test_prefill_and_other_geometries_take_the_general_kernel():
    R = ref()
    # prefill: 5 new rows per sequence, each sees the positions up to its own
    opt, qkv, keys, values, table, lens, starts, active, sinks, batch, physical = attention_case(128, 1, 5, [5, 140, 33], seed=3)
    k_ref, v_ref = keys.clone(), values.clone()
    want = torch.empty(batch * 5, 64 * 64, device="cuda")
    ws = torch.zeros(1 << 24, dtype=torch.uint8, device="cuda")
    ops = (ctypes.c_void_p * 8)(*[t.data_ptr() for t in (qkv, k_ref, v_ref, table, lens, starts, active, sinks)])
    assert R.ref_gpu_attention(ops, want.data_ptr(), ws.data_ptr(), batch, 5, table.shape[1], physical, 64, 8, 64, 1, 16, 128, 1, s()) == 0
    got = go.attention(opt, qkv, keys, values, table, lens, starts, active, sinks, batch, 5, physical)
    torch.cuda.synchronize()
    assert one_step(got, want, 2e-3) and torch.equal(keys, k_ref) and torch.equal(values, v_ref)
    # decode with 128-wide heads (not the grouped kernel's shape)
    opt, qkv, keys, values, table, lens, starts, active, sinks, batch, physical = attention_case(0, 0, 1, [9, 300, 40], q_heads=8, kv_heads=2, d=128, seed=4)
    k_ref, v_ref = keys.clone(), values.clone()
    want = torch.empty(batch, 8 * 128, device="cuda")
    ops = (ctypes.c_void_p * 8)(*[t.data_ptr() for t in (qkv, k_ref, v_ref, table, lens, starts, active, sinks)])
    assert R.ref_gpu_attention(ops, want.data_ptr(), ws.data_ptr(), batch, 1, table.shape[1], physical, 8, 2, 128, 1, 16, 0, 0, s()) == 0
    got = go.attention(opt, qkv, keys, values, table, lens, starts, active, sinks, batch, 1, physical)
    torch.cuda.synchronize()
    assert one_step(got, want, 2e-3)


def test_vocab_top1_pairs():
    R = ref()
    g = torch.Generator(device="cuda").manual_seed(5)
    logits = bf(torch.randn(4, 100500, device="cuda", generator=g))
    logits[1, 77] = logits[1, 90000] = 40.0
    logits[2, :] = 1.5
    for rank in (0, 1):
        want = torch.empty(4, 2, device="cuda")
        assert R.ref_gpu_vocab_top1(logits.data_ptr(), want.data_ptr(), 4, 100500, rank, s()) == 0
        got = go.vocab_top1(logits, rank)
        torch.cuda.synchronize()
        assert torch.equal(got, want)
    assert got[1, 1].item() == 100500 + 77 and got[2, 1].item() == 100500


def test_decode_gemv():
    R = ref()
    g = torch.Generator(device="cuda").manual_seed(6)
    # o_proj-like: 2880 rows over columns [4096, 8192) of a wider matrix
    w = (torch.randn(2880, 8192, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    x = torch.randn(4096, device="cuda", generator=g).to(torch.bfloat16)
    want = torch.empty(2880, dtype=torch.bfloat16, device="cuda")
    assert R.ref_gpu_decode_gemv(x.data_ptr(), w.data_ptr(), want.data_ptr(), 2880, 4096, 8192, 4096, 0, 0, 0, 0, s()) == 0
    got = go.decode_gemv(x, w, 2880, 4096, 4096)
    torch.cuda.synchronize()
    assert one_step(got.float()[None], want.float()[None], 1e-3) and (got == want).float().mean() >= 0.95
    # packed q/k/v weight of 64 + 8 + 8 heads, this rank's half
    wq = (torch.randn(80 * 64, 2880, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    xq = torch.randn(2880, device="cuda", generator=g).to(torch.bfloat16)
    rows = (32 + 8) * 64
    for rank in (0, 1):
        want = torch.empty(rows, dtype=torch.bfloat16, device="cuda")
        assert R.ref_gpu_decode_gemv(xq.data_ptr(), wq.data_ptr(), want.data_ptr(), rows, 2880, 2880, 0, 64, 8, 64, rank, s()) == 0
        got = go.decode_gemv(xq, wq, rows, 2880, 0, 64, 8, 64, rank)
        torch.cuda.synchronize()
        assert one_step(got.float()[None], want.float()[None], 1e-3)
    L = garnet_b200.lib()
    assert L.garnet_b200_gpt_oss_decode_gemv(xq.data_ptr(), wq.data_ptr(), want.data_ptr(), rows, 2881, 2880, 0, 0, 0, 0, 0, None) != 0
    assert L.garnet_b200_gpt_oss_rms_norm(None, None, None, 1, 1, 1e-5, None) != 0
