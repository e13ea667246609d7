"""The glue of a Qwen3 decode step on the GPU, through the C ABI, against the numpy oracle
(oracle/decode.py): attention over the paged KV cache with head norms, RoPE and the cache
append folded in; the list launch with RMS norm, SwiGLU and residual additions folded into
its linears; embedding and arg-max; and whole steps of a small decoder.

Tolerances (floating point; the oracle is evaluated in float64 with the same bf16 rounding
points): a result is a bf16 number, so it may differ from the oracle's by one rounding step
where the two fp32 values straddle a rounding boundary, plus a term well below the row's
scale for the fp32 summation order and the 15-bit block fixed point of the linears'
activations.  Every assertion states its bound."""
import ctypes

import numpy as np
import pytest
import torch

import garnet_b200
import oracle
from garnet_b200 import decode as dec
from oracle import decode as odec

pytestmark = pytest.mark.gpu


def t2n(t):
    return t.float().cpu().numpy().astype(np.float64)


def assert_bf16_close(got, want, rms_frac, what):
    """|got - want| <= 1.01 bf16 steps of |want| + rms_frac * rms(row of want)."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert np.isfinite(got).all(), what
    step = np.maximum(np.abs(want), 2.0 ** -120) * 2.0 ** -7
    rms = np.sqrt((want ** 2).mean(axis=-1, keepdims=True))
    excess = np.abs(got - want) - 1.01 * step - rms_frac * rms
    assert (excess <= 0).all(), f"{what}: worst excess {excess.max():.3e} (row scale {rms.max():.3e})"


def int4_pair(n, k, gen, scale=0.02):
    nib = torch.randint(0, 256, (n * k // 2,), dtype=torch.uint8, device="cuda", generator=gen)
    sc = (torch.randn(n, k // 128, device="cuda", generator=gen).abs() * (scale / 7.0)).to(torch.bfloat16)
    return nib, sc


def deq(pair, n, k):
    return odec.dequant(pair[0].cpu().numpy(), pair[1].float().cpu().numpy(), n, k)


def test_embedding_and_argmax():
    gen = torch.Generator(device="cuda").manual_seed(1)
    table = torch.randn(300, 256, device="cuda", generator=gen).to(torch.bfloat16)
    ids = torch.tensor([7, 299, 0, 12345, -3], dtype=torch.int32, device="cuda")     # the last two are clamped
    out = torch.zeros(5, 256, dtype=torch.bfloat16, device="cuda")
    dec.embedding_gather(table, ids, out)
    assert torch.equal(out, table[torch.tensor([7, 299, 0, 299, 0], device="cuda")])
    logits = torch.randn(4, 151936, device="cuda", generator=gen).to(torch.bfloat16)
    logits[1, 100] = logits[1, 90000] = 50.0          # a tie: the lowest index wins
    logits[2, :] = -1.0                                # all equal
    logits[3, 151935] = 60.0
    logits[3, 5] = float("nan")                        # never wins
    tok = torch.zeros(4, dtype=torch.int32, device="cuda")
    dec.argmax_bf16(logits, tok)
    want = [int(logits[0].float().argmax()), 100, 0, 151935]
    assert tok.cpu().tolist() == want


@pytest.mark.parametrize("q_heads,kv_heads", [(4, 2), (16, 8), (3, 3)])
def test_attention_decode_over_paged_cache(q_heads, kv_heads):
    cfg = dec.DecoderConfig(hidden=256, q_heads=q_heads, kv_heads=kv_heads, layers=1)
    gen = torch.Generator(device="cuda").manual_seed(q_heads)
    positions = [0, 15, 16, 127, 128, 300, 511]                # first slot, page edges, split edges, several splits
    batch, pages_per_seq = len(positions), 512 // cfg.page_size
    total_pages = batch * pages_per_seq + 3
    perm = torch.randperm(total_pages, generator=torch.Generator().manual_seed(3))[:batch * pages_per_seq]
    page_tables = perm.reshape(batch, pages_per_seq).to(torch.int32).cuda()
    kp = torch.randn(total_pages, cfg.page_size, kv_heads, 128, device="cuda", generator=gen).to(torch.bfloat16)
    vp = torch.randn(total_pages, cfg.page_size, kv_heads, 128, device="cuda", generator=gen).to(torch.bfloat16)
    qkv = (torch.randn(batch, cfg.qkv_width, device="cuda", generator=gen) * 1.5).to(torch.bfloat16)
    qn = (1 + 0.2 * torch.randn(128, device="cuda", generator=gen)).to(torch.bfloat16)
    kn = (1 + 0.2 * torch.randn(128, device="cuda", generator=gen)).to(torch.bfloat16)
    cos, sin = dec.rope_tables(512, 128, cfg.rope_theta)
    pos = torch.tensor(positions, dtype=torch.int32, device="cuda")
    o = odec.Decoder(cfg, dict(layers=[dict(q_norm=t2n(qn), k_norm=t2n(kn))]), [t2n(kp)], [t2n(vp)], page_tables.cpu().numpy(), cos, sin)
    want = o.attention(0, t2n(qkv), positions)
    attn = dec.PagedAttention(cfg, batch, 512, pages_per_seq, 512)
    out = torch.zeros(batch, q_heads * 128, dtype=torch.bfloat16, device="cuda")
    for _ in range(2):      # the second call finds the new rows already in the cache and the counters back at zero
        attn.run(qkv, qn, kn, torch.from_numpy(cos).cuda(), torch.from_numpy(sin).cuda(), kp, vp, page_tables, pos, out)
        torch.cuda.synchronize()
        # softmax-weighted means of bf16 values: one rounding step plus 2e-3 of the row's scale
        assert_bf16_close(t2n(out), want, 2e-3, "attention output")
    # the appended rows: v bit for bit, k (normalised and rotated on the device) within one rounding step
    for b, slot in enumerate(positions):
        page, off = int(page_tables[b, slot // cfg.page_size]), slot % cfg.page_size
        assert np.array_equal(t2n(vp[page, off]), o.value_pages[0][page, off])
        assert_bf16_close(t2n(kp[page, off]), o.key_pages[0][page, off], 1e-6, "appended k")
    # rows of other slots are untouched
    untouched = torch.ones(total_pages, cfg.page_size, dtype=torch.bool)
    for b, slot in enumerate(positions):
        untouched[int(page_tables[b, slot // cfg.page_size]), slot % cfg.page_size] = False
    assert np.array_equal(t2n(kp)[untouched.numpy()], o.key_pages[0][untouched.numpy()])


def test_attention_decode_rejects_bad_arguments():
    L = garnet_b200.lib()
    opt = dec.AttentionOptions(abi=1, struct_size=ctypes.sizeof(dec.AttentionOptions), q_heads=4, kv_heads=2, head_dim=64,
                               page_size=16, max_logical_pages=8, max_context=128, rope_positions=128, norm_eps=1e-6)
    n = ctypes.c_size_t(0)
    assert L.garnet_b200_attention_decode_workspace(ctypes.byref(opt), 1, ctypes.byref(n)) != 0      # head_dim
    opt.head_dim, opt.q_heads = 128, 3
    assert L.garnet_b200_attention_decode_workspace(ctypes.byref(opt), 1, ctypes.byref(n)) != 0      # 3 q heads over 2 kv heads
    opt.q_heads, opt.max_context = 4, 256
    assert L.garnet_b200_attention_decode_workspace(ctypes.byref(opt), 1, ctypes.byref(n)) != 0      # beyond the page table
    opt.max_context = 128
    assert L.garnet_b200_attention_decode_workspace(ctypes.byref(opt), 1, ctypes.byref(n)) == 0 and n.value > 0
    assert L.garnet_b200_attention_decode(ctypes.byref(opt), None, None, None, None, None, None, None, None, None, None, None,
                                          0, 1, 0, None) != 0


@pytest.mark.parametrize("m", [1, 3, 8])
def test_layer_glue_folded_into_the_list(m):
    """The list of one decoder layer after attention: o_proj + residual, norm + gate/up,
    SwiGLU + down + residual (taken from the first op's packets), norm + the next q/k/v -
    against the oracle, and each folded input on its own from memory."""
    H, I, QW, eps = 256, 384, 512, 1e-6
    gen = torch.Generator(device="cuda").manual_seed(m)
    o_w, gu_w, d_w, qkv_w = int4_pair(H, QW, gen), int4_pair(2 * I, H, gen, 0.08), int4_pair(H, I, gen), int4_pair(640, H, gen)
    mk = lambda pair, n, k: garnet_b200.W4A16Linear().prepare(pair[0], pair[1], n, k)   # noqa: E731
    lo, lgu, ld, lq = mk(o_w, H, QW), mk(gu_w, 2 * I, H), mk(d_w, H, I), mk(qkv_w, 640, H)
    bf = dict(dtype=torch.bfloat16, device="cuda")
    a = torch.randn(m, QW, device="cuda", generator=gen).to(torch.bfloat16)
    x0 = torch.randn(m, H, device="cuda", generator=gen).to(torch.bfloat16)
    w_post = (1 + 0.1 * torch.randn(H, device="cuda", generator=gen)).to(torch.bfloat16)
    w_in = (1 + 0.1 * torch.randn(H, device="cuda", generator=gen)).to(torch.bfloat16)
    x1, gu, x2, qkv = torch.zeros(m, H, **bf), torch.zeros(m, 2 * I, **bf), torch.zeros(m, H, **bf), torch.zeros(m, 640, **bf)
    lst = garnet_b200.GlueList([
        dict(linear=lo, x=a, y=x1, residual=x0),
        dict(linear=lgu, x=x1, y=gu, dep=0, norm_weight=w_post, norm_eps=eps),
        dict(linear=ld, x=gu, y=x2, dep=1, activation=1, residual_dep=0),
        dict(linear=lq, x=x2, y=qkv, dep=2, norm_weight=w_in, norm_eps=eps)], m=m)
    W = dict(o=deq(o_w, H, QW), gu=deq(gu_w, 2 * I, H), d=deq(d_w, H, I), q=deq(qkv_w, 640, H))
    bfr = lambda v: oracle.bf16_round(np.asarray(v, np.float32)).astype(np.float64)   # noqa: E731
    e_x1 = bfr(t2n(a) @ W["o"].T + t2n(x0))
    e_gu = bfr(odec.rms_norm(e_x1, t2n(w_post), eps) @ W["gu"].T)
    e_x2 = bfr(odec.silu_mul(e_gu, I) @ W["d"].T + e_x1)
    e_q = bfr(odec.rms_norm(e_x2, t2n(w_in), eps) @ W["q"].T)
    for _ in range(3):                      # the run tag moves on; stale packets of the previous run must not be taken
        lst.run()
        torch.cuda.synchronize()
        assert lst.fault() == 0
        assert_bf16_close(t2n(x1), e_x1, 3e-4, "o_proj + residual")
        assert_bf16_close(t2n(gu), e_gu, 6e-3, "norm + gate/up")            # inputs differ by bf16 steps of x1 and of the norm
        assert_bf16_close(t2n(x2), e_x2, 1.5e-2, "swiglu + down + residual")
        assert_bf16_close(t2n(qkv), e_q, 2.5e-2, "norm + q/k/v of the next layer")
    # each stage from the device's own previous stage (no accumulated difference): tight bounds
    s_gu = bfr(odec.rms_norm(t2n(x1), t2n(w_post), eps) @ W["gu"].T)
    s_x2 = bfr(odec.silu_mul(t2n(gu), I) @ W["d"].T + t2n(x1))
    s_q = bfr(odec.rms_norm(t2n(x2), t2n(w_in), eps) @ W["q"].T)
    assert_bf16_close(t2n(gu), s_gu, 1e-3, "norm + gate/up, stage alone")
    assert_bf16_close(t2n(x2), s_x2, 2e-3, "swiglu + down + residual, stage alone")
    assert_bf16_close(t2n(qkv), s_q, 1e-3, "norm + q/k/v, stage alone")
    # the same folded inputs read from memory instead of packets give the same bits
    gu2, x22, q2 = torch.zeros_like(gu), torch.zeros_like(x2), torch.zeros_like(qkv)
    garnet_b200.GlueList([dict(linear=lgu, x=x1, y=gu2, norm_weight=w_post, norm_eps=eps)], m=m).run()
    garnet_b200.GlueList([dict(linear=ld, x=gu, y=x22, activation=1, residual=x1)], m=m).run()
    garnet_b200.GlueList([dict(linear=lq, x=x2, y=q2, norm_weight=w_in, norm_eps=eps)], m=m).run()
    torch.cuda.synchronize()
    assert torch.equal(gu2, gu) and torch.equal(x22, x2) and torch.equal(q2, qkv)


def test_glue_list_rejects_bad_items():
    gen = torch.Generator(device="cuda").manual_seed(0)
    lin = garnet_b200.W4A16Linear().prepare(*int4_pair(256, 256, gen), 256, 256)
    wide = garnet_b200.W4A16Linear().prepare(*int4_pair(512, 256, gen), 512, 256)
    x = torch.zeros(1, 256, dtype=torch.bfloat16, device="cuda")
    y = torch.zeros(1, 512, dtype=torch.bfloat16, device="cuda")
    w = torch.ones(256, dtype=torch.bfloat16, device="cuda")
    bad = [
        [dict(linear=lin, x=x, y=y, norm_weight=w, norm_eps=0.0)],                                   # eps must be positive
        [dict(linear=lin, x=x, y=y, norm_weight=w, norm_eps=1e-6, activation=1)],                   # both on one input
        [dict(linear=lin, x=x, y=y), dict(linear=lin, x=y, y=x, dep=0, activation=1)] ,              # dep has n = 256, needs 512
        [dict(linear=wide, x=x, y=y), dict(linear=lin, x=x, y=x, residual_dep=0)],                   # residual of another width
        [dict(linear=lin, x=x, y=y, residual=x, residual_dep=0)],                                    # two residuals
    ]
    for calls in bad:
        with pytest.raises(garnet_b200.GarnetB200Error):
            garnet_b200.GlueList(calls, m=1)


def numpy_weights(cfg, w):
    H, I, qw = cfg.hidden, cfg.intermediate, cfg.q_heads * cfg.head_dim
    layers = [dict(in_norm=t2n(l["in_norm"]), post_norm=t2n(l["post_norm"]), q_norm=t2n(l["q_norm"]), k_norm=t2n(l["k_norm"]),
                   qkv=deq(l["qkv"], cfg.qkv_width, H), o=deq(l["o"], H, qw), gate_up=deq(l["gate_up"], 2 * I, H),
                   down=deq(l["down"], H, I)) for l in w["layers"]]
    return dict(embedding=t2n(w["embedding"]), final_norm=t2n(w["final_norm"]), lm_head=deq(w["lm_head"], cfg.vocab, H), layers=layers)


@pytest.mark.parametrize("graph", [False, True])
def test_decode_steps_of_a_small_decoder(graph):
    """Three steps of a 3-layer decoder (batch 2, sequences at different lengths) against the
    oracle fed the same tokens: logits within two rounding steps plus 3 % of the row's scale
    (differences of single bf16 steps in a residual stream are re-amplified by every norm), the
    residual stream of the first step much tighter, the caches equal to a rounding step."""
    cfg = dec.DecoderConfig(hidden=256, q_heads=4, kv_heads=2, intermediate=512, vocab=2048, layers=3)
    w = dec.synthetic_decoder(cfg, seed=5)
    batch, pages_per_seq = 2, 8
    total = batch * pages_per_seq
    gen = torch.Generator(device="cuda").manual_seed(9)
    kps = [torch.randn(total, cfg.page_size, cfg.kv_heads, 128, device="cuda", generator=gen).to(torch.bfloat16) for _ in range(cfg.layers)]
    vps = [torch.randn(total, cfg.page_size, cfg.kv_heads, 128, device="cuda", generator=gen).to(torch.bfloat16) for _ in range(cfg.layers)]
    page_tables = torch.randperm(total, generator=torch.Generator().manual_seed(1)).reshape(batch, pages_per_seq).to(torch.int32).cuda()
    step = dec.DecodeStep(cfg, w, batch, max_context=128, key_pages=kps, value_pages=vps, page_tables=page_tables)
    cos, sin = dec.rope_tables(pages_per_seq * cfg.page_size, 128, cfg.rope_theta)
    o = odec.Decoder(cfg, numpy_weights(cfg, w), [t2n(k) for k in kps], [t2n(v) for v in vps], page_tables.cpu().numpy(), cos, sin)
    if graph:
        step.token_in.copy_(torch.tensor([1, 2], dtype=torch.int32))
        step.positions.copy_(torch.tensor([3, 3], dtype=torch.int32))
        snapshot = [(k.clone(), v.clone()) for k, v in zip(kps, vps)]
        step.capture()                                  # the capture's warm-up run wrote rows at slot 3: put the caches back
        for (k0, v0), k, v in zip(snapshot, kps, vps):
            k.copy_(k0), v.copy_(v0)
    tokens, positions = np.array([11, 1999], np.int32), np.array([5, 40], np.int32)
    for it in range(3):
        step.token_in.copy_(torch.from_numpy(tokens))
        step.positions.copy_(torch.from_numpy(positions))
        step.run()
        torch.cuda.synchronize()
        assert step.fault() == 0
        e_tok, e_logits, trace = o.step(tokens, positions)
        got = t2n(step.logits)
        step_sz = np.maximum(np.abs(e_logits), 2.0 ** -120) * 2.0 ** -7
        rms = np.sqrt((e_logits ** 2).mean(axis=1, keepdims=True))
        assert (np.abs(got - e_logits) <= 2 * step_sz + 3e-2 * rms).all(), float((np.abs(got - e_logits) / rms).max())
        assert (np.abs(got - e_logits) <= 2 * step_sz + 3e-3 * rms).mean() >= 0.9
        if it == 0:
            assert_bf16_close(t2n(step.x[cfg.layers & 1]), trace[-1], 2e-2, "residual stream after the last layer")
        # greedy tokens agree wherever the oracle's margin is larger than the logit tolerance
        top2 = np.sort(e_logits, axis=1)[:, -2:]
        clear = (top2[:, 1] - top2[:, 0]) > 6e-2 * rms[:, 0] + 4 * step_sz.max(axis=1)
        dev_tok = step.token_out.cpu().numpy()
        assert np.array_equal(dev_tok[clear], e_tok[clear])
        assert np.array_equal(dev_tok, got.argmax(axis=1))          # and are the arg-max of the device's own logits
        tokens, positions = e_tok.copy(), positions + 1
    for i in range(cfg.layers):
        assert_bf16_close(t2n(vps[i]), o.value_pages[i], 3e-2, "value cache")
        assert_bf16_close(t2n(kps[i]), o.key_pages[i], 3e-2, "key cache")
