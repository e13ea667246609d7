"""The numpy oracle of the decode step (oracle/decode.py) against direct formulas, on the CPU:
the paged attention equals a dense softmax attention over the gathered context, RoPE is a
rotation (it keeps the norm of every (d, d + 64) pair up to the bf16 rounding), the RMS norm and
SwiGLU follow their definitions, and a step appends exactly one cache row per sequence."""
import numpy as np

from oracle import bf16_round
from oracle import decode as odec


class Cfg:
    hidden, q_heads, kv_heads, head_dim, intermediate, vocab, layers = 64, 4, 2, 128, 96, 50, 2
    eps, page_size = 1e-6, 16


def bf(a):
    return bf16_round(np.asarray(a, np.float32)).astype(np.float64)


def tables(positions, d=128, theta=1e6):
    inv = theta ** (-np.arange(0, d, 2, dtype=np.float64) / d)
    ang = np.arange(positions, dtype=np.float64)[:, None] * inv[None, :]
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


def test_norm_rope_and_swiglu_follow_their_definitions():
    rng = np.random.default_rng(0)
    x = bf(rng.normal(size=(3, 128)))
    w = bf(1 + 0.1 * rng.normal(size=128))
    n = odec.rms_norm(x, w, 1e-6)
    assert np.allclose(n, bf(x / np.sqrt((x ** 2).mean(axis=1, keepdims=True) + 1e-6) * w))
    cos, sin = tables(40)
    r = odec.rope(x, cos[17].astype(np.float64), sin[17].astype(np.float64))
    pair = lambda v: v[:, :64] ** 2 + v[:, 64:] ** 2   # noqa: E731
    assert np.allclose(pair(r), pair(x), rtol=2e-2, atol=1e-3)
    assert np.array_equal(odec.rope(x, cos[0].astype(np.float64), sin[0].astype(np.float64)), x)   # position 0: identity
    gu = bf(rng.normal(size=(2, 2 * 96)))
    g, u = gu[:, :96], gu[:, 96:]
    assert np.array_equal(odec.silu_mul(gu, 96), bf(g / (1 + np.exp(-g)) * u))


def test_paged_attention_equals_dense_attention_and_appends_one_row():
    cfg = Cfg()
    rng = np.random.default_rng(1)
    batch, pages_per_seq = 2, 4
    total = batch * pages_per_seq
    kp = [bf(rng.normal(size=(total, 16, cfg.kv_heads, 128)))]
    vp = [bf(rng.normal(size=(total, 16, cfg.kv_heads, 128)))]
    table = rng.permutation(total).reshape(batch, pages_per_seq).astype(np.int32)
    cos, sin = tables(64)
    ones = np.ones(128)
    o = odec.Decoder(cfg, dict(layers=[dict(q_norm=ones, k_norm=ones)]), [kp[0].copy()], [vp[0].copy()], table, cos, sin)
    qkv = bf(rng.normal(size=(batch, (cfg.q_heads + 2 * cfg.kv_heads) * 128)))
    positions = [5, 33]
    out = o.attention(0, qkv, positions)
    changed = (o.key_pages[0] != kp[0]).any(axis=(2, 3))
    assert changed.sum() == batch                       # one cache row per sequence
    for b, slot in enumerate(positions):
        page, off = table[b, slot // 16], slot % 16
        assert changed[page, off]
        v_new = qkv[b, (cfg.q_heads + cfg.kv_heads) * 128:].reshape(cfg.kv_heads, 128)
        assert np.array_equal(o.value_pages[0][page, off], v_new)
        # dense attention over the gathered context
        K = np.stack([o.key_pages[0][table[b, p // 16], p % 16] for p in range(slot + 1)])
        V = np.stack([o.value_pages[0][table[b, p // 16], p % 16] for p in range(slot + 1)])
        q = qkv[b, :cfg.q_heads * 128].reshape(cfg.q_heads, 128)
        qn = odec.rope(odec.rms_norm(q, ones, cfg.eps), cos[slot].astype(np.float64), sin[slot].astype(np.float64))
        for h in range(cfg.q_heads):
            s = K[:, h // 2] @ qn[h] / np.sqrt(128.0)
            p = np.exp(s - s.max())
            p /= p.sum()
            assert np.array_equal(out[b, h * 128:(h + 1) * 128], bf(p @ V[:, h // 2]))


def test_step_runs_and_is_deterministic():
    cfg = Cfg()
    rng = np.random.default_rng(2)
    H, I, qw, qkvw = cfg.hidden, cfg.intermediate, cfg.q_heads * 128, (cfg.q_heads + 2 * cfg.kv_heads) * 128
    layer = lambda: dict(in_norm=np.ones(H), post_norm=np.ones(H), q_norm=np.ones(128), k_norm=np.ones(128),   # noqa: E731
                         qkv=rng.normal(size=(qkvw, H)) * 0.05, o=rng.normal(size=(H, qw)) * 0.05,
                         gate_up=rng.normal(size=(2 * I, H)) * 0.05, down=rng.normal(size=(H, I)) * 0.05)
    w = dict(embedding=bf(rng.normal(size=(cfg.vocab, H))), final_norm=np.ones(H), lm_head=rng.normal(size=(cfg.vocab, H)) * 0.05,
             layers=[layer() for _ in range(cfg.layers)])
    table = np.arange(4, dtype=np.int32).reshape(1, 4)
    cos, sin = tables(64)
    runs = []
    for _ in range(2):
        kp = [np.zeros((4, 16, cfg.kv_heads, 128)) for _ in range(cfg.layers)]
        vp = [np.zeros((4, 16, cfg.kv_heads, 128)) for _ in range(cfg.layers)]
        o = odec.Decoder(cfg, w, kp, vp, table, cos, sin)
        tok, toks = np.array([7]), []
        for pos in range(3):
            tok, logits, _ = o.step(tok, np.array([pos]))
            assert np.isfinite(logits).all() and logits.shape == (1, cfg.vocab)
            toks.append(int(tok[0]))
        runs.append(toks)
        assert (np.abs(kp[0][0, :3]).sum(axis=(1, 2)) > 0).all() and np.abs(kp[0][0, 3:]).sum() == 0
    assert runs[0] == runs[1]
