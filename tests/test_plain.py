"""The plain implementation checked against itself and against hand-computed cases (no GPU)."""
import math

import numpy as np

import plain_llama as pl
from conftest import TINY_A, TINY_B
from ghost_infer_b200.parts.rope import rotary_inv_freq


def random_weights(cfg, seed):
    rng = np.random.default_rng(seed)
    H, KV = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d, hd, F, V = cfg["hidden_size"], cfg["head_dim"], cfg["intermediate_size"], cfg["vocab_size"]
    w = {"model.embed_tokens.weight": rng.normal(0, 0.05, (V, d)), "model.norm.weight": 1 + 0.1 * rng.normal(size=d)}
    if not cfg["tie_word_embeddings"]:
        w["lm_head.weight"] = rng.normal(0, 0.05, (V, d))
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        w[p + "input_layernorm.weight"] = 1 + 0.1 * rng.normal(size=d)
        w[p + "post_attention_layernorm.weight"] = 1 + 0.1 * rng.normal(size=d)
        w[p + "self_attn.q_proj.weight"] = rng.normal(0, 0.05, (H * hd, d))
        w[p + "self_attn.k_proj.weight"] = rng.normal(0, 0.05, (KV * hd, d))
        w[p + "self_attn.v_proj.weight"] = rng.normal(0, 0.05, (KV * hd, d))
        w[p + "self_attn.o_proj.weight"] = rng.normal(0, 0.05, (d, H * hd))
        w[p + "mlp.gate_proj.weight"] = rng.normal(0, 0.05, (F, d))
        w[p + "mlp.up_proj.weight"] = rng.normal(0, 0.05, (F, d))
        w[p + "mlp.down_proj.weight"] = rng.normal(0, 0.05, (d, F))
    return w


def test_rms_norm_by_hand():
    x = np.array([[3.0, 4.0]])
    y = pl.rms_norm(x, np.array([2.0, 0.5]), 0.5)
    s = 1 / math.sqrt(12.5 + 0.5)
    assert np.allclose(y, [[3 * s * 2, 4 * s * 0.5]])


def test_rope_pairs_and_position_zero():
    inv = np.array([1.0, 0.5], dtype=np.float32)
    x = np.arange(8, dtype=np.float64).reshape(1, 8) + 1      # two heads of 4
    assert np.allclose(pl.rope(x, [0], inv, 4), x)
    y = pl.rope(x, [3], inv, 4, "half")
    c, s = math.cos(3.0), math.sin(3.0)
    assert np.allclose(y[0, 0], 1 * c - 3 * s) and np.allclose(y[0, 2], 1 * s + 3 * c)     # pair (0, 2)
    c2, s2 = math.cos(1.5), math.sin(1.5)
    assert np.allclose(y[0, 5], 6 * c2 - 8 * s2) and np.allclose(y[0, 7], 6 * s2 + 8 * c2)  # head 1, pair (1, 3)
    z = pl.rope(x, [3], inv, 4, "adjacent")
    assert np.allclose(z[0, 0], 1 * c - 2 * s) and np.allclose(z[0, 1], 1 * s + 2 * c)      # pair (0, 1)
    # a rotation keeps each pair's length
    assert np.allclose((y ** 2).sum(), (x ** 2).sum())


def test_llama3_scaling_bands():
    sc = TINY_B["rope_scaling"]
    plain = pl.rotary_inv_freq(32, 500000.0, None).astype(np.float64)
    scaled = pl.rotary_inv_freq(32, 500000.0, sc).astype(np.float64)
    wavelen = 2 * math.pi / plain
    hi, lo = 32 / 4.0, 32 / 1.0
    kept, divided = wavelen < hi, wavelen > lo
    mid = ~kept & ~divided
    assert kept.any() and divided.any() and mid.any()           # all three regimes are in use
    assert np.allclose(scaled[kept], plain[kept], rtol=1e-6)
    assert np.allclose(scaled[divided], plain[divided] / 8.0, rtol=1e-6)
    assert np.all(scaled[mid] < plain[mid]) and np.all(scaled[mid] > plain[mid] / 8.0)
    # the product's table is the same numbers
    assert np.array_equal(rotary_inv_freq(32, 500000.0, sc).numpy(), pl.rotary_inv_freq(32, 500000.0, sc))
    assert np.array_equal(rotary_inv_freq(16, 10000.0, None).numpy(), pl.rotary_inv_freq(16, 10000.0, None))


def test_attention_is_causal_and_grouped():
    rng = np.random.default_rng(0)
    n, H, KV, hd = 6, 4, 2, 8
    q, k, v = rng.normal(size=(n, H * hd)), rng.normal(size=(n, KV * hd)), rng.normal(size=(n, KV * hd))
    full = pl.attention(q, k, v, H, KV, hd, 0.3)
    part = pl.attention(q[:4], k[:4], v[:4], H, KV, hd, 0.3)
    assert np.allclose(full[:4], part)                         # later tokens change nothing before them
    assert np.allclose(full[0], np.repeat(v[0].reshape(KV, hd), 2, axis=0).reshape(-1))  # heads 0,1 -> kv 0; 2,3 -> kv 1
    w1 = pl.attention(q, k, v, H, KV, hd, 0.3, window=1)
    assert np.allclose(w1, np.repeat(v.reshape(n, KV, hd), 2, axis=1).reshape(n, -1))     # a window of 1 sees itself only


def test_forward_prefix_property():
    for cfg, seed in ((TINY_A, 0), (TINY_B, 1)):
        w = random_weights(cfg, seed)
        toks = np.random.default_rng(seed).integers(0, cfg["vocab_size"], 20).tolist()
        full = pl.forward(cfg, w, toks)
        assert full.shape == (20, cfg["vocab_size"])
        assert np.allclose(full[:11], pl.forward(cfg, w, toks[:11]), atol=1e-12)


def test_tied_head_uses_the_embedding():
    w = random_weights(TINY_B, 3)
    toks = [1, 2, 3]
    a = pl.forward(TINY_B, w, toks)
    w2 = dict(w)
    w2["lm_head.weight"] = np.zeros_like(w["model.embed_tokens.weight"])
    assert np.array_equal(a, pl.forward(TINY_B, w2, toks))


def test_xorshift_and_greedy():
    r = pl.XorShift64Star(0)
    assert r.s == 1                                            # max(seed, 1)
    u = [pl.XorShift64Star(42).next_f32() for _ in range(2)]
    assert u[0] == u[1] and 0.0 <= u[0] < 1.0
    # first step by hand for state 1: s ^= s>>12 (1); s ^= s<<25; s ^= s>>27
    s = 1
    s ^= s >> 12
    s ^= (s << 25) & (2 ** 64 - 1)
    s ^= s >> 27
    assert pl.XorShift64Star(1).next_f32() == ((s * 0x2545F4914F6CDD1D % 2 ** 64) >> 40) / 2 ** 24
    assert pl.greedy([1.0, 3.0, 3.0, -1.0]) == 1               # the first of the highest
    assert pl.greedy([float("nan"), 2.0]) == 1


def test_distribution_cut_rules():
    logits = [0.0, math.log(2.0), math.log(4.0), math.log(1.0)]
    ids, w = pl.distribution(logits, 1.0, 0, 1.0)
    assert ids == [2, 1, 0, 3] and np.allclose(w, [0.5, 0.25, 0.125, 0.125])    # ties by token id
    ids, w = pl.distribution(logits, 1.0, 2, 1.0)
    assert ids == [2, 1] and np.allclose(w, [2 / 3, 1 / 3])
    ids, w = pl.distribution(logits, 1.0, 0, 0.7)
    assert ids == [2, 1]                                       # 0.5 < 0.7 <= 0.75: cut after the second
    ids, w = pl.distribution(logits, 0.5, 0, 1.0)
    assert np.allclose(w, np.array([16, 4, 1, 1]) / 22)


def test_sampling_frequencies():
    logits = [0.0, 1.0, 2.0, 0.5]
    rng = pl.XorShift64Star(7)
    n = 20000
    counts = np.zeros(4)
    for _ in range(n):
        counts[pl.sample(logits, 0.8, 0, 1.0, rng)] += 1
    p = np.exp(np.array(logits) / 0.8)
    p /= p.sum()
    assert np.abs(counts / n - p).max() < 0.012
