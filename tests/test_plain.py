"""The plain implementation checked against itself and against hand-computed cases (no GPU)."""
import math

import numpy as np
import pytest

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


# Rotary frequencies as literals.  They were worked out apart from both codes, with 60-digit decimal arithmetic
# (exp and ln of the decimal module, pi as a literal) from the rule itself: inv_freq_i = theta^(-2i/dim); with
# wavelen = 2 pi / inv_freq, a pair keeps its frequency if wavelen < orig / high, has it divided by `factor` if
# wavelen > orig / low, and otherwise takes ((1 - s) / factor + s) * inv_freq with s = (orig / wavelen - low) /
# (high - low); then rounded to float32.  The reference consumes such a table as `rope_freqs` = plain / scaled
# (src/model.rs:208-211, :768).  Tiny B (dim 32, theta 5e5, factor 8, low 1, high 4, orig 32) has one kept pair,
# one blended and fourteen divided; the 8B configuration (dim 128, orig 8192) has 29, 6 and 29.
INV_FREQ_TINY_B = [
    "0x1.0000000000000p+0", "0x1.b7a3860000000p-3", "0x1.8d275e0000000p-6", "0x1.5dc95a0000000p-7",
    "0x1.3411900000000p-8", "0x1.0f53860000000p-9", "0x1.ddee9c0000000p-11", "0x1.a4ee400000000p-12",
    "0x1.72ba440000000p-13", "0x1.46831a0000000p-14", "0x1.1f91f00000000p-15", "0x1.fa8b840000000p-17",
    "0x1.be21880000000p-18", "0x1.88ec220000000p-19", "0x1.5a0f4e0000000p-20", "0x1.30c94e0000000p-21"]
INV_FREQ_LLAMA_8B = [
    "0x1.0000000000000p+0", "0x1.a115820000000p-1", "0x1.53c38a0000000p-1", "0x1.14c7080000000p-1",
    "0x1.c2ef760000000p-2", "0x1.6f56fa0000000p-2", "0x1.2b3dc60000000p-2", "0x1.e788c20000000p-3",
    "0x1.8d275e0000000p-3", "0x1.4387400000000p-3", "0x1.078d3e0000000p-3", "0x1.ad63380000000p-4",
    "0x1.5dc95a0000000p-4", "0x1.1cf1300000000p-4", "0x1.d03cd00000000p-5", "0x1.7a2d080000000p-5",
    "0x1.3411900000000p-5", "0x1.f5ea7e0000000p-6", "0x1.98de920000000p-6", "0x1.4d12740000000p-6",
    "0x1.0f53860000000p-6", "0x1.ba0dd80000000p-7", "0x1.681ad80000000p-7", "0x1.2558fe0000000p-7",
    "0x1.ddee9c0000000p-8", "0x1.8554ea0000000p-8", "0x1.3d28040000000p-8", "0x1.025c6a0000000p-8",
    "0x1.a4ee400000000p-9", "0x1.1bfa0e0000000p-9", "0x1.67a2380000000p-10", "0x1.c12f3a0000000p-11",
    "0x1.132ba80000000p-11", "0x1.47e2160000000p-12", "0x1.765ba60000000p-13", "0x1.90d10c0000000p-14",
    "0x1.46831a0000000p-14", "0x1.09fb7e0000000p-14", "0x1.b159020000000p-15", "0x1.6103320000000p-15",
    "0x1.1f91f00000000p-15", "0x1.d484e00000000p-16", "0x1.7da9e80000000p-16", "0x1.36e8ea0000000p-16",
    "0x1.fa8b840000000p-17", "0x1.9ca3ea0000000p-17", "0x1.5024d60000000p-17", "0x1.11d4200000000p-17",
    "0x1.be21880000000p-18", "0x1.6b6d0e0000000p-18", "0x1.280d960000000p-18", "0x1.e257020000000p-19",
    "0x1.88ec220000000p-19", "0x1.4014d20000000p-19", "0x1.04be680000000p-19", "0x1.a8d0100000000p-20",
    "0x1.5a0f4e0000000p-20", "0x1.19e8020000000p-20", "0x1.cb4a9a0000000p-21", "0x1.76258e0000000p-21",
    "0x1.30c94e0000000p-21", "0x1.f091840000000p-22", "0x1.9483600000000p-22", "0x1.4985fe0000000p-22"]
LLAMA_8B_SCALING = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                    "original_max_position_embeddings": 8192}


def _ulps(a, b):
    a, b = np.asarray(a, dtype=np.float32), np.asarray(b, dtype=np.float32)
    return np.abs(a.view(np.int32).astype(np.int64) - b.view(np.int32).astype(np.int64))


@pytest.mark.parametrize("literals,dim,scaling", [(INV_FREQ_TINY_B, 32, TINY_B["rope_scaling"]),
                                                  (INV_FREQ_LLAMA_8B, 128, LLAMA_8B_SCALING)])
def test_rotary_frequencies_against_literals(literals, dim, scaling):
    """Both writings of the rule, the product's and the plain implementation's, give the literal table to one unit
    in the last place; so does the typed configuration's path to the product's part."""
    want = np.array([float.fromhex(h) for h in literals], dtype=np.float32)
    assert len(want) == dim // 2
    assert _ulps(pl.rotary_inv_freq(dim, 500000.0, scaling), want).max() <= 1
    assert _ulps(rotary_inv_freq(dim, 500000.0, scaling).numpy(), want).max() <= 1
    # through config.json's keys, as a model would get them
    from ghost_infer_b200.config import LlamaConfig
    from ghost_infer_b200.config.llama_spec import llama_rope_spec
    from ghost_infer_b200.parts.rope import Rotary
    raw = dict(TINY_B, head_dim=dim, hidden_size=3 * dim, rope_scaling=scaling)
    part = Rotary(llama_rope_spec(LlamaConfig.from_dict(raw)).params)
    assert _ulps(part.inv_freq_host.numpy(), want).max() <= 1
    # the literals themselves hold all three bands: kept pairs equal theta^(-2i/dim), divided ones an eighth of it
    plain = np.array([500000.0 ** (-2.0 * i / dim) for i in range(dim // 2)])
    ratio = plain / want.astype(np.float64)
    assert (np.abs(ratio - 1) < 1e-6).any() and (np.abs(ratio - 8) < 1e-5).any() and ((ratio > 1.001) & (ratio < 7.99)).any()


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
