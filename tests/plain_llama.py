"""A plain, slow implementation of the Llama 3 dense decoder and of the sampler, used as the oracle.

Whole sequences, no cache, one function per part, numpy only, float64 arithmetic by default.  It shares
no code with the package under test (it even reads safetensors files itself).  The reference's own
model code is Rust that cannot be compiled here (no cargo/rustc) and reads GGUF only, so this file
rests on the reference's formulas; every function cites the lines it restates
(paths are inside the ghost-infer project).
"""
from __future__ import annotations

import json
import math
import struct

import numpy as np


# ---------------------------------------------------------------------------------------------
# files
def read_safetensors(path):
    """name -> float64 array.  Layout: u64 header length, JSON header, raw little-endian data."""
    with open(path, "rb") as f:
        (hlen,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(hlen))
        data = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        raw = data[b:e]
        dt = info["dtype"]
        if dt == "F32":
            arr = np.frombuffer(raw, dtype="<f4").astype(np.float64)
        elif dt == "F64":
            arr = np.frombuffer(raw, dtype="<f8").astype(np.float64)
        elif dt == "F16":
            arr = np.frombuffer(raw, dtype="<f2").astype(np.float64)
        elif dt == "BF16":
            u = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            arr = u.view(np.float32).astype(np.float64)
        else:
            raise ValueError(f"{name}: dtype {dt}")
        out[name] = arr.reshape(info["shape"])
    return out


def read_model(model_dir):
    with open(f"{model_dir}/config.json") as f:
        cfg = json.load(f)
    return cfg, read_safetensors(f"{model_dir}/model.safetensors")


def bf16_round(x):
    """Round-to-nearest-even to bfloat16, returned as float64."""
    f = np.asarray(x, dtype=np.float32)
    u = f.view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(np.float32).astype(np.float64).reshape(f.shape)


# ---------------------------------------------------------------------------------------------
# parts
def embed(table, tokens):
    """x[b, :] = E[token_b, :], no scaling (src/model.rs:987-990)."""
    return table[np.asarray(tokens)]


def rms_norm(x, w, eps):
    """ms = sum(x^2) / d; y = x * (1 / sqrt(ms + eps)) * w (src/model.rs:919-928)."""
    ms = (x * x).sum(-1, keepdims=True) / x.shape[-1]
    return x * (1.0 / np.sqrt(ms + eps)) * w


def rotary_inv_freq(rotary_dim, theta, scaling):
    """inv_freq_i = theta ** (-2 i / rotary_dim) (src/model.rs:768), divided per pair by the llama3
    factors the reference reads from its file as `rope_freqs` (src/model.rs:30-31, :208-211).  The factors
    follow the llama3 rule from config.json's rope_scaling: wavelength 2 pi / f shorter than
    orig / high keeps f; longer than orig / low gives f / factor; between, a linear blend in
    orig / wavelength.  Rounded once to 32-bit, as the table the kernels use."""
    half = rotary_dim // 2
    f = np.array([theta ** (-(2.0 * i) / rotary_dim) for i in range(half)], dtype=np.float64)
    if scaling is not None:
        factor = scaling["factor"]
        low, high = scaling["low_freq_factor"], scaling["high_freq_factor"]
        orig = scaling["original_max_position_embeddings"]
        out = f.copy()
        for i in range(half):
            wavelen = 2.0 * math.pi / f[i]
            if wavelen > orig / low:
                out[i] = f[i] / factor
            elif wavelen >= orig / high:
                s = (orig / wavelen - low) / (high - low)
                out[i] = (1.0 - s) * f[i] / factor + s * f[i]
        f = out
    return f.astype(np.float32)


def rope(x, positions, inv_freq, head_dim, pairing="half"):
    """Rotation of every head of x [n, heads * head_dim] (src/model.rs:942-953): theta = pos * inv_freq_i
    in 32-bit; (a, b) <- (a cos - b sin, a sin + b cos); pairs (i, i + half) or (2i, 2i + 1)."""
    n = x.shape[0]
    rot = 2 * len(inv_freq)
    half = rot // 2
    heads = x.shape[1] // head_dim
    y = x.reshape(n, heads, head_dim).copy()
    ang = (np.asarray(positions, dtype=np.float32)[:, None] * inv_freq[None, :]).astype(np.float32).astype(np.float64)
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    if pairing == "half":
        ia, ib = np.arange(half), np.arange(half) + half
    else:
        ia, ib = 2 * np.arange(half), 2 * np.arange(half) + 1
    a, b = y[:, :, ia].copy(), y[:, :, ib].copy()
    y[:, :, ia] = a * c - b * s
    y[:, :, ib] = a * s + b * c
    return y.reshape(n, heads * head_dim)


def attention(q, k, v, n_heads, n_kv, head_dim, scale, window=None):
    """Causal grouped-query attention of one whole sequence (src/model.rs:1320-1419): head h reads kv head
    h // (H / KV); score = (q . k_t) * scale for t <= own position (and t > position - window); softmax with
    the maximum subtracted; output = sum p_t v_t; heads concatenated in order."""
    n = q.shape[0]
    group = n_heads // n_kv
    qh = q.reshape(n, n_heads, head_dim)
    kh = k.reshape(n, n_kv, head_dim)
    vh = v.reshape(n, n_kv, head_dim)
    out = np.zeros((n, n_heads, head_dim), dtype=q.dtype)
    pos = np.arange(n)
    visible = pos[None, :] <= pos[:, None]
    if window:
        visible &= pos[None, :] > pos[:, None] - window
    for h in range(n_heads):
        kvh = h // group
        s = (qh[:, h, :] @ kh[:, kvh, :].T) * scale
        s = np.where(visible, s, -np.inf)
        s = s - s.max(-1, keepdims=True)
        p = np.exp(s)
        p = p / p.sum(-1, keepdims=True)
        out[:, h, :] = p @ vh[:, kvh, :]
    return out.reshape(n, n_heads * head_dim)


def swiglu(x, w_gate, w_up, w_down):
    """g = Wgate x; u = Wup x; h = g / (1 + exp(-g)) * u; out = Wdown h (src/quant.rs:1135-1154,
    src/model.rs:1133-1147)."""
    g = x @ w_gate.T
    u = x @ w_up.T
    return (g / (1.0 + np.exp(-g)) * u) @ w_down.T


def layer(x, positions, w, prefix, cfg, inv_freq, act_round=None):
    """One decoder layer (src/model.rs:996-1147): x += Wo attention(rope(Wq n), rope(Wk n), Wv n) with
    n = rms_norm(x); x += swiglu(rms_norm(x)).  `act_round` (optional) rounds what a 16-bit engine would
    store between kernels; the residual stream stays unrounded."""
    r = act_round or (lambda t: t)
    H, KV = cfg["num_attention_heads"], cfg.get("num_key_value_heads") or cfg["num_attention_heads"]
    hd = cfg.get("head_dim") or cfg["hidden_size"] // H
    eps = cfg.get("rms_norm_eps", 1e-5)
    h = r(rms_norm(x, w[prefix + "input_layernorm.weight"], eps))
    q = r(h @ w[prefix + "self_attn.q_proj.weight"].T)
    k = r(h @ w[prefix + "self_attn.k_proj.weight"].T)
    v = r(h @ w[prefix + "self_attn.v_proj.weight"].T)
    q = r(rope(q, positions, inv_freq, hd))
    k = r(rope(k, positions, inv_freq, hd))
    a = r(attention(q, k, v, H, KV, hd, 1.0 / math.sqrt(hd)))
    x = x + a @ w[prefix + "self_attn.o_proj.weight"].T
    h = r(rms_norm(x, w[prefix + "post_attention_layernorm.weight"], eps))
    g = r(h @ w[prefix + "mlp.gate_proj.weight"].T)
    u = r(h @ w[prefix + "mlp.up_proj.weight"].T)
    act = r(g / (1.0 + np.exp(-g)) * u)
    return x + act @ w[prefix + "mlp.down_proj.weight"].T


def forward(cfg, w, tokens, act_round=None):
    """Logits [n, vocab] of one whole sequence: embedding, layers, final norm, head (the embedding table
    when tied) (src/model.rs:971-1192, :637-638)."""
    r = act_round or (lambda t: t)
    H = cfg["num_attention_heads"]
    hd = cfg.get("head_dim") or cfg["hidden_size"] // H
    inv_freq = rotary_inv_freq(hd, cfg.get("rope_theta", 10000.0), cfg.get("rope_scaling"))
    positions = np.arange(len(tokens))
    x = embed(w["model.embed_tokens.weight"], tokens)
    for i in range(cfg["num_hidden_layers"]):
        x = layer(x, positions, w, f"model.layers.{i}.", cfg, inv_freq, act_round)
    h = r(rms_norm(x, w["model.norm.weight"], cfg.get("rms_norm_eps", 1e-5)))
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return h @ head.T


# ---------------------------------------------------------------------------------------------
# sampling
class XorShift64Star:
    """src/sampler.rs:185-191; the state starts at max(seed, 1) (src/sampler.rs:41)."""

    def __init__(self, seed):
        self.s = max(int(seed), 1) & 0xFFFFFFFFFFFFFFFF

    def next_f32(self):
        s = self.s
        s ^= s >> 12
        s ^= (s << 25) & 0xFFFFFFFFFFFFFFFF
        s ^= s >> 27
        self.s = s
        return float(np.float32(((s * 0x2545F4914F6CDD1D) & 0xFFFFFFFFFFFFFFFF) >> 40) / np.float32(1 << 24))


def greedy(logits):
    """The highest logit, the first on ties (src/sampler.rs:136-142, src/main.rs:1180-1182)."""
    best, bi = -math.inf, 0
    for i, v in enumerate(logits):
        if v > best:
            best, bi = v, i
    return bi


def distribution(logits, temperature, top_k, top_p):
    """Candidates most likely first with their weights, and the kept mass (src/sampler.rs:259-291):
    top_k highest (0 = all), w = exp((l - max) / T) / total, cut after the first place where the running
    sum reaches top_p.  Equal logits are ordered by token id."""
    logits = np.asarray(logits, dtype=np.float32)
    order = sorted(range(len(logits)), key=lambda i: (-float(logits[i]), i))
    if top_k and top_k < len(order):
        order = order[:top_k]
    mx = float(logits[order[0]])
    w = np.exp((logits[order].astype(np.float64) - mx) / temperature)
    w = w / w.sum()
    cum, cut = 0.0, len(order)
    for i, p in enumerate(w):
        cum += p
        if cum >= top_p:
            cut = i + 1
            break
    return order[:cut], w[:cut]


def sample(logits, temperature, top_k, top_p, rng):
    """src/sampler.rs:205-218: r = u * mass; walk the candidates subtracting weights until r <= 0."""
    if temperature <= 0:
        return greedy(logits)
    ids, w = distribution(logits, temperature, top_k, top_p)
    r = rng.next_f32() * float(w.sum())
    for i, p in zip(ids, w):
        r -= p
        if r <= 0:
            return i
    return ids[-1]
