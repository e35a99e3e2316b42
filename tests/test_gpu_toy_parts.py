"""Parts and whole architectures that the library does not know are defined here, registered, built and
stepped, without a change to the library's files: a mixer with fixed-size state of its own (no cache), a
layer order that names a layer twice, and a layer that reads another layer's cache."""
import math

import numpy as np
import pytest
import torch

import ghost_infer_b200 as gi
from ghost_infer_b200.cache import StateRequest
from ghost_infer_b200.config import LlamaConfig, register_architecture, unregister_architecture
from ghost_infer_b200.config.llama_spec import build_llama_spec
from ghost_infer_b200.parts import Mixer, PartSpec, ScheduleEntry, WeightSpec, register, unregister
from ghost_infer_b200.parts.spec import LayerSpec, ModelSpec
from ghost_infer_b200.weights import write_random_model
from conftest import TINY_A
from gpu_helpers import check_logits
import plain_llama as pl

pytestmark = pytest.mark.gpu
DECAY = 0.5


class DecayMixer(Mixer):
    """state <- DECAY * state + h_t, token by token; output W state.  Its memory is one vector per sequence."""

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.d = int(params["hidden_size"])

    def weights(self):
        return [WeightSpec(self.prefix + "toy.weight", (self.d, self.d))]

    def state_request(self):
        return StateRequest((self.d,), torch.float32)

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.w = rt.place(tensors[self.prefix + "toy.weight"]).float()

    def forward(self, h, residual, step, memory):
        o = 0
        for slot, n in zip(step.host_slots, step.host_q_lens):
            s = memory.state[slot]
            rows = []
            for t in range(n):
                s = DECAY * s + h[o + t].float()
                rows.append(s)
            memory.state[slot] = s
            residual[o:o + n] += torch.stack(rows) @ self.w.T
            o += n


def toy_spec(cfg):
    base = build_llama_spec(cfg)
    layers = list(base.layers)
    l1 = layers[1]
    layers[1] = LayerSpec(prefix=l1.prefix, block=l1.block, mixer_norm=l1.mixer_norm,
                          mixer=PartSpec("toy_decay", {"hidden_size": cfg.hidden_size}), ffn_norm=l1.ffn_norm, ffn=l1.ffn)
    return ModelSpec(architecture="ToyStateForCausalLM", hidden_size=base.hidden_size, vocab_size=base.vocab_size,
                     max_positions=base.max_positions, embedding=base.embedding, layers=tuple(layers),
                     schedule=base.schedule, final_norm=base.final_norm, head=base.head)


def plain_toy_forward(cfg, w, tokens):
    """Layer 0 as the plain implementation has it; layer 1 with the decaying sum in place of attention."""
    inv = pl.rotary_inv_freq(cfg["head_dim"], cfg["rope_theta"], cfg["rope_scaling"])
    pos = np.arange(len(tokens))
    x = pl.embed(w["model.embed_tokens.weight"], tokens)
    x = pl.layer(x, pos, w, "model.layers.0.", cfg, inv)
    p = "model.layers.1."
    h = pl.rms_norm(x, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
    s = np.zeros(cfg["hidden_size"])
    rows = []
    for t in range(len(tokens)):
        s = DECAY * s + h[t]
        rows.append(s)
    x = x + np.stack(rows) @ w[p + "toy.weight"].T
    h = pl.rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
    x = x + pl.swiglu(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    return pl.rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"]) @ w["lm_head.weight"].T


def test_a_mixer_with_state_of_its_own(tmp_path):
    register("mixer", "toy_decay", DecayMixer)
    register_architecture("ToyStateForCausalLM", LlamaConfig.from_dict, toy_spec)
    try:
        raw = dict(TINY_A, architectures=["ToyStateForCausalLM"])
        d = str(tmp_path / "toy")
        write_random_model(d, raw, seed=3, dtype="float32", std=0.05, norm_jitter=0.1)
        model = gi.Model.from_pretrained(d, dtype="float32")
        assert "model.layers.1.toy.weight" in {w.name for w in model.weight_manifest()}
        assert "model.layers.1.self_attn.q_proj.weight" not in {w.name for w in model.weight_manifest()}
        cache = model.new_cache(max_tokens=64 * 16, max_seq_len=512)
        assert cache.state_bytes_per_sequence() == 64 * 4 and len(cache.groups) == 1 and len(cache.groups[0].entries) == 1
        eng = gi.Engine(model, cache)
        cfg, w = pl.read_model(d)
        rng = np.random.default_rng(0)
        for rnd in range(2):                          # twice: the second batch reuses slots, whose state must start at zero
            seqs = [rng.integers(0, 256, n).tolist() for n in (40, 9, 70)]
            slots = [cache.open_slot() for _ in seqs]
            cut = [30, 9, 1]
            out = eng.step([gi.StepEntry(s, t[:c], list(range(c))) for s, t, c in zip(slots, seqs, cut)]).cpu().numpy()
            got, o = [], 0
            for c in cut:
                got.append([out[o:o + c]])
                o += c
            fed = list(cut)
            while any(f < len(t) for f, t in zip(fed, seqs)):
                live = [i for i in range(3) if fed[i] < len(seqs[i])]
                out = eng.step([gi.StepEntry(slots[i], [seqs[i][fed[i]]], [0]) for i in live]).cpu().numpy()
                for r, i in enumerate(live):
                    got[i].append(out[r:r + 1])
                    fed[i] += 1
            for i, t in enumerate(seqs):
                check_logits(np.concatenate(got[i]), plain_toy_forward(cfg, w, t), "float32", f"toy round {rnd} request {i}")
            for s in slots:
                cache.close_slot(s)
    finally:
        unregister("mixer", "toy_decay")
        unregister_architecture("ToyStateForCausalLM")


def shared_spec(cfg):
    """Three runs over two layers: layer 0, layer 1, then layer 0 again reading the cache of its first run."""
    base = build_llama_spec(cfg)
    return ModelSpec(architecture="ToySharedForCausalLM", hidden_size=base.hidden_size, vocab_size=base.vocab_size,
                     max_positions=base.max_positions, embedding=base.embedding, layers=base.layers,
                     schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0, memory_of=0), ScheduleEntry(1)),
                     final_norm=base.final_norm, head=base.head)


def plain_shared_forward(cfg, w, tokens):
    H, KV, hd, eps = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["rms_norm_eps"]
    inv = pl.rotary_inv_freq(hd, cfg["rope_theta"], cfg["rope_scaling"])
    pos = np.arange(len(tokens))
    x = pl.embed(w["model.embed_tokens.weight"], tokens)
    kept = {}

    def run(x, layer, keep=None, reuse=None):
        p = f"model.layers.{layer}."
        h = pl.rms_norm(x, w[p + "input_layernorm.weight"], eps)
        q = pl.rope(h @ w[p + "self_attn.q_proj.weight"].T, pos, inv, hd)
        if reuse is None:
            k = pl.rope(h @ w[p + "self_attn.k_proj.weight"].T, pos, inv, hd)
            v = h @ w[p + "self_attn.v_proj.weight"].T
        else:
            k, v = kept[reuse]
        if keep is not None:
            kept[keep] = (k, v)
        x = x + pl.attention(q, k, v, H, KV, hd, 1 / math.sqrt(hd)) @ w[p + "self_attn.o_proj.weight"].T
        h = pl.rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
        return x + pl.swiglu(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])

    x = run(x, 0, keep=0)
    x = run(x, 1)
    x = run(x, 0, reuse=0)       # same weights, the first run's keys and values
    x = run(x, 1)                # same weights as the second run, a cache of its own
    return pl.rms_norm(x, w["model.norm.weight"], eps) @ w["lm_head.weight"].T


def test_a_layer_named_twice_and_a_shared_cache(tmp_path):
    register_architecture("ToySharedForCausalLM", LlamaConfig.from_dict, shared_spec)
    try:
        raw = dict(TINY_A, architectures=["ToySharedForCausalLM"])
        d = str(tmp_path / "shared")
        write_random_model(d, raw, seed=4, dtype="float32", std=0.05, norm_jitter=0.1)
        model = gi.Model.from_pretrained(d, dtype="float32")
        cache = model.new_cache(max_tokens=64 * 8, max_seq_len=512)
        assert len(cache.groups[0].entries) == 3          # three runs keep keys and values, the fourth borrows
        eng = gi.Engine(model, cache)
        cfg, w = pl.read_model(d)
        toks = np.random.default_rng(1).integers(0, 256, 80).tolist()
        s = cache.open_slot()
        outs = [eng.step([gi.StepEntry(s, toks[:50], list(range(50)))]).cpu().numpy()]
        for t in toks[50:]:
            outs.append(eng.step([gi.StepEntry(s, [t], [0])]).cpu().numpy())
        cache.close_slot(s)
        check_logits(np.concatenate(outs), plain_shared_forward(cfg, w, toks), "float32", "shared cache")
    finally:
        unregister_architecture("ToySharedForCausalLM")


# ---------------------------------------------------------------------------------------------------------
# A feed-forward with routing and another position encoding, both defined here.
from ghost_infer_b200.kernels import ops as _ops
from ghost_infer_b200.parts import FeedForward, PositionEncoding


class RoutedFfn(FeedForward):
    """Two experts, each one matrix; a router (32-bit logits) sends every token to the expert with the higher
    logit; the expert's output is scaled by the softmax weight of that logit."""

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.d = int(params["hidden_size"])
        self.n = int(params["experts"])

    def weights(self):
        return [WeightSpec(self.prefix + "moe.router.weight", (self.n, self.d))] + \
               [WeightSpec(self.prefix + f"moe.experts.{e}.weight", (self.d, self.d)) for e in range(self.n)]

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.router = rt.place(tensors[self.prefix + "moe.router.weight"]).float()
        self.experts = torch.stack([rt.place(tensors[self.prefix + f"moe.experts.{e}.weight"]).float() for e in range(self.n)])

    def forward(self, h, residual, step):
        x = h.float()
        logits = x @ self.router.T                              # router logits in 32-bit
        weight, pick = torch.softmax(logits, -1).max(-1)
        out = torch.einsum("td,tod->to", x, self.experts[pick])
        residual += out * weight[:, None]


class ScaledPositions(PositionEncoding):
    """No rotation: queries are scaled by 1 + slope * position (so scores depend on where the query stands)."""

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.slope = float(params["slope"])

    def encode_and_store(self, qkv, step, memory, n_heads, n_kv_heads, head_dim):
        q = qkv[:, :n_heads * head_dim]
        q.mul_((1.0 + self.slope * step.positions.float())[:, None].to(q.dtype))
        _ops.rope_cache_write(qkv, None, step.positions, step.token_slots, memory.block_table, memory.k, memory.v,
                              n_heads, n_kv_heads, head_dim, 0, False, memory.writes and memory.k is not None)


def routed_spec(cfg):
    base = build_llama_spec(cfg)
    layers = []
    for i, ls in enumerate(base.layers):
        mixer = PartSpec("gqa_attention", dict(ls.mixer.params, position=PartSpec("scaled_positions", {"slope": 0.02})))
        ffn = PartSpec("toy_routed", {"hidden_size": cfg.hidden_size, "experts": 2}) if i == 1 else ls.ffn
        layers.append(LayerSpec(prefix=ls.prefix, block=ls.block, mixer_norm=ls.mixer_norm, mixer=mixer,
                                ffn_norm=ls.ffn_norm, ffn=ffn))
    return ModelSpec(architecture="ToyRoutedForCausalLM", hidden_size=base.hidden_size, vocab_size=base.vocab_size,
                     max_positions=base.max_positions, embedding=base.embedding, layers=tuple(layers),
                     schedule=base.schedule, final_norm=base.final_norm, head=base.head)


def plain_routed_forward(cfg, w, tokens):
    H, KV, hd, eps = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["rms_norm_eps"]
    pos = np.arange(len(tokens))
    x = pl.embed(w["model.embed_tokens.weight"], tokens)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        h = pl.rms_norm(x, w[p + "input_layernorm.weight"], eps)
        q = (h @ w[p + "self_attn.q_proj.weight"].T) * (1.0 + 0.02 * pos)[:, None]
        k, v = h @ w[p + "self_attn.k_proj.weight"].T, h @ w[p + "self_attn.v_proj.weight"].T
        x = x + pl.attention(q, k, v, H, KV, hd, 1 / math.sqrt(hd)) @ w[p + "self_attn.o_proj.weight"].T
        h = pl.rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
        if i == 1:
            logits = h @ w[p + "moe.router.weight"].T
            e = np.exp(logits - logits.max(-1, keepdims=True))
            prob = e / e.sum(-1, keepdims=True)
            pick = prob.argmax(-1)
            out = np.stack([w[p + f"moe.experts.{pick[t]}.weight"] @ h[t] for t in range(len(tokens))])
            x = x + out * prob.max(-1)[:, None]
        else:
            x = x + pl.swiglu(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    return pl.rms_norm(x, w["model.norm.weight"], eps) @ w["lm_head.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_routed_feed_forward_and_another_position_encoding(tmp_path, dtype):
    register("feed_forward", "toy_routed", RoutedFfn)
    register("position", "scaled_positions", ScaledPositions)
    register_architecture("ToyRoutedForCausalLM", LlamaConfig.from_dict, routed_spec)
    try:
        raw = dict(TINY_A, architectures=["ToyRoutedForCausalLM"])
        d = str(tmp_path / "routed")
        write_random_model(d, raw, seed=5, dtype=dtype, std=0.05, norm_jitter=0.1)
        model = gi.Model.from_pretrained(d, dtype=dtype)
        names = {w.name for w in model.weight_manifest()}
        assert "model.layers.1.moe.router.weight" in names and "model.layers.1.mlp.gate_proj.weight" not in names
        cache = model.new_cache(max_tokens=64 * 16, max_seq_len=512)
        eng = gi.Engine(model, cache)
        cfg, w = pl.read_model(d)
        rng = np.random.default_rng(2)
        seqs = [rng.integers(0, 256, n).tolist() for n in (70, 12)]
        slots = [cache.open_slot() for _ in seqs]
        cut = [50, 12]
        out = eng.step([gi.StepEntry(s, t[:c], list(range(c))) for s, t, c in zip(slots, seqs, cut)]).cpu().numpy()
        got = [[out[:50]], [out[50:]]]
        runner = eng.decoder([slots[0]])                  # the graph path, with parts the library has never seen
        for j in range(50, 70):
            got[0].append(runner.forward(tokens=[seqs[0][j]]).cpu().numpy())
        for i, t in enumerate(seqs):
            ref = plain_routed_forward(cfg, w, t)
            if dtype == "float32":
                check_logits(np.concatenate(got[i]), ref, "float32", f"routed request {i}")
            else:
                # a 16-bit engine may route a token whose two router logits nearly tie to the other expert
                err = np.abs(np.concatenate(got[i]) - ref).max(-1)
                assert np.median(err) <= 0.025 * max(1.0, np.abs(ref).max()), float(np.median(err))
        for s in slots:
            cache.close_slot(s)
    finally:
        unregister("feed_forward", "toy_routed")
        unregister("position", "scaled_positions")
        unregister_architecture("ToyRoutedForCausalLM")
