"""Other arrangements of a layer's parts, defined and registered here without a change to the library: a block whose
mixer and feed-forward read the same norm and add side by side (three parts instead of four), and one with a norm
after the mixer and after the feed-forward as well as before them (six parts).  Both run whole prompts, one-token
steps and the recorded decode runner, against the formulas written out with the plain implementation's functions."""
import math

import numpy as np
import pytest
import torch

import ghost_infer_b200 as gi
from ghost_infer_b200.config import LlamaConfig, register_architecture, unregister_architecture
from ghost_infer_b200.config.llama_spec import build_llama_spec
from ghost_infer_b200.parts import Block, ExtraPart, register, unregister
from ghost_infer_b200.parts.spec import LayerSpec, ModelSpec
from ghost_infer_b200.weights import write_random_model
from conftest import TINY_A, TINY_D
from gpu_helpers import check_logits
import plain_llama as pl

pytestmark = pytest.mark.gpu


class ParallelResidual(Block):
    """x += mixer(n(x)) + ffn(n(x)): one norm, read by both."""

    def forward(self, x, step, memory):
        h = self.mixer_norm.forward(x)
        self.mixer.forward(h, x, step, memory)
        self.ffn.forward(h, x, step)


class SandwichResidual(Block):
    """x += post_a(mixer(pre_a(x))); x += post_b(ffn(pre_b(x))): the mixer and the feed-forward add into a stream of
    their own (zero before), whose norm is then added to x."""

    def forward(self, x, step, memory):
        y = torch.zeros_like(x)
        self.mixer.forward(self.mixer_norm.forward(x), y, step, memory)
        x += self.extra["post_mixer_norm"].forward(y).float()
        y = torch.zeros_like(x)
        self.ffn.forward(self.ffn_norm.forward(x), y, step)
        x += self.extra["post_ffn_norm"].forward(y).float()


def parallel_spec(cfg):
    base = build_llama_spec(cfg)
    layers = tuple(LayerSpec(prefix=ls.prefix, block="toy_parallel", mixer_norm=ls.mixer_norm, mixer=ls.mixer, ffn=ls.ffn)
                   for ls in base.layers)
    return ModelSpec(architecture="ToyParallelForCausalLM", hidden_size=base.hidden_size, vocab_size=base.vocab_size,
                     max_positions=base.max_positions, embedding=base.embedding, layers=layers, schedule=base.schedule,
                     final_norm=base.final_norm, head=base.head)


def sandwich_spec(cfg):
    base = build_llama_spec(cfg)
    layers = tuple(LayerSpec(prefix=ls.prefix, block="toy_sandwich", mixer_norm=ls.mixer_norm, mixer=ls.mixer,
                             ffn_norm=ls.ffn_norm, ffn=ls.ffn,
                             extra=(ExtraPart("post_mixer_norm", "norm", ls.mixer_norm, "post_mixer_norm."),
                                    ExtraPart("post_ffn_norm", "norm", ls.ffn_norm, "post_ffn_norm.")))
                   for ls in base.layers)
    return ModelSpec(architecture="ToySandwichForCausalLM", hidden_size=base.hidden_size, vocab_size=base.vocab_size,
                     max_positions=base.max_positions, embedding=base.embedding, layers=layers, schedule=base.schedule,
                     final_norm=base.final_norm, head=base.head)


def plain_forward(cfg, w, tokens, kind):
    H, KV, hd, eps = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["rms_norm_eps"]
    inv = pl.rotary_inv_freq(hd, cfg["rope_theta"], cfg["rope_scaling"])
    pos = np.arange(len(tokens))
    x = pl.embed(w["model.embed_tokens.weight"], tokens)

    def attn(p, h):
        q = pl.rope(h @ w[p + "self_attn.q_proj.weight"].T, pos, inv, hd)
        k = pl.rope(h @ w[p + "self_attn.k_proj.weight"].T, pos, inv, hd)
        v = h @ w[p + "self_attn.v_proj.weight"].T
        return pl.attention(q, k, v, H, KV, hd, 1 / math.sqrt(hd)) @ w[p + "self_attn.o_proj.weight"].T

    def ffn(p, h):
        return pl.swiglu(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])

    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        if kind == "parallel":
            h = pl.rms_norm(x, w[p + "input_layernorm.weight"], eps)
            x = x + attn(p, h) + ffn(p, h)
        else:
            a = attn(p, pl.rms_norm(x, w[p + "input_layernorm.weight"], eps))
            x = x + pl.rms_norm(a, w[p + "post_mixer_norm.weight"], eps)
            f = ffn(p, pl.rms_norm(x, w[p + "post_attention_layernorm.weight"], eps))
            x = x + pl.rms_norm(f, w[p + "post_ffn_norm.weight"], eps)
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else w["lm_head.weight"]
    return pl.rms_norm(x, w["model.norm.weight"], eps) @ head.T


@pytest.mark.parametrize("kind,block,spec", [("parallel", ParallelResidual, parallel_spec), ("sandwich", SandwichResidual, sandwich_spec)])
@pytest.mark.parametrize("base,dtype", [(TINY_A, "float32"), (TINY_D, "bfloat16")])
def test_other_arrangements_of_a_layer(tmp_path, kind, block, spec, base, dtype):
    arch = f"Toy{kind.capitalize()}ForCausalLM"
    register("block", f"toy_{kind}", block)
    register_architecture(arch, LlamaConfig.from_dict, spec)
    try:
        raw = dict(base, architectures=[arch])
        d = str(tmp_path / kind)
        write_random_model(d, raw, seed=11, dtype=dtype, std=0.05, norm_jitter=0.1)
        model = gi.Model.from_pretrained(d, dtype=dtype)
        names = {t.name for t in model.weight_manifest()}
        if kind == "parallel":
            assert not any("post_attention_layernorm" in n for n in names)          # the layer has one norm only
        else:
            assert "model.layers.0.post_mixer_norm.weight" in names and "model.layers.1.post_ffn_norm.weight" in names
        cfg, w = pl.read_model(d)
        llm = gi.LLM(model, dtype=dtype, max_tokens=64 * 12)
        eng, cache = llm.engine, llm.cache
        rng = np.random.default_rng(5)
        seqs = [rng.integers(0, raw["vocab_size"], n).tolist() for n in (90, 30)]
        refs = [plain_forward(cfg, w, t, kind) for t in seqs]
        slots = [cache.open_slot() for _ in seqs]
        cut = [70, 30]
        out = eng.step([gi.StepEntry(s, t[:c], list(range(c))) for s, t, c in zip(slots, seqs, cut)]).cpu().numpy()
        got = [[out[:70]], [out[70:]]]
        got[0].append(eng.step([gi.StepEntry(slots[0], [seqs[0][70]], [0])]).cpu().numpy())     # a plain one-token step
        runner = eng.decoder([slots[0]])                                                       # then the recorded ones
        for j in range(71, 90):
            got[0].append(runner.forward(tokens=[seqs[0][j]]).cpu().numpy())
        for i in range(2):
            check_logits(np.concatenate(got[i]), refs[i], dtype, f"{kind} {dtype} request {i}")
        for s in slots:
            cache.close_slot(s)
    finally:
        unregister("block", f"toy_{kind}")
        unregister_architecture(arch)
