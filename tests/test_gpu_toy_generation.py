"""Toy parts through the paths generation takes: the decode runner with and without its CUDA graph, and
`LLM.generate`.  Defined and registered here, none touching the library: an attention and a feed-forward whose
tensors live under other names; a mixer with state that plans its work in Python from the step's host-side lists
(it declares so, and its model then decodes launch by launch); the same mixer working from the device arrays alone
(recorded and replayed, padding rows and all); and one that reads the host lists without declaring it, which must be
refused in words rather than run wrongly."""
import numpy as np
import pytest
import torch

import ghost_infer_b200 as gi
from ghost_infer_b200.cache import StateRequest
from ghost_infer_b200.config import LlamaConfig, register_architecture, unregister_architecture
from ghost_infer_b200.config.llama_spec import build_llama_spec
from ghost_infer_b200.parts import Mixer, PartSpec, WeightSpec, register, unregister
from ghost_infer_b200.parts.spec import LayerSpec, ModelSpec
from ghost_infer_b200.weights import write_random_model
from conftest import TINY_A
from gpu_helpers import check_logits
import plain_llama as pl

pytestmark = pytest.mark.gpu
DECAY = 0.5


# ---- other tensor names ---------------------------------------------------------------------------------
ATTN_NAMES = {"q": "attn.wq.weight", "k": "attn.wk.weight", "v": "attn.wv.weight", "o": "attn.wo.weight"}
FFN_NAMES = {"gate": "ffn.w1.weight", "up": "ffn.w3.weight", "down": "ffn.w2.weight"}


def renamed_spec(cfg):
    base = build_llama_spec(cfg)
    layers = []
    for i, ls in enumerate(base.layers):
        layers.append(LayerSpec(
            prefix=f"blocks.{i}.", block=ls.block,
            mixer_norm=PartSpec("rmsnorm", dict(ls.mixer_norm.params, tensor_names={"weight": "scale"})),
            mixer=PartSpec("gqa_attention", dict(ls.mixer.params, tensor_names=ATTN_NAMES)),
            ffn_norm=PartSpec("rmsnorm", dict(ls.ffn_norm.params, tensor_names={"weight": "scale"})),
            ffn=PartSpec("swiglu", dict(ls.ffn.params, tensor_names=FFN_NAMES)),
            mixer_norm_prefix="norm1.", ffn_norm_prefix="norm2."))
    return ModelSpec(architecture="ToyRenamedForCausalLM", hidden_size=base.hidden_size, vocab_size=base.vocab_size,
                     max_positions=base.max_positions,
                     embedding=PartSpec("token_embedding", dict(base.embedding.params, tensor_names={"weight": "table"})),
                     layers=tuple(layers), schedule=base.schedule, final_norm=base.final_norm,
                     head=PartSpec("linear_head", dict(base.head.params, tensor_names={"weight": "out"})),
                     embedding_prefix="tok.", final_norm_prefix="final.", head_prefix="head.")


def standard_names(w, n_layers):
    """The renamed model's tensors under the names the plain implementation reads."""
    out = {"model.embed_tokens.weight": w["tok.table"], "model.norm.weight": w["final.weight"], "lm_head.weight": w["head.out"]}
    for i in range(n_layers):
        a, b = f"blocks.{i}.", f"model.layers.{i}."
        out[b + "input_layernorm.weight"] = w[a + "norm1.scale"]
        out[b + "post_attention_layernorm.weight"] = w[a + "norm2.scale"]
        for k, sub in ATTN_NAMES.items():
            out[b + f"self_attn.{k}_proj.weight"] = w[a + sub]
        for k, sub in FFN_NAMES.items():
            out[b + f"mlp.{k}_proj.weight"] = w[a + sub]
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_parts_under_other_tensor_names(tmp_path, dtype):
    register_architecture("ToyRenamedForCausalLM", LlamaConfig.from_dict, renamed_spec)
    try:
        raw = dict(TINY_A, architectures=["ToyRenamedForCausalLM"])
        d = str(tmp_path / "renamed")
        write_random_model(d, raw, seed=8, dtype=dtype, std=0.05, norm_jitter=0.1)
        model = gi.Model.from_pretrained(d, dtype=dtype)
        names = {w.name for w in model.weight_manifest()}
        assert {"tok.table", "head.out", "final.weight", "blocks.0.attn.wq.weight", "blocks.1.ffn.w2.weight",
                "blocks.0.norm1.scale"} <= names
        assert not any("self_attn" in n or "mlp." in n or "layernorm" in n for n in names)
        cfg, w = pl.read_model(d)
        w = standard_names(w, cfg["num_hidden_layers"])
        llm = gi.LLM(model, dtype=dtype, max_tokens=64 * 8)
        toks = np.random.default_rng(3).integers(0, 256, 90).tolist()
        s = llm.cache.open_slot()
        out = llm.engine.step([gi.StepEntry(s, toks[:70], list(range(70)))]).cpu().numpy()
        runner = llm.engine.decoder([s])
        rest = [runner.forward(tokens=[t]).cpu().numpy() for t in toks[70:]]
        llm.cache.close_slot(s)
        check_logits(np.concatenate([out] + rest), pl.forward(cfg, w, toks), dtype, "renamed tensors")
    finally:
        unregister_architecture("ToyRenamedForCausalLM")


# ---- a mixer with state, three ways -----------------------------------------------------------------------
class _Decay(Mixer):
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

    def by_host_lists(self, h, residual, step, memory):
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


class HostPlannedDecay(_Decay):
    plans_on_host = True            # forward() loops over the step's host-side lists

    def forward(self, h, residual, step, memory):
        self.by_host_lists(h, residual, step, memory)


class UndeclaredDecay(_Decay):
    def forward(self, h, residual, step, memory):
        self.by_host_lists(h, residual, step, memory)


class DevicePlannedDecay(_Decay):
    """One-token steps work from the device arrays alone (so they can be recorded and replayed); padding rows carry
    slot -1 and land in the state's trash row.  Prompts, which are never recorded, take the host lists."""

    def forward(self, h, residual, step, memory):
        if not step.is_decode:
            return self.by_host_lists(h, residual, step, memory)
        idx = step.token_slots.long()
        s = DECAY * memory.state[idx] + h.float()
        memory.state.index_copy_(0, torch.where(idx < 0, idx + memory.state.shape[0], idx), s)
        residual += s @ self.w.T


def decay_spec(arch, kind):
    def build(cfg):
        base = build_llama_spec(cfg)
        layers = list(base.layers)
        l1 = layers[1]
        layers[1] = LayerSpec(prefix=l1.prefix, block=l1.block, mixer_norm=l1.mixer_norm,
                              mixer=PartSpec(kind, {"hidden_size": cfg.hidden_size}), ffn_norm=l1.ffn_norm, ffn=l1.ffn)
        return ModelSpec(architecture=arch, hidden_size=base.hidden_size, vocab_size=base.vocab_size,
                         max_positions=base.max_positions, embedding=base.embedding, layers=tuple(layers),
                         schedule=base.schedule, final_norm=base.final_norm, head=base.head)
    return build


def plain_decay_forward(cfg, w, tokens):
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


def plain_greedy(cfg, w, prompt, n):
    toks, out = list(prompt), []
    for _ in range(n):
        t = int(np.argsort(-plain_decay_forward(cfg, w, toks)[-1], kind="stable")[0])
        out.append(t)
        toks.append(t)
    return out


@pytest.mark.parametrize("cls,graph_expected", [(HostPlannedDecay, False), (DevicePlannedDecay, True)])
def test_a_mixer_with_state_through_the_runner_and_through_generate(tmp_path, cls, graph_expected):
    arch = f"Toy{cls.__name__}ForCausalLM"
    register("mixer", "toy_decay_gen", cls)
    register_architecture(arch, LlamaConfig.from_dict, decay_spec(arch, "toy_decay_gen"))
    try:
        raw = dict(TINY_A, architectures=[arch])
        d = str(tmp_path / "toy")
        write_random_model(d, raw, seed=9, dtype="float32", std=0.05, norm_jitter=0.1)
        cfg, w = pl.read_model(d)
        llm = gi.LLM(d, dtype="float32", max_tokens=64 * 16)
        eng, cache = llm.engine, llm.cache
        assert eng.plans_on_host == (not graph_expected)
        rng = np.random.default_rng(4)
        # the runner, as generation drives it: three sequences (so a recorded step has a padding row), graph on and off
        for use_graph in (True, False):
            seqs = [rng.integers(0, 256, n).tolist() for n in (60, 25, 41)]
            starts = [30, 5, 40]
            slots = [cache.open_slot() for _ in seqs]
            eng.step([gi.StepEntry(s, t[:n], []) for s, t, n in zip(slots, seqs, starts)])
            runner = eng.decoder(slots, use_graph=use_graph)
            assert runner.use_graph == (use_graph and graph_expected)
            assert runner.rows == (4 if runner.use_graph else 3)
            got = [[] for _ in seqs]
            fed = list(starts)
            live = [0, 1, 2]
            while live:
                out = runner.forward(tokens=[seqs[i][fed[i]] for i in live]).cpu().numpy()
                for r, i in enumerate(live):
                    got[i].append(out[r])
                    fed[i] += 1
                still = [i for i in live if fed[i] < len(seqs[i])]
                if still != live and still:
                    runner = eng.decoder([slots[i] for i in still], use_graph=use_graph)
                live = still
            for i, t in enumerate(seqs):
                check_logits(np.stack(got[i]), plain_decay_forward(cfg, w, t)[starts[i]:], "float32",
                             f"{cls.__name__} graph {use_graph} request {i}")
            for s in slots:
                cache.close_slot(s)
        # and the entry point: two batches one after another, so that slots (and their state rows) are used again
        prompts = [rng.integers(0, 256, n).tolist() for n in (33, 4, 18, 9, 50)]
        res = llm.generate(prompts, max_new=7, temperature=0.0, stop_token_ids=(), batch_size=3)
        for p, r in zip(prompts, res):
            assert r.tokens == plain_greedy(cfg, w, p, 7)
        assert llm.last_stats.batches == 2 and cache.free_pages == cache.n_pages
    finally:
        unregister("mixer", "toy_decay_gen")
        unregister_architecture(arch)


def test_a_part_that_reads_host_lists_without_saying_so_is_refused_in_a_recorded_step(tmp_path):
    arch = "ToyUndeclaredForCausalLM"
    register("mixer", "toy_decay_undeclared", UndeclaredDecay)
    register_architecture(arch, LlamaConfig.from_dict, decay_spec(arch, "toy_decay_undeclared"))
    try:
        raw = dict(TINY_A, architectures=[arch])
        d = str(tmp_path / "toy")
        write_random_model(d, raw, seed=9, dtype="float32", std=0.05, norm_jitter=0.1)
        llm = gi.LLM(d, dtype="float32", max_tokens=64 * 8)
        s = llm.cache.open_slot()
        llm.engine.step([gi.StepEntry(s, [1, 2, 3], [])])           # fine: a plain step has the lists
        with pytest.raises(RuntimeError, match="plans_on_host"):
            llm.engine.decoder([s]).forward(tokens=[4])
        llm.cache.close_slot(s)
    finally:
        unregister("mixer", "toy_decay_undeclared")
        unregister_architecture(arch)
