"""Ways of cutting and batching the work that the other engine tests do not take, each against the plain
implementation: a sequence rewound and continued with other tokens (the reference lowers `pos` and goes on,
src/model.rs:799-821, src/cuda.rs:10202-10219); several sequences read in chunks through the generation loop, each at
a place of its own (src/cuda.rs:8543-8565); one step that holds sequences under way and a fresh prompt; the graph
runner across its length buckets; a model with a window through the entry point."""
import math

import numpy as np
import pytest
import torch

import ghost_infer_b200 as gi
from ghost_infer_b200.cache import pages_for
from ghost_infer_b200.config import LlamaConfig, register_architecture, unregister_architecture
from ghost_infer_b200.config.llama_spec import build_llama_spec
from ghost_infer_b200.engine.generate import GenerationLoop
from ghost_infer_b200.parts import PartSpec
from ghost_infer_b200.parts.spec import LayerSpec, ModelSpec
from ghost_infer_b200.sampling import DeviceSampler, SamplingParams
from ghost_infer_b200.weights import write_random_model
from conftest import TINY_A, TINY_D
from gpu_helpers import check_logits, make_engine, oracle, plain_logits, tokens_for
from test_gpu_model import poison_free_pages
import plain_llama as pl

pytestmark = pytest.mark.gpu

CASES = [("A", "float32"), ("B", "float32"), ("A", "bfloat16"), ("B", "bfloat16"), ("D", "bfloat16"), ("E", "bfloat16"),
         ("D", "float32"), ("E", "float32")]


@pytest.fixture(scope="module")
def engines(model_dirs):
    made = {}

    def get(name, dtype, **kw):
        key = (name, dtype, tuple(sorted(kw.items())))
        if key not in made:
            d = model_dirs(name, dtype)
            made[key] = (make_engine(d, dtype, **kw), d)
        return made[key]

    return get


def feed(eng, slot, toks, chunk):
    """The tokens in chunks of `chunk` (1: one-token steps), logits at every place."""
    outs = []
    for i in range(0, len(toks), chunk):
        part = toks[i:i + chunk]
        outs.append(eng.step([gi.StepEntry(slot, part, list(range(len(part))))]).cpu().numpy())
    return np.concatenate(outs)


# ---- (a) rewind, then other tokens --------------------------------------------------------------------------
@pytest.mark.parametrize("name,dtype", CASES)
def test_rewind_then_continue_with_other_tokens(engines, tiny_configs, name, dtype):
    """A prompt and twenty steps; the slot is rewound to a place inside an earlier page; a neighbour takes the pages
    that came back and fills them; the first sequence goes on with other tokens, in a chunk and in single steps.
    Then the same slot starts over after `reset`, without being closed.  Free pages hold NaN throughout."""
    eng, d = engines(name, dtype)
    cfg, cache = tiny_configs[name], eng.cache
    first = tokens_for(cfg, 150, 31)
    a = cache.open_slot()
    got = np.concatenate([feed(eng, a, first[:130], 130), feed(eng, a, first[130:150], 1)])
    check_logits(got, plain_logits(d, first), dtype, f"{name} {dtype} before the rewind")
    held = list(cache.groups[0].pages[a])
    assert len(held) == 3
    assert cache.truncate(a, 50) == 50 and cache.length(a) == 50         # inside the first page
    assert len(cache.groups[0].pages[a]) == 1 and cache.free_pages == cache.n_pages - 1
    poison_free_pages(eng)
    # a neighbour takes the pages that came back, and writes its own keys and values there
    b = cache.open_slot()
    other = tokens_for(cfg, 100, 32)
    got_b = feed(eng, b, other[:90], 90)
    assert set(cache.groups[0].pages[b]) == set(held[1:])
    # the first sequence goes on from position 50 with other tokens; it needs new pages, which are not its old ones
    second = first[:50] + tokens_for(cfg, 100, 33)
    got_a = np.concatenate([feed(eng, a, second[50:110], 60), feed(eng, a, second[110:150], 1)])
    got_b = np.concatenate([got_b, feed(eng, b, other[90:], 1)])
    check_logits(got_a, plain_logits(d, second)[50:], dtype, f"{name} {dtype} after the rewind")
    check_logits(got_b, plain_logits(d, other), dtype, f"{name} {dtype} the neighbour")
    # rewinding to where it stands, or further than it is, changes nothing
    assert cache.truncate(a, 150) == 150 and cache.truncate(a, 400) == 150
    # the slot starts over: no close, no open
    cache.reset(a)
    assert cache.length(a) == 0 and cache.slots.live(a)
    poison_free_pages(eng)
    third = tokens_for(cfg, 80, 34)
    got = np.concatenate([feed(eng, a, third[:70], 70), feed(eng, a, third[70:], 1)])
    check_logits(got, plain_logits(d, third), dtype, f"{name} {dtype} after the reset")
    # a rewind by a few tokens inside the last page, as a caller that takes back a reply's tail does
    assert cache.truncate(a, 75) == 75
    fourth = third[:75] + tokens_for(cfg, 6, 35)
    check_logits(feed(eng, a, fourth[75:], 1), plain_logits(d, fourth)[75:], dtype, f"{name} {dtype} short rewind")
    cache.close_slot(a)
    cache.close_slot(b)
    assert cache.free_pages == cache.n_pages


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("D", "bfloat16")])
def test_rewind_through_the_graph_runner(engines, tiny_configs, name, dtype):
    """The runner that generation uses, rewound between its steps: its graph reads lengths and pages anew."""
    eng, d = engines(name, dtype)
    cfg, cache = tiny_configs[name], eng.cache
    seqs = [tokens_for(cfg, 140, 36), tokens_for(cfg, 140, 37)]
    slots = [cache.open_slot() for _ in seqs]
    eng.step([gi.StepEntry(s, t[:100], []) for s, t in zip(slots, seqs)])
    runner = eng.decoder(slots)
    for j in range(100, 140):
        runner.forward(tokens=[t[j] for t in seqs])
    assert cache.truncate(slots[0], 60) == 60 and cache.truncate(slots[1], 110) == 110
    poison_free_pages(eng)
    new = [seqs[0][:60] + tokens_for(cfg, 40, 38), seqs[1][:110] + tokens_for(cfg, 40, 39)]
    refs = [plain_logits(d, t) for t in new]
    got = [[], []]
    for j in range(40):
        lg = runner.forward(tokens=[new[0][60 + j], new[1][110 + j]]).cpu().numpy()
        got[0].append(lg[0])
        got[1].append(lg[1])
    check_logits(np.stack(got[0]), refs[0][60:], dtype, f"{name} {dtype} runner after a rewind, request 0")
    check_logits(np.stack(got[1]), refs[1][110:], dtype, f"{name} {dtype} runner after a rewind, request 1")
    for s in slots:
        cache.close_slot(s)


# ---- (b) several sequences read in chunks -----------------------------------------------------------------------
class _GreedyOnDevice:
    def __init__(self, device):
        self.inner = DeviceSampler(SamplingParams(temperature=0.0, top_k=0, top_p=1.0, seed=1), device)

    def start(self, n):
        self.inner.start(n)

    def pick(self, logits, ids):
        return self.inner.pick(logits, ids)


@pytest.mark.parametrize("name,dtype", CASES[:6])
@pytest.mark.parametrize("limit", [7, 48, 64])
def test_several_sequences_read_in_chunks(engines, tiny_configs, name, dtype, limit):
    """The generation loop's own way of reading prompts with a bound on the tokens of a step: sequences stand at
    unequal places inside their prompts, a step gives some of them nothing, and a sequence's last chunk shares a step
    with another's first.  The logits after each prompt, and those of steps that follow (which read everything the
    chunks stored), are compared."""
    eng, d = engines(name, dtype)
    cfg, cache = tiny_configs[name], eng.cache
    lens = [150, 40, 97, 5]
    seqs = [tokens_for(cfg, n + 6, 60 + i) for i, n in enumerate(lens)]
    prompts = [t[:n] for t, n in zip(seqs, lens)]
    loop = GenerationLoop(eng, _GreedyOnDevice(eng.device), batch_size=4, max_step_tokens=limit)
    poison_free_pages(eng)
    slots = {i: cache.open_slot() for i in range(4)}
    steps_before = loop.stats.steps
    logits = loop._read_prompts(prompts, slots, [0, 1, 2, 3]).cpu().numpy()
    assert loop.stats.steps - steps_before == math.ceil(sum(lens) / limit)
    refs = [plain_logits(d, t) for t in seqs]
    for i in range(4):
        assert cache.length(slots[i]) == lens[i]
        check_logits(logits[i:i + 1], refs[i][lens[i] - 1:lens[i]], dtype, f"{name} {dtype} limit {limit} prompt {i}")
    got = [[] for _ in seqs]
    for j in range(6):
        out = eng.step([gi.StepEntry(slots[i], [seqs[i][lens[i] + j]], [0]) for i in range(4)]).cpu().numpy()
        for i in range(4):
            got[i].append(out[i])
    for i in range(4):
        check_logits(np.stack(got[i]), refs[i][lens[i]:], dtype, f"{name} {dtype} limit {limit} steps after prompt {i}")
    for s in slots.values():
        cache.close_slot(s)


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("D", "bfloat16")])
def test_generation_with_chunked_prompts_gives_the_same_tokens(model_dirs, tiny_configs, name, dtype):
    from test_gpu_generate import plain_greedy
    d = model_dirs(name, dtype)
    cfg = tiny_configs[name]
    llm = gi.LLM(d, dtype=dtype, max_tokens=64 * 32, max_seq_len=256, beyond_trained_positions=True)
    prompts = [tokens_for(cfg, n, 80 + i) for i, n in enumerate([130, 33, 70, 2])]
    whole = llm.generate(prompts, max_new=6, temperature=0.0, stop_token_ids=(), batch_size=4)
    cut = llm.generate(prompts, max_new=6, temperature=0.0, stop_token_ids=(), batch_size=4, max_step_tokens=50)
    for p, a, b in zip(prompts, whole, cut):
        want, _, margins = plain_greedy(d, p, 6)
        sure = 6
        if dtype == "bfloat16":
            near = [i for i, m in enumerate(margins) if m < 0.05]
            sure = near[0] if near else 6
        assert a.tokens[:sure] == want[:sure] and b.tokens[:sure] == want[:sure], (a.tokens, b.tokens, want)
    assert llm.cache.free_pages == llm.cache.n_pages


# ---- (c) sequences under way and a fresh prompt in one step -------------------------------------------------
@pytest.mark.parametrize("name,dtype", CASES)
def test_one_step_with_sequences_under_way_and_a_fresh_prompt(engines, tiny_configs, name, dtype):
    eng, d = engines(name, dtype)
    cfg, cache = tiny_configs[name], eng.cache
    seqs = [tokens_for(cfg, 45, 90), tokens_for(cfg, 135, 91), tokens_for(cfg, 70, 92), tokens_for(cfg, 3, 93)]
    refs = [plain_logits(d, t) for t in seqs]
    poison_free_pages(eng)
    s0, s1 = cache.open_slot(), cache.open_slot()
    eng.step([gi.StepEntry(s0, seqs[0][:40], []), gi.StepEntry(s1, seqs[1][:128], [])])
    s2, s3 = cache.open_slot(), cache.open_slot()
    # in the order of slots 2, 0, 3, 1: a fresh prompt first, the two under way between and after the fresh ones
    out = eng.step([gi.StepEntry(s2, seqs[2], list(range(70))), gi.StepEntry(s0, [seqs[0][40]], [0]),
                    gi.StepEntry(s3, seqs[3][:2], [1]), gi.StepEntry(s1, [seqs[1][128]], [0])]).cpu().numpy()
    check_logits(out[:70], refs[2], dtype, f"{name} {dtype} the fresh prompt")
    check_logits(out[70:71], refs[0][40:41], dtype, f"{name} {dtype} under way at 40")
    check_logits(out[71:72], refs[3][1:2], dtype, f"{name} {dtype} a two-token prompt")
    check_logits(out[72:73], refs[1][128:129], dtype, f"{name} {dtype} under way at 128, first row of a page")
    # and on: one token each for the first two, the rest of the short prompt
    out = eng.step([gi.StepEntry(s0, [seqs[0][41]], [0]), gi.StepEntry(s1, [seqs[1][129]], [0]),
                    gi.StepEntry(s3, seqs[3][2:], [0])]).cpu().numpy()
    check_logits(out, np.stack([refs[0][41], refs[1][129], refs[3][2]]), dtype, f"{name} {dtype} the step after")
    for s in (s0, s1, s2, s3):
        cache.close_slot(s)


# ---- (d) the graph runner across its length buckets ---------------------------------------------------------
@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "bfloat16"), ("D", "bfloat16"), ("E", "bfloat16"), ("E", "float32")])
def test_graph_runner_across_length_buckets(engines, tiny_configs, name, dtype):
    """Three sequences decode from positions 200, 30 and 100 to 620, 450 and 520: the longest crosses the buckets at 256
    and 512 (a new slice count, a new graph, an eager first step in mid-sequence), pages 4 to 10 are taken on the way."""
    eng, d = engines(name, dtype)
    cfg, cache = tiny_configs[name], eng.cache
    starts, steps = [200, 30, 100], 420
    seqs = [tokens_for(cfg, s + steps, 110 + i) for i, s in enumerate(starts)]
    refs = [plain_logits(d, t) for t in seqs]
    poison_free_pages(eng)
    slots = [cache.open_slot() for _ in seqs]
    eng.step([gi.StepEntry(s, t[:n], []) for s, t, n in zip(slots, seqs, starts)])
    runner = eng.decoder(slots)
    got = [[] for _ in seqs]
    graphs_before = len(eng._decode_graphs)
    for j in range(steps):
        lg = runner.forward(tokens=[t[n + j] for t, n in zip(seqs, starts)]).cpu().numpy()
        for i in range(3):
            got[i].append(lg[i])
    for i in range(3):
        check_logits(np.stack(got[i]), refs[i][starts[i]:], dtype, f"{name} {dtype} runner request {i}")
    if dtype == "float32":
        assert len(eng._decode_graphs) - graphs_before >= 2          # 32-bit slices follow the bucket: 256, 512, 1024
    for s in slots:
        cache.close_slot(s)


@pytest.mark.parametrize("name", ["D", "E"])
def test_decode_with_the_rotation_left_to_the_attention(model_dirs, tiny_configs, name):
    """The position encoding may leave a decode step's rotation and cache write to the attention kernel
    (`PositionEncoding.left_to_attention`, switched by `TUNE["attn_rope_inside"]`): through the runner that generation
    uses, across a page edge and a bucket edge, the logits are those of the plain implementation and, bit for bit,
    those of the step with the rotary kernel; one launch per layer fewer."""
    from ghost_infer_b200.kernels import ops
    cfg = tiny_configs[name]
    d = model_dirs(name, "bfloat16")
    starts, steps = [250, 61, 1], 70
    seqs = [tokens_for(cfg, s + steps, 130 + i) for i, s in enumerate(starts)]
    refs = [plain_logits(d, t) for t in seqs]
    outs, launches = [], []
    was = ops.TUNE["attn_rope_inside"], ops.TUNE["attn_keys_on_rows"]
    try:
        ops.TUNE["attn_keys_on_rows"] = False           # the kernel that can rotate by itself, in both runs
        for inside in (False, True):
            ops.TUNE["attn_rope_inside"] = inside
            eng = make_engine(d, "bfloat16")            # a fresh engine: recorded steps keep the kernels they were recorded with
            cache = eng.cache
            slots = [cache.open_slot() for _ in seqs]
            eng.step([gi.StepEntry(s, t[:n], []) for s, t, n in zip(slots, seqs, starts)])
            runner = eng.decoder(slots)
            got = []
            for j in range(steps):
                got.append(runner.forward(tokens=[t[n + j] for t, n in zip(seqs, starts)]).cpu().numpy().copy())
            outs.append(np.stack(got))
            launches.append(runner.launches_per_step())
            for s in slots:
                cache.close_slot(s)
    finally:
        ops.TUNE["attn_rope_inside"], ops.TUNE["attn_keys_on_rows"] = was
    for i in range(3):
        check_logits(outs[1][:, i], refs[i][starts[i]:], "bfloat16", f"{name} rotation inside the attention, request {i}")
    assert np.array_equal(outs[0], outs[1])
    assert launches[0] - launches[1] == cfg["num_hidden_layers"]


# ---- (e) a model with a window, through the entry point ------------------------------------------------------
def window_spec_for(window):
    def build(cfg):
        base = build_llama_spec(cfg)
        layers = []
        for ls in base.layers:
            mixer = PartSpec("gqa_attention", dict(ls.mixer.params, window=window))
            layers.append(LayerSpec(prefix=ls.prefix, block=ls.block, mixer_norm=ls.mixer_norm, mixer=mixer,
                                    ffn_norm=ls.ffn_norm, ffn=ls.ffn))
        return ModelSpec(architecture=f"ToyWindow{window}ForCausalLM", hidden_size=base.hidden_size,
                         vocab_size=base.vocab_size, max_positions=base.max_positions, embedding=base.embedding,
                         layers=tuple(layers), schedule=base.schedule, final_norm=base.final_norm, head=base.head)
    return build


def plain_window_forward(cfg, w, tokens, window):
    H, KV, hd, eps = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["rms_norm_eps"]
    inv = pl.rotary_inv_freq(hd, cfg["rope_theta"], cfg["rope_scaling"])
    pos = np.arange(len(tokens))
    x = pl.embed(w["model.embed_tokens.weight"], tokens)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        h = pl.rms_norm(x, w[p + "input_layernorm.weight"], eps)
        q = pl.rope(h @ w[p + "self_attn.q_proj.weight"].T, pos, inv, hd)
        k = pl.rope(h @ w[p + "self_attn.k_proj.weight"].T, pos, inv, hd)
        v = h @ w[p + "self_attn.v_proj.weight"].T
        x = x + pl.attention(q, k, v, H, KV, hd, 1 / math.sqrt(hd), window=window) @ w[p + "self_attn.o_proj.weight"].T
        h = pl.rms_norm(x, w[p + "post_attention_layernorm.weight"], eps)
        x = x + pl.swiglu(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else w["lm_head.weight"]
    return pl.rms_norm(x, w["model.norm.weight"], eps) @ head.T


@pytest.mark.parametrize("window", [37, 100])
@pytest.mark.parametrize("base,dtype", [(TINY_A, "float32"), (TINY_D, "bfloat16"), (TINY_D, "float32")])
def test_a_window_model_through_the_engine_and_the_entry_point(tmp_path, base, dtype, window):
    """Attention with a window in every layer.  The pool is small, so the pages a sequence gives back once its
    window has passed them are taken by its neighbour while it keeps attending; prompts are read in steps of 2 and
    of 48 tokens (chunks shorter and longer than the window), then 300 tokens are decoded through the graph runner;
    then greedy generation through `LLM.generate`."""
    arch = f"ToyWindow{window}ForCausalLM"
    register_architecture(arch, LlamaConfig.from_dict, window_spec_for(window))
    try:
        raw = dict(base, architectures=[arch], max_position_embeddings=1024)
        d = str(tmp_path / "win")
        write_random_model(d, raw, seed=6, dtype=dtype, std=0.05, norm_jitter=0.1)
        cfg, w = pl.read_model(d)
        model = gi.Model.from_pretrained(d, dtype=dtype)
        # a window of w needs at most ceil((w + 63) / 64) + 1 pages per sequence at any time; two sequences, one spare
        per_seq = (window + 63) // 64 + 2
        cache = model.new_cache(max_tokens=64 * (2 * per_seq + 1), max_slots=2, max_seq_len=1024)
        assert cache.groups[0].request.kind == "window"
        eng = gi.Engine(model, cache)
        for limit in (2, 48):
            seqs = [tokens_for(raw, 150 + 300, 120 + limit), tokens_for(raw, 90 + 300, 121 + limit)]
            refs = [plain_window_forward(cfg, w, t, window) for t in seqs]
            poison_free_pages(eng)
            slots = {0: cache.open_slot(), 1: cache.open_slot()}
            loop = GenerationLoop(eng, _GreedyOnDevice(eng.device), batch_size=2, max_step_tokens=limit)
            lg = loop._read_prompts([seqs[0][:150], seqs[1][:90]], slots, [0, 1]).cpu().numpy()
            check_logits(lg, np.stack([refs[0][149], refs[1][89]]), dtype, f"window {window} limit {limit} prompts")
            runner = eng.decoder([slots[0], slots[1]])
            got = [[], []]
            for j in range(300):
                out = runner.forward(tokens=[seqs[0][150 + j], seqs[1][90 + j]]).cpu().numpy()
                got[0].append(out[0])
                got[1].append(out[1])
                if j % 50 == 0:
                    poison_free_pages(eng)
            check_logits(np.stack(got[0]), refs[0][150:], dtype, f"window {window} limit {limit} request 0")
            check_logits(np.stack(got[1]), refs[1][90:], dtype, f"window {window} limit {limit} request 1")
            # the two sequences went through more pages than the pool has: pages were given back and used again
            assert pages_for(450) + pages_for(390) > cache.n_pages and cache.free_pages >= cache.n_pages - 2 * per_seq
            for s in slots.values():
                cache.close_slot(s)
            assert cache.free_pages == cache.n_pages
        del eng, cache, model
        # through the entry point: greedy tokens against the plain implementation
        llm = gi.LLM(d, dtype=dtype, max_tokens=64 * 12, max_seq_len=1024)
        prompts = [tokens_for(raw, n, 130 + i) for i, n in enumerate([140, 20])]
        res = llm.generate(prompts, max_new=24, temperature=0.0, stop_token_ids=(), batch_size=2, max_step_tokens=64)
        for p, r in zip(prompts, res):
            toks = list(p)
            for i, got_tok in enumerate(r.tokens):
                logits = plain_window_forward(cfg, w, toks, window)[-1]
                order = np.argsort(-logits, kind="stable")
                if got_tok != int(order[0]):
                    margin = logits[order[0]] - logits[order[1]]
                    assert dtype == "bfloat16" and margin < 0.05 and got_tok == int(order[1]), (i, got_tok, int(order[0]), margin)
                toks.append(got_tok)
            assert len(r.tokens) == 24 and r.finish_reason == "length"
        assert llm.cache.free_pages == llm.cache.n_pages
    finally:
        unregister_architecture(arch)
