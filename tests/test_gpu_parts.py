"""Each part alone, built from a `PartSpec` with sizes of its own, against the plain implementation's
function for that part."""
import math

import numpy as np
import pytest
import torch

from ghost_infer_b200.cache import CacheRequest, SequenceCache
from ghost_infer_b200.engine.step import Engine, StepContext, StepEntry
from ghost_infer_b200.parts import PartSpec, Runtime, lookup
import plain_llama as pl

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


def close(got, ref, dtype):
    got, ref = got.double().cpu().numpy(), np.asarray(ref)
    scale = max(1.0, np.abs(ref).max())
    bound = 3e-5 if dtype == torch.float32 else 0.02
    assert np.abs(got - ref).max() <= bound * scale, f"max error {np.abs(got - ref).max():.3e}, scale {scale:.2f}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    part = lookup("norm", "rmsnorm")({"size": 72, "eps": 2e-4}, "blk.n.")
    assert [(w.name, w.shape, w.init) for w in part.weights()] == [("blk.n.weight", (72,), "ones")]
    w = 1 + 0.3 * rnd(72, seed=1)
    part.bind({"blk.n.weight": w.to(dtype)}, Runtime(DEV, dtype))
    x = rnd(5, 72, seed=2, scale=2.0).to(DEV)
    ref = pl.rms_norm(x.double().cpu().numpy(), w.to(dtype).double().numpy(), 2e-4)
    close(part.forward(x), ref, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part(dtype):
    part = lookup("feed_forward", "swiglu")({"hidden_size": 40, "intermediate_size": 100}, "L.")
    names = {w.name: w.shape for w in part.weights()}
    assert names == {"L.mlp.gate_proj.weight": (100, 40), "L.mlp.up_proj.weight": (100, 40), "L.mlp.down_proj.weight": (40, 100)}
    t = {n: (rnd(*s, seed=i + 3, scale=0.2)).to(dtype) for i, (n, s) in enumerate(names.items())}
    part.bind(t, Runtime(DEV, dtype))
    h = rnd(6, 40, seed=9).to(dtype).to(DEV)
    res = rnd(6, 40, seed=10).to(DEV)
    before = res.clone()
    part.forward(h, res, None)
    f = lambda n: t[n].double().numpy()
    ref = pl.swiglu(h.double().cpu().numpy(), f("L.mlp.gate_proj.weight"), f("L.mlp.up_proj.weight"), f("L.mlp.down_proj.weight"))
    close(res - before, ref, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_and_head_parts(dtype):
    emb = lookup("embedding", "token_embedding")({"vocab_size": 77, "hidden_size": 24}, "emb.")
    head = lookup("head", "linear_head")({"vocab_size": 77, "hidden_size": 24, "tied": True}, "out.")
    assert head.weights() == [] and head.ignorable() == ["out.weight"]
    table = rnd(77, 24, seed=1).to(dtype)
    rt = Runtime(DEV, dtype)
    emb.bind({"emb.weight": table}, rt)
    head.bind({}, rt, emb)
    toks = torch.tensor([5, 76, 0], dtype=torch.int32, device=DEV)
    x = emb.forward(toks)
    assert torch.equal(x.cpu(), table[toks.cpu().long()].float())
    h = rnd(3, 24, seed=2).to(dtype).to(DEV)
    close(head.forward(h), h.double().cpu().numpy() @ table.double().numpy().T, dtype)
    untied = lookup("head", "linear_head")({"vocab_size": 77, "hidden_size": 24, "tied": False}, "out.")
    assert [(w.name, w.shape) for w in untied.weights()] == [("out.weight", (77, 24))]


def rope_spec(hd, scaling=None, rot=None, pairing="half", theta=10000.0):
    return PartSpec("rotary", {"head_dim": hd, "rotary_dim": rot or hd, "theta": theta, "pairing": pairing, "scaling": scaling})


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,KV,hd,window", [(6, 2, 32, None), (4, 4, 16, None), (5, 1, 48, 20)])
def test_attention_mixer_with_its_cache(dtype, H, KV, hd, window):
    """The mixer with a cache of its own: a prompt in one step, then tokens one at a time, in two slots at
    once; against the plain projections, rotation and attention over the whole sequence."""
    d = 56
    scaling = {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
               "original_max_position_embeddings": 16}
    spec = PartSpec("gqa_attention", {"hidden_size": d, "num_heads": H, "num_kv_heads": KV, "head_dim": hd,
                                      "scale": 0.3, "window": window, "position": rope_spec(hd, scaling)})
    mixer = lookup("mixer", "gqa_attention")(spec.params, "L.")
    t = {w.name: rnd(*w.shape, seed=i, scale=0.2).to(dtype) for i, w in enumerate(mixer.weights())}
    rt = Runtime(DEV, dtype)
    mixer.bind(t, rt)
    req = mixer.cache_request()
    assert req == (CacheRequest("window", KV, hd, window) if window else CacheRequest("full", KV, hd))
    cache = SequenceCache([(0, req, None, None)], max_tokens=64 * 8, max_slots=4, max_seq_len=512, dtype=dtype, device=DEV)

    class Bare:
        """Just enough of a model for the engine to build a step's index arrays."""
        def __init__(self):
            self.rt = rt
            self.spec = type("S", (), {"vocab_size": 10})()
    eng = Engine(Bare(), cache)
    n = [90, 70]
    hs = [rnd(n[i], d, seed=20 + i).to(dtype) for i in range(2)]
    slots = [cache.open_slot(), cache.open_slot()]
    got = [[], []]

    def run(entries_h):
        entries = [StepEntry(s, [0] * h.shape[0], []) for s, h in entries_h]
        cache.reserve([(e.slot, cache.length(e.slot) + len(e.tokens)) for e in entries])
        cache.sync_tables()
        ctx = eng.build_context(entries)
        h = torch.cat([h for _, h in entries_h]).to(DEV)
        res = torch.zeros(h.shape[0], d, device=DEV)
        mixer.forward(h, res, ctx, cache.memory(0))
        for e in entries:
            cache.commit(e.slot, cache.length(e.slot) + len(e.tokens))
        return res

    out = run([(slots[0], hs[0][:60]), (slots[1], hs[1][:3])])
    got[0].append(out[:60]); got[1].append(out[60:])
    fed = [60, 3]
    while fed[0] < n[0] or fed[1] < n[1]:
        live = [i for i in range(2) if fed[i] < n[i]]
        out = run([(slots[i], hs[i][fed[i]:fed[i] + 1]) for i in live])
        for r, i in enumerate(live):
            got[i].append(out[r:r + 1])
            fed[i] += 1
    inv = pl.rotary_inv_freq(hd, 10000.0, scaling)
    f = lambda k: t[f"L.self_attn.{k}_proj.weight"].double().numpy()
    for i in range(2):
        h = hs[i].double().numpy()
        r = pl.bf16_round if dtype == torch.bfloat16 else (lambda a: a)
        q, k, v = r(h @ f("q").T), r(h @ f("k").T), r(h @ f("v").T)
        q, k = pl.rope(q, np.arange(n[i]), inv, hd), pl.rope(k, np.arange(n[i]), inv, hd)
        a = pl.attention(q, k, v, H, KV, hd, 0.3, window)
        close(torch.cat(got[i]), a @ f("o").T, dtype)


def test_block_part_order():
    """The pre-norm arrangement calls norm, mixer, norm, feed-forward on the same residual, in that order."""
    calls = []

    class N:
        def __init__(self, tag): self.tag = tag
        def forward(self, x, rows=None):
            calls.append(("norm" + self.tag, float(x.sum())))
            return x * 2

    class M:
        def forward(self, h, residual, step, memory):
            calls.append(("mixer", float(h.sum())))
            residual += 1

    class F:
        def forward(self, h, residual, step):
            calls.append(("ffn", float(h.sum())))
            residual += 10

    block = lookup("block", "prenorm_residual")(N("1"), M(), N("2"), F())
    x = torch.ones(2, 3, device=DEV)
    block.forward(x, None, None)
    assert calls == [("norm1", 6.0), ("mixer", 12.0), ("norm2", 12.0), ("ffn", 24.0)]
    assert float(x.sum()) == 6 + 6 + 60
