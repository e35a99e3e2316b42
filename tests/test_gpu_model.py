"""The engine against the plain implementation: whole requests, the tail token by token, unequal batches
one after another with slots used again, long decoding, the first tokens; in 32-bit and in bfloat16."""
import numpy as np
import pytest
import torch

import ghost_infer_b200 as gi
from ghost_infer_b200.cache import CacheFullError
from gpu_helpers import check_logits, make_engine, plain_logits, tokens_for

pytestmark = pytest.mark.gpu

CASES = [("A", "float32", "float32"), ("B", "float32", "float32"), ("C", "float32", "bfloat16"),
         ("A", "bfloat16", "bfloat16"), ("B", "bfloat16", "bfloat16"), ("C", "bfloat16", "bfloat16"),
         ("B", "bfloat16", "float32"), ("D", "bfloat16", "bfloat16"), ("E", "bfloat16", "bfloat16"),
         ("E", "float32", "bfloat16")]


@pytest.fixture(scope="module")
def engines(model_dirs):
    made = {}

    def get(name, dtype, stored):
        key = (name, dtype, stored)
        if key not in made:
            d = model_dirs(name, stored)
            made[key] = (make_engine(d, dtype), d)
        return made[key]

    return get


def run_whole(eng, toks):
    s = eng.cache.open_slot()
    out = eng.step([gi.StepEntry(s, toks, list(range(len(toks))))]).cpu().numpy()
    eng.cache.close_slot(s)
    return out


@pytest.mark.parametrize("name,dtype,stored", CASES)
def test_each_request_alone_and_whole(engines, tiny_configs, name, dtype, stored):
    eng, d = engines(name, dtype, stored)
    for i, n in enumerate((1, 2, 31, 63, 64, 65, 130, 257)):
        toks = tokens_for(tiny_configs[name], n, 100 + i)
        check_logits(run_whole(eng, toks), plain_logits(d, toks), dtype, f"{name} {dtype} whole n={n}")
    assert eng.cache.free_pages == eng.cache.n_pages


@pytest.mark.parametrize("name,dtype,stored", CASES)
def test_last_32_tokens_one_by_one(engines, tiny_configs, name, dtype, stored):
    eng, d = engines(name, dtype, stored)
    for i, n in enumerate((33, 64, 97, 200)):
        toks = tokens_for(tiny_configs[name], n, 200 + i)
        ref = plain_logits(d, toks)
        s = eng.cache.open_slot()
        k = n - 32
        outs = [eng.step([gi.StepEntry(s, toks[:k], list(range(k)))]).cpu().numpy()]
        for t in toks[k:]:
            outs.append(eng.step([gi.StepEntry(s, [t], [0])]).cpu().numpy())
        eng.cache.close_slot(s)
        check_logits(np.concatenate(outs), ref, dtype, f"{name} {dtype} tail n={n}")


@pytest.mark.parametrize("name,dtype,stored", CASES)
def test_first_tokens(engines, tiny_configs, name, dtype, stored):
    eng, d = engines(name, dtype, stored)
    toks = tokens_for(tiny_configs[name], 4, 7)
    ref = plain_logits(d, toks)
    s = eng.cache.open_slot()
    outs = [eng.step([gi.StepEntry(s, [t], [0])]).cpu().numpy() for t in toks]     # a one-token prompt, then steps
    eng.cache.close_slot(s)
    check_logits(np.concatenate(outs), ref, dtype, f"{name} {dtype} first tokens")


def poison_free_pages(eng):
    """Fills every page no sequence holds with NaN: whoever reads a row it does not own shows it."""
    for g in eng.cache.groups:
        held = {p for pages in g.pages.values() for p in pages}
        free = [p for p in range(1, g.n_pages + 1) if p not in held]
        if free:
            idx = torch.tensor(free, device=g.k.device)
            g.k[:, idx] = float("nan")
            g.v[:, idx] = float("nan")


@pytest.mark.parametrize("name,dtype,stored", CASES)
def test_unequal_batches_one_after_another(engines, tiny_configs, name, dtype, stored):
    """Batches of unequal prompts; every request goes on token by token to its own length, the shorter
    ones end earlier; the next batch lands in the slots (and pages) the first one gave back."""
    eng, d = engines(name, dtype, stored)
    cfg = tiny_configs[name]
    plans = [[(130, 40), (5, 3), (64, 64), (33, 1)],       # (total length, prompt length)
             [(7, 7), (100, 90), (70, 1)],
             [(129, 64), (3, 2), (66, 65), (20, 10), (1, 1)]]
    for b, plan in enumerate(plans):
        poison_free_pages(eng)
        seqs = [tokens_for(cfg, total, 1000 + 10 * b + i) for i, (total, _) in enumerate(plan)]
        refs = [plain_logits(d, s) for s in seqs]
        slots = [eng.cache.open_slot() for _ in plan]
        assert slots == list(range(len(plan)))                        # slots are used again
        got = [[] for _ in plan]
        out = eng.step([gi.StepEntry(slots[i], seqs[i][:p], list(range(p))) for i, (_, p) in enumerate(plan)]).cpu().numpy()
        o = 0
        for i, (_, p) in enumerate(plan):
            got[i].append(out[o:o + p])
            o += p
        fed = [p for _, p in plan]
        live = [i for i, (total, p) in enumerate(plan) if p < total]
        for i in range(len(plan)):
            if i not in live:
                eng.cache.close_slot(slots[i])                        # ended with its prompt
        while live:
            out = eng.step([gi.StepEntry(slots[i], [seqs[i][fed[i]]], [0]) for i in live]).cpu().numpy()
            for r, i in enumerate(live):
                got[i].append(out[r:r + 1])
                fed[i] += 1
            for i in [i for i in live if fed[i] == len(seqs[i])]:
                eng.cache.close_slot(slots[i])
            live = [i for i in live if fed[i] < len(seqs[i])]
        for i in range(len(plan)):
            check_logits(np.concatenate(got[i]), refs[i], dtype, f"{name} {dtype} batch {b} request {i}")
        assert eng.cache.free_pages == eng.cache.n_pages and eng.cache.slots.free_slots == eng.cache.max_slots


@pytest.mark.parametrize("name,dtype,stored", [("A", "float32", "float32"), ("B", "bfloat16", "bfloat16"),
                                               ("D", "bfloat16", "bfloat16"), ("E", "bfloat16", "bfloat16")])
def test_long_decoding(engines, tiny_configs, name, dtype, stored):
    """Three prompt tokens, then 700 single-token steps: page after page, and contexts long enough for the
    decode kernel to cut them into slices."""
    eng, d = engines(name, dtype, stored)
    toks = tokens_for(tiny_configs[name], 703, 5)
    ref = plain_logits(d, toks)
    s = eng.cache.open_slot()
    outs = [eng.step([gi.StepEntry(s, toks[:3], [0, 1, 2])]).cpu().numpy()]
    for t in toks[3:]:
        outs.append(eng.step([gi.StepEntry(s, [t], [0])]).cpu().numpy())
    eng.cache.close_slot(s)
    check_logits(np.concatenate(outs), ref, dtype, f"{name} {dtype} long decoding")


@pytest.mark.parametrize("name,dtype,stored", [("B", "float32", "float32"), ("A", "bfloat16", "bfloat16")])
def test_chunked_prompt_and_partial_wants(engines, tiny_configs, name, dtype, stored):
    """A prompt cut into chunks of unequal size, logits asked only at some places."""
    eng, d = engines(name, dtype, stored)
    toks = tokens_for(tiny_configs[name], 150, 9)
    ref = plain_logits(d, toks)
    s = eng.cache.open_slot()
    a = eng.step([gi.StepEntry(s, toks[:70], [0, 69])]).cpu().numpy()
    assert eng.step([gi.StepEntry(s, toks[70:71], [])]) is None
    b = eng.step([gi.StepEntry(s, toks[71:150], [5, 78])]).cpu().numpy()
    eng.cache.close_slot(s)
    check_logits(np.concatenate([a, b]), ref[[0, 69, 76, 149]], dtype, f"{name} {dtype} chunks")


@pytest.mark.parametrize("name,dtype,stored", [("B", "bfloat16", "bfloat16"), ("E", "bfloat16", "bfloat16"), ("A", "float32", "float32")])
def test_a_place_wanted_twice(engines, tiny_configs, name, dtype, stored):
    """The same place named twice among the wanted ones, in a prompt and in one-token steps (where the last product
    of the last layer may leave partial sums to the final norm, which then reads that row for both)."""
    eng, d = engines(name, dtype, stored)
    toks = tokens_for(tiny_configs[name], 40, 12)
    ref = plain_logits(d, toks)
    s = eng.cache.open_slot()
    a = eng.step([gi.StepEntry(s, toks[:30], [29, 3, 29])]).cpu().numpy()
    check_logits(a, ref[[29, 3, 29]], dtype, f"{name} {dtype} prompt")
    assert np.array_equal(a[0], a[2])
    for i in range(30, 40):
        b = eng.step([gi.StepEntry(s, toks[i:i + 1], [0, 0, 0])]).cpu().numpy()
        check_logits(b, ref[[i, i, i]], dtype, f"{name} {dtype} token {i}")
        assert np.array_equal(b[0], b[1]) and np.array_equal(b[0], b[2])
    eng.cache.close_slot(s)


def test_host_checks_come_before_any_launch(engines):
    eng, _ = engines("A", "float32", "float32")
    s = eng.cache.open_slot()
    with pytest.raises(ValueError):
        eng.step([gi.StepEntry(s, [256], [0])])                      # token outside the vocabulary
    with pytest.raises(ValueError):
        eng.step([gi.StepEntry(s, [1, 2], [2])])                     # wanted place outside the tokens
    with pytest.raises(ValueError):
        eng.step([gi.StepEntry(s, [1], [0]), gi.StepEntry(s, [2], [0])])
    with pytest.raises(ValueError):
        eng.step([gi.StepEntry(s + 1, [1], [0])])                    # a slot nobody opened
    with pytest.raises(CacheFullError):
        eng.step([gi.StepEntry(s, [1] * 4000, [0])])
    assert eng.cache.length(s) == 0
    eng.cache.close_slot(s)


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_decoding_with_dependent_launch(model_dirs, tiny_configs, name):
    """Programmatic dependent launch lets a kernel start while its predecessor drains; results must not move.
    A batch decodes through the graph runner with it on, against the plain implementation and against itself off."""
    from ghost_infer_b200.kernels import ops
    d = model_dirs(name, "bfloat16")
    seqs = [tokens_for(tiny_configs[name], n, 40 + i) for i, n in enumerate((150, 90, 131))]
    refs = [plain_logits(d, s) for s in seqs]
    outs = {}
    was = ops.get_pdl()
    for pdl in (False, True):
        ops.set_pdl(pdl)
        try:
            eng = make_engine(d, "bfloat16")
            slots = [eng.cache.open_slot() for _ in seqs]
            eng.step([gi.StepEntry(s, t[:60], []) for s, t in zip(slots, seqs)])
            runner = eng.decoder(slots)
            got = [[] for _ in seqs]
            for j in range(60, 90):
                lg = runner.forward(tokens=[t[j] for t in seqs]).cpu().numpy()
                for i in range(len(seqs)):
                    got[i].append(lg[i])
            outs[pdl] = [np.stack(g) for g in got]
        finally:
            ops.set_pdl(was)
    for i in range(len(seqs)):
        check_logits(outs[True][i], refs[i][60:90], "bfloat16", f"{name} dependent launch request {i}")
        assert np.array_equal(outs[True][i], outs[False][i])
