"""The generation loop's decisions, with a stand-in for the step function and the sampler (no GPU)."""
from typing import List

import pytest
import torch

from ghost_infer_b200.cache import CacheFullError, CacheRequest, SequenceCache
from ghost_infer_b200.engine.generate import GenerationLoop

VOCAB = 50


class FakeEngine:
    """Next token = (last token + 1 + how many tokens the sequence holds) % VOCAB, as one-hot logits."""

    def __init__(self, max_tokens=64 * 64, max_slots=8, max_seq_len=4096):
        self.cache = SequenceCache([(0, CacheRequest("full", 1, 16), None, None)], max_tokens=max_tokens,
                                   max_slots=max_slots, max_seq_len=max_seq_len, dtype=torch.float32)
        self.calls: List[list] = []

    def step(self, entries):
        self.cache.reserve([(e.slot, self.cache.length(e.slot) + len(e.tokens)) for e in entries])
        rows = []
        self.calls.append([(e.slot, len(e.tokens)) for e in entries])
        for e in entries:
            n = self.cache.length(e.slot) + len(e.tokens)
            self.cache.commit(e.slot, n)
            for w in e.want:
                row = torch.zeros(VOCAB)
                row[(e.tokens[w] + 1 + n) % VOCAB] = 1.0
                rows.append(row)
        return torch.stack(rows) if rows else None


class ArgmaxSampler:
    def start(self, n):
        self.n = n

    def pick(self, logits, ids):
        return logits.argmax(-1).tolist()


def expected(prompt, max_new, stop=()):
    out, last, n = [], prompt[-1], len(prompt)
    while len(out) < max_new:
        t = (last + 1 + n) % VOCAB
        if t in stop:
            return out, "stop", t
        out.append(t)
        last, n = t, n + 1
    return out, "length", None


def test_unequal_prompts_lengths_and_batches():
    eng = FakeEngine()
    loop = GenerationLoop(eng, ArgmaxSampler(), batch_size=3)
    prompts = [[1, 2, 3], [4], [5, 6, 7, 8, 9], [10, 11], [12] * 40, [13, 14], [15]]
    res = loop.run(prompts, max_new=6)
    for p, r in zip(prompts, res):
        want, reason, _ = expected(p, 6)
        assert r.tokens == want and r.finish_reason == reason and r.prompt_tokens == len(p)
    assert loop.stats.batches == 3                       # 3 + 3 + 1 requests
    assert eng.calls[0] == [(0, 3), (1, 1), (2, 5)]      # all prompts of a batch in one step
    assert eng.cache.slots.free_slots == 8 and eng.cache.free_pages == 64
    # the second batch landed in the slots the first one gave back
    second = [c for c in eng.calls if c[0][1] in (2,)][0]
    assert [s for s, _ in second] == [0, 1, 2]


def test_stop_tokens_end_a_sequence_early_and_are_not_kept():
    eng = FakeEngine()
    prompts = [[1, 2, 3], [4], [20, 21]]
    # find what each would generate, then stop one of them on its third token
    free = [expected(p, 8)[0] for p in prompts]
    stop = {free[1][2]}
    loop = GenerationLoop(eng, ArgmaxSampler(), stop_token_ids=stop, batch_size=8)
    res = loop.run(prompts, max_new=8)
    for p, r in zip(prompts, res):
        want, reason, tok = expected(p, 8, stop)
        assert r.tokens == want and r.finish_reason == reason and r.stopped_on == tok
    assert res[1].finish_reason == "stop" and len(res[1].tokens) == 2
    # after the early end the batch goes on with the remaining sequences only
    sizes = [len(c) for c in eng.calls]
    assert sizes[0] == 3 and min(sizes) < 3 and sizes == sorted(sizes, reverse=True)
    # the stop token was never fed: the slot of request 1 received prompt + 2 tokens
    fed = sum(n for c in eng.calls for s, n in c if s == 1)
    assert fed == len(prompts[1]) + 2


def test_last_token_is_not_fed_and_counts():
    eng = FakeEngine()
    loop = GenerationLoop(eng, ArgmaxSampler(), batch_size=2)
    res = loop.run([[1, 2]], max_new=4)
    assert len(res[0].tokens) == 4 and loop.stats.gen_tokens == 4 and loop.stats.prompt_tokens == 2
    assert loop.stats.steps == 4                          # the prompt, then three fed tokens


def test_capacity_ends_a_sequence():
    """The reference's loop runs `while pos < ctx` and so yields ctx - prompt tokens: the logits after the last
    position of a full context are not sampled (src/main.rs:770)."""
    eng = FakeEngine(max_seq_len=8)
    loop = GenerationLoop(eng, ArgmaxSampler(), batch_size=2)
    res = loop.run([[1, 2, 3, 4, 5]], max_new=50)
    assert res[0].finish_reason == "capacity" and res[0].tokens == expected([1, 2, 3, 4, 5], 8 - 5)[0]
    assert loop.stats.gen_tokens == 3
    with pytest.raises(ValueError):
        loop.run([[1] * 8], max_new=2)                    # the prompt must leave room (src/main.rs:706)
    with pytest.raises(ValueError):
        loop.run([[]], max_new=2)                         # empty prompt (src/main.rs:703)


def test_batches_shrink_to_what_the_cache_holds():
    eng = FakeEngine(max_tokens=64 * 4)                   # 4 pages
    loop = GenerationLoop(eng, ArgmaxSampler(), batch_size=8)
    prompts = [[1] * 100, [2] * 100, [3] * 10, [4] * 10]  # 2 + 2 pages, then 1 + 1
    res = loop.run(prompts, max_new=3)
    assert loop.stats.batches == 2 and all(r.finish_reason == "length" for r in res)
    busy = FakeEngine(max_tokens=128)
    held = busy.cache.open_slot()
    busy.cache.reserve([(held, 100)])                     # somebody else holds every page
    with pytest.raises(CacheFullError):
        GenerationLoop(busy, ArgmaxSampler()).run([[1] * 70], max_new=1)


def test_max_new_zero_and_on_token():
    eng = FakeEngine()
    seen = []
    loop = GenerationLoop(eng, ArgmaxSampler(), batch_size=2, on_token=lambda i, t: seen.append((i, t)))
    assert loop.run([[1]], max_new=0)[0].tokens == []
    res = loop.run([[1], [2, 3]], max_new=2)
    assert sorted(seen) == sorted([(0, t) for t in res[0].tokens] + [(1, t) for t in res[1].tokens])


def test_prompts_read_in_several_steps():
    eng = FakeEngine()
    loop = GenerationLoop(eng, ArgmaxSampler(), batch_size=4, max_step_tokens=16)
    prompts = [[1] * 30, [2] * 5, [3] * 12]
    res = loop.run(prompts, max_new=3)
    for p, r in zip(prompts, res):
        assert r.tokens == expected(p, 3)[0]
    prompt_steps = [c for c in eng.calls if any(n > 1 for _, n in c)]
    assert all(sum(n for _, n in c) <= 16 for c in prompt_steps) and len(prompt_steps) == 3
    assert [n for c in prompt_steps for s, n in c if s == 0] == [16, 14]       # request 0 in two pieces


# ---- the loop that looks at tokens one step late takes the same decisions -------------------------------------
class FakeRunner:
    def __init__(self, eng, slots):
        self.eng, self.slots = eng, list(slots)

    def forward(self, tokens=None, dev_tokens=None):
        toks = dev_tokens.tolist() if tokens is None else list(tokens)
        from ghost_infer_b200.engine.step import StepEntry
        return self.eng.step([StepEntry(s, [int(t)], [0]) for s, t in zip(self.slots, toks)])


class PipelinedFakeEngine(FakeEngine):
    device = torch.device("cpu")

    def decoder(self, slots, use_graph=True):
        return FakeRunner(self, slots)


class DeviceArgmaxSampler(ArgmaxSampler):
    def pick_device(self, logits, ids):
        return logits.argmax(-1).to(torch.int32)


def run_both(prompts, max_new, stop=(), **kw):
    out = []
    for eng, sampler in ((FakeEngine(**kw), ArgmaxSampler()), (PipelinedFakeEngine(**kw), DeviceArgmaxSampler())):
        loop = GenerationLoop(eng, sampler, stop_token_ids=stop, batch_size=8)
        res = loop.run(prompts, max_new=max_new)
        out.append([(r.tokens, r.finish_reason, r.stopped_on) for r in res])
        assert eng.cache.free_pages == eng.cache.n_pages and eng.cache.slots.free_slots == eng.cache.max_slots
        assert loop.stats.gen_tokens == sum(len(r.tokens) + (r.finish_reason == "stop") for r in res)
    return out


def test_both_loops_agree_on_stops_lengths_and_the_context_s_end():
    prompts = [[1, 2, 3], [4], [20, 21], [7] * 5]
    free = [expected(p, 9)[0] for p in prompts]
    stop = {free[1][2], free[2][5]}
    simple, late = run_both(prompts, 9, stop=stop)
    assert simple == late
    assert [(r[0], r[1], r[2]) for r in simple] == [expected(p, 9, stop) for p in prompts]
    assert simple[1][1] == "stop" and simple[2][1] == "stop"
    simple, late = run_both([[1, 2, 3, 4, 5], [9, 9]], 50, max_seq_len=8)
    assert simple == late and [len(r[0]) for r in simple] == [3, 6] and all(r[1] == "capacity" for r in simple)


def test_both_loops_agree_when_the_pool_runs_full():
    """Three pages in all.  Two sequences of 60 tokens hold one page each and want a second one four steps on; only one
    more page is free, so the step that would take both new pages is refused.  A sequence that stops right then is
    known to the loop that looks at tokens at once, and late to the other, which must learn of it before it gives up."""
    prompts = [[1] * 60, [2] * 60]
    free = [expected(p, 12)[0] for p in prompts]
    # nobody stops: the step at length 65 finds one free page for two sequences; both end with "capacity"
    simple, late = run_both(prompts, 12, max_tokens=64 * 3)
    assert simple == late and all(r[1] == "capacity" and len(r[0]) == 5 for r in simple)
    # request 0 stops on the very token whose feeding would need the page: the other goes on and reaches its length
    simple, late = run_both(prompts, 12, stop={free[0][4]}, max_tokens=64 * 3)
    assert simple == late
    assert simple[0][1] == "stop" and len(simple[0][0]) == 4 and simple[1][1] == "length" and len(simple[1][0]) == 12
