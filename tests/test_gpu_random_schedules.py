"""Random ways of cutting and batching a handful of requests, each against the plain implementation.

The other engine tests walk schedules chosen by hand.  Here a generator draws them: one to five requests of 1 to 319
tokens; either every step takes some of the live requests and gives each a chunk of 1 to 300 of its next tokens (so a
step holds fresh prompts, chunks in mid-sequence and single tokens side by side, some requests sit a step out, and the
places whose logits are wanted are drawn too), or the prompts are read in one step and the rest goes one token at a
time through the runner that generation uses, which is rebuilt whenever a request ends.  Every row of logits that
comes back is compared.  The seeds are fixed: a failure names configuration and draw and can be run again."""
import numpy as np
import pytest

import ghost_infer_b200 as gi
from gpu_helpers import check_logits, make_engine, plain_logits, tokens_for

pytestmark = pytest.mark.gpu

CHUNKS = [1, 1, 2, 7, 33, 64, 65, 90, 130, 300]


def _chunks(rng, eng, d, cfg, dtype, what):
    cache = eng.cache
    n_req = int(rng.integers(1, 6))
    lens = [int(rng.integers(1, 320)) for _ in range(n_req)]
    seqs = [tokens_for(cfg, n, int(rng.integers(1 << 30))) for n in lens]
    refs = [plain_logits(d, t) for t in seqs]
    slots = [cache.open_slot() for _ in seqs]
    done = [0] * n_req
    rows = 0
    while any(done[i] < lens[i] for i in range(n_req)):
        live = [i for i in range(n_req) if done[i] < lens[i]]
        pick = [i for i in live if rng.random() < 0.7] or [live[0]]
        entries, wants = [], []
        for i in pick:
            n = int(min(lens[i] - done[i], rng.choice(CHUNKS)))
            w = sorted(set(int(x) for x in rng.integers(0, n, size=int(rng.integers(0, 3)))))
            if rng.random() < 0.5 and (n - 1) not in w:
                w.append(n - 1)
            entries.append(gi.StepEntry(slots[i], seqs[i][done[i]:done[i] + n], w))
            wants.append((i, done[i], w))
            done[i] += n
        lg = eng.step(entries)
        if sum(len(w) for _, _, w in wants):
            lg = lg.cpu().numpy()
            r = 0
            for i, base, w in wants:
                for x in w:
                    check_logits(lg[r:r + 1], refs[i][base + x:base + x + 1], dtype, f"{what}, request {i} of lengths {lens}, place {base + x}")
                    r += 1
            rows += r
    for s in slots:
        cache.close_slot(s)
    return rows


def _runner(rng, eng, d, cfg, dtype, what):
    cache = eng.cache
    n_req = int(rng.integers(1, 6))
    lens = [int(rng.integers(1, 320)) for _ in range(n_req)]
    seqs = [tokens_for(cfg, n, int(rng.integers(1 << 30))) for n in lens]
    refs = [plain_logits(d, t) for t in seqs]
    slots = [cache.open_slot() for _ in seqs]
    done = [max(1, n - int(rng.integers(0, 40))) for n in lens]
    lg = eng.step([gi.StepEntry(s, t[:c], [c - 1]) for s, t, c in zip(slots, seqs, done)]).cpu().numpy()
    for i in range(n_req):
        check_logits(lg[i:i + 1], refs[i][done[i] - 1:done[i]], dtype, f"{what}, prompt of request {i} of lengths {lens}")
    rows = n_req
    live = [i for i in range(n_req) if done[i] < lens[i]]
    while live:
        runner = eng.decoder([slots[i] for i in live])
        for _ in range(min(lens[i] - done[i] for i in live)):
            lg = runner.forward(tokens=[seqs[i][done[i]] for i in live]).cpu().numpy()
            for r, i in enumerate(live):
                check_logits(lg[r:r + 1], refs[i][done[i]:done[i] + 1], dtype, f"{what}, request {i} of lengths {lens}, place {done[i]}")
                done[i] += 1
            rows += len(live)
        live = [i for i in live if done[i] < lens[i]]
    for s in slots:
        cache.close_slot(s)
    return rows


@pytest.mark.parametrize("name,dtype", [("D", "bfloat16"), ("E", "bfloat16"), ("A", "float32"), ("B", "float32"),
                                        ("D", "float32"), ("B", "bfloat16")])
def test_drawn_schedules(model_dirs, tiny_configs, name, dtype):
    d, cfg = model_dirs(name, dtype), tiny_configs[name]
    eng = make_engine(d, dtype, max_tokens=64 * 64, max_seq_len=1024)
    rng = np.random.default_rng(sum(map(ord, name + dtype)))
    rows = 0
    for rnd in range(12):
        rows += _chunks(rng, eng, d, cfg, dtype, f"{name} {dtype} draw {rnd} in chunks")
        rows += _runner(rng, eng, d, cfg, dtype, f"{name} {dtype} draw {rnd} through the runner")
    assert rows > 200
    assert eng.cache.slots.free_slots == eng.cache.max_slots          # every slot came back
