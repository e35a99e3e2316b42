"""The 32-bit path gives the same bits for a token whatever else shares its step.

The reference checks that n one-token steps and one n-token batch give bit-identical rows
(GHOST_INFER_VERIFY_CHECK, src/main.rs:1306-1329) and keeps a fixed summation order for it (src/cuda.rs:748-766; slice
sizes from the token's own span, :1639-1644).  Here, in float32: a row computed by one-token steps has the same bits
alone, inside batches of other sizes and through the graph runner with its padding rows; a row computed as part of a
prompt has the same bits alone, in a batch, and however the prompt is cut into chunks.  The two kinds of row differ
from each other (a prompt's attention walks the keys in one running softmax, a one-token step cuts them into slices
that are merged afterwards): that difference is measured in units in the last place and bounded.
"""
import numpy as np
import pytest

import ghost_infer_b200 as gi
from gpu_helpers import check_logits, make_engine, plain_logits, tokens_for

pytestmark = pytest.mark.gpu
NAMES = ["A", "B", "D", "E"]


@pytest.fixture(scope="module")
def engines(model_dirs):
    made = {}

    def get(name):
        if name not in made:
            d = model_dirs(name, "float32")
            made[name] = (make_engine(d, "float32", max_tokens=64 * 64), d)
        return made[name]

    return get


def decode_rows(eng, seqs, starts, steps, runner=False):
    """Prompts `seqs[i][:starts[i]]` in one step, then `steps[i]` one-token steps each (a sequence that is done leaves);
    returns per sequence the logits of its one-token steps."""
    cache = eng.cache
    slots = [cache.open_slot() for _ in seqs]
    eng.step([gi.StepEntry(s, t[:n], []) for s, t, n in zip(slots, seqs, starts)])
    got = [[] for _ in seqs]
    fed = list(starts)
    run, run_for = None, None
    while True:
        live = [i for i in range(len(seqs)) if fed[i] < starts[i] + steps[i]]
        if not live:
            break
        if runner:
            if run_for != live:
                run, run_for = eng.decoder([slots[i] for i in live]), live
            out = run.forward(tokens=[seqs[i][fed[i]] for i in live]).cpu().numpy()
        else:
            out = eng.step([gi.StepEntry(slots[i], [seqs[i][fed[i]]], [0]) for i in live]).cpu().numpy()
        for r, i in enumerate(live):
            got[i].append(out[r].copy())
            fed[i] += 1
    for s in slots:
        cache.close_slot(s)
    return [np.stack(g) if g else np.zeros((0,)) for g in got]


@pytest.mark.parametrize("name", NAMES)
def test_one_token_steps_do_not_depend_on_batch_mates(engines, tiny_configs, name):
    eng, d = engines(name)
    cfg = tiny_configs[name]
    me = tokens_for(cfg, 330, 500)                       # 270 as a prompt, then 60 steps: slices of 256 keys, so two, then...
    mates = [tokens_for(cfg, n, 501 + i) for i, n in enumerate((700, 40, 300, 129))]
    alone = decode_rows(eng, [me], [270], [60])[0]
    check_logits(alone, plain_logits(d, me)[270:], "float32", f"{name} alone")
    # a batch of five: mates that are longer (more slices in the launch) and shorter, some leaving on the way
    five = decode_rows(eng, [mates[0], me, mates[1], mates[2], mates[3]], [600, 270, 10, 255, 64], [60, 60, 30, 45, 60])
    assert np.array_equal(five[1], alone)
    # the same through the graph runner, whose launches hold padding rows and a slice count set by a length bucket
    assert np.array_equal(decode_rows(eng, [me], [270], [60], runner=True)[0], alone)
    five_r = decode_rows(eng, [mates[0], me, mates[1], mates[2], mates[3]], [600, 270, 10, 255, 64], [60, 60, 30, 45, 60], runner=True)
    assert np.array_equal(five_r[1], alone)
    for a, b in zip(five, five_r):
        assert np.array_equal(a, b)
    # last of three and first of two
    assert np.array_equal(decode_rows(eng, [mates[3], mates[1], me], [64, 10, 270], [20, 20, 60])[2], alone)
    assert np.array_equal(decode_rows(eng, [me, mates[0]], [270, 650], [60, 10])[0], alone)


def prompt_rows(eng, entries_by_step, which):
    """Runs steps of (sequence index, tokens) entries, wanting every place of sequence `which`; returns its rows."""
    cache = eng.cache
    slots = {}
    rows = []
    for entries in entries_by_step:
        step = []
        for i, toks in entries:
            if i not in slots:
                slots[i] = cache.open_slot()
            step.append(gi.StepEntry(slots[i], toks, list(range(len(toks))) if i == which else []))
        out = eng.step(step)
        if out is not None:
            rows.append(out.cpu().numpy())
    for s in slots.values():
        cache.close_slot(s)
    return np.concatenate(rows)


@pytest.mark.parametrize("name", NAMES)
def test_prompt_rows_do_not_depend_on_batch_mates_or_on_the_cut(engines, tiny_configs, name):
    eng, d = engines(name)
    cfg = tiny_configs[name]
    me = tokens_for(cfg, 300, 510)
    m1, m2, m3 = (tokens_for(cfg, n, 511 + i) for i, n in enumerate((700, 33, 128)))
    alone = prompt_rows(eng, [[(0, me)]], 0)
    check_logits(alone, plain_logits(d, me), "float32", f"{name} prompt alone")
    assert np.array_equal(prompt_rows(eng, [[(1, m1), (0, me), (2, m2), (3, m3)]], 0), alone)       # a batch of four
    assert np.array_equal(prompt_rows(eng, [[(1, m2), (0, me)]], 0), alone)
    # more than 512 rows in the step and fewer: the norm's blocks must not follow the step's size
    assert np.array_equal(prompt_rows(eng, [[(0, me), (1, m1)]], 0), alone)
    # cut into chunks of 64, of 7, and unevenly, with a mate that is cut differently
    for size in (64, 7):
        steps = [[(0, me[i:i + size])] for i in range(0, 300, size)]
        assert np.array_equal(prompt_rows(eng, steps, 0), alone), f"chunks of {size}"
    uneven = [[(0, me[:100]), (1, m1[:300])], [(1, m1[300:310])], [(0, me[100:101]), (1, m1[310:700])], [(0, me[101:300]), (2, m2)]]
    assert np.array_equal(prompt_rows(eng, uneven, 0), alone)


@pytest.mark.parametrize("name", NAMES)
def test_prompt_rows_and_one_token_rows_differ_by_a_few_units_in_the_last_place(engines, tiny_configs, name):
    """The two ways are not the same arithmetic: the prompt kernel sums a row's keys in one running softmax over
    32-key tiles, the one-token kernel in slices of 256 keys (four warps each) merged afterwards; the same products
    summed in another order.  The difference is bounded here in units in the last place of the largest logit."""
    eng, d = engines(name)
    cfg = tiny_configs[name]
    me = tokens_for(cfg, 330, 500)
    whole = prompt_rows(eng, [[(0, me)]], 0)[270:]
    steps = decode_rows(eng, [me], [270], [60])[0]
    assert not np.array_equal(whole, steps)              # if they ever are equal, say so in the docstring
    scale = np.float32(np.abs(whole).max())
    ulp = np.spacing(scale)
    worst = float(np.abs(whole.astype(np.float64) - steps.astype(np.float64)).max() / ulp)
    print(f"{name}: prompt rows vs one-token rows differ by at most {worst:.1f} ulp of the largest logit ({scale:.3f})")
    assert worst <= 64.0
