"""Contexts of thousands of positions against the plain implementation: more pages per sequence than the other tests
reach (140), as many slices as a decode step ever cuts a context into (32), prompt steps of thousands of rows (row
tiles in several rounds of blocks, keys and values fetched over dozens of pages) and chunks that attend to thousands
of cached positions."""
import numpy as np
import pytest

import ghost_infer_b200 as gi
from ghost_infer_b200.weights import write_random_model
from conftest import TINY_D, TINY_E
from gpu_helpers import check_logits, tokens_for
import plain_llama as pl

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,base,dtype,n,chunk", [("E", TINY_E, "bfloat16", 9000, 4096), ("D", TINY_D, "bfloat16", 5000, 1500),
                                                     ("D", TINY_D, "float32", 3000, 1100)])
def test_thousands_of_positions(tmp_path, name, base, dtype, n, chunk):
    cfg = dict(base, max_position_embeddings=16384)
    d = str(tmp_path / "model")
    write_random_model(d, cfg, seed=3, dtype=dtype, std=0.05, norm_jitter=0.1)
    toks = tokens_for(cfg, n, 5)
    ref = pl.forward(*pl.read_model(d), toks)
    model = gi.Model.from_pretrained(d, dtype=dtype, device="cuda:0")
    cache = model.new_cache(max_tokens=64 * ((n + 63) // 64 + 2), max_seq_len=n + 64)
    eng = gi.Engine(model, cache)
    tail = 40
    cut = n - tail
    # the prompt in one step, logits wanted at its start, in its middle and at its end
    s = cache.open_slot()
    places = [0, cut // 2, cut - 1]
    lg = eng.step([gi.StepEntry(s, toks[:cut], places)]).cpu().numpy()
    check_logits(lg, ref[places], dtype, f"{name} {dtype}: prompt of {cut} tokens")
    # the tail one token at a time through the runner that generation uses
    runner = eng.decoder([s])
    got = [runner.forward(tokens=[toks[j]]).cpu().numpy()[0].copy() for j in range(cut, n)]
    check_logits(np.stack(got), ref[cut:], dtype, f"{name} {dtype}: positions {cut} to {n - 1} one by one")
    if dtype == "bfloat16":
        plan = eng._mixers[0].decode_plan(1, n, eng._sm_count, [n])
        assert plan[0] == min(32, n // 256)                  # the context was cut into that many slices
    cache.close_slot(s)
    # the same prompt in chunks, each attending to what the chunks before it left in the cache
    s = cache.open_slot()
    for a in range(0, cut, chunk):
        b = min(cut, a + chunk)
        lg = eng.step([gi.StepEntry(s, toks[a:b], [b - a - 1])]).cpu().numpy()
        check_logits(lg, ref[b - 1:b], dtype, f"{name} {dtype}: chunk ending at {b}")
    cache.close_slot(s)
    assert cache.slots.free_slots == cache.max_slots
