"""bin/trace_run driven as a user drives it: the same requests whole, with the last 32 tokens one by one,
and in batches of unequal lengths one after another, in 32-bit and in bfloat16."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from gpu_helpers import check_logits, plain_logits, tokens_for

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def build_trace(cfg):
    """Returns (steps, expect) where expect maps a step number to [(request tokens, places)]."""
    reqs = {f"r{i}": tokens_for(cfg, n, 300 + i) for i, n in enumerate((40, 5, 97, 64, 33))}
    steps, expect = [], {}

    def add(entries, end=()):
        n = len(steps)
        steps.append({"step": n, "entries": [{"id": i, "tokens": t, "want": w} for i, t, w in entries], "end": list(end)})
        wanted = [(i, p) for i, t, w in entries for p in w]
        if wanted:
            expect[n] = (entries, None)
        return n

    pos = {}
    # 1. each request alone and whole
    for rid, toks in reqs.items():
        add([(rid + "w", toks, list(range(len(toks))))], end=[rid + "w"])
    # 2. all but the last 32 tokens whole, the last 32 one by one
    for rid, toks in reqs.items():
        if len(toks) <= 32:
            continue
        k = len(toks) - 32
        add([(rid + "t", toks[:k], [k - 1])])
        for j in range(k, len(toks)):
            add([(rid + "t", [toks[j]], [0])], end=[rid + "t"] if j == len(toks) - 1 else [])
    # 3. two batches of unequal lengths; prompts of different sizes, then one token each; shorter ones end earlier
    for batch, ids in enumerate((["r0", "r1", "r2"], ["r3", "r4", "r1"])):
        cut = {rid: max(1, len(reqs[rid]) // 2) for rid in ids}
        names = {rid: f"{rid}b{batch}" for rid in ids}
        ends = [names[r] for r in ids if cut[r] == len(reqs[r])]
        add([(names[r], reqs[r][:cut[r]], list(range(cut[r]))) for r in ids], end=ends)
        fed = dict(cut)
        while True:
            live = [r for r in ids if fed[r] < len(reqs[r])]
            if not live:
                break
            ends = [names[r] for r in live if fed[r] + 1 == len(reqs[r])]
            add([(names[r], [reqs[r][fed[r]]], [0]) for r in live], end=ends)
            for r in live:
                fed[r] += 1
    return reqs, steps


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "bfloat16"), ("C", "float32"), ("C", "bfloat16"), ("E", "bfloat16")])
def test_trace_replay(tmp_path, model_dirs, tiny_configs, name, dtype):
    d = model_dirs(name, dtype)
    cfg = tiny_configs[name]
    reqs, steps = build_trace(cfg)
    out = tmp_path / "out"
    text = "\n".join(json.dumps(s) for s in steps) + "\n"
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype,
                        "--out", str(out), "--max-tokens", str(64 * 8)], input=text, capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-3000:]
    assert p.stdout.split("\n")[:len(steps)] == [f"done {i}" for i in range(len(steps))]
    refs = {rid: plain_logits(d, toks) for rid, toks in reqs.items()}
    place = {}                                   # request instance -> tokens fed so far
    vocab = cfg["vocab_size"]
    for s in steps:
        want_rows = []
        for e in s["entries"]:
            base = place.get(e["id"], 0)
            rid = e["id"][:2]
            for w in e["want"]:
                want_rows.append(refs[rid][base + w])
            place[e["id"]] = base + len(e["tokens"])
        f = out / f"{s['step']}.f32"
        if want_rows:
            got = np.fromfile(f, dtype="<f4").reshape(-1, vocab)
            check_logits(got, np.stack(want_rows), dtype, f"{name} {dtype} step {s['step']}")
        else:
            assert not f.exists()
