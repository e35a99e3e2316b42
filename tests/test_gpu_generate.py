"""Generation through the Python entry point and the command line, against the plain implementation."""
import os
import subprocess
import sys

import numpy as np
import pytest

import ghost_infer_b200 as gi
from gpu_helpers import check_logits, oracle, tokens_for
import plain_llama as pl

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def plain_greedy(model_dir, prompt, max_new, stop=()):
    """Greedy generation by recomputing the whole sequence for every token (src/main.rs:770-783)."""
    cfg, w = oracle(model_dir)
    toks, out, margins = list(prompt), [], []
    for _ in range(max_new):
        logits = pl.forward(cfg, w, toks)[-1]
        order = np.argsort(-logits, kind="stable")
        margins.append(float(logits[order[0]] - logits[order[1]]))
        t = int(order[0])
        if t in stop:
            return out, "stop", margins
        out.append(t)
        toks.append(t)
    return out, "length", margins


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("B", "bfloat16")])
def test_greedy_generation_matches_the_plain_implementation(model_dirs, tiny_configs, name, dtype):
    d = model_dirs(name, dtype)
    cfg = tiny_configs[name]
    llm = gi.LLM(d, dtype=dtype, max_tokens=64 * 32)
    lens = [5, 9, 13] if name == "A" else [1, 7, 40, 64]
    prompts = [tokens_for(cfg, n, 50 + i) for i, n in enumerate(lens)]
    res = llm.generate(prompts, max_new=8, temperature=0.0, stop_token_ids=(), batch_size=3)
    for p, r in zip(prompts, res):
        want, reason, margins = plain_greedy(d, p, 8)
        # a 16-bit engine may pick the other of two nearly equal logits; compare up to the first near-tie
        sure = len(want)
        if dtype == "bfloat16":
            near = [i for i, m in enumerate(margins) if m < 0.05]
            sure = near[0] if near else len(want)
        assert r.tokens[:sure] == want[:sure], f"prompt of {len(p)}: {r.tokens} vs {want}"
        assert r.finish_reason == "length" and len(r.tokens) == 8
    assert llm.last_stats.batches == (1 if name == "A" else 2)
    assert llm.cache.free_pages == llm.cache.n_pages


def test_stop_token_from_the_configuration(model_dirs, tiny_configs):
    d = model_dirs("A", "float32")
    llm = gi.LLM(d, dtype="float32", max_tokens=64 * 8)
    prompt = tokens_for(tiny_configs["A"], 6, 3)
    free, _, _ = plain_greedy(d, prompt, 6)
    res = llm.generate([prompt], max_new=6, temperature=0.0, stop_token_ids=[free[3]])
    first = free.index(free[3])
    assert res[0].tokens == free[:first] and res[0].finish_reason == "stop" and res[0].stopped_on == free[3]
    assert llm.stop_token_ids == (7,)                      # config.json's eos_token_id is the default stop set


def test_sampling_is_reproducible_and_does_not_depend_on_batch_mates(model_dirs, tiny_configs):
    d = model_dirs("B", "float32")
    cfg = tiny_configs["B"]
    llm = gi.LLM(d, dtype="float32", max_tokens=64 * 16)
    prompts = [tokens_for(cfg, n, 70 + i) for i, n in enumerate([1, 7, 40, 64])]
    kw = dict(max_new=16, temperature=0.8, top_k=40, top_p=0.9, seed=11, stop_token_ids=())
    a = [r.tokens for r in llm.generate(prompts, batch_size=4, **kw)]
    b = [r.tokens for r in llm.generate(prompts, batch_size=4, **kw)]
    c = [r.tokens for r in llm.generate(prompts, batch_size=1, **kw)]
    e = [r.tokens for r in llm.generate(prompts, batch_size=4, **dict(kw, seed=12))]
    assert a == b and a == c and a != e
    # request 0 draws from the reference's stream for that seed: check its first token against the plain sampler
    cfgp, w = oracle(d)
    first = pl.sample(pl.forward(cfgp, w, prompts[0])[-1], 0.8, 40, 0.9, pl.XorShift64Star(11))
    assert a[0][0] == first


def test_command_line_run(model_dirs, tiny_configs):
    d = model_dirs("A", "float32")
    prompt = tokens_for(tiny_configs["A"], 5, 1)
    want, _, _ = plain_greedy(d, prompt, 5, stop=(7,))
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "ghost-infer"), "run", d, "-p", ",".join(map(str, prompt)),
                        "-n", "5", "-t", "0", "--dtype", "float32", "--ctx", "128"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr
    assert p.stdout.split() == [str(t) for t in want]
    assert "[prompt 5 tok in" in p.stderr and "generated" in p.stderr
    bad = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "ghost-infer"), "run", d, "--nonsense"],
                         capture_output=True, text=True, timeout=600)
    assert bad.returncode == 1 and "unknown option --nonsense" in bad.stderr


def test_command_line_top_kvcheck_and_bench(tmp_path, model_dirs, tiny_configs):
    d = model_dirs("A", "float32")
    ids = tokens_for(tiny_configs["A"], 12, 2)
    exe = [sys.executable, os.path.join(ROOT, "bin", "ghost-infer")]
    # top: the ten most likely next tokens, and every logit as little-endian float32 when the variable is set
    dump = tmp_path / "logits.f32"
    cfg, w = oracle(d)
    ref = pl.forward(cfg, w, ids)[-1]
    for dtype in ("float32", "bfloat16"):
        p = subprocess.run(exe + ["top", d, ",".join(map(str, ids)), "--dtype", dtype], capture_output=True, text=True,
                           timeout=600, env=dict(os.environ, GHOST_INFER_LOGITS_OUT=str(dump)))
        assert p.returncode == 0, p.stderr
        got = np.fromfile(dump, dtype="<f4")
        assert got.shape == ref.shape
        check_logits(got, ref, dtype, f"top {dtype}")
        lines = [l for l in p.stdout.splitlines() if "logprob" in l]
        order = np.argsort(-ref, kind="stable")
        assert len(lines) == 10
        if dtype == "float32":
            assert [int(l.split()[0]) for l in lines] == [int(i) for i in order[:10]]
            lse = np.log(np.exp(ref - ref.max()).sum()) + ref.max()
            for l, i in zip(lines, order[:10]):
                assert abs(float(l.split()[-1]) - (ref[i] - lse)) < 2e-4      # four decimals are printed
        else:
            assert int(lines[0].split()[0]) in order[:2]
    # kvcheck: all but the last 4 ids as a prompt, those one at a time; pick and log-probability per token
    idf, out = tmp_path / "ids.txt", tmp_path / "kv.txt"
    idf.write_text(" ".join(map(str, ids)))
    full = pl.forward(cfg, w, ids)
    for dtype, tol in (("float32", 5e-5), ("bfloat16", 0.02)):
        p = subprocess.run(exe + ["kvcheck", d, str(idf), str(out), "4", "--dtype", dtype], capture_output=True, text=True,
                           timeout=600)
        assert p.returncode == 0, p.stderr
        rows = [l.split() for l in out.read_text().splitlines()]
        assert len(rows) == 4 and "mean NLL" in p.stderr
        for j, (pick, lp) in enumerate(rows):
            l = full[len(ids) - 5 + j]
            want = l[ids[len(ids) - 4 + j]] - (np.log(np.exp(l - l.max()).sum()) + l.max())
            assert abs(float(lp) - want) < tol            # the file keeps five decimals
            if dtype == "float32":
                assert int(pick) == int(np.argmax(l))
    # bench: the reference's fixed workload and its one-line result
    p = subprocess.run(exe + ["bench", d, "-n", "6", "--prompt-len", "20", "--batch", "2"], capture_output=True, text=True,
                       timeout=600, env=dict(os.environ, GHOST_INFER_BENCH_ROUNDS="2"))
    assert p.returncode == 0, p.stderr
    assert "prompt 20 tok x 2:" in p.stdout and "generate 6 tok x 2:" in p.stdout and p.stderr.count("round ") == 2


def test_time_per_kind_of_operation(model_dirs, tiny_configs):
    """The reference's profile buckets (src/profile.rs:7-46): with profiling on, every bucket the decoder uses has device
    time, steps run without a graph, and the tokens are the ones generation gives without it."""
    from ghost_infer_b200.kernels import ops
    d = model_dirs("E", "bfloat16")
    llm = gi.LLM(d, dtype="bfloat16", max_tokens=64 * 8)
    prompts = [tokens_for(tiny_configs["E"], n, 90 + i) for i, n in enumerate([20, 5])]
    plain = [r.tokens for r in llm.generate(prompts, max_new=6, temperature=0.0, stop_token_ids=(), batch_size=2)]
    assert not ops.profiling()
    was = ops.get_pdl()
    ops.profile_start()
    try:
        assert ops.profiling() and not ops.get_pdl()
        timed = [r.tokens for r in llm.generate(prompts, max_new=6, temperature=0.0, stop_token_ids=(), batch_size=2)]
        assert not llm.engine.decoder([0]).use_graph
    finally:
        buckets = ops.profile_stop()
    assert timed == plain and not ops.profiling() and ops.get_pdl() == was
    assert list(buckets) == ["embed", "norm", "qkv matmul", "rope+cache", "attention", "out matmul", "ffn matmul", "logits", "sampling"]
    assert all(ms > 0 for ms in buckets.values())
    # the command line prints them per token
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "ghost-infer"), "run", d, "-p", "1,2,3", "-n", "4", "-t", "0"],
                       capture_output=True, text=True, timeout=600, env=dict(os.environ, GHOST_INFER_PROFILE="1"))
    assert p.returncode == 0, p.stderr
    assert "[profile over" in p.stderr and "attention" in p.stderr and "ffn matmul" in p.stderr
