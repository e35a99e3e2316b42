"""Command line in the reference's manner (src/main.rs:36-92, :120-203, :205-248).

    ghost-infer inspect <model dir>
    ghost-infer top     <model dir> <token ids> [--dtype <t>]   next-token probabilities after the ids
    ghost-infer bench   <model dir> [-n <gen tokens>] [--prompt-len <n>] [--batch <n>]
    ghost-infer run     <model dir> -p <token ids> [options]
    ghost-infer kvcheck <model dir> <ids file> <out file> <tail> [--dtype <t>]
    ghost-infer random  <config.json> <out dir> [--seed <n>] [--dtype <t>]

Options keep the reference's names, meanings and defaults where it has them: -p/--prompt, -n/--max [256],
-t/--temp [0.7], --top-k [40], --top-p [0.9], --seed [time], --ctx [2048], --prompt-len [256], --gpu
(accepted; this library runs nowhere else).  Added: --dtype bfloat16|float32, --batch <n>.
A prompt is a list of token ids ("12,7,99" or "12 7 99"); several prompts are separated by ";".
"""
from __future__ import annotations

import json
import math
import os
import sys
import time
from dataclasses import dataclass, field
from typing import List, Optional

USAGE = """ghost-infer_b200 - run Llama 3 models from a safetensors folder on an NVIDIA B200

USAGE:
    ghost-infer inspect <model dir>
    ghost-infer top     <model dir> <token ids> [--dtype <t>]   (next-token probabilities after the ids)
    ghost-infer bench   <model dir> [-n <gen tokens>] [--prompt-len <n>] [--batch <n>]
    ghost-infer run     <model dir> -p <token ids> [options]
    ghost-infer kvcheck <model dir> <ids file> <out file> <tail> [--dtype <t>]
    ghost-infer random  <config.json> <out dir> [--seed <n>] [--dtype <t>]

OPTIONS:
    -p, --prompt <ids>    prompt as token ids, "1,2,3"; several prompts separated by ";" (run)
    -n, --max <n>         max new tokens per reply          [256]
    -t, --temp <f>        temperature, 0 = greedy            [0.7]
        --top-k <n>       keep the k most likely tokens, 0 = all [40]
        --top-p <f>       nucleus sampling cut-off           [0.9]
        --seed <n>        sampling seed                      [time]
        --ctx <n>         context window in tokens           [2048]
        --prompt-len <n>  prompt length (bench)              [256]
        --batch <n>       sequences per batch                [run: 8, bench: 1]
        --dtype <t>       bfloat16 or float32                [bfloat16]
        --gpu             accepted for compatibility: there is no other backend

ENVIRONMENT:
    GHOST_INFER_PROFILE=1     run: device time per kind of operation (steps then run kernel by kernel)
    GHOST_INFER_LOGITS_OUT=f  top: every logit of the last position as little-endian float32 into f
    GHOST_INFER_BENCH_ROUNDS  bench: rounds to take the best of [3]
"""


@dataclass
class Opts:
    model: str
    prompt: Optional[str] = None
    max_new: int = 256
    temp: float = 0.7
    top_k: int = 40
    top_p: float = 0.9
    seed: int = field(default_factory=time.time_ns)
    ctx: Optional[int] = None
    prompt_len: int = 256
    batch: Optional[int] = None
    dtype: str = "bfloat16"
    gpu: bool = True


class UsageError(Exception):
    pass


def parse_opts(args: List[str]) -> Opts:
    if not args:
        raise UsageError("missing model path")
    o = Opts(model=args[0])
    it = iter(args[1:])

    def val(name):
        try:
            return next(it)
        except StopIteration:
            raise UsageError(f"{name} needs a value") from None

    def num(s, name):
        try:
            return float(s)
        except ValueError:
            raise UsageError(f"{name}: \"{s}\" is not a number") from None

    for a in it:
        if a in ("-p", "--prompt"):
            o.prompt = val(a)
        elif a in ("-n", "--max"):
            o.max_new = int(num(val(a), a))
        elif a in ("-t", "--temp"):
            o.temp = num(val(a), a)
        elif a == "--top-k":
            o.top_k = int(num(val(a), a))
        elif a == "--top-p":
            o.top_p = num(val(a), a)
        elif a == "--seed":
            o.seed = int(num(val(a), a))
        elif a == "--ctx":
            o.ctx = int(num(val(a), a))
        elif a == "--prompt-len":
            o.prompt_len = int(num(val(a), a))
        elif a == "--batch":
            o.batch = int(num(val(a), a))
        elif a == "--dtype":
            o.dtype = val(a)
        elif a == "--gpu":
            o.gpu = True
        else:
            raise UsageError(f"unknown option {a}")
    return o


def parse_ids(text: str) -> List[List[int]]:
    prompts = []
    for part in text.split(";"):
        ids = [int(t) for t in part.replace(",", " ").split()]
        if ids:
            prompts.append(ids)
    if not prompts:
        raise UsageError("the prompt holds no token ids")
    return prompts


def _llm(o: Opts, max_tokens: int, ctx: Optional[int] = None):
    """`ctx`: the most tokens one sequence may hold; never more than the model's own positions, as the
    reference clamps its context (`ctx.min(max_ctx)`, src/model.rs:732)."""
    from .api import LLM
    from .engine.model import Model
    t = time.time()
    model = Model.from_pretrained(o.model, dtype=o.dtype)
    own = model.spec.max_positions
    if ctx is not None and ctx > own:
        print(f"[--ctx {ctx} is beyond the model's {own} positions: using {own}]", file=sys.stderr)
    llm = LLM(model, dtype=o.dtype, max_tokens=max_tokens, max_seq_len=own if ctx is None else min(ctx, own))
    cfg = llm.model.config
    print(f"[loaded {getattr(cfg, 'architecture', 'model')} ({o.dtype}) in {time.time() - t:.2f}s]", file=sys.stderr)
    return llm


def print_stats(st) -> None:
    """The reference's line (src/main.rs:1421-1438)."""
    print(f"[prompt {st.prompt_tokens} tok in {st.prompt_secs:.2f}s = {st.prompt_tokens / max(st.prompt_secs, 1e-9):.1f} tok/s"
          f" | generated {st.gen_tokens} tok in {st.gen_secs:.2f}s = {st.gen_tokens / max(st.gen_secs, 1e-9):.1f} tok/s]",
          file=sys.stderr)


def _profile_wanted() -> bool:
    return os.environ.get("GHOST_INFER_PROFILE", "") not in ("", "0")


def print_profile(buckets, tokens: int) -> None:
    """Device time per kind of operation and per token, in the reference's manner (src/profile.rs:36-46)."""
    total = sum(buckets.values()) or 1.0
    print(f"[profile over {tokens} tokens: device time per token, steps launched kernel by kernel]", file=sys.stderr)
    for name, ms in buckets.items():
        print(f"  {name:<12} {ms * 1e3 / max(1, tokens):>10.1f} us  {100.0 * ms / total:>5.1f}%", file=sys.stderr)


def cmd_run(o: Opts) -> None:
    if o.prompt is None:
        raise UsageError("run needs -p <token ids>")
    prompts = parse_ids(o.prompt)
    ctx = o.ctx or 2048
    batch = o.batch or 8
    llm = _llm(o, max_tokens=min(batch, len(prompts)) * ctx, ctx=ctx)
    if _profile_wanted():          # GHOST_INFER_PROFILE, as the reference's switch is called (src/profile.rs:20-29)
        from .kernels import ops
        ops.profile_start()
    results = llm.generate(prompts, max_new=o.max_new, temperature=o.temp, top_k=o.top_k, top_p=o.top_p,
                           seed=o.seed, batch_size=batch)
    for r in results:
        print(" ".join(str(t) for t in r.tokens))
    print_stats(llm.last_stats)
    if _profile_wanted():
        st = llm.last_stats
        print_profile(ops.profile_stop(), st.prompt_tokens + st.gen_tokens)


def cmd_top(model: str, ids_text: str, dtype: str = "bfloat16") -> None:
    """Top-10 next tokens after the ids; GHOST_INFER_LOGITS_OUT=<file> also dumps every logit as
    little-endian float32 (src/main.rs:1184-1205)."""
    import numpy as np
    from .engine.step import StepEntry
    ids = parse_ids(ids_text)[0]
    llm = _llm(Opts(model=model, dtype=dtype), max_tokens=len(ids) + 64)
    slot = llm.cache.open_slot()
    logits = llm.engine.step([StepEntry(slot, ids, [len(ids) - 1])])[0].cpu().numpy()
    llm.cache.close_slot(slot)
    out = os.environ.get("GHOST_INFER_LOGITS_OUT")
    if out:
        logits.astype("<f4").tofile(out)
    mx = float(logits.max())
    total = float(np.exp(logits.astype(np.float64) - mx).sum())
    print(f"{len(ids)} prompt tokens: {ids}")
    for i in np.argsort(-logits, kind="stable")[:10]:
        p = math.exp(float(logits[i]) - mx) / total
        print(f"{int(i):>7}  {p:>8.4f}  logprob {math.log(p):>8.4f}")


def cmd_kvcheck(model: str, ids_file: str, out_file: str, tail: int, dtype: str = "bfloat16") -> None:
    """All but the last `tail` ids as a prompt, those one at a time: per token the model's pick and the
    log-probability of the text's token (src/main.rs:1212-1239)."""
    import numpy as np
    from .engine.step import StepEntry
    with open(ids_file) as f:
        ids = parse_ids(f.read())[0]
    if len(ids) <= tail + 1:
        raise UsageError(f"the text has {len(ids)} tokens, not more than {tail}")
    llm = _llm(Opts(model=model, dtype=dtype), max_tokens=len(ids) + 64)
    slot = llm.cache.open_slot()
    split = len(ids) - tail
    t0 = time.time()
    logits = llm.engine.step([StepEntry(slot, ids[:split], [split - 1])])
    print(f"[read {split} tokens in {time.time() - t0:.1f}s]", file=sys.stderr)
    lines, nll = [], 0.0
    for tok in ids[split:]:
        l = logits[0].cpu().numpy().astype(np.float64)
        mx = l.max()
        lp = (l[tok] - mx) - math.log(np.exp(l - mx).sum())
        nll -= lp
        lines.append(f"{int(l.argmax())} {lp:.5f}\n")
        logits = llm.engine.step([StepEntry(slot, [tok], [0])])
    llm.cache.close_slot(slot)
    with open(out_file, "w") as f:
        f.writelines(lines)
    print(f"[{tail} tokens: mean NLL {nll / tail:.4f}, perplexity {math.exp(nll / tail):.3f}]", file=sys.stderr)


def cmd_bench(o: Opts) -> None:
    """Fixed workload: a prompt of --prompt-len tokens, then -n greedy tokens; best of 3 rounds; an FNV-1a
    hash of the tokens to compare builds (src/main.rs:1241-1285)."""
    import numpy as np
    batch = o.batch or 1
    llm = _llm(o, max_tokens=batch * (o.prompt_len + o.max_new + 8 + 64))
    vocab = llm.model.spec.vocab_size
    rng = np.random.default_rng(1)
    prompts = [rng.integers(0, vocab, size=o.prompt_len).tolist() for _ in range(batch)]
    best_pp = best_tg = 0.0
    rounds = max(1, int(os.environ.get("GHOST_INFER_BENCH_ROUNDS", "3")))
    for rnd in range(rounds):
        res = llm.generate(prompts, max_new=o.max_new, temperature=0.0, top_k=0, top_p=1.0, seed=1,
                           stop_token_ids=(), batch_size=batch)
        st = llm.last_stats
        h = 0xcbf29ce484222325
        for t in res[0].tokens:
            h = ((h ^ t) * 0x100000001b3) & 0xFFFFFFFFFFFFFFFF
        pp = st.prompt_tokens / max(st.prompt_secs, 1e-9)
        tg = st.gen_tokens / max(st.gen_secs, 1e-9)
        best_pp, best_tg = max(best_pp, pp), max(best_tg, tg)
        print(f"round {rnd}: {tg:.1f} tok/s, tokens {h:016x}", file=sys.stderr)
    print(f"prompt {o.prompt_len} tok x {batch}: {best_pp:>8.1f} tok/s | generate {o.max_new} tok x {batch}: {best_tg:>7.1f} tok/s | {o.dtype}")


def cmd_inspect(model_dir: str) -> None:
    from .config import read_config_json
    from .weights.loader import _open_files
    raw = read_config_json(model_dir)
    files = _open_files(model_dir)
    entries = [e for f in files for e in f.entries.values()]
    size = sum(e.end - e.begin for e in entries)
    print(f"safetensors  {len(raw)} config keys  {len(entries)} tensors  {size / 1e6:.1f} MB")
    print("\n== config ==")
    for k in sorted(raw):
        print(f"{k:<45} {json.dumps(raw[k])}")
    print("\n== tensors (first 12) ==")
    for e in sorted(entries, key=lambda e: e.name)[:12]:
        print(f"{e.name:<48} {e.dtype:<6} {list(e.shape)}")
    by_type = {}
    for e in entries:
        n = 1
        for s in e.shape:
            n *= s
        c, t = by_type.get(e.dtype, (0, 0))
        by_type[e.dtype] = (c + 1, t + n)
    print("\n== tensor types ==")
    for ty in sorted(by_type):
        c, t = by_type[ty]
        print(f"{ty:<8} {c:>4} tensors  {t / 1e6:>8.2f} M params")


def cmd_random(args: List[str]) -> None:
    from .weights import write_random_model
    if len(args) < 2:
        raise UsageError("random needs <config.json> <out dir>")
    seed, dtype = 0, "bfloat16"
    it = iter(args[2:])
    for a in it:
        if a == "--seed":
            seed = int(next(it))
        elif a == "--dtype":
            dtype = next(it)
        else:
            raise UsageError(f"unknown option {a}")
    with open(args[0]) as f:
        raw = json.load(f)
    write_random_model(args[1], raw, seed=seed, dtype=dtype)
    print(f"wrote {args[1]} (seed {seed}, {dtype})")


def _take_dtype(rest: List[str]):
    """Splits a trailing or embedded `--dtype <t>` off the positional arguments of `top` and `kvcheck`."""
    dtype, pos = "bfloat16", []
    it = iter(rest)
    for a in it:
        if a == "--dtype":
            try:
                dtype = next(it)
            except StopIteration:
                raise UsageError("--dtype needs a value") from None
        else:
            pos.append(a)
    return pos, dtype


def main(argv: Optional[List[str]] = None) -> int:
    args = list(sys.argv[1:] if argv is None else argv)
    cmd, rest = (args[0] if args else None), args[1:]
    try:
        if cmd in ("top", "kvcheck"):
            rest, dtype = _take_dtype(rest)
        if cmd == "inspect" and len(rest) == 1:
            cmd_inspect(rest[0])
        elif cmd == "top" and len(rest) == 2:
            cmd_top(rest[0], rest[1], dtype)
        elif cmd == "bench" and rest:
            cmd_bench(parse_opts(rest))
        elif cmd == "kvcheck" and len(rest) == 4:
            cmd_kvcheck(rest[0], rest[1], rest[2], int(rest[3]), dtype)
        elif cmd == "run" and rest:
            cmd_run(parse_opts(rest))
        elif cmd == "random":
            cmd_random(rest)
        else:
            sys.stderr.write(USAGE)
            return 2
    except UsageError as e:
        print(f"error: {e}", file=sys.stderr)
        return 1
    except Exception as e:  # the reference prints "error: ..." and exits 1 (src/main.rs:241-246)
        print(f"error: {e}", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
