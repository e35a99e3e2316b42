#!/usr/bin/env python3
"""Benchmark: Llama-3.1-8B-shaped random bf16 weights on one B200.

Prints ONE JSON line.  `value` is decoded tokens per second at batch 8 from 2,048-token contexts (device
time over `--steps` decode steps, sampling included); `e2e` is the same through the Python entry point
with host tokens in and out; `prefill` is one 2,048-token prompt; `points` holds decode at batch 1 and 64;
`roofline` relates the decode step's bytes (every weight once, plus the cache of the live requests) to the
measured copy bandwidth; `workloads` holds the baseline's other two shapes (Llama-3.2-1B: batch 64 with unequal
prompts; Llama-3.2-3B: batch 8 with 16,384-token prompts) run end to end through the entry point, each with its
own bytes per step and roofline fraction; `clocks_points` holds the SM clock seen during each timed point.
With --gpus N > 1 it says that this library runs on one GPU and exits with 2.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIG_8B = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 4096, "num_hidden_layers": 32, "num_attention_heads": 32,
    "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336, "vocab_size": 128256,
    "max_position_embeddings": 131072, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
}
CONTEXT = 8192
PROMPT = 2048


def _llama32(hidden, layers, heads, inter):
    return {
        "architectures": ["LlamaForCausalLM"], "hidden_size": hidden, "num_hidden_layers": layers, "num_attention_heads": heads,
        "num_key_value_heads": 8, "head_dim": hidden // heads, "intermediate_size": inter, "vocab_size": 128256,
        "max_position_embeddings": 131072, "rope_theta": 500000.0,
        "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                         "original_max_position_embeddings": 8192},
        "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
    }


# The other two workloads of the baseline: not the headline, run with --workload 1b / 3b.
WORKLOADS = {
    "1b": dict(config=_llama32(2048, 16, 32, 8192), batch=64, prompt=(128, 2048), new=256, step_tokens=None,
               name="Llama-3.2-1B shape, batch 64, prompts uniform in [128, 2048], 256 decode steps"),
    "3b": dict(config=_llama32(3072, 28, 24, 8192), batch=8, prompt=(16384, 16384), new=512, step_tokens=32768,
               name="Llama-3.2-3B shape, batch 8, 16,384-token prompts, 512 decode steps"),
}


def measure_workload(key, new_tokens=None, clocks=None, no_pdl=False):
    """One of the other baseline workloads, end to end through the Python entry point (host token ids in and out,
    sampling included); returns its record."""
    import numpy as np
    import torch
    import ghost_infer_b200 as gi
    from ghost_infer_b200.kernels import ops
    w = WORKLOADS[key]
    cfg = w["config"]
    ops.set_pdl(not no_pdl)
    rng = np.random.default_rng(0)
    lo, hi = w["prompt"]
    lens = rng.integers(lo, hi + 1, size=w["batch"]).tolist()
    prompts = [rng.integers(0, cfg["vocab_size"], size=n).tolist() for n in lens]
    new = new_tokens or w["new"]
    max_tokens = sum(((n + new + 63) // 64) * 64 for n in lens) + 64 * w["batch"]
    llm = gi.LLM(cfg, dtype="bfloat16", device="cuda:0", max_tokens=max_tokens, max_slots=w["batch"],
                 max_seq_len=hi + new + 64, seed=0)
    kw = dict(temperature=0.0, stop_token_ids=(), batch_size=w["batch"], max_step_tokens=w["step_tokens"])
    # warm-up with the whole batch: the first step of a shape obtains its device memory, which must not be timed
    llm.generate(prompts, max_new=4, **kw)
    torch.cuda.synchronize()
    t0 = time.time()
    llm.generate(prompts, max_new=new, time_steps_every=8, **kw)
    t1 = time.time()
    st = llm.last_stats
    layers = cfg["num_hidden_layers"]
    nums = model_numbers(cfg, layers)
    tied = bool(cfg.get("tie_word_embeddings"))
    weight_bytes = 2 * (layers * nums["linear_params_per_layer"] + nums["head_params"] + nums["norm_params"])
    steps = new - 1                     # every new token but the first (which the prompt step's logits give) costs a decode step
    mean_cached = sum(lens) + w["batch"] * (new / 2.0)
    step_bytes = weight_bytes + mean_cached * nums["kv_bytes_per_token"]
    ms = st.gen_secs * 1e3 / max(1, steps)
    pk = peaks()
    achieved = step_bytes / (ms * 1e-3) / 1e9
    dev_ms = sorted(st.step_ms)
    rec = {
        "name": w["name"], "value": round((st.gen_tokens - w["batch"]) / st.gen_secs, 1), "unit": "tokens/s", "ms_per_step": round(ms, 4),
        "device_ms_per_step_median": round(dev_ms[len(dev_ms) // 2], 4) if dev_ms else None,
        "steps": steps, "batch": w["batch"], "layers": layers, "layers_of_model": layers, "tied_head": tied,
        "prompt_tokens": st.prompt_tokens, "prompt_min": min(lens), "prompt_max": max(lens), "new_tokens": new,
        "bytes_per_step": int(step_bytes),
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "prefill": {"value": round(st.prompt_tokens / st.prompt_secs, 1), "tokens": st.prompt_tokens, "ms": round(st.prompt_secs * 1e3, 1)},
        "through": "LLM.generate: wall clock of the decode loop, host tokens in and out",
    }
    if clocks is not None:
        rec["clocks"] = clocks.window(t0, t1)
    del llm
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    return rec


def run_workload(key, args):
    """`--workload 1b|3b`: that workload alone, as one JSON line."""
    clocks = ClockSampler()
    clocks.start()
    rec = measure_workload(key, None if args.steps == 64 else max(4, args.steps), clocks, args.no_pdl)
    clocks.stop()
    print(json.dumps(dict(rec, metric=f"{rec['name']}: decode tok/s through LLM.generate", n_gpus=1, dtype="bf16", impl="ours",
                          data="synthetic")))
    return 0


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples the SM clock and the throttle reasons every 20 ms (NVML; nvidia-smi every 100 ms where NVML cannot be
    loaded) with the wall-clock time of each sample, so that every timed region can be given the samples that fell
    into it.  Reads only; no setting of the GPU is touched."""
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self):
        self.rows = []          # (time, sm MHz, max MHz, set of reasons)
        self.proc = None
        self._stop = threading.Event()
        self._thread = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(0)
            mx = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)
            masks = [pynvml.nvmlClocksEventReasonHwSlowdown, pynvml.nvmlClocksEventReasonHwThermalSlowdown,
                     pynvml.nvmlClocksEventReasonSwThermalSlowdown, pynvml.nvmlClocksEventReasonSwPowerCap]

            def loop():
                while not self._stop.wait(0.02):
                    try:
                        sm = pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)
                        bits = pynvml.nvmlDeviceGetCurrentClocksEventReasons(h)
                    except Exception:
                        continue
                    self.rows.append((time.time(), int(sm), int(mx), {n for n, m in zip(self.NAMES, masks) if bits & m}))

            self._thread = threading.Thread(target=loop, daemon=True)
            self._thread.start()
            return
        except Exception:
            pass
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self._thread = threading.Thread(target=self._read, daemon=True)
            self._thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            c = [x.strip() for x in line.split(",")]
            if len(c) >= 6 and c[0].isdigit() and c[1].isdigit():
                self.rows.append((time.time(), int(c[0]), int(c[1]),
                                  {n for i, n in enumerate(self.NAMES) if c[2 + i].lower().startswith("active")}))

    def window(self, t0=None, t1=None):
        """Median SM clock, the highest clock the GPU offers and every reason seen among the samples of [t0, t1]."""
        rows = [r for r in list(self.rows) if (t0 is None or r[0] >= t0) and (t1 is None or r[0] <= t1)]
        sm = sorted(r[1] for r in rows)
        reasons = sorted(set().union(*[r[3] for r in rows])) if rows else []
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max((r[2] for r in rows), default=None),
                "reasons": reasons, "samples": len(sm)}

    def stop(self):
        self._stop.set()
        if self.proc is not None:
            self.proc.terminate()
        return self.window()


def model_numbers(cfg, layers):
    d, H, KV, hd = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    F, V = cfg["intermediate_size"], cfg["vocab_size"]
    per_layer = (H + 2 * KV) * hd * d + d * H * hd + 3 * F * d
    return {"linear_params_per_layer": per_layer, "head_params": V * d, "norm_params": (2 * layers + 1) * d,
            "kv_bytes_per_token": 2 * layers * KV * hd * 2}


def decode_timeline(ops, decode_run, layers, steps, warmup, batch=8):
    """Prints, for the last decode step's streamed products (q/k/v, o, gate/up, down of every layer, then the head), the
    times of their blocks' stamps relative to the end of the product before: how long the kernels between two
    products take (the wait), how long a product streams, how far its blocks' ends spread."""
    import numpy as np
    per_step = 4 * layers + 1
    ops.stream_timeline_start(2 * per_step)
    decode_run(batch, steps, warmup)
    tl, n = ops.stream_timeline_stop()
    live = [i for i in range(tl.shape[0]) if tl[i, :, 0].max() > 0]
    order = sorted(live, key=lambda i: tl[i, :, 0][tl[i, :, 0] > 0].min())[-per_step:]
    names = ["q/k/v", "o", "gate/up", "down"]
    print(f"{n} launches stamped; the last step's {len(order)} streamed products, microseconds after the end of the product before")
    print(f"{'product':8s} {'first entry':>11s} {'wait over':>10s} {'first stage':>11s} {'last load':>10s} {'last product (min/med/max)':>27s} {'end (med/max)':>15s}")
    prev_end = None
    for k, i in enumerate(order):
        used = tl[i, :, 0] > 0
        t = tl[i, used, :]
        if prev_end is None:
            prev_end = t[:, 0].min()
        e = (t - prev_end).astype(np.float64) / 1e3          # the subtraction in integers: the clock's values need 61 bits
        name = names[k % 4] if k < len(order) - 1 else "head"
        print(f"{name:8s} {e[:, 0].min():11.2f} {np.median(e[:, 3]):10.2f} {np.median(e[:, 4]):11.2f} {np.median(e[:, 5]):10.2f} "
              f"{e[:, 6].min():9.2f}/{np.median(e[:, 6]):7.2f}/{e[:, 6].max():7.2f} {np.median(e[:, 7]):7.2f}/{e[:, 7].max():7.2f}")
        prev_end = t[:, 7].max()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the named configuration (recorded in config)")
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--workload", default="8b", choices=["8b", "1b", "3b"], help="8b: the headline; 1b, 3b: the baseline's other workloads")
    ap.add_argument("--tune", default="", help="overrides of kernel choices, e.g. small_skinny=0,attn_waves=2")
    ap.add_argument("--only", default="", choices=["", "prefill", "decode", "timeline"],
                    help="run one phase alone and print its time (a short program for a launch list under a profiler; no bench "
                         "line).  timeline: a table of when the streamed products of a decode step start, wait, stream and end")
    ap.add_argument("--batch", type=int, default=8, help="sequences per decode step for --only decode|timeline (the bench line is always batch 8)")
    ap.add_argument("--shape", default="8b", choices=["8b", "1b", "3b"], help="layer sizes for --only (the bench line is always the 8B shape)")
    ap.add_argument("--held", type=int, default=PROMPT, help="tokens each sequence holds for --only decode|timeline")
    ap.add_argument("--no-pdl", action="store_true", help="launch kernels strictly one after another (no programmatic dependent launch)")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "the reference is a Rust program for Windows that reads GGUF "
                          "files; it is no Python package, and cargo/rustc are not installed, so it cannot be built or installed here"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.tune:
        from ghost_infer_b200.kernels import ops as _ops
        for kv in filter(None, args.tune.split(",")):
            k, v = kv.split("=")
            _ops.TUNE[k] = type(_ops.TUNE[k])(float(v))
    if args.workload != "8b":
        return run_workload(args.workload, args)
    W = max(3, args.warmup)
    K = max(1, args.steps)

    import numpy as np
    import torch
    import ghost_infer_b200 as gi
    from ghost_infer_b200.kernels import ops

    dev = "cuda:0"
    ops.set_pdl(not args.no_pdl)
    cfg = dict(CONFIG_8B if not (args.only and args.shape != "8b") else WORKLOADS[args.shape]["config"])
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    layers = cfg["num_hidden_layers"]
    pk = peaks()
    nums = model_numbers(cfg, layers)
    t0 = time.time()
    llm = gi.LLM(cfg, dtype="bfloat16", device=dev, max_tokens=64 * CONTEXT, max_slots=64, max_seq_len=CONTEXT, seed=0)
    eng, cache = llm.engine, llm.cache
    for g in cache.groups:            # contexts stand in for prompts already read: random keys and values
        g.k.normal_(0.0, 0.5)
        g.v.normal_(0.0, 0.5)
    torch.cuda.synchronize()
    load_s = time.time() - t0
    rng = np.random.default_rng(0)
    V = cfg["vocab_size"]
    clocks = ClockSampler()

    def decode_run(batch, steps, warmup, held=PROMPT):
        """`steps` timed decode steps of `batch` sequences that each hold `held` tokens; device time."""
        slots = [cache.open_slot() for _ in range(batch)]
        cache.reserve([(s, held) for s in slots])
        for s in slots:
            cache.commit(s, held)
        toks = rng.integers(0, V, size=batch).tolist()
        runner = eng.decoder(slots)
        picked = torch.zeros(batch, dtype=torch.int32, device=dev)
        logits = runner.forward(tokens=toks)
        for _ in range(warmup):
            ops.sample(logits, 0.0, 0, 1.0, out=picked)
            logits = runner.forward(dev_tokens=picked)
        torch.cuda.synchronize()
        l0 = ops.launches
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):                       # a decode step: pick the token, run it
            ops.sample(logits, 0.0, 0, 1.0, out=picked)
            logits = runner.forward(dev_tokens=picked)
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop) / steps
        launched = ops.launches - l0
        ctx_tokens = sum(cache.length(s) for s in slots)
        for s in slots:
            cache.close_slot(s)
        return ms, launched, ctx_tokens

    if args.only == "timeline":
        return decode_timeline(ops, decode_run, layers, K, W, args.batch)
    if args.only == "decode":
        ms, n, _ = decode_run(args.batch, K, W, held=args.held)
        print(json.dumps({"only": "decode", "shape": args.shape, "layers": layers, "batch": args.batch, "held": args.held,
                          "ms_per_step": round(ms, 4), "launches_per_step": n // K}))
        return 0
    if args.only == "prefill":
        prompt = rng.integers(0, V, size=PROMPT).tolist()
        for i in range(W + K):
            if i == W:
                torch.cuda.synchronize()
                t0 = time.time()
            s = cache.open_slot()
            eng.step([gi.StepEntry(s, prompt, [PROMPT - 1])])
            cache.close_slot(s)
        torch.cuda.synchronize()
        print(json.dumps({"only": "prefill", "layers": layers, "tokens": PROMPT, "ms": round((time.time() - t0) * 1e3 / K, 3)}))
        return 0

    clocks.start()
    windows = {}

    def timed(name, fn):
        t_a = time.time()
        out = fn()
        windows[name] = (t_a, time.time())
        return out

    ms8, launches8, ctx8 = timed("decode_b8", lambda: decode_run(8, K, W))
    value = 8 * 1000.0 / ms8
    weight_bytes = 2 * (layers * nums["linear_params_per_layer"] + nums["head_params"] + nums["norm_params"])
    step_bytes = weight_bytes + ctx8 * nums["kv_bytes_per_token"]
    achieved = step_bytes / (ms8 * 1e-3) / 1e9

    points, point_steps = {}, max(50, K)
    point_frac = {}
    if not args.skip_points:
        for b in (1, 64):
            ms, _, ctx = timed(f"decode_b{b}", lambda: decode_run(b, point_steps, W))
            points[f"decode_b{b}"] = round(b * 1000.0 / ms, 1)
            point_frac[f"decode_b{b}"] = round((weight_bytes + ctx * nums["kv_bytes_per_token"]) / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        # the same batch of 8 with the cache's whole length behind it: the last timed step reads 8,192 positions
        ms, _, ctx = timed(f"decode_b8_ctx{CONTEXT}", lambda: decode_run(8, point_steps, W, held=CONTEXT - (W + point_steps + 1)))
        points[f"decode_b8_ctx{CONTEXT}"] = round(8 * 1000.0 / ms, 1)
        point_frac[f"decode_b8_ctx{CONTEXT}"] = round((weight_bytes + ctx * nums["kv_bytes_per_token"]) / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)

    # prefill: one prompt of 2,048 tokens, logits for its last place
    prompt = rng.integers(0, V, size=PROMPT).tolist()
    reps = 9

    def prefill_once():
        s = cache.open_slot()
        out = eng.step([gi.StepEntry(s, prompt, [PROMPT - 1])])
        cache.close_slot(s)
        return out

    def prefill_timed():
        """Every repetition timed by its own pair of events; the median stands (the power cap makes single ones wander)."""
        for _ in range(3):
            prefill_once()
        torch.cuda.synchronize()
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(reps + 1)]
        marks[0].record()
        for i in range(reps):
            prefill_once()
            marks[i + 1].record()
        torch.cuda.synchronize()
        each = sorted(a.elapsed_time(b) for a, b in zip(marks, marks[1:]))
        return each[len(each) // 2], each[0], each[-1]

    pre_ms, pre_min, pre_max = timed("prefill", prefill_timed)
    H, hd = cfg["num_attention_heads"], cfg["head_dim"]
    flops = 2.0 * PROMPT * layers * nums["linear_params_per_layer"] + 2.0 * nums["head_params"] \
        + layers * 4.0 * H * hd * (PROMPT * (PROMPT + 1) / 2)
    pre_frac = flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12)

    # end to end through the Python entry point: host token ids in, host token ids out, every step
    prompts = [rng.integers(0, V, size=PROMPT).tolist() for _ in range(8)]
    e2e_new = max(K, 256)      # long enough that the stretch after the prompt step (a power-capped clock) does not decide the figure
    llm.generate(prompts, max_new=3, temperature=0.0, stop_token_ids=(), batch_size=8)     # warm-up

    def e2e_run():
        llm.generate(prompts, max_new=e2e_new, temperature=0.0, stop_token_ids=(), batch_size=8, time_steps_every=8)
        return llm.last_stats

    st = timed("e2e", e2e_run)
    dev = [round(x, 4) for x in st.step_ms]
    e2e = {"value": round((st.gen_tokens - 8) / st.gen_secs, 1) if st.gen_secs > 0 else None, "unit": "tokens/s",
           "h2d_bytes_per_step": int(eng.bytes_h2d), "d2h_bytes_per_step": 8 * 4,
           "ms_per_step_wall": round(st.gen_secs * 1e3 / max(1, e2e_new - 1), 4),
           # device time per step over stretches of 8 steps (CUDA events in the loop): the first, the median, the last
           "ms_per_step_device": {"first": dev[0], "median": sorted(dev)[len(dev) // 2], "last": dev[-1], "stretches": len(dev)} if dev else None,
           "note": f"LLM.generate, batch 8, {PROMPT}-token prompts, {e2e_new} new tokens each; wall clock of the decode loop"}

    # the baseline's other two workloads, each a model of its own: this one's memory goes back first
    workloads = {}
    if not args.skip_points and not args.layers:
        del llm, eng, cache, prefill_once, prefill_timed, e2e_run, decode_run
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        for key in ("1b", "3b"):
            workloads[key] = measure_workload(key, None, clocks, args.no_pdl)
    clocks.stop()
    clk = clocks.window(*windows["decode_b8"])
    clocks_points = {name: clocks.window(*w) for name, w in windows.items()}
    for key, rec in workloads.items():
        clocks_points[f"workload_{key}"] = rec.pop("clocks", None)
    h2d_bytes = e2e["h2d_bytes_per_step"]

    line = {
        "metric": "Llama-3.1-8B bf16 decode tok/s @ batch 8 (2,048-token contexts)", "value": round(value, 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": round(ms8, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random N(0, 0.02) weights, uniform random token ids, random keys/values as contexts for the device-timed points",
        "impl": "ours",
        "config": {"model": "Llama-3.1-8B shape", "layers": layers, "layers_of_model": full_layers, "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": V, "global_batch": 8, "seq_len": CONTEXT,
                   "prompt_len": PROMPT, "parallelism": "1 gpu", "l2": "inputs larger than L2 (weights read once per step)",
                   "peaks": pk["source"], "load_s": round(load_s, 1)},
        "e2e": e2e,
        "gpu_launches": int(launches8),
        "prefill": {"value": round(PROMPT * 1000.0 / pre_ms, 1), "tokens": PROMPT, "ms": round(pre_ms, 3), "frac": round(pre_frac, 4),
                    "peak_tflops": pk["bf16_tflops"], "ms_min": round(pre_min, 3), "ms_max": round(pre_max, 3), "reps": reps,
                    "frac_of_sustained": round(flops / (pre_ms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": int(step_bytes)},
        "points": points,
        "points_roofline_frac": point_frac,
        "points_steps": point_steps,
        "workloads": workloads,
        "clocks": clk,
        "clocks_points": clocks_points,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
