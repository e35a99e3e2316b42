"""Times one kernel at one shape with CUDA events and relates it to the roofline.

    python -m ghost_infer_b200.kernels.microbench --kernel gemm_stream --m 8 --n 28672 --k 4096
    python -m ghost_infer_b200.kernels.microbench --kernel attn_decode --batch 8 --context 2048

Kernels: gemm_stream, gemm_skinny (decode products), gemm_tc (prefill product), attn_decode, attn_prefill (mma.sync),
attn_prefill_t5 (tcgen05),
rmsnorm, rope, sample.  Operands rotate through enough different buffers to exceed the L2 cache, so a bytes
figure is a DRAM figure.  The same command under `ncu --clock-control none -k regex:<kernel> -c 3` profiles exactly these launches.
The reference times whole runs only (`bench`, src/main.rs:1241-1285) and, per operation, wall-clock buckets
(src/profile.rs:7-46); per-kernel device timing is what a roofline needs.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from . import ops

L2_BYTES = 126 << 20


def _peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


def _time(fn, n_rot, iters, warmup):
    for i in range(warmup):
        fn(i % n_rot)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(iters):
        fn(i % n_rot)
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e3 / iters      # microseconds


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--kernel", required=True)
    ap.add_argument("--m", type=int, default=8)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--mode", default="store", choices=["store", "accum", "swiglu", "f32"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--own-tiles", type=int, default=0, help="attn_decode: slices of that many tiles of each sequence's own span")
    ap.add_argument("--tile-keys", type=int, default=0, help="attn_decode: 16 or 32 keys per tile (default: the engine's)")
    ap.add_argument("--merge-inside", type=int, default=-1, help="attn_decode: 1 = slices merged by the last block, 0 = by a second kernel")
    ap.add_argument("--tail", type=int, default=1, help="gemm_tc: 0 = full-width tiles only, 1 = narrower tiles in an unfilled last round")
    ap.add_argument("--stages", type=int, default=0, help="attn_decode: depth of each warp's ring of tiles (2 to 4)")
    ap.add_argument("--keys-on-rows", type=int, default=-1, help="attn_decode: warps per block of the kernel with the keys on the tile's rows (0: the other kernel; default: the engine's choice)")
    ap.add_argument("--shortest", type=int, default=0, help="attn_decode: lengths uniform in [shortest, context] instead of all equal")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--pdl", action="store_true")
    args = ap.parse_args()
    dev = "cuda:0"
    ops.set_pdl(args.pdl)
    if args.keys_on_rows >= 0:
        ops.TUNE["attn_keys_on_rows"] = args.keys_on_rows > 0
        if args.keys_on_rows > 0:
            ops.TUNE["attn_kr_warps"] = args.keys_on_rows
            if args.stages:
                ops.TUNE["attn_kr_stages"] = args.stages
    hbm, tflops, src = _peaks()
    bf = torch.bfloat16
    mode = {"store": ops.SKINNY_STORE_BF16, "accum": ops.SKINNY_ACCUM_F32, "swiglu": ops.SKINNY_SWIGLU, "f32": ops.SKINNY_STORE_F32}[args.mode]
    out = {"kernel": args.kernel, "peaks": src}
    if args.kernel in ("gemm_stream", "gemm_skinny", "gemm_tc"):
        M, N, K = args.m, args.n, args.k
        ops.gemm_tc_tail_tiles(bool(args.tail))
        n_rot = max(2, L2_BYTES * 2 // (N * K * 2) + 1)
        ws = [torch.randn(N, K, device=dev, dtype=bf) * 0.02 for _ in range(n_rot)]
        x = torch.randn(M, K, device=dev, dtype=bf)
        cols = N // 2 if args.mode == "swiglu" else N
        o = torch.zeros(M, cols, device=dev, dtype=bf if args.mode in ("store", "swiglu") else torch.float32)
        fn = {"gemm_stream": ops.gemm_stream, "gemm_skinny": ops.gemm_skinny, "gemm_tc": ops.gemm_tc}[args.kernel]
        us = _time(lambda i: fn(x, ws[i], mode, o), n_rot, args.iters, args.warmup)
        flops, nbytes = 2.0 * M * N * K, N * K * 2 + M * K * 2 + o.numel() * o.element_size()
        out.update(shape=[M, N, K], mode=args.mode, tail=args.tail, us=round(us, 2), tflops=round(flops / us / 1e6, 1),
                   gbs=round(nbytes / us / 1e3, 1), frac_hbm=round(nbytes / us / 1e3 / hbm, 3),
                   frac_tensor=round(flops / us / 1e6 / tflops, 3))
    elif args.kernel in ("attn_decode", "attn_prefill", "attn_prefill_t5"):
        B, S, H, KV, hd = args.batch, args.context, args.heads, args.kv_heads, args.head_dim
        pages_per = (S + 63) // 64
        n_sets = max(2, L2_BYTES * 2 // (B * pages_per * KV * 64 * hd * 2 * 2) + 1) if args.kernel == "attn_decode" else 1
        kc = torch.randn(n_sets * B * pages_per + 1, KV, 64, hd, device=dev, dtype=bf)
        vc = torch.randn_like(kc)
        tables = [(torch.arange(B * pages_per, dtype=torch.int32, device=dev).reshape(B, pages_per) + 1 + s * B * pages_per) for s in range(n_sets)]
        slots = torch.arange(B, dtype=torch.int32, device=dev)
        scale = hd ** -0.5
        if args.kernel == "attn_decode":
            q = torch.randn(B, (H + 2 * KV) * hd, device=dev, dtype=bf)
            lens = torch.full((B,), S, dtype=torch.int32, device=dev)
            if args.shortest:
                lens = torch.randint(args.shortest, S + 1, (B,), generator=torch.Generator().manual_seed(0)).to(torch.int32).to(dev)
            # the engine's choice (StepContext.decode_splits): one wave of as many blocks as an SM holds, slices of at least 128 keys
            sms = torch.cuda.get_device_properties(0).multi_processor_count
            per_sm = ops.attn_decode_blocks_per_sm(hd, True)
            splits, own = ops.attn_decode_plan(B, S, sms, H, KV, hd, None, bf, lens.tolist())
            if args.splits or args.own_tiles:
                splits, own = args.splits or 1, args.own_tiles
            tile = args.tile_keys or int(ops.TUNE["attn_tile_keys"])
            if own:
                splits = max(splits, (S + own * tile - 1) // (own * tile))
            inside = None if args.merge_inside < 0 else bool(args.merge_inside)
            o = torch.empty(B, H * hd, device=dev, dtype=bf)
            po = torch.empty(B * H * splits * hd, device=dev)
            pml = torch.empty(B * H * splits * 2, device=dev)
            us = _time(lambda i: ops.attn_decode_tc(q, kc, vc, tables[i], slots, lens, B, H, KV, hd, scale, None, splits, o, po, pml,
                                                    tile_keys=tile, own_tiles=own, merge_inside=inside, stages=args.stages or None),
                       n_sets, args.iters, args.warmup)
            nbytes = int(lens.sum()) * KV * hd * 2 * 2
            out.update(shape=[B, S, H, KV, hd], shortest=args.shortest, splits=splits, own_tiles=own, tile_keys=tile,
                       merge_inside=inside, stages=args.stages, keys_on_rows=int(ops.TUNE["attn_kr_warps"]) if ops.TUNE["attn_keys_on_rows"] else 0,
                       us=round(us, 2), gbs=round(nbytes / us / 1e3, 1), frac_hbm=round(nbytes / us / 1e3 / hbm, 3))
        else:
            q = torch.randn(B * S, (H + 2 * KV) * hd, device=dev, dtype=bf)
            cu = (torch.arange(B + 1, dtype=torch.int32, device=dev) * S)
            pos0 = torch.zeros(B, dtype=torch.int32, device=dev)
            o = torch.empty(B * S, H * hd, device=dev, dtype=bf)
            fn = ops.attn_prefill_t5 if args.kernel == "attn_prefill_t5" else ops.attn_prefill_tc
            us = _time(lambda i: fn(q, kc, vc, tables[0], cu, slots, pos0, B, S, H, KV, hd, scale, None, o),
                       1, args.iters, args.warmup)
            flops = 2.0 * B * H * hd * S * (S + 1)
            out.update(shape=[B, S, H, KV, hd], us=round(us, 2), tflops=round(flops / us / 1e6, 1),
                       frac_tensor=round(flops / us / 1e6 / tflops, 3))
    elif args.kernel == "rmsnorm":
        x = torch.randn(args.m, args.k, device=dev)
        w = torch.ones(args.k, device=dev, dtype=bf)
        us = _time(lambda i: ops.rmsnorm(x, w, 1e-5, bf), 1, args.iters, args.warmup)
        out.update(shape=[args.m, args.k], us=round(us, 2))
    elif args.kernel == "sample":
        logits = torch.randn(args.m, args.n, device=dev)
        state = torch.arange(1, args.m + 1, dtype=torch.int64, device=dev)
        us_g = _time(lambda i: ops.sample(logits, 0.0, 0, 1.0), 1, args.iters, args.warmup)
        us_s = _time(lambda i: ops.sample(logits, 0.7, 40, 0.9, state), 1, args.iters, args.warmup)
        us_t = _time(lambda i: ops.sample(logits, 0.7, 0, 1.0, state), 1, args.iters, args.warmup)
        us_p = _time(lambda i: ops.sample(logits, 0.7, 0, 0.9, state), 1, args.iters, args.warmup)
        out.update(shape=[args.m, args.n], us_greedy=round(us_g, 2), us_top_k_top_p=round(us_s, 2), us_temperature=round(us_t, 2),
                   us_top_p=round(us_p, 2))
    else:
        ap.error(f"unknown kernel {args.kernel}")
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
