"""Shared pieces of the GPU tests: the oracle's logits, engines over tiny models, and the tolerances.

Tolerances are set from the arithmetic, not from what passes:
* 32-bit path: products of a few hundred terms accumulated in float32 and a dozen dependent stages give
  relative errors of a few 1e-6; the bound is 3e-5 of the sequence's largest |logit| (at least 1).
* bfloat16 path: activations are rounded to 8 significant bits between kernels (relative 2^-9 each), a
  dozen roundings per layer add up like a random walk; the bound is 2.5% of the largest |logit| for the
  worst element and 0.6% for the root mean square.  A misplaced position, slot or head moves logits by
  tens of percent, far outside both.
"""
import numpy as np
import torch

import ghost_infer_b200 as gi
import plain_llama as pl

_ORACLE = {}


def oracle(model_dir):
    if model_dir not in _ORACLE:
        _ORACLE[model_dir] = pl.read_model(model_dir)
    return _ORACLE[model_dir]


def plain_logits(model_dir, tokens):
    cfg, w = oracle(model_dir)
    return pl.forward(cfg, w, list(tokens))


def make_engine(model_dir, dtype, max_tokens=64 * 48, max_seq_len=2048, max_slots=None):
    """The tiny models' own `max_position_embeddings` are small (128 to 1,024); the tests run sequences past
    them on purpose (pages, slices and buckets need length), which a cache only allows when asked."""
    model = gi.Model.from_pretrained(model_dir, dtype=dtype, device="cuda:0")
    cache = model.new_cache(max_tokens=max_tokens, max_seq_len=max_seq_len, max_slots=max_slots,
                            beyond_trained_positions=True)
    return gi.Engine(model, cache)


def check_logits(got, ref, dtype, what=""):
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    scale = max(1.0, float(np.abs(ref).max()))
    err = np.abs(got - ref)
    if dtype == "float32":
        assert err.max() <= 3e-5 * scale, f"{what}: max error {err.max():.3e} (scale {scale:.2f}) at {np.unravel_index(err.argmax(), err.shape)}"
    else:
        rms = float(np.sqrt((err ** 2).mean()))
        assert err.max() <= 0.025 * scale, f"{what}: max error {err.max():.3e} (scale {scale:.2f}) at {np.unravel_index(err.argmax(), err.shape)}"
        assert rms <= 0.006 * scale, f"{what}: rms error {rms:.3e} (scale {scale:.2f})"


def tokens_for(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab_size"], size=n).tolist()


def paged_from_dense(k_dense, v_dense, lens, n_pages_extra=3, seed=0, poison=float("nan")):
    """Scatters dense per-sequence keys/values [B, S, KV, hd] into shuffled pages.
    Returns (kcache, vcache [pages, KV, 64, hd], block_table int32 [B, max_pages]).  Rows past a sequence's
    length and unused pages are filled with `poison`, so that a kernel that reads them shows it."""
    B, S, KV, hd = k_dense.shape
    per = (S + 63) // 64
    total = B * per + n_pages_extra + 1
    g = torch.Generator().manual_seed(seed)
    order = (torch.randperm(total - 1, generator=g) + 1).tolist()
    kc = torch.full((total, KV, 64, hd), poison, dtype=k_dense.dtype, device=k_dense.device)
    vc = torch.full((total, KV, 64, hd), poison, dtype=k_dense.dtype, device=k_dense.device)
    kc[0] = 0
    vc[0] = 0
    bt = torch.zeros((B, per), dtype=torch.int32)
    it = iter(order)
    for b in range(B):
        for p in range((lens[b] + 63) // 64):
            page = next(it)
            bt[b, p] = page
            n = min(64, lens[b] - p * 64)
            kc[page, :, :n] = k_dense[b, p * 64:p * 64 + n].transpose(0, 1)
            vc[page, :, :n] = v_dense[b, p * 64:p * 64 + n].transpose(0, 1)
    return kc, vc, bt.to(k_dense.device)
