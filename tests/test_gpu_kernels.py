"""Each kernel alone against a plain float64/float32 PyTorch statement of the same operation, at sizes
other than the tiny models': odd widths, head sizes 16..256, several group sizes, long contexts."""
import math

import numpy as np
import contextlib

import pytest
import torch

from ghost_infer_b200.kernels import ops
from ghost_infer_b200.kernels.library import KernelError
from gpu_helpers import paged_from_dense
import plain_llama as pl

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=1.6e-2, atol=1.6e-2)


@contextlib.contextmanager
def keys_on_rows(warps=4, stages=2):
    """Inside, `ops.attn_decode_tc` runs the kernel that puts a tile's keys on the rows of its products."""
    was = {k: ops.TUNE[k] for k in ("attn_keys_on_rows", "attn_kr_warps", "attn_kr_stages")}
    ops.TUNE.update(attn_keys_on_rows=True, attn_kr_warps=warps, attn_kr_stages=stages)
    try:
        yield
    finally:
        ops.TUNE.update(was)


@contextlib.contextmanager
def heads_on_rows():
    """Inside, `ops.attn_decode_tc` runs the kernel with the group's heads on the rows of its products whatever the
    group's size (the kernel that can also merge its slices and rotate by itself)."""
    was = ops.TUNE["attn_keys_on_rows"]
    ops.TUNE["attn_keys_on_rows"] = False
    try:
        yield
    finally:
        ops.TUNE["attn_keys_on_rows"] = was


def rnd(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


@pytest.mark.parametrize("wdtype", DTYPES)
def test_embed(wdtype):
    table = rnd(301, 70, dtype=wdtype)
    toks = torch.tensor([0, 300, 5, 5, 299], dtype=torch.int32, device=DEV)
    out = ops.embed(table, toks)
    assert out.dtype == torch.float32 and torch.equal(out, table[toks.long()].float())


@pytest.mark.parametrize("odtype", DTYPES)
@pytest.mark.parametrize("wdtype", DTYPES)
@pytest.mark.parametrize("d", [70, 1000, 4096])
def test_rmsnorm(odtype, wdtype, d):
    x = rnd(9, d, seed=1, scale=3.0)
    w = (1 + 0.2 * rnd(d, seed=2)).to(wdtype)
    ref = (x.double() * torch.rsqrt((x.double() ** 2).mean(-1, keepdim=True) + 1e-3) * w.double())
    out = ops.rmsnorm(x, w, 1e-3, odtype)
    torch.testing.assert_close(out.double(), ref, **tol(odtype))
    rows = torch.tensor([8, 0, 3], dtype=torch.int32, device=DEV)
    out = ops.rmsnorm(x, w, 1e-3, odtype, rows=rows)
    torch.testing.assert_close(out.double(), ref[rows.long()], **tol(odtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul(dtype):
    gu = rnd(5, 2 * 301, dtype=dtype, seed=3, scale=2.0)
    g, u = gu[:, :301].double(), gu[:, 301:].double()
    ref = g / (1 + torch.exp(-g)) * u
    torch.testing.assert_close(ops.silu_mul(gu).double(), ref, **tol(dtype))


@pytest.mark.parametrize("adtype", DTYPES)
@pytest.mark.parametrize("wdtype", DTYPES)
@pytest.mark.parametrize("m,n,k", [(7, 96, 37), (1, 301, 80), (130, 65, 129), (64, 64, 16)])
def test_gemm_generic(adtype, wdtype, m, n, k):
    """Odd sizes, as the reference's own matmul test uses (37 x 96 x 7, src/quant.rs:1437-1461); the
    tolerance scales with the size of the terms, not of the sum."""
    a, w = rnd(m, k, dtype=adtype, seed=4), rnd(n, k, dtype=wdtype, seed=5)
    ref = a.double() @ w.double().T
    terms = (a.double().abs() @ w.double().abs().T)
    out = ops.gemm_generic(a, w, out_dtype=torch.float32)
    assert ((out.double() - ref).abs() <= 1e-6 * terms + 1e-7).all()
    out16 = ops.gemm_generic(a, w, out_dtype=torch.bfloat16)
    assert ((out16.double() - ref).abs() <= 2 ** -8 * ref.abs() + 1e-6 * terms + 1e-7).all()
    acc = rnd(m, n, seed=6)
    before = acc.clone()
    ops.gemm_generic(a, w, out=acc, accumulate=True)
    assert ((acc.double() - (before.double() + ref)).abs() <= 1e-6 * (terms + before.abs().double()) + 1e-6).all()


def test_gemm_strided_rows():
    a_full, w = rnd(10, 100, seed=7), rnd(33, 40, seed=8)
    a = a_full[:, 20:60]                       # rows 100 apart, 40 wide
    out_full = torch.zeros(10, 50, device=DEV)
    ops.gemm_generic(a, w, out=out_full[:, 5:38])
    torch.testing.assert_close(out_full[:, 5:38], a @ w.T, rtol=1e-5, atol=1e-5)
    assert float(out_full[:, :5].abs().sum()) == 0 and float(out_full[:, 38:].abs().sum()) == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hd,rot,adjacent", [(16, 16, False), (48, 48, False), (128, 128, False), (64, 32, False), (32, 32, True)])
def test_rope_and_cache_write(dtype, hd, rot, adjacent):
    H, KV, T = 5, 2, 6
    qkv = rnd(T, (H + 2 * KV) * hd, dtype=dtype, seed=9)
    orig = qkv.clone()
    positions = torch.tensor([0, 1, 63, 64, 200, 77], dtype=torch.int32, device=DEV)
    slots = torch.tensor([0, 0, 0, 0, 1, 1], dtype=torch.int32, device=DEV)
    bt = torch.tensor([[3, 1, 0, 0], [2, 5, 6, 4]], dtype=torch.int32, device=DEV)
    kc = torch.zeros(7, KV, 64, hd, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    inv = torch.from_numpy(pl.rotary_inv_freq(rot, 10000.0, None)).to(DEV)
    table = ops.rope_table(positions, inv)
    assert table.shape == (T, rot // 2, 2)
    ops.rope_cache_write(qkv, table, positions, slots, bt, kc, vc, H, KV, hd, rot, adjacent, True)
    pairing = "adjacent" if adjacent else "half"
    o = orig.double().cpu().numpy()
    pos = positions.cpu().numpy()

    def rot_ref(x, heads):
        x = x.reshape(T, heads, hd)
        y = x.copy()
        y[:, :, :rot] = pl.rope(x[:, :, :rot].reshape(T, heads * rot), pos, inv.cpu().numpy(), rot, pairing).reshape(T, heads, rot)
        return y.reshape(T, heads * hd)

    q_ref = rot_ref(o[:, :H * hd], H)
    k_ref = rot_ref(o[:, H * hd:(H + KV) * hd], KV)
    v_ref = o[:, (H + KV) * hd:]
    t = tol(dtype)
    np.testing.assert_allclose(qkv[:, :H * hd].double().cpu().numpy(), q_ref, rtol=t["rtol"], atol=t["atol"])
    assert torch.equal(qkv[:, H * hd:], orig[:, H * hd:])          # k and v rows are left as they were
    for i in range(T):
        page = int(bt[int(slots[i]), int(pos[i]) // 64])
        got_k = kc[page, :, int(pos[i]) % 64].double().cpu().numpy().reshape(-1)
        got_v = vc[page, :, int(pos[i]) % 64].double().cpu().numpy().reshape(-1)
        np.testing.assert_allclose(got_k, k_ref[i], rtol=t["rtol"], atol=t["atol"])
        np.testing.assert_array_equal(got_v, v_ref[i])
    assert float(kc[0].abs().sum()) == 0                            # nobody wrote to the trash page


def attention_ref(q, k, v, lens_q, pos0, H, KV, hd, scale, window):
    """q [B, Q, H*hd] at positions pos0[b]..; k, v dense [B, S, KV, hd].  float64."""
    out = torch.zeros_like(q, dtype=torch.float64)
    g = H // KV
    for b in range(q.shape[0]):
        for i in range(lens_q[b]):
            p = pos0[b] + i
            lo = max(0, p - window + 1) if window else 0
            for h in range(H):
                kk = k[b, lo:p + 1, h // g].double()
                vv = v[b, lo:p + 1, h // g].double()
                s = (kk @ q[b, i, h * hd:(h + 1) * hd].double()) * scale
                out[b, i, h * hd:(h + 1) * hd] = torch.softmax(s, 0) @ vv
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,KV,hd", [(4, 2, 16), (5, 1, 48), (8, 8, 64), (6, 2, 128), (2, 1, 256), (16, 2, 80)])
@pytest.mark.parametrize("window", [None, 37])
def test_attention_prefill(dtype, H, KV, hd, window):
    """Ragged batch: sequences that start at position 0 and one that goes on after 70 cached positions."""
    lens_q, pos0 = [1, 45, 100, 33], [0, 0, 0, 70]
    B, S = 4, 128
    k = rnd(B, S, KV, hd, dtype=dtype, seed=10)
    v = rnd(B, S, KV, hd, dtype=dtype, seed=11)
    q = rnd(B, max(lens_q), H * hd, dtype=dtype, seed=12)
    lens_kv = [p + n for p, n in zip(pos0, lens_q)]
    kc, vc, bt = paged_from_dense(k, v, lens_kv, seed=3)
    flat = torch.cat([q[b, :lens_q[b]] for b in range(B)])
    cu = torch.tensor([0] + list(np.cumsum(lens_q)), dtype=torch.int32, device=DEV)
    slots = torch.arange(B, dtype=torch.int32, device=DEV)
    out = torch.full_like(flat, float("nan"))
    ops.attn_prefill_generic(flat, kc, vc, bt, cu, slots, torch.tensor(pos0, dtype=torch.int32, device=DEV), B,
                             max(lens_q), H, KV, hd, 0.21, window, out)
    ref = attention_ref(q, k, v, lens_q, pos0, H, KV, hd, 0.21, window)
    ref = torch.cat([ref[b, :lens_q[b]] for b in range(B)])
    torch.testing.assert_close(out.double(), ref, **tol(dtype))


@pytest.mark.parametrize("H,KV,hd", [(8, 8, 64), (6, 2, 128), (3, 1, 64), (32, 8, 128)])
@pytest.mark.parametrize("window", [None, 37, 100])
def test_attention_prefill_tensor_cores(H, KV, hd, window):
    """The tensor-core prefill kernel: ragged lengths around its 64-row and 64-key tiles, a sequence that goes on
    after 70 and one after 200 cached positions, pages in shuffled order, unowned rows poisoned with NaN."""
    lens_q, pos0 = [1, 45, 64, 65, 200, 33, 130], [0, 0, 0, 0, 0, 70, 200]
    B, S = len(lens_q), 384
    k = rnd(B, S, KV, hd, dtype=torch.bfloat16, seed=10)
    v = rnd(B, S, KV, hd, dtype=torch.bfloat16, seed=11)
    q = rnd(B, max(lens_q), H * hd, dtype=torch.bfloat16, seed=12)
    lens_kv = [p + n for p, n in zip(pos0, lens_q)]
    kc, vc, bt = paged_from_dense(k, v, lens_kv, seed=3)
    flat = torch.cat([q[b, :lens_q[b]] for b in range(B)])
    cu = torch.tensor([0] + list(np.cumsum(lens_q)), dtype=torch.int32, device=DEV)
    slots = torch.arange(B, dtype=torch.int32, device=DEV)
    out = torch.full_like(flat, float("nan"))
    ops.attn_prefill_tc(flat, kc, vc, bt, cu, slots, torch.tensor(pos0, dtype=torch.int32, device=DEV), B,
                        max(lens_q), H, KV, hd, 0.21, window, out)
    ref = attention_ref(q, k, v, lens_q, pos0, H, KV, hd, 0.21, window)
    ref = torch.cat([ref[b, :lens_q[b]] for b in range(B)])
    torch.testing.assert_close(out.double(), ref, **tol(torch.bfloat16))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,KV,hd", [(4, 2, 16), (5, 1, 48), (8, 8, 64), (32, 8, 128), (2, 1, 256), (24, 2, 80)])
@pytest.mark.parametrize("window,splits", [(None, 1), (None, 5), (100, 1), (100, 3)])
def test_attention_decode(dtype, H, KV, hd, window, splits):
    lens = [1, 64, 65, 700, 333]
    B, S = len(lens), 704
    k = rnd(B, S, KV, hd, dtype=dtype, seed=13)
    v = rnd(B, S, KV, hd, dtype=dtype, seed=14)
    q = rnd(B, 1, H * hd, dtype=dtype, seed=15)
    kc, vc, bt = paged_from_dense(k, v, lens, seed=4)
    out = torch.full((B, H * hd), float("nan"), dtype=dtype, device=DEV)
    part_o = torch.full((B * H * splits * hd,), float("nan"), device=DEV)
    part_ml = torch.full((B * H * splits * 2,), float("nan"), device=DEV)
    ops.attn_decode_generic(q[:, 0], kc, vc, bt, torch.arange(B, dtype=torch.int32, device=DEV),
                            torch.tensor(lens, dtype=torch.int32, device=DEV), B, H, KV, hd, 0.17, window, splits, out,
                            part_o, part_ml)
    ref = attention_ref(q, k, v, [1] * B, [n - 1 for n in lens], H, KV, hd, 0.17, window)[:, 0]
    torch.testing.assert_close(out.double(), ref, **tol(dtype))


@pytest.mark.parametrize("tile_keys", [16, 32])
@pytest.mark.parametrize("H,KV,hd", [(8, 8, 64), (32, 8, 128), (24, 8, 128), (5, 1, 64), (40, 2, 128)])
@pytest.mark.parametrize("window,splits", [(None, 1), (None, 5), (100, 1), (100, 3)])
def test_attention_decode_tensor_cores(tile_keys, H, KV, hd, window, splits):
    """The tensor-core decode kernel: groups of 1, 3, 4, 5 and 20 heads (more than one 16-row tile), pages in
    shuffled order, rows past each sequence's end poisoned with NaN."""
    lens = [1, 31, 64, 65, 700, 333, 96]
    B, S = len(lens), 704
    k = rnd(B, S, KV, hd, dtype=torch.bfloat16, seed=13)
    v = rnd(B, S, KV, hd, dtype=torch.bfloat16, seed=14)
    q = rnd(B, 1, H * hd, dtype=torch.bfloat16, seed=15)
    kc, vc, bt = paged_from_dense(k, v, lens, seed=4)
    out = torch.full((B, H * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    part_o = torch.full((B * H * splits * hd,), float("nan"), device=DEV)
    part_ml = torch.full((B * H * splits * 2,), float("nan"), device=DEV)
    assert ops.attn_decode_tc_ok(q[:, 0], kc, hd)
    with heads_on_rows():
        ops.attn_decode_tc(q[:, 0], kc, vc, bt, torch.arange(B, dtype=torch.int32, device=DEV),
                           torch.tensor(lens, dtype=torch.int32, device=DEV), B, H, KV, hd, 0.17, window, splits, out,
                           part_o, part_ml, tile_keys=tile_keys)
    ref = attention_ref(q, k, v, [1] * B, [n - 1 for n in lens], H, KV, hd, 0.17, window)[:, 0]
    torch.testing.assert_close(out.double(), ref, **tol(torch.bfloat16))


@pytest.mark.parametrize("warps,stages", [(4, 2), (4, 3), (6, 2), (6, 3), (8, 2), (8, 3)])
@pytest.mark.parametrize("H,KV,hd", [(8, 8, 64), (32, 8, 64), (32, 8, 128), (24, 8, 128), (5, 1, 64), (40, 2, 128), (16, 2, 64)])
@pytest.mark.parametrize("window,splits,own_tiles", [(None, 1, 0), (None, 5, 0), (100, 1, 0), (100, 3, 0), (None, 13, 4)])
def test_attention_decode_keys_on_rows(warps, stages, H, KV, hd, window, splits, own_tiles):
    """The decode kernel with a tile's keys on the rows of its products and up to 8 heads on their columns: groups of 1,
    3, 4, 5, 8 and 20 heads (one to three blocks per kv head), 4 to 8 warps, pages in shuffled order, rows past each
    sequence's end poisoned with NaN, equal slices and slices of four tiles of each sequence's own span."""
    lens = [1, 31, 64, 65, 700, 333, 96, 15, 16, 17]
    B, S = len(lens), 704
    k = rnd(B, S, KV, hd, dtype=torch.bfloat16, seed=13)
    v = rnd(B, S, KV, hd, dtype=torch.bfloat16, seed=14)
    q = rnd(B, 1, H * hd, dtype=torch.bfloat16, seed=15)
    kc, vc, bt = paged_from_dense(k, v, lens, seed=4)
    out = torch.full((B, H * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    part_o = torch.full((B * H * splits * hd,), float("nan"), device=DEV)
    part_ml = torch.full((B * H * splits * 2,), float("nan"), device=DEV)
    ops.attn_decode_kr(q[:, 0], kc, vc, bt, torch.arange(B, dtype=torch.int32, device=DEV),
                       torch.tensor(lens, dtype=torch.int32, device=DEV), B, H, KV, hd, 0.17, window, splits, out,
                       part_o, part_ml, own_tiles=own_tiles, warps=warps, stages=stages)
    ref = attention_ref(q, k, v, [1] * B, [n - 1 for n in lens], H, KV, hd, 0.17, window)[:, 0]
    torch.testing.assert_close(out.double(), ref, **tol(torch.bfloat16))


@pytest.mark.parametrize("H,KV,hd", [(8, 8, 64), (32, 8, 128), (5, 1, 64), (40, 2, 128)])
@pytest.mark.parametrize("window", [None, 100])
@pytest.mark.parametrize("own_tiles,tile_keys", [(0, 16), (4, 16), (2, 32), (32, 16)])
def test_attention_decode_merges_its_slices_itself(H, KV, hd, window, own_tiles, tile_keys):
    """The slices merged by the block that finishes last, against the same launch merged by the second kernel: the same
    bits (both add the slices in slice order), and both the operation in 64-bit.  Slices of a fixed number of tiles of
    each sequence's own span: a sequence of one token uses one block, one of 700 many; the launch's other blocks
    leave at once.  Three launches in a row: the counters must be back at zero each time."""
    lens = [1, 31, 64, 65, 700, 333, 96, 129]
    B, S = len(lens), 704
    k = rnd(B, S, KV, hd, dtype=torch.bfloat16, seed=13)
    v = rnd(B, S, KV, hd, dtype=torch.bfloat16, seed=14)
    q = rnd(B, 1, H * hd, dtype=torch.bfloat16, seed=15)
    kc, vc, bt = paged_from_dense(k, v, lens, seed=4)
    slots, lens_t = torch.arange(B, dtype=torch.int32, device=DEV), torch.tensor(lens, dtype=torch.int32, device=DEV)
    splits = 5 if own_tiles == 0 else (704 + own_tiles * tile_keys - 1) // (own_tiles * tile_keys) + 2     # two more than any sequence needs
    ref = attention_ref(q, k, v, [1] * B, [n - 1 for n in lens], H, KV, hd, 0.17, window)[:, 0]
    outs = []
    for inside in (False, True, True, True):
        out = torch.full((B, H * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
        part_o = torch.full((B * H * splits * hd,), float("nan"), device=DEV)
        part_ml = torch.full((B * H * splits * 2,), float("nan"), device=DEV)
        with heads_on_rows():
            ops.attn_decode_tc(q[:, 0], kc, vc, bt, slots, lens_t, B, H, KV, hd, 0.17, window, splits, out, part_o, part_ml,
                               tile_keys=tile_keys, own_tiles=own_tiles, merge_inside=inside)
        torch.testing.assert_close(out.double(), ref, **tol(torch.bfloat16))
        outs.append(out)
    for o in outs[1:]:
        assert torch.equal(o, outs[0])
    assert int(ops._attn_merge_counters(torch.device(DEV)).abs().sum()) == 0


@pytest.mark.parametrize("decode", [False, True, "tc"])
@pytest.mark.parametrize("window", [None, 50])
def test_attention_finds_one_far_key(decode, window):
    """Random keys would hide a missed row among hundreds.  Here one key, far back (or exactly at the
    window's edge), is made to dominate the softmax, and its value is unlike every other."""
    H, KV, hd, n = 4, 2, 32, 600
    k = 0.01 * rnd(1, n, KV, hd, seed=16)
    v = 0.01 * rnd(1, n, KV, hd, seed=17)
    q = rnd(1, 1, H * hd, seed=18)
    pos = n - 1
    for kvh, target in ((0, 3), (1, pos - (window - 1) if window else 130)):
        # the key that matches the query of the group's first head, scaled up
        k[0, target, kvh] = 4.0 * q[0, 0, (kvh * 2) * hd:(kvh * 2 + 1) * hd]
        v[0, target, kvh] = 100.0 + kvh
        if window:
            k[0, pos - window, kvh] = 40.0 * q[0, 0, (kvh * 2) * hd:(kvh * 2 + 1) * hd]   # just outside: must not count
            v[0, pos - window, kvh] = -500.0
    if decode == "tc":
        H, KV, hd = 4, 2, 64
        k, v, q = [x.to(torch.bfloat16) for x in (torch.cat([k, k], -1), torch.cat([v, v], -1), torch.cat(
            [q.view(1, 1, 4, 32), torch.zeros(1, 1, 4, 32, device=DEV)], -1).reshape(1, 1, 4 * 64))]
    kc, vc, bt = paged_from_dense(k, v, [n], seed=5)
    ref = attention_ref(q, k, v, [1], [pos], H, KV, hd, 1.0, window)[:, 0]
    if window:
        assert float(ref[0, 2 * hd]) > 90                    # the edge key is inside and wins for head 2
        assert float(ref.min()) > -1                         # the key just outside the window plays no part
    else:
        assert float(ref[0, 2 * hd]) > 90
    out = torch.zeros((1, H * hd), device=DEV, dtype=q.dtype)
    one = torch.ones(1, dtype=torch.int32, device=DEV)
    if decode == "tc":
        po, pml = torch.zeros(H * 4 * hd, device=DEV), torch.zeros(H * 4 * 2, device=DEV)
        with heads_on_rows():
            ops.attn_decode_tc(q[:, 0], kc, vc, bt, 0 * one, n * one, 1, H, KV, hd, 1.0, window, 4, out, po, pml)
        torch.testing.assert_close(out.double(), ref, rtol=2e-2, atol=2e-2 * float(ref.abs().max()))
        out1 = torch.zeros_like(out)      # the decode kernel with the keys on the rows of its products
        with keys_on_rows(8, 3):
            ops.attn_decode_tc(q[:, 0], kc, vc, bt, 0 * one, n * one, 1, H, KV, hd, 1.0, window, 4, out1, po, pml)
        torch.testing.assert_close(out1.double(), ref, rtol=2e-2, atol=2e-2 * float(ref.abs().max()))
        out2 = torch.zeros_like(out)      # and the prefill kernel: the last position as a one-token chunk
        ops.attn_prefill_tc(q[:, 0], kc, vc, bt, torch.tensor([0, 1], dtype=torch.int32, device=DEV), 0 * one,
                            pos * one, 1, 1, H, KV, hd, 1.0, window, out2)
        torch.testing.assert_close(out2.double(), ref, rtol=2e-2, atol=2e-2 * float(ref.abs().max()))
        # and the tcgen05 prefill kernel, which takes the packed [q | k | v] rows
        packed = torch.cat([q[:, 0], torch.zeros(1, 2 * KV * hd, dtype=q.dtype, device=DEV)], -1).contiguous()
        out3 = torch.zeros_like(out)
        ops.attn_prefill_t5(packed, kc, vc, bt, torch.tensor([0, 1], dtype=torch.int32, device=DEV), 0 * one,
                            pos * one, 1, 1, H, KV, hd, 1.0, window, out3)
        assert ops.attn_prefill_t5_status() == 0
        torch.testing.assert_close(out3.double(), ref, rtol=2e-2, atol=2e-2 * float(ref.abs().max()))
        return
    if decode:
        po, pml = torch.zeros(H * 4 * hd, device=DEV), torch.zeros(H * 4 * 2, device=DEV)
        ops.attn_decode_generic(q[:, 0], kc, vc, bt, 0 * one, n * one, 1, H, KV, hd, 1.0, window, 4, out, po, pml)
    else:
        # the last position as a one-token chunk after n - 1 cached ones
        ops.attn_prefill_generic(q[:, 0], kc, vc, bt, torch.tensor([0, 1], dtype=torch.int32, device=DEV), 0 * one,
                                 pos * one, 1, 1, H, KV, hd, 1.0, window, out)
    torch.testing.assert_close(out.double(), ref, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("kernel,hd", [("generic", 32), ("mma", 64), ("tcgen05", 64), ("tcgen05", 128)])
@pytest.mark.parametrize("window", [None, 37, 64, 100])
@pytest.mark.parametrize("edge", ["newest", "oldest"])
def test_prompt_attention_edges_at_every_row(kernel, hd, window, edge):
    """Every row of a prompt is made to look at exactly one key: its own position (scores that grow with the key's
    position) or the oldest position it may see (scores that fall): the start, or the window's far edge.  The value
    of position j holds j, so the output names the key each row really used; one position off anywhere (a tile's
    border, a block's border, the window's edge) shows as a wrong number."""
    if edge == "oldest" and window is None:
        window_eff, first = None, lambda i: 0
    else:
        window_eff, first = window, (lambda i: max(0, i - window + 1)) if window else (lambda i: 0)
    H, KV, n, gap = 2, 1, 250, 10.0
    dtype = torch.float32 if kernel == "generic" else torch.bfloat16
    k = torch.zeros(1, n, KV, hd, dtype=dtype, device=DEV)
    v = torch.zeros(1, n, KV, hd, dtype=dtype, device=DEV)
    j = torch.arange(n, device=DEV, dtype=torch.float32)
    k[0, :, 0, 0] = (j if edge == "newest" else -j).to(dtype)          # whole numbers up to 256: exact in bfloat16
    v[0, :, 0, 0] = j.to(dtype)
    v[0, :, 0, 1] = 1.0
    packed = torch.zeros(n, (H + 2 * KV) * hd, dtype=dtype, device=DEV)
    packed[:, 0] = gap                                                   # both heads ask the same
    packed[:, hd] = gap
    kc, vc, bt = paged_from_dense(k, v, [n], seed=6)
    cu = torch.tensor([0, n], dtype=torch.int32, device=DEV)
    zero = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.full((n, H * hd), float("nan"), dtype=dtype, device=DEV)
    if kernel == "generic":
        ops.attn_prefill_generic(packed, kc, vc, bt, cu, zero, zero, 1, n, H, KV, hd, 1.0, window_eff, out)
    elif kernel == "mma":
        ops.attn_prefill_tc(packed, kc, vc, bt, cu, zero, zero, 1, n, H, KV, hd, 1.0, window_eff, out)
    else:
        ops.attn_prefill_t5(packed, kc, vc, bt, cu, zero, zero, 1, n, H, KV, hd, 1.0, window_eff, out)
        assert ops.attn_prefill_t5_status() == 0
    want = torch.tensor([float(i if edge == "newest" else first(i)) for i in range(n)], device=DEV, dtype=torch.float64)
    for h in range(H):
        got = out[:, h * hd].double()
        # the next key weighs e^-10 of the chosen one, and positions are whole numbers: half a position is a fault
        assert float((got - want).abs().max()) < 0.3, (h, int((got - want).abs().argmax()), got[:8], want[:8])
        torch.testing.assert_close(out[:, h * hd + 1].double(), torch.ones(n, device=DEV, dtype=torch.float64), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("kernel,hd", [("generic", 32), ("mma", 64), ("mma", 128), ("keys", 64), ("keys", 128)])
@pytest.mark.parametrize("window,splits", [(None, 1), (None, 3), (37, 1), (64, 4), (100, 2)])
@pytest.mark.parametrize("edge", ["newest", "oldest"])
def test_decode_attention_edges_at_every_length(kernel, hd, window, splits, edge):
    """The same for one-token steps: sequences of many lengths around the tiles' and pages' borders, each made to
    look at its newest position or at the oldest it may see."""
    lens = list(range(1, 36)) + [47, 48, 49, 63, 64, 65, 66, 100, 101, 127, 128, 129, 130, 191, 192, 193, 250]
    B, S, H, KV, gap = len(lens), 256, 2, 1, 10.0
    dtype = torch.float32 if kernel == "generic" else torch.bfloat16
    k = torch.zeros(B, S, KV, hd, dtype=dtype, device=DEV)
    v = torch.zeros(B, S, KV, hd, dtype=dtype, device=DEV)
    j = torch.arange(S, device=DEV, dtype=torch.float32)
    k[:, :, 0, 0] = (j if edge == "newest" else -j).to(dtype)
    v[:, :, 0, 0] = j.to(dtype)
    q = torch.zeros(B, H * hd, dtype=dtype, device=DEV)
    q[:, 0] = gap
    q[:, hd] = gap
    kc, vc, bt = paged_from_dense(k, v, lens, seed=8)
    out = torch.full((B, H * hd), float("nan"), dtype=dtype, device=DEV)
    po = torch.full((B * H * splits * hd,), float("nan"), device=DEV)
    pml = torch.full((B * H * splits * 2,), float("nan"), device=DEV)
    slots = torch.arange(B, dtype=torch.int32, device=DEV)
    dev_lens = torch.tensor(lens, dtype=torch.int32, device=DEV)
    fn = ops.attn_decode_generic if kernel == "generic" else ops.attn_decode_tc
    with (keys_on_rows() if kernel == "keys" else heads_on_rows()):
        fn(q, kc, vc, bt, slots, dev_lens, B, H, KV, hd, 1.0, window, splits, out, po, pml)
    want = torch.tensor([float(n - 1 if edge == "newest" else (max(0, n - window) if window else 0)) for n in lens],
                        device=DEV, dtype=torch.float64)
    for h in range(H):
        got = out[:, h * hd].double()
        assert float((got - want).abs().max()) < 0.3, (h, lens[int((got - want).abs().argmax())], got, want)


def test_argmax_first_on_ties_and_nan():
    logits = torch.zeros(4, 1000, device=DEV)
    logits[0, 17] = 3.0
    logits[0, 800] = 3.0                 # the first of the highest wins (src/sampler.rs:136-142)
    logits[1, 999] = 1.0
    logits[2, :] = -5.0
    logits[2, 500] = float("nan")        # NaN never wins (src/cuda.rs:3540-3570)
    logits[2, 501] = -4.0
    logits[3, :] = float("-inf")
    out = ops.sample(logits, 0.0, 0, 1.0).cpu().tolist()
    assert out == [17, 999, 501, 0]


@pytest.mark.parametrize("vocab", [301, 5000, 128256])
@pytest.mark.parametrize("temp,top_k,top_p", [(0.8, 0, 1.0), (0.7, 40, 0.9), (1.5, 0, 0.9), (0.3, 5, 1.0), (1.0, 1000, 0.5), (2.0, 3, 0.2)])
def test_sampler_matches_the_plain_sampler(vocab, temp, top_k, top_p):
    """Same logits, same generator stream: the device picks what the plain walk over the sorted list picks.
    Several draws per row advance the state as the plain generator does."""
    rows = 6
    g = torch.Generator().manual_seed(vocab)
    logits = (torch.randn(rows, vocab, generator=g) * 2.0)
    logits[1, :50] = logits[1, 0]                       # ties, ordered by token id
    logits[2] = torch.round(logits[2])                  # many ties
    logits[3, 7 % vocab] = 1e30                         # one logit far above all others (nothing else near its key)
    logits[4] = -logits[4].abs() - 5.0                  # negative only
    dev = logits.to(DEV)
    seeds = [1, 2, 3, 99, 2 ** 40 + 7, 12345]
    state = torch.tensor(seeds, dtype=torch.int64, device=DEV)
    gens = [pl.XorShift64Star(s) for s in seeds]
    for draw in range(3):
        got = ops.sample(dev, temp, top_k, top_p, state).cpu().tolist()
        for r in range(rows):
            want = pl.sample(logits[r].numpy(), temp, top_k, top_p, gens[r])
            assert got[r] == want, f"row {r} draw {draw}: device {got[r]}, plain {want}"
    assert [int(s) & (2 ** 64 - 1) for s in state.cpu().tolist()] == [g_.s for g_ in gens]


def test_sampler_frequencies_and_state_index():
    logits = torch.tensor([[0.0, 1.0, 2.0, 0.5, -1.0]] * 512, device=DEV)
    state = torch.arange(1, 1025, dtype=torch.int64, device=DEV)
    idx = torch.arange(512, 1024, dtype=torch.int32, device=DEV)      # rows use states 512..1023
    counts = np.zeros(5)
    for _ in range(40):
        got = ops.sample(logits, 0.8, 0, 1.0, state, idx).cpu().numpy()
        counts += np.bincount(got, minlength=5)
    assert torch.equal(state[:512].cpu(), torch.arange(1, 513, dtype=torch.int64))   # the other states are untouched
    p = np.exp(np.array([0.0, 1.0, 2.0, 0.5, -1.0]) / 0.8)
    p /= p.sum()
    assert np.abs(counts / counts.sum() - p).max() < 0.012


def test_kernels_refuse_what_they_cannot_do():
    from ghost_infer_b200.kernels import KernelError
    with pytest.raises(KernelError):
        ops.rmsnorm(torch.zeros(2, 8), torch.ones(8), 1e-5, torch.float32)          # no CPU path
    with pytest.raises(KernelError):
        ops.gemm_generic(rnd(2, 8), rnd(3, 9))                                       # widths that do not meet
    with pytest.raises(KernelError):
        ops.gemm_generic(rnd(2, 8).half(), rnd(3, 8).half())                         # a dtype nobody wrote
    H, KV, hd = 2, 1, 272
    q = rnd(1, H * hd)
    kc = torch.zeros(2, KV, 64, hd, device=DEV)
    one = torch.ones(1, dtype=torch.int32, device=DEV)
    with pytest.raises(KernelError) as e:
        ops.attn_decode_generic(q, kc, kc, one.reshape(1, 1), 0 * one, one, 1, H, KV, hd, 1.0, None, 1, torch.zeros_like(q))
    assert "272" in str(e.value)


@pytest.mark.parametrize("m", [1, 3, 8, 9, 16, 17, 40, 64])
@pytest.mark.parametrize("n,k", [(100, 72), (96, 4096), (33, 264), (6144, 512)])
def test_gemm_skinny(m, n, k):
    """The decode product: few rows of activations, W rows that are no multiple of the block's 32, a K that is
    a multiple of 8 but not of 32; store, float store and accumulation."""
    a, w = rnd(m, k, dtype=torch.bfloat16, seed=20), rnd(n, k, dtype=torch.bfloat16, seed=21)
    assert ops.skinny_ok(a, w)
    ref = a.double() @ w.double().T
    terms = a.double().abs() @ w.double().abs().T
    out = ops.gemm_skinny(a, w, ops.SKINNY_STORE_F32)
    assert ((out.double() - ref).abs() <= 2e-6 * terms + 1e-7).all()
    out16 = ops.gemm_skinny(a, w, ops.SKINNY_STORE_BF16)
    assert ((out16.double() - ref).abs() <= 2 ** -8 * ref.abs() + 2e-6 * terms + 1e-7).all()
    acc = rnd(m, n, seed=22)
    before = acc.clone()
    ops.gemm_skinny(a, w, ops.SKINNY_ACCUM_F32, acc)
    assert ((acc.double() - (before.double() + ref)).abs() <= 2e-6 * (terms + before.abs().double()) + 1e-6).all()
    # a row gives the same bits alone and inside a batch (fixed summation order, src/cuda.rs:748-766)
    alone = ops.gemm_skinny(a[m - 1:m].contiguous(), w, ops.SKINNY_STORE_F32)
    assert torch.equal(alone[0], out[m - 1])


@pytest.mark.parametrize("m", [1, 8, 13, 64])
@pytest.mark.parametrize("f,k", [(176, 64), (24, 4096), (14336 // 8, 128)])
def test_gemm_skinny_swiglu(m, f, k):
    a = rnd(m, k, dtype=torch.bfloat16, seed=23)
    g, u = rnd(f, k, dtype=torch.bfloat16, seed=24, scale=0.3), rnd(f, k, dtype=torch.bfloat16, seed=25, scale=0.3)
    w = torch.stack([g.view(f // 8, 8, k), u.view(f // 8, 8, k)], dim=1).reshape(2 * f, k).contiguous()
    gd, ud = a.double() @ g.double().T, a.double() @ u.double().T
    ref = gd / (1 + torch.exp(-gd)) * ud
    out = ops.swiglu_interleaved(a, w)
    assert out.shape == (m, f) and out.dtype == torch.bfloat16
    torch.testing.assert_close(out.double(), ref, rtol=1e-2, atol=1e-3 * float(ref.abs().max()))
    # more rows than the decode kernel takes: the product, then the interleaved elementwise kernel
    big = rnd(70, k, dtype=torch.bfloat16, seed=26)
    gd, ud = big.double() @ g.double().T, big.double() @ u.double().T
    torch.testing.assert_close(ops.swiglu_interleaved(big, w).double(), gd / (1 + torch.exp(-gd)) * ud, rtol=2e-2,
                               atol=1e-2 * float((gd * ud).abs().max()))


@pytest.mark.parametrize("tile_n", [128, 256])
@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (130, 96, 72), (65, 264, 200), (700, 512, 4096), (2048, 1000, 512)])
def test_gemm_tensor_cores(tile_n, m, n, k):
    """The tcgen05 / TMA product: whole tiles, and rows, columns and K that stop inside a tile (zero-filled by
    TMA, masked at the store); store in both precisions and accumulation into a float matrix."""
    a, w = rnd(m, k, dtype=torch.bfloat16, seed=30), rnd(n, k, dtype=torch.bfloat16, seed=31)
    assert ops.tc_ok(a, w)
    ref = a.double() @ w.double().T
    terms = a.double().abs() @ w.double().abs().T
    out = ops.gemm_tc(a, w, ops.SKINNY_STORE_F32, tile_n=tile_n)
    assert ops.gemm_tc_status() == 0
    assert ((out.double() - ref).abs() <= 2e-6 * terms + 1e-7).all(), float((out.double() - ref).abs().max())
    out16 = ops.gemm_tc(a, w, ops.SKINNY_STORE_BF16, tile_n=tile_n)
    assert ((out16.double() - ref).abs() <= 2 ** -8 * ref.abs() + 2e-6 * terms + 1e-7).all()
    acc = rnd(m, n, seed=32)
    before = acc.clone()
    ops.gemm_tc(a, w, ops.SKINNY_ACCUM_F32, acc, tile_n=tile_n)
    assert ((acc.double() - (before.double() + ref)).abs() <= 2e-6 * (terms + before.abs().double()) + 1e-6).all()
    assert ops.gemm_tc_status() == 0


@pytest.mark.parametrize("tile_n", [128, 256])
@pytest.mark.parametrize("m,f,k", [(200, 176, 64), (129, 1000, 520)])
def test_gemm_tensor_cores_swiglu(tile_n, m, f, k):
    a = rnd(m, k, dtype=torch.bfloat16, seed=33)
    g, u = rnd(f, k, dtype=torch.bfloat16, seed=34, scale=0.3), rnd(f, k, dtype=torch.bfloat16, seed=35, scale=0.3)
    w = torch.stack([g.view(f // 8, 8, k), u.view(f // 8, 8, k)], dim=1).reshape(2 * f, k).contiguous()
    gd, ud = a.double() @ g.double().T, a.double() @ u.double().T
    ref = gd / (1 + torch.exp(-gd)) * ud
    out = ops.gemm_tc(a, w, ops.SKINNY_SWIGLU, tile_n=tile_n)
    assert ops.gemm_tc_status() == 0
    torch.testing.assert_close(out.double(), ref, rtol=1e-2, atol=1e-3 * float(ref.abs().max()))


@pytest.mark.parametrize("pdl", [False, True])
@pytest.mark.parametrize("m", [1, 8, 13, 16, 17, 32, 50, 64])
@pytest.mark.parametrize("n,k", [(100, 72), (128, 64), (6144, 4096), (4096, 14336), (1000, 520), (40000, 264), (19100, 200)])
def test_gemm_stream(pdl, m, n, k):
    """The persistent stream-K decode product: tiles cut between blocks (summed by whoever arrives last, in
    K order), rows of W that stop inside a tile, K that stops inside a block, every token-tile width."""
    a, w = rnd(m, k, dtype=torch.bfloat16, seed=40), rnd(n, k, dtype=torch.bfloat16, seed=41)
    ref = a.double() @ w.double().T
    terms = a.double().abs() @ w.double().abs().T
    out = ops.gemm_stream(a, w, ops.SKINNY_STORE_F32, pdl=pdl)
    assert ops.gemm_stream_status() == 0
    assert ((out.double() - ref).abs() <= 2e-6 * terms + 1e-7).all(), float((out.double() - ref).abs().max())
    again = ops.gemm_stream(a, w, ops.SKINNY_STORE_F32, pdl=pdl)
    assert torch.equal(out, again)                    # the same bits whoever arrived last
    out16 = ops.gemm_stream(a, w, ops.SKINNY_STORE_BF16, pdl=pdl)
    assert ((out16.double() - ref).abs() <= 2 ** -8 * ref.abs() + 2e-6 * terms + 1e-7).all()
    acc = rnd(m, n, seed=42)
    before = acc.clone()
    ops.gemm_stream(a, w, ops.SKINNY_ACCUM_F32, acc, pdl=pdl)
    assert ((acc.double() - (before.double() + ref)).abs() <= 2e-6 * (terms + before.abs().double()) + 1e-6).all()
    assert ops.gemm_stream_status() == 0


@pytest.mark.parametrize("mode", ["store", "f32", "swiglu"])
@pytest.mark.parametrize("m,tiles,k", [(8, 120, 264), (64, 147, 512), (20, 119, 72), (5, 118, 264)])
def test_gemm_stream_one_block_per_tile(mode, m, tiles, k):
    """A product that finishes its own sums and has a few tiles fewer than there are SMs runs one block per tile (no
    tile is cut between blocks): 119 tiles and more on 148 SMs.  Against the 64-bit product, with the rule on and
    off, and with a last tile that is not full."""
    n = tiles * 128 - (0 if mode == "swiglu" else 40)
    a, w = rnd(m, k, dtype=torch.bfloat16, seed=80), rnd(n, k, dtype=torch.bfloat16, seed=81, scale=0.1)
    ref = a.double() @ w.double().T
    code = {"store": ops.SKINNY_STORE_BF16, "f32": ops.SKINNY_STORE_F32, "swiglu": ops.SKINNY_SWIGLU}[mode]
    if mode == "swiglu":
        r = ref.view(m, n // 16, 2, 8)
        ref = (torch.nn.functional.silu(r[:, :, 0]) * r[:, :, 1]).reshape(m, n // 2)
    was = ops.TUNE["stream_whole_percent"]
    try:
        for percent in (80, 0, 80):
            ops.TUNE["stream_whole_percent"] = percent
            out = ops.gemm_stream(a, w, code)
            torch.testing.assert_close(out.double(), ref, **tol(torch.float32 if mode == "f32" else torch.bfloat16))
    finally:
        ops.TUNE["stream_whole_percent"] = was
        ops.gemm_stream(a[:1], w[:128], ops.SKINNY_STORE_BF16)      # tells the library the old value again
    assert ops.gemm_stream_status() == 0


def test_gemm_stream_time_stamps():
    """With a buffer given, every block of a streamed product notes the clock along its life, in order; without
    one, nothing is written."""
    a, w = rnd(8, 4096, dtype=torch.bfloat16, seed=40), rnd(6144, 4096, dtype=torch.bfloat16, seed=41)
    ops.stream_timeline_start(4)
    ops.gemm_stream(a, w, ops.SKINNY_STORE_F32)
    ops.gemm_stream(a, w, ops.SKINNY_STORE_F32)
    stamps, n = ops.stream_timeline_stop()
    assert n == 2 and stamps.shape == (4, 256, 8)
    assert (stamps[2:] == 0).all()
    for launch in stamps[:2]:
        blocks = launch[launch[:, 0] > 0]
        assert 1 <= len(blocks) <= 256
        for a_ev, b_ev in ((0, 1), (1, 3), (3, 4), (4, 6), (5, 6), (6, 7)):
            assert (blocks[:, a_ev] <= blocks[:, b_ev]).all(), (a_ev, b_ev)
    assert stamps[1, :, 0].max() >= stamps[0, :, 7][stamps[0, :, 7] > 0].min()     # the second launch came later
    out = ops.gemm_stream(a, w, ops.SKINNY_STORE_F32)                               # switched off again: results as ever
    assert ops.gemm_stream_status() == 0
    terms = a.double().abs() @ w.double().abs().T
    assert ((out.double() - a.double() @ w.double().T).abs() <= 2e-6 * terms + 1e-7).all()


@pytest.mark.parametrize("m", [1, 8, 20, 64])
@pytest.mark.parametrize("f,k", [(176, 64), (1000, 4096), (14336, 512)])
def test_gemm_stream_swiglu(m, f, k):
    a = rnd(m, k, dtype=torch.bfloat16, seed=43)
    g, u = rnd(f, k, dtype=torch.bfloat16, seed=44, scale=0.3), rnd(f, k, dtype=torch.bfloat16, seed=45, scale=0.3)
    w = torch.stack([g.view(f // 8, 8, k), u.view(f // 8, 8, k)], dim=1).reshape(2 * f, k).contiguous()
    gd, ud = a.double() @ g.double().T, a.double() @ u.double().T
    ref = gd / (1 + torch.exp(-gd)) * ud
    out = ops.gemm_stream(a, w, ops.SKINNY_SWIGLU)
    assert ops.gemm_stream_status() == 0
    assert out.shape == (m, f)
    torch.testing.assert_close(out.double(), ref, rtol=1e-2, atol=1e-3 * float(ref.abs().max()))


@pytest.mark.parametrize("m", [1, 8, 16, 40])
@pytest.mark.parametrize("n,k", [(4096, 4096), (4096, 14336), (512, 264), (2048, 128)])
def test_deferred_accumulation_is_settled_by_the_norm(m, n, k):
    """A decode product that adds into the residual stream may leave the partial sums of tiles cut between blocks
    in scratch; the norm that reads the stream next adds them (and writes the settled rows back)."""
    a, w = rnd(m, k, dtype=torch.bfloat16, seed=50), rnd(n, k, dtype=torch.bfloat16, seed=51, scale=0.05)
    wn = (1 + 0.1 * rnd(n, seed=52)).to(torch.bfloat16)
    x0 = rnd(m, n, seed=53)
    want_x = x0.double() + a.double() @ w.double().T
    want_h = want_x * torch.rsqrt((want_x ** 2).mean(-1, keepdim=True) + 1e-5) * wn.double()
    # through the norm
    x = ops.as_carrier(x0.clone())
    with ops.defer_into(x):
        ops.linear(a, w, out=x, accumulate=True)
    assert ops.has_pending(x)
    h = ops.rmsnorm(x, wn, 1e-5, torch.bfloat16)
    assert not ops.has_pending(x)
    torch.testing.assert_close(x.double(), want_x, rtol=1e-5, atol=1e-4)
    torch.testing.assert_close(h.double(), want_h, rtol=1.6e-2, atol=1.6e-2)
    # selected rows only (the final norm): those rows are settled
    x = ops.as_carrier(x0.clone())
    with ops.defer_into(x):
        ops.linear(a, w, out=x, accumulate=True)
    rows = torch.tensor([m - 1, 0], dtype=torch.int32, device=DEV)
    h = ops.rmsnorm(x, wn, 1e-5, torch.float32, rows=rows)
    torch.testing.assert_close(h.double(), want_h[rows.long()], rtol=1e-4, atol=1e-4)
    # settled on its own, and twice the same bits
    outs = []
    for _ in range(2):
        x = ops.as_carrier(x0.clone())
        with ops.defer_into(x):
            ops.linear(a, w, out=x, accumulate=True)
        ops.settle(x)
        outs.append(x.clone())
    torch.testing.assert_close(outs[0].double(), want_x, rtol=1e-5, atol=1e-4)
    assert torch.equal(outs[0], outs[1])
    # outside a deferring context nothing is left pending
    x = ops.as_carrier(x0.clone())
    ops.linear(a, w, out=x, accumulate=True)
    assert not ops.has_pending(x)
    torch.testing.assert_close(x.double(), want_x, rtol=1e-5, atol=1e-4)
    # a second accumulation while one is pending settles the first before it adds
    x = ops.as_carrier(x0.clone())
    with ops.defer_into(x):
        ops.linear(a, w, out=x, accumulate=True)
        ops.linear(a, w, out=x, accumulate=True)
    ops.settle(x)
    torch.testing.assert_close(x.double(), x0.double() + 2 * (a.double() @ w.double().T), rtol=1e-5, atol=2e-4)
    # what is pending travels with the tensor: a plain tensor is never deferred into ...
    plain = x0.clone()
    with ops.defer_into(plain):
        ops.linear(a, w, out=plain, accumulate=True)
    assert not ops.has_pending(plain)
    torch.testing.assert_close(plain.double(), want_x, rtol=1e-5, atol=1e-4)
    # ... any torch operation on a carrier settles first (a reader that forgets cannot see rows without their sums) ...
    x = ops.as_carrier(x0.clone())
    with ops.defer_into(x):
        ops.linear(a, w, out=x, accumulate=True)
    pending_before = ops.has_pending(x)
    got = x[:, :7] + 0.0
    assert not ops.has_pending(x)
    torch.testing.assert_close(got.double(), want_x[:, :7], rtol=1e-5, atol=1e-4)
    # ... and a kernel that does not settle refuses a tensor with sums pending instead of reading it
    x = ops.as_carrier(x0.clone())
    with ops.defer_into(x):
        ops.linear(a, w, out=x, accumulate=True)
    if ops.has_pending(x):
        assert pending_before
        with pytest.raises(KernelError, match="pending"):
            ops.gemm_generic(x, torch.zeros(8, n, device=DEV))
        ops.drop_pending(x)


@pytest.mark.parametrize("m", [1, 8, 20])
@pytest.mark.parametrize("H,KV,hd,rot", [(32, 8, 128, 128), (6, 2, 64, 32), (5, 1, 48, 48)])
def test_deferred_store_is_settled_by_the_rotary_kernel(m, H, KV, hd, rot):
    """The q/k/v product of a decode step may leave partial sums instead of values; the kernel that rotates and
    writes the cache adds them.  Bit for bit what the plain store followed by the same kernel gives."""
    d = 264
    n = (H + 2 * KV) * hd
    a, w = rnd(m, d, dtype=torch.bfloat16, seed=60), rnd(n, d, dtype=torch.bfloat16, seed=61, scale=0.1)
    positions = torch.arange(5, 5 + m, dtype=torch.int32, device=DEV)
    slots = torch.zeros(m, dtype=torch.int32, device=DEV)
    bt = torch.tensor([[2, 1]], dtype=torch.int32, device=DEV)
    inv = torch.from_numpy(pl.rotary_inv_freq(rot, 10000.0, None)).to(DEV)
    table = ops.rope_table(positions, inv)
    outs = []
    for defer in (False, True):
        kc = torch.zeros(3, KV, 64, hd, dtype=torch.bfloat16, device=DEV)
        vc = torch.zeros_like(kc)
        if defer:
            with ops.defer_store():
                qkv = ops.linear(a, w, out_dtype=torch.bfloat16)
            assert ops.has_pending(qkv)
        else:
            qkv = ops.linear(a, w, out_dtype=torch.bfloat16)
            assert not ops.has_pending(qkv)
        ops.rope_cache_write(qkv, table, positions, slots, bt, kc, vc, H, KV, hd, rot, False, True)
        assert not ops.has_pending(qkv)
        outs.append((qkv[:, :H * hd].clone(), kc, vc))
    for x, y in zip(outs[0], outs[1]):
        assert torch.equal(x, y)
    ref_v = (a.double() @ w.double().T)[:, (H + KV) * hd:]
    got_v = outs[1][2][2, :, 5:5 + m].transpose(0, 1).reshape(m, KV * hd).double()
    torch.testing.assert_close(got_v, ref_v, rtol=1.6e-2, atol=1.6e-2)


@pytest.mark.parametrize("hd", [128, 64])
@pytest.mark.parametrize("H,KV", [(4, 2), (32, 8), (3, 1)])
@pytest.mark.parametrize("window", [None, 37, 100])
@pytest.mark.parametrize("pairing", [0, 2])
def test_attention_prefill_tcgen05(H, KV, window, hd, pairing, request):
    """The tcgen05 prefill kernel (head sizes 128 and 64): ragged lengths around its 128-row and 64-key tiles,
    sequences that go on after cached positions, pages in shuffled order, unowned rows poisoned with NaN.  With one
    query tile per block and with two (the block's barriers are made anew between them)."""
    ops.attn_prefill_t5_pairing(pairing)
    request.addfinalizer(lambda: ops.attn_prefill_t5_pairing(1))
    lens_q, pos0 = [1, 45, 128, 129, 300, 33, 130, 520], [0, 0, 0, 0, 0, 70, 200, 10]
    B, S = len(lens_q), 576
    k = rnd(B, S, KV, hd, dtype=torch.bfloat16, seed=10)
    v = rnd(B, S, KV, hd, dtype=torch.bfloat16, seed=11)
    q = rnd(B, max(lens_q), (H + 2 * KV) * hd, dtype=torch.bfloat16, seed=12)
    lens_kv = [p + n for p, n in zip(pos0, lens_q)]
    kc, vc, bt = paged_from_dense(k, v, lens_kv, seed=3)
    flat = torch.cat([q[b, :lens_q[b]] for b in range(B)])
    cu = torch.tensor([0] + list(np.cumsum(lens_q)), dtype=torch.int32, device=DEV)
    slots = torch.arange(B, dtype=torch.int32, device=DEV)
    ref = attention_ref(q[:, :, :H * hd], k, v, lens_q, pos0, H, KV, hd, 0.21, window)
    ref = torch.cat([ref[b, :lens_q[b]] for b in range(B)])
    pos0_t = torch.tensor(pos0, dtype=torch.int32, device=DEV)
    # Many launches of the same case: what goes wrong in this kernel goes wrong by timing (a warp of a block that falls
    # behind the others), most easily where a block has few key tiles (a window), and then in one launch of dozens.
    for _ in range(16 if window else 4):
        out = torch.full((flat.shape[0], H * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops.attn_prefill_t5(flat, kc, vc, bt, cu, slots, pos0_t, B, max(lens_q), H, KV, hd, 0.21, window, out)
        assert ops.attn_prefill_t5_status() == 0
        torch.testing.assert_close(out.double(), ref, **tol(torch.bfloat16))


def test_prefill_kernels_chain_under_dependent_launch():
    """Norm, product, rotary + cache write, tcgen05 attention and an accumulating product in a row, with and without
    programmatic dependent launch: each kernel may start while its predecessor drains, the bits must not move."""
    H, KV, hd, d, T = 4, 2, 128, 256, 300
    x0 = rnd(T, d, seed=70)
    wn = (1 + 0.1 * rnd(d, seed=71)).to(torch.bfloat16)
    wqkv = rnd((H + 2 * KV) * hd, d, dtype=torch.bfloat16, seed=72, scale=0.1)
    wo = rnd(d, H * hd, dtype=torch.bfloat16, seed=73, scale=0.1)
    positions = torch.arange(T, dtype=torch.int32, device=DEV)
    slots = torch.zeros(T, dtype=torch.int32, device=DEV)
    bt = torch.arange(1, 6, dtype=torch.int32, device=DEV).reshape(1, 5)
    inv = torch.from_numpy(pl.rotary_inv_freq(hd, 10000.0, None)).to(DEV)
    cu = torch.tensor([0, T], dtype=torch.int32, device=DEV)
    zero = torch.zeros(1, dtype=torch.int32, device=DEV)
    outs = []
    was = ops.get_pdl()
    for pdl in (False, True, True):
        ops.set_pdl(pdl)
        try:
            x = x0.clone()
            kc = torch.zeros(6, KV, 64, hd, dtype=torch.bfloat16, device=DEV)
            vc = torch.zeros_like(kc)
            h = ops.rmsnorm(x, wn, 1e-5, torch.bfloat16)
            qkv = ops.linear(h, wqkv, out_dtype=torch.bfloat16)
            table = ops.rope_table(positions, inv)
            ops.rope_cache_write(qkv, table, positions, slots, bt, kc, vc, H, KV, hd, hd, False, True)
            att = torch.empty(T, H * hd, dtype=torch.bfloat16, device=DEV)
            ops.attn_prefill_t5(qkv, kc, vc, bt, cu, zero, zero, 1, T, H, KV, hd, hd ** -0.5, None, att)
            ops.linear(att, wo, out=x, accumulate=True)
            torch.cuda.synchronize()
            outs.append(x.clone())
        finally:
            ops.set_pdl(was)
    assert ops.gemm_tc_status() == 0 and ops.attn_prefill_t5_status() == 0
    assert torch.isfinite(outs[0]).all() and float((outs[0] - x0).abs().max()) > 0
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[1], outs[2])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hd,rot", [(16, 16), (128, 128), (64, 32), (48, 32)])
def test_rope_and_cache_write_for_a_prompt(dtype, hd, rot):
    """Many tokens at once take the kernel with 16-byte accesses (when the sizes allow it): the same numbers as the
    plain formula, two sequences in different slots, positions that cross pages."""
    H, KV, T = 5, 2, 90
    qkv = rnd(T, (H + 2 * KV) * hd, dtype=dtype, seed=80)
    orig = qkv.clone()
    positions = torch.cat([torch.arange(60, 110), torch.arange(0, 40)]).to(torch.int32).to(DEV)
    slots = torch.cat([torch.zeros(50), torch.ones(40)]).to(torch.int32).to(DEV)
    bt = torch.tensor([[3, 1], [2, 4]], dtype=torch.int32, device=DEV)
    kc = torch.zeros(5, KV, 64, hd, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    inv = torch.from_numpy(pl.rotary_inv_freq(rot, 500000.0, None)).to(DEV)
    table = ops.rope_table(positions, inv)
    ops.rope_cache_write(qkv, table, positions, slots, bt, kc, vc, H, KV, hd, rot, False, True)
    o = orig.double().cpu().numpy()
    pos = positions.cpu().numpy()

    def rot_ref(x, heads):
        x = x.reshape(T, heads, hd)
        y = x.copy()
        y[:, :, :rot] = pl.rope(x[:, :, :rot].reshape(T, heads * rot), pos, inv.cpu().numpy(), rot, "half").reshape(T, heads, rot)
        return y.reshape(T, heads * hd)

    q_ref, k_ref, v_ref = rot_ref(o[:, :H * hd], H), rot_ref(o[:, H * hd:(H + KV) * hd], KV), o[:, (H + KV) * hd:]
    t = tol(dtype)
    np.testing.assert_allclose(qkv[:, :H * hd].double().cpu().numpy(), q_ref, rtol=t["rtol"], atol=t["atol"])
    assert torch.equal(qkv[:, H * hd:], orig[:, H * hd:])
    for i in range(T):
        page = int(bt[int(slots[i]), int(pos[i]) // 64])
        np.testing.assert_allclose(kc[page, :, int(pos[i]) % 64].double().cpu().numpy().reshape(-1), k_ref[i], rtol=t["rtol"], atol=t["atol"])
        np.testing.assert_array_equal(vc[page, :, int(pos[i]) % 64].double().cpu().numpy().reshape(-1), v_ref[i])
    assert float(kc[0].abs().sum()) == 0


@pytest.mark.parametrize("H,KV,hd,rot", [(32, 8, 128, 128), (6, 2, 64, 32), (5, 1, 64, 64), (40, 2, 128, 64), (8, 8, 128, 128)])
@pytest.mark.parametrize("window,splits", [(None, 1), (None, 5), (100, 3)])
@pytest.mark.parametrize("defer", [False, True])
def test_decode_attention_rotates_and_stores_by_itself(H, KV, hd, rot, window, splits, defer):
    """The decode attention given the rows as the q/k/v product left them (with partial sums pending or not) and the
    table of angles, against the rotary kernel followed by the attention: the same bits in the output and in every
    byte of the cache.  The cache rows of the newest positions hold NaN beforehand, so a block that reads its last tile
    before the key and value are stored shows; lengths of 1, at page and tile edges, and long ones; a group of 20 heads
    (two blocks per kv head, both of which store); a rotated part smaller than the head."""
    lens = [1, 31, 64, 65, 700, 333, 96, 129, 16, 17]
    B, S, d = len(lens), 704, 264
    k = rnd(B, S, KV, hd, dtype=torch.bfloat16, seed=13)
    v = rnd(B, S, KV, hd, dtype=torch.bfloat16, seed=14)
    a, w = rnd(B, d, dtype=torch.bfloat16, seed=60), rnd((H + 2 * KV) * hd, d, dtype=torch.bfloat16, seed=61, scale=0.1)
    slots, lens_t = torch.arange(B, dtype=torch.int32, device=DEV), torch.tensor(lens, dtype=torch.int32, device=DEV)
    pos = lens_t - 1
    table = ops.rope_table(pos, torch.from_numpy(pl.rotary_inv_freq(rot, 10000.0, None)).to(DEV))
    results = []
    for inside in (False, True, True):
        kc, vc, bt = paged_from_dense(k, v, lens, seed=4)
        for b, n in enumerate(lens):
            page, off = int(bt[b, (n - 1) // 64]), (n - 1) % 64
            kc[page, :, off] = float("nan")
            vc[page, :, off] = float("nan")
        if defer:
            with ops.defer_store():
                qkv = ops.linear(a, w, out_dtype=torch.bfloat16)
            assert ops.has_pending(qkv)
        else:
            qkv = ops.linear(a, w, out_dtype=torch.bfloat16)
        out = torch.full((B, H * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
        part_o = torch.full((B * H * splits * hd,), float("nan"), device=DEV)
        part_ml = torch.full((B * H * splits * 2,), float("nan"), device=DEV)
        if not inside:
            ops.rope_cache_write(qkv, table, pos, slots, bt, kc, vc, H, KV, hd, rot, False, True)
        with heads_on_rows():       # the same kernel in both arms
            ops.attn_decode_tc(qkv, kc, vc, bt, slots, lens_t, B, H, KV, hd, 0.17, window, splits, out, part_o, part_ml,
                               rope=(table, rot) if inside else None)
        assert not ops.has_pending(qkv)
        assert not bool(torch.isnan(out.float()).any())
        results.append((out, kc, vc))
    for out, kc, vc in results[1:]:
        assert torch.equal(out, results[0][0])
        # NaN poison fills the same unused rows in every run: compare the bits
        assert torch.equal(kc.view(torch.int16), results[0][1].view(torch.int16))
        assert torch.equal(vc.view(torch.int16), results[0][2].view(torch.int16))
    # and the stored value is the product's
    ref_v = (a.double() @ w.double().T)[:, (H + KV) * hd:]
    got = torch.stack([results[1][2][int(bt[b, (n - 1) // 64]), :, (n - 1) % 64].reshape(KV * hd) for b, n in enumerate(lens)])
    torch.testing.assert_close(got.double(), ref_v, rtol=1.6e-2, atol=1.6e-2)


@pytest.mark.parametrize("H,KV,hd", [(32, 8, 128), (3, 1, 128), (5, 1, 64), (4, 2, 64), (6, 3, 64)])
@pytest.mark.parametrize("m,k", [(200, 264), (65, 64), (1000, 512)])
@pytest.mark.parametrize("write_cache", [True, False])
def test_prompt_product_rotates_and_stores_in_its_epilogue(H, KV, hd, m, k, write_cache):
    """The q/k/v product of a prompt step with the rotation and the cache write in its epilogue, against the plain
    product followed by the rotary kernel: the same bits in the queries' columns and in every byte of the cache.
    Three sequences of unequal lengths that start inside pages, one of them a padding row's slot (-1, the trash page);
    head counts that make a group of 128 columns straddle queries and keys, or end half-way (7 heads of 64); a last
    row tile that is not full."""
    n = (H + 2 * KV) * hd
    a, w = rnd(m, k, dtype=torch.bfloat16, seed=90), rnd(n, k, dtype=torch.bfloat16, seed=91, scale=0.1)
    cuts = [0, m // 3, m // 3 + 1, m]                       # tokens of sequence i: cuts[i] .. cuts[i + 1]
    starts = [37, 64, 5]
    positions = torch.cat([torch.arange(s0, s0 + (cuts[i + 1] - cuts[i])) for i, s0 in enumerate(starts)]).to(torch.int32).to(DEV)
    slots = torch.cat([torch.full((cuts[i + 1] - cuts[i],), sl, dtype=torch.int32) for i, sl in enumerate([1, -1, 0])]).to(DEV)
    pages = (max(starts) + m + 63) // 64 + 1
    bt = (torch.randperm(2 * pages, generator=torch.Generator().manual_seed(3)) + 1).to(torch.int32).reshape(2, pages).to(DEV)
    table = ops.rope_table(positions, torch.from_numpy(pl.rotary_inv_freq(hd, 10000.0, None)).to(DEV))
    results = []
    for fused in (False, True):
        kc = torch.full((2 * pages + 1, KV, 64, hd), float("nan"), dtype=torch.bfloat16, device=DEV)
        vc = torch.full_like(kc, float("nan"))
        if fused:
            qkv = ops.gemm_tc_qkv_rope(a, w, table, positions, slots, bt, kc, vc, H, KV, hd, write_cache)
        else:
            qkv = ops.gemm_tc(a, w, ops.SKINNY_STORE_BF16)
            ops.rope_cache_write(qkv, table, positions, slots, bt, kc, vc, H, KV, hd, hd, False, write_cache)
        results.append((qkv[:, :H * hd].clone(), kc, vc))
    assert ops.gemm_tc_status() == 0
    assert torch.equal(results[0][0], results[1][0])
    assert torch.equal(results[0][1].view(torch.int16), results[1][1].view(torch.int16))
    assert torch.equal(results[0][2].view(torch.int16), results[1][2].view(torch.int16))
    assert not bool(torch.isnan(results[1][0].float()).any())
    if write_cache:       # the value rows are the product's
        ref_v = (a.double() @ w.double().T)[:cuts[1], (H + KV) * hd:]
        got = torch.stack([results[1][2][int(bt[1, (37 + t) // 64]), :, (37 + t) % 64].reshape(KV * hd) for t in range(cuts[1])])
        torch.testing.assert_close(got.double(), ref_v, rtol=1.6e-2, atol=1.6e-2)
    else:
        assert bool(torch.isnan(results[1][1].float()).all())


@pytest.mark.parametrize("inside", [False, True])
@pytest.mark.parametrize("H,KV,hd,lens,hidden,splits", [(4, 2, 64, [102, 102], 192, 2), (4, 2, 64, [140, 111, 7], 192, 3),
                                                         (3, 1, 128, [102, 90], 264, 2), (32, 8, 64, [700] * 4, 2048, 4),
                                                         (32, 8, 128, [513] * 3, 4096, 3)])
def test_a_replayed_step_reads_what_its_own_kernels_wrote(H, KV, hd, lens, hidden, splits, inside):
    """Product, rotation + cache write (a kernel of its own, or inside the attention) and decode attention recorded in a CUDA graph with dependent launch: each
    kernel starts while the one before it still runs and must not read that kernel's results before its dependency
    wait.  The graph's buffers hold other values before the first replay (the queries' rows are filled with NaN, the
    cache rows of the new position with zeros), so a read that comes too early shows.  Compared bit for bit with the
    same three kernels launched one by one."""
    B = len(lens)
    S = ((max(lens) + 63) // 64) * 64
    k = rnd(B, S, KV, hd, dtype=torch.bfloat16, seed=70)
    v = rnd(B, S, KV, hd, dtype=torch.bfloat16, seed=71)
    kc, vc, bt = paged_from_dense(k, v, lens, seed=1, poison=0.0)
    w = rnd((H + 2 * KV) * hd, hidden, dtype=torch.bfloat16, seed=72, scale=0.05)
    h = rnd(B, hidden, dtype=torch.bfloat16, seed=73)
    inv = torch.rand(hd // 2, device=DEV)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    slots = torch.arange(B, dtype=torch.int32, device=DEV)
    lens_t = torch.tensor(lens, dtype=torch.int32, device=DEV)
    kept = {}

    def layer():
        with ops.defer_store():
            qkv = ops.linear(h, w, out_dtype=torch.bfloat16)
        table = ops.rope_table(pos, inv)
        if not inside:
            ops.rope_cache_write(qkv, table, pos, slots, bt, kc, vc, H, KV, hd, hd, False, True)
        out = torch.empty(B, H * hd, dtype=torch.bfloat16, device=DEV)
        po = torch.empty(B * H * splits * hd, device=DEV)
        pml = torch.empty(B * H * splits * 2, device=DEV)
        ops.attn_decode_tc(qkv, kc, vc, bt, slots, lens_t, B, H, KV, hd, 0.125, None, splits, out, po, pml,
                           rope=(table, hd) if inside else None)
        kept.update(qkv=qkv, table=table, po=po, pml=pml)
        return out

    was = ops.get_pdl()
    ops.set_pdl(True)
    try:
        want = layer().clone()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            out = layer()
        for _ in range(2):
            for t in kept.values():
                t.fill_(float("nan"))
            for b in range(B):
                page, off = int(bt[b, (lens[b] - 1) // 64]), (lens[b] - 1) % 64
                kc[page, :, off] = 0
                vc[page, :, off] = 0
            torch.cuda.synchronize()
            g.replay()
            torch.cuda.synchronize()
            assert torch.equal(out, want)
    finally:
        ops.set_pdl(was)


@pytest.mark.parametrize("mode", ["store", "accum", "swiglu", "f32"])
@pytest.mark.parametrize("m,n,k", [(2048, 4096, 256), (2048, 6144, 128), (2000, 4000, 264), (1100, 8192, 64), (300, 38400, 64)])
def test_tensor_core_product_with_narrower_tiles_in_the_last_round(mode, m, n, k):
    """Shapes whose 128 x 256 tiles do not fill the last round of blocks: the last columns are cut into narrower tiles
    (another TMA box, another instruction width, fewer epilogue chunks).  Every element is still one sum in k order: the
    same bits as with full-width tiles, and the product itself within the tolerance."""
    a = rnd(m, k, dtype=torch.bfloat16, seed=80)
    w = rnd(n, k, dtype=torch.bfloat16, seed=81, scale=0.1)
    code = {"store": ops.SKINNY_STORE_BF16, "accum": ops.SKINNY_ACCUM_F32, "swiglu": ops.SKINNY_SWIGLU, "f32": ops.SKINNY_STORE_F32}[mode]
    base = rnd(m, n, seed=82) if mode == "accum" else None
    outs = []
    try:
        for tail in (True, False):
            ops.gemm_tc_tail_tiles(tail)
            out = base.clone() if base is not None else None
            outs.append(ops.gemm_tc(a, w, code, out))
            assert ops.gemm_tc_status() == 0
    finally:
        ops.gemm_tc_tail_tiles(True)
    assert torch.equal(outs[0], outs[1])
    full = a.double() @ w.double().T
    if mode == "swiglu":
        g = full.view(m, n // 16, 2, 8)[:, :, 0].reshape(m, n // 2)
        u = full.view(m, n // 16, 2, 8)[:, :, 1].reshape(m, n // 2)
        ref = g / (1 + torch.exp(-g)) * u
        torch.testing.assert_close(outs[0].double(), ref, rtol=2e-2, atol=1e-2 * float(ref.abs().max()))
    elif mode == "accum":
        torch.testing.assert_close(outs[0].double(), base.double() + full, rtol=1e-4, atol=1e-3)
    else:
        torch.testing.assert_close(outs[0].double(), full, rtol=1e-2 if mode == "store" else 1e-4, atol=1e-3 * float(full.abs().max()))


@pytest.mark.parametrize("hd", [128, 64])
@pytest.mark.parametrize("slow_warp", [0, 3])
def test_prompt_attention_with_one_row_warp_far_behind_the_others(hd, slow_warp):
    """In the tcgen05 prompt attention four warps own 32 query rows each.  Here the rows of one warp meet a larger
    maximum at every tile (their scores grow with the key's position: the accumulator is rescaled each time, which
    waits for the output product before), while all other rows see equal scores and run ahead.  A warp a tile ahead
    must not be counted for the one behind: the slow rows' outputs name the newest key (values hold their position),
    the others the mean of what they see.  (With one barrier for both score buffers this case went wrong about once
    in some ten thousand blocks, when the slow warp was also held up by the SM's other block: the test walks the path,
    it cannot force the timing.)"""
    H, KV, n, gap = 2, 1, 1536, 12.0
    k = torch.zeros(1, n, KV, hd, device=DEV)
    k[0, :, 0, 0] = torch.arange(n, device=DEV) * gap
    v = torch.zeros(1, n, KV, hd, device=DEV)
    v[0, :, 0, :] = (torch.arange(n, device=DEV, dtype=torch.float32) / 64.0)[:, None]
    q = torch.zeros(1, n, (H + 2 * KV) * hd, device=DEV)
    rows = torch.arange(n, device=DEV)
    slow = (rows % 128) // 32 == slow_warp
    for h in range(H):
        q[0, slow, h * hd] = 1.0
    k, v, q = k.to(torch.bfloat16), v.to(torch.bfloat16), q.to(torch.bfloat16)
    kc, vc, bt = paged_from_dense(k, v, [n], seed=7)
    cu = torch.tensor([0, n], dtype=torch.int32, device=DEV)
    zero = torch.zeros(1, dtype=torch.int32, device=DEV)
    ref = attention_ref(q[:, :, :H * hd], k, v, [n], [0], H, KV, hd, 1.0, None)[0]
    for pairing in (0, 2, 1):
        ops.attn_prefill_t5_pairing(pairing)
        try:
            for _ in range(3):
                out = torch.full((n, H * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
                ops.attn_prefill_t5(q[0], kc, vc, bt, cu, zero, zero, 1, n, H, KV, hd, 1.0, None, out)
                assert ops.attn_prefill_t5_status() == 0
                torch.testing.assert_close(out.double(), ref, rtol=2e-2, atol=2e-2)
        finally:
            ops.attn_prefill_t5_pairing(1)
