"""The decode attention's entry point that allocates nothing, called through its exported C symbol.

Some callers of this library cannot ask for device memory: a program without an allocator of its own, a
plug-in under somebody else's memory budget, a loop that may not stall on cudaMalloc.  For them
`gi_attn_decode_tc_noalloc` keeps the slices' scratch in an array inside the library.  This test calls it as
such a caller would, with nothing but pointers to inputs and outputs, twice in a row with different shapes (so
the second call meets whatever the first left in the array), and checks each result bit for bit against the entry
point that takes scratch from the caller, and both against the operation written out in 64-bit.  It is collected
last, so a run that stops at the first failure has already run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SCRATCH_FLOATS = 2 * 1024 * 1024


def _lib():
    from ghost_infer_b200.kernels import build
    lib = ctypes.CDLL(build.library_path(create=True, verbose=False))
    P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_float
    lib.gi_attn_decode_tc_noalloc.argtypes = [P, L, P, L, P, P, P, I, P, P, I, I, I, I, F, I, I, P]
    lib.gi_attn_decode_tc_noalloc.restype = I
    lib.gi_attn_decode_tc.argtypes = [P, L, P, P, P, L, P, P, P, I, P, P, I, I, I, I, F, I, I, P]
    lib.gi_attn_decode_tc.restype = I
    lib.gi_last_error.restype = ctypes.c_char_p
    return lib


def _case(lens, H, KV, hd, seed):
    from gpu_helpers import paged_from_dense
    g = torch.Generator().manual_seed(seed)
    B, S = len(lens), ((max(lens) + 63) // 64) * 64
    k = torch.randn(B, S, KV, hd, generator=g).to(torch.bfloat16).to(DEV)
    v = torch.randn(B, S, KV, hd, generator=g).to(torch.bfloat16).to(DEV)
    q = torch.randn(B, H * hd, generator=g).to(torch.bfloat16).to(DEV)
    kc, vc, bt = paged_from_dense(k, v, lens, seed=seed)
    slots = torch.arange(B, dtype=torch.int32, device=DEV)
    lens_t = torch.tensor(lens, dtype=torch.int32, device=DEV)
    return q, kc, vc, bt, slots, lens_t, k, v


def _plain(q, k, v, lens, H, KV, hd, scale, window):
    """The operation itself in 64-bit, written out here: the judge of both entry points."""
    out = torch.zeros(q.shape, dtype=torch.float64, device=q.device)
    g = H // KV
    for b, n in enumerate(lens):
        lo = max(0, n - window) if window else 0
        for h in range(H):
            kk, vv = k[b, lo:n, h // g].double(), v[b, lo:n, h // g].double()
            s = (kk @ q[b, h * hd:(h + 1) * hd].double()) * scale
            out[b, h * hd:(h + 1) * hd] = torch.softmax(s, 0) @ vv
    return out


def _both(lib, q, kc, vc, bt, slots, lens_t, H, KV, hd, window, splits):
    B = q.shape[0]
    stream = torch.cuda.current_stream().cuda_stream
    got = torch.full((B, H * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    rc = lib.gi_attn_decode_tc_noalloc(got.data_ptr(), H * hd, q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(),
                                       bt.data_ptr(), bt.shape[1], slots.data_ptr(), lens_t.data_ptr(), B, H, KV, hd,
                                       0.2, window, splits, stream)
    assert rc == 0, lib.gi_last_error()
    want = torch.full_like(got, float("nan"))
    part_o = torch.empty(B * H * splits * hd, device=DEV)
    part_ml = torch.empty(B * H * splits * 2, device=DEV)
    rc = lib.gi_attn_decode_tc(want.data_ptr(), H * hd, part_o.data_ptr(), part_ml.data_ptr(), q.data_ptr(), q.stride(0),
                               kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), bt.shape[1], slots.data_ptr(),
                               lens_t.data_ptr(), B, H, KV, hd, 0.2, window, splits, stream)
    assert rc == 0, lib.gi_last_error()
    torch.cuda.synchronize()
    return got, want


def _check(lib, lens, H, KV, hd, window, splits, seed):
    q, kc, vc, bt, slots, lens_t, k, v = _case(lens, H, KV, hd, seed)
    got, want = _both(lib, q, kc, vc, bt, slots, lens_t, H, KV, hd, window, splits)
    # the same kernel with its scratch elsewhere: not one bit may differ
    assert torch.equal(got, want)
    # and both are the operation: bfloat16 results of 64-bit sums (8 significant bits, probabilities rounded to
    # bfloat16 before they meet the values)
    ref = _plain(q, k, v, lens, H, KV, hd, 0.2, window)
    torch.testing.assert_close(got.double(), ref, rtol=1.6e-2, atol=1.6e-2)
    torch.testing.assert_close(want.double(), ref, rtol=1.6e-2, atol=1.6e-2)


def test_two_calls_in_a_row_match_the_entry_point_that_takes_scratch():
    lib = _lib()
    # first call: many slices of long contexts; second call: other sizes, so its slices land on what the first left;
    # third: one slice (no scratch is touched); fourth: the first again, on what the others left
    for lens, H, KV, hd, window, splits, seed in (([700, 333, 64, 1], 32, 8, 128, 0, 6, 1),
                                                  ([129, 500, 31], 6, 2, 64, 100, 3, 2),
                                                  ([200, 77], 8, 2, 128, 0, 1, 3),
                                                  ([700, 333, 64, 1], 32, 8, 128, 0, 6, 1)):
        _check(lib, lens, H, KV, hd, window, splits, seed)


def test_the_largest_request_the_built_in_scratch_holds_is_served_and_the_next_refused():
    """A request needs sequences x heads x slices x (head size + 2) floats.  With the head sizes the kernel takes that
    last factor is 66 or 130, and the limit, 2^21, has no odd factor: no request lands on the limit itself.  So the
    case here is the largest that fits for its heads and slices (8 x 32 x 63 x 130 = 2,096,640 of 2,097,152), checked
    like the others, and beside it one more sequence (2,358,720), which is refused."""
    lib = _lib()
    H, KV, hd, splits = 32, 8, 128, 63
    B = SCRATCH_FLOATS // (H * splits * (hd + 2))
    assert B == 8 and SCRATCH_FLOATS - B * H * splits * (hd + 2) < H * splits * (hd + 2)
    _check(lib, [130 + 61 * i for i in range(B)], H, KV, hd, 0, splits, 5)
    q, kc, vc, bt, slots, lens_t, _, _ = _case([5] * (B + 1), H, KV, hd, 6)
    out = torch.zeros((B + 1, H * hd), dtype=torch.bfloat16, device=DEV)
    rc = lib.gi_attn_decode_tc_noalloc(out.data_ptr(), H * hd, q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(),
                                       bt.data_ptr(), bt.shape[1], slots.data_ptr(), lens_t.data_ptr(), B + 1, H, KV, hd,
                                       0.2, 0, splits, torch.cuda.current_stream().cuda_stream)
    assert rc != 0 and "scratch" in lib.gi_last_error().decode()


def test_a_request_beyond_the_built_in_scratch_is_refused():
    lib = _lib()
    H, KV, hd, splits = 32, 8, 128, 16
    B = SCRATCH_FLOATS // (H * splits * (hd + 2)) + 1
    q, kc, vc, bt, slots, lens_t, _, _ = _case([5] * B, H, KV, hd, 3)
    out = torch.zeros((B, H * hd), dtype=torch.bfloat16, device=DEV)
    rc = lib.gi_attn_decode_tc_noalloc(out.data_ptr(), H * hd, q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(),
                                       bt.data_ptr(), bt.shape[1], slots.data_ptr(), lens_t.data_ptr(), B, H, KV, hd,
                                       0.2, 0, splits, torch.cuda.current_stream().cuda_stream)
    assert rc != 0
    msg = lib.gi_last_error().decode()
    assert "scratch" in msg and str(SCRATCH_FLOATS) in msg
    torch.cuda.synchronize()
    assert float(out.float().abs().sum()) == 0          # nothing was launched
