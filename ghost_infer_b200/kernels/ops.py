"""Typed Python wrappers over the kernel library's C entry points.

Each wrapper checks shapes, dtypes, devices and contiguity on the host (the reference validates
token ids, capacity and sizes before any launch: src/model.rs:974-982, src/cuda.rs:8644-8652), then
launches on torch's current stream.  Tensors are torch tensors on a CUDA device; nothing here runs on
the CPU and nothing falls back to library code.
"""
from __future__ import annotations

import contextlib
import ctypes
import os
import weakref
from ctypes import c_float, c_int, c_long, c_void_p
from typing import Dict, Optional, Tuple

import torch

from .library import KernelError, last_error, load

F32, BF16 = 0, 1
GEMM_STORE, GEMM_ACCUM_F32 = 0, 1

_DT = {torch.float32: F32, torch.bfloat16: BF16}


class SettleT(ctypes.Structure):
    """gi_settle_t: where a deferred product left its partial sums and how it had cut its work."""
    _fields_ = [("partials", c_void_p), ("tile_first_cta", c_void_p), ("tile_last_cta", c_void_p),
                ("cta_first_tile", c_void_p), ("nt", c_int)]


_bound = None


def _bind():
    global _bound
    if _bound is not None:
        return _bound
    lib = load()
    P, I, L, F = c_void_p, c_int, c_long, c_float
    sigs = {
        "gi_embed": [P, P, I, P, I, I, I, P],
        "gi_rmsnorm": [P, I, P, P, I, P, I, I, F, P],
        "gi_rmsnorm_settle": [P, I, P, P, I, P, I, I, F, SettleT, P],
        "gi_settle": [P, SettleT, P, I, I, P],
        "gi_gemm_stream_geometry": [I, I, I, ctypes.POINTER(c_int), ctypes.POINTER(c_int), ctypes.POINTER(c_int)],
        "gi_silu_mul": [P, P, I, I, I, I, P],
        "gi_gemm_skinny_bf16": [P, I, P, P, I, I, I, L, L, L, P],
        "gi_gemm_generic": [P, I, I, P, I, P, I, I, I, I, L, L, L, P],
        "gi_rope_table": [P, P, P, I, I, P],
        "gi_rope_cache_write": [P, I, L, P, P, P, P, I, P, P, I, I, I, I, I, I, I, P],
        "gi_rope_cache_write_settle": [P, I, L, P, P, P, P, I, P, P, I, I, I, I, I, I, I, SettleT, P],
        "gi_attn_prefill_generic": [P, L, P, L, I, P, P, P, I, P, P, P, I, I, I, I, I, F, I, P],
        "gi_attn_decode_generic": [P, L, P, P, P, L, I, P, P, P, I, P, P, I, I, I, I, F, I, I, I, P],
        "gi_gemm_stream_bf16": [P, I, P, P, P, P, I, I, I, I, L, L, L, I, P],
        "gi_gemm_stream_bf16_ex": [P, I, P, P, P, P, I, I, I, I, L, L, L, I, P, I, I, L, I, I, P],
        "gi_gemm_stream_status": [P],
        "gi_gemm_tc_bf16": [P, I, P, P, I, I, I, L, L, L, I, P],
        "gi_gemm_tc_status": [P],
        "gi_attn_prefill_tc": [P, L, P, L, P, P, P, I, P, P, P, I, I, I, I, I, F, I, P],
        "gi_attn_prefill_t5": [P, L, P, L, L, P, P, L, P, I, P, P, P, I, I, I, I, I, F, I, P],
        "gi_attn_prefill_t5_status": [P],
        "gi_attn_decode_tc": [P, L, P, P, P, L, P, P, P, I, P, P, I, I, I, I, F, I, I, P],
        "gi_attn_decode_tc_ex": [P, L, P, P, P, L, P, P, P, I, P, P, I, I, I, I, F, I, I, I, P],
        "gi_attn_decode_tc_merged": [P, L, P, P, P, I, P, L, P, P, P, I, P, P, I, I, I, I, F, I, I, I, I, I, P],
        "gi_attn_decode_tc_rope": [P, L, P, P, P, I, P, L, P, P, P, I, P, P, I, I, I, I, F, I, I, I, I, I, P, I, SettleT, P],
        "gi_attn_decode_kr": [P, L, P, P, P, L, P, P, P, I, P, P, I, I, I, I, F, I, I, I, I, I, P],
        "gi_gemm_tc_qkv_rope": [P, P, P, I, I, I, L, L, L, P, P, P, P, I, P, P, I, I, I, I, P],
        "gi_sample": [P, P, L, I, I, F, I, F, P, P, P],
    }
    for name, argtypes in sigs.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = c_int
    lib.gi_gemm_stream_scratch_floats.restype = c_long
    if os.environ.get("GHOST_INFER_PDL") in ("0", "1"):         # the process-wide default of set_pdl
        lib.gi_set_pdl(int(os.environ["GHOST_INFER_PDL"]))
    _bound = lib
    return lib


launches = 0   # kernels launched through this module since import (benchmarks report the difference)


def _check(lib, rc: int, n: int = 1) -> None:
    global launches
    if rc != 0:
        raise KernelError(last_error(lib) or f"kernel entry point failed with code {rc}")
    launches += n


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _dt(t: torch.Tensor, what: str) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"{what}: dtype {t.dtype} is not supported (float32 or bfloat16)") from None


def _cuda(t: torch.Tensor, what: str, settles: bool = False) -> None:
    """`settles`: the kernel about to read `t` adds pending partial sums itself; any other kernel must not meet them."""
    if not t.is_cuda:
        raise KernelError(f"{what} must live on a CUDA device; there is no CPU path")
    if not settles and type(t) is Carrier and t.__dict__.get("_gi_pending") is not None:
        raise KernelError(f"{what}: partial sums of a deferred product are pending for this tensor; "
                          f"only a kernel that settles them (or ops.settle) may read it")


def _rows(t: torch.Tensor, what: str) -> int:
    """Leading dimension (in elements) of a 2-D tensor whose rows are contiguous."""
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{what} must be 2-D with contiguous rows, got shape {tuple(t.shape)} strides {t.stride()}")
    return t.stride(0)


def _i32(t: Optional[torch.Tensor], what: str):
    if t is None:
        return None
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{what} must be a contiguous int32 tensor")
    _cuda(t, what)
    return t.data_ptr()


# ---- time per kind of operation ----------------------------------------------------------------------------
# The reference sums wall-clock time into eight named buckets ("embed", "norm+quant", "qkv matmul", "rope+cache",
# "attention", "out matmul", "ffn matmul", "logits"), switched on by GHOST_INFER_PROFILE, synchronising after each
# operation and running without its CUDA graph meanwhile (src/profile.rs:7-46, src/cuda.rs:8054-8063, :9993-9996).
# Here the parts name the bucket of what they launch (`with ops.bucket("attention"):`), and while profiling is on a
# pair of CUDA events brackets each such stretch on the launching stream: device time, no synchronisation inside a
# step.  Steps are then launched kernel by kernel (no graph replay, no dependent launch, which would let one bucket's
# kernels run inside another's stretch).  Off, `bucket` hands out one shared do-nothing context.
BUCKETS = ("embed", "norm", "qkv matmul", "rope+cache", "attention", "out matmul", "ffn matmul", "logits", "sampling")


class _NoBucket:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NO_BUCKET = _NoBucket()
_profile_marks: Optional[list] = None      # (bucket, start event, end event) while profiling
_profile_pdl_was: Optional[bool] = None


class _Bucket:
    __slots__ = ("name", "start")

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        self.start = torch.cuda.Event(enable_timing=True)
        self.start.record()
        return self

    def __exit__(self, *exc):
        end = torch.cuda.Event(enable_timing=True)
        end.record()
        if _profile_marks is not None:
            _profile_marks.append((self.name, self.start, end))
        return False


def bucket(name: str):
    """A context for the launches of one kind of operation; it costs nothing unless profiling is on."""
    return _NO_BUCKET if _profile_marks is None else _Bucket(name)


def profiling() -> bool:
    return _profile_marks is not None


def profile_start() -> None:
    """From now on the device time of every bucketed stretch is recorded (steps run without graph and dependent launch)."""
    global _profile_marks, _profile_pdl_was
    if _profile_marks is None:
        _profile_pdl_was = get_pdl()
        set_pdl(False)
    _profile_marks = []


def profile_stop() -> Dict[str, float]:
    """Stops recording.  Returns milliseconds of device time per bucket, in the order of BUCKETS (others after)."""
    global _profile_marks, _profile_pdl_was
    marks, _profile_marks = _profile_marks or [], None
    if _profile_pdl_was is not None:
        set_pdl(_profile_pdl_was)
        _profile_pdl_was = None
    torch.cuda.synchronize()
    totals: Dict[str, float] = {}
    for name, a, b in marks:
        totals[name] = totals.get(name, 0.0) + a.elapsed_time(b)
    order = [n for n in BUCKETS if n in totals] + sorted(n for n in totals if n not in BUCKETS)
    return {n: totals[n] for n in order}


# ------------------------------------------------------------------------------------------------
def embed(table: torch.Tensor, tokens: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    lib = _bind()
    _cuda(table, "embedding table")
    if table.dim() != 2 or not table.is_contiguous():
        raise KernelError("the embedding table must be a contiguous [vocab, width] matrix")
    n, (vocab, d) = tokens.numel(), table.shape
    if out is None:
        out = torch.empty((n, d), dtype=torch.float32, device=table.device)
    _check(lib, lib.gi_embed(out.data_ptr(), table.data_ptr(), _dt(table, "embedding table"), _i32(tokens, "tokens"),
                             n, d, vocab, _stream()))
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
            rows: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    lib = _bind()
    _cuda(x, "rmsnorm input", settles=True)
    if x.dtype != torch.float32 or x.dim() != 2 or not x.is_contiguous():
        raise KernelError("rmsnorm input must be a contiguous float32 [rows, width] matrix")
    d = x.shape[1]
    if weight.numel() != d or not weight.is_contiguous():
        raise KernelError(f"rmsnorm weight has {weight.numel()} values, the rows are {d} wide")
    n = x.shape[0] if rows is None else rows.numel()
    if out is None:
        out = torch.empty((n, d), dtype=out_dtype, device=x.device)
    pending = _take_pending(x)
    if pending is not None and (pending[1] or d % 4 != 0):
        x.__dict__["_gi_pending"] = pending         # not this kernel's kind of sums: the plain way
        settle(x)
        pending = None
    if pending is not None:
        pending = pending[0]
        # a deferred product left partial sums for this stream: add them while the rows are read anyway (and write
        # the settled rows back; with a selection of rows nothing is written back: the selection may name a row twice,
        # and the stream's other rows stay unsettled, so whoever selects rows must be the stream's last reader)
        _check(lib, lib.gi_rmsnorm_settle(out.data_ptr(), _dt(out, "rmsnorm output"), x.data_ptr(), weight.data_ptr(),
                                          _dt(weight, "rmsnorm weight"), _i32(rows, "rows"), n, d, float(eps), pending,
                                          _stream()))
        return out
    _check(lib, lib.gi_rmsnorm(out.data_ptr(), _dt(out, "rmsnorm output"), x.data_ptr(), weight.data_ptr(),
                               _dt(weight, "rmsnorm weight"), _i32(rows, "rows"), n, d, float(eps), _stream()))
    return out


# ---- deferred accumulation into the residual stream ---------------------------------------------------
# The decode product cuts tiles of W between blocks; adding such a tile's partial sums into the residual
# stream needs an exchange between blocks at the kernel's end.  When the stream's next reader is a norm, which
# reads every row anyway, the product leaves the partial sums in scratch and the norm adds them (in a fixed
# order).  What is pending travels with the tensor itself: only a `Carrier` can have sums pending, the record
# is an attribute of that object (so it dies with it and no other tensor at the same address inherits it),
# any torch operation on it settles first, and a kernel wrapper that does not settle refuses it.
_METADATA = frozenset((
    "get:shape", "get:dtype", "get:device", "get:is_cuda", "get:ndim", "get:layout", "get:requires_grad", "get:is_cpu",
    "get:is_meta", "get:names", "get:grad_fn", "get:is_leaf", "get:_base",
    "data_ptr", "stride", "size", "dim", "numel", "nelement", "element_size", "storage_offset", "is_contiguous",
    "is_floating_point", "is_complex", "get_device", "__len__", "ndimension", "__repr__", "__format__"))


class Carrier(torch.Tensor):
    """A device tensor that a deferred product may leave partial sums for (the residual stream of a step; the
    q/k/v rows on their way to the kernel that rotates and stores).  Shares its storage with the plain tensor
    it was made from.  Reading its sizes, strides and address is free; every other torch operation on it first
    adds what is pending (one kernel launch), so that no reader can see rows without their sums."""

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        name = getattr(func, "__name__", "")
        if name == "__get__":
            name = "get:" + getattr(getattr(func, "__self__", None), "__name__", "")
        if name not in _METADATA:
            for a in args:
                if type(a) is Carrier and a.__dict__.get("_gi_pending") is not None:
                    settle(a)
        with torch._C.DisableTorchFunctionSubclass():
            return func(*args, **(kwargs or {}))


def as_carrier(t: torch.Tensor) -> torch.Tensor:
    """`t` as a tensor that deferred products may leave partial sums for (same storage)."""
    return t if type(t) is Carrier else t.as_subclass(Carrier)


_pending_scratch: Dict[int, torch.Tensor] = {}
_defer_target: Optional[torch.Tensor] = None


def _take_pending(x: torch.Tensor):
    if type(x) is not Carrier:
        return None
    return x.__dict__.pop("_gi_pending", None)


@contextlib.contextmanager
def defer_into(x: torch.Tensor):
    """Inside, a product accumulated into `x` (this very object, a `Carrier`) may leave partial sums pending.
    Whoever reads `x` next settles them: `rmsnorm` while it reads the rows, anything else through `settle`."""
    global _defer_target
    prev = _defer_target
    _defer_target = x if (TUNE["defer_residual"] and type(x) is Carrier and x.is_cuda) else None
    try:
        yield
    finally:
        _defer_target = prev


_defer_store = False


@contextlib.contextmanager
def defer_store():
    """Inside, a decode product that stores bfloat16 rows may leave the tiles cut between blocks as partial sums
    (its result is then a `Carrier`).  `rope_cache_write` adds them while it reads the rows."""
    global _defer_store
    prev = _defer_store
    _defer_store = bool(TUNE["defer_residual"])
    try:
        yield
    finally:
        _defer_store = prev


def has_pending(x: torch.Tensor) -> bool:
    return type(x) is Carrier and x.__dict__.get("_gi_pending") is not None


def settle(x: torch.Tensor) -> None:
    """Adds pending partial sums (if any) to every row of the matrix `x`."""
    pending = _take_pending(x)
    if pending is None:
        return
    lib = _bind()
    rec, store = pending
    if store:
        raise KernelError("partial sums of a stored product are pending: only rope_cache_write settles those")
    _check(lib, lib.gi_settle(x.data_ptr(), rec, None, x.shape[0], x.shape[1], _stream()))


def drop_pending(x: torch.Tensor) -> None:
    """Forgets partial sums pending for `x` (the stream is not read again)."""
    _take_pending(x)


def _defer_ok(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    return (_defer_target is not None and out is _defer_target and out.dtype == torch.float32
            and out.is_contiguous() and out.shape[1] % 4 == 0 and out.shape[1] <= 8192 and out.data_ptr() % 16 == 0
            and not has_pending(out))


def _gemm_stream_deferred(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int = 4) -> torch.Tensor:
    lib = _bind()
    key = a.device.index if a.device.index is not None else torch.cuda.current_device()
    if key not in _pending_scratch:
        _pending_scratch[key] = torch.empty(int(lib.gi_gemm_stream_scratch_floats()), dtype=torch.float32, device=a.device)
    scratch = _pending_scratch[key]
    m, k = a.shape
    n = w.shape[0]
    _, counters = _stream_buffers(a.device)
    _check(lib, lib.gi_gemm_stream_bf16_ex(out.data_ptr(), mode, a.data_ptr(), w.data_ptr(), scratch.data_ptr(),
                                           counters.data_ptr(), counters.numel(), m, n, k, a.stride(0), w.stride(0),
                                           out.stride(0), -1, *_next_weights(w, mode), _stream()))
    n_ctas, kb, nt = c_int(0), c_int(0), c_int(0)
    lib.gi_gemm_stream_geometry(m, n, k, ctypes.byref(n_ctas), ctypes.byref(kb), ctypes.byref(nt))
    tabs = _settle_tables(a.device, (n + 127) // 128, kb.value, n_ctas.value)
    out.__dict__["_gi_pending"] = (SettleT(scratch.data_ptr(), tabs[0].data_ptr(), tabs[1].data_ptr(), tabs[2].data_ptr(), nt.value),
                                   mode == SKINNY_STORE_DEFER)
    return out


_settle_tabs: Dict[tuple, tuple] = {}


def _settle_tables(device: torch.device, n_tiles: int, kb_per_tile: int, n_ctas: int):
    """Which blocks held pieces of which tile, as the streamed product cuts its work: block c takes the units
    [c * U / G, (c + 1) * U / G) of the U = tiles x K-blocks units.  Built once per shape, kept on the device."""
    key = (str(device), n_tiles, kb_per_tile, n_ctas)
    if key not in _settle_tabs:
        units = n_tiles * kb_per_tile
        starts = [c * units // n_ctas for c in range(n_ctas + 1)]
        import bisect
        cta_of = lambda u: bisect.bisect_right(starts, u) - 1
        first = [cta_of(t * kb_per_tile) for t in range(n_tiles)]
        last = [cta_of((t + 1) * kb_per_tile - 1) for t in range(n_tiles)]
        first_tile = [starts[c] // kb_per_tile for c in range(n_ctas)]
        _settle_tabs[key] = tuple(torch.tensor(v, dtype=torch.int32, device=device) for v in (first, last, first_tile))
    return _settle_tabs[key]


def silu_mul(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None, interleaved: bool = False) -> torch.Tensor:
    """silu(gate) * up over rows [gate | up], or, `interleaved`, rows of blocks [8 gate | 8 up]."""
    lib = _bind()
    _cuda(gate_up, "gate/up rows")
    if gate_up.dim() != 2 or not gate_up.is_contiguous() or gate_up.shape[1] % 2:
        raise KernelError("gate/up rows must be a contiguous [rows, 2 * width] matrix")
    n, f = gate_up.shape[0], gate_up.shape[1] // 2
    if out is None:
        out = torch.empty((n, f), dtype=gate_up.dtype, device=gate_up.device)
    _check(lib, lib.gi_silu_mul(out.data_ptr(), gate_up.data_ptr(), _dt(gate_up, "gate/up rows"), n, f, int(interleaved),
                                _stream()))
    return out


def gemm_generic(a: torch.Tensor, w: torch.Tensor, *, out: Optional[torch.Tensor] = None,
                 out_dtype: Optional[torch.dtype] = None, accumulate: bool = False) -> torch.Tensor:
    """out[M, N] (+)= a[M, K] @ w[N, K]^T with 32-bit accumulation on CUDA cores."""
    lib = _bind()
    _cuda(a, "activations")
    _cuda(w, "weights")
    lda, ldw = _rows(a, "activations"), _rows(w, "weights")
    m, k = a.shape
    n, kw = w.shape
    if k != kw:
        raise KernelError(f"matrix product: activations are {k} wide, the weights take {kw}")
    if out is None:
        if accumulate:
            raise KernelError("matrix product: accumulation needs an output to add to")
        out = torch.empty((m, n), dtype=out_dtype or a.dtype, device=a.device)
    ldo = _rows(out, "output")
    if out.shape != (m, n):
        raise KernelError(f"matrix product: output is {tuple(out.shape)}, wanted {(m, n)}")
    mode = GEMM_ACCUM_F32 if accumulate else GEMM_STORE
    _check(lib, lib.gi_gemm_generic(out.data_ptr(), _dt(out, "output"), mode, a.data_ptr(), _dt(a, "activations"),
                                    w.data_ptr(), _dt(w, "weights"), m, n, k, lda, ldw, ldo, _stream()))
    return out


SKINNY_STORE_BF16, SKINNY_STORE_F32, SKINNY_ACCUM_F32, SKINNY_SWIGLU, SKINNY_ACCUM_DEFER, SKINNY_STORE_DEFER = 0, 1, 2, 3, 4, 5
SKINNY_MAX_ROWS = 64


def skinny_ok(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the decode product kernel takes these operands: bfloat16, at most 64 rows, 16-byte rows."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.dim() == 2 and w.dim() == 2
            and 0 < a.shape[0] <= SKINNY_MAX_ROWS and a.shape[1] % 8 == 0 and a.stride(1) == 1 and w.stride(1) == 1
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_skinny(a: torch.Tensor, w: torch.Tensor, mode: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[M, N] (op)= a[M, K] @ w[N, K]^T for M <= 64, bfloat16 operands, tensor cores, bound by the bytes of w.
    mode SKINNY_SWIGLU: w's rows are interleaved [8 gate | 8 up] and out is [M, N / 2] = silu(gate) * up."""
    lib = _bind()
    _cuda(a, "activations")
    _cuda(w, "weights")
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("the decode product kernel takes bfloat16 operands")
    lda, ldw = _rows(a, "activations"), _rows(w, "weights")
    m, k = a.shape
    n, kw = w.shape
    if k != kw:
        raise KernelError(f"matrix product: activations are {k} wide, the weights take {kw}")
    cols = n // 2 if mode == SKINNY_SWIGLU else n
    want = {SKINNY_STORE_BF16: torch.bfloat16, SKINNY_SWIGLU: torch.bfloat16}.get(mode, torch.float32)
    if out is None:
        if mode == SKINNY_ACCUM_F32:
            raise KernelError("matrix product: accumulation needs an output to add to")
        out = torch.empty((m, cols), dtype=want, device=a.device)
    if out.shape != (m, cols) or out.dtype != want:
        raise KernelError(f"matrix product: output is {tuple(out.shape)} {out.dtype}, wanted {(m, cols)} {want}")
    ldo = _rows(out, "output")
    _check(lib, lib.gi_gemm_skinny_bf16(out.data_ptr(), mode, a.data_ptr(), w.data_ptr(), m, n, k, lda, ldw, ldo, _stream()))
    return out


# Choices measured on a B200; benchmarks may override them to try alternatives.
TUNE = {"small_skinny": False, "attn_waves": 1.0, "attn_tile_keys": 16, "defer_residual": True, "attn_prefill_tcgen05": True, "prefetch_units": 16,
        "attn_merge_inside": False, "attn_own_slices": False, "attn_stages_hd64": 2, "attn_stages_hd128": 3, "attn_rope_inside": False, "stream_whole_percent": 80,
        "attn_keys_on_rows": True, "attn_kr_warps": 6, "attn_kr_stages": 2, "qkv_rope_epilogue": True, "attn_min_slice": 256}
USE_STREAM = True    # decode products through the persistent stream-K kernel (else the mma.sync kernel)


def set_pdl(on: bool) -> None:
    """Programmatic dependent launch: consecutive kernels of a stream that support it overlap one's start with
    the other's end (and the decode product prefetches weights meanwhile).  Process-wide; on unless switched off
    here or by GHOST_INFER_PDL=0 in the environment."""
    lib = _bind()
    lib.gi_set_pdl(int(bool(on)))


def get_pdl() -> bool:
    return bool(_bind().gi_get_pdl())


_STREAM_COUNTERS = 8192
_stream_scratch = {}


def _stream_buffers(device: torch.device):
    """Scratch of the streamed product, one set per device, allocated once (its address is baked into graphs)."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _stream_scratch:
        lib = _bind()
        n = int(lib.gi_gemm_stream_scratch_floats())
        _stream_scratch[key] = (torch.empty(n, dtype=torch.float32, device=device),
                                torch.zeros(_STREAM_COUNTERS, dtype=torch.int32, device=device))
    return _stream_scratch[key]


_whole_percent = 80    # what the library was last told (its own default)


def gemm_stream(a: torch.Tensor, w: torch.Tensor, mode: int, out: Optional[torch.Tensor] = None,
                pdl: Optional[bool] = None) -> torch.Tensor:
    """out[M, N] (op)= a[M, K] @ w[N, K]^T for M <= 64: persistent, TMA-fed, tcgen05, stream-K balanced; the decode
    step's product.  Modes as gemm_skinny's."""
    lib = _bind()
    _cuda(a, "activations")
    _cuda(w, "weights")
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("the streamed product takes bfloat16 operands")
    lda, ldw = _rows(a, "activations"), _rows(w, "weights")
    m, k = a.shape
    n, kw = w.shape
    if k != kw:
        raise KernelError(f"matrix product: activations are {k} wide, the weights take {kw}")
    cols = n // 2 if mode == SKINNY_SWIGLU else n
    want = {SKINNY_STORE_BF16: torch.bfloat16, SKINNY_SWIGLU: torch.bfloat16}.get(mode, torch.float32)
    if out is None:
        if mode == SKINNY_ACCUM_F32:
            raise KernelError("matrix product: accumulation needs an output to add to")
        out = torch.empty((m, cols), dtype=want, device=a.device)
    if out.shape != (m, cols) or out.dtype != want:
        raise KernelError(f"matrix product: output is {tuple(out.shape)} {out.dtype}, wanted {(m, cols)} {want}")
    ldo = _rows(out, "output")
    scratch, counters = _stream_buffers(a.device)
    if (n + 127) // 128 > counters.numel():
        raise KernelError(f"the streamed product takes at most {counters.numel() * 128} rows of weights")
    global _whole_percent
    if _whole_percent != int(TUNE["stream_whole_percent"]):
        _whole_percent = int(TUNE["stream_whole_percent"])
        lib.gi_gemm_stream_whole_tiles(_whole_percent)
    _check(lib, lib.gi_gemm_stream_bf16_ex(out.data_ptr(), mode, a.data_ptr(), w.data_ptr(), scratch.data_ptr(),
                                           counters.data_ptr(), counters.numel(), m, n, k, lda, ldw, ldo,
                                           -1 if pdl is None else int(pdl), *_next_weights(w, mode), _stream()))
    return out


# ---- which matrix the next streamed product reads -----------------------------------------------------
# A decode step runs the same products in the same order every time.  Each streamed product remembers which
# matrix followed it the last time and tells its kernel, which asks the L2 cache for that matrix's first units
# while it drains, so the memory does not idle across the kernel boundary.  A wrong guess only costs bandwidth.
_followed_by: Dict[int, tuple] = {}            # weights' address -> (weak reference to the next weights, that product's mode)
_last_streamed: Optional[int] = None


def _next_weights(w: torch.Tensor, mode: int):
    """(pointer, rows, columns, row stride, mode, units ahead) of the product that followed `w`'s last time, or nothing."""
    global _last_streamed
    here = w.data_ptr()
    if _last_streamed is not None and _last_streamed != here:
        if len(_followed_by) > 4096:                     # models come and go: forget the weights that are gone
            for key in [k for k, (ref, _) in _followed_by.items() if ref() is None]:
                del _followed_by[key]
        _followed_by[_last_streamed] = (weakref.ref(w), mode)
    _last_streamed = here
    ref, next_mode = _followed_by.get(here, (None, 0))
    nxt = ref() if ref is not None else None
    ahead = int(TUNE["prefetch_units"])
    if (nxt is None or ahead <= 0 or nxt.dtype != torch.bfloat16 or nxt.dim() != 2 or nxt.stride(1) != 1
            or nxt.device != w.device):
        return None, 0, 0, 0, 0, 0
    return nxt.data_ptr(), nxt.shape[0], nxt.shape[1], nxt.stride(0), next_mode, ahead


_timeline_buf: Optional[torch.Tensor] = None


def stream_timeline_start(slots: int, device="cuda") -> None:
    """From now on each streamed product's blocks note the nanosecond clock at eight places of their life, launch n
    into slot n mod `slots` (a launch captured in a CUDA graph keeps its slot).  For timelines of a decode step."""
    global _timeline_buf
    lib = _bind()
    _timeline_buf = torch.zeros((slots, 256, 8), dtype=torch.int64, device=device)
    lib.gi_gemm_stream_timeline.restype = c_long
    lib.gi_gemm_stream_timeline.argtypes = [c_void_p, c_int]
    lib.gi_gemm_stream_timeline(_timeline_buf.data_ptr(), slots)


def stream_timeline_stop():
    """Stops the stamping.  Returns (stamps [slots, 256 blocks, 8 events] as an int64 array, launches stamped).
    Events: 0 entry, 1 set up, 2 the SM's number, 3 dependency wait over, 4 first stage landed, 5 last load issued,
    6 last product issued, 7 last epilogue done."""
    global _timeline_buf
    lib = _bind()
    lib.gi_gemm_stream_timeline.restype = c_long
    lib.gi_gemm_stream_timeline.argtypes = [c_void_p, c_int]
    n = int(lib.gi_gemm_stream_timeline(None, 0))
    torch.cuda.synchronize()
    out = _timeline_buf.cpu().numpy() if _timeline_buf is not None else None
    _timeline_buf = None
    return out, n


def gemm_stream_status() -> int:
    lib = _bind()
    status = ctypes.c_int(0)
    _check(lib, lib.gi_gemm_stream_status(ctypes.byref(status)), 0)
    return status.value


def _decode_product(a: torch.Tensor, w: torch.Tensor, mode: int, out: Optional[torch.Tensor]) -> torch.Tensor:
    """The streamed product has a fixed cost of a few microseconds (set-up, and partial sums that cross blocks)
    and then runs at the memory's speed; the register-fed kernel starts faster and streams slower.  Alone, the
    latter wins for at most 8 rows against less than 64 MB of weights; inside a decode step with dependent
    launch the streamed one wins everywhere (it fetches weights while its predecessor drains), so it is the
    default and `TUNE["small_skinny"]` switches the other choice on."""
    small = TUNE["small_skinny"] and a.shape[0] <= 8 and w.shape[0] * w.shape[1] * 2 < (64 << 20)
    if USE_STREAM and not small and (w.shape[0] + 127) // 128 <= _STREAM_COUNTERS:
        if mode == SKINNY_ACCUM_F32:
            if _defer_ok(a, w, out):
                return _gemm_stream_deferred(a, w, out)
            settle(out)          # something is pending for this stream already: add it before adding more
        if mode == SKINNY_STORE_BF16 and _defer_store and out is None and w.shape[0] % 8 == 0:
            out = as_carrier(torch.empty((a.shape[0], w.shape[0]), dtype=torch.bfloat16, device=a.device))
            return _gemm_stream_deferred(a, w, out, SKINNY_STORE_DEFER)
        return gemm_stream(a, w, mode, out)
    return gemm_skinny(a, w, mode, out)


TC_TILE_N = 256     # width of the tensor-core product's output tile (128 or 256)


def tc_ok(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the tcgen05 product takes these operands: bfloat16, rows 16 bytes apart, 16-byte aligned."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.dim() == 2 and w.dim() == 2
            and a.shape[0] > 0 and a.shape[1] % 8 == 0 and a.stride(1) == 1 and w.stride(1) == 1
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc(a: torch.Tensor, w: torch.Tensor, mode: int, out: Optional[torch.Tensor] = None,
            tile_n: Optional[int] = None) -> torch.Tensor:
    """out[M, N] (op)= a[M, K] @ w[N, K]^T on tcgen05 tensor cores with TMA-fed operands; modes as gemm_skinny's."""
    lib = _bind()
    _cuda(a, "activations")
    _cuda(w, "weights")
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("the tensor-core product takes bfloat16 operands")
    lda, ldw = _rows(a, "activations"), _rows(w, "weights")
    m, k = a.shape
    n, kw = w.shape
    if k != kw:
        raise KernelError(f"matrix product: activations are {k} wide, the weights take {kw}")
    cols = n // 2 if mode == SKINNY_SWIGLU else n
    want = {SKINNY_STORE_BF16: torch.bfloat16, SKINNY_SWIGLU: torch.bfloat16}.get(mode, torch.float32)
    if out is None:
        if mode == SKINNY_ACCUM_F32:
            raise KernelError("matrix product: accumulation needs an output to add to")
        out = torch.empty((m, cols), dtype=want, device=a.device)
    if out.shape != (m, cols) or out.dtype != want:
        raise KernelError(f"matrix product: output is {tuple(out.shape)} {out.dtype}, wanted {(m, cols)} {want}")
    ldo = _rows(out, "output")
    _check(lib, lib.gi_gemm_tc_bf16(out.data_ptr(), mode, a.data_ptr(), w.data_ptr(), m, n, k, lda, ldw, ldo,
                                    int(tile_n or TC_TILE_N), _stream()))
    return out


def qkv_rope_ok(h: torch.Tensor, w: torch.Tensor, memory, head_dim: int, rotary_dim: int) -> bool:
    """Whether the prompt step's q/k/v product can rotate and store in its epilogue (`gemm_tc_qkv_rope`): the
    tensor-core product takes the operands, heads of 64 or 128 values rotated whole, a bfloat16 cache or none to write."""
    if not (TUNE["qkv_rope_epilogue"] and tc_ok(h, w) and h.shape[0] > SKINNY_MAX_ROWS and head_dim in (64, 128)
            and rotary_dim == head_dim):
        return False
    if memory.writes and memory.k is not None:
        return memory.k.dtype == torch.bfloat16 and memory.k.is_contiguous() and memory.v.is_contiguous()
    return True


def gemm_tc_qkv_rope(h: torch.Tensor, w: torch.Tensor, table: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor,
                     block_table: Optional[torch.Tensor], kcache: Optional[torch.Tensor], vcache: Optional[torch.Tensor],
                     n_heads: int, n_kv: int, head_dim: int, write_cache: bool) -> torch.Tensor:
    """The packed [q | k | v] rows of a prompt step, h @ w^T, with the rotation by `table` (pairs (i, i + half), the
    whole head) and the cache write in the product's epilogue: the queries' columns of the result are rotated, the
    keys' and values' columns are not written (they went to the cache; with `write_cache` false, nowhere).  The same
    bits as the plain product followed by `rope_cache_write`."""
    lib = _bind()
    _cuda(h, "activations")
    _cuda(w, "weights")
    if h.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("the tensor-core product takes bfloat16 operands")
    lda, ldw = _rows(h, "activations"), _rows(w, "weights")
    m, k = h.shape
    n, kw = w.shape
    if k != kw or n != (n_heads + 2 * n_kv) * head_dim:
        raise KernelError(f"q/k/v product: activations {tuple(h.shape)}, weights {tuple(w.shape)}, wanted {(n_heads + 2 * n_kv) * head_dim} rows of weights")
    if table.dtype != torch.float32 or not table.is_contiguous() or table.numel() != m * (head_dim // 2) * 2:
        raise KernelError("the table of angles must hold tokens x head_dim / 2 float32 (cos, sin) pairs")
    if write_cache:
        if kcache is None or vcache is None or block_table is None:
            raise KernelError("cache write without a cache")
        if kcache.dtype != torch.bfloat16 or vcache.dtype != torch.bfloat16:
            raise KernelError(f"the cache is {kcache.dtype}, the step runs in bfloat16")
        if tuple(kcache.shape[1:]) != (n_kv, 64, head_dim) or not kcache.is_contiguous() or not vcache.is_contiguous():
            raise KernelError(f"cache pages must be contiguous [pages, {n_kv}, 64, {head_dim}], got {tuple(kcache.shape)}")
    out = torch.empty((m, n), dtype=torch.bfloat16, device=h.device)
    _check(lib, lib.gi_gemm_tc_qkv_rope(
        out.data_ptr(), h.data_ptr(), w.data_ptr(), m, n, k, lda, ldw, _rows(out, "output"), table.data_ptr(),
        _i32(positions, "positions"), _i32(slots, "slots"), _i32(block_table, "block table"),
        block_table.shape[1] if block_table is not None else 0,
        kcache.data_ptr() if (write_cache and kcache is not None) else None,
        vcache.data_ptr() if (write_cache and vcache is not None) else None,
        n_heads, n_kv, head_dim, int(write_cache), _stream()))
    return out


def gemm_tc_tail_tiles(on: bool) -> None:
    """The tensor-core product cuts the columns of an unfilled last round of blocks into narrower tiles that fit one
    round (on by default); off, every tile has the full width.  Process-wide; for measurements and tests."""
    lib = _bind()
    lib.gi_gemm_tc_tail_tiles(int(bool(on)))


def gemm_tc_status() -> int:
    """0 if every wait inside the tensor-core product was met since the last call; synchronises the device."""
    lib = _bind()
    status = ctypes.c_int(0)
    _check(lib, lib.gi_gemm_tc_status(ctypes.byref(status)), 0)
    return status.value


def check_status() -> None:
    """Raises if any bounded wait inside the tensor-core kernels ran out since the last call (the kernel then left
    through its normal exit with its work undone: the results of that launch are not to be trusted).  Reads and
    clears the kernels' status words; synchronises the device."""
    bad = []
    for name, fn in (("prompt product", gemm_tc_status), ("decode product", gemm_stream_status),
                     ("prompt attention", attn_prefill_t5_status)):
        code = fn()
        if code:
            bad.append(f"{name} (wait {code})")
    if bad:
        raise KernelError("a wait inside a kernel ran out of tries: " + ", ".join(bad) + "; results since the last check are not to be trusted")


def _tc_out_ok(out: Optional[torch.Tensor], mode: int, cols: int) -> bool:
    """The tensor-core product stores 16 bytes at a time: output rows must start on 16-byte boundaries."""
    align = 8 if mode in (SKINNY_STORE_BF16, SKINNY_SWIGLU) else 4
    if out is None:
        return cols % align == 0
    return out.stride(1) == 1 and out.stride(0) % align == 0 and out.data_ptr() % 16 == 0


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """float32 [tokens, pairs, 2]: (cos, sin) of position * frequency, angles formed in 32-bit."""
    lib = _bind()
    _cuda(positions, "positions")
    if inv_freq.dtype != torch.float32 or not inv_freq.is_contiguous():
        raise KernelError("the rotary frequency table must be contiguous float32")
    n, half = positions.numel(), inv_freq.numel()
    table = torch.empty((n, half, 2), dtype=torch.float32, device=positions.device)
    _check(lib, lib.gi_rope_table(table.data_ptr(), _i32(positions, "positions"), inv_freq.data_ptr(), n, 2 * half, _stream()))
    return table


def rope_cache_write(qkv: torch.Tensor, table: Optional[torch.Tensor], positions: torch.Tensor, slots: torch.Tensor,
                     block_table: Optional[torch.Tensor], kcache: Optional[torch.Tensor],
                     vcache: Optional[torch.Tensor], n_heads: int, n_kv: int, head_dim: int,
                     rotary_dim: int, adjacent: bool, write_cache: bool) -> None:
    """Rotates the q and k parts of the packed rows by the angles of `table` (q in place, k into the cache)
    and copies v into the cache."""
    lib = _bind()
    _cuda(qkv, "q/k/v rows", settles=True)
    ld = _rows(qkv, "q/k/v rows")
    n = qkv.shape[0]
    if qkv.shape[1] != (n_heads + 2 * n_kv) * head_dim:
        raise KernelError(f"q/k/v rows are {qkv.shape[1]} wide, wanted {(n_heads + 2 * n_kv) * head_dim}")
    if rotary_dim:
        if table is None or table.dtype != torch.float32 or table.numel() != n * (rotary_dim // 2) * 2:
            raise KernelError("the table of angles must hold tokens x rotary_dim / 2 float32 (cos, sin) pairs")
    if write_cache:
        if kcache is None or vcache is None or block_table is None:
            raise KernelError("cache write without a cache")
        if kcache.dtype != qkv.dtype or vcache.dtype != qkv.dtype:
            raise KernelError(f"the cache is {kcache.dtype}, the step runs in {qkv.dtype}")
        if tuple(kcache.shape[1:]) != (n_kv, 64, head_dim) or not kcache.is_contiguous() or not vcache.is_contiguous():
            raise KernelError(f"cache pages must be contiguous [pages, {n_kv}, 64, {head_dim}], got {tuple(kcache.shape)}")
    max_pages = block_table.shape[1] if block_table is not None else 0
    args = (qkv.data_ptr(), _dt(qkv, "q/k/v rows"), ld, table.data_ptr() if table is not None else None,
            _i32(positions, "positions"), _i32(slots, "slots"), _i32(block_table, "block table"), max_pages,
            kcache.data_ptr() if kcache is not None else None, vcache.data_ptr() if vcache is not None else None,
            n, n_heads, n_kv, head_dim, rotary_dim, int(adjacent), int(write_cache))
    pending = _take_pending(qkv)
    if pending is not None:       # the product left partial sums instead of some of these rows' values
        if not pending[1]:
            raise KernelError("rope_cache_write met partial sums of an accumulating product")
        _check(lib, lib.gi_rope_cache_write_settle(*args, pending[0], _stream()))
    else:
        _check(lib, lib.gi_rope_cache_write(*args, _stream()))


def attn_prefill_generic(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_table: torch.Tensor,
                         cu_seqlens: torch.Tensor, seq_slots: torch.Tensor, seq_pos0: torch.Tensor, n_seqs: int,
                         max_q_len: int, n_heads: int, n_kv: int, head_dim: int, scale: float,
                         window: Optional[int], out: torch.Tensor) -> torch.Tensor:
    lib = _bind()
    _cuda(q, "queries")
    ldq, ldo = _rows(q, "queries"), _rows(out, "attention output")
    if kcache.dtype != q.dtype or out.dtype != q.dtype:
        raise KernelError("queries, cache and attention output must share a dtype")
    _check(lib, lib.gi_attn_prefill_generic(
        out.data_ptr(), ldo, q.data_ptr(), ldq, _dt(q, "queries"), kcache.data_ptr(), vcache.data_ptr(),
        _i32(block_table, "block table"), block_table.shape[1], _i32(cu_seqlens, "cu_seqlens"),
        _i32(seq_slots, "slots"), _i32(seq_pos0, "start positions"), n_seqs, max_q_len, n_heads, n_kv, head_dim,
        float(scale), int(window or 0), _stream()))
    return out


def attn_decode_generic(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_table: torch.Tensor,
                        seq_slots: torch.Tensor, seq_lens: torch.Tensor, n_seqs: int, n_heads: int, n_kv: int,
                        head_dim: int, scale: float, window: Optional[int], n_splits: int, out: torch.Tensor,
                        part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None,
                        own_tiles: int = 0) -> torch.Tensor:
    """`own_tiles` > 0: slice s of a sequence is tiles [s * own_tiles, (s + 1) * own_tiles) of its own span (32 keys a
    tile), whatever `n_splits` is, which must then cover the longest sequence; 0: every span is cut into `n_splits`
    equal slices."""
    lib = _bind()
    _cuda(q, "queries")
    ldq, ldo = _rows(q, "queries"), _rows(out, "attention output")
    if kcache.dtype != q.dtype or out.dtype != q.dtype:
        raise KernelError("queries, cache and attention output must share a dtype")
    if n_splits > 1:
        if part_o is None or part_ml is None:
            raise KernelError("attention slices need scratch memory")
        if part_o.dtype != torch.float32 or part_o.numel() < n_seqs * n_heads * n_splits * head_dim:
            raise KernelError("attention scratch for outputs is too small")
        if part_ml.dtype != torch.float32 or part_ml.numel() < n_seqs * n_heads * n_splits * 2:
            raise KernelError("attention scratch for maxima and sums is too small")
    _check(lib, lib.gi_attn_decode_generic(
        out.data_ptr(), ldo, part_o.data_ptr() if part_o is not None else None,
        part_ml.data_ptr() if part_ml is not None else None, q.data_ptr(), ldq, _dt(q, "queries"),
        kcache.data_ptr(), vcache.data_ptr(), _i32(block_table, "block table"), block_table.shape[1],
        _i32(seq_slots, "slots"), _i32(seq_lens, "lengths"), n_seqs, n_heads, n_kv, head_dim, float(scale),
        int(window or 0), int(n_splits), int(own_tiles), _stream()), 2 if n_splits > 1 else 1)
    return out


def attn_prefill_tc(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_table: torch.Tensor,
                    cu_seqlens: torch.Tensor, seq_slots: torch.Tensor, seq_pos0: torch.Tensor, n_seqs: int,
                    max_q_len: int, n_heads: int, n_kv: int, head_dim: int, scale: float,
                    window: Optional[int], out: torch.Tensor) -> torch.Tensor:
    """As attn_prefill_generic, for bfloat16 and head size 64 or 128, on tensor cores."""
    lib = _bind()
    _cuda(q, "queries")
    ldq, ldo = _rows(q, "queries"), _rows(out, "attention output")
    if q.dtype != torch.bfloat16 or kcache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("the tensor-core prefill attention takes bfloat16 queries, cache and output")
    _check(lib, lib.gi_attn_prefill_tc(
        out.data_ptr(), ldo, q.data_ptr(), ldq, kcache.data_ptr(), vcache.data_ptr(),
        _i32(block_table, "block table"), block_table.shape[1], _i32(cu_seqlens, "cu_seqlens"),
        _i32(seq_slots, "slots"), _i32(seq_pos0, "start positions"), n_seqs, max_q_len, n_heads, n_kv, head_dim,
        float(scale), int(window or 0), _stream()))
    return out


def attn_prefill_t5(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_table: torch.Tensor,
                    cu_seqlens: torch.Tensor, seq_slots: torch.Tensor, seq_pos0: torch.Tensor, n_seqs: int,
                    max_q_len: int, n_heads: int, n_kv: int, head_dim: int, scale: float,
                    window: Optional[int], out: torch.Tensor) -> torch.Tensor:
    """As attn_prefill_generic, for bfloat16 and head size 64 or 128, on tcgen05 tensor cores with TMA-fed operands.
    `q` is the whole packed [tokens, (H + 2 KV) * head_dim] matrix (its first columns are the queries)."""
    lib = _bind()
    _cuda(q, "queries")
    ldq, ldo = _rows(q, "queries"), _rows(out, "attention output")
    if q.dtype != torch.bfloat16 or kcache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("the tcgen05 prefill attention takes bfloat16 queries, cache and output")
    if not kcache.is_contiguous() or not vcache.is_contiguous() or q.shape[1] != (n_heads + 2 * n_kv) * head_dim:
        raise KernelError("the tcgen05 prefill attention takes the packed q/k/v rows and contiguous cache pages")
    _check(lib, lib.gi_attn_prefill_t5(
        out.data_ptr(), ldo, q.data_ptr(), ldq, q.shape[0], kcache.data_ptr(), vcache.data_ptr(), kcache.shape[0],
        _i32(block_table, "block table"), block_table.shape[1], _i32(cu_seqlens, "cu_seqlens"),
        _i32(seq_slots, "slots"), _i32(seq_pos0, "start positions"), n_seqs, max_q_len, n_heads, n_kv, head_dim,
        float(scale), int(window or 0), _stream()))
    return out


def attn_prefill_t5_pairing(mode: int) -> None:
    """Query tiles two to a block in the tcgen05 prompt attention: 0 never, 1 where the launch then is one round of
    blocks (the default), 2 always.  Process-wide; for measurements and tests."""
    _bind().gi_attn_prefill_t5_pairing(int(mode))


def attn_prefill_t5_status() -> int:
    lib = _bind()
    status = ctypes.c_int(0)
    _check(lib, lib.gi_attn_prefill_t5_status(ctypes.byref(status)), 0)
    return status.value


def attn_decode_tc_ok(q: torch.Tensor, kcache: torch.Tensor, head_dim: int) -> bool:
    """Whether the tensor-core decode attention takes these operands: bfloat16, head size 64 or 128, 16-byte rows."""
    return (q.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16 and head_dim in (64, 128)
            and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0)


_ATTN_COUNTERS = 1 << 16
_attn_counters: Dict[int, torch.Tensor] = {}


def _attn_merge_counters(device: torch.device) -> torch.Tensor:
    """Arrival counters of the decode attention's merge, one set per device, allocated once (their address is baked
    into recorded steps) and zero between launches (the kernel leaves them so)."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _attn_counters:
        _attn_counters[key] = torch.zeros(_ATTN_COUNTERS, dtype=torch.int32, device=device)
    return _attn_counters[key]


def attn_decode_tc(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_table: torch.Tensor,
                   seq_slots: torch.Tensor, seq_lens: torch.Tensor, n_seqs: int, n_heads: int, n_kv: int,
                   head_dim: int, scale: float, window: Optional[int], n_splits: int, out: torch.Tensor,
                   part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None,
                   tile_keys: Optional[int] = None, own_tiles: int = 0, merge_inside: Optional[bool] = None,
                   stages: Optional[int] = None, rope: Optional[Tuple[torch.Tensor, int]] = None) -> torch.Tensor:
    """`tile_keys`: 32 (one block per SM, deep rings) or 16 (two blocks per SM); default TUNE["attn_tile_keys"].
    `own_tiles` > 0: slices of that many tiles of each sequence's own span (`n_splits` must then cover the longest
    sequence); 0: every span is cut into `n_splits` equal slices.  `merge_inside`: the slices are merged by the block
    that finishes last instead of by a second kernel (default TUNE["attn_merge_inside"]).
    `rope` = (table of angles [sequences, pairs, 2], rotary size): `q` holds the packed [q | k | v] rows as the
    product left them (partial sums may be pending); the kernel rotates q and k by the table, pairs (i, i + half),
    and stores k and v at each sequence's newest position itself, instead of `rope_cache_write` before it."""
    lib = _bind()
    _cuda(q, "queries", settles=rope is not None)
    ldq, ldo = _rows(q, "queries"), _rows(out, "attention output")
    if q.dtype != torch.bfloat16 or kcache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("the tensor-core decode attention takes bfloat16 queries, cache and output")
    if n_splits > 1:
        if part_o is None or part_ml is None:
            raise KernelError("attention slices need scratch memory")
        if part_o.dtype != torch.float32 or part_o.numel() < n_seqs * n_heads * n_splits * head_dim:
            raise KernelError("attention scratch for outputs is too small")
        if part_ml.dtype != torch.float32 or part_ml.numel() < n_seqs * n_heads * n_splits * 2:
            raise KernelError("attention scratch for maxima and sums is too small")
    tile_keys = int(tile_keys or TUNE["attn_tile_keys"])
    if own_tiles and n_splits * own_tiles * tile_keys < 1:
        raise KernelError("attention: slices of no keys")
    chunks = (n_heads // max(1, n_kv) + 15) // 16
    inside = TUNE["attn_merge_inside"] if merge_inside is None else merge_inside
    counters = None
    if inside and n_splits > 1 and n_seqs * n_kv * chunks <= _ATTN_COUNTERS:
        counters = _attn_merge_counters(q.device)
    args = (out.data_ptr(), ldo, part_o.data_ptr() if part_o is not None else None,
            part_ml.data_ptr() if part_ml is not None else None,
            counters.data_ptr() if counters is not None else None, counters.numel() if counters is not None else 0,
            q.data_ptr(), ldq, kcache.data_ptr(), vcache.data_ptr(),
            _i32(block_table, "block table"), block_table.shape[1], _i32(seq_slots, "slots"), _i32(seq_lens, "lengths"),
            n_seqs, n_heads, n_kv, head_dim, float(scale), int(window or 0), int(n_splits), int(own_tiles),
            tile_keys, int(stages if stages is not None else attn_decode_stages(head_dim)))
    n_launches = 2 if (n_splits > 1 and counters is None) else 1
    if rope is None and counters is None and TUNE["attn_keys_on_rows"] and n_heads // max(1, n_kv) <= 8:
        # the keys of a tile on the rows of the products, up to 8 heads on their columns (a wider group would need
        # two blocks that read the same keys: it keeps the kernel with 16 heads on the rows)
        return attn_decode_kr(q, kcache, vcache, block_table, seq_slots, seq_lens, n_seqs, n_heads, n_kv, head_dim, scale,
                              window, n_splits, out, part_o, part_ml, own_tiles=own_tiles)
    if rope is None:
        _check(lib, lib.gi_attn_decode_tc_merged(*args, _stream()), n_launches)
        return out
    table, rotary_dim = rope
    if q.shape[0] < n_seqs or q.shape[1] != (n_heads + 2 * n_kv) * head_dim:
        raise KernelError(f"q/k/v rows are {tuple(q.shape)}, wanted {n_seqs} rows of {(n_heads + 2 * n_kv) * head_dim}")
    if table.dtype != torch.float32 or not table.is_contiguous() or table.numel() != q.shape[0] * (rotary_dim // 2) * 2:
        raise KernelError("the table of angles must hold rows x rotary_dim / 2 float32 (cos, sin) pairs")
    if tuple(kcache.shape[1:]) != (n_kv, 64, head_dim) or not kcache.is_contiguous() or not vcache.is_contiguous():
        raise KernelError(f"cache pages must be contiguous [pages, {n_kv}, 64, {head_dim}], got {tuple(kcache.shape)}")
    pending = _take_pending(q)
    if pending is not None and not pending[1]:
        raise KernelError("the decode attention met partial sums of an accumulating product")
    settle_t = pending[0] if pending is not None else SettleT(None, None, None, None, 0)
    _check(lib, lib.gi_attn_decode_tc_rope(*args, table.data_ptr(), int(rotary_dim), settle_t, _stream()), n_launches)
    return out


def sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float,
           rng_state: Optional[torch.Tensor] = None, state_index: Optional[torch.Tensor] = None,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of `logits` (float32).  temperature <= 0: the highest logit, first on ties."""
    lib = _bind()
    _cuda(logits, "logits")
    if logits.dtype != torch.float32:
        raise KernelError("logits must be float32")
    ld = _rows(logits, "logits")
    n, vocab = logits.shape
    if out is None:
        out = torch.empty((n,), dtype=torch.int32, device=logits.device)
    if rng_state is not None:
        if rng_state.dtype != torch.int64 or not rng_state.is_contiguous():
            raise KernelError("generator states must be a contiguous int64 tensor")
        _cuda(rng_state, "generator states")
    _check(lib, lib.gi_sample(out.data_ptr(), logits.data_ptr(), ld, n, vocab, float(temperature), int(top_k),
                              float(top_p), rng_state.data_ptr() if rng_state is not None else None,
                              _i32(state_index, "state index"), _stream()))
    return out


# ------------------------------------------------------------------------------------------------
# Dispatchers: the one place where a kernel is chosen for an operation.
def linear(h: torch.Tensor, w: torch.Tensor, *, out: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None, accumulate: bool = False) -> torch.Tensor:
    want = out.dtype if out is not None else (out_dtype or h.dtype)
    if accumulate and out is not None and not (skinny_ok(h, w) and USE_STREAM):
        settle(out)
    mode = SKINNY_ACCUM_F32 if accumulate else {torch.bfloat16: SKINNY_STORE_BF16, torch.float32: SKINNY_STORE_F32}.get(want)
    if mode is not None:
        if skinny_ok(h, w):
            return _decode_product(h, w, mode, out)
        if tc_ok(h, w) and _tc_out_ok(out, mode, w.shape[0]):
            return gemm_tc(h, w, mode, out)
    return gemm_generic(h, w, out=out, out_dtype=out_dtype, accumulate=accumulate)


def swiglu_interleaved(h: torch.Tensor, w_interleaved: torch.Tensor) -> torch.Tensor:
    """silu(Wgate h) * (Wup h) where `w_interleaved` holds gate and up rows in blocks [8 gate | 8 up]."""
    if skinny_ok(h, w_interleaved):
        return _decode_product(h, w_interleaved, SKINNY_SWIGLU, None)
    if tc_ok(h, w_interleaved) and w_interleaved.shape[0] % 16 == 0:
        return gemm_tc(h, w_interleaved, SKINNY_SWIGLU)
    gu = linear(h, w_interleaved, out_dtype=h.dtype)
    return silu_mul(gu, interleaved=True)


def attn_decode_stages(head_dim: int) -> int:
    """Depth of each warp's ring of key/value tiles in the tensor-core decode attention."""
    return int(TUNE["attn_stages_hd64"] if head_dim == 64 else TUNE["attn_stages_hd128"])


def attn_decode_blocks_per_sm(head_dim: int, fast: bool) -> float:
    """How many blocks of the decode attention one SM holds (its shared memory decides: a block's rings of key and
    value tiles are 96 KB at head size 128 and 64 KB at head size 64 with 16-key tiles), times TUNE["attn_waves"]:
    the slice count fills that many places once."""
    if not fast:
        per_sm = 2
    elif TUNE["attn_keys_on_rows"]:
        # the kernel with a tile's keys on the rows of its products: 8 rows of queries, and each warp's ring of
        # `stages` x (16 keys + 16 values); 80 registers a thread at head size 64, up to 127 at 128
        warps, stages = int(TUNE["attn_kr_warps"]), int(TUNE["attn_kr_stages"])
        smem = 8 * head_dim * 2 + warps * stages * 2 * 16 * head_dim * 2 + 1152
        regs = 65536 // (warps * 32 * (80 if head_dim == 64 else 128))
        per_sm = max(1, min(regs, (227 * 1024) // smem))
    elif TUNE["attn_tile_keys"] == 16:
        # a block's shared memory: 16 rows of queries, and four warps' rings of `stages` x (16 keys + 16 values)
        smem = 16 * head_dim * 2 + 4 * attn_decode_stages(head_dim) * 2 * 16 * head_dim * 2 + 1152
        regs = 4 if head_dim == 64 else 3          # blocks per SM that the registers allow (121 and 168 a thread)
        per_sm = min(regs, (227 * 1024) // smem)
    else:
        per_sm = 1
    return per_sm * TUNE["attn_waves"]


OWN_LENGTH_TILES = 8      # 32-bit decode attention: a slice is this many 32-key tiles of the sequence's own span


def attn_decode_plan(n_seqs: int, max_kv_len: int, sm_count: int, n_heads: int, n_kv: int, head_dim: int,
                     window: Optional[int], dtype: torch.dtype, kv_lens=None):
    """How the decode attention cuts contexts into slices, as (slices in the launch, tiles per slice).

    bfloat16, few sequences: tiles per slice 0 = every sequence is cut into the same number of slices, as many as
    fill the GPU once (blocks that wait for a second round cost more than longer slices), at least 256 positions of the
    longest sequence's present length each (measured at batch 1 to 4 of the 8B shape with 2,048 cached positions: 8
    slices beat 16 and 4, and 32, which the length bucket's upper end alone would allow, cost 3.5 % of the step).
    bfloat16, so many sequences that one slice each fills more than half the GPU, and their lengths (`kv_lens`) known:
    slices of a fixed number of tiles of each sequence's own span, the shortest for which all blocks still find a
    place at once; long sequences are then cut and short ones are not, so that no block is much longer than the rest.
    float32: slices of a fixed length counted from the start of the sequence's own span, so that a sequence's
    sums are formed in the same order whatever else the step holds (the reference sizes its slices from the
    token's own span for the same reason, src/cuda.rs:1639-1644, :8432-8437); the launch holds as many slices as
    the longest sequence needs, and shorter ones leave theirs empty."""
    if dtype == torch.float32:
        span = max_kv_len if not window else min(max_kv_len, int(window) + 31)
        tiles = (span + 31) // 32 + (1 if window else 0)
        return max(1, (tiles + OWN_LENGTH_TILES - 1) // OWN_LENGTH_TILES), OWN_LENGTH_TILES
    fast = dtype == torch.bfloat16 and head_dim in (64, 128)
    # heads of a group that one block takes: 16 in the tensor-core kernels (groups of more than 8 heads go to the one
    # that has the heads on the rows of its tile), 8 in the plain kernel
    rows_per_block = 16 if fast else 8
    group = n_heads // n_kv
    chunks = (group + rows_per_block - 1) // rows_per_block
    blocks = max(1, n_seqs * n_kv * chunks)
    places = int(attn_decode_blocks_per_sm(head_dim, fast) * sm_count)
    if 2 * blocks <= places or not fast:
        # slices of at least TUNE["attn_min_slice"] positions of the longest sequence as it is now (a plan is kept while
        # the sequences grow to the end of their length bucket, up to twice as long)
        longest = max_kv_len if not kv_lens else min(max_kv_len, max(int(n) for n in kv_lens))
        return int(max(1, min(places // blocks, 32, longest // int(TUNE["attn_min_slice"])))), 0
    if kv_lens is not None and TUNE["attn_own_slices"] and blocks < places:
        tile = int(TUNE["attn_tile_keys"])
        span = (lambda n: n) if not window else (lambda n: min(n, int(window) + 2 * tile))
        # the lengths a little ahead of now: the plan is kept while the sequences grow
        lens = [span(min(int(n) + 64, max_kv_len)) for n in kv_lens]
        idle = max(0, n_seqs - len(lens))                    # padding rows: one tile each
        longest = span(max_kv_len)
        unit = max(1, 256 // tile)
        own = unit
        while own * tile < longest:
            need = (sum((n + own * tile - 1) // (own * tile) for n in lens) + idle) * n_kv * chunks
            if need <= places:
                return max(1, (longest + own * tile - 1) // (own * tile)), own
            own += unit
    return 1, 0


def attn_decode_kr(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_table: torch.Tensor,
                   seq_slots: torch.Tensor, seq_lens: torch.Tensor, n_seqs: int, n_heads: int, n_kv: int,
                   head_dim: int, scale: float, window: Optional[int], n_splits: int, out: torch.Tensor,
                   part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None, own_tiles: int = 0,
                   warps: Optional[int] = None, stages: Optional[int] = None) -> torch.Tensor:
    """The tensor-core decode attention with a tile's 16 keys on the rows of its products and up to 8 heads of a group on
    their columns (wider groups take several blocks per kv head).  Same operands and scratch as `attn_decode_tc`;
    `warps` per block (4, 6 or 8) and `stages` of each warp's ring (2 or 3) default to TUNE's."""
    lib = _bind()
    _cuda(q, "queries")
    ldq, ldo = _rows(q, "queries"), _rows(out, "attention output")
    if q.dtype != torch.bfloat16 or kcache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("the tensor-core decode attention takes bfloat16 queries, cache and output")
    if n_splits > 1:
        if part_o is None or part_ml is None:
            raise KernelError("attention slices need scratch memory")
        if part_o.dtype != torch.float32 or part_o.numel() < n_seqs * n_heads * n_splits * head_dim:
            raise KernelError("attention scratch for outputs is too small")
        if part_ml.dtype != torch.float32 or part_ml.numel() < n_seqs * n_heads * n_splits * 2:
            raise KernelError("attention scratch for maxima and sums is too small")
    _check(lib, lib.gi_attn_decode_kr(
        out.data_ptr(), ldo, part_o.data_ptr() if part_o is not None else None,
        part_ml.data_ptr() if part_ml is not None else None, q.data_ptr(), ldq, kcache.data_ptr(), vcache.data_ptr(),
        _i32(block_table, "block table"), block_table.shape[1], _i32(seq_slots, "slots"), _i32(seq_lens, "lengths"),
        n_seqs, n_heads, n_kv, head_dim, float(scale), int(window or 0), int(n_splits), int(own_tiles),
        int(warps or TUNE["attn_kr_warps"]), int(stages or TUNE["attn_kr_stages"]), _stream()), 2 if n_splits > 1 else 1)
    return out


def attn_rope_inside_ok(qkv: torch.Tensor, memory, step, head_dim: int) -> bool:
    """Whether a step's rotation and cache write can be left to its attention kernel (`attention(..., rope=)`): a
    decode step on the tensor-core kernel that writes its own cache."""
    return bool(TUNE["attn_rope_inside"] and step.is_decode and memory.k is not None and memory.writes
                and attn_decode_tc_ok(qkv, memory.k, head_dim) and qkv.shape[0] == step.n_seqs)


def attention(qkv: torch.Tensor, memory, step, n_heads: int, n_kv: int, head_dim: int, scale: float,
              window: Optional[int], out: torch.Tensor, plan=None, rope=None) -> torch.Tensor:
    """Attention of a step's tokens over the cache (which already holds the step's own keys and values).
    The queries are the first n_heads * head_dim columns of the packed rows `qkv`.  `plan`: what
    `attn_decode_plan` gave for a decode step (worked out here when absent).  `rope` = (table, rotary size), only
    where `attn_rope_inside_ok` holds: the rows are not rotated and the cache lacks the step's keys and values;
    the kernel does both."""
    if memory.k is None:
        raise KernelError("attention needs a cache to read from")
    if rope is not None and not attn_rope_inside_ok(qkv, memory, step, head_dim):
        raise KernelError("this step's attention cannot rotate and store by itself")
    if step.is_decode:
        fast = attn_decode_tc_ok(qkv, memory.k, head_dim)
        if plan is None:
            plan = attn_decode_plan(step.n_seqs, step.max_kv_len, step.sm_count, n_heads, n_kv, head_dim, window, qkv.dtype)
        n_splits, own_tiles = plan
        part_o = part_ml = None
        if n_splits > 1:
            part_o = torch.empty((step.n_seqs * n_heads * n_splits * head_dim,), dtype=torch.float32, device=qkv.device)
            part_ml = torch.empty((step.n_seqs * n_heads * n_splits * 2,), dtype=torch.float32, device=qkv.device)
        if fast:
            return attn_decode_tc(qkv, memory.k, memory.v, memory.block_table, step.seq_slots, step.seq_lens,
                                  step.n_seqs, n_heads, n_kv, head_dim, scale, window, n_splits, out, part_o, part_ml,
                                  own_tiles=own_tiles, rope=rope)
        return attn_decode_generic(qkv, memory.k, memory.v, memory.block_table, step.seq_slots, step.seq_lens,
                                   step.n_seqs, n_heads, n_kv, head_dim, scale, window, n_splits, out, part_o, part_ml,
                                   own_tiles=own_tiles)
    if attn_decode_tc_ok(qkv, memory.k, head_dim) and out.stride(0) % 2 == 0:
        # tcgen05 (scores and output in tensor memory); mma.sync when that is switched off or the rows do not suit TMA
        t5 = (TUNE["attn_prefill_tcgen05"] and head_dim in (64, 128) and out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0
              and qkv.shape[1] == (n_heads + 2 * n_kv) * head_dim and memory.k.is_contiguous())
        kernel = attn_prefill_t5 if t5 else attn_prefill_tc
    else:
        kernel = attn_prefill_generic
    return kernel(qkv, memory.k, memory.v, memory.block_table, step.cu_seqlens, step.seq_slots,
                  step.seq_pos0, step.n_seqs, step.max_q_len, n_heads, n_kv, head_dim, scale, window, out)
