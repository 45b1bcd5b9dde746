"""Python face of the kernel library: loads the shared library that
`csrc/build.py` builds and wraps each C entry point in a function that takes
torch tensors (as storage only: pointers, shapes and dtypes are read, no torch
operator runs).  Kernels launch on torch's current CUDA stream, so they order with
torch's allocator and can be captured into CUDA graphs.

There is no fallback: without the library, or on a device that is not sm_100,
every call raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_void_p, c_int, c_float, c_longlong, c_char_p
from typing import Optional

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    pass


_lib = None


def lib():
    """The loaded library (built at the first call if needed)."""
    global _lib
    if _lib is None:
        path = _build.ensure_built()
        try:
            _lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load the kernel library {path}: {e}") from None
        _lib.rb_last_error.restype = c_char_p
        if _lib.rb_abi_version() != 1:
            raise KernelError("kernel library has another ABI version")
        if os.environ.get("REINFER_B200_GEMM_SCHEDULE"):
            # 0: one CTA per tile, 1: persistent CTAs (default) for prompt portions
            _lib.rb_set_gemm_persistent(int(os.environ["REINFER_B200_GEMM_SCHEDULE"]))
        if os.environ.get("REINFER_B200_GEMM_TOKEN_LANES"):
            # prompt portions: 1 a token per accumulator lane (default), 0 a feature per lane
            _lib.rb_set_gemm_token_lanes(int(os.environ["REINFER_B200_GEMM_TOKEN_LANES"]))
        if os.environ.get("REINFER_B200_GEMM_GATED_STREAM"):
            # the gated pair over 65 .. 128 tokens: 1 the streaming kernel with a token per lane (default), 0 a feature per lane
            _lib.rb_set_gemm_gated_stream(int(os.environ["REINFER_B200_GEMM_GATED_STREAM"]))
        if os.environ.get("REINFER_B200_GEMM_TILE_ROWS"):
            # prompt portions: 256 or 224 weight rows a tile; default chosen per product
            _lib.rb_set_gemm_tile_features(int(os.environ["REINFER_B200_GEMM_TILE_ROWS"]))
        if os.environ.get("REINFER_B200_PDL", "1") == "0":
            _lib.rb_set_pdl(0)          # launch every kernel fully serialised (for comparisons)
    return _lib


_checked_device = False


def require_device() -> None:
    """Fail loudly unless a CUDA device of compute capability 10.x is current."""
    global _checked_device
    if _checked_device:
        return
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device: reinfer_b200 runs on a B200 (sm_100a) only and has no CPU path")
    cc = lib().rb_device_cc()
    if cc < 0:
        raise KernelError(f"CUDA error {-cc} while reading the device's compute capability")
    if cc // 10 != 10:
        raise KernelError(f"device has compute capability {cc / 10:.1f}; the kernels are built for sm_100a only")
    _checked_device = True


launches = 0          # kernels of this library launched so far (every wrapper passes through _check)


class SegmentProfiler:
    """CUDA-event times of the launches of a step, by named segment (the idea of the reference's DecodeProfiler
    and PrefillProfiler: cudaEvent pairs around named segments, crates/cuda/src/engine.rs:928-1408, 6675-6975).
    While a profiler is installed (`set_profiler`) every wrapper records an event behind its launch; a launch's
    time is the span from the event before it to its own, so the launches are seen one after the other, without
    the overlap that programmatic dependent launch gives them in a plain run: compare shares, as with a profiler.
    Each wrapper also says what the launch has to compute and to move, which gives achieved FLOP/s and bytes/s."""

    def __init__(self) -> None:
        self.marks = []                                     # (name, flops, bytes, event)
        self.start = None

    def begin(self) -> None:
        self.marks = []
        self.start = torch.cuda.Event(enable_timing=True)
        self.start.record()

    def mark(self, name: str, flops: float, nbytes: float) -> None:
        if self.start is None:
            return
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self.marks.append((name, flops, nbytes, ev))

    def summary(self):
        """name -> {"n", "us", "tflops", "gbs"} (synchronises); insertion order = order of first launch."""
        torch.cuda.synchronize()
        out, prev = {}, self.start
        for name, flops, nbytes, ev in self.marks:
            us = prev.elapsed_time(ev) * 1e3
            prev = ev
            d = out.setdefault(name, {"n": 0, "us": 0.0, "flops": 0.0, "bytes": 0.0})
            d["n"] += 1; d["us"] += us; d["flops"] += flops; d["bytes"] += nbytes
        for d in out.values():
            t = max(d["us"], 1e-9) * 1e-6
            d["tflops"] = d.pop("flops") / t / 1e12
            d["gbs"] = d.pop("bytes") / t / 1e9
        return out


_profiler: Optional["SegmentProfiler"] = None


def set_profiler(p: Optional["SegmentProfiler"]) -> Optional["SegmentProfiler"]:
    """Install (or, with None, remove) the profiler that the wrappers report to; returns the previous one."""
    global _profiler
    old, _profiler = _profiler, p
    return old


def _check(rc: int, what: str, flops: float = 0.0, nbytes: float = 0.0) -> None:
    global launches
    launches += 1
    if _profiler is not None and rc == 0:
        _profiler.mark(what, flops, nbytes)
    if rc == 0:
        return
    if rc < 0:
        raise KernelError(f"{what}: {lib().rb_last_error().decode()}")
    raise KernelError(f"{what}: CUDA error {rc} at launch")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> c_void_p:
    """torch's current stream as a raw handle (by torch's own short way where it has one: a step makes hundreds of
    launches and each asks)."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} is not float32 or bfloat16") from None


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


# ------------------------------------------------------------------ wrappers
def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, slot_token: Optional[torch.Tensor] = None,
                 entry_slot: Optional[torch.Tensor] = None, tok_entry: Optional[torch.Tensor] = None,
                 pos_table: Optional[torch.Tensor] = None, positions: Optional[torch.Tensor] = None,
                 scale: float = 1.0, rounded: Optional[torch.Tensor] = None) -> None:
    """out[t,:] (float32) = table[ids[t],:]; where ids[t] < 0 and the slot tables are given, the id is
    slot_token[entry_slot[tok_entry[t]]]: the token that the sampler left in the request's slot.  With a table of
    learned position vectors (the embedding table's dtype) the row pos_table[positions[t]] is added.  `scale`
    multiplies the rows; `rounded` (bfloat16, out's shape) receives them once more, rounded."""
    _need(out.dtype == torch.float32 and ids.dtype == torch.int32, "embed_gather: out float32, ids int32")
    _need(table.is_contiguous() and out.is_contiguous(), "embed_gather: contiguous tensors")
    _need(rounded is None or (rounded.dtype == torch.bfloat16 and rounded.is_contiguous() and rounded.shape == out.shape),
          "embed_gather: the rounded copy is bfloat16 of out's shape")
    if pos_table is not None:
        _need(pos_table.dtype == table.dtype and pos_table.is_contiguous() and pos_table.shape[1] == table.shape[1] and
              positions is not None, "embed_gather: a position table of the embedding's dtype and width, with positions")
    _check(lib().rb_embed_gather(_p(table), dt(table), _p(ids), _p(slot_token), _p(entry_slot), _p(tok_entry), _p(out),
                                 c_int(ids.numel()), c_int(table.shape[1]), c_int(table.shape[0]),
                                 _p(pos_table), _p(positions if pos_table is not None else None),
                                 c_int(pos_table.shape[0] if pos_table is not None else 0), c_float(float(scale)),
                                 _p(rounded), _stream()), "embed_gather")


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], w: torch.Tensor, out: torch.Tensor,
                eps: float, row_idx: Optional[torch.Tensor] = None) -> None:
    """x (float32, [rows,h]) += delta if given; out[r] = rmsnorm(x[row_idx[r] or r]) * w.
    delta has x's shape, or one more leading dimension: partial sums [S, rows, h] that are added in
    ascending order (what a split product leaves).  With row_idx the sum is formed for the gathered
    rows only and x itself is left unchanged."""
    _need(x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous(), "rmsnorm: x float32 contiguous")
    h = x.shape[-1]
    rows = out.numel() // h
    n_delta = 0
    if delta is not None:
        _need(delta.is_contiguous() and delta.numel() % x.numel() == 0 and delta.shape[-1] == h, "rmsnorm: delta has x's shape (or a stack of it)")
        n_delta = delta.numel() // x.numel()
    _check(lib().rb_add_rmsnorm(_p(x), _p(delta), c_int(dt(delta) if delta is not None else F32), c_int(n_delta),
                                c_longlong(x.numel()), _p(w), c_int(dt(w)),
                                _p(out), c_int(dt(out)), _p(row_idx), c_int(rows), c_int(h), c_float(eps),
                                _stream()), "add_rmsnorm")


def residual_rowscale(x: torch.Tensor, delta: Optional[torch.Tensor], w: torch.Tensor):
    """x (float32 [rows,h]) += delta (x's shape, or a stack of partial sums added in ascending order); returns
    (y, sumsq): y = bfloat16(x * w) and sumsq [rows, parts] float32, the sum of x^2 by chunks of columns.  The
    product that reads y multiplies its results for row r by 1/sqrt(sum(sumsq[r]) / h + eps): the RMS norm with
    its division moved behind the product (gemm_bf16(..., row_scale=(sumsq, h, eps)))."""
    _need(x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 2, "rowscale: x float32 [rows,h] contiguous")
    rows, h = x.shape
    n_delta = 0
    if delta is not None:
        _need(delta.dtype == torch.float32 and delta.is_contiguous() and delta.numel() % x.numel() == 0 and delta.shape[-1] == h,
              "rowscale: delta float32 with x's shape (or a stack of it)")
        n_delta = delta.numel() // x.numel()
    parts = int(lib().rb_rowscale_parts(c_int(h)))
    y = torch.empty((rows, h), dtype=torch.bfloat16, device=x.device)
    sumsq = torch.empty((rows, parts), dtype=torch.float32, device=x.device)
    _check(lib().rb_residual_rowscale(_p(x), _p(delta), c_int(n_delta), c_longlong(x.numel()), _p(w), c_int(dt(w)),
                                      _p(y), _p(sumsq), c_int(rows), c_int(h), _stream()), "residual_rowscale")
    return y, sumsq


def residual_add(x: torch.Tensor, delta: torch.Tensor) -> None:
    _need(x.dtype == torch.float32 and x.is_contiguous() and delta.is_contiguous() and x.numel() == delta.numel(),
          "residual_add: x float32, same size")
    _check(lib().rb_residual_add(_p(x), _p(delta), c_int(dt(delta)), c_longlong(x.numel()), _stream()), "residual_add")


def qknorm_rope_append(qkv: torch.Tensor, qw: Optional[torch.Tensor], kw: Optional[torch.Tensor],
                       inv_freq: Optional[torch.Tensor], positions: Optional[torch.Tensor],
                       kv_slot: Optional[torch.Tensor], q_out: torch.Tensor, cache: Optional[torch.Tensor],
                       QH: int, KH: int, d: int, rot: int, page_size: int, eps: float,
                       k_out: Optional[torch.Tensor] = None, cs_table: Optional[torch.Tensor] = None) -> None:
    """Per-head RMSNorm of q and k (if weights are given), rotation of the first `rot` dims (if
    rot > 0), q -> q_out, k and v -> the cache at kv_slot (or k -> k_out, v untouched)."""
    n = qkv.shape[0]
    _need(qkv.is_contiguous() and q_out.is_contiguous(), "qknorm_rope_append: contiguous")
    _need(qkv.shape[-1] == (QH + 2 * KH) * d, "qknorm_rope_append: qkv width")
    wd = dt(qw) if qw is not None else F32
    if qw is not None:
        _need(kw is not None and kw.dtype == qw.dtype, "qknorm_rope_append: q/k norm weights of one dtype")
    _check(lib().rb_qknorm_rope_append(_p(qkv), c_int(dt(qkv)), _p(qw), _p(kw), c_int(wd), _p(inv_freq), _p(cs_table),
                                       _p(positions), _p(kv_slot), _p(q_out), _p(k_out), _p(cache),
                                       c_int(dt(cache) if cache is not None else dt(qkv)),
                                       c_int(n), c_int(QH), c_int(KH), c_int(d), c_int(rot), c_int(page_size),
                                       c_float(eps), _stream()), "qknorm_rope_append")


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """(cos, sin) of positions[t] * inv_freq[p] as float32 [T, half, 2]: computed once per step, read by every layer."""
    T, half = positions.numel(), inv_freq.numel()
    cs = torch.empty((T, half, 2), dtype=torch.float32, device=positions.device)
    _check(lib().rb_rope_table(_p(positions), _p(inv_freq), _p(cs), c_int(T), c_int(half), _stream()), "rope_table")
    return cs


def kv_append(k: torch.Tensor, v: torch.Tensor, kv_slot: torch.Tensor, cache: torch.Tensor,
              KH: int, d: int, page_size: int) -> None:
    """k, v: [T, KH*d] views (row stride free, heads contiguous) -> cache pages."""
    _need(k.dtype == v.dtype == cache.dtype, "kv_append: one dtype")
    _need(k.stride(-1) == 1 and v.stride(-1) == 1, "kv_append: rows contiguous")
    _check(lib().rb_kv_append(_p(k), c_longlong(k.stride(0)), _p(v), c_longlong(v.stride(0)), _p(kv_slot), _p(cache),
                              c_int(dt(k)), c_int(k.shape[0]), c_int(KH), c_int(d), c_int(page_size), _stream()),
           "kv_append")


def swiglu(gu: torch.Tensor, out: torch.Tensor) -> None:
    _need(gu.is_contiguous() and out.is_contiguous() and gu.dtype == out.dtype, "swiglu: contiguous, one dtype")
    F_ = out.shape[-1]
    _need(gu.shape[-1] == 2 * F_, "swiglu: input is [gate | up]")
    _check(lib().rb_swiglu(_p(gu), _p(out), c_int(dt(gu)), c_int(out.numel() // F_), c_int(F_), _stream()), "swiglu")


def gemm_ref(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, accumulate: bool = False) -> None:
    """c[M,N] (=|+=) a[M,K] @ w[N,K]^T on the CUDA cores in 32-bit."""
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and tuple(c.shape) == (M, N), "gemm: shapes")
    _need(a.stride(1) == 1 and w.stride(1) == 1 and c.stride(1) == 1, "gemm: rows contiguous")
    _check(lib().rb_gemm_ref(_p(a), c_int(dt(a)), _p(w), c_int(dt(w)), _p(c), c_int(dt(c)), c_int(int(accumulate)),
                             c_int(M), c_int(N), c_int(K), c_longlong(a.stride(0)), c_longlong(w.stride(0)),
                             c_longlong(c.stride(0)), _stream()), f"gemm_fma {N}x{K}", 2.0 * M * N * K,
           float(M * K * a.element_size() + N * K * w.element_size() + M * N * c.element_size()))


def paged_attention_ref(q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, tok_row: torch.Tensor,
                        positions: torch.Tensor, out: torch.Tensor, QH: int, KH: int, d: int, page_size: int,
                        window: int, scale: float, work=(0.0, 0.0), dv: int = 0, chunk: int = 0,
                        penalty=None, out_scale: float = 1.0, bias: Optional[torch.Tensor] = None,
                        more: Optional["AttentionExtras"] = None) -> None:
    """The plain attention over the paged cache.  dv: the value heads' size where it differs from d (the cache of a
    layer is then [page][K: KH x page x d | V: KH x page x dv]); chunk: a token sees only the keys of its own chunk
    of that many positions; penalty = (r1, r2), float32 [QH] each: score -= r1 ln(1 + r2 (i - j)); out_scale
    multiplies the output before it is rounded; bias: float32 [QH, rows], score += bias[h, min(i - j, rows - 1)];
    more: soft cap, sink, values inside the keys and output gate (AttentionExtras)."""
    _need(q.is_contiguous() and out.is_contiguous() and cache.is_contiguous() and block_table.is_contiguous(),
          "attention: contiguous")
    _need(q.dtype == cache.dtype == out.dtype, "attention: one dtype for q, cache and out")
    r1 = r2 = None
    if penalty is not None:
        r1, r2 = penalty
        _need(r1.dtype == torch.float32 and r2.dtype == torch.float32 and r1.numel() == QH and r2.numel() == QH,
              "attention: the distance penalty is two float32 vectors, one number per query head each")
    _check(lib().rb_paged_attention_ref(_p(q), _p(cache), c_int(dt(q)), _p(block_table), _p(tok_row), _p(positions),
                                        _p(out), c_int(q.shape[0]), c_int(QH), c_int(KH), c_int(d), c_int(page_size),
                                        c_int(block_table.shape[1]), c_int(window), c_float(scale), c_int(dv), c_int(chunk),
                                        _p(r1), _p(r2), c_float(out_scale), *_bias_args(bias, QH),
                                        *(more or _NO_EXTRAS).flat(QH, dv or d), _stream()),
           "paged_attention_ref", *work)


class _FaMore(ctypes.Structure):
    _fields_ = [("softcap", c_float), ("sink", c_void_p), ("v_in_k", c_int), ("gate", c_void_p), ("gate_stride", c_longlong)]


class AttentionExtras:
    """Options of the attention kernels beyond mask, penalty and bias: `softcap` > 0 squashes the scaled scores to
    cap * tanh(score / cap); `sink` (float32 [QH]) joins each head's softmax denominator as exp(sink[h]) without a
    value; `v_in_k`: the values are the first dv columns of the key rows and the pages hold keys only; `gate` (float32
    rows [T, >= QH * dv], rows contiguous inside): the output is multiplied by sigmoid(gate[t, h * dv + i])."""

    def __init__(self, softcap: float = 0.0, sink: Optional[torch.Tensor] = None, v_in_k: bool = False,
                 gate: Optional[torch.Tensor] = None):
        self.softcap, self.sink, self.v_in_k, self.gate = float(softcap or 0.0), sink, bool(v_in_k), gate

    def check(self, QH: int, dv: int) -> None:
        _need(self.sink is None or (self.sink.dtype == torch.float32 and self.sink.is_contiguous() and self.sink.numel() == QH),
              "attention: the sink is one float32 number per query head")
        _need(self.gate is None or (self.gate.dtype == torch.float32 and self.gate.dim() == 2 and self.gate.stride(1) == 1 and
                                    self.gate.shape[1] == QH * dv), "attention: the gate is float32 [T, query heads * value size]")

    def flat(self, QH: int, dv: int):
        """The arguments as the plain kernel's entry point takes them, one by one."""
        self.check(QH, dv)
        return (c_float(self.softcap), _p(self.sink), c_int(int(self.v_in_k)), _p(self.gate),
                c_longlong(self.gate.stride(0) if self.gate is not None else 0))

    def struct(self, QH: int, dv: int):
        """The arguments as the flash kernels' entry points take them: a pointer to one record."""
        self.check(QH, dv)
        self._rec = _FaMore(self.softcap, self.sink.data_ptr() if self.sink is not None else None, int(self.v_in_k),
                            self.gate.data_ptr() if self.gate is not None else None,
                            self.gate.stride(0) if self.gate is not None else 0)
        return ctypes.byref(self._rec)


_NO_EXTRAS = AttentionExtras()


def _more_arg(more: Optional[AttentionExtras], QH: int, dv: int):
    return c_void_p(0) if more is None else more.struct(QH, dv)


def _bias_args(bias, QH: int):
    """(pointer, rows) of a distance-bias table: float32 [QH, rows] (a head's biases by distance lie side by side), the
    last entry of a head for every greater distance."""
    if bias is None:
        return c_void_p(0), c_int(0)
    _need(bias.dtype == torch.float32 and bias.is_contiguous() and bias.dim() == 2 and bias.shape[0] == QH and bias.shape[1] > 0,
          "attention: the distance bias is a float32 table [query heads, distances]")
    return _p(bias), c_int(bias.shape[1])


def fa_group_chunk(group: int) -> int:
    """Query heads of one kv head that share a row tile: the largest divisor of the group up to 16."""
    for c in range(16, 0, -1):
        if group % c == 0:
            return c
    return 1


def _penalty_args(penalty, QH: int):
    if penalty is None:
        return c_void_p(0), c_void_p(0)
    r1, r2 = penalty
    _need(r1.dtype == torch.float32 and r2.dtype == torch.float32 and r1.numel() == QH and r2.numel() == QH,
          "attention: the distance penalty is two float32 vectors, one number per query head each")
    return _p(r1), _p(r2)


def fa_decode(q, cache, block_table, cu_q, kv_len, out, first_entry: int, n_entries: int, first_tok: int, n_splits: int,
              QH: int, KH: int, d: int, page_size: int, window: int, scale: float, work=(0.0, 0.0),
              chunk: int = 0, penalty=None, out_scale: float = 1.0, dv: int = 0, bias: Optional[torch.Tensor] = None,
              more: Optional[AttentionExtras] = None) -> None:
    """Split-K flash decoding (tensor cores) for entries that bring one token each.  chunk, penalty = (r1, r2),
    out_scale, dv and bias as in paged_attention_ref."""
    part_o = part_lse = None
    if n_splits > 1:
        part_o = torch.empty(n_entries * QH * n_splits * (dv or d), dtype=torch.float32, device=q.device)
        part_lse = torch.empty(n_entries * QH * n_splits, dtype=torch.float32, device=q.device)
    _check(lib().rb_fa_decode(_p(q), _p(cache), _p(block_table), _p(cu_q), _p(kv_len), _p(out), _p(part_o), _p(part_lse),
                              c_int(first_entry), c_int(n_entries), c_int(first_tok), c_int(n_splits), c_int(QH), c_int(KH),
                              c_int(d), c_int(page_size), c_int(block_table.shape[1]), c_int(window), c_float(scale),
                              c_int(chunk), *_penalty_args(penalty, QH), c_float(out_scale), c_int(dv), *_bias_args(bias, QH),
                              _more_arg(more, QH, dv or d), _stream()), "fa_decode", *work)
    if n_splits > 1:
        global launches
        launches += 1                      # the merge kernel


class StreamChain:
    """Which constant ranges (weights) the streaming kernels of one forward pass read, in order.

    A decode step is bound by memory traffic, and memory idles while one product drains and the small
    kernels after it run.  So a streaming kernel (a product over few tokens, decode attention) is told
    which weights the next one reads and calls their first bytes into L2 once its own loads are issued.
    The order is not declared by anyone: every pass writes down what it streamed, and a pass whose
    ranges match the last complete pass step by step learns from it what comes next; after the last
    range comes the first (the next step).  A pass that runs other kernels (a prompt) or another order
    just gets no hint until two passes agree again.
    """

    def __init__(self) -> None:
        self.known: list = []           # (address, bytes) of the last complete pass; bytes == 0: a marker, nothing to fetch
        self.now: list = []
        self.live = False

    def begin(self) -> None:
        self.now = []
        self.live = True

    def end(self) -> None:
        if self.live:
            self.known = self.now
        self.live = False

    def step(self, address: int, nbytes: int):
        """Note that a kernel streams this range now; returns (address, bytes) of what follows, or None."""
        if not self.live:
            return None
        i = len(self.now)
        self.now.append((address, nbytes))
        k = self.known
        if i < len(k) and k[i] == (address, nbytes) and len(k) > 1:
            nxt = k[(i + 1) % len(k)]
            if nxt[1] > 0 and nxt[0] % 16 == 0:
                return nxt
        return None


_chain: Optional[StreamChain] = None
L2_PREFETCH_BYTES = int(float(os.environ.get("REINFER_B200_L2_PREFETCH_MB", "12")) * (1 << 20))
DEFER_SUMS = os.environ.get("REINFER_B200_DEFER_SUMS", "1") != "0"   # split products leave their last sum to the next norm
STREAMING_TOKENS = 64                       # products over at most this many tokens count as weight streaming


def set_chain(chain: Optional[StreamChain]) -> Optional[StreamChain]:
    """Make `chain` the one that the streaming kernels consult (None: no hints); returns the previous one."""
    global _chain
    old, _chain = _chain, chain
    return old


def row_scale_ok(T: int) -> bool:
    """Whether the tensor-core products over T tokens apply the factor of rows that lack it (RowScaled input)."""
    return bool(lib().rb_gemm_row_scale_ok(c_int(int(T))))


def _row_scale_args(row_scale, T: int):
    """(sumsq pointer, parts, width, eps) arguments of a product whose rows still lack their RMS factor."""
    if row_scale is None:
        return c_void_p(0), c_int(0), c_int(0), c_float(0.0)
    sumsq, width, eps = row_scale
    _need(sumsq.dtype == torch.float32 and sumsq.is_contiguous() and sumsq.dim() == 2 and sumsq.shape[0] == T,
          "gemm: row factors come as float32 [tokens, parts]")
    return _p(sumsq), c_int(sumsq.shape[1]), c_int(int(width)), c_float(float(eps))


def _next_range(t: Optional[torch.Tensor], marker: int = 0):
    """(pointer, bytes) arguments of the range that follows tensor t (or the marker) in the active chain."""
    if _chain is None or L2_PREFETCH_BYTES <= 0:
        return c_void_p(0), c_longlong(0)
    nxt = _chain.step(t.data_ptr(), t.numel() * t.element_size()) if t is not None else _chain.step(marker, 0)
    if nxt is None:
        return c_void_p(0), c_longlong(0)
    return c_void_p(nxt[0]), c_longlong(min(nxt[1], L2_PREFETCH_BYTES))


DECODE_SLOTS = 296                          # CTAs of the decode attention that are resident at once (two per SM)
# Clusters merge their splits themselves only while they fill at most this share of the places the device reports: a
# cluster needs its places on one GPC at once, and near the limit clusters wait for one another (measured: 13 splits
# of 16 pairs on 208 of 221 places, 7 splits of 40 pairs on 280 of 296, each 4 % slower a step than a neighbouring count)
CLUSTER_FILL = 0.9
MAX_CLUSTER_SPLITS = 16                     # splits that can merge inside one cluster (more than 8: not portable, asked of the device)
_cluster_slots: dict = {}


def decode_cluster_slots(d: int, n: int) -> int:
    """CTAs of the decode attention that can be resident at once as clusters of n: the fixed figure for portable
    clusters, what the device's occupancy calculation says for larger ones (0: cannot be launched)."""
    if n <= 8:
        return DECODE_SLOTS
    key = (d, n)
    if key not in _cluster_slots:
        _cluster_slots[key] = min(DECODE_SLOTS, int(lib().rb_fa_decode_cluster_slots(c_int(d), c_int(n))))
    return _cluster_slots[key]


def decode_merges_in_cluster(n_entries: int, QH: int, KH: int, d: int, n_splits: int) -> bool:
    """Whether fa_decode_tma's splits would be the CTAs of clusters that merge their results themselves."""
    ctas = n_entries * KH * (QH // KH // fa_group_chunk(QH // KH)) * n_splits
    return bool(ATTN_CLUSTER_MERGE and 2 <= n_splits <= min(MAX_CLUSTER_SPLITS, d) and ctas <= CLUSTER_FILL * decode_cluster_slots(d, n_splits))


def fa_decode_tma(q, cache, block_table, cu_q, kv_len, out, first_entry: int, n_entries: int, first_tok: int, n_splits: int,
                  QH: int, KH: int, d: int, page_size: int, window: int, scale: float, work=(0.0, 0.0),
                  bias: Optional[torch.Tensor] = None, more: Optional["AttentionExtras"] = None) -> None:
    """Split-K flash decoding with the key/value tiles brought in by TMA (page size a power of two >= 8); bias as in
    paged_attention_ref; more: soft cap, and - with one split or splits that merge in their cluster - sink and gate.
    Up to 16 splits whose CTAs are all resident at once form clusters that merge their results themselves (no scratch,
    no merge kernel); several waves of CTAs, or more splits, go through scratch and the merge kernel (clusters
    that wait for a free place on one GPC were measured slower there)."""
    part_o = part_lse = None
    in_kernel = decode_merges_in_cluster(n_entries, QH, KH, d, n_splits)
    _need(more is None or not more.v_in_k, "fa_decode_tma: the pages hold keys and values")
    extras = (more or _NO_EXTRAS).flat(QH, d)
    if n_splits > 1 and not in_kernel:
        part_o = torch.empty(n_entries * QH * n_splits * d, dtype=torch.float32, device=q.device)
        part_lse = torch.empty(n_entries * QH * n_splits, dtype=torch.float32, device=q.device)
    nw, nb = _next_range(None, marker=cache.data_ptr())
    _check(lib().rb_fa_decode_tma(_p(q), _p(cache), c_longlong(cache.shape[0]), _p(block_table), _p(cu_q), _p(kv_len), _p(out),
                                  _p(part_o), _p(part_lse), c_int(first_entry), c_int(n_entries), c_int(first_tok),
                                  c_int(n_splits), c_int(QH), c_int(KH), c_int(d), c_int(page_size),
                                  c_int(block_table.shape[1]), c_int(window), c_float(scale), nw, nb, *_bias_args(bias, QH),
                                  extras[0], extras[1], extras[3], extras[4], _stream()),
           "fa_decode_tma", *work)


def fa_prefill_tma(q, cache, block_table, cu_q, kv_len, out, first_entry: int, n_entries: int, n_tiles: int,
                   QH: int, KH: int, d: int, page_size: int, window: int, scale: float, work=(0.0, 0.0)) -> None:
    """Paged causal flash attention with the key/value tiles brought in by TMA."""
    _check(lib().rb_fa_prefill_tma(_p(q), _p(cache), c_longlong(cache.shape[0]), _p(block_table), _p(cu_q), _p(kv_len), _p(out),
                                   c_int(first_entry), c_int(n_entries), c_int(n_tiles), c_int(QH), c_int(KH), c_int(d),
                                   c_int(page_size), c_int(block_table.shape[1]), c_int(window), c_float(scale), _stream()),
           "fa_prefill_tma", *work)


def fa_prefill_tc(q, cache, block_table, cu_q, kv_len, out, first_entry: int, n_entries: int, q_lens,
                  QH: int, KH: int, d: int, page_size: int, window: int, scale: float, work=(0.0, 0.0),
                  chunk: int = 0, penalty=None, out_scale: float = 1.0, bias: Optional[torch.Tensor] = None,
                  more: Optional["AttentionExtras"] = None) -> None:
    """Paged causal flash attention on the tcgen05 tensor cores (scores and the weighted sum in tensor memory):
    head size 128, page size a power of two >= 8.  q_lens: the token counts of the entries (host).  chunk (a multiple
    of 64), penalty = (r1, r2), out_scale and bias as in paged_attention_ref; more: soft cap, sink and gate (not values
    inside the keys)."""
    _need(more is None or not more.v_in_k, "fa_prefill_tc: the pages hold keys and values")
    extras = (more or _NO_EXTRAS).flat(QH, d)
    gc = int(lib().rb_fa_prefill_tc_group(c_int(QH), c_int(KH)))
    tpt = int(lib().rb_fa_prefill_tc_rows()) // gc              # tokens that one CTA takes
    n_tiles = sum(-(-int(n) // tpt) for n in q_lens)
    _check(lib().rb_fa_prefill_tc(_p(q), _p(cache), c_longlong(cache.shape[0]), _p(block_table), _p(cu_q), _p(kv_len), _p(out),
                                  c_int(first_entry), c_int(n_entries), c_int(n_tiles), c_int(QH), c_int(KH), c_int(d),
                                  c_int(page_size), c_int(block_table.shape[1]), c_int(window), c_float(scale), c_int(chunk),
                                  *_penalty_args(penalty, QH), c_float(out_scale), *_bias_args(bias, QH), extras[0], extras[1],
                                  extras[3], extras[4], _stream()),
           "fa_prefill_tc", *work)


def tma_pages(page_size: int) -> bool:
    return page_size >= 8 and page_size & (page_size - 1) == 0


def fa_prefill(q, cache, block_table, cu_q, kv_len, out, first_entry: int, n_entries: int, n_tiles: int,
               QH: int, KH: int, d: int, page_size: int, window: int, scale: float, work=(0.0, 0.0),
               chunk: int = 0, penalty=None, out_scale: float = 1.0, dv: int = 0, bias: Optional[torch.Tensor] = None,
               more: Optional[AttentionExtras] = None) -> None:
    """Paged causal flash attention (tensor cores) for entries that bring several tokens.  chunk, penalty = (r1, r2),
    out_scale, dv and bias as in paged_attention_ref."""
    _check(lib().rb_fa_prefill(_p(q), _p(cache), _p(block_table), _p(cu_q), _p(kv_len), _p(out), c_int(first_entry),
                               c_int(n_entries), c_int(n_tiles), c_int(QH), c_int(KH), c_int(d), c_int(page_size),
                               c_int(block_table.shape[1]), c_int(window), c_float(scale), c_int(chunk),
                               *_penalty_args(penalty, QH), c_float(out_scale), c_int(dv), *_bias_args(bias, QH),
                               _more_arg(more, QH, dv or d), _stream()),
           "fa_prefill", *work)


USE_TMA_ATTENTION = os.environ.get("REINFER_B200_TMA_ATTENTION", "1") != "0"
ATTN_CLUSTER_MERGE = os.environ.get("REINFER_B200_ATTN_CLUSTER", "1") != "0"
USE_TC_ATTENTION = os.environ.get("REINFER_B200_TC_ATTENTION", "1") != "0"
MIXED_OVERLAP = os.environ.get("REINFER_B200_MIXED_OVERLAP", "1") != "0"   # decode attention beside the portions' attention
_side_streams: dict = {}


def _side_stream(device) -> "torch.cuda.Stream":
    key = torch.device(device).index or 0
    if key not in _side_streams:
        _side_streams[key] = torch.cuda.Stream(device=device)
    return _side_streams[key]
def decode_splits(ctas: int, tiles: int, slots: int = DECODE_SLOTS, head_dim: int = 128, cluster_slots=None,
                  total_tiles: Optional[int] = None) -> int:
    """How many CTAs share one (request, kv head)'s keys: the split count with the least estimated time (ties to
    the smaller).  `ctas` (request, kv head) pairs, the longest of `tiles` 64-key tiles, `total_tiles` over all pairs
    (default: all as long as the longest).  The estimate is fitted to measurements of the kernel at batch 1..64 and
    4k..32k keys, alone and inside whole decode steps:
      - every resident CTA has the first three tiles of its share on their way before the kernels in front of it
        have finished; what is left streams at the memory bandwidth, less what the CTAs' fill and drain cost,
        which weighs the more the fewer tiles a CTA walks:   bytes left / 6.5 TB/s * (1 + 2.7 / tiles per CTA)
      - a CTA alone streams a 64-key tile of 128-wide heads in about a microsecond and needs about five to start
        and finish; the kernel lasts as long as the CTA with most tiles:   (most tiles per CTA - 3) * 1 us + 5 us
        (requests of unequal lengths: the longest alone decides this term, so splitting pays although the
        CTAs then come in several waves)
      - the larger of the two counts, plus the merge: about 2 us inside a cluster (up to 16 splits, all CTAs
        resident at once: `cluster_slots(n)` says how many CTAs that is for clusters of more than 8), else a merge
        kernel of about 6 us + 0.1 us per split (a launch more in the step's chain; at 9 and 12 requests the count
        that still merges in its clusters beat the next one, which does not, by 2-3.5 us a layer).
      - more CTAs than can be resident come in waves: the full waves stream at the bandwidth, but the CTAs of a
        part-filled last wave run with few others and cannot use what the rest left free - each walks its tiles at a
        lone CTA's pace.  (40-56 requests over 4k keys, one split: 384 CTAs on 296 places took as long as 512;
        three splits took a tenth off the step at 40 and 48 requests, none at 56.)"""
    if _FORCED_SPLITS:
        return max(1, min(_FORCED_SPLITS, tiles))
    key = None
    if cluster_slots is None:
        key = (ctas, tiles, slots, head_dim, total_tiles, ATTN_CLUSTER_MERGE)
        if key in _splits_memo:
            return _splits_memo[key]
        cluster_slots = lambda n: decode_cluster_slots(head_dim, n)
    if total_tiles is None:
        total_tiles = ctas * tiles
    total_tiles = max(min(total_tiles, ctas * tiles), 1)
    tile_us = head_dim / 128.0                              # a lone CTA's time for one tile
    tile_bw_us = 64 * head_dim * 4 / 6.5e6                  # one tile's bytes at the device's bandwidth
    ahead = 3                                               # tiles a CTA requests before it has to wait
    best, best_cost = 1, None
    for n in range(1, max(1, min(64, tiles)) + 1):
        per = -(-tiles // n)                                # the longest request's CTAs
        per_avg = max(total_tiles / (ctas * n), 1.0)
        early = min(total_tiles, min(ctas * n, slots) * ahead)
        t_bw = (total_tiles - early) * tile_bw_us * (1.0 + 2.7 / per_avg)
        t_lat = max(0, per - ahead) * tile_us + 5.0
        if n == 1:
            merge = 0.0
        elif n <= min(MAX_CLUSTER_SPLITS, head_dim) and ATTN_CLUSTER_MERGE and \
                ctas * n <= CLUSTER_FILL * (slots if n <= 8 else min(slots, cluster_slots(n))):
            merge = 2.0
        else:
            merge = 6.0 + 0.1 * n
        t_wave = 0.0
        if ctas * n > slots:
            full, rest = divmod(ctas * n, slots)
            fill_drain = 1.0 + 2.7 / per_avg
            wave = per_avg * max(tile_us, slots * tile_bw_us) * fill_drain
            t_wave = full * wave
            if rest:
                # (the CTAs of a wave end within about a seventh of its length of one another, and the next begin as
                # they do: that much of the last wave runs beside the one before it)
                t_wave += per_avg * max(tile_us, rest * tile_bw_us) * fill_drain - 0.15 * wave
        cost = max(t_bw, t_lat, t_wave) + merge
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = n, cost
    if key is not None:
        if len(_splits_memo) > 4096:
            _splits_memo.clear()
        _splits_memo[key] = best
    return best


_splits_memo: dict = {}
# REINFER_B200_ATTN_SPLITS=n: every decode attention launch splits its keys n ways (a development switch, to measure the model against)
_FORCED_SPLITS = int(os.environ.get("REINFER_B200_ATTN_SPLITS", "0") or 0)


def attention(ctx, q: torch.Tensor, cache: torch.Tensor, group, out: torch.Tensor, QH: int, KH: int, d: int,
              window: int, scale: float) -> None:
    """Attention of a step's tokens over their requests' pages.  float32 (and head sizes the
    tensor-core kernels do not take) runs the plain kernel; bfloat16 runs flash decoding for the
    entries with one token and the paged flash prefill kernel for the others."""
    n_dec, E = ctx.n_decode, ctx.n_entries
    dec_work = pre_work = (0.0, 0.0)
    if _profiler is not None:
        def work(first, last):
            """(flops, bytes) that attention over entries first..last-1 has to do: two products of 2*d per (query head,
            key) pair the causal mask lets through, and every key and value of the request read once."""
            fl = by = 0.0
            for e in range(first, last):
                n, s0 = ctx.q_start[e + 1] - ctx.q_start[e], ctx.start_pos[e]
                pairs = n * s0 + n * (n + 1) / 2
                if window:
                    pairs = min(pairs, n * window)
                fl += 4.0 * QH * d * pairs
                by += ((min(s0 + n, window + n) if window else s0 + n) * KH * 2 + 2 * n * QH) * d * q.element_size()
            return fl, by
        dec_work, pre_work = work(0, n_dec), work(n_dec, E)
    if q.dtype != torch.bfloat16 or d % 8 or d > 256:
        paged_attention_ref(q, cache, group.block_table, ctx.tok_entry, ctx.positions, out, QH, KH, d,
                            group.page_size, window, scale, work=(dec_work[0] + pre_work[0], dec_work[1] + pre_work[1]))
        return
    _need(q.is_contiguous() and out.is_contiguous() and cache.is_contiguous() and group.block_table.is_contiguous(),
          "attention: contiguous")
    gc = fa_group_chunk(QH // KH)
    joined = None
    if n_dec:
        pairs = KH * (QH // KH // gc)
        ctas = n_dec * pairs
        tiles = ctx.decode_kv_tiles[1] if ctx.decode_kv_tiles else -(-ctx.max_kv_len // 64)
        total = ctx.decode_kv_tiles[0] * pairs if ctx.decode_kv_tiles else None
        plan = getattr(ctx, "decode_plan", None)              # a captured step: the split it was made for
        n_splits = max(1, min(int(plan), tiles)) if isinstance(plan, int) and not _FORCED_SPLITS else \
            decode_splits(ctas, tiles, head_dim=d, total_tiles=total)
        decode = fa_decode_tma if (tma_pages(group.page_size) and USE_TMA_ATTENTION) else fa_decode
        if E > n_dec and MIXED_OVERLAP and _profiler is None and not torch.cuda.is_current_stream_capturing():
            # A step with prompt portions beside decoding requests: the two attention kernels read the same inputs
            # and write different rows, and the decoding requests' kernel leaves most SMs idle (a few CTAs with long
            # chains).  It runs on a stream of its own beside the portions' kernel; the main stream goes on when
            # both are done.
            main = torch.cuda.current_stream()
            ready = torch.cuda.Event()
            ready.record(main)
            side = _side_stream(q.device)
            side.wait_event(ready)
            with torch.cuda.stream(side):
                decode(q, cache, group.block_table, ctx.cu_q, ctx.kv_len, out, 0, n_dec, 0, n_splits, QH, KH, d,
                       group.page_size, window, scale, work=dec_work)
                joined = torch.cuda.Event()
                joined.record(side)
        else:
            decode(q, cache, group.block_table, ctx.cu_q, ctx.kv_len, out, 0, n_dec, 0, n_splits, QH, KH, d,
                   group.page_size, window, scale, work=dec_work)
    if E > n_dec and d == 128 and USE_TC_ATTENTION and USE_TMA_ATTENTION and tma_pages(group.page_size):
        fa_prefill_tc(q, cache, group.block_table, ctx.cu_q, ctx.kv_len, out, n_dec, E - n_dec,
                      [ctx.q_start[e + 1] - ctx.q_start[e] for e in range(n_dec, E)], QH, KH, d, group.page_size, window, scale,
                      work=pre_work)
    elif E > n_dec:
        tpt = 64 // gc
        n_tiles = sum(-(-(ctx.q_start[e + 1] - ctx.q_start[e]) // tpt) for e in range(n_dec, E))
        prefill = fa_prefill_tma if (tma_pages(group.page_size) and USE_TMA_ATTENTION) else fa_prefill
        prefill(q, cache, group.block_table, ctx.cu_q, ctx.kv_len, out, n_dec, E - n_dec, n_tiles, QH, KH, d,
                group.page_size, window, scale, work=pre_work)
    if joined is not None:
        torch.cuda.current_stream().wait_event(joined)


def sample(logits: torch.Tensor, row_idx: Optional[torch.Tensor], params: torch.Tensor, history: Optional[torch.Tensor],
           work: torch.Tensor, out_tokens: torch.Tensor, rows: int) -> None:
    """params: uint8 tensor holding `rows` RbSampleParams records (see sampling/sampler.py)."""
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "sample: float32 logits")
    vocab = logits.shape[1]
    hist_cap = history.shape[1] if history is not None else 0
    _need(work.numel() >= rows * vocab and work.dtype == torch.float32, "sample: scratch of rows*vocab floats")
    _check(lib().rb_sample(_p(logits), c_longlong(logits.stride(0)), _p(row_idx), _p(params), _p(history),
                           c_int(hist_cap), _p(work), _p(out_tokens), c_int(rows), c_int(vocab), _stream()), "sample")


def sample_slots(logits: torch.Tensor, row_slot: torch.Tensor, slot_params: torch.Tensor, slot_history: torch.Tensor,
                 slot_token: torch.Tensor, work: torch.Tensor, out_tokens: torch.Tensor, rows: int) -> None:
    """One token per row of `logits`, every request's parameters, seed, draw count and recent tokens taken from
    (and the token written to) its slot: row r belongs to slot row_slot[r] (csrc/sampler.cu)."""
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "sample_slots: float32 logits")
    vocab = logits.shape[1]
    _need(work.numel() >= rows * vocab and work.dtype == torch.float32, "sample_slots: scratch of rows*vocab floats")
    _need(row_slot.dtype == torch.int32 and slot_token.dtype == torch.int32 and slot_history.dtype == torch.int32 and
          slot_params.dtype == torch.uint8 and slot_params.is_contiguous() and slot_history.is_contiguous(),
          "sample_slots: int32 tables, records as bytes")
    _check(lib().rb_sample_slots(_p(logits), c_longlong(logits.stride(0)), _p(row_slot), _p(slot_params), _p(slot_history),
                                 c_int(slot_history.shape[1]), _p(slot_token), _p(work), _p(out_tokens), c_int(rows),
                                 c_int(vocab), _stream()), "sample_slots")


_gemm_ws = None
GEMM_WS_FLOATS = 8 << 20          # 32 MB of split-K partials


def set_gemm_token_lanes(value: int) -> int:
    """Which form the tensor-core product over several token tiles takes: 1 a token per accumulator lane, 0 a
    feature per lane.  Returns the old setting; for tests and comparisons."""
    return int(lib().rb_set_gemm_token_lanes(c_int(int(value))))


def set_gemm_tile_features(value: int) -> int:
    """Weight rows per tile of the products over several token tiles (token-lane forms): 256 (four stages in
    flight), 224 (five), or 0 = chosen per product by the rounds its tiles need over the SMs.  Returns the old
    setting; for tests and comparisons."""
    return int(lib().rb_set_gemm_tile_features(c_int(int(value))))


def gemm_bf16(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, accumulate: bool = False, splits: int = 0,
              row_scale=None) -> None:
    """c[T,N] (=|+=) a[T,K] @ w[N,K]^T on the tensor cores (tcgen05, TMA); bf16 operands, float
    accumulation, c bfloat16 or float32.  Operands that TMA cannot address (a row stride that is no
    multiple of 8 elements, a base that is not 16-byte aligned) go to the plain kernel instead."""
    global _gemm_ws
    T, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and tuple(c.shape) == (T, N), "gemm: shapes")
    _need(a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "gemm_bf16: bfloat16 operands")
    _need(a.stride(1) == 1 and w.stride(1) == 1 and c.stride(1) == 1, "gemm: rows contiguous")
    if a.stride(0) % 8 or w.stride(0) % 8 or a.data_ptr() % 16 or w.data_ptr() % 16:
        _need(row_scale is None, "gemm: row factors need operands that TMA can address")
        return gemm_ref(a, w, c, accumulate)
    if _gemm_ws is None or _gemm_ws.device != a.device:
        _gemm_ws = torch.empty(GEMM_WS_FLOATS, dtype=torch.float32, device=a.device)
    nw, nb = _next_range(w) if T <= STREAMING_TOKENS else (c_void_p(0), c_longlong(0))
    _check(lib().rb_gemm_bf16(_p(a), _p(w), _p(c), c_int(dt(c)), c_int(int(accumulate)), c_int(T), c_int(N), c_int(K),
                              c_longlong(a.stride(0)), c_longlong(w.stride(0)), c_longlong(c.stride(0)),
                              _p(_gemm_ws), c_longlong(_gemm_ws.numel()), c_int(splits), nw, nb,
                              *_row_scale_args(row_scale, T), _stream()), f"gemm {N}x{K}",
           2.0 * T * N * K, 2.0 * (T * K + N * K) + T * N * c.element_size())


# REINFER_B200_QKV_HEADS=0: the q/k/v projection and the per-head work as two kernels at every size (a development switch).
QKV_HEADS = os.environ.get("REINFER_B200_QKV_HEADS", "1") != "0"


def gemm_qkv_heads(a: torch.Tensor, w_qkv: torch.Tensor, q_out: torch.Tensor, cache: torch.Tensor, kv_slot: torch.Tensor,
                   cs_table: torch.Tensor, q_w: torch.Tensor, k_w: torch.Tensor, QH: int, KH: int, page_size: int, eps: float,
                   row_scale=None) -> bool:
    """The q/k/v projection of a prompt portion with the per-head work in its epilogue (heads of 128): q_out [T, QH, 128]
    gets the normalised, rotated queries, the cache pages the keys and values at kv_slot.  cs_table [T, 64, 2] float32
    from rope_table.  Returns False (and does nothing) where this form does not apply - at most 256 tokens, operands
    that TMA cannot address - and the caller runs the product and qknorm_rope_append one after the other."""
    T, K = a.shape
    if not QKV_HEADS:
        return False
    if T <= 256 or a.dtype != torch.bfloat16 or w_qkv.dtype != torch.bfloat16 or q_out.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16:
        return False
    if row_scale is not None and not row_scale_ok(T):
        return False
    if a.stride(1) != 1 or w_qkv.stride(1) != 1 or a.stride(0) % 8 or w_qkv.stride(0) % 8 or a.data_ptr() % 16 or w_qkv.data_ptr() % 16:
        return False
    _need(w_qkv.shape == ((QH + 2 * KH) * 128, K), "gemm_qkv_heads: weight shape")
    _need(q_out.is_contiguous() and tuple(q_out.shape) == (T, QH, 128) and cache.is_contiguous(), "gemm_qkv_heads: q_out [T, QH, 128], cache contiguous")
    _need(q_w.dtype == k_w.dtype and q_w.numel() == 128 and k_w.numel() == 128 and q_w.is_contiguous() and k_w.is_contiguous(),
          "gemm_qkv_heads: norm weights [128] of one dtype")
    _need(cs_table.dtype == torch.float32 and cs_table.is_contiguous() and cs_table.numel() == T * 128, "gemm_qkv_heads: table [T, 64, 2] float32")
    _need(kv_slot.dtype == torch.int32 and kv_slot.numel() >= T, "gemm_qkv_heads: kv_slot int32 [T]")
    N = (QH + 2 * KH) * 128
    _check(lib().rb_gemm_qkv_heads(_p(a), _p(w_qkv), c_int(T), c_int(K), c_longlong(a.stride(0)), c_longlong(w_qkv.stride(0)),
                                   c_int(QH), c_int(KH), _p(q_out), _p(cache), _p(kv_slot), _p(cs_table), _p(q_w), _p(k_w),
                                   c_int(dt(q_w)), c_float(eps), c_int(page_size), *_row_scale_args(row_scale, T), _stream()),
           f"gemm+heads {N}x{K}", 2.0 * T * N * K, float(T * K * 2 + N * K * 2 + T * N * 2))
    return True


def gemm_qkv_heads_stream(a, w_qkv: torch.Tensor, q_out: torch.Tensor, cache: torch.Tensor, kv_slot: Optional[torch.Tensor],
                          positions: torch.Tensor, inv_freq: torch.Tensor, q_w: Optional[torch.Tensor], k_w: Optional[torch.Tensor],
                          QH: int, KH: int, page_size: int, eps: float, row_scale=None) -> bool:
    """The q/k/v projection of a decode step's few rows (heads of 128) whose cluster does the per-head work on its sums:
    q_out [T, QH, 128] gets the normalised, rotated queries, the cache pages the keys and values at kv_slot (None:
    nothing is stored).  Returns False (and does nothing) where this form does not apply, and the caller runs the
    product and qknorm_rope_append one after the other."""
    T, K = a.shape
    if not (QKV_HEADS and 0 < T <= STREAMING_TOKENS and K >= 128 and a.dtype == torch.bfloat16 and w_qkv.dtype == torch.bfloat16 and
            q_out.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16):
        return False
    if a.stride(1) != 1 or w_qkv.stride(1) != 1 or a.stride(0) % 8 or w_qkv.stride(0) % 8 or a.data_ptr() % 16 or w_qkv.data_ptr() % 16:
        return False
    _need(w_qkv.shape == ((QH + 2 * KH) * 128, K), "gemm_qkv_heads_stream: weight shape")
    _need(q_out.is_contiguous() and tuple(q_out.shape) == (T, QH, 128) and cache.is_contiguous(), "gemm_qkv_heads_stream: q_out [T, QH, 128], cache contiguous")
    _need((q_w is None) == (k_w is None), "gemm_qkv_heads_stream: q and k norm weights come together")
    if q_w is not None:
        _need(q_w.dtype == k_w.dtype and q_w.numel() == 128 and k_w.numel() == 128 and q_w.is_contiguous() and k_w.is_contiguous(),
              "gemm_qkv_heads_stream: norm weights [128] of one dtype")
    _need(inv_freq.dtype == torch.float32 and inv_freq.numel() == 64 and inv_freq.is_contiguous(), "gemm_qkv_heads_stream: inv_freq float32 [64]")
    _need(positions.dtype == torch.int32 and positions.numel() >= T, "gemm_qkv_heads_stream: positions int32 [T]")
    _need(kv_slot is None or (kv_slot.dtype == torch.int32 and kv_slot.numel() >= T), "gemm_qkv_heads_stream: kv_slot int32 [T]")
    N = (QH + 2 * KH) * 128
    nw, nb = _next_range(w_qkv)
    _check(lib().rb_gemm_qkv_heads_stream(_p(a), _p(w_qkv), c_int(T), c_int(K), c_longlong(a.stride(0)), c_longlong(w_qkv.stride(0)),
                                          c_int(QH), c_int(KH), _p(q_out), _p(cache), _p(kv_slot), _p(positions), _p(inv_freq),
                                          _p(q_w), _p(k_w), c_int(dt(q_w) if q_w is not None else 0), c_float(eps), c_int(page_size),
                                          nw, nb, *_row_scale_args(row_scale, T), _stream()),
           f"gemm+heads {N}x{K}", 2.0 * T * N * K, float(T * K * 2 + N * K * 2 + T * N * 2))
    return True


def gemm_bf16_partials(a: torch.Tensor, w: torch.Tensor, row_scale=None) -> Optional[torch.Tensor]:
    """Partial sums [S, T, N] (float32) of a[T,K] @ w[N,K]^T over S ranges of K, for a consumer that adds them
    up itself (add_rmsnorm with a stacked delta): the split product then needs no reduction of its own, and
    none of its CTAs waits for another.  None if this product is not one for the streaming kernel (more than
    STREAMING_TOKENS tokens, operands that TMA cannot address): the caller then runs the plain form."""
    T, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K, "gemm: shapes")
    if not (0 < T <= STREAMING_TOKENS and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16):
        return None
    if a.stride(1) != 1 or w.stride(1) != 1 or a.stride(0) % 8 or w.stride(0) % 8 or a.data_ptr() % 16 or w.data_ptr() % 16:
        return None
    S = int(lib().rb_gemm_partials_plan(c_int(T), c_int(N), c_int(K)))
    out = torch.empty((S, T, N), dtype=torch.float32, device=a.device)
    nw, nb = _next_range(w)
    _check(lib().rb_gemm_bf16_partials(_p(a), _p(w), _p(out), c_int(S), c_int(T), c_int(N), c_int(K),
                                       c_longlong(a.stride(0)), c_longlong(w.stride(0)), nw, nb,
                                       *_row_scale_args(row_scale, T), _stream()), f"gemm {N}x{K}",
           2.0 * T * N * K, 2.0 * (T * K + N * K) + 4.0 * S * T * N)
    return out


# REINFER_B200_PRODUCT_NORM=0: a decode step's o and down projections never prepare the next norm's rows themselves
# (they leave partial sums, or add into the residual, and the norm runs as a kernel of its own).
PRODUCT_NORM = os.environ.get("REINFER_B200_PRODUCT_NORM", "1") != "0"


def gemm_bf16_residual_norm(a: torch.Tensor, w: torch.Tensor, residual: torch.Tensor, norm_w: torch.Tensor, row_scale=None,
                            dyt=None):
    """residual[T,N] (float32) += a[T,K] @ w[N,K]^T for a decode step's few rows, the product reduced inside a
    cluster whose CTAs also prepare what the RMS norm with weight norm_w would make of the new residual: returns
    (rows, sumsq) as residual_rowscale does (rows = bfloat16(residual * norm_w), sumsq [T, N/128] the sum of squares
    by tiles of 128 columns), or None (and does nothing) where this form does not apply.  With dyt = (bias, alpha),
    tensors of norm_w's dtype, the norm is Dynamic Tanh: rows = bfloat16(tanh(alpha residual) norm_w + bias), complete,
    and sumsq is None."""
    T, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and tuple(residual.shape) == (T, N), "gemm: shapes")
    if not (PRODUCT_NORM and 0 < T <= STREAMING_TOKENS and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and
            residual.dtype == torch.float32 and N % 128 == 0 and K >= 128 and norm_w.numel() == N and norm_w.is_contiguous() and
            norm_w.dtype in (torch.float32, torch.bfloat16) and norm_w.data_ptr() % 16 == 0):
        return None
    if a.stride(1) != 1 or w.stride(1) != 1 or a.stride(0) % 8 or w.stride(0) % 8 or a.data_ptr() % 16 or w.data_ptr() % 16 or \
            residual.stride(1) != 1 or residual.stride(0) % 4 or residual.data_ptr() % 16:
        return None
    bias = alpha = None
    if dyt is not None:
        bias, alpha = dyt
        if not (bias.dtype == alpha.dtype == norm_w.dtype and bias.is_contiguous() and bias.numel() == N and alpha.numel() == 1 and
                bias.data_ptr() % 16 == 0):
            return None
    rows = torch.empty((T, N), dtype=torch.bfloat16, device=a.device)
    sumsq = torch.empty((T, N // 128), dtype=torch.float32, device=a.device) if dyt is None else None
    nw, nb = _next_range(w)
    _check(lib().rb_gemm_bf16_residual_norm(_p(a), _p(w), _p(residual), c_int(T), c_int(N), c_int(K), c_longlong(a.stride(0)),
                                            c_longlong(w.stride(0)), c_longlong(residual.stride(0)), _p(norm_w), c_int(dt(norm_w)),
                                            _p(rows), _p(sumsq), nw, nb, *_row_scale_args(row_scale, T), _p(bias), _p(alpha),
                                            _stream()),
           f"gemm+{'dyt' if dyt is not None else 'norm'} {N}x{K}", 2.0 * T * N * K, 2.0 * (T * K + N * K) + 14.0 * T * N)
    return rows, sumsq


def gemm_bf16_swiglu(a: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor, splits: int = 0, row_scale=None,
                     act: str = "silu", bias: Optional[torch.Tensor] = None, gates: Optional[torch.Tensor] = None, ff: int = 0) -> bool:
    """out[T,F] (bf16) = silu(a Wg^T) * (a Wu^T), w_gate_up = [Wg; Wu] of shape [2F, K]: one tensor-core
    product with two accumulators and the activation in its epilogue.  Returns False (and does
    nothing) if TMA cannot address the operands; the caller then runs the two-kernel form.
    Options of the epilogue, as in glu_act: `act` ("silu" or "gelu_tanh"), `bias` (float32 [2F], added to gate and up
    before the activation), `gates` (float32 [T, F // ff]: a factor per token and block of ff features)."""
    T, K = a.shape
    F_ = out.shape[1]
    _need(bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == 2 * F_), "gemm_swiglu: the bias is float32 [2F]")
    _need(gates is None or (ff > 0 and F_ % ff == 0 and gates.dtype == torch.float32 and gates.is_contiguous() and
                            tuple(gates.shape) == (T, F_ // ff)), "gemm_swiglu: gates float32 [T, F / ff]")
    _need(w_gate_up.shape == (2 * F_, K) and out.shape[0] == T, "gemm_swiglu: shapes")
    _need(a.dtype == w_gate_up.dtype == out.dtype == torch.bfloat16, "gemm_swiglu: bfloat16 tensors")
    _need(a.stride(1) == 1 and w_gate_up.stride(1) == 1 and out.stride(1) == 1, "gemm_swiglu: rows contiguous")
    if a.stride(0) % 8 or w_gate_up.stride(0) % 8 or a.data_ptr() % 16 or w_gate_up.data_ptr() % 16:
        return False
    nw, nb = _next_range(w_gate_up) if T <= STREAMING_TOKENS else (c_void_p(0), c_longlong(0))
    _check(lib().rb_gemm_bf16_swiglu(_p(a), _p(w_gate_up), _p(out), c_int(T), c_int(F_), c_int(K),
                                     c_longlong(a.stride(0)), c_longlong(w_gate_up.stride(0)), c_longlong(out.stride(0)),
                                     c_int(splits), nw, nb, *_row_scale_args(row_scale, T), _p(bias), c_int(GLU_ACTS[act]), _p(gates),
                                     c_int(ff), _stream()),
           f"gemm+swiglu {2 * F_}x{K}", 4.0 * T * F_ * K, 2.0 * (T * K + 2 * F_ * K + T * F_))
    return True


# ------------------------------------------------------------------ statistics-free norm, soft cap, short convolution, recurrences
def dyt(x: torch.Tensor, delta: Optional[torch.Tensor], w: torch.Tensor, b: torch.Tensor, alpha: torch.Tensor,
        out: torch.Tensor, row_idx: Optional[torch.Tensor] = None) -> None:
    """x (float32 [rows, h]) += delta (x's shape or a stack of partial sums, float32, added in ascending order);
    out[r] = tanh(alpha x[row_idx[r] or r]) w + b.  With row_idx x itself stays as it is."""
    _need(x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous(), "dyt: x float32 contiguous")
    _need(w.dtype == b.dtype == alpha.dtype and alpha.numel() == 1, "dyt: weight, bias and alpha of one dtype")
    h = x.shape[-1]
    rows = out.numel() // h
    n_delta = 0
    if delta is not None:
        _need(delta.dtype == torch.float32 and delta.is_contiguous() and delta.numel() % x.numel() == 0 and delta.shape[-1] == h,
              "dyt: delta float32 with x's shape (or a stack of it)")
        n_delta = delta.numel() // x.numel()
    _check(lib().rb_dyt(_p(x), _p(delta), c_int(n_delta), c_longlong(x.numel()), _p(w), _p(b), _p(alpha), c_int(dt(w)),
                        _p(out), c_int(dt(out)), _p(row_idx), c_int(rows), c_int(h), _stream()), "dyt",
           0.0, float(rows * h * (4 + out.element_size())))


def softcap(x: torch.Tensor, cap: float) -> None:
    """x <- cap tanh(x / cap) in place (float32)."""
    _need(x.dtype == torch.float32 and x.is_contiguous(), "softcap: float32 contiguous")
    _check(lib().rb_softcap(_p(x), c_longlong(x.numel()), c_float(cap), _stream()), "softcap")


def tanh_(x: torch.Tensor) -> None:
    """tanh in place on a block [rows, cols] whose rows may be strided."""
    _need(x.dim() == 2 and x.stride(1) == 1, "tanh_: rows contiguous")
    _check(lib().rb_unary(_p(x), c_int(dt(x)), c_longlong(x.stride(0)), c_int(x.shape[0]), c_int(x.shape[1]), c_int(0),
                          _stream()), "tanh")


def head_norm_gate(o: torch.Tensor, w: torch.Tensor, gate: torch.Tensor, out: torch.Tensor, H: int, dv: int, eps: float,
                   gate_fn: str, out_scale: float = 1.0) -> None:
    """o [T, H, dv] float32 -> out [T, H*dv] (rows may be strided): o over its root mean square per head, times w
    ([dv]: one weight for all heads; [H*dv]: one per head), times sigmoid or silu of gate [T, H*dv], times out_scale."""
    T = o.shape[0]
    _need(o.dtype == torch.float32 and o.is_contiguous() and w.dtype == torch.float32 and w.numel() in (dv, H * dv),
          "head_norm_gate: o and w float32, w one row or one per head")
    _need(gate.dtype == out.dtype and gate.stride(1) == 1 and out.stride(1) == 1, "head_norm_gate: gate and out of one dtype")
    _check(lib().rb_head_norm_gate(_p(o), _p(w), c_int(int(w.numel() == H * dv and H > 1)), _p(gate), c_longlong(gate.stride(0)),
                                   c_int({"sigmoid": 0, "silu": 1}[gate_fn]), _p(out), c_longlong(out.stride(0)),
                                   c_int(dt(out)), c_int(T), c_int(H), c_int(dv), c_float(eps), c_float(out_scale),
                                   _stream()), "head_norm_gate", 0.0, float(T * H * dv * (4 + 2 * out.element_size())))


def shortconv(u: torch.Tensor, w: torch.Tensor, state: torch.Tensor, y: torch.Tensor, cu_q: torch.Tensor,
              entry_slot: torch.Tensor, n_entries: int, max_q_len: int, silu: bool) -> None:
    """y[t, c] = act(sum_j w[c, j] u[t - taps + 1 + j, c]) per request; inputs before the step come from the request's
    slot in state [slots, taps-1, C] float32 (zeros for a new request), which is left holding the last taps-1 inputs."""
    C, taps = w.shape
    _need(w.dtype == torch.float32 and w.is_contiguous() and state.dtype == torch.float32 and state.is_contiguous(),
          "shortconv: float32 taps and state")
    _need(u.shape[1] == C and y.shape[1] == C and u.stride(1) == 1 and y.stride(1) == 1 and u.dtype == y.dtype,
          "shortconv: u and y [T, C] of one dtype")
    _need(tuple(state.shape[1:]) == (taps - 1, C), "shortconv: state [slots, taps-1, C]")
    _check(lib().rb_shortconv(_p(u), c_longlong(u.stride(0)), _p(w), _p(state), _p(y), c_longlong(y.stride(0)), c_int(dt(u)),
                              _p(cu_q), _p(entry_slot), c_int(n_entries), c_int(max_q_len), c_int(C), c_int(taps),
                              c_int(int(silu)), _stream()), "shortconv", 0.0, float(2 * u.shape[0] * C * u.element_size()))


def unit_heads_append(x: torch.Tensor, kv_slot: Optional[torch.Tensor], q_out: torch.Tensor, cache: torch.Tensor,
                      QH: int, KH: int, dk: int, dv: int, page_size: int, eps: float) -> None:
    """x [T, (QH+KH) dk + KH dv]: q and k heads over their root mean square (no weight), q -> q_out [T, QH, dk],
    k and v into the token's cache slot (layout of paged_attention_ref with dv)."""
    _need(x.stride(1) == 1 and x.shape[1] == (QH + KH) * dk + KH * dv and q_out.is_contiguous() and x.dtype == q_out.dtype == cache.dtype,
          "unit_heads_append: x [T, q|k|v], one dtype")
    _check(lib().rb_unit_heads_append(_p(x), c_longlong(x.stride(0)), _p(kv_slot), _p(q_out), _p(cache), c_int(dt(x)),
                                      c_int(x.shape[0]), c_int(QH), c_int(KH), c_int(dk), c_int(dv), c_int(page_size),
                                      c_float(eps), _stream()), "unit_heads_append")


def chunk_attention(ctx, q: torch.Tensor, cache: torch.Tensor, group, out: torch.Tensor, QH: int, KH: int, dk: int, dv: int,
                    chunk: int, scale: float, penalty, out_scale: float = 1.0) -> None:
    """Attention of a step's tokens over the keys of their own chunk, with the logarithmic distance penalty
    (parts/chunk_attention.py).  q [T, QH, dk], out [T, QH, dv]."""
    n_dec, E = ctx.n_decode, ctx.n_entries
    dec_work = pre_work = (0.0, 0.0)
    if _profiler is not None:
        def work(first, last):
            """(flops, bytes) of entries first..last-1: two products per (query head, visible key) pair, the keys and
            values of the chunks the portion touches read once."""
            pairs = keys = toks = 0.0
            for e in range(first, last):
                n, s0 = ctx.q_start[e + 1] - ctx.q_start[e], ctx.start_pos[e]
                pairs += sum((p % chunk) + 1 for p in range(s0, s0 + n)) if n <= 4096 else n * (chunk + 1) / 2
                keys += (s0 + n) - (s0 // chunk * chunk)
                toks += n
            return 2.0 * QH * (dk + dv) * pairs, (keys * KH * (dk + dv) + toks * QH * (dk + dv)) * q.element_size()
        dec_work, pre_work = work(0, n_dec), work(n_dec, E)
    if q.dtype != torch.bfloat16 or dk != dv or dk % 8 or dk > 256:
        # 32-bit, or value heads of their own size: the plain kernel
        paged_attention_ref(q, cache, group.block_table, ctx.tok_entry, ctx.positions, out, QH, KH, dk, group.page_size, 0, scale,
                            work=(dec_work[0] + pre_work[0], dec_work[1] + pre_work[1]), dv=dv, chunk=chunk, penalty=penalty,
                            out_scale=out_scale)
        return
    gc = fa_group_chunk(QH // KH)
    if n_dec:
        # a token's keys are those of its chunk: at most chunk / 64 tiles; they are split over CTAs while that fills the device
        ctas = n_dec * KH * (QH // KH // gc)
        n_splits = max(1, min(DECODE_SLOTS // max(ctas, 1), -(-chunk // 256), 16))
        fa_decode(q, cache, group.block_table, ctx.cu_q, ctx.kv_len, out, 0, n_dec, 0, n_splits, QH, KH, dk, group.page_size, 0,
                  scale, work=dec_work, chunk=chunk, penalty=penalty, out_scale=out_scale)
    if E > n_dec and dk == 128 and chunk % 64 == 0 and USE_TC_ATTENTION and USE_TMA_ATTENTION and tma_pages(group.page_size):
        # heads of 128, chunks in whole key tiles: the tcgen05 kernel
        fa_prefill_tc(q, cache, group.block_table, ctx.cu_q, ctx.kv_len, out, n_dec, E - n_dec,
                      [ctx.q_start[e + 1] - ctx.q_start[e] for e in range(n_dec, E)], QH, KH, dk, group.page_size, 0, scale,
                      work=pre_work, chunk=chunk, penalty=penalty, out_scale=out_scale)
    elif E > n_dec:
        tpt = 64 // gc
        n_tiles = sum(-(-(ctx.q_start[e + 1] - ctx.q_start[e]) // tpt) for e in range(n_dec, E))
        fa_prefill(q, cache, group.block_table, ctx.cu_q, ctx.kv_len, out, n_dec, E - n_dec, n_tiles, QH, KH, dk, group.page_size,
                   0, scale, work=pre_work, chunk=chunk, penalty=penalty, out_scale=out_scale)


def residual_outnorm(x: torch.Tensor, y: torch.Tensor, w: torch.Tensor, eps: float, mult: float,
                     rounded: Optional[torch.Tensor] = None, extra=None, next_w: Optional[torch.Tensor] = None):
    """x (float32 [rows, h]) += mult * rms(y) * w with y float32 [rows, h] or a stack [S, rows, h] of partial sums
    (added in ascending order) and rms(y) = y / sqrt(mean(y^2) + eps); `rounded` (bfloat16 [rows, h]) receives
    the new x once more, rounded.  extra = (a float32 [rows], src [rows, h]): y[r,:] gets a[r] * src[r,:] added first.
    next_w (float32 [h], the weight of the norm that reads x next): returns (rows, sumsq) as residual_rowscale does -
    bfloat16(x * next_w) and the rows' sums of squares [rows, parts] - so that norm costs no launch; else None."""
    _need(x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 2, "outnorm: x float32 [rows, h] contiguous")
    rows, h = x.shape
    _need(y.dtype == torch.float32 and y.is_contiguous() and y.shape[-1] == h and y.numel() % max(x.numel(), 1) == 0 and y.numel() >= x.numel(),
          "outnorm: y float32 with x's shape (or a stack of it)")
    _need(rounded is None or (rounded.dtype == torch.bfloat16 and rounded.is_contiguous() and rounded.shape == x.shape),
          "outnorm: the rounded copy is bfloat16 of x's shape")
    if rows == 0:
        return None
    ea = es = None
    if extra is not None:
        ea, es = extra
        _need(ea.dtype == torch.float32 and ea.numel() == rows and es.is_contiguous() and tuple(es.shape) == (rows, h),
              "outnorm: the extra term is a float32 factor per row and rows of x's shape")
    n_rows = n_sumsq = None
    parts = 0
    if next_w is not None:
        _need(next_w.dtype == torch.float32 and next_w.is_contiguous() and next_w.numel() == h, "outnorm: the next norm's weight is float32 [h]")
        parts = int(lib().rb_rowscale_parts(c_int(h)))
        n_rows = torch.empty((rows, h), dtype=torch.bfloat16, device=x.device)
        n_sumsq = torch.empty((rows, parts), dtype=torch.float32, device=x.device)
    _check(lib().rb_residual_outnorm(_p(x), _p(y), c_int(y.numel() // x.numel()), c_longlong(x.numel()), _p(w), c_int(dt(w)),
                                     _p(rounded), c_int(rows), c_int(h), c_float(eps), c_float(mult), _p(ea), _p(es),
                                     c_int(dt(es) if es is not None else F32), _p(next_w), _p(n_rows), _p(n_sumsq), c_int(parts), _stream()),
           "residual_outnorm", 0.0, float((y.numel() + 2 * x.numel()) * 4 + (2 * x.numel() if rounded is not None else 0) +
                                          (2 * x.numel() if next_w is not None else 0)))
    return None if next_w is None else (n_rows, n_sumsq)


def round_rows(x: torch.Tensor) -> torch.Tensor:
    """bfloat16 copy of float32 rows."""
    _need(x.dtype == torch.float32 and x.is_contiguous(), "round_rows: float32 contiguous")
    out = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
    _check(lib().rb_round_rows(_p(x), _p(out), c_longlong(x.numel()), _stream()), "round_rows", 0.0, 6.0 * x.numel())
    return out


def norm_heads_append(x: torch.Tensor, qw: torch.Tensor, kw: Optional[torch.Tensor], positions: Optional[torch.Tensor],
                      kv_slot: Optional[torch.Tensor], q_out: torch.Tensor, cache: Optional[torch.Tensor],
                      QH: int, KH: int, d: int, dv: int, q_group: int, k_group: int, values_are_keys: bool, page_size: int,
                      eps: float, temp=None) -> None:
    """x [T, q | k | v] (v absent when the values are the keys): RMS norm of q over groups of q_group columns (d: per
    head with a weight [d]; QH*d: the whole projection) and of k likewise, q times 1 + coef ln(floor((p+1)/every) + 1)
    with temp = (coef, every), q -> q_out [T, QH, d], normalised k and the values (projected, or k before its norm)
    into the token's cache slot.  kv_slot None: only the queries are prepared."""
    _need(x.stride(1) == 1 and q_out.is_contiguous() and x.dtype == q_out.dtype, "norm_heads_append: rows contiguous, one dtype")
    need = QH * d if kv_slot is None else (QH + KH) * d + (0 if values_are_keys else KH * dv)
    _need(x.shape[1] >= need, "norm_heads_append: x holds q | k | v")
    _need(cache is None or cache.dtype == x.dtype, "norm_heads_append: the cache has the activations' dtype")
    _need(kw is None or kw.dtype == qw.dtype, "norm_heads_append: norm weights of one dtype")
    coef, every = (float(temp[0]), int(temp[1])) if temp is not None else (0.0, 0)
    _check(lib().rb_norm_heads_append(_p(x), c_longlong(x.stride(0)), c_int(dt(x)), _p(qw), _p(kw), c_int(dt(qw)),
                                      _p(positions), _p(kv_slot), _p(q_out), _p(cache if kv_slot is not None else None),
                                      c_int(x.shape[0]), c_int(QH), c_int(KH), c_int(d), c_int(dv), c_int(q_group), c_int(k_group),
                                      c_int(int(bool(values_are_keys))), c_int(page_size), c_float(eps), c_float(coef), c_int(every),
                                      _stream()), "norm_heads_append")


MOE_MODES = {"scores": 0, "chosen_logits": 1}


def moe_route(z: torch.Tensor, corr: Optional[torch.Tensor], experts: int, top: int, mode: str = "scores"):
    """z float32 [T, n] router outputs -> (gates float32 [T, experts], ident float32 [T] or None): softmax over all n,
    the `top` largest of score + corr chosen, gates = the chosen scores (zero elsewhere), ident = the sum of the chosen
    scores among the outputs experts..n-1 (experts that are the identity).  mode "chosen_logits": corr is a bias of the
    logits, the `top` largest logits are chosen and gates = the softmax over the chosen logits alone."""
    _need(z.dtype == torch.float32 and z.is_contiguous() and z.dim() == 2, "moe_route: z float32 [T, n]")
    T, n = z.shape
    _need(corr is None or (corr.dtype == torch.float32 and corr.numel() == n), "moe_route: the correction is float32 [n]")
    gates = torch.empty((T, experts), dtype=torch.float32, device=z.device)
    ident = torch.empty((T,), dtype=torch.float32, device=z.device) if n > experts else None
    _check(lib().rb_moe_route(_p(z), _p(corr), _p(gates), _p(ident), c_int(T), c_int(n), c_int(experts), c_int(top), c_int(MOE_MODES[mode]),
                              _stream()), "moe_route")
    return gates, ident


def moe_router(x: torch.Tensor, w: torch.Tensor, corr: Optional[torch.Tensor], experts: int, top: int, mode: str = "scores"):
    """The router's product z = x w^T (32-bit, one fixed order per output) and moe_route's choice in one kernel:
    x [T, h], w [n, h] -> (gates float32 [T, experts], ident float32 [T] or None)."""
    _need(x.is_contiguous() and w.is_contiguous() and x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1],
          "moe_router: x [T, h], w [n, h] contiguous")
    T, n = x.shape[0], w.shape[0]
    _need(corr is None or (corr.dtype == torch.float32 and corr.numel() == n), "moe_router: the correction is float32 [n]")
    gates = torch.empty((T, experts), dtype=torch.float32, device=x.device)
    ident = torch.empty((T,), dtype=torch.float32, device=x.device) if n > experts else None
    _check(lib().rb_moe_router(_p(x), c_int(dt(x)), _p(w), c_int(dt(w)), _p(corr), _p(gates), _p(ident), c_int(T), c_int(x.shape[1]),
                               c_int(n), c_int(experts), c_int(top), c_int(MOE_MODES[mode]), _stream()), "moe_router",
           2.0 * T * n * x.shape[1], float(x.numel() * x.element_size() + w.numel() * w.element_size()))
    return gates, ident


def relu2_gate(u: torch.Tensor, gates: torch.Tensor, ff: int) -> torch.Tensor:
    """act[t, e*ff + c] = relu(u[t, e*ff + c])^2 * gates[t, e], in u's dtype."""
    T, E = gates.shape
    _need(u.is_contiguous() and u.shape == (T, E * ff) and gates.dtype == torch.float32 and gates.is_contiguous(),
          "relu2_gate: u [T, experts * ff], gates float32 [T, experts]")
    act = torch.empty_like(u)
    _check(lib().rb_relu2_gate(_p(u), _p(gates), _p(act), c_int(dt(u)), c_int(T), c_int(E), c_int(ff), _stream()), "relu2_gate",
           0.0, 2.0 * u.numel() * u.element_size())
    return act


def rows_axpy(dst: torch.Tensor, a: torch.Tensor, src: torch.Tensor, store: bool = False) -> None:
    """dst[t,:] (float32) += a[t] * src[t,:]  (store: = instead of +=)."""
    _need(dst.dtype == torch.float32 and dst.is_contiguous() and src.is_contiguous() and dst.shape == src.shape and
          a.dtype == torch.float32 and a.numel() == dst.shape[0], "rows_axpy: dst float32 [T, h], a float32 [T], src [T, h]")
    _check(lib().rb_rows_axpy(_p(dst), _p(a), _p(src), c_int(dt(src)), c_int(dst.shape[0]), c_int(dst.shape[1]),
                              c_int(int(store)), _stream()), "rows_axpy")


def moe_grouped_experts(x: torch.Tensor, gates: torch.Tensor, top: int, w_gate_up: torch.Tensor, w_down: torch.Tensor, ff: int,
                        act: str, dst: torch.Tensor, store: bool = False) -> bool:
    """dst[t] (+)= sum over the experts e that token t chose of gates[t, e] * W_down,e (f(W_gate,e x[t]) * (W_up,e x[t])), computing
    only the chosen (token, expert) pairs: the tokens' rows are copied into an array sorted by expert (every expert's stretch
    padded to whole tiles of 128 rows) and two grouped tensor-core products run over it (csrc/moe_group.cu, rb_gemm_bf16_grouped).
    x [T, h] bfloat16; gates float32 [T, E], zero where an expert was not chosen, at most `top` non-zero a row; w_gate_up
    [2 E ff, h] = [all experts' gate rows; all experts' up rows]; w_down [h, E ff], the experts side by side; dst float32
    [T, h].  Nothing comes back to the host.  Returns False (and does nothing) where this form does not apply."""
    T, h = x.shape
    E = gates.shape[1]
    if x.dtype != torch.bfloat16 or w_gate_up.dtype != torch.bfloat16 or w_down.dtype != torch.bfloat16 or T == 0 or T > 65535:
        return False
    if h % 8 or ff % 8 or x.data_ptr() % 16 or w_gate_up.data_ptr() % 16 or w_down.data_ptr() % 16 or not (x.is_contiguous() and
            w_gate_up.is_contiguous() and w_down.is_contiguous()):
        return False
    _need(tuple(w_gate_up.shape) == (2 * E * ff, h) and tuple(w_down.shape) == (h, E * ff) and gates.dtype == torch.float32 and
          gates.is_contiguous() and dst.dtype == torch.float32 and dst.is_contiguous() and tuple(dst.shape) == (T, h), "moe_grouped_experts: shapes")
    dev = x.device
    tiles = -(-(T * top + E * 127) // 128)
    ints = torch.empty(E + T * E + E + tiles + 1 + T * top, dtype=torch.int32, device=dev)
    count, pos, seg, tile_group, live, rows = torch.split(ints, [E, T * E, E, tiles, 1, T * top])
    w = torch.empty((T, top), dtype=torch.float32, device=dev)
    xs = torch.empty((tiles * 128, h), dtype=torch.bfloat16, device=dev)
    _check(lib().rb_moe_group_plan(_p(x), c_int(dt(x)), _p(gates), _p(count), _p(pos), _p(seg), _p(tile_group), _p(live), _p(rows), _p(w),
                                   _p(xs), c_int(T), c_int(E), c_int(h), c_int(top), c_int(tiles), _stream()), "moe_group_plan",
           0.0, float((1 + top) * T * h * 2))
    global launches
    launches += 2
    inner = torch.empty((tiles * 128, ff), dtype=torch.bfloat16, device=dev)
    _check(lib().rb_gemm_bf16_grouped(_p(xs), _p(w_gate_up), _p(inner), c_int(1), c_int(tiles * 128), c_int(ff), c_int(h), c_int(E),
                                      c_longlong(h), c_longlong(h), c_longlong(ff), _p(tile_group), _p(live), c_int(GLU_ACTS[act]), _stream()),
           f"gemm+swiglu grouped {2 * ff}x{h}", 4.0 * T * top * ff * h, 2.0 * (T * top * (h + ff) + 2 * E * ff * h))
    y = torch.empty((tiles * 128, h), dtype=torch.float32, device=dev)
    _check(lib().rb_gemm_bf16_grouped(_p(inner), _p(w_down), _p(y), c_int(0), c_int(tiles * 128), c_int(h), c_int(ff), c_int(E),
                                      c_longlong(ff), c_longlong(E * ff), c_longlong(h), _p(tile_group), _p(live), c_int(0), _stream()),
           f"gemm grouped {h}x{ff}", 2.0 * T * top * ff * h, 2.0 * (T * top * ff + E * ff * h) + 4.0 * T * top * h)
    _check(lib().rb_moe_group_combine(_p(dst), _p(y), _p(rows), _p(w), c_int(T), c_int(h), c_int(top), c_int(int(store)), _stream()),
           "moe_group_combine", 0.0, float(T * h * 4 * (top + 2)))
    return True


GLU_ACTS = {"silu": 0, "gelu_tanh": 1}


def glu_act(gu: torch.Tensor, out: torch.Tensor, act: str = "silu", bias: Optional[torch.Tensor] = None,
            gates: Optional[torch.Tensor] = None, ff: int = 0) -> None:
    """gu [T, gate: F | up: F] (float32 or the activation dtype; rows may be strided) -> out [T, F]:
    f(gate + bias) * (up + bias) * gates[t, c // ff].  bias float32 [2F] and gates float32 [T, F // ff] are optional."""
    T, F_ = out.shape
    _need(gu.dim() == 2 and gu.stride(1) == 1 and gu.shape == (T, 2 * F_) and out.is_contiguous(), "glu_act: gu [T, 2F], out [T, F]")
    _need(bias is None or (bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == 2 * F_), "glu_act: the bias is float32 [2F]")
    _need(gates is None or (ff > 0 and F_ % ff == 0 and gates.dtype == torch.float32 and gates.is_contiguous() and
                            tuple(gates.shape) == (T, F_ // ff)), "glu_act: gates float32 [T, F / ff]")
    _check(lib().rb_glu_act(_p(gu), c_longlong(gu.stride(0)), c_int(dt(gu)), _p(bias), c_int(GLU_ACTS[act]), _p(gates), c_int(ff),
                            _p(out), c_int(dt(out)), c_int(T), c_int(F_), _stream()), f"glu_act {act}",
           0.0, float(T * F_ * (2 * gu.element_size() + out.element_size())))


def add_row_vector(x: torch.Tensor, b: torch.Tensor) -> None:
    """x[t, :] += b for every row of the float32 stream."""
    _need(x.dtype == torch.float32 and x.is_contiguous() and b.is_contiguous() and b.numel() == x.shape[1], "add_row_vector: x float32 [T, h], b [h]")
    _check(lib().rb_add_row_vector(_p(x), _p(b), c_int(dt(b)), c_int(x.shape[0]), c_int(x.shape[1]), _stream()), "add_row_vector")


def diff_heads(a: torch.Tensor, out: torch.Tensor, lam: float, eps: float, out_scale: float, H: int, G: int, dv: int,
               gate: Optional[torch.Tensor] = None) -> None:
    """The output stage of differential attention: a [T, 2H, dv] holds the two maps' outputs of every head (map m of head
    g R + r at row (2g + m) R + r, R = H / G); out [T, H, dv] = rms_eps(a1 - lam a2) * out_scale * sigmoid(gate[t, h]).
    gate: float32 rows [T, H] (rows may be strided) or None."""
    T = a.shape[0]
    _need(a.is_contiguous() and out.is_contiguous() and a.dtype == out.dtype and a.numel() == T * 2 * H * dv and
          out.numel() == T * H * dv, "diff_heads: a [T, 2H, dv], out [T, H, dv], one dtype")
    _need(gate is None or (gate.dtype == torch.float32 and gate.dim() == 2 and gate.stride(1) == 1 and gate.shape == (T, H)),
          "diff_heads: the gate is float32 [T, H]")
    _check(lib().rb_diff_heads(_p(a), c_int(dt(a)), c_float(lam), c_float(eps), c_float(out_scale), _p(gate),
                               c_longlong(gate.stride(0) if gate is not None else 0), _p(out), c_int(T), c_int(H), c_int(G),
                               c_int(dv), _stream()), "diff_heads", 0.0, float(3 * T * H * dv * a.element_size()))


def biased_attention(ctx, q: torch.Tensor, cache: torch.Tensor, group, out: torch.Tensor, QH: int, KH: int, dk: int, dv: int,
                     window: int, scale: float, bias: Optional[torch.Tensor], more: Optional[AttentionExtras] = None) -> None:
    """Softmax attention of a step's tokens over their requests' pages, causal or in a sliding window, with a
    learned bias by distance (float32 [QH, rows]; a head's last entry serves every greater distance) added to the scaled
    scores, and value heads of their own size.  q [T, QH, dk], out [T, QH, dv].  more: soft cap, sink, values inside
    the keys, output gate (AttentionExtras); the decode kernel whose tiles come by TMA and the tcgen05 prefill kernel take
    all but values inside the keys."""
    n_dec, E = ctx.n_decode, ctx.n_entries
    dec_work = pre_work = (0.0, 0.0)
    if _profiler is not None:
        def work(first, last):
            """(flops, bytes) of entries first..last-1: two products per (query head, visible key) pair, the visible keys
            and values read once."""
            pairs = keys = toks = 0.0
            for e in range(first, last):
                n, s0 = ctx.q_start[e + 1] - ctx.q_start[e], ctx.start_pos[e]
                full = n * s0 + n * (n + 1) / 2
                pairs += min(full, n * window) if window else full
                keys += min(s0 + n, window + n) if window else s0 + n
                toks += n
            stored = dk if (more is not None and more.v_in_k) else dk + dv
            return 2.0 * QH * (dk + dv) * pairs, (keys * KH * stored + toks * QH * (dk + dv)) * q.element_size()
        dec_work, pre_work = work(0, n_dec), work(n_dec, E)
    if q.dtype != torch.bfloat16 or dk % 8 or dv % 8 or max(dk, dv) > 256:
        # 32-bit, or head sizes the tensor-core kernels do not take: the plain kernel
        paged_attention_ref(q, cache, group.block_table, ctx.tok_entry, ctx.positions, out, QH, KH, dk, group.page_size, window, scale,
                            work=(dec_work[0] + pre_work[0], dec_work[1] + pre_work[1]), dv=dv, bias=bias, more=more)
        return
    gc = fa_group_chunk(QH // KH)
    if n_dec:
        # the keys a token sees (all before it, or its window) are split over CTAs while that fills the device
        ctas = n_dec * KH * (QH // KH // gc)
        keys = min(ctx.max_kv_len, window + 63) if window else ctx.max_kv_len
        per = 256 if ctas * -(-keys // 256) >= DECODE_SLOTS // 2 else 128     # few heads and requests: finer splits fill the device
        n_splits = max(1, min(DECODE_SLOTS // max(ctas, 1), -(-keys // per), 16))
        tma = dk == dv and (more is None or not more.v_in_k) and tma_pages(group.page_size) and USE_TMA_ATTENTION
        if tma and more is not None and (more.sink is not None or more.gate is not None) and n_splits > 1:
            tma = decode_merges_in_cluster(n_dec, QH, KH, dk, n_splits)        # sink and gate enter where the splits come together
        if tma:
            # key size = value size: the kernel whose tiles come by TMA (up to 16 splits merge inside their cluster)
            fa_decode_tma(q, cache, group.block_table, ctx.cu_q, ctx.kv_len, out, 0, n_dec, 0, n_splits, QH, KH, dk, group.page_size,
                          window, scale, work=dec_work, bias=bias, more=more)
        else:
            fa_decode(q, cache, group.block_table, ctx.cu_q, ctx.kv_len, out, 0, n_dec, 0, n_splits, QH, KH, dk, group.page_size,
                      window, scale, work=dec_work, dv=dv, bias=bias, more=more)
    if E > n_dec and dk == 128 and dv == 128 and (more is None or not more.v_in_k) and USE_TC_ATTENTION and USE_TMA_ATTENTION and \
            tma_pages(group.page_size):
        # heads of 128: the tcgen05 kernel
        fa_prefill_tc(q, cache, group.block_table, ctx.cu_q, ctx.kv_len, out, n_dec, E - n_dec,
                      [ctx.q_start[e + 1] - ctx.q_start[e] for e in range(n_dec, E)], QH, KH, dk, group.page_size, window, scale,
                      work=pre_work, bias=bias, more=more)
    elif E > n_dec:
        tpt = 64 // gc
        n_tiles = sum(-(-(ctx.q_start[e + 1] - ctx.q_start[e]) // tpt) for e in range(n_dec, E))
        fa_prefill(q, cache, group.block_table, ctx.cu_q, ctx.kv_len, out, n_dec, E - n_dec, n_tiles, QH, KH, dk, group.page_size,
                   window, scale, work=pre_work, dv=dv, bias=bias, more=more)


def rotary_heads_append(x: torch.Tensor, bias: Optional[torch.Tensor], positions: torch.Tensor, freq: Optional[torch.Tensor],
                        rot: int, mag: float, kv_slot: Optional[torch.Tensor], q_out: torch.Tensor, cache: torch.Tensor,
                        QH: int, KH: int, dk: int, dv: int, page_size: int, vmix: int = 0,
                        lam: Optional[torch.Tensor] = None, v_first: Optional[torch.Tensor] = None, half_split: bool = False) -> None:
    """x [T, q | k | v | ...] (float32 or bfloat16 rows): + bias (float32 over q | k | v), neighbouring dimensions (2i, 2i+1)
    (with half_split: dimensions i and i + rot/2)
    of the first `rot` of every q and k head rotated by position * freq[i] with cosine and sine times `mag`, q -> q_out
    [T, QH, dk], k and v into the token's cache slot (pages [K: KH x page x dk | V: KH x page x dv]).  vmix 1: the values
    (with bias) are also left in v_first (float32 [T, KH * dv]); vmix 2: v <- (1 - lam) v + lam v_first first."""
    _need(x.stride(1) == 1 and x.shape[1] >= (QH + KH) * dk + KH * dv and q_out.is_contiguous() and cache.dtype == q_out.dtype,
          "rotary_heads_append: x holds q | k | v, rows contiguous; q_out and the cache of one dtype")
    _need(bias is None or (bias.dtype == torch.float32 and bias.numel() >= (QH + KH) * dk + KH * dv), "rotary_heads_append: a float32 bias over q | k | v")
    _need(freq is None or (freq.dtype == torch.float32 and freq.numel() >= rot // 2), "rotary_heads_append: float32 frequencies, one a pair")
    _need(v_first is None or (v_first.dtype == torch.float32 and v_first.is_contiguous() and v_first.numel() == x.shape[0] * KH * dv),
          "rotary_heads_append: the first values are float32 [T, KH * dv]")
    _need(lam is None or (lam.dtype == torch.float32 and lam.numel() == 1), "rotary_heads_append: the mixing weight is one float32 number")
    _check(lib().rb_rotary_heads_append(_p(x), c_longlong(x.stride(0)), c_int(dt(x)), _p(bias), _p(positions), _p(freq), c_int(rot),
                                        c_float(mag), _p(kv_slot), _p(q_out), _p(cache), c_int(dt(q_out)), c_int(x.shape[0]), c_int(QH),
                                        c_int(KH), c_int(dk), c_int(dv), c_int(page_size), c_int(vmix), _p(lam), _p(v_first), c_int(int(half_split)),
                                        _stream()),
           "rotary_heads_append", 0.0, float(x.shape[0] * ((QH + KH) * dk + KH * dv) * (x.element_size() + q_out.element_size())))


def latent_prep(x: torch.Tensor, na: int, nc: int, nr: int, wa: torch.Tensor, wc: torch.Tensor, eps: float, positions: torch.Tensor,
                freq: Optional[torch.Tensor], rot: int, mag: float, kv_slot: Optional[torch.Tensor], a_out: torch.Tensor,
                cache: torch.Tensor, page_size: int) -> None:
    """x [T, a | c | r] (float32 or bfloat16 rows): a_out = rms(a) * wa; the token's cache slot (a one-head cache whose
    pages hold keys only, [page, nc + nr]) gets rms(c) * wc and r with its first `rot` dimensions rotated in neighbouring
    pairs.  Norm weights float32, as stored."""
    _need(x.stride(1) == 1 and x.shape[1] >= na + nc + nr and a_out.is_contiguous() and a_out.shape[-1] == na, "latent_prep: x holds a | c | r")
    _need(wa.dtype == torch.float32 and wc.dtype == torch.float32 and wa.numel() == na and wc.numel() == nc, "latent_prep: float32 norm weights")
    _need(cache.dtype == a_out.dtype, "latent_prep: the cache has the activations' dtype")
    _check(lib().rb_latent_prep(_p(x), c_longlong(x.stride(0)), c_int(dt(x)), c_int(na), c_int(nc), c_int(nr), _p(wa), _p(wc), c_float(eps),
                                _p(positions), _p(freq), c_int(rot), c_float(mag), _p(kv_slot), _p(a_out), _p(cache), c_int(dt(a_out)),
                                c_int(x.shape[0]), c_int(page_size), _stream()),
           "latent_prep", 0.0, float(x.shape[0] * (na + nc + nr) * (x.element_size() + a_out.element_size())))


def rotate_pairs(src: torch.Tensor, dst: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor, rot: int, mag: float) -> None:
    """src, dst [T, H, width] views (last dimension contiguous, strides of their own, one dtype): dst = src with neighbouring
    dimensions (2i, 2i+1) of the first `rot` rotated by position * freq[i], cosine and sine times `mag`."""
    _need(src.dim() == 3 and dst.shape == src.shape and src.stride(2) == 1 and dst.stride(2) == 1 and src.dtype == dst.dtype,
          "rotate_pairs: two [T, H, width] views of one dtype")
    T, H, width = src.shape
    _check(lib().rb_rotate_pairs(_p(src), c_longlong(src.stride(0)), c_longlong(src.stride(1)), _p(dst), c_longlong(dst.stride(0)),
                                 c_longlong(dst.stride(1)), c_int(dt(src)), _p(positions), _p(freq), c_int(T), c_int(H), c_int(width),
                                 c_int(rot), c_float(mag), _stream()), "rotate_pairs", 0.0, float(2 * src.numel() * src.element_size()))


def heads_linear(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, tail=None, gate: Optional[torch.Tensor] = None) -> None:
    """y[t, h, :n_out] = w[h] x[t, h, :n_in] for every head: x [T, H, n_in (+ tail)] and y [T, H, n_out (+ tail)] views (last
    dimension contiguous), w [H, n_out, n_in] contiguous.  tail = (positions, freq, rot, mag): the columns of x behind
    the head's inputs go behind the head's outputs in y, their first `rot` dimensions rotated in neighbouring pairs.
    bfloat16: one tensor-core launch for all heads (tail included); else the plain kernel (32-bit sums in ascending order)
    and `rotate_pairs`.  Either way a token's result does not depend on the batch.  gate: float32 rows [T, H * n_out]
    (rows may be strided) whose sigmoid multiplies the outputs before they are rounded."""
    _need(x.dim() == 3 and y.dim() == 3 and w.dim() == 3 and w.is_contiguous() and x.stride(2) == 1 and y.stride(2) == 1, "heads_linear: views")
    T, H = x.shape[0], x.shape[1]
    n_out, n_in = w.shape[1], w.shape[2]
    n_tail = x.shape[2] - n_in
    _need(w.shape[0] == H and n_tail >= 0 and tuple(y.shape) == (T, H, n_out + n_tail) and x.dtype == y.dtype and
          (n_tail == 0 or tail is not None), "heads_linear: shapes")
    _need(gate is None or (gate.dtype == torch.float32 and gate.dim() == 2 and gate.stride(1) == 1 and gate.shape == (T, H * n_out)),
          "heads_linear: the gate is float32 [T, heads * outputs]")
    if T == 0:
        return
    g_row = c_longlong(gate.stride(0) if gate is not None else 0)
    positions, freq, rot, mag = tail if (tail is not None and n_tail) else (None, None, 0, 1.0)
    if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and n_in % 8 == 0 and x.stride(0) % 8 == 0 and x.stride(1) % 8 == 0 and \
            x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0:
        _check(lib().rb_heads_linear_mma(_p(x), c_longlong(x.stride(0)), c_longlong(x.stride(1)), _p(w), _p(y), c_longlong(y.stride(0)),
                                         c_longlong(y.stride(1)), c_int(T), c_int(H), c_int(n_in), c_int(n_out), c_int(n_tail), c_int(rot),
                                         _p(positions), _p(freq), c_float(mag), _p(gate), g_row, _stream()),
               f"heads_linear {n_out}x{n_in}", 2.0 * T * H * n_in * n_out,
               float(H * n_in * n_out * 2 + T * H * (n_in + n_out + 2 * n_tail) * 2))
        return
    _check(lib().rb_heads_linear(_p(x), c_longlong(x.stride(0)), c_longlong(x.stride(1)), c_int(dt(x)), _p(w), c_int(dt(w)), _p(y),
                                 c_longlong(y.stride(0)), c_longlong(y.stride(1)), c_int(T), c_int(H), c_int(n_in), c_int(n_out), _p(gate), g_row,
                                 _stream()),
           f"heads_linear {n_out}x{n_in}", 2.0 * T * H * n_in * n_out,
           float(H * n_in * n_out * w.element_size() + T * H * (n_in + n_out) * x.element_size()))
    if n_tail:
        rotate_pairs(x[:, :, n_in:], y[:, :, n_out:], positions, freq, rot, mag)


RECURRENCE_FORMS = {"diagonal": 0, "delta_old_state": 1, "delta_gated_state": 2}
RECURRENCE_GATES = {"sigmoid_root": 0, "exp_sigmoid": 1, "exp_softplus": 2}


def recurrence(form: str, gate: str, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, z: torch.Tensor,
               z_bias: Optional[torch.Tensor], state: torch.Tensor, out: torch.Tensor, cu_q: torch.Tensor,
               entry_slot: torch.Tensor, n_entries: int, H: int, Hk: int, dk: int, dv: int, *, gate_param: float = 0.0,
               q_scale: float = 1.0, unit_qk: bool = False, a_pre: Optional[torch.Tensor] = None,
               a_bias: Optional[torch.Tensor] = None, b_pre: Optional[torch.Tensor] = None,
               rate: Optional[torch.Tensor] = None, max_q_len: int = 1 << 30, gate_per_head: bool = False) -> None:
    """The token-by-token recurrence over state [slots, H, dk, dv] (float32) of csrc/recurrence.cu.  q, k [T, Hk*dk],
    v [T, H*dv], a_pre [T, H*dk], b_pre [T, H] in the activation dtype (rows may be strided); z [T, H*dk] float32;
    z_bias, a_bias [H*dk] and rate [H] float32; out [T, H, dv] float32.  max_q_len: the step's longest portion (the
    default says "unknown: may be long").  gate_per_head: one gate per head and token, z [T, H] and z_bias [H]."""
    _need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (H, dk, dv),
          "recurrence: state float32 [slots, H, dk, dv]")
    _need(out.dtype == torch.float32 and out.is_contiguous() and z.dtype == torch.float32, "recurrence: out and z float32")
    for t in (q, k, v, z, a_pre, b_pre):
        _need(t is None or t.stride(-1) == 1, "recurrence: rows contiguous")
    _need(q.dtype == k.dtype == v.dtype, "recurrence: q, k, v of one dtype")
    for t in (z_bias, a_bias, rate):
        _need(t is None or (t.dtype == torch.float32 and t.is_contiguous()), "recurrence: small vectors float32")
    ld = lambda t: c_longlong(t.stride(0) if t is not None else 0)
    T = q.shape[0]
    # a step with a portion longer than one tile has its gates and unit vectors prepared ahead, in parallel over the
    # step's tokens, into a scratch buffer (a decode step, whose captured form has max_q_len 1, never takes it)
    prep = None
    if max_q_len > int(lib().rb_recurrence_tile(c_int(dk))):
        prep = torch.empty(T * H * int(lib().rb_recurrence_record_floats(c_int(RECURRENCE_FORMS[form]), c_int(dk), c_int(dv))),
                           dtype=torch.float32, device=q.device)
    _check(lib().rb_recurrence(c_int(RECURRENCE_FORMS[form]), c_int(RECURRENCE_GATES[gate]), c_int(dt(q)),
                               _p(q), ld(q), _p(k), ld(k), _p(v), ld(v), _p(z), ld(z), _p(z_bias), c_int(int(gate_per_head)),
                               _p(a_pre), ld(a_pre), _p(a_bias), _p(b_pre), ld(b_pre), _p(rate),
                               c_float(gate_param), c_float(q_scale), c_int(int(unit_qk)),
                               _p(state), _p(out), _p(cu_q), _p(entry_slot), c_int(n_entries), c_int(H), c_int(Hk),
                               c_int(dk), c_int(dv), _p(prep), c_int(T), c_int(max_q_len), _stream()), f"recurrence {form}",
           6.0 * T * H * dk * dv, float(T * H * (2 * dk + 2 * dv) * 4 + 2 * n_entries * H * dk * dv * 4))
    if prep is not None:
        global launches
        launches += 1                      # the preparation kernel


def random_normal(out: torch.Tensor, base: int, mean: float, std: float) -> None:
    """out[i] = mean + std * n_i, n_i the i-th normal of the counter stream that starts at `base`
    (weights/random.py states the function); out float32 or bfloat16, contiguous."""
    _need(out.is_contiguous(), "random_normal: contiguous tensor")
    _check(lib().rb_random_normal(_p(out), c_int(dt(out)), c_longlong(out.numel()), ctypes.c_ulonglong(base & ((1 << 64) - 1)),
                                  ctypes.c_double(mean), ctypes.c_double(std), _stream()), "random_normal")


def random_ints(out: torch.Tensor, base: int) -> None:
    _need(out.is_contiguous() and out.dtype == torch.int32, "random_ints: contiguous int32 tensor")
    _check(lib().rb_random_ints(_p(out), c_longlong(out.numel()), ctypes.c_ulonglong(base & ((1 << 64) - 1)), _stream()),
           "random_ints")


def kernel_error(reset: bool = True) -> int:
    """The error word that a kernel sets when one of its bounded waits gives up (0 = none).
    Synchronises the device."""
    words = [int(fn(c_int(int(reset)))) for fn in (lib().rb_gemm_error, lib().rb_attn_error, lib().rb_attn_tc_error,
                                                   lib().rb_selftest_error)]
    if reset and any(words):
        lib().rb_status_clear()
    return next((w for w in words if w), 0)


_status_word = None
STATUS_UNITS = {1: "tensor-core product (gemm_tc.cu)", 2: "paged attention (attention_tma.cu)",
                3: "tensor-core prefill attention (attention_tc.cu)", 4: "bounded-wait self-test (selftest.cu)"}


def status_word() -> int:
    """The host's copy of the kernels' error word: 0, or the code of the first bounded wait that gave up.
    A plain load from pinned memory that the kernels write to; no call into the device, no synchronisation.
    What it shows is complete for every kernel the host has already waited for."""
    global _status_word
    if _status_word is None:
        fn = lib().rb_status_host
        fn.restype = ctypes.POINTER(c_int)
        ptr = fn()
        if not ptr:
            raise KernelError(f"status word: {lib().rb_last_error().decode()}")
        _status_word = ptr
    return int(_status_word[0])


def describe_status(code: int) -> str:
    unit, where = (code >> 16) & 0xFF, code & 0xFF
    return f"a bounded wait gave up at point {where} of the {STATUS_UNITS.get(unit, f'unit {unit}')}"


def clear_status() -> int:
    """Clear the status word and the kernels' own words after an error was handled (synchronises the device)."""
    status_word()
    return int(lib().rb_status_clear())


def test_bounded_wait(limit_ns: int, gave_up: Optional[torch.Tensor] = None) -> None:
    """Launch the self-test kernel whose wait nobody answers (selftest.cu); it gives up after `limit_ns`."""
    status_word()                       # the word must be bound before a kernel can write it
    _check(lib().rb_test_bounded_wait(ctypes.c_ulonglong(int(limit_ns)), _p(gave_up), _stream()), "test_bounded_wait")


def sample_params_size() -> int:
    return int(lib().rb_sample_params_size())
