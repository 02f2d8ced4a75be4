"""The compiled sm_100a kernels, called with torch tensors.

The library is plain C (``csrc/*.cu``), loaded with ctypes; each wrapper
checks types and layouts, passes raw device pointers and the current
stream, and raises :class:`KernelError` with the library's message when a
launcher refuses its arguments.  There is no other implementation behind
these functions: without the compiled library, or on a device that is not
sm_100, they raise.
"""

from __future__ import annotations

import ctypes
import functools
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

F32, BF16 = 0, 1
EPI_NONE, EPI_SOFTCAP, EPI_GEGLU = 0, 1, 2
EPI_SWIGLU = 4          # the gated epilogue with SiLU (weight-streaming and paired tcgen05 products)
EPI_RELU2 = 5           # the square of max(y, 0), value by value (the same two products)
# the clipped gate, g sigmoid(1.702 g) (u + 1) with g = min(g, cap), u = clamp(u, -cap, cap): the
# products' ``cap`` carries the limit (the same two products)
EPI_CLIPPED = 6
EPI_GELU = 7            # the exact (erf) gelu, value by value (the same two products)
GATED_EPILOGUES = (EPI_GEGLU, EPI_SWIGLU, EPI_CLIPPED)
ROPE_HALF_SPLIT, ROPE_INTERLEAVED = 0, 1
ACT_GELU_TANH, ACT_SILU = 0, 1          # of the gated feed-forward
ACT_RELU_SQUARED = 2                    # of the feed-forward without a gate (activate)
ACT_TANH = 3                            # tanh, value by value (activate)
GATE_SILU, GATE_SIGMOID = 0, 1          # of head_norm_gate
SCORE_SOFTMAX_TOP, SCORE_SIGMOID = 0, 1     # of the routers: what a chosen expert's weight is
FORM_CLIPPED_GATED, FORM_PLAIN_GELU = 0, 1  # of the routed experts: what an expert computes

_lib = None


class KernelError(RuntimeError):
    pass


def library():
    """Load (compiling first if needed) the kernel library."""
    global _lib
    if _lib is not None:
        return _lib
    from ..csrc.build import ensure_built
    path = ensure_built()
    lib = ctypes.CDLL(path)
    lib.sib_last_error.restype = ctypes.c_char_p
    lib.sib_attention_rows_scratch_bytes.restype = c_longlong
    if lib.sib_compiled_arch() != 100:
        raise KernelError(f"{path} was not compiled for sm_100a")
    _lib = lib
    return lib


def require_device(device: torch.device) -> None:
    """Fail loudly unless ``device`` is a CUDA device of compute capability 10.x."""
    if device.type != "cuda" or not torch.cuda.is_available():
        raise KernelError("strata_inference_b200 runs on an sm_100 CUDA device only; "
                          f"got device '{device}' (there is no CPU path)")
    major, minor = torch.cuda.get_device_capability(device)
    if major != 10:
        raise KernelError(f"strata_inference_b200 is compiled for sm_100a; device '{device}' "
                          f"has compute capability {major}.{minor}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> c_void_p:
    """The current stream of the current device (asked for at every launch: it changes
    under graph capture).  torch's raw getter costs a fraction of a microsecond, the Stream
    object several."""
    if _raw_stream is not None:
        return c_void_p(_raw_stream(torch.cuda.current_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"element type {dtype} is not supported (float32 and bfloat16 are)")


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


_launches = 0


def launch_count() -> int:
    """How many launcher calls of this library succeeded so far in this process
    (a launcher that merges split partial results launches two kernels and counts once)."""
    return _launches


def _check(rc: int) -> None:
    global _launches
    if rc != 0:
        raise KernelError(library().sib_last_error().decode())
    _launches += 1


def _want(t: torch.Tensor, dtype: torch.dtype, name: str, contiguous: bool = True) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name}: expected a CUDA tensor")
    if t.dtype != dtype:
        raise KernelError(f"{name}: expected {dtype}, got {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name}: expected a contiguous tensor")


# --------------------------------------------------------------------------
# Per-kernel timing.  Inside ``with KernelProfile() as prof:`` every launcher of this
# module (and whatever else is wrapped in ``prof.region``) is bracketed by CUDA events;
# ``prof.rows()`` then gives, per kernel class, the calls, the device time and the bytes
# and operations that the work needs by its shapes.  Outside such a block the wrappers
# cost one comparison.  The reference's counterpart is a device synchronisation and a
# wall-clock figure per layer (src/model/layer.rs:1265,1365-1375).

_profile: Optional["KernelProfile"] = None
# Set while a chain of deferred steps is being collected (parts/base.py ProductChain): called
# before any other launch of this module, so that the chain's kernel runs first.
_pending: Optional[Callable[[], None]] = None


def set_pending(flush: Optional[Callable[[], None]]) -> None:
    global _pending
    _pending = flush


class KernelProfile:
    """``plan``: an earlier profile of the same launch sequence.  With a plan the events
    are made for recording inside a CUDA graph (they are re-recorded by every replay) and
    each launch takes its kernel class and work from the plan, in order, instead of
    working them out (which may read device memory and cannot be done while capturing)."""

    def __init__(self, plan: Optional["KernelProfile"] = None):
        self.events: List[Tuple[str, torch.cuda.Event, torch.cuda.Event, float, float]] = []
        self.plan = [(n, b, f) for n, _, _, b, f in plan.events] if plan is not None else None
        self._next = 0

    def __enter__(self) -> "KernelProfile":
        global _profile
        self._outer, _profile = _profile, self
        return self

    def __exit__(self, *exc) -> None:
        global _profile
        _profile = self._outer

    def planned(self) -> Tuple[str, float, float]:
        item = self.plan[self._next % len(self.plan)]
        self._next += 1
        return item

    def region(self, name: str, nbytes: float, flops: float):
        return _Region(self, name, nbytes, flops)

    def rows(self, last: Optional[int] = None) -> List[Dict]:
        """One row per kernel class, longest first (synchronises the device).  ``last``:
        only the last so many launches (the ones a graph replays)."""
        torch.cuda.synchronize()
        table: Dict[str, Dict] = {}
        for name, start, end, nbytes, flops in (self.events[-last:] if last else self.events):
            r = table.setdefault(name, {"name": name, "calls": 0, "ms": 0.0, "bytes": 0.0,
                                        "flops": 0.0})
            r["calls"] += 1
            r["ms"] += start.elapsed_time(end)
            r["bytes"] += nbytes
            r["flops"] += flops
        return sorted(table.values(), key=lambda r: -r["ms"])


class _Region:
    def __init__(self, prof, name, nbytes, flops):
        self.prof = prof
        if prof.plan is not None:
            name, nbytes, flops = prof.planned()
        self.name, self.nbytes, self.flops = name, nbytes, flops

    def __enter__(self):
        external = self.prof.plan is not None
        self.start = torch.cuda.Event(enable_timing=True, external=external)
        self.end = torch.cuda.Event(enable_timing=True, external=external)
        self.start.record()
        return self

    def __exit__(self, *exc):
        self.end.record()
        self.prof.events.append((self.name, self.start, self.end, float(self.nbytes),
                                 float(self.flops)))


def profile_region(name: str, nbytes: float, flops: float):
    """A region of the active profile, or nothing when none is active."""
    return _profile.region(name, nbytes, flops) if _profile is not None else _NO_REGION


class _NoRegion:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NO_REGION = _NoRegion()


def recording_allowed() -> bool:
    """False while a profile without a plan is active: its events and the work it reads
    from the device cannot go into a CUDA graph, so steps are not recorded meanwhile."""
    return _profile is None or _profile.plan is not None


def _nbytes(*tensors) -> int:
    return sum(t.numel() * t.element_size() for t in tensors if t is not None)


def _timed(work: Callable):
    """Wrap a launcher: under an active profile it is timed and ``work(*args)`` gives
    (kernel class, bytes, operations) from the call's arguments."""
    def deco(fn):
        @functools.wraps(fn)
        def wrapper(*args, **kw):
            if _pending is not None:
                _pending()          # deferred work that this launch may depend on goes first
            if _profile is None:
                return fn(*args, **kw)
            name, nbytes, flops = ("", 0, 0) if _profile.plan is not None else work(*args, **kw)
            with _profile.region(name, nbytes, flops):
                return fn(*args, **kw)
        return wrapper
    return deco


def _attention_cache_work(kind, row_pos, k_pool, n_heads, head_dim, window, rows, value_dim=None,
                          chunk=0):
    """Keys and values a row at ``row_pos`` reads from the cache (reads the positions back:
    only done under a profile)."""
    seen = row_pos.to(torch.int64) + 1
    if chunk > 0:
        seen = row_pos.to(torch.int64) % chunk + 1
    elif window > 0:
        seen = seen.clamp(max=window)
    keys = int(seen.sum().item())
    n_kv = k_pool.shape[1]
    nbytes = keys * n_kv * (head_dim + (value_dim or head_dim)) * k_pool.element_size()
    return kind, nbytes, 4.0 * keys * n_heads * head_dim


def _prompt_work(kind, qkv, seq_len, n_heads, head_dim, window):
    """Prompts from position 0: (query, key) pairs inside the causal mask and the window."""
    pairs = 0
    for n in seq_len.to(torch.int64).tolist():
        if window and n > window:
            pairs += window * (window + 1) // 2 + (n - window) * window
        else:
            pairs += n * (n + 1) // 2
    return kind, _nbytes(qkv) + qkv.shape[0] * n_heads * head_dim * qkv.element_size(), \
        4.0 * pairs * n_heads * head_dim


# --------------------------------------------------------------------------

@_timed(lambda tokens, table, scale, out: ("embed_rows", 2 * _nbytes(out), 0))
def embed_rows(tokens: torch.Tensor, table: torch.Tensor, scale: float,
               out: torch.Tensor) -> torch.Tensor:
    """out[r] = scale * table[tokens[r]] in 32-bit."""
    _want(tokens, torch.int32, "tokens")
    _want(out, torch.float32, "out")
    rows, hidden = out.shape
    if tokens.numel() != rows or table.shape[1] != hidden or not table.is_contiguous():
        raise KernelError("embed_rows: shapes do not fit")
    _check(library().sib_embed_rows(_ptr(tokens), _ptr(table), _code(table.dtype), _ptr(out),
                                    c_int(rows), c_int(hidden), c_float(scale), _stream()))
    return out


def randn_fill(dst: torch.Tensor, rows: int, cols: int, group: int, group_stride: int, key: int,
               offset: float, std: float, stored_dtype: torch.dtype) -> None:
    """Seeded normal values for a stored tensor of [rows, cols], written to ``dst``: a view
    [runs, rows a run, cols] into the weight buffer whose runs may lie apart (see
    csrc/randn_fill.cu).  ``key`` is the tensor's 64-bit key."""
    if not dst.is_cuda or dst.stride(2) != 1 or dst.stride(1) != cols:
        raise KernelError("randn_fill: destination runs must be rows of `cols` contiguous elements")
    runs, per_run, _ = dst.shape
    if runs * per_run != rows or (runs > 1 and (per_run != group or dst.stride(0) != group_stride * cols)):
        raise KernelError("randn_fill: the destination view does not fit the run layout")
    _check(library().sib_randn_fill(
        _ptr(dst), _code(dst.dtype), c_longlong(rows), c_longlong(cols),
        c_longlong(group if runs > 1 else 0), c_longlong(group_stride if runs > 1 else 0),
        ctypes.c_ulonglong(key), c_float(offset), c_float(std),
        c_int(BF16 if stored_dtype == torch.bfloat16 else F32), _stream()))


@_timed(lambda gate_up, out, group=0, act=ACT_GELU_TANH: ("gelu_mul", _nbytes(gate_up, out), 0))
def gelu_mul(gate_up: torch.Tensor, out: torch.Tensor, group: int = 0,
             act: int = ACT_GELU_TANH) -> torch.Tensor:
    """out[r, i] = act(gate(r, i)) * up(r, i), act the tanh-GELU or SiLU; gate_up rows are
    [gates | ups] (group 0) or groups of ``group`` gates followed by their ups."""
    rows, inter = out.shape
    _want(gate_up, out.dtype, "gate_up")
    _want(out, out.dtype, "out")
    if tuple(gate_up.shape) != (rows, 2 * inter):
        raise KernelError("gelu_mul: gate_up must be [rows, 2 * intermediate]")
    _check(library().sib_gated_mul(_ptr(gate_up), _ptr(out), _code(out.dtype), c_int(rows),
                                   c_int(inter), c_int(group), c_int(act), _stream()))
    return out


@_timed(lambda x, out: ("cast_rows", _nbytes(x, out), 0))
def cast_rows(x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out = x in out's element type (the 32-bit stream as activations)."""
    _want(x, x.dtype, "x")
    _want(out, out.dtype, "out")
    if x.numel() != out.numel():
        raise KernelError("cast_rows: x and out differ in size")
    _check(library().sib_cast_rows(_ptr(x), _code(x.dtype), _ptr(out), _code(out.dtype),
                                   c_longlong(x.numel()), _stream()))
    return out


@_timed(lambda x, cap: ("softcap", 2 * _nbytes(x), 0))
def softcap_(x: torch.Tensor, cap: float) -> torch.Tensor:
    """x = cap * tanh(x / cap) in place (32-bit)."""
    _want(x, torch.float32, "x")
    _check(library().sib_softcap(_ptr(x), c_longlong(x.numel()), c_float(cap), _stream()))
    return x


@_timed(lambda x, gain, eps, out, rows=None: (
    "rms_norm", out.shape[0] * x.shape[1] * x.element_size() + _nbytes(out), 0))
def rms_norm(x: torch.Tensor, gain: torch.Tensor, eps: float, out: torch.Tensor,
             rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[i] = rms(x[rows[i] if rows else i]) * gain; statistics in 32-bit.  ``x`` may be a
    view of the leading columns of a wider buffer."""
    _want(gain, torch.float32, "gain")
    _want(x, x.dtype, "x", contiguous=False)
    _want(out, out.dtype, "out")
    n, hidden = out.shape
    if x.shape[1] != hidden or gain.numel() != hidden or x.stride(1) != 1:
        raise KernelError("rms_norm: shapes do not fit")
    if rows is not None:
        _want(rows, torch.int32, "rows")
        if rows.numel() != n:
            raise KernelError("rms_norm: one row index per output row")
    elif x.shape[0] != n:
        raise KernelError("rms_norm: x and out differ in rows")
    _check(library().sib_rms_norm(_ptr(x), _code(x.dtype), _ptr(rows), _ptr(gain), c_float(eps),
                                  _ptr(out), _code(out.dtype), c_int(n), c_int(hidden),
                                  c_longlong(x.stride(0)), _stream()))
    return out


@_timed(lambda a, post_gain, post_eps, h, pre_gain, pre_eps, out: (
    "add_rms_norm", _nbytes(a, out) + 2 * _nbytes(h), 0))
def add_rms_norm(a: torch.Tensor, post_gain: Optional[torch.Tensor], post_eps: float,
                 h: torch.Tensor, pre_gain: Optional[torch.Tensor], pre_eps: float,
                 out: Optional[torch.Tensor]) -> None:
    """h += rms(a) * post_gain (or a when post_gain is None); out = rms(h) * pre_gain."""
    _want(h, torch.float32, "h")
    _want(a, a.dtype, "a")
    rows, hidden = h.shape
    if tuple(a.shape) != (rows, hidden):
        raise KernelError("add_rms_norm: a and h differ in shape")
    for g, nm in ((post_gain, "post_gain"), (pre_gain, "pre_gain")):
        if g is not None:
            _want(g, torch.float32, nm)
            if g.numel() != hidden:
                raise KernelError(f"add_rms_norm: {nm} has the wrong length")
    if pre_gain is not None:
        if out is None:
            raise KernelError("add_rms_norm: pre_gain needs out")
        _want(out, a.dtype, "out")
    _check(library().sib_add_rms_norm(_ptr(a), _code(a.dtype), _ptr(post_gain), c_float(post_eps),
                                      _ptr(h), _ptr(pre_gain), c_float(pre_eps), _ptr(out),
                                      c_int(rows), c_int(hidden), _stream()))


@_timed(lambda x, w, b, alpha, out, rows=None: (
    "dyt_norm", out.shape[0] * x.shape[1] * x.element_size() + _nbytes(out), 0))
def dyt_norm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, alpha: torch.Tensor,
             out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[i] = tanh(alpha x[rows[i] if rows else i]) * w + b, element by element in 32-bit;
    ``alpha`` is one 32-bit value on the device."""
    _want(x, x.dtype, "x")
    _want(out, out.dtype, "out")
    n, hidden = out.shape
    _f32(w, hidden, "w")
    _f32(b, hidden, "b")
    _f32(alpha, 1, "alpha")
    if x.shape[1] != hidden:
        raise KernelError("dyt_norm: shapes do not fit")
    if rows is not None:
        _want(rows, torch.int32, "rows")
        if rows.numel() != n:
            raise KernelError("dyt_norm: one row index per output row")
    elif x.shape[0] != n:
        raise KernelError("dyt_norm: x and out differ in rows")
    _check(library().sib_dyt_norm(_ptr(x), _code(x.dtype), _ptr(rows), _ptr(w), _ptr(b), _ptr(alpha),
                                  _ptr(out), _code(out.dtype), c_int(n), c_int(hidden), _stream()))
    return out


@_timed(lambda a, post, h, pre, out, scale=1.0: ("add_dyt_norm", _nbytes(a, out) + 2 * _nbytes(h), 0))
def add_dyt_norm(a: torch.Tensor, post, h: torch.Tensor, pre, out: Optional[torch.Tensor],
                 scale: float = 1.0) -> None:
    """h += scale * dyt_post(a) (or scale * a when ``post`` is None); out = dyt_pre(h) (or h as
    activations when ``pre`` is None and out is given).  ``post`` and ``pre``: (w, b, alpha) of
    a Dynamic Tanh, 32-bit on the device."""
    _want(h, torch.float32, "h")
    _want(a, a.dtype, "a")
    rows, hidden = h.shape
    if tuple(a.shape) != (rows, hidden):
        raise KernelError("add_dyt_norm: a and h differ in shape")
    for triple, nm in ((post, "post"), (pre, "pre")):
        if triple is not None:
            _f32(triple[0], hidden, nm + " weight")
            _f32(triple[1], hidden, nm + " bias")
            _f32(triple[2], 1, nm + " alpha")
    if out is not None:
        _want(out, a.dtype, "out")
        if tuple(out.shape) != (rows, hidden):
            raise KernelError("add_dyt_norm: out and h differ in shape")
    elif pre is not None:
        raise KernelError("add_dyt_norm: the next norm needs out")
    pw, pb, pa = post if post is not None else (None, None, None)
    qw, qb, qa = pre if pre is not None else (None, None, None)
    _check(library().sib_add_dyt_norm(_ptr(a), _code(a.dtype), _ptr(pw), _ptr(pb), _ptr(pa), _ptr(h),
                                      _ptr(qw), _ptr(qb), _ptr(qa), _ptr(out), c_int(rows),
                                      c_int(hidden), c_float(scale), _stream()))


@_timed(lambda ctx, table, bigram, last_token, out, *a: ("bigram_embed", 3 * _nbytes(out), 0))
def bigram_embed(ctx, table: torch.Tensor, bigram: torch.Tensor, last_token: torch.Tensor,
                 out: torch.Tensor, scale: float, buckets: int, mul_prev: int, mul_cur: int) -> torch.Tensor:
    """out[r] = scale * table[token] + bigram[(previous * mul_prev + token * mul_cur) mod
    buckets] (row ``buckets`` at a sequence's first position), 32-bit; then
    ``last_token[slot]`` (int32, one per slot) becomes each sequence's last token of the step."""
    _want(out, torch.float32, "out")
    _want(last_token, torch.int32, "last_token")
    rows, hidden = out.shape
    if (ctx.tokens.numel() != rows or table.shape[1] != hidden or tuple(bigram.shape) != (buckets + 1, hidden)
            or not table.is_contiguous() or not bigram.is_contiguous() or table.dtype != bigram.dtype):
        raise KernelError("bigram_embed: shapes do not fit")
    _check(library().sib_bigram_embed(
        _ptr(ctx.tokens), _ptr(table), _ptr(bigram), _code(table.dtype), _ptr(ctx.row_pos),
        _ptr(ctx.row_seq), _ptr(ctx.seq_slot), _ptr(ctx.seq_start), _ptr(ctx.seq_end),
        _ptr(ctx.seq_row0), _ptr(last_token), _ptr(out), c_int(rows), c_int(ctx.n_seqs), c_int(hidden),
        c_float(scale), c_int(buckets), c_longlong(mul_prev), c_longlong(mul_cur), _stream()))
    return out


@_timed(lambda x, out, act: ("activate", _nbytes(x, out), 0))
def activate(x: torch.Tensor, out: torch.Tensor, act: int) -> torch.Tensor:
    """out = act(x) value by value (ACT_RELU_SQUARED: max(x, 0) squared; ACT_TANH)."""
    _want(x, out.dtype, "x")
    _want(out, out.dtype, "out")
    if x.numel() != out.numel():
        raise KernelError("activate: x and out differ in size")
    _check(library().sib_activate(_ptr(x), _ptr(out), _code(out.dtype), c_longlong(x.numel()),
                                  c_int(act), _stream()))
    return out


@_timed(lambda a, b, out: ("pair_rows", _nbytes(a, b, out), 0))
def pair_rows(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[r] = [a[r] | b[r]] in out's element type; a and b are 32-bit ``[rows, hidden]``."""
    _want(a, torch.float32, "a")
    _want(b, torch.float32, "b")
    _want(out, out.dtype, "out")
    rows, hidden = a.shape
    if tuple(b.shape) != (rows, hidden) or tuple(out.shape) != (rows, 2 * hidden):
        raise KernelError("pair_rows: shapes do not fit")
    _check(library().sib_pair_rows(_ptr(a), _ptr(b), _ptr(out), _code(out.dtype), c_int(rows),
                                   c_int(hidden), _stream()))
    return out


@_timed(lambda t, e, col0, y: ("gelu_gate_rows", _nbytes(t, y) * 2, 0))
def gelu_gate_rows(t: torch.Tensor, e: torch.Tensor, col0: int, y: torch.Tensor) -> torch.Tensor:
    """y[r, j] = gelu_tanh(t[r, j]) * e[r, col0 + j]; ``e`` 32-bit rows (a view is fine)."""
    _want(t, y.dtype, "t")
    _want(y, y.dtype, "y")
    _want(e, torch.float32, "e", contiguous=False)
    rows, width = t.shape
    if tuple(y.shape) != (rows, width) or e.shape[0] != rows or e.stride(1) != 1 or e.shape[1] < col0 + width:
        raise KernelError("gelu_gate_rows: shapes do not fit")
    _check(library().sib_gelu_gate_rows(_ptr(t), _ptr(e), c_longlong(e.stride(0)), c_int(col0), _ptr(y),
                                        _code(y.dtype), c_int(rows), c_int(width), _stream()))
    return y


@_timed(lambda a, b, wa, wb, y, eps: ("pair_norm_mean", _nbytes(a, b, y), 0))
def pair_norm_mean(a: torch.Tensor, b: torch.Tensor, wa: torch.Tensor, wb: torch.Tensor,
                   y: torch.Tensor, eps: float) -> torch.Tensor:
    """y = (a / rms(a) * wa + b / rms(b) * wb) / 2 row by row (csrc/norm.cu); statistics and
    the sum are 32-bit."""
    rows, width = y.shape
    for t, nm in ((a, "a"), (b, "b"), (y, "y")):
        _want(t, y.dtype, nm)
        if tuple(t.shape) != (rows, width):
            raise KernelError("pair_norm_mean: shapes do not fit")
    _f32(wa, width, "wa")
    _f32(wb, width, "wb")
    _check(library().sib_pair_norm_mean(_ptr(a), _ptr(b), _ptr(wa), _ptr(wb), _ptr(y), _code(y.dtype),
                                        c_int(rows), c_int(width), c_float(eps), _stream()))
    return y


@_timed(lambda logits, bias, ids, weights, *a: ("router_topk", _nbytes(logits, ids, weights), 0))
def router_topk(logits: torch.Tensor, bias: Optional[torch.Tensor], ids: torch.Tensor,
                weights: torch.Tensor, score: int = SCORE_SOFTMAX_TOP) -> None:
    """Per row of the 32-bit ``logits`` (+ ``bias``): the ``top`` = ids.shape[1] largest (ties: the
    lower index) into ``ids`` (int32) and into ``weights`` the softmax over those alone
    (SCORE_SOFTMAX_TOP) or each one's own sigmoid (SCORE_SIGMOID)."""
    rows, experts = logits.shape
    top = ids.shape[1]
    _want(logits, torch.float32, "logits")
    _want(ids, torch.int32, "ids")
    _f32(weights, rows * top, "weights")
    if bias is not None:
        _f32(bias, experts, "bias")
    if ids.shape[0] != rows:
        raise KernelError("router_topk: one row of choices per row of logits")
    _check(library().sib_router_topk(_ptr(logits), _ptr(bias), _ptr(ids), _ptr(weights), c_int(rows),
                                     c_int(experts), c_int(top), c_int(score), _stream()))


@_timed(lambda x, w, bias, ids, weights, *a: ("router_rows", _nbytes(x, w), 2.0 * x.shape[0] * w.numel()))
def router_rows(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], ids: torch.Tensor,
                weights: torch.Tensor, score: int = SCORE_SOFTMAX_TOP) -> None:
    """Few rows: z = w x (+ ``bias``) with the 32-bit matrix ``w`` ``[experts, width]`` and the
    choice of :func:`router_topk`, in one launch; sums are 32-bit."""
    rows, width = x.shape
    experts, top = w.shape[0], ids.shape[1]
    _want(x, x.dtype, "x", contiguous=False)
    _want(w, torch.float32, "w")
    _want(ids, torch.int32, "ids")
    _f32(weights, rows * top, "weights")
    if bias is not None:
        _f32(bias, experts, "bias")
    if w.shape[1] != width or ids.shape[0] != rows or x.stride(1) != 1:
        raise KernelError("router_rows: shapes do not fit")
    # (with 16 experts and more the logits are made by many blocks and left here for the choice)
    logits = torch.empty((rows, experts), dtype=torch.float32, device=x.device) if experts >= 16 else None
    _check(library().sib_router_rows(_ptr(x), c_longlong(x.stride(0)), _code(x.dtype), _ptr(w), _ptr(bias),
                                     _ptr(ids), _ptr(weights), c_int(rows), c_int(width),
                                     c_int(experts), c_int(top), c_int(score), _ptr(logits), _stream()))


@_timed(lambda gu, y, row_weight, limit, alpha, *a: ("expert_activate", _nbytes(gu, y), 0))
def expert_activate(gu: torch.Tensor, y: torch.Tensor, row_weight: Optional[torch.Tensor],
                    limit: float, alpha: float, form: int = FORM_CLIPPED_GATED,
                    group: int = 0) -> torch.Tensor:
    """FORM_CLIPPED_GATED: y = g * sigmoid(alpha g) * (u + 1), g = min(gate, limit), u = clamp(up,
    -limit, limit), from rows ``[gate (ff) | up (ff)]``; with ``row_weight`` every row times its
    32-bit weight.  FORM_PLAIN_GELU: y = gelu(row_weight * up), the exact gelu, from rows ``[up
    (ff)]``.  ``group`` 8: gates and ups lie interleaved in eights (8 gates, then their 8 ups)."""
    rows, ff = y.shape
    _want(gu, y.dtype, "gu", contiguous=False)
    _want(y, y.dtype, "y")
    if gu.shape[0] != rows or gu.shape[1] != (1 if form == FORM_PLAIN_GELU else 2) * ff or gu.stride(1) != 1:
        raise KernelError("expert_activate: rows of gate | up (or of up alone)")
    if row_weight is not None:
        _f32(row_weight, rows, "row_weight")
    _check(library().sib_expert_activate(_ptr(gu), c_longlong(gu.stride(0)), _ptr(y), _ptr(row_weight),
                                         _code(y.dtype), c_int(rows), c_int(ff), c_float(limit),
                                         c_float(alpha), c_int(form), c_int(group), _stream()))
    return y


_PAIR_ORDER: dict = {}


@_timed(lambda x, w_gu, w_down, ids, weights, base, out, limit, alpha, form=0: (
    "routed_rows", min(ids.numel(), w_down.shape[0]) * (2 if form else 3) * w_down.shape[1] * w_down.shape[2]
    * x.element_size(), (4.0 if form else 6.0) * ids.numel() * w_down.shape[1] * w_down.shape[2]))
def routed_rows(x: torch.Tensor, w_gu: torch.Tensor, w_down: torch.Tensor, ids: torch.Tensor,
                weights: torch.Tensor, base: Optional[torch.Tensor], out: torch.Tensor,
                limit: float, alpha: float, form: int = FORM_CLIPPED_GATED) -> torch.Tensor:
    """The chosen experts of every row, each (row, expert) pair streaming its expert's matrices
    (csrc/routed.cu): ``w_gu`` ``[experts, 2 ff, width]`` (gate rows, then up rows), ``w_down``
    ``[experts, width, ff]``; out = base + sum_k weights[r, k] down(act(gate, up)) in 32-bit.
    FORM_PLAIN_GELU: ``w_gu`` ``[experts, ff, width]`` (up rows alone), out = base + sum_k
    down(gelu(weights[r, k] * up)).
    With more pairs than half the experts the kernels go expert by expert instead (an expert's
    matrices are read once for all the pairs that chose it)."""
    rows, width = x.shape
    top = ids.shape[1]
    experts, _, ff = w_down.shape
    _want(x, x.dtype, "x", contiguous=False)
    for t, nm in ((w_gu, "w_gu"), (w_down, "w_down"), (out, "out")):
        _want(t, x.dtype, nm)
    _want(ids, torch.int32, "ids")
    _f32(weights, rows * top, "weights")
    if tuple(w_gu.shape) != (experts, (1 if form == FORM_PLAIN_GELU else 2) * ff, width) \
            or w_down.shape[1] != width or x.stride(1) != 1 \
            or tuple(out.shape) != (rows, width) or ids.shape[0] != rows:
        raise KernelError("routed_rows: shapes do not fit")
    if base is not None:
        _want(base, x.dtype, "base")
    mid = torch.empty((rows * top, ff), dtype=x.dtype, device=x.device)
    pairs = rows * top
    if 2 * pairs > experts and (max(width, ff) + 4 + pairs) * 4 <= 48 * 1024:
        # more pairs than half the experts: expert-major, an expert's matrices read once
        order = _PAIR_ORDER.get((pairs, x.device))
        if order is None:
            order = _PAIR_ORDER[(pairs, x.device)] = torch.arange(pairs, dtype=torch.int32, device=x.device)
        ys = torch.empty((pairs, width), dtype=x.dtype, device=x.device)
        _check(library().sib_routed_by_expert(
            _ptr(x), c_longlong(x.stride(0)), _ptr(w_gu), _ptr(w_down), _ptr(ids), _ptr(weights),
            _ptr(base), _ptr(mid), _ptr(ys), _ptr(order), _ptr(out), _code(x.dtype), c_int(rows),
            c_int(width), c_int(ff), c_int(top), c_int(experts), c_float(limit), c_float(alpha),
            c_int(form), _stream()))
        return out
    _check(library().sib_routed_rows(
        _ptr(x), c_longlong(x.stride(0)), _ptr(w_gu), _ptr(w_down), _ptr(ids), _ptr(weights),
        _ptr(base), _ptr(mid), _ptr(out), _code(x.dtype), c_int(rows), c_int(width), c_int(ff),
        c_int(top), c_float(limit), c_float(alpha), c_int(form), _stream()))
    return out


@_timed(lambda ys, where, weights, base, out: ("routed_combine", _nbytes(ys, out), 0))
def routed_combine(ys: torch.Tensor, where: torch.Tensor, weights: Optional[torch.Tensor],
                   base: Optional[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
    """out[r] = base[r] + sum_k weights[r, k] ys[where[r, k]] in 32-bit: the rows' sums over the
    outputs of their (row, expert) pairs, which lie sorted by expert.  ``weights`` None: the plain
    sum."""
    rows, width = out.shape
    top = where.shape[1]
    _want(ys, out.dtype, "ys")
    _want(out, out.dtype, "out")
    _want(where, torch.int32, "where")
    if weights is not None:
        _f32(weights, rows * top, "weights")
    if ys.shape[1] != width or where.shape[0] != rows:
        raise KernelError("routed_combine: shapes do not fit")
    if base is not None:
        _want(base, out.dtype, "base")
    _check(library().sib_routed_combine(_ptr(ys), _ptr(where), _ptr(weights), _ptr(base), _ptr(out),
                                        _code(out.dtype), c_int(rows), c_int(width), c_int(top),
                                        _stream()))
    return out


@_timed(lambda qkv, *a, **kw: ("rope_store", 2 * _nbytes(qkv), 0))
def rope_store(qkv: torch.Tensor, row_pos, row_seq, seq_slot, seq_end,
               inv_freq: Optional[torch.Tensor], rotary_dim: int, style: int,
               k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
               page_table: Optional[torch.Tensor], page_tokens: int, ring_tokens: int,
               n_heads: int, n_kv: int, head_dim: int) -> None:
    """Rotate q and k of the packed rows in place and write k, v into the paged cache."""
    _want(qkv, qkv.dtype, "qkv")
    rows = qkv.shape[0]
    if qkv.shape[1] != (n_heads + 2 * n_kv) * head_dim:
        raise KernelError("rope_store: qkv width does not fit the head counts")
    if inv_freq is not None:
        _want(inv_freq, torch.float32, "inv_freq")
        if inv_freq.numel() * 2 != rotary_dim:
            raise KernelError("rope_store: one frequency per rotated pair")
    max_pages = 0
    if k_pool is not None:
        _want(k_pool, qkv.dtype, "k_pool")
        _want(v_pool, qkv.dtype, "v_pool")
        _want(page_table, torch.int32, "page_table")
        max_pages = page_table.shape[1]
        if tuple(k_pool.shape[1:]) != (n_kv, page_tokens, head_dim):
            raise KernelError("rope_store: pool layout must be [pages, kv_heads, page_tokens, head_dim]")
    _check(library().sib_rope_store(
        _ptr(qkv), _code(qkv.dtype), _ptr(row_pos), _ptr(row_seq), _ptr(seq_slot), _ptr(seq_end),
        _ptr(inv_freq), c_int(rotary_dim), c_int(style), _ptr(k_pool), _ptr(v_pool),
        _ptr(page_table), c_int(max_pages), c_int(page_tokens), c_int(ring_tokens), c_int(rows),
        c_int(n_heads), c_int(n_kv), c_int(head_dim), _stream()))


@_timed(lambda proj, qkv, *a, **kw: ("head_prepare", _nbytes(proj) + 2 * _nbytes(qkv), 0))
def head_prepare(proj: torch.Tensor, qkv: torch.Tensor, bias: Optional[torch.Tensor],
                 q_gain: Optional[torch.Tensor], k_gain: Optional[torch.Tensor], eps: float,
                 inv_freq: Optional[torch.Tensor], rotary_dim: int,
                 v_first: Optional[torch.Tensor], lam: Optional[torch.Tensor], row_pos, row_seq,
                 seq_slot, seq_end, k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
                 page_table: Optional[torch.Tensor], page_tokens: int, ring_tokens: int,
                 n_heads: int, n_kv: int, key_dim: int, value_dim: int, pad: int,
                 style: int = ROPE_HALF_SPLIT) -> torch.Tensor:
    """From a projected row ``[q heads | k heads | v heads | ...]`` to the packed q|k|v rows
    the attention kernels read, heads ``pad`` wide (csrc/head_prepare.cu): bias, per-head RMS
    norm of q and k with a gain, partial rotation (``style``: half-split pairs or
    neighbouring ones), values mixed with ``v_first`` (a view
    ``[rows, n_kv * its own head width]`` of an earlier layer's packed rows) by ``lam``, and
    k and v written into the paged cache."""
    rows = proj.shape[0]
    _want(proj, qkv.dtype, "proj", contiguous=False)
    _want(qkv, qkv.dtype, "qkv")
    need = n_heads * key_dim + n_kv * (key_dim + value_dim)
    if proj.stride(1) != 1 or proj.shape[1] < need:
        raise KernelError("head_prepare: a projected row must hold q, k and v side by side")
    if tuple(qkv.shape) != (rows, (n_heads + 2 * n_kv) * pad):
        raise KernelError("head_prepare: the packed rows do not fit the head counts")
    for t, n, nm in ((bias, need, "bias"), (q_gain, key_dim, "q_gain"), (k_gain, key_dim, "k_gain"),
                     (inv_freq, rotary_dim // 2, "inv_freq"), (lam, 1, "lam")):
        if t is not None:
            _want(t, torch.float32, nm)
            if t.numel() != n:
                raise KernelError(f"head_prepare: {nm} has {t.numel()} values, expected {n}")
    v_stride = v_pad = 0
    if v_first is not None:
        _want(v_first, qkv.dtype, "v_first", contiguous=False)
        v_pad = v_first.shape[1] // max(n_kv, 1)
        if v_first.stride(1) != 1 or tuple(v_first.shape) != (rows, n_kv * v_pad) or v_pad < value_dim \
                or lam is None:
            raise KernelError("head_prepare: v_first must be [rows, kv heads x width] with lam")
        v_stride = v_first.stride(0)
    max_pages = 0
    if k_pool is not None:
        _want(k_pool, qkv.dtype, "k_pool")
        _want(v_pool, qkv.dtype, "v_pool")
        _want(page_table, torch.int32, "page_table")
        max_pages = page_table.shape[1]
        want = (n_kv, page_tokens, pad)
        if tuple(k_pool.shape[1:]) != want or tuple(v_pool.shape[1:]) != want:
            raise KernelError("head_prepare: pool layout must be [pages, kv_heads, page_tokens, width]")
    _check(library().sib_head_prepare(
        _ptr(proj), c_longlong(proj.stride(0)), _ptr(qkv), _code(qkv.dtype), _ptr(bias),
        _ptr(q_gain), _ptr(k_gain), c_float(eps), _ptr(inv_freq), c_int(rotary_dim if inv_freq is not None else 0),
        _ptr(v_first), c_longlong(v_stride), c_int(v_pad), _ptr(lam), _ptr(row_pos), _ptr(row_seq), _ptr(seq_slot),
        _ptr(seq_end), _ptr(k_pool), _ptr(v_pool), _ptr(page_table), c_int(max_pages),
        c_int(page_tokens), c_int(ring_tokens), c_int(rows), c_int(n_heads), c_int(n_kv),
        c_int(key_dim), c_int(value_dim), c_int(pad), c_int(1 if style == ROPE_INTERLEAVED else 0),
        _stream()))
    return qkv


@_timed(lambda qkv, view, *a, **kw: ("pool_store", 2 * _nbytes(qkv) // 3, 0))
def pool_store(qkv: torch.Tensor, view, ctx, n_heads: int, n_kv: int, pad: int) -> None:
    """For every block of ``view.need.pool`` positions whose last position this step brings:
    the mean of the block's keys and the mean of its values, as the packed rows ``qkv`` (this
    step's positions) and the cache ``view`` (earlier ones) hold them, into the block's cells
    (csrc/head_prepare.cu pool_store)."""
    _want(qkv, qkv.dtype, "qkv")
    if view.cell_k is None or view.need.pool <= 0:
        raise KernelError("pool_store: the cache keeps no cells of blocks")
    if tuple(qkv.shape) != (ctx.n_rows, (n_heads + 2 * n_kv) * pad):
        raise KernelError("pool_store: the packed rows do not fit the head counts")
    for t in (view.k, view.v, view.cell_k, view.cell_v):
        _want(t, qkv.dtype, "cache")
        if t.shape[1] != n_kv or t.shape[3] != pad:
            raise KernelError("pool_store: keys and values must be cached `pad` wide")
    _check(library().sib_pool_store(
        _ptr(qkv), _ptr(view.k), _ptr(view.v), _ptr(view.page_table), c_int(view.page_table.shape[1]),
        c_int(view.page_tokens), c_int(view.ring_tokens), _ptr(view.cell_k), _ptr(view.cell_v),
        _ptr(view.cell_table), c_int(view.cell_table.shape[1]), c_int(view.cell_page_tokens),
        _ptr(ctx.seq_slot), _ptr(ctx.seq_start), _ptr(ctx.seq_end), _ptr(ctx.seq_row0),
        _code(qkv.dtype), c_int(ctx.n_seqs), c_int(ctx.max_count), c_int(n_heads), c_int(n_kv),
        c_int(pad), c_int(view.need.pool), _stream()))


@_timed(lambda o, gate, y, *a: ("head_gate", _nbytes(o, y), 0))
def head_gate(o: torch.Tensor, gate: Optional[torch.Tensor], y: torch.Tensor, n_heads: int,
              value_dim: int, pad: int) -> torch.Tensor:
    """y[r, h, :] = o[r, h, :value_dim] * sigmoid(gate[r, h]); ``o`` has heads ``pad`` wide,
    ``gate`` is a view ``[rows, n_heads]`` (None: no gate, only the narrowing)."""
    rows = o.shape[0]
    _want(o, y.dtype, "o")
    _want(y, y.dtype, "y")
    if tuple(o.shape) != (rows, n_heads * pad) or tuple(y.shape) != (rows, n_heads * value_dim):
        raise KernelError("head_gate: shapes do not fit the head counts")
    stride = 0
    if gate is not None:
        _want(gate, y.dtype, "gate", contiguous=False)
        if tuple(gate.shape) != (rows, n_heads) or gate.stride(1) != 1:
            raise KernelError("head_gate: one gate value per row and head")
        stride = gate.stride(0)
    _check(library().sib_head_gate(_ptr(o), _ptr(gate), c_longlong(stride), _ptr(y), _code(y.dtype),
                                   c_int(rows), c_int(n_heads), c_int(value_dim), c_int(pad),
                                   _stream()))
    return y


@_timed(lambda proj, q_lat, q_rows, k_rows, *a, **kw: ("latent_prepare", _nbytes(q_lat, q_rows, k_rows) * 2, 0))
def latent_prepare(proj: torch.Tensor, q_lat: torch.Tensor, q_rows: torch.Tensor, k_rows: torch.Tensor,
                   c_gain: torch.Tensor, eps: float, inv_freq: Optional[torch.Tensor], rot: int, ctx,
                   k_pool: Optional[torch.Tensor], page_table: Optional[torch.Tensor],
                   page_tokens: int, ring_tokens: int, n_heads: int, q_dim: int, rot_dim: int,
                   rank: int, pad: int, down: Optional[torch.Tensor] = None) -> None:
    """Between the projections and the attention over a shared latent (csrc/head_prepare.cu):
    ``proj`` rows hold the query heads (``q_dim`` + ``rot_dim`` each) and then the down
    projection (``rank`` + ``rot_dim``), unless ``down`` (a view ``[rows, rank + rot_dim]``) gives
    the latter where the queries come from a product of their own; ``q_lat`` ``[heads, rows, rank]`` are the queries
    already multiplied into the latent's space.  Writes ``q_rows`` ``[rows, heads * pad]``
    (not with ``q_lat`` and ``q_rows`` None), ``k_rows`` ``[rows, pad]`` and the cache cells of
    the rows."""
    rows = proj.shape[0]
    _want(proj, proj.dtype, "proj", contiguous=False)
    if (q_lat is None) != (q_rows is None):
        raise KernelError("latent_prepare: q_lat and q_rows come together (None: the key rows only)")
    for t, shape, nm in ((q_lat, (n_heads, rows, rank), "q_lat"), (q_rows, (rows, n_heads * pad), "q_rows"),
                         (k_rows, (rows, pad), "k_rows")):
        if t is None:
            continue
        _want(t, proj.dtype, nm)
        if tuple(t.shape) != shape:
            raise KernelError(f"latent_prepare: {nm} must be {shape}")
    if proj.stride(1) != 1 or proj.shape[1] < n_heads * (q_dim + rot_dim) + (0 if down is not None else rank + rot_dim):
        raise KernelError("latent_prepare: a projected row must hold the query heads and the down projection")
    if down is not None:
        _want(down, proj.dtype, "down", contiguous=False)
        if down.stride(1) != 1 or down.shape[0] != rows or down.shape[1] < rank + rot_dim:
            raise KernelError("latent_prepare: down must be [rows, rank + rot_dim]")
    _f32(c_gain, rank, "c_gain")
    if rot:
        _f32(inv_freq, rot // 2, "inv_freq")
    max_pages = 0
    if k_pool is not None:
        _want(k_pool, proj.dtype, "k_pool")
        if tuple(k_pool.shape[1:]) != (1, page_tokens, pad) or page_table is None:
            raise KernelError("latent_prepare: pool layout must be [pages, 1, page_tokens, pad]")
        max_pages = page_table.shape[1]
    _check(library().sib_latent_prepare(
        _ptr(proj), c_longlong(proj.stride(0)), _ptr(q_lat), _ptr(q_rows), _ptr(k_rows),
        _code(proj.dtype), _ptr(c_gain), c_float(eps), _ptr(inv_freq if rot else None), c_int(rot),
        _ptr(ctx.row_pos), _ptr(ctx.row_seq), _ptr(ctx.seq_slot), _ptr(ctx.seq_end), _ptr(k_pool),
        _ptr(page_table), c_int(max_pages), c_int(page_tokens), c_int(ring_tokens), c_int(rows),
        c_int(n_heads), c_int(q_dim), c_int(rot_dim), c_int(rank), c_int(pad), _ptr(down),
        c_longlong(down.stride(0) if down is not None else 0), _stream()))


@_timed(lambda proj, k_rows, k_heads, v_heads, qkv, *a, **kw: ("latent_expand", _nbytes(k_heads, v_heads, qkv) * 1.3, 0))
def latent_expand(proj: torch.Tensor, k_rows: torch.Tensor, k_heads: torch.Tensor, v_heads: torch.Tensor,
                  qkv: torch.Tensor, inv_freq: Optional[torch.Tensor], rot: int, row_pos, n_heads: int,
                  q_dim: int, rot_dim: int, value_dim: int, rank: int, pad: int, head_width: int) -> torch.Tensor:
    """Packed rows for the prompt attention kernels from keys and values made per head
    (csrc/head_prepare.cu): ``qkv[r]`` = query heads ``[unrotated | rotated | 0]``, key heads
    ``[k_heads | the row's shared rotated part (from k_rows) | 0]``, value heads ``[v_heads | 0]``,
    every head ``head_width`` wide."""
    rows = proj.shape[0]
    _want(proj, proj.dtype, "proj", contiguous=False)
    for t, shape, nm in ((k_rows, (rows, pad), "k_rows"), (k_heads, (rows, n_heads * q_dim), "k_heads"),
                         (v_heads, (rows, n_heads * value_dim), "v_heads"),
                         (qkv, (rows, 3 * n_heads * head_width), "qkv")):
        _want(t, proj.dtype, nm)
        if tuple(t.shape) != shape:
            raise KernelError(f"latent_expand: {nm} must be {shape}")
    if proj.stride(1) != 1 or proj.shape[1] < n_heads * (q_dim + rot_dim):
        raise KernelError("latent_expand: a projected row must hold the query heads")
    if rot:
        _f32(inv_freq, rot // 2, "inv_freq")
    _check(library().sib_latent_expand(
        _ptr(proj), c_longlong(proj.stride(0)), _ptr(k_rows), _ptr(k_heads), _ptr(v_heads), _ptr(qkv),
        _code(proj.dtype), _ptr(inv_freq if rot else None), c_int(rot), _ptr(row_pos), c_int(rows),
        c_int(n_heads), c_int(q_dim), c_int(rot_dim), c_int(value_dim), c_int(rank), c_int(pad),
        c_int(head_width), _stream()))
    return qkv


def _f32(t: Optional[torch.Tensor], n: int, name: str) -> None:
    if t is None:
        raise KernelError(f"{name} is needed")
    _want(t, torch.float32, name)
    if t.numel() != n:
        raise KernelError(f"{name} has {t.numel()} values, expected {n}")


@_timed(lambda proj, conv_w, a_log, dt_bias, state, hist_offset, qn, kn, vc, beta, decay, *a, **kw: (
    "delta_prepare", _nbytes(proj, qn, kn, vc, beta, decay), 0))
def delta_prepare(proj: torch.Tensor, conv_w: torch.Tensor, a_log: torch.Tensor,
                  dt_bias: torch.Tensor, state: torch.Tensor, hist_offset: int, qn: torch.Tensor,
                  kn: torch.Tensor, vc: torch.Tensor, beta: torch.Tensor, decay: torch.Tensor, ctx,
                  n_heads: int, n_kv: int, key_dim: int, value_dim: int, taps: int) -> None:
    """First step of the gated delta rule (csrc/recurrent.cu): from projected rows
    ``[q | k | v | gate | b | a]`` the convolved, activated and unit-length q and k, the
    convolved v, beta and the decay, all 32-bit; then the convolution history of every
    sequence is brought up to the step's end.  ``state``: ``[slots, floats]``, the history
    ``[taps - 1, channels]`` begins at ``hist_offset``."""
    rows = proj.shape[0]
    _want(proj, proj.dtype, "proj")
    _want(state, torch.float32, "state")
    nqk, nv = n_kv * key_dim, n_heads * value_dim
    if proj.shape[1] != 2 * nqk + 2 * nv + 2 * n_heads:
        raise KernelError("delta_prepare: a projected row must hold q, k, v, gate, b and a")
    _f32(conv_w, (2 * nqk + nv) * taps, "conv_w")
    _f32(a_log, n_heads, "a_log")
    _f32(dt_bias, n_heads, "dt_bias")
    for t, n, nm in ((qn, rows * nqk, "qn"), (kn, rows * nqk, "kn"), (vc, rows * nv, "vc"),
                     (beta, rows * n_heads, "beta"), (decay, rows * n_heads, "decay")):
        _f32(t, n, nm)
    if state.shape[1] < hist_offset + (taps - 1) * (2 * nqk + nv):
        raise KernelError("delta_prepare: the state is too small for the history")
    _check(library().sib_delta_prepare(
        _ptr(proj), c_longlong(proj.stride(0)), _code(proj.dtype), _ptr(conv_w), _ptr(a_log),
        _ptr(dt_bias), _ptr(state), c_longlong(state.stride(0)), c_longlong(hist_offset), _ptr(qn),
        _ptr(kn), _ptr(vc), _ptr(beta), _ptr(decay), _ptr(ctx.row_pos), _ptr(ctx.row_seq),
        _ptr(ctx.seq_slot), _ptr(ctx.seq_start), _ptr(ctx.seq_end), _ptr(ctx.seq_row0), c_int(rows),
        c_int(ctx.n_seqs), c_int(n_heads), c_int(n_kv), c_int(key_dim), c_int(value_dim),
        c_int(taps), _stream()))


def _scan_work(kind, rows, n_seqs, n_heads, key_dim, cols):
    state = n_seqs * n_heads * key_dim * cols * 4
    return kind, 2 * state + rows * n_heads * (2 * key_dim + 2 * cols) * 4, \
        7.0 * rows * n_heads * key_dim * cols


@_timed(lambda qn, kn, vc, decay, beta, state, out, ctx, n_heads, n_kv, key_dim, value_dim: _scan_work(
    "delta_scan", out.shape[0], ctx.n_seqs, n_heads, key_dim, value_dim))
def delta_scan(qn: torch.Tensor, kn: torch.Tensor, vc: torch.Tensor, decay: torch.Tensor,
               beta: torch.Tensor, state: torch.Tensor, out: torch.Tensor, ctx, n_heads: int,
               n_kv: int, key_dim: int, value_dim: int) -> torch.Tensor:
    """The gated delta rule over the step's rows, sequence by sequence, from and into the
    slots' matrices ``state[slot, :heads * value_dim * key_dim]``; ``out`` 32-bit
    ``[rows, heads * value_dim]``."""
    rows = out.shape[0]
    _want(state, torch.float32, "state")
    _f32(out, rows * n_heads * value_dim, "out")
    if state.shape[1] < n_heads * value_dim * key_dim:
        raise KernelError("delta_scan: the state is too small for the matrices")
    _check(library().sib_delta_scan(
        _ptr(qn), _ptr(kn), _ptr(vc), _ptr(decay), _ptr(beta), _ptr(state),
        c_longlong(state.stride(0)), _ptr(out), _ptr(ctx.seq_slot), _ptr(ctx.seq_start),
        _ptr(ctx.seq_end), _ptr(ctx.seq_row0), c_int(rows), c_int(ctx.n_seqs), c_int(n_heads),
        c_int(n_kv), c_int(key_dim), c_int(value_dim), _stream()))
    return out


@_timed(lambda proj, bias_i, bias_f, cap, state, out, m_out, ctx, n_heads, key_dim, value_dim: _scan_work(
    "memory_scan", out.shape[0], ctx.n_seqs, n_heads, key_dim, value_dim + 1))
def memory_scan(proj: torch.Tensor, bias_i: torch.Tensor, bias_f: torch.Tensor, cap: float,
                state: torch.Tensor, out: torch.Tensor, m_out: torch.Tensor, ctx, n_heads: int,
                key_dim: int, value_dim: int) -> torch.Tensor:
    """The matrix memory with exponential gates over the step's rows.  ``proj``:
    ``[q | k | v | gate | i | f]`` per row; ``out`` 32-bit ``[rows, heads * (value_dim + 1)]``
    (the last column of a head is <n, q>), ``m_out`` ``[rows, heads]`` the running maxima;
    ``state[slot]``: the matrices with n as one more column, then the maxima."""
    rows = proj.shape[0]
    _want(proj, proj.dtype, "proj")
    _want(state, torch.float32, "state")
    nq, nv = n_heads * key_dim, n_heads * value_dim
    if proj.shape[1] != 2 * nq + 2 * nv + 2 * n_heads:
        raise KernelError("memory_scan: a projected row must hold q, k, v, gate, i and f")
    _f32(bias_i, n_heads, "bias_i")
    _f32(bias_f, n_heads, "bias_f")
    _f32(out, rows * n_heads * (value_dim + 1), "out")
    _f32(m_out, rows * n_heads, "m_out")
    if state.shape[1] < n_heads * (value_dim + 1) * key_dim + n_heads:
        raise KernelError("memory_scan: the state is too small")
    _check(library().sib_memory_scan(
        _ptr(proj), c_longlong(proj.stride(0)), _code(proj.dtype), c_longlong(2 * nq + 2 * nv),
        c_longlong(2 * nq + 2 * nv + n_heads), _ptr(bias_i), _ptr(bias_f), c_float(cap), _ptr(state),
        c_longlong(state.stride(0)), _ptr(out), _ptr(m_out), _ptr(ctx.seq_slot), _ptr(ctx.seq_start),
        _ptr(ctx.seq_end), _ptr(ctx.seq_row0), c_int(rows), c_int(ctx.n_seqs), c_int(n_heads),
        c_int(key_dim), c_int(value_dim), _stream()))
    return out


@_timed(lambda proj, inv_freq, rot, row_pos, qn, kn, vc, *a: (
    "retention_prepare", proj.shape[0] * (qn.shape[1] * 2 + vc.shape[1]) * proj.element_size()
    + _nbytes(qn, kn, vc), 0))
def retention_prepare(proj: torch.Tensor, inv_freq: Optional[torch.Tensor], rot: int, row_pos,
                      qn: torch.Tensor, kn: torch.Tensor, vc: torch.Tensor, n_heads: int,
                      key_dim: int, value_dim: int, k_scale: float, silu: bool = False) -> None:
    """From projected rows ``[q | k | v | ...]``: q and k rotated on their first ``rot``
    dimensions (half-split pairs), k times ``k_scale``, v as it is; all 32-bit.  ``silu``: q, k
    and v pass SiLU first."""
    rows = proj.shape[0]
    _want(proj, proj.dtype, "proj", contiguous=False)
    if proj.stride(1) != 1 or proj.shape[1] < n_heads * (2 * key_dim + value_dim):
        raise KernelError("retention_prepare: a projected row must hold q, k and v")
    for t, n, nm in ((qn, rows * n_heads * key_dim, "qn"), (kn, rows * n_heads * key_dim, "kn"),
                     (vc, rows * n_heads * value_dim, "vc")):
        _f32(t, n, nm)
    if rot:
        _f32(inv_freq, rot // 2, "inv_freq")
    _check(library().sib_retention_prepare(
        _ptr(proj), c_longlong(proj.stride(0)), _code(proj.dtype), _ptr(inv_freq if rot else None),
        c_int(rot), _ptr(row_pos), _ptr(qn), _ptr(kn), _ptr(vc), c_int(rows), c_int(n_heads),
        c_int(key_dim), c_int(value_dim), c_float(k_scale), c_int(1 if silu else 0), _stream()))


@_timed(lambda qn, kn, vc, decay, state, out, ctx, n_heads, key_dim, value_dim: _scan_work(
    "retention_scan", out.shape[0], ctx.n_seqs, n_heads, key_dim, value_dim))
def retention_scan(qn: torch.Tensor, kn: torch.Tensor, vc: torch.Tensor, decay: torch.Tensor,
                   state: torch.Tensor, out: torch.Tensor, ctx, n_heads: int, key_dim: int,
                   value_dim: int) -> torch.Tensor:
    """S <- decay_h S + k v^T, o = S^T q over the step's rows, sequence by sequence, from and
    into the slots' matrices ``state[slot, :heads * value_dim * key_dim]``; ``out`` 32-bit
    ``[rows, heads * value_dim]``; ``decay`` one 32-bit value per head."""
    rows = out.shape[0]
    _want(state, torch.float32, "state")
    _f32(qn, rows * n_heads * key_dim, "qn")
    _f32(kn, rows * n_heads * key_dim, "kn")
    _f32(vc, rows * n_heads * value_dim, "vc")
    _f32(decay, n_heads, "decay")
    _f32(out, rows * n_heads * value_dim, "out")
    if state.shape[1] < n_heads * value_dim * key_dim:
        raise KernelError("retention_scan: the state is too small for the matrices")
    _check(library().sib_retention_scan(
        _ptr(qn), _ptr(kn), _ptr(vc), _ptr(decay), _ptr(state), c_longlong(state.stride(0)),
        _ptr(out), _ptr(ctx.seq_slot), _ptr(ctx.seq_start), _ptr(ctx.seq_end), _ptr(ctx.seq_row0),
        c_int(rows), c_int(ctx.n_seqs), c_int(n_heads), c_int(key_dim), c_int(value_dim), _stream()))
    return out


@_timed(lambda o, m, w, gate, y, *a: ("head_norm_gate", _nbytes(o, y) + _nbytes(y), 0))  # (+ the gates)
def head_norm_gate(o: torch.Tensor, m: Optional[torch.Tensor], w: Optional[torch.Tensor],
                   gate: torch.Tensor, y: torch.Tensor, n_heads: int, value_dim: int, eps: float,
                   act: int) -> torch.Tensor:
    """y[r, h, :] = x / rms(x) * w * act(gate[r, h, :]) with x the head's 32-bit output
    (``o`` ``[rows, heads * cols]``, the first ``value_dim`` columns of a head; with ``m``
    divided by max(|column value_dim|, e^-m) + 1e-6 first).  ``w``: one weight per column
    shared by the heads, or one per head and column, or None for none.  ``gate``: a view ``[rows, heads *
    value_dim]``.  act: GATE_SILU or GATE_SIGMOID."""
    rows = y.shape[0]
    _want(o, torch.float32, "o")
    _want(y, y.dtype, "y")
    if w is not None:
        _want(w, torch.float32, "w")
    _want(gate, y.dtype, "gate", contiguous=False)
    cols = o.shape[1] // n_heads
    if tuple(y.shape) != (rows, n_heads * value_dim) or o.shape[0] != rows or cols < value_dim:
        raise KernelError("head_norm_gate: shapes do not fit the head counts")
    if w is not None and w.numel() not in (value_dim, n_heads * value_dim):
        raise KernelError("head_norm_gate: the weight is per column or per head and column")
    if tuple(gate.shape) != (rows, n_heads * value_dim) or gate.stride(1) != 1:
        raise KernelError("head_norm_gate: one gate value per output")
    if m is not None:
        _f32(m, rows * n_heads, "m")
    _check(library().sib_head_norm_gate(
        _ptr(o), _ptr(m), _ptr(w), c_int(0 if w is None or w.numel() == value_dim else value_dim), _ptr(gate),
        c_longlong(gate.stride(0)), _ptr(y), _code(y.dtype), c_int(rows), c_int(n_heads),
        c_int(value_dim), c_int(cols), c_float(eps), c_int(act), _stream()))
    return y


@_timed(lambda q, k, v, keep, take, state, out, ctx, n_heads, n_kv, key_dim, value_dim: _scan_work(
    "gated_scan", out.shape[0], ctx.n_seqs, n_heads, key_dim, value_dim))
def gated_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, keep: torch.Tensor,
               take: torch.Tensor, state: torch.Tensor, out: torch.Tensor, ctx, n_heads: int,
               n_kv: int, key_dim: int, value_dim: int) -> torch.Tensor:
    """S <- keep S + take k v^T, o = S^T q with ``keep`` and ``take`` 32-bit ``[rows, heads]``
    (csrc/recurrent.cu).  ``q``, ``k`` (``n_kv`` key heads of ``key_dim``) and ``v`` (``n_heads``
    heads of ``value_dim``) are 32-bit views whose rows may be columns of one buffer."""
    rows = out.shape[0]
    _want(state, torch.float32, "state")
    for t, n, nm in ((q, n_kv * key_dim, "q"), (k, n_kv * key_dim, "k"), (v, n_heads * value_dim, "v")):
        _want(t, torch.float32, nm, contiguous=False)
        if tuple(t.shape) != (rows, n) or t.stride(1) != 1:
            raise KernelError(f"gated_scan: {nm} must be [rows, {n}] with unit column stride")
    _f32(keep, rows * n_heads, "keep")
    _f32(take, rows * n_heads, "take")
    _f32(out, rows * n_heads * value_dim, "out")
    if state.shape[1] < n_heads * value_dim * key_dim:
        raise KernelError("gated_scan: the state is too small for the matrices")
    _check(library().sib_gated_scan(
        _ptr(q), _ptr(k), _ptr(v), c_longlong(q.stride(0)), c_longlong(k.stride(0)),
        c_longlong(v.stride(0)), _ptr(keep), _ptr(take), _ptr(state), c_longlong(state.stride(0)),
        _ptr(out), _ptr(ctx.seq_slot), _ptr(ctx.seq_start), _ptr(ctx.seq_end), _ptr(ctx.seq_row0),
        c_int(rows), c_int(ctx.n_seqs), c_int(n_heads), c_int(n_kv), c_int(key_dim),
        c_int(value_dim), _stream()))
    return out


@_timed(lambda proj, conv_w, conv_b, a_log, dt_bias, state, hist_offset, xbc, keep, take, *a, **kw: (
    "ssm_prepare", _nbytes(proj, xbc, keep, take), 0))
def ssm_prepare(proj: torch.Tensor, conv_w: torch.Tensor, conv_b: torch.Tensor, a_log: torch.Tensor,
                dt_bias: torch.Tensor, state: torch.Tensor, hist_offset: int, xbc: torch.Tensor,
                keep: torch.Tensor, take: torch.Tensor, ctx, n_heads: int, inner: int,
                channels: int, taps: int) -> None:
    """First step of the state-space layer (csrc/recurrent.cu): from projected rows
    ``[z (inner) | x (inner) | B | C | dt (heads)]`` the convolved (with bias) and activated
    channels x | B | C, the step size softplus(dt + dt_bias) (``take``) and the decay
    exp(-exp(A_log) step) (``keep``), all 32-bit; then every sequence's convolution history
    (``state[slot, hist_offset:]``, ``[taps - 1, channels]``) is brought up to the step's end."""
    rows = proj.shape[0]
    _want(proj, proj.dtype, "proj")
    _want(state, torch.float32, "state")
    if proj.shape[1] != inner + channels + n_heads:
        raise KernelError("ssm_prepare: a projected row must hold z, the channels and dt")
    _f32(conv_w, channels * taps, "conv_w")
    _f32(conv_b, channels, "conv_b")
    _f32(a_log, n_heads, "a_log")
    _f32(dt_bias, n_heads, "dt_bias")
    _f32(xbc, rows * channels, "xbc")
    _f32(keep, rows * n_heads, "keep")
    _f32(take, rows * n_heads, "take")
    if state.shape[1] < hist_offset + (taps - 1) * channels:
        raise KernelError("ssm_prepare: the state is too small for the history")
    _check(library().sib_ssm_prepare(
        _ptr(proj), c_longlong(proj.stride(0)), _code(proj.dtype), _ptr(conv_w), _ptr(conv_b),
        _ptr(a_log), _ptr(dt_bias), _ptr(state), c_longlong(state.stride(0)), c_longlong(hist_offset),
        _ptr(xbc), _ptr(keep), _ptr(take), _ptr(ctx.row_pos), _ptr(ctx.row_seq), _ptr(ctx.seq_slot),
        _ptr(ctx.seq_start), _ptr(ctx.seq_end), _ptr(ctx.seq_row0), c_int(rows), c_int(ctx.n_seqs),
        c_int(n_heads), c_int(inner), c_int(channels), c_int(taps), _stream()))


@_timed(lambda o, xbc, z, skip, w, y, *a: ("ssm_finish", 2 * _nbytes(o) + 2 * _nbytes(y), 0))
def ssm_finish(o: torch.Tensor, xbc: torch.Tensor, z: torch.Tensor, skip: torch.Tensor,
               w: torch.Tensor, y: torch.Tensor, inner: int, value_dim: int, parts: int,
               eps: float) -> torch.Tensor:
    """y = (o + skip_h x) * silu(z), divided by its root mean square in ``parts`` equal parts
    of a row, times ``w``.  ``o`` 32-bit ``[rows, inner]``; x the first ``inner`` columns of
    the 32-bit ``xbc``; ``z`` a view ``[rows, inner]`` in y's type."""
    rows = y.shape[0]
    _f32(o, rows * inner, "o")
    _want(xbc, torch.float32, "xbc")
    _want(y, y.dtype, "y")
    _want(z, y.dtype, "z", contiguous=False)
    _f32(skip, inner // value_dim, "skip")
    _f32(w, inner, "w")
    if tuple(z.shape) != (rows, inner) or z.stride(1) != 1 or tuple(y.shape) != (rows, inner):
        raise KernelError("ssm_finish: one gate value per output")
    _check(library().sib_ssm_finish(
        _ptr(o), _ptr(xbc), c_longlong(xbc.stride(0)), _ptr(z), c_longlong(z.stride(0)), _ptr(skip),
        _ptr(w), _ptr(y), _code(y.dtype), c_int(rows), c_int(inner), c_int(value_dim), c_int(parts),
        c_float(eps), _stream()))
    return y


@_timed(lambda proj, a_col, decay_in, w0, a_bias, prep, *a: ("general_delta_prepare", _nbytes(proj, prep), 0))
def gdelta_prepare(proj: torch.Tensor, a_col: int, decay_in: torch.Tensor, w0: torch.Tensor,
                   a_bias: torch.Tensor, prep: torch.Tensor, n_heads: int, dim: int) -> torch.Tensor:
    """First step of the generalized delta rule (csrc/general_delta.cu): from projected rows
    ``[r | k | v | ...]`` with the removal rates' inputs at column ``a_col`` and the decays'
    inputs ``decay_in`` the six 32-bit vectors per row and head that the recurrence reads:
    r | k | w | u | a u | v (``prep`` ``[rows, heads, 6, dim]``)."""
    rows = proj.shape[0]
    n = n_heads * dim
    _want(proj, proj.dtype, "proj")
    _want(decay_in, proj.dtype, "decay_in", contiguous=False)
    if proj.shape[1] < max(3 * n, a_col + n) or tuple(decay_in.shape) != (rows, n) or decay_in.stride(1) != 1:
        raise KernelError("general_delta_prepare: the projected rows do not hold r, k, v and a")
    _f32(w0, n, "w0")
    _f32(a_bias, n, "a_bias")
    _f32(prep, rows * n * 6, "prep")
    _check(library().sib_gdelta_prepare(
        _ptr(proj), c_longlong(proj.stride(0)), c_longlong(a_col), _ptr(decay_in),
        c_longlong(decay_in.stride(0)), _code(proj.dtype), _ptr(w0), _ptr(a_bias), _ptr(prep),
        c_int(rows), c_int(n_heads), c_int(dim), _stream()))
    return prep


@_timed(lambda prep, state, out, ctx, n_heads, dim: (
    "general_delta_scan", 2 * ctx.n_seqs * n_heads * dim * dim * 4 + _nbytes(prep, out),
    8.0 * out.shape[0] * n_heads * dim * dim))
def gdelta_scan(prep: torch.Tensor, state: torch.Tensor, out: torch.Tensor, ctx, n_heads: int,
                dim: int) -> torch.Tensor:
    """The generalized delta rule over the step's rows, sequence by sequence, from and into the
    slots' matrices ``state[slot, :heads * dim * dim]``; ``out`` 32-bit ``[rows, heads * dim]``."""
    rows = out.shape[0]
    _want(state, torch.float32, "state")
    _f32(prep, rows * n_heads * 6 * dim, "prep")
    _f32(out, rows * n_heads * dim, "out")
    if state.shape[1] < n_heads * dim * dim:
        raise KernelError("general_delta_scan: the state is too small for the matrices")
    _check(library().sib_gdelta_scan(
        _ptr(prep), _ptr(state), c_longlong(state.stride(0)), _ptr(out), _ptr(ctx.seq_slot),
        _ptr(ctx.seq_start), _ptr(ctx.seq_end), _ptr(ctx.seq_row0), c_int(rows), c_int(ctx.n_seqs),
        c_int(n_heads), c_int(dim), _stream()))
    return out


def attention_rows_scratch_bytes(rows: int, n_heads: int, head_dim: int, splits: int) -> int:
    return int(library().sib_attention_rows_scratch_bytes(c_int(rows), c_int(n_heads),
                                                          c_int(head_dim), c_int(splits)))


@_timed(lambda q, q_stride, k_new, v_new, kv_stride, k_pool, v_pool, page_table, page_tokens,
        ring_tokens, row_pos, row_seq, seq_slot, seq_start, seq_row0, out, scratch, n_heads, n_kv,
        head_dim, scale, softcap, window, splits, sink=None, values_in_keys=False, cells=None,
        cells_only=False, chunk=0: (
            ("attention_rows (blocks)", _nbytes(out), 0) if cells_only else
            _attention_cache_work("attention_rows (cache)", row_pos, k_pool, n_heads, head_dim,
                                  window, out.shape[0], chunk=chunk) if k_pool is not None else
            ("attention_rows (prompt)", 2 * _nbytes(out) * (1 + 2 * n_kv / n_heads),
             2.0 * (row_pos.to(torch.int64) + 1).sum().item() * 2 * n_heads * head_dim)))
def attention_rows(q: torch.Tensor, q_stride: int, k_new: Optional[torch.Tensor],
                   v_new: Optional[torch.Tensor], kv_stride: int,
                   k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
                   page_table: Optional[torch.Tensor], page_tokens: int, ring_tokens: int,
                   row_pos, row_seq, seq_slot, seq_start, seq_row0, out: torch.Tensor,
                   scratch: Optional[torch.Tensor], n_heads: int, n_kv: int, head_dim: int,
                   scale: float, softcap: float, window: int, splits: int,
                   sink: Optional[torch.Tensor] = None, values_in_keys: bool = False,
                   cells=None, cells_only: bool = False, chunk: int = 0) -> torch.Tensor:
    """General attention of independent rows (see csrc/attention_rows.cu).  ``chunk`` > 0
    (without a window): a row sees the positions of its own chunk of that many, chunks
    counted from the sequence's first position.  ``sink``: one
    32-bit value per query head whose exponential joins the softmax's denominator.
    ``values_in_keys``: a value is its key's cell (``v_new`` / ``v_pool`` are not read).
    ``cells``: a cache view (``KVView``) with cells of pooled blocks; a row then also sees
    the blocks that lie wholly before its window, one key and one value each.

    ``q``, ``k_new``, ``v_new`` may be views into one packed buffer; only
    their first elements' addresses and the strides are used."""
    rows = out.shape[0]
    _want(out, out.dtype, "out")
    if q.dtype != out.dtype:
        raise KernelError("attention_rows: q and out differ in type")
    max_pages = page_table.shape[1] if page_table is not None else 0
    if k_pool is not None and tuple(k_pool.shape[1:]) != (n_kv, page_tokens, head_dim):
        raise KernelError("attention_rows: pool layout must be [pages, kv_heads, page_tokens, head_dim]")
    if splits > 1:
        need = attention_rows_scratch_bytes(rows, n_heads, head_dim, splits)
        if scratch is None or scratch.numel() * scratch.element_size() < need:
            raise KernelError(f"attention_rows: {need} bytes of scratch memory are needed")
    if sink is not None:
        _f32(sink, n_heads, "sink")
    if cells_only:
        if cells is None or splits != 1:
            raise KernelError("attention_rows: the blocks alone need their cache and one split")
        _f32(scratch, rows * n_heads * (head_dim + 2), "scratch")
    _check(library().sib_attention_rows(
        _ptr(q), c_int(q_stride), _ptr(k_new), _ptr(v_new), c_int(kv_stride), _ptr(k_pool),
        _ptr(v_pool), _ptr(page_table), c_int(max_pages), c_int(page_tokens), c_int(ring_tokens),
        _ptr(row_pos), _ptr(row_seq), _ptr(seq_slot), _ptr(seq_start), _ptr(seq_row0), _ptr(out),
        _ptr(scratch), _code(out.dtype), c_int(rows), c_int(n_heads), c_int(n_kv), c_int(head_dim),
        c_float(scale), c_float(softcap), c_int(window), c_int(chunk), c_int(splits), _ptr(sink),
        c_int(1 if values_in_keys else 0),
        _ptr(cells.cell_k if cells is not None else None),
        _ptr(cells.cell_v if cells is not None else None),
        _ptr(cells.cell_table if cells is not None else None),
        c_int(cells.need.pool if cells is not None else 0),
        c_int(cells.cell_table.shape[1] if cells is not None else 0),
        c_int(cells.cell_page_tokens if cells is not None else 0),
        c_int(1 if cells_only else 0), _stream()))
    return out


def attention_latent_supports(n_heads: int, width: int) -> bool:
    return bool(library().sib_attention_latent_supports(c_int(n_heads), c_int(width)))


@_timed(lambda q, k_new, k_pool, page_table, page_tokens, ring_tokens, ctx, out, scratch, sink, n_heads,
        width, scale, window, splits, rows_per_tile=1: (
            _attention_cache_work("attention_latent (cache)", ctx.row_pos, k_pool, n_heads, width, window,
                                  out.shape[0], value_dim=0) if k_new is None else
            ("attention_latent (prompt)", _nbytes(q, k_new, out),
             4.0 * float(((ctx.row_pos.to(torch.int64) + 1).clamp(max=window) if window
                          else ctx.row_pos.to(torch.int64) + 1).sum().item()) * n_heads * width)))
def attention_latent(q: torch.Tensor, k_new: Optional[torch.Tensor], k_pool: Optional[torch.Tensor],
                     page_table: Optional[torch.Tensor], page_tokens: int, ring_tokens: int, ctx,
                     out: torch.Tensor, scratch: Optional[torch.Tensor], sink: Optional[torch.Tensor],
                     n_heads: int, width: int, scale: float, window: int, splits: int,
                     rows_per_tile: int = 1) -> torch.Tensor:
    """bfloat16 attention of every head over ONE shared row per position, on the tensor
    cores (csrc/attention_latent.cu): ``q`` and ``out`` ``[rows, heads * width]``, keys (which
    are the values too) from the step's rows ``k_new`` ``[rows, width]`` or from the cache
    ``k_pool`` ``[pages, 1, page_tokens, width]``; ``sink`` one 32-bit value per head."""
    rows = out.shape[0]
    _want(q, torch.bfloat16, "q")
    _want(out, torch.bfloat16, "out")
    if tuple(q.shape) != (rows, n_heads * width) or tuple(out.shape) != (rows, n_heads * width):
        raise KernelError("attention_latent: q and out must be [rows, heads * width]")
    max_pages = 0
    if k_new is not None:
        _want(k_new, torch.bfloat16, "k_new")
        if tuple(k_new.shape) != (rows, width):
            raise KernelError("attention_latent: k_new must be [rows, width]")
    else:
        _want(k_pool, torch.bfloat16, "k_pool")
        if tuple(k_pool.shape[1:]) != (1, page_tokens, width) or page_table is None:
            raise KernelError("attention_latent: pool layout must be [pages, 1, page_tokens, width]")
        max_pages = page_table.shape[1]
    if splits > 1:
        need = attention_rows_scratch_bytes(rows, n_heads, width, splits)
        if scratch is None or scratch.numel() * scratch.element_size() < need:
            raise KernelError(f"attention_latent: {need} bytes of scratch memory are needed")
    if sink is not None:
        _f32(sink, n_heads, "sink")
    _check(library().sib_attention_latent(
        _ptr(q), _ptr(k_new), _ptr(k_pool if k_new is None else None),
        _ptr(page_table if k_new is None else None), c_int(max_pages), c_int(page_tokens),
        c_int(ring_tokens), _ptr(ctx.row_pos), _ptr(ctx.row_seq), _ptr(ctx.seq_slot),
        _ptr(ctx.seq_start), _ptr(ctx.seq_row0), _ptr(out), _ptr(scratch), _ptr(sink), c_int(rows),
        c_int(n_heads), c_int(width), c_float(scale), c_int(window), c_int(splits),
        c_int(rows_per_tile), _stream()))
    return out


def attention_decode_supports(n_heads: int, n_kv: int, head_dim: int, page_tokens: int) -> bool:
    return bool(library().sib_attention_decode_supports(c_int(n_heads), c_int(n_kv),
                                                        c_int(head_dim), c_int(page_tokens)))


def attention_decode_resident_warps(n_heads: int, n_kv: int, head_dim: int, warps: int = 4) -> int:
    """Warps of the decode attention kernel that the current device holds at a time for this
    shape, in blocks of ``warps`` warps (0: not a shape the kernel takes)."""
    return int(library().sib_attention_decode_resident_warps_of(c_int(n_heads), c_int(n_kv),
                                                                c_int(head_dim), c_int(warps)))


@_timed(lambda q, q_stride, k_pool, v_pool, page_table, page_tokens, ring_tokens, row_pos, row_seq,
        seq_slot, out, scratch, tickets, n_heads, n_kv, head_dim, scale, softcap, window, splits,
        warps=4, fresh=0, chunk=0, sink=None: _attention_cache_work(
            "attention_decode", row_pos, k_pool, n_heads, head_dim, window, out.shape[0], chunk=chunk))
def attention_decode(q: torch.Tensor, q_stride: int, k_pool: torch.Tensor, v_pool: torch.Tensor,
                     page_table: torch.Tensor, page_tokens: int, ring_tokens: int, row_pos,
                     row_seq, seq_slot, out: torch.Tensor, scratch: Optional[torch.Tensor],
                     tickets: Optional[torch.Tensor], n_heads: int, n_kv: int, head_dim: int,
                     scale: float, softcap: float, window: int, splits: int,
                     warps: int = 4, fresh: int = 0, chunk: int = 0,
                     sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of single rows over the bfloat16 cache (see csrc/attention_decode.cu).
    ``splits`` blocks of ``warps`` warps share the keys of a (row, kv head); with more than one they
    need ``scratch`` for their partial results and ``tickets``: int32 counters, one
    per (row, kv head), zero before the first call (every call leaves them zero).
    ``fresh``: the most positions of a sequence that the kernel before this one wrote (the
    rows a sequence has in this step); keys below them are fetched while that kernel still
    runs.  0: every load waits for it.  ``chunk`` > 0 (without a window): a row sees the
    positions of its own chunk; ``sink``: one 32-bit value per query head whose exponential
    joins the softmax's denominator."""
    global _launches
    rows = out.shape[0]
    _want(out, torch.bfloat16, "out")
    _want(k_pool, torch.bfloat16, "k_pool")
    _want(v_pool, torch.bfloat16, "v_pool")
    _want(page_table, torch.int32, "page_table")
    if q.dtype != torch.bfloat16:
        raise KernelError("attention_decode: q must be bfloat16")
    if tuple(k_pool.shape[1:]) != (n_kv, page_tokens, head_dim):
        raise KernelError("attention_decode: pool layout must be [pages, kv_heads, page_tokens, head_dim]")
    if splits > 1:
        need = attention_rows_scratch_bytes(rows, n_heads, head_dim, splits)
        if scratch is None or scratch.numel() * scratch.element_size() < need:
            raise KernelError(f"attention_decode: {need} bytes of scratch memory are needed")
        if tickets is None or tickets.dtype != torch.int32 or tickets.numel() < rows * n_kv:
            raise KernelError(f"attention_decode: {rows * n_kv} int32 ticket counters are needed")
    if sink is not None:
        _f32(sink, n_heads, "sink")
    _check(library().sib_attention_decode_masked(
        _ptr(q), c_int(q_stride), _ptr(k_pool), _ptr(v_pool), _ptr(page_table),
        c_int(page_table.shape[1]), c_int(page_tokens), c_int(ring_tokens), _ptr(row_pos),
        _ptr(row_seq), _ptr(seq_slot), _ptr(out), _ptr(scratch), _ptr(tickets), c_int(rows),
        c_int(n_heads), c_int(n_kv), c_int(head_dim), c_float(scale), c_float(softcap),
        c_int(window), c_int(splits), c_int(warps), c_int(fresh), c_int(chunk), _ptr(sink), _stream()))
    return out


def attention_prefill_supports(n_heads: int, n_kv: int, head_dim: int) -> bool:
    return bool(library().sib_attention_prefill_supports(c_int(n_heads), c_int(n_kv),
                                                         c_int(head_dim)))


@_timed(lambda qkv, out, seq_row0, seq_len, n_seqs, max_len, n_heads, n_kv, head_dim, scale,
        softcap, window: _prompt_work("attention_prefill (mma.sync)", qkv, seq_len, n_heads,
                                      head_dim, window))
def attention_prefill(qkv: torch.Tensor, out: torch.Tensor, seq_row0, seq_len, n_seqs: int,
                      max_len: int, n_heads: int, n_kv: int, head_dim: int, scale: float,
                      softcap: float, window: int) -> torch.Tensor:
    """Attention of packed bfloat16 prompts that start at position 0 over their
    own (rotated) keys and values (see csrc/attention_prefill.cu)."""
    _want(qkv, torch.bfloat16, "qkv")
    _want(out, torch.bfloat16, "out")
    if out.shape[0] != qkv.shape[0] or out.shape[1] != n_heads * head_dim:
        raise KernelError("attention_prefill: out must be [rows, heads * head_dim]")
    _check(library().sib_attention_prefill(
        _ptr(qkv), c_int(qkv.shape[1]), _ptr(out), _ptr(seq_row0), _ptr(seq_len), c_int(n_seqs),
        c_int(max_len), c_int(n_heads), c_int(n_kv), c_int(head_dim), c_float(scale),
        c_float(softcap), c_int(window), _stream()))
    return out


def attention_prefill_tc_supports(n_heads: int, n_kv: int, head_dim: int, width: int) -> bool:
    return bool(library().sib_attention_prefill_tc_supports(c_int(n_heads), c_int(n_kv),
                                                            c_int(head_dim), c_int(width)))


def attention_prefill_tc_split(n_seqs: int, max_len: int, n_heads: int, n_kv: int,
                               head_dim: int):
    """(bytes of scratch memory, ticket counters) that a launch of this shape needs to split
    its long blocks of query rows; (0, 0) if it would not split."""
    nbytes, n_tickets = c_longlong(0), c_int(0)
    from ctypes import byref
    library().sib_attention_prefill_tc_split(c_int(n_seqs), c_int(max_len), c_int(n_heads),
                                             c_int(n_kv), c_int(head_dim), byref(nbytes),
                                             byref(n_tickets))
    return int(nbytes.value), int(n_tickets.value)


def attention_prefill_tc_plan(lens: Sequence[int], n_heads: int, n_kv: int, head_dim: int,
                              window: int, first_query: Optional[Sequence[int]] = None):
    """(work items, bytes of scratch memory, ticket counters) of a launch for prompts of these
    lengths that runs as a balanced list of work items; (0, 0, 0) if it would run as a grid.
    ``first_query``: per sequence, the position from which rows are queries."""
    from ctypes import byref
    nbytes, n_tickets = c_longlong(0), c_int(0)
    arr = (c_int * len(lens))(*[int(n) for n in lens])
    q0 = None if first_query is None else (c_int * len(lens))(*[int(n) for n in first_query])
    n_items = library().sib_attention_prefill_tc_plan(arr, q0, c_int(len(lens)), c_int(n_heads),
                                                      c_int(n_kv), c_int(head_dim), c_int(window),
                                                      byref(nbytes), byref(n_tickets))
    return int(n_items), int(nbytes.value), int(n_tickets.value)


@_timed(lambda qkv, out, seq_row0, seq_len, n_seqs, max_len, n_heads, n_kv, head_dim, scale,
        softcap, window, scratch=None, tickets=None, host_lens=None, seq_q0=None,
        host_q0=None, sink=None, extra=None: _prompt_work(
            "attention_prefill_tc (tcgen05)", qkv, seq_len, n_heads, head_dim, window))
def attention_prefill_tc(qkv: torch.Tensor, out: torch.Tensor, seq_row0, seq_len, n_seqs: int,
                         max_len: int, n_heads: int, n_kv: int, head_dim: int, scale: float,
                         softcap: float, window: int, scratch: Optional[torch.Tensor] = None,
                         tickets: Optional[torch.Tensor] = None,
                         host_lens: Optional[Sequence[int]] = None,
                         seq_q0: Optional[torch.Tensor] = None,
                         host_q0: Optional[Sequence[int]] = None,
                         sink: Optional[torch.Tensor] = None,
                         extra: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The prompt attention on tcgen05 (see csrc/attention_prefill_tc.cu).  ``sink``: one 32-bit
    value per head whose exponential joins every row's denominator (no cap then).  ``extra``:
    32-bit ``[rows, heads, head_dim + 2]``, per row and head the (max, sum, accumulator) of keys
    that another kernel has summed (``attention_rows`` with ``cells_only``), joined with this
    kernel's own sums before the last division (no cap, no sink then).  With ``scratch``
    and ``tickets`` (int32, zero before the first call; every call leaves them zero) of the
    sizes ``attention_prefill_tc_split`` gives, a launch that cannot fill the device runs its
    long blocks of query rows as two halves.  With ``host_lens`` (the prompts' lengths, as
    ``seq_len`` holds them on the device) and memory of the sizes ``attention_prefill_tc_plan``
    gives, the launch is a list of work items ordered by their work, with the blocks split
    that make the busiest SM's share smallest.  ``seq_q0`` (int32 on the device, ``host_q0``
    the same on the host): per sequence the position from which rows are queries; the rows
    before it bring keys and values only and their output rows are not written."""
    _want(qkv, torch.bfloat16, "qkv")
    _want(out, torch.bfloat16, "out")
    if out.shape[0] != qkv.shape[0] or out.shape[1] != n_heads * head_dim:
        raise KernelError("attention_prefill_tc: out must be [rows, heads * head_dim]")
    if tickets is not None:
        _want(tickets, torch.int32, "tickets")
    if sink is not None:
        _f32(sink, n_heads, "sink")
    if extra is not None:
        _f32(extra, qkv.shape[0] * n_heads * (head_dim + 2), "extra")
    _check(library().sib_attention_prefill_tc(
        _ptr(qkv), c_int(qkv.shape[1]), c_int(qkv.shape[0]), _ptr(out), _ptr(seq_row0),
        _ptr(seq_len), c_int(n_seqs), c_int(max_len), c_int(n_heads), c_int(n_kv), c_int(head_dim),
        c_float(scale), c_float(softcap), c_int(window), _ptr(scratch),
        c_longlong(scratch.numel() * scratch.element_size() if scratch is not None else 0),
        _ptr(tickets), c_int(tickets.numel() if tickets is not None else 0),
        None if host_lens is None else (c_int * len(host_lens))(*[int(n) for n in host_lens]),
        _ptr(seq_q0),
        None if host_q0 is None else (c_int * len(host_q0))(*[int(n) for n in host_q0]),
        _ptr(sink), _ptr(extra), _stream()))
    return out


@_timed(lambda packed, k_pool, *a, **kw: ("gather_kv_rows", 0, 0))
def gather_kv_rows(packed: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                   page_table: torch.Tensor, seq_slot: torch.Tensor, seq_from: torch.Tensor,
                   seq_upto: torch.Tensor, seq_row0: torch.Tensor, most: int, page_tokens: int,
                   ring_tokens: int, n_heads: int, n_kv: int, head_dim: int) -> torch.Tensor:
    """Keys and values of the positions [seq_from[b], seq_upto[b]) that sequence b holds in
    the paged cache, into rows seq_row0[b] + position of the packed q|k|v buffer (q columns
    of those rows: zero).  ``most``: the most positions of any sequence."""
    _want(packed, torch.bfloat16, "packed")
    _want(k_pool, torch.bfloat16, "k_pool")
    _want(v_pool, torch.bfloat16, "v_pool")
    for t, name in ((page_table, "page_table"), (seq_slot, "seq_slot"), (seq_from, "seq_from"),
                    (seq_upto, "seq_upto"), (seq_row0, "seq_row0")):
        _want(t, torch.int32, name)
    if packed.shape[1] != (n_heads + 2 * n_kv) * head_dim:
        raise KernelError("gather_kv_rows: the packed rows do not fit the head counts")
    _check(library().sib_gather_kv_rows(
        _ptr(packed), _ptr(k_pool), _ptr(v_pool), _ptr(page_table), _ptr(seq_slot), _ptr(seq_from),
        _ptr(seq_upto), _ptr(seq_row0), c_int(seq_slot.numel()), c_int(most), c_int(n_heads),
        c_int(n_kv), c_int(head_dim), c_int(page_table.shape[1]), c_int(page_tokens),
        c_int(ring_tokens), _stream()))
    return packed


def attention_prefill_tc_error(clear: bool = True) -> int:
    """0, or the code left by a block of attention_prefill_tc whose bounded wait ran out
    (synchronises the device)."""
    torch.cuda.synchronize()
    return int(library().sib_attention_prefill_tc_error(c_int(1 if clear else 0)))


SKINNY_MAX_ROWS = 64


def _product_work(kind, x, w, out):
    return (f"{kind} {w.shape[0]}x{w.shape[1]}", _nbytes(w, out) + x.shape[0] * x.shape[1]
            * x.element_size(), 2.0 * x.shape[0] * w.shape[0] * w.shape[1])


@_timed(lambda x, w, out, epilogue=EPI_NONE, cap=0.0: _product_work("skinny_linear", x, w, out))
def skinny_linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_NONE,
                  cap: float = 0.0) -> torch.Tensor:
    """out = x . w^T for at most 64 rows of bfloat16 x (see csrc/linear_skinny.cu)."""
    _want(x, torch.bfloat16, "x", contiguous=False)
    _want(w, torch.bfloat16, "w")
    _want(out, out.dtype, "out", contiguous=False)
    R, K = x.shape
    N = w.shape[0]
    n_out = N // 2 if epilogue in GATED_EPILOGUES else N
    if w.shape[1] != K or tuple(out.shape) != (R, n_out) or x.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("skinny_linear: shapes do not fit")
    _check(library().sib_skinny_linear(_ptr(w), _ptr(x), _ptr(out), _code(out.dtype), c_int(R),
                                       c_int(N), c_int(K), c_int(x.stride(0)),
                                       c_int(out.stride(0)), c_int(epilogue), c_float(cap),
                                       _stream()))
    return out


def linear_stream_supports(R: int, N: int, K: int, x_stride: int) -> bool:
    return bool(library().sib_linear_stream_supports(c_int(R), c_int(N), c_int(K), c_int(x_stride)))


@_timed(lambda x, w, out, epilogue=EPI_NONE, cap=0.0, ksplit=0, stages=0: _product_work(
    "linear_stream", x, w, out))
def linear_stream(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_NONE,
                  cap: float = 0.0, ksplit: int = 0, stages: int = 0) -> torch.Tensor:
    """out = x . w^T for at most 16 rows of bfloat16 x, the weights staged through shared
    memory by TMA (see csrc/linear_stream.cu).  ``ksplit`` blocks of a cluster share a tile
    of weight rows, ``stages`` tiles are in flight per block; 0 lets the launcher choose."""
    _want(x, torch.bfloat16, "x", contiguous=False)
    _want(w, torch.bfloat16, "w")
    _want(out, out.dtype, "out", contiguous=False)
    R, K = x.shape
    N = w.shape[0]
    n_out = N // 2 if epilogue in GATED_EPILOGUES else N
    if w.shape[1] != K or tuple(out.shape) != (R, n_out) or x.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("linear_stream: shapes do not fit")
    _check(library().sib_linear_stream(_ptr(w), _ptr(x), _ptr(out), _code(out.dtype), c_int(R),
                                       c_int(N), c_int(K), c_int(x.stride(0)),
                                       c_int(out.stride(0)), c_int(epilogue), c_float(cap),
                                       c_int(ksplit), c_int(stages), _stream()))
    return out


def linear_rows_tc_max_rows() -> int:
    return int(library().sib_linear_rows_tc_max_rows())


@_timed(lambda x, w, out, epilogue=EPI_NONE, cap=0.0, ksplit=0, stages=0: _product_work(
    "linear_rows_tc", x, w, out))
def linear_rows_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_NONE,
                   cap: float = 0.0, ksplit: int = 0, stages: int = 0) -> torch.Tensor:
    """out = x . w^T for at most 128 rows of bfloat16 x on the tcgen05 tensor cores, the
    weights streamed through a ring of TMA stages (see csrc/linear_rows_tc.cu).  ``ksplit``
    blocks of a cluster share a tile of 128 weight rows, ``stages`` stages are in flight per
    block; 0 lets the launcher choose."""
    _want(x, torch.bfloat16, "x", contiguous=False)
    _want(w, torch.bfloat16, "w")
    _want(out, out.dtype, "out", contiguous=False)
    R, K = x.shape
    N = w.shape[0]
    n_out = N // 2 if epilogue in GATED_EPILOGUES else N
    if w.shape[1] != K or tuple(out.shape) != (R, n_out) or x.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("linear_rows_tc: shapes do not fit")
    _check(library().sib_linear_rows_tc(_ptr(w), _ptr(x), _ptr(out), _code(out.dtype), c_int(R),
                                        c_int(N), c_int(K), c_int(x.stride(0)),
                                        c_int(out.stride(0)), c_int(epilogue), c_float(cap),
                                        c_int(ksplit), c_int(stages), _stream()))
    return out


@_timed(lambda x, w, out, *a, **kw: _product_work("skinny_linear_rope", x, w, out))
def skinny_linear_rope(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, row_pos, row_seq,
                       seq_slot, seq_end, inv_freq: torch.Tensor,
                       k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
                       page_table: Optional[torch.Tensor], page_tokens: int, ring_tokens: int,
                       n_heads: int, n_kv: int, head_dim: int) -> torch.Tensor:
    """The q|k|v product of at most 16 bfloat16 rows that also rotates q and k (half-split
    pairs over the whole head) and writes k and v into the paged cache as well as into
    ``out`` (see csrc/linear_skinny.cu, RopeTail).  ``n_kv == 0``: q rows only, nothing stored."""
    _want(x, torch.bfloat16, "x", contiguous=False)
    _want(w, torch.bfloat16, "w")
    _want(out, torch.bfloat16, "out", contiguous=False)
    _want(inv_freq, torch.float32, "inv_freq")
    R, K = x.shape
    N = (n_heads + 2 * n_kv) * head_dim
    if tuple(w.shape) != (N, K) or tuple(out.shape) != (R, N) or x.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("skinny_linear_rope: shapes do not fit the head counts")
    if inv_freq.numel() * 2 != head_dim:
        raise KernelError("skinny_linear_rope: one frequency per pair of the whole head")
    max_pages = 0
    if n_kv:
        _want(k_pool, torch.bfloat16, "k_pool")
        _want(v_pool, torch.bfloat16, "v_pool")
        _want(page_table, torch.int32, "page_table")
        max_pages = page_table.shape[1]
        if tuple(k_pool.shape[1:]) != (n_kv, page_tokens, head_dim):
            raise KernelError("skinny_linear_rope: pool layout must be [pages, kv_heads, page_tokens, head_dim]")
    _check(library().sib_skinny_linear_rope(
        _ptr(w), _ptr(x), _ptr(out), c_int(R), c_int(K), c_int(x.stride(0)), c_int(out.stride(0)),
        _ptr(row_pos), _ptr(row_seq), _ptr(seq_slot), _ptr(seq_end), _ptr(inv_freq),
        _ptr(k_pool) if n_kv else c_void_p(0), _ptr(v_pool) if n_kv else c_void_p(0),
        _ptr(page_table) if n_kv else c_void_p(0), c_int(max_pages), c_int(page_tokens),
        c_int(ring_tokens), c_int(n_heads), c_int(n_kv), c_int(head_dim), _stream()))
    return out


def gemm_tcgen05_supports(R: int, N: int, K: int, x_stride: int) -> bool:
    return bool(library().sib_gemm_tcgen05_supports(c_int(R), c_int(N), c_int(K),
                                                    c_longlong(x_stride)))


@_timed(lambda x, w, out, epilogue=EPI_NONE, cap=0.0, one_block=False: _product_work(
    "gemm_tcgen05", x, w, out))
def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_NONE,
                 cap: float = 0.0, one_block: bool = False) -> torch.Tensor:
    """out = x . w^T for bfloat16 x and w on tcgen05 (see csrc/gemm_tcgen05.cu).  More than
    128 rows go to the kernel that works on pairs of SMs unless ``one_block`` is set."""
    _want(x, torch.bfloat16, "x", contiguous=False)
    _want(w, torch.bfloat16, "w")
    _want(out, out.dtype, "out", contiguous=False)
    R, K = x.shape
    N = w.shape[0]
    n_out = N // 2 if epilogue in GATED_EPILOGUES else N
    if w.shape[1] != K or tuple(out.shape) != (R, n_out) or x.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm_tcgen05: shapes do not fit")
    entry = library().sib_gemm_tcgen05_one_block if one_block else library().sib_gemm_tcgen05
    _check(entry(_ptr(w), _ptr(x), _ptr(out), _code(out.dtype), c_int(R), c_int(N), c_int(K),
                 c_longlong(x.stride(0)), c_int(out.stride(0)), c_int(epilogue), c_float(cap),
                 _stream()))
    return out


def gemm_tcgen05_error(clear: bool = True) -> int:
    """0, or the code left by a block of gemm_tcgen05 whose bounded wait ran out
    (synchronises the device)."""
    torch.cuda.synchronize()
    return int(library().sib_gemm_tcgen05_error(c_int(1 if clear else 0)))


@_timed(lambda logits, *a, **kw: ("sample_rows", _nbytes(logits), 0))
def sample_rows(logits: torch.Tensor, temperature: float, top_k: int, top_p: float,
                rng_state: Optional[torch.Tensor], out: torch.Tensor,
                rng_index: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of 32-bit logits; advances each row's generator by one draw.
    ``rng_index[row]`` (int32) says which element of ``rng_state`` a row uses."""
    _want(logits, torch.float32, "logits", contiguous=False)
    _want(out, torch.int32, "out")
    rows, vocab = logits.shape
    if logits.stride(1) != 1 or out.numel() != rows:
        raise KernelError("sample_rows: shapes do not fit")
    if rng_state is not None:
        _want(rng_state, torch.int64, "rng_state")
        if rng_index is None and rng_state.numel() != rows:
            raise KernelError("sample_rows: one generator state per row")
        if rng_index is not None:
            _want(rng_index, torch.int32, "rng_index")
    _check(library().sib_sample_rows(_ptr(logits), c_longlong(logits.stride(0)), c_int(rows),
                                     c_int(vocab), c_float(temperature), c_int(top_k),
                                     c_float(top_p), _ptr(rng_state), _ptr(rng_index), _ptr(out),
                                     _stream()))
    return out


class KernelWatch:
    """The verdicts of kernels whose waits are bounded, brought to the host without a
    synchronisation of their own.

    ``fetch()`` enqueues an asynchronous copy of the device's error words into a pinned
    buffer on the current stream; after the caller's next synchronisation of that stream
    (the read of the sampled tokens, the copy of the logits) ``check()`` looks at the
    buffer and raises :class:`KernelError` naming the kernel and its code if a wait ran
    out, after clearing the word.  The reference logs a failed launch and goes on
    (src/backend/cuda/mod.rs:379-397)."""

    def __init__(self):
        lib = library()
        lib.sib_error_word_name.restype = ctypes.c_char_p
        self.n = int(lib.sib_error_words())
        self.host = torch.zeros(self.n, dtype=torch.int32).pin_memory()
        self.names = [lib.sib_error_word_name(c_int(i)).decode() for i in range(self.n)]
        self.pending = False

    def fetch(self) -> None:
        if library().sib_kernel_errors_fetch(c_void_p(self.host.data_ptr()), _stream()) != 0:
            raise KernelError(library().sib_last_error().decode())
        self.pending = True

    def check(self) -> None:
        """Call after the stream that ``fetch`` ran on has been synchronised."""
        if not self.pending:
            return
        self.pending = False
        words = self.host.tolist()
        bad = [(i, c) for i, c in enumerate(words) if c]
        if not bad:
            return
        for i, _ in bad:
            set_kernel_error(i, 0)
        self.host.zero_()
        raise KernelError("; ".join(
            f"a bounded wait of {self.names[i] or 'kernel %d' % i} ran out (code {c}): "
            f"its output is incomplete" for i, c in bad))


def set_kernel_error(word: int, code: int) -> None:
    """Set a device error word from the host (0 clears it; tests use it to stand for a
    kernel that gave up)."""
    if library().sib_kernel_error_set(c_int(word), c_int(code), _stream()) != 0:
        raise KernelError(library().sib_last_error().decode())


# --------------------------------------------------------------------------
# decode_chain: several dependent few-row steps as one kernel (csrc/decode_chain.cu)

CHAIN_PRODUCT, CHAIN_NORM = 0, 1
EPI_ROPE = 3


class ChainPhase(ctypes.Structure):
    """Mirrors SibChainPhase of csrc/decode_chain.h."""
    _fields_ = [
        ("kind", c_int), ("epi", c_int),
        ("w", c_void_p), ("x", c_void_p), ("y", c_void_p),
        ("N", c_int), ("K", c_int), ("x_stride", c_int), ("y_stride", c_int), ("out_f32", c_int),
        ("cap", c_float),
        ("row_pos", c_void_p), ("row_seq", c_void_p), ("seq_slot", c_void_p), ("seq_end", c_void_p),
        ("inv_freq", c_void_p), ("k_pool", c_void_p), ("v_pool", c_void_p), ("page_table", c_void_p),
        ("n_heads", c_int), ("n_kv", c_int), ("head_dim", c_int), ("max_pages", c_int),
        ("page_tokens", c_int), ("ring_tokens", c_int),
        ("a", c_void_p), ("post_gain", c_void_p), ("h", c_void_p), ("pre_gain", c_void_p),
        ("out", c_void_p), ("rows", c_void_p),
        ("post_eps", c_float), ("pre_eps", c_float),
        ("hidden", c_int), ("a_stride", c_int), ("out_stride", c_int),
    ]


def _addr(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


def chain_product(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_NONE,
                  cap: float = 0.0, rope: Optional[dict] = None) -> ChainPhase:
    """A product phase: out = epilogue(x . w^T).  ``rope``: the arguments of
    ``skinny_linear_rope`` by name, for the q|k|v product that rotates and stores."""
    _want(x, torch.bfloat16, "x", contiguous=False)
    _want(w, torch.bfloat16, "w")
    R, K = x.shape
    N = w.shape[0]
    n_out = N // 2 if epilogue in GATED_EPILOGUES else N
    if w.shape[1] != K or tuple(out.shape) != (R, n_out) or x.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("chain_product: shapes do not fit")
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError("chain_product: outputs are bfloat16 or float32")
    ph = ChainPhase(kind=CHAIN_PRODUCT, epi=EPI_ROPE if rope is not None else epilogue,
                    w=w.data_ptr(), x=x.data_ptr(), y=out.data_ptr(), N=N, K=K,
                    x_stride=x.stride(0), y_stride=out.stride(0),
                    out_f32=1 if out.dtype == torch.float32 else 0, cap=cap)
    if rope is not None:
        n_kv = rope["n_kv"]
        for name in ("row_pos", "row_seq", "seq_slot", "seq_end"):
            _want(rope[name], torch.int32, name)
            setattr(ph, name, rope[name].data_ptr())
        _want(rope["inv_freq"], torch.float32, "inv_freq")
        if rope["inv_freq"].numel() * 2 != rope["head_dim"]:
            raise KernelError("chain_product: one frequency per pair of the whole head")
        ph.inv_freq = rope["inv_freq"].data_ptr()
        if n_kv:
            _want(rope["k_pool"], torch.bfloat16, "k_pool")
            _want(rope["v_pool"], torch.bfloat16, "v_pool")
            _want(rope["page_table"], torch.int32, "page_table")
            if tuple(rope["k_pool"].shape[1:]) != (n_kv, rope["page_tokens"], rope["head_dim"]):
                raise KernelError("chain_product: pool layout must be [pages, kv_heads, page_tokens, head_dim]")
            ph.k_pool, ph.v_pool = rope["k_pool"].data_ptr(), rope["v_pool"].data_ptr()
            ph.page_table = rope["page_table"].data_ptr()
            ph.max_pages = rope["page_table"].shape[1]
        ph.n_heads, ph.n_kv, ph.head_dim = rope["n_heads"], n_kv, rope["head_dim"]
        ph.page_tokens, ph.ring_tokens = rope["page_tokens"], rope["ring_tokens"]
    return ph


def chain_norm(a: Optional[torch.Tensor], post_gain: Optional[torch.Tensor], post_eps: float,
               h: torch.Tensor, pre_gain: Optional[torch.Tensor], pre_eps: float,
               out: Optional[torch.Tensor], rows: Optional[torch.Tensor] = None) -> ChainPhase:
    """A "norm, add, norm" phase (see ``add_rms_norm``); without ``a`` a plain norm of the
    rows of h that ``rows`` names."""
    _want(h, torch.float32, "h")
    hidden = h.shape[1]
    if a is not None:
        _want(a, torch.bfloat16, "a", contiguous=False)
        if tuple(a.shape) != tuple(h.shape) or a.stride(1) != 1:
            raise KernelError("chain_norm: a and h differ in shape")
    for gname, gt in (("post_gain", post_gain), ("pre_gain", pre_gain)):
        if gt is not None:
            _want(gt, torch.float32, gname)
            if gt.numel() != hidden:
                raise KernelError(f"chain_norm: {gname} has the wrong length")
    if pre_gain is not None:
        if out is None:
            raise KernelError("chain_norm: pre_gain needs out")
        _want(out, torch.bfloat16, "out", contiguous=False)
    if rows is not None:
        _want(rows, torch.int32, "rows")
    return ChainPhase(kind=CHAIN_NORM, a=_addr(a), post_gain=_addr(post_gain), h=h.data_ptr(),
                      pre_gain=_addr(pre_gain), out=_addr(out), rows=_addr(rows),
                      post_eps=post_eps, pre_eps=pre_eps, hidden=hidden,
                      a_stride=a.stride(0) if a is not None else 0,
                      out_stride=out.stride(0) if out is not None else 0)


def decode_chain_max_phases() -> int:
    return int(library().sib_decode_chain_max_phases())


def _chain_work(phases, rows, sync, stages=0):
    nbytes = flops = 0
    for ph in phases:
        if ph.kind == CHAIN_PRODUCT:
            nbytes += ph.N * ph.K * 2 + rows * (ph.K + ph.N) * 2
            flops += 2.0 * rows * ph.N * ph.K
        else:
            nbytes += rows * ph.hidden * 12
    return f"decode_chain of {len(phases)}", nbytes, flops


@_timed(_chain_work)
def _decode_chain(phases, rows, sync, stages=0):
    arr = (ChainPhase * len(phases))(*phases)
    _check(library().sib_decode_chain(arr, c_int(len(phases)), c_int(rows), c_int(stages),
                                      _ptr(sync), _stream()))


def decode_chain(phases, rows: int, sync: torch.Tensor, stages: int = 0) -> None:
    """Run ``phases`` (from ``chain_product`` / ``chain_norm``) in order as one kernel for a
    step of ``rows`` rows.  ``sync``: two int32 counters on the device, zero before the
    first call (every call leaves them zero)."""
    _want(sync, torch.int32, "sync")
    if sync.numel() < 2:
        raise KernelError("decode_chain: two counters are needed")
    _decode_chain(list(phases), rows, sync, stages)
