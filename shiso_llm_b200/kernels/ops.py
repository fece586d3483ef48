"""The kernel table: one Python function per CUDA kernel, launched on the current stream.

Every function checks shapes, types, contiguity and device, then calls the C launcher
with raw pointers.  Nothing here computes on the CPU and nothing calls a library
routine for the model's arithmetic; if the extension cannot be loaded the first call
raises.  Inputs must be CUDA tensors.
"""

from __future__ import annotations

from typing import Optional

import torch

from .library import KernelLibraryError, library

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}

# How many kernels were launched through this table (bench.py reports it).
launch_count = 0


class KernelError(RuntimeError):
    pass


_ERRORS = {
    1001: "unsupported element type",
    1002: "unsupported shape",
    1003: "misaligned pointer or stride",
    1004: "unsupported combination",
}


def require() -> None:
    """Loads the extension now, or raises with the reason."""
    if not torch.cuda.is_available():
        raise KernelLibraryError("no CUDA device: this engine has no CPU path")
    library()


def _code(t: torch.Tensor) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"element type {t.dtype} is not float32 or bfloat16") from None


def _ptr(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_DEVICE_INDEX = None  # the one device this process's kernel library works on, once bound


def resolve_binding(wanted_index, bound_index, current_index) -> int:
    """Which device an engine asked for ends up on, or the refusal.  ``wanted_index`` is the
    index the caller named (None for a bare "cuda"), ``bound_index`` the device the library is
    bound to already (None: not yet), ``current_index`` the process's current device."""
    index = current_index if wanted_index is None else wanted_index
    if bound_index is not None and index != bound_index:
        raise KernelError(
            f"this process's kernel library works on cuda:{bound_index} (attributes of its kernels and its status word "
            f"live there); an engine on cuda:{index} needs a process of its own"
        )
    return index


def bind_device(device) -> int:
    """Binds the kernel library to ``device`` (a torch.device of type cuda) and makes it the
    current device; returns its index.  The library keeps per-process state for one device -
    which kernels were given their shared-memory attribute, the status word of the bounded
    waits - and every launch goes to the current device's
    stream, so all engines of a process share one device; another one is refused here, before
    a pointer of one device could reach a kernel on another."""
    global _DEVICE_INDEX
    device = torch.device(device)
    if device.type != "cuda":
        raise KernelError(f"the CUDA kernels cannot run on {device}")
    index = resolve_binding(device.index, _DEVICE_INDEX, torch.cuda.current_device())
    if index >= torch.cuda.device_count():
        raise KernelError(f"cuda:{index} does not exist: this process sees {torch.cuda.device_count()} device(s)")
    torch.cuda.set_device(index)
    _DEVICE_INDEX = index
    return index


def _stream() -> int:
    """The current stream's handle.  Asked for at every launch (a graph capture changes it), so
    through torch's raw binding where it exists: the public call costs 13 us of Python per launch,
    a third of a kernel-by-kernel step's host time."""
    global _DEVICE_INDEX
    if _RAW_STREAM is None:
        return torch.cuda.current_stream().cuda_stream
    if _DEVICE_INDEX is None:
        _DEVICE_INDEX = torch.cuda.current_device()
    return _RAW_STREAM(_DEVICE_INDEX)


def _check(t: torch.Tensor, name: str, dtype=None, ndim=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name}: expected a CUDA tensor, got one on {t.device}")
    if not t.is_contiguous():
        raise KernelError(f"{name}: expected a contiguous tensor")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: expected {dtype}, got {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise KernelError(f"{name}: expected {ndim} dimensions, got shape {tuple(t.shape)}")


_region = None  # the open profile region, if any (kernels/profile.py)
_plain_library = library


class _TimedLibrary:
    """The kernel library while a region is open: an event is recorded before every call."""

    def __init__(self, lib):
        self._lib = lib

    def __getattr__(self, name):
        fn = getattr(self._lib, name)
        if not name.startswith("shiso_"):
            return fn

        def call(*args):
            if _region is not None:
                _region.before()
            return fn(*args)

        return call


def profile_start() -> None:
    """Opens a region: until ``profile_stop`` every launch stands between two events."""
    global _region, library
    from .profile import Region

    if _region is not None:
        raise KernelError("a profile region is already open")
    require()
    timed = _TimedLibrary(_plain_library())
    library = lambda: timed  # noqa: E731
    _region = Region(torch)


def profile_stop():
    """Closes the region: ((kernel, shape, launches, microseconds) in launch order, host
    microseconds, microseconds from the first launch's start to the last one's end)."""
    global _region, library
    if _region is None:
        raise KernelError("no profile region is open")
    region, _region = _region, None
    library = _plain_library
    return region.close()


def _done(status: int, what: str, launches: int = 1, shape=()) -> None:
    global launch_count
    if status != 0:
        why = _ERRORS.get(status)
        if why is None:
            why = f"CUDA error {status} at launch"
        raise KernelError(f"{what}: {why} (status {status})")
    launch_count += launches
    if _region is not None:
        _region.mark(what, "x".join(str(int(d)) for d in shape), launches)


# --------------------------------------------------------------------------- rows


def embed(ids: torch.Tensor, table: torch.Tensor, feed_index=None, fed_tokens=None, scale: float = 1.0) -> torch.Tensor:
    """Rows of ``table`` for ``ids``, times ``scale`` (in float32).  Where ``feed_index[t] >= 0`` the
    id is read on the device from ``fed_tokens[feed_index[t]]`` instead (a token picked a step
    earlier that the host has not seen)."""
    _check(ids, "ids", torch.int32, 1)
    _check(table, "embedding table", None, 2)
    tokens, (vocab, hidden) = ids.shape[0], table.shape
    if (feed_index is None) != (fed_tokens is None):
        raise KernelError("embed: feed_index and fed_tokens come together")
    if feed_index is not None:
        _check(feed_index, "feed_index", torch.int32, 1)
        _check(fed_tokens, "fed_tokens", torch.int32, 1)
        if feed_index.shape[0] != tokens:
            raise KernelError(f"feed_index has {feed_index.shape[0]} entries for {tokens} rows")
    out = torch.empty((tokens, hidden), dtype=torch.float32, device=table.device)
    status = library().shiso_embed_scaled(
        _ptr(ids), _ptr(feed_index), _ptr(fed_tokens), _ptr(table), _code(table), _ptr(out), tokens, hidden, vocab, float(scale), _stream()
    )
    _done(status, "embed", shape=(tokens, hidden))
    return out


def stream_add(residual, deltas, vector, in_place=True):
    """``residual + sum(deltas) + vector``: float32 rows ``[T, H]``, up to three blocks of rows of the
    same shape (float32 or bfloat16 each) and a float32 vector ``[H]`` added to every row (or None).
    Written into ``residual``, or with ``in_place=False`` into rows of their own; returns them."""
    _check(residual, "residual", torch.float32, 2)
    tokens, hidden = residual.shape
    deltas = tuple(deltas)
    if len(deltas) > 3:
        raise KernelError(f"{len(deltas)} blocks of rows to add; the kernel takes three")
    for d in deltas:
        _check(d, "rows to add", None, 2)
        if d.shape != residual.shape:
            raise KernelError(f"rows of {tuple(d.shape)} added to a residual of {tuple(residual.shape)}")
    if vector is not None:
        _check(vector, "vector", torch.float32, 1)
        if vector.shape[0] != hidden:
            raise KernelError(f"a vector of {vector.shape[0]} for rows of {hidden}")
    out = residual if in_place else torch.empty_like(residual)
    d = list(deltas) + [None] * (3 - len(deltas))
    status = library().shiso_stream_add(
        _ptr(residual), _ptr(out), _ptr(d[0]), _code(d[0]) if d[0] is not None else 0, _ptr(d[1]), _code(d[1]) if d[1] is not None else 0,
        _ptr(d[2]), _code(d[2]) if d[2] is not None else 0, _ptr(vector), tokens, hidden, _stream(),
    )
    _done(status, "stream_add", shape=(tokens, hidden))
    return out


def add_dyt(residual, deltas, alpha, w, b, out_dtype, rows=None):
    """``tanh(alpha * x) * w + b`` of ``x = residual + sum(deltas)``: ``residual`` float32 ``[T, H]``,
    up to two ``deltas`` ``[T, H]`` in the output type.  Without ``rows`` the sum is stored back into
    ``residual``; with ``rows`` (int32) only those rows are summed and squashed, into ``[len(rows), H]``."""
    _check(residual, "residual", torch.float32, 2)
    _check(w, "norm weight", torch.float32, 1)
    _check(b, "norm bias", torch.float32, 1)
    tokens, hidden = residual.shape
    if w.shape[0] != hidden or b.shape[0] != hidden:
        raise KernelError(f"norm weight / bias of {w.shape[0]} / {b.shape[0]} entries for rows of {hidden}")
    deltas = tuple(deltas)
    if len(deltas) > 2:
        raise KernelError(f"{len(deltas)} block outputs to add; the kernel takes two")
    for d in deltas:
        _check(d, "delta", out_dtype, 2)
        if d.shape != residual.shape:
            raise KernelError(f"delta {tuple(d.shape)} does not match the residual {tuple(residual.shape)}")
    out_rows = tokens
    if rows is not None:
        _check(rows, "rows", torch.int32, 1)
        out_rows = rows.shape[0]
    out = torch.empty((out_rows, hidden), dtype=out_dtype, device=residual.device)
    d = list(deltas) + [None] * (2 - len(deltas))
    status = library().shiso_add_dyt(
        _ptr(residual), _ptr(d[0]), _ptr(d[1]), _ptr(rows), _ptr(w), _ptr(b), float(alpha), _ptr(out), _code(out), out_rows, hidden, _stream()
    )
    _done(status, "dyt" if not deltas else "add + dyt", shape=(out_rows, hidden))
    return out


def gather_rows(x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    _check(x, "x", torch.float32, 2)
    _check(rows, "rows", torch.int32, 1)
    out = torch.empty((rows.shape[0], x.shape[1]), dtype=torch.float32, device=x.device)
    _done(library().shiso_gather_rows(_ptr(x), _ptr(rows), _ptr(out), rows.shape[0], x.shape[1], _stream()), "gather_rows")
    return out


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    return add_rmsnorm(x, None, w, eps, out_dtype, None)


def add_rmsnorm(residual, delta, w, eps, out_dtype, rows=None):
    """``residual`` float32 [T, H]; ``delta`` [T, H] in the output type or None; returns
    norm(residual + delta).  Without ``rows`` the sum is stored back into ``residual``."""
    _check(residual, "residual", torch.float32, 2)
    _check(w, "norm weight", torch.float32, 1)
    tokens, hidden = residual.shape
    if w.shape[0] != hidden:
        raise KernelError(f"norm weight has {w.shape[0]} entries for rows of {hidden}")
    if delta is not None:
        _check(delta, "delta", out_dtype, 2)
        if delta.shape != residual.shape:
            raise KernelError(f"delta {tuple(delta.shape)} does not match the residual {tuple(residual.shape)}")
    out_rows = tokens
    if rows is not None:
        _check(rows, "rows", torch.int32, 1)
        out_rows = rows.shape[0]
    out = torch.empty((out_rows, hidden), dtype=out_dtype, device=residual.device)
    status = library().shiso_rmsnorm(
        _ptr(residual), _ptr(delta), _ptr(rows), _ptr(w), _ptr(out), _code(out), out_rows, hidden, float(eps), _stream()
    )
    _done(status, "rmsnorm" if delta is None else "add + rmsnorm", shape=(out_rows, hidden))
    return out


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    _check(gate_up, "gate_up", None, 2)
    tokens, two_inter = gate_up.shape
    if two_inter % 2:
        raise KernelError(f"gate_up rows of {two_inter} cannot be split in two halves")
    out = torch.empty((tokens, two_inter // 2), dtype=gate_up.dtype, device=gate_up.device)
    _done(library().shiso_swiglu(_ptr(gate_up), _ptr(out), _code(gate_up), tokens, two_inter // 2, _stream()), "swiglu")
    return out


# --------------------------------------------------------------------------- matrix products


_SM_COUNT = None
PROMPT_MIN_TOKENS = 193  # from here the persistent tensor-memory kernels (tokens as the MMA's M operand): plain products on pairs of SMs; below, 64-token tiles with K split over a cluster are faster
# Portions of a few hundred rows times a matrix of few rows: the kernel for long portions would have a
# handful of 256 x 256 tiles for 74 pairs of SMs and walk a long K alone.  Up to FEW_PAIR_TILES such
# tiles, and while tiles of 128 features x 64 tokens stay within the CTAs that are resident at once, the
# product runs as those tiles on single SMs with K split over a cluster (576 rows: 2048 x 5632 31.2 ->
# 22.2 us, 2048 x 2048 14.9 -> 12.3 us, 3072 x 2048 17.2 -> 14.6 us; 1024 x 4608 at 512 rows 26.2 -> 12.5 us;
# 6144 x 2048 at 512 rows would lose, 18.0 -> 28.2 us, and is left where it was).
FEW_PAIR_TILES = 36
FEW_TILES_MAX_TOKENS = 1024
PAIR_MIN_TOKENS_GLU = 512  # gate/up pairs below this stay on single SMs: the pairs' 256-token tiles would leave a second, nearly empty wave


def _sm_count() -> int:
    global _SM_COUNT
    if _SM_COUNT is None:
        _SM_COUNT = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _SM_COUNT


STREAM_KERNEL_MAX_TOKENS = 8  # up to here the persistent weight-streaming kernel runs the product (9..16 rows measured slower there than in the tensor-memory kernel)


def _few_pair_tiles(tokens: int, n: int) -> bool:
    """Whether a plain bfloat16 product of this shape runs as token tiles of 64 in the kernel for
    few rows rather than as 256 x 256 tiles on SM pairs (the rule stands at FEW_PAIR_TILES)."""
    return (
        PROMPT_MIN_TOKENS <= tokens <= FEW_TILES_MAX_TOKENS
        and -(-tokens // 256) * -(-n // 256) <= FEW_PAIR_TILES and -(-tokens // 64) * -(-n // 128) <= 2 * _sm_count()
    )


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x[T, K] @ w[N, K]^T`` with float accumulation.

    bfloat16 x bfloat16 runs on the tensor cores (tcgen05, accumulators in TMEM); the true
    32-bit path and mixed types run the CUDA-core kernel, whose rows do not depend on the
    batch."""
    _check(x, "x", None, 2)
    _check(w, "w", None, 2)
    tokens, k = x.shape
    n, k2 = w.shape
    if k != k2:
        raise KernelError(f"x has rows of {k}, the matrix has rows of {k2}")
    if bias is not None:
        _check(bias, "bias", torch.float32, 1)
    out = torch.empty((tokens, n), dtype=out_dtype, device=x.device)
    lib = library()
    both_bf16 = x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    if both_bf16 and k % 8 == 0 and tokens <= STREAM_KERNEL_MAX_TOKENS:
        status = lib.shiso_gemm_stream(
            _ptr(x), _ptr(w), _ptr(bias), _ptr(out), _code(out), tokens, n, k, 0, _sm_count(), _stream()
        )
        _done(status, "linear (streaming)", shape=(tokens, n, k))
        return out
    if both_bf16 and _few_pair_tiles(tokens, n) and lib.shiso_gemm_tcgen05_supported(k, _ptr(x), _ptr(w)):
        status = lib.shiso_gemm_tcgen05_tokens64(
            _ptr(x), _ptr(w), _ptr(bias), _ptr(out), _code(out), tokens, n, k, _sm_count(), _stream()
        )
        _done(status, "linear (tcgen05, token tiles of 64)", shape=(tokens, n, k))
        return out
    if both_bf16 and tokens >= PROMPT_MIN_TOKENS and n % 8 == 0 and lib.shiso_gemm_tcgen05_supported(k, _ptr(x), _ptr(w)):
        status = lib.shiso_gemm_tcgen05_pair(
            _ptr(x), _ptr(w), _ptr(bias), _ptr(out), _code(out), tokens, n, k, 0, _sm_count(), _stream()
        )
        _done(status, "linear (tcgen05, persistent)", shape=(tokens, n, k))
        return out
    if both_bf16 and lib.shiso_gemm_tcgen05_supported(k, _ptr(x), _ptr(w)):
        status = lib.shiso_gemm_tcgen05(
            _ptr(x), _ptr(w), _ptr(bias), _ptr(out), _code(out), tokens, n, k, _sm_count(), _stream()
        )
        _done(status, "linear (tcgen05)", shape=(tokens, n, k))
        return out
    status = lib.shiso_gemm_simple(
        _ptr(x), _code(x), _ptr(w), _code(w), _ptr(bias), _ptr(out), _code(out), tokens, n, k, _stream()
    )
    _done(status, "linear", shape=(tokens, n, k))
    return out


def linear_swiglu(x: torch.Tensor, gate_up: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """``silu(x @ gate^T) * (x @ up^T)`` for ``gate_up = [gate; up]`` of shape ``[2I, K]``.
    In bfloat16 the activation is applied in the product's epilogue (the streaming kernel for a
    handful of rows, the tensor-memory kernel with two accumulators otherwise); other types
    run the product and then the activation kernel."""
    _check(x, "x", None, 2)
    _check(gate_up, "gate_up", None, 2)
    tokens, k = x.shape
    two_inter = gate_up.shape[0]
    if two_inter % 2 or gate_up.shape[1] != k:
        raise KernelError(f"gate/up matrix of shape {tuple(gate_up.shape)} does not fit rows of {k}")
    if (
        x.dtype == torch.bfloat16 and gate_up.dtype == torch.bfloat16 and out_dtype == torch.bfloat16
        and tokens <= STREAM_KERNEL_MAX_TOKENS and k % 8 == 0
    ):
        out = torch.empty((tokens, two_inter // 2), dtype=out_dtype, device=x.device)
        status = library().shiso_gemm_stream(
            _ptr(x), _ptr(gate_up), 0, _ptr(out), _code(out), tokens, two_inter, k, two_inter // 2,
            _sm_count(), _stream(),
        )
        _done(status, "linear_swiglu (streaming)", shape=(tokens, two_inter, k))
        return out
    lib = library()
    if (
        x.dtype == torch.bfloat16 and gate_up.dtype == torch.bfloat16
        and lib.shiso_gemm_tcgen05_supported(k, _ptr(x), _ptr(gate_up))
    ):
        out = torch.empty((tokens, two_inter // 2), dtype=out_dtype, device=x.device)
        if tokens >= PROMPT_MIN_TOKENS and (two_inter // 2) % 8 == 0:
            product = lib.shiso_gemm_tcgen05_pair if tokens >= PAIR_MIN_TOKENS_GLU else lib.shiso_gemm_tcgen05_prompt
            status = product(
                _ptr(x), _ptr(gate_up), 0, _ptr(out), _code(out), tokens, two_inter // 2, k, two_inter // 2,
                _sm_count(), _stream(),
            )
            _done(status, "linear_swiglu (tcgen05, persistent)", shape=(tokens, two_inter, k))
            return out
        status = lib.shiso_gemm_tcgen05_swiglu(
            _ptr(x), _ptr(gate_up), _ptr(out), _code(out), tokens, two_inter // 2, k, _stream()
        )
        _done(status, "linear_swiglu (tcgen05)", shape=(tokens, two_inter, k))
        return out
    return swiglu(linear(x, gate_up, out_dtype))


_GLU_ACTS = {"silu": 0, "gelu_tanh": 1, "swish_clamped": 2}


def glu_act(gate_up: torch.Tensor, act: str, limit: float = 0.0) -> torch.Tensor:
    """The gated pair over rows ``[gate | up]``: "silu" ``silu(g) u``; "gelu_tanh" ``gelu(g) u`` in
    its tanh form; "swish_clamped" ``g' sigmoid(1.702 g') (u' + 1)`` with ``g' = min(g, limit)`` and
    ``u' = clamp(u, -limit, limit)``.  Evaluated in float32."""
    _check(gate_up, "gate_up", None, 2)
    if act not in _GLU_ACTS:
        raise KernelError(f"gated pair {act!r}: expected one of {sorted(_GLU_ACTS)}")
    tokens, two_inter = gate_up.shape
    if two_inter % 2:
        raise KernelError(f"gate_up rows of {two_inter} cannot be split in two halves")
    out = torch.empty((tokens, two_inter // 2), dtype=gate_up.dtype, device=gate_up.device)
    status = library().shiso_glu_act(_ptr(gate_up), _ptr(out), _code(gate_up), tokens, two_inter // 2, _GLU_ACTS[act], float(limit), _stream())
    _done(status, f"glu_act ({act})", shape=(tokens, two_inter // 2))
    return out


def linear_glu(x: torch.Tensor, gate_up: torch.Tensor, out_dtype: torch.dtype, act: str, limit: float = 0.0) -> torch.Tensor:
    """``act(x @ gate^T, x @ up^T)`` for ``gate_up = [gate; up]`` (the pairs of ``glu_act``).  In
    bfloat16 the pair is applied in the product's epilogue, by the kernels and at the sizes of
    ``linear_swiglu`` (exponential and reciprocal from the special-function unit); other types run
    the product and then the activation kernel."""
    if act == "silu":
        return linear_swiglu(x, gate_up, out_dtype)
    if act not in _GLU_ACTS:
        raise KernelError(f"gated pair {act!r}: expected one of {sorted(_GLU_ACTS)}")
    _check(x, "x", None, 2)
    _check(gate_up, "gate_up", None, 2)
    tokens, k = x.shape
    two_inter = gate_up.shape[0]
    if two_inter % 2 or gate_up.shape[1] != k:
        raise KernelError(f"gate/up matrix of shape {tuple(gate_up.shape)} does not fit rows of {k}")
    inter, code = two_inter // 2, _GLU_ACTS[act]
    lib = library()
    if x.dtype == torch.bfloat16 and gate_up.dtype == torch.bfloat16 and out_dtype == torch.bfloat16:
        if tokens <= STREAM_KERNEL_MAX_TOKENS and k % 8 == 0:
            out = torch.empty((tokens, inter), dtype=out_dtype, device=x.device)
            status = lib.shiso_gemm_stream_glu(_ptr(x), _ptr(gate_up), _ptr(out), _code(out), tokens, inter, k, code, float(limit),
                                               _sm_count(), _stream())
            _done(status, f"linear_glu {act} (streaming)", shape=(tokens, two_inter, k))
            return out
        if lib.shiso_gemm_tcgen05_supported(k, _ptr(x), _ptr(gate_up)):
            out = torch.empty((tokens, inter), dtype=out_dtype, device=x.device)
            if tokens >= PROMPT_MIN_TOKENS and inter % 8 == 0:
                product = lib.shiso_gemm_tcgen05_pair_glu if tokens >= PAIR_MIN_TOKENS_GLU else lib.shiso_gemm_tcgen05_prompt_glu
                status = product(_ptr(x), _ptr(gate_up), _ptr(out), _code(out), tokens, inter, k, code, float(limit), _sm_count(), _stream())
                _done(status, f"linear_glu {act} (tcgen05, persistent)", shape=(tokens, two_inter, k))
                return out
            status = lib.shiso_gemm_tcgen05_glu(_ptr(x), _ptr(gate_up), _ptr(out), _code(out), tokens, inter, k, code, float(limit), _stream())
            _done(status, f"linear_glu {act} (tcgen05)", shape=(tokens, two_inter, k))
            return out
    return glu_act(linear(x, gate_up, out_dtype), act, limit)


STREAM_MAX_TOKENS = 8  # rows for which the weight-streaming kernel runs the product-into-stream / scaled-product pair
GLU_ONE_TILE_MAX_TOKENS = 64  # above one token tile the scaled gate/up pair runs as a plain product and the activation kernel: a gate/up CTA has an SM to itself, so two token tiles are 88 CTAs that each walk the whole K (20.9 us at 128 rows of the 1.2B shape against 17.8 us; decode at batch 96 / 128 +3.2 / +2.0 %)
FUSED_NORM_MAX_TOKENS = 192  # up to here (all the rows it takes) the tensor-memory kernel (tokens as the MMA's N operand) runs the pair: decode at batch 9 / 16 / 32 / 64 gained 11 / 10 / 4 / 1 % over product + norm kernel when the pair was built, batch 80 / 96 / 128 gain 4.2 / 4.2 / 3.6 % since a warp finishes whole tokens of the split products


class ScaledRows:
    """Rows that still lack their RMS scale: ``x`` is bfloat16 ``(residual * norm weight)`` and
    ``partials[c, t]`` are sums of squares of token ``t`` whose total over ``c`` gives the mean
    square.  ``linear_scaled`` applies the scale after its product."""

    def __init__(self, x, partials, eps):
        self.x, self.partials, self.eps = x, partials, float(eps)


def linear_into_stream(x, w, residual, next_norm_w, eps, bias=None):
    """A block's output projection, the residual add and the first half of the next RMS norm in
    one launch, for up to 192 bfloat16 rows and for the products of a few hundred rows that run
    as token tiles of 64 (``_few_pair_tiles``): returns ``(residual + x @ w^T, ScaledRows)`` -
    ``residual`` (float32 ``[T, N]``) itself is not changed - or None when sizes or types are
    not the ones the kernels take.  A handful of rows run in the weight-streaming kernel, more
    in the tensor-memory kernel whose threads own a feature each, so that a warp reads and
    writes neighbouring values of a token's row.  (The product into the stream in the
    tensor-memory kernels for long prompts was measured slower than product + row kernel:
    there a thread owns a row, and its strided reads and writes of the stream cost more than
    the row kernel they replace.  Applying the row scale is one factor a thread there, so those
    kernels do take the rows this one leaves: ``linear_scaled``.)"""
    tokens, k = x.shape
    n = w.shape[0]
    if (
        x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or residual.dtype != torch.float32
        or k % 8 or w.shape[1] != k or n % 8
        or (tokens > FUSED_NORM_MAX_TOKENS and not _few_pair_tiles(tokens, n))
    ):
        return None
    lib = library()
    streaming = tokens <= min(STREAM_MAX_TOKENS, STREAM_KERNEL_MAX_TOKENS)
    if not streaming and not lib.shiso_gemm_tcgen05_supported(k, _ptr(x), _ptr(w)):
        return None
    _check(x, "x", torch.bfloat16, 2)
    _check(w, "w", torch.bfloat16, 2)
    _check(residual, "residual", torch.float32, 2)
    _check(next_norm_w, "norm weight", torch.float32, 1)
    if residual.shape != (tokens, n) or next_norm_w.shape[0] != n:
        raise KernelError(f"a residual of shape {tuple(residual.shape)} beside a product of {tokens} x {n}")
    if bias is not None:
        _check(bias, "bias", torch.float32, 1)
    summed = torch.empty_like(residual)
    rows = torch.empty((tokens, n), dtype=torch.bfloat16, device=x.device)
    if streaming:
        partials = torch.empty((-(-n // 16), 16), dtype=torch.float32, device=x.device)
        status = lib.shiso_gemm_stream_into(
            _ptr(x), _ptr(w), _ptr(bias), _ptr(residual), _ptr(summed), _ptr(next_norm_w), _ptr(rows), _ptr(partials),
            tokens, n, k, _sm_count(), _stream(),
        )
    else:
        partials = torch.empty((lib.shiso_gemm_tcgen05_into_partial_rows(n), tokens), dtype=torch.float32, device=x.device)
        status = lib.shiso_gemm_tcgen05_into(
            _ptr(x), _ptr(w), _ptr(bias), _ptr(residual), _ptr(summed), _ptr(next_norm_w), _ptr(rows), _ptr(partials),
            tokens, n, k, _sm_count(), _stream(),
        )
    _done(status, "linear_into_stream" + (" (streaming)" if streaming else " (tcgen05)"), shape=(tokens, n, k))
    return summed, ScaledRows(rows, partials, eps)


def linear_scaled(rows: ScaledRows, w, out_dtype, glu=False):
    """``rmsnorm(..) @ w^T`` (SwiGLU over the gate/up pair ``w`` when ``glu``) for rows that
    ``linear_into_stream`` left: the row scale is applied to the accumulators."""
    x = rows.x
    _check(x, "x", torch.bfloat16, 2)
    _check(w, "w", torch.bfloat16, 2)
    tokens, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k or (glu and n % 2):
        raise KernelError(f"a matrix of shape {tuple(w.shape)} for rows of {k}")
    if tokens > FUSED_NORM_MAX_TOKENS:
        return _linear_scaled_long(rows, w, out_dtype, glu)
    if glu and tokens > GLU_ONE_TILE_MAX_TOKENS and out_dtype == torch.bfloat16 and (n // 2) % 8 == 0:
        return swiglu(linear_scaled(rows, w, out_dtype, False))
    inter = n // 2 if glu else 0
    out = torch.empty((tokens, inter if glu else n), dtype=out_dtype, device=x.device)
    lib = library()
    if tokens <= min(STREAM_MAX_TOKENS, STREAM_KERNEL_MAX_TOKENS):
        status = lib.shiso_gemm_stream_scaled(
            _ptr(x), _ptr(rows.partials), rows.partials.shape[0], rows.eps, _ptr(w), _ptr(out), _code(out),
            tokens, n, k, inter, _sm_count(), _stream(),
        )
    else:
        status = lib.shiso_gemm_tcgen05_scaled(
            _ptr(x), _ptr(rows.partials), rows.partials.shape[0], rows.partials.shape[1], rows.eps, _ptr(w), _ptr(out),
            _code(out), tokens, n, k, inter, _sm_count(), _stream(),
        )
    _done(status, "linear_scaled", shape=(tokens, n, k))
    return out


def _linear_scaled_long(rows: ScaledRows, w, out_dtype, glu):
    """``linear_scaled`` for more than 192 rows: the kernel ``linear`` / ``linear_swiglu`` would
    take for the shape, with the row scale in its epilogue."""
    x = rows.x
    tokens, k = x.shape
    n = w.shape[0]
    lib = library()
    partials = rows.partials
    if n % 8 or k % 8 or (glu and (n // 2) % 8):
        # widths the prompt kernels do not take: the kernel for up to 192 rows takes any, a
        # slice of the rows at a time (the partial sums' columns are the tokens)
        out = torch.empty((tokens, n // 2 if glu else n), dtype=out_dtype, device=x.device)
        stride = partials.shape[1]
        for first in range(0, tokens, FUSED_NORM_MAX_TOKENS):
            count = min(FUSED_NORM_MAX_TOKENS, tokens - first)
            status = lib.shiso_gemm_tcgen05_scaled(
                _ptr(x[first : first + count]), partials.data_ptr() + 4 * first, partials.shape[0], stride, rows.eps, _ptr(w),
                _ptr(out[first : first + count]), _code(out), count, n, k, n // 2 if glu else 0, _sm_count(), _stream(),
            )
            _done(status, "linear_scaled (a slice of the rows)", shape=(count, n, k))
        return out
    if glu:
        inter = n // 2
        out = torch.empty((tokens, inter), dtype=out_dtype, device=x.device)
        product = lib.shiso_gemm_tcgen05_pair_scaled if tokens >= PAIR_MIN_TOKENS_GLU else lib.shiso_gemm_tcgen05_prompt_scaled
        status = product(_ptr(x), _ptr(partials), partials.shape[0], partials.shape[1], rows.eps, _ptr(w), _ptr(out), _code(out),
                         tokens, inter, k, inter, _sm_count(), _stream())
        _done(status, "linear_scaled + swiglu (tcgen05, persistent)", shape=(tokens, n, k))
        return out
    out = torch.empty((tokens, n), dtype=out_dtype, device=x.device)
    if _few_pair_tiles(tokens, n) and lib.shiso_gemm_tcgen05_supported(k, _ptr(x), _ptr(w)):
        status = lib.shiso_gemm_tcgen05_scaled(
            _ptr(x), _ptr(partials), partials.shape[0], partials.shape[1], rows.eps, _ptr(w), _ptr(out), _code(out),
            tokens, n, k, 0, _sm_count(), _stream(),
        )
        _done(status, "linear_scaled (tcgen05, token tiles of 64)", shape=(tokens, n, k))
        return out
    status = lib.shiso_gemm_tcgen05_pair_scaled(
        _ptr(x), _ptr(partials), partials.shape[0], partials.shape[1], rows.eps, _ptr(w), _ptr(out), _code(out),
        tokens, n, k, 0, _sm_count(), _stream(),
    )
    _done(status, "linear_scaled (tcgen05, persistent)", shape=(tokens, n, k))
    return out


def linear_add_rmsnorm(x, w, residual, norm_w, eps, out_dtype):
    """A block's output projection, the residual add and the next RMS norm:
    ``residual += x @ w^T`` (float32, in place) and returns ``rmsnorm(residual) * norm_w``.
    Two launches: the product, then the fused add + norm row kernel.  (One launch, with the
    CTA that finishes last normalising, was measured at 10.5 us against 6.1 us for the pair
    in a dependent-launch chain and was dropped.)"""
    return add_rmsnorm(residual, linear(x, w, out_dtype), norm_w, eps, out_dtype)


CONV_FUSED_MAX_TAPS = 4  # taps the weight-streaming kernel's convolution epilogue takes


def linear_short_conv(x, in_proj, taps, bias, state, step):
    """The short conv's input projection followed by the gated convolution; ``x`` is a tensor or
    ``ScaledRows``.  For a handful of bfloat16 rows, one per sequence, the convolution runs in
    the product's epilogue (a tile of the weight-streaming kernel is then the B, C and x rows of
    five channels); else the product and the convolution kernel run one after the other."""
    rows = x if isinstance(x, ScaledRows) else None
    xt = rows.x if rows is not None else x
    tokens, k = xt.shape
    hidden, n_taps = taps.shape
    if (
        xt.dtype == torch.bfloat16 and in_proj.dtype == torch.bfloat16 and tokens <= STREAM_KERNEL_MAX_TOKENS
        and getattr(step, "all_decode", False) and 2 <= n_taps <= CONV_FUSED_MAX_TAPS and k % 8 == 0
    ):
        _check(xt, "x", torch.bfloat16, 2)
        _check(in_proj, "in_proj", torch.bfloat16, 2)
        _check(taps, "conv taps", torch.float32, 2)
        if in_proj.shape != (3 * hidden, k):
            raise KernelError(f"an input projection of shape {tuple(in_proj.shape)} for {hidden} channels of rows of {k}")
        if state.dtype != torch.float32 or not state.is_cuda or state.dim() != 3:
            raise KernelError("conv state: expected a float32 CUDA tensor [slots, taps-1, hidden]")
        if state.shape[1:] != (n_taps - 1, hidden) or state.stride(2) != 1 or state.stride(1) != hidden:
            raise KernelError(f"conv state of shape {tuple(state.shape)} / strides {state.stride()} does not fit {n_taps} taps x {hidden}")
        if bias is not None:
            _check(bias, "conv bias", torch.float32, 1)
        y = torch.empty((tokens, hidden), dtype=xt.dtype, device=xt.device)
        status = library().shiso_gemm_stream_conv(
            _ptr(xt), _ptr(rows.partials) if rows is not None else 0, rows.partials.shape[0] if rows is not None else 0,
            rows.eps if rows is not None else 0.0, _ptr(in_proj), _ptr(taps), _ptr(bias), state.data_ptr(), state.stride(0),
            _ptr(step.seq_of_token), _ptr(step.state_slots), _ptr(y), _code(y), tokens, hidden, k, n_taps,
            _sm_count(), _stream(),
        )
        _done(status, "linear_short_conv (streaming)", shape=(tokens, 3 * hidden, k))
        return y
    proj = linear_scaled(rows, in_proj, xt.dtype) if rows is not None else linear(xt, in_proj, xt.dtype)
    return short_conv(proj, taps, bias, state, step)


def linear_simple(x, w, out_dtype, bias=None):
    """The CUDA-core product for any element types (used by tests to compare kernels)."""
    _check(x, "x", None, 2)
    _check(w, "w", None, 2)
    out = torch.empty((x.shape[0], w.shape[0]), dtype=out_dtype, device=x.device)
    status = library().shiso_gemm_simple(
        _ptr(x), _code(x), _ptr(w), _code(w), _ptr(bias), _ptr(out), _code(out), x.shape[0], w.shape[0], x.shape[1], _stream()
    )
    _done(status, "linear")
    return out


CARRIES_STATUS = True  # argmax and sample take ``status_out``
GAVE_UP = "a kernel gave up waiting on a barrier; what it wrote is not valid"


def check_kernel_status() -> None:
    """Raises when a bounded wait inside a kernel ran out since the status word was last read
    (here, or by a token-picking kernel that was given a place for it).  Synchronises the
    device; not for use while a stream is being captured."""
    status = library().shiso_gemm_tcgen05_status()
    if status != 0:
        raise KernelError(f"{GAVE_UP} (status {status})")


def selftest_bounded_wait(limit_cycles: int = 4000) -> None:
    """Launches one CTA that waits ``limit_cycles`` clock cycles on a barrier nobody arrives at
    and then gives up, as any kernel here does when a wait runs out: the status word is set and
    the kernel returns.  For tests of what the host does then."""
    _done(library().shiso_selftest_bounded_wait(int(limit_cycles), _stream()), "selftest_bounded_wait")


# --------------------------------------------------------------------------- short convolution


def short_conv(proj, taps, bias, state, step):
    """``proj[T, 3H]`` -> ``y[T, H]``; ``state`` is the float32 view ``[slots, taps-1, H]`` of
    the slot buffer (rows of one slot contiguous) and is updated for the step's sequences."""
    _check(proj, "proj", None, 2)
    _check(taps, "conv taps", torch.float32, 2)
    tokens, h3 = proj.shape
    hidden, n_taps = taps.shape
    if h3 != 3 * hidden:
        raise KernelError(f"proj rows of {h3} are not 3 x {hidden}")
    if state.dtype != torch.float32 or not state.is_cuda or state.dim() != 3:
        raise KernelError("conv state: expected a float32 CUDA tensor [slots, taps-1, hidden]")
    if state.shape[1:] != (n_taps - 1, hidden) or state.stride(2) != 1 or state.stride(1) != hidden:
        raise KernelError(f"conv state of shape {tuple(state.shape)} / strides {state.stride()} does not fit {n_taps} taps x {hidden}")
    if bias is not None:
        _check(bias, "conv bias", torch.float32, 1)
    y = torch.empty((tokens, hidden), dtype=proj.dtype, device=proj.device)
    status = library().shiso_short_conv(
        _ptr(proj), _code(proj), _ptr(taps), _ptr(bias), state.data_ptr(), state.stride(0),
        _ptr(step.seq_of_token), _ptr(step.q_start), _ptr(step.state_slots), _ptr(y),
        tokens, step.num_seqs, hidden, n_taps, 1, int(getattr(step, "max_q_len", 0)), _stream(),
    )
    _done(status, "short_conv", 2, shape=(tokens, hidden))
    return y


# --------------------------------------------------------------------------- attention


def qk_norm_rope_store(qkv, heads, kv_heads, head_dim, q_w, k_w, eps, inv_freq, rotary_dim, step,
                       k_cache, v_cache, block_table, page_size, store, interleaved=False):
    """Per-head norm, rotation and cache store.  The rotation pairs are ``(i, i + rotary_dim/2)``,
    or neighbours ``(2i, 2i + 1)`` with ``interleaved``."""
    _check(qkv, "qkv", None, 2)
    tokens, width = qkv.shape
    if width != (heads + 2 * kv_heads) * head_dim:
        raise KernelError(f"qkv rows of {width} are not ({heads} + 2 x {kv_heads}) x {head_dim}")
    for name, t in (("q norm weight", q_w), ("k norm weight", k_w)):
        if t is not None:
            _check(t, name, torch.float32, 1)
            if t.shape[0] != head_dim:
                raise KernelError(f"{name} has {t.shape[0]} entries for heads of {head_dim}")
    if rotary_dim:
        _check(inv_freq, "inv_freq", torch.float32, 1)
        if inv_freq.shape[0] != rotary_dim // 2:
            raise KernelError(f"inv_freq has {inv_freq.shape[0]} entries for a rotation over {rotary_dim}")
    _check(block_table, "block table", torch.int32, 2)
    do_store = bool(store) and kv_heads > 0
    if do_store:
        for name, t in (("k cache", k_cache), ("v cache", v_cache)):
            _check(t, name, qkv.dtype, 4)
            if t.shape[1:] != (page_size, kv_heads, head_dim):
                raise KernelError(f"{name} of shape {tuple(t.shape)} does not fit pages of {page_size} x {kv_heads} x {head_dim}")
    q = torch.empty((tokens, heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    status = library().shiso_qk_norm_rope_store(
        _ptr(qkv), _code(qkv), _ptr(q_w), _ptr(k_w), _ptr(inv_freq) if rotary_dim else 0,
        _ptr(step.positions), _ptr(step.seq_of_token), _ptr(block_table), block_table.shape[1],
        _ptr(k_cache) if do_store else 0, _ptr(v_cache) if do_store else 0, _ptr(q),
        tokens, heads, kv_heads, head_dim, int(rotary_dim), page_size, float(eps), int(do_store), int(bool(interleaved)),
        _stream(),
    )
    _done(status, "qk_norm_rope_store", shape=(tokens, heads + 2 * kv_heads, head_dim))
    return q


MAX_DECODE_GROUP = 16  # query heads per KV head the decode kernel serves from one read (rows of one MMA tile)
DECODE_HEAD_DIMS = tuple(range(16, 129, 16))  # larger head sizes take the general kernel
PREFILL_MAX_HEAD_DIM = 128  # the tiled prompt kernel keeps a row's output in registers
TC_ATTENTION_MIN_TOKENS = 256  # steps from here on, with a portion of at least ...
TC_ATTENTION_MIN_PORTION = 128  # ... this many rows, take the tensor-memory attention kernel (head size 64)


_WIDE_CLUSTERS = None


def _wide_clusters() -> bool:
    """Whether the fused decode kernel may be launched as clusters of 16 CTAs on this device."""
    global _WIDE_CLUSTERS
    if _WIDE_CLUSTERS is None:
        _WIDE_CLUSTERS = int(library().shiso_decode_attention_fused_max_parts()) >= 16
    return _WIDE_CLUSTERS


def decode_splits(tokens: int, kv_heads: int, capacity: int, fused: bool = False) -> int:
    """Into how many parts a decode kernel cuts a sequence's keys.  It depends on the launch
    shape only, never on current lengths, so a captured step stays valid.  The two-launch
    kernel wants enough CTAs (tokens x KV heads x parts) to fill the SMs a few times over, no
    part shorter than 128 keys of the table's capacity.  The fused kernel streams a long part
    at full rate through its ring, and every CTA costs it a start and a hand-over at the end:
    it wants one wave of the two CTAs an SM holds (measured when three fitted: batch 8 x 8 KV
    heads x 2,190 keys took 14.8 us in 4 parts, 16.5 in 6, 21 in 10; batch 32 30 us whole, 43 in 2)."""
    if fused:
        # the parts of a (sequence, KV head) are a thread-block cluster: at most 8, or 16 where the
        # device places such clusters and one or two sequences leave room for them (a part of two
        # tiles instead of four: batch 1 x 2,158 keys)
        room = 2 * _sm_count() // (tokens * kv_heads)
        most = 16 if room >= 16 and _wide_clusters() else 8
        return max(1, min(most, room, -(-capacity // 128)))
    return max(1, min(16, -(-4 * _sm_count() // (tokens * kv_heads)), -(-capacity // 128)))


DECODE_FROM_QKV_MAX_TOKENS = 64  # rows up to which attention takes the qkv rows itself: one launch fewer per layer, and the keys and values move before the predecessor ends (batch 8 / 16 / 32 / 64 decode 1 / 1.8 / 2.0 / 1.0 % faster; no change at 96 and 128 rows)


def decode_attention_from_qkv(qkv, heads, kv_heads, head_dim, q_w, k_w, eps, inv_freq, rotary_dim, step,
                              k_cache, v_cache, block_table, page_size, store, scale, window, interleaved=False, keep_first=0):
    """``qk_norm_rope_store`` and ``paged_attention`` in one launch for steps of single tokens:
    the attention kernel takes the rows of the qkv product, norms and rotates the queries and
    each token's new key itself, and (with ``store``) writes the new key and value into the
    caches, with the bits ``qk_norm_rope_store`` would write.  bfloat16, heads of 64 rotated
    whole, both norms present, a handful of rows; None when the step or the sizes are others (the
    caller then runs the two kernels).  With a ``window``, the first ``keep_first`` positions of a
    sequence stay visible."""
    lib = library()
    if (
        qkv.shape[0] > DECODE_FROM_QKV_MAX_TOKENS or qkv.dtype != torch.bfloat16 or not getattr(step, "all_decode", False) or q_w is None or k_w is None
        or interleaved
        or inv_freq is None or head_dim != 64 or rotary_dim != 64 or kv_heads <= 0
        or not lib.shiso_decode_attention_fused_supported(heads, kv_heads, head_dim, page_size)
    ):
        return None
    _check(qkv, "qkv", torch.bfloat16, 2)
    tokens, width = qkv.shape
    if width != (heads + 2 * kv_heads) * head_dim:
        raise KernelError(f"qkv rows of {width} are not ({heads} + 2 x {kv_heads}) x {head_dim}")
    for name, t in (("k cache", k_cache), ("v cache", v_cache)):
        _check(t, name, torch.bfloat16, 4)
        if t.shape[1:] != (page_size, kv_heads, head_dim):
            raise KernelError(f"{name} of shape {tuple(t.shape)} does not fit pages of {page_size} x {kv_heads} x {head_dim}")
    _check(block_table, "block table", torch.int32, 2)
    _check(q_w, "q norm weight", torch.float32, 1)
    _check(k_w, "k norm weight", torch.float32, 1)
    _check(inv_freq, "inv_freq", torch.float32, 1)
    if q_w.shape[0] != head_dim or k_w.shape[0] != head_dim or inv_freq.shape[0] != rotary_dim // 2:
        raise KernelError("norm weights of the head size and one frequency per rotated pair are expected")
    out = torch.empty((tokens, heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    if keep_first and window:
        # the keys a row reads are bounded by the window, whatever the table could hold
        splits = decode_splits(tokens, kv_heads, min(block_table.shape[1] * page_size, int(window) + int(keep_first) + 128), True)
        status = lib.shiso_decode_attention_from_qkv_kept(
            _ptr(qkv), _ptr(q_w), _ptr(k_w), _ptr(inv_freq), float(eps), _ptr(k_cache), _ptr(v_cache), _ptr(block_table),
            block_table.shape[1], _ptr(step.positions), _ptr(step.seq_of_token), _ptr(out),
            tokens, heads, kv_heads, head_dim, page_size, k_cache.shape[0], float(scale), int(window), int(keep_first), splits,
            int(bool(store)), _stream(),
        )
        _done(status, "decode_attention_from_qkv (kept first)", shape=(tokens, heads, head_dim))
        return out
    splits = decode_splits(tokens, kv_heads, block_table.shape[1] * page_size, True)
    status = lib.shiso_decode_attention_from_qkv(
        _ptr(qkv), _ptr(q_w), _ptr(k_w), _ptr(inv_freq), float(eps), _ptr(k_cache), _ptr(v_cache), _ptr(block_table),
        block_table.shape[1], _ptr(step.positions), _ptr(step.seq_of_token), _ptr(out),
        tokens, heads, kv_heads, head_dim, page_size, k_cache.shape[0], float(scale), int(window), splits, int(bool(store)),
        _stream(),
    )
    _done(status, "decode_attention_from_qkv", shape=(tokens, heads, head_dim))
    return out


def paged_attention(q, heads, kv_heads, head_dim, k_cache, v_cache, block_table, page_size, scale, window, step,
                    general=False):
    """Attention of every row over its sequence's cache.  Steps of single tokens in bfloat16
    take the split-key decode kernel (keys and values read once per KV head); other bfloat16
    steps take the tiled tensor-core kernel; float32 and head sizes above 128 take the general
    kernel.  ``general=True`` forces the general kernel (tests compare the routes)."""
    _check(q, "q", None, 2)
    tokens = q.shape[0]
    if q.shape[1] != heads * head_dim:
        raise KernelError(f"q rows of {q.shape[1]} are not {heads} x {head_dim}")
    for name, t in (("k cache", k_cache), ("v cache", v_cache)):
        _check(t, name, q.dtype, 4)
        if t.shape[1:] != (page_size, kv_heads, head_dim):
            raise KernelError(f"{name} of shape {tuple(t.shape)} does not fit pages of {page_size} x {kv_heads} x {head_dim}")
    _check(block_table, "block table", torch.int32, 2)
    out = torch.empty_like(q)
    lib = library()
    if general:
        pass
    elif (
        q.dtype == torch.bfloat16 and getattr(step, "all_decode", False)
        and heads // kv_heads <= MAX_DECODE_GROUP and head_dim in DECODE_HEAD_DIMS
    ):
        fused = bool(lib.shiso_decode_attention_fused_supported(heads, kv_heads, head_dim, page_size))
        splits = decode_splits(tokens, kv_heads, block_table.shape[1] * page_size, fused)
        if fused:
            # keys and values by TMA, the parts merged through their cluster's shared memory: one launch
            status = lib.shiso_decode_attention_fused(
                _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1], _ptr(step.positions),
                _ptr(step.seq_of_token), _ptr(out), tokens, heads, kv_heads, head_dim,
                page_size, k_cache.shape[0], float(scale), int(window), splits, _stream(),
            )
            _done(status, "decode_attention (fused)", shape=(tokens, heads, head_dim))
            return out
        scratch = torch.empty((tokens * heads * splits * (head_dim + 2),), dtype=torch.float32, device=q.device)
        status = lib.shiso_decode_attention(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1], _ptr(step.positions),
            _ptr(step.seq_of_token), _ptr(scratch), _ptr(out), tokens, heads, kv_heads, head_dim, page_size,
            float(scale), int(window), splits, _stream(),
        )
        _done(status, "decode_attention", 2, shape=(tokens, heads, head_dim))
        return out
    elif (
        q.dtype == torch.bfloat16 and tokens >= TC_ATTENTION_MIN_TOKENS
        and getattr(step, "max_q_len", tokens) >= TC_ATTENTION_MIN_PORTION
        and lib.shiso_prefill_attention_tc_supported(head_dim, page_size)
    ):
        # long portions: products in tensor memory, 128 query rows per CTA
        starts = getattr(step, "h_q_start", None)
        if starts:
            tiles = sum(-(-(b - a) // 128) for a, b in zip(starts[:-1], starts[1:]))
        else:
            tiles = tokens // 128 + step.num_seqs
        status = lib.shiso_prefill_attention_tc(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1], _ptr(step.q_start),
            _ptr(step.start_pos), _ptr(out), tokens, step.num_seqs, tiles, heads, kv_heads, page_size,
            k_cache.shape[0], float(scale), int(window), _stream(),
        )
        _done(status, "prefill_attention (tcgen05)", shape=(tokens, heads, head_dim))
        return out
    elif q.dtype == torch.bfloat16 and head_dim % 16 == 0 and head_dim <= PREFILL_MAX_HEAD_DIM:
        starts = getattr(step, "h_q_start", None)
        if starts:
            tiles = sum(-(-(b - a) // 64) for a, b in zip(starts[:-1], starts[1:]))
        else:
            tiles = tokens // 64 + step.num_seqs
        status = lib.shiso_prefill_attention(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1], _ptr(step.q_start),
            _ptr(step.start_pos), _ptr(out), step.num_seqs, tiles, heads, kv_heads, head_dim, page_size,
            float(scale), int(window), _stream(),
        )
        _done(status, "prefill_attention", shape=(tokens, heads, head_dim))
        return out
    status = lib.shiso_paged_attention(
        _ptr(q), _code(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1],
        _ptr(step.positions), _ptr(step.seq_of_token), _ptr(out), tokens, heads, kv_heads, head_dim,
        page_size, float(scale), int(window), _stream(),
    )
    _done(status, "paged_attention", shape=(tokens, heads, head_dim))
    return out


# --------------------------------------------------------------------------- hashed-pair embedding, copies of the stream


def _slot_rows(state: torch.Tensor, name: str, dtype) -> int:
    """The distance, in elements, between two slots of a per-request state view whose rows are
    contiguous inside a slot."""
    if not state.is_cuda or state.dtype != dtype:
        raise KernelError(f"{name}: expected a {dtype} CUDA tensor, got {state.dtype} on {state.device}")
    inner = 1
    for size, stride in zip(reversed(state.shape[1:]), reversed(state.stride()[1:])):
        if size != 1 and stride != inner:
            raise KernelError(f"{name}: a slot's values must be contiguous, strides are {state.stride()}")
        inner *= size
    return state.stride(0)


def embed_hashed_pair(ids, table, pair_table, scale, buckets, mul_prev, mul_cur, step, state, feed_index=None, fed_tokens=None):
    """``scale * table[id] + pair_table[(previous id * mul_prev + id * mul_cur) mod buckets]``, row
    ``buckets`` of the pair table for a sequence's first token; float32 rows.  ``state`` (int32
    ``[slots, 1]``) holds each request's last token + 1 and is brought up to date."""
    _check(ids, "ids", torch.int32, 1)
    _check(table, "embedding table", None, 2)
    _check(pair_table, "pair table", table.dtype, 2)
    tokens, (vocab, hidden) = ids.shape[0], table.shape
    if pair_table.shape != (buckets + 1, hidden):
        raise KernelError(f"a pair table of shape {tuple(pair_table.shape)} for {buckets} buckets and rows of {hidden}")
    if (feed_index is None) != (fed_tokens is None):
        raise KernelError("embed: feed_index and fed_tokens come together")
    stride = _slot_rows(state, "token state", torch.int32)
    out = torch.empty((tokens, hidden), dtype=torch.float32, device=table.device)
    status = library().shiso_embed_hashed_pair(
        _ptr(ids), _ptr(feed_index), _ptr(fed_tokens), _ptr(table), _ptr(pair_table), _code(table), _ptr(step.seq_of_token),
        _ptr(step.q_start), _ptr(step.start_pos), _ptr(step.state_slots), state.data_ptr(), stride, _ptr(out),
        tokens, step.num_seqs, hidden, vocab, float(scale), int(buckets), int(mul_prev), int(mul_cur), _stream(),
    )
    _done(status, "embed_hashed_pair", 2, shape=(tokens, hidden))
    return out


def _hyper_mix(source, y, mix, write, copies, read, weight, eps, out_dtype, want_sum):
    single = source.dim() == 2
    _check(source, "stream", torch.float32, 2 if single else 3)
    tokens, hidden = source.shape[-2:]
    if not single and source.shape[0] != copies:
        raise KernelError(f"{source.shape[0]} copies of the stream where {copies} are expected")
    lanes = None
    if y is not None:
        _check(y, "sublayer output", None, 2)
        _check(mix, "mixing matrix", torch.float32, 2)
        _check(write, "write vector", torch.float32, 1)
        if y.shape != (tokens, hidden) or mix.shape != (copies, copies) or write.shape[0] != copies:
            raise KernelError("a sublayer output, mixing matrix or write vector of the wrong shape")
        if not want_sum:
            lanes = source if not single else torch.empty((copies, tokens, hidden), dtype=torch.float32, device=source.device)
    normed = summed = None
    act = out_dtype
    if read is not None:
        _check(read, "read vector", torch.float32, 1)
        _check(weight, "norm weight", torch.float32, 1)
        if read.shape[0] != copies or weight.shape[0] != hidden:
            raise KernelError("a read vector or norm weight of the wrong shape")
        normed = torch.empty((tokens, hidden), dtype=out_dtype, device=source.device)
    if want_sum:
        summed = torch.empty((tokens, hidden), dtype=torch.float32, device=source.device)
    if y is not None:
        if act is None:
            act = y.dtype
        elif y.dtype != act:
            raise KernelError(f"a sublayer output of {y.dtype} beside normed rows of {act}")
    status = library().shiso_hyper_mix(
        _ptr(source), 0 if single else tokens * hidden, _ptr(y), _ptr(mix) if y is not None else 0,
        _ptr(write) if y is not None else 0, _ptr(lanes), tokens * hidden, _ptr(read), _ptr(weight) if read is not None else 0,
        float(eps), _ptr(normed), _ptr(summed), _CODES[act if act is not None else torch.float32], tokens, hidden, copies, _stream(),
    )
    _done(status, "hyper_mix", shape=(copies, tokens, hidden))
    return lanes, normed, summed


def hyper_mix_read(source, y, mix, write, copies, read, weight, eps, out_dtype):
    """Copies of the residual stream: writes a sublayer's output into them and reads them for the
    next sublayer, in one launch.  ``source`` is float32 ``[copies, T, H]``, or ``[T, H]`` standing
    for every copy.  With ``y``: ``x_r' = sum_s mix[s, r] x_s + write[r] * y`` (in place, or into a
    new buffer when ``source`` was a single stream).  Returns ``(the copies written or None, rows)``
    with ``rows = rmsnorm(sum_r read[r] x_r') * weight`` in ``out_dtype``."""
    lanes, normed, _ = _hyper_mix(source, y, mix, write, copies, read, weight, eps, out_dtype, False)
    return lanes, normed


def hyper_mix_sum(source, y, mix, write):
    """The sum of the copies after a last write (``y`` may be None): float32 ``[T, H]``."""
    copies = source.shape[0] if source.dim() == 3 else mix.shape[0]
    return _hyper_mix(source, y, mix, write, copies, None, None, 0.0, None, True)[2]


# --------------------------------------------------------------------------- time mixing, recurrences


def token_shift_blend(x, mu, state, step):
    """``out[c] = x_t + (x_{t-1} - x_t) * mu[c]`` for every row of ``mu``; ``x_{t-1}`` is the row
    before in the same sequence, the request's kept row (``state``, float32 ``[slots, H]``) for a
    portion's first token, zeros at position 0.  The kept rows are brought up to date."""
    _check(x, "x", None, 2)
    _check(mu, "blend weights", torch.float32, 2)
    tokens, hidden = x.shape
    if mu.shape[1] != hidden or state.shape[1:] != (hidden,):
        raise KernelError(f"blend weights {tuple(mu.shape)} or kept rows {tuple(state.shape)} do not fit rows of {hidden}")
    stride = _slot_rows(state, "kept rows", torch.float32)
    out = torch.empty((mu.shape[0], tokens, hidden), dtype=x.dtype, device=x.device)
    status = library().shiso_token_shift_blend(
        _ptr(x), _code(x), _ptr(mu), state.data_ptr(), stride, _ptr(step.seq_of_token), _ptr(step.q_start), _ptr(step.start_pos),
        _ptr(step.state_slots), _ptr(out), tokens, step.num_seqs, hidden, mu.shape[0], _stream(),
    )
    _done(status, "token_shift_blend", 2, shape=(mu.shape[0], tokens, hidden))
    return out


_UNARY = {"tanh": 0, "silu": 1, "relu2": 2, "copy": 3}  # copy: the values in another element type


def unary(x, kind, out_dtype):
    _check(x, "x", None, None)
    out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    _done(library().shiso_unary(_ptr(x), _code(x), _ptr(out), _code(out), x.numel(), _UNARY[kind], _stream()), f"unary ({kind})",
          shape=tuple(x.shape))
    return out


def _rows(t, name, dtype, width=None) -> int:
    """The row stride of a 2-D tensor whose rows are contiguous (a column range of a wider one)."""
    if not t.is_cuda or t.dim() != 2 or t.stride(1) != 1 or (dtype is not None and t.dtype != dtype):
        raise KernelError(f"{name}: expected 2-D CUDA rows of {dtype} with unit column stride, got {t.dtype} {tuple(t.shape)} {t.stride()}")
    if width is not None and t.shape[1] != width:
        raise KernelError(f"{name}: rows of {t.shape[1]} where {width} are expected")
    return t.stride(0)


RECURRENCE_SPLIT_MIN_PORTION = 64  # portions from here on may share a head's value columns out over several CTAs


def recurrence_supported(dim: int, vdim: int) -> bool:
    return bool(library().shiso_decay_recurrence_supported(int(dim), int(vdim)))


def decay_recurrence(q, k, v, out, state, step, heads, dim, vdim, eps, *, decay_logits=None, decay_bias=None, bonus=None,
                     head_decay=None, head_loss=None, inv_freq=None, rotary_dim=0, key_scale=1.0, out_weight=None, gate=None,
                     out_scale=1.0):
    """A matrix state ``S[dim, vdim]`` per head (``state``, float32 ``[slots, heads, dim, vdim]``),
    walked over each sequence's rows in order.  With ``decay_logits`` (float32 ``[T, heads * dim]``),
    ``decay_bias`` and ``bonus``: ``w = exp(-exp(logits + bias))``, ``o = (S + diag(bonus) k v^T)^T q``,
    then ``S = diag(w) S + k v^T``.  With ``head_decay`` (float32 ``[heads]``; ``head_loss`` = 1 - decay, formed in higher
    precision, is what the kernel multiplies by - when it is not given it is formed here): q and k rotated by the
    position (half-split pairs over ``rotary_dim``), k times ``key_scale``, ``S = decay S + k v^T``,
    then ``o = S^T q``.  ``o`` is brought to unit RMS per head, times ``out_weight``, times
    ``silu(gate)``, times ``out_scale``, into ``out``.  q, k, v, gate and out may be column ranges."""
    act = q.dtype
    tokens = q.shape[0]
    q_ld, k_ld = _rows(q, "q", act, heads * dim), _rows(k, "k", act, heads * dim)
    v_ld, out_ld = _rows(v, "v", act, heads * vdim), _rows(out, "out", act, heads * vdim)
    gate_ld = _rows(gate, "gate", act, heads * vdim) if gate is not None else 0
    if state.shape[1:] != (heads, dim, vdim):
        raise KernelError(f"a state of shape {tuple(state.shape)} for {heads} heads of {dim} x {vdim}")
    stride = _slot_rows(state, "recurrent state", torch.float32)
    logits_ld = 0
    if decay_logits is not None:
        logits_ld = _rows(decay_logits, "decay logits", torch.float32, heads * dim)
        _check(decay_bias, "decay bias", torch.float32, 1)
        _check(bonus, "bonus", torch.float32, 2)
        if decay_bias.shape[0] != heads * dim or bonus.shape != (heads, dim):
            raise KernelError("a decay bias or bonus of the wrong shape")
    if head_decay is not None:
        _check(head_decay, "head decay", torch.float32, 1)
        if head_decay.shape[0] != heads:
            raise KernelError(f"{head_decay.shape[0]} decays for {heads} heads")
        if head_loss is None:
            head_loss = (1.0 - head_decay.double()).float()
        _check(head_loss, "head loss", torch.float32, 1)
        if head_loss.shape[0] != heads:
            raise KernelError(f"{head_loss.shape[0]} values of 1 - decay for {heads} heads")
    if rotary_dim:
        _check(inv_freq, "inv_freq", torch.float32, 1)
        if inv_freq.shape[0] != rotary_dim // 2:
            raise KernelError(f"inv_freq has {inv_freq.shape[0]} entries for a rotation over {rotary_dim}")
    if out_weight is not None:
        _check(out_weight, "output weight", torch.float32, 1)
        if out_weight.shape[0] != heads * vdim:
            raise KernelError(f"an output weight of {out_weight.shape[0]} for {heads} heads of {vdim}")
    # Long portions: a head's value columns are shared out over several CTAs (few heads and sequences
    # would leave most SMs idle while one walks thousands of tokens); the outputs' unit RMS, weight
    # and gate then follow in a row kernel.  The split depends on the step's shape only.
    col_parts, raw = 1, None
    if not getattr(step, "all_decode", False) and getattr(step, "max_q_len", tokens) >= RECURRENCE_SPLIT_MIN_PORTION:
        while (col_parts < 8 and heads * step.num_seqs * col_parts < _sm_count() and vdim % (2 * col_parts) == 0
               and vdim // (2 * col_parts) >= 8 and recurrence_supported(dim, vdim // (2 * col_parts))):
            col_parts *= 2
        if col_parts > 1:
            raw = torch.empty((tokens, heads * vdim), dtype=torch.float32, device=q.device)
    status = library().shiso_decay_recurrence(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), gate.data_ptr() if gate is not None else 0, q_ld, k_ld, v_ld, gate_ld,
        out.data_ptr(), out_ld, _CODES[act], state.data_ptr(), stride, _ptr(step.q_start), _ptr(step.state_slots),
        _ptr(step.positions), _ptr(decay_logits), logits_ld, _ptr(decay_bias), _ptr(bonus), _ptr(head_loss),
        _ptr(inv_freq) if rotary_dim else 0, int(rotary_dim), float(key_scale), _ptr(out_weight), float(eps), float(out_scale),
        _ptr(raw), col_parts, tokens, step.num_seqs, heads, dim, vdim, _stream(),
    )
    _done(status, "decay_recurrence" + (f" (columns over {col_parts} CTAs)" if raw is not None else ""), 2 if raw is not None else 1,
          shape=(tokens, heads, dim, vdim))
    return out


# --------------------------------------------------------------------------- windowed attention with pooled blocks


def _paged(cache, name, dtype, page_size):
    _check(cache, name, dtype, 4)
    if cache.shape[1] != page_size:
        raise KernelError(f"{name} of shape {tuple(cache.shape)} does not have pages of {page_size}")


def store_kv(k, v, kv_heads, dim, vdim, step, k_cache, v_cache, block_table, page_size):
    """A step's keys and values, as they are, into the paged caches (``k`` and ``v`` may be column ranges)."""
    act = k.dtype
    k_ld, v_ld = _rows(k, "k", act, kv_heads * dim), _rows(v, "v", act, kv_heads * vdim)
    _paged(k_cache, "k cache", act, page_size)
    _paged(v_cache, "v cache", act, page_size)
    if k_cache.shape[2:] != (kv_heads, dim) or v_cache.shape[2:] != (kv_heads, vdim):
        raise KernelError(f"caches of shape {tuple(k_cache.shape)} / {tuple(v_cache.shape)} for {kv_heads} heads of {dim} / {vdim}")
    _check(block_table, "block table", torch.int32, 2)
    status = library().shiso_store_kv(
        k.data_ptr(), k_ld, v.data_ptr(), v_ld, _CODES[act], _ptr(step.positions), _ptr(step.seq_of_token), _ptr(block_table),
        block_table.shape[1], _ptr(k_cache), _ptr(v_cache), k.shape[0], kv_heads, dim, vdim, page_size, _stream(),
    )
    _done(status, "store_kv", shape=(k.shape[0], kv_heads, dim + vdim))


def pool_kv(k_cache, v_cache, block_table, pooled_k, pooled_v, pooled_table, page_size, pool, step):
    """For every row of the step whose position ends a block of ``pool`` positions: the means of
    the block's cached keys and values (float32) as row ``position // pool`` of the pooled caches."""
    _paged(k_cache, "k cache", None, page_size)
    _paged(v_cache, "v cache", k_cache.dtype, page_size)
    _paged(pooled_k, "pooled k cache", torch.float32, page_size)
    _paged(pooled_v, "pooled v cache", torch.float32, page_size)
    if pooled_k.shape[2:] != k_cache.shape[2:] or pooled_v.shape[2:] != v_cache.shape[2:]:
        raise KernelError("pooled caches whose heads differ from the caches they summarise")
    _check(block_table, "block table", torch.int32, 2)
    _check(pooled_table, "pooled block table", torch.int32, 2)
    if pooled_table.shape != block_table.shape:
        raise KernelError("the two block tables of a step have one shape")
    kv_heads, dim, vdim = k_cache.shape[2], k_cache.shape[3], v_cache.shape[3]
    status = library().shiso_pool_kv(
        _ptr(k_cache), _ptr(v_cache), _code(k_cache), _ptr(block_table), _ptr(pooled_k), _ptr(pooled_v), _ptr(pooled_table),
        block_table.shape[1], _ptr(step.positions), _ptr(step.seq_of_token), step.num_tokens, kv_heads, dim, vdim, page_size,
        int(pool), _stream(),
    )
    _done(status, "pool_kv", shape=(step.num_tokens, kv_heads, dim + vdim))


def pooled_window_attention(q, heads, k_cache, v_cache, block_table, pooled_k, pooled_v, pooled_table, page_size, scale,
                            window, pool, step, out, out_scale=1.0):
    """Softmax attention of every row over the last ``window`` positions of its sequence and, in
    the same softmax, the pooled key and value of every block of ``pool`` positions that lies
    wholly behind the window; ``out`` (a column range, like ``q``) gets the result times ``out_scale``."""
    act = q.dtype
    kv_heads, dim, vdim = k_cache.shape[2], k_cache.shape[3], v_cache.shape[3]
    q_ld, out_ld = _rows(q, "q", act, heads * dim), _rows(out, "out", act, heads * vdim)
    _paged(k_cache, "k cache", act, page_size)
    _paged(v_cache, "v cache", act, page_size)
    _paged(pooled_k, "pooled k cache", torch.float32, page_size)
    _paged(pooled_v, "pooled v cache", torch.float32, page_size)
    _check(block_table, "block table", torch.int32, 2)
    _check(pooled_table, "pooled block table", torch.int32, 2)
    if pooled_table.shape != block_table.shape:
        raise KernelError("the two block tables of a step have one shape")
    lib = library()
    tokens = q.shape[0]
    seen = None
    if (
        act == torch.bfloat16 and dim == vdim and tokens >= TC_ATTENTION_MIN_TOKENS
        and getattr(step, "max_q_len", tokens) >= TC_ATTENTION_MIN_PORTION
        and lib.shiso_prefill_attention_tc_supported(dim, page_size) and q_ld % 8 == 0 and out_ld % 8 == 0
        and q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0
    ):
        # long portions: the window's tokens by the tensor-memory kernel, which leaves each row's
        # normalised result and the logarithm of its softmax sum; the pooled blocks are folded in after
        starts = getattr(step, "h_q_start", None)
        if starts:
            tiles = sum(-(-(b - a) // 128) for a, b in zip(starts[:-1], starts[1:]))
        else:
            tiles = tokens // 128 + step.num_seqs
        seen = torch.empty((tokens, heads), dtype=torch.float32, device=q.device)
        status = lib.shiso_prefill_attention_tc_open(
            q.data_ptr(), q_ld, _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1], _ptr(step.q_start),
            _ptr(step.start_pos), out.data_ptr(), out_ld, _ptr(seen), float(out_scale), tokens, step.num_seqs, tiles, heads, kv_heads, page_size,
            k_cache.shape[0], float(scale), int(window), _stream(),
        )
        _done(status, "prefill_attention (tcgen05, window of pooled_window_attention)", shape=(tokens, heads, dim))
    status = lib.shiso_pooled_window_attention(
        q.data_ptr(), q_ld, _CODES[act], _ptr(k_cache), _ptr(v_cache), _ptr(block_table), _ptr(pooled_k), _ptr(pooled_v),
        _ptr(pooled_table), block_table.shape[1], _ptr(step.positions), _ptr(step.seq_of_token), out.data_ptr(), out_ld,
        _ptr(seen), tokens, heads, kv_heads, dim, vdim, page_size, float(scale), int(window), int(pool), float(out_scale), _stream(),
    )
    _done(status, "pooled_window_attention" + (" (pooled blocks)" if seen is not None else ""), shape=(tokens, heads, dim))
    return out


# --------------------------------------------------------------------------- attention with a parameterised mask and weighting

_HEAD_NORMS = {None: 0, "before": 1, "after": 2}
_MASKS = {"window": 0, "chunk": 1}
MASKED_MAX_HEAD_DIM = 256  # what the kernels of this group keep of a head in a warp's registers
MASKED_MAX_SPLITS = 16  # CTAs that share a (row, head)'s keys in the general kernel
NO_WINDOW = 1 << 30  # a window of this size or more reaches back to the start of any sequence: the kernels that know "no window" are told so
MASKED_SCRATCH_BYTES = 64 << 20  # their partial results, at most; larger steps take one CTA a (row, head)


def head_prepare_store(proj, heads, kv_heads, dim, vdim, q_w, k_w, eps, norm_order, inv_freq, rotary_dim, magnitude, step,
                       k_cache, v_cache, block_table, page_size, store=True):
    """Prepares the heads of ``proj[T, heads*dim | kv_heads*dim | kv_heads*vdim | ...]`` in place:
    an RMS norm over every query and key head (``norm_order`` None, "before" or "after" the
    rotation; weights ``q_w`` / ``k_w`` of ``[dim]`` or None for a unit norm), the half-split
    rotation of the first ``rotary_dim`` entries by ``position * inv_freq`` with cosine and sine
    times ``magnitude``.  Queries are written back where they stood; keys and the values (copied
    as they are) go to the paged caches.  Returns the query columns."""
    act = proj.dtype
    q_cols, k_cols, v_cols = heads * dim, kv_heads * dim, kv_heads * vdim
    ld = _rows(proj, "projected rows", act)
    if proj.shape[1] < q_cols + k_cols + v_cols:
        raise KernelError(f"projected rows of {proj.shape[1]} do not hold {heads} + {kv_heads} heads of {dim} and {kv_heads} of {vdim}")
    if norm_order not in _HEAD_NORMS:
        raise KernelError(f"head norm order {norm_order!r}: expected None, 'before' or 'after'")
    for name, t in (("q norm weight", q_w), ("k norm weight", k_w)):
        if t is not None:
            _check(t, name, torch.float32, 1)
            if t.shape[0] != dim:
                raise KernelError(f"{name} has {t.shape[0]} entries for heads of {dim}")
    if rotary_dim:
        _check(inv_freq, "inv_freq", torch.float32, 1)
        if inv_freq.shape[0] != rotary_dim // 2:
            raise KernelError(f"inv_freq has {inv_freq.shape[0]} entries for a rotation over {rotary_dim}")
    _check(block_table, "block table", torch.int32, 2)
    if store:
        _paged(k_cache, "k cache", act, page_size)
        _paged(v_cache, "v cache", act, page_size)
        if k_cache.shape[2:] != (kv_heads, dim) or v_cache.shape[2:] != (kv_heads, vdim):
            raise KernelError(f"caches of shape {tuple(k_cache.shape)} / {tuple(v_cache.shape)} for {kv_heads} heads of {dim} / {vdim}")
    status = library().shiso_head_prepare_store(
        proj.data_ptr(), ld, _CODES[act], 0, q_cols, q_cols + k_cols, _ptr(q_w), _ptr(k_w), _ptr(inv_freq) if rotary_dim else 0,
        _ptr(step.positions), _ptr(step.seq_of_token), _ptr(block_table), block_table.shape[1],
        _ptr(k_cache) if store else 0, _ptr(v_cache) if store else 0, proj.shape[0], heads, kv_heads, dim, vdim, int(rotary_dim),
        page_size, float(eps), float(magnitude), _HEAD_NORMS[norm_order], int(bool(store)), _stream(),
    )
    _done(status, "head_prepare_store", shape=(proj.shape[0], heads + kv_heads, dim))
    return proj[:, :q_cols]


def gate_rows(x, gate):
    """``x *= sigmoid(gate)`` entry by entry, in place; both ``[T, C]`` in one type (column ranges may be given).  Returns ``x``."""
    x_ld = _rows(x, "rows", None)
    gate_ld = _rows(gate, "gate", x.dtype, x.shape[1])
    if gate.shape[0] != x.shape[0]:
        raise KernelError(f"{gate.shape[0]} gate rows for {x.shape[0]} rows")
    status = library().shiso_gate_rows(x.data_ptr(), x_ld, gate.data_ptr(), gate_ld, _code(x), x.shape[0], x.shape[1], _stream())
    _done(status, "gate_rows", shape=tuple(x.shape))
    return x


def joined_norm_store(proj, heads, kv_heads, dim, vdim, q_w, k_w, eps, q_temperature, values_from_keys, step, k_cache, v_cache,
                      block_table, page_size):
    """Prepares ``proj[T, heads*dim | kv_heads*dim | (kv_heads*vdim) | ...]`` in place: ONE RMS norm over
    all query columns together (weight ``q_w[heads*dim]``) and one over all key columns
    (``k_w[kv_heads*dim]``); the queries times ``1 + coef * ln(floor((p + 1) / every) + 1)`` at
    position ``p`` when ``q_temperature = (coef, every)``.  Queries are written back where they
    stood, normed keys go to the paged key cache, and the value cache gets the value columns or,
    with ``values_from_keys``, the key columns as they came.  Returns the query columns."""
    act = proj.dtype
    q_cols, k_cols, v_cols = heads * dim, kv_heads * dim, kv_heads * vdim
    ld = _rows(proj, "projected rows", act)
    if values_from_keys and vdim != dim:
        raise KernelError(f"values that are the keys have their size {dim}, not {vdim}")
    if proj.shape[1] < q_cols + k_cols + (0 if values_from_keys else v_cols):
        raise KernelError(f"projected rows of {proj.shape[1]} do not hold {heads} + {kv_heads} heads of {dim}")
    _check(q_w, "q norm weight", torch.float32, 1)
    _check(k_w, "k norm weight", torch.float32, 1)
    if q_w.shape[0] != q_cols or k_w.shape[0] != k_cols:
        raise KernelError(f"norm weights of {q_w.shape[0]} / {k_w.shape[0]} entries for {q_cols} query and {k_cols} key columns")
    _check(block_table, "block table", torch.int32, 2)
    _paged(k_cache, "k cache", act, page_size)
    _paged(v_cache, "v cache", act, page_size)
    if k_cache.shape[2:] != (kv_heads, dim) or v_cache.shape[2:] != (kv_heads, vdim):
        raise KernelError(f"caches of shape {tuple(k_cache.shape)} / {tuple(v_cache.shape)} for {kv_heads} heads of {dim} / {vdim}")
    coef, every = q_temperature if q_temperature is not None else (0.0, 0)
    status = library().shiso_joined_norm_store(
        proj.data_ptr(), ld, _CODES[act], q_cols, k_cols, q_cols if values_from_keys else q_cols + k_cols, v_cols, _ptr(q_w), _ptr(k_w),
        _ptr(step.positions), _ptr(step.seq_of_token), _ptr(block_table), block_table.shape[1], _ptr(k_cache), _ptr(v_cache),
        proj.shape[0], page_size, float(eps), float(coef), int(every), _stream(),
    )
    _done(status, "joined_norm_store", shape=(proj.shape[0], heads + kv_heads, dim))
    return proj[:, :q_cols]


def masked_attention(q, heads, k_cache, v_cache, block_table, page_size, scale, mask, size, keep_first, step, *, sigmoid=False,
                     key_bias=None, softcap=None, gate=None, general=False, gate_per_element=False):
    """Attention of every row over the keys its mask shows: ``mask`` "window" (the last ``size``
    positions and the first ``keep_first`` of the sequence) or "chunk" (the positions of the row's
    own run of ``size``, counted from 0).  Scores ``(q . k) * scale``, capped as
    ``softcap * tanh(score / softcap)`` when a cap is given; weights a softmax, or with ``sigmoid``
    one ``sigmoid(score + key_bias[head])`` per key, not normalised.  ``gate[T, heads]`` (logits)
    multiplies each head's output by its sigmoid; with ``gate_per_element`` it is ``[T, heads * vdim]``
    and every output entry has a gate of its own.  ``q`` and ``gate`` may be column ranges.
    Returns ``[T, heads * vdim]``.  bfloat16 steps that hold prompt portions take the tiled
    tensor-core kernel (key sizes in multiples of 16 up to 256, value sizes up to 128); steps of
    single tokens, float32 and other sizes take the general kernel, as does ``general=True``
    (tests compare the routes)."""
    act = q.dtype
    kv_heads, dim, vdim = k_cache.shape[2], k_cache.shape[3], v_cache.shape[3]
    q_ld = _rows(q, "q", act, heads * dim)
    _paged(k_cache, "k cache", act, page_size)
    _paged(v_cache, "v cache", act, page_size)
    _check(block_table, "block table", torch.int32, 2)
    if mask not in _MASKS:
        raise KernelError(f"mask {mask!r}: expected 'window' or 'chunk'")
    if key_bias is not None:
        _check(key_bias, "key bias", torch.float32, 1)
        if key_bias.shape[0] != heads:
            raise KernelError(f"key bias has {key_bias.shape[0]} entries for {heads} heads")
    gate_ld = _rows(gate, "gate", act, heads * (vdim if gate_per_element else 1)) if gate is not None else 0
    wide = int(bool(gate is not None and gate_per_element))
    tokens = q.shape[0]
    out = torch.empty((tokens, heads * vdim), dtype=act, device=q.device)
    lib = library()
    what = f"({mask}, {'sigmoid' if sigmoid else 'softmax'})"
    # A softmax over a window (with or without kept first tokens), heads of 64, no cap and no gate is
    # what the framework's tensor-memory prompt kernel and its TMA decode kernel compute: they take
    # the first positions as tiles of their own ahead of the window's.
    # (A gate per output entry is applied behind them by a row kernel; a gate per head keeps the kernels that know it.)
    plain_window = (
        not general and act == torch.bfloat16 and mask == "window" and not sigmoid and not softcap and (gate is None or wide)
        and dim == vdim and q.data_ptr() % 16 == 0 and q_ld % 8 == 0
    )
    if (
        plain_window and getattr(step, "all_decode", False) and heads // kv_heads <= MAX_DECODE_GROUP
        and lib.shiso_decode_attention_fused_supported(heads, kv_heads, dim, page_size)
    ):
        splits = decode_splits(tokens, kv_heads, min(block_table.shape[1] * page_size, size + keep_first + 2 * 64), True)
        status = lib.shiso_decode_attention_fused_kept(
            q.data_ptr(), q_ld, _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1], _ptr(step.positions),
            _ptr(step.seq_of_token), _ptr(out), tokens, heads, kv_heads, dim, page_size, k_cache.shape[0], float(scale),
            0 if size >= NO_WINDOW else int(size), int(keep_first), splits, _stream(),
        )
        _done(status, f"decode_attention (fused) {what}", shape=(tokens, heads, dim))
        return gate_rows(out, gate) if wide else out
    if (
        plain_window and not getattr(step, "all_decode", False) and tokens >= TC_ATTENTION_MIN_TOKENS
        and getattr(step, "max_q_len", tokens) >= TC_ATTENTION_MIN_PORTION
        and lib.shiso_prefill_attention_tc_supported(dim, page_size)
    ):
        starts = getattr(step, "h_q_start", None)
        if starts:
            tiles = sum(-(-(b - a) // 128) for a, b in zip(starts[:-1], starts[1:]))
        else:
            tiles = tokens // 128 + step.num_seqs
        status = lib.shiso_prefill_attention_tc_kept(
            q.data_ptr(), q_ld, _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1], _ptr(step.q_start),
            _ptr(step.start_pos), _ptr(out), heads * vdim, tokens, step.num_seqs, tiles, heads, kv_heads, page_size,
            k_cache.shape[0], float(scale), 0 if size >= NO_WINDOW else int(size), int(keep_first), _stream(),
        )
        _done(status, f"prefill_attention (tcgen05) {what}", shape=(tokens, heads, dim))
        return gate_rows(out, gate) if wide else out
    if (
        not general and act == torch.bfloat16 and not getattr(step, "all_decode", False)
        and lib.shiso_masked_attention_tiles_supported(dim, vdim)
    ):
        starts = getattr(step, "h_q_start", None)
        if starts:
            tiles = sum(-(-(b - a) // 64) for a, b in zip(starts[:-1], starts[1:]))
        else:
            tiles = tokens // 64 + step.num_seqs
        status = lib.shiso_masked_attention_tiles(
            q.data_ptr(), q_ld, _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1], _ptr(step.q_start),
            _ptr(step.start_pos), _ptr(out), heads * vdim, gate.data_ptr() if gate is not None else 0, gate_ld, _ptr(key_bias),
            step.num_seqs, tiles, heads, kv_heads, dim, vdim, page_size, float(scale), float(softcap or 0.0), _MASKS[mask], int(size),
            int(keep_first), int(bool(sigmoid)), wide, _stream(),
        )
        _done(status, f"masked_attention_tiles {what}", shape=(tokens, heads, dim))
        return out
    # CTAs a (row, head): one per 256 keys the mask can show (a number of the layer, not of the
    # step), while their partial results stay small; a second launch adds them up
    splits = max(1, min(MASKED_MAX_SPLITS, -(-(int(size) + int(keep_first)) // 256)))
    if tokens * heads * splits * (vdim + 2) * 4 > MASKED_SCRATCH_BYTES:
        splits = 1
    scratch = torch.empty((tokens * heads * splits * (vdim + 2),), dtype=torch.float32, device=q.device) if splits > 1 else None
    status = lib.shiso_masked_attention(
        q.data_ptr(), q_ld, _CODES[act], _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1], _ptr(step.positions),
        _ptr(step.seq_of_token), _ptr(out), heads * vdim, gate.data_ptr() if gate is not None else 0, gate_ld, _ptr(key_bias),
        tokens, heads, kv_heads, dim, vdim, page_size, float(scale), float(softcap or 0.0), _MASKS[mask], int(size), int(keep_first),
        int(bool(sigmoid)), splits, _ptr(scratch), wide, _stream(),
    )
    _done(status, f"masked_attention {what}", 2 if splits > 1 else 1, shape=(tokens, heads, dim))
    return out


# --------------------------------------------------------------------------- norms on a sublayer's output, polynomial activation


def norm_into(residual, y, w, eps, want_rows=True):
    """``residual += y * rsqrt(mean(y^2) + eps) * w`` (float32 rows, in place); returns the new
    residual rows in ``y``'s type - the residual itself when that is float32 - or None when not wanted."""
    _check(residual, "residual", torch.float32, 2)
    _check(y, "sublayer output", None, 2)
    _check(w, "norm weight", torch.float32, 1)
    tokens, hidden = residual.shape
    if y.shape != residual.shape or w.shape[0] != hidden:
        raise KernelError(f"output {tuple(y.shape)} and weight {tuple(w.shape)} do not match the residual {tuple(residual.shape)}")
    out = torch.empty_like(y) if want_rows and y.dtype != torch.float32 else None
    _done(library().shiso_norm_into(_ptr(residual), _ptr(y), _code(y), _ptr(w), _ptr(out), tokens, hidden, float(eps), _stream()),
          "norm_into", shape=(tokens, hidden))
    if not want_rows:
        return None
    return residual if out is None else out


def polynorm(z, coefficients, eps, out_dtype):
    """``a N(z) + b N(z^2) + c N(z^3) + e`` per row, ``N(u) = u * rsqrt(mean(u^2) + eps)``;
    ``coefficients`` = float32 ``[a, b, c, e]``."""
    ld = _rows(z, "z", out_dtype)
    _check(coefficients, "coefficients", torch.float32, 1)
    if coefficients.shape[0] != 4:
        raise KernelError(f"{coefficients.shape[0]} coefficients where a, b, c and e are expected")
    out = torch.empty(z.shape, dtype=out_dtype, device=z.device)
    _done(library().shiso_polynorm(z.data_ptr(), ld, _CODES[out_dtype], _ptr(coefficients), _ptr(out), z.shape[0], z.shape[1], float(eps),
                                   _stream()), "polynorm", shape=tuple(z.shape))
    return out


# --------------------------------------------------------------------------- layer norm, norms in groups


def add_layernorm(residual, deltas, w, eps, out_dtype, rows=None):
    """Layer norm with a weight and no bias of ``residual`` (float32 ``[T, H]``) plus up to two
    block outputs ``deltas`` (tensors of the output type); the sum is formed in float32 and,
    without ``rows``, stored back.  With ``rows`` only those rows are summed and normalised."""
    _check(residual, "residual", torch.float32, 2)
    _check(w, "norm weight", torch.float32, 1)
    tokens, hidden = residual.shape
    if w.shape[0] != hidden:
        raise KernelError(f"norm weight has {w.shape[0]} entries for rows of {hidden}")
    deltas = tuple(deltas)
    if len(deltas) > 2:
        raise KernelError(f"{len(deltas)} block outputs wait to be added; the kernel takes two")
    for d in deltas:
        _check(d, "delta", out_dtype, 2)
        if d.shape != residual.shape:
            raise KernelError(f"delta {tuple(d.shape)} does not match the residual {tuple(residual.shape)}")
    out_rows = tokens
    if rows is not None:
        _check(rows, "rows", torch.int32, 1)
        out_rows = rows.shape[0]
    out = torch.empty((out_rows, hidden), dtype=out_dtype, device=residual.device)
    status = library().shiso_add_layernorm(
        _ptr(residual), _ptr(deltas[0]) if deltas else 0, _ptr(deltas[1]) if len(deltas) > 1 else 0, _ptr(rows), _ptr(w), _ptr(out),
        _code(out), out_rows, hidden, float(eps), _stream(),
    )
    _done(status, "layernorm" if not deltas else f"add {len(deltas)} + layernorm", shape=(out_rows, hidden))
    return out


_GATE_MODES = {None: 0, "silu_before": 1, "sigmoid_after": 2}


def group_rmsnorm(x, weight, eps, groups, out_dtype, gate=None, gate_mode=None):
    """Rows ``x[T, W]`` (float32 or the output type; a column range may be given) in ``groups`` equal
    parts, each divided by its own root mean square, times ``weight``.  ``gate_mode``
    ``"silu_before"`` multiplies the rows by ``silu(gate)`` first, ``"sigmoid_after"`` the result by
    ``sigmoid(gate)``; ``gate`` is ``[T, W]`` of the output type (a column range may be given)."""
    tokens, width = x.shape
    x_ld = _rows(x, "x", None, width)
    if x.dtype not in (torch.float32, out_dtype):
        raise KernelError(f"rows of {x.dtype} for an output of {out_dtype}")
    _check(weight, "norm weight", torch.float32, 1)
    if weight.shape[0] != width or groups < 1 or width % groups:
        raise KernelError(f"a weight of {weight.shape[0]} or {groups} groups for rows of {width}")
    if (gate is None) != (gate_mode is None) or gate_mode not in _GATE_MODES:
        raise KernelError(f"gate mode {gate_mode!r} with{'out' if gate is None else ''} a gate")
    gate_ld = _rows(gate, "gate", out_dtype, width) if gate is not None else 0
    out = torch.empty((tokens, width), dtype=out_dtype, device=x.device)
    status = library().shiso_group_rmsnorm(
        x.data_ptr(), _code(x), x_ld, gate.data_ptr() if gate is not None else 0, gate_ld, _ptr(weight), _ptr(out), _code(out),
        tokens, width, int(groups), _GATE_MODES[gate_mode], float(eps), _stream(),
    )
    _done(status, "group_rmsnorm", shape=(tokens, width, groups))
    return out


# --------------------------------------------------------------------------- causal convolution, scalar-decay recurrences


def causal_conv(x, taps, bias, state, step, silu=True):
    """``y_t[c] = act(bias[c] + sum_j taps[c, j] x_{t-(L-1)+j}[c])`` per sequence (``x[T, C]``, a column
    range may be given); ``state`` (float32 ``[slots, L-1, C]``) holds each request's last ``L - 1``
    inputs and is brought up to date."""
    tokens, channels = x.shape
    x_ld = _rows(x, "x", None, channels)
    _check(taps, "conv taps", torch.float32, 2)
    n_taps = taps.shape[1]
    if taps.shape[0] != channels:
        raise KernelError(f"taps for {taps.shape[0]} channels, rows of {channels}")
    if bias is not None:
        _check(bias, "conv bias", torch.float32, 1)
    if state.shape[1:] != (n_taps - 1, channels):
        raise KernelError(f"conv state of shape {tuple(state.shape)} does not fit {n_taps} taps x {channels}")
    stride = _slot_rows(state, "conv state", torch.float32)
    y = torch.empty((tokens, channels), dtype=x.dtype, device=x.device)
    status = library().shiso_causal_conv(
        x.data_ptr(), x_ld, _code(x), _ptr(taps), _ptr(bias), state.data_ptr(), stride, _ptr(step.seq_of_token), _ptr(step.q_start),
        _ptr(step.state_slots), _ptr(y), tokens, step.num_seqs, channels, n_taps, int(bool(silu)), _stream(),
    )
    _done(status, "causal_conv", 2, shape=(tokens, channels))
    return y


def state_recurrence(q, k, v, state, step, heads, groups, dim, vdim, *, silu_inputs=False, head_loss=None,
                     dt=None, dt_bias=None, a_log=None, skip=None):
    """A matrix state ``S[dim, vdim]`` per head (``state``, float32 ``[slots, heads, dim, vdim]``) walked
    over each sequence's rows in order: ``S = a S + b k v^T``, ``o = S^T q + skip v``.  With
    ``head_loss`` (float32 ``[heads]``, one minus the head's decay): ``a = 1 - head_loss``, ``b = 1``.
    With ``dt`` (``[T, heads]``): ``b = softplus(dt + dt_bias)``, ``a = exp(-exp(a_log) b)``.  q and k
    are ``[T, groups * dim]``, head ``h`` reading group ``h // (heads / groups)``; ``silu_inputs``
    applies silu to q, k and v on load.  All inputs may be column ranges.  Returns float32
    ``[T, heads * vdim]``."""
    act = q.dtype
    tokens = q.shape[0]
    q_ld, k_ld = _rows(q, "q", act, groups * dim), _rows(k, "k", act, groups * dim)
    v_ld = _rows(v, "v", act, heads * vdim)
    if state.shape[1:] != (heads, dim, vdim):
        raise KernelError(f"a state of shape {tuple(state.shape)} for {heads} heads of {dim} x {vdim}")
    stride = _slot_rows(state, "recurrent state", torch.float32)
    if (dt is None) == (head_loss is None):
        raise KernelError("a recurrence takes either a decay per head or a step size per token and head")
    dt_ld = 0
    if dt is not None:
        dt_ld = _rows(dt, "dt", act, heads)
        for name, t in (("dt bias", dt_bias), ("a_log", a_log)):
            _check(t, name, torch.float32, 1)
            if t.shape[0] != heads:
                raise KernelError(f"{name} has {t.shape[0]} entries for {heads} heads")
    else:
        _check(head_loss, "head loss", torch.float32, 1)
        if head_loss.shape[0] != heads:
            raise KernelError(f"{head_loss.shape[0]} values of 1 - decay for {heads} heads")
    if skip is not None:
        _check(skip, "skip", torch.float32, 1)
        if skip.shape[0] != heads:
            raise KernelError(f"{skip.shape[0]} skip weights for {heads} heads")
    out = torch.empty((tokens, heads * vdim), dtype=torch.float32, device=q.device)
    status = library().shiso_state_recurrence(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), dt.data_ptr() if dt is not None else 0, q_ld, k_ld, v_ld, dt_ld, _CODES[act],
        _ptr(dt_bias), _ptr(a_log), _ptr(skip), _ptr(head_loss), state.data_ptr(), stride, _ptr(step.q_start), _ptr(step.state_slots),
        _ptr(out), tokens, step.num_seqs, heads, groups, dim, vdim, int(bool(silu_inputs)), _sm_count(), _stream(),
    )
    _done(status, "state_recurrence", shape=(tokens, heads, dim, vdim))
    return out


# --------------------------------------------------------------------------- latent attention


def _heads3(t, name, dtype):
    """Row and head strides of ``[T, H, W]`` whose last dimension is contiguous."""
    if not t.is_cuda or t.dim() != 3 or (t.shape[2] > 1 and t.stride(2) != 1) or (dtype is not None and t.dtype != dtype):
        raise KernelError(f"{name}: expected [T, H, W] CUDA rows of {dtype} with unit column stride, got {t.dtype} {tuple(t.shape)} {t.stride()}")
    return t.stride(0), t.stride(1)


def latent_store(rows, rank, norm_w, eps, inv_freq, rotary_dim, step, k_cache, block_table, page_size, magnitude=1.0, interleaved=False):
    """Each row ``[latent (rank) | shared key part]`` (a column range may be given): the latent
    RMS-normed with ``norm_w``, the rest rotated by the row's position (half-split pairs over
    ``rotary_dim``, or neighbours with ``interleaved``; cosine and sine times ``magnitude``); stored
    as the position's row of ``k_cache [pages, page_size, 1, width]``."""
    tokens, width = rows.shape
    ld = _rows(rows, "rows", k_cache.dtype, width)
    _paged(k_cache, "latent cache", rows.dtype, page_size)
    if k_cache.shape[2:] != (1, width):
        raise KernelError(f"a cache of shape {tuple(k_cache.shape)} for rows of {width}")
    _check(norm_w, "latent norm weight", torch.float32, 1)
    if norm_w.shape[0] != rank:
        raise KernelError(f"a norm weight of {norm_w.shape[0]} for a latent of {rank}")
    if rotary_dim:
        _check(inv_freq, "inv_freq", torch.float32, 1)
        if inv_freq.shape[0] != rotary_dim // 2:
            raise KernelError(f"inv_freq has {inv_freq.shape[0]} entries for a rotation over {rotary_dim}")
    _check(block_table, "block table", torch.int32, 2)
    status = library().shiso_latent_store(
        rows.data_ptr(), ld, _code(rows), _ptr(norm_w), _ptr(inv_freq) if rotary_dim else 0, _ptr(step.positions),
        _ptr(step.seq_of_token), _ptr(block_table), block_table.shape[1], _ptr(k_cache), tokens, int(rank), width, int(rotary_dim),
        page_size, float(eps), float(magnitude), int(bool(interleaved)), _stream(),
    )
    _done(status, "latent_store", shape=(tokens, width))


def rotate_heads(x, out, inv_freq, rotary_dim, step, magnitude=1.0, interleaved=False):
    """``x[T, H, W]`` with the half-split pairs (neighbours with ``interleaved``) of its first
    ``rotary_dim`` columns turned by each row's position, cosine and sine times ``magnitude``, into
    ``out[T, H, W]``; both may be column ranges of wider rows."""
    act = x.dtype
    x_ld, x_hs = _heads3(x, "x", act)
    out_ld, out_hs = _heads3(out, "out", act)
    if x.shape != out.shape:
        raise KernelError(f"rows of {tuple(x.shape)} into {tuple(out.shape)}")
    if rotary_dim:
        _check(inv_freq, "inv_freq", torch.float32, 1)
        if inv_freq.shape[0] != rotary_dim // 2:
            raise KernelError(f"inv_freq has {inv_freq.shape[0]} entries for a rotation over {rotary_dim}")
    tokens, heads, width = x.shape
    status = library().shiso_rotate_heads(
        x.data_ptr(), x_ld, x_hs, out.data_ptr(), out_ld, out_hs, _CODES[act], _ptr(inv_freq) if rotary_dim else 0,
        _ptr(step.positions), tokens, heads, width, int(rotary_dim), float(magnitude), int(bool(interleaved)), _stream(),
    )
    _done(status, "rotate_heads", shape=(tokens, heads, width))


def head_linear(x, w, out, gate=None):
    """A product per head: ``out[t, h] = w[h] x[t, h]`` for ``x[T, H, K]``, ``w[H, N, K]``, ``out[T, H, N]``
    (x and out may be column ranges); with ``gate[T, H]`` (a column range of rows of x's type) the
    head's result is multiplied by ``sigmoid(gate[t, h])``.  Float accumulation on CUDA cores."""
    x_ld, x_hs = _heads3(x, "x", None)
    out_ld, out_hs = _heads3(out, "out", None)
    _check(w, "w", None, 3)
    tokens, heads, k = x.shape
    n = w.shape[1]
    if w.shape != (heads, n, k) or out.shape != (tokens, heads, n):
        raise KernelError(f"x {tuple(x.shape)}, w {tuple(w.shape)} and out {tuple(out.shape)} do not fit")
    gate_ld = _rows(gate, "gate", x.dtype, heads) if gate is not None else 0
    status = library().shiso_head_linear(
        x.data_ptr(), x_ld, x_hs, _code(x), _ptr(w), _code(w), out.data_ptr(), out_ld, out_hs, _code(out),
        gate.data_ptr() if gate is not None else 0, gate_ld, tokens, heads, n, k, _stream(),
    )
    _done(status, "head_linear", shape=(tokens, heads, n, k))
    return out


LATENT_DECODE_SHARE_KEYS = 256  # a decode step's keys are shared out over CTAs in ranges of about this many (a run of 32 per warp) ...
LATENT_MAX_SHARES = 16  # ... up to this many CTAs a (row, head group)


LATENT_MMA_MIN_PORTION = 8  # steps whose longest portion has at least this many rows take the tensor-core kernel (bfloat16)


def latent_attention(q_lat, rank, k_cache, block_table, page_size, scale, step, general=False):
    """Causal softmax attention of ``q_lat[T, H, W]`` against the cached rows ``k_cache[pages, page_size,
    1, W]`` of each row's sequence; the values are the first ``rank`` entries of the same rows.
    Returns ``[T, H, rank]`` in the input type.  bfloat16 steps with prompt portions take the
    tensor-core kernel (16 rows of a sequence and eight heads a CTA) where the widths allow it;
    steps of single tokens, float32 and other widths the general kernel, which ``general=True`` forces."""
    _check(q_lat, "q", None, 3)
    tokens, heads, width = q_lat.shape
    _paged(k_cache, "latent cache", q_lat.dtype, page_size)
    if k_cache.shape[2:] != (1, width) or not 0 < rank <= width:
        raise KernelError(f"a cache of shape {tuple(k_cache.shape)} for queries of {width} and a latent of {rank}")
    _check(block_table, "block table", torch.int32, 2)
    out = torch.empty((tokens, heads, rank), dtype=q_lat.dtype, device=q_lat.device)
    lib = library()
    if (
        not general and q_lat.dtype == torch.bfloat16 and not getattr(step, "all_decode", False)
        and getattr(step, "max_q_len", tokens) >= LATENT_MMA_MIN_PORTION and lib.shiso_latent_prefill_supported(int(rank), width)
    ):
        starts = getattr(step, "h_q_start", None)
        if starts:
            tiles = sum(-(-(b - a) // 16) for a, b in zip(starts[:-1], starts[1:]))
        else:
            tiles = tokens // 16 + step.num_seqs
        status = lib.shiso_latent_prefill(
            _ptr(q_lat), _ptr(k_cache), _ptr(block_table), block_table.shape[1], _ptr(step.q_start), _ptr(step.start_pos), _ptr(out),
            step.num_seqs, tiles, heads, int(rank), width, page_size, float(scale), _stream(),
        )
        _done(status, "latent_attention (mma, prompt portions)", shape=(tokens, heads, width))
        return out
    # steps of single tokens at long contexts: a row's keys go to several CTAs (the split depends on the step's shape only)
    shares, scratch = 1, None
    if getattr(step, "all_decode", False):
        context = block_table.shape[1] * page_size
        shares = max(1, min(LATENT_MAX_SHARES, context // LATENT_DECODE_SHARE_KEYS, 2 * _sm_count() // max(1, tokens * -(-heads // 4))))  # two CTAs fit an SM
        if shares > 1:
            scratch = torch.empty((tokens * heads * shares * (rank + 2),), dtype=torch.float32, device=q_lat.device)
    status = library().shiso_latent_attention(
        _ptr(q_lat), _code(q_lat), _ptr(k_cache), _ptr(block_table), block_table.shape[1], _ptr(step.positions),
        _ptr(step.seq_of_token), _ptr(out), _ptr(scratch), tokens, heads, int(rank), width, page_size, float(scale), shares, _stream(),
    )
    _done(status, "latent_attention", 2 if shares > 1 else 1, shape=(tokens, heads, width))
    return out


# --------------------------------------------------------------------------- mixture of experts


def moe_route(logits, top, group_count, group_keep, scale, sigmoid=False, renormalize=False, correction=None, renorm_eps=0.0):
    """For every row of ``logits`` (float32 ``[T, E]``, a column range may be given): scores (softmax
    over all experts, or sigmoids), the ``top`` largest among the experts of the ``group_keep`` best
    of ``group_count`` groups of neighbours (a group's value is its largest), ranked by score +
    ``correction[e]`` where a correction (float32 ``[E]``) is given, and their weights: the scores
    themselves (divided by their sum + ``renorm_eps`` with ``renormalize``) times ``scale``.  Returns
    ids int32 and weights float32, both ``[T, top]``, best first."""
    ld = _rows(logits, "router logits", torch.float32)
    tokens, experts = logits.shape
    if correction is not None:
        _check(correction, "router correction", torch.float32, 1)
        if correction.shape[0] != experts:
            raise KernelError(f"a correction of {correction.shape[0]} entries for {experts} experts")
    ids = torch.empty((tokens, top), dtype=torch.int32, device=logits.device)
    weights = torch.empty((tokens, top), dtype=torch.float32, device=logits.device)
    status = library().shiso_moe_route(
        logits.data_ptr(), ld, _ptr(correction), _ptr(ids), _ptr(weights), tokens, experts, int(top), int(group_count), int(group_keep),
        float(scale), int(bool(sigmoid)), int(bool(renormalize)), float(renorm_eps), _stream(),
    )
    _done(status, "moe_route", shape=(tokens, experts, top))
    return ids, weights


MOE_MAX_EXPERTS = 256  # router outputs the grouping kernels keep in shared memory


def routed_experts(x, ids, weights, gate_up, down, extra=None, act="silu", limit=0.0, extra_gate=None, identity=0):
    """``out[t] = extra[t] + sum_j weights[t, j] * expert_{ids[t, j]}(x[t])`` with gated experts
    ``down[e] pair(gate x, up x)`` (``act`` / ``limit``: the pairs of ``glu_act``), ``gate_up[e] =
    [gate; up]``: ``x[T, H]``, ``gate_up[E, 2F, H]``, ``down[E, H, F]``.  Ids ``E .. E + identity - 1`` are
    identity experts: one adds ``weights[t, j] * x[t]``.  ``extra_gate`` (float32 ``[T, 1]``, a column
    range may be given) multiplies ``extra[t]`` by its sigmoid.  The (row, choice) pairs are grouped
    by expert on the device; nothing about the routing reaches the host."""
    _check(x, "x", None, 2)
    _check(ids, "expert ids", torch.int32, 2)
    _check(weights, "expert weights", torch.float32, 2)
    _check(gate_up, "gate/up matrices", None, 3)
    _check(down, "down matrices", gate_up.dtype, 3)
    tokens, hidden = x.shape
    experts, two_ff, _ = gate_up.shape
    top = ids.shape[1]
    if ids.shape != (tokens, top) or weights.shape != ids.shape or gate_up.shape[2] != hidden or down.shape != (experts, hidden, two_ff // 2):
        raise KernelError("ids, weights or expert matrices of the wrong shape")
    if extra is not None:
        _check(extra, "extra", x.dtype, 2)
        if extra.shape != x.shape:
            raise KernelError(f"extra rows of {tuple(extra.shape)} beside {tuple(x.shape)}")
    if act not in _GLU_ACTS:
        raise KernelError(f"gated pair {act!r}: expected one of {sorted(_GLU_ACTS)}")
    gate_ld = 0
    if extra_gate is not None:
        if extra is None:
            raise KernelError("a gate on extra rows that are absent")
        gate_ld = _rows(extra_gate, "extra gate", torch.float32, 1)
        if extra_gate.shape[0] != tokens:
            raise KernelError(f"{extra_gate.shape[0]} gates for {tokens} rows")
    ff, total = two_ff // 2, tokens * top
    if identity < 0 or experts + identity > MOE_MAX_EXPERTS:
        raise KernelError(f"{experts} experts and {identity} identity experts; the grouping kernels take {MOE_MAX_EXPERTS} in all")
    ints = torch.empty((experts + identity + 3 * total,), dtype=torch.int32, device=x.device)
    mid = torch.empty((total, ff), dtype=x.dtype, device=x.device)
    y = torch.empty((total, hidden), dtype=torch.float32, device=x.device)
    out = torch.empty_like(x)
    status = library().shiso_routed_experts(
        _ptr(x), _code(x), _ptr(ids), _ptr(weights), _ptr(gate_up), _ptr(down), _code(gate_up), _ptr(extra),
        extra_gate.data_ptr() if extra_gate is not None else 0, gate_ld, _ptr(out), _ptr(ints),
        _ptr(mid), _ptr(y), tokens, hidden, ff, experts, int(identity), top, _GLU_ACTS[act], float(limit), _stream(),
    )
    _done(status, "routed_experts", 6, shape=(tokens, top, experts, ff, hidden))
    return out


# --------------------------------------------------------------------------- sampling


def _picks(out, rows, device):
    if out is None:
        return torch.empty((rows,), dtype=torch.int32, device=device)
    _check(out, "out", torch.int32, 1)
    if out.shape[0] != rows:
        raise KernelError(f"out has {out.shape[0]} entries for {rows} rows")
    return out


def _status_place(status_out) -> int:
    if status_out is None:
        return 0
    _check(status_out, "status_out", torch.int32, 1)
    if status_out.shape[0] != 1:
        raise KernelError("status_out is one int32")
    return status_out.data_ptr()


def suppress(logits: torch.Tensor, rows: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """Sets ``logits[rows[i], ids[i]]`` to -inf, in place, before a pick
    (crates/shiso-engine/src/sampling.rs:156-174; kernels/cuda/sample/sample.cu:18-26)."""
    _check(logits, "logits", torch.float32, 2)
    _check(rows, "rows", torch.int32, 1)
    _check(ids, "ids", torch.int32, 1)
    if rows.shape != ids.shape:
        raise KernelError(f"{rows.shape[0]} rows for {ids.shape[0]} ids")
    _done(library().shiso_suppress(_ptr(logits), _ptr(rows), _ptr(ids), rows.shape[0], logits.shape[0], logits.shape[1],
                                   _stream()), "suppress")
    return logits


def words_to_host(src: torch.Tensor, host: torch.Tensor) -> bool:
    """``host[:n] = src`` for int32 ``src`` on the device and pinned ``host``, as a kernel in the
    stream that stores into the host's memory in place: a step's tokens reach the host without a
    turn of the copy engine between two kernels (decode at batch 8 loses 2 to 3 % to that turn).
    The host reads them after an event, as after a copy.  False when the device cannot address
    the memory; the caller then copies."""
    _check(src, "src", torch.int32, 1)
    if host.is_cuda or host.dtype != torch.int32 or not host.is_contiguous() or not host.is_pinned() or host.numel() < src.numel():
        return False
    status = library().shiso_copy_words(_ptr(src), host.data_ptr(), src.numel(), 2, _stream())
    if status == 1004:  # memory the device cannot address
        return False
    _done(status, "words_to_host", shape=(src.numel(),))
    return True


def words_from_host(host: torch.Tensor, dst: torch.Tensor) -> bool:
    """``dst = host[:n]`` for pinned int32 ``host`` and ``dst`` on the device, as a kernel in the
    stream that loads from the host's memory in place (a step's few KB of positions and block
    tables).  The host may write the buffer again after an event that follows, as after a copy.
    False when the device cannot address the memory; the caller then copies."""
    _check(dst, "dst", torch.int32, 1)
    if host.is_cuda or host.dtype != torch.int32 or not host.is_contiguous() or not host.is_pinned() or host.numel() < dst.numel():
        return False
    status = library().shiso_copy_words(host.data_ptr(), _ptr(dst), dst.numel(), 1, _stream())
    if status == 1004:  # memory the device cannot address
        return False
    _done(status, "words_from_host", shape=(dst.numel(),))
    return True


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None, status_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The index of each row's largest value (the smallest index among equals), int32, written
    to ``out`` when one is given.  ``status_out`` (one int32) receives the status word of the
    bounded waits, which is cleared: see ``check_kernel_status``."""
    _check(logits, "logits", torch.float32, 2)
    rows, vocab = logits.shape
    out = _picks(out, rows, logits.device)
    status = _status_place(status_out)
    if vocab >= 8192:
        # chunks of at least 1,024 values; no more blocks (rows x chunks)
        # than a few waves: 64 rows x 64 chunks of four values a thread took 13.6 us for 17 MB
        chunks = max(1, min(128, -(-vocab // 1024), -(-4 * _sm_count() // rows)))
        scratch = torch.empty((2 * rows * chunks,), dtype=torch.float32, device=logits.device)
        code = library().shiso_argmax_chunked(_ptr(logits), _ptr(out), _ptr(scratch), rows, vocab, chunks, status, _stream())
        _done(code, "argmax", 2)
        return out
    _done(library().shiso_argmax(_ptr(logits), _ptr(out), rows, vocab, status, _stream()), "argmax")
    return out


def sample(logits, temperature, top_k, top_p, min_p, keys, positions, out=None, status_out=None) -> torch.Tensor:
    """Keyed sampling, one row per request: float32 ``temperature``/``top_p``/``min_p``,
    int32 ``top_k`` (0 = off) and ``positions``, int64 ``keys``, all of length rows.
    ``status_out`` as in ``argmax``."""
    _check(logits, "logits", torch.float32, 2)
    rows = logits.shape[0]
    for name, t, dt in (
        ("temperature", temperature, torch.float32), ("top_k", top_k, torch.int32),
        ("top_p", top_p, torch.float32), ("min_p", min_p, torch.float32),
        ("keys", keys, torch.int64), ("positions", positions, torch.int32),
    ):
        _check(t, name, dt, 1)
        if t.shape[0] != rows:
            raise KernelError(f"{name} has {t.shape[0]} entries for {rows} rows")
    out = _picks(out, rows, logits.device)
    status = library().shiso_sample(
        _ptr(logits), _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(min_p), _ptr(keys), _ptr(positions),
        _ptr(out), rows, logits.shape[1], _status_place(status_out), _stream(),
    )
    _done(status, "sample")
    return out
