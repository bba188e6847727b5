"""Python faces of the CUDA entry points: argument checks, the launch, the error.

Every function here runs a hand-written kernel on the current CUDA stream.  There is no
CPU or library fallback: tensors that are not on a CUDA device, or sizes that a kernel
does not take, raise ``KernelError`` with the reason.
"""

from __future__ import annotations

import ctypes
import os
import weakref

import torch

from .build import ATTENTION_SOURCES, CORE_SOURCES, load_library

_ERRORS = {
    1: "unsupported dtype (kernels take float32 and bfloat16)",
    2: "a size this kernel does not take",
    3: "a pointer or stride is not aligned as the kernel needs",
    4: "the CUDA launch failed",
    5: "a size beyond the kernel's stated maximum",
}


class KernelError(RuntimeError):
    pass


_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}


#: Programmatic dependent launch of the kernels (a kernel's set-up and weight loads overlap the tail
#: of the kernel before it).  The reference's switch keeps its name: DRYFT_PDL=off|on|early
#: (engine/kernels/cuda_small.py:22); anything but "off" turns it on.
PDL = os.environ.get("DRYFT_PDL", "early") != "off"
_PDL_APPLIED: set = set()


def _with_pdl(lib, setter: str):
    if id(lib) not in _PDL_APPLIED:
        getattr(lib, setter)(1 if PDL else 0)
        _PDL_APPLIED.add(id(lib))
    return lib


def set_pdl(enabled: bool) -> None:
    """Switches programmatic dependent launch on or off for every kernel launched from now on."""
    global PDL
    PDL = bool(enabled)
    _PDL_APPLIED.clear()


#: The tcgen05 kernels bound every wait on an mbarrier; a wait that runs out records a code, the CTA
#: frees its tensor memory and returns, and the step's numbers are not valid.  Each device has one
#: small int32 buffer that receives these codes (one word per kernel family), so that the host can
#: read it with a step's results instead of synchronising for it.
STATUS_WORDS = 8
_STATUS_UNITS = {"gemm_decode": 0, "gemm_pair": 1, "attention_prefill_tc": 2, "attention_decode": 3}
_STATUS: dict[int, torch.Tensor] = {}
_STATUS_BOUND: set = set()
_STATUS_LIBRARIES: list = []          # (library, units) of every library that was handed a status word


def status_words(device=None) -> torch.Tensor:
    """The int32 status buffer of ``device`` (default: the current one); all zero while nothing failed."""
    index = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    held = _STATUS.get(index)
    if held is None:
        held = _STATUS[index] = torch.zeros(STATUS_WORDS, dtype=torch.int32, device=f"cuda:{index}")
    return held


def _bind_status(lib, units: tuple[str, ...]):
    """Tells ``lib``'s kernels (on the current device) which words of the status buffer are theirs."""
    index = torch.cuda.current_device()
    if (id(lib), index) not in _STATUS_BOUND:
        words = status_words(index)
        for unit in units:
            rc = getattr(lib, f"dfi_{unit}_set_status_word")(ctypes.c_void_p(words.data_ptr() + 4 * _STATUS_UNITS[unit]))
            if rc != 0:
                raise KernelError(f"could not hand the status word to {unit}")
        _STATUS_BOUND.add((id(lib), index))
        if not any(held is lib for held, _ in _STATUS_LIBRARIES):
            _STATUS_LIBRARIES.append((lib, units))
    return lib


def raise_for_status(values, device=None) -> None:
    """``values``: a host copy of ``status_words``.  If any word is set, clears the words and every
    stream-K counter of the device (a kernel that gave up may have left tickets behind) and raises."""
    values = [int(v) for v in values]
    if not any(values):
        return
    if torch.cuda.is_available():
        index = torch.cuda.current_device() if device is None else torch.device(device).index or 0
        torch.cuda.synchronize(index)
        status_words(index).zero_()
        for lib, units in _STATUS_LIBRARIES:
            for unit in units:
                getattr(lib, f"dfi_{unit}_error")(1)
        for table in (_ATTENTION_SCRATCH, _DECODE_SCRATCH, _GEMM_SCRATCH):
            for device_key, held in table.items():
                if torch.device(device_key).index == index:
                    held[1].zero_()
    names = {v: k for k, v in _STATUS_UNITS.items()}
    failed = ", ".join(f"{names.get(i, f'word {i}')} (wait code {v})" for i, v in enumerate(values) if v)
    raise KernelError(f"a bounded wait ran out in a tcgen05 kernel: {failed}; the results of the step are not valid")


def check_status(device=None) -> None:
    """Reads the status buffer (this synchronises) and raises ``KernelError`` if a wait ran out."""
    raise_for_status(status_words(device).tolist(), device)


def wait_selftest(unit: str, limit: int = 1, code: int = 77, head_dim: int = 128) -> None:
    """Launches ``unit``'s one-CTA self-test kernel: it waits ``limit`` tries on a barrier that nothing
    arrives on, records ``code`` as a real kernel's wait would, frees its tensor memory and returns."""
    lib = _attention_library(head_dim) if unit.startswith("attention") else _core()
    _check(getattr(lib, f"dfi_{unit}_wait_selftest")(ctypes.c_uint(limit), int(code), _stream()), f"{unit} self-test")


def _core():
    return _bind_status(_with_pdl(load_library("dfi_core", CORE_SOURCES), "dfi_set_pdl"), ("gemm_decode", "gemm_pair"))


def _code(t: torch.Tensor) -> int:
    if t.dtype not in _DTYPE_CODE:
        raise KernelError(f"unsupported dtype {t.dtype}: kernels take float32 and bfloat16")
    return _DTYPE_CODE[t.dtype]


def _need_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("the kernels run on a CUDA device only (tensor is on %s); there is no CPU path" % t.device)


def _ptr(t: torch.Tensor | None):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


_HELD_STREAM: ctypes.c_void_p | None = None


def _stream():
    if _HELD_STREAM is not None:
        return _HELD_STREAM
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class on_current_stream:
    """Within this block the kernels are launched on the stream that is current at its entry, looked up
    once instead of at every launch (the look-up costs as much as a launch).  The caller does not
    switch streams inside the block."""

    def __enter__(self):
        global _HELD_STREAM
        self.before = _HELD_STREAM
        _HELD_STREAM = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        return self

    def __exit__(self, *exc):
        global _HELD_STREAM
        _HELD_STREAM = self.before
        return False


#: kernels launched through this module since import (a step captured in a CUDA graph counts
#: once at capture; replays are counted by the caller)
LAUNCHES = 0


def _check(rc: int, what: str, detail: str = "") -> None:
    global LAUNCHES
    LAUNCHES += 1
    if rc != 0:
        raise KernelError(f"{what}: {_ERRORS.get(rc, f'error {rc}')}{' (' + detail + ')' if detail else ''}")


def _f(x: float):
    return ctypes.c_float(x)


def embedding(table: torch.Tensor, ids: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """``table[ids] * scale`` for int32 ``ids [rows]``."""
    _need_cuda(table, ids)
    assert ids.dtype == torch.int32 and table.is_contiguous()
    rows, (vocab, hidden) = ids.numel(), table.shape
    out = torch.empty((rows, hidden), dtype=table.dtype, device=table.device)
    _check(_core().dfi_embedding(_ptr(table), _ptr(ids), _ptr(out), rows, hidden, vocab, _code(table), _stream()),
           "embedding")
    if scale != 1.0:
        scale_add(out, None, scale)
    return out


def scale_add(a: torch.Tensor, b: torch.Tensor | None, scale: float = 1.0) -> torch.Tensor:
    """``a = a * scale + b`` in place (float32 arithmetic, one rounding); ``b`` may be None."""
    _need_cuda(a, b)
    assert a.is_contiguous() and (b is None or (b.is_contiguous() and b.shape == a.shape and b.dtype == a.dtype))
    _check(_core().dfi_scale_add(_ptr(a), _ptr(b), ctypes.c_longlong(a.numel()), _f(scale), _code(a), _stream()),
           "scale_add")
    return a


def add_rows(residual: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    """``residual += delta`` in place: the residual sum where no norm follows it."""
    return scale_add(residual, delta, 1.0)


def transform_logits(logits: torch.Tensor, scale: float = 1.0, softcap: float = 0.0) -> torch.Tensor:
    """``logits * scale`` and then, with ``softcap`` c > 0, ``c * tanh(x / c)``: in place, float32."""
    _need_cuda(logits)
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    _check(_core().dfi_scale_cap(_ptr(logits), ctypes.c_longlong(logits.numel()), _f(scale), _f(softcap), _stream()),
           "transform_logits")
    return logits


def gather_rows(x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    """``x[rows]`` for int32 ``rows`` on the device."""
    _need_cuda(x, rows)
    assert rows.dtype == torch.int32 and x.is_contiguous() and x.dim() == 2
    out = torch.empty((rows.numel(), x.shape[1]), dtype=x.dtype, device=x.device)
    _check(_core().dfi_gather_rows(_ptr(x), _ptr(rows), _ptr(out), rows.numel(), x.shape[1], _code(x), _stream()),
           "gather_rows")
    return out


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``x * rsqrt(mean(x^2) + eps) * weight`` per row; ``weight`` is float32."""
    _need_cuda(x, weight)
    assert x.is_contiguous() and x.dim() == 2 and weight.dtype == torch.float32 and weight.numel() == x.shape[1]
    out = torch.empty_like(x)
    _check(_core().dfi_rmsnorm(_ptr(x), _ptr(None), _ptr(weight), _ptr(out), x.shape[0], x.shape[1], _f(eps),
                               _code(x), _stream()), "rms_norm")
    return out


def add_rms_norm(residual: torch.Tensor, delta: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``residual += delta`` in place (float32 sum), then the RMSNorm of the new residual."""
    _need_cuda(residual, delta, weight)
    assert residual.is_contiguous() and delta.is_contiguous() and residual.shape == delta.shape
    assert residual.dtype == delta.dtype and weight.dtype == torch.float32 and weight.numel() == residual.shape[1]
    out = torch.empty_like(residual)
    _check(_core().dfi_rmsnorm(_ptr(residual), _ptr(delta), _ptr(weight), _ptr(out), residual.shape[0],
                               residual.shape[1], _f(eps), _code(residual), _stream()), "add_rms_norm")
    return out


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` for ``gate_up [rows, 2*inter]`` with the gate half first."""
    _need_cuda(gate_up)
    assert gate_up.is_contiguous() and gate_up.dim() == 2 and gate_up.shape[1] % 2 == 0
    rows, inter = gate_up.shape[0], gate_up.shape[1] // 2
    out = torch.empty((rows, inter), dtype=gate_up.dtype, device=gate_up.device)
    for start in range(0, rows, 65535):
        part = gate_up[start:start + 65535]
        _check(_core().dfi_swiglu(_ptr(part), _ptr(out[start:start + 65535]), part.shape[0], inter,
                                  _code(gate_up), _stream()), "swiglu")
    return out


def qk_norm_rope_write(qkv: torch.Tensor, n_q: int, n_kv: int, head_dim: int, q_weight, k_weight, eps: float,
                       cos, sin, row_pos: torch.Tensor, row_seq: torch.Tensor, cache) -> torch.Tensor:
    """Per-head RMSNorm (if weights are given) and rotation (if tables are given: ``cos``/``sin
    [positions, rotary_dim / 2]`` rotate the first ``rotary_dim <= head_dim`` elements of a head) of the
    query and key heads of ``qkv [rows, (n_q + 2 n_kv) * head_dim]``; queries are
    rewritten in place, keys and values go to ``cache`` (a ``LayerCache``) at each row's
    position unless ``cache.writes`` is false.  Returns the query view ``[rows, n_q * head_dim]``.
    """
    _need_cuda(qkv, row_pos, row_seq, cache.k, cache.v, cache.block_table)
    rows, width = qkv.shape
    assert qkv.is_contiguous() and width == (n_q + 2 * n_kv) * head_dim
    assert row_pos.dtype == torch.int32 and row_seq.dtype == torch.int32
    assert cache.k.dtype == qkv.dtype and cache.k.is_contiguous() and cache.v.is_contiguous()
    assert cache.k.shape[1] == n_kv and cache.k.shape[3] == head_dim and cache.k.shape[2] == cache.page_size
    if head_dim % 4 or head_dim > 256:
        raise KernelError(f"qk_norm_rope_write: head_dim {head_dim} must be a multiple of 4 and at most 256")
    for w in (q_weight, k_weight):
        assert w is None or (w.dtype == torch.float32 and w.numel() == head_dim)
    rotary_dim = head_dim
    if cos is not None:
        assert cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.shape == sin.shape
        assert cos.is_contiguous() and sin.is_contiguous()
        rotary_dim = 2 * cos.shape[1]
        if rotary_dim > head_dim:
            raise KernelError(f"qk_norm_rope_write: tables for {rotary_dim} rotating elements, heads of {head_dim}")
    _check(_core().dfi_qk_norm_rope_write(
        _ptr(qkv), rows, width, n_q, n_kv, head_dim, _ptr(q_weight), _ptr(k_weight), _f(eps), _ptr(cos), _ptr(sin),
        rotary_dim, _ptr(row_pos), _ptr(row_seq), _ptr(cache.k), _ptr(cache.v), _ptr(cache.block_table),
        cache.block_table.shape[1], cache.page_size, cache.ring_tokens, 1 if cache.writes else 0, _code(qkv),
        _stream()), "qk_norm_rope_write", f"head_dim {head_dim}")
    return qkv[:, : n_q * head_dim]


def attention_generic(q: torch.Tensor, cache, row_seq: torch.Tensor, row_pos: torch.Tensor, n_q: int, n_kv: int,
                      head_dim: int, scale: float, window: int = 0) -> torch.Tensor:
    """Causal attention of every query row over its sequence's cached keys up to the
    row's own position (and not further back than ``window`` keys, if given).
    ``q`` may be a column slice of a wider matrix (its row stride is passed on)."""
    _need_cuda(q, cache.k, row_seq, row_pos)
    rows = q.shape[0]
    assert q.stride(1) == 1 and q.shape[1] == n_q * head_dim
    vec = 4 if q.dtype == torch.float32 else 8
    if head_dim % vec or head_dim > 256:
        raise KernelError(f"attention: head_dim {head_dim} must be a multiple of {vec} and at most 256")
    if n_q % n_kv:
        raise KernelError(f"attention: {n_q} query heads are not a multiple of {n_kv} key/value heads")
    out = torch.empty((rows, n_q * head_dim), dtype=q.dtype, device=q.device)
    _check(_core().dfi_attention_generic(
        _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(cache.k), _ptr(cache.v), _ptr(cache.block_table),
        cache.block_table.shape[1], _ptr(row_seq), _ptr(row_pos), rows, n_q, n_kv, head_dim, cache.page_size,
        cache.ring_tokens, window, _f(scale), _code(q), _stream()), "attention", f"head_dim {head_dim}")
    return out


def _attention_library(head_dim: int):
    return _bind_status(_with_pdl(load_library(f"dfi_attention_d{head_dim}", ATTENTION_SOURCES,
                                               [f"-DDFI_HEAD_DIM={head_dim}"]), "dfi_attention_set_pdl"),
                        ("attention_prefill_tc", "attention_decode"))


_RETIRED_SCRATCH: list = []


def _scratch(table: dict, device, floats: int, counters: int):
    """The scratch of one kernel family on ``device``: room for partial sums and zeroed counters, made
    once at the size its first caller asks for (the engine always asks for the same: one wave of CTAs,
    65,536 counters).  A later call that needs more gets a new one; the old one is kept for good, because
    CUDA graphs captured earlier still name its address."""
    held = table.get(device)
    if held is None or held[0].numel() < floats or held[1].numel() < counters:
        if held is not None:
            _RETIRED_SCRATCH.append(held)
        held = (torch.empty(max(floats, held[0].numel() if held else 0), dtype=torch.float32, device=device),
                torch.zeros(max(counters, 65536, held[1].numel() if held else 0), dtype=torch.int32, device=device))
        table[device] = held
    return held


DECODE_ATTENTION_MAX_SEQS = 1024
_ATTENTION_SCRATCH: dict = {}


def attention_prefill(q, cache, ctx, n_q: int, n_kv: int, head_dim: int, scale: float, window: int = 0):
    """Tensor-core flash attention (bfloat16) for any number of query rows per sequence."""
    _need_cuda(q, cache.k)
    assert q.dtype == torch.bfloat16 and q.stride(1) == 1 and q.shape[1] == n_q * head_dim
    out = torch.empty((q.shape[0], n_q * head_dim), dtype=q.dtype, device=q.device)
    _check(_attention_library(head_dim).dfi_attention_prefill(
        _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(cache.k), _ptr(cache.v), _ptr(cache.block_table),
        cache.block_table.shape[1], _ptr(ctx.cu_rows), _ptr(ctx.seq_start), ctx.n_seqs, ctx.max_q_len, n_q, n_kv,
        cache.page_size, cache.ring_tokens, window, _f(scale), _stream()), "attention_prefill",
        f"head_dim {head_dim}, {n_q}/{n_kv} heads")
    return out


def attention_prefill_tc(q, cache, ctx, n_q: int, n_kv: int, head_dim: int, scale: float, window: int = 0,
                         tiles_per_cta: int = 0):
    """Flash attention for prompts on tcgen05 (head sizes 64 and 128): TMA-fed pages of keys and values,
    scores and the page's output in tensor memory, one thread per query row for the softmax.
    ``tiles_per_cta``: 1 or 2 query tiles of 128 rows a CTA; 0 lets the launch choose (two, unless the
    shares are short or that would leave half the SMs without a CTA)."""
    _need_cuda(q, cache.k)
    assert q.dtype == torch.bfloat16 and q.stride(1) == 1 and q.shape[1] == n_q * head_dim
    lib = _attention_library(head_dim)
    if not lib.dfi_attention_prefill_tc_available():
        raise KernelError(f"attention_prefill_tc: head_dim {head_dim} has no tcgen05 kernel (64 and 128 have)")
    out = torch.empty((q.shape[0], n_q * head_dim), dtype=q.dtype, device=q.device)
    _check(lib.dfi_attention_prefill_tc(
        _ptr(q), q.shape[0], q.stride(0), _ptr(out), out.stride(0), _ptr(cache.k), _ptr(cache.v),
        ctypes.c_longlong(cache.k.shape[0]), _ptr(cache.block_table), cache.block_table.shape[1], _ptr(ctx.cu_rows),
        _ptr(ctx.seq_start), ctx.n_seqs, ctx.max_q_len, n_q, n_kv, cache.page_size, cache.ring_tokens, window,
        _f(scale), int(tiles_per_cta), _stream()), "attention_prefill_tc", f"head_dim {head_dim}, {n_q}/{n_kv} heads")
    return out


def attention_tc_error(head_dim: int, reset: bool = True) -> int:
    """0, or the code of the first bounded wait that ran out in the tcgen05 attention kernel (synchronises)."""
    return _attention_library(head_dim).dfi_attention_prefill_tc_error(int(reset))


class TokenPrep:
    """What ``attention_decode`` needs to prepare the step's tokens itself: the raw projection ``qkv
    [sequences, (n_q + 2 n_kv) * head_dim]``, the per-head norm weights (or None), its eps, and the
    rotation tables (or None)."""

    __slots__ = ("qkv", "q_weight", "k_weight", "eps", "cos", "sin")

    def __init__(self, qkv, q_weight, k_weight, eps, cos, sin):
        self.qkv, self.q_weight, self.k_weight, self.eps, self.cos, self.sin = qkv, q_weight, k_weight, eps, cos, sin


def decode_prepares_tokens(qkv: torch.Tensor, ctx, n_q: int, n_kv: int, head_dim: int, cos=None) -> bool:
    """True if ``attention_decode`` can take this step's raw projection (``prep=``) instead of queries
    prepared by ``qk_norm_rope_write``: a bfloat16 step of one token per sequence with a head size that
    is a power of two, whose rotation (if any) takes the whole head."""
    return (qkv.is_cuda and (cos is None or 2 * cos.shape[1] == head_dim) and qkv.dtype == torch.bfloat16 and ctx.all_decode and head_dim in (16, 32, 64, 128)
            and n_q // n_kv <= 16 and ctx.n_seqs <= DECODE_ATTENTION_MAX_SEQS and qkv.stride(1) == 1
            and qkv.stride(0) % 4 == 0 and bool(_attention_library(head_dim).dfi_attention_decode_prepares()))


#: Lengths (in keys) at which the decode attention's launch shape changes with ``ctx.max_kv_len`` (the
#: kernel library names the same ones: ``dfi_attention_decode_kv_step``)
DECODE_KV_STEPS = (2048, 5120, 10240)


def decode_kv_limit(longest: int, max_context: int) -> int:
    """What a decode step whose longest sequence holds ``longest`` keys says as its ``max_kv_len``: the
    smallest of ``DECODE_KV_STEPS`` that covers it, at most ``max_context``.  A step launched (or a graph
    captured) under a limit serves every step whose sequences stay within it."""
    for step in DECODE_KV_STEPS:
        if longest <= step:
            return min(step, max_context)
    return max_context


def attention_decode(q, cache, ctx, n_q: int, n_kv: int, head_dim: int, scale: float, window: int = 0,
                     n_ctas: int | None = None, prep: TokenPrep | None = None):
    """Tensor-core attention (bfloat16) for steps with one query row per sequence: the pages of
    all sequences are dealt to ``n_ctas`` CTAs (default: as many as run at once) in equal runs, and
    the parts of a sequence that end up in different CTAs are merged by the last of them to finish.

    With ``prep`` (and ``q`` None) the kernel also does what ``qk_norm_rope_write`` does for the step's
    tokens: per-head norm and rotation of q and k, and (if ``cache.writes``) the new key and value
    into the cache.

    ``ctx.decode_plans`` (a dict that lives as long as one pass through the model, or absent): how the
    launch deals its pages is then worked out once, by a small kernel before the first launch that deals
    these pages, and the launches of the other layers read it instead of working it out CTA by CTA."""
    if prep is not None:
        q = prep.qkv
        _need_cuda(q, cache.k)
        assert q.dtype == torch.bfloat16 and q.shape == (ctx.n_seqs, (n_q + 2 * n_kv) * head_dim)
    else:
        _need_cuda(q, cache.k)
        assert q.dtype == torch.bfloat16 and q.stride(1) == 1 and q.shape == (ctx.n_seqs, n_q * head_dim)
    lib = _attention_library(head_dim)
    if not n_ctas:
        n_ctas = lib.dfi_attention_decode_wave()
    n_ctas = min(n_ctas, 4096)
    lib.dfi_attention_decode_scratch_floats.restype = ctypes.c_longlong
    floats, n_counters = lib.dfi_attention_decode_scratch_floats(n_ctas), ctx.n_seqs * n_kv
    held = _scratch(_ATTENTION_SCRATCH, q.device, floats, n_counters)
    out = torch.empty((q.shape[0], n_q * head_dim), dtype=q.dtype, device=q.device)
    max_kv_len = int(getattr(ctx, "max_kv_len", 0) or 0)
    plans, fresh = None, 0
    shared = getattr(ctx, "decode_plans", None)
    if shared is not None:
        # everything the plans depend on: the launches of one pass that agree in it deal the same pages
        key = ("attention_decode", head_dim, ctx.seq_start.data_ptr(), ctx.n_seqs, n_q, n_kv, window, n_ctas, max_kv_len)
        plans = shared.get(key)
        if plans is None:
            lib.dfi_attention_decode_plan_bytes.restype = ctypes.c_longlong
            plans = shared[key] = torch.empty(lib.dfi_attention_decode_plan_bytes(n_ctas), dtype=torch.uint8, device=q.device)
            fresh = 1
            global LAUNCHES
            LAUNCHES += 1                        # the call then launches the planning kernel too
    if prep is not None:
        _check(lib.dfi_attention_decode_prepared(
            _ptr(q), q.stride(0), _ptr(prep.q_weight), _ptr(prep.k_weight), _f(prep.eps), _ptr(prep.cos), _ptr(prep.sin),
            int(cache.writes), _ptr(out), out.stride(0), _ptr(cache.k), _ptr(cache.v), ctypes.c_longlong(cache.k.shape[0]),
            _ptr(cache.block_table),
            cache.block_table.shape[1], _ptr(ctx.seq_start), ctx.n_seqs, n_q, n_kv, cache.page_size, cache.ring_tokens,
            window, _f(scale), n_ctas, _ptr(held[0]), _ptr(held[1]), max_kv_len, _ptr(plans), fresh, _stream()),
            "attention_decode", f"head_dim {head_dim}, {n_q}/{n_kv} heads, tokens prepared inside")
        return out
    _check(lib.dfi_attention_decode(
        _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(cache.k), _ptr(cache.v), ctypes.c_longlong(cache.k.shape[0]),
        _ptr(cache.block_table),
        cache.block_table.shape[1], _ptr(ctx.seq_start), ctx.n_seqs, n_q, n_kv, cache.page_size, cache.ring_tokens,
        window, _f(scale), n_ctas, _ptr(held[0]), _ptr(held[1]), max_kv_len, _ptr(plans), fresh, _stream()),
        "attention_decode", f"head_dim {head_dim}, {n_q}/{n_kv} heads")
    return out


def attention(q: torch.Tensor, cache, ctx, n_q: int, n_kv: int, head_dim: int, scale: float,
              window: int = 0) -> torch.Tensor:
    """Attention of a step's query rows over the cache, by the kernel that fits: the
    tensor-core kernels for bfloat16 and head sizes in steps of 16 up to 128 (prompts with head
    size 64 or 128 on tcgen05, the others and decoding on mma.sync), the plain kernel for float32
    and for head sizes up to 256."""
    if q.dtype == torch.bfloat16 and head_dim % 16 == 0 and head_dim <= 128:
        if ctx.all_decode and n_q // n_kv <= 16 and ctx.n_seqs <= DECODE_ATTENTION_MAX_SEQS:
            return attention_decode(q, cache, ctx, n_q, n_kv, head_dim, scale, window)
        if head_dim in (64, 128):
            return attention_prefill_tc(q, cache, ctx, n_q, n_kv, head_dim, scale, window)
        return attention_prefill(q, cache, ctx, n_q, n_kv, head_dim, scale, window)
    return attention_generic(q, cache, ctx.row_seq, ctx.row_pos, n_q, n_kv, head_dim, scale, window)


def argmax(logits: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """Index of the largest float32 logit per row (lowest index on ties), int32."""
    _need_cuda(logits)
    assert logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1
    if out is None:
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
    assert out.dtype == torch.int32 and out.numel() == logits.shape[0] and out.is_contiguous()
    _check(_core().dfi_argmax(_ptr(logits), logits.shape[0], logits.stride(0), logits.shape[1], _ptr(out), _stream()),
           "argmax")
    return out


def sample_temperature(logits: torch.Tensor, uniforms: torch.Tensor, temperature: float,
                       out: torch.Tensor | None = None) -> torch.Tensor:
    """One draw per row from ``softmax(logits / temperature)`` by inverse CDF at ``uniforms [rows]``."""
    _need_cuda(logits, uniforms)
    assert logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1
    assert uniforms.dtype == torch.float32 and uniforms.numel() == logits.shape[0]
    if not temperature > 0:
        raise KernelError("sample_temperature: temperature must be positive (use argmax for greedy)")
    if out is None:
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
    assert out.dtype == torch.int32 and out.numel() == logits.shape[0] and out.is_contiguous()
    _check(_core().dfi_sample_temperature(_ptr(logits), logits.shape[0], logits.stride(0), logits.shape[1],
                                          _ptr(uniforms), _f(temperature), _ptr(out), _stream()),
           "sample_temperature")
    return out


_GEMM_SCRATCH: dict = {}
SKINNY_MAX_ROWS = 64

#: Tiles of 128 rows x 64 k per CTA that a decode kernel asks into L2 for the product after it (``NextWeights``).
#: Measured at Qwen3-4B sizes, batch 8: 4 tiles take 2 % off the step, 8 tiles 0.6 %, 16 tiles add 2.6 %.  0: none.
NEXT_TILES = int(os.environ.get("DRYFT_NEXT_TILES", "4"))


def _gemm_scratch(device, n_ctas: int, counters: int):
    """The stream-K scratch of a device: room for every CTA's partial sums, and zeroed counters."""
    lib = _core()
    lib.dfi_skinny_gemm_partial_floats.restype = ctypes.c_longlong
    floats = lib.dfi_skinny_gemm_partial_floats(n_ctas)
    return _scratch(_GEMM_SCRATCH, device, floats, counters)


def skinny_linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype | None = None,
                  swiglu: bool = False, n_ctas: int | None = None) -> torch.Tensor:
    """``x @ weight.T`` (or, with ``swiglu``, ``silu(x @ gate.T) * (x @ up.T)`` for ``weight = [gate; up]``)
    for at most 64 rows of bfloat16 ``x``: the decode step's matrix product, bound by reading ``weight`` once.
    ``n_ctas`` (default: one per SM) is how many persistent CTAs share the work."""
    _need_cuda(x, weight)
    m, k = x.shape
    assert x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.shape[1] == k
    assert x.is_contiguous() and weight.is_contiguous()
    if m > SKINNY_MAX_ROWS or k % 8:
        raise KernelError(f"skinny_linear takes at most {SKINNY_MAX_ROWS} rows and K in steps of 8, got {m} x {k}")
    n = weight.shape[0] // 2 if swiglu else weight.shape[0]
    out_dtype = out_dtype or x.dtype
    lib = _core()
    if not n_ctas:
        n_ctas = lib.dfi_sm_count()
    partials, counters = _gemm_scratch(x.device, n_ctas, lib.dfi_skinny_gemm_counters(n, int(swiglu)))
    out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    _check(lib.dfi_skinny_gemm(_ptr(x), _ptr(weight), _ptr(out), m, n, k, int(swiglu), n_ctas, _ptr(partials),
                               _ptr(counters), _DTYPE_CODE[out_dtype], _stream()), "skinny_linear",
           f"{m} x {k} by {weight.shape[0]} x {k}")
    return out


def tc_error(reset: bool = True) -> int:
    """0, or the code of the first bounded wait that ran out in the decode product's kernel (synchronises)."""
    return _core().dfi_gemm_decode_error(int(reset))


_DECODE_SCRATCH: dict = {}


def pair_linear(x: torch.Tensor, weight: torch.Tensor, swiglu: bool = False) -> torch.Tensor:
    """``x @ weight.T`` (with ``swiglu``: ``silu(x @ gate.T) * (x @ up.T)`` for ``weight = [gate; up]``) in
    bfloat16 for many rows: the persistent tcgen05 kernel that runs each 256 x 256 tile on a pair of SMs
    (``csrc/gemm_tcgen05_pair.cu``)."""
    _need_cuda(x, weight)
    m, k = x.shape
    assert x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.shape[1] == k
    assert x.is_contiguous() and weight.is_contiguous()
    if k % 8:
        raise KernelError(f"pair_linear takes K in steps of 8, got {k}")
    n = weight.shape[0] // 2 if swiglu else weight.shape[0]
    out = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    _check(_core().dfi_gemm_pair(_ptr(x), _ptr(weight), _ptr(out), m, n, k, n, int(swiglu), _stream()), "pair_linear",
           f"{m} x {k} by {weight.shape[0]} x {k}")
    return out


def pair_error(reset: bool = True) -> int:
    """The error word of the pair kernel: 0, or the code of the wait that ran out."""
    return _core().dfi_gemm_pair_error(int(reset))


#: rows from which the pair kernel is used for the SwiGLU product (below, the library product + SwiGLU kernel is as fast or faster)
PAIR_MIN_ROWS = 1024

#: Which kernel takes a prompt's plain bfloat16 products (more than 64 rows): "library" (the default: the
#: library's GEMM, as in the reference's prefill, which measured faster on these shapes) or "own" (the
#: pair kernel for every one of them, so that the whole step runs on this package's kernels).
PREFILL_GEMM = os.environ.get("DRYFT_PREFILL_GEMM", "library")


class ScaledRows:
    """Rows ``w (.) r`` of an RMS norm that still lack their factor ``1 / rms(r)``: the product that
    reads them applies it to its result.  ``ssq [parts, stride]`` holds partial sums of squares of
    ``r`` per row; ``dim`` and ``eps`` are the norm's.  With ``ssq`` None the rows are complete (the
    factor is in them): what a product over many rows hands on, where a kernel of its own normalises."""

    __slots__ = ("rows", "ssq", "dim", "eps")

    def __init__(self, rows: torch.Tensor, ssq: torch.Tensor, dim: int, eps: float):
        self.rows, self.ssq, self.dim, self.eps = rows, ssq, dim, eps

    @property
    def shape(self):
        return self.rows.shape

    @property
    def dtype(self):
        return self.rows.dtype


def add_norm_fusable(rows: torch.Tensor) -> bool:
    """True if a product whose result is a delta of the residual ``rows`` can add it there itself and hand on
    the rows of the next norm (``linear(..., add_norm=...)``): the decode kernel in its epilogue, the
    library's product over many rows with the residual as its addend."""
    return (rows.is_cuda and rows.dtype == torch.bfloat16 and rows.dim() == 2 and rows.shape[1] % 8 == 0
            and rows.is_contiguous())


class NextWeights:
    """A word about the weights a decode step streams next: ``weight [N, K]`` (with ``swiglu``: ``[gate; up]``
    of ``2 N`` rows) of the product that follows the kernel this is given to (``then=``).  The kernel asks
    the first tiles behind that product's opening ring into L2 once its own stream has been asked for.  A
    hint: results never depend on it, and kernels that cannot use it ignore it.  It does not keep the
    matrix alive."""

    __slots__ = ("_weight", "swiglu", "_hints", "__weakref__")

    def __init__(self, weight: torch.Tensor, swiglu: bool = False):
        self._weight, self.swiglu = weakref.ref(weight), bool(swiglu)
        self._hints: dict = {}

    @property
    def weight(self) -> torch.Tensor | None:
        return self._weight()

    def hint(self, rows: int):
        """The kernels' form of the hint for a step of ``rows`` rows (a host buffer), or None."""
        w = self.weight
        if w is None or NEXT_TILES <= 0 or not w.is_cuda or w.dtype != torch.bfloat16 \
                or not 0 < rows <= SKINNY_MAX_ROWS or w.dim() != 2 or w.shape[1] % 8 or not w.is_contiguous():
            return None
        key = (w.data_ptr(), rows)
        held = self._hints.get(key)
        if held is None:
            lib = _core()
            held = ctypes.create_string_buffer(lib.dfi_next_stream_bytes())
            n = w.shape[0] // 2 if self.swiglu else w.shape[0]
            rc = lib.dfi_gemm_decode_next_stream(held, _ptr(w), rows, n, w.shape[1], int(self.swiglu), 0, NEXT_TILES)
            held = held if rc == 0 else False
            self._hints = {key: held}            # one entry: a part's weights stay where they are between steps
        return held or None


_NEXT_WEIGHTS: dict = {}


def next_weights(weight: torch.Tensor | None, swiglu: bool = False) -> NextWeights | None:
    """The ``NextWeights`` of a matrix, made once for each tensor object (None for None)."""
    if weight is None:
        return None
    key = (id(weight), bool(swiglu))
    held = _NEXT_WEIGHTS.get(key)
    if held is None or held.weight is not weight:
        held = _NEXT_WEIGHTS[key] = NextWeights(weight, swiglu)
        weakref.finalize(weight, _NEXT_WEIGHTS.pop, key, None)
    return held


def _hint(then: NextWeights | None, rows: int):
    return then.hint(rows) if then is not None else None


def decode_linear(x, weight: torch.Tensor, out_dtype: torch.dtype | None = None,
                  swiglu: bool = False, n_ctas: int | None = None, add_norm=None, then: NextWeights | None = None):
    """``x @ weight.T`` (with ``swiglu``: ``silu(x @ gate.T) * (x @ up.T)`` for ``weight = [gate; up]``)
    for at most 64 rows of bfloat16 ``x``: the decode step's product as a persistent stream-K kernel on
    tcgen05, with TMA loads and the accumulator in tensor memory.  ``n_ctas``: CTAs that share the
    work (default one per SM).

    ``x`` may be ``ScaledRows``: their factor is applied to the result.  ``add_norm = (residual,
    norm_weight, eps)``: the product is a residual delta; ``residual`` is updated in place and the call
    returns the ``ScaledRows`` of ``rms_norm(residual) * norm_weight`` for the next product.  ``then``: the
    weights of the product that the step runs after this one (see ``NextWeights``)."""
    scaled = x if isinstance(x, ScaledRows) else None
    if scaled is not None:
        x = scaled.rows
        if scaled.ssq is None:
            scaled = None                        # complete rows: nothing left to apply
    _need_cuda(x, weight)
    m, k = x.shape
    assert x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.shape[1] == k
    assert x.is_contiguous() and weight.is_contiguous()
    if m > SKINNY_MAX_ROWS or k % 8:
        raise KernelError(f"decode_linear takes at most {SKINNY_MAX_ROWS} rows and K in steps of 8, got {m} x {k}")
    n = weight.shape[0] // 2 if swiglu else weight.shape[0]
    out_dtype = out_dtype or x.dtype
    lib = _core()
    if not n_ctas:
        n_ctas = lib.dfi_sm_count()
    lib.dfi_gemm_decode_partial_floats.restype = ctypes.c_longlong
    floats, counters = lib.dfi_gemm_decode_partial_floats(n_ctas), lib.dfi_gemm_decode_counters(n, int(swiglu))
    held = _scratch(_DECODE_SCRATCH, x.device, floats, counters)
    out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    what = f"{m} x {k} by {weight.shape[0]} x {k}"
    hint = _hint(then, m)
    if scaled is None and add_norm is None:
        _check(lib.dfi_gemm_decode(_ptr(x), _ptr(weight), _ptr(out), m, n, k, int(swiglu), n_ctas, _ptr(held[0]),
                                   _ptr(held[1]), _DTYPE_CODE[out_dtype], hint, _stream()), "decode_linear", what)
        return out
    in_ssq, in_parts, in_dim, in_eps = None, 0, 0, 0.0
    if scaled is not None:
        assert scaled.ssq.dtype == torch.float32 and scaled.ssq.shape[1] == lib.dfi_gemm_decode_ssq_stride()
        in_ssq, in_parts, in_dim, in_eps = _ptr(scaled.ssq), scaled.ssq.shape[0], scaled.dim, scaled.eps
    residual = norm_weight = out_ssq = ssq = None
    if add_norm is not None:
        res, norm_w, eps = add_norm
        if swiglu or out_dtype != torch.bfloat16:
            raise KernelError("decode_linear adds a residual to a plain bfloat16 product only")
        assert res.shape == (m, n) and res.dtype == torch.bfloat16 and res.is_contiguous()
        assert norm_w.shape == (n,) and norm_w.dtype == torch.float32
        ssq = torch.empty((lib.dfi_gemm_decode_ssq_parts(m, n, k, n_ctas), lib.dfi_gemm_decode_ssq_stride()),
                          dtype=torch.float32, device=x.device)
        residual, norm_weight, out_ssq = _ptr(res), _ptr(norm_w), _ptr(ssq)
    _check(lib.dfi_gemm_decode_fused(_ptr(x), _ptr(weight), _ptr(out), m, n, k, int(swiglu), n_ctas, _ptr(held[0]),
                                     _ptr(held[1]), _DTYPE_CODE[out_dtype], in_ssq, in_parts, in_dim,
                                     ctypes.c_float(in_eps), residual, norm_weight, out_ssq, hint, _stream()),
           "decode_linear", what)
    if add_norm is not None:
        return ScaledRows(out, ssq, n, float(add_norm[2]))
    return out


def simt_linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``x @ weight.T`` on the float32 pipes (``csrc/gemm_simt.cu``): every product and sum in float32 in
    the order of k.  Any sizes; float32 operands, or bfloat16 ones with a bfloat16 or float32 result."""
    _need_cuda(x, weight)
    assert x.dim() == 2 and weight.dim() == 2 and x.shape[1] == weight.shape[1] and x.dtype == weight.dtype
    x, weight = x.contiguous(), weight.contiguous()
    out_dtype = out_dtype or x.dtype
    if out_dtype not in _DTYPE_CODE or (x.dtype == torch.float32 and out_dtype != torch.float32):
        raise KernelError(f"simt_linear: {x.dtype} operands cannot give a {out_dtype} result")
    out = torch.empty((x.shape[0], weight.shape[0]), dtype=out_dtype, device=x.device)
    _check(_core().dfi_gemm_simt(_ptr(x), _ptr(weight), _ptr(out), x.shape[0], weight.shape[0], x.shape[1], _code(x),
                                 _DTYPE_CODE[out_dtype], _stream()), "simt_linear",
           f"{x.shape[0]} x {x.shape[1]} by {weight.shape[0]} x {weight.shape[1]}")
    return out


def linear(x, weight: torch.Tensor, out_dtype: torch.dtype | None = None, add_norm=None,
           then: NextWeights | None = None):
    """``x @ weight.T`` for ``weight [out, in]`` as stored in the model file.

    bfloat16 with at most 64 rows (decoding) runs the hand-written stream-K tcgen05 kernel; larger
    bfloat16 products go to the library's GEMM, as the reference's prefill does
    (engine/engine.py:881-884), or with ``DRYFT_PREFILL_GEMM=own`` to the pair kernel.  float32
    operands, and bfloat16 matrices whose width is no multiple of 8 (which the TMA-fed kernels do not
    take), run the plain float32-pipe kernel of this package: true 32-bit, no library, no
    reduced-precision mode.  ``out_dtype=torch.float32`` keeps bfloat16 products unrounded (used for
    logits).  ``ScaledRows`` in, ``add_norm`` and ``then`` are those of ``decode_linear``; the other
    kernels ignore ``then``.  ``add_norm`` over more than 64 bfloat16 rows: the library's product takes the
    residual as its addend and the norm kernel follows; the ``ScaledRows`` returned are complete.
    """
    if isinstance(x, ScaledRows) and x.ssq is None:
        x = x.rows
    if isinstance(x, ScaledRows) or (add_norm is not None and x.shape[0] <= SKINNY_MAX_ROWS):
        # only made and asked for where the decode kernel runs (add_norm_fusable)
        return decode_linear(x, weight, out_dtype, add_norm=add_norm, then=then)
    _need_cuda(x, weight)
    if add_norm is not None:
        # Many rows: the residual is the product's addend (float32 sum on the accumulator, rounded once), so the
        # delta is never written and the norm reads one tensor.
        residual, norm_weight, eps = add_norm
        assert x.dtype == torch.bfloat16 and residual.dtype == torch.bfloat16 and residual.is_contiguous()
        assert residual.shape == (x.shape[0], weight.shape[0]) and x.shape[1] == weight.shape[1]
        if PREFILL_GEMM == "own" and x.is_contiguous() and weight.is_contiguous():
            normed = add_rms_norm(residual, pair_linear(x, weight), norm_weight, eps)
        else:
            residual.addmm_(x, weight.t())
            normed = rms_norm(residual, norm_weight, eps)
        return ScaledRows(normed, None, weight.shape[0], float(eps))
    assert x.dim() == 2 and weight.dim() == 2 and x.shape[1] == weight.shape[1] and x.dtype == weight.dtype
    if x.dtype == torch.float32 or x.shape[1] % 8:
        return simt_linear(x, weight, out_dtype)
    if x.shape[0] <= SKINNY_MAX_ROWS and x.is_contiguous():
        return decode_linear(x, weight, out_dtype, then=then)
    if out_dtype is not None and out_dtype != x.dtype:
        return torch.mm(x, weight.t(), out_dtype=out_dtype)
    if PREFILL_GEMM == "own" and x.is_contiguous() and weight.is_contiguous():
        return pair_linear(x, weight)
    return torch.mm(x, weight.t())


def linear_swiglu(x, gate_up: torch.Tensor, then: NextWeights | None = None) -> torch.Tensor:
    """``silu(x @ gate.T) * (x @ up.T)`` for the fused matrix ``gate_up = [gate; up]``: one kernel
    for bfloat16 (the decode kernel for few rows, the pair kernel for many), else the product followed by
    the SwiGLU kernel."""
    if isinstance(x, ScaledRows) and x.ssq is None:
        x = x.rows
    if isinstance(x, ScaledRows):
        return decode_linear(x, gate_up, swiglu=True, then=then)
    if x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and x.is_contiguous():
        if x.shape[0] <= SKINNY_MAX_ROWS:
            return decode_linear(x, gate_up, swiglu=True, then=then)
        if (x.shape[0] >= PAIR_MIN_ROWS or PREFILL_GEMM == "own") and gate_up.is_contiguous():
            return pair_linear(x, gate_up, swiglu=True)          # prompts: the activation on the accumulator
    return swiglu(linear(x, gate_up))
