"""Typed wrappers over the kernel library: they check dtypes, layouts and devices, and pass raw
pointers with the current CUDA stream.  Every function needs CUDA tensors; none has a CPU path.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import lib as _lib
from .lib import KernelError

F32, BF16 = 0, 1
_c_void_p, _c_int, _c_long, _c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_float


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"dtype {dtype} has no kernel (float32 and bfloat16 do)")


def _stream() -> ctypes.c_void_p:
    return _c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return _c_void_p(0 if t is None else t.data_ptr())


def _check(t: torch.Tensor, name: str, dtype: Optional[torch.dtype] = None, dense: bool = True) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} is on {t.device}; the kernels run on CUDA only")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} has dtype {t.dtype}, expected {dtype}")
    if dense and not t.is_contiguous():
        raise KernelError(f"{name} is not contiguous")


def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t] = float(table[ids[t]]); out is float32 [tokens, hidden]."""
    _check(table, "table"); _check(ids, "ids", torch.int32); _check(out, "out", torch.float32)
    vocab, hidden = table.shape
    tokens = ids.numel()
    if out.shape != (tokens, hidden):
        raise KernelError(f"embed: out is {tuple(out.shape)}, expected {(tokens, hidden)}")
    _lib.core().call("mrun_embed", _ptr(table), dtype_code(table.dtype), _ptr(ids), _ptr(out),
                     _c_int(tokens), _c_int(hidden), _c_int(vocab), _stream())
    return out


def add_rmsnorm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """resid (+= delta) then out = rmsnorm(resid) * weight; with ``rows`` only those rows are
    normed and resid is left as it is."""
    _check(resid, "resid", torch.float32); _check(weight, "weight", torch.float32); _check(out, "out")
    hidden = resid.shape[-1]
    n_rows = resid.shape[0] if rows is None else rows.numel()
    if delta is not None:
        _check(delta, "delta", out.dtype)
        if delta.shape != resid.shape:
            raise KernelError(f"add_rmsnorm: delta {tuple(delta.shape)} vs resid {tuple(resid.shape)}")
    if rows is not None:
        _check(rows, "rows", torch.int32)
    if weight.numel() != hidden or out.shape != (n_rows, hidden):
        raise KernelError(f"add_rmsnorm: weight {tuple(weight.shape)}, out {tuple(out.shape)}, "
                          f"expected hidden {hidden}, rows {n_rows}")
    _lib.core().call("mrun_add_rmsnorm", _ptr(resid), _ptr(delta), _ptr(weight), _c_float(eps), _ptr(out),
                     dtype_code(out.dtype), _ptr(rows), _c_int(n_rows), _c_int(hidden), _stream())
    return out


def rotary_table(positions: torch.Tensor, inv_freq: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t, j] = (cos, sin)(positions[t] * inv_freq[j]); inv_freq is float64."""
    _check(positions, "positions", torch.int32); _check(inv_freq, "inv_freq", torch.float64)
    _check(out, "out", torch.float32)
    tokens, half = positions.numel(), inv_freq.numel()
    if out.shape != (tokens, half, 2):
        raise KernelError(f"rotary_table: out is {tuple(out.shape)}, expected {(tokens, half, 2)}")
    _lib.core().call("mrun_rotary_table", _ptr(positions), _ptr(inv_freq), _ptr(out), _c_int(tokens),
                     _c_int(half), _stream())
    return out


def qk_norm_rope_cache(qkv: torch.Tensor, heads: int, kv_heads: int, head_dim: int,
                       q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                       rot: Optional[torch.Tensor], rotary_dim: int, slots: Optional[torch.Tensor],
                       k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                       page_size: int) -> None:
    """In place on the q part of ``qkv``; k and v go into the pages that ``slots`` names."""
    _check(qkv, "qkv")
    tokens = qkv.shape[0]
    if qkv.shape[1] != (heads + 2 * kv_heads) * head_dim:
        raise KernelError(f"qk_norm_rope_cache: qkv is {tuple(qkv.shape)}, expected width "
                          f"{(heads + 2 * kv_heads) * head_dim}")
    for name, w in (("q_weight", q_weight), ("k_weight", k_weight)):
        if w is not None:
            _check(w, name, torch.float32)
            if w.numel() != head_dim:
                raise KernelError(f"qk_norm_rope_cache: {name} has {w.numel()} elements, head_dim is {head_dim}")
    if rot is not None:
        _check(rot, "rot", torch.float32)
        if rot.shape != (tokens, rotary_dim // 2, 2):
            raise KernelError(f"qk_norm_rope_cache: rot is {tuple(rot.shape)}, expected "
                              f"{(tokens, rotary_dim // 2, 2)}")
    if slots is not None:
        _check(slots, "slots", torch.int32)
        if slots.numel() != tokens:
            raise KernelError("qk_norm_rope_cache: one slot per token is needed")
        for name, c in (("k_cache", k_cache), ("v_cache", v_cache)):
            _check(c, name, qkv.dtype)
            if c.dim() != 4 or c.shape[1:] != (kv_heads, page_size, head_dim):
                raise KernelError(f"qk_norm_rope_cache: {name} is {tuple(c.shape)}, expected "
                                  f"[pages, {kv_heads}, {page_size}, {head_dim}]")
    _lib.core().call("mrun_qk_norm_rope_cache", _ptr(qkv), dtype_code(qkv.dtype), _ptr(q_weight),
                     _ptr(k_weight), _c_float(eps), _ptr(rot), _c_int(rotary_dim if rot is not None else 0),
                     _ptr(slots), _ptr(k_cache), _ptr(v_cache), _c_int(tokens), _c_int(heads),
                     _c_int(kv_heads), _c_int(head_dim), _c_int(page_size), _stream())


def paged_attention_generic(q: torch.Tensor, q_stride: int, out: torch.Tensor, k_cache: torch.Tensor,
                            v_cache: torch.Tensor, block_tables: torch.Tensor, token_slot: torch.Tensor,
                            positions: torch.Tensor, heads: int, scale: float, window: int = 0) -> torch.Tensor:
    """Attention of every token over its request's pages, 32-bit arithmetic on CUDA cores.

    ``q`` may be a view into a wider buffer: row t starts ``q_stride`` elements after row t-1.
    ``block_tables`` has one row per state slot; ``token_slot[t]`` names the row of token t.
    """
    _check(q, "q", dense=False); _check(out, "out", q.dtype)
    _check(k_cache, "k_cache", q.dtype); _check(v_cache, "v_cache", q.dtype)
    _check(block_tables, "block_tables", torch.int32); _check(token_slot, "token_slot", torch.int32)
    _check(positions, "positions", torch.int32)
    pages, kv_heads, page_size, head_dim = k_cache.shape
    tokens = positions.numel()
    if v_cache.shape != k_cache.shape:
        raise KernelError("paged_attention: k and v caches differ in shape")
    if out.shape != (tokens, heads * head_dim) or token_slot.numel() != tokens:
        raise KernelError(f"paged_attention: out {tuple(out.shape)} / token_slot {token_slot.numel()} "
                          f"do not match {tokens} tokens of {heads}x{head_dim}")
    if block_tables.dim() != 2:
        raise KernelError("paged_attention: block_tables must be [slots, max_blocks]")
    _lib.core().call("mrun_paged_attention_generic", _ptr(q), _c_long(q_stride), _ptr(out), _ptr(k_cache),
                     _ptr(v_cache), dtype_code(q.dtype), _ptr(block_tables), _c_int(block_tables.shape[1]),
                     _ptr(token_slot), _ptr(positions), _c_int(tokens), _c_int(heads), _c_int(kv_heads),
                     _c_int(head_dim), _c_int(page_size), _c_long(pages * kv_heads * page_size),
                     _c_float(scale), _c_int(window), _stream())
    return out


GATE_FUNCTIONS = {"silu": 1, "gelu_tanh": 2}      # codes of the C ABI (MRUN_GATE_*); 0 = no gated epilogue


def gate_code(activation: str) -> int:
    try:
        return GATE_FUNCTIONS[activation]
    except KeyError:
        raise KernelError(f"no kernel has the gate function {activation!r} "
                          f"(known: {', '.join(sorted(GATE_FUNCTIONS))})") from None


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False, activation: str = "silu") -> torch.Tensor:
    """out = act(gate) * up.  Plain layout: gate_up[:, :I] are the gates, gate_up[:, I:] the ups.
    Interleaved: runs of eight gates followed by the eight ups of the same outputs."""
    _check(gate_up, "gate_up"); _check(out, "out", gate_up.dtype)
    tokens, inter = out.shape
    if gate_up.shape != (tokens, 2 * inter):
        raise KernelError(f"swiglu: gate_up {tuple(gate_up.shape)} vs out {tuple(out.shape)}")
    _lib.core().call("mrun_swiglu", _ptr(gate_up), _ptr(out), dtype_code(out.dtype), _c_int(tokens),
                     _c_int(inter), _c_int(8 if interleaved else 0), _c_int(gate_code(activation)), _stream())
    return out


def add_bias(y: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """y[t, n] += bias[n] in place; bias is float32."""
    _check(y, "y"); _check(bias, "bias", torch.float32)
    if y.dim() != 2 or bias.numel() != y.shape[1]:
        raise KernelError(f"add_bias: y {tuple(y.shape)} vs bias {tuple(bias.shape)}")
    _lib.core().call("mrun_add_bias", _ptr(y), dtype_code(y.dtype), _ptr(bias), _c_int(y.shape[0]),
                     _c_int(y.shape[1]), _stream())
    return y


SKINNY_ROWS = 16      # the decode GEMM takes up to this many rows


def skinny_ok(x, w: torch.Tensor) -> bool:
    """Whether the decode GEMM takes this product: few rows, bf16, K a multiple of 32."""
    if isinstance(x, NormedRows):
        x = x.xw
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[0] <= SKINNY_ROWS
            and x.shape[1] % 32 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0)


SUMS_UNIT = 2.0 ** -30        # a row's total of squares is a 64-bit integer in these units


class NormedRows:
    """The output of an RMSNorm whose row scale has not been applied yet: ``xw`` holds
    bf16(stream * norm weight) and ``sums`` (int64, a row each) each row's total of squares of the stream
    in units of 2^-30.  The decode GEMM takes it as its x and applies rsqrt(total / width + eps)
    to its own sums (so does the tcgen05 GEMM for 17 to 128 rows); :meth:`finish` makes the plain
    normed rows."""

    def __init__(self, xw: torch.Tensor, sums: torch.Tensor, eps: float):
        self.xw, self.sums, self.eps = xw, sums, float(eps)

    @property
    def shape(self):
        return self.xw.shape

    @property
    def dtype(self):
        return self.xw.dtype

    @property
    def device(self):
        return self.xw.device

    def finish(self) -> torch.Tensor:
        tokens, width = self.xw.shape
        out = torch.empty_like(self.xw)
        _lib.core().call("mrun_norm_finish", _ptr(self.xw), _ptr(self.sums), _c_float(self.eps), _ptr(out),
                         _c_int(tokens), _c_int(width), _stream())
        return out


class RowSums:
    """Zeroed per-row totals for the products of one step: one buffer per device, cleared once at
    the start of a step (:meth:`begin_step`: one memset, which a captured step replays) and handed
    out slice by slice, so that no product clears its own."""

    ROWS = 16 * 1024
    _arenas = {}

    @classmethod
    def begin_step(cls, device: torch.device) -> None:
        arena = cls._arenas.get(device)
        if arena is None:
            arena = cls._arenas[device] = [torch.zeros(cls.ROWS, dtype=torch.int64, device=device), 0]
        arena[0].zero_()                   # always: a captured step must clear what other steps left
        arena[1] = 0

    @classmethod
    def take(cls, device: torch.device, rows: int = 16) -> torch.Tensor:
        """The next ``rows`` zeroed totals of the step (a multiple of 16 is taken), or a fresh
        zeroed tensor outside a step or when the step has used all of its buffer."""
        rows = -(-rows // 16) * 16
        arena = cls._arenas.get(device)
        if arena is None or arena[1] + rows > cls.ROWS:
            return torch.zeros(rows, dtype=torch.int64, device=device)
        arena[1] += rows
        return arena[0][arena[1] - rows:arena[1]]


class PendingLinear:
    """A product ``x @ w.T`` that has not run yet: a part returns it as its output where the norm
    that follows can run it with the residual sum and the norm folded into its epilogue
    (:func:`linear_into_norm`).  :meth:`compute` runs it as an ordinary product."""

    def __init__(self, x: torch.Tensor, w: torch.Tensor):
        self.x, self.w = x, w

    @property
    def shape(self):
        return (self.x.shape[0], self.w.shape[0])

    def compute(self) -> torch.Tensor:
        return linear(self.x, self.w)


def _normed(x):
    """(rows, totals pointer, eps) of a product's x, which may be :class:`NormedRows`."""
    if isinstance(x, NormedRows):
        return x.xw, _ptr(x.sums), _c_float(x.eps)
    return x, _ptr(None), _c_float(0.0)


def gemm_skinny(x, w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16,
                swiglu_rows: bool = False, activation: str = "silu", rows: int = 0) -> torch.Tensor:
    """y = x @ w.T for at most 16 rows, reading w once at HBM speed.  ``swiglu_rows``: w holds gate
    and up rows interleaved in runs of eight and y = act(gate) * up has half as many columns.
    ``x`` may be :class:`NormedRows`.  ``w`` is a weight: the kernel asks for its first rows while
    the decode GEMM launched before it may still be running, so it must not be that launch's
    output (x, the stream and every output are touched only after that kernel has finished).
    ``rows``: the rows of w a block takes (8..16; 0: the count that fills the device most evenly)."""
    x, sums, eps = _normed(x)
    _check(x, "x", torch.bfloat16, dense=False); _check(w, "w", torch.bfloat16)
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise KernelError(f"gemm_skinny: x {tuple(x.shape)} vs w {tuple(w.shape)}")
    out = torch.empty((m, n // 2 if swiglu_rows else n), dtype=out_dtype, device=x.device)
    _lib.core().call("mrun_gemm_skinny", _ptr(x), _ptr(w), _ptr(out), dtype_code(out_dtype),
                     _c_int(gate_code(activation) if swiglu_rows else 0), _c_int(m), _c_int(n), _c_int(k),
                     _c_long(x.stride(0) if m > 1 else max(k, x.stride(0))), _c_long(out.shape[1]),
                     sums, eps, _ptr(None), _ptr(None), _ptr(None), _ptr(None), _c_int(rows), _stream())
    return out


def norm_fusable(pending, resid: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether :func:`linear_into_norm` takes this pending product and residual stream."""
    return (isinstance(pending, PendingLinear) and (skinny_ok(pending.x, pending.w) or tc5_ok(pending.x, pending.w))
            and resid.dtype == torch.float32 and resid.is_contiguous() and resid.shape == pending.shape
            and resid.shape[1] % 32 == 0 and weight.numel() == resid.shape[1])


def linear_into_norm(pending: PendingLinear, resid: torch.Tensor, weight: torch.Tensor, eps: float,
                     rows: int = 0) -> NormedRows:
    """resid += pending.x @ pending.w.T (32-bit, in place) and the RMSNorm of the new rows with
    ``weight``, as :class:`NormedRows`: one kernel (the decode GEMM up to 16 rows, the tcgen05
    GEMM up to 128)."""
    skinny = skinny_ok(pending.x, pending.w)
    x, in_sums, in_eps = _normed(pending.x)
    w = pending.w
    _check(x, "x", torch.bfloat16, dense=False); _check(w, "w", torch.bfloat16)
    _check(resid, "resid", torch.float32); _check(weight, "weight", torch.float32)
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k or resid.shape != (m, n) or weight.numel() != n:
        raise KernelError(f"linear_into_norm: x {tuple(x.shape)}, w {tuple(w.shape)}, resid {tuple(resid.shape)}, "
                          f"weight {tuple(weight.shape)}")
    xw = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    out_sums = RowSums.take(x.device, m)
    head = (_ptr(x), _ptr(w), _ptr(None), dtype_code(torch.bfloat16), _c_int(0), _c_int(m), _c_int(n), _c_int(k),
            _c_long(x.stride(0) if m > 1 else max(k, x.stride(0))), _c_long(n), in_sums, in_eps, _ptr(resid),
            _ptr(weight), _ptr(xw), _ptr(out_sums))
    if skinny:
        _lib.core().call("mrun_gemm_skinny", *head, _c_int(rows), _stream())
    else:
        _lib.core().call("mrun_gemm_tc5", *head, _c_int(0), _ptr(_tc5_status(x.device)), _stream())
    return NormedRows(xw, out_sums, eps)


def gemm_f32_nt(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x @ w.T in IEEE 32-bit with a fixed summation order.  x may have a row stride."""
    _check(x, "x", torch.float32, dense=False); _check(w, "w", torch.float32)
    if x.dim() != 2 or w.dim() != 2 or x.shape[1] != w.shape[1] or x.stride(1) != 1:
        raise KernelError(f"gemm_f32_nt: x {tuple(x.shape)} (strides {x.stride()}) vs w {tuple(w.shape)}")
    m, k = x.shape
    n = w.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=torch.float32, device=x.device)
    _check(out, "out", torch.float32)
    if out.shape != (m, n):
        raise KernelError(f"gemm_f32_nt: out is {tuple(out.shape)}, expected {(m, n)}")
    _lib.core().call("mrun_gemm_f32_nt", _ptr(x), _ptr(w), _ptr(out), _c_int(m), _c_int(n), _c_int(k),
                     _c_long(x.stride(0) if m > 1 else k), _c_long(n), _stream())
    return out


TC5_ROWS = 128            # the tcgen05 GEMM takes up to this many rows
# Whether products of 17 to 128 rows go to the tcgen05 GEMM.  Off: measured on B200 at the
# Qwen3-8B shapes it loses to the vendor library at 32, 64 and 128 rows (a kernel that holds tensor
# memory has its multiprocessor to itself, so nothing of its start overlaps the kernel before).
TC5_GEMM = False


def _tc5_status(device: torch.device) -> torch.Tensor:
    return status_word(device, "gemm_tc5", {1: "the TMA producer", 2: "the MMA issuer", 3: "the epilogue",
                                            4: "the exchange inside a cluster"})


def tc5_ok(x, w: torch.Tensor) -> bool:
    """Whether the tcgen05 GEMM takes this product: 17..128 rows, bf16, K a multiple of 64."""
    if isinstance(x, NormedRows):
        x = x.xw
    return (TC5_GEMM and isinstance(x, torch.Tensor) and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and x.dim() == 2 and SKINNY_ROWS < x.shape[0] <= TC5_ROWS
            and x.shape[1] % 64 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and w.is_contiguous() and w.data_ptr() % 16 == 0)


_sm_count = {}


def sm_count(device: torch.device) -> int:
    n = _sm_count.get(device)
    if n is None:
        n = _sm_count[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return n


def gemm_tc5(x, w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16, swiglu_rows: bool = False,
             activation: str = "silu", split: int = 0) -> torch.Tensor:
    """y = x @ w.T for 1..128 rows on the tcgen05 tensor cores (TMA-fed, accumulators in tensor
    memory, k split over thread-block clusters whose blocks exchange partial sums through
    distributed shared memory; ``split`` = 0 lets the library choose the cluster size).
    ``swiglu_rows`` as in :func:`gemm_skinny`; ``x`` may be :class:`NormedRows`; ``w`` is a weight
    (its first tiles are asked for before the kernel before has finished).  A wait inside the
    kernel that runs out sets the status word that :func:`tc5_check` reads."""
    x, sums, eps = _normed(x)
    _check(x, "x", torch.bfloat16, dense=False); _check(w, "w", torch.bfloat16)
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise KernelError(f"gemm_tc5: x {tuple(x.shape)} vs w {tuple(w.shape)}")
    out = torch.empty((m, n // 2 if swiglu_rows else n), dtype=out_dtype, device=x.device)
    _lib.core().call("mrun_gemm_tc5", _ptr(x), _ptr(w), _ptr(out), dtype_code(out_dtype),
                     _c_int(gate_code(activation) if swiglu_rows else 0), _c_int(m), _c_int(n), _c_int(k),
                     _c_long(x.stride(0) if m > 1 else max(k, x.stride(0))), _c_long(out.shape[1]),
                     sums, eps, _ptr(None), _ptr(None), _ptr(None), _ptr(None), _c_int(split),
                     _ptr(_tc5_status(x.device)), _stream())
    return out


_status_words = {}       # (device, kernel name) -> (int32[1] on the device, {code: role})


def status_word(device: torch.device, kernel: str, roles: dict) -> torch.Tensor:
    """The word a kernel with bounded waits reports into (zero = fine), one per device and kernel,
    never reallocated, so that captured graphs may keep its address.  :func:`tc5_check` reads it."""
    entry = _status_words.get((device, kernel))
    if entry is None:
        entry = _status_words[(device, kernel)] = (torch.zeros(1, dtype=torch.int32, device=device), dict(roles))
    return entry[0]


def tc5_check(device: Optional[torch.device] = None) -> None:
    """Raises if a tcgen05 kernel on the device gave up on a wait (and clears its status word)."""
    for (dev, kernel), (status, roles) in list(_status_words.items()):
        if device is not None and dev != device:
            continue
        code = int(status.item())
        if code:
            status.zero_()
            raise KernelError(f"{kernel}: {roles.get(code, 'a role')} waited longer than its budget on {dev}; "
                              f"the results of that call are invalid")


def linear(x, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
           bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x @ w.T (+ bias).  float32: this library's own IEEE kernel.  bfloat16 with at most 16
    rows (decode): this library's weight-streaming tensor-core kernel (``x`` may then be
    :class:`NormedRows`).  bfloat16 otherwise (prefill): the vendor GEMM library with 32-bit
    accumulation (the reference calls its array library's matmul for the same products and adds
    an optional bias after it, crates/mrun-engine/src/load.rs:294-306)."""
    if isinstance(x, NormedRows):
        if skinny_ok(x, w) or tc5_ok(x, w):
            y = (gemm_skinny if skinny_ok(x, w) else gemm_tc5)(x, w, out_dtype or torch.bfloat16)
            return y if bias is None else add_bias(y, bias)
        x = x.finish()
    if x.dtype == torch.float32:
        y = gemm_f32_nt(x, w)
    else:
        _check(x, "x", torch.bfloat16, dense=False); _check(w, "w", torch.bfloat16)
        if skinny_ok(x, w):
            y = gemm_skinny(x, w, out_dtype or torch.bfloat16)
        elif tc5_ok(x, w):
            y = gemm_tc5(x, w, out_dtype or torch.bfloat16)
        elif out_dtype is None or out_dtype == torch.bfloat16:
            y = torch.mm(x, w.t())
        else:
            y = torch.mm(x, w.t(), out_dtype=out_dtype)
    return y if bias is None else add_bias(y, bias)


def linear_or_pending(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None):
    """The last product of a part whose caller accepts a :class:`PendingLinear`: left pending in
    bfloat16 without a bias (the norm after it then runs it with the residual sum folded in: in
    the decode GEMM's epilogue up to 16 rows, as the vendor GEMM's accumulate-into-C above),
    computed otherwise."""
    if bias is None and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        return PendingLinear(x, w)
    return linear(x, w, bias=bias)


def accumulate_ok(pending, resid: torch.Tensor) -> bool:
    """Whether :func:`linear_add_into` takes this pending product and residual stream."""
    return (isinstance(pending, PendingLinear) and isinstance(pending.x, torch.Tensor) and not tc5_ok(pending.x, pending.w)
            and not skinny_ok(pending.x, pending.w)
            and pending.x.dtype == torch.bfloat16 and pending.w.dtype == torch.bfloat16 and pending.x.dim() == 2
            and resid.dtype == torch.float32 and resid.is_contiguous() and tuple(resid.shape) == tuple(pending.shape))


def linear_add_into(resid: torch.Tensor, pending: PendingLinear) -> torch.Tensor:
    """resid += pending.x @ pending.w.T in place: the vendor GEMM with bfloat16 operands, 32-bit
    accumulation and the 32-bit stream as its C and D, so that the product is never rounded to
    bfloat16, written and read again (prompt portions and decode batches above 16 rows)."""
    return torch.addmm(resid, pending.x, pending.w.t(), out_dtype=torch.float32, out=resid)


def sample(logits: torch.Tensor, out: torch.Tensor, temperature: Optional[torch.Tensor] = None,
           top_p: Optional[torch.Tensor] = None, top_k: Optional[torch.Tensor] = None,
           min_p: Optional[torch.Tensor] = None, keys: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of float32 logits; per-row parameter arrays, None = neutral."""
    _check(logits, "logits", torch.float32); _check(out, "out", torch.int32)
    rows, vocab = logits.shape
    for name, t, dt in (("temperature", temperature, torch.float32), ("top_p", top_p, torch.float32),
                        ("top_k", top_k, torch.int32), ("min_p", min_p, torch.float32),
                        ("keys", keys, torch.int64)):
        if t is not None:
            _check(t, name, dt)
            if t.numel() < rows:
                raise KernelError(f"sample: {name} has {t.numel()} entries for {rows} rows")
    if out.numel() < rows:
        raise KernelError(f"sample: out has {out.numel()} entries for {rows} rows")
    _lib.core().call("mrun_sample", _ptr(logits), _c_int(rows), _c_int(vocab), _ptr(temperature), _ptr(top_p),
                     _ptr(top_k), _ptr(min_p), _ptr(keys), _ptr(out), _stream())
    return out


def top_logprobs(logits: torch.Tensor, n: int):
    """(ids int32 [rows, n], log-probabilities float32 [rows, n]) of the n most likely tokens of
    each row of float32 logits, most likely first, ties by the smaller id."""
    _check(logits, "logits", torch.float32)
    rows, vocab = logits.shape
    n = max(1, min(int(n), vocab))
    ids = torch.empty((rows, n), dtype=torch.int32, device=logits.device)
    values = torch.empty((rows, n), dtype=torch.float32, device=logits.device)
    _lib.core().call("mrun_top_logprobs", _ptr(logits), _c_int(rows), _c_int(vocab), _c_int(n), _ptr(ids),
                     _ptr(values), _stream())
    return ids, values


def apply_token_mask(logits: torch.Tensor, rows: torch.Tensor, words: torch.Tensor, mask_vocab: torch.Tensor) -> None:
    """In place: logits[rows[m], i] = -inf wherever bit i of words[m] is clear or i >= mask_vocab[m].
    ``words``: int32 [masks, words a mask] (the bits of unsigned 32-bit words), 32 tokens a word."""
    _check(logits, "logits", torch.float32); _check(rows, "rows", torch.int32)
    _check(words, "words", torch.int32); _check(mask_vocab, "mask_vocab", torch.int32)
    masks = rows.numel()
    if words.dim() != 2 or words.shape[0] != masks or mask_vocab.numel() != masks:
        raise KernelError(f"apply_token_mask: {masks} rows, words {tuple(words.shape)}, {mask_vocab.numel()} vocabularies")
    _lib.core().call("mrun_apply_token_mask", _ptr(logits), _c_int(logits.shape[1]), _ptr(rows), _ptr(words),
                     _c_int(words.shape[1]), _ptr(mask_vocab), _c_int(masks), _stream())


def repetition_penalty(logits: torch.Tensor, recent: torch.Tensor, penalty: torch.Tensor) -> None:
    """In place: the logits of the ids in recent[row] (negative = empty) are penalised."""
    _check(logits, "logits", torch.float32); _check(recent, "recent", torch.int32)
    _check(penalty, "penalty", torch.float32)
    rows, vocab = logits.shape
    if recent.dim() != 2 or recent.shape[0] != rows or penalty.numel() < rows:
        raise KernelError(f"repetition_penalty: recent {tuple(recent.shape)}, penalty {penalty.numel()}, rows {rows}")
    _lib.core().call("mrun_repetition_penalty", _ptr(logits), _c_int(rows), _c_int(vocab), _ptr(recent),
                     _c_int(recent.shape[1]), _ptr(penalty), _stream())


def scatter_i32(dst: torch.Tensor, index: torch.Tensor, value: torch.Tensor) -> None:
    """dst.view(-1)[index[i]] = value[i] for int32 tensors."""
    _check(dst, "dst", torch.int32); _check(index, "index", torch.int32); _check(value, "value", torch.int32)
    if index.numel() != value.numel():
        raise KernelError("scatter_i32: index and value differ in length")
    _lib.core().call("mrun_scatter_i32", _ptr(dst), _ptr(index), _ptr(value), _c_int(index.numel()),
                     _c_long(dst.numel()), _stream())


def select_tokens(ids: torch.Tensor, previous: torch.Tensor, source: torch.Tensor) -> None:
    """ids[r] = previous[source[r]] where source[r] >= 0 (int32 tensors)."""
    _check(ids, "ids", torch.int32); _check(previous, "previous", torch.int32); _check(source, "source", torch.int32)
    if source.numel() != ids.numel():
        raise KernelError("select_tokens: one source per row is needed")
    _lib.core().call("mrun_select_tokens", _ptr(ids), _ptr(previous), _ptr(source), _c_int(ids.numel()),
                     _c_int(previous.numel()), _stream())

