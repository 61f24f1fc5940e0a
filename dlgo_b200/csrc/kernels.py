"""Python face of the CUDA entry points: tensors in, checked, launched on the
current stream.  Nothing here computes; a missing or failing library raises."""
from __future__ import annotations

import ctypes
from typing import Sequence, List, Optional

import torch

from . import build

F32, BF16 = 0, 1
_STATUS = {
    -1: "a size this kernel does not take",
    -2: "a pointer or stride that breaks an alignment rule",
    -3: "an element type this kernel does not take",
    -4: "a CUDA driver entry point could not be found",
    -5: "the kernel gave up a bounded wait on the device",
}


class KernelError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, not {dt}")


LAUNCHES = 0  # kernels of this package launched (or captured into a graph) so far

# Per-kernel timing a user can switch on (the reference's DLGO_PROFILE, examples/benchmark/main.go:24-28): while
# on, a CUDA event follows every launch of this package; the time between two consecutive events is the time of
# the later launch (kernels of one stream run in order).  Meant for runs without CUDA graphs.
_profile_events: Optional[list] = None


def profile_start() -> None:
    """Begin timing every launch of this package on the current stream."""
    global _profile_events
    first = torch.cuda.Event(enable_timing=True)
    first.record()
    _profile_events = [("", first)]


def profile_stop() -> List[tuple]:
    """End the timing; returns [(entry point, launches, total ms)] sorted by time, most first."""
    global _profile_events
    events, _profile_events = _profile_events or [], None
    if len(events) < 2:
        return []
    torch.cuda.synchronize()
    total: dict = {}
    for (_, before), (name, after) in zip(events, events[1:]):
        n, ms = total.get(name, (0, 0.0))
        total[name] = (n + 1, ms + before.elapsed_time(after))
    return sorted(((k, n, ms) for k, (n, ms) in total.items()), key=lambda r: -r[2])


def _check(status: int, what: str, launches: int = 1) -> None:
    global LAUNCHES
    if status == 0:
        LAUNCHES += launches
        if _profile_events is not None and launches > 0 and not torch.cuda.is_current_stream_capturing():
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            _profile_events.append((what, ev))
        return
    if status < 0:
        raise KernelError(f"{what}: refused ({_STATUS.get(status, status)})")
    raise KernelError(f"{what}: CUDA error {status} at launch")


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream() -> ctypes.c_void_p:
    # the raw handle of the current stream of the current device (a C call; current_stream() builds objects)
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice()))


def _need(t: torch.Tensor, dt: Optional[torch.dtype], name: str) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must live on the GPU (there is no CPU path)")
    if dt is not None and t.dtype != dt:
        raise KernelError(f"{name} must be {dt}, is {t.dtype}")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


def _lib(name: str) -> ctypes.CDLL:
    return build.load_library(name)


_i, _f, _p, _ll = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_longlong


# ------------------------------------------------------------------ elementwise
def embed(tokens: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None,
          copies: Optional[int] = None, scale: float = 1.0) -> torch.Tensor:
    """out[t, :] = table[tokens[t], :] * scale as fp32; with ``copies`` = s, out[t, c, :] for c < s (all equal)."""
    _need(tokens, torch.int32, "tokens")
    _need(table, None, "table")
    T, (V, d) = tokens.numel(), table.shape
    if out is None:
        out = torch.empty((T, d) if copies is None else (T, copies, d), dtype=torch.float32, device=table.device)
    _need(out, torch.float32, "out")
    st = _lib("elementwise").dlgo_embed(_ptr(tokens), _ptr(table), _i(dtype_code(table.dtype)), _ptr(out), _i(T), _i(d),
                                        _i(V), _i(copies or 1), _f(scale), _stream())
    _check(st, "embed")
    return out


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, out_dtype: torch.dtype,
            rows: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Row-wise RMSNorm of fp32 ``x``; with ``rows`` only those rows, in that order."""
    _need(x, torch.float32, "x")
    _need(w, torch.float32, "w")
    d = x.shape[-1]
    if w.numel() != d:
        raise KernelError(f"rmsnorm: weight has {w.numel()} elements, rows have {d}")
    R = x.shape[0] if rows is None else rows.numel()
    if rows is not None:
        _need(rows, torch.int32, "rows")
    if out is None:
        out = torch.empty((R, d), dtype=out_dtype, device=x.device)
    _need(out, out_dtype, "out")
    st = _lib("elementwise").dlgo_rmsnorm(_ptr(x), _ptr(w), _ptr(out), _i(dtype_code(out_dtype)), _ptr(rows), _i(R),
                                          _i(d), _f(eps), _stream())
    _check(st, "rmsnorm")
    return out


def add_rmsnorm(x: torch.Tensor, parts: torch.Tensor, w: Optional[torch.Tensor], eps: float,
                out_dtype: Optional[torch.dtype], rows: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """``x += parts.sum(0)`` (slices in order, in place), then RMSNorm of the new rows; with ``w`` None
    only the sum.  ``parts`` is [S, T, d] fp32."""
    _need(x, torch.float32, "x")
    if parts.dtype != torch.float32 or parts.dim() != 3 or parts.stride(2) != 1 or parts.stride(1) != x.shape[1]:
        raise KernelError("add_rmsnorm: parts must be [S, T, d] float32 with contiguous rows")
    d = x.shape[-1]
    R = x.shape[0] if rows is None else rows.numel()
    out = None
    if w is not None:
        _need(w, torch.float32, "w")
        out = torch.empty((R, d), dtype=out_dtype, device=x.device)
    if rows is not None:
        _need(rows, torch.int32, "rows")
    st = _lib("elementwise").dlgo_add_rmsnorm(
        _ptr(x), _ptr(parts), _i(parts.shape[0]), _ll(parts.stride(0)), _ptr(w), _ptr(out),
        _i(dtype_code(out_dtype) if w is not None else F32), _ptr(rows), _i(R), _i(d), _f(eps), _stream())
    _check(st, "add_rmsnorm")
    return out


def swiglu(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None, block: Optional[int] = None) -> torch.Tensor:
    """[T, 2F] (gate | up) -> [T, F].  ``block``: gate and up columns alternate in blocks of this many columns
    (a divisor of F) instead of two halves."""
    _need(gate_up, None, "gate_up")
    T, F2 = gate_up.shape
    F = F2 // 2
    if out is None:
        out = torch.empty((T, F), dtype=gate_up.dtype, device=gate_up.device)
    _need(out, gate_up.dtype, "out")
    if block is None or block == F:
        st = _lib("elementwise").dlgo_swiglu(_ptr(gate_up), _ptr(out), _i(dtype_code(gate_up.dtype)), _i(T), _i(F),
                                             _stream())
    else:
        if block <= 0 or F % block:
            raise KernelError(f"swiglu: blocks of {block} columns do not divide {F}")
        st = _lib("elementwise").dlgo_swiglu_blocks(_ptr(gate_up), _ptr(out), _i(dtype_code(gate_up.dtype)), _i(T),
                                                    _i(F), _i(block), _stream())
    _check(st, "swiglu")
    return out


# ----------------------------------------------- residual streams and their norms
NORM_NONE, NORM_RMS, NORM_DYT = 0, 1, 2
ACT_NONE, ACT_RELU2, ACT_SILU, ACT_GELU_TANH = 0, 1, 2, 3
ACT_TANH = 4           # (the elementwise bias_act only)
MOE_ACT_SWIGLU = 4     # (moe_gemm_tc only: W's rows in blocks of MOE_SWIGLU_BLOCK gate rows and as many up rows)
MOE_SWIGLU_BLOCK = 16
GATE_SIGMOID, GATE_SILU = 0, 1
MAX_STREAMS = 8


def streams_step(X: torch.Tensor, *, y: Optional[torch.Tensor] = None, y_bias: Optional[torch.Tensor] = None,
                 mix: Optional[torch.Tensor] = None, write: Optional[torch.Tensor] = None, clear_y: bool = False,
                 read: Optional[torch.Tensor] = None, norm_kind: int = NORM_NONE,
                 norm_w: Optional[torch.Tensor] = None, norm_b: Optional[torch.Tensor] = None,
                 norm_alpha: Optional[torch.Tensor] = None, eps: float = 0.0,
                 out_dtype: Optional[torch.dtype] = None, rows: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """One hand-over on residual streams ``X`` [T, s, d] (fp32, in place).

    Write part (with ``y`` [T, d] fp32): ``X[t, q] = sum_r mix[r, q] X[t, r] + write[q] * (y[t] + y_bias)``,
    all streams at once from the old values; ``clear_y`` leaves zeros in ``y``.  Read part (with
    ``out_dtype``): ``u = sum_r read[r] X[t, r]`` (``read`` None: the plain sum) through the norm
    (``NORM_DYT``: tanh(alpha u) w + b; ``NORM_RMS``; ``NORM_NONE``: u itself) into a new [R, d] tensor;
    ``rows`` picks the rows to read (read part only)."""
    _need(X, torch.float32, "X")
    if X.dim() != 3:
        raise KernelError("streams_step: X must be [tokens, streams, hidden]")
    T, s, d = X.shape
    if s > MAX_STREAMS:
        raise KernelError(f"streams_step: at most {MAX_STREAMS} streams, got {s}")
    if y is not None:
        _need(y, torch.float32, "y")
        if tuple(y.shape) != (T, d) or mix is None or write is None or rows is not None:
            raise KernelError("streams_step: the write part needs y [T, d], mix, write, and no row selection")
        _need(mix, torch.float32, "mix")
        _need(write, torch.float32, "write")
        if tuple(mix.shape) != (s, s) or write.numel() != s:
            raise KernelError("streams_step: mix must be [s, s] and write [s]")
    for n, t in (("y_bias", y_bias), ("read", read), ("norm_w", norm_w), ("norm_b", norm_b), ("norm_alpha", norm_alpha)):
        if t is not None:
            _need(t, torch.float32, n)
    if rows is not None:
        _need(rows, torch.int32, "rows")
    R = T if rows is None else rows.numel()
    out = None
    if out_dtype is not None:
        if norm_kind != NORM_NONE and (norm_w is None or norm_w.numel() != d):
            raise KernelError("streams_step: the norm needs a weight of the hidden size")
        if norm_kind == NORM_DYT and norm_alpha is None:
            raise KernelError("streams_step: Dynamic Tanh needs alpha")
        out = torch.empty((R, d), dtype=out_dtype, device=X.device)
    elif y is None:
        return None
    st = _lib("streams").dlgo_streams_step(
        _ptr(X), _i(T), _i(s), _i(d), _ptr(y), _ptr(y_bias), _ptr(mix), _ptr(write), _i(1 if clear_y else 0),
        _ptr(read), _i(norm_kind), _ptr(norm_w), _ptr(norm_b), _ptr(norm_alpha), _f(eps), _ptr(out),
        _i(dtype_code(out_dtype) if out_dtype is not None else F32), _ptr(rows), _i(R), _stream())
    _check(st, "streams_step")
    return out


def bias_act(z: torch.Tensor, bias: Optional[torch.Tensor], act: int, out_dtype: torch.dtype,
             in_place: bool = False) -> torch.Tensor:
    """``act(z + bias)`` for fp32 ``z`` [T, n] (unit inner stride), into ``out_dtype``; ``in_place`` (fp32) writes z."""
    if z.dtype != torch.float32 or z.dim() != 2 or z.stride(1) != 1:
        raise KernelError("bias_act: z must be 2-D float32 with unit inner stride")
    T, n = z.shape
    if bias is not None:
        _need(bias, torch.float32, "bias")
        if bias.numel() != n:
            raise KernelError(f"bias_act: bias has {bias.numel()} elements, rows have {n}")
    if in_place:
        if out_dtype != torch.float32:
            raise KernelError("bias_act: in place only in float32")
        out = z
    else:
        out = torch.empty((T, n), dtype=out_dtype, device=z.device)
    st = _lib("streams").dlgo_bias_act(_ptr(z), _i(z.stride(0)), _ptr(bias), _ptr(out), _i(dtype_code(out_dtype)),
                                       _i(out.stride(0)), _i(T), _i(n), _i(act), _stream())
    _check(st, "bias_act")
    return out


def gated_rmsnorm(o: torch.Tensor, gate: torch.Tensor, w: Optional[torch.Tensor], eps: float, out_dtype: torch.dtype,
                  group: Optional[int] = None, gate_act: int = GATE_SIGMOID, scale: float = 1.0) -> torch.Tensor:
    """``rms(o) * w * g(gate) * scale`` row by row; o and gate are fp32 [T, n] views with unit inner stride.
    ``group``: the mean square is taken over each run of ``group`` neighbours (a head) on its own instead of the
    whole row; ``w`` None: no weight; ``gate_act``: sigmoid or silu of the gate."""
    for n_, t in (("o", o), ("gate", gate)):
        if t.dtype != torch.float32 or t.dim() != 2 or t.stride(1) != 1:
            raise KernelError(f"gated_rmsnorm: {n_} must be 2-D float32 with unit inner stride")
    T, n = o.shape
    if w is not None:
        _need(w, torch.float32, "w")
    if tuple(gate.shape) != (T, n) or (w is not None and w.numel() != n):
        raise KernelError("gated_rmsnorm: shapes differ")
    group = n if group is None else int(group)
    if group <= 0 or n % group:
        raise KernelError(f"gated_rmsnorm: rows of {n} do not split into groups of {group}")
    out = torch.empty((T, n), dtype=out_dtype, device=o.device)
    st = _lib("streams").dlgo_gated_rmsnorm(_ptr(o), _i(o.stride(0)), _ptr(gate), _i(gate.stride(0)), _ptr(w), _ptr(out),
                                            _i(dtype_code(out_dtype)), _i(T), _i(n), _f(eps), _i(group), _i(gate_act),
                                            _f(scale), _stream())
    _check(st, "gated_rmsnorm")
    return out


# ------------------------------------------------------------- latent attention
def latent_norm_append(proj: torch.Tensor, kv_off: int, kv_rank: int, w_kv: torch.Tensor, q_off: int, q_rank: int,
                       w_q: Optional[torch.Tensor], eps: float, token_pos: torch.Tensor, token_seq: torch.Tensor,
                       seq_slot: torch.Tensor, page_table: torch.Tensor, pages: torch.Tensor,
                       write_cache: bool = True) -> Optional[torch.Tensor]:
    """RMS norms of the latents in fp32 ``proj`` [T, ld]: columns ``kv_off ...`` go (normed, times ``w_kv``) to
    the paged cache ``pages`` [n, 1, page, kv_rank] at each token's position; with ``q_rank`` > 0 columns
    ``q_off ...`` come back normed (times ``w_q``) as [T, q_rank] in the cache's type."""
    if proj.dtype != torch.float32 or proj.dim() != 2 or proj.stride(1) != 1:
        raise KernelError("latent_norm_append: proj must be 2-D float32 with unit inner stride")
    _need(w_kv, torch.float32, "w_kv")
    _need(pages, None, "pages")
    for n, t in (("token_pos", token_pos), ("token_seq", token_seq), ("seq_slot", seq_slot), ("page_table", page_table)):
        _need(t, torch.int32, n)
    T = proj.shape[0]
    if pages.shape[-1] != kv_rank or w_kv.numel() != kv_rank:
        raise KernelError("latent_norm_append: the cache's rows and the norm weight must have kv_rank elements")
    cq = None
    if q_rank > 0:
        _need(w_q, torch.float32, "w_q")
        cq = torch.empty((T, q_rank), dtype=pages.dtype, device=proj.device)
    st = _lib("latent_attention").dlgo_latent_norm_append(
        _ptr(proj), _i(proj.stride(0)), _i(T), _i(kv_off), _i(kv_rank), _ptr(w_kv), _i(q_off), _i(q_rank), _ptr(w_q),
        _ptr(cq), _f(eps), _ptr(token_pos), _ptr(token_seq), _ptr(seq_slot), _ptr(page_table), _i(page_table.shape[1]),
        _ptr(pages), _i(dtype_code(pages.dtype)), _i(pages.shape[-2]), _i(1 if write_cache else 0), _stream())
    _check(st, "latent_norm_append")
    return cq


def latent_rope_append(proj: torch.Tensor, kv_off: int, kv_rank: int, w_kv: torch.Tensor, q_off: int, num_heads: int,
                       q_head: int, rope: int, freq: torch.Tensor, amplitude: float, eps: float,
                       token_pos: torch.Tensor, token_seq: torch.Tensor, seq_slot: torch.Tensor,
                       page_table: torch.Tensor, pages: torch.Tensor, write_cache: bool = True) -> None:
    """Latents with a rotated key part, from fp32 ``proj`` [T, ld]: columns ``kv_off ...`` hold ``kv_rank`` numbers
    that are RMS-normed (times ``w_kv``) and ``rope`` numbers that turn with the position in neighbouring pairs
    (angle ``float(pos) * freq[i]``, cosine and sine times ``amplitude``); both go to the token's row of the paged
    cache ``pages`` [n, 1, page, kv_rank + rope].  The queries at ``q_off`` ([heads, q_head] per token) turn IN
    PLACE in the last ``rope`` numbers of every head."""
    if proj.dtype != torch.float32 or proj.dim() != 2 or proj.stride(1) != 1:
        raise KernelError("latent_rope_append: proj must be 2-D float32 with unit inner stride")
    _need(w_kv, torch.float32, "w_kv")
    _need(freq, torch.float32, "freq")
    _need(pages, None, "pages")
    for n, t in (("token_pos", token_pos), ("token_seq", token_seq), ("seq_slot", seq_slot), ("page_table", page_table)):
        _need(t, torch.int32, n)
    if pages.shape[-1] != kv_rank + rope or w_kv.numel() != kv_rank or freq.numel() != rope // 2:
        raise KernelError("latent_rope_append: cache rows hold kv_rank + rope numbers; rope / 2 frequencies")
    if q_off + num_heads * q_head > proj.shape[1] or kv_off + kv_rank + rope > proj.shape[1]:
        raise KernelError("latent_rope_append: the columns named lie outside proj")
    st = _lib("latent_attention").dlgo_latent_rope_append(
        _ptr(proj), _i(proj.stride(0)), _i(proj.shape[0]), _i(kv_off), _i(kv_rank), _ptr(w_kv), _i(q_off),
        _i(num_heads), _i(q_head), _i(rope), _ptr(freq), _f(amplitude), _f(eps), _ptr(token_pos), _ptr(token_seq),
        _ptr(seq_slot), _ptr(page_table), _i(page_table.shape[1]), _ptr(pages), _i(dtype_code(pages.dtype)),
        _i(pages.shape[-2]), _i(1 if write_cache else 0), _stream())
    _check(st, "latent_rope_append")


def latent_attention(q: torch.Tensor, w_k: torch.Tensor, w_v: torch.Tensor, sink: Optional[torch.Tensor],
                     pages: torch.Tensor, page_table: torch.Tensor, seq_slot: torch.Tensor, token_seq: torch.Tensor,
                     token_pos: torch.Tensor, num_heads: int, qk_dim: int, v_dim: int, scale: float,
                     window: int = 0) -> torch.Tensor:
    """Causal attention of packed tokens over cached latents ``pages`` [n, 1, page, rank]: per head
    ``softmax((Wk^T q) . c * scale) c`` carried out through ``Wv``; ``q`` [T, >= H*qk_dim] (fp32 or the cache's
    type), ``w_k`` [H*qk_dim, rank], ``w_v`` [H*v_dim, rank] in the cache's type.  Returns [T, H*v_dim]."""
    _need(pages, None, "pages")
    _need(w_k, pages.dtype, "w_k")
    _need(w_v, pages.dtype, "w_v")
    if q.dtype not in (torch.float32, pages.dtype) or q.dim() != 2 or q.stride(1) != 1:
        raise KernelError("latent_attention: q must be 2-D, float32 or the cache's type, with unit inner stride")
    if sink is not None:
        _need(sink, torch.float32, "sink")
    for n, t in (("page_table", page_table), ("seq_slot", seq_slot), ("token_seq", token_seq), ("token_pos", token_pos)):
        _need(t, torch.int32, n)
    T, rank = q.shape[0], pages.shape[-1]
    if tuple(w_k.shape) != (num_heads * qk_dim, rank) or tuple(w_v.shape) != (num_heads * v_dim, rank):
        raise KernelError("latent_attention: the up-projections do not fit heads, sizes and rank")
    out = torch.empty((T, num_heads * v_dim), dtype=pages.dtype, device=q.device)
    st = _lib("latent_attention").dlgo_latent_attention(
        _ptr(q), _i(1 if q.dtype == torch.float32 else 0), _i(q.stride(0)), _ptr(w_k), _ptr(w_v), _ptr(sink),
        _ptr(pages), _i(dtype_code(pages.dtype)), _ptr(page_table), _i(page_table.shape[1]), _i(pages.shape[-2]),
        _ptr(seq_slot), _ptr(token_seq), _ptr(token_pos), _ptr(out), _i(out.stride(0)), _i(T), _i(num_heads),
        _i(qk_dim), _i(v_dim), _i(rank), _f(scale), _i(window), _stream())
    _check(st, "latent_attention")
    return out


def latent_attention_few_takes(dtype: torch.dtype, rank: int) -> bool:
    """Whether the three-launch kernels take this rank (a latent row is read 16 bytes at a time)."""
    v = 4 if dtype == torch.float32 else 8
    return rank % v == 0 and rank <= 256 * v


def latent_attention_few(q: torch.Tensor, w_k: torch.Tensor, w_v: torch.Tensor, sink: Optional[torch.Tensor],
                         pages: torch.Tensor, page_table: torch.Tensor, seq_slot: torch.Tensor,
                         token_seq: torch.Tensor, token_pos: torch.Tensor, num_heads: int, qk_dim: int, v_dim: int,
                         scale: float, window: int, n_slices: int, q_lat: torch.Tensor,
                         parts: torch.Tensor) -> torch.Tensor:
    """:func:`latent_attention` for steps of few tokens, as three launches that each fill the GPU: the queries
    into latent space (``q_lat`` [T, H, rank] fp32 scratch), the softmax over every token's visible latents cut
    into ``n_slices`` slices (``parts`` [T, H, n_slices, rank + 2] fp32 scratch), and the slices' meeting, the
    sink and the way out through Wv."""
    _need(pages, None, "pages")
    _need(w_k, pages.dtype, "w_k")
    _need(w_v, pages.dtype, "w_v")
    if q.dtype not in (torch.float32, pages.dtype) or q.dim() != 2 or q.stride(1) != 1:
        raise KernelError("latent_attention_few: q must be 2-D, float32 or the cache's type, with unit inner stride")
    if sink is not None:
        _need(sink, torch.float32, "sink")
    for n, t in (("page_table", page_table), ("seq_slot", seq_slot), ("token_seq", token_seq), ("token_pos", token_pos)):
        _need(t, torch.int32, n)
    T, rank = q.shape[0], pages.shape[-1]
    if tuple(w_k.shape) != (num_heads * qk_dim, rank) or tuple(w_v.shape) != (num_heads * v_dim, rank):
        raise KernelError("latent_attention_few: the up-projections do not fit heads, sizes and rank")
    if q_lat.dtype != torch.float32 or q_lat.numel() < T * num_heads * rank or parts.dtype != torch.float32 or \
            parts.numel() < T * num_heads * n_slices * (rank + 2):
        raise KernelError("latent_attention_few: scratch too small")
    out = torch.empty((T, num_heads * v_dim), dtype=pages.dtype, device=q.device)
    st = _lib("latent_attention").dlgo_latent_attention_few(
        _ptr(q), _i(1 if q.dtype == torch.float32 else 0), _i(q.stride(0)), _ptr(w_k), _ptr(w_v), _ptr(sink),
        _ptr(pages), _i(dtype_code(pages.dtype)), _ptr(page_table), _i(page_table.shape[1]), _i(pages.shape[-2]),
        _ptr(seq_slot), _ptr(token_seq), _ptr(token_pos), _ptr(out), _i(out.stride(0)), _i(T), _i(num_heads),
        _i(qk_dim), _i(v_dim), _i(rank), _f(scale), _i(window), _i(n_slices), _ptr(q_lat), _ptr(parts), _stream())
    _check(st, "latent_attention_few", 3)
    return out


def latent_attention_tiles_takes(dtype: torch.dtype, num_heads: int, rank: int) -> bool:
    """Whether the few-token kernels that serve all heads of a token from one tile of keys take these sizes."""
    if dtype not in (torch.float32, torch.bfloat16):
        return False
    return bool(_lib("latent_attention").dlgo_latent_attention_tiles_takes(_i(dtype_code(dtype)), _i(num_heads), _i(rank)))


def latent_attention_tiles(q: torch.Tensor, w_k: torch.Tensor, w_v: torch.Tensor, sink: Optional[torch.Tensor],
                           pages: torch.Tensor, page_table: torch.Tensor, seq_slot: torch.Tensor,
                           token_seq: torch.Tensor, token_pos: torch.Tensor, num_heads: int, qk_dim: int, v_dim: int,
                           scale: float, window: int, n_slices: int, q_lat: torch.Tensor,
                           parts: torch.Tensor) -> torch.Tensor:
    """:func:`latent_attention_few` with every latent row read once per token instead of once per head: four
    launches (queries into latent space; tiles of 32 keys in shared memory serving all heads, a block per token and
    slice of the keys; the slices' meeting; out through ``w_v``).  Same arguments and scratch."""
    _need(pages, None, "pages")
    _need(w_k, pages.dtype, "w_k")
    _need(w_v, pages.dtype, "w_v")
    if q.dtype not in (torch.float32, pages.dtype) or q.dim() != 2 or q.stride(1) != 1:
        raise KernelError("latent_attention_tiles: q must be 2-D, float32 or the cache's type, with unit inner stride")
    if sink is not None:
        _need(sink, torch.float32, "sink")
    for n, t in (("page_table", page_table), ("seq_slot", seq_slot), ("token_seq", token_seq), ("token_pos", token_pos)):
        _need(t, torch.int32, n)
    T, rank = q.shape[0], pages.shape[-1]
    if tuple(w_k.shape) != (num_heads * qk_dim, rank) or tuple(w_v.shape) != (num_heads * v_dim, rank):
        raise KernelError("latent_attention_tiles: the up-projections do not fit heads, sizes and rank")
    if q_lat.dtype != torch.float32 or q_lat.numel() < T * num_heads * rank or parts.dtype != torch.float32 or \
            parts.numel() < T * num_heads * n_slices * (rank + 2):
        raise KernelError("latent_attention_tiles: scratch too small")
    out = torch.empty((T, num_heads * v_dim), dtype=pages.dtype, device=q.device)
    st = _lib("latent_attention").dlgo_latent_attention_tiles(
        _ptr(q), _i(1 if q.dtype == torch.float32 else 0), _i(q.stride(0)), _ptr(w_k), _ptr(w_v), _ptr(sink),
        _ptr(pages), _i(dtype_code(pages.dtype)), _ptr(page_table), _i(page_table.shape[1]), _i(pages.shape[-2]),
        _ptr(seq_slot), _ptr(token_seq), _ptr(token_pos), _ptr(out), _i(out.stride(0)), _i(T), _i(num_heads),
        _i(qk_dim), _i(v_dim), _i(rank), _f(scale), _i(window), _i(n_slices), _ptr(q_lat), _ptr(parts), _stream())
    _check(st, "latent_attention_tiles", 4)
    return out


def latent_gather(pages: torch.Tensor, page_table: torch.Tensor, tmp_pages: torch.Tensor, n_tmp: int,
                  seq_slot: torch.Tensor) -> torch.Tensor:
    """Rows [n_tmp * page, rank] of the cached latents of the pages listed in ``tmp_pages`` [n_tmp, 3]
    (sequence of the step, its page index, written rows); rows that are not written are zero."""
    _need(pages, None, "pages")
    for n, t in (("page_table", page_table), ("tmp_pages", tmp_pages), ("seq_slot", seq_slot)):
        _need(t, torch.int32, n)
    page_size, rank = pages.shape[-2], pages.shape[-1]
    out = torch.empty((n_tmp * page_size, rank), dtype=pages.dtype, device=pages.device)
    st = _lib("latent_attention").dlgo_latent_gather(_ptr(pages), _i(dtype_code(pages.dtype)), _ptr(page_table),
                                                     _i(page_table.shape[1]), _i(page_size), _ptr(tmp_pages), _i(n_tmp),
                                                     _ptr(seq_slot), _ptr(out), _i(rank), _stream())
    _check(st, "latent_gather")
    return out


def attention_prefill_tc_rows(q: torch.Tensor, kv: torch.Tensor, k_col: int, v_col: int, n_pages: int,
                              page_table: torch.Tensor, tiles: torch.Tensor, seq_rows: torch.Tensor,
                              token_pos: torch.Tensor, num_heads: int, head_dim: int, scale: float, window: int = 0,
                              sink: Optional[torch.Tensor] = None, split: bool = True) -> torch.Tensor:
    """Prompt attention on the tensor cores over keys and values made for the step: ``kv`` [n_pages * 64, ld]
    bf16 holds every head's keys from column ``k_col`` and values from ``v_col`` (head h at + h * head_dim),
    row = page * 64 + key; ``page_table`` [sequences of the step, pages] maps a sequence's page index to a page
    of these rows; ``seq_rows`` [sequences] names each sequence's row of that table.  ``sink`` [heads] joins the
    denominator.  ``split``: probabilities enter P V as two bfloat16 terms.  Returns [T, heads * head_dim]."""
    for n, t in (("q", q), ("kv", kv)):
        if t.dtype != torch.bfloat16 or t.dim() != 2 or t.stride(1) != 1:
            raise KernelError(f"attention_prefill_tc_rows: {n} must be 2-D bfloat16 with unit inner stride")
    for n, t in (("page_table", page_table), ("tiles", tiles), ("seq_rows", seq_rows), ("token_pos", token_pos)):
        _need(t, torch.int32, n)
    if sink is not None:
        _need(sink, torch.float32, "sink")
    T = q.shape[0]
    out = torch.empty((T, num_heads * head_dim), dtype=torch.bfloat16, device=q.device)
    es = kv.element_size()
    st = _lib("attention_prefill_tc").dlgo_attention_prefill_tc_rows(
        _ptr(q), _i(T), _i(q.stride(0)), _p(kv.data_ptr() + k_col * es), _p(kv.data_ptr() + v_col * es), _i(n_pages),
        _i(kv.stride(0)), _ptr(page_table), _i(page_table.shape[1]), _ptr(tiles), _i(tiles.shape[0]), _ptr(seq_rows),
        _ptr(token_pos), _ptr(out), _i(out.stride(0)), _i(num_heads), _i(head_dim), _i(window), _f(scale), _ptr(sink),
        _i(1 if split else 0), _stream())
    _check(st, "attention_prefill_tc_rows")
    return out


# ---------------------------------------------------------- lightning attention
def lightning_scan(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, tiles: torch.Tensor, n_seqs: int,
                   seq_slot: torch.Tensor, decay: torch.Tensor, state: torch.Tensor, num_heads: int, qk_dim: int,
                   v_dim: int, silu: bool = True) -> torch.Tensor:
    """Decayed linear attention of packed tokens, sequence by sequence in token order, continuing each
    sequence's fp32 state ``state`` [slots, H, qk_dim, v_dim] (in place).  ``proj`` [T, ld] fp32 holds the
    q, k and v projections at the given column offsets (with ``silu``, silu is applied here); ``tiles`` [n_seqs, 3] lists
    (sequence, first packed token, count).  Returns fp32 [T, H*v_dim]."""
    if proj.dtype != torch.float32 or proj.dim() != 2 or proj.stride(1) != 1:
        raise KernelError("lightning_scan: proj must be 2-D float32 with unit inner stride")
    _need(tiles, torch.int32, "tiles")
    _need(seq_slot, torch.int32, "seq_slot")
    _need(decay, torch.float32, "decay")
    _need(state, torch.float32, "state")
    if tuple(state.shape[1:]) != (num_heads, qk_dim, v_dim) or decay.numel() != num_heads:
        raise KernelError("lightning_scan: state must be [slots, heads, qk_dim, v_dim] and decay [heads]")
    T = proj.shape[0]
    out = torch.empty((T, num_heads * v_dim), dtype=torch.float32, device=proj.device)
    st = _lib("lightning").dlgo_lightning_scan(_ptr(proj), _i(proj.stride(0)), _i(q_off), _i(k_off), _i(v_off),
                                               _ptr(tiles), _i(n_seqs), _ptr(seq_slot), _ptr(decay), _ptr(state),
                                               _ptr(out), _i(out.stride(0)), _i(num_heads), _i(qk_dim), _i(v_dim),
                                               _i(1 if silu else 0), _stream())
    _check(st, "lightning_scan")
    return out


def lightning_segments_takes(qk_dim: int) -> bool:
    """Whether the segment kernels (the state's columns in registers, segments side by side) take this qk size."""
    return qk_dim in (32, 64, 128)


def lightning_segments(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, tiles: torch.Tensor, n_tiles: int,
                       direct: bool, seq_slot: torch.Tensor, decay: torch.Tensor, state: torch.Tensor,
                       scratch: Optional[torch.Tensor], num_heads: int, qk_dim: int, v_dim: int,
                       silu: bool = True) -> torch.Tensor:
    """:func:`lightning_scan` with every sequence's tokens cut into consecutive segments (``tiles`` [n_tiles, 3],
    a sequence's segments in token order) that run side by side: each first computes its own end state from
    zero, then starts from the decayed sum of what lies before it.  ``direct``: one segment per sequence (no
    first pass); else ``scratch`` holds 2 * n_tiles * H * qk_dim * v_dim floats."""
    if proj.dtype != torch.float32 or proj.dim() != 2 or proj.stride(1) != 1:
        raise KernelError("lightning_segments: proj must be 2-D float32 with unit inner stride")
    _need(tiles, torch.int32, "tiles")
    _need(seq_slot, torch.int32, "seq_slot")
    _need(decay, torch.float32, "decay")
    _need(state, torch.float32, "state")
    if tuple(state.shape[1:]) != (num_heads, qk_dim, v_dim) or decay.numel() != num_heads:
        raise KernelError("lightning_segments: state must be [slots, heads, qk_dim, v_dim] and decay [heads]")
    if not direct:
        need = 2 * n_tiles * num_heads * qk_dim * v_dim
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
            raise KernelError(f"lightning_segments: {n_tiles} segments need {need} floats of scratch")
    T = proj.shape[0]
    out = torch.empty((T, num_heads * v_dim), dtype=torch.float32, device=proj.device)
    st = _lib("lightning").dlgo_lightning_segments(
        _ptr(proj), _i(proj.stride(0)), _i(q_off), _i(k_off), _i(v_off), _ptr(tiles), _i(n_tiles),
        _i(1 if direct else 0), _ptr(seq_slot), _ptr(decay), _ptr(state), _ptr(scratch), _ptr(out), _i(out.stride(0)),
        _i(num_heads), _i(qk_dim), _i(v_dim), _i(1 if silu else 0), _stream())
    _check(st, "lightning_segments", 1 if direct else 2)
    return out


def rotate_scale(proj: torch.Tensor, q_off: int, k_off: int, freq: Optional[torch.Tensor], rot: int,
                 token_pos: torch.Tensor, num_heads: int, qk_dim: int, k_scale: float) -> None:
    """In place on the fp32 projection rows ``proj`` [T, ld]: the first ``rot`` numbers of every q and k head
    (``num_heads`` heads of ``qk_dim`` at the column offsets) turn in pairs (i, i + rot/2) by the angle
    ``float(position) * freq[i]``; keys are then multiplied by ``k_scale``."""
    if proj.dtype != torch.float32 or proj.dim() != 2 or proj.stride(1) != 1:
        raise KernelError("rotate_scale: proj must be 2-D float32 with unit inner stride")
    _need(token_pos, torch.int32, "token_pos")
    if rot:
        _need(freq, torch.float32, "freq")
        if freq.numel() != rot // 2:
            raise KernelError("rotate_scale: one frequency per rotated pair")
    hi = max(q_off, k_off) + num_heads * qk_dim
    if hi > proj.shape[1] or abs(q_off - k_off) < num_heads * qk_dim:
        raise KernelError("rotate_scale: q and k columns must lie inside the rows and apart")
    st = _lib("lightning").dlgo_rotate_scale(_ptr(proj), _i(proj.stride(0)), _i(q_off), _i(k_off),
                                             _ptr(freq if rot else None), _i(rot), _ptr(token_pos), _i(proj.shape[0]),
                                             _i(num_heads), _i(qk_dim), _f(k_scale), _stream())
    _check(st, "rotate_scale")


# ------------------------------------------------------------------ time mixing
def token_shift_mix(x: torch.Tensor, mu: torch.Tensor, token_seq: torch.Tensor, seq_slot: torch.Tensor,
                    state: torch.Tensor, prev_off: int, out_dtype: torch.dtype) -> torch.Tensor:
    """Blends of every token's input with the previous token's: ``out[s, t] = x[t] + (x[t-1] - x[t]) * mu[s]`` for the
    fp32 rows ``x`` [T, d] and ``mu`` [n, d]; a sequence's first token of the step reads its predecessor from the
    sequence's row of ``state`` [slots, row] (fp32) at column ``prev_off``.  Returns [n, T, d] in ``out_dtype``."""
    _need(x, torch.float32, "x")
    _need(mu, torch.float32, "mu")
    _need(token_seq, torch.int32, "token_seq")
    _need(seq_slot, torch.int32, "seq_slot")
    T, d = x.shape
    if state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 or prev_off + d > state.shape[1]:
        raise KernelError("token_shift_mix: state must be 2-D float32 rows that hold d numbers at prev_off")
    if mu.dim() != 2 or mu.shape[1] != d:
        raise KernelError("token_shift_mix: mu must be [n, d]")
    out = torch.empty((mu.shape[0], T, d), dtype=out_dtype, device=x.device)
    st = _lib("timemix").dlgo_token_shift_mix(_ptr(x), _ptr(mu), _i(mu.shape[0]), _ptr(token_seq), _ptr(seq_slot),
                                              _ptr(state), _ll(state.stride(0)), _i(prev_off), _ptr(out),
                                              _i(dtype_code(out_dtype)), _i(T), _i(d), _stream())
    _check(st, "token_shift_mix")
    return out


def wkv_segments_takes(head_dim: int) -> bool:
    """Whether the segment kernels (the state's columns in registers, segments side by side) take this head size."""
    return head_dim in (32, 64, 128)


def wkv_scratch_floats(n_tiles: int, num_heads: int, head_dim: int) -> int:
    return n_tiles * num_heads * (2 * head_dim * head_dim + head_dim)


def wkv(r: torch.Tensor, k: torch.Tensor, v: torch.Tensor, zw: torch.Tensor, w0: torch.Tensor, u: torch.Tensor,
        tiles: torch.Tensor, n_tiles: int, direct: bool, segments: bool, seq_slot: torch.Tensor, state: torch.Tensor,
        x: Optional[torch.Tensor], scratch: Optional[torch.Tensor], num_heads: int, head_dim: int) -> torch.Tensor:
    """The recurrence with a per-token, per-channel decay ``w = exp(-exp(zw + w0))`` and the bonus ``u`` for the
    current token, over packed tokens, continuing each sequence's state.  r, k, v, zw: fp32 [T, H * n]
    (contiguous); w0, u: fp32 [H * n]; ``state`` [slots, row] fp32 rows of H * n * n state numbers followed, when
    ``x`` (fp32 [T, d]) is given, by the d numbers of the sequence's last input, which is stored there.
    ``segments``: ``tiles`` cuts sequences into segments that run side by side (head sizes 32 / 64 / 128; unless
    ``direct``, with ``scratch`` of :func:`wkv_scratch_floats`); else one row of ``tiles`` per sequence, any head
    size.  Returns fp32 [T, H * n]."""
    T = r.shape[0]
    ld = num_heads * head_dim
    for n_, t in (("r", r), ("k", k), ("v", v), ("zw", zw)):
        _need(t, torch.float32, n_)
        if tuple(t.shape) != (T, ld):
            raise KernelError(f"wkv: {n_} must be [{T}, {ld}]")
    for n_, t in (("w0", w0), ("u", u)):
        _need(t, torch.float32, n_)
        if t.numel() != ld:
            raise KernelError(f"wkv: {n_} must hold one number per head and channel")
    _need(tiles, torch.int32, "tiles")
    _need(seq_slot, torch.int32, "seq_slot")
    d = 0
    if x is not None:
        _need(x, torch.float32, "x")
        d = x.shape[1]
    if state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 or \
            state.shape[1] < ld * head_dim + d:
        raise KernelError("wkv: state must be 2-D float32 rows of heads * n * n (+ d) numbers")
    out = torch.empty((T, ld), dtype=torch.float32, device=r.device)
    lib = _lib("timemix")
    if segments:
        if not direct:
            need = wkv_scratch_floats(n_tiles, num_heads, head_dim)
            if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
                raise KernelError(f"wkv: {n_tiles} segments need {need} floats of scratch")
        st = lib.dlgo_wkv_segments(_ptr(r), _ptr(k), _ptr(v), _ptr(zw), _i(ld), _ptr(w0), _ptr(u), _ptr(tiles),
                                   _i(n_tiles), _i(1 if direct else 0), _ptr(seq_slot), _ptr(state),
                                   _ll(state.stride(0)), _ptr(x), _i(d), _ptr(scratch), _ptr(out), _i(num_heads),
                                   _i(head_dim), _stream())
        _check(st, "wkv_segments", 1 if direct else 2)
    else:
        st = lib.dlgo_wkv_scan(_ptr(r), _ptr(k), _ptr(v), _ptr(zw), _i(ld), _ptr(w0), _ptr(u), _ptr(tiles), _i(n_tiles),
                               _ptr(seq_slot), _ptr(state), _ll(state.stride(0)), _ptr(x), _i(d), _ptr(out),
                               _i(num_heads), _i(head_dim), _stream())
        _check(st, "wkv_scan")
    return out


# ------------------------------------------------------ layer norm, norm of a sublayer's result
NORMED_LAYER, NORMED_RMS = 0, 1


def layernorm_rows(x: torch.Tensor, w: torch.Tensor, eps: float, out_dtype: torch.dtype,
                   rows: Optional[torch.Tensor] = None, kind: int = NORMED_LAYER, in_place: bool = False) -> torch.Tensor:
    """``(x - mean) / sqrt(var + eps) * w`` (or, ``kind`` NORMED_RMS, ``x / sqrt(mean(x^2) + eps) * w``) of the fp32
    rows ``x`` [T, d], or of the rows listed in ``rows`` (int32), in ``out_dtype``; ``in_place``: x is rewritten."""
    _need(x, torch.float32, "x")
    _need(w, torch.float32, "w")
    T, d = x.shape
    if w.numel() != d:
        raise KernelError("layernorm_rows: one weight per channel")
    if rows is not None:
        _need(rows, torch.int32, "rows")
    R = T if rows is None else rows.numel()
    if in_place:
        if rows is not None or out_dtype != torch.float32:
            raise KernelError("layernorm_rows: in place only for all rows in float32")
        out = x
    else:
        out = torch.empty((R, d), dtype=out_dtype, device=x.device)
    st = _lib("layernorm").dlgo_layernorm_rows(_ptr(x), _ptr(w), _ptr(out), _i(dtype_code(out_dtype)), _ptr(rows), _i(R),
                                               _i(d), _i(kind), _f(eps), _stream())
    _check(st, "layernorm_rows")
    return out


def add_normed(x: torch.Tensor, y: torch.Tensor, w: torch.Tensor, eps: float, act_dtype: Optional[torch.dtype],
               kind: int = NORMED_LAYER, clear_y: bool = True) -> Optional[torch.Tensor]:
    """``x <- x + norm(y) * w`` on the fp32 residual stream ``x`` [T, d], in place (``y`` fp32 [T, d], left zero with
    ``clear_y``); returns the new rows in ``act_dtype`` (None: no copy)."""
    _need(x, torch.float32, "x")
    _need(y, torch.float32, "y")
    _need(w, torch.float32, "w")
    T, d = x.shape
    if tuple(y.shape) != (T, d) or w.numel() != d:
        raise KernelError("add_normed: y must have x's shape and w one element per channel")
    act = None if act_dtype is None else torch.empty((T, d), dtype=act_dtype, device=x.device)
    st = _lib("layernorm").dlgo_add_normed(_ptr(x), _ptr(y), _ptr(w), _ptr(act),
                                           _i(dtype_code(act_dtype or torch.float32)), _i(T), _i(d), _i(kind), _f(eps),
                                           _i(1 if clear_y else 0), _stream())
    _check(st, "add_normed")
    return act


# --------------------------------------- queries and keys normed as a whole, cache append, head gates
def wholenorm_append(proj: torch.Tensor, w_q: Optional[torch.Tensor], w_k: Optional[torch.Tensor], eps: float,
                     token_pos: torch.Tensor, token_seq: torch.Tensor, seq_slot: torch.Tensor,
                     page_table: torch.Tensor, kpages: torch.Tensor, vpages: torch.Tensor, num_heads: int,
                     num_kv_heads: int, qk_dim: int, v_dim: int, has_gate: bool, gate_scale: float, write_cache: bool,
                     clear: bool, out_dtype: torch.dtype):
    """From the fp32 rows ``proj`` [T, >= Hq qk + Hkv (qk + v) (+ Hq)]: queries and keys each divided by the root mean
    square over ALL their numbers and multiplied by ``w_q`` / ``w_k`` (None: left as they are); keys and values
    appended to their pages ``[pages, kv_heads, page_size, hd]`` with zeros behind a head's own numbers; returns
    (queries [T, Hq * hd] in ``out_dtype``, gates [T, Hq] fp32 = sigmoid(logit) * gate_scale, or None)."""
    if proj.dtype != torch.float32 or proj.dim() != 2 or proj.stride(1) != 1:
        raise KernelError("wholenorm_append: proj must be 2-D float32 with unit inner stride")
    for n_, t in (("w_q", w_q), ("w_k", w_k)):
        if t is not None:
            _need(t, torch.float32, n_)
    if (w_q is not None and w_q.numel() != num_heads * qk_dim) or (w_k is not None and w_k.numel() != num_kv_heads * qk_dim):
        raise KernelError("wholenorm_append: the norm weights must cover the whole projections")
    for n_, t in (("token_pos", token_pos), ("token_seq", token_seq), ("seq_slot", seq_slot), ("page_table", page_table)):
        _need(t, torch.int32, n_)
    _need(kpages, out_dtype, "kpages")
    _need(vpages, out_dtype, "vpages")
    P, hkv, ps, hd = kpages.shape
    if hkv != num_kv_heads or tuple(vpages.shape) != tuple(kpages.shape):
        raise KernelError("wholenorm_append: pages must be [pages, kv_heads, page_size, hd], keys and values alike")
    T = proj.shape[0]
    q = torch.empty((T, num_heads * hd), dtype=out_dtype, device=proj.device)
    gate = torch.empty((T, num_heads), dtype=torch.float32, device=proj.device) if has_gate else None
    st = _lib("wholenorm_append").dlgo_wholenorm_append(
        _ptr(proj), _i(proj.stride(0)), _ptr(w_q), _ptr(w_k), _f(eps), _ptr(token_pos), _ptr(token_seq), _ptr(seq_slot),
        _ptr(page_table), _i(page_table.shape[1]), _ptr(kpages), _ptr(vpages), _ptr(q), _ptr(gate),
        _i(dtype_code(out_dtype)), _i(T), _i(num_heads), _i(num_kv_heads), _i(qk_dim), _i(v_dim), _i(hd), _i(ps),
        _i(1 if has_gate else 0), _f(gate_scale), _i(1 if write_cache else 0), _i(1 if clear else 0), _stream())
    _check(st, "wholenorm_append")
    return q, gate


CONV_MAX_TAPS = 8


def conv_rope_append(proj: torch.Tensor, bias: Optional[torch.Tensor], taps: Optional[torch.Tensor],
                     state: Optional[torch.Tensor], freq: Optional[torch.Tensor], rot: int, amplitude: float,
                     token_pos: torch.Tensor, token_seq: torch.Tensor, seq_slot: torch.Tensor,
                     page_table: torch.Tensor, kpages: torch.Tensor, vpages: torch.Tensor, num_heads: int,
                     num_kv_heads: int, qk_dim: int, v_dim: int, tiles: Optional[torch.Tensor], n_tiles: int,
                     write_cache: bool = True, one_token_each: bool = False, clear_proj: bool = False) -> torch.Tensor:
    """From the fp32 result ``proj`` [T, >= C] of a q | k | v projection (heads of ``qk_dim``, ``qk_dim`` and ``v_dim``
    numbers, C in all): ``+ bias`` [C]; a causal convolution over time per channel with ``taps`` [C, n] (the last
    tap on the token itself), whose reach before the step's first token of a sequence is read from ``state``
    [slots, n - 1, C] (fp32; afterwards it holds the sequence's last n - 1 projected rows: a second launch over
    ``tiles`` [n_tiles, 3], one row (sequence, first packed token, count) per sequence of the step, which a step
    whose sequences bring one token each, ``one_token_each``, may do without; such a step may also hand ``proj`` as
    a sum to be left zero, ``clear_proj``, where :func:`conv_rope_append_clears` says so); rotation of the first ``rot`` numbers
    of every q and k head in neighbouring pairs (angle ``float(pos) * freq[i]``, cosine and sine times
    ``amplitude``); k and v into their page rows, q returned [T, heads * hd] in the cache's type, heads laid out
    ``hd`` = the pages' head size wide with zeros behind their own numbers."""
    if proj.dtype != torch.float32 or proj.dim() != 2 or proj.stride(1) != 1:
        raise KernelError("conv_rope_append: proj must be 2-D float32 with unit inner stride")
    C = (num_heads + num_kv_heads) * qk_dim + num_kv_heads * v_dim
    hd = kpages.shape[-1]
    if proj.shape[1] < C or kpages.shape != vpages.shape or kpages.dtype != vpages.dtype:
        raise KernelError("conv_rope_append: proj has too few columns, or keys and values differ in shape")
    n_taps = 1
    for n, t, numel in (("bias", bias, C), ("freq", freq, rot // 2)):
        if t is not None:
            _need(t, torch.float32, n)
            if t.numel() != numel:
                raise KernelError(f"conv_rope_append: {n} has {t.numel()} numbers, wanted {numel}")
    if taps is not None:
        _need(taps, torch.float32, "taps")
        if taps.dim() != 2 or taps.shape[0] != C or not 1 <= taps.shape[1] <= CONV_MAX_TAPS:
            raise KernelError(f"conv_rope_append: taps must be [channels, 1..{CONV_MAX_TAPS}]")
        n_taps = taps.shape[1]
    if n_taps > 1:
        if state is None or tiles is None:
            raise KernelError("conv_rope_append: a convolution needs the sequences' state and the step's sequences")
        _need(state, torch.float32, "state")
        _need(tiles, torch.int32, "tiles")
        if state[0].numel() != (n_taps - 1) * C:
            raise KernelError("conv_rope_append: a state row holds (taps - 1) * channels numbers")
    for n, t in (("token_pos", token_pos), ("token_seq", token_seq), ("seq_slot", seq_slot), ("page_table", page_table)):
        _need(t, torch.int32, n)
    _need(kpages, None, "kpages")
    _need(vpages, None, "vpages")
    T = proj.shape[0]
    q = torch.empty((T, num_heads * hd), dtype=kpages.dtype, device=proj.device)
    st = _lib("conv_rope_append").dlgo_conv_rope_append(
        _ptr(proj), _i(proj.stride(0)), _i(T), _ptr(bias), _ptr(taps), _i(n_taps), _ptr(state), _ptr(freq), _i(rot),
        _f(amplitude), _ptr(token_pos), _ptr(token_seq), _ptr(seq_slot), _ptr(page_table), _i(page_table.shape[1]),
        _i(kpages.shape[-2]), _ptr(q), _ptr(kpages), _ptr(vpages), _i(dtype_code(kpages.dtype)), _i(num_heads),
        _i(num_kv_heads), _i(qk_dim), _i(v_dim), _i(hd), _i(1 if write_cache else 0), _ptr(tiles), _i(n_tiles),
        _i(1 if one_token_each else 0), _i(1 if clear_proj else 0), _stream())
    _check(st, "conv_rope_append", 2 if n_taps > 1 else 1)
    return q


def conv_rope_append_clears(qk_dim: int, v_dim: int, head_dim: int, ld: int, n_taps: int) -> bool:
    """Whether :func:`conv_rope_append` can clear ``proj`` (row stride ``ld``) behind it in a step of one token a sequence."""
    return bool(_lib("conv_rope_append").dlgo_conv_rope_append_clears(_i(qk_dim), _i(v_dim), _i(head_dim), _i(ld), _i(n_taps)))


def gated_residual(x: torch.Tensor, y: Optional[torch.Tensor], gate: Optional[torch.Tensor],
                   gate_bias: Optional[torch.Tensor], *, y_bias: Optional[torch.Tensor] = None, history: Optional[torch.Tensor] = None, depth: int = 0,
                   average: Optional[torch.Tensor] = None, norm_w: Optional[torch.Tensor] = None, eps: float = 0.0,
                   out_dtype: Optional[torch.dtype] = None, clear_y: bool = True,
                   clear_gate: bool = False) -> Optional[torch.Tensor]:
    """``x += (y + y_bias) * sigmoid(gate + gate_bias)`` on the fp32 stream ``x`` [T, d] (``gate`` None: ``x += y +
    y_bias``; ``y`` None: nothing is added; ``y_bias`` [d]: a bias the sublayer left to this pass), ``y`` left zero
    (and ``gate`` with ``clear_gate``: a sum that a contraction's slices add themselves into); with ``depth`` = n > 0, x is then stored as entry n - 1 of ``history``
    [>= n, T, d] and replaced by ``sum_j average[j] * history[j]`` over j < n; with ``norm_w``, the RMS norm of the
    new x times ``norm_w`` comes back in ``out_dtype``."""
    _need(x, torch.float32, "x")
    T, d = x.shape
    if y is not None:
        _need(y, torch.float32, "y")
        if tuple(y.shape) != (T, d):
            raise KernelError("gated_residual: y must have x's shape")
    ldg = 0
    if gate is not None:
        if gate.dtype != torch.float32 or gate.dim() != 2 or gate.stride(1) != 1 or gate.shape[0] != T or gate.shape[1] < d:
            raise KernelError("gated_residual: gate must be fp32 [T, >= d] with unit inner stride")
        ldg = gate.stride(0)
    for n, t in (("gate_bias", gate_bias), ("y_bias", y_bias)):
        if t is not None:
            _need(t, torch.float32, n)
            if t.numel() != d:
                raise KernelError(f"gated_residual: {n} must hold {d} numbers")
    stride = 0
    if depth > 0:
        _need(history, torch.float32, "history")
        _need(average, torch.float32, "average")
        if history.dim() != 3 or history.shape[0] < depth or tuple(history.shape[1:]) != (T, d) or average.numel() != depth:
            raise KernelError("gated_residual: history must be [>= depth, T, d] and average hold depth numbers")
        stride = history.stride(0)
    out = None
    if norm_w is not None:
        _need(norm_w, torch.float32, "norm_w")
        out = torch.empty((T, d), dtype=out_dtype, device=x.device)
    st = _lib("gated_residual").dlgo_gated_residual(
        _ptr(x), _ptr(y), _ptr(y_bias), _ptr(gate), _i(ldg), _ptr(gate_bias), _ptr(history), _ll(stride), _i(depth), _ptr(average),
        _ptr(norm_w), _f(eps), _ptr(out), _i(dtype_code(out_dtype) if out is not None else F32), _i(T), _i(d),
        _i(1 if clear_y else 0), _i(1 if clear_gate else 0), _stream())
    _check(st, "gated_residual")
    return out


def scale_softcap(logits: torch.Tensor, scale: float, cap: float) -> torch.Tensor:
    """``logits <- cap * tanh(logits * scale / cap)`` in place on contiguous fp32 (``cap`` <= 0: ``logits * scale``)."""
    _need(logits, torch.float32, "logits")
    st = _lib("gated_residual").dlgo_scale_softcap(_ptr(logits), _ll(logits.numel()), _f(scale), _f(cap), _stream())
    _check(st, "scale_softcap")
    return logits


def scale_heads(a: torch.Tensor, gate: torch.Tensor, head_dim: int) -> torch.Tensor:
    """``a[t, h, :] *= gate[t, h]`` in place for ``a`` [T, H * head_dim] (float32 or bfloat16) and fp32 ``gate`` [T, H]."""
    _need(a, None, "a")
    _need(gate, torch.float32, "gate")
    T, n = a.shape
    H = gate.shape[1]
    if n != H * head_dim or gate.shape[0] != T:
        raise KernelError("scale_heads: a must be [T, H * head_dim] and gate [T, H]")
    st = _lib("wholenorm_append").dlgo_scale_heads(_ptr(a), _ptr(gate), _i(dtype_code(a.dtype)), _i(T), _i(H),
                                                   _i(head_dim), _stream())
    _check(st, "scale_heads")
    return a


# ------------------------------------------------------------------------ GEMM
EPI_STORE, EPI_STORE_F32, EPI_ADD_F32 = 0, 1, 2


def gemm_simt(x: torch.Tensor, w: torch.Tensor, epilogue: int = EPI_STORE,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x[M, K] . w[N, K]^T on the fp32 pipes; epilogue stores (x's type or fp32) or adds into fp32 ``out``."""
    _need(w, x.dtype, "w")
    if x.dim() != 2 or x.stride(1) != 1:
        raise KernelError("gemm: x must be 2-D with unit inner stride")
    M, K = x.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelError(f"gemm: x has K={K}, w has K={K2}")
    if out is None:
        if epilogue == EPI_ADD_F32:
            raise KernelError("gemm: the add epilogue needs the tensor to add into")
        out = torch.empty((M, N), dtype=x.dtype if epilogue == EPI_STORE else torch.float32, device=x.device)
    if out.dim() != 2 or out.stride(1) != 1 or out.shape != (M, N):
        raise KernelError(f"gemm: out must be [{M}, {N}] with unit inner stride")
    want = x.dtype if epilogue == EPI_STORE else torch.float32
    if out.dtype != want:
        raise KernelError(f"gemm: out must be {want}")
    st = _lib("gemm_simt").dlgo_gemm_simt(_ptr(x), _ptr(w), _ptr(out), _i(dtype_code(x.dtype)), _i(M), _i(N), _i(K),
                                          _i(x.stride(0)), _i(w.stride(0)), _i(out.stride(0)), _i(epilogue), _stream())
    _check(st, "gemm_simt")
    return out


# --------------------------------------------------------------- rope + append
def rope_append(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, token_pos: torch.Tensor,
                token_seq: torch.Tensor, seq_slot: torch.Tensor, page_table: torch.Tensor,
                kpages: torch.Tensor, vpages: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                rotary_dim: int, interleaved: bool, write_cache: bool = True,
                parts: Optional[torch.Tensor] = None, clear_parts: bool = False) -> None:
    """Rotate q (in place) and k, and store k and v at their positions' pages.

    ``parts`` ([S, T, ld] fp32): the projection's unsummed K-slices; they are added here and ``qkv``
    only receives the rotated q.  ``clear_parts``: the kernel leaves zeros where it read
    ``parts`` (a sum that the projection adds into and that must be zero again for the next step)."""
    _need(qkv, None, "qkv")
    _need(cos, torch.float32, "cos")
    _need(sin, torch.float32, "sin")
    for n, t in (("token_pos", token_pos), ("token_seq", token_seq), ("seq_slot", seq_slot), ("page_table", page_table)):
        _need(t, torch.int32, n)
    _need(kpages, qkv.dtype, "kpages")
    _need(vpages, qkv.dtype, "vpages")
    T = qkv.shape[0]
    page_size = kpages.shape[-2]
    st = _lib("rope_append").dlgo_rope_append(
        _ptr(qkv), _i(dtype_code(qkv.dtype)), _i(T), _i(qkv.stride(0)), _ptr(cos), _ptr(sin), _ptr(token_pos),
        _ptr(token_seq), _ptr(seq_slot), _ptr(page_table), _i(page_table.shape[1]), _ptr(kpages), _ptr(vpages),
        _i(num_heads), _i(num_kv_heads), _i(head_dim), _i(rotary_dim), _i(page_size), _i(1 if interleaved else 0),
        _i(1 if write_cache else 0), _ptr(parts), _i(0 if parts is None else parts.shape[0]),
        _ll(0 if parts is None else parts.stride(0)), _i(1 if clear_parts else 0), _stream())
    _check(st, "rope_append")


# ------------------------------------------- head norm + rotation from frequencies + append
def headnorm_rope_append(proj: torch.Tensor, bias: Optional[torch.Tensor], w_q: Optional[torch.Tensor],
                         w_k: Optional[torch.Tensor], eps: float, freq: Optional[torch.Tensor], rotary_dim: int,
                         token_pos: torch.Tensor, token_seq: torch.Tensor, seq_slot: torch.Tensor,
                         page_table: torch.Tensor, kpages: torch.Tensor, vpages: torch.Tensor, num_heads: int,
                         num_kv_heads: int, head_dim: int, values_from_keys: bool, write_cache: bool = True,
                         clear: bool = False, norm_dim: Optional[int] = None) -> torch.Tensor:
    """From the fp32 projection ``proj`` [T, ld] (query heads, key heads and, unless ``values_from_keys``, value
    heads; ``bias`` fp32 per column added first): per-head RMS norm of queries and keys with the weights ``w_q`` /
    ``w_k`` (None: no norm), rotation of the first ``rotary_dim`` numbers of each head (pairs (i, i + rotary_dim/2))
    by the fp32 angle ``float(position) * freq[i]``, keys and values stored at their positions' pages (with
    ``values_from_keys`` a value is its key as projected, before norm and rotation).  Returns the queries
    [T, heads * head_dim] in the cache's type.  ``clear`` leaves zeros in ``proj``.  ``norm_dim``: the number of
    entries the head norm's mean runs over (heads laid out with trailing zeros; default ``head_dim``)."""
    if proj.dtype != torch.float32 or proj.dim() != 2 or proj.stride(1) != 1:
        raise KernelError("headnorm_rope_append: proj must be 2-D float32 with unit inner stride")
    for n, t in (("bias", bias), ("w_q", w_q), ("w_k", w_k), ("freq", freq)):
        if t is not None:
            _need(t, torch.float32, n)
    for n, t in (("token_pos", token_pos), ("token_seq", token_seq), ("seq_slot", seq_slot), ("page_table", page_table)):
        _need(t, torch.int32, n)
    _need(kpages, None, "kpages")
    _need(vpages, kpages.dtype, "vpages")
    T = proj.shape[0]
    cols = (num_heads + (1 if values_from_keys else 2) * num_kv_heads) * head_dim
    if proj.shape[1] < cols or (bias is not None and bias.numel() != cols):
        raise KernelError(f"headnorm_rope_append: the projection (and its bias) must have {cols} columns")
    for n, t in (("w_q", w_q), ("w_k", w_k)):
        if t is not None and t.numel() != head_dim:
            raise KernelError(f"headnorm_rope_append: {n} must have head_dim elements")
    if rotary_dim and (freq is None or freq.numel() != rotary_dim // 2):
        raise KernelError("headnorm_rope_append: one frequency per rotated pair")
    if kpages.shape[-1] != head_dim or kpages.shape[-3] != num_kv_heads:
        raise KernelError("headnorm_rope_append: the cache's pages do not fit the heads")
    q = torch.empty((T, num_heads * head_dim), dtype=kpages.dtype, device=proj.device)
    st = _lib("headnorm_rope").dlgo_headnorm_rope_append(
        _ptr(proj), _i(proj.stride(0)), _ptr(bias), _ptr(w_q), _ptr(w_k), _f(eps), _ptr(freq), _i(rotary_dim),
        _ptr(token_pos), _ptr(token_seq), _ptr(seq_slot), _ptr(page_table), _i(page_table.shape[1]), _ptr(kpages),
        _ptr(vpages), _ptr(q), _i(dtype_code(kpages.dtype)), _i(T), _i(num_heads), _i(num_kv_heads), _i(head_dim),
        _i(kpages.shape[-2]), _i(1 if values_from_keys else 0), _i(1 if write_cache else 0), _i(1 if clear else 0),
        _i(norm_dim or head_dim), _stream())
    _check(st, "headnorm_rope_append")
    return q


# ------------------------------------------------------- norm after the residual sum
def scaled_add_rmsnorm(x: torch.Tensor, y: Optional[torch.Tensor], layer_scale: Optional[torch.Tensor],
                       w: Optional[torch.Tensor], skip: float, eps: float, act_dtype: Optional[torch.dtype],
                       clear_y: bool = True) -> Optional[torch.Tensor]:
    """``x <- rms(skip * x + layer_scale * y) * w`` on the fp32 residual stream ``x`` [T, d], in place (``y`` fp32
    [T, d], left zero with ``clear_y``); returns the new rows in ``act_dtype`` (None: no copy).  With ``y`` and ``w``
    None only the copy is made."""
    _need(x, torch.float32, "x")
    T, d = x.shape
    for n, t in (("y", y), ("layer_scale", layer_scale), ("w", w)):
        if t is not None:
            _need(t, torch.float32, n)
    if y is not None and tuple(y.shape) != (T, d):
        raise KernelError("scaled_add_rmsnorm: y must have x's shape")
    for n, t in (("layer_scale", layer_scale), ("w", w)):
        if t is not None and t.numel() != d:
            raise KernelError(f"scaled_add_rmsnorm: {n} must have one element per channel")
    act = None if act_dtype is None else torch.empty((T, d), dtype=act_dtype, device=x.device)
    st = _lib("postnorm").dlgo_scaled_add_rmsnorm(
        _ptr(x), _ptr(y), _ptr(layer_scale), _ptr(w), _ptr(act), _i(dtype_code(act_dtype or torch.float32)), _i(T),
        _i(d), _f(skip), _f(eps), _i(1 if clear_y else 0), _stream())
    _check(st, "scaled_add_rmsnorm")
    return act


# ------------------------------------------------------------------ routed experts
MOE_FEW_ROWS, MOE_TILE_ROWS, MOE_TC_ROWS, MOE_TC_PAIR_ROWS = 8, 64, 128, 256      # rows per tile of the grouped contractions


def moe_router(h: torch.Tensor, w_router: torch.Tensor, correction: Optional[torch.Tensor], n_outputs: int,
               has_gate: bool, top: int, groups: int, keep: int, sigmoid_scores: bool = False,
               renormalize: bool = False, plan: Optional[tuple] = None, logit_bias: Optional[torch.Tensor] = None):
    """Router of a mixture of experts for ``h`` [T, d]: returns (chosen outputs [T, top] int32, their weights
    [T, top] fp32, gate [T] fp32 or None, plan).  ``w_router`` is fp32 [n_outputs (+ 1 gate row), d].
    ``plan`` = (experts that hold tensors, rows per tile): the :class:`MoEPlan` of :func:`moe_plan` is made as well,
    in the choice's own launch where the step has few tokens, else by a launch of its own; without it None."""
    _need(w_router, torch.float32, "w_router")
    if h.dim() != 2 or h.stride(1) != 1:
        raise KernelError("moe_router: h must be 2-D with unit inner stride")
    T, d = h.shape
    rows = n_outputs + (1 if has_gate else 0)
    if tuple(w_router.shape) != (rows, d):
        raise KernelError(f"moe_router: the router's weight must be [{rows}, {d}]")
    if correction is not None:
        _need(correction, torch.float32, "correction")
        if correction.numel() != n_outputs:
            raise KernelError("moe_router: one correction per router output")
    if logit_bias is not None:
        _need(logit_bias, torch.float32, "logit_bias")
        if logit_bias.numel() != n_outputs:
            raise KernelError("moe_router: one logit bias per router output")
    idx = torch.empty((T, top), dtype=torch.int32, device=h.device)
    wt = torch.empty((T, top), dtype=torch.float32, device=h.device)
    gate = torch.empty((T,), dtype=torch.float32, device=h.device) if has_gate else None
    z = torch.empty((T, rows), dtype=torch.float32, device=h.device)
    p = _empty_plan(T * top, plan[0], plan[1], h.device) if plan is not None and plan[0] > 0 else None
    fused = ctypes.c_int(0)
    st = _lib("moe").dlgo_moe_router(
        _ptr(h), _i(dtype_code(h.dtype)), _i(h.stride(0)), _ptr(w_router), _ptr(correction), _ptr(logit_bias), _ptr(z), _ptr(idx),
        _ptr(wt), _ptr(gate), _i(T), _i(d), _i(n_outputs), _i(1 if has_gate else 0), _i(top), _i(groups), _i(keep),
        _i(1 if sigmoid_scores else 0), _i(1 if renormalize else 0), _i(plan[0] if p is not None else 0),
        _i(plan[1] if p is not None else 0), _ptr(p.offsets if p is not None else None),
        _ptr(p.sorted_pair if p is not None else None), _ptr(p.tile_expert if p is not None else None),
        _ptr(p.tile_row0 if p is not None else None), _ptr(p.n_tiles if p is not None else None),
        _i(p.max_tiles if p is not None else 0), ctypes.byref(fused), _stream())
    _check(st, "moe_router", 2)
    if p is not None and not fused.value:
        p = moe_plan(idx, plan[0], plan[1], p)
    return idx, wt, gate, p


class MoEPlan:
    """Device-side lists of a step's (token, choice) pairs sorted by expert (see :func:`moe_plan`)."""

    __slots__ = ("offsets", "sorted_pair", "tile_expert", "tile_row0", "n_tiles", "max_tiles", "tile_rows", "pairs")


def _empty_plan(pairs: int, n_experts: int, tile_rows: int, device: torch.device) -> MoEPlan:
    p = MoEPlan()
    p.pairs, p.tile_rows = pairs, tile_rows
    p.max_tiles = (pairs + tile_rows - 1) // tile_rows + n_experts
    buf = torch.empty((n_experts + 1 + pairs + 2 * p.max_tiles + 1,), dtype=torch.int32, device=device)
    o = 0
    p.offsets = buf[o:o + n_experts + 1]; o += n_experts + 1
    p.sorted_pair = buf[o:o + pairs]; o += pairs
    p.tile_expert = buf[o:o + p.max_tiles]; o += p.max_tiles
    p.tile_row0 = buf[o:o + p.max_tiles]; o += p.max_tiles
    p.n_tiles = buf[o:o + 1]
    return p


def moe_plan(idx: torch.Tensor, n_experts: int, tile_rows: int, into: Optional[MoEPlan] = None) -> MoEPlan:
    """Sort the pairs of ``idx`` [T, top] by expert, on the device: offsets per expert, the sorted list of pair
    numbers (token * top + choice), and row tiles of ``tile_rows`` rows.  Outputs >= ``n_experts`` enter no list."""
    _need(idx, torch.int32, "idx")
    pairs = idx.numel()
    p = into if into is not None else _empty_plan(pairs, n_experts, tile_rows, idx.device)
    st = _lib("moe").dlgo_moe_plan(_ptr(idx), _i(pairs), _i(n_experts), _i(tile_rows), _ptr(p.offsets),
                                   _ptr(p.sorted_pair), _ptr(p.tile_expert), _ptr(p.tile_row0), _ptr(p.n_tiles),
                                   _i(p.max_tiles), _stream())
    _check(st, "moe_plan")
    return p


def moe_gemm(plan: MoEPlan, a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, gather_div: Optional[int],
             scatter: bool, act: int) -> torch.Tensor:
    """Grouped contraction over the plan's sorted rows: ``out[o(r)] = act(a[s(r)] . w[expert(r)]^T)`` with ``w``
    [experts, N, K].  ``gather_div`` d: ``s(r) = pair(r) // d`` (rows of ``a`` are tokens), None: ``s(r) = r``;
    ``scatter``: ``o(r) = pair(r)``, else ``o(r) = r``.  ``out`` is fp32 or ``a``'s type."""
    _need(w, a.dtype, "w")
    if a.dim() != 2 or a.stride(1) != 1 or out.dim() != 2 or out.stride(1) != 1 or w.dim() != 3:
        raise KernelError("moe_gemm: a and out must be 2-D with unit inner stride, w [experts, N, K]")
    _need(w, None, "w")
    E, N, Kd = w.shape
    if a.shape[1] != Kd or out.shape[1] != N or out.dtype not in (torch.float32, a.dtype):
        raise KernelError("moe_gemm: shapes or types do not fit")
    kind = 0 if plan.tile_rows == MOE_FEW_ROWS else 1
    if kind == 1 and plan.tile_rows != MOE_TILE_ROWS:
        raise KernelError(f"moe_gemm: the plan's tiles must have {MOE_FEW_ROWS} or {MOE_TILE_ROWS} rows")
    st = _lib("moe").dlgo_moe_gemm(
        _i(kind), _i(dtype_code(a.dtype)), _ptr(a), _ll(a.stride(0)), _ptr(plan.sorted_pair if gather_div else None),
        _i(gather_div or 1), _ptr(w), _ptr(out), _ll(out.stride(0)), _ptr(plan.sorted_pair if scatter else None),
        _ptr(plan.offsets), _ptr(plan.tile_expert), _ptr(plan.tile_row0), _ptr(plan.n_tiles), _i(plan.max_tiles),
        _i(N), _i(Kd), _i(act), _i(1 if out.dtype == torch.float32 else 0), _stream())
    _check(st, "moe_gemm")
    return out


def moe_gemm_tc_takes(dtype: torch.dtype, n: int, k: int) -> bool:
    """Whether the tensor-core grouped contraction takes a weight [experts, n, k] of this type."""
    return dtype == torch.bfloat16 and n > 0 and k > 0 and k % 8 == 0


def moe_gather_rows(plan: MoEPlan, src: torch.Tensor, div: int, scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rows of ``src`` in the plan's sorted order: ``dst[r] = src[pair(r) // div]`` for the rows that belong to
    an expert (the others are left unwritten).  Rows must be a multiple of 16 bytes.  ``scale`` (fp32, one number
    per pair; bfloat16 rows only): ``dst[r] = scale[pair(r)] * src[pair(r) // div]``."""
    if scale is not None:
        _need(scale, torch.float32, "scale")
        if src.dtype != torch.bfloat16 or scale.numel() != plan.pairs:
            raise KernelError("moe_gather_rows: a scale goes with bfloat16 rows, one number per pair")
    if src.dim() != 2 or src.stride(1) != 1:
        raise KernelError("moe_gather_rows: src must be 2-D with unit inner stride")
    if not src.is_cuda:
        raise KernelError("moe_gather_rows: src must live on the GPU")
    dst = torch.empty((plan.pairs, src.shape[1]), dtype=src.dtype, device=src.device)
    n_exp = plan.offsets.numel() - 1
    st = _lib("moe_tc").dlgo_moe_gather_rows(
        _ptr(src), _ll(src.stride(0) * src.element_size()), _ptr(dst), _i(src.shape[1] * src.element_size()),
        _ptr(plan.sorted_pair), _ptr(plan.offsets[n_exp:]), _i(div), _i(plan.pairs), _ptr(scale), _stream())
    _check(st, "moe_gather_rows")
    return dst


def moe_gemm_tc(plan: MoEPlan, a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, scatter: bool, act: int) -> torch.Tensor:
    """The grouped contraction on the tensor cores (bfloat16, a plan with tiles of 128 rows): ``a`` holds the rows
    in sorted order, ``w`` is [experts, N, K]; ``out`` (bfloat16 or fp32) receives row r, or with ``scatter`` row
    pair(r)."""
    _need(a, torch.bfloat16, "a")
    _need(w, torch.bfloat16, "w")
    if (plan.tile_rows not in (MOE_TC_ROWS, MOE_TC_PAIR_ROWS) or w.dim() != 3 or a.dim() != 2 or out.dim() != 2 or
            out.stride(1) != 1):
        raise KernelError("moe_gemm_tc: a plan with tiles of 128 rows (or 256: CTA pairs), a and out 2-D, w [experts, N, K]")
    E, N, Kd = w.shape
    if act == MOE_ACT_SWIGLU and (N % (2 * MOE_SWIGLU_BLOCK) or plan.tile_rows != MOE_TC_ROWS):
        raise KernelError("moe_gemm_tc: silu(gate) * up needs whole blocks of gate and up rows and tiles of 128 rows")
    n_out = N // 2 if act == MOE_ACT_SWIGLU else N
    if a.shape[1] != Kd or out.shape[1] != n_out or out.dtype not in (torch.float32, torch.bfloat16):
        raise KernelError("moe_gemm_tc: shapes or types do not fit")
    st = _lib("moe_tc").dlgo_moe_gemm_tc(
        _ptr(a), _ll(a.shape[0]), _ll(a.stride(0)), _ptr(w), _i(E), _ptr(out), _ll(out.stride(0)),
        _ptr(plan.sorted_pair if scatter else None), _ptr(plan.offsets), _ptr(plan.tile_expert), _ptr(plan.tile_row0),
        _ptr(plan.n_tiles), _i(plan.max_tiles), _i(plan.tile_rows), _i(N), _i(Kd), _i(act),
        _i(1 if out.dtype == torch.float32 else 0), _stream())
    _check(st, "moe_gemm_tc")
    return out


def moe_scale_rows(h: torch.Tensor, wt: torch.Tensor) -> torch.Tensor:
    """For experts whose weight multiplies their input: rows [T * top, d] with ``rows[t * top + k] = wt[t, k] *
    h[t]`` in ``h``'s type (the product in fp32)."""
    _need(wt, torch.float32, "wt")
    if h.dim() != 2 or h.stride(1) != 1 or wt.dim() != 2 or wt.shape[0] != h.shape[0]:
        raise KernelError("moe_scale_rows: h [T, d] with unit inner stride, wt [T, top]")
    T, d = h.shape
    top = wt.shape[1]
    rows = torch.empty((T * top, d), dtype=h.dtype, device=h.device)
    st = _lib("moe").dlgo_moe_scale_rows(_ptr(h), _i(dtype_code(h.dtype)), _i(h.stride(0)), _ptr(wt), _ptr(rows),
                                         _i(T * top), _i(d), _i(top), _stream())
    _check(st, "moe_scale_rows")
    return rows


def moe_combine(y: torch.Tensor, pair_out: Optional[torch.Tensor], h: torch.Tensor, idx: torch.Tensor,
                wt: Optional[torch.Tensor], n_experts: int, shared: Optional[torch.Tensor] = None,
                gate: Optional[torch.Tensor] = None) -> None:
    """``y[t] += sum_k wt[t, k] * (pair_out[t * top + k] if idx[t, k] < n_experts else h[t]) + gate[t] * shared[t]``
    (sums in fp32; ``gate`` None: 1; ``wt`` None: every weight 1; ``pair_out`` fp32 or of ``h``'s type)."""
    _need(y, torch.float32, "y")
    _need(idx, torch.int32, "idx")
    if wt is not None:
        _need(wt, torch.float32, "wt")
    T, d = y.shape
    top = idx.shape[1]
    if h.dim() != 2 or h.stride(1) != 1 or tuple(h.shape) != (T, d):
        raise KernelError("moe_combine: h must be [T, d] with unit inner stride")
    if pair_out is not None:
        _need(pair_out, None, "pair_out")
        if pair_out.dtype not in (torch.float32, h.dtype):
            raise KernelError("moe_combine: pair_out must be float32 or of h's type")
        if tuple(pair_out.shape) != (T * top, d):
            raise KernelError("moe_combine: pair_out must be [T * top, d]")
    elif n_experts > 0:
        raise KernelError("moe_combine: experts without their outputs")
    for n, t in (("shared", shared), ("gate", gate)):
        if t is not None:
            _need(t, torch.float32, n)
    st = _lib("moe").dlgo_moe_combine(_ptr(y), _ptr(pair_out),
                                      _i(1 if pair_out is None or pair_out.dtype == torch.float32 else 0), _ptr(h),
                                      _i(dtype_code(h.dtype)), _i(h.stride(0)),
                                      _ptr(idx), _ptr(wt), _ptr(shared), _ptr(gate), _i(T), _i(d), _i(top),
                                      _i(n_experts), _stream())
    _check(st, "moe_combine")


# ------------------------------------------------------------------- attention
ATT_ROW_ELEMS = 128 * 32  # rows of a block times head_dim may not exceed this


def attention_tile_shape(head_dim: int, group: int, decode: bool) -> tuple[int, int]:
    """(tokens per tile, query heads of a kv head per block) that the kernel takes."""
    rows = max(1, ATT_ROW_ELEMS // head_dim)
    rows = min(rows, 32)
    gchunk = min(group, rows)
    qt = 1 if decode else max(1, min(8, rows // gchunk))
    return qt, gchunk


def attention_scratch_floats(T: int, num_heads: int, head_dim: int, n_splits: int) -> int:
    return 0 if n_splits <= 1 else T * num_heads * n_splits * (head_dim + 2)


def attention(q: torch.Tensor, ldq: int, T: int, kpages: torch.Tensor, vpages: torch.Tensor,
              page_table: torch.Tensor, tiles: torch.Tensor, tile_tokens_max: int, seq_slot: torch.Tensor,
              token_pos: torch.Tensor, out: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
              scale: float, window: int = 0, n_splits: int = 1, gchunk: int = 1,
              scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal grouped-query attention of T packed tokens over the paged cache."""
    _need(out, q.dtype, "out")
    _need(kpages, q.dtype, "kpages")
    _need(vpages, q.dtype, "vpages")
    for n, t in (("page_table", page_table), ("tiles", tiles), ("seq_slot", seq_slot), ("token_pos", token_pos)):
        _need(t, torch.int32, n)
    if n_splits > 1:
        need = attention_scratch_floats(T, num_heads, head_dim, n_splits)
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
            raise KernelError(f"attention: {n_splits} slices need {need} floats of scratch")
    st = _lib("attention").dlgo_attention(
        _ptr(q), _i(dtype_code(q.dtype)), _i(T), _i(ldq), _ptr(kpages), _ptr(vpages), _ptr(page_table),
        _i(page_table.shape[1]), _ptr(tiles), _i(tiles.shape[0]), _i(tile_tokens_max), _ptr(seq_slot),
        _ptr(token_pos), _ptr(out), _i(out.stride(0)), _ptr(scratch), _i(num_heads), _i(num_kv_heads), _i(head_dim),
        _i(kpages.shape[-2]), _i(n_splits), _i(gchunk), _i(window), _f(scale), _stream())
    _check(st, "attention", 2 if n_splits > 1 else 1)
    return out


# -------------------------------------------------------------------- sampling
def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """First index of each row's maximum (int32 on the device)."""
    _need(logits, torch.float32, "logits")
    R, V = logits.shape
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    _need(out, torch.int32, "out")
    lib = _lib("sampling")
    chunks = lib.dlgo_argmax_chunks(_i(R), _i(V))
    pv = pi = None
    if chunks > 1:
        pv = torch.empty((R * chunks,), dtype=torch.float32, device=logits.device)
        pi = torch.empty((R * chunks,), dtype=torch.int32, device=logits.device)
    st = lib.dlgo_argmax(_ptr(logits), _i(R), _i(logits.stride(0)), _i(V), _ptr(out), _ptr(pv), _ptr(pi), _stream())
    _check(st, "argmax", 2 if chunks > 1 else 1)
    return out


_argmax_host_buffers: dict = {}


def argmax_to_host(logits: torch.Tensor) -> list:
    """First index of each row's maximum, as a list of ints on the host: the kernels, the copy into a
    pinned buffer and the wait for it in one native call."""
    _need(logits, torch.float32, "logits")
    R, V = logits.shape
    key = (logits.device.index, R, V)
    buf = _argmax_host_buffers.get(key)
    lib = _lib("sampling")
    if buf is None:
        chunks = lib.dlgo_argmax_chunks(_i(R), _i(V))
        host = torch.zeros((R,), dtype=torch.int32).pin_memory()
        buf = _argmax_host_buffers[key] = (
            torch.empty((R,), dtype=torch.int32, device=logits.device),
            torch.empty((R * chunks,), dtype=torch.float32, device=logits.device) if chunks > 1 else None,
            torch.empty((R * chunks,), dtype=torch.int32, device=logits.device) if chunks > 1 else None,
            host, host.numpy(), 2 if chunks > 1 else 1)
    out, pv, pi, host, host_np, launches = buf
    st = lib.dlgo_argmax_host(_ptr(logits), _i(R), _i(logits.stride(0)), _i(V), _ptr(out), _ptr(pv), _ptr(pi),
                              _ptr(host), _stream())
    _check(st, "argmax", launches)
    return host_np.tolist()


def greedy_run_graph(host_inputs: torch.Tensor, graph_exec: int, host_ids: torch.Tensor,
                     stop_ids: Sequence[int], max_steps: int, device_index: int, launches_per_step: int) -> List[List[int]]:
    """Up to ``max_steps`` greedy decode steps of one batch in one native call (dlgo_greedy_run_graph).
    The captured step begins with the copy of its inputs out of ``host_inputs`` and ends with the argmax
    and the copy of the ids into ``host_ids`` (pinned int32 [B]);
    ``host_inputs`` (pinned int32 [3, B]: ids, positions, slots) holds the first step's inputs and is
    advanced in place.  Returns the ids chosen, a list per step, ending with the step in which a
    sequence chose a stop id."""
    import numpy as np
    B = host_ids.numel()
    stops = np.asarray(sorted(int(t) for t in stop_ids), dtype=np.int32)
    tokens = np.empty((max_steps, B), dtype=np.int32)
    n = _lib("sampling").dlgo_greedy_run_graph(
        ctypes.c_void_p(host_inputs.data_ptr()), _i(B), ctypes.c_void_p(graph_exec),
        ctypes.c_void_p(host_ids.data_ptr()), stops.ctypes.data_as(ctypes.c_void_p), _i(len(stops)), _i(max_steps),
        tokens.ctypes.data_as(ctypes.c_void_p), ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(device_index)))
    if n <= 0:
        raise KernelError(f"greedy_run_graph: error {n}")
    global LAUNCHES
    LAUNCHES += launches_per_step * n
    return tokens[:n].tolist()


def sampled_run_graph(host_inputs: torch.Tensor, graph_exec: int, host_ids: torch.Tensor, stop_ids: Sequence[int],
                      max_steps: int, draw_inputs: torch.Tensor, window: int, device_index: int,
                      launches_per_step: int) -> List[List[int]]:
    """:func:`greedy_run_graph` for sampled decoding (dlgo_sampled_run_graph): the captured step also copies
    ``draw_inputs`` (pinned int32: [2] seed, [B] requests, [B] draw indices, [B, window] recent tokens,
    [B] tokens produced so far) and ends with the filters and the draw; draw indices and windows are
    advanced in place."""
    import numpy as np
    B = host_ids.numel()
    if draw_inputs.numel() != 2 + 3 * B + B * window or draw_inputs.dtype != torch.int32 or not draw_inputs.is_pinned():
        raise KernelError("sampled_run_graph: draw_inputs must be pinned int32 [2 + 3 B + B window]")
    stops = np.asarray(sorted(int(t) for t in stop_ids), dtype=np.int32)
    tokens = np.empty((max_steps, B), dtype=np.int32)
    n = _lib("sampling").dlgo_sampled_run_graph(
        ctypes.c_void_p(host_inputs.data_ptr()), _i(B), ctypes.c_void_p(graph_exec),
        ctypes.c_void_p(host_ids.data_ptr()), stops.ctypes.data_as(ctypes.c_void_p), _i(len(stops)), _i(max_steps),
        tokens.ctypes.data_as(ctypes.c_void_p), ctypes.c_void_p(draw_inputs.data_ptr()), _i(window),
        ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(device_index)))
    if n <= 0:
        raise KernelError(f"sampled_run_graph: error {n}")
    global LAUNCHES
    LAUNCHES += launches_per_step * n
    return tokens[:n].tolist()


def sample(logits: torch.Tensor, temperature: torch.Tensor, request: torch.Tensor, draw: torch.Tensor, seed: int,
           out: Optional[torch.Tensor] = None, seed_dev: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row from softmax(logits / temperature) by inverse CDF; the uniform is a function of
    (seed, draw, request).  ``seed_dev`` (two int32 on the device, 8-byte aligned): the kernel reads the seed
    there instead (a captured step whose seed changes between replays)."""
    _need(logits, torch.float32, "logits")
    _need(temperature, torch.float32, "temperature")
    _need(request, torch.int32, "request")
    _need(draw, torch.int32, "draw")
    R, V = logits.shape
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    if seed_dev is not None and (seed_dev.dtype != torch.int32 or seed_dev.numel() < 2 or not seed_dev.is_cuda):
        raise KernelError("sample: seed_dev must be two int32 on the GPU")
    lib = _lib("sampling")
    chunks = int(lib.dlgo_sample_chunks(_i(V)))       # > 0: a large vocabulary, drawn from in two kernels
    part = torch.empty((R * chunks * 2,), dtype=torch.float32, device=logits.device) if chunks > 0 else None
    st = lib.dlgo_sample(_ptr(logits), _i(R), _i(logits.stride(0)), _i(V), _ptr(temperature), _ptr(request),
                         _ptr(draw), ctypes.c_ulonglong(seed & (2 ** 64 - 1)), _ptr(seed_dev), _ptr(out), _ptr(part),
                         _stream())
    _check(st, "sample", 2 if chunks > 0 else 1)
    return out


def uniform(seed: int, draw: torch.Tensor, request: torch.Tensor) -> torch.Tensor:
    _need(draw, torch.int32, "draw")
    _need(request, torch.int32, "request")
    out = torch.empty((draw.numel(),), dtype=torch.float32, device=draw.device)
    st = _lib("sampling").dlgo_uniform(ctypes.c_ulonglong(seed & (2 ** 64 - 1)), _ptr(draw), _ptr(request), _ptr(out),
                                       _i(draw.numel()), _stream())
    _check(st, "uniform")
    return out


# ------------------------------------------------------- tensor-core contraction
TC_STORE, TC_STORE_F32, TC_ADD_F32, TC_SWIGLU, TC_PARTIAL, TC_RED_F32 = 0, 1, 2, 3, 4, 5
TC_TILE_M, TC_TILE_K = 128, 64


def gemm_tc_workspace_floats(ra: int, rb: int, bn: int, splits: int) -> int:
    if splits <= 1:
        return 0
    return ((ra + TC_TILE_M - 1) // TC_TILE_M) * ((rb + bn - 1) // bn) * splits * bn * TC_TILE_M


def gemm_tc(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, transposed: bool, epilogue: int, bn: int,
            splits: int = 1, workspace: Optional[torch.Tensor] = None,
            counters: Optional[torch.Tensor] = None, static_operand: int = 0, pair_tile: int = 0) -> torch.Tensor:
    """D[Ra, Rb] = a[Ra, K] . b[Rb, K]^T on the tensor cores (bf16 in, fp32 accumulate).

    ``out`` receives D (``transposed``: D^T) through ``epilogue``; with ``splits`` > 1 the K range is
    shared by that many CTAs per tile, which needs ``workspace`` (fp32) and zeroed ``counters`` (int32).
    ``static_operand`` (1: a, 2: b) names the operand that holds weights no earlier kernel writes.
    ``pair_tile`` (128 or 256): many tokens, 256 x pair_tile tiles computed by pairs of CTAs (cta_group::2).
    ``TC_PARTIAL`` (transposed only): every K-slice leaves its fp32 tile in ``out`` [splits, Rb, Ra] for the
    reader to add in order.  ``TC_RED_F32`` (transposed only): every K-slice adds itself into the fp32
    ``out`` with reductions at the memory; no workspace, and the order of the adds (the sum's last bits) is
    not fixed.
    """
    if epilogue == TC_RED_F32 and not transposed:
        raise KernelError("gemm_tc: the atomic add is for transposed products")
    for n, t in (("a", a), ("b", b)):
        if not t.is_cuda or t.dtype != torch.bfloat16 or t.dim() != 2 or t.stride(1) != 1:
            raise KernelError(f"gemm_tc: {n} must be a 2-D bfloat16 GPU tensor with unit inner stride")
    ra, k = a.shape
    rb, k2 = b.shape
    if k != k2:
        raise KernelError(f"gemm_tc: a has K={k}, b has K={k2}")
    if out.stride(-1) != 1:
        raise KernelError("gemm_tc: out must have unit inner stride")
    if splits > 1 and epilogue not in (TC_PARTIAL, TC_RED_F32):
        need = gemm_tc_workspace_floats(ra, rb, bn, splits)
        tiles = ((ra + TC_TILE_M - 1) // TC_TILE_M) * ((rb + bn - 1) // bn)
        if workspace is None or workspace.numel() < need or counters is None or counters.numel() < tiles:
            raise KernelError(f"gemm_tc: {splits} K-slices need {need} floats of workspace and {tiles} counters")
    if epilogue == TC_PARTIAL:
        # out is [slices, rb, ra]: the kernel's row stride is that of one slice's rows
        if not transposed or out.dim() != 3 or out.dtype != torch.float32 or \
                tuple(out.shape) != (splits, rb, ra) or out.stride(0) != rb * out.stride(1) or out.stride(1) < ra:
            raise KernelError(f"gemm_tc: partials go to a float32 [{splits}, {rb}, {ra}] tensor of a transposed product")
        ldo = out.stride(1)
    else:
        want_shape = (rb, ra) if transposed else (ra, rb)
        if epilogue == TC_SWIGLU:
            want_shape = (rb, ra // 2) if transposed else (ra, rb // 2)
        if out.dim() != 2 or tuple(out.shape) != want_shape:
            raise KernelError(f"gemm_tc: out must be {list(want_shape)}, is {list(out.shape)}")
        want_dtype = torch.bfloat16 if epilogue in (TC_STORE, TC_SWIGLU) else torch.float32
        if out.dtype != want_dtype:
            raise KernelError(f"gemm_tc: out must be {want_dtype}")
        ldo = out.stride(0)
    st = _lib("gemm_tc").dlgo_gemm_tc(_ptr(a), _i(ra), _i(a.stride(0)), _ptr(b), _i(rb), _i(b.stride(0)), _i(k),
                                      _ptr(out), _i(ldo), _i(1 if transposed else 0), _i(epilogue), _i(bn),
                                      _i(splits), _ptr(workspace), _ptr(counters), _i(static_operand), _i(pair_tile),
                                      _stream())
    _check(st, "gemm_tc")
    return out


def gemm_tc_bias_act(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, transposed: bool, bn: int,
                     bias: Optional[torch.Tensor], act: int, splits: int = 1, workspace: Optional[torch.Tensor] = None,
                     counters: Optional[torch.Tensor] = None, static_operand: int = 0, pair_tile: int = 0) -> torch.Tensor:
    """:func:`gemm_tc` whose epilogue writes ``act(D + bias)`` as bfloat16: ``bias`` (fp32, one number per row of
    the weight operand, or None) and the activation (``ACT_*``) are applied in fp32 on the accumulator.  The
    weight is ``a`` when ``transposed`` (few tokens) and ``b`` otherwise."""
    for n, t in (("a", a), ("b", b)):
        if not t.is_cuda or t.dtype != torch.bfloat16 or t.dim() != 2 or t.stride(1) != 1:
            raise KernelError(f"gemm_tc_bias_act: {n} must be a 2-D bfloat16 GPU tensor with unit inner stride")
    ra, k = a.shape
    rb, k2 = b.shape
    if k != k2:
        raise KernelError(f"gemm_tc_bias_act: a has K={k}, b has K={k2}")
    want_shape = (rb, ra) if transposed else (ra, rb)
    if out.dtype != torch.bfloat16 or out.dim() != 2 or tuple(out.shape) != want_shape or out.stride(1) != 1:
        raise KernelError(f"gemm_tc_bias_act: out must be bfloat16 {list(want_shape)} with unit inner stride")
    if bias is not None:
        _need(bias, torch.float32, "bias")
        if bias.numel() != (ra if transposed else rb):
            raise KernelError("gemm_tc_bias_act: one bias per row of the weight")
    if splits > 1:
        need = gemm_tc_workspace_floats(ra, rb, bn, splits)
        tiles = ((ra + TC_TILE_M - 1) // TC_TILE_M) * ((rb + bn - 1) // bn)
        if workspace is None or workspace.numel() < need or counters is None or counters.numel() < tiles:
            raise KernelError(f"gemm_tc_bias_act: {splits} K-slices need {need} floats of workspace and {tiles} counters")
    st = _lib("gemm_tc").dlgo_gemm_tc_bias_act(
        _ptr(a), _i(ra), _i(a.stride(0)), _ptr(b), _i(rb), _i(b.stride(0)), _i(k), _ptr(out), _i(out.stride(0)),
        _i(1 if transposed else 0), _i(bn), _i(splits), _ptr(workspace), _ptr(counters), _i(static_operand),
        _i(pair_tile), _ptr(bias), _i(act), _stream())
    _check(st, "gemm_tc_bias_act")
    return out


class RopeArgs(ctypes.Structure):
    """What the q|k|v projection's epilogue needs to rotate q and k and to append k and v (DlgoRopeArgs)."""
    _fields_ = [("cos_t", _p), ("sin_t", _p), ("token_pos", _p), ("token_seq", _p), ("seq_slot", _p),
                ("page_table", _p), ("max_pages", _i), ("kpages", _p), ("vpages", _p), ("Hq", _i), ("Hkv", _i),
                ("hd", _i), ("write_cache", _i)]


def rope_args(cos: torch.Tensor, sin: torch.Tensor, token_pos: torch.Tensor, token_seq: torch.Tensor,
              seq_slot: torch.Tensor, page_table: torch.Tensor, kpages: torch.Tensor, vpages: torch.Tensor,
              num_heads: int, num_kv_heads: int, head_dim: int, write_cache: bool) -> RopeArgs:
    """Checked :class:`RopeArgs`; the caller keeps the tensors alive while a launch may read them."""
    _need(cos, torch.float32, "cos")
    _need(sin, torch.float32, "sin")
    for n, t in (("token_pos", token_pos), ("token_seq", token_seq), ("seq_slot", seq_slot), ("page_table", page_table)):
        _need(t, torch.int32, n)
    _need(kpages, torch.bfloat16, "kpages")
    _need(vpages, torch.bfloat16, "vpages")
    if cos.dim() != 2 or cos.shape[1] * 2 != head_dim or sin.shape != cos.shape:
        raise KernelError("rope_args: whole-head rotation tables [positions, head_dim / 2] only")
    if kpages.shape[-2] != 64 or kpages.shape[-1] != head_dim or kpages.shape[-3] != num_kv_heads:
        raise KernelError("rope_args: pages must be [pages, kv heads, 64, head_dim]")
    return RopeArgs(cos.data_ptr(), sin.data_ptr(), token_pos.data_ptr(), token_seq.data_ptr(), seq_slot.data_ptr(),
                    page_table.data_ptr(), page_table.shape[1], kpages.data_ptr(), vpages.data_ptr(), num_heads,
                    num_kv_heads, head_dim, 1 if write_cache else 0)


def gemm_tc_rope_takes(out_features: int, in_features: int, num_heads: int, num_kv_heads: int, head_dim: int,
                       page_size: int) -> bool:
    """Whether :func:`gemm_tc_rope` takes a q|k|v weight [out, in] with these heads and pages."""
    import os
    return os.environ.get("DLGO_TC_DIRECT_EPILOGUE") is None and bool(_lib("gemm_tc").dlgo_gemm_tc_rope_takes(
        _i(out_features), _i(in_features), _i(num_heads), _i(num_kv_heads), _i(head_dim), _i(page_size)))


def gemm_tc_rope(x: torch.Tensor, w: torch.Tensor, qkv: torch.Tensor, pair_tile: int, rope: RopeArgs) -> torch.Tensor:
    """The q|k|v projection of a prompt step (``x`` [T, K] . ``w`` [(Hq + 2 Hkv) hd, K]^T on the tensor cores)
    whose epilogue rotates q and k in fp32 (whole head, split-half pairing), rounds once, writes the q heads to
    ``qkv`` [T, out] and appends k and v to the tokens' rows of their pages; the k and v columns of ``qkv`` are
    not written.  ``pair_tile``: 256 (CTA pairs) or 0."""
    for n, t in (("x", x), ("w", w)):
        if not t.is_cuda or t.dtype != torch.bfloat16 or t.dim() != 2 or t.stride(1) != 1:
            raise KernelError(f"gemm_tc_rope: {n} must be a 2-D bfloat16 GPU tensor with unit inner stride")
    T, k = x.shape
    n_out, k2 = w.shape
    if k != k2 or qkv.dtype != torch.bfloat16 or tuple(qkv.shape) != (T, n_out) or qkv.stride(1) != 1:
        raise KernelError("gemm_tc_rope: x [T, K], w [out, K] and a bfloat16 qkv [T, out] with unit inner stride")
    st = _lib("gemm_tc").dlgo_gemm_tc_rope(_ptr(x), _i(T), _i(x.stride(0)), _ptr(w), _i(n_out), _i(w.stride(0)), _i(k),
                                           _ptr(qkv), _i(qkv.stride(0)), _i(pair_tile), ctypes.byref(rope), _stream())
    _check(st, "gemm_tc_rope")
    return qkv


def check_device_errors() -> None:
    """Raise if a kernel gave up a bounded wait on the device since the last check (synchronises)."""
    for lib, fn in (("gemm_tc", "dlgo_gemm_tc_error"), ("attention_prefill_tc", "dlgo_attention_tc_error"),
                    ("moe_tc", "dlgo_moe_tc_error")):
        if lib in build._loaded:
            v = getattr(build._loaded[lib], fn)()
            if v != 0:
                raise KernelError(f"a tensor-core kernel ({lib}) gave up a bounded wait on the device; "
                                  "its results are invalid")
    if "decode_layers" in build._loaded:
        v = build._loaded["decode_layers"].dlgo_decode_layers_error()
        if v == 1:
            raise KernelError("the persistent decode kernel gave up a bounded wait on the device; its results are "
                              "invalid and its counters must be zeroed again (build a new engine)")
        if v != 0:
            raise KernelError("a token's position had no page in the cache's table (persistent decode kernel)")
    for lib, fn in (("rope_append", "dlgo_rope_append_error"), ("headnorm_rope", "dlgo_headnorm_rope_error"),
                    ("wholenorm_append", "dlgo_wholenorm_append_error")):
        if lib in build._loaded and getattr(build._loaded[lib], fn)() != 0:
            raise KernelError("a token's position had no page in the cache's table: its keys and values were not "
                              "stored and the step's results are invalid")


# ------------------------------------------------------------ decode attention
def attention_decode_mma_takes(dtype: torch.dtype, head_dim: int, page_size: int, n_splits: int) -> bool:
    """Whether the tensor-core decode kernel takes these sizes (bfloat16, heads of 64 or 128, 1..8 slices)."""
    return dtype == torch.bfloat16 and bool(
        _lib("attention_decode_mma").dlgo_attention_decode_mma_takes(_i(head_dim), _i(page_size), _i(n_splits)))


def attention_decode_mma_fuses_rope(num_heads: int, num_kv_heads: int, head_dim: int, rotary_dim: int,
                                    interleaved: bool) -> bool:
    """Whether the kernel can sum the projection's slices, rotate and append itself: whole-head rotation
    in the split-half pairing, at most 8 query heads per kv head."""
    return rotary_dim == head_dim and not interleaved and num_heads // num_kv_heads <= 8


def attention_decode_mma(q: Optional[torch.Tensor], ldq: int, B: int, kpages: torch.Tensor, vpages: torch.Tensor,
                         page_table: torch.Tensor, seq_slot: torch.Tensor, token_pos: torch.Tensor,
                         out: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                         window: int = 0, n_splits: int = 1, keys_per_tile: int = 16,
                         scratch: Optional[torch.Tensor] = None, parts: Optional[torch.Tensor] = None,
                         cos: Optional[torch.Tensor] = None, sin: Optional[torch.Tensor] = None,
                         write_cache: bool = True, clear_parts: bool = False) -> torch.Tensor:
    """Attention of one new token per sequence over its cached keys and values, bfloat16, on the
    tensor cores (mma.sync); 2..8 slices combine inside a thread-block cluster, more go through
    ``scratch`` (``attention_scratch_floats`` floats) and a second kernel.  With ``parts`` (the q|k|v
    projection as fp32 [slices, sequences, columns], unrotated) the kernel sums the slices, rotates q and k
    and appends k and v itself; ``clear_parts`` (one slice, at most 8 page slices): the sum is left zero."""
    for n, t in (("out", out), ("kpages", kpages), ("vpages", vpages)):
        _need(t, torch.bfloat16, n)
    for n, t in (("page_table", page_table), ("seq_slot", seq_slot), ("token_pos", token_pos)):
        _need(t, torch.int32, n)
    if seq_slot.numel() < B or token_pos.numel() < B or out.shape[0] < B:
        raise KernelError("attention_decode_mma: fewer rows than sequences")
    if out.shape[1] < num_heads * head_dim:
        raise KernelError("attention_decode_mma: out needs a column per head dimension")
    S = part_stride = 0
    if parts is None:
        _need(q, torch.bfloat16, "q")
        if q.shape[0] < B or q.shape[1] < num_heads * head_dim:
            raise KernelError("attention_decode_mma: q needs a row per sequence and a column per head dimension")
    else:
        # the projection's unsummed slices [S, B, ldq] (q | k | v heads), rotated and appended by the kernel
        _need(parts, torch.float32, "parts")
        _need(cos, torch.float32, "cos")
        _need(sin, torch.float32, "sin")
        if parts.dim() != 3 or parts.shape[1] < B or parts.shape[2] != ldq or \
                ldq < (num_heads + 2 * num_kv_heads) * head_dim or cos.shape[1] != head_dim // 2:
            raise KernelError("attention_decode_mma: parts must be [slices, sequences, q|k|v columns] with cos/sin "
                              "tables of head_dim / 2 columns")
        if not attention_decode_mma_fuses_rope(num_heads, num_kv_heads, head_dim, head_dim, False):
            raise KernelError("attention_decode_mma: these head counts cannot take the fused rotation")
        S, part_stride = parts.shape[0], parts.stride(0)
        if clear_parts and (S != 1 or n_splits > 8):
            raise KernelError("attention_decode_mma: only one summed slice read by at most 8 page slices can be cleared")
    if parts is None and clear_parts:
        raise KernelError("attention_decode_mma: clear_parts goes with parts")
    page_size = kpages.shape[-2]
    if n_splits > 8:
        need = attention_scratch_floats(B, num_heads, head_dim, n_splits)
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
            raise KernelError(f"attention_decode_mma: {n_splits} slices need {need} floats of scratch")
    st = _lib("attention_decode_mma").dlgo_attention_decode_mma(
        _ptr(q), _i(B), _i(ldq), _ptr(kpages), _ptr(vpages), _ptr(page_table), _i(page_table.shape[1]),
        _ptr(seq_slot), _ptr(token_pos), _ptr(out), _i(out.stride(0)), _i(num_heads), _i(num_kv_heads), _i(head_dim),
        _i(page_size), _i(n_splits), _i(window), _f(scale), _i(keys_per_tile),
        _ptr(scratch if n_splits > 8 else None), _ptr(parts), _i(S), _ll(part_stride), _ptr(cos), _ptr(sin),
        _i(1 if write_cache else 0), _i(1 if clear_parts else 0), _stream())
    _check(st, "attention_decode_mma", 2 if n_splits > 8 else 1)
    return out


def attention_decode_takes(dtype: torch.dtype, head_dim: int, page_size: int) -> bool:
    return bool(_lib("attention_decode").dlgo_attention_decode_takes(_i(dtype_code(dtype)), _i(head_dim), _i(page_size)))


def attention_decode(q: torch.Tensor, ldq: int, B: int, kpages: torch.Tensor, vpages: torch.Tensor,
                     page_table: torch.Tensor, seq_slot: torch.Tensor, token_pos: torch.Tensor, out: torch.Tensor,
                     num_heads: int, num_kv_heads: int, head_dim: int, scale: float, window: int = 0,
                     n_splits: int = 1, scratch: Optional[torch.Tensor] = None,
                     counters: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of one new token per sequence over its cached keys and values.

    ``counters`` (int32, zero, at least ``B * num_kv_heads * ceil(group / 4)``): with them the slice that
    finishes last combines the partial results; without them a second kernel does."""
    _need(out, q.dtype, "out")
    _need(kpages, q.dtype, "kpages")
    _need(vpages, q.dtype, "vpages")
    for n, t in (("page_table", page_table), ("seq_slot", seq_slot), ("token_pos", token_pos)):
        _need(t, torch.int32, n)
    if n_splits > 1 and not (scratch is None and n_splits <= 8):   # up to 8 slices can combine in a cluster
        need = attention_scratch_floats(B, num_heads, head_dim, n_splits)
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
            raise KernelError(f"attention_decode: {n_splits} slices need {need} floats of scratch")
        if counters is not None:
            _need(counters, torch.int32, "counters")
            if counters.numel() < B * num_kv_heads * ((num_heads // num_kv_heads + 3) // 4):
                raise KernelError("attention_decode: too few counters")
    st = _lib("attention_decode").dlgo_attention_decode(
        _ptr(q), _i(dtype_code(q.dtype)), _i(B), _i(ldq), _ptr(kpages), _ptr(vpages), _ptr(page_table),
        _i(page_table.shape[1]), _ptr(seq_slot), _ptr(token_pos), _ptr(out), _i(out.stride(0)), _ptr(scratch),
        _ptr(counters), _i(num_heads), _i(num_kv_heads), _i(head_dim), _i(kpages.shape[-2]), _i(n_splits), _i(window),
        _f(scale), _stream())
    _check(st, "attention_decode", 2 if (n_splits > 1 and counters is None and scratch is not None) else 1)
    return out


# ------------------------------------------------------ tensor-core prefill attention
PREFILL_TC_TILE = 128


def attention_prefill_tc_takes(dtype: torch.dtype, head_dim: int, page_size: int) -> bool:
    return dtype == torch.bfloat16 and head_dim in (64, 128) and page_size == 64


def attention_prefill_tc(q: torch.Tensor, ldq: int, T: int, kpages: torch.Tensor, vpages: torch.Tensor,
                         page_table: torch.Tensor, tiles: torch.Tensor, seq_slot: torch.Tensor,
                         token_pos: torch.Tensor, out: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                         scale: float, window: int = 0) -> torch.Tensor:
    """Causal attention of packed prompt tokens on the tensor cores; tiles hold at most 128 tokens each."""
    _need(out, torch.bfloat16, "out")
    _need(kpages, torch.bfloat16, "kpages")
    _need(vpages, torch.bfloat16, "vpages")
    if q.dtype != torch.bfloat16:
        raise KernelError("attention_prefill_tc: q must be bfloat16")
    for n, t in (("page_table", page_table), ("tiles", tiles), ("seq_slot", seq_slot), ("token_pos", token_pos)):
        _need(t, torch.int32, n)
    st = _lib("attention_prefill_tc").dlgo_attention_prefill_tc(
        _ptr(q), _i(T), _i(ldq), _ptr(kpages), _ptr(vpages), _i(kpages.shape[0]), _ptr(page_table),
        _i(page_table.shape[1]), _ptr(tiles), _i(tiles.shape[0]), _ptr(seq_slot), _ptr(token_pos), _ptr(out),
        _i(out.stride(0)), _i(num_heads), _i(num_kv_heads), _i(head_dim), _i(window), _f(scale), _stream())
    _check(st, "attention_prefill_tc")
    return out


# ------------------------------------------------------------------- filters
FILTER_MAX_K, FILTER_MAX_RECENT = 2048, 64


def filter_logits(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, min_p: float, penalty: float,
                  recent: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Repetition penalty, temperature, top-k (0: off, else up to 2048), top-p and min-p in one kernel.
    Returns the filtered, temperature-scaled logits; dropped tokens hold -inf.  ``recent`` is
    [rows, <= 64] int32 with -1 for "none"."""
    if not logits.is_cuda or logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("logits must be float32 [rows, vocab] on the GPU with unit stride along the vocabulary")
    R, V = logits.shape
    work = torch.empty((R, V), dtype=torch.float32, device=logits.device)
    n_recent = 0
    if recent is not None:
        _need(recent, torch.int32, "recent")
        n_recent = recent.shape[1]
    st = _lib("sampling").dlgo_filter(_ptr(logits), _i(R), _i(logits.stride(0)), _i(V), _ptr(work), _f(temperature),
                                      _i(top_k), _f(top_p), _f(min_p), _f(penalty), _ptr(recent), _i(n_recent),
                                      _stream())
    _check(st, "filter")
    return work


def filter_draw_chunks(V: int, top_k: int) -> int:
    """Chunks of the vocabulary :func:`filter_draw` works in, or 0 where it does not take the sizes (top-k off or
    above 256, a very large vocabulary): the caller then uses :func:`filter_logits` and :func:`sample`."""
    return int(_lib("sampling").dlgo_filter_draw_chunks(_i(V), _i(top_k)))


def filter_draw(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, min_p: float, penalty: float,
                recent: Optional[torch.Tensor], request: torch.Tensor, draw: torch.Tensor, seed: int,
                out: Optional[torch.Tensor] = None, seed_dev: Optional[torch.Tensor] = None) -> torch.Tensor:
    """:func:`filter_logits` followed by :func:`sample` for a small top-k, without a pass of one block over the
    whole row: blocks over chunks of the vocabulary list what top-k can keep, one block per row filters and
    draws from that list (csrc/sampling.cu)."""
    if not logits.is_cuda or logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("logits must be float32 [rows, vocab] on the GPU with unit stride along the vocabulary")
    R, V = logits.shape
    lib = _lib("sampling")
    C = int(lib.dlgo_filter_draw_chunks(_i(V), _i(top_k)))
    if C == 0:
        raise KernelError(f"filter_draw does not take top_k={top_k} with a vocabulary of {V}")
    cap = int(lib.dlgo_filter_draw_cap(_i(top_k)))
    _need(request, torch.int32, "request")
    _need(draw, torch.int32, "draw")
    n_recent = 0
    if recent is not None:
        _need(recent, torch.int32, "recent")
        n_recent = recent.shape[1]
    if seed_dev is not None and (seed_dev.dtype != torch.int32 or seed_dev.numel() < 2 or not seed_dev.is_cuda):
        raise KernelError("filter_draw: seed_dev must be two int32 on the GPU")
    dev = logits.device
    cand_v = torch.empty((R * C * cap,), dtype=torch.float32, device=dev)
    cand_i = torch.empty((R * C * cap + R * C,), dtype=torch.int32, device=dev)      # indices, then counts
    work = torch.empty((R, V), dtype=torch.float32, device=dev)      # (rows with more ties than the lists hold)
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=dev)
    st = lib.dlgo_filter_draw(_ptr(logits), _i(R), _i(logits.stride(0)), _i(V), _ptr(work), _f(temperature), _i(top_k),
                              _f(top_p), _f(min_p), _f(penalty), _ptr(recent), _i(n_recent), _ptr(cand_v),
                              _ptr(cand_i), _p(cand_i.data_ptr() + 4 * R * C * cap), _ptr(request), _ptr(draw),
                              ctypes.c_ulonglong(seed & (2 ** 64 - 1)), _ptr(seed_dev), _ptr(out), _stream())
    _check(st, "filter_draw", 2)
    return out


# ------------------------------------------------------------------ host side of a decode step
class HostStep:
    """The runtime calls of a decode step's launch as one native call: inputs out of a pinned buffer,
    an event that frees the buffer, the captured graph."""

    def __init__(self) -> None:
        lib = _lib("hoststep")
        lib.dlgo_hoststep_create.restype = ctypes.c_void_p
        self._lib = lib
        self._h = ctypes.c_void_p(lib.dlgo_hoststep_create())
        if not self._h:
            raise KernelError("hoststep: no event")

    def wait(self) -> None:
        st = self._lib.dlgo_hoststep_wait(self._h)
        if st != 0:
            raise KernelError(f"hoststep: CUDA error {st} while waiting for the input copy")

    def launch(self, dev_inputs: torch.Tensor, host_inputs: torch.Tensor, graph_exec: int, device_index: int) -> None:
        st = self._lib.dlgo_hoststep_launch(
            self._h, _ptr(dev_inputs), ctypes.c_void_p(host_inputs.data_ptr()),
            _ll(host_inputs.numel() * host_inputs.element_size()), ctypes.c_void_p(graph_exec),
            ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(device_index)))
        if st != 0:
            raise KernelError(f"hoststep: CUDA error {st} at the launch of a decode step")

    def __del__(self) -> None:
        try:
            self._lib.dlgo_hoststep_destroy(self._h)
        except Exception:
            pass


# ------------------------------------------------- a run of layers as one persistent kernel (decode steps)
def decode_layers_takes(tokens: int, hidden: int, num_heads: int, num_kv_heads: int, head_dim: int, ffn: int,
                        page_size: int) -> bool:
    """Whether the persistent decode kernel takes these sizes (see csrc/decode_layers.cu)."""
    return bool(_lib("decode_layers").dlgo_decode_layers_takes(_i(tokens), _i(hidden), _i(num_heads), _i(num_kv_heads),
                                                               _i(head_dim), _i(ffn), _i(page_size)))


def decode_layers_grid() -> int:
    return int(_lib("decode_layers").dlgo_decode_layers_grid())


def decode_layers_describe(layers: Sequence[dict], hidden: int, num_heads: int, num_kv_heads: int, head_dim: int,
                           ffn: int, device: torch.device) -> torch.Tensor:
    """The descriptor array of a run of layers, in device memory.  Each entry of ``layers`` gives the tensors
    ``w_qkv, w_o, w_gu, w_down`` (bfloat16, contiguous), ``norm1_w, norm2_w`` (float32), ``kpages, vpages``, and
    ``eps1, eps2, write_cache``.  The caller keeps those tensors alive as long as the descriptors are used."""
    lib = _lib("decode_layers")
    size = int(lib.dlgo_decode_layers_desc_bytes())
    raw = ctypes.create_string_buffer(size * len(layers) + 64)
    base = (ctypes.addressof(raw) + 63) & ~63
    for i, L in enumerate(layers):
        for n in ("w_qkv", "w_o", "w_gu", "w_down"):
            _need(L[n], torch.bfloat16, n)
        for n in ("norm1_w", "norm2_w"):
            _need(L[n], torch.float32, n)
        if L["kpages"].dtype != torch.bfloat16 or L["vpages"].dtype != torch.bfloat16:
            raise KernelError("decode_layers: the cache must be bfloat16")
        st = lib.dlgo_decode_layers_describe(
            ctypes.c_void_p(base + i * size), _ptr(L["w_qkv"]), _ptr(L["w_o"]), _ptr(L["w_gu"]), _ptr(L["w_down"]),
            _ptr(L["norm1_w"]), _ptr(L["norm2_w"]), _f(L["eps1"]), _f(L["eps2"]), _ptr(L["kpages"]), _ptr(L["vpages"]),
            _i(1 if L["write_cache"] else 0), _i(hidden), _i(num_heads), _i(num_kv_heads), _i(head_dim), _i(ffn))
        _check(st, "decode_layers_describe", 0)
    host = torch.frombuffer(bytearray(ctypes.string_at(base, size * len(layers))), dtype=torch.uint8)
    # device allocations are 256-byte aligned, which the tensor maps inside need
    return host.to(device)


def decode_layers_scratch_floats(tokens: int, num_heads: int, head_dim: int, n_splits: int) -> int:
    return int(_lib("decode_layers").dlgo_decode_layers_scratch_floats(_i(tokens), _i(num_heads), _i(head_dim),
                                                                         _i(n_splits)))


def decode_layers(desc: torch.Tensor, n_layers: int, residual: torch.Tensor, hidden: int, num_heads: int,
                  num_kv_heads: int, head_dim: int, ffn: int, scale: float, qkv_sum: torch.Tensor,
                  scale1: torch.Tensor, attn_out: torch.Tensor, h: torch.Tensor, scratch: Optional[torch.Tensor],
                  tickets: torch.Tensor, page_table: torch.Tensor, seq_slot: torch.Tensor, token_pos: torch.Tensor,
                  cos: torch.Tensor, sin: torch.Tensor, page_size: int, n_splits: int, sync: torch.Tensor,
                  first: bool = False) -> None:
    """``n_layers`` decoder layers on the residual stream [T, hidden] (fp32, in place), one new token per
    sequence: see csrc/decode_layers.cu.  ``qkv_sum``, ``tickets`` and ``sync`` must be zero and are left zero."""
    T = residual.shape[0]
    _need(residual, torch.float32, "residual")
    _need(qkv_sum, torch.float32, "qkv_sum")
    _need(scale1, torch.float32, "scale1")
    _need(attn_out, torch.bfloat16, "attn_out")
    _need(h, torch.bfloat16, "h")
    for n, t in (("tickets", tickets), ("page_table", page_table), ("seq_slot", seq_slot), ("token_pos", token_pos),
                 ("sync", sync)):
        _need(t, torch.int32, n)
    _need(cos, torch.float32, "cos")
    _need(sin, torch.float32, "sin")
    qkv_n = (num_heads + 2 * num_kv_heads) * head_dim
    if (residual.shape[1] != hidden or qkv_sum.numel() < T * qkv_n or scale1.numel() < T or
            attn_out.numel() < T * num_heads * head_dim or h.numel() < T * ffn or tickets.numel() < T * num_kv_heads or
            sync.numel() < 2 or seq_slot.numel() < T or token_pos.numel() < T):
        raise KernelError("decode_layers: a buffer is too small for these sizes")
    if cos.shape[1] * 2 != head_dim or sin.shape != cos.shape:
        raise KernelError("decode_layers: whole-head rotation tables [positions, head_dim / 2] only")
    if n_splits > 1:
        need = decode_layers_scratch_floats(T, num_heads, head_dim, n_splits)
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
            raise KernelError(f"decode_layers: {n_splits} page slices need {need} floats of scratch")
    st = _lib("decode_layers").dlgo_decode_layers(
        _ptr(desc), _i(n_layers), _i(T), _i(hidden), _i(num_heads), _i(num_kv_heads), _i(head_dim), _i(ffn), _f(scale),
        _ptr(residual), _i(residual.stride(0)), _ptr(qkv_sum), _ptr(scale1), _ptr(attn_out), _ptr(h), _ptr(scratch),
        _ptr(tickets), _ptr(page_table), _i(page_table.shape[1]), _ptr(seq_slot), _ptr(token_pos), _ptr(cos), _ptr(sin),
        _i(page_size), _i(n_splits), _i(0), _ptr(sync), _i(1 if first else 0), _stream())
    _check(st, "decode_layers")


# ------------------------------------------------------------------ the layer loop of a prompt step, native
class PromptEntryPoints(ctypes.Structure):
    _fields_ = [(n, _p) for n in ("rmsnorm", "gemm_tc", "rope_append", "attention", "gemm_tc_rope")]


class PromptShape(ctypes.Structure):
    _fields_ = [(n, _i) for n in ("hidden", "heads", "kv_heads", "head_dim", "ffn", "rotary_dim", "interleaved",
                                  "window", "page_size")] + [("scale", _f)]


class PromptLayer(ctypes.Structure):
    _fields_ = [("w_qkv", _p), ("w_o", _p), ("w_gate_up", _p), ("w_down", _p), ("norm1_w", _p), ("norm2_w", _p),
                ("eps1", _f), ("eps2", _f), ("kpages", _p), ("vpages", _p), ("n_pages", _i), ("write_cache", _i)]


class PromptStep(ctypes.Structure):
    _fields_ = [("tokens", _i), ("residual", _p), ("x", _p), ("qkv", _p), ("attn_out", _p), ("h", _p), ("cos_t", _p),
                ("sin_t", _p), ("token_pos", _p), ("token_seq", _p), ("seq_slot", _p), ("page_table", _p),
                ("max_pages", _i), ("tiles", _p), ("n_tiles", _i), ("bn", _i * 4), ("pair", _i * 4), ("fuse_rope", _i)]


PROMPT_CALLS = ("mixer norm", "q/k/v projection", "rotation and cache append (0 launches where the projection does it)", "attention", "output projection",
                "feed-forward norm", "gate/up projection", "down projection")


def prompt_entry_points() -> PromptEntryPoints:
    """Addresses of the entry points that the native layer loop calls (their libraries are loaded, and
    compiled first if need be)."""
    def address(lib: str, fn: str) -> int:
        return ctypes.cast(getattr(_lib(lib), fn), ctypes.c_void_p).value
    return PromptEntryPoints(address("elementwise", "dlgo_rmsnorm"), address("gemm_tc", "dlgo_gemm_tc"),
                             address("rope_append", "dlgo_rope_append"),
                             address("attention_prefill_tc", "dlgo_attention_prefill_tc"),
                             address("gemm_tc", "dlgo_gemm_tc_rope"))


def prompt_layers_describe(layers: Sequence[dict]) -> tuple:
    """The host-side descriptor array of a run of layers: (ctypes array, the tensors it points at, which the
    caller keeps alive with it).  Each entry gives ``w_qkv, w_o, w_gate_up, w_down`` (bfloat16, contiguous),
    ``norm1_w, norm2_w`` (float32), ``kpages, vpages`` (bfloat16) and ``eps1, eps2, write_cache``."""
    arr = (PromptLayer * len(layers))()
    keep = []
    for i, L in enumerate(layers):
        for n in ("w_qkv", "w_o", "w_gate_up", "w_down", "kpages", "vpages"):
            _need(L[n], torch.bfloat16, n)
        for n in ("norm1_w", "norm2_w"):
            _need(L[n], torch.float32, n)
        a = arr[i]
        for n in ("w_qkv", "w_o", "w_gate_up", "w_down", "norm1_w", "norm2_w", "kpages", "vpages"):
            setattr(a, n, L[n].data_ptr())
            keep.append(L[n])
        a.eps1, a.eps2 = L["eps1"], L["eps2"]
        a.n_pages, a.write_cache = L["kpages"].shape[0], 1 if L["write_cache"] else 0
    return arr, keep


def prompt_layers(entry: PromptEntryPoints, shape: PromptShape, layers: ctypes.Array, step: PromptStep) -> None:
    """Run ``len(layers)`` pre-norm layers of a prompt step: eight launches a layer (seven where the q/k/v
    projection rotates and appends in its epilogue: ``step.fuse_rope``), issued from one native loop
    (csrc/prompt_layers.cu).  The caller has checked types and sizes of what ``step`` points at."""
    failed = _i(-1)
    n = len(layers)
    st = _lib("prompt_layers").dlgo_prompt_layers(ctypes.byref(entry), ctypes.byref(shape), layers, _i(n),
                                                  ctypes.byref(step), ctypes.byref(failed), _stream())
    if st != 0 and failed.value >= 0:
        _check(st, f"prompt_layers (layer {failed.value // 8} of the run, {PROMPT_CALLS[failed.value % 8]})")
    _check(st, "prompt_layers", (7 if step.fuse_rope else 8) * n)
