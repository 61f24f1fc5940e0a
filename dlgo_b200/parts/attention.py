"""Grouped-query attention over the cache, with rotary positions.

Reference (models/llm/forward.go:207-290): q, k, v projections in one dispatch
(:224), rotation of every q and k head at the token's position (:246-252),
append to the cache (:257), per head ``softmax(q.k * scale)`` over positions
``0..pos`` and the weighted sum of values with kv head ``h / (Hq/Hkv)``
(:258-278), output projection (:286); the caller adds the result to the
residual (:163).  Prompts run the same steps over all their positions and read
keys and values back from the cache (models/llm/forward_batch.go:135-210).

Every constant is a parameter: head counts, head size, score scale, an optional
window (keys t > pos - window only), the name of the position encoding to use,
and the cache group the layer's keys and values belong to.
"""
from __future__ import annotations

import os
from typing import Any, Callable, Dict, Mapping, Optional

import torch

from ..csrc import kernels as K
from .base import CacheNeed, Mixer, ParamSpec, PositionEncoding, StateNeed
from .linear import ADD_F32, STORE, STORE_F32, Linear, stack_rows
from .registry import MIXERS

_CLUSTER_MAX = int(os.environ.get("DLGO_ATTN_CLUSTER_MAX", 8))     # slices up to this many combine in a cluster
_MMA_KEYS = int(os.environ.get("DLGO_ATTN_MMA_KEYS", 32))    # keys per warp iteration of the tensor-core decode kernel (0: off)
# few tokens: the projection's K-slices meet in one fp32 sum (reductions at the memory) that is zero between steps
_QKV_SUM = int(os.environ.get("DLGO_ATTN_QKV_SUM", 1))
# ... which the tensor-core decode kernel reads itself: it rotates q and k, appends k and v and clears the sum, so
# the rotation needs no launch of its own.  Measured on a B200 (Llama 3.2 1B sizes): 0.789 -> 0.761 ms a step at
# batch 8, 1.31 -> 1.28 ms at batch 64.
_FUSE_ROPE = int(os.environ.get("DLGO_ATTN_FUSE_ROPE", 1))
_FUSE_ROPE_MAX_HEAD = 64
# prompts: the q|k|v projection's epilogue rotates and appends (0: the rotation kernel runs behind it)
_PROMPT_ROPE = int(os.environ.get("DLGO_PROMPT_ROPE", 1))


_DECODE_BLOCKS = int(os.environ.get("DLGO_ATTN_BLOCKS", 0))   # blocks wanted in flight for decode attention (0: as many as are resident)


def _sm_count(device: torch.device) -> int:
    from .tensor_core import sm_count
    return sm_count(device)


class GQAAttention(Mixer):
    head_multiple = 16      # head sizes this mixer's kernels take

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                 window: Optional[int] = None, position_encoding: Optional[str] = "rope",
                 cache_group: str = "full"):
        super().__init__(hidden_size=hidden_size, num_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=head_dim,
                         scale=scale, window=window, position_encoding=position_encoding, cache_group=cache_group)
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads ({num_heads}) must be a multiple of num_kv_heads ({num_kv_heads})")
        if head_dim % self.head_multiple:
            raise ValueError(f"head_dim must be a multiple of {self.head_multiple}, got {head_dim}")
        if window is not None and window <= 0:
            raise ValueError(f"window must be positive or None, got {window}")
        self.hidden_size = int(hidden_size)
        self.num_heads = int(num_heads)
        self.num_kv_heads = int(num_kv_heads)
        self.head_dim = int(head_dim)
        self.scale = float(scale)
        self.window = None if window is None else int(window)
        self.position_encoding = position_encoding
        self.cache_group = cache_group
        self.chunk: Optional[int] = None      # a subclass may cut the sequence into chunks instead of a window
        self.q_dim = self.num_heads * self.head_dim
        self.kv_dim = self.num_kv_heads * self.head_dim
        self.wqkv: Optional[Linear] = None
        self.wo: Optional[Linear] = None
        self._no_rotation: Optional[torch.Tensor] = None

    # --------------------------------------------------------------- declarations
    def param_specs(self) -> Dict[str, ParamSpec]:
        return {
            "q_proj.weight": ParamSpec((self.q_dim, self.hidden_size)),
            "k_proj.weight": ParamSpec((self.kv_dim, self.hidden_size)),
            "v_proj.weight": ParamSpec((self.kv_dim, self.hidden_size)),
            "o_proj.weight": ParamSpec((self.hidden_size, self.q_dim)),
        }

    def cache_need(self) -> CacheNeed:
        return CacheNeed(self.cache_group, self.num_kv_heads, self.head_dim, self.window)

    def load(self, get: Callable[[str], torch.Tensor], runtime: Any) -> None:
        # one fused projection: rows q | k | v (the reference splits a fused tensor
        # the other way round, models/llm/loader.go:267-279)
        parts = [runtime.compute_copy(get(n)) for n in ("q_proj.weight", "k_proj.weight", "v_proj.weight")]
        self.wqkv = Linear(torch.cat(parts, dim=0), runtime)
        self.wo = Linear(get("o_proj.weight"), runtime)
        self._no_rotation = torch.zeros((1, 1), dtype=torch.float32, device=runtime.device)

    def span(self) -> int:
        """Which keys a query sees besides the causal rule, as the attention kernels take it: a window w as w, chunks
        of c positions as -c, every key as 0."""
        if self.window:
            return self.window
        return -self.chunk if self.chunk else 0

    # -------------------------------------------------------------------- forward
    def _decode_slices(self, ctx: Any, cache: Any, T: int, group: int, pages: int):
        """(page slices per sequence, scratch, counters) of the decode kernels: slices so that every SM has
        several blocks (whole waves: rounded down); 2..8 slices form a thread-block cluster and combine
        through distributed shared memory, more (one very long sequence alone) go through scratch memory."""
        # (as many blocks as are resident at once: four per SM, two for heads above 64, whose kernel takes twice
        # the registers; measured on a B200 at the layer sizes of Llama 3.2 3B, heads of 128, batch 8: 4 slices
        # in one wave 1.83 ms a step, 8 slices in two waves 2.04 ms)
        blocks = _DECODE_BLOCKS or (4 if self.head_dim <= 64 else 2) * _sm_count(cache.keys.device)
        base_blocks = T * self.num_kv_heads * ((group + 3) // 4)
        n_splits = max(1, min(pages, blocks // base_blocks))
        scratch = counters = None
        if n_splits > _CLUSTER_MAX and pages <= 64 and _CLUSTER_MAX > 1:
            n_splits = _CLUSTER_MAX
        if n_splits > _CLUSTER_MAX:
            scratch = ctx.scratch("attention", K.attention_scratch_floats(T, self.num_heads, self.head_dim, n_splits))
            counters = ctx.zeros("attention_counters", T * self.num_kv_heads * ((group + 3) // 4))
        return n_splits, scratch, counters

    def fuses_prompt_rope(self, ctx: Any, cache: Any, positions: Mapping[str, PositionEncoding]) -> bool:
        """Whether this step's q|k|v projection rotates and appends in its own epilogue: a prompt step in
        bfloat16 of more tokens than the few-token kernel takes, whole-head rotation in the split-half pairing,
        heads and pages the tensor-core kernel takes."""
        if ctx.decode or self.position_encoding is None or not _PROMPT_ROPE:
            return False
        pe = positions[self.position_encoding]
        return (pe.rotary_dim == self.head_dim and not pe.interleaved and cache.keys.dtype == torch.bfloat16 and
                self.wqkv.rope_qkv_takes(ctx.n_tokens, self.num_heads, self.num_kv_heads, self.head_dim,
                                         cache.page_size))

    def _decode_plan(self, ctx: Any, cache: Any, act: torch.dtype):
        """(decode kernel?, tensor-core decode kernel?, page slices, scratch, counters, pages of the longest
        sequence) for this step's attention."""
        T = ctx.n_tokens
        group = self.num_heads // self.num_kv_heads
        longest = ctx.capacity if ctx.captured else ctx.max_len
        pages = max(1, (longest + cache.page_size - 1) // cache.page_size)
        decode_kernel = ctx.decode and K.attention_decode_takes(act, self.head_dim, cache.page_size)
        n_splits, scratch, counters = self._decode_slices(ctx, cache, T, group, pages) if decode_kernel else (1, None, None)
        mma = (decode_kernel and _MMA_KEYS > 0 and
               K.attention_decode_mma_takes(act, self.head_dim, cache.page_size, n_splits))
        return decode_kernel, mma, n_splits, scratch, counters, pages

    def _attend(self, qkv: torch.Tensor, ctx: Any, cache: Any, out: torch.Tensor, decode_kernel: bool, mma: bool,
                n_splits: int, scratch: Any, counters: Any, pages: int) -> None:
        """Attention of the step's (rotated) queries, the first columns of ``qkv``'s rows, over the cache,
        into ``out`` [T, heads * head_dim], by whichever kernel takes the step."""
        T = ctx.n_tokens
        x = qkv
        group = self.num_heads // self.num_kv_heads
        if mma:
            K.attention_decode_mma(qkv, qkv.stride(0), T, cache.keys, cache.values, cache.page_table, ctx.seq_slot,
                                   ctx.token_pos, out, self.num_heads, self.num_kv_heads, self.head_dim, self.scale,
                                   self.span(), n_splits, _MMA_KEYS, scratch)
        elif decode_kernel:
            K.attention_decode(qkv, qkv.stride(0), T, cache.keys, cache.values, cache.page_table, ctx.seq_slot,
                               ctx.token_pos, out, self.num_heads, self.num_kv_heads, self.head_dim, self.scale,
                               self.span(), n_splits, scratch, counters)
        elif not ctx.decode and K.attention_prefill_tc_takes(qkv.dtype, self.head_dim, cache.page_size):
            # prompts: 128 query rows per CTA on the tensor cores
            tiles, n_tiles, _ = ctx.tiles(K.PREFILL_TC_TILE, heaviest_first=True)
            K.attention_prefill_tc(qkv, qkv.stride(0), T, cache.keys, cache.values, cache.page_table, tiles,
                                   ctx.seq_slot, ctx.token_pos, out, self.num_heads, self.num_kv_heads,
                                   self.head_dim, self.scale, self.span())
        else:
            qt, gchunk = K.attention_tile_shape(self.head_dim, group, ctx.decode)
            tiles, n_tiles, tile_max = ctx.tiles(qt)
            n_gchunks = (group + gchunk - 1) // gchunk
            base_blocks = n_tiles * self.num_kv_heads * n_gchunks
            target = 2 * _sm_count(x.device)
            n_splits = max(1, min(pages, -(-target // base_blocks))) if ctx.decode else 1
            scratch = None
            if n_splits > 1:
                scratch = ctx.scratch("attention",
                                      K.attention_scratch_floats(T, self.num_heads, self.head_dim, n_splits))
            K.attention(qkv, qkv.stride(0), T, cache.keys, cache.values, cache.page_table, tiles, tile_max,
                        ctx.seq_slot, ctx.token_pos, out, self.num_heads, self.num_kv_heads, self.head_dim,
                        self.scale, self.span(), n_splits, gchunk, scratch)

    def _project_out(self, out: torch.Tensor, residual: torch.Tensor, ctx: Any) -> None:
        parts = self.wo.partials(out, for_residual=True) if hasattr(ctx, "defer") else None
        if parts is not None:
            ctx.defer(residual, parts)      # the next norm adds the slices to the residual
        else:
            self.wo(out, ADD_F32, residual)

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: Any, cache: Any,
                state: Optional[torch.Tensor], positions: Mapping[str, PositionEncoding]) -> None:
        T = ctx.n_tokens
        group = self.num_heads // self.num_kv_heads
        if self.position_encoding is not None:
            pe = positions[self.position_encoding]
            cos, sin, rot, inter = pe.cos, pe.sin, pe.rotary_dim, pe.interleaved
        else:
            cos = sin = self._no_rotation
            rot, inter = 0, False
        act = self.wqkv.weight.dtype
        n_cols = self.q_dim + 2 * self.kv_dim
        # bfloat16, common head sizes, one token per sequence: scores and weighted sum on the tensor cores
        decode_kernel, mma, n_splits, scratch, counters, pages = self._decode_plan(ctx, cache, act)
        out = torch.empty((T, self.q_dim), dtype=act, device=x.device)
        qkv = None
        rotated = False
        if _QKV_SUM and self.wqkv.sums_slices_at_memory(T):
            # few tokens: the projection's K-slices add themselves, at the memory, into one fp32 sum that is zero
            # between steps; whoever rotates reads it once and leaves zeros behind
            qkv_sum = ctx.zeros(f"qkv_sum{n_cols}", T * n_cols, torch.float32)[:T * n_cols].view(1, T, n_cols)
            # (heads of 64 only: at 128 the kernel is at its register limit and the fused form measured 2 to 3 %
            # slower in a whole step at the layer sizes of Llama 3.2 3B and 3.1 8B, batch 8)
            fuse = (mma and _FUSE_ROPE and n_splits <= 8 and self.head_dim <= _FUSE_ROPE_MAX_HEAD and
                    K.attention_decode_mma_fuses_rope(self.num_heads, self.num_kv_heads, self.head_dim, rot, inter))
            self.wqkv(x, ADD_F32, qkv_sum[0])
            if fuse:
                # the decode kernel rotates, appends and clears itself: no launch for the rotation
                K.attention_decode_mma(None, n_cols, T, cache.keys, cache.values, cache.page_table, ctx.seq_slot,
                                       ctx.token_pos, out, self.num_heads, self.num_kv_heads, self.head_dim,
                                       self.scale, self.span(), n_splits, _MMA_KEYS, None, qkv_sum, cos, sin,
                                       cache.writes, clear_parts=True)
                rotated = True
            else:
                qkv = torch.empty((T, n_cols), dtype=x.dtype, device=x.device)
                K.rope_append(qkv, cos, sin, ctx.token_pos, ctx.token_seq, ctx.seq_slot, cache.page_table, cache.keys,
                              cache.values, self.num_heads, self.num_kv_heads, self.head_dim, rot, inter, cache.writes,
                              qkv_sum, True)
        elif self.fuses_prompt_rope(ctx, cache, positions):
            # prompts: the projection's epilogue rotates q and k and appends k and v (no launch for that, and
            # one rounding to bfloat16 instead of two)
            rope = K.rope_args(cos, sin, ctx.token_pos, ctx.token_seq, ctx.seq_slot, cache.page_table, cache.keys,
                               cache.values, self.num_heads, self.num_kv_heads, self.head_dim, cache.writes)
            qkv = self.wqkv.rope_qkv(x, rope)
        else:
            # ... or leaves its K-slices unsummed for the rotation to add in order; else the finished product
            qkv_parts = self.wqkv.partials(x, single_ok=False)
            qkv = (self.wqkv(x, STORE) if qkv_parts is None else
                   torch.empty((T, n_cols), dtype=x.dtype, device=x.device))
            K.rope_append(qkv, cos, sin, ctx.token_pos, ctx.token_seq, ctx.seq_slot, cache.page_table, cache.keys,
                          cache.values, self.num_heads, self.num_kv_heads, self.head_dim, rot, inter, cache.writes,
                          qkv_parts, False)
        if not rotated:
            self._attend(qkv, ctx, cache, out, decode_kernel, mma, n_splits, scratch, counters, pages)
        self._project_out(out, residual, ctx)


class KeysAsValuesAttention(GQAAttention):
    """Grouped-query attention whose values are its keys as projected: there is no value projection, and what a
    position contributes to the weighted sum is its key BEFORE the head norm and the rotation.

        q = Wq h (+ bq),  k = Wk h (+ bk),  v = k
        q, k <- head norm (per head: u / sqrt(mean(u^2) + eps) * w, one weight of head_dim numbers shared by all
                heads; ``head_norm``), then the rotation of the first numbers of each head (the position encoding
                named by ``position_encoding`` gives how many and at which frequencies)
        out  = Wo softmax(q . k * scale) v            (causal, over the cache)

    The cache keeps two rows per position and kv head like any grouped-query mixer: the normed and rotated key,
    and the key as projected (the value).  The projection's result stays fp32 until bias, norm and rotation are
    done (one kernel, which also appends to the cache); scores, softmax and the weighted sum run in the same
    attention kernels as :class:`GQAAttention`.  ``names``: tensor names below the part's prefix."""

    head_multiple = 8       # (16 bytes of bfloat16: what the general attention kernel reads at a time)

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                 bias: bool = False, head_norm: bool = False, eps: float = 1e-6, window: Optional[int] = None,
                 position_encoding: Optional[str] = None, cache_group: str = "full",
                 names: Optional[Mapping[str, str]] = None):
        # A head size that is no multiple of 8 is laid out as the next multiple: the projection gets zero rows, the
        # output projection zero columns, so the added numbers are zeros everywhere (queries, both cache rows,
        # attention's result) and change neither a score nor a sum; the head norm's mean runs over the true size.
        self.true_head_dim = int(head_dim)
        padded = -(-self.true_head_dim // self.head_multiple) * self.head_multiple
        super().__init__(hidden_size, num_heads, num_kv_heads, padded, scale, window, position_encoding, cache_group)
        self.params.update(head_dim=head_dim, bias=bias, head_norm=head_norm, eps=eps, names=names)
        self.bias = bool(bias)
        self.head_norm = bool(head_norm)
        self.eps = float(eps)
        self.names = {"q": "q_proj.weight", "k": "k_proj.weight", "q_bias": "q_proj.bias", "k_bias": "k_proj.bias",
                      "q_norm": "q_norm.weight", "k_norm": "k_norm.weight", "out": "o_proj.weight"}
        self.names.update(names or {})
        self.wqk: Optional[Linear] = None
        self.b_qk: Optional[torch.Tensor] = None
        self.w_qnorm: Optional[torch.Tensor] = None
        self.w_knorm: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        n, hd = self.names, self.true_head_dim
        q_dim, kv_dim = self.num_heads * hd, self.num_kv_heads * hd
        specs = {n["q"]: ParamSpec((q_dim, self.hidden_size)), n["k"]: ParamSpec((kv_dim, self.hidden_size)),
                 n["out"]: ParamSpec((self.hidden_size, q_dim))}
        if self.bias:
            specs[n["q_bias"]] = ParamSpec((q_dim,))
            specs[n["k_bias"]] = ParamSpec((kv_dim,))
        if self.head_norm:
            specs[n["q_norm"]] = ParamSpec((hd,), "one_plus_normal")
            specs[n["k_norm"]] = ParamSpec((hd,), "one_plus_normal")
        return specs

    def _pad_heads(self, t: torch.Tensor, dim: int) -> torch.Tensor:
        """``t`` with every head's ``true_head_dim`` entries along ``dim`` followed by zeros up to ``head_dim``."""
        hd, hp = self.true_head_dim, self.head_dim
        if hd == hp:
            return t
        shape = list(t.shape)
        heads = shape[dim] // hd
        t = t.reshape(shape[:dim] + [heads, hd] + shape[dim + 1:])
        pad = torch.zeros(shape[:dim] + [heads, hp - hd] + shape[dim + 1:], dtype=t.dtype, device=t.device)
        return torch.cat([t, pad], dim=dim + 1).reshape(shape[:dim] + [heads * hp] + shape[dim + 1:])

    def load(self, get: Callable[[str], torch.Tensor], runtime: Any) -> None:
        n = self.names
        self.wqk = Linear(torch.cat([self._pad_heads(runtime.compute_copy(get(n["q"])), 0),
                                     self._pad_heads(runtime.compute_copy(get(n["k"])), 0)], dim=0), runtime)
        self.wo = Linear(self._pad_heads(runtime.compute_copy(get(n["out"])), 1).contiguous(), runtime)
        if self.bias:       # added to the fp32 result of the projection
            self.b_qk = torch.cat([self._pad_heads(get(n["q_bias"]).to(torch.float32), 0),
                                   self._pad_heads(get(n["k_bias"]).to(torch.float32), 0)]).contiguous()
        if self.head_norm:  # norms are 32-bit in every precision
            self.w_qnorm = self._pad_heads(get(n["q_norm"]).to(torch.float32), 0).contiguous()
            self.w_knorm = self._pad_heads(get(n["k_norm"]).to(torch.float32), 0).contiguous()

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: Any, cache: Any,
                state: Optional[torch.Tensor], positions: Mapping[str, PositionEncoding]) -> None:
        T = ctx.n_tokens
        freq, rot = None, 0
        if self.position_encoding is not None:
            pe = positions[self.position_encoding]
            if getattr(pe, "interleaved", False) or getattr(pe, "amplitude", 1.0) != 1.0:
                raise ValueError("this mixer's kernel rotates pairs (i, i + rot/2) with plain cosine and sine")
            freq, rot = pe.frequencies, pe.rotary_dim
        act = self.wqk.weight.dtype
        n_cols = self.q_dim + self.kv_dim
        decode_kernel, mma, n_splits, scratch, counters, pages = self._decode_plan(ctx, cache, act)
        if _QKV_SUM and self.wqk.sums_slices_at_memory(T):
            # few tokens: the projection's K-slices add themselves into one fp32 sum that is zero between steps;
            # the norm-and-rotation kernel reads it once and leaves zeros behind
            proj = ctx.zeros(f"qk_sum{n_cols}", T * n_cols, torch.float32)[:T * n_cols].view(T, n_cols)
            self.wqk(x, ADD_F32, proj)
            clear = True
        else:
            proj = self.wqk(x, STORE_F32)
            clear = False
        q = K.headnorm_rope_append(proj, self.b_qk, self.w_qnorm, self.w_knorm, self.eps, freq, rot, ctx.token_pos,
                                   ctx.token_seq, ctx.seq_slot, cache.page_table, cache.keys, cache.values,
                                   self.num_heads, self.num_kv_heads, self.head_dim, True, cache.writes, clear,
                                   norm_dim=self.true_head_dim)
        out = torch.empty((T, self.q_dim), dtype=act, device=x.device)
        self._attend(q, ctx, cache, out, decode_kernel, mma, n_splits, scratch, counters, pages)
        self._project_out(out, residual, ctx)


class WholeNormAttention(GQAAttention):
    """Grouped-query softmax attention without positions, whose queries and keys are normed over their WHOLE
    projection, whose keys and values may differ in size, and whose heads are gated:

        q = Wq h,  k = Wk h,  v = Wv h                        (H x qk_dim, G x qk_dim, G x v_dim numbers)
        q <- q / sqrt(mean over all H qk_dim numbers of q^2 + eps) * wq      (``qk_norm``; likewise k with wk)
        out_h = softmax over the visible keys of (q_h . k_g * scale) v_g     (g = h // (H / G); ``window`` w: keys j
                                                                             with 0 <= i - j < w)
        out_h <- out_h * sigmoid(Wg h)_h                                     (``head_gate``: one number per head)
        result = Wo [out_1 .. out_H] * out_scale

    Heads are laid out ``head_dim`` = max(qk_dim, v_dim) (rounded up to a multiple of 8) numbers wide with zeros
    behind their own numbers, so that keys and values share the page shape and the kernels of
    :class:`GQAAttention` run unchanged; the output projection gets zero columns.  The projection's result stays
    fp32 until norm and gate are done (one kernel, which also appends to the cache).  ``names``: tensor names
    below the part's prefix."""

    head_multiple = 8

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, qk_dim: int, v_dim: int, scale: float,
                 eps: float = 1e-6, window: Optional[int] = None, qk_norm: bool = True, head_gate: bool = False,
                 cache_group: str = "full", out_scale: float = 1.0, names: Optional[Mapping[str, str]] = None):
        self.qk_dim, self.v_dim = int(qk_dim), int(v_dim)
        if self.qk_dim <= 0 or self.v_dim <= 0:
            raise ValueError("qk_dim and v_dim must be positive")
        padded = -(-max(self.qk_dim, self.v_dim) // self.head_multiple) * self.head_multiple
        super().__init__(hidden_size, num_heads, num_kv_heads, padded, scale, window, None, cache_group)
        self.params = dict(hidden_size=hidden_size, num_heads=num_heads, num_kv_heads=num_kv_heads, qk_dim=qk_dim,
                           v_dim=v_dim, scale=scale, eps=eps, window=window, qk_norm=qk_norm, head_gate=head_gate,
                           cache_group=cache_group, out_scale=out_scale, names=names)
        self.eps = float(eps)
        self.qk_norm, self.head_gate = bool(qk_norm), bool(head_gate)
        self.out_scale = float(out_scale)
        self.names = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "q_norm": "q_norm.weight",
                      "k_norm": "k_norm.weight", "gate": "g_proj.weight", "out": "o_proj.weight"}
        self.names.update(names or {})
        self.w_in: Optional[Linear] = None        # rows q | k | v | gate
        self.w_qnorm: Optional[torch.Tensor] = None
        self.w_knorm: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        n, d = self.names, self.hidden_size
        H, G, dk, dv = self.num_heads, self.num_kv_heads, self.qk_dim, self.v_dim
        specs = {n["q"]: ParamSpec((H * dk, d)), n["k"]: ParamSpec((G * dk, d)), n["v"]: ParamSpec((G * dv, d)),
                 n["out"]: ParamSpec((d, H * dv))}
        if self.qk_norm:
            specs[n["q_norm"]] = ParamSpec((H * dk,), "one_plus_normal")
            specs[n["k_norm"]] = ParamSpec((G * dk,), "one_plus_normal")
        if self.head_gate:
            specs[n["gate"]] = ParamSpec((H, d))
        return specs

    def load(self, get: Callable[[str], torch.Tensor], runtime: Any) -> None:
        n = self.names
        rows = [runtime.compute_copy(get(n[k])) for k in ("q", "k", "v")]
        if self.head_gate:
            rows.append(runtime.compute_copy(get(n["gate"])))
        self.w_in = Linear(stack_rows(rows), runtime)
        wo = runtime.compute_copy(get(n["out"]))
        hd, dv, H = self.head_dim, self.v_dim, self.num_heads
        if dv != hd:        # zero columns where the heads' layout has zeros
            wide = torch.zeros((wo.shape[0], H, hd), dtype=wo.dtype, device=wo.device)
            wide[:, :, :dv] = wo.view(wo.shape[0], H, dv)
            wo = wide.view(wo.shape[0], H * hd)
        self.wo = Linear(wo.contiguous(), runtime)
        if self.qk_norm:    # norms are 32-bit in every precision
            self.w_qnorm = get(n["q_norm"]).to(torch.float32).contiguous()
            self.w_knorm = get(n["k_norm"]).to(torch.float32).contiguous()

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: Any, cache: Any,
                state: Optional[torch.Tensor], positions: Mapping[str, PositionEncoding]) -> None:
        T = ctx.n_tokens
        act = self.w_in.weight.dtype
        n_cols = self.w_in.out_features
        decode_kernel, mma, n_splits, scratch, counters, pages = self._decode_plan(ctx, cache, act)
        if _QKV_SUM and self.w_in.sums_slices_at_memory(T):
            # few tokens: the projection's K-slices add themselves into one fp32 sum that is zero between steps;
            # the norm-and-append kernel reads it once and leaves zeros behind
            proj = ctx.zeros(f"qkvg_sum{n_cols}", T * n_cols, torch.float32)[:T * n_cols].view(T, n_cols)
            self.w_in(x, ADD_F32, proj)
            clear = True
        else:
            proj = self.w_in(x, STORE_F32)
            clear = False
        q, gate = K.wholenorm_append(proj, self.w_qnorm, self.w_knorm, self.eps, ctx.token_pos, ctx.token_seq,
                                     ctx.seq_slot, cache.page_table, cache.keys, cache.values, self.num_heads,
                                     self.num_kv_heads, self.qk_dim, self.v_dim, self.head_gate, self.out_scale,
                                     cache.writes, clear, act)
        out = torch.empty((T, self.q_dim), dtype=act, device=x.device)
        self._attend(q, ctx, cache, out, decode_kernel, mma, n_splits, scratch, counters, pages)
        if gate is None and self.out_scale != 1.0:      # no gates to carry the constant factor
            gate = torch.full((T, self.num_heads), self.out_scale, dtype=torch.float32, device=x.device)
        if gate is not None:
            K.scale_heads(out, gate, self.head_dim)
        self._project_out(out, residual, ctx)


_WHOLE_SEQUENCE = 1 << 30


class ShortConvAttention(GQAAttention):
    """Grouped-query softmax attention whose projections carry biases and pass through a short causal convolution
    over time before the rotation, whose keys and values may differ in size, and whose mask may be cut into chunks:

        q = Wq h + bq,  k = Wk h + bk,  v = Wv h + bv                 (``bias``; H x qk_dim, G x qk_dim, G x v_dim)
        u_t <- sum_j taps[c, j] * u_(t - n + 1 + j)  per channel c    (``conv_taps`` n > 1; zeros before the sequence)
        q, k: the rotation named by ``position_encoding`` (neighbouring pairs of the first numbers of each head)
        out_h = softmax over the visible keys of (q_h . k_g * scale) v_g     g = h // (H / G)
        visible: j <= i and, with ``window`` w, i - j < w; or, with ``chunk`` c, floor(i / c) = floor(j / c)
        result = Wo [out_1 .. out_H] + bo

    The sequence's last n - 1 projected rows (with their biases, fp32) are its state.  Heads are laid out
    ``head_dim`` = max(qk_dim, v_dim) (rounded up to a multiple of 8) numbers wide with zeros behind their own
    numbers, so that keys and values share the page shape and the kernels of :class:`GQAAttention` run unchanged.
    The projection's result stays fp32 until bias, convolution and rotation are done (one kernel, which also
    appends to the cache; a second small one keeps the state).  A chunked mixer keeps all its pages: the cache
    manager's window bookkeeping is for sliding windows.  ``names``: tensor names below the part's prefix."""

    head_multiple = 8
    can_defer_bias = True       # a caller may add :attr:`output_bias` itself, in its next pass over the result

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, qk_dim: int, v_dim: int, scale: float,
                 bias: bool = False, conv_taps: Optional[int] = None, window: Optional[int] = None,
                 chunk: Optional[int] = None, position_encoding: Optional[str] = None, cache_group: str = "full",
                 names: Optional[Mapping[str, str]] = None):
        self.qk_dim, self.v_dim = int(qk_dim), int(v_dim)
        if self.qk_dim <= 0 or self.v_dim <= 0:
            raise ValueError("qk_dim and v_dim must be positive")
        if window is not None and chunk is not None:
            raise ValueError("a window or chunks, not both")
        if chunk is not None and chunk <= 0:
            raise ValueError(f"chunk must be positive or None, got {chunk}")
        taps = int(conv_taps or 1)          # (None: no convolution and no taps in the file; 1: one tap per channel)
        if not 1 <= taps <= K.CONV_MAX_TAPS:
            raise ValueError(f"conv_taps must be 1 to {K.CONV_MAX_TAPS}, got {conv_taps}")
        padded = -(-max(self.qk_dim, self.v_dim) // self.head_multiple) * self.head_multiple
        super().__init__(hidden_size, num_heads, num_kv_heads, padded, scale, window, position_encoding, cache_group)
        self.params = dict(hidden_size=hidden_size, num_heads=num_heads, num_kv_heads=num_kv_heads, qk_dim=qk_dim,
                           v_dim=v_dim, scale=scale, bias=bias, conv_taps=conv_taps, window=window, chunk=chunk,
                           position_encoding=position_encoding, cache_group=cache_group, names=names)
        self.chunk = None if chunk is None else int(chunk)
        self.bias = bool(bias)
        self.taps = taps
        self.has_conv = conv_taps is not None and int(conv_taps) >= 1
        self.channels = (self.num_heads + self.num_kv_heads) * self.qk_dim + self.num_kv_heads * self.v_dim
        self.names = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "out": "o_proj.weight",
                      "q_bias": "q_proj.bias", "k_bias": "k_proj.bias", "v_bias": "v_proj.bias",
                      "out_bias": "o_proj.bias", "q_conv": "q_conv.weight", "k_conv": "k_conv.weight",
                      "v_conv": "v_conv.weight"}
        self.names.update(names or {})
        self.w_in: Optional[Linear] = None        # rows q | k | v
        self.b_in: Optional[torch.Tensor] = None
        self.output_bias: Optional[torch.Tensor] = None
        self.w_taps: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        n, d = self.names, self.hidden_size
        H, G, dk, dv = self.num_heads, self.num_kv_heads, self.qk_dim, self.v_dim
        sizes = {"q": H * dk, "k": G * dk, "v": G * dv}
        specs = {n[key]: ParamSpec((rows, d)) for key, rows in sizes.items()}
        specs[n["out"]] = ParamSpec((d, H * dv))
        if self.bias:
            for key, rows in sizes.items():
                specs[n[key + "_bias"]] = ParamSpec((rows,))
            specs[n["out_bias"]] = ParamSpec((d,))
        if self.has_conv:
            for key, rows in sizes.items():
                specs[n[key + "_conv"]] = ParamSpec((rows, self.taps), "last_one_plus_normal")
        return specs

    def cache_need(self) -> CacheNeed:
        return CacheNeed(self.cache_group, self.num_kv_heads, self.head_dim, self.window)

    def state_need(self) -> Optional[StateNeed]:
        return StateNeed(((self.taps - 1) * self.channels,), torch.float32) if self.taps > 1 else None

    def load(self, get: Callable[[str], torch.Tensor], runtime: Any) -> None:
        n = self.names
        self.w_in = Linear(stack_rows([runtime.compute_copy(get(n[key])) for key in ("q", "k", "v")]), runtime)
        wo = runtime.compute_copy(get(n["out"]))
        hd, dv, H = self.head_dim, self.v_dim, self.num_heads
        if dv != hd:        # zero columns where the heads' layout has zeros
            wide = torch.zeros((wo.shape[0], H, hd), dtype=wo.dtype, device=wo.device)
            wide[:, :, :dv] = wo.view(wo.shape[0], H, dv)
            wo = wide.view(wo.shape[0], H * hd)
        self.wo = Linear(wo.contiguous(), runtime)
        if self.bias:       # added in fp32: to the projection's fp32 result, and to the fp32 sum the mixer adds into
            self.b_in = torch.cat([get(n[key + "_bias"]).to(torch.float32) for key in ("q", "k", "v")]).contiguous()
            self.output_bias = get(n["out_bias"]).to(torch.float32).contiguous()
        if self.has_conv:
            self.w_taps = torch.cat([get(n[key + "_conv"]).to(torch.float32) for key in ("q", "k", "v")],
                                    dim=0).contiguous()

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: Any, cache: Any,
                state: Optional[torch.Tensor], positions: Mapping[str, PositionEncoding],
                defer_bias: bool = False) -> None:
        """``defer_bias``: the caller adds :attr:`output_bias` itself."""
        T = ctx.n_tokens
        act = self.w_in.weight.dtype
        freq, rot, amplitude = None, 0, 1.0
        if self.position_encoding is not None:
            pe = positions[self.position_encoding]
            if not pe.interleaved:
                raise ValueError("this mixer's kernel rotates neighbouring pairs: the encoding must be 'interleaved'")
            freq, rot, amplitude = pe.frequencies, pe.rotary_dim, pe.amplitude
        tiles, n_tiles = None, 0
        if self.taps > 1:
            if state is None:
                raise RuntimeError("a mixer with a convolution over time needs its state")
            state = state.view(state.shape[0], -1)
            tiles, n_tiles, _ = ctx.tiles(1 if ctx.decode else _WHOLE_SEQUENCE)
        decode_kernel, mma, n_splits, scratch, counters, pages = self._decode_plan(ctx, cache, act)
        n_cols = self.w_in.out_features
        clear = (ctx.decode and _QKV_SUM and self.w_in.sums_slices_at_memory(T) and
                 K.conv_rope_append_clears(self.qk_dim, self.v_dim, self.head_dim, n_cols, self.taps))
        if clear:
            # decoding: the projection's K-slices add themselves into one fp32 sum that is zero between steps; the
            # kernel behind it reads a token's row once and leaves zeros
            proj = ctx.zeros(f"qkv_conv_sum{n_cols}", T * n_cols, torch.float32)[:T * n_cols].view(T, n_cols)
            self.w_in(x, ADD_F32, proj)
        else:
            proj = self.w_in(x, STORE_F32)
        q = K.conv_rope_append(proj, self.b_in, self.w_taps, state, freq, rot, amplitude, ctx.token_pos, ctx.token_seq,
                               ctx.seq_slot, cache.page_table, cache.keys, cache.values, self.num_heads,
                               self.num_kv_heads, self.qk_dim, self.v_dim, tiles, n_tiles, cache.writes, ctx.decode, clear)
        out = torch.empty((T, self.q_dim), dtype=act, device=x.device)
        self._attend(q, ctx, cache, out, decode_kernel, mma, n_splits, scratch, counters, pages)
        if self.output_bias is not None and not defer_bias:
            K.bias_act(residual, self.output_bias, K.ACT_NONE, torch.float32, in_place=True)
        self.wo(out, ADD_F32, residual)


MIXERS.register("gqa_attention", GQAAttention)
MIXERS.register("short_conv_attention", ShortConvAttention)
MIXERS.register("wholenorm_attention", WholeNormAttention)
MIXERS.register("keys_as_values_attention", KeysAsValuesAttention)
