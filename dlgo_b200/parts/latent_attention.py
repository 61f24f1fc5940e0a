"""Attention over a cache of latents, without positions.

Every position keeps ONE vector for all heads: ``c = rms(Wd h) * g`` of ``kv_rank`` numbers.  A head's keys
and values are linear in it (``k = Wk c``, ``v = Wv c``), so the cache holds only ``c`` and the kernel never
builds keys or values: ``score = (Wk^T q) . c * scale`` and ``out = Wv (sum_j p_j c_j)``.

Options, all constants of the part:

* ``q_rank``: the queries go through a latent of their own, ``q = Wu rms(Wq h) * gq``; ``None``: ``q = Wq h``
* ``window``: position i sees j with ``0 <= i - j < window``; ``None``: every j <= i
* ``sink``: a learned number per head joins the softmax's denominator as ``exp(sink)`` (no key, no value,
  not scaled)
* ``rope_dim`` r with ``position_encoding``: the down-projection has ``kv_rank + r`` rows; the last r are one key
  part shared by all heads, which turns with the position (neighbouring pairs) and is cached behind the latent;
  a head's query is ``[qk_dim unrotated | r rotated]`` and ``score = (q_u . Wk c + q_r . k_r) * scale``.  The
  kernels stay as they are: a cache row is ``[c | k_r]``, the key matrix of a head becomes ``[[Wk, 0], [0, I]]``
  and its value matrix ``[Wv, 0]``, so the unit block carries the rotated part through the same sums

The down-projections of queries and latents are one contraction with an fp32 result, because their RMS
norms are taken in fp32; scores, softmax and the weighted sum are fp32 in every precision.
"""
from __future__ import annotations

import os
from typing import Any, Callable, Dict, Mapping, Optional

import torch

from ..csrc import kernels as K
from .base import CacheNeed, Mixer, ParamSpec, PositionEncoding
from .linear import ADD_F32, STORE, STORE_F32, Linear
from .registry import MIXERS

_NAMES = {"q": "q_proj.weight", "q_down": "q_a_proj.weight", "q_norm": "q_a_norm.weight", "q_up": "q_b_proj.weight",
          "kv_down": "kv_a_proj.weight", "kv_norm": "kv_a_norm.weight", "k_up": "k_b_proj.weight",
          "v_up": "v_b_proj.weight", "sink": "sinks", "out": "o_proj.weight"}


# prompt steps of at least this many tokens make the step's keys and values and run on the tensor cores
PROMPT_TC_MIN_TOKENS = int(os.environ.get("DLGO_LATENT_TC_MIN_TOKENS", 64))


FEW_TOKENS = 64      # steps of up to this many tokens run the three-launch kernels
SLICE_BLOCKS_PER_SM = int(os.environ.get("DLGO_LATENT_SLICE_BLOCKS", 4))   # blocks of the softmax launch wanted per SM
TILE_BLOCKS_PER_SM = int(os.environ.get("DLGO_LATENT_TILE_BLOCKS", 2))     # ... of the launch that serves all heads from one tile


class LatentAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, qk_dim: int, v_dim: int, kv_rank: int, scale: float,
                 eps: float, q_rank: Optional[int] = None, window: Optional[int] = None, sink: bool = False,
                 cache_group: str = "latent", names: Optional[Mapping[str, str]] = None, rope_dim: int = 0,
                 position_encoding: Optional[str] = None):
        super().__init__(hidden_size=hidden_size, num_heads=num_heads, qk_dim=qk_dim, v_dim=v_dim, kv_rank=kv_rank,
                         scale=scale, eps=eps, q_rank=q_rank, window=window, sink=sink, cache_group=cache_group,
                         names=names, rope_dim=rope_dim, position_encoding=position_encoding)
        if not 0 < kv_rank + rope_dim <= 1024:
            raise ValueError(f"kv_rank (+ rope_dim) must be 1 to 1024, got {kv_rank} + {rope_dim}")
        if rope_dim < 0 or rope_dim % 2 or (rope_dim > 0) != (position_encoding is not None):
            raise ValueError("rope_dim must be even, and positive exactly when a position encoding is named")
        if rope_dim and q_rank is not None:
            raise ValueError("a rotated key part goes with queries projected in one step (q_rank None)")
        if window is not None and window <= 0:
            raise ValueError(f"window must be positive or None, got {window}")
        self.hidden_size, self.n_heads = int(hidden_size), int(num_heads)
        self.qk_dim, self.v_dim, self.kv_rank = int(qk_dim), int(v_dim), int(kv_rank)
        self.q_rank = None if q_rank is None else int(q_rank)
        self.scale, self.eps = float(scale), float(eps)
        self.window = None if window is None else int(window)
        self.has_sink = bool(sink)
        self.cache_group = cache_group
        self.rope_dim = int(rope_dim)
        self.position_encoding = position_encoding
        # what the kernels see: a query head and a cache row carry the rotated part behind their own numbers
        self.q_head = self.qk_dim + self.rope_dim
        self.row = self.kv_rank + self.rope_dim
        self.names = dict(_NAMES)
        self.names.update(names or {})
        self.w_down: Optional[Linear] = None      # rows: query part (q_down or q) | kv_down
        self.w_q_up: Optional[Linear] = None
        self.w_k_up: Optional[torch.Tensor] = None
        self.w_v_up: Optional[torch.Tensor] = None
        self.wo: Optional[Linear] = None
        self.q_norm: Optional[torch.Tensor] = None
        self.kv_norm: Optional[torch.Tensor] = None
        self.sink: Optional[torch.Tensor] = None

    # --------------------------------------------------------------- declarations
    def param_specs(self) -> Dict[str, ParamSpec]:
        n, d, H = self.names, self.hidden_size, self.n_heads
        specs = {
            n["kv_down"]: ParamSpec((self.row, d)),
            n["kv_norm"]: ParamSpec((self.kv_rank,), "one_plus_normal"),
            n["k_up"]: ParamSpec((H * self.qk_dim, self.kv_rank)),
            n["v_up"]: ParamSpec((H * self.v_dim, self.kv_rank)),
            n["out"]: ParamSpec((d, H * self.v_dim)),
        }
        if self.q_rank is not None:
            specs[n["q_down"]] = ParamSpec((self.q_rank, d))
            specs[n["q_norm"]] = ParamSpec((self.q_rank,), "one_plus_normal")
            specs[n["q_up"]] = ParamSpec((H * self.qk_dim, self.q_rank))
        else:
            specs[n["q"]] = ParamSpec((H * self.q_head, d))
        if self.has_sink:
            specs[n["sink"]] = ParamSpec((H,))
        return specs

    def cache_need(self) -> CacheNeed:
        # one "kv head" whose rows are the latents; keys and values are the same plane
        return CacheNeed(self.cache_group, 1, self.row, self.window, planes=1)

    def load(self, get: Callable[[str], torch.Tensor], runtime: Any) -> None:
        n = self.names
        first = get(n["q_down"] if self.q_rank is not None else n["q"])
        self.w_down = Linear(torch.cat([runtime.compute_copy(first), runtime.compute_copy(get(n["kv_down"]))], dim=0),
                             runtime)
        self.kv_norm = get(n["kv_norm"]).to(torch.float32).contiguous()
        if self.q_rank is not None:
            self.q_norm = get(n["q_norm"]).to(torch.float32).contiguous()
            self.w_q_up = Linear(get(n["q_up"]), runtime)
        # one matrix [Wk; Wv]: the per-token kernel reads its halves, a prompt step multiplies by all of it
        wk, wv = runtime.compute_copy(get(n["k_up"])), runtime.compute_copy(get(n["v_up"]))
        if self.rope_dim:
            H, dk, dv, R, r = self.n_heads, self.qk_dim, self.v_dim, self.kv_rank, self.rope_dim
            wide = torch.zeros((H, dk + r, R + r), dtype=wk.dtype, device=wk.device)
            wide[:, :dk, :R] = wk.view(H, dk, R)
            wide[:, dk:, R:] = torch.eye(r, dtype=wk.dtype, device=wk.device)
            wk = wide.view(H * (dk + r), R + r)
            wv = torch.cat([wv, torch.zeros((H * dv, r), dtype=wv.dtype, device=wv.device)], dim=1)
        self.w_kv_up = Linear(torch.cat([wk, wv], dim=0), runtime)
        self.w_k_up = self.w_kv_up.weight[:self.n_heads * self.q_head]
        self.w_v_up = self.w_kv_up.weight[self.n_heads * self.q_head:]
        if self.has_sink:
            self.sink = get(n["sink"]).to(torch.float32).contiguous()
        self.wo = Linear(get(n["out"]), runtime)

    # -------------------------------------------------------------------- forward
    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: Any, cache: Any,
                state: Optional[torch.Tensor], positions: Mapping[str, PositionEncoding]) -> None:
        n_q = self.q_rank if self.q_rank is not None else self.n_heads * self.q_head
        proj = self.w_down(x, STORE_F32)                       # [T, n_q + kv_rank (+ rope_dim)] fp32
        if self.rope_dim:
            pe = positions[self.position_encoding]
            if not pe.interleaved or pe.rotary_dim != self.rope_dim:
                raise ValueError("the rotated part turns in neighbouring pairs, all of it")
            K.latent_rope_append(proj, n_q, self.kv_rank, self.kv_norm, 0, self.n_heads, self.q_head, self.rope_dim,
                                 pe.frequencies, pe.amplitude, self.eps, ctx.token_pos, ctx.token_seq, ctx.seq_slot,
                                 cache.page_table, cache.keys, cache.writes)
            cq = None
        else:
            cq = K.latent_norm_append(proj, n_q, self.kv_rank, self.kv_norm, 0, self.q_rank or 0, self.q_norm,
                                      self.eps, ctx.token_pos, ctx.token_seq, ctx.seq_slot, cache.page_table,
                                      cache.keys, cache.writes)
        q = self.w_q_up(cq, STORE) if self.q_rank is not None else proj[:, :n_q]
        if self.prompt_on_tensor_cores(ctx, cache):
            out = self._prompt_tc(q, ctx, cache)
            self.wo(out, ADD_F32, residual)
            return
        T, H, R = ctx.n_tokens, self.n_heads, self.row
        if T <= FEW_TOKENS and K.latent_attention_tiles_takes(cache.keys.dtype, H, R):
            # decoding: a block per token and slice of its keys serves all heads from one tile of latents; slices
            # so that the GPU has a couple of blocks per SM, of 32 keys or more each
            longest = ctx.capacity if ctx.captured else ctx.max_len
            span = min(longest, self.window) if self.window else longest
            from .tensor_core import sm_count
            n_slices = max(1, min((TILE_BLOCKS_PER_SM * sm_count(x.device)) // T, span // 32, 32))
            out = K.latent_attention_tiles(q, self.w_k_up, self.w_v_up, self.sink, cache.keys, cache.page_table,
                                           ctx.seq_slot, ctx.token_seq, ctx.token_pos, H, self.q_head, self.v_dim,
                                           self.scale, self.window or 0, n_slices,
                                           ctx.scratch("latent_q", T * H * R),
                                           ctx.scratch("latent_parts", T * H * n_slices * (R + 2)))
            self.wo(out, ADD_F32, residual)
            return
        if T <= FEW_TOKENS and K.latent_attention_few_takes(cache.keys.dtype, R):
            # decoding: enough blocks for the whole GPU whatever the batch (a token's keys in slices of 64 or more)
            longest = ctx.capacity if ctx.captured else ctx.max_len
            span = min(longest, self.window) if self.window else longest
            from .tensor_core import sm_count
            n_slices = max(1, min((SLICE_BLOCKS_PER_SM * sm_count(x.device)) // (T * H), span // 32, 32))
            out = K.latent_attention_few(q, self.w_k_up, self.w_v_up, self.sink, cache.keys, cache.page_table,
                                         ctx.seq_slot, ctx.token_seq, ctx.token_pos, H, self.q_head, self.v_dim,
                                         self.scale, self.window or 0, n_slices,
                                         ctx.scratch("latent_q", T * H * R),
                                         ctx.scratch("latent_parts", T * H * n_slices * (R + 2)))
            self.wo(out, ADD_F32, residual)
            return
        out = K.latent_attention(q, self.w_k_up, self.w_v_up, self.sink, cache.keys, cache.page_table, ctx.seq_slot,
                                 ctx.token_seq, ctx.token_pos, self.n_heads, self.q_head, self.v_dim, self.scale,
                                 self.window or 0)
        self.wo(out, ADD_F32, residual)


    # ------------------------------------------------------- prompts on the tensor cores
    def prompt_on_tensor_cores(self, ctx: Any, cache: Any) -> bool:
        """A prompt step in bfloat16 of enough tokens, heads of 64 or 128 with equal key and value sizes."""
        return (not ctx.decode and ctx.n_tokens >= PROMPT_TC_MIN_TOKENS and cache.keys.dtype == torch.bfloat16 and
                self.q_head == self.v_dim and
                K.attention_prefill_tc_takes(torch.bfloat16, self.q_head, cache.page_size))

    def _prompt_tc(self, q: torch.Tensor, ctx: Any, cache: Any) -> torch.Tensor:
        """Keys and values of every position the step's tokens see, made from the cached latents by one
        contraction with [Wk; Wv], then the tensor-core prompt attention over those rows (scores fp32 in tensor
        memory, softmax fp32, probabilities as two bfloat16 terms)."""
        ps = cache.page_size
        pages, table_rows = [], []
        for i, (start, n) in enumerate(zip(ctx.seq_start_host, ctx.seq_ntok_host)):
            first = (max(0, start - self.window + 1) if self.window else 0) // ps
            last = (start + n - 1) // ps
            row = [-1] * (last + 1)
            for lp in range(first, last + 1):
                row[lp] = len(pages)
                pages.append((i, lp, min(ps, start + n - lp * ps)))
            table_rows.append(row)
        width = max(len(r) for r in table_rows)
        meta = torch.tensor([v for p in pages for v in p] + [v for r in table_rows for v in r + [-1] * (width - len(r))],
                            dtype=torch.int32).to(q.device, non_blocking=True)
        n_tmp = len(pages)
        tmp_pages = meta[:3 * n_tmp].view(n_tmp, 3)
        tmp_table = meta[3 * n_tmp:].view(len(table_rows), width)
        seq_rows = ctx._scratch.get("seq_rows")             # sequence i of the step reads row i of the table
        if seq_rows is None or seq_rows.numel() < ctx.n_seqs:
            seq_rows = ctx._scratch["seq_rows"] = torch.arange(max(ctx.n_seqs, 64), dtype=torch.int32, device=q.device)
        latents = K.latent_gather(cache.keys, cache.page_table, tmp_pages, n_tmp, ctx.seq_slot)
        kv = self.w_kv_up(latents, STORE)                      # [pages * 64, H * (qk_dim + v_dim)]
        if q.dtype != torch.bfloat16:
            q = K.bias_act(q, None, K.ACT_NONE, torch.bfloat16)
        tiles, _, _ = ctx.tiles(K.PREFILL_TC_TILE, heaviest_first=True)
        return K.attention_prefill_tc_rows(q, kv, 0, self.n_heads * self.q_head, n_tmp, tmp_table, tiles, seq_rows,
                                           ctx.token_pos, self.n_heads, self.q_head, self.scale, self.window or 0,
                                           self.sink)


MIXERS.register("latent_attention", LatentAttention)
