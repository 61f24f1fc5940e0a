"""Linear attention with a fixed decay per head over a fixed-size state: "lightning attention", and retention.

Per head, with ``q = silu(Wq h)``, ``k = silu(Wk h)`` (``qk_dim`` numbers) and ``v = silu(Wv h)``
(``v_dim`` numbers): ``S_t = decay * S_(t-1) + k_t v_t^T`` and ``o_t = S_t^T q_t``, no other scale.  The heads'
outputs side by side are RMS-normed together (weight ``norm``), multiplied by ``sigmoid(Wg h)`` and projected
by ``Wo``.  The state [heads, qk_dim, v_dim] is fp32, zero at a sequence's start, and is carried in the
sequence's slot of the state area from step to step; no position is cached.

q, k, v and the gate come from one contraction with an fp32 result; silu, decay, state, norm and gate are
computed in fp32 in every precision.

:class:`Retention` is the same recurrence with other surroundings: ``q = Wq h`` and ``k = Wk h`` without an
activation but with rotary positions (and a constant factor on k), ``v = Wv h``; every head's output is divided by
its own root mean square (no weight) and multiplied by ``silu(Wg h)`` before ``Wo``.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Mapping, Optional, Sequence

import torch

from ..csrc import kernels as K
from .base import Mixer, ParamSpec, PositionEncoding, StateNeed
from .linear import ADD_F32, STORE_F32, Linear, stack_rows
from .registry import MIXERS

_NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "gate": "g_proj.weight",
          "out": "o_proj.weight", "norm": "norm.weight"}
_WHOLE_SEQUENCE = 1 << 30      # a "tile" as long as any sequence's tokens of one step
SEGMENT = 128                  # tokens of a segment where a prompt's segments run side by side


class LightningAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, qk_dim: int, v_dim: int, decay: Sequence[float], eps: float,
                 names: Optional[Mapping[str, str]] = None):
        super().__init__(hidden_size=hidden_size, num_heads=num_heads, qk_dim=qk_dim, v_dim=v_dim, decay=tuple(decay),
                         eps=eps, names=names)
        if len(decay) != num_heads:
            raise ValueError(f"one decay per head: {len(decay)} for {num_heads} heads")
        self.hidden_size, self.n_heads = int(hidden_size), int(num_heads)
        self.qk_dim, self.v_dim = int(qk_dim), int(v_dim)
        self.decay_values = tuple(float(x) for x in decay)
        self.eps = float(eps)
        self.names = dict(_NAMES)
        self.names.update(names or {})
        self.w_in: Optional[Linear] = None        # rows q | k | v | gate
        self.wo: Optional[Linear] = None
        self.norm: Optional[torch.Tensor] = None
        self.decay: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        n, d, H = self.names, self.hidden_size, self.n_heads
        return {
            n["q"]: ParamSpec((H * self.qk_dim, d)), n["k"]: ParamSpec((H * self.qk_dim, d)),
            n["v"]: ParamSpec((H * self.v_dim, d)), n["gate"]: ParamSpec((H * self.v_dim, d)),
            n["out"]: ParamSpec((d, H * self.v_dim)), n["norm"]: ParamSpec((H * self.v_dim,), "one_plus_normal"),
        }

    def state_need(self) -> StateNeed:
        return StateNeed((self.n_heads, self.qk_dim, self.v_dim), torch.float32)

    def load(self, get: Callable[[str], torch.Tensor], runtime: Any) -> None:
        n = self.names
        self.w_in = Linear(torch.cat([runtime.compute_copy(get(n[k])) for k in ("q", "k", "v", "gate")], dim=0), runtime)
        self.wo = Linear(get(n["out"]), runtime)
        self.norm = get(n["norm"]).to(torch.float32).contiguous()
        self.decay = torch.tensor(self.decay_values, dtype=torch.float64).to(torch.float32).to(runtime.device)

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: Any, cache: Any,
                state: Optional[torch.Tensor], positions: Mapping[str, PositionEncoding]) -> None:
        if state is None:
            raise RuntimeError("lightning attention needs its state")
        H, dk, dv = self.n_heads, self.qk_dim, self.v_dim
        proj = self.w_in(x, STORE_F32)                      # [T, 2 H dk + 2 H dv] fp32
        if K.lightning_segments_takes(dk):
            # the state's columns in registers; a prompt's segments side by side
            tiles, n_tiles, _ = ctx.tiles(1 if ctx.decode else SEGMENT)
            direct = ctx.decode or n_tiles == ctx.n_seqs
            scratch = None if direct else ctx.scratch("lightning_segments", 2 * n_tiles * H * dk * dv)
            o = K.lightning_segments(proj, 0, H * dk, 2 * H * dk, tiles, n_tiles, direct, ctx.seq_slot, self.decay,
                                     state, scratch, H, dk, dv)
        else:
            tiles, n_seqs, _ = ctx.tiles(1 if ctx.decode else _WHOLE_SEQUENCE)
            o = K.lightning_scan(proj, 0, H * dk, 2 * H * dk, tiles, n_seqs, ctx.seq_slot, self.decay, state, H, dk, dv)
        a = K.gated_rmsnorm(o, proj[:, 2 * H * dk + H * dv:], self.norm, self.eps, self.wo.weight.dtype)
        self.wo(a, ADD_F32, residual)


class Retention(Mixer):
    """``S_t = decay_h S_(t-1) + k_t v_t^T``, ``o_t = S_t^T q_t`` per head, with q and k turned by the position
    (``position_encoding`` names rotary frequencies; None: no rotation), k multiplied by ``k_scale`` after the
    rotation, each head's o divided by its root mean square (``eps``), the heads side by side multiplied by
    ``silu(Wg h)`` and projected by ``Wo``.  ``out_scale``: a constant factor on the result (for a mixer that is one
    of several whose results are added).  ``names``: tensor names below the part's prefix."""

    def __init__(self, hidden_size: int, num_heads: int, qk_dim: int, v_dim: int, decay: Sequence[float], eps: float,
                 position_encoding: Optional[str] = None, k_scale: float = 1.0, out_scale: float = 1.0,
                 names: Optional[Mapping[str, str]] = None):
        super().__init__(hidden_size=hidden_size, num_heads=num_heads, qk_dim=qk_dim, v_dim=v_dim, decay=tuple(decay),
                         eps=eps, position_encoding=position_encoding, k_scale=k_scale, out_scale=out_scale, names=names)
        if len(decay) != num_heads:
            raise ValueError(f"one decay per head: {len(decay)} for {num_heads} heads")
        self.hidden_size, self.n_heads = int(hidden_size), int(num_heads)
        self.qk_dim, self.v_dim = int(qk_dim), int(v_dim)
        self.decay_values = tuple(float(x) for x in decay)
        self.eps = float(eps)
        self.position_encoding = position_encoding
        self.k_scale, self.out_scale = float(k_scale), float(out_scale)
        self.names = {k: v for k, v in _NAMES.items() if k != "norm"}
        self.names.update(names or {})
        self.w_in: Optional[Linear] = None        # rows q | k | v | gate
        self.wo: Optional[Linear] = None
        self.decay: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        n, d, H = self.names, self.hidden_size, self.n_heads
        return {
            n["q"]: ParamSpec((H * self.qk_dim, d)), n["k"]: ParamSpec((H * self.qk_dim, d)),
            n["v"]: ParamSpec((H * self.v_dim, d)), n["gate"]: ParamSpec((H * self.v_dim, d)),
            n["out"]: ParamSpec((d, H * self.v_dim)),
        }

    def state_need(self) -> StateNeed:
        return StateNeed((self.n_heads, self.qk_dim, self.v_dim), torch.float32)

    def load(self, get: Callable[[str], torch.Tensor], runtime: Any) -> None:
        n = self.names
        self.w_in = Linear(stack_rows(runtime.compute_copy(get(n[k])) for k in ("q", "k", "v", "gate")), runtime)
        self.wo = Linear(get(n["out"]), runtime)
        self.decay = torch.tensor(self.decay_values, dtype=torch.float64).to(torch.float32).to(runtime.device)

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: Any, cache: Any,
                state: Optional[torch.Tensor], positions: Mapping[str, PositionEncoding]) -> None:
        if state is None:
            raise RuntimeError("retention needs its state")
        H, dk, dv = self.n_heads, self.qk_dim, self.v_dim
        proj = self.w_in(x, STORE_F32)                      # [T, 2 H dk + 2 H dv (+ padding)] fp32
        freq, rot = None, 0
        if self.position_encoding is not None:
            pe = positions[self.position_encoding]
            if getattr(pe, "interleaved", False) or getattr(pe, "amplitude", 1.0) != 1.0:
                raise ValueError("this mixer's kernel rotates pairs (i, i + rot/2) with plain cosine and sine")
            freq, rot = pe.frequencies, pe.rotary_dim
        if rot or self.k_scale != 1.0:
            K.rotate_scale(proj, 0, H * dk, freq, rot, ctx.token_pos, H, dk, self.k_scale)
        if K.lightning_segments_takes(dk):
            tiles, n_tiles, _ = ctx.tiles(1 if ctx.decode else SEGMENT)
            direct = ctx.decode or n_tiles == ctx.n_seqs
            scratch = None if direct else ctx.scratch("lightning_segments", 2 * n_tiles * H * dk * dv)
            o = K.lightning_segments(proj, 0, H * dk, 2 * H * dk, tiles, n_tiles, direct, ctx.seq_slot, self.decay,
                                     state, scratch, H, dk, dv, silu=False)
        else:
            tiles, n_seqs, _ = ctx.tiles(1 if ctx.decode else _WHOLE_SEQUENCE)
            o = K.lightning_scan(proj, 0, H * dk, 2 * H * dk, tiles, n_seqs, ctx.seq_slot, self.decay, state, H, dk, dv,
                                 silu=False)
        g0 = 2 * H * dk + H * dv
        a = K.gated_rmsnorm(o, proj[:, g0:g0 + H * dv], None, self.eps, self.wo.weight.dtype, group=dv,
                            gate_act=K.GATE_SILU, scale=self.out_scale)
        self.wo(a, ADD_F32, residual)


MIXERS.register("lightning_attention", LightningAttention)
MIXERS.register("retention", Retention)
