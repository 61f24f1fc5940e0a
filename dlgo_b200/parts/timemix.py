"""Time mixing: a recurrence over a fixed-size state whose decay depends on the token.

With h the mixer's input and h' the previous token's input (zeros before a sequence's first token), every
projection reads its own blend ``m_s = h + (h' - h) * mu_s`` for s in r, k, v, g, w:

    r = Wr m_r,  k = Wk m_k,  v = Wv m_v                      (heads x head_dim numbers each)
    gate = silu(Wg m_g)
    w = exp(-exp(W2 tanh(W1 m_w) + w0))                       per head and key channel, in (0, 1)
    per head:  o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t      (the bonus u counts for the current token only)
               S_t = diag(w_t) S_(t-1) + k_t v_t^T
    result = Wo (o / rms(o) per head * norm * gate) * out_scale

The state of a sequence is S [heads, head_dim, head_dim] followed by its last input (hidden_size numbers), fp32,
zero when the slot is taken; no position is cached.  The blends are formed from the fp32 residual stream where the
block offers it; tanh, the decay's exponentials, the state, the per-head norm and the gate are fp32 in every
precision, and so are the results of all projections that enter the recurrence.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Mapping, Optional

import torch

from ..csrc import kernels as K
from .base import Mixer, ParamSpec, PositionEncoding, StateNeed
from .linear import ADD_F32, STORE_F32, Linear
from .registry import MIXERS

_NAMES = {"mu": "mu.{}", "r": "r_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "gate": "g_proj.weight",
          "out": "o_proj.weight", "decay_down": "w1.weight", "decay_up": "w2.weight", "decay_bias": "w0",
          "bonus": "u", "norm": "norm.weight"}
_BLENDS = ("r", "k", "v", "g", "w")
SEGMENT = 128                  # tokens of a segment where a prompt's segments run side by side
_WHOLE_SEQUENCE = 1 << 30


class TimeMix(Mixer):
    """``decay_rank``: width of the decay's small projection.  ``out_scale``: a constant factor on the result.
    ``names``: tensor names below the part's prefix (``mu`` with a place for the blend's letter)."""

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, decay_rank: int, eps: float,
                 out_scale: float = 1.0, names: Optional[Mapping[str, str]] = None):
        super().__init__(hidden_size=hidden_size, num_heads=num_heads, head_dim=head_dim, decay_rank=decay_rank,
                         eps=eps, out_scale=out_scale, names=names)
        self.hidden_size, self.n_heads, self.head_size = int(hidden_size), int(num_heads), int(head_dim)
        self.decay_rank = int(decay_rank)
        if min(self.hidden_size, self.n_heads, self.head_size, self.decay_rank) <= 0:
            raise ValueError("sizes must be positive")
        self.eps, self.out_scale = float(eps), float(out_scale)
        self.names = dict(_NAMES)
        self.names.update(names or {})
        self.inner = self.n_heads * self.head_size
        self.mu: Optional[torch.Tensor] = None            # [5, d] fp32 in the order r, k, v, g, w
        self.w_r = self.w_k = self.w_v = self.w_g = self.w_down = self.w_up = self.wo = None
        self.w0: Optional[torch.Tensor] = None
        self.bonus: Optional[torch.Tensor] = None
        self.norm: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        n, d, m = self.names, self.hidden_size, self.inner
        specs = {n["mu"].format(s): ParamSpec((d,)) for s in _BLENDS}
        for key in ("r", "k", "v", "gate"):
            specs[n[key]] = ParamSpec((m, d))
        specs[n["decay_down"]] = ParamSpec((self.decay_rank, d))
        specs[n["decay_up"]] = ParamSpec((m, self.decay_rank))
        specs[n["decay_bias"]] = ParamSpec((m,))
        specs[n["bonus"]] = ParamSpec((self.n_heads, self.head_size))
        specs[n["norm"]] = ParamSpec((m,), "one_plus_normal")
        specs[n["out"]] = ParamSpec((d, m))
        return specs

    def state_need(self) -> StateNeed:
        return StateNeed((self.inner * self.head_size + self.hidden_size,), torch.float32)

    def load(self, get: Callable[[str], torch.Tensor], runtime: Any) -> None:
        n = self.names
        self.mu = torch.stack([get(n["mu"].format(s)).to(torch.float32) for s in _BLENDS], dim=0).contiguous()
        self.w_r, self.w_k, self.w_v, self.w_g = (Linear(get(n[key]), runtime) for key in ("r", "k", "v", "gate"))
        self.w_down = Linear(get(n["decay_down"]), runtime)
        self.w_up = Linear(get(n["decay_up"]), runtime)
        self.wo = Linear(get(n["out"]), runtime)
        # what enters the recurrence is 32-bit in every precision
        self.w0 = get(n["decay_bias"]).to(torch.float32).contiguous()
        self.bonus = get(n["bonus"]).to(torch.float32).reshape(-1).contiguous()
        self.norm = get(n["norm"]).to(torch.float32).contiguous()

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: Any, cache: Any,
                state: Optional[torch.Tensor], positions: Mapping[str, PositionEncoding]) -> None:
        if state is None:
            raise RuntimeError("time mixing needs its state")
        H, n, d = self.n_heads, self.head_size, self.hidden_size
        act = self.wo.weight.dtype
        h32 = getattr(ctx, "sublayer_input_f32", None)
        if h32 is None or h32.shape != x.shape:
            h32 = x if x.dtype == torch.float32 else x.float()
        st = state.view(state.shape[0], -1)
        blends = K.token_shift_mix(h32, self.mu, ctx.token_seq, ctx.seq_slot, st, H * n * n, act)     # [5, T, d]
        r = self.w_r(blends[0], STORE_F32)
        k = self.w_k(blends[1], STORE_F32)
        v = self.w_v(blends[2], STORE_F32)
        g = self.w_g(blends[3], STORE_F32)
        low = K.bias_act(self.w_down(blends[4], STORE_F32), None, K.ACT_TANH, act)
        zw = self.w_up(low, STORE_F32)
        if K.wkv_segments_takes(n):
            tiles, n_tiles, _ = ctx.tiles(1 if ctx.decode else SEGMENT)
            direct = ctx.decode or n_tiles == ctx.n_seqs
            scratch = None if direct else ctx.scratch("wkv_segments", K.wkv_scratch_floats(n_tiles, H, n))
            o = K.wkv(r, k, v, zw, self.w0, self.bonus, tiles, n_tiles, direct, True, ctx.seq_slot, st, h32, scratch, H, n)
        else:
            tiles, n_seqs, _ = ctx.tiles(1 if ctx.decode else _WHOLE_SEQUENCE)
            o = K.wkv(r, k, v, zw, self.w0, self.bonus, tiles, n_seqs, True, False, ctx.seq_slot, st, h32, None, H, n)
        a = K.gated_rmsnorm(o, g, self.norm, self.eps, act, group=n, gate_act=K.GATE_SILU, scale=self.out_scale)
        self.wo(a, ADD_F32, residual)


MIXERS.register("time_mix", TimeMix)
