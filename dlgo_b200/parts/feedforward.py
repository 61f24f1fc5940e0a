"""SwiGLU feed-forward: ``y = Wd . (silu(Wg . x) * (Wu . x))``.

Reference (models/llm/forward.go:293-298): gate and up projections in one
dispatch, ``h = g / (1 + exp(-g)) * u`` (ops/activation.go:8-38), down
projection; the caller adds the result to the residual (:169).  Dense: no
experts, no routing.
"""
from __future__ import annotations

import os
from typing import Any, Callable, Dict, Mapping, Optional

import torch

from ..csrc import kernels as K
from .base import FeedForward, ParamSpec
from .linear import ADD_F32, STORE, STORE_F32, Linear
from .registry import FEED_FORWARDS


class SwiGLU(FeedForward):
    """``names``: tensor names of gate, up and down below the part's prefix."""

    def __init__(self, hidden_size: int, intermediate_size: int, names: Optional[Mapping[str, str]] = None):
        super().__init__(hidden_size=hidden_size, intermediate_size=intermediate_size, names=names)
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.names = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}
        self.names.update(names or {})
        self.w_gate_up: Optional[Linear] = None
        self.w_down: Optional[Linear] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        n = self.names
        return {
            n["gate"]: ParamSpec((self.intermediate_size, self.hidden_size)),
            n["up"]: ParamSpec((self.intermediate_size, self.hidden_size)),
            n["down"]: ParamSpec((self.hidden_size, self.intermediate_size)),
        }

    def load(self, get: Callable[[str], torch.Tensor], runtime: Any) -> None:
        gate = runtime.compute_copy(get(self.names["gate"]))
        up = runtime.compute_copy(get(self.names["up"]))
        f, d = self.intermediate_size, self.hidden_size
        self.fused = False
        if runtime.dtype == torch.bfloat16 and f % 16 == 0 and d % 8 == 0:
            # blocks of 16 gate rows followed by their 16 up rows: the contraction's epilogue then
            # holds a gate value and its up value side by side and writes silu(g) * u directly
            inter = torch.stack([gate.view(f // 16, 16, d), up.view(f // 16, 16, d)], dim=1).reshape(2 * f, d)
            self.w_gate_up = Linear(inter.contiguous(), runtime, fused_swiglu=True)
            self.fused = True
        else:
            self.w_gate_up = Linear(torch.cat([gate, up], dim=0), runtime)
        self.w_down = Linear(get(self.names["down"]), runtime)

    def forward(self, x: Any, residual: torch.Tensor, ctx: Any) -> None:
        if self.fused:
            h = self.w_gate_up(x)
        else:
            h = K.swiglu(self.w_gate_up(x, STORE))
        parts = self.w_down.partials(h, for_residual=True) if ctx is not None and hasattr(ctx, "defer") else None
        if parts is not None:
            ctx.defer(residual, parts)      # the next norm adds the slices to the residual
        else:
            self.w_down(h, ADD_F32, residual)


_FUSED_BIAS_ACT = os.environ.get("DLGO_FUSED_BIAS_ACT", "1") != "0"


class ReluSquaredMLP(FeedForward):
    """Dense two-matrix feed-forward with the square of relu between: ``y = Wd . relu(Wu . x + bu)^2 + bd``
    (``bias`` False: no bu, bd).  ``names``: tensor names below the part's prefix.  Bias and activation run in
    fp32 on the contraction's accumulator (its epilogue on the tensor cores), or, with ``DLGO_FUSED_BIAS_ACT=0``,
    in a launch of their own on its fp32 result."""

    can_defer_bias = True

    def __init__(self, hidden_size: int, intermediate_size: int, bias: bool = False,
                 names: Optional[Mapping[str, str]] = None):
        super().__init__(hidden_size=hidden_size, intermediate_size=intermediate_size, bias=bias, names=names)
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.bias = bool(bias)
        self.names = {"up": "up_proj.weight", "up_bias": "up_proj.bias", "down": "down_proj.weight",
                      "down_bias": "down_proj.bias"}
        self.names.update(names or {})
        self.w_up: Optional[Linear] = None
        self.w_down: Optional[Linear] = None
        self.b_up: Optional[torch.Tensor] = None
        self.output_bias: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        n, f, d = self.names, self.intermediate_size, self.hidden_size
        specs = {n["up"]: ParamSpec((f, d)), n["down"]: ParamSpec((d, f))}
        if self.bias:
            specs[n["up_bias"]] = ParamSpec((f,))
            specs[n["down_bias"]] = ParamSpec((d,))
        return specs

    def load(self, get: Callable[[str], torch.Tensor], runtime: Any) -> None:
        n = self.names
        self.w_up = Linear(get(n["up"]), runtime)
        self.w_down = Linear(get(n["down"]), runtime)
        if self.bias:
            self.b_up = get(n["up_bias"]).to(torch.float32).contiguous()
            self.output_bias = get(n["down_bias"]).to(torch.float32).contiguous()

    def forward(self, x: Any, residual: torch.Tensor, ctx: Any, defer_bias: bool = False) -> None:
        """``defer_bias``: the caller adds :attr:`output_bias` itself (fused into its next pass over the result)."""
        if _FUSED_BIAS_ACT:
            h = self.w_up.bias_act(x, self.b_up, K.ACT_RELU2)      # bias and relu squared in the contraction's epilogue
        else:
            h = K.bias_act(self.w_up(x, STORE_F32), self.b_up, K.ACT_RELU2, self.w_down.weight.dtype)
        if self.output_bias is not None and not defer_bias:
            K.bias_act(residual, self.output_bias, K.ACT_NONE, torch.float32, in_place=True)
        self.w_down(h, ADD_F32, residual)


FEED_FORWARDS.register("swiglu", SwiGLU)
FEED_FORWARDS.register("relu2_mlp", ReluSquaredMLP)
