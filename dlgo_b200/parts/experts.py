"""Routed experts: a mixture-of-experts feed-forward.

    z = Wr h (+ b)                   router logits, fp32 (the router's weight is kept in fp32; ``logit_bias``: a stored
                                     bias that is part of the logits, unlike ``correction``)
    s = softmax(z)  (or sigmoid(z))  over ALL router outputs
    c = s + correction               choice scores (``correction``: a stored per-output bias used for choosing only)
    outputs form ``group_count`` equal groups of neighbours; a group's score is its largest c; only outputs of
    the ``group_keep`` best groups can be chosen (the others count as minus infinity); the ``top`` largest c win
    y = sum over the chosen e of s_e * expert_e(h)            (``renormalize``: s_e / sum of the chosen s)
    expert_e(h) = Wdown_e act(Wup_e h)                        for e < num_experts
                  (``gated``: Wdown_e (silu(Wgate_e h) * (Wup_e h)), a third matrix per expert)
    expert_e(h) = h                                           for the ``identity_experts`` outputs after them
    y += gate * shared(h),  gate = sigmoid(w_g . h) per token (``shared_size``, ``shared_gate``)
    ``weight_on`` = "input": y = sum over the chosen e of expert_e(s_e * h) instead (the weight multiplies what the
    expert reads, which differs from the above as soon as an expert is not linear)

Every constant above is a parameter.  Nothing returns to the host between the router and the result: the
(token, choice) pairs are sorted by expert on the device, the experts run as two grouped contractions over the
sorted rows (bfloat16: on tcgen05 from a couple of dozen pairs a step on, tiles of 128 rows; else tiles of 8 rows
with a warp per output, or 64 x 64 tiles on the fp32 pipes for float32 prompts), and a last pass adds the weighted
results in the order the choices were made, so a step can be captured in a CUDA graph and a token's result does not
depend on the rest of the batch.
"""
from __future__ import annotations

import os
from typing import Any, Callable, Dict, Mapping, Optional

import torch

from ..csrc import kernels as K
from .base import FeedForward, ParamSpec
from .linear import STORE_F32, Linear
from .registry import FEED_FORWARDS

_ACTS = {"none": K.ACT_NONE, "relu2": K.ACT_RELU2, "silu": K.ACT_SILU, "gelu_tanh": K.ACT_GELU_TANH}
# pairs per expert (on average) up to which the 8-row tiles run; beyond, the larger tiles
_FEW_PAIRS_PER_EXPERT = int(os.environ.get("DLGO_MOE_FEW_PAIRS", 8))
_TENSOR_CORES = os.environ.get("DLGO_MOE_TC", "1") != "0"       # 0: the fp32-pipe tiles also in bfloat16
# bfloat16: pairs of a step from which the tcgen05 kernel runs instead of the 8-row tiles.  Measured on a B200 at
# width 2,048 with 56 experts of 1,024, 8 chosen (ms a decode step, 8-row tiles against tcgen05): batch 1, 0.518 /
# 0.662; batch 2, 0.620 / 0.694; batch 4, 0.745 / 0.717; batch 8, 0.880 / 0.735; batch 32, 1.58 / 0.894.
# With experts of a megabyte (width 1,024, experts of 512) the 8-row tiles still win at 32 pairs: 0.372 / 0.420.
_TC_MIN_PAIRS = int(os.environ.get("DLGO_MOE_TC_MIN_PAIRS", 0))      # 0: 24, or 128 for experts below 2 MB
# prompts (more than 2,048 pairs): CTA pairs on two row tiles of an expert that share one weight tile
_TC_PAIRS = os.environ.get("DLGO_MOE_TC_PAIR", "0") != "0"
_FUSED_SWIGLU = os.environ.get("DLGO_MOE_FUSED_SWIGLU", "1") != "0"     # 0: gated experts' silu(gate) * up as a pass of its own


class RoutedExperts(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int, num_experts: int, top: int,
                 identity_experts: int = 0, group_count: int = 1, group_keep: int = 1, score: str = "softmax",
                 renormalize: bool = False, correction: bool = False, activation: str = "relu2",
                 shared_size: Optional[int] = None, shared_gate: bool = False,
                 names: Optional[Mapping[str, str]] = None, logit_bias: bool = False, gated: bool = False,
                 weight_on: str = "output"):
        super().__init__(hidden_size=hidden_size, intermediate_size=intermediate_size, num_experts=num_experts, top=top,
                         identity_experts=identity_experts, group_count=group_count, group_keep=group_keep,
                         score=score, renormalize=renormalize, correction=correction, activation=activation,
                         shared_size=shared_size, shared_gate=shared_gate, names=names, logit_bias=logit_bias,
                         gated=gated, weight_on=weight_on)
        if weight_on not in ("output", "input"):
            raise ValueError(f"weight_on must be 'output' or 'input', got {weight_on!r}")
        if weight_on == "input" and identity_experts:
            raise ValueError("identity experts take their weight on the output")
        self.weight_on_input = weight_on == "input"
        self.logit_bias = bool(logit_bias)
        self.gated = bool(gated)
        if self.gated and activation != "silu":
            raise ValueError("gated experts multiply silu(gate) by up: the activation must be 'silu'")
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.num_experts = int(num_experts)
        self.identity_experts = int(identity_experts)
        self.n_outputs = self.num_experts + self.identity_experts
        self.top = int(top)
        self.group_count, self.group_keep = int(group_count), int(group_keep)
        if score not in ("softmax", "sigmoid"):
            raise ValueError(f"score must be 'softmax' or 'sigmoid', got {score!r}")
        if activation not in _ACTS:
            raise ValueError(f"activation must be one of {sorted(_ACTS)}, got {activation!r}")
        if self.n_outputs <= 0 or self.n_outputs % self.group_count or not 0 < self.group_keep <= self.group_count:
            raise ValueError("the router's outputs must form equal groups of which some are kept")
        if not 0 < self.top <= self.group_keep * (self.n_outputs // self.group_count):
            raise ValueError("top must be positive and no more than the kept groups hold")
        self.sigmoid_scores = score == "sigmoid"
        self.renormalize = bool(renormalize)
        self.correction = bool(correction)
        self.act = _ACTS[activation]
        self.shared_size = None if shared_size is None else int(shared_size)
        self.shared_gate = bool(shared_gate) and self.shared_size is not None
        self.names = {"router": "router.weight", "correction": "router.bias", "logit_bias": "router.logit_bias",
                      "gate": "gate_proj.weight", "expert": "experts.{}.",
                      "up": "up_proj.weight", "down": "down_proj.weight", "shared_up": "shared.up_proj.weight",
                      "shared_down": "shared.down_proj.weight", "shared_gate": "shared.gate.weight"}
        self.names.update(names or {})
        self.w_router: Optional[torch.Tensor] = None        # fp32 [outputs (+ gate row), hidden]
        self.b_choice: Optional[torch.Tensor] = None
        self.b_logit: Optional[torch.Tensor] = None
        self.w_up: Optional[torch.Tensor] = None            # [experts, ff, hidden]
        self.w_down: Optional[torch.Tensor] = None          # [experts, hidden, ff]
        self.shared_up: Optional[Linear] = None
        self.shared_down: Optional[Linear] = None
        self.on_tensor_cores = False

    def param_specs(self) -> Dict[str, ParamSpec]:
        n, d, f = self.names, self.hidden_size, self.intermediate_size
        specs = {n["router"]: ParamSpec((self.n_outputs, d))}
        if self.correction:
            specs[n["correction"]] = ParamSpec((self.n_outputs,))
        if self.logit_bias:
            specs[n["logit_bias"]] = ParamSpec((self.n_outputs,))
        for e in range(self.num_experts):
            p = n["expert"].format(e)
            if self.gated:
                specs[p + n["gate"]] = ParamSpec((f, d))
            specs[p + n["up"]] = ParamSpec((f, d))
            specs[p + n["down"]] = ParamSpec((d, f))
        if self.shared_size is not None:
            specs[n["shared_up"]] = ParamSpec((self.shared_size, d))
            specs[n["shared_down"]] = ParamSpec((d, self.shared_size))
            if self.shared_gate:
                specs[n["shared_gate"]] = ParamSpec((1, d))
        return specs

    def load(self, get: Callable[[str], torch.Tensor], runtime: Any) -> None:
        n = self.names
        rows = [get(n["router"]).to(torch.float32)]
        if self.shared_gate:
            rows.append(get(n["shared_gate"]).to(torch.float32).reshape(1, self.hidden_size))
        self.w_router = torch.cat(rows, dim=0).contiguous()      # routers are 32-bit in every precision
        if self.correction:
            self.b_choice = get(n["correction"]).to(torch.float32).contiguous()
        if self.logit_bias:
            self.b_logit = get(n["logit_bias"]).to(torch.float32).contiguous()
        if self.num_experts:
            ups = [runtime.compute_copy(get(n["expert"].format(e) + n["up"])) for e in range(self.num_experts)]
            self.gate_block = self.intermediate_size
            if self.gated:
                # an expert's first matrix: its gate rows, then its up rows; in bfloat16, where the tensor-core
                # contraction forms silu(gate) * up on its accumulator, blocks of 16 gate rows and their 16 up rows
                f, B = self.intermediate_size, K.MOE_SWIGLU_BLOCK
                gates = [runtime.compute_copy(get(n["expert"].format(e) + n["gate"])) for e in range(self.num_experts)]
                if _TENSOR_CORES and _FUSED_SWIGLU and runtime.dtype == torch.bfloat16 and f % B == 0:
                    self.gate_block = B
                    ups = [torch.stack([g.view(f // B, B, -1), u.view(f // B, B, -1)], dim=1).reshape(2 * f, -1)
                           for g, u in zip(gates, ups)]
                else:
                    ups = [torch.cat([g, u], dim=0) for g, u in zip(gates, ups)]
            downs = [runtime.compute_copy(get(n["expert"].format(e) + n["down"])) for e in range(self.num_experts)]
            self.w_up = torch.stack(ups, dim=0).contiguous()
            self.w_down = torch.stack(downs, dim=0).contiguous()
            self.on_tensor_cores = (_TENSOR_CORES and
                                    K.moe_gemm_tc_takes(self.w_up.dtype, self.w_up.shape[1], self.hidden_size) and
                                    K.moe_gemm_tc_takes(self.w_down.dtype, self.hidden_size, self.intermediate_size))
        if self.shared_size is not None:
            self.shared_up = Linear(get(n["shared_up"]), runtime)
            self.shared_down = Linear(get(n["shared_down"]), runtime)

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: Any) -> None:
        T, d = x.shape
        pairs = T * self.top
        # which grouped kernel the step takes decides the plan's tile rows; the plan is made with the choice
        tc_from = _TC_MIN_PAIRS or (24 if self.intermediate_size * self.hidden_size >= (1 << 20) else 128)
        on_tc = self.on_tensor_cores and pairs >= tc_from
        few = pairs <= _FEW_PAIRS_PER_EXPERT * max(self.num_experts, 1)
        tile_rows = ((K.MOE_TC_PAIR_ROWS if _TC_PAIRS and pairs > 2048 else K.MOE_TC_ROWS) if on_tc else
                     (K.MOE_FEW_ROWS if few else K.MOE_TILE_ROWS))
        idx, wt, gate, plan = K.moe_router(x, self.w_router, self.b_choice, self.n_outputs, self.shared_gate, self.top,
                                           self.group_count, self.group_keep, self.sigmoid_scores, self.renormalize,
                                           plan=(self.num_experts, tile_rows), logit_bias=self.b_logit)
        pair_out = None
        src, div, scale = x, self.top, None
        if self.weight_on_input:
            # an expert reads its row multiplied by the pair's weight: on the tensor-core path the copy into sorted
            # order multiplies on its way, else a pass makes a row per pair; the combine then adds the experts'
            # results as they are
            if on_tc:
                scale = wt
            else:
                src, div = K.moe_scale_rows(x, wt), 1
            wt = None
        if self.num_experts:
            # (gated: the first contraction leaves gate and up values side by side; silu(gate) * up is formed on the
            # tensor-core kernel's accumulator where the rows alternate in blocks, else by a pass of its own)
            act = K.ACT_NONE if self.gated else self.act
            fused = self.gated and on_tc and self.gate_block == K.MOE_SWIGLU_BLOCK and tile_rows == K.MOE_TC_ROWS
            hidden = torch.empty((pairs, self.intermediate_size if fused else self.w_up.shape[1]), dtype=x.dtype,
                                 device=x.device)
            pair_out = torch.empty((pairs, d), dtype=x.dtype, device=x.device)    # (sums of these stay fp32)
            if on_tc:
                # bfloat16: the tokens' rows copied into sorted order, then both contractions on tcgen05
                rows = K.moe_gather_rows(plan, src, div, scale)
                K.moe_gemm_tc(plan, rows, self.w_up, hidden, False, K.MOE_ACT_SWIGLU if fused else act)
                if self.gated and not fused:
                    hidden = K.swiglu(hidden, block=self.gate_block)
                K.moe_gemm_tc(plan, hidden, self.w_down, pair_out, True, K.ACT_NONE)
            else:
                K.moe_gemm(plan, src, self.w_up, hidden, div, False, act)                  # rows gathered by token (or pair)
                if self.gated:
                    hidden = K.swiglu(hidden, block=self.gate_block)
                K.moe_gemm(plan, hidden, self.w_down, pair_out, None, True, K.ACT_NONE)    # rows scattered by pair
        shared = None
        if self.shared_size is not None:
            shared = self.shared_down(self.shared_up.bias_act(x, None, self.act), STORE_F32)
        K.moe_combine(residual, pair_out, x, idx, wt, self.num_experts, shared, gate)


FEED_FORWARDS.register("routed_experts", RoutedExperts)
