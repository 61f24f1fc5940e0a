"""RMSNorm: ``out = x * (1 / sqrt(mean(x^2) + eps)) * w`` (ops/norm.go:10-32),
statistics in fp32 on the fp32 residual stream, output in the run's precision.  Beside it: Dynamic Tanh, and the
layer norm with a weight and no bias."""
from __future__ import annotations

from typing import Any, Callable, Dict, Optional

import torch

from ..csrc import kernels as K
from .base import Norm, ParamSpec
from .registry import NORMS


class RMSNorm(Norm):
    """``one_plus``: the tensor is stored around zero and the norm multiplies by ``1 + w`` (the sum is made once,
    in fp32, when the weights are loaded).  ``name``: the tensor's name below the part's prefix."""

    def __init__(self, size: int, eps: float, one_plus: bool = False, name: str = "weight"):
        super().__init__(size=size, eps=eps, one_plus=one_plus, name=name)
        self.size = int(size)
        self.eps = float(eps)
        self.one_plus = bool(one_plus)
        self.name = name
        self.weight: Optional[torch.Tensor] = None
        self.out_dtype: Optional[torch.dtype] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {self.name: ParamSpec((self.size,), "normal" if self.one_plus else "one_plus_normal")}

    def load(self, get: Callable[[str], torch.Tensor], runtime: Any) -> None:
        w = get(self.name).to(torch.float32)
        self.weight = (w + 1.0 if self.one_plus else w).contiguous()
        self.out_dtype = runtime.dtype

    def forward(self, residual: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        return K.rmsnorm(residual, self.weight, self.eps, self.out_dtype, rows)

    def forward_fused(self, residual: torch.Tensor, parts: torch.Tensor,
                      rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``residual += parts.sum(0)`` and the norm of the new rows, in one pass."""
        return K.add_rmsnorm(residual, parts, self.weight, self.eps, self.out_dtype, rows)


RMSNorm.normed_kind = K.NORMED_RMS       # for arrangements that norm a sublayer's result (kernels.add_normed)


class LayerNorm(Norm):
    """``out = (x - mean(x)) / sqrt(var(x) + eps) * w`` with the variance as the mean of the squared deviations;
    a weight, no bias.  ``name``: the tensor's name below the part's prefix."""

    normed_kind = K.NORMED_LAYER

    def __init__(self, size: int, eps: float, name: str = "weight"):
        super().__init__(size=size, eps=eps, name=name)
        self.size = int(size)
        self.eps = float(eps)
        self.name = name
        self.weight: Optional[torch.Tensor] = None
        self.out_dtype: Optional[torch.dtype] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {self.name: ParamSpec((self.size,), "one_plus_normal")}

    def load(self, get: Callable[[str], torch.Tensor], runtime: Any) -> None:
        self.weight = get(self.name).to(torch.float32).contiguous()
        self.out_dtype = runtime.dtype

    def forward(self, residual: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        return K.layernorm_rows(residual, self.weight, self.eps, self.out_dtype, rows, self.normed_kind)

    def forward_in_place(self, x: torch.Tensor) -> torch.Tensor:
        """The fp32 rows ``x`` rewritten with their norm (a norm on the embedding: the stream stays fp32)."""
        return K.layernorm_rows(x, self.weight, self.eps, torch.float32, None, self.normed_kind, in_place=True)


class DynamicTanh(Norm):
    """Dynamic Tanh: ``out = tanh(alpha * x) * w + b`` element by element, with a learned scalar ``alpha``;
    no mean, no variance, no eps.  ``names`` gives the tensor names of weight, bias and alpha below the
    part's prefix."""

    kind = K.NORM_DYT

    def __init__(self, size: int, names: Optional[Dict[str, str]] = None):
        super().__init__(size=size, names=names)
        self.size = int(size)
        self.names = {"weight": "weight", "bias": "bias", "alpha": "alpha"}
        self.names.update(names or {})
        self.eps = 0.0
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None
        self.alpha: Optional[torch.Tensor] = None
        self.out_dtype: Optional[torch.dtype] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {self.names["weight"]: ParamSpec((self.size,), "one_plus_normal"),
                self.names["bias"]: ParamSpec((self.size,)),
                self.names["alpha"]: ParamSpec((), "one_plus_normal")}

    def load(self, get: Callable[[str], torch.Tensor], runtime: Any) -> None:
        self.weight = get(self.names["weight"]).to(torch.float32).contiguous()
        self.bias = get(self.names["bias"]).to(torch.float32).contiguous()
        self.alpha = get(self.names["alpha"]).to(torch.float32).reshape(1).contiguous()
        self.out_dtype = runtime.dtype

    def forward(self, residual: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        return self.forward_streams(residual.view(residual.shape[0], 1, -1), None, rows)

    def forward_streams(self, streams: torch.Tensor, read: Optional[torch.Tensor] = None,
                        rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The norm of ``sum_r read[r] * streams[:, r]`` (``read`` None: the plain sum) for streams [T, s, d]."""
        return K.streams_step(streams, read=read, norm_kind=K.NORM_DYT, norm_w=self.weight, norm_b=self.bias,
                              norm_alpha=self.alpha, out_dtype=self.out_dtype, rows=rows)

    def step_args(self) -> Dict[str, Any]:
        """This norm as arguments of :func:`kernels.streams_step` (for a caller that fuses it with a write)."""
        return dict(norm_kind=K.NORM_DYT, norm_w=self.weight, norm_b=self.bias, norm_alpha=self.alpha,
                    out_dtype=self.out_dtype)


def _rms_forward_streams(self, streams: torch.Tensor, read: Optional[torch.Tensor] = None,
                         rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    return K.streams_step(streams, read=read, rows=rows, **self.step_args())


def _rms_step_args(self) -> Dict[str, Any]:
    return dict(norm_kind=K.NORM_RMS, norm_w=self.weight, eps=self.eps, out_dtype=self.out_dtype)


RMSNorm.forward_streams = _rms_forward_streams
RMSNorm.step_args = _rms_step_args

NORMS.register("rmsnorm", RMSNorm)
NORMS.register("dynamic_tanh", DynamicTanh)
NORMS.register("layernorm", LayerNorm)
