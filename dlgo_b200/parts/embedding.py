"""Token embedding and the output head.

Embedding: ``x = E[token, :]`` with no scaling for this architecture
(models/llm/forward.go:132-135).  Head: ``logits = O . x`` in fp32, with
``O = E`` when the weights are tied (models/llm/forward.go:193-197,
models/llm/loader.go:74-76).
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Optional, Sequence

import torch

from ..csrc import kernels as K
from .base import ParamSpec, Part
from .linear import STORE_F32, Linear
from .registry import EMBEDDINGS, HEADS


class TokenEmbedding(Part):
    """``name``: the table's tensor name below the part's prefix.  ``norm``: a norm applied to the looked-up rows
    before they become the residual stream, as ``(kind, params)`` of the norm registry (its tensor names are
    relative to the embedding's prefix as well); it must offer ``forward_in_place`` on fp32 rows.  ``scale``: a constant
    every looked-up number is multiplied by (in fp32)."""

    def __init__(self, vocab_size: int, hidden_size: int, name: str = "weight", norm: Optional[Sequence[Any]] = None,
                 scale: float = 1.0):
        super().__init__(vocab_size=vocab_size, hidden_size=hidden_size, name=name, norm=norm, scale=scale)
        self.scale = float(scale)
        self.vocab_size = int(vocab_size)
        self.hidden_size = int(hidden_size)
        self.name = name
        self.table: Optional[torch.Tensor] = None
        self.norm: Any = None
        if norm is not None:
            from ..config.spec import PartSpec
            from .registry import NORMS
            kind, params = norm
            self.norm = NORMS.build(PartSpec(kind, dict(params)))
            if not hasattr(self.norm, "forward_in_place"):
                raise ValueError(f"the norm {kind!r} cannot rewrite fp32 rows in place")

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs = {self.name: ParamSpec((self.vocab_size, self.hidden_size))}
        if self.norm is not None:
            specs.update(self.norm.param_specs())
        return specs

    def load(self, get: Callable[[str], torch.Tensor], runtime: Any) -> None:
        self.table = runtime.compute_copy(get(self.name)).contiguous()
        if self.norm is not None:
            self.norm.load(get, runtime)

    def forward(self, token_ids: torch.Tensor, copies: Optional[int] = None) -> torch.Tensor:
        """fp32 rows [T, hidden]; with ``copies`` = s, [T, s, hidden] with every copy equal (residual streams)."""
        if self.norm is None:
            return K.embed(token_ids, self.table, copies=copies, scale=self.scale)
        if copies is not None:
            raise ValueError("a normed embedding feeds a single residual stream")
        return self.norm.forward_in_place(K.embed(token_ids, self.table, scale=self.scale))


class LinearHead(Part):
    """``tied_to`` names the tensor (absolute name) the head shares, or ``None`` for a weight of its own.
    ``scale`` s and ``softcap`` c: ``logits <- c * tanh(s * logits / c)`` (c None: ``s * logits``), in fp32."""

    def __init__(self, vocab_size: int, hidden_size: int, tied_to: Optional[str] = None, name: str = "weight",
                 scale: float = 1.0, softcap: Optional[float] = None):
        super().__init__(vocab_size=vocab_size, hidden_size=hidden_size, tied_to=tied_to, name=name, scale=scale,
                         softcap=softcap)
        if softcap is not None and softcap <= 0:
            raise ValueError(f"softcap must be positive or None, got {softcap}")
        self.scale = float(scale)
        self.softcap = None if softcap is None else float(softcap)
        self.vocab_size = int(vocab_size)
        self.hidden_size = int(hidden_size)
        self.tied_to = tied_to
        self.name = name
        self.proj: Optional[Linear] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {} if self.tied_to else {self.name: ParamSpec((self.vocab_size, self.hidden_size))}

    def load(self, get: Callable[[str], torch.Tensor], runtime: Any) -> None:
        self.proj = Linear(get(self.name), runtime)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        logits = self.proj(x, STORE_F32)
        if self.scale != 1.0 or self.softcap is not None:
            K.scale_softcap(logits, self.scale, self.softcap or 0.0)
        return logits


EMBEDDINGS.register("token_embedding", TokenEmbedding)
HEADS.register("linear_head", LinearHead)
