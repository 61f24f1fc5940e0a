"""Several mixers side by side: all read the same input, and the result is the sum of theirs, each with a
constant factor.

``mixers`` lists ``(tensor-name prefix below this part's, PartSpec of the mixer, factor)``.  A member carries its
factor itself (its ``out_scale``), inside the last fp32 pass before its output projection, so the members simply add
into the same fp32 target one after another and no pass over the sum is needed.  At most one member may keep
positions in the cache (the group's pages are then this part's); members with a fixed-size state get their part
of one flat fp32 state row per sequence.
"""
from __future__ import annotations

import math
from typing import Any, Callable, Dict, List, Mapping, Optional, Sequence, Tuple

import torch

from ..config.spec import PartSpec
from .base import CacheNeed, Mixer, ParamSpec, PositionEncoding, StateNeed
from .registry import MIXERS


class ParallelMixers(Mixer):
    def __init__(self, mixers: Sequence[Tuple[str, Any, float]]):
        super().__init__(mixers=mixers)
        if not mixers:
            raise ValueError("parallel mixers need at least one member")
        self.members: List[Tuple[str, Mixer]] = []
        for prefix, spec, factor in mixers:
            if not isinstance(spec, PartSpec):
                spec = PartSpec(spec[0], dict(spec[1]))
            member = MIXERS.build(spec.with_params(out_scale=float(factor)))
            self.members.append((str(prefix), member))
        if sum(1 for _, m in self.members if m.cache_need() is not None) > 1:
            raise ValueError("at most one of several mixers side by side may keep positions in the cache")
        # members with state: (member index, first float of its part, floats, shape)
        self._state_parts: List[Tuple[int, int, int, Tuple[int, ...]]] = []
        off = 0
        for i, (_, m) in enumerate(self.members):
            need = m.state_need()
            if need is None:
                continue
            if need.dtype != torch.float32:
                raise ValueError("members' states are joined in one fp32 row")
            n = int(math.prod(need.shape))
            self._state_parts.append((i, off, n, tuple(need.shape)))
            off += n
        self._state_floats = off

    def param_specs(self) -> Dict[str, ParamSpec]:
        specs: Dict[str, ParamSpec] = {}
        for prefix, m in self.members:
            for rel, ps in m.param_specs().items():
                specs[prefix + rel] = ps
        return specs

    def cache_need(self) -> Optional[CacheNeed]:
        for _, m in self.members:
            need = m.cache_need()
            if need is not None:
                return need
        return None

    def state_need(self) -> Optional[StateNeed]:
        if not self._state_parts:
            return None
        if len(self._state_parts) == 1:
            return StateNeed(self._state_parts[0][3], torch.float32)      # the one member's own shape
        return StateNeed((self._state_floats,), torch.float32)

    def load(self, get: Callable[[str], torch.Tensor], runtime: Any) -> None:
        for prefix, m in self.members:
            m.load(lambda rel, _p=prefix: get(_p + rel), runtime)

    def prepare(self, runtime: Any) -> None:
        for _, m in self.members:
            m.prepare(runtime)

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: Any, cache: Any,
                state: Optional[torch.Tensor], positions: Mapping[str, PositionEncoding]) -> None:
        parts = {i: (off, n, shape) for i, off, n, shape in self._state_parts}
        for i, (_, m) in enumerate(self.members):
            st = None
            if i in parts:
                if state is None:
                    raise RuntimeError("a member of the parallel mixers needs its state")
                off, n, shape = parts[i]
                # (one member with state: the row is its own; several: a member's columns of the flat row, rows
                # `state.stride(0)` apart, which the member's kernels must take)
                st = state if len(parts) == 1 else state[:, off:off + n].view((state.shape[0],) + shape)
            m.forward(x, residual, ctx, cache if m.cache_need() is not None else None, st, positions)
            if hasattr(ctx, "settle"):
                ctx.settle(residual)        # slices a member left unsummed go in before the next member adds


MIXERS.register("parallel_mixers", ParallelMixers)
