"""Arrangements of a layer's parts.

``prenorm`` is the reference's standard wiring (models/llm/forward.go:144-169):
``r = x + mixer(norm(x))``, then ``x = r + ffn(norm(r))``.  The residual stream
is one fp32 tensor that mixer and feed-forward add into.
"""
from __future__ import annotations

from typing import Any, Mapping, Optional

import torch

from ..csrc import kernels as K
from .base import Block, ParamSpec, Part, PositionEncoding
from .registry import BLOCKS, CONNECTIONS


def norm_of(norm: Any, residual: torch.Tensor, ctx: Any) -> torch.Tensor:
    """The norm of the residual stream, adding first whatever the previous part left pending
    (fused into the norm's pass where the norm offers that)."""
    pending = ctx.take_pending() if hasattr(ctx, "take_pending") else None
    if pending is not None:
        if hasattr(norm, "forward_fused"):
            return norm.forward_fused(residual, pending)
        ctx.pending = pending
        ctx.settle(residual)
    return norm.forward(residual)


class PreNormBlock(Block):
    handles_pending = True   # reads the residual only through norm_of

    def __init__(self, mixer: Any, ffn: Any, norms: Mapping[str, Any], connections: Any = None):
        super().__init__(mixer, ffn, norms, connections)
        missing = [r for r in ("mixer_norm", "ffn_norm") if r not in self.norms]
        if missing or mixer is None or ffn is None:
            raise ValueError("a pre-norm block needs a mixer, a feed-forward and the norms 'mixer_norm' and 'ffn_norm'"
                             + (f" (missing: {', '.join(missing)})" if missing else ""))
        self.mixer_norm = self.norms["mixer_norm"]
        self.ffn_norm = self.norms["ffn_norm"]

    def forward(self, residual: torch.Tensor, ctx: Any, cache: Any, state: Optional[torch.Tensor],
                positions: Mapping[str, PositionEncoding]) -> None:
        x = norm_of(self.mixer_norm, residual, ctx)
        self.mixer.forward(x, residual, ctx, cache, state, positions)
        x = norm_of(self.ffn_norm, residual, ctx)
        self.ffn.forward(x, residual, ctx)


class HyperConnection(Part):
    """How one sublayer sits on ``streams`` residual streams x_1 .. x_s: it reads ``u = sum_r read[r] x_r`` and
    its result y returns as ``x_q <- sum_r mix[r, q] x_r + write[q] * y`` for every q at once (``mix`` is
    indexed [from, to]).  With one stream, read = write = mix = 1 this is the plain residual sum.
    ``names``: tensor names of the three below the part's prefix."""

    def __init__(self, streams: int, names: Optional[Mapping[str, str]] = None):
        super().__init__(streams=streams, names=names)
        if not 1 <= int(streams) <= K.MAX_STREAMS:
            raise ValueError(f"streams must be 1 to {K.MAX_STREAMS}, got {streams}")
        self.streams = int(streams)
        self.names = {"read": "read", "write": "write", "mix": "mix"}
        self.names.update(names or {})
        self.read: Optional[torch.Tensor] = None
        self.write: Optional[torch.Tensor] = None
        self.mix: Optional[torch.Tensor] = None

    def param_specs(self):
        s = self.streams
        return {self.names["read"]: ParamSpec((s,), "one_plus_normal"),
                self.names["write"]: ParamSpec((s,), "one_plus_normal"),
                self.names["mix"]: ParamSpec((s, s), "identity_plus_normal")}

    def load(self, get: Any, runtime: Any) -> None:
        # coefficients of the residual sum: fp32 in every precision
        self.read = get(self.names["read"]).to(torch.float32).contiguous()
        self.write = get(self.names["write"]).to(torch.float32).contiguous()
        self.mix = get(self.names["mix"]).to(torch.float32).contiguous()


class HyperPreNormBlock(Block):
    """Pre-norm layer on several residual streams [tokens, streams, hidden] (fp32): every sublayer that is
    there (``mixer``, then ``ffn``) reads the streams through its connection and its norm and writes back
    through the connection.  A sublayer adds its result into a zeroed [tokens, hidden] buffer, as it would
    into a single residual stream; the write reads that buffer and leaves it zero for the next sublayer.
    The write of one sublayer and the read and norm of the next are one launch (also across layers: the
    last write of a layer is left for the next layer's first read, or for whoever reads the streams next)."""

    handles_pending = False
    on_streams = True

    def __init__(self, mixer: Any, ffn: Any, norms: Mapping[str, Any], connections: Any = None):
        super().__init__(mixer, ffn, norms, connections)
        self.sublayers = []
        for part, norm, conn in ((mixer, "mixer_norm", "mixer_conn"), (ffn, "ffn_norm", "ffn_conn")):
            if part is None:
                continue
            if norm not in self.norms or conn not in self.connections:
                raise ValueError(f"a block on residual streams needs the norm {norm!r} and the connection {conn!r}")
            if not hasattr(self.norms[norm], "step_args"):
                raise ValueError(f"the norm {norm!r} cannot read residual streams")
            self.sublayers.append((part, self.norms[norm], self.connections[conn]))
        if mixer is None:
            raise ValueError("a block needs a mixer")

    def forward(self, streams: torch.Tensor, ctx: Any, cache: Any, state: Optional[torch.Tensor],
                positions: Mapping[str, PositionEncoding]) -> None:
        T, s, d = streams.shape
        y = ctx.zeros(f"sublayer_out{d}", T * d, torch.float32)[:T * d].view(T, d)
        for part, norm, conn in self.sublayers:
            owed = ctx.take_owed_write() if hasattr(ctx, "take_owed_write") else None
            if owed is not None:
                x = K.streams_step(streams, read=conn.read, **owed, **norm.step_args())
            else:
                x = norm.forward_streams(streams, conn.read)
            bias = None
            if part is self.mixer:
                part.forward(x, y, ctx, cache, state, positions)
            elif getattr(part, "can_defer_bias", False):
                part.forward(x, y, ctx, defer_bias=True)      # the write adds the output bias in its own pass
                bias = part.output_bias
            else:
                part.forward(x, y, ctx)
            ctx.settle(y)
            write = dict(y=y, y_bias=bias, mix=conn.mix, write=conn.write, clear_y=True)
            if hasattr(ctx, "owe_write"):
                ctx.owe_write(streams, write)
            else:
                K.streams_step(streams, **write)


class LayerScale(Part):
    """How a sublayer's result y joins the residual stream x in a layer that norms after the sum:
    ``skip_scale * x + scale * y`` with ``scale`` one learned number per channel and ``skip_scale`` a constant.
    ``name``: the tensor's name below the part's prefix."""

    def __init__(self, size: int, skip_scale: float = 1.0, name: str = "weight"):
        super().__init__(size=size, skip_scale=skip_scale, name=name)
        self.size = int(size)
        self.skip_scale = float(skip_scale)
        self.name = name
        self.scale: Optional[torch.Tensor] = None

    def param_specs(self):
        return {self.name: ParamSpec((self.size,), "one_plus_normal")}

    def load(self, get: Any, runtime: Any) -> None:
        self.scale = get(self.name).to(torch.float32).contiguous()      # part of the residual sum: fp32


class PostNormBlock(Block):
    """Norm after the sum: ``x <- norm1(a x + s1 * mixer(x))``, then ``x <- norm2(a x + s2 * ffn(x))``, where the
    sublayers read x itself and (a, s) come from the sublayer's connection (:class:`LayerScale`).  A layer
    without a feed-forward ends after the first line.  The residual stream stays fp32; a sublayer adds its result
    into a zeroed fp32 [tokens, hidden] buffer as it would into a residual stream, and ONE launch forms the sum,
    norms it, rewrites x, leaves the buffer zero and makes the copy of x in the run's type that the next
    contractions read."""

    handles_pending = False

    def __init__(self, mixer: Any, ffn: Any, norms: Mapping[str, Any], connections: Any = None):
        super().__init__(mixer, ffn, norms, connections)
        if mixer is None:
            raise ValueError("a block needs a mixer")
        self.sublayers = []
        for part, norm, conn in ((mixer, "mixer_norm", "mixer_conn"), (ffn, "ffn_norm", "ffn_conn")):
            if part is None:
                continue
            if norm not in self.norms or conn not in self.connections:
                raise ValueError(f"a post-norm block needs the norm {norm!r} and the connection {conn!r}")
            n, c = self.norms[norm], self.connections[conn]
            if not (hasattr(n, "weight") and hasattr(n, "eps") and hasattr(c, "scale") and hasattr(c, "skip_scale")):
                raise ValueError(f"a post-norm block needs an RMS norm as {norm!r} and a layer scale as {conn!r}")
            self.sublayers.append((part, n, c))

    def forward(self, residual: torch.Tensor, ctx: Any, cache: Any, state: Optional[torch.Tensor],
                positions: Mapping[str, PositionEncoding]) -> None:
        T, d = residual.shape
        dtype = ctx.runtime.dtype
        y = ctx.zeros(f"sublayer_out{d}", T * d, torch.float32)[:T * d].view(T, d)
        # x in the run's type: float32 runs read the residual stream itself; else the copy the previous
        # block's last norm made, or (first layer) a copy made now
        if dtype == torch.float32:
            x = residual
        else:
            kept = getattr(ctx, "residual_copy", None)
            x = kept[1] if kept is not None and kept[0] is residual else \
                K.scaled_add_rmsnorm(residual, None, None, None, 1.0, 0.0, dtype)
        for part, norm, conn in self.sublayers:
            if part is self.mixer:
                part.forward(x, y, ctx, cache, state, positions)
            else:
                part.forward(x, y, ctx)
            ctx.settle(y)
            copy = K.scaled_add_rmsnorm(residual, y, conn.scale, norm.weight, conn.skip_scale, norm.eps,
                                        None if dtype == torch.float32 else dtype, clear_y=True)
            x = residual if copy is None else copy
        ctx.residual_copy = (residual, x)


class ResultNormBlock(Block):
    """Norm on the sublayer's RESULT only: ``x <- x + norm1(mixer(x))``, then ``x <- x + norm2(ffn(x))``; the
    sublayers read x itself.  A layer without a feed-forward ends after the first line.  The norms are any that
    :func:`kernels.add_normed` knows (a layer norm with a weight, an RMS norm: ``normed_kind``, ``weight``, ``eps``).
    The residual stream stays fp32; a sublayer adds its result into a zeroed fp32 [tokens, hidden] buffer as it
    would into a residual stream, and ONE launch norms that buffer, adds it to x, leaves the buffer zero and makes
    the copy of x in the run's type that the next contractions read.  A sublayer that wants x unrounded (a
    recurrence's inputs) finds the fp32 stream as ``ctx.sublayer_input_f32``."""

    handles_pending = False

    def __init__(self, mixer: Any, ffn: Any, norms: Mapping[str, Any], connections: Any = None):
        super().__init__(mixer, ffn, norms, connections)
        if mixer is None:
            raise ValueError("a block needs a mixer")
        self.sublayers = []
        for part, role in ((mixer, "mixer_norm"), (ffn, "ffn_norm")):
            if part is None:
                continue
            n = self.norms.get(role)
            if n is None or not (hasattr(n, "normed_kind") and hasattr(n, "weight") and hasattr(n, "eps")):
                raise ValueError(f"a result-norm block needs a layer norm or an RMS norm as {role!r}")
            self.sublayers.append((part, n))

    def forward(self, residual: torch.Tensor, ctx: Any, cache: Any, state: Optional[torch.Tensor],
                positions: Mapping[str, PositionEncoding]) -> None:
        T, d = residual.shape
        dtype = ctx.runtime.dtype
        y = ctx.zeros(f"sublayer_out{d}", T * d, torch.float32)[:T * d].view(T, d)
        if dtype == torch.float32:
            x = residual
        else:
            kept = getattr(ctx, "residual_copy", None)
            x = kept[1] if kept is not None and kept[0] is residual else \
                K.scaled_add_rmsnorm(residual, None, None, None, 1.0, 0.0, dtype)
        ctx.sublayer_input_f32 = residual
        for part, norm in self.sublayers:
            if part is self.mixer:
                part.forward(x, y, ctx, cache, state, positions)
            else:
                part.forward(x, y, ctx)
            ctx.settle(y)
            copy = K.add_normed(residual, y, norm.weight, norm.eps, None if dtype == torch.float32 else dtype,
                                norm.normed_kind, clear_y=True)
            x = residual if copy is None else copy
        ctx.sublayer_input_f32 = None
        ctx.residual_copy = (residual, x)


class ResidualGate(Part):
    """A gate on a sublayer's result before it joins the residual stream: ``sigmoid(W h + b)`` element by element,
    with h the sublayer's own input; W is [size, size].  ``names``: tensor names of W and b below the part's
    prefix."""

    def __init__(self, size: int, names: Optional[Mapping[str, str]] = None):
        super().__init__(size=size, names=names)
        self.size = int(size)
        self.names = {"weight": "weight", "bias": "bias"}
        self.names.update(names or {})
        self.proj: Any = None
        self.bias: Optional[torch.Tensor] = None

    def param_specs(self):
        return {self.names["weight"]: ParamSpec((self.size, self.size)), self.names["bias"]: ParamSpec((self.size,))}

    def load(self, get: Any, runtime: Any) -> None:
        from .linear import Linear
        self.proj = Linear(get(self.names["weight"]), runtime)
        self.bias = get(self.names["bias"]).to(torch.float32).contiguous()      # added to the fp32 logits

    def logits(self, h: torch.Tensor, ctx: Any = None) -> tuple:
        """(``W h`` as fp32 [T, size], whether the reader must leave zeros behind); bias and sigmoid belong to the
        pass that applies the gate.  With few tokens the contraction's K-slices add themselves into a sum that is
        zero between uses (the reader clears it), which spares the slices' meeting in a workspace."""
        T = h.shape[0]
        if ctx is not None and self.proj.sums_slices_at_memory(T):
            n = T * self.size
            z = ctx.zeros(f"gate_logits{self.size}", n, torch.float32)[:n].view(T, self.size)
            self.proj(h, K.EPI_ADD_F32, z)
            return z, True
        return self.proj(h, K.EPI_STORE_F32), False


class DepthAverage(Part):
    """What a layer hands on is a weighted sum over the depth of the model: with X_0 the embedding's output and X_j
    the result of the layer j - 1 before this averaging, the layer with ``depth`` = n hands on
    ``sum_(j < n) a[j] X_j`` (so the first layer has n = 2).  ``total``: the largest ``depth`` in the model (the step
    keeps that many copies of the stream).  ``name``: the tensor's name below the part's prefix."""

    def __init__(self, depth: int, total: int, name: str = "weight"):
        super().__init__(depth=depth, total=total, name=name)
        if not 2 <= int(depth) <= int(total):
            raise ValueError(f"depth must be 2 to total ({total}), got {depth}")
        self.depth, self.total = int(depth), int(total)
        self.name = name
        self.weights: Optional[torch.Tensor] = None

    def param_specs(self):
        return {self.name: ParamSpec((self.depth,), "last_one_plus_normal")}

    def load(self, get: Any, runtime: Any) -> None:
        self.weights = get(self.name).to(torch.float32).contiguous()       # part of the residual sum: fp32
        self.one = torch.ones((1,), dtype=torch.float32, device=self.weights.device)


class GatedPreNormBlock(Block):
    """Pre-norm layer whose sublayers return through a gate, optionally followed by an average over the depth:

        x <- x + sigmoid(G1 n1 + b1) * mixer(n1),   n1 = norm1(x)
        x <- x + sigmoid(G2 n2 + b2) * ffn(n2),     n2 = norm2(x)          (a layer without feed-forward ends above)
        x <- sum_j a[j] X_j                                                (``depth_average``; X_j: see DepthAverage)

    Connections: ``mixer_gate`` and ``ffn_gate`` (:class:`ResidualGate`; a sublayer without one is added as it is),
    ``depth_average`` (:class:`DepthAverage`).  The residual stream stays fp32; a sublayer adds its result into a
    zeroed fp32 [tokens, hidden] buffer as it would into a residual stream, and ONE launch applies the gate, adds,
    leaves the buffer zero, forms the depth average where the layer ends, and norms what the next sublayer reads
    (across layers too: a layer whose successor in the run order is of this kind norms for it, ``link_next``)."""

    handles_pending = False

    def __init__(self, mixer: Any, ffn: Any, norms: Mapping[str, Any], connections: Any = None):
        super().__init__(mixer, ffn, norms, connections)
        if mixer is None:
            raise ValueError("a block needs a mixer")
        self.sublayers = []
        for part, norm, gate in ((mixer, "mixer_norm", "mixer_gate"), (ffn, "ffn_norm", "ffn_gate")):
            if part is None:
                continue
            n = self.norms.get(norm)
            if n is None or not (hasattr(n, "weight") and hasattr(n, "eps")) or getattr(n, "normed_kind", None) != K.NORMED_RMS:
                raise ValueError(f"a gated pre-norm block needs an RMS norm as {norm!r}")
            g = self.connections.get(gate)
            if g is not None and not hasattr(g, "logits"):
                raise ValueError(f"the connection {gate!r} must be a residual gate")
            self.sublayers.append((part, n, g))
        self.average = self.connections.get("depth_average")
        if self.average is not None and not hasattr(self.average, "depth"):
            raise ValueError("the connection 'depth_average' must be a depth average")
        self._next_norm: Any = None
        self._next_known = False

    def link_next(self, nxt: Any) -> None:
        """Told by the model which block follows this one in the run order: if it is always the same block of this
        kind, this block's last launch also norms the stream with that block's first norm."""
        norm = nxt.sublayers[0][1] if isinstance(nxt, GatedPreNormBlock) else None
        if self._next_known and norm is not self._next_norm:
            norm = None             # (a layer that runs in several places with different successors)
        self._next_norm, self._next_known = norm, True

    def forward(self, residual: torch.Tensor, ctx: Any, cache: Any, state: Optional[torch.Tensor],
                positions: Mapping[str, PositionEncoding]) -> None:
        T, d = residual.shape
        dtype = ctx.runtime.dtype
        y = ctx.zeros(f"sublayer_out{d}", T * d, torch.float32)[:T * d].view(T, d)
        avg, history = self.average, None
        if avg is not None:
            history = ctx.scratch("depth_history", avg.total * T * d)[:avg.total * T * d].view(avg.total, T, d)
            if avg.depth == 2:      # the model's first layer: what arrives is the embedding's output X_0
                K.gated_residual(residual, None, None, None, history=history, depth=1, average=avg.one)
        first_norm = self.sublayers[0][1]
        ahead, ctx.normed_ahead = getattr(ctx, "normed_ahead", None), None
        x = ahead[2] if ahead is not None and ahead[0] is residual and ahead[1] is first_norm else \
            first_norm.forward(residual)
        last = len(self.sublayers) - 1
        nn = self._next_norm
        tail = dict(norm_w=nn.weight, eps=nn.eps, out_dtype=dtype) if nn is not None else {}
        for i, (part, norm, gate) in enumerate(self.sublayers):
            # (a sublayer that ends with a bias may leave it to the pass that applies the gate)
            defer = {"defer_bias": True} if getattr(part, "can_defer_bias", False) else {}
            if part is self.mixer:
                part.forward(x, y, ctx, cache, state, positions, **defer)
            else:
                part.forward(x, y, ctx, **defer)
            ctx.settle(y)
            logits, clear = gate.logits(x, ctx) if gate is not None else (None, False)
            bias = gate.bias if gate is not None else None
            y_bias = part.output_bias if defer else None
            if i < last:
                nxt = self.sublayers[i + 1][1]
                x = K.gated_residual(residual, y, logits, bias, y_bias=y_bias, norm_w=nxt.weight, eps=nxt.eps,
                                     out_dtype=dtype, clear_gate=clear)
            elif avg is not None:
                x = K.gated_residual(residual, y, logits, bias, y_bias=y_bias, history=history, depth=avg.depth,
                                     average=avg.weights, clear_gate=clear, **tail)
            else:
                x = K.gated_residual(residual, y, logits, bias, y_bias=y_bias, clear_gate=clear, **tail)
        if nn is not None:
            ctx.normed_ahead = (residual, nn, x)


BLOCKS.register("prenorm", PreNormBlock)
BLOCKS.register("gated_prenorm", GatedPreNormBlock)
BLOCKS.register("result_norm", ResultNormBlock)
BLOCKS.register("hyper_prenorm", HyperPreNormBlock)
BLOCKS.register("postnorm", PostNormBlock)
CONNECTIONS.register("hyper_connection", HyperConnection)
CONNECTIONS.register("layer_scale", LayerScale)
CONNECTIONS.register("residual_gate", ResidualGate)
CONNECTIONS.register("depth_average", DepthAverage)
