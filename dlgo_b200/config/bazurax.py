"""Typed configuration of the Bazurax design, read from its config.json keys.

A Bazurax model is a list of layers that norm a sublayer's RESULT before it joins the residual stream
(``x <- x + LN(mixer(x))``, ``x <- x + LN(ff(x))``, layer norms with a weight and no bias); the embedding is
normed too, and the head is the embedding table.  A layer's mixer is a retention (linear attention with a
fixed decay per head and rotary positions) or two mixers side by side whose results are added with fixed
factors: grouped-query softmax attention in a sliding window (queries and keys normed over their whole
projection, no positions, a sigmoid gate per head) and a time-mixing recurrence with a per-token decay.
The feed-forward is a gated dense one, a mixture of gated experts, or absent:

    {"architecture": "Bazurax", "vocab": V, "width": d, "norm": {"eps": e},
     "layers": [{"type": "retention",
                 "mixer": {"heads": H, "dim": n, "vdim": m, "decay": [H numbers], "rot": {"base": b, "dims": r}},
                 "mlp": null | {"kind": "dense", "ff": f}
                             | {"kind": "moe", "expert": {"ff": f}, "router": {"experts": E, "top": k}}},
                {"type": "parallel",
                 "mixer": {"left": {"heads": H, "kv_heads": G, "dim": n, "vdim": m, "scale": s, "mask": {"size": w}},
                           "right": {"heads": H2, "dim": n2},
                           "left_scale": a, "right_scale": c},
                 "mlp": ...}, ...]}

Tensor names: ``embed``, ``embed.norm``, ``final.norm`` and, for layer i, ``l<i>.norm1|norm2``;
retention ``l<i>.mix.q|k|v|g|o``; parallel ``l<i>.mix.left.q|k|v|g|o``, ``l<i>.mix.left.q.norm|k.norm``,
``l<i>.mix.right.mu.r|k|v|g|w``, ``l<i>.mix.right.r|k|v|g|o|w1|w2|w0|u|norm``; feed-forwards
``l<i>.mlp.gate|up|down`` or ``l<i>.mlp.router``, ``l<i>.mlp.router.b``, ``l<i>.mlp.e<j>.gate|up|down``.

The width of the decay's small projection (``w1`` [rank, d], ``w2`` [H2 n2, rank]) is no key of the file: it
is the shape of ``w1`` in the weight file (or, for a configuration without weights, the optional key
``right.rank``).  Every other size and every constant that can differ between two models of the design
comes from the keys; what the design fixes is in the parts this description names.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional, Tuple, Union

from .llama import _as, _need, _opt
from .monolix import _obj
from .registry import ConfigError, register_architecture
from .spec import ArchitectureSpec, LayerSpec, PartSpec, RunEntry

MIXER_KINDS = ("retention", "parallel")
# Positions enter only through angles computed from the position itself, and the recurrences have no horizon:
# the cache's size bounds a sequence.
NO_CONTEXT_LIMIT = 1 << 20


@dataclass(frozen=True)
class BazuraxRetention:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]
    rot_base: Optional[float]       # None: no rotation
    rot_dims: int


@dataclass(frozen=True)
class BazuraxWindowAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int


@dataclass(frozen=True)
class BazuraxTimeMix:
    heads: int
    dim: int
    rank: int                       # width of the decay's small projection
    rank_given: bool                # the key was in the file (else the size came from the weights)


@dataclass(frozen=True)
class BazuraxParallel:
    left: BazuraxWindowAttention
    right: BazuraxTimeMix
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class BazuraxDense:
    ff: int


@dataclass(frozen=True)
class BazuraxMoE:
    ff: int
    experts: int
    top: int


@dataclass(frozen=True)
class BazuraxLayer:
    kind: str
    mixer: Union[BazuraxRetention, BazuraxParallel]
    mlp: Union[None, BazuraxDense, BazuraxMoE]


def _retention(m: Mapping[str, Any], where: str) -> BazuraxRetention:
    heads, dim, vdim = _need(m, "heads", int), _need(m, "dim", int), _need(m, "vdim", int)
    if heads <= 0 or dim <= 0 or vdim <= 0:
        raise ConfigError(f"config.json: {where}heads, dim and vdim must be positive")
    decay = m.get("decay")
    if not isinstance(decay, (list, tuple)) or len(decay) != heads:
        raise ConfigError(f"config.json: {where}decay must list one number per head ({heads})")
    decay = tuple(_as(x, "decay", float) for x in decay)
    rot = _obj(m, "rot", where, required=False)
    base, dims = None, 0
    if rot is not None:
        base, dims = _need(rot, "base", float), _need(rot, "dims", int)
        if dims % 2 or not 0 <= dims <= dim or base <= 0:
            raise ConfigError(f"config.json: {where}rot.dims must be even and at most dim, rot.base positive")
        if dims == 0:
            base = None
    return BazuraxRetention(heads, dim, vdim, decay, base, dims)


def _window_attention(m: Mapping[str, Any], where: str) -> BazuraxWindowAttention:
    heads, kv, dim, vdim = _need(m, "heads", int), _need(m, "kv_heads", int), _need(m, "dim", int), _need(m, "vdim", int)
    if heads <= 0 or kv <= 0 or dim <= 0 or vdim <= 0 or heads % kv:
        raise ConfigError(f"config.json: {where}heads must be a positive multiple of kv_heads, dim and vdim positive")
    window = _need(_obj(m, "mask", where), "size", int)
    if window <= 0:
        raise ConfigError(f"config.json: {where}mask.size must be positive")
    return BazuraxWindowAttention(heads, kv, dim, vdim, _need(m, "scale", float), window)


def _time_mix(m: Mapping[str, Any], where: str, w1_shape: Optional[Tuple[int, ...]]) -> BazuraxTimeMix:
    heads, dim = _need(m, "heads", int), _need(m, "dim", int)
    if heads <= 0 or dim <= 0:
        raise ConfigError(f"config.json: {where}heads and dim must be positive")
    given = m.get("rank") is not None
    if given:
        rank = _need(m, "rank", int)
    elif w1_shape is not None and len(w1_shape) == 2:
        rank = int(w1_shape[0])
    else:
        raise ConfigError(f"config.json: {where}the width of the decay's small projection is the shape of the weight "
                          f"file's 'w1' tensor; without weights give it as {where}rank")
    if rank <= 0:
        raise ConfigError(f"config.json: {where}rank must be positive")
    return BazuraxTimeMix(heads, dim, rank, given)


def _mlp(mlp: Mapping[str, Any], where: str) -> Union[BazuraxDense, BazuraxMoE]:
    kind = mlp.get("kind")
    if kind == "dense":
        ff = _need(mlp, "ff", int)
        if ff <= 0:
            raise ConfigError(f"config.json: {where}ff must be positive")
        return BazuraxDense(ff)
    if kind == "moe":
        ff = _need(_obj(mlp, "expert", where), "ff", int)
        r = _obj(mlp, "router", where)
        experts, top = _need(r, "experts", int), _need(r, "top", int)
        if ff <= 0 or experts <= 0 or not 0 < top <= experts:
            raise ConfigError(f"config.json: {where}ff and experts must be positive and top between 1 and experts")
        return BazuraxMoE(ff, experts, top)
    raise ConfigError(f"config.json: {where}kind is {kind!r}; this design has 'dense' and 'moe' (or null for none)")


@dataclass(frozen=True)
class BazuraxConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[BazuraxLayer, ...]
    architecture: str = "Bazurax"

    shapes_from_file = True         # (a class attribute: the registry then hands from_dict the file's tensor shapes)

    # ------------------------------------------------------------------ parsing
    @classmethod
    def from_dict(cls, d: Mapping[str, Any], shapes: Optional[Mapping[str, Tuple[int, ...]]] = None) -> "BazuraxConfig":
        layers_in = d.get("layers")
        if not isinstance(layers_in, (list, tuple)) or not layers_in:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers: List[BazuraxLayer] = []
        for i, L in enumerate(layers_in):
            where = f"layers[{i}]."
            if not isinstance(L, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = L.get("type")
            if kind not in MIXER_KINDS:
                raise ConfigError(f"config.json: {where}type is {kind!r}; this design has {', '.join(MIXER_KINDS)}")
            m = _obj(L, "mixer", where)
            if kind == "retention":
                mixer: Any = _retention(m, where + "mixer.")
            else:
                w1 = None if shapes is None else shapes.get(f"l{i}.mix.right.w1")
                mixer = BazuraxParallel(_window_attention(_obj(m, "left", where + "mixer."), where + "mixer.left."),
                                        _time_mix(_obj(m, "right", where + "mixer."), where + "mixer.right.", w1),
                                        _need(m, "left_scale", float), _need(m, "right_scale", float))
            mlp_in = L.get("mlp")
            if mlp_in is not None and not isinstance(mlp_in, dict):
                raise ConfigError(f"config.json: {where}mlp must be null or an object")
            layers.append(BazuraxLayer(kind, mixer, None if mlp_in is None else _mlp(mlp_in, where + "mlp.")))
        vocab, width = _need(d, "vocab", int), _need(d, "width", int)
        if vocab <= 0 or width <= 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive")
        return cls(vocab=vocab, width=width, norm_eps=_need(_obj(d, "norm", ""), "eps", float), layers=tuple(layers),
                   architecture=str(d.get("architecture") or (d.get("architectures") or ["Bazurax"])[0]))

    def to_dict(self) -> Dict[str, Any]:
        layers = []
        for L in self.layers:
            if L.kind == "retention":
                a = L.mixer
                m: Dict[str, Any] = {"heads": a.heads, "dim": a.dim, "vdim": a.vdim, "decay": list(a.decay)}
                if a.rot_base is not None:
                    m["rot"] = {"base": a.rot_base, "dims": a.rot_dims}
            else:
                p = L.mixer
                right: Dict[str, Any] = {"heads": p.right.heads, "dim": p.right.dim}
                if p.right.rank_given:
                    right["rank"] = p.right.rank
                m = {"left": {"heads": p.left.heads, "kv_heads": p.left.kv_heads, "dim": p.left.dim, "vdim": p.left.vdim,
                              "scale": p.left.scale, "mask": {"size": p.left.window}},
                     "right": right, "left_scale": p.left_scale, "right_scale": p.right_scale}
            if L.mlp is None:
                mlp = None
            elif isinstance(L.mlp, BazuraxDense):
                mlp = {"kind": "dense", "ff": L.mlp.ff}
            else:
                mlp = {"kind": "moe", "expert": {"ff": L.mlp.ff}, "router": {"experts": L.mlp.experts, "top": L.mlp.top}}
            layers.append({"type": L.kind, "mixer": m, "mlp": mlp})
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "layers": layers}

    # ------------------------------------------------------- architecture as data
    def _retention_spec(self, a: BazuraxRetention) -> Tuple[PartSpec, Optional[str]]:
        pe = None if a.rot_base is None else f"rotary_{a.dim}_{a.rot_dims}_{a.rot_base!r}"
        return PartSpec("retention", {
            "hidden_size": self.width, "num_heads": a.heads, "qk_dim": a.dim, "v_dim": a.vdim, "decay": a.decay,
            "eps": self.norm_eps, "position_encoding": pe, "k_scale": a.dim ** -0.5,
            "names": {"q": "q", "k": "k", "v": "v", "gate": "g", "out": "o"}}), pe

    def _parallel_spec(self, p: BazuraxParallel, cache_group: str) -> PartSpec:
        left = PartSpec("wholenorm_attention", {
            "hidden_size": self.width, "num_heads": p.left.heads, "num_kv_heads": p.left.kv_heads,
            "qk_dim": p.left.dim, "v_dim": p.left.vdim, "scale": p.left.scale, "eps": self.norm_eps,
            "window": p.left.window, "qk_norm": True, "head_gate": True, "cache_group": cache_group,
            "names": {"q": "q", "k": "k", "v": "v", "q_norm": "q.norm", "k_norm": "k.norm", "gate": "g", "out": "o"}})
        right = PartSpec("time_mix", {
            "hidden_size": self.width, "num_heads": p.right.heads, "head_dim": p.right.dim, "decay_rank": p.right.rank,
            "eps": self.norm_eps,
            "names": {"mu": "mu.{}", "r": "r", "k": "k", "v": "v", "gate": "g", "out": "o", "decay_down": "w1",
                      "decay_up": "w2", "decay_bias": "w0", "bonus": "u", "norm": "norm"}})
        return PartSpec("parallel_mixers", {"mixers": (("left.", left, p.left_scale), ("right.", right, p.right_scale))})

    def _ffn_spec(self, mlp: Union[BazuraxDense, BazuraxMoE]) -> PartSpec:
        if isinstance(mlp, BazuraxDense):
            return PartSpec("swiglu", {"hidden_size": self.width, "intermediate_size": mlp.ff,
                                       "names": {"gate": "gate", "up": "up", "down": "down"}})
        return PartSpec("routed_experts", {
            "hidden_size": self.width, "intermediate_size": mlp.ff, "num_experts": mlp.experts, "top": mlp.top,
            "score": "softmax", "renormalize": True, "logit_bias": True, "gated": True, "activation": "silu",
            "names": {"router": "router", "logit_bias": "router.b", "expert": "e{}.", "gate": "gate", "up": "up",
                      "down": "down"}})

    def architecture_spec(self) -> ArchitectureSpec:
        d = self.width
        norm = PartSpec("layernorm", {"size": d, "eps": self.norm_eps, "name": ""})
        layers: List[LayerSpec] = []
        positions: Dict[str, PartSpec] = {}
        for i, L in enumerate(self.layers):
            if L.kind == "retention":
                mixer, pe = self._retention_spec(L.mixer)
                if pe is not None:
                    positions[pe] = PartSpec("rotary_frequencies", {"head_dim": L.mixer.dim, "rotary_dim": L.mixer.rot_dims,
                                                                    "theta": L.mixer.rot_base})
            else:
                mixer = self._parallel_spec(L.mixer, "window")
            norms = {"mixer_norm": norm}
            names = {"mixer": "mix.", "mixer_norm": "norm1"}
            ffn = None
            if L.mlp is not None:
                ffn = self._ffn_spec(L.mlp)
                norms["ffn_norm"] = norm
                names.update({"ffn": "mlp.", "ffn_norm": "norm2"})
            layers.append(LayerSpec(prefix=f"l{i}.", block="result_norm", mixer=mixer, ffn=ffn, norms=norms, names=names))
        spec = ArchitectureSpec(
            name=self.architecture, hidden_size=d, vocab_size=self.vocab, max_positions=NO_CONTEXT_LIMIT,
            embedding=PartSpec("token_embedding", {
                "vocab_size": self.vocab, "hidden_size": d, "name": "embed",
                "norm": ("layernorm", {"size": d, "eps": self.norm_eps, "name": "embed.norm"})}),
            embedding_prefix="",
            layers=layers, order=[RunEntry(i) for i in range(len(layers))],
            final_norm=norm, final_norm_prefix="final.norm",
            head=PartSpec("linear_head", {"vocab_size": self.vocab, "hidden_size": d, "tied_to": "embed"}),
            head_prefix="",
            position_encodings=positions,
            bos_token_id=None, stop_token_ids=(),
        )
        spec.validate()
        return spec


register_architecture("Bazurax", BazuraxConfig)
