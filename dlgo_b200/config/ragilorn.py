"""Typed configuration of the Ragilorn design, read from its config.json keys.

A Ragilorn model is a list of pre-norm layers whose sublayers return to the residual stream through a learned
sigmoid gate and whose results are averaged over the depth of the model before the next layer reads them.  A
layer's mixer is grouped-query attention with biases, a short causal convolution over time on q, k and v,
rotary positions (YaRN-scaled, neighbouring pairs) on part of each head and a mask cut into chunks; or latent
attention (one compressed vector per position plus one rotated key part shared by all heads).  The feed-forward
is a gated dense one, a mixture of gated experts (sigmoid scores, the weight on the expert's input), or absent:

    {"architecture": "Ragilorn", "vocab": V, "width": d, "norm": {"eps": e}, "embedding": {"scale": s},
     "logit_scale": a, "logit_softcap": c,
     "layers": [{"type": "attention" | "latent_attention",
                 "mixer": {...sizes and constants of the mixer...},
                 "mlp": null | {"kind": "dense", "ff": f}
                             | {"kind": "moe", "expert": {"ff": f}, "router": {"experts": n, "top": k}}}, ...]}

Tensor names: ``embed``, ``head``, ``final.norm`` and, for layer i, ``l<i>.norm1|norm2``, ``l<i>.rg1|rg2[.b]``,
``l<i>.dwa``, ``l<i>.mix.*``, ``l<i>.mlp.*``.

Every size and every constant that can differ between two models of the design comes from the file; constants the
design fixes (which norm, which activation, the pairing of the rotation) are in the parts this description names.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional, Tuple

from .llama import _as, _need, _opt
from .registry import ConfigError, register_architecture
from .spec import ArchitectureSpec, LayerSpec, PartSpec, RunEntry

MIXER_KINDS = ("attention", "latent_attention")
# The design names no context limit (angles are formed from the position itself); the cache's size bounds a sequence.
NO_CONTEXT_LIMIT = 1 << 20


def _obj(d: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}{key!r} must be an object")
    return v


def _positive(d: Mapping[str, Any], key: str, where: str) -> int:
    try:
        v = _need(d, key, int)
    except ConfigError as e:
        raise ConfigError(f"config.json: {where}{key}: {e}") from None
    if v <= 0:
        raise ConfigError(f"config.json: {where}{key} must be positive, got {v}")
    return v


@dataclass(frozen=True)
class Rotation:
    base: float
    dims: int
    # YaRN: (factor, original context, fast, slow), or None for plain frequencies
    scaling: Optional[Tuple[float, float, float, float]] = None

    @classmethod
    def read(cls, rot: Mapping[str, Any], where: str) -> "Rotation":
        base, dims = _need(rot, "base", float), _positive(rot, "dims", where)
        if dims % 2 or base <= 1.0:
            raise ConfigError(f"config.json: {where}dims must be even and base above 1")
        sc = rot.get("scaling")
        scaling = None
        if sc is not None:
            if not isinstance(sc, dict):
                raise ConfigError(f"config.json: {where}scaling must be an object or null")
            scaling = tuple(_need(sc, k, float) for k in ("factor", "original", "fast", "slow"))
            if scaling[0] <= 0 or scaling[1] <= 0 or scaling[2] <= 0 or scaling[3] <= 0:
                raise ConfigError(f"config.json: {where}scaling's numbers must be positive")
        return cls(base, dims, scaling)

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            d["scaling"] = dict(zip(("factor", "original", "fast", "slow"), self.scaling))
        return d

    def part(self, head_dim: int) -> PartSpec:
        scaling = None
        if self.scaling is not None:
            f, o, fast, slow = self.scaling
            scaling = {"rope_type": "yarn", "factor": f, "original_max_position_embeddings": o, "beta_fast": fast,
                       "beta_slow": slow}
        return PartSpec("rotary_frequencies", {"head_dim": head_dim, "rotary_dim": self.dims, "theta": self.base,
                                               "scaling": scaling, "pairing": "interleaved"})

    def key(self) -> str:
        return "rot:" + ":".join(repr(v) for v in (self.base, self.dims) + (self.scaling or ()))


@dataclass(frozen=True)
class RagilornMixer:
    kind: str                   # one of MIXER_KINDS
    heads: int
    dim: int                    # per-head query/key size (latent attention: the unrotated part)
    vdim: int
    scale: float
    rot: Optional[Rotation]
    kv_heads: int = 1           # attention
    conv: Optional[int] = None  # attention: taps of the convolution over time (None: no convolution)
    chunk: Optional[int] = None  # attention: mask.size
    kv_rank: int = 0            # latent attention
    rot_dim: int = 0            # latent attention: size of the rotated part


@dataclass(frozen=True)
class RagilornMLP:
    kind: str                   # "dense" or "moe"
    ff: int
    experts: int = 0
    top: int = 0


@dataclass(frozen=True)
class RagilornConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    logit_scale: float
    logit_softcap: Optional[float]
    layers: Tuple[Tuple[RagilornMixer, Optional[RagilornMLP]], ...]
    architecture: str = "Ragilorn"

    # ------------------------------------------------------------------ parsing
    @staticmethod
    def _mixer(kind: str, m: Mapping[str, Any], where: str) -> RagilornMixer:
        heads, dim, vdim = (_positive(m, k, where) for k in ("heads", "dim", "vdim"))
        scale = _need(m, "scale", float)
        rot_in = m.get("rot")
        rot = Rotation.read(_obj(m, "rot", where), where + "rot.") if rot_in is not None else None
        if kind == "attention":
            kv = _opt(m, "kv_heads", int, heads)
            if kv <= 0 or heads % kv:
                raise ConfigError(f"config.json: {where}kv_heads ({kv}) must divide heads ({heads})")
            conv = _opt(m, "conv", int, None) or None       # (absent, null or 0: no convolution)
            if conv is not None and conv < 1:
                raise ConfigError(f"config.json: {where}conv must be at least 1, got {conv}")
            chunk = None
            if m.get("mask") is not None:
                chunk = _positive(_obj(m, "mask", where), "size", where + "mask.")
            if rot is not None and rot.dims > dim:
                raise ConfigError(f"config.json: {where}rot.dims ({rot.dims}) exceeds dim ({dim})")
            return RagilornMixer(kind, heads, dim, vdim, scale, rot, kv_heads=kv, conv=conv, chunk=chunk)
        kv_rank, rot_dim = _positive(m, "kv_rank", where), _positive(m, "rot_dim", where)
        if rot is None:
            raise ConfigError(f"config.json: {where}rot is required: the shared key part turns with the position")
        if rot_dim % 2:
            raise ConfigError(f"config.json: {where}rot_dim must be even, got {rot_dim}")
        # the rotated vector is the whole rot_dim part
        return RagilornMixer(kind, heads, dim, vdim, scale, Rotation(rot.base, rot_dim, rot.scaling), kv_rank=kv_rank,
                             rot_dim=rot_dim)

    @staticmethod
    def _mlp(mlp: Any, where: str) -> Optional[RagilornMLP]:
        if mlp is None:
            return None
        if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
            raise ConfigError(f"config.json: {where}mlp must be null or an object of kind 'dense' or 'moe'")
        if mlp["kind"] == "dense":
            return RagilornMLP("dense", _positive(mlp, "ff", where + "mlp."))
        ff = _positive(_obj(mlp, "expert", where + "mlp."), "ff", where + "mlp.expert.")
        r = _obj(mlp, "router", where + "mlp.")
        experts, top = _positive(r, "experts", where + "mlp.router."), _positive(r, "top", where + "mlp.router.")
        if top > experts:
            raise ConfigError(f"config.json: {where}mlp.router.top ({top}) exceeds experts ({experts})")
        return RagilornMLP("moe", ff, experts, top)

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "RagilornConfig":
        layers_in = d.get("layers")
        if not isinstance(layers_in, (list, tuple)) or not layers_in:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers: List[Tuple[RagilornMixer, Optional[RagilornMLP]]] = []
        for i, L in enumerate(layers_in):
            where = f"layers[{i}]."
            if not isinstance(L, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = L.get("type")
            if kind not in MIXER_KINDS:
                raise ConfigError(f"config.json: {where}type is {kind!r}; this design has {', '.join(MIXER_KINDS)}")
            layers.append((cls._mixer(kind, _obj(L, "mixer", where), where + "mixer."), cls._mlp(L.get("mlp"), where)))
        vocab, width = _need(d, "vocab", int), _need(d, "width", int)
        if vocab <= 0 or width <= 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive")
        emb = d.get("embedding")
        cap = _opt(d, "logit_softcap", float, None)
        if cap is not None and cap <= 0:
            raise ConfigError(f"config.json: 'logit_softcap' must be positive or null, got {cap}")
        return cls(vocab=vocab, width=width, norm_eps=_need(_obj(d, "norm", ""), "eps", float),
                   embedding_scale=_opt(emb, "scale", float, 1.0) if isinstance(emb, dict) else 1.0,
                   logit_scale=_opt(d, "logit_scale", float, 1.0), logit_softcap=cap, layers=tuple(layers),
                   architecture=str(d.get("architecture") or (d.get("architectures") or ["Ragilorn"])[0]))

    def to_dict(self) -> Dict[str, Any]:
        layers = []
        for m, f in self.layers:
            mixer: Dict[str, Any] = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale}
            if m.rot is not None:
                mixer["rot"] = m.rot.to_dict()
            if m.kind == "attention":
                mixer["kv_heads"] = m.kv_heads
                if m.conv is not None:
                    mixer["conv"] = m.conv
                if m.chunk is not None:
                    mixer["mask"] = {"size": m.chunk}
            else:
                mixer.update(kv_rank=m.kv_rank, rot_dim=m.rot_dim)
            mlp: Any = None
            if f is not None and f.kind == "dense":
                mlp = {"kind": "dense", "ff": f.ff}
            elif f is not None:
                mlp = {"kind": "moe", "expert": {"ff": f.ff}, "router": {"experts": f.experts, "top": f.top}}
            layers.append({"type": m.kind, "mixer": mixer, "mlp": mlp})
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale},
                "logit_scale": self.logit_scale, "logit_softcap": self.logit_softcap, "layers": layers}

    # ------------------------------------------------------- architecture as data
    def _mixer_spec(self, m: RagilornMixer, positions: Dict[str, PartSpec]) -> PartSpec:
        pe = None
        if m.rot is not None:
            pe = m.rot.key()
            positions.setdefault(pe, m.rot.part(m.dim if m.kind == "attention" else m.rot_dim))
        if m.kind == "attention":
            # layers whose keys and values have one shape share an allocation
            return PartSpec("short_conv_attention", {
                "hidden_size": self.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "qk_dim": m.dim,
                "v_dim": m.vdim, "scale": m.scale, "bias": True, "conv_taps": m.conv, "chunk": m.chunk,
                "position_encoding": pe, "cache_group": "full",
                "names": {"q": "q", "k": "k", "v": "v", "out": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b",
                          "out_bias": "o.b", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv"}})
        return PartSpec("latent_attention", {
            "hidden_size": self.width, "num_heads": m.heads, "qk_dim": m.dim, "v_dim": m.vdim, "kv_rank": m.kv_rank,
            "scale": m.scale, "eps": self.norm_eps, "rope_dim": m.rot_dim, "position_encoding": pe,
            "cache_group": "latent",
            "names": {"q": "q", "kv_down": "dkv", "kv_norm": "dkv.norm", "k_up": "uk", "v_up": "uv", "out": "o"}})

    def _ffn_spec(self, f: RagilornMLP) -> PartSpec:
        if f.kind == "dense":
            return PartSpec("swiglu", {"hidden_size": self.width, "intermediate_size": f.ff,
                                       "names": {"gate": "gate", "up": "up", "down": "down"}})
        return PartSpec("routed_experts", {
            "hidden_size": self.width, "intermediate_size": f.ff, "num_experts": f.experts, "top": f.top,
            "score": "sigmoid", "renormalize": False, "activation": "silu", "gated": True, "weight_on": "input",
            "names": {"router": "router", "expert": "e{}.", "gate": "gate", "up": "up", "down": "down"}})

    def architecture_spec(self) -> ArchitectureSpec:
        d, n = self.width, len(self.layers)
        norm = PartSpec("rmsnorm", {"size": d, "eps": self.norm_eps, "name": ""})
        gate = PartSpec("residual_gate", {"size": d, "names": {"weight": "", "bias": ".b"}})
        positions: Dict[str, PartSpec] = {}
        layers: List[LayerSpec] = []
        for i, (m, f) in enumerate(self.layers):
            norms = {"mixer_norm": norm}
            connections = {"mixer_gate": gate,
                           "depth_average": PartSpec("depth_average", {"depth": i + 2, "total": n + 1, "name": "dwa"})}
            names = {"mixer": "mix.", "mixer_norm": "norm1", "mixer_gate": "rg1", "depth_average": ""}
            ffn = None
            if f is not None:
                ffn = self._ffn_spec(f)
                norms["ffn_norm"] = norm
                connections["ffn_gate"] = gate
                names.update({"ffn": "mlp.", "ffn_norm": "norm2", "ffn_gate": "rg2"})
            layers.append(LayerSpec(prefix=f"l{i}.", block="gated_prenorm", mixer=self._mixer_spec(m, positions),
                                    ffn=ffn, norms=norms, names=names, connections=connections))
        spec = ArchitectureSpec(
            name=self.architecture, hidden_size=d, vocab_size=self.vocab, max_positions=NO_CONTEXT_LIMIT,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": d, "name": "embed",
                                                   "scale": self.embedding_scale}),
            embedding_prefix="",
            layers=layers, order=[RunEntry(i) for i in range(n)],
            final_norm=norm, final_norm_prefix="final.norm",
            head=PartSpec("linear_head", {"vocab_size": self.vocab, "hidden_size": d, "tied_to": None, "name": "head",
                                          "scale": self.logit_scale, "softcap": self.logit_softcap}),
            head_prefix="",
            position_encodings=positions,
            bos_token_id=None, stop_token_ids=(),
        )
        spec.validate()
        return spec


register_architecture("Ragilorn", RagilornConfig)
