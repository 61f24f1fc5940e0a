"""Small Ragilorn configurations with weights of a useful size, and helpers that run the engine and the plain
implementation on them.  The configurations differ from one another in every size and in the order of their
layers, and include values that are 1 (one head, one kv head, one expert, one chosen, a chunk of one, an
embedding scale of 1) or absent (no convolution, no chunks, no scaling of the rotation, no rotation, no logit cap, a
layer without feed-forward) and values that models often make equal but that need not be (key and value sizes, the
rotated share of a head, heads and kv heads)."""
from __future__ import annotations

import functools
import json
import os
from typing import Dict, Optional, Sequence, Tuple

import torch

from bazurax_configs import RowCheck, assert_rows, random_tokens, row_error      # noqa: F401  (shared test helpers)


def yarn(factor, original, fast=32.0, slow=1.0):
    return {"factor": factor, "original": original, "fast": fast, "slow": slow}


def att(heads, kv, dim, vdim, scale, rot_dims=0, base=10000.0, scaling=None, conv=None, chunk=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
        if scaling:
            m["rot"]["scaling"] = scaling
    if conv:
        m["conv"] = conv
    if chunk:
        m["mask"] = {"size": chunk}
    return m


def lat(heads, dim, rot_dim, vdim, kv_rank, scale, base=10000.0, scaling=None):
    rot = {"base": base, "dims": rot_dim}
    if scaling:
        rot["scaling"] = scaling
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale, "rot": rot}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def layer(mixer, mlp):
    return {"type": "latent_attention" if "kv_rank" in mixer else "attention", "mixer": mixer, "mlp": mlp}


def model(vocab, width, layers, eps=1e-5, emb=1.0, logit_scale=1.0, softcap=None):
    return {"architecture": "Ragilorn", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "embedding": {"scale": emb}, "logit_scale": logit_scale, "logit_softcap": softcap, "layers": layers}


CONFIGS: Dict[str, dict] = {
    # latent attention first; heads of 24 with values of 40 and three taps; a layer without feed-forward; a causal
    # layer without convolution or chunks whose whole head turns; top 3 of 6
    "P": model(150, 72, [
        layer(lat(3, 24, 8, 20, 40, 0.25, 5000.0, yarn(3.0, 64)), moe(40, 6, 3)),
        layer(att(6, 3, 24, 40, 0.3, 12, 7000.0, yarn(2.0, 100, 16.0, 2.0), conv=3, chunk=37), None),
        layer(att(4, 4, 16, 8, 0.4, 16, 300.0), dense(56)),
        layer(lat(2, 16, 16, 24, 18, 0.3, 900.0), dense(88))], emb=0.7, logit_scale=2.0, softcap=2.5),
    # one head everywhere it can be; one expert of which one is chosen; chunks longer than most prompts and a chunk
    # of one; two taps; no rotation at all in one layer; no cap on the logits; width 48
    "Q": model(97, 48, [
        layer(att(1, 1, 40, 16, 0.2, 8, 50000.0, yarn(8.0, 32), conv=2, chunk=500), moe(24, 1, 1)),
        layer(att(2, 1, 12, 20, 0.5, 0, conv=5, chunk=1), moe(16, 5, 1)),
        layer(lat(1, 8, 4, 40, 9, 0.4, 100.0, yarn(1.5, 16, 4.0, 0.5)), None)], eps=1e-6),
    # head sizes 64 and 128 (the tensor-core attention kernels), chunks of 64, 70 and 129, latent rows of 128 and
    # 192 numbers, top 2 of 8, width 128
    "R": model(260, 128, [
        layer(att(4, 2, 64, 64, 0.125, 32, 100000.0, yarn(4.0, 128), conv=4, chunk=70), dense(192)),
        layer(lat(4, 32, 32, 64, 96, 0.15, 1e6, yarn(2.0, 256)), moe(64, 8, 2)),
        layer(att(2, 1, 128, 64, 0.09, 64, 500000.0, yarn(2.0, 2048), conv=4, chunk=64), moe(64, 8, 2)),
        layer(lat(2, 64, 64, 128, 128, 0.1, 10000.0), dense(96)),
        layer(att(8, 2, 32, 128, 0.2, 32, 10000.0, None, conv=None, chunk=129), None)],
              eps=1e-6, emb=0.4, logit_scale=3.0, softcap=4.0),
}
SEEDS = {"P": 41, "Q": 42, "R": 43}


def tensor_shapes(cfg: dict) -> Dict[str, Tuple[int, ...]]:
    """Names and shapes of a configuration's tensors, from the design's description (not from the package)."""
    d, V = cfg["width"], cfg["vocab"]
    s: Dict[str, Tuple[int, ...]] = {"embed": (V, d), "head": (V, d), "final.norm": (d,)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        s.update({p + "norm1": (d,), p + "rg1": (d, d), p + "rg1.b": (d,), p + "dwa": (i + 2,)})
        H, dk, dv = m["heads"], m["dim"], m["vdim"]
        if L["type"] == "attention":
            G = m["kv_heads"]
            for n, rows in (("q", H * dk), ("k", G * dk), ("v", G * dv)):
                s[p + "mix." + n] = (rows, d)
                s[p + "mix." + n + ".b"] = (rows,)
                if m.get("conv"):
                    s[p + "mix." + n + ".conv"] = (rows, m["conv"])
            s.update({p + "mix.o": (d, H * dv), p + "mix.o.b": (d,)})
        else:
            R, r = m["kv_rank"], m["rot_dim"]
            s.update({p + "mix.q": (H * (dk + r), d), p + "mix.dkv": (R + r, d), p + "mix.dkv.norm": (R,),
                      p + "mix.uk": (H * dk, R), p + "mix.uv": (H * dv, R), p + "mix.o": (d, H * dv)})
        mlp = L["mlp"]
        if mlp is None:
            continue
        s.update({p + "norm2": (d,), p + "rg2": (d, d), p + "rg2.b": (d,)})
        if mlp["kind"] == "dense":
            s.update({p + "mlp.gate": (mlp["ff"], d), p + "mlp.up": (mlp["ff"], d), p + "mlp.down": (d, mlp["ff"])})
        else:
            f, E = mlp["expert"]["ff"], mlp["router"]["experts"]
            s[p + "mlp.router"] = (E, d)
            for e in range(E):
                s.update({f"{p}mlp.e{e}.gate": (f, d), f"{p}mlp.e{e}.up": (f, d), f"{p}mlp.e{e}.down": (d, f)})
    return s


def make_weights(cfg: dict, seed: int, sharpen: float = 3.0, mild: bool = False) -> Dict[str, torch.Tensor]:
    """Weights (bfloat16): matrices ~ N(0, 1/in), the embedding N(0, 1), norm weights around 1, biases of visible
    size, taps of visible size on every position, depth weights that give every earlier layer a share.  Query
    matrices are multiplied by ``sharpen`` so that the softmax is far from uniform and a wrong, missing or extra key
    moves the logits; routers are scaled up so that choices are not near ties.  ``mild`` (whole models in
    bfloat16): flatter softmaxes and routers, and experts whose results are a quarter as large, so that a router's
    near tie that rounding tips the other way stays one row's affair instead of colouring, through that position's
    keys and values, every later row of its sequence (float32 runs carry the sharp cases)."""
    if mild:
        sharpen = 1.5
    g = torch.Generator().manual_seed(seed)
    w = {}
    shapes = tensor_shapes(cfg)
    for name in sorted(shapes):
        shape = shapes[name]
        r = torch.randn(shape, generator=g)
        if name == "embed":
            t = r
        elif name.endswith(".conv"):
            t = 0.4 * r
            t[:, -1] += 1.0
        elif name.endswith(".dwa"):
            t = 0.3 * r
            t[-1] += 1.0
        elif name.endswith(".b"):
            t = 0.3 * r
        elif "norm" in name:
            t = 1.0 + 0.2 * r
        elif name.endswith(".router"):
            t = (1.0 if mild else 3.0) * r / shape[1] ** 0.5
        elif mild and ".mlp.e" in name and name.endswith(".down"):
            t = 0.25 * r / shape[1] ** 0.5
        elif name.endswith("mix.q"):
            t = sharpen * r / shape[1] ** 0.5
        else:
            t = r / shape[1] ** 0.5
        w[name] = t.to(torch.bfloat16)
    return w


def config_of(cfg: dict):
    from dlgo_b200.config.ragilorn import RagilornConfig
    return RagilornConfig.from_dict(cfg)


def write_model(name: str, out_dir: str, sharpen: float = 3.0, mild: bool = False) -> str:
    from dlgo_b200.weights import save_tensors
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(CONFIGS[name], f)
    save_tensors(os.path.join(out_dir, "model.safetensors"), make_weights(CONFIGS[name], SEEDS[name], sharpen, mild=mild))
    return out_dir


@functools.lru_cache(maxsize=64)
def _plain_cached(model_dir: str, tokens: tuple) -> torch.Tensor:
    import plain_ragilorn as P
    cfg, w = P.read_model(model_dir, torch.float64)
    return P.forward(cfg, w, list(tokens)).to(torch.float32)


def plain_logits(model_dir: str, tokens: Sequence[int]) -> torch.Tensor:
    """Logits [T, vocab] of the plain implementation (float64 arithmetic) for one whole sequence."""
    return _plain_cached(model_dir, tuple(int(t) for t in tokens))
