"""A plain, slow implementation of the Bazurax design, one function per mechanism, written from its
equations only.  It shares no code with the package: it reads config.json and the safetensors file
itself and computes whole sequences on the CPU with torch in float32 or float64, token by token where
the design is a recurrence.

Notation: x is the residual stream [T, width]; a sublayer reads x itself and its result is normed before
it joins the stream:  x <- x + LN1(mixer(x)),  x <- x + LN2(ff(x)),  LN(u) = (u - mean) / sqrt(var + eps) * w.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional, Tuple

import torch

_DT = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32, "F64": torch.float64}


def read_model(model_dir: str, dtype: torch.dtype = torch.float64) -> Tuple[dict, Dict[str, torch.Tensor]]:
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    with open(os.path.join(model_dir, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        head = json.loads(f.read(n))
        blob = f.read()
    w = {}
    for name, info in head.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        t = torch.frombuffer(bytearray(blob[a:b]), dtype=_DT[info["dtype"]]).reshape(info["shape"])
        w[name] = t.to(dtype) if t.is_floating_point() else t
    return cfg, w


# ------------------------------------------------------------------------------------------ small pieces
def layer_norm(u: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    m = u.mean(-1, keepdim=True)
    var = ((u - m) ** 2).mean(-1, keepdim=True)
    return (u - m) / torch.sqrt(var + eps) * weight


def unit_rms(u: torch.Tensor, eps: float) -> torch.Tensor:
    return u / torch.sqrt((u * u).mean(-1, keepdim=True) + eps)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def rotate_half(t: torch.Tensor, base: float, dims: int, first: int = 0) -> torch.Tensor:
    """t [T, heads, dim], row n at position first + n: among the first `dims` entries of every head, entry i
    turns with entry i + dims/2 by the angle position * base^(-2i/dims); the other entries stay."""
    T = t.shape[0]
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=torch.float64)
    ang = (first + torch.arange(T, dtype=torch.float64))[:, None] * f[None, :]
    c, s = torch.cos(ang).to(t.dtype)[:, None, :], torch.sin(ang).to(t.dtype)[:, None, :]
    a, b = t[..., :half], t[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, t[..., dims:]], dim=-1)


# ------------------------------------------------------------------------------------------------ mixers
def retention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """Linear attention with one fixed decay per head, no softmax and no denominator."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, dk)
    k = (h @ w[p + "k"].T).view(T, H, dk)
    v = (h @ w[p + "v"].T).view(T, H, dv)
    rot = m.get("rot")
    if rot and rot["dims"]:
        q, k = rotate_half(q, rot["base"], rot["dims"]), rotate_half(k, rot["base"], rot["dims"])
    k = k * dk ** -0.5
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        lam = float(m["decay"][hd])
        S = torch.zeros(dk, dv, dtype=h.dtype)
        for t in range(T):
            S = lam * S + torch.outer(k[t, hd], v[t, hd])
            out[t, hd] = S.T @ q[t, hd]
    out = unit_rms(out, eps).reshape(T, H * dv)
    return (out * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def window_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """Grouped-query softmax attention inside a sliding window, queries and keys normed over their whole
    projection, no positions, one sigmoid gate per head."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = unit_rms(h @ w[p + "q"].T, eps) * w[p + "q.norm"]
    k = unit_rms(h @ w[p + "k"].T, eps) * w[p + "k.norm"]
    q, k = q.view(T, H, dk), k.view(T, G, dk)
    v = (h @ w[p + "v"].T).view(T, G, dv)
    gate = torch.sigmoid(h @ w[p + "g"].T)          # [T, H]
    size = m["mask"]["size"]
    per = H // G
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for i in range(T):
        lo = max(0, i - size + 1)
        for hd in range(H):
            g = hd // per
            s = (k[lo:i + 1, g] @ q[i, hd]) * m["scale"]
            out[i, hd] = torch.softmax(s, dim=0) @ v[lo:i + 1, g]
    out = out * gate[:, :, None]
    return out.reshape(T, H * dv) @ w[p + "o"].T


def time_mix(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """A recurrence whose decay depends on the token, per head and key channel, with a bonus for the
    current token; every projection reads its own blend of this token's input and the previous one's."""
    T, d = h.shape
    H, n = m["heads"], m["dim"]
    prev = torch.cat([torch.zeros(1, d, dtype=h.dtype), h[:-1]], dim=0)
    mix = {s: h + (prev - h) * w[p + "mu." + s] for s in "rkvgw"}
    r = (mix["r"] @ w[p + "r"].T).view(T, H, n)
    k = (mix["k"] @ w[p + "k"].T).view(T, H, n)
    v = (mix["v"] @ w[p + "v"].T).view(T, H, n)
    gate = silu(mix["g"] @ w[p + "g"].T)
    decay = torch.exp(-torch.exp(torch.tanh(mix["w"] @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"])).view(T, H, n)
    u = w[p + "u"]                                   # [H, n]
    out = torch.zeros(T, H, n, dtype=h.dtype)
    for hd in range(H):
        S = torch.zeros(n, n, dtype=h.dtype)
        for t in range(T):
            kv = torch.outer(k[t, hd], v[t, hd])
            out[t, hd] = (S + u[hd][:, None] * kv).T @ r[t, hd]
            S = decay[t, hd][:, None] * S + kv
    out = unit_rms(out, eps).reshape(T, H * n) * w[p + "norm"]
    return (out * gate) @ w[p + "o"].T


def parallel(h, w, p, m, eps):
    return (m["left_scale"] * window_attention(h, w, p + "left.", m["left"], eps) +
            m["right_scale"] * time_mix(h, w, p + "right.", m["right"], eps))


# ---------------------------------------------------------------------------------------- feed-forwards
def gated_mlp(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def router(h, w, p, r) -> Tuple[torch.Tensor, torch.Tensor]:
    """Chosen experts [T, top] and their weights: the largest logits win (the earlier of equals), and the
    weights are the softmax over the winners' logits alone."""
    z = h.to(w[p + "router"].dtype) @ w[p + "router"].T + w[p + "router.b"]
    val, idx = torch.sort(z, dim=-1, descending=True, stable=True)
    val, idx = val[:, :r["top"]], idx[:, :r["top"]]
    return idx, torch.softmax(val, dim=-1)


def experts(h, w, p, mlp):
    idx, wt = router(h, w, p, mlp["router"])
    y = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            y[t] += wt[t, j].to(h.dtype) * gated_mlp(h[t:t + 1], w, f"{p}e{e}.")[0]
    return y


# ------------------------------------------------------------------------------------------- whole model
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence; ``layers_out`` collects the stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = layer_norm(w["embed"][torch.tensor(tokens, dtype=torch.long)], w["embed.norm"], eps)
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        if L["type"] == "retention":
            y = retention(x, w, p + "mix.", L["mixer"], eps)
        elif L["type"] == "parallel":
            y = parallel(x, w, p + "mix.", L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        x = x + layer_norm(y, w[p + "norm1"], eps)
        mlp = L.get("mlp")
        if mlp is not None:
            y = gated_mlp(x, w, p + "mlp.") if mlp["kind"] == "dense" else experts(x, w, p + "mlp.", mlp)
            x = x + layer_norm(y, w[p + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return layer_norm(x, w["final.norm"], eps) @ w["embed"].T


def greedy_generate(cfg: dict, w: Dict[str, torch.Tensor], prompt: List[int], n: int) -> List[int]:
    """n tokens, each the largest logit after the whole sequence so far (recomputed from the start every time)."""
    seq, out = list(prompt), []
    for _ in range(n):
        t = int(forward(cfg, w, seq)[-1].argmax())
        out.append(t)
        seq.append(t)
    return out
