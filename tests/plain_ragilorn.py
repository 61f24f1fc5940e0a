"""A plain, slow implementation of the Ragilorn design, one function per mechanism, written from its
equations only.  It shares no code with the package: it reads config.json and the safetensors file
itself and computes whole sequences on the CPU with torch in float32 or float64.

Notation: X_0 = E[token] * s_e is the embedding's output; layer i turns its input x into
    y = x + sigmoid(G1 n1 + b1) * mixer(n1),   n1 = N1(x)
    X_(i+1) = y + sigmoid(G2 n2 + b2) * ff(n2),   n2 = N2(y)
and hands on  sum_(j <= i+1) a_i[j] X_j ;  N(u) = u / sqrt(mean(u^2) + eps) * w.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional, Tuple

import torch

_DT = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32, "F64": torch.float64}


def read_model(model_dir: str, dtype: torch.dtype = torch.float32) -> Tuple[dict, Dict[str, torch.Tensor]]:
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


def rms_norm(u: torch.Tensor, weight: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    r = u / torch.sqrt((u * u).mean(-1, keepdim=True) + eps)
    return r if weight is None else r * weight


def short_conv(u: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """u [T, C] over time, taps [C, n]: y_t = sum_j taps[:, j] * u_(t - n + 1 + j), zeros before the start."""
    T, C = u.shape
    n = taps.shape[1]
    padded = torch.cat([torch.zeros(n - 1, C, dtype=u.dtype), u], dim=0)
    y = torch.zeros_like(u)
    for j in range(n):
        y = y + taps[:, j] * padded[j:j + T]
    return y


def yarn_frequencies(rot: dict) -> Tuple[List[float], float]:
    """Frequencies of the pairs and the factor on cosine and sine."""
    dims, base = rot["dims"], rot["base"]
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = sc["factor"], sc["original"]

    def where(turns):
        return dims * math.log(orig / (2 * math.pi * turns)) / (2 * math.log(base))
    lo = max(math.floor(where(sc["fast"])), 0)
    hi = min(math.ceil(where(sc["slow"])), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate_pairs(t: torch.Tensor, rot: dict, first: int = 0) -> torch.Tensor:
    """t [T, heads, dim], row p at position first + p: of the first rot.dims entries of every head, entry 2i
    turns with entry 2i + 1."""
    T = t.shape[0]
    dims = rot["dims"]
    f, m = yarn_frequencies(rot)
    ang = torch.arange(first, first + T, dtype=torch.float64)[:, None] * torch.tensor(f, dtype=torch.float64)[None, :]
    c = (torch.cos(ang) * m).to(t.dtype)[:, None, :]
    s = (torch.sin(ang) * m).to(t.dtype)[:, None, :]
    u, v = t[..., 0:dims:2], t[..., 1:dims:2]
    turned = torch.stack([u * c - v * s, v * c + u * s], dim=-1).flatten(-2)
    return torch.cat([turned, t[..., dims:]], dim=-1)


def visible(T: int, chunk: Optional[int]) -> torch.Tensor:
    """[T, T] True where query i sees key j."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if chunk:
        ok = ok & (i // chunk == j // chunk)
    return ok


def softmax_attend(q, k, v, scale, ok):
    """q [T, H, d], k [T, H, d], v [T, H, dv], ok [T, T] -> [T, H, dv]."""
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    s = s.masked_fill(~ok[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hij,jhd->ihd", p, v)


def attention(h, w, p, m):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = h @ w[p + "q"].T + w[p + "q.b"]
    k = h @ w[p + "k"].T + w[p + "k.b"]
    v = h @ w[p + "v"].T + w[p + "v.b"]
    if m.get("conv"):
        q, k, v = short_conv(q, w[p + "q.conv"]), short_conv(k, w[p + "k.conv"]), short_conv(v, w[p + "v.conv"])
    q, k, v = q.view(T, H, d), k.view(T, G, d), v.view(T, G, dv)
    if m.get("rot"):
        q, k = rotate_pairs(q, m["rot"]), rotate_pairs(k, m["rot"])
    per = H // G
    k = k.repeat_interleave(per, dim=1)
    v = v.repeat_interleave(per, dim=1)
    mask = m.get("mask")
    out = softmax_attend(q, k, v, m["scale"], visible(T, mask["size"] if mask else None))
    return out.reshape(T, H * dv) @ w[p + "o"].T + w[p + "o.b"]


def latent_attention(h, w, p, m, eps):
    T = h.shape[0]
    H, d, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = (h @ w[p + "q"].T).view(T, H, d + dr)
    down = h @ w[p + "dkv"].T
    c = rms_norm(down[:, :R], w[p + "dkv.norm"], eps)
    kr = down[:, R:].view(T, 1, dr)
    rot = dict(m["rot"])
    rot["dims"] = dr
    qr = rotate_pairs(q[..., d:].contiguous(), rot)
    kr = rotate_pairs(kr, rot).expand(T, H, dr)
    kn = (c @ w[p + "uk"].T).view(T, H, d)
    v = (c @ w[p + "uv"].T).view(T, H, dv)
    out = softmax_attend(torch.cat([q[..., :d], qr], -1), torch.cat([kn, kr], -1), v, m["scale"], visible(T, None))
    return out.reshape(T, H * dv) @ w[p + "o"].T


def gated_ff(h, gate, up, down):
    return (torch.nn.functional.silu(h @ gate.T) * (h @ up.T)) @ down.T


def route(h, router, top):
    """Chosen experts [T, top] and their weights: sigmoid of the logits, largest first, as they are."""
    s = torch.sigmoid(h.to(torch.float32) @ router.to(torch.float32).T)
    wt, idx = torch.topk(s, top, dim=-1)
    return idx, wt.to(h.dtype)


def experts(h, w, p, mlp):
    idx, wt = route(h, w[p + "router"], mlp["router"]["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(idx[t].tolist(), wt[t]):
            q = f"{p}e{e}."
            out[t] += gated_ff((a * h[t])[None], w[q + "gate"], w[q + "up"], w[q + "down"])[0]
    return out


def feed_forward(h, w, p, mlp):
    if mlp["kind"] == "dense":
        return gated_ff(h, w[p + "gate"], w[p + "up"], w[p + "down"])
    return experts(h, w, p, mlp)


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens, layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence; ``layers_out`` collects what every layer hands on."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    history = [x]
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        n1 = rms_norm(x, w[p + "norm1"], eps)
        if L["type"] == "attention":
            y = attention(n1, w, p + "mix.", L["mixer"])
        elif L["type"] == "latent_attention":
            y = latent_attention(n1, w, p + "mix.", L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        x = x + torch.sigmoid(n1 @ w[p + "rg1"].T + w[p + "rg1.b"]) * y
        if L.get("mlp") is not None:
            n2 = rms_norm(x, w[p + "norm2"], eps)
            y = feed_forward(n2, w, p + "mlp.", L["mlp"])
            x = x + torch.sigmoid(n2 @ w[p + "rg2"].T + w[p + "rg2.b"]) * y
        history.append(x)
        a = w[p + "dwa"]
        x = sum(a[j] * history[j] for j in range(i + 2))
        if layers_out is not None:
            layers_out.append(x)
    z = rms_norm(x, w["final.norm"], eps) @ w["head"].T * cfg["logit_scale"]
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(z / cap) if cap else z


def greedy_generate(cfg: dict, w: Dict[str, torch.Tensor], prompt, n: int) -> List[int]:
    tokens = list(prompt)
    for _ in range(n):
        tokens.append(int(forward(cfg, w, tokens)[-1].argmax()))
    return tokens[len(prompt):]
