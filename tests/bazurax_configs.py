"""Small Bazurax configurations with weights of a useful size, and helpers that run the engine and the plain
implementation on them.  The configurations differ from one another in every size and in the order of their
layers, and include values that are 1 (one head, one kv head, one expert, a window of one) or absent (no
rotation, a layer without feed-forward) and values that models often make equal but that need not be (key and
value sizes, the recurrence's inner width and the model's, the decays of two heads, the two factors of the
parallel mixers)."""
from __future__ import annotations

import functools
import json
import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch


def ret(heads, dim, vdim, decay, rot_dims=0, base=10000.0):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
    return m


def win(heads, kv, dim, vdim, scale, size):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": size}}


def par(left, r_heads, r_dim, left_scale=1.0, right_scale=1.0):
    return {"left": left, "right": {"heads": r_heads, "dim": r_dim}, "left_scale": left_scale, "right_scale": right_scale}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def model(vocab, width, layers, eps=1e-5):
    return {"architecture": "Bazurax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


CONFIGS: Dict[str, dict] = {
    # parallel mixers first; heads of 24 with values of 40, a recurrence whose inner width (3 x 16) is not the
    # model's; a retention with partial rotation and no feed-forward; one without rotation; a window of one
    "P": model(150, 72, [
        layer("parallel", par(win(6, 3, 24, 40, 0.3, 37), 3, 16, 0.7, 1.3), moe(40, 6, 3)),
        layer("retention", ret(3, 24, 16, (0.9, 0.97, 0.995), 12, 5000.0), None),
        layer("retention", ret(2, 32, 40, (0.99, 0.95)), dense(56)),
        layer("parallel", par(win(4, 4, 16, 8, 0.5, 1), 1, 40, 1.1, 0.4), dense(88))]),
    # one head everywhere it can be; one expert of which one is chosen; a window longer than most prompts; the whole
    # head rotated with a small base; width 48
    "Q": model(97, 48, [
        layer("retention", ret(1, 40, 24, (0.98,), 40, 300.0), moe(24, 1, 1)),
        layer("parallel", par(win(5, 1, 40, 16, 0.2, 150), 2, 24, 0.5, 0.5), None),
        layer("retention", ret(4, 16, 16, (0.999, 0.9, 0.5, 0.96875), 8, 1e6), moe(16, 5, 1))], eps=1e-6),
    # head sizes 64, 32 and 128 (the kernels that keep the state in registers and the tensor-core attention),
    # top 2 of 8, windows of 64 and 70, width 128
    "R": model(260, 128, [
        layer("retention", ret(3, 64, 32, (0.96875, 0.998, 0.9), 32, 100000.0), dense(192)),
        layer("parallel", par(win(4, 2, 64, 64, 0.125, 70), 2, 32, 0.6, 0.5), moe(64, 8, 2)),
        layer("retention", ret(1, 128, 64, (0.99,), 128, 10000.0), moe(64, 8, 2)),
        layer("parallel", par(win(2, 1, 32, 128, 0.2, 64), 1, 128, 1.0, 1.0), dense(96)),
        layer("parallel", par(win(8, 2, 128, 64, 0.1, 129), 2, 64, 0.9, 0.8), None)], eps=1e-6),
}
SEEDS = {"P": 31, "Q": 32, "R": 33}


def rank_of(i: int) -> int:
    """Width of layer i's small decay projection in the test weights (it is no key of the configuration)."""
    return (5, 16, 3, 24, 8)[i % 5]


def tensor_shapes(cfg: dict) -> Dict[str, Tuple[int, ...]]:
    """Names and shapes of a configuration's tensors, from the design's description (not from the package)."""
    d, V = cfg["width"], cfg["vocab"]
    s: Dict[str, Tuple[int, ...]] = {"embed": (V, d), "embed.norm": (d,), "final.norm": (d,)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        s[p + "norm1"] = (d,)
        if L["type"] == "retention":
            H, dk, dv = m["heads"], m["dim"], m["vdim"]
            s.update({p + "mix.q": (H * dk, d), p + "mix.k": (H * dk, d), p + "mix.v": (H * dv, d),
                      p + "mix.g": (H * dv, d), p + "mix.o": (d, H * dv)})
        else:
            a, b = m["left"], m["right"]
            H, G, dk, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            q = p + "mix.left."
            s.update({q + "q": (H * dk, d), q + "k": (G * dk, d), q + "v": (G * dv, d), q + "q.norm": (H * dk,),
                      q + "k.norm": (G * dk,), q + "g": (H, d), q + "o": (d, H * dv)})
            r, inner, rank = p + "mix.right.", b["heads"] * b["dim"], rank_of(i)
            for x in "rkvgw":
                s[r + "mu." + x] = (d,)
            for x in "rkvg":
                s[r + x] = (inner, d)
            s.update({r + "w1": (rank, d), r + "w2": (inner, rank), r + "w0": (inner,), r + "u": (b["heads"], b["dim"]),
                      r + "norm": (inner,), r + "o": (d, inner)})
        mlp = L["mlp"]
        if mlp is None:
            continue
        s[p + "norm2"] = (d,)
        if mlp["kind"] == "dense":
            s.update({p + "mlp.gate": (mlp["ff"], d), p + "mlp.up": (mlp["ff"], d), p + "mlp.down": (d, mlp["ff"])})
        else:
            f, E = mlp["expert"]["ff"], mlp["router"]["experts"]
            s[p + "mlp.router"] = (E, d)
            s[p + "mlp.router.b"] = (E,)
            for e in range(E):
                s.update({f"{p}mlp.e{e}.gate": (f, d), f"{p}mlp.e{e}.up": (f, d), f"{p}mlp.e{e}.down": (d, f)})
    return s


def make_weights(cfg: dict, seed: int, sharpen: float = 3.0, mild: bool = False) -> Dict[str, torch.Tensor]:
    """Weights (bfloat16): matrices ~ N(0, 1/in), the embedding N(0, 1), norm weights around 1, blends in (0, 1),
    decay biases around -1.5 (decays between 0.3 and 0.98 a token), bonuses and router biases of visible size.  The
    whole-projection norm weights are multiplied by ``sharpen`` so that the softmax is far from uniform and a
    wrong, missing or extra key moves the logits; routers are scaled up so that choices are not near ties.
    ``mild`` (whole models in bfloat16): flatter softmaxes and routers, so that a near tie that rounding tips the
    other way stays one row's affair (float32 runs carry the sharp cases)."""
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
        elif name.endswith(".q.norm") or name.endswith(".k.norm"):
            t = (1.0 + 0.2 * r) * sharpen ** 0.5
        elif ".mu." in name:
            t = torch.rand(shape, generator=g)
        elif name.endswith(".w0"):
            t = -1.5 + 1.0 * r
        elif name.endswith(".u"):
            t = 0.5 * r
        elif name.endswith(".router.b"):
            t = 0.5 * r
        elif "norm" in name:
            t = 1.0 + 0.2 * r
        elif name.endswith(".router"):
            t = (1.0 if mild else 3.0) * r / shape[1] ** 0.5
        elif name.endswith(".w2"):
            t = 1.5 * r / shape[1] ** 0.5
        else:
            t = r / shape[1] ** 0.5
        w[name] = t.to(torch.bfloat16)
    return w


def config_of(cfg: dict, w: Dict[str, torch.Tensor]):
    """The package's typed configuration, with the sizes that only the tensors give."""
    from dlgo_b200.config.bazurax import BazuraxConfig
    return BazuraxConfig.from_dict(cfg, shapes={n: tuple(t.shape) for n, t in w.items()})


def write_model(name: str, out_dir: str, sharpen: float = 3.0, mild: bool = False) -> str:
    from dlgo_b200.weights import save_tensors
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(CONFIGS[name], f)
    save_tensors(os.path.join(out_dir, "model.safetensors"), make_weights(CONFIGS[name], SEEDS[name], sharpen, mild=mild))
    return out_dir


def random_tokens(n: int, vocab: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


@functools.lru_cache(maxsize=64)
def _plain_cached(model_dir: str, tokens: tuple) -> torch.Tensor:
    import plain_bazurax as P
    cfg, w = P.read_model(model_dir, torch.float64)
    return P.forward(cfg, w, list(tokens)).to(torch.float32)


def plain_logits(model_dir: str, tokens: Sequence[int]) -> torch.Tensor:
    """Logits [T, vocab] of the plain implementation (float64 arithmetic) for one whole sequence."""
    return _plain_cached(model_dir, tuple(int(t) for t in tokens))


def row_error(got: torch.Tensor, ref: torch.Tensor) -> torch.Tensor:
    """Per row: root mean square of the difference (mean taken off) over the root mean square of the reference."""
    d = got.double() - ref.double()
    d = d - d.mean(-1, keepdim=True)
    r = ref.double() - ref.double().mean(-1, keepdim=True)
    return (d.pow(2).mean(-1) / r.pow(2).mean(-1).clamp_min(1e-30)).sqrt()


# A wrong, missing or extra key, a lost state, a wrong expert or a lost bias moves a row by 0.1 to 1 on this
# measure; float32 rounding stays below 1e-5 and bfloat16 rounding below 5e-2 through these few layers.  In bfloat16
# a router's near tie may fall the other way for a single token, which moves that row like a fault, and through
# the recurrences the rows after it a little: a few rows may differ.
TOL = {"float32": 1e-4, "bfloat16": 8e-2}


def assert_rows(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str) -> None:
    got = got.detach().float().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    e = row_error(got, ref)
    worst = int(e.argmax())
    if dtype == "bfloat16" and e.numel() >= 20:
        assert float(e.median()) <= TOL[dtype] / 3 and float((e > TOL[dtype]).float().mean()) <= 0.1, \
            f"{what}: median {float(e.median()):.3e}, {int((e > TOL[dtype]).sum())} of {e.numel()} rows over {TOL[dtype]:.1e}"
        return
    assert float(e.max()) <= TOL[dtype], f"{what}: row {worst} differs by {float(e.max()):.3e} (allowed {TOL[dtype]:.1e})"


class RowCheck:
    """Rows checked one at a time (decoded steps): float32 rows are asserted at once; bfloat16 rows are collected
    and judged together by :func:`assert_rows`' quantile rule when :meth:`done` is called."""

    def __init__(self, dtype: str, what: str):
        self.dtype, self.what, self.got, self.ref = dtype, what, [], []

    def add(self, got: torch.Tensor, ref: torch.Tensor, what: str) -> None:
        if self.dtype == "float32":
            assert_rows(got, ref, self.dtype, what)
        else:
            self.got.append(got.detach().float().cpu())
            self.ref.append(ref)

    def done(self) -> None:
        if self.got:
            assert_rows(torch.cat(self.got), torch.cat(self.ref), self.dtype, self.what)
