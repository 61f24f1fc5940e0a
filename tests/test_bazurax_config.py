"""Bazurax without a GPU: the configuration's keys, parts and constants, expected tensors, cache and state needs
and refusals; the plain implementation's pieces against hand-made cases; and the test weights' sensitivity."""
import copy
import json
import math
import os

import pytest
import torch

import plain_bazurax as P
from bazurax_configs import (CONFIGS, SEEDS, config_of, dense, layer, make_weights, model, moe, par, random_tokens, rank_of,
                             ret, row_error, tensor_shapes, win, write_model)

from dlgo_b200.config import ConfigError, config_from_dict, load_config
from dlgo_b200.engine.model import CausalLM


def plain_of(cfg, w, tokens):
    return P.forward(cfg, {k: v.double() for k, v in w.items()}, tokens).float()


def test_registry_and_keys():
    w = make_weights(CONFIGS["P"], 1)
    cfg = config_of(CONFIGS["P"], w)
    assert type(cfg).__name__ == "BazuraxConfig" and cfg.vocab == 150 and cfg.width == 72 and cfg.norm_eps == 1e-5
    assert [L.kind for L in cfg.layers] == ["parallel", "retention", "retention", "parallel"]
    p = cfg.layers[0].mixer
    a, b = p.left, p.right
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.window) == (6, 3, 24, 40, 0.3, 37)
    assert (b.heads, b.dim, b.rank) == (3, 16, rank_of(0)) and (p.left_scale, p.right_scale) == (0.7, 1.3)
    r = cfg.layers[1].mixer
    assert (r.heads, r.dim, r.vdim, r.decay, r.rot_base, r.rot_dims) == (3, 24, 16, (0.9, 0.97, 0.995), 5000.0, 12)
    assert cfg.layers[2].mixer.rot_base is None and cfg.layers[1].mlp is None
    e = cfg.layers[0].mlp
    assert (e.ff, e.experts, e.top) == (40, 6, 3) and cfg.layers[2].mlp.ff == 56
    assert config_of(cfg.to_dict(), w) == cfg


def test_the_decay_projection_s_width_comes_from_the_weight_file(tmp_path):
    d = write_model("Q", str(tmp_path / "q"))
    cfg = load_config(d)
    assert cfg.layers[1].mixer.right.rank == rank_of(1)
    with pytest.raises(ConfigError) as e:           # no weights at hand: the configuration says what it misses
        config_from_dict(CONFIGS["Q"])
    assert "rank" in str(e.value)
    c = copy.deepcopy(CONFIGS["Q"])
    c["layers"][1]["mixer"]["right"]["rank"] = 7
    assert config_from_dict(c).layers[1].mixer.right.rank == 7


def test_parts_and_their_constants():
    w = make_weights(CONFIGS["P"], 1)
    spec = config_of(CONFIGS["P"], w).architecture_spec()
    assert spec.name == "Bazurax" and spec.head.kind == "linear_head" and spec.head.params["tied_to"] == "embed"
    assert spec.embedding.params["norm"][0] == "layernorm" and spec.final_norm.kind == "layernorm"
    assert [ls.block for ls in spec.layers] == ["result_norm"] * 4
    assert [ls.mixer.kind for ls in spec.layers] == ["parallel_mixers", "retention", "retention", "parallel_mixers"]
    assert [None if ls.ffn is None else ls.ffn.kind for ls in spec.layers] == ["routed_experts", None, "swiglu", "swiglu"]
    (lp, left, ls_), (rp, right, rs_) = spec.layers[0].mixer.params["mixers"]
    assert (lp, rp, ls_, rs_) == ("left.", "right.", 0.7, 1.3)
    assert left.kind == "wholenorm_attention" and left.params["window"] == 37 and left.params["scale"] == 0.3
    assert left.params["qk_dim"] == 24 and left.params["v_dim"] == 40 and left.params["head_gate"] and left.params["qk_norm"]
    assert right.kind == "time_mix" and right.params["decay_rank"] == rank_of(0) and right.params["head_dim"] == 16
    m = spec.layers[1].mixer.params
    assert m["k_scale"] == 24 ** -0.5 and m["decay"] == (0.9, 0.97, 0.995) and m["position_encoding"] is not None
    assert spec.position_encodings[m["position_encoding"]].params == {"head_dim": 24, "rotary_dim": 12, "theta": 5000.0}
    assert spec.layers[2].mixer.params["position_encoding"] is None
    f = spec.layers[0].ffn.params
    assert f["logit_bias"] and f["gated"] and f["renormalize"] and f["top"] == 3 and f["num_experts"] == 6


def test_expected_tensors_are_the_design_s():
    for name, c in CONFIGS.items():
        w = make_weights(c, 1)
        t = CausalLM(config_of(c, w).architecture_spec()).expected_tensors()
        assert {n: tuple(ps.shape) for n, ps in t.items()} == tensor_shapes(c), name


def test_cache_and_state_needs():
    c = CONFIGS["P"]
    m = CausalLM(config_of(c, make_weights(c, 1)).architecture_spec())
    needs, borrows, states = m.cache_needs()
    assert borrows == [None] * 4 and needs[1] is None and needs[2] is None
    # keys and values share a page shape: the larger of the two sizes, as the next multiple of eight
    assert (needs[0].num_kv_heads, needs[0].head_dim, needs[0].window) == (3, 40, 37)
    assert (needs[3].num_kv_heads, needs[3].head_dim, needs[3].window) == (4, 16, 1)
    size = {i: math.prod(s.shape) if not isinstance(s, (list, tuple)) else sum(math.prod(x.shape) for x in s) for i, s in states.items()}
    assert size[1] == 3 * 24 * 16 and size[2] == 2 * 32 * 40
    assert size[0] == 3 * 16 * 16 + 72 and size[3] == 1 * 40 * 40 + 72          # the recurrence's state and the last input


@pytest.mark.parametrize("change, where", [
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=4), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["left"]["mask"].update(size=0), "mask"),
    (lambda c: c["layers"][0]["mixer"]["left"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mixer"].pop("right_scale"), "right_scale"),
    (lambda c: c["layers"][0]["mixer"].pop("right"), "right"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.9, 0.8]), "decay"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=13), "rot"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=26), "rot"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=7), "top"),
    (lambda c: c["layers"][0]["mlp"].update(kind="relu"), "kind"),
    (lambda c: c["layers"][0].update(type="attention"), "type"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.update(layers=[]), "layers"),
])
def test_refusals(change, where):
    c = copy.deepcopy(CONFIGS["P"])
    change(c)
    with pytest.raises(ConfigError) as e:
        config_of(c, make_weights(CONFIGS["P"], 1))
    assert where in str(e.value)


def test_random_model_mode_knows_the_design(tmp_path):
    from dlgo_b200.weights.random_init import write_random_model
    c = copy.deepcopy(CONFIGS["Q"])
    c["layers"][1]["mixer"]["right"]["rank"] = rank_of(1)
    out = write_random_model(config_from_dict(c), 3, str(tmp_path / "m"))
    cfg, w = P.read_model(out)
    assert cfg["architecture"] == "Bazurax" and {n: tuple(t.shape) for n, t in w.items()} == tensor_shapes(CONFIGS["Q"])
    assert abs(float(w["l0.norm1"].float().mean()) - 1) < 0.05          # plain norm weights lie around one
    assert load_config(out).layers[1].mixer.right.rank == rank_of(1)
    assert torch.isfinite(P.forward(cfg, {k: v.double() for k, v in w.items()}, [1, 2, 3])).all()


# ------------------------------------------------------------------------ the oracle's pieces
def test_layer_norm_by_hand():
    u = torch.tensor([[1.0, 2.0, 3.0, 6.0]], dtype=torch.float64)
    w = torch.tensor([1.0, 2.0, 1.0, 0.5], dtype=torch.float64)
    # mean 3, squared deviations 4 1 0 9 -> variance 3.5
    assert torch.allclose(P.layer_norm(u, w, 0.0), torch.tensor([[-2.0, -2.0, 0.0, 1.5]], dtype=torch.float64) / 3.5 ** 0.5)
    assert torch.allclose(P.layer_norm(u, w, 0.5), torch.tensor([[-2.0, -2.0, 0.0, 1.5]], dtype=torch.float64) / 2.0)


def test_rotation_by_hand():
    t = torch.zeros(3, 1, 6, dtype=torch.float64)
    t[:, 0, 0] = 1.0          # pairs (0, 2) and (1, 3) of the first four numbers; 4 and 5 pass
    t[:, 0, 5] = 7.0
    r = P.rotate_half(t, 100.0, 4)
    for p in range(3):
        assert torch.allclose(r[p, 0], torch.tensor([math.cos(p), 0.0, math.sin(p), 0.0, 0.0, 7.0], dtype=torch.float64))
    t = torch.zeros(2, 1, 4, dtype=torch.float64)
    t[:, 0, 1] = 1.0          # second pair turns at 100^(-2/4) = 0.1 rad a position
    assert torch.allclose(P.rotate_half(t, 100.0, 4)[1, 0], torch.tensor([0.0, math.cos(0.1), 0.0, math.sin(0.1)], dtype=torch.float64))


def test_retention_by_hand():
    """One head of one key and one value channel, no rotation, identity projections: o_t = sum_s decay^(t-s) k_s v_s q_t,
    whose unit norm is its sign."""
    m = ret(1, 1, 1, (0.5,))
    one = torch.ones(1, 1, dtype=torch.float64)
    w = {"q": one, "k": one * 2.0, "v": one * 3.0, "g": one, "o": one}
    h = torch.tensor([[1.0], [-1.0], [2.0]], dtype=torch.float64)
    # S: 6, 0.5 * 6 + 6 = 9, 0.5 * 9 + 24 = 28.5 (all positive); o = S q has the sign of h; times silu(h)
    got = P.retention(h, w, "", m, 0.0)
    assert torch.allclose(got, torch.sign(h) * P.silu(h))
    # with a wide head the norm divides by the root mean square over the value channels
    m = ret(1, 1, 2, (0.5,))
    w = {"q": one, "k": one, "v": torch.tensor([[3.0], [4.0]], dtype=torch.float64), "g": torch.ones(2, 1, dtype=torch.float64),
         "o": torch.eye(2, dtype=torch.float64)}
    got = P.retention(h[:1], w, "", m, 0.0)
    assert torch.allclose(got, torch.tensor([[3.0, 4.0]], dtype=torch.float64) / 12.5 ** 0.5 * P.silu(h[:1]))


def test_window_by_hand():
    """A window of two with equal scores: each output is the mean of this value and the one before."""
    m = win(1, 1, 1, 1, 1.0, 2)
    one = torch.ones(1, 1, dtype=torch.float64)
    w = {"q": one * 0.0, "k": one, "v": one, "q.norm": torch.ones(1, dtype=torch.float64), "k.norm": torch.ones(1, dtype=torch.float64),
         "g": one * 0.0, "o": one}
    h = torch.tensor([[1.0], [3.0], [7.0], [-1.0]], dtype=torch.float64)
    got = P.window_attention(h, w, "", m, 1e-6)
    assert torch.allclose(got, 0.5 * torch.tensor([[1.0], [2.0], [5.0], [3.0]], dtype=torch.float64))       # gate sigmoid(0)


def test_time_mix_by_hand():
    """One head of one channel with blends of one half: the second token's output is (S_1 + u k v) r with S_1 = k_1 v_1,
    and the decay enters only at the third."""
    m = {"heads": 1, "dim": 1}
    one = torch.ones(1, 1, dtype=torch.float64)
    w = {f"mu.{s}": torch.full((1,), 0.5, dtype=torch.float64) for s in "rkvgw"}
    w.update({"r": one, "k": one, "v": one, "g": one, "w1": one * 0.0, "w2": one, "w0": torch.tensor([math.log(math.log(2.0))], dtype=torch.float64),
              "u": one * 3.0, "norm": torch.ones(1, dtype=torch.float64), "o": one})
    h = torch.tensor([[2.0], [4.0], [-6.0]], dtype=torch.float64)
    # blends: 1, 3, -1 (each the mean with the token before, zeros before the first); decay exp(-exp(w0)) = 1/2
    # o_1 = 3 * 1 * 1 = 3; S_1 = 1; o_2 = (1 + 3 * 9) * 3 = 84; S_2 = 0.5 + 9 = 9.5; o_3 = (9.5 + 3) * (-1) = -12.5
    x = torch.tensor([1.0, 3.0, -1.0], dtype=torch.float64)
    want = torch.tensor([1.0, 1.0, -1.0], dtype=torch.float64) * P.silu(x)          # unit norm of one channel: the sign
    assert torch.allclose(P.time_mix(h, w, "", m, 0.0)[:, 0], want)
    w["norm"] = torch.ones(1, dtype=torch.float64) * 2.0
    assert torch.allclose(P.time_mix(h, w, "", m, 0.0)[:, 0], 2.0 * want)


def test_time_mix_state_by_hand():
    """Two channels: the bonus counts for the current token only, and the decay multiplies the state's key rows."""
    m = {"heads": 1, "dim": 2}
    I = torch.eye(2, dtype=torch.float64)
    w = {f"mu.{s}": torch.zeros(2, dtype=torch.float64) for s in "rkvgw"}
    w.update({"r": I, "k": I, "v": I, "g": I, "w1": torch.zeros(1, 2, dtype=torch.float64), "w2": torch.zeros(2, 1, dtype=torch.float64),
              "w0": torch.tensor([math.log(math.log(2.0)), math.log(math.log(4.0))], dtype=torch.float64),
              "u": torch.tensor([[10.0, 100.0]], dtype=torch.float64), "norm": torch.ones(2, dtype=torch.float64), "o": I})
    h = torch.tensor([[1.0, 2.0], [1.0, 1.0], [1.0, 1.0]], dtype=torch.float64)
    # S_1 = k v^T = [[1, 2], [2, 4]]; o_2 = (S_1 + diag(u) 1 1^T)^T r = [1 + 10 + 2 + 100, 2 + 10 + 4 + 100] = [113, 116]
    # S_2 = diag(1/2, 1/4) S_1 + 1 1^T = [[1.5, 2], [1.5, 2]]; o_3 = [1.5 + 10 + 1.5 + 100, 2 + 10 + 2 + 100] = [113, 114]
    o = torch.tensor([[113.0, 116.0], [113.0, 114.0]], dtype=torch.float64)
    want = o / (o * o).mean(-1, keepdim=True).sqrt() * P.silu(h[1:])
    assert torch.allclose(P.time_mix(h, w, "", m, 0.0)[1:], want)


def test_router_by_hand():
    w = {"router": torch.eye(4, dtype=torch.float64), "router.b": torch.tensor([0.0, 0.0, 5.0, 0.0], dtype=torch.float64)}
    h = torch.tensor([[3.0, 1.0, -3.0, 2.0]], dtype=torch.float64)
    idx, wt = P.router(h, w, "", {"experts": 4, "top": 2})          # logits 3 1 2 2: the bias lifts the third; ties: the earlier
    assert idx.tolist() == [[0, 2]]
    assert torch.allclose(wt, torch.softmax(torch.tensor([[3.0, 2.0]], dtype=torch.float64), -1))
    idx, wt = P.router(h, w, "", {"experts": 4, "top": 1})
    assert idx.tolist() == [[0]] and float(wt) == 1.0


def test_every_mechanism_shows_in_the_test_weights():
    """Knocking a mechanism out of the oracle's inputs moves the logits far beyond the tolerances."""
    for name in CONFIGS:
        cfg = CONFIGS[name]
        w = make_weights(cfg, SEEDS[name])
        tokens = random_tokens(60, cfg["vocab"], 2)
        ref = plain_of(cfg, w, tokens)
        knock = {"router bias": (lambda n: n.endswith(".router.b"), 0.0), "bonus": (lambda n: n.endswith(".u"), 0.0),
                 "blends": (lambda n: ".mu." in n, 0.0), "decay bias": (lambda n: n.endswith(".w0"), -8.0),
                 "decay projection": (lambda n: n.endswith(".w2"), 0.0), "whole norm": (lambda n: n.endswith(".k.norm"), 1.0),
                 "group norm": (lambda n: n.endswith("right.norm"), 1.0), "head gate": (lambda n: n.endswith("left.g"), 0.0),
                 "embedding norm": (lambda n: n == "embed.norm", 1.0), "result norm": (lambda n: n.endswith("norm1"), 1.0)}
        for what, (pick, value) in knock.items():
            if what == "router bias" and name == "Q":
                continue                                     # one expert, or one of five by a wide margin
            w2 = {k: (torch.full_like(v, value) if pick(k) else v) for k, v in w.items()}
            assert float(row_error(plain_of(cfg, w2, tokens), ref).median()) > 1e-2, (name, what)
        for path, value, what in [(("left", "mask", "size"), None, "window"), (("left_scale",), 0.0, "left factor"),
                                  (("right_scale",), 0.0, "right factor"), (("left", "scale"), 0.01, "score scale")]:
            c2 = copy.deepcopy(cfg)
            for L in c2["layers"]:
                if L["type"] != "parallel":
                    continue
                at = L["mixer"]
                for k in path[:-1]:
                    at = at[k]
                at[path[-1]] = value if value is not None else at[path[-1]] + 5 if at[path[-1]] < 30 else at[path[-1]] // 3
            e = row_error(plain_of(c2, w, tokens), ref)
            assert float(e.max() if what == "window" else e.median()) > 1e-2, (name, what)
        c2 = copy.deepcopy(cfg)
        for L in c2["layers"]:
            if L["type"] == "retention":
                L["mixer"]["decay"] = [0.5 * x for x in L["mixer"]["decay"]]
                L["mixer"].pop("rot", None)
        assert float(row_error(plain_of(c2, w, tokens), ref).median()) > 1e-2, (name, "decay and rotation")
