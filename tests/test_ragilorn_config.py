"""Ragilorn without a GPU: configuration and registry, parts and their constants, expected tensors, cache and state
needs, refusals, the random-weights mode, and the plain implementation's pieces by hand."""
import copy
import json
import math

import pytest
import torch

import plain_ragilorn as P
from ragilorn_configs import CONFIGS, SEEDS, att, dense, lat, layer, make_weights, model, moe, tensor_shapes, yarn, random_tokens, row_error


def spec_of(cfg):
    from dlgo_b200.config import config_from_dict
    return config_from_dict(cfg).architecture_spec()


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_expected_tensors_are_the_design_s(name):
    from dlgo_b200.engine.model import CausalLM
    m = CausalLM(spec_of(CONFIGS[name]))
    got = {n: tuple(ps.shape) for n, ps in m.expected_tensors().items()}
    assert got == tensor_shapes(CONFIGS[name])


def test_registry_and_round_trip():
    from dlgo_b200.config import RagilornConfig, config_from_dict, registered_architectures
    assert "Ragilorn" in registered_architectures()
    for cfg in CONFIGS.values():
        c = config_from_dict(cfg)
        assert isinstance(c, RagilornConfig)
        assert config_from_dict(c.to_dict()) == c
        assert config_from_dict(json.loads(json.dumps(c.to_dict()))) == c


def test_parts_carry_the_file_s_constants():
    spec = spec_of(CONFIGS["P"])
    assert spec.embedding.params["scale"] == 0.7
    assert spec.head.params["scale"] == 2.0 and spec.head.params["softcap"] == 2.5
    l0, l1, l2, l3 = spec.layers
    assert [l.block for l in spec.layers] == ["gated_prenorm"] * 4
    assert l0.mixer.kind == "latent_attention" and l0.mixer.params["rope_dim"] == 8 and l0.mixer.params["kv_rank"] == 40
    assert l0.ffn.kind == "routed_experts" and l0.ffn.params["weight_on"] == "input" and l0.ffn.params["top"] == 3
    assert l0.ffn.params["score"] == "sigmoid" and not l0.ffn.params["renormalize"] and l0.ffn.params["gated"]
    assert l1.mixer.kind == "short_conv_attention" and l1.mixer.params["conv_taps"] == 3 and l1.mixer.params["chunk"] == 37
    assert l1.ffn is None and set(l1.norms) == {"mixer_norm"} and "ffn_gate" not in l1.connections
    assert l2.mixer.params["chunk"] is None and l2.mixer.params["conv_taps"] is None
    assert [l.connections["depth_average"].params["depth"] for l in spec.layers] == [2, 3, 4, 5]
    assert all(l.connections["depth_average"].params["total"] == 5 for l in spec.layers)
    # every distinct rotation is a position encoding of its own; neighbouring pairs; YaRN where the file has it
    pes = spec.position_encodings
    assert len(pes) == 4 and all(p.params["pairing"] == "interleaved" for p in pes.values())
    pe = pes[l1.mixer.params["position_encoding"]]
    assert pe.params["rotary_dim"] == 12 and pe.params["theta"] == 7000.0
    assert pe.params["scaling"] == {"rope_type": "yarn", "factor": 2.0, "original_max_position_embeddings": 100.0,
                                    "beta_fast": 16.0, "beta_slow": 2.0}
    assert pes[l2.mixer.params["position_encoding"]].params["scaling"] is None
    # the latent layer's rotated vector is its rot_dim part whatever rot.dims says
    cfg = copy.deepcopy(CONFIGS["P"])
    cfg["layers"][0]["mixer"]["rot"]["dims"] = 6
    assert spec_of(cfg).position_encodings[spec_of(cfg).layers[0].mixer.params["position_encoding"]].params["rotary_dim"] == 8
    assert spec_of(CONFIGS["Q"]).layers[1].mixer.params["position_encoding"] is None


def test_cache_and_state_needs():
    from dlgo_b200.engine.model import CausalLM
    needs, borrows, states = CausalLM(spec_of(CONFIGS["P"])).cache_needs()
    assert borrows == [None] * 4
    assert (needs[0].planes, needs[0].head_dim, needs[0].num_kv_heads) == (1, 48, 1)          # latent 40 + rotated 8
    assert (needs[1].planes, needs[1].head_dim, needs[1].num_kv_heads, needs[1].window) == (2, 40, 3, None)
    assert (needs[2].head_dim, needs[2].num_kv_heads) == (16, 4)
    assert (needs[3].planes, needs[3].head_dim) == (1, 34)
    assert set(states) == {1} and states[1].shape == (2 * (6 * 24 + 3 * 24 + 3 * 40),)       # (taps - 1) x channels


@pytest.mark.parametrize("path, value, word", [
    (("layers", 0, "type"), "attn", "type"),
    (("layers", 1, "mixer", "kv_heads"), 4, "kv_heads"),
    (("layers", 1, "mixer", "rot", "dims"), 7, "dims"),
    (("layers", 1, "mixer", "rot", "dims"), 26, "dims"),
    (("layers", 1, "mixer", "mask", "size"), 0, "size"),
    (("layers", 0, "mixer", "kv_rank"), None, "kv_rank"),
    (("layers", 0, "mixer", "rot_dim"), 5, "rot_dim"),
    (("layers", 0, "mlp", "router", "top"), 7, "top"),
    (("layers", 2, "mlp", "kind"), "glu", "mlp"),
    (("layers", 1, "mixer", "rot", "scaling", "factor"), None, "factor"),
    (("norm",), None, "norm"),
    (("logit_softcap",), -1.0, "logit_softcap"),
])
def test_refusals_name_the_key(path, value, word):
    from dlgo_b200.config import ConfigError, config_from_dict
    cfg = copy.deepcopy(CONFIGS["P"])
    d = cfg
    for k in path[:-1]:
        d = d[k]
    d[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        config_from_dict(cfg)
    assert word in str(e.value)


def test_random_weights_mode(tmp_path):
    from dlgo_b200.config import config_from_dict
    from dlgo_b200.weights.random_init import write_random_model
    out = write_random_model(config_from_dict(CONFIGS["Q"]), 5, str(tmp_path / "m"))
    cfg, w = P.read_model(out, torch.float32)
    assert {n: tuple(t.shape) for n, t in w.items()} == tensor_shapes(CONFIGS["Q"])
    assert abs(float(w["l0.mix.q.conv"][:, -1].mean()) - 1.0) < 0.1 and abs(float(w["l1.dwa"][-1]) - 1.0) < 0.1
    assert torch.isfinite(P.forward(cfg, w, [1, 2, 3, 4])).all()


# ------------------------------------------------------------------ the plain implementation's pieces by hand
def test_short_convolution_by_hand():
    u = torch.tensor([[1.0, 10.0], [2.0, 20.0], [3.0, 30.0], [4.0, 40.0]])
    taps = torch.tensor([[0.5, 0.25, 1.0], [0.0, -1.0, 2.0]])          # the last tap is the token's own
    y = P.short_conv(u, taps)
    assert torch.allclose(y[:, 0], torch.tensor([1.0, 2.25, 4.0, 5.75]))
    assert torch.allclose(y[:, 1], torch.tensor([20.0, 30.0, 40.0, 50.0]))


def test_rotation_of_neighbouring_pairs_by_hand():
    rot = {"base": 100.0, "dims": 4}
    t = torch.tensor([[[1.0, 0.0, 0.0, 2.0, 7.0, 8.0]]] * 3)            # one head of six, four turn
    out = P.rotate_pairs(t, rot, first=1)                                # positions 1, 2, 3
    for r, p in enumerate((1, 2, 3)):
        a0, a1 = p * 1.0, p * 100.0 ** -0.5
        want = [math.cos(a0), math.sin(a0), -2 * math.sin(a1), 2 * math.cos(a1), 7.0, 8.0]
        assert torch.allclose(out[r, 0], torch.tensor(want), atol=1e-6)


def test_yarn_by_hand_and_in_the_package():
    from dlgo_b200.parts.rope import rotary_amplitude, rotary_frequencies
    rot = {"base": 10000.0, "dims": 16, "scaling": yarn(4.0, 64, 8.0, 1.0)}
    f, amp = P.yarn_frequencies(rot)
    assert amp == pytest.approx(0.1 * math.log(4.0) + 1.0)
    # where(t) = 16 ln(64 / (2 pi t)) / (2 ln 10000): where(8) = 0.209.. -> lo 0; where(1) = 2.01.. -> hi 3
    plain = [10000.0 ** (-2 * i / 16) for i in range(8)]
    ramp = [0.0, 1 / 3, 2 / 3, 1.0, 1.0, 1.0, 1.0, 1.0]
    assert f == pytest.approx([p / 4 * r + p * (1 - r) for p, r in zip(plain, ramp)])
    sc = {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 64, "beta_fast": 8.0, "beta_slow": 1.0}
    assert rotary_frequencies(16, 10000.0, sc) == pytest.approx(f, rel=1e-12)
    assert rotary_amplitude(sc) == pytest.approx(amp) and rotary_amplitude(None) == 1.0
    for cfg in CONFIGS.values():
        for L in cfg["layers"]:
            r = L["mixer"].get("rot")
            if r and r.get("scaling"):
                s = r["scaling"]
                sc = {"rope_type": "yarn", "factor": s["factor"], "original_max_position_embeddings": s["original"],
                      "beta_fast": s["fast"], "beta_slow": s["slow"]}
                dims = L["mixer"].get("rot_dim", r["dims"])
                assert rotary_frequencies(dims, r["base"], sc) == pytest.approx(P.yarn_frequencies({**r, "dims": dims})[0], rel=1e-12)
    # a ramp whose ends meet: hi - lo = 0 is replaced by 0.001, so index lo itself stays plain and all above are scaled
    f2, _ = P.yarn_frequencies({"base": 10000.0, "dims": 16, "scaling": yarn(2.0, 64, 2.0, 2.0)})
    assert f2[0] == plain[0] and f2[1] == plain[1] and f2[2] == pytest.approx(plain[2] / 2)


def test_chunks_by_hand():
    ok = P.visible(7, 3)
    assert ok.tolist() == [[j <= i and i // 3 == j // 3 for j in range(7)] for i in range(7)]
    assert P.visible(4, None).tolist() == [[j <= i for j in range(4)] for i in range(4)]


def test_router_and_weights_on_the_input_by_hand():
    h = torch.tensor([[1.0, 0.0], [0.0, 2.0]], dtype=torch.float64)
    router = torch.tensor([[2.0, 0.0], [0.0, 1.0], [-1.0, -1.0]], dtype=torch.float64)
    idx, wt = P.route(h, router, 2)
    assert idx.tolist() == [[0, 1], [1, 0]]
    assert torch.allclose(wt, torch.sigmoid(torch.tensor([[2.0, 0.0], [2.0, 0.0]], dtype=torch.float64)))     # not renormalized
    # one expert, chosen by both tokens: the result is expert(w h), not w expert(h)
    w = {"m.router": torch.tensor([[1.0, 1.0]], dtype=torch.float64), "m.e0.gate": torch.eye(2, dtype=torch.float64),
         "m.e0.up": torch.eye(2, dtype=torch.float64), "m.e0.down": torch.eye(2, dtype=torch.float64)}
    out = P.experts(h, w, "m.", {"router": {"top": 1}})
    a = torch.sigmoid(torch.tensor([1.0, 2.0], dtype=torch.float64))
    for t in range(2):
        x = a[t] * h[t]
        assert torch.allclose(out[t], torch.nn.functional.silu(x) * x)
        assert not torch.allclose(out[t], a[t] * torch.nn.functional.silu(h[t]) * h[t])


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_every_mechanism_moves_the_logits(name):
    """Knocking any one mechanism out of the test weights or configuration moves the logits far beyond the
    tolerances of the GPU tests, so those tests would see it missing."""
    cfg = CONFIGS[name]
    w = {k: v.double() for k, v in make_weights(cfg, SEEDS[name]).items()}
    tokens = random_tokens(80, cfg["vocab"], 3)
    ref = P.forward(cfg, w, tokens)

    def moved(cfg2, w2, least=0.02):
        return float(row_error(P.forward(cfg2, w2, tokens), ref).max()) > least

    def without(fn):
        c, v = copy.deepcopy(cfg), dict(w)
        fn(c, v)
        return c, v
    knocks = []
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        knocks.append(lambda c, v, p=p: v.__setitem__(p + "rg1", torch.zeros_like(v[p + "rg1"])))
        knocks.append(lambda c, v, p=p: v.__setitem__(p + "rg1.b", torch.zeros_like(v[p + "rg1.b"])))
        knocks.append(lambda c, v, p=p, i=i: v.__setitem__(p + "dwa", torch.eye(i + 2, dtype=torch.float64)[-1]))
        m = L["mixer"]
        if m.get("conv"):
            knocks.append(lambda c, v, i=i: c["layers"][i]["mixer"].__setitem__("conv", None))
        if m.get("mask") and m["mask"]["size"] < 80:
            knocks.append(lambda c, v, i=i: c["layers"][i]["mixer"].__setitem__("mask", None))
        if m.get("rot"):
            knocks.append(lambda c, v, i=i: c["layers"][i]["mixer"]["rot"].__setitem__("base", c["layers"][i]["mixer"]["rot"]["base"] * 3))
            if m["rot"].get("scaling"):
                knocks.append(lambda c, v, i=i: c["layers"][i]["mixer"]["rot"].__setitem__("scaling", None))
        if L["type"] == "attention":
            b = "mix.v.b" if (m.get("mask") or {}).get("size") == 1 else "mix.k.b"      # (one visible key: its score cancels)
            knocks.append(lambda c, v, p=p, b=b: v.__setitem__(p + b, torch.zeros_like(v[p + b])))
            knocks.append(lambda c, v, p=p: v.__setitem__(p + "mix.o.b", torch.zeros_like(v[p + "mix.o.b"])))
        else:
            knocks.append(lambda c, v, p=p: v.__setitem__(p + "mix.dkv.norm", torch.ones_like(v[p + "mix.dkv.norm"])))
        if L["mlp"] is not None:
            knocks.append(lambda c, v, p=p: v.__setitem__(p + "rg2", torch.zeros_like(v[p + "rg2"])))
    knocks.append(lambda c, v: c["embedding"].__setitem__("scale", c["embedding"]["scale"] * 1.5))
    knocks.append(lambda c, v: c.__setitem__("logit_scale", c["logit_scale"] * 1.5))
    if cfg["logit_softcap"]:
        knocks.append(lambda c, v: c.__setitem__("logit_softcap", None))
    for k, fn in enumerate(knocks):
        assert moved(*without(fn)), f"knock-out {k} of {name} is invisible"
