"""Bazurax on the GPU against the plain implementation (tests/plain_bazurax.py): every mechanism alone (its
kernels, and one-layer models that hold nothing else), then whole models through the engine's step function, its
cache and state, and the public entry point."""
import copy
import json
import math
import os

import pytest
import torch

import plain_bazurax as P
from bazurax_configs import (CONFIGS, SEEDS, RowCheck, assert_rows, config_of, dense, layer, make_weights, model, moe, par,
                             plain_logits, random_tokens, ret, row_error, win, write_model)

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
DEV = "cuda:0"


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    root = tmp_path_factory.mktemp("bazurax")
    out = {(n, "float32"): write_model(n, str(root / n)) for n in CONFIGS}
    out.update({(n, "bfloat16"): write_model(n, str(root / (n + "_mild")), mild=True) for n in CONFIGS})
    return out


_engines = {}


def engine_for(model_dir, dtype, **kw):
    from dlgo_b200.engine.engine import Engine
    key = (model_dir, dtype, tuple(sorted(kw.items())))
    if key not in _engines:
        kw.setdefault("max_tokens", 4096)
        _engines[key] = Engine(model_dir, dtype=dtype, **kw)
    return _engines[key]


def engine_of(cfg, w, dtype, **kw):
    from dlgo_b200.engine.engine import Engine
    kw.setdefault("max_tokens", 2048)
    return Engine(spec=config_of(cfg, w).architecture_spec(), tensors=w, dtype=dtype, **kw)


def plain_of(cfg, w, tokens):
    return P.forward(cfg, {k: v.double() for k, v in w.items()}, tokens).float()


def run_whole(eng, tokens):
    s = eng.take_slot()
    try:
        return eng.step([s], [tokens], [list(range(len(tokens)))])
    finally:
        eng.free_slot(s)


def prefill_then_decode(eng, tokens, start):
    s = eng.take_slot()
    got = [eng.step([s], [tokens[:start]], [list(range(start))]).clone()]
    got += [eng.step([s], [tokens[p:p + 1]]).clone() for p in range(start, len(tokens))]
    eng.free_slot(s)
    return torch.cat(got)


# ------------------------------------------------------------------ mechanisms alone: the kernels
@pytest.mark.parametrize("T", [3, 100])
@pytest.mark.parametrize("act_dtype", [torch.float32, torch.bfloat16])
def test_layer_norm_and_the_norm_of_a_result(T, act_dtype):
    from dlgo_b200.csrc import kernels as K
    g = torch.Generator().manual_seed(T)
    loose = dict(rtol=1e-2, atol=1e-2) if act_dtype == torch.bfloat16 else dict(rtol=1e-5, atol=1e-5)
    for d in (40, 72, 1000, 4096):
        # rows with a mean far from zero: the variance is of the deviations, not the mean square
        x, y = torch.randn(T, d, generator=g), 3.0 + 2.0 * torch.randn(T, d, generator=g)
        w, eps = 1 + 0.2 * torch.randn(d, generator=g), 1e-5
        ref = P.layer_norm(y.double(), w.double(), eps)
        out = K.layernorm_rows(y.to(DEV), w.to(DEV), eps, act_dtype)
        assert torch.allclose(out.cpu().double(), ref, **loose)
        rows = torch.tensor([T - 1, 0], dtype=torch.int32)
        out = K.layernorm_rows(y.to(DEV), w.to(DEV), eps, act_dtype, rows.to(DEV))
        assert torch.allclose(out.cpu().double(), ref[[T - 1, 0]], **loose)
        yd = y.to(DEV)
        assert K.layernorm_rows(yd, w.to(DEV), eps, torch.float32, in_place=True) is yd
        assert torch.allclose(yd.cpu().double(), ref, rtol=1e-5, atol=1e-5)
        xd, yd = x.to(DEV), y.to(DEV)
        act = K.add_normed(xd, yd, w.to(DEV), eps, None if act_dtype == torch.float32 else act_dtype, K.NORMED_LAYER, clear_y=True)
        assert torch.allclose(xd.cpu().double(), x.double() + ref, rtol=1e-5, atol=1e-5)      # the stream stays fp32
        assert float(yd.abs().max()) == 0.0                                                  # left zero for the next sublayer
        if act_dtype == torch.float32:
            assert act is None
        else:
            assert torch.equal(act.float(), xd.to(act_dtype).float())
        xd, yd = x.to(DEV), y.to(DEV)
        K.add_normed(xd, yd, w.to(DEV), eps, None, K.NORMED_RMS, clear_y=False)
        assert torch.allclose(xd.cpu().double(), x.double() + P.unit_rms(y.double(), eps) * w.double(), rtol=1e-5, atol=1e-5)
        assert torch.equal(yd.cpu(), y)


@pytest.mark.parametrize("H, dk, rot", [(3, 24, 12), (1, 40, 40), (2, 64, 32), (4, 16, 0), (2, 128, 128), (5, 6, 2)])
def test_rotation_and_key_scale(H, dk, rot):
    from dlgo_b200.csrc import kernels as K
    g = torch.Generator().manual_seed(dk)
    pos = torch.tensor([0, 1, 2, 63, 64, 1000, 70001, 5, 130], dtype=torch.int32)
    T, base, ks, extra = pos.numel(), 3000.0, dk ** -0.5, 11
    proj = torch.randn(T, 2 * H * dk + extra, generator=g)
    q, k = proj[:, :H * dk].double().view(T, H, dk), proj[:, H * dk:2 * H * dk].double().view(T, H, dk)
    if rot:
        f = torch.tensor([base ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float64)
        q = torch.stack([P.rotate_half(q[t:t + 1], base, rot, first=int(pos[t]))[0] for t in range(T)])
        k = torch.stack([P.rotate_half(k[t:t + 1], base, rot, first=int(pos[t]))[0] for t in range(T)])
    pd = proj.to(DEV)
    K.rotate_scale(pd, 0, H * dk, f.float().to(DEV) if rot else None, rot, pos.to(DEV), H, dk, ks)
    got = pd.cpu().double()
    assert torch.equal(got[:, 2 * H * dk:], proj[:, 2 * H * dk:].double())              # what follows is not touched
    for t in range(T):
        # fp32 angles: an angle of 70001 rad carries an absolute error of ~4e-3 rad
        tol = 3e-4 if int(pos[t]) <= 1000 else 2e-2
        assert torch.allclose(got[t, :H * dk].view(H, dk), q[t], atol=tol * 4, rtol=tol), (t, "q")
        assert torch.allclose(got[t, H * dk:2 * H * dk].view(H, dk), k[t] * ks, atol=tol, rtol=tol), (t, "k")


@pytest.mark.parametrize("act_dtype", [torch.float32, torch.bfloat16])
def test_blends_with_the_previous_token(act_dtype):
    """Three sequences in one step: one that starts (its predecessor is the slot's zeros), one that goes on from a
    stored input, one of a single token."""
    from dlgo_b200.csrc import kernels as K
    g = torch.Generator().manual_seed(4)
    d, off = 40, 24
    lens, slots = [5, 3, 1], [2, 0, 3]
    x = torch.randn(sum(lens), d, generator=g)
    mu = torch.rand(5, d, generator=g)
    state = torch.zeros(4, off + d)
    state[:, :off] = 7.0
    state[0, off:] = torch.randn(d, generator=g)
    state[3, off:] = torch.randn(d, generator=g)
    token_seq = torch.tensor(sum(([i] * n for i, n in enumerate(lens)), []), dtype=torch.int32)
    prev, at = [], 0
    for i, n in enumerate(lens):
        prev += [state[slots[i], off:]] + [x[at + j] for j in range(n - 1)]
        at += n
    prev = torch.stack(prev).double()
    ref = x.double()[None] + (prev - x.double())[None] * mu.double()[:, None]
    out = K.token_shift_mix(x.to(DEV), mu.to(DEV), token_seq.to(DEV), torch.tensor(slots, dtype=torch.int32, device=DEV),
                            state.to(DEV), off, act_dtype)
    tol = 2e-2 if act_dtype == torch.bfloat16 else 1e-6
    assert torch.allclose(out.cpu().double(), ref, atol=tol, rtol=tol)


@pytest.mark.parametrize("n, top", [(6, 3), (1, 1), (5, 1), (8, 2), (12, 2), (64, 8), (33, 5)])
def test_router_with_a_bias_on_the_logits(n, top):
    from dlgo_b200.csrc import kernels as K
    g = torch.Generator().manual_seed(n)
    T, d = 57, 72
    h = torch.randn(T, d, generator=g)
    w = {"router": (3.0 * torch.randn(n, d, generator=g) / d ** 0.5), "router.b": 2.0 * torch.randn(n, generator=g)}
    idx_ref, wt_ref = P.router(h.double(), {k: v.double() for k, v in w.items()}, "", {"experts": n, "top": top})
    idx, wt, gate, _ = K.moe_router(h.to(DEV), w["router"].to(DEV), None, n, False, top, 1, 1, False, True,
                                    logit_bias=w["router.b"].to(DEV))
    z = h.double() @ w["router"].double().T + w["router.b"].double()
    for t in range(T):
        got, want = idx[t].tolist(), idx_ref[t].tolist()
        if sorted(got) != sorted(want):                 # only a near tie may differ
            a, b = (set(got) - set(want)).pop(), (set(want) - set(got)).pop()
            assert abs(float(z[t, a] - z[t, b])) < 1e-4
            continue
        order = [got.index(e) for e in want]
        assert torch.allclose(wt[t].cpu().double()[order], wt_ref[t], atol=1e-5)
    without, _ = P.router(h.double(), {"router": w["router"].double(), "router.b": torch.zeros(n, dtype=torch.float64)}, "",
                          {"experts": n, "top": top})
    assert n == 1 or not torch.equal(without, idx_ref)          # the bias decides some choices


@pytest.mark.parametrize("act_dtype", [torch.float32, torch.bfloat16])
def test_unit_norm_per_head_and_gate(act_dtype):
    from dlgo_b200.csrc import kernels as K
    g = torch.Generator().manual_seed(2)
    tol = 2e-2 if act_dtype == torch.bfloat16 else 1e-5
    for H, dv in ((3, 16), (1, 40), (2, 128), (5, 6)):
        T, eps, scale = 9, 1e-5, 0.7
        o = 5.0 * torch.randn(T, H * dv, generator=g)
        gate = torch.randn(T, H * dv, generator=g)
        w = 1 + 0.3 * torch.randn(H * dv, generator=g)
        ref = P.unit_rms(o.double().view(T, H, dv), eps).reshape(T, H * dv) * P.silu(gate.double()) * scale
        out = K.gated_rmsnorm(o.to(DEV), gate.to(DEV), None, eps, act_dtype, group=dv, gate_act=K.GATE_SILU, scale=scale)
        assert torch.allclose(out.cpu().double(), ref, atol=tol, rtol=tol)
        out = K.gated_rmsnorm(o.to(DEV), gate.to(DEV), w.to(DEV), eps, act_dtype, group=dv, gate_act=K.GATE_SILU, scale=scale)
        assert torch.allclose(out.cpu().double(), ref * w.double(), atol=tol, rtol=tol)
        a = torch.randn(T, H * dv, generator=g)
        hg = torch.rand(T, H, generator=g)
        ad = a.to(DEV).to(act_dtype)
        K.scale_heads(ad, hg.to(DEV), dv)
        want = a.to(act_dtype).double().view(T, H, dv) * hg.double()[:, :, None]
        assert torch.allclose(ad.cpu().double().view(T, H, dv), want, atol=tol, rtol=tol)


# --------------------------------------------------- mechanisms alone: one-layer models that hold nothing else
def one_layer(kind, mixer, mlp=None, width=48, vocab=60):
    return model(vocab, width, [layer(kind, copy.deepcopy(mixer), mlp)], eps=1e-6)


def check_model(cfg, w, dtype, what, n=150, start=70, seed=6):
    """Whole prompt, and a prompt followed by token-by-token decoding, against the oracle."""
    tokens = random_tokens(n, cfg["vocab"], seed)
    ref = plain_of(cfg, w, tokens)
    eng = engine_of(cfg, w, dtype)
    assert_rows(run_whole(eng, tokens), ref, dtype, f"{what}: whole")
    assert_rows(prefill_then_decode(eng, tokens, start), ref, dtype, f"{what}: prefill then decode")
    assert_rows(prefill_then_decode(eng, tokens[:40], 1), ref[:40], dtype, f"{what}: decoded from the first token")
    return eng


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H, dk, dv, rot", [(3, 24, 16, 12), (1, 40, 24, 40), (2, 32, 40, 0), (2, 64, 32, 32), (1, 128, 64, 64),
                                            (4, 16, 16, 8), (2, 64, 100, 64), (5, 6, 2, 2),
                                            (2, 32, 30, 16), (1, 64, 130, 32), (1, 32, 136, 0)])
def test_retention_alone(H, dk, dv, rot, dtype):
    decay = [1.0 - 2.0 ** -(2 + i) for i in range(H)]
    cfg = one_layer("retention", ret(H, dk, dv, decay, rot, 700.0))
    w = make_weights(cfg, dk + dv)
    check_model(cfg, w, dtype, f"retention {H}x{dk}x{dv}", n=300, start=140)      # (prompts longer than a segment)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H, G, dk, dv, size", [(6, 3, 24, 40, 37), (4, 4, 16, 8, 1), (5, 1, 40, 16, 150), (4, 2, 64, 64, 70),
                                                (2, 1, 32, 128, 64), (8, 2, 128, 64, 129), (3, 3, 20, 12, 2), (2, 2, 12, 100, 65)])
def test_window_attention_alone(H, G, dk, dv, size, dtype):
    """The time mixing beside it counts for nothing (its factor is zero), so the logits are the attention's."""
    cfg = one_layer("parallel", par(win(H, G, dk, dv, 0.9 * dk ** -0.5, size), 1, 8, 1.0, 0.0))
    w = make_weights(cfg, dk + dv + size)
    check_model(cfg, w, dtype, f"window attention {H}/{G}x{dk}x{dv} w{size}", n=200, start=60)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H, n, width", [(3, 16, 72), (1, 40, 48), (2, 32, 48), (2, 64, 96), (1, 128, 64), (5, 6, 40)])
def test_time_mixing_alone(H, n, width, dtype):
    """The attention beside it counts for nothing.  The recurrence's inner width is not the model's."""
    cfg = one_layer("parallel", par(win(1, 1, 8, 8, 0.3, 4), H, n, 0.0, 1.0), width=width)
    w = make_weights(cfg, n + width)
    check_model(cfg, w, dtype, f"time mixing {H}x{n}", n=300, start=140)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("mlp", [dense(56), dense(33), moe(40, 6, 3), moe(24, 1, 1), moe(16, 5, 1), moe(64, 12, 4), moe(20, 3, 3)],
                         ids=["dense56", "dense33", "moe6top3", "moe1", "moe5top1", "moe12top4", "moe3top3"])
def test_feed_forwards_alone(mlp, dtype):
    """Behind a mixer whose state forgets at once (a retention with a fast decay and tiny sizes)."""
    cfg = one_layer("retention", ret(1, 8, 8, (0.25,)), mlp, width=64, vocab=80)
    w = make_weights(cfg, 17, mild=(dtype == "bfloat16"))
    check_model(cfg, w, dtype, "feed-forward", n=90, start=30)


@pytest.mark.parametrize("dtype", DTYPES)
def test_experts_on_many_tokens(dtype):
    """Sizes that the tensor-core contractions of the experts take in bfloat16, on prompts of several tiles."""
    cfg = one_layer("retention", ret(1, 8, 8, (0.25,)), moe(64, 8, 2), width=128, vocab=200)
    w = make_weights(cfg, 18, mild=(dtype == "bfloat16"))
    tokens = random_tokens(700, cfg["vocab"], 3)
    assert_rows(run_whole(engine_of(cfg, w, dtype), tokens), plain_of(cfg, w, tokens), dtype, "experts, 700 tokens")


@pytest.mark.parametrize("T", [5, 300])
@pytest.mark.parametrize("d, ff, E, top", [(128, 64, 6, 2), (72, 16, 3, 3), (256, 160, 2, 1)])
def test_gated_experts_on_the_tensor_cores(T, d, ff, E, top):
    """silu(gate) * up formed on the grouped tensor-core contraction's accumulator (an expert's rows in blocks of
    16 gate rows and their 16 up rows) and by the pass of its own over both layouts, against fp32 formulas."""
    from dlgo_b200.csrc import kernels as K
    g = torch.Generator().manual_seed(T + d + ff)
    B = K.MOE_SWIGLU_BLOCK
    h = torch.randn(T, d, generator=g).to(torch.bfloat16)
    gate = (torch.randn(E, ff, d, generator=g) / d ** 0.5).to(torch.bfloat16)
    up = (torch.randn(E, ff, d, generator=g) / d ** 0.5).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    blocks = torch.stack([gate.view(E, ff // B, B, d), up.view(E, ff // B, B, d)], dim=2).reshape(E, 2 * ff, d)
    ref = torch.zeros(T * top, ff)
    for t in range(T):
        for j in range(top):
            e = int(idx[t, j])
            a, b = gate[e].float() @ h[t].float(), up[e].float() @ h[t].float()
            ref[t * top + j] = a * torch.sigmoid(a) * b
    plan = K.moe_plan(idx.to(DEV), E, K.MOE_TC_ROWS)
    rows = K.moe_gather_rows(plan, h.to(DEV), top)
    total = int(plan.offsets[-1])
    assert total == T * top
    pair = plan.sorted_pair[:total].long().cpu()
    hid = torch.full((T * top, ff), float("nan"), dtype=torch.bfloat16, device=DEV)
    K.moe_gemm_tc(plan, rows, blocks.to(DEV), hid, False, K.MOE_ACT_SWIGLU)
    both = torch.full((T * top, 2 * ff), float("nan"), dtype=torch.bfloat16, device=DEV)
    K.moe_gemm_tc(plan, rows, blocks.to(DEV), both, False, K.ACT_NONE)
    halves = torch.full((T * top, 2 * ff), float("nan"), dtype=torch.bfloat16, device=DEV)
    K.moe_gemm_tc(plan, rows, torch.cat([gate, up], dim=1).to(DEV), halves, False, K.ACT_NONE)
    K.check_device_errors()
    tol = 2e-2 * float(ref.abs().max())
    for what, got in (("fused", hid), ("pass over blocks", K.swiglu(both, block=B)), ("pass over halves", K.swiglu(halves))):
        out = torch.zeros(T * top, ff)
        out[pair] = got[:total].float().cpu()
        assert torch.isfinite(out).all(), what
        assert torch.allclose(out, ref, rtol=2e-2, atol=tol), (what, float((out - ref).abs().max()))


# ---------------------------------------------- a key that carries the answer: far away, and at the window's edge
def standing_out(cfg, w):
    """(query token b, key token a, filler f) for a one-layer model whose first mixer is the window attention: a's
    score with b stands far above f's with b and b's own, summed over heads."""
    wd = {k: v.double() for k, v in w.items()}
    m, eps = cfg["layers"][0]["mixer"]["left"], cfg["norm"]["eps"]
    x = P.layer_norm(wd["embed"], wd["embed.norm"], eps)
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = (P.unit_rms(x @ wd["l0.mix.left.q"].T, eps) * wd["l0.mix.left.q.norm"]).view(-1, H, d)
    k = (P.unit_rms(x @ wd["l0.mix.left.k"].T, eps) * wd["l0.mix.left.k.norm"]).view(-1, G, d)
    k = k.repeat_interleave(H // G, dim=1)
    s = torch.einsum("bhd,ahd->ba", q, k) * m["scale"]
    s.fill_diagonal_(-1e9)
    b, a = divmod(int(s.argmax()), s.shape[1])
    s[b, a] = 1e9
    s[b, b] = 1e9
    return b, a, int(s[b].argmin())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H, G, dk, dv, size", [(2, 1, 24, 16, 100), (4, 2, 64, 64, 131), (2, 2, 32, 64, 64), (2, 1, 64, 128, 200)])
def test_a_key_just_inside_and_just_outside_the_window(H, G, dk, dv, size, dtype):
    """One key carries the answer.  The query sees it at distance size - 1 and no longer at distance size, in a prompt
    and decoded, wherever the pair lies among the pages."""
    cfg = one_layer("parallel", par(win(H, G, dk, dv, 1.0, size), 1, 8, 1.0, 0.0))
    w = make_weights(cfg, 5 + size, sharpen=12.0)
    b, a, f = standing_out(cfg, w)
    eng = engine_of(cfg, w, dtype)
    for n in (size + 3, 390):
        without = plain_of(cfg, w, [f] * n + [b])
        for dist in (1, size - 2, size - 1, size, size + 1):
            tokens = [f] * n + [b]
            tokens[n - dist] = a
            ref = plain_of(cfg, w, tokens)
            seen = float(row_error(without[-1:], ref[-1:])) > 0.2
            assert seen == (dist < size), (n, dist)                          # the oracle's window is the design's
            s = eng.take_slot()
            assert_rows(eng.step([s], [tokens], [[n]]), ref[-1:], dtype, f"key at distance {dist} of {n} (prompt)")
            eng.free_slot(s)
            for cut in (n, n - dist + 1 if dist > 1 else n, max(1, n - size - 1)):
                s = eng.take_slot()
                eng.step([s], [tokens[:cut]], [[]])
                for p in range(cut, n):
                    eng.step([s], [tokens[p:p + 1]], [[]])
                assert_rows(eng.step([s], [tokens[-1:]]), ref[-1:], dtype, f"key at distance {dist} of {n} (decoded from {cut})")
                eng.free_slot(s)
    eng.cache.book.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_far_token_in_the_retention_s_state(dtype):
    """One token hundreds of positions back still shows through a slow decay, in a prompt, decoded, and in a prompt cut
    into portions; with a fast decay beside it (another head) that forgets."""
    cfg = one_layer("retention", ret(2, 32, 24, (0.999, 0.5), 16, 200.0))
    w = make_weights(cfg, 8)
    n = 500
    base = random_tokens(n, cfg["vocab"], 3)
    other = list(base)
    other[7] = (base[7] + 1) % cfg["vocab"]
    ref, ref_other = plain_of(cfg, w, base), plain_of(cfg, w, other)
    # one token among hundreds: it moves the last row by half a percent, fifty times the float32 tolerance
    assert float(row_error(ref_other[-1:], ref[-1:])) > 3e-3
    eng = engine_of(cfg, w, dtype)
    for tokens, r in ((base, ref), (other, ref_other)):
        assert_rows(run_whole(eng, tokens)[-3:], r[-3:], dtype, "far token (prompt)")
        assert_rows(prefill_then_decode(eng, tokens, 450)[-3:], r[-3:], dtype, "far token (decoded)")
        s = eng.take_slot()
        for at in range(0, n - 2, 83):
            eng.step([s], [tokens[at:min(at + 83, n - 2)]], [[]])
        got = eng.step([s], [tokens[n - 2:]], [[0, 1]])
        eng.free_slot(s)
        assert_rows(got, r[-2:], dtype, "far token (portions)")
    if dtype == "float32":
        assert float(row_error(run_whole(eng, other)[-1:].float().cpu(), ref[-1:])) > 3e-3


# ------------------------------------------------------------------------------- whole models
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompts(dirs, name, dtype):
    eng = engine_for(dirs[name, dtype], dtype)
    V = CONFIGS[name]["vocab"]
    rows = RowCheck(dtype, f"{name}: whole prompts")
    for n in (1, 2, 3, 63, 64, 65, 127, 128, 129, 211, 300):
        tokens = random_tokens(n, V, 100 + n)
        rows.add(run_whole(eng, tokens), plain_logits(dirs[name, dtype], tokens), f"{name}: prompt of {n}")
    rows.done()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_prefill_then_token_by_token(dirs, name, graphs, dtype):
    """A short prompt, then more than two pages of decoding, past every window (with and without captured steps)."""
    eng = engine_for(dirs[name, dtype], dtype, cuda_graphs=graphs)
    V = CONFIGS[name]["vocab"]
    tokens = random_tokens(190, V, 7)
    ref = plain_logits(dirs[name, dtype], tokens)
    for start in (1, 5):
        assert_rows(prefill_then_decode(eng, tokens, start), ref, dtype, f"{name}: decoding from {start}")
    eng.cache.book.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_portions(dirs, name, dtype):
    eng = engine_for(dirs[name, dtype], dtype)
    V = CONFIGS[name]["vocab"]
    tokens = random_tokens(300, V, 8)
    ref = plain_logits(dirs[name, dtype], tokens)
    for cuts in ([2] * 150, [3, 61, 1, 63, 2, 170], [64, 64, 64, 108], [7, 293], [299, 1], [129, 2, 128, 41], [1, 1, 298]):
        s = eng.take_slot()
        got, at = [], 0
        for c in cuts:
            got.append(eng.step([s], [tokens[at:at + c]], [list(range(c))]).clone())
            at += c
        eng.free_slot(s)
        assert_rows(torch.cat(got), ref, dtype, f"{name}: portions {cuts[:3]}...")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_unequal_batch_against_each_alone(dirs, name, dtype):
    eng = engine_for(dirs[name, dtype], dtype)
    V = CONFIGS[name]["vocab"]
    lens = [1, 140, 2, 266, 31]
    seqs = [random_tokens(n + 40, V, 50 + n) for n in lens]
    refs = [plain_logits(dirs[name, dtype], t) for t in seqs]
    slots = [eng.take_slot() for _ in seqs]
    got = eng.step(slots, [t[:n] for t, n in zip(seqs, lens)], [list(range(n)) for n in lens])
    off = 0
    rows = RowCheck(dtype, f"{name}: a mixed batch")
    for i, n in enumerate(lens):
        rows.add(got[off:off + n], refs[i][:n], f"{name}: sequence {i} of a mixed prompt batch")
        off += n
    rows.done()
    rows = RowCheck(dtype, f"{name}: decoded together")
    live = list(range(len(seqs)))
    for step in range(40):
        if step in (9, 17, 30):
            eng.free_slot(slots[live.pop(0)])
        out = eng.step([slots[i] for i in live], [[seqs[i][lens[i] + step]] for i in live])
        for j, i in enumerate(live):
            rows.add(out[j:j + 1], refs[i][lens[i] + step:lens[i] + step + 1],
                     f"{name}: sequence {i}, decoded step {step} in a batch of {len(live)}")
    rows.done()
    for i in live:
        eng.free_slot(slots[i])
    eng.cache.book.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_pages_slots_and_states_used_again(dirs, dtype):
    """A small cache whose pages go round several times, poisoned where nothing was written; a slot's state must be
    zero again when the slot is taken anew."""
    name = "P"
    eng = engine_for(dirs[name, dtype], dtype, max_tokens=512, max_slots=3)
    eng.cache.poison()
    V = CONFIGS[name]["vocab"]
    rows = RowCheck(dtype, "pages and slots used again")
    for r in range(5):
        lens = [150 + 7 * r, 90 - r, 60 + r]
        seqs = [random_tokens(n, V, 300 + 10 * r + i) for i, n in enumerate(lens)]
        slots = [eng.take_slot() for _ in seqs]
        got = eng.step(slots, seqs, [[n - 4, n - 3, n - 2, n - 1] for n in lens])
        assert torch.isfinite(got).all()                          # nothing unwritten reached a result
        for i, n in enumerate(lens):
            rows.add(got[4 * i:4 * i + 4], plain_logits(dirs[name, dtype], seqs[i])[n - 4:], f"round {r}, sequence {i}")
        for s in (slots[1], slots[0], slots[2]):
            eng.free_slot(s)
    rows.done()
    eng.cache.book.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(dirs, dtype):
    name = "Q"
    eng = engine_for(dirs[name, dtype], dtype)
    V = CONFIGS[name]["vocab"]
    tokens = random_tokens(420, V, 9)
    ref = plain_logits(dirs[name, dtype], tokens)
    s = eng.take_slot()
    eng.step([s], [tokens[:20]], [[]])
    rows = RowCheck(dtype, "long decoding")
    for p in range(20, len(tokens)):
        out = eng.step([s], [tokens[p:p + 1]])
        if p % 17 == 0 or p >= len(tokens) - 8:
            rows.add(out.clone(), ref[p:p + 1], f"decoded position {p}")
    rows.done()
    eng.free_slot(s)


def test_greedy_generation_through_the_entry_point(dirs):
    import dlgo_b200
    for name in ("P", "R"):
        dtype = "float32"
        llm = dlgo_b200.load_llm(dirs[name, dtype], dtype=dtype, max_tokens=2048)
        cfg, w = P.read_model(dirs[name, dtype], torch.float64)
        prompts = [random_tokens(n, cfg["vocab"], 70 + n) for n in (1, 9, 70)]
        got = llm.generate(prompts, max_tokens=12, greedy=True, ignore_eos=True)
        for p, g in zip(prompts, got):
            want = P.greedy_generate(cfg, w, p, 12)
            if g != want:                      # only a near tie may differ
                k = next(i for i in range(12) if g[i] != want[i])
                lg = P.forward(cfg, w, p + want[:k])[-1]
                assert float(lg[want[k]] - lg[g[k]]) < 1e-4 * float(lg.abs().max()), (name, g, want)
        info = llm.model_info()
        assert info.architecture == "Bazurax" and info.layers == len(cfg["layers"]) and info.vocab_size == cfg["vocab"]
        out = llm.generate(prompts[:2], max_tokens=5, temperature=0.8, top_k=20, seed=3, ignore_eos=True)
        assert all(len(o) == 5 and all(0 <= t < cfg["vocab"] for t in o) for o in out)


def test_trace_replay_command(dirs, tmp_path):
    """bin/trace_run on a Bazurax folder: a mixed batch, then decoding, against the plain implementation."""
    import subprocess
    import sys
    import numpy as np
    name, dtype = "P", "float32"
    V = CONFIGS[name]["vocab"]
    a, b = random_tokens(30, V, 1), random_tokens(75, V, 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:28], "want": [0, 27]}, {"id": "b", "tokens": b[:70], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[28:29], "want": [0]}, {"id": "b", "tokens": b[70:71], "want": [0]}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[29:30], "want": []}, {"id": "b", "tokens": b[71:72], "want": [0]}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "b", "tokens": b[72:73], "want": [0]}], "end": ["b"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", dirs[name, dtype], "--dtype", "float32",
                        "--out", str(out), "--max-tokens", "256"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
    ra, rb = plain_logits(dirs[name, dtype], a), plain_logits(dirs[name, dtype], b)
    want = {0: torch.stack([ra[0], ra[27]]), 1: torch.stack([ra[28], rb[70]]), 2: rb[71:72], 3: rb[72:73]}
    for i, ref in want.items():
        got = torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, V))
        assert_rows(got, ref, "float32", f"step {i}")
