"""Ragilorn on the GPU against the plain implementation (tests/plain_ragilorn.py): every mechanism alone (its
kernels, and one-layer models that hold nothing else), then whole models through the engine's step function, its
cache and state, and the public entry point."""
import copy
import json
import math
import os

import pytest
import torch

import plain_ragilorn as P
from ragilorn_configs import (CONFIGS, SEEDS, RowCheck, assert_rows, att, config_of, dense, lat, layer, make_weights, model,
                              moe, plain_logits, random_tokens, row_error, write_model, yarn)

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
DEV = "cuda:0"


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    root = tmp_path_factory.mktemp("ragilorn")
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
    return Engine(spec=config_of(cfg).architecture_spec(), tensors=w, dtype=dtype, **kw)


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


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


# ------------------------------------------------------------------ mechanisms alone: the kernels
@pytest.mark.parametrize("act_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, G, dk, dv, rot, taps", [(3, 1, 24, 40, 12, 3), (2, 2, 16, 8, 16, 1), (1, 1, 7, 5, 4, 2),
                                                     (4, 2, 64, 64, 32, 4), (2, 1, 128, 64, 0, 8)])
def test_bias_convolution_rotation_and_append(H, G, dk, dv, rot, taps, act_dtype):
    """Two sequences over three steps (a prompt portion each, a portion of fewer tokens than the taps reach, one
    token each): the convolution reads across the steps through the state; keys and values land in their pages."""
    from dlgo_b200.csrc import kernels as K
    g = torch.Generator().manual_seed(H * dk + taps)
    C = (H + G) * dk + G * dv
    hd = -(-max(dk, dv) // 8) * 8
    lens = [[5, 2, 1], [70, 1, 1]]
    total = [sum(l) for l in lens]
    u = [torch.randn(n, C, generator=g) for n in total]
    bias = 0.5 * torch.randn(C, generator=g)
    w_taps = torch.randn(C, taps, generator=g) if taps > 1 else None
    rotd = {"base": 300.0, "dims": rot, "scaling": yarn(2.0, 16, 4.0, 1.0)}
    freq, amp = (P.yarn_frequencies(rotd) if rot else ([], 1.0))
    ref = []
    for s in range(2):
        y = (u[s] + bias).double()
        if taps > 1:
            y = P.short_conv(y, w_taps.double())
        q, k, v = y[:, :H * dk].view(-1, H, dk), y[:, H * dk:(H + G) * dk].view(-1, G, dk), y[:, (H + G) * dk:].view(-1, G, dv)
        if rot:
            q, k = P.rotate_pairs(q, rotd), P.rotate_pairs(k, rotd)
        ref.append((q, k, v))
    PS, n_pages = 64, 6
    kp = torch.full((n_pages, G, PS, hd), float("nan"), dtype=act_dtype, device=DEV)
    vp = torch.full_like(kp, float("nan"))
    table = i32([[4, 1, -1], [2, 5, 0]])
    state = torch.zeros(3, (taps - 1) * C, device=DEV) if taps > 1 else None
    slots = [2, 0]           # rows of the state; rows of the page table are the slots too
    table_by_slot = torch.full((3, 3), -1, dtype=torch.int32, device=DEV)
    table_by_slot[2], table_by_slot[0] = table[0], table[1]
    done = [0, 0]
    tol = dict(rtol=2e-2, atol=2e-2) if act_dtype == torch.bfloat16 else dict(rtol=1e-5, atol=1e-5)
    for step in range(3):
        rows, pos, seq, tiles = [], [], [], []
        for s in range(2):
            n = lens[s][step]
            tiles.append([s, len(pos), n])
            rows.append(u[s][done[s]:done[s] + n])
            pos += list(range(done[s], done[s] + n))
            seq += [s] * n
        proj = torch.cat(rows).to(DEV)
        q = K.conv_rope_append(proj, bias.to(DEV), None if w_taps is None else w_taps.to(DEV), state,
                               torch.tensor(freq, dtype=torch.float32, device=DEV) if rot else None, rot, amp, i32(pos),
                               i32(seq), i32(slots), table_by_slot, kp, vp, H, G, dk, dv, i32(tiles), 2)
        q = q.float().cpu().view(-1, H, hd)
        at = 0
        for s in range(2):
            n = lens[s][step]
            assert torch.allclose(q[at:at + n, :, :dk].double(), ref[s][0][done[s]:done[s] + n], **tol), (step, s)
            assert (q[at:at + n, :, dk:] == 0).all()
            at += n
            done[s] += n
    for s in range(2):
        for p in range(total[s]):
            page = int(table[s][p // PS])
            krow, vrow = kp[page, :, p % PS].float().cpu(), vp[page, :, p % PS].float().cpu()
            assert torch.allclose(krow[:, :dk].double(), ref[s][1][p], **tol), (s, p)
            assert torch.allclose(vrow[:, :dv].double(), ref[s][2][p], **tol), (s, p)
            assert (krow[:, dk:] == 0).all() and (vrow[:, dv:] == 0).all()
    if taps > 1:      # the state is the last taps - 1 projected rows with their bias, oldest first
        for s in range(2):
            want = (u[s] + bias)[-(taps - 1):].reshape(-1)
            assert torch.allclose(state[slots[s]].cpu(), want, atol=1e-6)


@pytest.mark.parametrize("act_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, dk, r, R", [(3, 24, 8, 40), (1, 8, 4, 9), (4, 32, 32, 96), (2, 64, 64, 128)])
def test_latents_with_a_rotated_key_part(H, dk, r, R, act_dtype):
    from dlgo_b200.csrc import kernels as K
    g = torch.Generator().manual_seed(H + R)
    T, eps = 9, 1e-5
    n_q = H * (dk + r)
    proj = torch.randn(T, n_q + R + r + 3, generator=g)
    w = 1 + 0.2 * torch.randn(R, generator=g)
    rotd = {"base": 1000.0, "dims": r, "scaling": yarn(3.0, 8, 2.0, 0.5)}
    freq, amp = P.yarn_frequencies(rotd)
    pos = [100, 101, 102, 103, 0, 1, 2, 63, 64]
    PS = 64
    pages = torch.full((4, 1, PS, R + r), float("nan"), dtype=act_dtype, device=DEV)
    table = i32([[3, 1], [0, 2]])
    seq = [0, 0, 0, 0, 1, 1, 1, 1, 1]
    dev = proj.to(DEV)
    K.latent_rope_append(dev, n_q, R, w.to(DEV), 0, H, dk + r, r, torch.tensor(freq, dtype=torch.float32, device=DEV), amp,
                         eps, i32(pos), i32(seq), i32([0, 1]), table, pages.view(4, PS, R + r))
    tol = dict(rtol=2e-2, atol=2e-2) if act_dtype == torch.bfloat16 else dict(rtol=1e-5, atol=1e-5)
    got_q = dev[:, :n_q].cpu().view(T, H, dk + r)
    for t in range(T):
        q = proj[t, :n_q].view(1, H, dk + r).double()
        want = torch.cat([q[..., :dk], P.rotate_pairs(q[..., dk:].contiguous(), rotd, first=pos[t])], -1)
        assert torch.allclose(got_q[t].double(), want[0], rtol=1e-5, atol=1e-5)          # queries stay fp32, in place
        c = P.rms_norm(proj[t, n_q:n_q + R].double(), w.double(), eps)
        kr = P.rotate_pairs(proj[t, n_q + R:n_q + R + r].view(1, 1, r).double(), rotd, first=pos[t])[0, 0]
        row = pages[int(table[seq[t]][pos[t] // PS]), 0, pos[t] % PS].float().cpu().double()
        assert torch.allclose(row, torch.cat([c, kr]), **tol), t
    assert torch.equal(dev[:, n_q:].cpu(), proj[:, n_q:])                                   # nothing else is rewritten


@pytest.mark.parametrize("act_dtype", [torch.float32, torch.bfloat16])
def test_gate_depth_average_and_norm(act_dtype):
    from dlgo_b200.csrc import kernels as K
    g = torch.Generator().manual_seed(5)
    loose = dict(rtol=1e-2, atol=1e-2) if act_dtype == torch.bfloat16 else dict(rtol=1e-5, atol=1e-5)
    for T, d in ((3, 40), (70, 72), (5, 1000), (2, 4096)):
        x, y = torch.randn(T, d, generator=g), torch.randn(T, d, generator=g)
        gl, gb = 2 * torch.randn(T, d + 8, generator=g), torch.randn(d, generator=g)
        w, eps = 1 + 0.2 * torch.randn(d, generator=g), 1e-5
        hist = torch.randn(4, T, d, generator=g)
        avg = torch.randn(3, generator=g)
        want_x = x.double() + torch.sigmoid(gl[:, :d].double() + gb.double()) * y.double()
        # gate, add, clear, norm of the sum
        xd, yd = x.to(DEV), y.to(DEV)
        out = K.gated_residual(xd, yd, gl.to(DEV)[:, :d], gb.to(DEV), norm_w=w.to(DEV), eps=eps, out_dtype=act_dtype)
        assert torch.allclose(xd.cpu().double(), want_x, rtol=1e-6, atol=1e-6) and not yd.any()
        assert torch.allclose(out.float().cpu().double(), P.rms_norm(want_x, w.double(), eps), **loose)
        # a bias that the sublayer left to this pass joins its result before the gate
        yb = torch.randn(d, generator=g)
        xd, yd = x.to(DEV), y.to(DEV)
        K.gated_residual(xd, yd, gl.to(DEV)[:, :d], gb.to(DEV), y_bias=yb.to(DEV))
        biased = x.double() + torch.sigmoid(gl[:, :d].double() + gb.double()) * (y.double() + yb.double())
        assert torch.allclose(xd.cpu().double(), biased, rtol=1e-6, atol=1e-6) and not yd.any()
        # gate, add, then the average over three entries of which the sum is the last
        xd, yd, hd = x.to(DEV), y.to(DEV), hist.to(DEV)
        assert K.gated_residual(xd, yd, gl.to(DEV)[:, :d], gb.to(DEV), history=hd, depth=3, average=avg.to(DEV)) is None
        mixed = avg[0].double() * hist[0].double() + avg[1].double() * hist[1].double() + avg[2].double() * want_x
        assert torch.allclose(xd.cpu().double(), mixed, rtol=1e-5, atol=1e-5)
        assert torch.allclose(hd[2].cpu().double(), want_x, rtol=1e-6, atol=1e-6)
        assert torch.equal(hd[:2].cpu(), hist[:2]) and torch.equal(hd[3].cpu(), hist[3])
        # no gate: a plain sum; nothing to add: the stream is stored as the first entry
        xd, yd = x.to(DEV), y.to(DEV)
        K.gated_residual(xd, yd, None, None)
        assert torch.allclose(xd.cpu(), x + y)
        K.gated_residual(xd, None, None, None, history=hd, depth=1, average=torch.ones(1, device=DEV))
        assert torch.equal(hd[0], xd) and torch.allclose(xd.cpu(), x + y)


def test_scaled_embedding_and_capped_logits():
    from dlgo_b200.csrc import kernels as K
    g = torch.Generator().manual_seed(2)
    table = torch.randn(50, 72, generator=g).to(torch.bfloat16)
    ids = [3, 49, 0, 3]
    for scale in (1.0, 0.37):
        out = K.embed(i32(ids), table.to(DEV), scale=scale).cpu()
        assert torch.equal(out, table[ids].float() * torch.tensor(scale, dtype=torch.float32))
    z = 6 * torch.randn(7, 33, generator=g)
    for scale, cap in ((0.25, 15.0), (2.0, 1.5), (0.5, 0.0)):
        got = K.scale_softcap(z.to(DEV), scale, cap).cpu().double()
        want = z.double() * scale
        want = cap * torch.tanh(want / cap) if cap else want
        assert torch.allclose(got, want, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("act_dtype", [torch.float32, torch.bfloat16])
def test_rows_multiplied_by_their_experts_weights(act_dtype):
    from dlgo_b200.csrc import kernels as K
    g = torch.Generator().manual_seed(4)
    h = torch.randn(11, 40, generator=g).to(act_dtype)
    wt = torch.rand(11, 3, generator=g)
    rows = K.moe_scale_rows(h.to(DEV), wt.to(DEV))
    want = (wt[:, :, None] * h.float()[:, None, :]).reshape(33, 40).to(act_dtype)
    assert torch.equal(rows.cpu(), want)
    if act_dtype == torch.bfloat16:
        # the same product on the way into sorted order (the tensor-core experts' copy)
        idx = torch.randint(0, 4, (11, 3), generator=g, dtype=torch.int32)
        plan = K.moe_plan(idx.to(DEV), 4, K.MOE_TC_ROWS)
        got = K.moe_gather_rows(plan, h.to(DEV), 3, scale=wt.to(DEV)).cpu()
        assert torch.equal(got, want[plan.sorted_pair.cpu().long()])
    # weights of one in the combine
    y = torch.zeros(11, 40, device=DEV)
    pair_out = torch.randn(33, 40, generator=g).to(act_dtype)
    K.moe_combine(y, pair_out.to(DEV), h.to(DEV), torch.zeros(11, 3, dtype=torch.int32, device=DEV), None, 1)
    assert torch.allclose(y.cpu(), pair_out.float().view(11, 3, 40).sum(1), atol=1e-5)


# --------------------------------------------------- mechanisms alone: one-layer models that hold nothing else
def one_layer(mixer, mlp=None, width=48, vocab=60, **kw):
    return model(vocab, width, [layer(copy.deepcopy(mixer), mlp)], eps=1e-6, **kw)


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
@pytest.mark.parametrize("H, G, dk, dv, rot, conv, chunk", [
    (6, 3, 24, 40, 12, 3, 37), (4, 4, 16, 8, 16, None, None), (5, 1, 40, 16, 8, 2, 150), (4, 2, 64, 64, 32, 4, 70),
    (2, 1, 32, 128, 32, 4, 64), (8, 2, 128, 64, 64, 4, 129), (3, 3, 20, 12, 0, 5, 2), (2, 2, 12, 100, 4, 8, 65),
    (5, 1, 128, 48, 96, 3, 88), (2, 1, 64, 64, 64, None, 1)])
def test_attention_alone(H, G, dk, dv, rot, conv, chunk, dtype):
    cfg = one_layer(att(H, G, dk, dv, 0.9 * dk ** -0.5, rot, 20000.0, yarn(2.0, 64) if rot else None, conv, chunk))
    w = make_weights(cfg, dk + dv + (chunk or 0))
    check_model(cfg, w, dtype, f"attention {H}/{G}x{dk}x{dv} rot {rot} conv {conv} chunk {chunk}", n=200, start=60)


@pytest.mark.parametrize("dtype", DTYPES)
def test_sizes_off_every_grid(dtype):
    """A width, a vocabulary and head sizes that are no multiple of 8 (contractions on the fp32 pipes also in bfloat16,
    the plain forms of the row kernels), a convolution of one tap, experts of an odd width."""
    cfg = model(61, 100, [layer(att(5, 5, 12, 18, 0.3, 6, 900.0, yarn(2.0, 20), conv=1, chunk=50), moe(30, 3, 2)),
                          layer(lat(3, 10, 6, 14, 22, 0.3, 500.0), dense(52)),
                          layer(att(2, 1, 7, 5, 0.4, 4, 70.0, None, conv=3), None)], eps=1e-6, emb=1.3, logit_scale=1.5, softcap=3.0)
    w = make_weights(cfg, 23, mild=(dtype == "bfloat16"))
    assert w["l0.mix.q.conv"].shape == (60, 1)
    check_model(cfg, w, dtype, "sizes off every grid", n=130, start=55)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H, dk, r, dv, R", [(3, 24, 8, 20, 40), (1, 8, 4, 40, 9), (4, 32, 32, 64, 96), (2, 64, 64, 128, 128),
                                             (6, 64, 16, 72, 112), (2, 16, 16, 24, 18), (2, 96, 32, 128, 160)])
def test_latent_attention_alone(H, dk, r, dv, R, dtype):
    cfg = one_layer(lat(H, dk, r, dv, R, 0.9 * (dk + r) ** -0.5, 3000.0, yarn(4.0, 32)))
    w = make_weights(cfg, dk + dv + R)
    check_model(cfg, w, dtype, f"latent attention {H}x({dk}+{r})x{dv} rank {R}", n=200, start=60)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("mlp", [dense(56), dense(33), moe(40, 6, 3), moe(24, 1, 1), moe(16, 5, 1), moe(64, 12, 4), moe(20, 3, 3), None],
                         ids=["dense56", "dense33", "moe6top3", "moe1", "moe5top1", "moe12top4", "moe3top3", "none"])
def test_feed_forwards_alone(mlp, dtype):
    """Behind a mixer that sees one key (a chunk of one)."""
    cfg = one_layer(att(1, 1, 8, 8, 0.3, 0, chunk=1), mlp, width=64, vocab=80, emb=0.6, logit_scale=2.0, softcap=3.0)
    w = make_weights(cfg, 17, mild=(dtype == "bfloat16"))
    check_model(cfg, w, dtype, "feed-forward", n=90, start=30)


@pytest.mark.parametrize("dtype", DTYPES)
def test_experts_on_many_tokens(dtype):
    """Sizes that the tensor-core contractions of the experts take in bfloat16, on prompts of several tiles."""
    cfg = one_layer(att(1, 1, 8, 8, 0.3, 0, chunk=1), moe(64, 8, 2), width=128, vocab=200)
    w = make_weights(cfg, 18, mild=(dtype == "bfloat16"))
    tokens = random_tokens(700, cfg["vocab"], 3)
    assert_rows(run_whole(engine_of(cfg, w, dtype), tokens), plain_of(cfg, w, tokens), dtype, "experts, 700 tokens")


# ---------------------------------------------- a key that carries the answer: far away, and at a chunk's edge
def standing_out(cfg, w):
    """(query token b, key token a, filler f) for a one-layer attention model without convolution or rotation: a's
    score with b stands far above f's with b and b's own, summed over heads."""
    wd = {k: v.double() for k, v in w.items()}
    m, eps = cfg["layers"][0]["mixer"], cfg["norm"]["eps"]
    x = P.rms_norm(wd["embed"] * cfg["embedding"]["scale"], wd["l0.norm1"], eps)
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = (x @ wd["l0.mix.q"].T + wd["l0.mix.q.b"]).view(-1, H, d)
    k = (x @ wd["l0.mix.k"].T + wd["l0.mix.k.b"]).view(-1, G, d).repeat_interleave(H // G, dim=1)
    s = torch.einsum("bhd,ahd->ba", q, k) * m["scale"]
    s.fill_diagonal_(-1e9)
    b, a = divmod(int(s.argmax()), s.shape[1])
    s[b, a] = 1e9
    s[b, b] = 1e9
    return b, a, int(s[b].argmin())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H, G, dk, dv, size", [(2, 1, 24, 16, 100), (4, 2, 64, 64, 131), (2, 2, 32, 64, 64), (2, 1, 128, 64, 88)])
def test_a_key_just_inside_and_just_outside_the_chunk(H, G, dk, dv, size, dtype):
    """One key carries the answer.  The query sees it as the first position of its own chunk and no longer as the
    last of the chunk before, in a prompt and decoded, wherever the edge lies among the pages; chunks count from
    position 0 of the sequence, not from where the prompt was cut."""
    cfg = one_layer(att(H, G, dk, dv, 1.0, 0, chunk=size))
    w = make_weights(cfg, 5 + size, sharpen=12.0)
    b, a, f = standing_out(cfg, w)
    eng = engine_of(cfg, w, dtype)
    for n_chunks, inside in ((1, 0), (1, size - 1), (3, 1), (3, size - 1), (2, size // 2)):
        # the query sits `inside` positions into chunk number n_chunks; the key at the chunk's first position, at the
        # last of the chunk before, and far back in the sequence's first chunk
        qpos = n_chunks * size + inside
        edge = n_chunks * size
        without = plain_of(cfg, w, [f] * qpos + [b])
        for kpos in (edge, edge - 1, edge + inside // 2, 1):
            if kpos >= qpos:
                continue
            tokens = [f] * qpos + [b]
            tokens[kpos] = a
            ref = plain_of(cfg, w, tokens)
            seen = float(row_error(without[-1:], ref[-1:])) > 0.2
            assert seen == (kpos >= edge), (qpos, kpos)                          # the oracle's chunks are the design's
            s = eng.take_slot()
            assert_rows(eng.step([s], [tokens], [[qpos]]), ref[-1:], dtype, f"key at {kpos}, query at {qpos} (prompt)")
            eng.free_slot(s)
            for cut in (qpos, max(1, edge - 3)):
                s = eng.take_slot()
                eng.step([s], [tokens[:cut]], [[]])
                for p in range(cut, qpos):
                    eng.step([s], [tokens[p:p + 1]], [[]])
                assert_rows(eng.step([s], [tokens[-1:]]), ref[-1:], dtype, f"key at {kpos}, query at {qpos} (decoded from {cut})")
                eng.free_slot(s)
            for first in (edge + 1 if edge + 1 < qpos else edge - 2, edge - 1):      # a portion that starts inside a chunk
                s = eng.take_slot()
                eng.step([s], [tokens[:first]], [[]])
                got = eng.step([s], [tokens[first:]], [[qpos - first]])
                assert_rows(got, ref[-1:], dtype, f"key at {kpos}, query at {qpos} (portion from {first})")
                eng.free_slot(s)
    eng.cache.book.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_far_key_among_hundreds_in_latent_attention(dtype):
    """Causal latent attention sees every earlier position: one key far back carries the answer, in a prompt, in
    portions and decoded."""
    cfg = one_layer(lat(2, 32, 16, 24, 48, 1.0, 10000.0, yarn(2.0, 64)))
    w = make_weights(cfg, 77, sharpen=10.0)
    eng = engine_of(cfg, w, dtype)
    wd = {k: v.double() for k, v in w.items()}
    V = cfg["vocab"]
    # the pair of tokens whose score (at equal positions far apart the rotated part matters little: rank by the whole) is largest
    best, pair = -1.0, None
    for b in range(0, V, 7):
        for a in range(1, V, 5):
            if a == b:
                continue
            base = plain_of(cfg, w, [3] * 400 + [b])[-1:]
            moved = float(row_error(plain_of(cfg, w, [3] * 10 + [a] + [3] * 389 + [b])[-1:], base))
            if moved > best:
                best, pair = moved, (a, b)
        if best > 0.3:
            break
    assert best > 0.2, best
    a, b = pair
    for kpos in (0, 10, 63, 64, 200, 398):
        tokens = [3] * 400 + [b]
        tokens[kpos] = a
        ref = plain_of(cfg, w, tokens)
        s = eng.take_slot()
        assert_rows(eng.step([s], [tokens], [[400]]), ref[-1:], dtype, f"far key at {kpos} (prompt)")
        eng.free_slot(s)
        s = eng.take_slot()
        eng.step([s], [tokens[:130]], [[]])
        eng.step([s], [tokens[130:399]], [[]])
        eng.step([s], [tokens[399:400]], [[]])
        assert_rows(eng.step([s], [tokens[400:]]), ref[-1:], dtype, f"far key at {kpos} (portions, then decoded)")
        eng.free_slot(s)


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
    """A short prompt, then more than two pages of decoding, past every chunk's edge (with and without captured steps)."""
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
    """A small cache whose pages go round several times, poisoned where nothing was written; a slot's convolution
    state must be zero again when the slot is taken anew."""
    name = "P"
    eng = engine_for(dirs[name, dtype], dtype, max_tokens=512, max_slots=3)
    eng.cache.poison()
    V = CONFIGS[name]["vocab"]
    rows = RowCheck(dtype, "pages and slots used again")
    for r in range(5):
        lens = [150 + 7 * r, 90 - r, 60 + r]
        seqs = [random_tokens(n, V, 300 + 10 * r + i) for i, n in enumerate(lens)]
        slots = [eng.take_slot() for _ in seqs]
        got = eng.step(slots, seqs, [[0, 1, n - 2, n - 1] for n in lens])
        assert torch.isfinite(got).all()                          # nothing unwritten reached a result
        for i, n in enumerate(lens):
            ref = plain_logits(dirs[name, dtype], seqs[i])
            rows.add(got[4 * i:4 * i + 4], ref[[0, 1, n - 2, n - 1]], f"round {r}, sequence {i}")
        for s in (slots[1], slots[0], slots[2]):
            eng.free_slot(s)
    rows.done()
    eng.cache.book.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(dirs, dtype):
    name = "Q"
    eng = engine_for(dirs[name, dtype], dtype)
    V = CONFIGS[name]["vocab"]
    tokens = random_tokens(620, V, 9)          # past the chunk of 500
    ref = plain_logits(dirs[name, dtype], tokens)
    s = eng.take_slot()
    eng.step([s], [tokens[:20]], [[]])
    rows = RowCheck(dtype, "long decoding")
    for p in range(20, len(tokens)):
        out = eng.step([s], [tokens[p:p + 1]])
        if p % 17 == 0 or p in (498, 499, 500, 501) or p >= len(tokens) - 8:
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
        assert info.architecture == "Ragilorn" and info.layers == len(cfg["layers"]) and info.vocab_size == cfg["vocab"]
        out = llm.generate(prompts[:2], max_tokens=5, temperature=0.8, top_k=20, seed=3, ignore_eos=True)
        assert all(len(o) == 5 and all(0 <= t < cfg["vocab"] for t in o) for o in out)


def test_trace_replay_command(dirs, tmp_path):
    """bin/trace_run on a Ragilorn folder: a mixed batch, then decoding, against the plain implementation."""
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


# ------------------------------------------------- latent attention for few tokens: tiles of keys that serve all heads
@pytest.mark.parametrize("act_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, dk, dv, rank, window, sink", [(16, 24, 20, 48, 0, False), (1, 8, 40, 16, 0, True), (3, 16, 8, 136, 70, False),
                                                           (8, 32, 32, 128, 0, False), (24, 16, 24, 264, 33, True), (32, 8, 16, 576, 0, False),
                                                           (9, 12, 10, 648, 0, False)])
def test_latent_attention_from_tiles_of_keys(H, dk, dv, rank, window, sink, act_dtype):
    """Tokens of several sequences at positions around page and tile borders, keys in slices of unequal sizes (some
    empty): scores, softmax (with a window and a sink) and the way out against their formulas."""
    from dlgo_b200.csrc import kernels as K
    assert K.latent_attention_tiles_takes(act_dtype, H, rank)
    g = torch.Generator().manual_seed(H + rank)
    PS = 64
    lens = [1, 31, 32, 33, 64, 65, 200, 129]                      # the token of sequence i sits at position lens[i] - 1
    n_pages = sum(-(-n // PS) for n in lens)
    pages = (torch.randn(n_pages, PS, rank, generator=g) * 0.7).to(act_dtype)
    order = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((len(lens), 4), -1, dtype=torch.int32)
    at = 0
    for i, n in enumerate(lens):
        for p in range(-(-n // PS)):
            table[i, p] = order[at]
            at += 1
    wk = (torch.randn(H * dk, rank, generator=g) / rank ** 0.5).to(act_dtype)
    wv = (torch.randn(H * dv, rank, generator=g) / rank ** 0.5).to(act_dtype)
    q = torch.randn(len(lens), H * dk + 5, generator=g) * 2.0
    sk = torch.randn(H, generator=g) if sink else None
    scale = 0.3
    T = len(lens)
    for n_slices in (1, 3, 7):
        out = K.latent_attention_tiles(q.to(DEV)[:, :H * dk], wk.to(DEV), wv.to(DEV), None if sk is None else sk.to(DEV),
                                       pages.to(DEV), table.to(DEV), i32(list(range(T))), i32(list(range(T))),
                                       i32([n - 1 for n in lens]), H, dk, dv, scale, window, n_slices,
                                       torch.empty(T * H * rank, device=DEV),
                                       torch.empty(T * H * n_slices * (rank + 2), device=DEV)).float().cpu().double()
        for i, n in enumerate(lens):
            rows = torch.cat([pages[int(table[i, p])] for p in range(-(-n // PS))]).double()[:n]
            if window:
                rows = rows[max(0, n - window):]
            for h in range(H):
                ql = wk.double()[h * dk:(h + 1) * dk].T @ q[i, h * dk:(h + 1) * dk].double()
                s = rows @ ql * scale
                if sk is not None:
                    s = torch.cat([s, sk[h:h + 1].double()])
                pr = torch.softmax(s, 0)[:rows.shape[0]]
                want = wv.double()[h * dv:(h + 1) * dv] @ (pr @ rows)
                tol = 3e-2 if act_dtype == torch.bfloat16 else 1e-4
                assert torch.allclose(out[i, h * dv:(h + 1) * dv], want, rtol=tol, atol=tol * float(want.abs().max())), \
                    (n_slices, i, h, float((out[i, h * dv:(h + 1) * dv] - want).abs().max()))
