"""Monolix on the GPU against the plain implementation (tests/plain_monolix.py): every mechanism alone, then
whole models through the engine's step function, its cache, and the public entry point."""
import copy
import json
import os

import pytest
import torch

import plain_monolix as P
from monolix_configs import (CONFIGS, SEEDS, RowCheck, assert_rows, att, layer, make_weights, moe, plain_logits, random_tokens,
                             row_error, write_model)

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
DEV = "cuda:0"


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    root = tmp_path_factory.mktemp("monolix")
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
    from dlgo_b200.config import config_from_dict
    from dlgo_b200.engine.engine import Engine
    kw.setdefault("max_tokens", 2048)
    return Engine(spec=config_from_dict(cfg).architecture_spec(), tensors=w, dtype=dtype, **kw)


def plain_of(cfg, w, tokens):
    return P.forward(cfg, {k: v.double() for k, v in w.items()}, tokens).float()


def run_whole(eng, tokens):
    s = eng.take_slot()
    try:
        return eng.step([s], [tokens], [list(range(len(tokens)))])
    finally:
        eng.free_slot(s)


# ------------------------------------------------------------------ mechanisms alone: the kernels
@pytest.mark.parametrize("T", [3, 100])
@pytest.mark.parametrize("act_dtype", [torch.float32, torch.bfloat16])
def test_norm_after_the_sum(T, act_dtype):
    from dlgo_b200.csrc import kernels as K
    g = torch.Generator().manual_seed(T)
    for d in (40, 72, 1000):
        x, y = torch.randn(T, d, generator=g), torch.randn(T, d, generator=g)
        ls, w = 1 + 0.3 * torch.randn(d, generator=g), 1 + 0.2 * torch.randn(d, generator=g)
        skip, eps = 1.75, 1e-5
        u = skip * x.double() + ls.double() * y.double()
        ref = P.rms(u, eps) * w.double()
        xd, yd = x.to(DEV), y.to(DEV)
        act = K.scaled_add_rmsnorm(xd, yd, ls.to(DEV), w.to(DEV), skip, eps, act_dtype, clear_y=True)
        assert torch.allclose(xd.cpu().double(), ref, rtol=1e-5, atol=1e-5)
        assert torch.allclose(act.cpu().double(), ref, rtol=1e-2 if act_dtype == torch.bfloat16 else 1e-5, atol=1e-2 if act_dtype == torch.bfloat16 else 1e-5)
        assert float(yd.abs().max()) == 0.0                       # left zero for the next sublayer
        # copy only
        c = K.scaled_add_rmsnorm(xd, None, None, None, 1.0, 0.0, act_dtype)
        assert torch.equal(c.float(), xd.to(act_dtype).float())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("Hq, Hkv, hd, rot", [(6, 3, 24, 12), (4, 4, 16, 16), (5, 1, 40, 8), (2, 2, 64, 0), (8, 4, 128, 64)])
def test_head_norm_rotation_and_append(Hq, Hkv, hd, rot, dtype):
    """Bias, per-head norm, rotation at far positions, and the cache rows: the key row normed and rotated, the
    value row the key as projected."""
    from dlgo_b200.csrc import kernels as K
    g = torch.Generator().manual_seed(hd)
    T, ps, base, eps = 7, 64, 30000.0, 1e-6
    pos = torch.tensor([0, 1, 63, 64, 1000, 70001, 5], dtype=torch.int32)
    cols = (Hq + Hkv) * hd
    proj = torch.randn(T, cols, generator=g)
    bias = 0.5 * torch.randn(cols, generator=g)
    wq, wk = 1 + 0.3 * torch.randn(hd, generator=g), 1 + 0.3 * torch.randn(hd, generator=g)
    u = (proj + bias).double()
    q = P.rms(u[:, :Hq * hd].view(T, Hq, hd), eps) * wq.double()
    k = P.rms(u[:, Hq * hd:].view(T, Hkv, hd), eps) * wk.double()
    if rot:
        half = rot // 2
        f = torch.tensor([base ** (-2.0 * i / rot) for i in range(half)], dtype=torch.float64)
        ang = pos.double()[:, None] * f[None]
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]

        def turn(t):
            a, b = t[..., :half], t[..., half:rot]
            return torch.cat([a * c - b * s, b * c + a * s, t[..., rot:]], -1)
        q, k = turn(q), turn(k)
    n_pages = 1200
    kp = torch.zeros(n_pages, Hkv, ps, hd, dtype=dtype, device=DEV)
    vp = torch.zeros_like(kp)
    # every token a sequence of its own; page p of a slot is physical page (slot * 7 + p * 13) % n_pages
    table = torch.full((T, 70001 // ps + 1), -1, dtype=torch.int32)
    phys = []
    for t in range(T):
        page = (t * 7 + (int(pos[t]) // ps) * 13) % n_pages
        table[t, int(pos[t]) // ps] = page
        phys.append(page)
    freq = None if not rot else torch.tensor([base ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float64).float().to(DEV)
    pd = proj.to(DEV)
    qo = K.headnorm_rope_append(pd, bias.to(DEV), wq.to(DEV), wk.to(DEV), eps, freq, rot, pos.to(DEV),
                                torch.arange(T, dtype=torch.int32, device=DEV), torch.arange(T, dtype=torch.int32, device=DEV),
                                table.to(DEV), kp, vp, Hq, Hkv, hd, True, True, True)
    K.check_device_errors()
    # fp32 angles: an angle of 70001 rad carries an absolute error of ~4e-3 rad, so far positions are compared
    # against fp32-angle tolerances
    tol = 3e-2 if dtype == torch.bfloat16 else 2e-2
    near = 2e-2 if dtype == torch.bfloat16 else 3e-4           # (an fp32 angle of 1000 rad is good to 6e-5 rad)
    for t in range(T):
        lim = near if int(pos[t]) <= 1000 else tol
        assert torch.allclose(qo[t].cpu().double().view(Hq, hd), q[t], atol=lim * 4, rtol=lim), (t, "q")
        row = int(pos[t]) % ps
        assert torch.allclose(kp[phys[t], :, row].cpu().double(), k[t], atol=lim * 4, rtol=lim), (t, "k")
        assert torch.allclose(vp[phys[t], :, row].cpu().double(), u[t, Hq * hd:].view(Hkv, hd), atol=near * 4, rtol=near), (t, "v")
    assert float(pd.abs().max()) == 0.0                            # the sum is left zero


def _route_cases():
    # (outputs, experts with tensors, top, groups, keep)
    return [(20, 15, 4, 5, 3), (8, 6, 3, 4, 2), (5, 5, 1, 1, 1), (4, 1, 2, 2, 2), (8, 8, 2, 2, 1), (64, 60, 8, 8, 4),
            (33, 30, 5, 3, 2)]


@pytest.mark.parametrize("n, E, top, groups, keep", _route_cases())
def test_router_choice_and_weights(n, E, top, groups, keep):
    """Scores over all outputs, corrections that change the choice but not the weights, groups whose losers
    count as minus infinity (corrections make choice scores negative), identity outputs included."""
    from dlgo_b200.csrc import kernels as K
    g = torch.Generator().manual_seed(n * 7 + top)
    T, d = 50, 48
    h = torch.randn(T, d, generator=g)
    Wr = 2.0 * torch.randn(n, d, generator=g) / d ** 0.5
    wg = torch.randn(1, d, generator=g) / d ** 0.5
    corr = 0.3 * torch.randn(n, generator=g) - 0.2                # mostly negative choice scores
    idx, wt, gate, plan = K.moe_router(h.to(DEV), torch.cat([Wr, wg]).to(DEV), corr.to(DEV), n, True, top, groups, keep,
                                       plan=(E, K.MOE_FEW_ROWS))
    z = h.double() @ Wr.double().T
    for t in range(T):
        want_idx, want_w = P.route(z[t], corr.double(), top, groups, keep)
        assert idx[t].tolist() == want_idx, (t, idx[t].tolist(), want_idx)
        assert torch.allclose(wt[t].cpu().double(), want_w, rtol=1e-5, atol=1e-7)
    assert torch.allclose(gate.cpu().double(), torch.sigmoid(h.double() @ wg.double().T)[:, 0], rtol=1e-5, atol=1e-7)
    # the plan made along with the choice (in the same launch for the first tokens alone) equals one made from idx
    for toks in (T, 5):
        i2, _, _, p2 = K.moe_router(h[:toks].to(DEV), torch.cat([Wr, wg]).to(DEV), corr.to(DEV), n, True, top, groups,
                                    keep, plan=(E, K.MOE_FEW_ROWS))
        want = K.moe_plan(i2, E, K.MOE_FEW_ROWS)
        assert torch.equal(i2, idx[:toks]) and torch.equal(p2.offsets, want.offsets) and torch.equal(p2.n_tiles, want.n_tiles)
        nt, total = int(want.n_tiles), int(want.offsets[-1])
        assert torch.equal(p2.tile_expert[:nt], want.tile_expert[:nt]) and torch.equal(p2.tile_row0[:nt], want.tile_row0[:nt])
        off = want.offsets.tolist()
        for e in range(E):       # the same pairs per expert, in whatever order
            assert sorted(p2.sorted_pair[off[e]:off[e + 1]].tolist()) == sorted(want.sorted_pair[off[e]:off[e + 1]].tolist())
        assert total == int((i2 < E).sum())
    # without the correction the choice differs somewhere (the test's numbers show the mechanism)
    idx0, _, _, _ = K.moe_router(h.to(DEV), Wr.to(DEV), None, n, False, top, groups, keep)
    if n > top:
        assert not torch.equal(idx0, idx)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [1, 5, 33, 300])
@pytest.mark.parametrize("d, ff, E, ident, top", [(48, 40, 6, 2, 3), (72, 24, 1, 3, 2), (50, 36, 5, 0, 1), (128, 88, 10, 3, 4)])
def test_experts_grouped_contractions(T, d, ff, E, ident, top, dtype):
    """Plan, the two grouped contractions (tiles of 8 rows and of 64) and the combine against a loop over
    tokens; identity experts return the input; sizes that are no multiple of 8 take the scalar loads."""
    from dlgo_b200.csrc import kernels as K
    g = torch.Generator().manual_seed(T + d)
    n = E + ident
    h = torch.randn(T, d, generator=g).to(dtype)
    up = (torch.randn(E, ff, d, generator=g) / d ** 0.5).to(dtype)
    down = (torch.randn(E, d, ff, generator=g) / ff ** 0.5).to(dtype)
    idx = torch.stack([torch.randperm(n, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    wt = torch.rand(T, top, generator=g)
    shared = torch.randn(T, d, generator=g)
    gate = torch.rand(T, generator=g)
    ref = torch.zeros(T, d, dtype=torch.float64)
    for t in range(T):
        for k in range(top):
            e = int(idx[t, k])
            o = h[t].double() if e >= E else P.relu2_expert(h[t].double(), up[e].double(), down[e].double())
            ref[t] += wt[t, k].double() * o
    ref += gate.double()[:, None] * shared.double()
    for rows in (K.MOE_FEW_ROWS, K.MOE_TILE_ROWS):
        plan = K.moe_plan(idx.to(DEV), E, rows)
        off = plan.offsets.cpu().tolist()
        assert off[-1] == int((idx < E).sum()) and off == sorted(off)
        hid = torch.empty(T * top, ff, dtype=dtype, device=DEV)
        K.moe_gemm(plan, h.to(DEV), up.to(DEV), hid, top, False, K.ACT_RELU2)
        po = torch.full((T * top, d), float("nan"), device=DEV)
        K.moe_gemm(plan, hid, down.to(DEV), po, None, True, K.ACT_NONE)
        y = torch.zeros(T, d, device=DEV)
        K.moe_combine(y, po, h.to(DEV), idx.to(DEV), wt.to(DEV), E, shared.to(DEV), gate.to(DEV))
        tol = 3e-2 if dtype == torch.bfloat16 else 1e-4            # (the hidden activations are rounded to bfloat16)
        assert torch.allclose(y.cpu().double(), ref, rtol=tol, atol=tol * float(ref.abs().max())), (rows, float((y.cpu().double() - ref).abs().max()))


@pytest.mark.parametrize("T", [3, 130, 700])
@pytest.mark.parametrize("d, ff, E, ident, top", [(256, 192, 5, 1, 3), (128, 80, 11, 3, 4), (72, 40, 3, 0, 2), (512, 320, 2, 0, 1)])
def test_experts_on_the_tensor_cores(T, d, ff, E, ident, top):
    """The grouped contraction on tcgen05 (tiles of 128 sorted rows; an expert's last tile runs into the next
    expert's rows, a weight tile into the next expert's weight: neither may be stored) against the fp32-pipe
    tiles, which the test above checks against a loop over tokens."""
    from dlgo_b200.csrc import kernels as K
    g = torch.Generator().manual_seed(T + d)
    n = E + ident
    h = torch.randn(T, d, generator=g).to(torch.bfloat16).to(DEV)
    up = (torch.randn(E, ff, d, generator=g) / d ** 0.5).to(torch.bfloat16).to(DEV)
    down = (torch.randn(E, d, ff, generator=g) / ff ** 0.5).to(torch.bfloat16).to(DEV)
    idx = torch.stack([torch.randperm(n, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    if T > 100:
        idx[: T // 2, 0] = 0                                   # one expert with many tiles, some with few rows
    idx = idx.to(DEV)
    assert K.moe_gemm_tc_takes(torch.bfloat16, ff, d) and K.moe_gemm_tc_takes(torch.bfloat16, d, ff)
    ref_plan = K.moe_plan(idx, E, K.MOE_TILE_ROWS)
    hid_ref = torch.zeros(T * top, ff, dtype=torch.bfloat16, device=DEV)
    K.moe_gemm(ref_plan, h, up, hid_ref, top, False, K.ACT_RELU2)
    out_ref = torch.zeros(T * top, d, device=DEV)
    K.moe_gemm(ref_plan, hid_ref, down, out_ref, None, True, K.ACT_NONE)
    for tile_rows in (K.MOE_TC_ROWS, K.MOE_TC_PAIR_ROWS):       # one CTA per tile at a time; CTA pairs on two tiles
        plan = K.moe_plan(idx, E, tile_rows)
        rows = K.moe_gather_rows(plan, h, top)
        hid = torch.full((T * top, ff), float("nan"), dtype=torch.bfloat16, device=DEV)
        K.moe_gemm_tc(plan, rows, up, hid, False, K.ACT_RELU2)
        out = torch.zeros(T * top, d, device=DEV)
        K.moe_gemm_tc(plan, hid, down, out, True, K.ACT_NONE)
        K.check_device_errors()
        total = int(plan.offsets[-1])
        assert total == int((idx < E).sum())
        # sorted rows of the two plans differ in order within an expert: compare through the pair numbers
        a = torch.zeros(T * top, ff, device=DEV)
        a[plan.sorted_pair[:total].long()] = hid[:total].float()
        b = torch.zeros(T * top, ff, device=DEV)
        b[ref_plan.sorted_pair[:total].long()] = hid_ref[:total].float()
        assert torch.isfinite(hid[:total].float()).all()
        assert torch.allclose(a, b, rtol=2e-2, atol=2e-2 * float(b.abs().max())), tile_rows
        assert torch.allclose(out, out_ref, rtol=3e-2, atol=3e-2 * float(out_ref.abs().max())), \
            (tile_rows, float((out - out_ref).abs().max()))


# ---------------------------------------------- one layer: a key that carries the answer
def one_layer(mixer, mlp=None, width=48, vocab=60, alpha=1.0):
    return {"architecture": "Monolix", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "postln_alpha": alpha,
            "layers": [layer(copy.deepcopy(mixer), mlp)]}


def standing_out(cfg, w):
    """(query token b, key token a, filler f) for a one-layer model without rotation: a's score with b stands
    far above f's with b and b's own, summed over heads."""
    wd = {k: v.double() for k, v in w.items()}
    m, eps = cfg["layers"][0]["mixer"], cfg["norm"]["eps"]
    x = wd["embed"]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = P.rms((x @ wd["l0.mix.q"].T + wd["l0.mix.q.b"]).view(-1, H, d), eps) * wd["l0.mix.q.norm"]
    k = P.rms((x @ wd["l0.mix.k"].T + wd["l0.mix.k.b"]).view(-1, G, d), eps) * wd["l0.mix.k.norm"]
    k = k.repeat_interleave(H // G, dim=1)
    s = torch.einsum("bhd,ahd->ba", q, k) * m["scale"]
    s.fill_diagonal_(-1e9)
    b, a = divmod(int(s.argmax()), s.shape[1])
    s[b, a] = 1e9
    s[b, b] = 1e9
    return b, a, int(s[b].argmin())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("mixer", [att(2, 1, 24, 0, scale=0.5), att(4, 2, 64, 0, scale=0.3)], ids=["heads24", "heads64"])
def test_one_far_key_among_hundreds(mixer, dtype):
    """One key far back carries the answer: the prompt's last token and a decoded token must both find it,
    whichever page and row it lies in."""
    cfg = one_layer(mixer)
    w = make_weights(cfg, 5, sharpen=12.0)
    b, a, f = standing_out(cfg, w)
    n = 390
    eng = engine_of(cfg, w, dtype)
    without = plain_of(cfg, w, [f] * n + [b])
    for far_pos in (0, 1, 63, 64, 200, 388):
        tokens = [f] * n + [b]
        tokens[far_pos] = a
        ref = plain_of(cfg, w, tokens)
        assert float(row_error(without[-1:], ref[-1:])) > 0.2        # the far key matters in the oracle
        s = eng.take_slot()
        assert_rows(eng.step([s], [tokens], [[n]]), ref[-1:], dtype, f"far key at {far_pos} (prompt)")
        eng.free_slot(s)
        s = eng.take_slot()
        eng.step([s], [tokens[:-1]], [[]])
        assert_rows(eng.step([s], [tokens[-1:]]), ref[-1:], dtype, f"far key at {far_pos} (decoded)")
        eng.free_slot(s)


@pytest.mark.parametrize("dtype", DTYPES)
def test_rotation_turns_with_the_distance(dtype):
    """With rotation the same two tokens score differently at different distances; the engine follows the
    oracle at every distance, in prompts cut anywhere and decoded, far beyond the first pages."""
    cfg = one_layer(att(2, 2, 32, 16, base=50.0, scale=0.6))
    w = make_weights(cfg, 9, sharpen=10.0)
    tokens = random_tokens(300, cfg["vocab"], 4)
    ref = plain_of(cfg, w, tokens)
    norot = copy.deepcopy(cfg)
    del norot["layers"][0]["mixer"]["rot"]
    assert float(row_error(plain_of(norot, w, tokens), ref).median()) > 0.1      # the rotation matters here
    eng = engine_of(cfg, w, dtype)
    assert_rows(run_whole(eng, tokens), ref, dtype, "whole")
    s = eng.take_slot()
    got = [eng.step([s], [tokens[:130]], [list(range(130))]).clone()]
    got += [eng.step([s], [tokens[p:p + 1]]).clone() for p in range(130, 300)]
    eng.free_slot(s)
    assert_rows(torch.cat(got), ref, dtype, "prefill then decode")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dim, rot", [(20, 10), (12, 12), (36, 0), (100, 50)])
def test_head_sizes_that_are_no_multiple_of_eight(dim, rot, dtype):
    """Such a head is laid out with trailing zeros; norm, rotation, scores and sums see the true size."""
    cfg = {"architecture": "Monolix", "vocab": 90, "width": 56, "norm": {"eps": 1e-6}, "postln_alpha": 1.5,
           "layers": [layer(att(4, 2, dim, rot, base=300.0, scale=0.4), moe(24, 3, 1, 2, 2, 1, 16)),
                      layer(att(4, 2, dim, rot, base=300.0, scale=0.4), moe(24, 3, 1, 2, 2, 1, 16), 0)]}
    w = make_weights(cfg, dim, mild=(dtype == "bfloat16"))
    tokens = random_tokens(150, cfg["vocab"], 6)
    ref = plain_of(cfg, w, tokens)
    eng = engine_of(cfg, w, dtype)
    assert_rows(run_whole(eng, tokens), ref, dtype, "whole")
    s = eng.take_slot()
    got = [eng.step([s], [tokens[:70]], [list(range(70))]).clone()]
    got += [eng.step([s], [tokens[p:p + 1]]).clone() for p in range(70, 150)]
    eng.free_slot(s)
    assert_rows(torch.cat(got), ref, dtype, "prefill then decode")


def test_a_layer_may_use_a_later_layer_s_tensors():
    cfg = copy.deepcopy(CONFIGS["R"])
    cfg["layers"][0]["weights_of"] = 2            # 0 -> 2 -> 1: layer 1 holds the tensors
    cfg["layers"][1].pop("weights_of")
    cfg["layers"][2]["weights_of"] = 1
    w = make_weights(cfg, 4)
    tokens = random_tokens(90, cfg["vocab"], 6)
    assert_rows(run_whole(engine_of(cfg, w, "float32"), tokens), plain_of(cfg, w, tokens), "float32", "whole")


@pytest.mark.parametrize("dtype", DTYPES)
def test_values_are_the_keys_as_projected(dtype):
    """What is summed is the key before norm and rotation, with its bias: an oracle that sums the normed and
    rotated key instead differs visibly, and the engine agrees with the right one."""
    cfg = one_layer(att(3, 1, 16, 8, scale=0.5))
    w = make_weights(cfg, 3)
    tokens = random_tokens(80, cfg["vocab"], 5)
    ref = plain_of(cfg, w, tokens)
    wd = {k: v.double() for k, v in w.items()}
    m, eps = cfg["layers"][0]["mixer"], cfg["norm"]["eps"]
    x = wd["embed"][torch.tensor(tokens)]
    T, H, d = len(tokens), m["heads"], m["dim"]
    q = P.rotate(P.rms((x @ wd["l0.mix.q"].T + wd["l0.mix.q.b"]).view(T, H, d), eps) * wd["l0.mix.q.norm"], m["rot"]["base"], m["rot"]["dims"])
    k = P.rotate(P.rms((x @ wd["l0.mix.k"].T + wd["l0.mix.k.b"]).view(T, 1, d), eps) * wd["l0.mix.k.norm"], m["rot"]["base"], m["rot"]["dims"])
    sc = torch.einsum("ihd,jd->hij", q, k[:, 0]) * m["scale"]
    sc = sc.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
    wrong = torch.einsum("hij,jd->ihd", torch.softmax(sc, -1), k[:, 0]).reshape(T, H * d) @ wd["l0.mix.o"].T
    xw = P.one_plus_norm(cfg["postln_alpha"] * x + wd["l0.ls1"] * wrong, wd["l0.norm1"], eps)
    wrong_logits = (P.one_plus_norm(xw, wd["final.norm"], eps) @ wd["head"].T).float()
    assert float(row_error(wrong_logits, ref).median()) > 0.05
    assert_rows(run_whole(engine_of(cfg, w, dtype), tokens), ref, dtype, "values")


# ------------------------------------------------------------------------------- whole models
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompts(dirs, name, dtype):
    eng = engine_for(dirs[name, dtype], dtype)
    V = CONFIGS[name]["vocab"]
    rows = RowCheck(dtype, f"{name}: whole prompts")
    for n in (1, 2, 3, 63, 64, 65, 129, 211):
        tokens = random_tokens(n, V, 100 + n)
        rows.add(run_whole(eng, tokens), plain_logits(dirs[name, dtype], tokens), f"{name}: prompt of {n}")
    rows.done()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_prefill_then_token_by_token(dirs, name, graphs, dtype):
    """A short prompt, then more than two pages of decoding (with and without captured steps)."""
    eng = engine_for(dirs[name, dtype], dtype, cuda_graphs=graphs)
    V = CONFIGS[name]["vocab"]
    tokens = random_tokens(170, V, 7)
    ref = plain_logits(dirs[name, dtype], tokens)
    for start in (1, 5):
        s = eng.take_slot()
        got = [eng.step([s], [tokens[:start]], [list(range(start))]).clone()]
        for p in range(start, len(tokens)):
            got.append(eng.step([s], [tokens[p:p + 1]]).clone())
        eng.free_slot(s)
        assert_rows(torch.cat(got), ref, dtype, f"{name}: decoding from {start}")
    eng.cache.book.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_portions(dirs, name, dtype):
    eng = engine_for(dirs[name, dtype], dtype)
    V = CONFIGS[name]["vocab"]
    tokens = random_tokens(200, V, 8)
    ref = plain_logits(dirs[name, dtype], tokens)
    for cuts in ([2] * 100, [3, 61, 1, 63, 2, 70], [64, 64, 64, 8], [7, 193], [199, 1], [100, 2, 98]):
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
    lens = [1, 140, 2, 66, 31]
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
def test_pages_and_slots_used_again(dirs, dtype):
    """A small cache whose pages go round several times, poisoned where nothing was written."""
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
        assert info.architecture == "Monolix" and info.layers == len(cfg["layers"])
        assert (info.heads, info.kv_heads) == (cfg["layers"][0]["mixer"]["heads"], cfg["layers"][0]["mixer"]["kv_heads"])
        out = llm.generate(prompts[:2], max_tokens=5, temperature=0.8, top_k=20, seed=3, ignore_eos=True)
        assert all(len(o) == 5 and all(0 <= t < cfg["vocab"] for t in o) for o in out)


def test_trace_replay_command(dirs, tmp_path):
    """bin/trace_run on a Monolix folder: a mixed batch, then decoding, against the plain implementation."""
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
