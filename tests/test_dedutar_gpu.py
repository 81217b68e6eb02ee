"""Dedutar on the GPU against the plain implementation (tests/plain_dedutar.py): every mechanism alone, then
whole models through the engine's step function, its cache and state, and the public entry point."""
import copy
import json
import os

import pytest
import torch

import plain_dedutar as P
from dedutar_configs import CONFIGS, SEEDS, assert_rows, make_weights, plain_logits, random_tokens, row_error, write_model

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


def _dev():
    return torch.device("cuda:0")


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    root = tmp_path_factory.mktemp("dedutar")
    out = {(n, "float32"): write_model(n, str(root / n)) for n in CONFIGS}
    # bfloat16 runs get milder queries and keys: through nine layers of very peaked softmaxes, rounding alone
    # flips near ties between two keys and moves single rows as far as a fault would
    out.update({(n, "bfloat16"): write_model(n, str(root / (n + "_mild")), sharpen=1.5) for n in CONFIGS})
    return out


_engines = {}


def engine_for(model_dir, dtype, **kw):
    from dlgo_b200.engine.engine import Engine
    key = (model_dir, dtype, tuple(sorted(kw.items())))
    if key not in _engines:
        kw.setdefault("max_tokens", 4096)
        _engines[key] = Engine(model_dir, dtype=dtype, **kw)
    return _engines[key]


def run_whole(eng, tokens):
    s = eng.take_slot()
    try:
        return eng.step([s], [tokens], [list(range(len(tokens)))])
    finally:
        eng.free_slot(s)


# ------------------------------------------------------------------ mechanisms alone: the small kernels
@pytest.mark.parametrize("s", [1, 2, 5])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_streams_write_and_read(s, out_dtype):
    from dlgo_b200.csrc import kernels as K
    g = torch.Generator().manual_seed(s)
    T, d = 37, 88
    X = torch.randn(T, s, d, generator=g)
    y = torch.randn(T, d, generator=g)
    bias = torch.randn(d, generator=g)
    w = {"c.in": torch.randn(s, generator=g), "c.out": torch.randn(s, generator=g), "c.mix": torch.randn(s, s, generator=g),
         "n": 1 + 0.1 * torch.randn(d, generator=g), "n.b": 0.1 * torch.randn(d, generator=g), "n.alpha": torch.tensor(0.7)}
    # the plain write: the sublayer returns y + bias whatever it reads
    Xs = X.permute(1, 0, 2).double()
    wd = {k: v.double() for k, v in w.items()}
    new = P.hyper_sublayer(Xs, wd, "c.", lambda u: (y + bias).double())
    u = torch.einsum("s,std->td", wd["c.in"], new)
    want_dyt = P.dynamic_tanh(u, wd, "n")
    want_rms = P.rms(u, 1e-5) * wd["n"]
    dev = _dev()
    tol = 1e-5 if out_dtype == torch.float32 else 1.6e-2
    for kind, want in ((K.NORM_DYT, want_dyt), (K.NORM_RMS, want_rms), (K.NORM_NONE, u)):
        Xg, yg = X.to(dev).clone(), y.to(dev).clone()
        out = K.streams_step(Xg, y=yg, y_bias=bias.to(dev), mix=w["c.mix"].to(dev), write=w["c.out"].to(dev), clear_y=True,
                             read=w["c.in"].to(dev), norm_kind=kind, norm_w=w["n"].to(dev), norm_b=w["n.b"].to(dev),
                             norm_alpha=w["n.alpha"].reshape(1).to(dev), eps=1e-5, out_dtype=out_dtype)
        assert float((Xg.cpu().double() - new.permute(1, 0, 2)).abs().max()) < 1e-5
        assert float(yg.abs().max()) == 0.0                          # left zero for the next sublayer
        assert float((out.cpu().double() - want).abs().max()) <= tol * float(want.abs().max())
        # the same in two launches, and the read alone on chosen rows
        Xg2, yg2 = X.to(dev).clone(), y.to(dev).clone()
        assert K.streams_step(Xg2, y=yg2, y_bias=bias.to(dev), mix=w["c.mix"].to(dev), write=w["c.out"].to(dev)) is None
        assert torch.equal(Xg2, Xg) and torch.equal(yg2.cpu(), y)    # not cleared unless asked
        rows = torch.tensor([5, 0, 36, 5], dtype=torch.int32, device=dev)
        part = K.streams_step(Xg2, read=w["c.in"].to(dev), norm_kind=kind, norm_w=w["n"].to(dev), norm_b=w["n.b"].to(dev),
                              norm_alpha=w["n.alpha"].reshape(1).to(dev), eps=1e-5, out_dtype=out_dtype, rows=rows)
        assert torch.equal(part, out[rows.long()])
    # the plain sum of the streams (the model's last read)
    total = K.streams_step(X.to(dev), norm_kind=K.NORM_NONE, out_dtype=torch.float32)
    assert float((total.cpu() - X.sum(1)).abs().max()) < 1e-5


def test_bias_activation_and_gated_norm():
    from dlgo_b200.csrc import kernels as K
    g = torch.Generator().manual_seed(3)
    dev = _dev()
    z = 2 * torch.randn(19, 130, generator=g)
    b = torch.randn(130, generator=g)
    zd = (z + b).double()
    for act, want in ((K.ACT_RELU2, torch.relu(zd) ** 2), (K.ACT_SILU, P.silu(zd)), (K.ACT_GELU_TANH, P.gelu_tanh(zd)),
                      (K.ACT_NONE, zd)):
        got = K.bias_act(z.to(dev), b.to(dev), act, torch.float32)
        assert float((got.cpu().double() - want).abs().max()) < 1e-5
        got16 = K.bias_act(z.to(dev), b.to(dev), act, torch.bfloat16)
        assert float((got16.float().cpu().double() - want).abs().max()) <= 8e-3 * float(want.abs().max())
    # a column slice (row stride larger than the width), in place
    wide = torch.randn(7, 50, generator=g).to(dev)
    view = wide[:, 10:30]
    ref = (view.cpu() + b[:20])
    K.bias_act(view, b[:20].contiguous().to(dev), K.ACT_NONE, torch.float32, in_place=True)
    assert float((wide[:, 10:30].cpu() - ref).abs().max()) < 1e-6
    o = torch.randn(11, 96, generator=g) * 3
    gate = torch.randn(11, 200, generator=g)
    w = 1 + 0.1 * torch.randn(96, generator=g)
    want = P.rms(o.double(), 1e-5) * w.double() * torch.sigmoid(gate[:, 100:196].double())
    got = K.gated_rmsnorm(o.to(dev), gate.to(dev)[:, 100:196], w.to(dev), 1e-5, torch.float32)
    assert float((got.cpu().double() - want).abs().max()) < 1e-5


# ------------------------------------------------- mechanisms alone: one mixer in a model of one layer
def one_layer(layer, streams=1, width=48, vocab=60):
    layer = copy.deepcopy(layer)
    layer["mlp"] = None
    return {"architecture": "Dedutar", "vocab": vocab, "width": width, "streams": streams, "norm": {"eps": 1e-6},
            "loop": None, "layers": [layer]}


def engine_of(cfg, w, dtype, **kw):
    from dlgo_b200.config import config_from_dict
    from dlgo_b200.engine.engine import Engine
    kw.setdefault("max_tokens", 2048)
    return Engine(spec=config_from_dict(cfg).architecture_spec(), tensors=w, dtype=dtype, **kw)


def plain_of(cfg, w, tokens):
    return P.forward(cfg, {k: v.double() for k, v in w.items()}, tokens).float()


def token_scores(cfg, w):
    """Layer 0 has no positions: the score of query token b with key token a depends on the two tokens only.
    Returns [b, a] summed over heads (before the softmax)."""
    wd = {k: v.double() for k, v in w.items()}
    m, eps = cfg["layers"][0]["mixer"], cfg["norm"]["eps"]
    u = wd["embed"] * wd["l0.hc1.in"].sum()
    h = P.dynamic_tanh(u, wd, "l0.norm1")
    if cfg["layers"][0]["type"] == "latent_attention":
        q = (P.rms(h @ wd["l0.mix.dq"].T, eps) * wd["l0.mix.dq.norm"]) @ wd["l0.mix.uq"].T
    else:
        q = h @ wd["l0.mix.q"].T
    c = P.rms(h @ wd["l0.mix.dkv"].T, eps) * wd["l0.mix.dkv.norm"]
    k = c @ wd["l0.mix.uk"].T
    H, dk = m["heads"], m["dim"]
    return torch.einsum("bhd,ahd->ba", q.view(-1, H, dk), k.view(-1, H, dk)) * m["scale"]


def standing_out(cfg, w):
    """(query token b, key token a, filler f): a's score with b stands far above f's with b and b's own."""
    s = token_scores(cfg, w)
    s.fill_diagonal_(-1e9)
    b, a = divmod(int(s.argmax()), s.shape[1])
    s[b, a] = 1e9
    s[b, b] = 1e9
    f = int(s[b].argmin())
    return b, a, f


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", ["latent_attention", "latent_attention_2"])
def test_one_far_key_among_hundreds(kind, dtype):
    """One key far back carries the answer: the prompt's last token and a decoded token must both find it."""
    layer = CONFIGS["Q"]["layers"][0] if kind == "latent_attention_2" else \
        {"type": kind, "mixer": {"heads": 2, "dim": 16, "vdim": 24, "kv_rank": 40, "q_rank": 24, "scale": 0.25,
                                 "mask": {"size": 400}}}
    cfg = one_layer(layer)
    w = make_weights(cfg, 5, sharpen=16.0)
    b, a, f = standing_out(cfg, w)
    n = 390
    for far_pos in (0, 1, 63, 64, 200):
        tokens = [f] * n + [b]
        tokens[far_pos] = a
        ref = plain_of(cfg, w, tokens)
        without = plain_of(cfg, w, [f] * n + [b])
        assert float(row_error(without[-1:], ref[-1:])) > 0.2        # the far key matters in the oracle
        eng = engine_of(cfg, w, dtype)
        s = eng.take_slot()
        got = eng.step([s], [tokens], [[n]])
        assert_rows(got, ref[-1:], dtype, f"far key at {far_pos} (prompt)")
        eng.free_slot(s)
        s = eng.take_slot()
        eng.step([s], [tokens[:-1]], [[]])
        got = eng.step([s], [tokens[-1:]])
        assert_rows(got, ref[-1:], dtype, f"far key at {far_pos} (decoded)")
        eng.free_slot(s)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [1, 2, 40, 64, 65, 130])
def test_window_edge(window, dtype):
    """The key that carries the answer sits just inside or just outside the window: in a prompt and decoded."""
    layer = {"type": "latent_attention", "mixer": {"heads": 3, "dim": 8, "vdim": 16, "kv_rank": 24, "q_rank": 16,
                                                   "scale": 0.35, "mask": {"size": window}}}
    cfg = one_layer(layer, streams=2)
    w = make_weights(cfg, 6, sharpen=16.0)
    b, a, f = standing_out(cfg, w)
    n = 200
    eng = engine_of(cfg, w, dtype)
    refs = {}
    for dist in (window - 1, window):            # inside, outside
        if dist == 0:
            continue                               # (the query itself: a window of one position)
        tokens = [f] * n + [b]
        tokens[n - dist] = a
        refs[dist] = ref = plain_of(cfg, w, tokens)
        s = eng.take_slot()
        got = eng.step([s], [tokens], [[n - 1, n]])
        assert_rows(got, ref[n - 1:], dtype, f"window {window}, key at distance {dist} (prompt)")
        eng.free_slot(s)
        s = eng.take_slot()
        eng.step([s], [tokens[:n - 3]], [[]])
        for p in range(n - 3, n + 1):
            got = eng.step([s], [tokens[p:p + 1]])
        assert_rows(got, ref[n:], dtype, f"window {window}, key at distance {dist} (decoded)")
        eng.free_slot(s)
    if window > 1:
        assert float(row_error(refs[window - 1][-1:], refs[window][-1:])) > 0.2     # the edge shows in the oracle


@pytest.mark.parametrize("dim", [64, 128])
@pytest.mark.parametrize("kind, window", [("latent_attention_2", None), ("latent_attention", 100),
                                          ("latent_attention", 64), ("latent_attention", 1000)])
def test_latent_prompts_on_the_tensor_cores(kind, window, dim):
    """bfloat16 prompt steps with heads of 64 and 128 make the step's keys and values and run on the tensor
    cores: whole prompts, portions that read back what earlier portions cached (also behind a window whose pages
    were given back), unequal batches, a sink, and one far key that carries the answer."""
    from dlgo_b200.csrc import kernels as K
    dtype = "bfloat16"
    m = {"heads": 3, "dim": dim, "vdim": dim, "kv_rank": 96, "scale": dim ** -0.5}
    if kind == "latent_attention":
        m.update(q_rank=48, mask={"size": window})
    cfg = one_layer({"type": kind, "mixer": m}, streams=2, width=64)
    w = make_weights(cfg, 9, sharpen=16.0)
    b, a, f = standing_out(cfg, w)
    n = 330
    tokens = random_tokens(n, cfg["vocab"], 4)
    ref = plain_of(cfg, w, tokens)
    eng = engine_of(cfg, w, dtype)
    K.profile_start()
    got = run_whole(eng, tokens)
    names = {k for k, _, _ in K.profile_stop()}
    assert "attention_prefill_tc_rows" in names and "latent_attention" not in names
    assert_rows(got, ref, dtype, "whole prompt")
    for cuts in ([130, 200], [64, 64, 202], [100, 70, 96, 64], [329, 1]):
        s = eng.take_slot()
        out, at = [], 0
        for c in cuts:
            out.append(eng.step([s], [tokens[at:at + c]], [list(range(c))]).clone())
            at += c
        eng.free_slot(s)
        assert_rows(torch.cat(out), ref, dtype, f"portions {cuts}")
    # unequal prompts in one step
    lens = [70, 330, 129, 64]
    slots = [eng.take_slot() for _ in lens]
    out = eng.step(slots, [tokens[:k] for k in lens], [list(range(k)) for k in lens])
    off = 0
    for k in lens:
        assert_rows(out[off:off + k], ref[:k], dtype, f"a prompt of {k} in a batch")
        off += k
    for s in slots:
        eng.free_slot(s)
    # the key that carries the answer: far back, at a page's border, just inside and just outside the window
    places = [0, 63, 64, 191] if window is None else [n - window, n - window + 1]
    for place in places:
        if place < 0:
            continue
        seq = [f] * n + [b]
        seq[place] = a
        r2 = plain_of(cfg, w, seq)
        s = eng.take_slot()
        got = eng.step([s], [seq], [[n - 1, n]])
        eng.free_slot(s)
        assert_rows(got, r2[n - 1:], dtype, f"key at {place}")
    if window is not None and window < n:
        inside, outside = [f] * n + [b], [f] * n + [b]
        inside[n - window + 1] = a
        outside[n - window] = a
        assert float(row_error(plain_of(cfg, w, inside)[-1:], plain_of(cfg, w, outside)[-1:])) > 0.2


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rank", [21, 18, 72, 264])
def test_latent_ranks_of_any_size(rank, dtype):
    """Ranks that are odd, even but no multiple of a 16-byte piece, and beyond one piece per lane: prompt,
    portions and decoding agree with the plain implementation."""
    layer = {"type": "latent_attention", "mixer": {"heads": 2, "dim": 12, "vdim": 20, "kv_rank": rank, "q_rank": 9,
                                                   "scale": 0.3, "mask": {"size": 50}}}
    cfg = one_layer(layer, streams=1, width=40)
    w = make_weights(cfg, 10, sharpen=2.0)
    tokens = random_tokens(90, cfg["vocab"], 6)
    ref = plain_of(cfg, w, tokens)
    eng = engine_of(cfg, w, dtype)
    assert_rows(run_whole(eng, tokens), ref, dtype, "whole")
    s = eng.take_slot()
    got = [eng.step([s], [tokens[:70]], [list(range(70))]).clone()]
    got.append(eng.step([s], [tokens[70:75]], [list(range(5))]).clone())
    for p in range(75, 90):
        got.append(eng.step([s], [tokens[p:p + 1]]).clone())
    eng.free_slot(s)
    assert_rows(torch.cat(got), ref, dtype, "prompt, a portion, decoding")


@pytest.mark.parametrize("dtype", DTYPES)
def test_sink_counts_once_and_unscaled(dtype):
    layer = {"type": "latent_attention_2", "mixer": {"heads": 4, "dim": 8, "vdim": 8, "kv_rank": 16, "scale": 0.5}}
    cfg = one_layer(layer, streams=3)
    w = make_weights(cfg, 7)
    tokens = random_tokens(70, cfg["vocab"], 1)
    eng = engine_of(cfg, w, dtype)
    ref = plain_of(cfg, w, tokens)
    assert_rows(run_whole(eng, tokens), ref, dtype, "with sinks")
    w2 = dict(w)
    w2["l0.mix.sink"] = torch.full_like(w["l0.mix.sink"], -30.0)      # a sink that weighs nothing
    ref2 = plain_of(cfg, w2, tokens)
    assert float(row_error(ref2, ref).max()) > 0.05                  # leaving the sink out shows
    assert_rows(run_whole(engine_of(cfg, w2, dtype), tokens), ref2, dtype, "sinks of no weight")
    w3 = dict(w)
    w3["l0.mix.sink"] = torch.tensor([9.0, -3.0, 4.0, 0.0]).to(torch.bfloat16)   # one that dominates, first token too
    assert_rows(run_whole(engine_of(cfg, w3, dtype), tokens), plain_of(cfg, w3, tokens), dtype, "a dominating sink")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decay", [[1.0, 0.0, 0.5], [0.999, 0.9, 0.99]])
@pytest.mark.parametrize("dim, vdim", [(16, 24), (32, 40), (64, 160), (128, 16), (200, 160)])
def test_lightning_state_is_carried(dim, vdim, decay, dtype):
    """qk sizes of both kernels (the state in shared memory; in registers with a prompt cut into segments that
    run side by side), value sizes below, at and above a block's columns, and a state too large for one block."""
    layer = {"type": "lightning", "mixer": {"heads": 3, "dim": dim, "vdim": vdim, "decay": decay}}
    cfg = one_layer(layer, streams=2)
    w = make_weights(cfg, 8)
    tokens = random_tokens(300, cfg["vocab"], 2)
    ref = plain_of(cfg, w, tokens)
    eng = engine_of(cfg, w, dtype)
    assert_rows(run_whole(eng, tokens), ref, dtype, "whole")
    for cuts in ([1, 1, 2, 3, 60, 64, 169], [299, 1], [2] * 150, [129, 128, 43], [10, 290]):
        s = eng.take_slot()
        got, at = [], 0
        for c in cuts:
            got.append(eng.step([s], [tokens[at:at + c]], [list(range(c))]).clone())   # (a decode step's logits live until the next)
            at += c
        eng.free_slot(s)
        assert_rows(torch.cat(got), ref, dtype, f"portions {cuts[:4]}...")
    # a slot that is taken again starts from a zero state
    s = eng.take_slot()
    eng.step([s], [tokens[:40]], [[]])
    eng.free_slot(s)
    s2 = eng.take_slot()
    assert s2 == s
    assert_rows(eng.step([s2], [tokens[:9]], [list(range(9))]), ref[:9], dtype, "slot used again")
    eng.free_slot(s2)


# ------------------------------------------------------------------------------- whole models
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompts(dirs, name, dtype):
    eng = engine_for(dirs[name, dtype], dtype)
    V = CONFIGS[name]["vocab"]
    for n in (1, 2, 3, 63, 64, 65, 129, 211):
        tokens = random_tokens(n, V, 100 + n)
        assert_rows(run_whole(eng, tokens), plain_logits(dirs[name, dtype], tokens), dtype, f"{name}: prompt of {n}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_prefill_then_token_by_token(dirs, name, graphs, dtype):
    """A short prompt, then more than two pages of decoding: windows slide over decoded tokens, pages of
    windowed layers are given back, states are carried."""
    eng = engine_for(dirs[name, dtype], dtype, cuda_graphs=graphs)
    V = CONFIGS[name]["vocab"]
    tokens = random_tokens(190, V, 7)
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
            got.append(eng.step([s], [tokens[at:at + c]], [list(range(c))]).clone())   # (a decode step's logits live until the next)
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
    for i, n in enumerate(lens):
        assert_rows(got[off:off + n], refs[i][:n], dtype, f"{name}: sequence {i} of a mixed prompt batch")
        off += n
    # decoded together; the shorter ones leave the batch one after another
    live = list(range(len(seqs)))
    for step in range(40):
        if step in (9, 17, 30):
            eng.free_slot(slots[live.pop(0)])
        out = eng.step([slots[i] for i in live], [[seqs[i][lens[i] + step]] for i in live])
        for j, i in enumerate(live):
            assert_rows(out[j:j + 1], refs[i][lens[i] + step:lens[i] + step + 1], dtype,
                        f"{name}: sequence {i}, decoded step {step} in a batch of {len(live)}")
    for i in live:
        eng.free_slot(slots[i])
    eng.cache.book.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_pages_and_slots_used_again(dirs, dtype):
    """A small cache whose pages go round several times, poisoned where nothing was written."""
    name = "Q"
    eng = engine_for(dirs[name, dtype], dtype, max_tokens=512, max_slots=3)
    eng.cache.poison()
    V = CONFIGS[name]["vocab"]
    for r in range(5):
        lens = [150 + 7 * r, 90 - r, 60 + r]
        seqs = [random_tokens(n, V, 300 + 10 * r + i) for i, n in enumerate(lens)]
        slots = [eng.take_slot() for _ in seqs]
        got = eng.step(slots, seqs, [[n - 2, n - 1] for n in lens])
        for i, n in enumerate(lens):
            assert_rows(got[2 * i:2 * i + 2], plain_logits(dirs[name, dtype], seqs[i])[n - 2:], dtype, f"round {r}, sequence {i}")
        for s in (slots[1], slots[0], slots[2]):
            eng.free_slot(s)
    eng.cache.book.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(dirs, dtype):
    name = "R"
    eng = engine_for(dirs[name, dtype], dtype)
    V = CONFIGS[name]["vocab"]
    tokens = random_tokens(420, V, 9)
    ref = plain_logits(dirs[name, dtype], tokens)
    s = eng.take_slot()
    eng.step([s], [tokens[:20]], [[]])
    for p in range(20, len(tokens)):
        out = eng.step([s], [tokens[p:p + 1]])
        if p % 37 == 0 or p >= len(tokens) - 3:
            assert_rows(out, ref[p:p + 1], dtype, f"decoded position {p}")
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
        assert llm.model_info().architecture == "Dedutar"
        # sampled generation runs through the same loop and kernels
        out = llm.generate(prompts[:2], max_tokens=5, temperature=0.8, top_k=20, seed=3, ignore_eos=True)
        assert all(len(o) == 5 and all(0 <= t < cfg["vocab"] for t in o) for o in out)


def test_trace_replay_command(dirs, tmp_path):
    """bin/trace_run on a Dedutar folder: a mixed batch, then decoding, against the plain implementation."""
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


@pytest.mark.parametrize("tokens", [1, 8, 17, 64, 65, 300])
@pytest.mark.parametrize("n, k", [(384, 320), (200, 96), (1024, 512)])
def test_contraction_with_bias_and_activation(tokens, n, k):
    """The tensor-core contraction's bias + activation epilogue (few tokens: weight rows as the tile's rows, with
    and without K-slices; many tokens: weight rows as its columns) against fp32 arithmetic."""
    from dlgo_b200.csrc import kernels as K
    from dlgo_b200.engine.runtime import Runtime
    from dlgo_b200.parts.linear import Linear
    g = torch.Generator().manual_seed(tokens + n)
    dev = _dev()
    w = (torch.randn(n, k, generator=g) / k ** 0.5).to(torch.bfloat16)
    x = torch.randn(tokens, k, generator=g).to(torch.bfloat16)
    b = torch.randn(n, generator=g)
    lin = Linear(w.to(dev), Runtime("cuda:0", "bfloat16"))
    z = x.double() @ w.double().T + b.double()
    for act, want in ((K.ACT_RELU2, torch.relu(z) ** 2), (K.ACT_NONE, z), (K.ACT_SILU, P.silu(z)), (K.ACT_GELU_TANH, P.gelu_tanh(z))):
        got = lin.bias_act(x.to(dev), b.to(dev), act)
        assert got.dtype == torch.bfloat16 and tuple(got.shape) == (tokens, n)
        assert float((got.float().cpu().double() - want).abs().max()) <= 1e-2 * float(want.abs().max())
    got = lin.bias_act(x.to(dev), None, K.ACT_RELU2)
    want = torch.relu(x.double() @ w.double().T) ** 2
    assert float((got.float().cpu().double() - want).abs().max()) <= 1e-2 * float(want.abs().max())
