"""Monolix without a GPU: the configuration's keys, run order, parts and constants, expected tensors, cache needs
and refusals; the plain implementation's pieces against hand-made cases; and the test weights' sensitivity."""
import copy

import pytest
import torch

import plain_monolix as P
from monolix_configs import CONFIGS, SEEDS, att, layer, make_weights, moe, random_tokens, row_error

from dlgo_b200.config import ConfigError, config_from_dict
from dlgo_b200.engine.model import CausalLM


def plain_of(cfg, w, tokens):
    return P.forward(cfg, {k: v.double() for k, v in w.items()}, tokens).float()


def test_registry_and_keys():
    cfg = config_from_dict(CONFIGS["P"])
    assert type(cfg).__name__ == "MonolixConfig" and cfg.vocab == 150 and cfg.width == 72
    assert cfg.postln_alpha == 1.7 and cfg.norm_eps == 1e-5
    assert [L.weights_of for L in cfg.layers] == [None, 0, None, 0]          # a chain ends where the tensors are
    a = cfg.layers[0].mixer
    assert (a.heads, a.kv_heads, a.dim, a.scale, a.rot_base, a.rot_dims) == (6, 3, 24, 0.3, 5000.0, 12)
    e = cfg.layers[0].mlp
    assert (e.ff, e.experts, e.identity, e.top, e.group_count, e.group_keep, e.shared_ff) == (40, 6, 2, 3, 4, 2, 56)
    assert cfg.layers[2].mlp is None and cfg.layers[2].mixer.rot_base is None
    again = config_from_dict(cfg.to_dict())
    assert again == cfg


def test_run_order_shares_tensors_but_not_caches():
    spec = config_from_dict(CONFIGS["P"]).architecture_spec()
    assert [ls.prefix for ls in spec.layers] == ["l0.", "l2."]
    assert [(e.layer, e.cache_of) for e in spec.order] == [(0, None), (0, None), (1, None), (0, None)]
    model = CausalLM(spec)
    needs, borrows, states = model.cache_needs()
    assert borrows == [None] * 4 and not states
    assert [(n.num_kv_heads, n.head_dim, n.planes, n.window) for n in needs] == [(3, 24, 2, None)] * 2 + [(1, 32, 2, None), (3, 24, 2, None)]


def test_a_head_size_that_is_no_multiple_of_eight_is_laid_out_as_the_next_one():
    cfg = {"architecture": "Monolix", "vocab": 50, "width": 40, "norm": {"eps": 1e-6}, "postln_alpha": 1.0,
           "layers": [layer(att(3, 1, 20, 10), None)]}
    model = CausalLM(config_from_dict(cfg).architecture_spec())
    shape = {n: tuple(ps.shape) for n, ps in model.expected_tensors().items()}
    assert shape["l0.mix.q"] == (60, 40) and shape["l0.mix.k"] == (20, 40) and shape["l0.mix.o"] == (40, 60)
    assert shape["l0.mix.q.norm"] == (20,)
    needs, _, _ = model.cache_needs()
    assert (needs[0].num_kv_heads, needs[0].head_dim) == (1, 24)


def test_weights_of_may_name_a_later_layer_and_chains_end_at_the_holder():
    c = copy.deepcopy(CONFIGS["R"])
    c["layers"][0]["weights_of"] = 2            # 0 -> 2 -> 1: layer 1 holds the tensors
    c["layers"][1].pop("weights_of")
    c["layers"][2]["weights_of"] = 1
    cfg = config_from_dict(c)
    assert [L.weights_of for L in cfg.layers] == [1, None, 1]
    spec = cfg.architecture_spec()
    assert [ls.prefix for ls in spec.layers] == ["l1."] and [e.layer for e in spec.order] == [0, 0, 0]
    w = make_weights(c, 3)
    assert all(n.startswith("l1.") or "." not in n or n.startswith("final") for n in w)
    assert P.weights_layer(c, 0) == 1 and P.weights_layer(c, 2) == 1
    c["layers"][1]["weights_of"] = 0            # a circle
    with pytest.raises(ConfigError):
        config_from_dict(c)


def test_expected_tensors():
    t = CausalLM(config_from_dict(CONFIGS["P"]).architecture_spec()).expected_tensors()
    shape = {n: tuple(ps.shape) for n, ps in t.items()}
    assert shape["embed"] == (150, 72) and shape["head"] == (150, 72) and shape["final.norm"] == (72,)
    assert shape["l0.mix.q"] == (144, 72) and shape["l0.mix.k"] == (72, 72) and shape["l0.mix.o"] == (72, 144)
    assert shape["l0.mix.q.b"] == (144,) and shape["l0.mix.k.b"] == (72,)
    assert shape["l0.mix.q.norm"] == (24,) and shape["l0.mix.k.norm"] == (24,)
    assert shape["l0.mlp.router"] == (8, 72) and shape["l0.mlp.correction"] == (8,)
    assert shape["l0.mlp.e5.up"] == (40, 72) and shape["l0.mlp.e5.down"] == (72, 40) and "l0.mlp.e6.up" not in shape
    assert shape["l0.mlp.shared.up"] == (56, 72) and shape["l0.mlp.shared.down"] == (72, 56) and shape["l0.mlp.shared.sg"] == (1, 72)
    assert shape["l0.ls1"] == (72,) and shape["l0.ls2"] == (72,) and shape["l0.norm1"] == (72,) and shape["l0.norm2"] == (72,)
    assert not any(n.startswith("l1.") or n.startswith("l3.") for n in shape)          # they use layer 0's
    assert "l2.norm1" in shape and "l2.ls1" in shape and "l2.norm2" not in shape and "l2.mlp.router" not in shape
    assert not any(".v" in n for n in shape)                                             # the values are the keys
    q = CausalLM(config_from_dict(CONFIGS["Q"]).architecture_spec()).expected_tensors()
    assert "l0.mlp.correction" in q and "l0.mlp.shared.up" not in q and tuple(q["l1.mlp.router"].shape) == (4, 48)


@pytest.mark.parametrize("change, where", [
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=4), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"].update(vdim=32), "vdim"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=13), "rot"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=26), "rot"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "top"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=3), "groups"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(keep=5), "groups"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "kind"),
    (lambda c: c["layers"][0].update(type="recurrent"), "type"),
    (lambda c: c["layers"][1].update(weights_of=1), "weights_of"),
    (lambda c: c["layers"][1].update(mixer=dict(c["layers"][1]["mixer"], heads=3)), "sizes differ"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_refusals(change, where):
    c = copy.deepcopy(CONFIGS["P"])
    change(c)
    with pytest.raises(ConfigError) as e:
        config_from_dict(c)
    assert where in str(e.value) or where == "sizes differ"


def test_random_model_mode_knows_the_design(tmp_path):
    from dlgo_b200.weights.random_init import write_random_model
    out = write_random_model(config_from_dict(CONFIGS["Q"]), 3, str(tmp_path / "m"))
    cfg, w = P.read_model(out)
    assert cfg["architecture"] == "Monolix" and set(w) == set(make_weights(CONFIGS["Q"], 1))
    assert abs(float(w["l0.norm1"].float().mean())) < 0.05 and abs(float(w["l0.ls1"].float().mean()) - 1) < 0.05


# ------------------------------------------------------------------------ the oracle's pieces
def test_route_by_hand():
    # 8 outputs in 4 groups of 2, keep 2, top 3.  softmax of equal logits is 1/8 each, so the correction decides.
    z = torch.zeros(8, dtype=torch.float64)
    corr = torch.tensor([0.0, -0.5, 0.3, -0.9, 0.2, 0.25, -0.3, -0.2], dtype=torch.float64)
    idx, wt = P.route(z, corr, 3, 4, 2)
    # group bests: .125, .425, .375, -.075 -> groups 1 and 2 are kept; among 2, 3, 4, 5 the best three are 2, 5, 4
    assert idx == [2, 5, 4] and torch.allclose(wt, torch.full((3,), 0.125, dtype=torch.float64))
    # all choice scores negative: losers of the group round must not come back as zeros
    idx, _ = P.route(z, corr - 1.0, 3, 4, 2)
    assert idx == [2, 5, 4]
    # weights are the plain scores, not renormalised
    z = torch.tensor([2.0, 1.0, 0.0, -1.0], dtype=torch.float64)
    idx, wt = P.route(z, torch.zeros(4, dtype=torch.float64), 2, 1, 1)
    s = torch.softmax(z, 0)
    assert idx == [0, 1] and torch.allclose(wt, s[:2]) and float(wt.sum()) < 1


def test_rotation_by_hand():
    t = torch.zeros(3, 1, 6, dtype=torch.float64)
    t[:, 0, 0] = 1.0          # pairs (0, 2) and (1, 3) of the first four numbers; 4 and 5 pass
    t[:, 0, 5] = 7.0
    r = P.rotate(t, 100.0, 4)
    for p in range(3):
        assert torch.allclose(r[p, 0], torch.tensor([torch.cos(torch.tensor(float(p))), 0.0, torch.sin(torch.tensor(float(p))), 0.0, 0.0, 7.0], dtype=torch.float64))
    t = torch.zeros(2, 1, 4, dtype=torch.float64)
    t[:, 0, 1] = 1.0          # second pair turns at 100^(-2/4) = 0.1 rad a position
    r = P.rotate(t, 100.0, 4)
    assert torch.allclose(r[1, 0], torch.tensor([0.0, 0.9950041652780258, 0.0, 0.09983341664682815], dtype=torch.float64))


def test_layer_by_hand():
    """One token, one head, zero biases and unit norms: attention returns Wo k, the layer is norm(a x + ls * that)."""
    cfg = {"architecture": "Monolix", "vocab": 5, "width": 8, "norm": {"eps": 0.0}, "postln_alpha": 2.0,
           "layers": [layer(att(1, 1, 8, 0, scale=1.0), None)]}
    w = {k: v.double() for k, v in make_weights(cfg, 1).items()}
    x = w["embed"][3]
    k = w["l0.mix.k"] @ x + w["l0.mix.k.b"]
    u = 2.0 * x + w["l0.ls1"] * (w["l0.mix.o"] @ k)
    u = u / u.pow(2).mean().sqrt() * (1 + w["l0.norm1"])
    u = u / u.pow(2).mean().sqrt() * (1 + w["final.norm"])
    assert torch.allclose(P.forward(cfg, w, [3])[0], w["head"] @ u, atol=1e-12)


def test_every_mechanism_shows_in_the_test_weights():
    """Knocking a mechanism out of the oracle's inputs moves the logits far beyond the tolerances: biases, the
    router's correction, layer scales, one-plus norm weights, head norm weights, the skip scale."""
    for name in CONFIGS:
        cfg = CONFIGS[name]
        w = make_weights(cfg, SEEDS[name])
        tokens = random_tokens(40, cfg["vocab"], 2)
        ref = plain_of(cfg, w, tokens)
        knock = {"bias": (lambda n: n.endswith(".b"), 0.0), "correction": (lambda n: n.endswith(".correction"), 0.0),
                 "layer scale": (lambda n: ".ls" in n, 1.0), "norm": (lambda n: n.endswith("norm1") or n == "final.norm", 0.0),
                 "head norm": (lambda n: n.endswith(".k.norm"), 1.0)}
        for what, (pick, value) in knock.items():
            if what == "correction" and name == "R":
                continue                                     # one kept group of two with top 2: nothing to choose
            w2 = {k: (torch.full_like(v, value) if pick(k) else v) for k, v in w.items()}
            assert float(row_error(plain_of(cfg, w2, tokens), ref).median()) > 1e-2, (name, what)
        c2 = copy.deepcopy(cfg)
        c2["postln_alpha"] = cfg["postln_alpha"] + 1.0
        assert float(row_error(plain_of(c2, w, tokens), ref).median()) > 1e-2, (name, "skip scale")


