"""The Dedutar configuration: its keys, the run order, the parts it names, the tensors it expects (CPU)."""
import copy

import pytest
import torch

from dedutar_configs import CONFIGS, make_weights
from dlgo_b200.config import ConfigError, DedutarConfig, config_from_dict
from dlgo_b200.engine.model import CausalLM

import plain_dedutar as P


def test_chosen_by_name_under_either_key():
    c = config_from_dict(CONFIGS["P"])
    assert isinstance(c, DedutarConfig)
    d = dict(CONFIGS["P"])
    d["architectures"] = [d.pop("architecture")]
    assert isinstance(config_from_dict(d), DedutarConfig)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_run_order_and_round_trip(name):
    cfg = CONFIGS[name]
    c = config_from_dict(cfg)
    assert c.run_order() == P.run_order(cfg)
    spec = c.architecture_spec()
    assert [e.layer for e in spec.order] == P.run_order(cfg)
    assert all(e.cache_of is None for e in spec.order)          # every pass keeps its own cache
    assert spec.streams == cfg["streams"]
    again = config_from_dict(c.to_dict())
    assert again == c


def test_loop_shapes():
    base = copy.deepcopy(CONFIGS["P"])
    for loop, want in ((None, [0, 1, 2, 3, 4]), ({"start": 0, "stop": 5, "times": 2}, [0, 1, 2, 3, 4] * 2),
                       ({"start": 4, "stop": 5, "times": 3}, [0, 1, 2, 3, 4, 4, 4]),
                       ({"start": 2, "stop": 2, "times": 4}, [0, 1, 2, 3, 4]),
                       ({"start": 0, "stop": 2, "times": 1}, [0, 1, 2, 3, 4])):
        base["loop"] = loop
        assert config_from_dict(base).run_order() == want == P.run_order(base)


def test_parts_carry_the_constants():
    spec = config_from_dict(CONFIGS["P"]).architecture_spec()
    l0, l1, l2 = spec.layers[0], spec.layers[1], spec.layers[2]
    assert l0.mixer.kind == "latent_attention" and l0.mixer.params["window"] == 7 and l0.mixer.params["q_rank"] == 40
    assert not l0.mixer.params["sink"]
    assert l1.mixer.kind == "lightning_attention" and tuple(l1.mixer.params["decay"]) == (0.9, 0.5)
    assert l2.mixer.kind == "latent_attention" and l2.mixer.params["sink"] and l2.mixer.params["window"] is None
    assert l2.mixer.params["q_rank"] is None and l2.ffn is None and set(l2.norms) == {"mixer_norm"}
    assert l0.ffn.kind == "relu2_mlp" and l0.ffn.params["intermediate_size"] == 160
    assert l0.block == "hyper_prenorm" and set(l0.connections) == {"mixer_conn", "ffn_conn"}
    assert spec.final_norm.kind == "dynamic_tanh"


def test_expected_tensors_and_cache_needs():
    cfg = CONFIGS["P"]
    model = CausalLM(config_from_dict(cfg).architecture_spec())
    exp = model.expected_tensors()
    assert tuple(exp["l0.mix.dq"].shape) == (40, 96) and tuple(exp["l0.mix.uq"].shape) == (48, 40)
    assert tuple(exp["l0.mix.uv"].shape) == (72, 48) and tuple(exp["l0.mix.dkv.norm"].shape) == (48,)
    assert tuple(exp["l2.mix.sink"].shape) == (2,) and tuple(exp["l2.mix.q"].shape) == (48, 96)
    assert tuple(exp["l1.mix.g"].shape) == (80, 96) and tuple(exp["l1.mix.norm"].shape) == (80,)
    assert tuple(exp["l0.hc1.mix"].shape) == (3, 3) and tuple(exp["l0.norm1.alpha"].shape) == ()
    assert "l2.norm2" not in exp and "l2.mlp.up" not in exp and "l2.hc2.in" not in exp
    assert tuple(exp["l0.mlp.up.b"].shape) == (160,) and tuple(exp["final.norm.b"].shape) == (96,)
    assert set(make_weights(cfg, 0)) == set(exp)
    needs, borrows, states = model.cache_needs()
    order = P.run_order(cfg)
    for i, layer in enumerate(order):
        kind = cfg["layers"][layer]["type"]
        if kind == "lightning":
            m = cfg["layers"][layer]["mixer"]
            assert needs[i] is None and states[i].shape == (m["heads"], m["dim"], m["vdim"])
            assert states[i].dtype == torch.float32
        else:
            m = cfg["layers"][layer]["mixer"]
            assert needs[i].head_dim == m["kv_rank"] and needs[i].num_kv_heads == 1 and needs[i].planes == 1
            assert needs[i].window == (m["mask"]["size"] if "mask" in m else None) and i not in states


@pytest.mark.parametrize("change, match", [
    (lambda d: d["layers"][0].__setitem__("type", "attention"), "type"),
    (lambda d: d["layers"][1]["mixer"].__setitem__("decay", [0.5]), "decay"),
    (lambda d: d["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda d: d["layers"][0]["mixer"].pop("mask"), "mask"),
    (lambda d: d["layers"][0]["mixer"].pop("q_rank"), "q_rank"),
    (lambda d: d["layers"][0].__setitem__("mlp", {"kind": "experts", "ff": 8}), "dense"),
    (lambda d: d.__setitem__("loop", {"start": 3, "stop": 2, "times": 2}), "loop"),
    (lambda d: d.__setitem__("streams", 0), "streams"),
    (lambda d: d.pop("norm"), "norm"),
    (lambda d: d.pop("width"), "width"),
])
def test_refusals(change, match):
    d = copy.deepcopy(CONFIGS["P"])
    change(d)
    with pytest.raises(ConfigError, match=match):
        config_from_dict(d)


def test_plain_mechanisms_agree_with_direct_formulas():
    """The oracle's own pieces against formulas written out once more by hand, on tiny inputs."""
    torch.manual_seed(0)
    x = torch.randn(5, 6, dtype=torch.float64)
    assert torch.allclose(P.rms(x, 1e-3), x / (x.pow(2).mean(-1, keepdim=True) + 1e-3).sqrt())
    # a sublayer on streams with read = 1/s, mix = I, write = 1 and s equal streams is the plain residual sum
    X = x[None].repeat(3, 1, 1)
    w = {"p.in": torch.full((3,), 1 / 3, dtype=torch.float64), "p.mix": torch.eye(3, dtype=torch.float64),
         "p.out": torch.ones(3, dtype=torch.float64)}
    Y = P.hyper_sublayer(X, w, "p.", lambda u: 2 * u)
    assert torch.allclose(Y, 3 * X)
    # lightning attention with decay 1 is causal linear attention: o_t = sum_{j<=t} (q_t . k_j) v_j
    h = torch.randn(7, 4, dtype=torch.float64)
    ws = {"m.q": torch.randn(6, 4, dtype=torch.float64), "m.k": torch.randn(6, 4, dtype=torch.float64),
          "m.v": torch.randn(10, 4, dtype=torch.float64), "m.g": torch.zeros(10, 4, dtype=torch.float64),
          "m.norm": torch.ones(10, dtype=torch.float64), "m.o": torch.eye(10, dtype=torch.float64)}
    got = P.lightning(h, ws, "m.", {"heads": 2, "dim": 3, "vdim": 5, "decay": [1.0, 1.0]}, 0.0)
    q, k, v = (P.silu(h @ ws[n].T) for n in ("m.q", "m.k", "m.v"))
    o = torch.zeros(7, 10, dtype=torch.float64)
    for a in range(2):
        s = torch.tril(q[:, 3 * a:3 * a + 3] @ k[:, 3 * a:3 * a + 3].T)
        o[:, 5 * a:5 * a + 5] = s @ v[:, 5 * a:5 * a + 5]
    assert torch.allclose(got, P.rms(o, 0.0) * 0.5)
