"""Small Dedutar configurations with weights of a useful size, and helpers that run the engine and the plain
implementation on them.  The configurations differ from one another in every size, and include values that
are 1 (one stream, one head, a window of one position, one pass) and values that models often make equal
but that need not be (qk size and value size, heads of different layers, ranks)."""
from __future__ import annotations

import functools
import json
import os
from typing import Dict, List, Sequence

import torch


def _lat(heads, dim, vdim, rank, q_rank, window, ff):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "q_rank": q_rank,
                      "scale": dim ** -0.5, "mask": {"size": window}},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _lat2(heads, dim, vdim, rank, ff):
    return {"type": "latent_attention_2",
            "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": 1.3 * dim ** -0.5},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _lin(heads, dim, vdim, decay, ff):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


CONFIGS: Dict[str, dict] = {
    # three streams, the middle two layers run twice, a window that ends inside the first page
    "P": {"architecture": "Dedutar", "vocab": 200, "width": 96, "streams": 3, "norm": {"eps": 1e-5},
          "loop": {"start": 1, "stop": 3, "times": 2},
          "layers": [_lat(3, 16, 24, 48, 40, 7, 160), _lin(2, 16, 40, [0.9, 0.5], 112), _lat2(2, 24, 16, 32, None),
                     _lin(3, 8, 16, [0.999, 0.97, 0.7], None), _lat(2, 8, 8, 24, 16, 33, 64)]},
    # one stream, no loop, one head, a window longer than a page and a window of one position, a layer first
    # that has no feed-forward
    "Q": {"architecture": "Dedutar", "vocab": 131, "width": 64, "streams": 1, "norm": {"eps": 1e-6},
          "loop": None,
          "layers": [_lat2(1, 32, 48, 80, None), _lat(1, 24, 16, 66, 24, 70, 72), _lin(1, 32, 32, [0.98], 96),
                     _lat(4, 8, 16, 16, 8, 1, 48), _lat2(5, 16, 8, 40, 40)]},
    # two streams, the whole model is the loop (three passes), windows at and around the page size
    "R": {"architecture": "Dedutar", "vocab": 90, "width": 48, "streams": 2, "norm": {"eps": 1e-6},
          "loop": {"start": 0, "stop": 3, "times": 3},
          "layers": [_lat(2, 16, 16, 32, 32, 64, 80), _lin(2, 24, 8, [0.8, 0.95], 40), _lat(3, 8, 24, 20, 12, 65, None)]},
}
SEEDS = {"P": 11, "Q": 12, "R": 13}


def make_weights(cfg: dict, seed: int, sharpen: float = 4.0) -> Dict[str, torch.Tensor]:
    """Weights (bfloat16) for the tensors the package expects of this configuration: matrices ~ N(0, 1/in),
    the embedding N(0, 1), norm weights near 1, stream coefficients near the plain residual sum.  Query and
    key up-projections are scaled by ``sharpen`` so that the softmax is far from uniform and a wrong, missing
    or extra key moves the logits; sinks are made comparable to the largest scores."""
    from dlgo_b200.config import config_from_dict
    from dlgo_b200.engine.model import CausalLM
    g = torch.Generator().manual_seed(seed)
    expected = CausalLM(config_from_dict(cfg).architecture_spec()).expected_tensors()
    w = {}
    for name in sorted(expected):
        shape = tuple(expected[name].shape)
        r = torch.randn(shape, generator=g)
        tail = name.split(".", 1)[1] if "." in name else name
        if name == "embed":
            t = r
        elif name.endswith(".alpha"):
            t = 0.8 + 0.2 * r
        elif ".hc" in name and name.endswith(".in"):
            t = 1.0 / shape[0] + 0.3 * r
        elif ".hc" in name and name.endswith(".out"):
            t = 1.0 + 0.3 * r
        elif ".hc" in name and name.endswith(".mix"):
            t = torch.eye(shape[0]) + 0.2 * r
        elif name.endswith(".sink"):
            t = 2.0 + 2.0 * r
        elif name.endswith(".b"):
            t = 0.2 * r
        elif len(shape) == 1:
            t = 1.0 + 0.2 * r                      # norm weights
        else:
            t = r / shape[1] ** 0.5
            if tail in ("mix.uq", "mix.uk") or (tail == "mix.q" and f"{name[:-1]}dkv" in expected):
                t = t * sharpen ** 0.5
        w[name] = t.to(torch.bfloat16)
    return w


def write_model(name: str, out_dir: str, sharpen: float = 4.0) -> str:
    from dlgo_b200.weights import save_tensors
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(CONFIGS[name], f)
    save_tensors(os.path.join(out_dir, "model.safetensors"), make_weights(CONFIGS[name], SEEDS[name], sharpen))
    return out_dir


def random_tokens(n: int, vocab: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


@functools.lru_cache(maxsize=64)
def _plain_cached(model_dir: str, tokens: tuple) -> torch.Tensor:
    import plain_dedutar as P
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


# A wrong, missing or extra key, a lost state or a sink left out moves a row by 0.2 to 1 on this measure; float32
# rounding through up to nine sharpened layers reaches 3e-5, bfloat16 rounding 6e-2.
TOL = {"float32": 1e-4, "bfloat16": 1.2e-1}


def assert_rows(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str) -> None:
    got = got.detach().float().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    e = row_error(got, ref)
    worst = int(e.argmax())
    if dtype == "bfloat16" and e.numel() >= 20:
        # small latents (a dozen numbers) are RMS-normed: where such a vector nearly cancels, bfloat16 rounding
        # of its inputs turns its direction, and a single row moves as far as a fault would move most rows
        assert float(e.median()) <= TOL[dtype] / 4 and float((e > TOL[dtype]).float().mean()) <= 0.1, \
            f"{what}: median {float(e.median()):.3e}, {int((e > TOL[dtype]).sum())} of {e.numel()} rows over {TOL[dtype]:.1e}"
        return
    assert float(e.max()) <= TOL[dtype], f"{what}: row {worst} differs by {float(e.max()):.3e} (allowed {TOL[dtype]:.1e})"
