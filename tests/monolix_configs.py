"""Small Monolix configurations with weights of a useful size, and helpers that run the engine and the plain
implementation on them.  The configurations differ from one another in every size, and include values that
are 1 (one kv head, one expert chosen, one group) or absent (no identity experts, no shared expert, no groups,
no rotation, a layer without feed-forward) and values that models often make equal but that need not be."""
from __future__ import annotations

import functools
import json
import os
from typing import Dict, List, Optional, Sequence

import torch


def att(heads, kv, dim, rot_dims, base=10000.0, scale=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": scale if scale is not None else dim ** -0.5}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
    return m


def moe(ff, experts, identity, top, count, keep, shared):
    r = {"experts": experts, "identity": identity, "top": top}
    if count:
        r["groups"] = {"count": count, "keep": keep}
    m = {"kind": "moe", "expert": {"ff": ff}, "router": r}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def layer(mixer, mlp, weights_of=None):
    L = {"type": "attention", "mixer": mixer, "mlp": mlp}
    if weights_of is not None:
        L["weights_of"] = weights_of
    return L


_A = att(6, 3, 24, 12, base=5000.0, scale=0.3)
_A_mlp = moe(40, 6, 2, 3, 4, 2, 56)
_B1 = att(4, 4, 16, 16, scale=0.4)
_B2 = att(5, 1, 40, 8, base=777.0, scale=0.2)
_C = att(4, 2, 64, 32, base=100000.0)
_Cm = moe(64, 8, 0, 2, 2, 1, 32)

CONFIGS: Dict[str, dict] = {
    # layers 1 and 3 run with layer 0's tensors (caches of their own), layer 2 has its own and no feed-forward;
    # identity experts, groups, a shared expert; partial rotation; heads of 24
    "P": {"architecture": "Monolix", "vocab": 150, "width": 72, "norm": {"eps": 1e-5}, "postln_alpha": 1.7,
          "layers": [layer(_A, _A_mlp), layer(_A, _A_mlp, 0), layer(att(3, 1, 32, 0, scale=0.25), None),
                     layer(_A, _A_mlp, 1)]},
    # every layer its own sizes: as many kv heads as heads with the whole head rotated; one kv head with heads of
    # 40; top 1 without groups, identity experts or shared expert; all router outputs but one are identities
    "Q": {"architecture": "Monolix", "vocab": 97, "width": 48, "norm": {"eps": 1e-6}, "postln_alpha": 1.0,
          "layers": [layer(_B1, moe(24, 5, 0, 1, 0, 0, None)), layer(_B2, moe(16, 1, 3, 2, 2, 2, 24)),
                     layer(_B1, moe(24, 5, 0, 1, 0, 0, None), 0)]},
    # heads of 64 (the tensor-core attention kernels in bfloat16), one kept group of two, width 128
    "R": {"architecture": "Monolix", "vocab": 260, "width": 128, "norm": {"eps": 1e-6}, "postln_alpha": 3.0,
          "layers": [layer(_C, _Cm), layer(_C, _Cm, 0), layer(_C, _Cm, 0)]},
}
SEEDS = {"P": 21, "Q": 22, "R": 23}


def make_weights(cfg: dict, seed: int, sharpen: float = 3.0, tensors: Optional[dict] = None,
                 mild: bool = False) -> Dict[str, torch.Tensor]:
    """Weights (bfloat16) for the tensors the package expects of this configuration: matrices ~ N(0, 1/in), the
    embedding N(0, 1), norm weights stored around zero, head norm weights and layer scales near 1, biases and
    corrections of visible size.  Head norm weights are multiplied by ``sharpen`` so that the softmax is far
    from uniform and a wrong, missing or extra key moves the logits; routers are scaled up so that choices
    are not near ties.  ``mild`` (whole models in bfloat16): a router's near tie that rounding tips the other way
    swaps an expert, and through peaked attention that one token moves every later row of its sequence as far as
    a fault would; mild weights have flatter softmaxes, flatter routers and a feed-forward that weighs a third,
    so that such a swap stays one row's affair (float32 runs and the kernels' own tests carry the sharp cases)."""
    if mild:
        sharpen = 1.5
    from dlgo_b200.config import config_from_dict
    from dlgo_b200.engine.model import CausalLM
    g = torch.Generator().manual_seed(seed)
    expected = tensors or CausalLM(config_from_dict(cfg).architecture_spec()).expected_tensors()
    w = {}
    for name in sorted(expected):
        shape = tuple(expected[name].shape)
        r = torch.randn(shape, generator=g)
        if name == "embed":
            t = r
        elif name.endswith(".q.norm") or name.endswith(".k.norm"):
            t = (1.0 + 0.2 * r) * sharpen ** 0.5
        elif name.endswith(".correction"):
            t = 0.15 * r
        elif name.endswith(".b"):
            t = 0.3 * r
        elif ".ls" in name:
            t = (1.0 + 0.3 * r) * (0.3 if mild and name.endswith("ls2") else 1.0)
        elif "norm" in name:
            t = 0.2 * r                             # stored around zero: the norm multiplies by 1 + w
        elif name.endswith(".router"):
            t = (1.0 if mild else 3.0) * r / shape[1] ** 0.5
        else:
            t = r / shape[1] ** 0.5
        w[name] = t.to(torch.bfloat16)
    return w


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
    import plain_monolix as P
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


# A wrong, missing or extra key, a wrong expert or a lost bias moves a row by 0.1 to 1 on this measure; float32
# rounding stays below 1e-5 and bfloat16 rounding below 5e-2 through these few layers.  In bfloat16 a router's
# near tie may fall the other way for a single token, which moves that row like a fault: a few rows may differ.
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
    and judged together by :func:`assert_rows`' quantile rule when :meth:`done` is called, since a router's near
    tie that rounding tips the other way moves a single row as far as a fault would move most."""

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
