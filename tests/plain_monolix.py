"""A plain, slow implementation of the Monolix design, one function per mechanism, written from its
equations only.  It shares no code with the package: it reads config.json and the safetensors file
itself and computes whole sequences on the CPU with torch in float32 or float64.

Notation: x is the residual stream [T, width]; h is a sublayer's input (x itself: the design norms
AFTER the sum); a layer is  x <- N1(alpha x + ls1 * mixer(x)),  x <- N2(alpha x + ls2 * ff(x))  with
N(u) = u / sqrt(mean(u^2) + eps) * (1 + w).
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional, Tuple

import torch

_DT = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32, "F64": torch.float64}


def read_model(model_dir: str, dtype: torch.dtype = torch.float32) -> Tuple[dict, Dict[str, torch.Tensor]]:
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    with open(os.path.join(model_dir, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        head = json.loads(f.read(n))
        blob = f.read()
    w = {}
    for name, info in head.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        t = torch.frombuffer(bytearray(blob[a:b]), dtype=_DT[info["dtype"]]).reshape(info["shape"])
        w[name] = t.to(dtype) if t.is_floating_point() else t
    return cfg, w


def weights_layer(cfg: dict, i: int) -> int:
    """The layer whose tensors layer i uses."""
    while cfg["layers"][i].get("weights_of") is not None:
        i = cfg["layers"][i]["weights_of"]
    return i


def rms(u: torch.Tensor, eps: float) -> torch.Tensor:
    return u / torch.sqrt((u * u).mean(-1, keepdim=True) + eps)


def one_plus_norm(u, weight, eps):
    return rms(u, eps) * (1 + weight)


def rotate(t: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """t [T, heads, dim], row p at position p: the first `dims` entries of every head turn, entry i with
    entry i + dims/2 by the angle p * base^(-2i/dims)."""
    T = t.shape[0]
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=torch.float64)
    ang = torch.arange(T, dtype=torch.float64)[:, None] * f[None, :]
    c, s = torch.cos(ang).to(t.dtype)[:, None, :], torch.sin(ang).to(t.dtype)[:, None, :]
    u, v = t[..., :half], t[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, t[..., dims:]], dim=-1)


def attention(h, w, p, m, eps):
    """Grouped-query attention whose values are the keys as projected (before norm and rotation)."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, d)
    v = k
    q = rms(q, eps) * w[p + "q.norm"]
    k = rms(k, eps) * w[p + "k.norm"]
    rot = m.get("rot")
    if rot:
        q, k = rotate(q, rot["base"], rot["dims"]), rotate(k, rot["base"], rot["dims"])
    out = torch.zeros(T, H, d, dtype=h.dtype)
    per = H // G
    for i in range(T):
        for a in range(H):
            g = a // per
            s = (k[:i + 1, g] @ q[i, a]) * m["scale"]
            e = torch.exp(s - s.max())
            out[i, a] = (e / e.sum()) @ v[:i + 1, g]
    return out.reshape(T, H * d) @ w[p + "o"].T


def relu2_expert(h, up, down):
    return (torch.relu(h @ up.T) ** 2) @ down.T


def route(z: torch.Tensor, correction: torch.Tensor, top: int, groups: int, keep: int):
    """z [n] router logits of one token -> (chosen indices, their weights).  Weights are the softmax
    scores; the choice is by score + correction among the experts of the `keep` groups whose best
    choice score is largest."""
    s = torch.softmax(z, dim=-1)
    c = s + correction
    n = z.numel()
    size = n // groups
    best = c.view(groups, size).max(dim=1).values
    kept = torch.topk(best, keep).indices.tolist()
    allowed = torch.full((n,), float("-inf"), dtype=c.dtype)
    for g in kept:
        allowed[g * size:(g + 1) * size] = c[g * size:(g + 1) * size]
    idx = torch.topk(allowed, top).indices
    return idx.tolist(), s[idx]


def moe(h, w, p, mlp):
    r = mlp["router"]
    E, ident, top = r["experts"], r.get("identity", 0), r["top"]
    grp = r.get("groups") or {"count": 1, "keep": 1}
    z = h.to(torch.float32).to(h.dtype) @ w[p + "router"].T
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        idx, wt = route(z[t], w[p + "correction"], top, grp["count"], grp["keep"])
        for e, a in zip(idx, wt):
            if e >= E:                      # an identity expert: the input itself
                out[t] += a * h[t]
            else:
                out[t] += a * relu2_expert(h[t], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"])
    if mlp.get("shared"):
        g = torch.sigmoid(h @ w[p + "shared.sg"].T)         # [T, 1]
        out = out + g * relu2_expert(h, w[p + "shared.up"], w[p + "shared.down"])
    return out


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence."""
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    x = w["embed"][torch.tensor(tokens)]
    for i, L in enumerate(cfg["layers"]):
        j = weights_layer(cfg, i)
        p = f"l{j}."
        y = attention(x, w, p + "mix.", L["mixer"], eps)
        x = one_plus_norm(alpha * x + w[p + "ls1"] * y, w[p + "norm1"], eps)
        if L.get("mlp") is not None:
            y = moe(x, w, p + "mlp.", L["mlp"])
            x = one_plus_norm(alpha * x + w[p + "ls2"] * y, w[p + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x)
    return one_plus_norm(x, w["final.norm"], eps) @ w["head"].T


def greedy_generate(cfg, w, prompt: List[int], n: int) -> List[int]:
    seq, out = list(prompt), []
    for _ in range(n):
        t = int(forward(cfg, w, seq)[-1].argmax())
        out.append(t)
        seq.append(t)
    return out
