"""A plain, slow implementation of the Dedutar design, one function per mechanism, written from its
equations only.  It shares no code with the package: it reads config.json and the safetensors file
itself and computes whole sequences on the CPU with torch in float32 or float64.

Notation: h is a sublayer's input [T, width]; X are the residual streams [s, T, width].
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


def run_order(cfg: dict) -> List[int]:
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def dynamic_tanh(x, w, prefix):
    return torch.tanh(w[prefix + ".alpha"] * x) * w[prefix] + w[prefix + ".b"]


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z / (1 + torch.exp(-z))


def feed_forward(h, w, p):
    z = h @ w[p + "up"].T + w[p + "up.b"]
    z = torch.relu(z) ** 2
    return z @ w[p + "down"].T + w[p + "down.b"]


def latent_attention(h, w, p, m, eps, queries_through_latent: bool, window: Optional[int], sink: bool):
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    if queries_through_latent:
        cq = rms(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
        q = cq @ w[p + "uq"].T
    else:
        q = h @ w[p + "q"].T
    c = rms(h @ w[p + "dkv"].T, eps) * w[p + "dkv.norm"]
    k = (c @ w[p + "uk"].T).view(T, H, dk)
    v = (c @ w[p + "uv"].T).view(T, H, dv)
    q = q.view(T, H, dk)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for i in range(T):
        lo = 0 if window is None else max(0, i - window + 1)
        for a in range(H):
            s = (k[lo:i + 1, a] @ q[i, a]) * m["scale"]
            mx = s.max()
            if sink:
                mx = torch.maximum(mx, w[p + "sink"][a])
            e = torch.exp(s - mx)
            den = e.sum()
            if sink:
                den = den + torch.exp(w[p + "sink"][a] - mx)
            out[i, a] = (e / den) @ v[lo:i + 1, a]
    return out.reshape(T, H * dv) @ w[p + "o"].T


def lightning(h, w, p, m, eps):
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).view(T, H, dk)
    k = silu(h @ w[p + "k"].T).view(T, H, dk)
    v = silu(h @ w[p + "v"].T).view(T, H, dv)
    decay = torch.tensor(m["decay"], dtype=h.dtype)
    S = torch.zeros(H, dk, dv, dtype=h.dtype)
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        S = decay[:, None, None] * S + k[t, :, :, None] * v[t, :, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    o = rms(o.reshape(T, H * dv), eps) * w[p + "norm"]
    o = o * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def mixer(h, w, layer: int, spec: dict, eps: float):
    p = f"l{layer}.mix."
    m, kind = spec["mixer"], spec["type"]
    if kind == "latent_attention":
        return latent_attention(h, w, p, m, eps, True, m["mask"]["size"], False)
    if kind == "latent_attention_2":
        return latent_attention(h, w, p, m, eps, False, None, True)
    if kind == "lightning":
        return lightning(h, w, p, m, eps)
    raise ValueError(kind)


def hyper_sublayer(X, w, p, fn):
    """X [s, T, d] -> new X: read with `in`, run the sublayer, mix the old streams and add `out` * y."""
    u = torch.einsum("s,std->td", w[p + "in"], X)
    y = fn(u)
    return torch.einsum("sr,std->rtd", w[p + "mix"], X) + w[p + "out"][:, None, None] * y[None]


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens)]
    X = x[None].repeat(cfg["streams"], 1, 1)
    for i in run_order(cfg):
        spec = cfg["layers"][i]
        X = hyper_sublayer(X, w, f"l{i}.hc1.", lambda u: mixer(dynamic_tanh(u, w, f"l{i}.norm1"), w, i, spec, eps))
        if spec["mlp"] is not None:
            X = hyper_sublayer(X, w, f"l{i}.hc2.",
                               lambda u: feed_forward(dynamic_tanh(u, w, f"l{i}.norm2"), w, f"l{i}.mlp."))
        if layers_out is not None:
            layers_out.append(X.sum(0))
    return dynamic_tanh(X.sum(0), w, "final.norm") @ w["head"].T


def greedy_generate(cfg, w, prompt: List[int], n: int) -> List[int]:
    seq, out = list(prompt), []
    for _ in range(n):
        t = int(forward(cfg, w, seq)[-1].argmax())
        out.append(t)
        seq.append(t)
    return out
