"""Typed configuration of the Monolix design, read from its config.json keys.

A Monolix model is a list of layers that norm AFTER the residual sum, each a grouped-query attention
mixer whose values are its keys as projected, plus an optional mixture-of-experts feed-forward; a layer
may run with the tensors of another layer (earlier or later in the list) while keeping a cache of its own:

    {"architecture": "Monolix", "vocab": V, "width": d, "norm": {"eps": e}, "postln_alpha": a,
     "layers": [{"type": "attention",
                 "mixer": {"heads": H, "kv_heads": G, "dim": n, "vdim": n, "scale": s,
                           "rot": {"base": b, "dims": r}},
                 "mlp": null | {"kind": "moe", "expert": {"ff": f},
                                "router": {"experts": E, "identity": I, "top": k,
                                           "groups": {"count": c, "keep": m}},
                                "shared": {"ff": fs}},
                 "weights_of": j (optional)}, ...]}

Tensor names: ``embed``, ``head``, ``final.norm`` and, for a layer i with tensors of its own,
``l<i>.norm1|norm2``, ``l<i>.ls1|ls2``, ``l<i>.mix.q|k[.b|.norm]``, ``l<i>.mix.o``,
``l<i>.mlp.router|correction``, ``l<i>.mlp.e<j>.up|down``, ``l<i>.mlp.shared.up|down|sg``.

Every size and every constant that can differ between two models of the design comes from the file;
what the design fixes (which norm, which activation, how experts are chosen) is in the parts this
description names.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional, Tuple

from .llama import _as, _need, _opt
from .registry import ConfigError, register_architecture
from .spec import ArchitectureSpec, LayerSpec, PartSpec, RunEntry

MIXER_KINDS = ("attention",)
# The rotation is computed from the position itself and the design names no context limit; the cache's
# size bounds a sequence.
NO_CONTEXT_LIMIT = 1 << 20


def _obj(d: Mapping[str, Any], key: str, where: str, required: bool = True) -> Optional[Mapping[str, Any]]:
    v = d.get(key)
    if v is None and not required:
        return None
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}{key!r} must be an object")
    return v


@dataclass(frozen=True)
class MonolixAttention:
    heads: int
    kv_heads: int
    dim: int
    scale: float
    rot_base: Optional[float]       # None: no rotation
    rot_dims: int


@dataclass(frozen=True)
class MonolixMoE:
    ff: int
    experts: int                    # experts that hold tensors
    identity: int                   # router outputs beyond them whose expert is the input itself
    top: int
    group_count: int
    group_keep: int
    shared_ff: Optional[int]        # None: no shared expert


@dataclass(frozen=True)
class MonolixLayer:
    kind: str
    mixer: MonolixAttention
    mlp: Optional[MonolixMoE]
    weights_of: Optional[int]       # the layer whose tensors this one uses (None: its own)


def _attention(m: Mapping[str, Any], where: str) -> MonolixAttention:
    heads, kv, dim = _need(m, "heads", int), _need(m, "kv_heads", int), _need(m, "dim", int)
    if heads <= 0 or kv <= 0 or dim <= 0 or heads % kv:
        raise ConfigError(f"config.json: {where}heads must be a positive multiple of kv_heads, dim positive")
    vdim = _opt(m, "vdim", int, dim)
    if vdim != dim:
        raise ConfigError(f"config.json: {where}vdim is {vdim} but the values are the keys, of size {dim}")
    rot = _obj(m, "rot", where, required=False)
    base, dims = None, 0
    if rot is not None:
        base, dims = _need(rot, "base", float), _need(rot, "dims", int)
        if dims % 2 or not 0 <= dims <= dim or base <= 0:
            raise ConfigError(f"config.json: {where}rot.dims must be even and at most dim, rot.base positive")
        if dims == 0:
            base = None
    return MonolixAttention(heads, kv, dim, _need(m, "scale", float), base, dims)


def _moe(mlp: Mapping[str, Any], where: str) -> MonolixMoE:
    if mlp.get("kind") != "moe":
        raise ConfigError(f"config.json: {where}kind is {mlp.get('kind')!r}; this design has 'moe' (or null for none)")
    r = _obj(mlp, "router", where)
    experts, ident, top = _need(r, "experts", int), _opt(r, "identity", int, 0), _need(r, "top", int)
    groups = _obj(r, "groups", where + "router.", required=False)
    count, keep = (1, 1) if groups is None else (_need(groups, "count", int), _need(groups, "keep", int))
    n = experts + ident
    if experts < 0 or ident < 0 or n <= 0 or count <= 0 or n % count or not 0 < keep <= count:
        raise ConfigError(f"config.json: {where}router: {experts} + {ident} outputs do not form {count} equal groups "
                          f"of which {keep} are kept")
    if not 0 < top <= keep * (n // count):
        raise ConfigError(f"config.json: {where}router.top is {top}; the kept groups hold {keep * (n // count)}")
    ff = _need(_obj(mlp, "expert", where), "ff", int) if experts else 0
    shared = _obj(mlp, "shared", where, required=False)
    shared_ff = None if shared is None else _need(shared, "ff", int)
    if (experts and ff <= 0) or (shared_ff is not None and shared_ff <= 0):
        raise ConfigError(f"config.json: {where}ff sizes must be positive")
    return MonolixMoE(ff, experts, ident, top, count, keep, shared_ff)


@dataclass(frozen=True)
class MonolixConfig:
    vocab: int
    width: int
    norm_eps: float
    postln_alpha: float
    layers: Tuple[MonolixLayer, ...]
    architecture: str = "Monolix"

    # ------------------------------------------------------------------ parsing
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "MonolixConfig":
        layers_in = d.get("layers")
        if not isinstance(layers_in, (list, tuple)) or not layers_in:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers: List[MonolixLayer] = []
        for i, L in enumerate(layers_in):
            where = f"layers[{i}]."
            if not isinstance(L, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = L.get("type")
            if kind not in MIXER_KINDS:
                raise ConfigError(f"config.json: {where}type is {kind!r}; this design has {', '.join(MIXER_KINDS)}")
            mixer = _attention(_obj(L, "mixer", where), where + "mixer.")
            mlp_in = L.get("mlp")
            if mlp_in is not None and not isinstance(mlp_in, dict):
                raise ConfigError(f"config.json: {where}mlp must be null or an object")
            mlp = None if mlp_in is None else _moe(mlp_in, where + "mlp.")
            of = L.get("weights_of")
            if of is not None:
                of = _as(of, "weights_of", int)
                if not 0 <= of < len(layers_in) or of == i:
                    raise ConfigError(f"config.json: {where}weights_of names layer {of}; it must name another layer")
            layers.append(MonolixLayer(kind, mixer, mlp, of))
        # a chain of weights_of ends at the layer that holds the tensors (which may come later in the file)
        for i, L in enumerate(layers):
            of, seen = L.weights_of, {i}
            while of is not None and layers[of].weights_of is not None:
                if of in seen:
                    raise ConfigError(f"config.json: layers[{i}].weights_of runs in a circle")
                seen.add(of)
                of = layers[of].weights_of
            if of is not None:
                if of in seen:
                    raise ConfigError(f"config.json: layers[{i}].weights_of runs in a circle")
                if (layers[of].mixer, layers[of].mlp) != (L.mixer, L.mlp):
                    raise ConfigError(f"config.json: layers[{i}] uses the tensors of layer {of} but its sizes differ")
                layers[i] = MonolixLayer(L.kind, L.mixer, L.mlp, of)
        vocab, width = _need(d, "vocab", int), _need(d, "width", int)
        if vocab <= 0 or width <= 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive")
        return cls(vocab=vocab, width=width, norm_eps=_need(_obj(d, "norm", ""), "eps", float),
                   postln_alpha=_opt(d, "postln_alpha", float, 1.0), layers=tuple(layers),
                   architecture=str(d.get("architecture") or (d.get("architectures") or ["Monolix"])[0]))

    def to_dict(self) -> Dict[str, Any]:
        layers = []
        for L in self.layers:
            a = L.mixer
            m: Dict[str, Any] = {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.dim, "scale": a.scale}
            if a.rot_base is not None:
                m["rot"] = {"base": a.rot_base, "dims": a.rot_dims}
            mlp = None
            if L.mlp is not None:
                e = L.mlp
                mlp = {"kind": "moe", "expert": {"ff": e.ff},
                       "router": {"experts": e.experts, "identity": e.identity, "top": e.top,
                                  "groups": {"count": e.group_count, "keep": e.group_keep}}}
                if e.shared_ff is not None:
                    mlp["shared"] = {"ff": e.shared_ff}
            entry: Dict[str, Any] = {"type": L.kind, "mixer": m, "mlp": mlp}
            if L.weights_of is not None:
                entry["weights_of"] = L.weights_of
            layers.append(entry)
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "postln_alpha": self.postln_alpha, "layers": layers}

    # ------------------------------------------------------- architecture as data
    def _mixer_spec(self, a: MonolixAttention) -> Tuple[PartSpec, Optional[str]]:
        pe = None if a.rot_base is None else f"rotary_{a.rot_dims}_{a.rot_base!r}"
        return PartSpec("keys_as_values_attention", {
            "hidden_size": self.width, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim,
            "scale": a.scale, "bias": True, "head_norm": True, "eps": self.norm_eps, "position_encoding": pe,
            "cache_group": "full",
            "names": {"q": "q", "k": "k", "q_bias": "q.b", "k_bias": "k.b", "q_norm": "q.norm", "k_norm": "k.norm",
                      "out": "o"}}), pe

    def _ffn_spec(self, e: MonolixMoE) -> PartSpec:
        return PartSpec("routed_experts", {
            "hidden_size": self.width, "intermediate_size": e.ff, "num_experts": e.experts,
            "identity_experts": e.identity, "top": e.top, "group_count": e.group_count, "group_keep": e.group_keep,
            "score": "softmax", "renormalize": False, "correction": True, "activation": "relu2",
            "shared_size": e.shared_ff, "shared_gate": True,
            "names": {"router": "router", "correction": "correction", "expert": "e{}.", "up": "up", "down": "down",
                      "shared_up": "shared.up", "shared_down": "shared.down", "shared_gate": "shared.sg"}})

    def architecture_spec(self) -> ArchitectureSpec:
        d = self.width
        norm = PartSpec("rmsnorm", {"size": d, "eps": self.norm_eps, "one_plus": True, "name": ""})
        scale = PartSpec("layer_scale", {"size": d, "skip_scale": self.postln_alpha, "name": ""})
        layers: List[LayerSpec] = []
        place: Dict[int, int] = {}          # layer of the file -> index among the layers that hold tensors
        positions: Dict[str, PartSpec] = {}
        order: List[RunEntry] = []
        for i, L in enumerate(self.layers):
            if L.weights_of is not None:
                continue
            mixer, pe = self._mixer_spec(L.mixer)
            if pe is not None:
                positions[pe] = PartSpec("rotary_frequencies", {"head_dim": L.mixer.dim, "rotary_dim": L.mixer.rot_dims,
                                                                "theta": L.mixer.rot_base})
            norms = {"mixer_norm": norm}
            connections = {"mixer_conn": scale}
            names = {"mixer": "mix.", "mixer_norm": "norm1", "mixer_conn": "ls1"}
            ffn = None
            if L.mlp is not None:
                ffn = self._ffn_spec(L.mlp)
                norms["ffn_norm"] = norm
                connections["ffn_conn"] = scale
                names.update({"ffn": "mlp.", "ffn_norm": "norm2", "ffn_conn": "ls2"})
            place[i] = len(layers)
            layers.append(LayerSpec(prefix=f"l{i}.", block="postnorm", mixer=mixer, ffn=ffn, norms=norms,
                                    names=names, connections=connections))
        # every layer of the file is one run entry: shared tensors, a cache of its own
        order = [RunEntry(place[i if L.weights_of is None else L.weights_of]) for i, L in enumerate(self.layers)]
        spec = ArchitectureSpec(
            name=self.architecture, hidden_size=d, vocab_size=self.vocab, max_positions=NO_CONTEXT_LIMIT,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": d, "name": "embed"}),
            embedding_prefix="",
            layers=layers, order=order,
            final_norm=norm, final_norm_prefix="final.norm",
            head=PartSpec("linear_head", {"vocab_size": self.vocab, "hidden_size": d, "tied_to": None,
                                          "name": "head"}),
            head_prefix="",
            position_encodings=positions,
            bos_token_id=None, stop_token_ids=(),
        )
        spec.validate()
        return spec


register_architecture("Monolix", MonolixConfig)
