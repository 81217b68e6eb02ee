"""Typed configuration of the Dedutar design, read from its config.json keys.

A Dedutar model is a list of layers, each a mixer of one of three kinds plus an
optional dense feed-forward, wired through several residual streams
("hyper-connections") with Dynamic-Tanh norms, and a run order in which one
span of layers may repeat with shared weights:

    {"architecture": "Dedutar", "vocab": V, "width": d, "streams": s, "norm": {"eps": e},
     "loop": {"start": a, "stop": b, "times": n},
     "layers": [{"type": "lightning" | "latent_attention" | "latent_attention_2",
                 "mixer": {...sizes and constants of the mixer...},
                 "mlp": null | {"kind": "dense", "ff": f}}, ...]}

Tensor names: ``embed``, ``head``, ``final.norm[.b|.alpha]`` and, for layer i,
``l<i>.norm1|norm2[.b|.alpha]``, ``l<i>.hc1|hc2.in|out|mix``, ``l<i>.mix.*``,
``l<i>.mlp.up|down[.b]``.

Every size and every constant that can differ between two models of the design
comes from the file; constants the design fixes (which norm, which activation,
which mixer kinds exist) are in the parts this description names.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional, Tuple

from .llama import _as, _need, _opt
from .registry import ConfigError, register_architecture
from .spec import ArchitectureSpec, LayerSpec, PartSpec, RunEntry

MIXER_KINDS = ("lightning", "latent_attention", "latent_attention_2")
# The design has no position encoding and names no context limit; the cache's size bounds a sequence.
NO_CONTEXT_LIMIT = 1 << 20


def _obj(d: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}{key!r} must be an object")
    return v


@dataclass(frozen=True)
class DedutarLayer:
    kind: str                           # one of MIXER_KINDS
    mixer: Tuple[Tuple[str, Any], ...]  # the mixer's keys as read, in sorted order (hashable)
    ff: Optional[int]                   # feed-forward width, None for a layer without one

    def m(self) -> Dict[str, Any]:
        return dict(self.mixer)


@dataclass(frozen=True)
class DedutarConfig:
    vocab: int
    width: int
    streams: int
    norm_eps: float
    layers: Tuple[DedutarLayer, ...]
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    architecture: str = "Dedutar"

    # ------------------------------------------------------------------ parsing
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "DedutarConfig":
        layers_in = d.get("layers")
        if not isinstance(layers_in, (list, tuple)) or not layers_in:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers: List[DedutarLayer] = []
        for i, L in enumerate(layers_in):
            where = f"layers[{i}]."
            if not isinstance(L, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = L.get("type")
            if kind not in MIXER_KINDS:
                raise ConfigError(f"config.json: {where}type is {kind!r}; this design has {', '.join(MIXER_KINDS)}")
            m = dict(_obj(L, "mixer", where))
            for key in ("heads", "dim", "vdim"):
                if _need(m, key, int) <= 0:
                    raise ConfigError(f"config.json: {where}mixer.{key} must be positive")
            if kind == "lightning":
                decay = m.get("decay")
                if not isinstance(decay, (list, tuple)) or len(decay) != m["heads"]:
                    raise ConfigError(f"config.json: {where}mixer.decay must list one number per head")
                m["decay"] = tuple(_as(x, "decay", float) for x in decay)
            else:
                if _need(m, "kv_rank", int) <= 0:
                    raise ConfigError(f"config.json: {where}mixer.kv_rank must be positive")
                m["scale"] = _need(m, "scale", float)
                if kind == "latent_attention" and _need(m, "q_rank", int) <= 0:
                    raise ConfigError(f"config.json: {where}mixer.q_rank must be positive")
                mask = m.pop("mask", None)
                if mask is not None:
                    size = _need(_obj({"mask": mask}, "mask", where + "mixer."), "size", int)
                    if size <= 0:
                        raise ConfigError(f"config.json: {where}mixer.mask.size must be positive")
                    m["window"] = size
                elif kind == "latent_attention":
                    raise ConfigError(f"config.json: {where}mixer.mask.size is required for a windowed mixer")
            mlp = L.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: {where}mlp must be null or an object of kind 'dense'")
                ff = _need(mlp, "ff", int)
                if ff <= 0:
                    raise ConfigError(f"config.json: {where}mlp.ff must be positive")
            layers.append(DedutarLayer(kind, tuple(sorted(m.items())), ff))
        n = len(layers)
        loop = d.get("loop")
        a, b, times = 0, 0, 1
        if loop is not None:
            if not isinstance(loop, dict):
                raise ConfigError("config.json: 'loop' must be an object or null")
            a, b, times = _need(loop, "start", int), _need(loop, "stop", int), _need(loop, "times", int)
            if not (0 <= a <= b <= n) or times < 1:
                raise ConfigError(f"config.json: loop {a}..{b} x {times} does not fit {n} layers")
        streams = _opt(d, "streams", int, 1)
        if streams < 1 or streams > 8:
            raise ConfigError(f"config.json: 'streams' must be 1 to 8, got {streams}")
        vocab, width = _need(d, "vocab", int), _need(d, "width", int)
        if vocab <= 0 or width <= 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive")
        return cls(vocab=vocab, width=width, streams=streams,
                   norm_eps=_need(_obj(d, "norm", ""), "eps", float), layers=tuple(layers),
                   loop_start=a, loop_stop=b, loop_times=times,
                   architecture=str(d.get("architecture") or (d.get("architectures") or ["Dedutar"])[0]))

    def to_dict(self) -> Dict[str, Any]:
        layers = []
        for L in self.layers:
            m = L.m()
            if "decay" in m:
                m["decay"] = list(m["decay"])
            if "window" in m:
                m["mask"] = {"size": m.pop("window")}
            layers.append({"type": L.kind, "mixer": m, "mlp": None if L.ff is None else {"kind": "dense", "ff": L.ff}})
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "streams": self.streams,
                "norm": {"eps": self.norm_eps}, "layers": layers,
                "loop": {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}}

    # ------------------------------------------------------- architecture as data
    def run_order(self) -> List[int]:
        """Layer indices in the order they run: the looped span repeats in a row, the rest follow."""
        n = len(self.layers)
        span = list(range(self.loop_start, self.loop_stop))
        return list(range(self.loop_start)) + span * self.loop_times + list(range(self.loop_stop, n))

    def _mixer_spec(self, L: DedutarLayer) -> PartSpec:
        m, d = L.m(), self.width
        if L.kind == "lightning":
            return PartSpec("lightning_attention", {
                "hidden_size": d, "num_heads": m["heads"], "qk_dim": m["dim"], "v_dim": m["vdim"],
                "decay": tuple(m["decay"]), "eps": self.norm_eps,
                "names": {"q": "q", "k": "k", "v": "v", "gate": "g", "out": "o", "norm": "norm"}})
        names = {"kv_down": "dkv", "kv_norm": "dkv.norm", "k_up": "uk", "v_up": "uv", "out": "o"}
        params: Dict[str, Any] = {
            "hidden_size": d, "num_heads": m["heads"], "qk_dim": m["dim"], "v_dim": m["vdim"],
            "kv_rank": m["kv_rank"], "scale": m["scale"], "eps": self.norm_eps, "window": m.get("window"),
            "q_rank": None, "sink": False}
        if L.kind == "latent_attention":
            params["q_rank"] = m["q_rank"]
            names.update({"q_down": "dq", "q_norm": "dq.norm", "q_up": "uq"})
        else:
            params["sink"] = True
            names.update({"q": "q", "sink": "sink"})
        # layers whose needs are equal share one allocation; the window is part of a group's name because a
        # windowed group gives pages back early
        params["cache_group"] = "latent" if params["window"] is None else f"latent_w{params['window']}"
        params["names"] = names
        return PartSpec("latent_attention", params)

    def architecture_spec(self) -> ArchitectureSpec:
        d = self.width
        norm = PartSpec("dynamic_tanh", {"size": d, "names": {"weight": "", "bias": ".b", "alpha": ".alpha"}})
        conn = PartSpec("hyper_connection", {"streams": self.streams,
                                             "names": {"read": "in", "write": "out", "mix": "mix"}})
        layers: List[LayerSpec] = []
        for i, L in enumerate(self.layers):
            norms = {"mixer_norm": norm}
            connections = {"mixer_conn": conn}
            names = {"mixer": "mix.", "mixer_norm": "norm1", "mixer_conn": "hc1."}
            ffn = None
            if L.ff is not None:
                ffn = PartSpec("relu2_mlp", {"hidden_size": d, "intermediate_size": L.ff, "bias": True,
                                             "names": {"up": "up", "up_bias": "up.b", "down": "down",
                                                       "down_bias": "down.b"}})
                norms["ffn_norm"] = norm
                connections["ffn_conn"] = conn
                names.update({"ffn": "mlp.", "ffn_norm": "norm2", "ffn_conn": "hc2."})
            layers.append(LayerSpec(prefix=f"l{i}.", block="hyper_prenorm", mixer=self._mixer_spec(L), ffn=ffn,
                                    norms=norms, names=names, connections=connections))
        spec = ArchitectureSpec(
            name=self.architecture, hidden_size=d, vocab_size=self.vocab, max_positions=NO_CONTEXT_LIMIT,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab, "hidden_size": d, "name": "embed"}),
            embedding_prefix="",
            layers=layers,
            order=[RunEntry(i) for i in self.run_order()],     # every pass of a repeated layer keeps its own cache
            final_norm=norm, final_norm_prefix="final.norm",
            head=PartSpec("linear_head", {"vocab_size": self.vocab, "hidden_size": d, "tied_to": None,
                                          "name": "head"}),
            head_prefix="",
            position_encodings={},
            bos_token_id=None, stop_token_ids=(),
            streams=self.streams,
        )
        spec.validate()
        return spec


register_architecture("Dedutar", DedutarConfig)
