"""Typed configuration of the Titedra decoder, read from ``config.json``.

Titedra is a small decoder whose layers put an RMS norm (gain stored around zero: ``1 + w``)
before AND after each branch, ``x + norm_b(branch(norm_a(x)))``.  Every layer's mixer is a latent
attention (:mod:`scratch_llm_b200.parts.latent_attention`: low-rank latents for queries and for
keys/values, one cached vector per token, a rotated key part shared by all heads, an output gate
per head); its feed-forward is a dense SwiGLU, a routed one (sigmoid router with a correction,
groups scored by their two best, weights not renormalised, experts ``W_down relu(W_up h)^2``), or
absent.  ``loop`` runs the layers ``start .. stop - 1`` ``times`` times in a row with the same
tensors, each pass with cache entries of its own; before the first layer of every pass the stream
is replaced by ``W_in [x; x0]`` with the embedding output ``x0``
(:mod:`scratch_llm_b200.parts.stream_join`).  The embedding is multiplied by ``embedding.scale``
and the logits by ``logit_scale``.

config.json::

    {"architecture": "Titedra", "vocab": V, "width": d, "norm": {"eps": e},
     "embedding": {"scale": s}, "logit_scale": t,
     "loop": {"start": a, "stop": b, "times": n},
     "layers": [{"type": "latent_attention",
                 "mixer": {"heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank", "scale",
                           "rot": {"base", "dims"}},
                 "mlp": {"kind": "dense", "ff": f}},
                {..., "mlp": {"kind": "moe", "expert": {"ff"},
                              "router": {"experts", "top", "groups": {"count", "keep"}}}},
                {..., "mlp": null}]}

Tensors: ``embed``, ``head``, ``final.norm``, ``loop.in`` and per layer i ``l<i>.norm1``,
``l<i>.norm1b``, ``l<i>.norm2``, ``l<i>.norm2b``, ``l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,g,o}``
and ``l<i>.mlp.{gate,up,down}`` or ``l<i>.mlp.{router,correction,e<j>.up,e<j>.down}``.
"""

from __future__ import annotations

import copy
import math
from dataclasses import dataclass, field
from typing import Any, Mapping

from .spec import JoinSpec, LayerSpec, ModelSpec, PartSpec, Run

#: the design has no longest position; this bounds the rotary tables and the block tables
#: (config.json may carry another bound as "max_position")
DEFAULT_MAX_POSITION = 1 << 17


def _positive_int(value: Any, what: str) -> int:
    if not isinstance(value, int) or isinstance(value, bool) or value < 1:
        raise ValueError(f"{what} must be a positive integer, got {value!r}")
    return value


def _number(value: Any, what: str) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(value):
        raise ValueError(f"{what} must be a number, got {value!r}")
    return float(value)


@dataclass(frozen=True)
class TitedraConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple[Mapping[str, Any], ...]
    embedding_scale: float = 1.0
    logit_scale: float = 1.0
    loop: Mapping[str, int] | None = None
    max_position: int = DEFAULT_MAX_POSITION
    raw: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)

    architecture = "Titedra"

    def __post_init__(self) -> None:
        _positive_int(self.vocab, "vocab")
        _positive_int(self.width, "width")
        _positive_int(self.max_position, "max_position")
        _number(self.embedding_scale, "embedding.scale")
        _number(self.logit_scale, "logit_scale")
        if not (self.norm_eps >= 0 and math.isfinite(self.norm_eps)):
            raise ValueError(f"norm.eps must not be negative, got {self.norm_eps!r}")
        if not self.layers:
            raise ValueError("layers must list at least one layer")
        for i, layer in enumerate(self.layers):
            self._check_layer(i, layer)
        if self.loop is not None:
            for key in ("start", "stop", "times"):
                if not isinstance(self.loop.get(key), int) or isinstance(self.loop.get(key), bool):
                    raise ValueError(f"loop.{key} must be an integer, got {self.loop.get(key)!r}")
            a, b, n = self.loop["start"], self.loop["stop"], self.loop["times"]
            if not 0 <= a < b <= len(self.layers) or n < 1:
                raise ValueError(f"loop must name a span of layers and a count of at least 1, "
                                 f"got start {a}, stop {b}, times {n} for {len(self.layers)} "
                                 "layers")

    @staticmethod
    def _check_layer(i: int, layer: Mapping[str, Any]) -> None:
        kind, m = layer.get("type"), layer.get("mixer")
        if kind != "latent_attention":
            raise ValueError(f"layer {i}: type must be 'latent_attention', got {kind!r}")
        if not isinstance(m, Mapping):
            raise ValueError(f"layer {i}: 'mixer' must give the mixer's sizes")
        for key in ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank"):
            _positive_int(m.get(key), f"layer {i}: mixer.{key}")
        _number(m.get("scale"), f"layer {i}: mixer.scale")
        rot = m.get("rot")
        if not isinstance(rot, Mapping):
            raise ValueError(f"layer {i}: mixer.rot must give the rotation's base and dims")
        dims = _positive_int(rot.get("dims"), f"layer {i}: mixer.rot.dims")
        if dims % 2 or dims > m["rot_dim"]:
            raise ValueError(f"layer {i}: rot.dims must be even and at most rot_dim")
        if not _number(rot.get("base"), f"layer {i}: mixer.rot.base") > 0:
            raise ValueError(f"layer {i}: rot.base must be positive")
        mlp = layer.get("mlp")
        if mlp is None:
            return
        if mlp.get("kind") == "dense":
            _positive_int(mlp.get("ff"), f"layer {i}: mlp.ff")
        elif mlp.get("kind") == "moe":
            r = mlp.get("router") or {}
            _positive_int(r.get("experts"), f"layer {i}: mlp.router.experts")
            _positive_int(r.get("top"), f"layer {i}: mlp.router.top")
            _positive_int((mlp.get("expert") or {}).get("ff"), f"layer {i}: mlp.expert.ff")
            groups = r.get("groups")
            if groups is not None:
                _positive_int(groups.get("count"), f"layer {i}: mlp.router.groups.count")
                _positive_int(groups.get("keep"), f"layer {i}: mlp.router.groups.keep")
        else:
            raise ValueError(f"layer {i}: mlp.kind must be 'dense' or 'moe', "
                             f"got {mlp.get('kind')!r}")

    # -- config.json ---------------------------------------------------------------------

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "TitedraConfig":
        missing = [k for k in ("vocab", "width", "layers") if k not in raw]
        if missing:
            raise ValueError(f"config.json lacks required keys: {', '.join(missing)}")
        loop = raw.get("loop")
        return cls(vocab=raw["vocab"], width=raw["width"],
                   norm_eps=_number((raw.get("norm") or {}).get("eps", 0.0), "norm.eps"),
                   layers=tuple(copy.deepcopy(dict(layer)) for layer in raw["layers"]),
                   embedding_scale=(raw.get("embedding") or {}).get("scale", 1.0),
                   logit_scale=raw.get("logit_scale", 1.0),
                   loop=None if loop is None else dict(loop),
                   max_position=raw.get("max_position", DEFAULT_MAX_POSITION),
                   raw=copy.deepcopy(dict(raw)))

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab,
                               "width": self.width, "norm": {"eps": self.norm_eps},
                               "embedding": {"scale": self.embedding_scale},
                               "logit_scale": self.logit_scale,
                               "layers": [copy.deepcopy(dict(layer)) for layer in self.layers]}
        if self.loop is not None:
            out["loop"] = dict(self.loop)
        if self.max_position != DEFAULT_MAX_POSITION:
            out["max_position"] = self.max_position
        return out

    @property
    def vocab_size(self) -> int:
        return self.vocab

    # -- layers as data ------------------------------------------------------------------

    def run_layers(self) -> list[tuple[int, bool]]:
        """The layers in the order they run, each with whether a pass of the loop starts there
        (the stream is joined with the embedding output right before it)."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, False) for i in range(n)]
        a, b, times = self.loop["start"], self.loop["stop"], self.loop["times"]
        order = [(i, False) for i in range(a)]
        for _ in range(times):
            order += [(i, i == a) for i in range(a, b)]
        return order + [(i, False) for i in range(b, n)]

    def _mixer(self, m: Mapping[str, Any]) -> tuple[PartSpec, PartSpec]:
        mixer = PartSpec("latent_attention", {
            "hidden_size": self.width, "n_heads": m["heads"], "dim": m["dim"],
            "rot_dim": m["rot_dim"], "value_dim": m["vdim"], "q_rank": m["q_rank"],
            "kv_rank": m["kv_rank"], "scale": float(m["scale"]), "eps": self.norm_eps,
            "gate": True})
        position = PartSpec("rotary", {
            "head_dim": m["rot_dim"] + m["rot_dim"] % 2, "theta": float(m["rot"]["base"]),
            "max_position": self.max_position, "interleaved": False,
            "rot_dims": m["rot"]["dims"]})
        return mixer, position

    def _feed_forward(self, mlp: Mapping[str, Any]) -> PartSpec:
        if mlp["kind"] == "dense":
            return PartSpec("swiglu", {"hidden_size": self.width, "intermediate_size": mlp["ff"],
                                       "names": {"gate": "gate", "up": "up", "down": "down"}})
        r = mlp["router"]
        groups = r.get("groups") or {"count": 1, "keep": 1}
        return PartSpec("routed_experts", {
            "hidden_size": self.width, "expert_size": mlp["expert"]["ff"],
            "experts": r["experts"], "top": r["top"], "groups": groups["count"],
            "keep_groups": groups["keep"], "score": "sigmoid", "group_score": "top2",
            "renormalize": False, "expert": "sqrelu"})

    def model_spec(self) -> ModelSpec:
        norm = PartSpec("rmsnorm", {"size": self.width, "eps": self.norm_eps, "name": "",
                                    "offset": 1.0})
        names = {"mixer": "mix", "mixer_norm": "norm1", "mixer_out_norm": "norm1b",
                 "feed_forward": "mlp", "feed_forward_norm": "norm2",
                 "feed_forward_out_norm": "norm2b"}
        layers = []
        for i, layer in enumerate(self.layers):
            mixer, position = self._mixer(layer["mixer"])
            parts = {"mixer": mixer, "mixer_norm": norm, "mixer_out_norm": norm,
                     "position": position}
            if layer.get("mlp") is not None:
                parts["feed_forward"] = self._feed_forward(layer["mlp"])
                parts["feed_forward_norm"] = parts["feed_forward_out_norm"] = norm
            layers.append(LayerSpec(f"l{i}", "sandwich", parts, names))
        runs = self.run_layers()
        joins = ()
        if any(starts for _, starts in runs):
            joins = (JoinSpec(PartSpec("concat_linear", {"size": self.width, "name": ""}),
                              "loop.in"),)
        order = tuple(Run(layer=i, cache=c, join=0 if starts else None)
                      for c, (i, starts) in enumerate(runs))
        return ModelSpec(
            hidden_size=self.width, vocab_size=self.vocab, max_position=self.max_position,
            layers=tuple(layers), order=order, final_norm=norm, embed_name="embed",
            final_norm_name="final.norm", lm_head_name="head", tie_embeddings=False,
            embedding_multiplier=float(self.embedding_scale),
            logit_scale=float(self.logit_scale), joins=joins)
