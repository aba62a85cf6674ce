"""Typed configuration of the Tubevik decoder, read from ``config.json``.

Tubevik is a small decoder whose layers have ONE layer norm (gain and offset) in front of a
mixer and a feed-forward that run side by side on its output, ``x + m * (mixer(h) + ff(h))``
with ``h = LN(x)`` and ``m`` = ``residual_mult``.  The embedded tokens pass a layer norm before
the first layer; the logits pass a tanh cap.  ``layers`` lists the layers, each with one of two
mixers:

* ``attention``: grouped-query attention with biases on q, k and v, an RMS norm over the whole
  query projection and over the whole key projection before the rotation, a rotation of halves
  with blended (YaRN) frequencies, a tanh cap on the scores, a sliding window and one sigmoid
  output gate per head (:mod:`scratch_llm_b200.parts.normed_attention`).  With ``kv_from: j``
  the layer has no keys and values of its own and reads layer j's cache entry;
* ``parallel``: two mixers on the same input (:mod:`scratch_llm_b200.parts.side_by_side`):
  ``left``, attention in chunks with a rotation of adjacent pairs on the first ``rot.dims``
  entries of a head, an RMS norm per head after it and a sink of score 0; ``right``, the gated
  delta rule with one decay per key channel through a low-rank pair and a low-rank sigmoid gate
  (:mod:`scratch_llm_b200.parts.delta_rule`).

The feed-forward (``mlp``, or null) is gated with clamps
(:class:`scratch_llm_b200.parts.feed_forward.ClampedGLU`).

config.json::

    {"architecture": "Tubevik", "vocab": V, "width": d, "norm": {"eps": e},
     "residual_mult": m, "logit_softcap": c,
     "layers": [{"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "softcap",
                           "mask": {"size"}, "rot": {"base", "dims", "scaling": {"factor",
                           "original", "fast", "slow"}}, "kv_from": j (optional)},
                 "mlp": {"kind": "dense", "ff": f, "limit": l} | null},
                {"type": "parallel",
                 "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale",
                                    "mask": {"size"}, "rot": {"base", "dims"}},
                           "right": {"heads", "kv_heads", "dim", "vdim", "conv"},
                           "left_scale", "right_scale"}, "mlp": ...}, ...]}

Tensors: ``embed``, ``embed.norm`` (+ ``.b``), ``final.norm`` (+ ``.b``), ``head``, and per layer
i ``l<i>.norm1`` (+ ``.b``), ``l<i>.mix.*`` (``l<i>.mix.left.*`` / ``l<i>.mix.right.*``),
``l<i>.mlp.{gate,up,down}``.
"""

from __future__ import annotations

import copy
import math
from dataclasses import dataclass, field
from typing import Any, Mapping

from .spec import LayerSpec, ModelSpec, PartSpec, Run

#: constants the design fixes
GATE_SLOPE = 1.702           # the feed-forward's gate is g * sigmoid(1.702 g)
YARN_MAGNITUDE = 0.1         # cos and sin are multiplied by 0.1 ln(factor) + 1
#: the design has no longest position; this bounds the engine's block tables and rotary tables
#: (config.json may carry another bound as "max_position")
DEFAULT_MAX_POSITION = 1 << 16


def _positive_int(value: Any, what: str) -> int:
    if not isinstance(value, int) or isinstance(value, bool) or value < 1:
        raise ValueError(f"{what} must be a positive integer, got {value!r}")
    return value


def _number(value: Any, what: str) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(value):
        raise ValueError(f"{what} must be a number, got {value!r}")
    return float(value)


def _positive(value: Any, what: str) -> float:
    if not _number(value, what) > 0:
        raise ValueError(f"{what} must be positive, got {value!r}")
    return float(value)


def _check_heads(m: Mapping[str, Any], where: str) -> None:
    for key in ("heads", "kv_heads", "dim", "vdim"):
        _positive_int(m.get(key), f"{where}.{key}")
    if m["heads"] % m["kv_heads"]:
        raise ValueError(f"{where}: {m['heads']} heads do not group evenly over "
                         f"{m['kv_heads']} kv_heads")


def _check_rotation(rot: Any, dim: int, where: str, scaling: bool) -> None:
    if not isinstance(rot, Mapping):
        raise ValueError(f"{where}.rot must give the rotation's base and dims")
    _positive(rot.get("base"), f"{where}.rot.base")
    dims = _positive_int(rot.get("dims"), f"{where}.rot.dims")
    if dims % 2 or dims > dim:
        raise ValueError(f"{where}.rot.dims must be even and at most dim = {dim}, got {dims}")
    sc = rot.get("scaling")
    if sc is not None:
        if not scaling:
            raise ValueError(f"{where}.rot.scaling: this mixer's rotation has no scaling")
        for key in ("factor", "original", "fast", "slow"):
            _positive(sc.get(key) if isinstance(sc, Mapping) else None,
                      f"{where}.rot.scaling.{key}")


@dataclass(frozen=True)
class TubevikConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    layers: tuple[Mapping[str, Any], ...]
    logit_softcap: float = 0.0
    max_position: int = DEFAULT_MAX_POSITION
    raw: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)

    architecture = "Tubevik"

    def __post_init__(self) -> None:
        _positive_int(self.vocab, "vocab")
        _positive_int(self.width, "width")
        _positive_int(self.max_position, "max_position")
        _positive(self.norm_eps, "norm.eps")
        _number(self.residual_mult, "residual_mult")
        if _number(self.logit_softcap, "logit_softcap") < 0:
            raise ValueError(f"logit_softcap must not be negative, got {self.logit_softcap!r}")
        if not self.layers:
            raise ValueError("layers must list at least one layer")
        for i, layer in enumerate(self.layers):
            self._check_layer(i, layer)

    def _check_layer(self, i: int, layer: Mapping[str, Any]) -> None:
        kind, m = layer.get("type"), layer.get("mixer")
        if kind not in ("attention", "parallel"):
            raise ValueError(f"layer {i}: type must be 'attention' or 'parallel', got {kind!r}")
        if not isinstance(m, Mapping):
            raise ValueError(f"layer {i}: 'mixer' must give the mixer's sizes")
        if kind == "attention":
            self._check_attention(i, m)
        else:
            left, right = m.get("left"), m.get("right")
            if not isinstance(left, Mapping) or not isinstance(right, Mapping):
                raise ValueError(f"layer {i}: a parallel mixer gives 'left' and 'right'")
            where = f"layer {i}: mixer.left"
            _check_heads(left, where)
            _number(left.get("scale"), f"{where}.scale")
            _positive_int((left.get("mask") or {}).get("size"), f"{where}.mask.size")
            _check_rotation(left.get("rot"), left["dim"], where, scaling=False)
            where = f"layer {i}: mixer.right"
            _check_heads(right, where)
            _positive_int(right.get("conv"), f"{where}.conv")
            _number(m.get("left_scale"), f"layer {i}: mixer.left_scale")
            _number(m.get("right_scale"), f"layer {i}: mixer.right_scale")
        mlp = layer.get("mlp")
        if mlp is not None:
            if not isinstance(mlp, Mapping) or mlp.get("kind") != "dense":
                raise ValueError(f"layer {i}: mlp.kind must be 'dense', got "
                                 f"{mlp.get('kind') if isinstance(mlp, Mapping) else mlp!r}")
            _positive_int(mlp.get("ff"), f"layer {i}: mlp.ff")
            _positive(mlp.get("limit"), f"layer {i}: mlp.limit")

    def _check_attention(self, i: int, m: Mapping[str, Any]) -> None:
        where = f"layer {i}: mixer"
        _check_heads(m, where)
        _number(m.get("scale"), f"{where}.scale")
        if m.get("softcap") is not None and not _number(m["softcap"], f"{where}.softcap") >= 0:
            raise ValueError(f"{where}.softcap must not be negative")
        _positive_int((m.get("mask") or {}).get("size"), f"{where}.mask.size")
        _check_rotation(m.get("rot"), m["dim"], where, scaling=True)
        src = m.get("kv_from")
        if src is None:
            return
        if not isinstance(src, int) or isinstance(src, bool) or not 0 <= src < i:
            raise ValueError(f"{where}.kv_from must name an earlier layer, got {src!r}")
        other = self.layers[src]
        if other.get("type") != "attention" or other["mixer"].get("kv_from") is not None:
            raise ValueError(f"{where}.kv_from names layer {src}, which is not an attention layer "
                             "with keys and values of its own")
        o = other["mixer"]
        same = all(o.get(k) == m.get(k) for k in ("heads", "kv_heads", "dim", "vdim")) and \
            dict(o.get("rot") or {}) == dict(m.get("rot") or {})
        if not same:
            raise ValueError(f"{where}: layer {src}, whose keys and values this layer uses, must "
                             "have the same head counts, sizes and rotation")

    # -- config.json ---------------------------------------------------------------------

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "TubevikConfig":
        missing = [k for k in ("vocab", "width", "norm", "layers", "residual_mult")
                   if k not in raw]
        if missing:
            raise ValueError(f"config.json lacks required keys: {', '.join(missing)}")
        return cls(vocab=raw["vocab"], width=raw["width"],
                   norm_eps=_number((raw["norm"] or {}).get("eps"), "norm.eps"),
                   residual_mult=raw["residual_mult"],
                   layers=tuple(copy.deepcopy(dict(layer)) for layer in raw["layers"]),
                   logit_softcap=raw.get("logit_softcap") or 0.0,
                   max_position=raw.get("max_position", DEFAULT_MAX_POSITION),
                   raw=copy.deepcopy(dict(raw)))

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab,
                               "width": self.width, "norm": {"eps": self.norm_eps},
                               "residual_mult": self.residual_mult,
                               "logit_softcap": self.logit_softcap,
                               "layers": [copy.deepcopy(dict(layer)) for layer in self.layers]}
        if self.max_position != DEFAULT_MAX_POSITION:
            out["max_position"] = self.max_position
        return out

    @property
    def vocab_size(self) -> int:
        return self.vocab

    # -- layers as data ------------------------------------------------------------------

    def _rotary(self, m: Mapping[str, Any], interleaved: bool) -> PartSpec:
        rot = m["rot"]
        args: dict[str, Any] = {"head_dim": m["dim"] + m["dim"] % 2, "theta": float(rot["base"]),
                                "max_position": self.max_position, "interleaved": interleaved,
                                "rot_dims": rot["dims"]}
        if rot.get("scaling") is not None:
            args["yarn"] = {k: float(rot["scaling"][k])
                            for k in ("factor", "original", "fast", "slow")}
            args["yarn_magnitude"] = YARN_MAGNITUDE
        return PartSpec("rotary", args)

    def _attention(self, m: Mapping[str, Any]) -> PartSpec:
        return PartSpec("normed_attention", {
            "hidden_size": self.width, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"],
            "head_dim": m["dim"], "value_dim": m["vdim"], "scale": float(m["scale"]),
            "eps": self.norm_eps, "bias": True, "qk_norm": "wide",
            "softcap": float(m.get("softcap") or 0.0), "window": m["mask"]["size"],
            "head_gate": True, "borrow_kv": m.get("kv_from") is not None})

    def _parallel(self, m: Mapping[str, Any]) -> PartSpec:
        left, right = m["left"], m["right"]
        return PartSpec("side_by_side", {
            "left": {"kind": "normed_attention", "args": {
                "hidden_size": self.width, "n_heads": left["heads"],
                "n_kv_heads": left["kv_heads"], "head_dim": left["dim"],
                "value_dim": left["vdim"], "scale": float(left["scale"]), "eps": self.norm_eps,
                "qk_norm": "unit_after", "chunk": left["mask"]["size"], "zero_sink": True}},
            "right": {"kind": "gated_delta_rule", "args": {
                "hidden_size": self.width, "n_heads": right["heads"],
                "n_kv_heads": right["kv_heads"], "key_dim": right["dim"],
                "value_dim": right["vdim"], "conv_taps": right["conv"], "eps": self.norm_eps,
                "decay_rank": -1, "gate_rank": -1, "gate_activation": "sigmoid"}},
            "left_scale": float(m["left_scale"]), "right_scale": float(m["right_scale"])})

    def model_spec(self) -> ModelSpec:
        norm = PartSpec("layernorm", {"size": self.width, "eps": self.norm_eps, "name": ""})
        layers, order = [], []
        entry_of: dict[int, int] = {}       # layer -> the cache entry its run writes
        for i, layer in enumerate(self.layers):
            m = layer["mixer"]
            if layer["type"] == "attention":
                parts = {"mixer": self._attention(m), "position": self._rotary(m, False)}
            else:
                parts = {"mixer": self._parallel(m), "position": self._rotary(m["left"], True)}
            parts["norm"] = norm
            mlp = layer.get("mlp")
            if mlp is not None:
                parts["feed_forward"] = PartSpec("clamped_glu", {
                    "hidden_size": self.width, "intermediate_size": mlp["ff"],
                    "limit": float(mlp["limit"]), "slope": GATE_SLOPE})
            layers.append(LayerSpec(f"l{i}", "shared_norm", parts,
                                    {"mixer": "mix", "norm": "norm1", "feed_forward": "mlp"},
                                    {"residual_mult": float(self.residual_mult)}))
            src = m.get("kv_from") if layer["type"] == "attention" else None
            if src is None:
                entry_of[i] = len(entry_of)
                order.append(Run(layer=i, cache=entry_of[i]))
            else:
                order.append(Run(layer=i, cache=entry_of[src], write=False))
        return ModelSpec(
            hidden_size=self.width, vocab_size=self.vocab, max_position=self.max_position,
            layers=tuple(layers), order=tuple(order), final_norm=norm, embed_name="embed",
            final_norm_name="final.norm", lm_head_name="head", tie_embeddings=False,
            logit_softcap=float(self.logit_softcap), embed_norm=norm,
            embed_norm_name="embed.norm")
