"""Two mixers side by side on the same input: ``left_scale * Left(x) + right_scale * Right(x)``.

Each side is any registered mixer, named by its kind and arguments; its tensors live below the
sub-prefixes ``left`` and ``right`` (or as ``names`` says).  A layer has one cache entry, and
this mixer shares it out: paged keys and values for the side that wants them (at most one side
may), per-request state for each side that keeps some (the entry's state tensors are the left
side's followed by the right side's).  Nothing is added here: the result is handed on as a
weighted sum (:class:`~.stream.Terms`) for a block and a norm that take one.
"""

from __future__ import annotations

from typing import Any, Mapping

import torch

from .base import BuildContext, CacheView, KVSpec, Mixer, PositionEncoding
from .registry import MIXERS, register_mixer
from .stream import Terms


def _as_tuple(v) -> tuple:
    return () if v is None else tuple(v) if isinstance(v, (tuple, list)) else (v,)


@register_mixer("side_by_side")
class SideBySide(Mixer):
    #: forward() returns a weighted sum of tensors, not a tensor
    returns_terms = True

    def __init__(self, left: Mapping[str, Any], right: Mapping[str, Any], left_scale: float = 1.0,
                 right_scale: float = 1.0, names: Mapping[str, str] | None = None) -> None:
        """``left`` / ``right``: ``{"kind": <a key of MIXERS>, "args": {...}}``."""
        self.sides = []
        for what, spec in (("left", left), ("right", right)):
            kind = spec["kind"]
            if kind not in MIXERS:
                raise ValueError(f"unknown mixer {kind!r} for the {what} side; registered: "
                                 f"{', '.join(sorted(MIXERS))}")
            self.sides.append(MIXERS[kind](**dict(spec.get("args", {}))))
        self.scales = (float(left_scale), float(right_scale))
        self.names = {"left": "left", "right": "right", **(names or {})}
        self.prefixes = (self.names["left"], self.names["right"])
        if sum(side.kv_spec() is not None for side in self.sides) > 1:
            raise ValueError("both sides want paged keys and values: a layer's cache entry has "
                             "one set of pages")

    @property
    def capturable(self) -> bool:
        return all(getattr(side, "capturable", True) for side in self.sides)

    @property
    def pad_safe(self) -> bool:
        return all(getattr(side, "pad_safe", False) for side in self.sides)

    @property
    def head_dim(self):
        return next((side.head_dim for side in self.sides
                     if side.kv_spec() is not None and hasattr(side, "head_dim")), None)

    # ------------------------------------------------------------------------------ cache

    def kv_spec(self) -> KVSpec | None:
        return next((spec for spec in (side.kv_spec() for side in self.sides)
                     if spec is not None), None)

    def state_spec(self):
        specs = sum((_as_tuple(side.state_spec()) for side in self.sides), ())
        return specs or None

    def kernel_jobs(self, dtype: torch.dtype):
        jobs = []
        for side in self.sides:
            if hasattr(side, "kernel_jobs"):
                said = side.kernel_jobs(dtype)
                if said is None:
                    return None
                jobs += said
        return jobs

    # ---------------------------------------------------------------------------- weights

    def param_specs(self):
        return {f"{prefix}.{name}": spec for prefix, side in zip(self.prefixes, self.sides)
                for name, spec in side.param_specs().items()}

    def load(self, tensors: Mapping[str, torch.Tensor], ctx: BuildContext) -> None:
        for prefix, side in zip(self.prefixes, self.sides):
            side.load({name: tensors[f"{prefix}.{name}"] for name in side.param_specs()}, ctx)

    # ---------------------------------------------------------------------------- forward

    def _views(self, cache: CacheView) -> list[CacheView]:
        """What each side sees of the layer's cache entry: the pages for the side that has keys,
        its own share of the state tensors in the form it declared them."""
        states = _as_tuple(cache.state)
        views, at = [], 0
        for side in self.sides:
            declared = side.state_spec()
            n = len(_as_tuple(declared))
            mine = states[at:at + n]
            at += n
            state = None if n == 0 else mine if isinstance(declared, (tuple, list)) else mine[0]
            paged = side.kv_spec() is not None
            views.append(CacheView(pages=cache.pages if paged else None,
                                   block_table=cache.block_table if paged else None,
                                   page_size=cache.page_size, state=state))
        return views

    def forward(self, x, batch, cache: CacheView, write: bool, position: PositionEncoding):
        out = None
        for side, scale, view in zip(self.sides, self.scales, self._views(cache)):
            term = Terms.of(side.forward(x, batch, view, write, position), scale)
            out = term if out is None else out + term
        return out

    # -- for a block that multiplies several branches' activations by one joined output matrix

    def out_segments(self):
        """Both sides' output matrices, each with its side's weight in the sum; None if a side
        cannot hand out its activations."""
        segments = []
        for side, scale in zip(self.sides, self.scales):
            if not hasattr(side, "out_segments"):
                return None
            mine = side.out_segments()
            if mine is None:
                return None
            if len(mine) != 1:
                return None
            segments += [(w, c * scale) for w, c in mine]
        return segments

    def release_out(self) -> None:
        for side in self.sides:
            side.release_out()

    def activations_into(self, x, batch, cache: CacheView, write: bool, position, outs) -> None:
        for i, (side, view) in enumerate(zip(self.sides, self._views(cache))):
            side.activations_into(x, batch, view, write, position, outs[i:i + 1])
