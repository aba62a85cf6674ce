"""Position encodings.

``rotary``: cos and sin of ``position * theta^(-2j/head_dim)`` in a 32-bit table of
``max_position`` rows, built exactly as the reference builds its buffers
(src/scratch_llm/model.py:195-202); the rotation itself runs in the fused rotate-and-store
kernel in 32-bit.  ``interleaved`` True rotates the adjacent pairs (x[2j], x[2j+1]) as the
reference does (src/scratch_llm/model.py:204-220); False rotates (x[j], x[j + head_dim/2]),
the layout of checkpoints saved for the split-half rotation.

Two options for other designs: ``rot_dims`` rotates only the first ``rot_dims`` entries of a head
(the tables then have ``rot_dims / 2`` columns and the pairs are taken among those entries, the
rest of the head passes unchanged), and ``scaling_factor`` divides every frequency (linear
position scaling).  With either, the frequencies ``theta^(-2j / rot_dims) / scaling_factor`` are
formed in 64-bit and rounded once; the angle ``position * frequency`` is 32-bit arithmetic.

``yarn`` (a mapping ``factor``, ``original``, ``fast``, ``slow``): every frequency f_i is blended
with ``f_i / factor`` by a ramp over the pair index i.  With ``pair(t) = dims * ln(original /
(2 pi t)) / (2 ln theta)``, ``lo = max(floor(pair(fast)), 0)`` and ``hi = min(ceil(pair(slow)),
dims - 1)``, the ramp is ``r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)`` and the frequency
``f_i / factor * r_i + f_i * (1 - r_i)``; cos and sin are both multiplied by
``yarn_magnitude * ln(factor) + 1``.

``none``: no position encoding (a mixer that needs none, or a test part).
"""

from __future__ import annotations

import math
from typing import Any, Mapping

import torch

from .base import BuildContext, PositionEncoding
from .registry import register_position_encoding


@register_position_encoding("rotary")
class Rotary(PositionEncoding):
    rotary_tables = True
    pad_safe = True   # a table lookup per token; padding tokens have position 0

    def __init__(self, head_dim: int, theta: float, max_position: int,
                 interleaved: bool = True, rot_dims: int | None = None,
                 scaling_factor: float = 1.0, yarn: Mapping[str, Any] | None = None,
                 yarn_magnitude: float = 0.1) -> None:
        if head_dim % 2:
            raise ValueError(f"rotary positions need an even head size, got {head_dim}")
        if rot_dims is not None and (rot_dims % 2 or not 2 <= rot_dims <= head_dim):
            raise ValueError(f"rot_dims must be even and between 2 and the head size "
                             f"{head_dim}, got {rot_dims}")
        if not scaling_factor > 0:
            raise ValueError(f"scaling_factor must be positive, got {scaling_factor}")
        self.head_dim, self.theta = head_dim, float(theta)
        self.max_position, self.interleaved = max_position, bool(interleaved)
        self.rot_dims, self.scaling_factor = rot_dims, float(scaling_factor)
        self.yarn = None if yarn is None else {k: float(yarn[k])
                                               for k in ("factor", "original", "fast", "slow")}
        if self.yarn is not None and not (self.yarn["factor"] > 0 and self.yarn["original"] > 0
                                          and self.yarn["fast"] > 0 and self.yarn["slow"] > 0):
            raise ValueError(f"yarn scaling needs positive factor, original, fast and slow, "
                             f"got {yarn!r}")
        self.yarn_magnitude = float(yarn_magnitude)
        self.cos: torch.Tensor | None = None
        self.sin: torch.Tensor | None = None

    def tables(self) -> tuple[torch.Tensor, torch.Tensor]:
        """The table on the CPU in 32-bit: the reference's, or, with ``rot_dims`` or a scaling
        factor, frequencies from 64-bit and 32-bit angles."""
        if self.yarn is not None:
            dims = self.rot_dims or self.head_dim
            y = self.yarn

            def pair(turns: float) -> float:
                return dims * math.log(y["original"] / (2.0 * math.pi * turns)) \
                    / (2.0 * math.log(self.theta))

            lo = max(math.floor(pair(y["fast"])), 0)
            hi = min(math.ceil(pair(y["slow"])), dims - 1)
            freqs64 = []
            for j in range(dims // 2):
                f = self.theta ** (-2.0 * j / dims) / self.scaling_factor
                ramp = min(max((j - lo) / max(hi - lo, 0.001), 0.0), 1.0)
                freqs64.append(f / y["factor"] * ramp + f * (1.0 - ramp))
            inv_freq = torch.tensor(freqs64, dtype=torch.float64).float()
            freqs = torch.arange(self.max_position).float()[:, None] * inv_freq[None, :]
            mag = self.yarn_magnitude * math.log(y["factor"]) + 1.0
            return freqs.cos() * mag, freqs.sin() * mag
        if self.rot_dims is not None or self.scaling_factor != 1.0:
            dims = self.rot_dims or self.head_dim
            inv_freq = torch.tensor([self.theta ** (-2.0 * j / dims) / self.scaling_factor
                                     for j in range(dims // 2)], dtype=torch.float64).float()
            freqs = torch.arange(self.max_position).float()[:, None] * inv_freq[None, :]
            return freqs.cos(), freqs.sin()
        inv_freq = 1.0 / (self.theta ** (torch.arange(0, self.head_dim, 2).float()
                                         / self.head_dim))
        freqs = torch.outer(torch.arange(self.max_position).float(), inv_freq)
        return freqs.cos(), freqs.sin()

    def load(self, tensors: Mapping[str, torch.Tensor], ctx: BuildContext) -> None:
        cos, sin = self.tables()
        self.cos = cos.to(ctx.device).contiguous()
        self.sin = sin.to(ctx.device).contiguous()

    def apply(self, q, k, positions):  # the attention mixer uses the tables instead
        raise NotImplementedError("rotary positions are applied by the fused kernel")


@register_position_encoding("none")
class NoPosition(PositionEncoding):
    pad_safe = True

    def __init__(self, **_: object) -> None:
        pass

    def apply(self, q, k, positions) -> None:
        return None
