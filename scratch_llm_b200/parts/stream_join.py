"""Joins of the residual stream with the embedding output, between runs of layers.

``concat_linear``: ``x <- W [x; x0]`` with ``W`` [hidden, 2 hidden] (the stream's half first) and
``x0`` the embedding output.  A model that runs a span of layers several times with the same
weights does this before each pass, so that every pass sees the tokens themselves again.  Both
halves are rounded to the compute dtype for the product; its result is the new 32-bit stream.
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..kernels import ops
from ..weights.loader import ParamSpec
from .base import BuildContext, StreamJoin
from .linear import Linear
from .registry import register_stream_join


@register_stream_join("concat_linear")
class ConcatLinear(StreamJoin):
    pad_safe = True   # every token by itself

    def __init__(self, size: int, name: str = "") -> None:
        """``name``: the matrix's tensor name below the part's prefix ("" = the prefix itself)."""
        self.size, self.name = size, name
        self.w: Linear | None = None
        self.dtype = torch.float32

    def kernel_jobs(self, dtype: torch.dtype):
        return [ops.core_job("sllm_stream_ops")]

    def param_specs(self) -> dict[str, ParamSpec]:
        return {self.name: ParamSpec((self.size, 2 * self.size))}

    def load(self, tensors: Mapping[str, torch.Tensor], ctx: BuildContext) -> None:
        self.w = Linear(tensors[self.name].to(device=ctx.device, dtype=ctx.dtype).contiguous())
        self.dtype = ctx.dtype

    def forward(self, resid: torch.Tensor, first: torch.Tensor) -> torch.Tensor:
        both = torch.empty((resid.shape[0], 2 * self.size), dtype=self.dtype, device=resid.device)
        ops.concat_cast(resid, first, both)
        return self.w(both, out_dtype=torch.float32)
