"""Dense SwiGLU feed-forward: ``W_down( silu(W_gate x) * (W_up x) )`` without biases
(src/scratch_llm/model.py:223-237 of the reference; its w1 is the gate, w3 the up and w2 the
down matrix).  Gate and up are fused into one [2F, d] matrix at load.
"""

from __future__ import annotations

import math
from typing import Mapping

import torch

from ..kernels import ops
from ..weights.loader import ParamSpec
from .base import BuildContext, FeedForward
from .linear import Linear
from .registry import register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    pad_safe = True   # every token by itself
    accepts_sink = True   # forward() takes sink=: the down projection may feed the stream itself

    def accepts_normed(self, n_tokens: int) -> bool:
        return self.gate_up is not None and self.gate_up.takes_normed(n_tokens, swiglu=True)

    def __init__(self, hidden_size: int, intermediate_size: int,
                 names: Mapping[str, str] | None = None, activation: str = "silu") -> None:
        """``activation``: what the gate passes through, "silu" or "gelu_tanh"."""
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"unknown activation {activation!r}")
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.activation = activation
        self.names = {"gate": "gate_proj.weight", "up": "up_proj.weight",
                      "down": "down_proj.weight", **(names or {})}
        self.gate_up: Linear | None = None
        self.down: Linear | None = None

    def param_specs(self) -> dict[str, ParamSpec]:
        d, f = self.hidden_size, self.intermediate_size
        return {self.names["gate"]: ParamSpec((f, d)), self.names["up"]: ParamSpec((f, d)),
                self.names["down"]: ParamSpec((d, f))}

    def load(self, tensors: Mapping[str, torch.Tensor], ctx: BuildContext) -> None:
        put = lambda t: t.to(device=ctx.device, dtype=ctx.dtype)  # noqa: E731
        self.gate_up = Linear(torch.cat([put(tensors[self.names["gate"]]),
                                         put(tensors[self.names["up"]])], 0).contiguous())
        self.down = Linear(put(tensors[self.names["down"]]).contiguous())

    def forward(self, x, sink=None):
        y = self.gate_up.gated(x, self.activation)
        return self.down(y) if sink is None else sink.finish(self.down, y)


@register_feed_forward("geglu")
class GeGLU(SwiGLU):
    """The same with the tanh form of gelu on the gate: ``W_down( gelu(W_gate x) * (W_up x) )``."""

    def __init__(self, hidden_size: int, intermediate_size: int,
                 names: Mapping[str, str] | None = None, activation: str = "gelu_tanh") -> None:
        super().__init__(hidden_size, intermediate_size, names, activation)

    def kernel_jobs(self, dtype):
        jobs = [ops.core_job("sllm_stream_ops")]
        if dtype == torch.bfloat16:     # prompt steps from 1,024 tokens on: the fused tcgen05 product
            jobs.append(ops.core_job("sllm_gemm_tcgen05"))
        return jobs


@register_feed_forward("act_mlp")
class ActMLP(FeedForward):
    """A feed-forward without a gate: ``W_down act(W_up x)``, without biases.  ``activation``
    "xielu": with the two numbers p, q of the tensor ``act``,
    ``softplus(p) z^2 + z / 2`` for z > 0 and ``(1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2``
    for z <= 0; the two factors are formed once at load, in 64-bit."""

    pad_safe = True   # every token by itself

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "xielu",
                 names: Mapping[str, str] | None = None) -> None:
        if activation not in ops.PARAM_ACTIVATIONS:
            raise ValueError(f"unknown activation {activation!r}")
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.activation = activation
        self.names = {"up": "up", "down": "down", "act": "act", **(names or {})}
        self.up: Linear | None = None
        self.down: Linear | None = None
        self.factors = (0.0, 0.0)

    def kernel_jobs(self, dtype):
        return [ops.core_job("sllm_stream_ops")]

    def param_specs(self) -> dict[str, ParamSpec]:
        d, f = self.hidden_size, self.intermediate_size
        return {self.names["up"]: ParamSpec((f, d)), self.names["down"]: ParamSpec((d, f)),
                self.names["act"]: ParamSpec((2,), "gain")}

    def load(self, tensors: Mapping[str, torch.Tensor], ctx: BuildContext) -> None:
        put = lambda t: t.to(device=ctx.device, dtype=ctx.dtype).contiguous()  # noqa: E731
        self.up, self.down = Linear(put(tensors[self.names["up"]])), \
            Linear(put(tensors[self.names["down"]]))
        p, q = tensors[self.names["act"]].to(torch.float64).tolist()
        softplus = lambda z: max(z, 0.0) + math.log1p(math.exp(-abs(z)))  # noqa: E731
        self.factors = (softplus(p), 0.5 + softplus(q))

    def forward(self, x):
        z = self.up(x)
        return self.down(ops.param_act(z, torch.empty_like(z), self.activation, *self.factors))


@register_feed_forward("clamped_glu")
class ClampedGLU(FeedForward):
    """A gated feed-forward with clamps: with ``g = min(W_gate x, limit)`` and
    ``u = clamp(W_up x, -limit, limit)``, ``W_down( g * sigmoid(slope * g) * (u + 1) )``, without
    biases.  Gate and up are fused into one [2F, d] matrix at load."""

    pad_safe = True   # every token by itself

    def __init__(self, hidden_size: int, intermediate_size: int, limit: float,
                 slope: float = 1.702, names: Mapping[str, str] | None = None) -> None:
        if not (limit > 0 and math.isfinite(limit)):
            raise ValueError(f"limit must be positive, got {limit!r}")
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.limit, self.slope = float(limit), float(slope)
        self.names = {"gate": "gate", "up": "up", "down": "down", **(names or {})}
        self.gate_up: Linear | None = None
        self.down: Linear | None = None

    def kernel_jobs(self, dtype):
        jobs = [ops.core_job("sllm_stream_ops")]
        if dtype == torch.bfloat16:     # prompt steps from 1,024 tokens on: the fused tcgen05 product
            jobs.append(ops.core_job("sllm_gemm_tcgen05"))
        return jobs

    def param_specs(self) -> dict[str, ParamSpec]:
        d, f = self.hidden_size, self.intermediate_size
        return {self.names["gate"]: ParamSpec((f, d)), self.names["up"]: ParamSpec((f, d)),
                self.names["down"]: ParamSpec((d, f))}

    def load(self, tensors: Mapping[str, torch.Tensor], ctx: BuildContext) -> None:
        put = lambda t: t.to(device=ctx.device, dtype=ctx.dtype)  # noqa: E731
        self.gate_up = Linear(torch.cat([put(tensors[self.names["gate"]]),
                                         put(tensors[self.names["up"]])], 0).contiguous())
        self.down = Linear(put(tensors[self.names["down"]]).contiguous())

    def activations(self, x, out: torch.Tensor | None = None) -> torch.Tensor:
        """What the down matrix multiplies, [N, F]; ``out``: where to put it (may be a column
        slice of a wider buffer)."""
        return self.gate_up.gated(x, ("clamped", self.limit, self.slope), out=out)

    def forward(self, x):
        return self.down(self.activations(x))

    # -- for a block that multiplies several branches' activations by one joined output matrix

    def out_segments(self):
        return [(self.down.weight, 1.0)]

    def release_out(self) -> None:
        self.down = None

    def activations_into(self, x, outs) -> None:
        self.activations(x, out=outs[0])
