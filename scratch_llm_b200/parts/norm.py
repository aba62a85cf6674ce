"""RMSNorm fused with the add of the pending residual delta.

``x * rsqrt(mean(x^2) + eps) * weight`` in 32-bit, eps inside the root, the weight after the
normalisation, one rounding at the end (src/scratch_llm/model.py:149-162 of the reference; its
eps is fixed at 1e-5 in code, here it is a parameter).
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..kernels import ops
from ..weights.loader import ParamSpec
from .base import BuildContext, Norm
from .registry import register_norm
from .stream import Current, Normed, Terms


@register_norm("rmsnorm")
class RMSNorm(Norm):
    pad_safe = True   # every token by itself
    #: the norm's factor is one number per token: the product before it may prepare it and the
    #: product after it may apply it (scratch_llm_b200.parts.stream)
    deferrable = True

    def __init__(self, size: int, eps: float, name: str = "weight", offset: float = 0.0) -> None:
        """``name``: the gain's tensor name below the part's prefix; "" if the prefix itself is
        the tensor's name.  ``offset``: the gain is ``offset + w`` of the stored ``w`` (1.0 for
        gains that are stored around zero), formed once at load in 32-bit."""
        self.size, self.eps, self.name, self.offset = size, float(eps), name, float(offset)
        self.weight: torch.Tensor | None = None
        self.dtype = torch.float32

    def param_specs(self) -> dict[str, ParamSpec]:
        return {self.name: ParamSpec((self.size,), "gain")}

    def load(self, tensors: Mapping[str, torch.Tensor], ctx: BuildContext) -> None:
        self.weight = tensors[self.name].to(device=ctx.device, dtype=torch.float32).contiguous()
        if self.offset:
            self.weight += self.offset
        self.dtype = ctx.dtype

    def forward(self, resid: torch.Tensor, delta: torch.Tensor | None,
                out_rows: torch.Tensor | None = None):
        if isinstance(delta, Normed):
            # the product before this norm has already put its output into the stream and
            # prepared this norm: what is left is the tokens' factor, which the next product applies
            if delta.norm is not self or out_rows is not None:
                raise ValueError("a deferred norm reached a norm it was not prepared for")
            return delta
        if isinstance(delta, Current):
            delta = None
        n = resid.shape[0] if out_rows is None else out_rows.numel()
        out = torch.empty((n, self.size), dtype=self.dtype, device=resid.device)
        return ops.add_rmsnorm(resid, delta, self.weight, self.eps, out, out_rows)

    def add_normed(self, resid: torch.Tensor, delta: torch.Tensor,
                   cast_out: torch.Tensor | None = None, then: "RMSNorm | None" = None):
        """``resid += rmsnorm(delta)``; with ``then`` (another norm of this kind and size) also
        returns ``then(resid)`` from the same pass."""
        if then is None:
            ops.add_normed(resid, delta, self.weight, self.eps, cast_out)
            return None
        out = torch.empty_like(delta)
        ops.add_normed(resid, delta, self.weight, self.eps, cast_out,
                       (then.weight, then.eps, out))
        return out

    def chains_with(self, other) -> bool:
        return isinstance(other, RMSNorm) and other.size == self.size


@register_norm("dyt")
class DynamicTanh(Norm):
    """A tanh in the place of a norm: ``tanh(alpha * x) * w + b`` element by element, with one
    scalar ``alpha`` and the vectors ``w`` and ``b``.  No mean or variance is computed (an ``eps``
    is accepted and unused), so the arithmetic has no row-wide step: the same kernel can mix in
    the previous token's result (a token shift, ``fuses_token_mix``), and the norm of a branch's
    output chains with the norm in front of the next branch (``add_normed(..., then=)``).

    Tensors below the part's prefix: the gain under ``name`` ("" = the prefix itself), the scalar
    under ``<name>.alpha`` and the offset under ``<name>.b``."""

    pad_safe = True            # every element by itself
    fuses_token_mix = True     # forward(..., token_mix=) mixes with the previous token's result

    def __init__(self, size: int, eps: float = 0.0, name: str = "") -> None:
        self.size, self.eps, self.name = size, float(eps), name
        self.alpha = 1.0
        self.weight: torch.Tensor | None = None
        self.bias: torch.Tensor | None = None
        self.dtype = torch.float32

    def _sub(self, what: str) -> str:
        return f"{self.name}.{what}" if self.name else what

    def kernel_jobs(self, dtype: torch.dtype):
        return [ops.core_job("sllm_tanh_norm")]

    def param_specs(self) -> dict[str, ParamSpec]:
        return {self.name: ParamSpec((self.size,), "gain"),
                self._sub("alpha"): ParamSpec((), "gain"),
                self._sub("b"): ParamSpec((self.size,), "gain")}

    def load(self, tensors: Mapping[str, torch.Tensor], ctx: BuildContext) -> None:
        f32 = lambda t: t.to(device=ctx.device, dtype=torch.float32).contiguous()  # noqa: E731
        self.weight, self.bias = f32(tensors[self.name]), f32(tensors[self._sub("b")])
        self.alpha = float(tensors[self._sub("alpha")].to(torch.float32))
        self.dtype = ctx.dtype

    def params(self) -> tuple[float, torch.Tensor, torch.Tensor]:
        return self.alpha, self.weight, self.bias

    def forward(self, resid: torch.Tensor, delta=None, out_rows: torch.Tensor | None = None,
                token_mix=None):
        """``token_mix = (mu, state, batch, write)``: every token's result is mixed with the
        previous token's (see :func:`scratch_llm_b200.kernels.ops.dyt_norm`); the state of rows
        that bring several tokens is stored by a second launch."""
        if isinstance(delta, Current):
            delta = None
        if delta is not None:
            raise ValueError("this norm takes a stream with nothing pending")
        n = resid.shape[0] if out_rows is None else out_rows.numel()
        out = torch.empty((n, self.size), dtype=self.dtype, device=resid.device)
        shift = None
        if token_mix is not None:
            mu, state, batch, write = token_mix
            shift = (mu, state, batch.token_row, batch.row_start, batch.row_slot, write)
        ops.dyt_norm(resid, self.alpha, self.weight, self.bias, out, out_rows, shift)
        if token_mix is not None and write and batch.n_multi:
            ops.dyt_state_update(resid, self.alpha, self.weight, self.bias, state,
                                 batch.row_start, batch.row_slot, batch.n_rows, self.dtype)
        return out

    def add_normed(self, resid: torch.Tensor, delta: torch.Tensor,
                   cast_out: torch.Tensor | None = None, then: "DynamicTanh | None" = None):
        """``resid += dyt(delta)``; with ``then`` (another norm of this kind) also returns
        ``then(resid)`` from the same pass."""
        if cast_out is not None:
            raise ValueError("this norm hands on the next norm's output (then=), not a copy")
        if then is None:
            ops.dyt_add(resid, delta, self.alpha, self.weight, self.bias)
            return None
        out = torch.empty_like(delta)
        ops.dyt_add(resid, delta, self.alpha, self.weight, self.bias, then.params(), out)
        return out

    def chains_with(self, other) -> bool:
        return isinstance(other, DynamicTanh)


@register_norm("layernorm")
class LayerNorm(Norm):
    """``(x - mean) / sqrt(var + eps) * w + b`` with the variance as the mean of the squared
    deviations, all in 32-bit with one rounding at the end.  Tensors below the part's prefix: the
    gain under ``name`` ("" = the prefix itself) and the offset under ``<name>.b``.

    What is pending for the stream may be a tensor or a weighted sum of several
    (:class:`~.stream.Terms`): the kernel adds them in while it reads the stream."""

    pad_safe = True       # every token by itself
    takes_terms = True    # forward() accepts a Terms as what is pending

    def __init__(self, size: int, eps: float, name: str = "") -> None:
        self.size, self.eps, self.name = size, float(eps), name
        self.weight: torch.Tensor | None = None
        self.bias: torch.Tensor | None = None
        self.dtype = torch.float32

    def _bias_name(self) -> str:
        return f"{self.name}.b" if self.name else "b"

    def kernel_jobs(self, dtype: torch.dtype):
        return [ops.core_job("sllm_layer_norm")]

    def param_specs(self) -> dict[str, ParamSpec]:
        return {self.name: ParamSpec((self.size,), "gain"),
                self._bias_name(): ParamSpec((self.size,), "gain")}

    def load(self, tensors: Mapping[str, torch.Tensor], ctx: BuildContext) -> None:
        f32 = lambda t: t.to(device=ctx.device, dtype=torch.float32).contiguous()  # noqa: E731
        self.weight, self.bias = f32(tensors[self.name]), f32(tensors[self._bias_name()])
        self.dtype = ctx.dtype

    @staticmethod
    def _terms(delta) -> tuple:
        if delta is None or isinstance(delta, Current):
            return ()
        if isinstance(delta, Terms):
            return delta.items
        if isinstance(delta, Normed):
            raise ValueError("a layer norm's factor is not one number per token: nothing can "
                             "hand it over")
        return ((delta, 1.0),)

    def forward(self, resid: torch.Tensor, delta=None, out_rows: torch.Tensor | None = None):
        n = resid.shape[0] if out_rows is None else out_rows.numel()
        out = torch.empty((n, self.size), dtype=self.dtype, device=resid.device)
        return ops.add_layernorm(resid, self._terms(delta), self.weight, self.bias, self.eps,
                                 out, out_rows)

    def in_place(self, resid: torch.Tensor) -> torch.Tensor:
        """The stream replaced by its norm (32-bit), as a model does to its embedding output."""
        return ops.add_layernorm(resid, (), self.weight, self.bias, self.eps, resid)
