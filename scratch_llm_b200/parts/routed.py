"""A routed feed-forward (mixture of experts): ``experts`` small gated feed-forwards of which
every token uses ``top``, chosen by a router.

    z = W_router x                      (32-bit)          s = softmax(z) over ALL router outputs
    choice = s + correction             (the weights below use s, without the correction)
    the outputs form ``groups`` equal groups of neighbours; a group's score is its largest
    choice score and only the best ``keep_groups`` groups stay eligible
    the ``top`` eligible outputs with the largest choice scores are chosen;
    weight_i = s_i / (sum of the chosen s + 1e-20)
    out = sum_i weight_i * Expert_i(x)  [+ Shared(x)]

The last ``identity`` router outputs are identity experts: their output is x itself, they have no
tensors.  Experts and the shared expert: ``W_down(silu(W_gate x) * (W_up x))`` without biases.
Tensors below the part's prefix: ``router``, ``correction``, ``e<i>.{gate,up,down}`` and
``shared.{gate,up,down}``.

Variants for other designs, each a constructor argument: ``score="sigmoid"`` (s = sigmoid(z), every
output by itself, instead of the softmax), ``group_score="top2"`` (a group's score is the sum of
its two largest choice scores instead of its largest), ``renormalize=False`` (the weights are the
chosen scores s themselves) and ``expert="sqrelu"`` (experts without a gate,
``W_down(relu(W_up x)^2)``, tensors ``e<i>.{up,down}``).

Nothing of a step is read on the host: the router's kernel sorts the (token, choice) pairs by
expert on the device and the grouped products walk a tile list, so steps can be recorded into
CUDA graphs.  Every product of a token is one chain over the reduction in ascending order and the
choices are added in the router's order, so a token's result does not depend on the batch.
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..kernels import ops
from ..weights.loader import ParamSpec
from .base import BuildContext, FeedForward
from .feed_forward import SwiGLU
from .linear import Linear
from .registry import register_feed_forward


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    pad_safe = True   # every token by itself (padding tokens are routed like any other, unread)

    def __init__(self, hidden_size: int, expert_size: int, experts: int, top: int,
                 identity: int = 0, groups: int = 1, keep_groups: int = 1,
                 shared_size: int | None = None, score: str = "softmax",
                 group_score: str = "max", renormalize: bool = True,
                 expert: str = "gated_silu") -> None:
        total = experts + identity
        if experts < 0 or identity < 0 or total < 1:
            raise ValueError("a router needs at least one output")
        if not 1 <= top <= min(total, 32):
            raise ValueError(f"top must be between 1 and min(router outputs, 32), got {top}")
        if groups < 1 or total % groups or not 1 <= keep_groups <= groups:
            raise ValueError(f"{total} router outputs do not form {groups} equal groups of "
                             f"which {keep_groups} are kept")
        if keep_groups * (total // groups) < top:
            raise ValueError("the kept groups hold fewer outputs than are chosen")
        if score not in ("softmax", "sigmoid") or group_score not in ("max", "top2") \
                or expert not in ("gated_silu", "sqrelu"):
            raise ValueError(f"unknown router or expert variant: score {score!r}, group_score "
                             f"{group_score!r}, expert {expert!r}")
        self.flags = (ops.MOE_SIGMOID if score == "sigmoid" else 0) \
            | (ops.MOE_GROUP_TOP2 if group_score == "top2" else 0) \
            | (0 if renormalize else ops.MOE_RAW_WEIGHTS)
        #: what the experts' first grouped product does: silu(gate) * up, or relu(up)^2
        self.first = ops.MOE_GATED if expert == "gated_silu" else ops.MOE_SQRELU
        self.hidden_size, self.expert_size = hidden_size, expert_size
        self.experts, self.identity, self.top = experts, identity, top
        self.groups, self.keep_groups = groups, keep_groups
        self.shared = None if shared_size is None else SwiGLU(
            hidden_size, shared_size, names={"gate": "shared.gate", "up": "shared.up",
                                             "down": "shared.down"})
        self.router: Linear | None = None
        self.correction = self.gate_up = self.down = None

    def _tensor_cores(self, dtype) -> bool:
        return dtype == torch.bfloat16 and self.experts > 0 and \
            ops.moe_tc_supports(self.hidden_size, self.expert_size)

    def kernel_jobs(self, dtype):
        jobs = [ops.core_job("sllm_moe")]
        if self._tensor_cores(dtype):
            jobs.append(ops.core_job("sllm_moe_tc"))
        if dtype == torch.bfloat16 and self.shared is not None:
            jobs.append(ops.core_job("sllm_gemm_tcgen05"))   # the shared expert's long steps
        return jobs

    def param_specs(self) -> dict[str, ParamSpec]:
        d, f, total = self.hidden_size, self.expert_size, self.experts + self.identity
        specs = {"router": ParamSpec((total, d)), "correction": ParamSpec((total,), "gain")}
        for e in range(self.experts):
            if self.first == ops.MOE_GATED:
                specs[f"e{e}.gate"] = ParamSpec((f, d))
            specs[f"e{e}.up"] = ParamSpec((f, d))
            specs[f"e{e}.down"] = ParamSpec((d, f))
        if self.shared is not None:
            specs.update(self.shared.param_specs())
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], ctx: BuildContext) -> None:
        put = lambda t: t.to(device=ctx.device, dtype=ctx.dtype)  # noqa: E731
        self.router = Linear(put(tensors["router"]).contiguous())
        self.correction = tensors["correction"].to(device=ctx.device,
                                                   dtype=torch.float32).contiguous()
        if self.experts:
            # [E, 2 F, d]: an expert's gate rows, then its up rows (without a gate: [E, F, d]);
            # [E, d, F]
            if self.first == ops.MOE_GATED:
                self.gate_up = torch.stack([torch.cat([put(tensors[f"e{e}.gate"]),
                                                       put(tensors[f"e{e}.up"])], 0)
                                            for e in range(self.experts)]).contiguous()
            else:
                self.gate_up = torch.stack([put(tensors[f"e{e}.up"])
                                            for e in range(self.experts)]).contiguous()
            self.down = torch.stack([put(tensors[f"e{e}.down"])
                                     for e in range(self.experts)]).contiguous()
        if self.shared is not None:
            self.shared.load(tensors, ctx)

    def forward(self, x):
        n, d = x.shape
        logits = self.router(x, out_dtype=torch.float32)
        tensor_cores = self._tensor_cores(x.dtype)
        ids, weights, pair_token, pair_place, meta, max_tiles, rows = ops.moe_route(
            logits, self.correction, None, self.experts, self.groups, self.keep_groups, self.top,
            tile_rows=ops.MOE_TC_TILE_ROWS if tensor_cores else None,
            gather_from=x if tensor_cores else None, flags=self.flags)
        pairs = n * self.top
        y = torch.empty((max(pairs, 1), d), dtype=torch.float32, device=x.device)
        if self.experts:
            hidden = torch.empty((pairs, self.expert_size), dtype=x.dtype, device=x.device)
            if tensor_cores:
                # bfloat16: the tokens' rows in the sorted order, then both products on tcgen05
                if rows is None:     # (steps of few tokens: the router has copied them itself)
                    rows = ops.moe_gather_rows(x, pair_token, torch.empty(
                        (pairs, d), dtype=x.dtype, device=x.device))
                ops.moe_tc_product(rows, self.gate_up, hidden, meta, max_tiles, gated=self.first)
                ops.moe_tc_product(hidden, self.down, y, meta, max_tiles, gated=False)
            else:
                ops.moe_product(x, self.gate_up, hidden, meta, pair_token, max_tiles,
                                gated=self.first)
                ops.moe_product(hidden, self.down, y, meta, pair_token, max_tiles, gated=False)
        shared = self.shared.forward(x) if self.shared is not None else None
        out = torch.empty_like(x)
        return ops.moe_combine(y, x, shared, ids, weights, pair_place, self.experts, out)
