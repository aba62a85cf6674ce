"""The gated delta rule as a mixer: a recurrent layer whose state per request is one matrix
``S`` [key_dim, value_dim] per head in 32-bit, plus the last inputs of a short convolution.

    q, k = W_q x, W_k x  (n_kv_heads x key_dim),   v = W_v x  (n_heads x value_dim)
    each through a causal convolution over time per channel (``conv_taps`` taps, the last one
    is the current token's, zeros before the start) and silu;
    k, q made unit vectors per head (eps 1e-6 inside the root), q also times key_dim^(-1/2);
    beta = sigmoid(W_b x),  g = exp(-exp(A_log) * softplus(W_a x + dt_bias))   (one per head)
    S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
    out = W_o ( rmsnorm_per_head(o) * gain * silu(W_g x) )

Two options for other designs.  ``decay_rank`` (a number, or -1 for "as the tensors say"): ONE
DECAY PER KEY CHANNEL instead of one per head, through a low-rank pair of matrices,

    g = exp(-exp(A_log_h) * softplus(W_a2 (W_a1 x) + dt_bias))          laid out heads x key_dim

(``a1`` [rank, d], ``a2`` [H key_dim, rank], ``dt_bias`` [H key_dim]), acting on the rows of S
that belong to key channels; the second product, softplus and the exponentials are 32-bit.
``gate_rank`` (likewise): the output gate through a low-rank pair, ``act(W_g2 (W_g1 x))``
(``g1`` [rank, d], ``g2`` [H value_dim, rank]); ``gate_activation`` "silu" or "sigmoid".

Head h reads key/query head ``h // (n_heads / n_kv_heads)``.  What enters the recurrence (unit
vectors, gates, decays, the state) is 32-bit; the projections, the convolution and silu run in
the compute dtype.  The state lives in the cache manager's state slots
(:meth:`state_spec`: the matrix and the convolution's carried inputs), so a request may be fed
in portions of any size, beside other requests, and its slot is used again after it ends.
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..kernels import ops
from ..weights.loader import ParamSpec
from .base import BuildContext, CacheView, Mixer, PositionEncoding, StateSpec
from .linear import Linear
from .registry import register_mixer


@register_mixer("gated_delta_rule")
class GatedDeltaRule(Mixer):
    pad_safe = True   # padding tokens belong to no row: the recurrence never sees them

    def __init__(self, hidden_size: int, n_heads: int, n_kv_heads: int, key_dim: int,
                 value_dim: int, conv_taps: int, eps: float,
                 names: Mapping[str, str] | None = None, decay_rank: int | None = None,
                 gate_rank: int | None = None, gate_activation: str = "silu") -> None:
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads do not group evenly over {n_kv_heads} key heads")
        if not 1 <= key_dim <= ops.DELTA_MAX_KEY_DIM:
            raise ValueError(f"key size {key_dim}: the delta-rule kernel takes 1 to "
                             f"{ops.DELTA_MAX_KEY_DIM}")
        if decay_rank is not None and key_dim > ops.DELTA_CHANNEL_MAX_KEY_DIM:
            raise ValueError(f"key size {key_dim}: with a decay per channel the delta-rule kernel "
                             f"takes up to {ops.DELTA_CHANNEL_MAX_KEY_DIM}")
        if gate_activation not in ("silu", "sigmoid"):
            raise ValueError(f"gate_activation must be 'silu' or 'sigmoid', got {gate_activation!r}")
        if not 1 <= conv_taps <= 16:
            raise ValueError(f"the short convolution takes 1 to 16 taps, got {conv_taps}")
        self.hidden_size, self.n_heads, self.n_kv_heads = hidden_size, n_heads, n_kv_heads
        self.key_dim, self.value_dim, self.conv_taps = key_dim, value_dim, conv_taps
        self.eps = float(eps)
        self.decay_rank, self.gate_rank = decay_rank, gate_rank
        self.gate_activation = gate_activation
        self.names = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "a": "a", "b": "b",
                      "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv",
                      "A_log": "A_log", "dt_bias": "dt_bias", "norm": "norm", "a1": "a1",
                      "a2": "a2", "g1": "g1", "g2": "g2", **(names or {})}
        self.dtype = torch.float32
        self.proj: Linear | None = None     # [q; k; v; g]
        self.ab: Linear | None = None       # [a; b]
        self.o: Linear | None = None
        self.taps = self.taps_t = self.a_log = self.dt_bias = self.gain = None
        self.a2t = self.g2t = None          # the low-rank pairs' second matrices, [rank, out]

    @property
    def conv_channels(self) -> int:
        return 2 * self.n_kv_heads * self.key_dim + self.n_heads * self.value_dim

    def state_spec(self):
        S = StateSpec((self.n_heads, self.value_dim, self.key_dim), torch.float32)
        if self.conv_taps == 1:
            return S
        return (S, StateSpec((self.conv_taps - 1, self.conv_channels), self.dtype))

    def kernel_jobs(self, dtype: torch.dtype):
        return [ops.core_job("sllm_recurrent_ops"), ops.delta_rule_library(self.key_dim)]

    def param_specs(self) -> dict[str, ParamSpec]:
        n, d = self.names, self.hidden_size
        kd, vd = self.n_kv_heads * self.key_dim, self.n_heads * self.value_dim
        K, H = self.conv_taps, self.n_heads
        specs = {n["q"]: ParamSpec((kd, d)), n["k"]: ParamSpec((kd, d)), n["v"]: ParamSpec((vd, d)),
                 n["o"]: ParamSpec((d, vd)), n["b"]: ParamSpec((H, d)),
                 n["q_conv"]: ParamSpec((kd, K), "gain"), n["k_conv"]: ParamSpec((kd, K), "gain"),
                 n["v_conv"]: ParamSpec((vd, K), "gain"), n["A_log"]: ParamSpec((H,), "gain"),
                 n["norm"]: ParamSpec((self.value_dim,), "gain")}
        if self.decay_rank is None:
            specs[n["a"]] = ParamSpec((H, d))
            specs[n["dt_bias"]] = ParamSpec((H,), "gain")
        else:
            specs[n["a1"]] = ParamSpec((self.decay_rank, d))
            specs[n["a2"]] = ParamSpec((H * self.key_dim, self.decay_rank))
            specs[n["dt_bias"]] = ParamSpec((H * self.key_dim,), "gain")
        if self.gate_rank is None:
            specs[n["g"]] = ParamSpec((vd, d))
        else:
            specs[n["g1"]] = ParamSpec((self.gate_rank, d))
            specs[n["g2"]] = ParamSpec((vd, self.gate_rank))
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], ctx: BuildContext) -> None:
        put = lambda t: t.to(device=ctx.device, dtype=ctx.dtype)  # noqa: E731
        f32 = lambda t: t.to(device=ctx.device, dtype=torch.float32).contiguous()  # noqa: E731
        n = self.names
        self.dtype = ctx.dtype
        wide = "qkv" + ("g" if self.gate_rank is None else "")
        self.proj = Linear(torch.cat([put(tensors[n[k]]) for k in wide], 0).contiguous())
        # the narrow projections, with a 32-bit output: [a | a1; b; g1]
        narrow = [tensors[n["a"]] if self.decay_rank is None else tensors[n["a1"]], tensors[n["b"]]]
        if self.decay_rank is not None:
            if tensors[n["a1"]].shape[0] != tensors[n["a2"]].shape[1]:
                raise ValueError("the decay's low-rank matrices do not fit each other")
            self.decay_rank = tensors[n["a1"]].shape[0]
            self.a2t = f32(tensors[n["a2"]]).t().contiguous()
        if self.gate_rank is not None:
            if tensors[n["g1"]].shape[0] != tensors[n["g2"]].shape[1]:
                raise ValueError("the gate's low-rank matrices do not fit each other")
            self.gate_rank = tensors[n["g1"]].shape[0]
            self.g2t = f32(tensors[n["g2"]]).t().contiguous()
            narrow.append(tensors[n["g1"]])
        self.ab = Linear(torch.cat([put(t) for t in narrow], 0).contiguous())
        self.o = Linear(put(tensors[n["o"]]).contiguous())
        self.taps = torch.cat([f32(tensors[n[k]]) for k in ("q_conv", "k_conv", "v_conv")], 0)
        self.taps_t = self.taps.t().contiguous()
        self.a_log, self.dt_bias = f32(tensors[n["A_log"]]), f32(tensors[n["dt_bias"]])
        self.gain = f32(tensors[n["norm"]])

    def forward(self, x, batch, cache: CacheView, write: bool, position: PositionEncoding):
        return self.o(self.heads_out(x, batch, cache, write, position))

    def heads_out(self, x, batch, cache: CacheView, write: bool, position: PositionEncoding,
                  out: torch.Tensor | None = None) -> torch.Tensor:
        """The heads' read-outs, normed and gated [N, H * value_dim]: what the output matrix
        multiplies.  ``out``: where to put them (may be a column slice)."""
        H, G, D, V, K = self.n_heads, self.n_kv_heads, self.key_dim, self.value_dim, self.conv_taps
        C = self.conv_channels
        state = cache.state if isinstance(cache.state, tuple) else (cache.state, None)
        S, carried = state
        n = x.shape[0]
        proj = self.proj(x)                                   # [N, C + H V]
        ab = self.ab(x, out_dtype=torch.float32)              # [N, 2 H]: gates in 32-bit
        act = torch.empty((n, C), dtype=proj.dtype, device=proj.device)
        ops.conv_silu(proj, self.taps, carried, batch.token_row, batch.row_start, batch.row_slot,
                      act, self.taps_t)
        if write:
            ops.conv_state_update(proj, K, carried, batch.row_start, batch.row_slot, batch.n_rows)
        if not write:
            raise NotImplementedError("a run that only reads another run's recurrent state")
        # (padding tokens belong to no row: their read-out stays zero)
        o = (torch.zeros if batch.padded else torch.empty)((n, H * V), dtype=torch.float32,
                                                           device=proj.device)
        max_new = 1 if batch.n_multi == 0 else 0
        if self.decay_rank is None:
            ops.delta_rule(act, ab, self.a_log, self.dt_bias, S, batch.row_start, batch.row_slot,
                           o, batch.n_rows, H, G, D, V, max_new=max_new)
            b_end = 2 * H
        else:
            # the logarithms of the channels' decays, 32-bit from the first product's output on
            # (a low-rank gate's second product rides along in the same launch)
            log_decay = torch.empty((n, H * D), dtype=torch.float32, device=proj.device)
            if self.gate_rank is not None:
                gate = torch.empty((n, H * V), dtype=proj.dtype, device=proj.device)
                also = (self.decay_rank + H, self.g2t, gate)
            ops.lowrank_expand(ab, 0, self.a2t, log_decay, bias=self.dt_bias,
                               rate_log=self.a_log, per_rate=D,
                               also=also if self.gate_rank is not None else None)
            ops.delta_rule(act, ab, None, None, S, batch.row_start, batch.row_slot, o,
                           batch.n_rows, H, G, D, V, max_new=max_new, log_decay=log_decay,
                           b_col=self.decay_rank, longest=batch.max_new)
            b_end = self.decay_rank + H
        if self.gate_rank is None:
            gate = proj[:, C:C + H * V]
        elif self.decay_rank is None:
            gate = torch.empty((n, H * V), dtype=proj.dtype, device=proj.device)
            ops.lowrank_expand(ab, b_end, self.g2t, gate)
        if out is None:
            out = torch.empty(o.shape, dtype=gate.dtype, device=o.device)
        ops.head_norm_gate(o, gate, self.gain, self.eps, out, self.n_heads,
                           gate_activation=self.gate_activation)
        return out

    # -- for a block that multiplies several branches' activations by one joined output matrix

    def out_segments(self):
        """[(the output matrix [hidden, H * value_dim], its weight in the layer's sum)]."""
        return [(self.o.weight, 1.0)]

    def release_out(self) -> None:
        self.o = None

    def activations_into(self, x, batch, cache: CacheView, write: bool, position, outs) -> None:
        self.heads_out(x, batch, cache, write, position, out=outs[0])
