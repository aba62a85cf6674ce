"""Grouped-query attention with rotary positions whose queries and keys are normed, for designs
that do one or several of:

* biases on the q, k and v projections (``bias``);
* an RMS norm over the WHOLE query projection and over the whole key projection, before they
  are split into heads and rotated, with a gain per column (``qk_norm="wide"``);
* an RMS norm per head without gains AFTER the rotation (``qk_norm="unit_after"``);
* a tanh cap on the scaled scores, ``cap * tanh(s / cap)`` (``softcap``);
* a sliding window (``window``: query i sees keys j with ``0 <= i - j < window``) or chunks
  (``chunk``: query i sees keys j <= i with ``i // chunk == j // chunk``, counted from the
  sequence's start, however the prompt was cut);
* a sink of score 0 in the softmax's denominator, with no value (``zero_sink``);
* a sigmoid output gate with ONE number per head, read from the mixer's input (``head_gate``);
* keys and values BORROWED from another layer's cache entry (``borrow_kv``): the mixer then has
  no key or value tensors, its run reads the entry the other layer's run wrote in the same step
  (the run order says which), with its own queries and mask.

The values may have another size than queries and keys (``value_dim``): heads are padded with
zero rows of the projections up to a common multiple of 16, the head size of the kernels and of
the cache; the norms divide by the true sizes.  Norms, rotation and softmax are 32-bit; the
cache holds the keys after norm and rotation.
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..kernels import ops
from ..weights.loader import ParamSpec
from .attention import TC_MIN_PACKED_QUERIES, decode_splits
from .base import BuildContext, CacheView, KVSpec, Mixer, PositionEncoding
from .linear import Linear
from .registry import register_mixer


@register_mixer("normed_attention")
class NormedAttention(Mixer):
    pad_safe = True   # padding tokens are neither normed nor stored; empty rows leave the kernels

    def __init__(self, hidden_size: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 scale: float, eps: float, value_dim: int | None = None, bias: bool = False,
                 qk_norm: str | None = None, softcap: float = 0.0, window: int | None = None,
                 chunk: int | None = None, zero_sink: bool = False, head_gate: bool = False,
                 borrow_kv: bool = False,
                 names: Mapping[str, str] | None = None) -> None:
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} query heads do not group evenly over {n_kv_heads} "
                             "kv heads")
        if qk_norm not in (None, "wide", "unit_after"):
            raise ValueError(f"qk_norm must be None, 'wide' or 'unit_after', got {qk_norm!r}")
        if window is not None and chunk is not None:
            raise ValueError("a mixer has a window or chunks, not both")
        for what, v in (("window", window), ("chunk", chunk)):
            if v is not None and v < 1:
                raise ValueError(f"{what} must be at least 1, got {v}")
        if softcap < 0:
            raise ValueError(f"softcap must not be negative, got {softcap}")
        self.qk_dim, self.v_dim = head_dim, head_dim if value_dim is None else value_dim
        if min(self.qk_dim, self.v_dim) < 1:
            raise ValueError("head sizes must be positive")
        # the common head size of the kernels and of the cache's pages
        self.head_dim = -(-max(self.qk_dim, self.v_dim) // 16) * 16
        if self.head_dim > 512:
            raise ValueError(f"head sizes {self.qk_dim} / {self.v_dim}: the attention kernels "
                             "take up to 512")
        self.hidden_size, self.n_heads, self.n_kv_heads = hidden_size, n_heads, n_kv_heads
        self.scale, self.eps, self.softcap = float(scale), float(eps), float(softcap)
        self.window, self.chunk = window, chunk
        self.has_bias, self.qk_norm = bool(bias), qk_norm
        self.zero_sink, self.has_gate, self.borrow_kv = bool(zero_sink), bool(head_gate), bool(borrow_kv)
        self.names = {"q": "q", "k": "k", "v": "v", "o": "o", "g": "g", "q_norm": "q.norm",
                      "k_norm": "k.norm", **(names or {})}
        for n in "qkv":
            self.names.setdefault(n + "_bias", self.names[n] + ".b")
        self.proj: Linear | None = None      # [q; k; v; gate] (k and v absent when borrowed)
        self.o: Linear | None = None
        self.bias = self.q_gain = self.k_gain = self.sinks = None

    # ------------------------------------------------------------------------------ cache

    def kv_spec(self) -> KVSpec:
        """The entry this mixer writes, or (borrowed keys) what it needs of the entry it reads:
        a chunk never looks further back than its own length, so it is kept like a window."""
        return KVSpec(self.n_kv_heads, self.head_dim, self.window or self.chunk)

    def _tensor_cores(self, dtype: torch.dtype) -> bool:
        return dtype == torch.bfloat16 and self.head_dim <= ops.MMA_MAX_HEAD_DIM

    def kernel_jobs(self, dtype: torch.dtype):
        jobs = [ops.core_job("sllm_norm_rope_cache")]
        if self.has_gate:
            jobs.append(ops.core_job("sllm_latent_attention"))    # (its per-head gate kernel)
        if self._tensor_cores(dtype):
            jobs.append(ops.attention_mma_library(self.head_dim))
            if self.head_dim % 64 == 0:
                jobs.append(ops.attention_tc_library(self.head_dim))
        else:
            jobs.append(ops.attention_library(self.head_dim))
        return jobs

    # ---------------------------------------------------------------------------- weights

    @property
    def gate_cols(self) -> int:
        """The gate's columns in the fused projection: one per head, up to a multiple of 8 (rows
        of the projection then start on 16-byte boundaries)."""
        return -(-self.n_heads // 8) * 8 if self.has_gate else 0

    def param_specs(self) -> dict[str, ParamSpec]:
        H, G, d, n = self.n_heads, self.n_kv_heads, self.hidden_size, self.names
        specs = {n["q"]: ParamSpec((H * self.qk_dim, d)), n["o"]: ParamSpec((d, H * self.v_dim))}
        if not self.borrow_kv:
            specs[n["k"]] = ParamSpec((G * self.qk_dim, d))
            specs[n["v"]] = ParamSpec((G * self.v_dim, d))
        if self.has_bias:
            specs[n["q_bias"]] = ParamSpec((H * self.qk_dim,), "gain")
            if not self.borrow_kv:
                specs[n["k_bias"]] = ParamSpec((G * self.qk_dim,), "gain")
                specs[n["v_bias"]] = ParamSpec((G * self.v_dim,), "gain")
        if self.qk_norm == "wide":
            specs[n["q_norm"]] = ParamSpec((H * self.qk_dim,), "gain")
            if not self.borrow_kv:
                specs[n["k_norm"]] = ParamSpec((G * self.qk_dim,), "gain")
        if self.has_gate:
            specs[n["g"]] = ParamSpec((H, d))
        return specs

    def _padded_rows(self, t: torch.Tensor, heads: int, size: int) -> torch.Tensor:
        """[heads * size, ...] -> [heads * head_dim, ...] with zeros after each head's rows."""
        if size == self.head_dim:
            return t
        out = t.new_zeros((heads, self.head_dim) + tuple(t.shape[1:]))
        out[:, :size] = t.reshape((heads, size) + tuple(t.shape[1:]))
        return out.view((heads * self.head_dim,) + tuple(t.shape[1:]))

    def load(self, tensors: Mapping[str, torch.Tensor], ctx: BuildContext) -> None:
        put = lambda t: t.to(device=ctx.device, dtype=ctx.dtype)  # noqa: E731
        f32 = lambda t: t.to(device=ctx.device, dtype=torch.float32)  # noqa: E731
        H, G, n = self.n_heads, self.n_kv_heads, self.names
        sizes = {"q": (H, self.qk_dim), "k": (G, self.qk_dim), "v": (G, self.v_dim)}
        mine = "q" if self.borrow_kv else "qkv"
        blocks = [self._padded_rows(put(tensors[n[c]]), *sizes[c]) for c in mine]
        if self.has_gate:
            gate = put(tensors[n["g"]])
            pad = gate.new_zeros((self.gate_cols - H, gate.shape[1]))
            blocks += [gate, pad]
        self.proj = Linear(torch.cat(blocks, 0).contiguous())
        o = put(tensors[n["o"]])
        self.o = Linear(self._padded_rows(o.t(), H, self.v_dim).t().contiguous())
        if self.has_bias:
            self.bias = torch.cat([self._padded_rows(f32(tensors[n[c + "_bias"]]), *sizes[c])
                                   for c in mine], 0).contiguous()
        if self.qk_norm == "wide":
            self.q_gain = self._padded_rows(f32(tensors[n["q_norm"]]), *sizes["q"]).contiguous()
            if not self.borrow_kv:
                self.k_gain = self._padded_rows(f32(tensors[n["k_norm"]]), *sizes["k"]).contiguous()
        if self.zero_sink:
            self.sinks = torch.zeros(H, dtype=torch.float32, device=ctx.device)

    # ---------------------------------------------------------------------------- forward

    def forward(self, x, batch, cache: CacheView, write: bool, position: PositionEncoding):
        return self.o(self.heads_out(x, batch, cache, write, position))

    def heads_out(self, x, batch, cache: CacheView, write: bool, position: PositionEncoding,
                  out: torch.Tensor | None = None) -> torch.Tensor:
        """The concatenated heads' outputs [N, H * head_dim], gated: what
        the output matrix multiplies.  ``out``: where to put them (may be a column slice; in a
        padded step it must hold zeros, since padding tokens get no attention output)."""
        H, G, hd = self.n_heads, self.n_kv_heads, self.head_dim
        if self.borrow_kv == write:
            raise ValueError("a mixer with keys of its own writes its cache entry; one that "
                             "borrows them reads another run's")
        if not position.rotary_tables:
            raise ValueError("this mixer rotates its queries and keys by a table of angles")
        proj = self.proj(x)
        ops.norm_rope_kv_write(proj, batch.positions, batch.token_row, cache.pages,
                               cache.block_table, cache.page_size, H, G, hd, self.qk_dim, self.eps,
                               has_kv=not self.borrow_kv, write=write, bias=self.bias,
                               q_gain=self.q_gain, k_gain=self.k_gain,
                               unit_after=self.qk_norm == "unit_after", cos=position.cos,
                               sin=position.sin, interleaved=position.interleaved)
        q = proj[:, :H * hd]
        if out is None:
            # (padding tokens get no attention output: zeros, so that what follows stays finite)
            out = (torch.zeros if batch.padded else torch.empty)(
                (proj.shape[0], H * hd), dtype=proj.dtype, device=proj.device)
        g0 = (H + (0 if self.borrow_kv else 2 * G)) * hd
        gate = proj[:, g0:g0 + H] if self.has_gate else None
        if self._tensor_cores(proj.dtype):
            # (the gate in the kernels' epilogues, where they have one)
            if self._attend_tensor_cores(q, out, batch, cache, gate):
                gate = None
        else:
            ops.attention_simt(q, cache.pages, cache.block_table, cache.page_size,
                               batch.row_start, batch.row_pos0, out, batch.n_rows, batch.max_new,
                               H, G, hd, self.scale, self.window, None, self.sinks,
                               softcap=self.softcap, chunk=self.chunk)
        if gate is not None:
            ops.head_gate(out, gate, H)
        return out

    def _attend_tensor_cores(self, q, out, batch, cache: CacheView, gate) -> bool:
        """Rows with several new tokens go to the tcgen05 kernel where the longest of them fills
        one of its query tiles, else to the wide ``mma.sync`` kernel; rows with one token to the
        split kernel (as :class:`~.attention.GQAttention` does).  All take the cap, the chunks
        and the sink.  Returns whether the gate was applied (the tcgen05 kernel has none: a step
        that uses it gates all of its rows afterwards)."""
        H, G, hd = self.n_heads, self.n_kv_heads, self.head_dim
        gated = True
        common = (q, cache.pages, cache.block_table, cache.page_size, batch.row_start,
                  batch.row_pos0, out)
        if batch.n_multi and batch.max_new_multi * (H // G) >= TC_MIN_PACKED_QUERIES and \
                out.stride(0) % 8 == 0 and \
                ops.attention_tc_supports(H, G, hd, cache.page_size, self.window, biased=True):
            # scores, probabilities and output in tensor memory
            ops.attention_tc(*common, batch.multi_rows, batch.n_multi, batch.max_new_multi, H, G,
                             hd, self.scale, self.window, None, self.sinks, biased=True,
                             softcap=self.softcap, chunk=self.chunk)
            gated, gate = False, None
        elif batch.n_multi:
            ops.attention_mma(*common, batch.multi_rows, batch.n_multi, batch.max_new_multi, H, G,
                              hd, self.scale, self.window, split=False, sinks=self.sinks,
                              softcap=self.softcap, chunk=self.chunk, gate=gate)
        if batch.n_single:
            reach = self.window or self.chunk
            context = batch.context_bucket if reach is None \
                else min(batch.context_bucket, reach + 64)
            n_splits = decode_splits(batch.n_single * G * (-(-(H // G) // 16)), context,
                                     ops.attention_decode_slots(hd))
            scratch = None
            if n_splits > 1:
                scratch = torch.empty(ops.attention_mma_scratch_floats(q.shape[0], H, hd, n_splits),
                                      dtype=torch.float32, device=q.device)
            ctas = batch.n_single * G * (-(-(H // G) // 16)) * n_splits
            ops.attention_mma(*common, batch.single_rows, batch.n_single, 1, H, G, hd, self.scale,
                              self.window, split=True, n_splits=n_splits, scratch=scratch,
                              sinks=self.sinks, softcap=self.softcap, chunk=self.chunk, gate=gate,
                              merge_inside=ctas <= ops.attention_decode_slots(hd))
        return gated

    # -- for a block that multiplies several branches' activations by one joined output matrix

    def out_segments(self):
        """[(the output matrix [hidden, H * head_dim], its weight in the layer's sum)]."""
        return [(self.o.weight, 1.0)]

    def release_out(self) -> None:
        self.o = None

    def activations_into(self, x, batch, cache: CacheView, write: bool, position, outs) -> None:
        self.heads_out(x, batch, cache, write, position, out=outs[0])
