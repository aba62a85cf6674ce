"""Latent attention: queries, keys and values pass through low-rank latents, and the cache holds
one latent per token instead of keys and values per head.

    c_q = rmsnorm(W_dq x) g_q                q_h = W_uq,h c_q = [q_h^n (dim) | q_h^r (rot_dim)]
    [c' | k^r] = W_dkv x                     c = rmsnorm(c') g_kv   (kv_rank entries)
    k_h = [W_uk,h c | rot(k^r)]              v_h = W_uv,h c         (k^r is shared by all heads)
    score_h(i, j) = scale * (q_h^n(i) . W_uk,h c(j) + rot(q_h^r(i)) . rot(k^r(j))),  j <= i
    o_h = sigmoid(W_g x)_h * sum_j softmax_j(score_h) v_h(j)        out = W_o [o_1 .. o_H]

Only ``c`` and ``rot(k^r)`` are cached, as ONE vector per token.  The products with W_uk and W_uv
are moved to the query's side (the absorbed form), which needs no key or value per head at all:

    score_h(i, j) = scale * [W_uk,h^T q_h^n(i) | rot(q_h^r(i))] . [c(j) | rot(k^r(j))]
    o_h = gate * W_uv,h (sum_j p_h(i, j) c(j))

so the attention itself is the engine's paged attention with one kv head whose "key" is the cached
vector and whose "value" is the same vector's leading ``kv_rank`` entries (a cache of one plane,
:class:`~.base.KVSpec` ``planes=1``); all query heads share every cache tile they read.  The
rotation (split-half pairing over the first ``rot_dims`` entries of the rotated part) comes from
the layer's rotary position encoding, whose tables have ``rot_dims / 2`` columns.

Every size is a constructor argument; ``gate`` False leaves the output gate out.  Norms,
rotation, scores and softmax are 32-bit; the cache and the products' operands have the compute
dtype.
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


#: cached vectors of up to this many entries: the split decode kernel's last CTA merges the
#: splits itself.  Beyond it the merge kernel, which spreads a row's heads over CTAs, is faster
#: than one CTA walking 16 heads of long vectors (at 256 entries: 13 + 8 us against 26 us).
MERGE_INSIDE_MAX_DIM = 128


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    pad_safe = True   # padding tokens are not stored; rows without tokens leave the kernels

    def __init__(self, hidden_size: int, n_heads: int, dim: int, rot_dim: int, value_dim: int,
                 q_rank: int, kv_rank: int, scale: float, eps: float, gate: bool = True,
                 names: Mapping[str, str] | None = None) -> None:
        if min(hidden_size, n_heads, dim, value_dim, q_rank, kv_rank) < 1 or rot_dim < 0:
            raise ValueError("latent attention: sizes must be positive")
        self.hidden_size, self.n_heads, self.dim, self.rot_dim = hidden_size, n_heads, dim, rot_dim
        self.value_dim, self.q_rank, self.kv_rank = value_dim, q_rank, kv_rank
        self.scale, self.eps, self.has_gate = float(scale), float(eps), bool(gate)
        #: the cached vector's size: latent, rotated key part, zeros up to a multiple of 16
        self.head_dim = -(-(kv_rank + rot_dim) // 16) * 16
        if self.head_dim > ops.SIMT_MAX_HEAD_DIM:
            raise ValueError(f"kv_rank + rot_dim = {kv_rank + rot_dim}: the attention kernels "
                             f"take cached vectors of up to {ops.SIMT_MAX_HEAD_DIM} entries")
        self.names = {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv",
                      "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv", "g": "g", "o": "o",
                      **(names or {})}
        self.down: Linear | None = None     # [dq; dkv; g] in one product
        self.uq: Linear | None = None
        self.o: Linear | None = None
        self.uk = self.uk_t = self.uv = self.uv_t = self.q_gain = self.kv_gain = None
        self._small = False

    def kv_spec(self) -> KVSpec:
        return KVSpec(1, self.head_dim, None, planes=1)

    def _tensor_cores(self, dtype: torch.dtype) -> bool:
        return dtype == torch.bfloat16 and self.head_dim <= ops.MMA_MAX_HEAD_DIM

    def kernel_jobs(self, dtype: torch.dtype):
        jobs = [ops.core_job("sllm_latent_attention")]
        if self._tensor_cores(dtype):
            jobs.append(ops.attention_mma_library(self.head_dim))
            if ops.attention_tc_supports(self.n_heads, 1, self.head_dim, 16, None):
                jobs.append(ops.attention_tc_library(self.head_dim))
        else:
            jobs.append(ops.attention_library(self.head_dim))
        return jobs

    def param_specs(self) -> dict[str, ParamSpec]:
        n, H, d = self.names, self.n_heads, self.hidden_size
        specs = {n["dq"]: ParamSpec((self.q_rank, d)),
                 n["dq_norm"]: ParamSpec((self.q_rank,), "gain"),
                 n["uq"]: ParamSpec((H * (self.dim + self.rot_dim), self.q_rank)),
                 n["dkv"]: ParamSpec((self.kv_rank + self.rot_dim, d)),
                 n["dkv_norm"]: ParamSpec((self.kv_rank,), "gain"),
                 n["uk"]: ParamSpec((H * self.dim, self.kv_rank)),
                 n["uv"]: ParamSpec((H * self.value_dim, self.kv_rank)),
                 n["o"]: ParamSpec((d, H * self.value_dim))}
        if self.has_gate:
            specs[n["g"]] = ParamSpec((H, d))
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], ctx: BuildContext) -> None:
        put = lambda t: t.to(device=ctx.device, dtype=ctx.dtype)  # noqa: E731
        f32 = lambda t: t.to(device=ctx.device, dtype=torch.float32).contiguous()  # noqa: E731
        n, H = self.names, self.n_heads
        blocks = [put(tensors[n["dq"]]), put(tensors[n["dkv"]])]
        if self.has_gate:
            blocks.append(put(tensors[n["g"]]))
        self.down = Linear(torch.cat(blocks, 0).contiguous())
        self.uq = Linear(put(tensors[n["uq"]]).contiguous())
        self.o = Linear(put(tensors[n["o"]]).contiguous())
        self.uk = put(tensors[n["uk"]]).view(H, self.dim, self.kv_rank).contiguous()
        # [H, kv_rank, dim]: the absorb product's matrix with the reduction index last
        self.uk_t = self.uk.transpose(1, 2).contiguous()
        self.uv = put(tensors[n["uv"]]).view(H, self.value_dim, self.kv_rank).contiguous()
        # [H, kv_rank, value_dim]: the value product's matrix with the output index last, for
        # steps of few tokens (uk has that layout for the absorb product as it is)
        self.uv_t = self.uv.transpose(1, 2).contiguous()
        self._small = ctx.dtype == torch.bfloat16 \
            and ops.latent_small_supports(self.dim, self.kv_rank) \
            and ops.latent_small_supports(self.kv_rank, self.value_dim)
        self.q_gain, self.kv_gain = f32(tensors[n["dq_norm"]]), f32(tensors[n["dkv_norm"]])

    # ------------------------------------------------------------------------- forward

    def forward(self, x, batch, cache: CacheView, write: bool, position: PositionEncoding):
        if not getattr(position, "rotary_tables", False):
            raise ValueError("latent attention needs a rotary position encoding's tables")
        cos, sin = position.cos, position.sin
        H, d, r, R, V, Dp = (self.n_heads, self.dim, self.rot_dim, self.kv_rank, self.value_dim,
                             self.head_dim)
        n = x.shape[0]
        a = self.down(x)                                        # [N, q_rank + R + r (+ H)]
        cq = torch.empty((n, self.q_rank), dtype=a.dtype, device=a.device)
        ops.latent_prep(a, self.q_rank, self.q_rank, R, r, self.q_gain, self.kv_gain, self.eps,
                        batch.positions, batch.token_row, cos, sin, cq, cache.pages,
                        cache.block_table, cache.page_size, write)
        q = self.uq(cq)                                         # [N, H * (d + r)]
        qlat = torch.empty((n, H * Dp), dtype=q.dtype, device=q.device)
        small = self._small and n <= ops.LATENT_SMALL_MAX_TOKENS
        gate = a[:, self.q_rank + R + r:] if self.has_gate else None
        if small:
            # steps of few tokens: absorb product and rotation in one launch, value product and
            # gate in another
            ops.latent_small(q, d + r, self.uk, qlat, Dp, rot=(r, batch.positions, cos, sin))
            olat = (torch.zeros if batch.padded else torch.empty)(
                (n, H * Dp), dtype=q.dtype, device=q.device)
            self._attend(qlat, olat, batch, cache)
            o = torch.empty((n, H * V), dtype=q.dtype, device=q.device)
            ops.latent_small(olat, Dp, self.uv_t, o, V, gate=gate)
            return self.o(o)
        if q.dtype == torch.bfloat16:
            # the library's batched product, one batch per head, straight into its columns
            torch.bmm(q.view(n, H, d + r)[:, :, :d].transpose(0, 1), self.uk,
                      out=qlat.view(n, H, Dp)[:, :, :R].transpose(0, 1))
        else:
            ops.head_product(q, d + r, self.uk_t, qlat, Dp)
        ops.latent_q_rot(q, H, d, r, batch.positions, cos, sin, qlat, R)
        # (padding tokens get no attention output: zeros, so that what follows stays finite)
        olat = (torch.zeros if batch.padded else torch.empty)(
            (n, H * Dp), dtype=q.dtype, device=q.device)
        self._attend(qlat, olat, batch, cache)
        o = torch.empty((n, H * V), dtype=q.dtype, device=q.device)
        if q.dtype == torch.bfloat16:
            torch.bmm(olat.view(n, H, Dp)[:, :, :R].transpose(0, 1), self.uv.transpose(1, 2),
                      out=o.view(n, H, V).transpose(0, 1))
        else:
            ops.head_product(olat, Dp, self.uv, o, V)
        if self.has_gate:
            ops.head_gate(o, gate, H)
        return self.o(o)

    def _attend(self, q, out, batch, cache: CacheView) -> None:
        """One kv head, every query head in its group, the cached vector as key and value."""
        H, Dp = self.n_heads, self.head_dim
        common = (q, cache.pages, cache.block_table, cache.page_size, batch.row_start,
                  batch.row_pos0, out)
        if not self._tensor_cores(q.dtype):
            ops.attention_simt(*common, batch.n_rows, batch.max_new, H, 1, Dp, self.scale, None)
            return
        if batch.n_multi:
            if ops.attention_tc_supports(H, 1, Dp, cache.page_size, None) \
                    and batch.max_new_multi * H >= TC_MIN_PACKED_QUERIES:
                ops.attention_tc(*common, batch.multi_rows, batch.n_multi, batch.max_new_multi,
                                 H, 1, Dp, self.scale)
            else:
                ops.attention_mma(*common, batch.multi_rows, batch.n_multi, batch.max_new_multi,
                                  H, 1, Dp, self.scale, None, split=False)
        if batch.n_single:
            base = batch.n_single * (-(-H // 16))
            n_splits = decode_splits(base, batch.context_bucket, ops.attention_decode_slots(Dp))
            scratch = None
            if n_splits > 1:
                scratch = torch.empty(ops.attention_mma_scratch_floats(q.shape[0], H, Dp, n_splits),
                                      dtype=torch.float32, device=q.device)
            ops.attention_mma(*common, batch.single_rows, batch.n_single, 1, H, 1, Dp, self.scale,
                              None, split=True, n_splits=n_splits, scratch=scratch,
                              merge_inside=Dp <= MERGE_INSIDE_MAX_DIM
                              and base * n_splits <= ops.attention_decode_slots(Dp))
