"""The generic decoder: embedding, the layers of a :class:`ModelSpec` in its run order, final
norm, output matrix on the wanted rows only.

embed -> blocks -> final norm -> output matrix is src/scratch_llm/model.py:471-505 of the
reference, which computes logits at every position (:480) and lets callers slice the last one
(src/scratch_llm/serving/continuous.py:496-498); here only the rows named by
``batch.logit_index`` pass through the final norm and the output matrix.
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..config.spec import ModelSpec, PartSpec
from ..kernels import ops
from ..parts import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, SIDE_INPUTS,
                     STREAM_JOINS, TOKEN_MIXES, BuildContext, CacheView, KVSpec, StateSpec, make)
from ..parts.linear import Linear
from ..parts.stream import Current, Normed, StreamSink
from ..weights.loader import ParamSpec


def _spec_key(spec: PartSpec):
    return (spec.kind, tuple(sorted((k, repr(v)) for k, v in spec.args.items())))


#: kind of part (a value of a block's ``ROLES``) -> (registry, name used in error messages)
PART_KINDS = {"mixer": (MIXERS, "mixer"), "feed_forward": (FEED_FORWARDS, "feed-forward"),
              "norm": (NORMS, "norm"), "position": (POSITION_ENCODINGS, "position encoding"),
              "side": (SIDE_INPUTS, "side input"), "token_mix": (TOKEN_MIXES, "token mix")}


def _tensor_name(prefix: str, name: str) -> str:
    """A part's tensor name in the model folder: below the part's prefix; the prefix itself for
    the name ""; and as it stands, without its "/", for an absolute name (a tensor that several
    parts share, which then all receive the same device tensor)."""
    if name.startswith("/"):
        return name[1:]
    return f"{prefix}.{name}" if name else prefix


class _HeadEntry:
    """The output matrix as the part that follows the final norm: it can finish a norm handed
    over to it where its product can (see :mod:`scratch_llm_b200.parts.stream`)."""

    def __init__(self, model: "DecoderModel") -> None:
        self.model = model

    def accepts_normed(self, n_tokens: int) -> bool:
        head = self.model.lm_head
        return head is not None and head.takes_normed(n_tokens)


class DecoderModel:
    def __init__(self, spec: ModelSpec) -> None:
        self.spec = spec
        self.ctx: BuildContext | None = None
        positions: dict = {}
        self.blocks = []
        self._named_parts: list[tuple[str, object]] = []
        for layer in spec.layers:
            try:
                block_cls = BLOCKS[layer.block]
            except KeyError:
                raise ValueError(f"unknown block {layer.block!r}; registered: "
                                 f"{', '.join(sorted(BLOCKS))}") from None
            roles = dict(getattr(block_cls, "ROLES", {}))
            optional = set(getattr(block_cls, "OPTIONAL_ROLES", ()))
            if not (set(roles) - optional <= set(layer.parts) <= set(roles)):
                raise ValueError(f"layer {layer.prefix!r}: block {layer.block!r} has the roles "
                                 f"{sorted(roles)} (optional: {sorted(optional)}), the layer's "
                                 f"spec gives {sorted(layer.parts)}")
            roles = {role: kind for role, kind in roles.items() if role in layer.parts}
            if sum(kind == "mixer" for kind in roles.values()) > 1:
                raise ValueError(f"block {layer.block!r} has several mixers: a layer has one "
                                 "cache entry, which one mixer owns")
            built = {}
            for role, kind in roles.items():
                part_spec = layer.parts[role]
                if kind not in PART_KINDS:
                    raise ValueError(f"block {layer.block!r}: role {role!r} has the unknown kind "
                                     f"{kind!r} (kinds: {', '.join(PART_KINDS)})")
                table, what = PART_KINDS[kind]
                if kind == "position":   # one table serves every layer that asks for the same
                    key = _spec_key(part_spec)
                    if key not in positions:
                        positions[key] = make(table, what, part_spec)
                    built[role] = positions[key]
                else:
                    built[role] = make(table, what, part_spec)
                    self._named_parts.append(
                        (f"{layer.prefix}.{layer.names.get(role, role)}", built[role]))
            block = block_cls(**built, **dict(getattr(layer, "block_args", None) or {}))
            block.parts = built          # role -> part, for whoever walks the model's parts
            block.cache_owner = next((built[r] for r, k in roles.items() if k == "mixer"), None)
            self.blocks.append(block)
        self._positions = list(positions.values())
        # joins of the stream with the embedding output that some runs ask for
        self.joins = []
        for join in spec.joins:
            part = make(STREAM_JOINS, "stream join", join.part)
            self.joins.append(part)
            self._named_parts.append((join.prefix, part))
        self._keeps_first = any(run.join is not None for run in spec.order)
        #: for looking into a model: called as ``stream_probe(run index, resid, pending)`` after
        #: every run of a layer in steps that run eagerly (the stream is ``resid`` plus what is
        #: pending, if anything is); None in normal use
        self.stream_probe = None
        # per run: the (norm, part) the NEXT run's block starts with, for blocks that ask
        self._next_entry: list = []
        for i, run in enumerate(spec.order):
            block = self.blocks[run.layer]
            nxt = self.blocks[spec.order[i + 1].layer] if i + 1 < len(spec.order) else None
            entry = nxt.entry() if nxt is not None and hasattr(nxt, "entry") else None
            self._next_entry.append(entry if getattr(block, "takes_next_entry", False) else None)
        self.final_norm = make(NORMS, "norm", spec.final_norm)
        self._named_parts.append((spec.final_norm_name, self.final_norm))
        # a norm between the embedding and the first layer, for designs that have one
        self.embed_norm = None
        if spec.embed_norm is not None:
            self.embed_norm = make(NORMS, "norm", spec.embed_norm)
            if not hasattr(self.embed_norm, "in_place"):
                raise ValueError(f"norm {spec.embed_norm.kind!r} cannot norm the stream in place, "
                                 "which the norm after the embedding does")
            self._named_parts.append((spec.embed_norm_name, self.embed_norm))
        # what the first run starts with, for the embedding (if that block says, its norm's
        # factor is one number per token and its gain a vector `weight`)
        first = self.blocks[spec.order[0].layer] if spec.order else None
        entry = first.entry() if first is not None and hasattr(first, "entry") else None
        self._first_entry = entry if (entry is not None and getattr(entry[0], "deferrable", False)
                                      and hasattr(entry[1], "accepts_normed")
                                      and spec.embed_norm is None) else None
        # the last run may prepare the final norm for the output matrix in steps that want the
        # logits of every token in order (decode steps), where no rows are gathered in between
        last = self.blocks[spec.order[-1].layer] if spec.order else None
        self._final_entry = ((self.final_norm, _HeadEntry(self))
                             if getattr(last, "takes_next_entry", False) else None)
        self._first_wants_current = bool(getattr(first, "wants_current", False))
        self._inv_freq: torch.Tensor | None = None
        self.embedding: torch.Tensor | None = None
        self.lm_head: Linear | None = None

    def all_parts(self):
        """Every part of the model and every block, once (a position encoding that several
        layers share comes once)."""
        seen: dict[int, object] = {}
        for block in self.blocks:
            seen.setdefault(id(block), block)
            for part in block.parts.values():
                seen.setdefault(id(part), part)
        for part in self.joins:
            seen.setdefault(id(part), part)
        seen.setdefault(id(self.final_norm), self.final_norm)
        if self.embed_norm is not None:
            seen.setdefault(id(self.embed_norm), self.embed_norm)
        return list(seen.values())

    # --------------------------------------------------------------------------- weights

    def param_specs(self) -> dict[str, ParamSpec]:
        s = self.spec
        specs = {s.embed_name: ParamSpec((s.vocab_size, s.hidden_size))}
        for prefix, part in self._named_parts:
            for name, p in part.param_specs().items():
                full = _tensor_name(prefix, name)
                if full in specs and specs[full] != p:
                    raise ValueError(f"two parts want the tensor {full!r} with different specs")
                specs[full] = p
        if not s.tie_embeddings:
            specs[s.lm_head_name] = ParamSpec((s.vocab_size, s.hidden_size))
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor], ctx: BuildContext) -> None:
        s = self.spec
        self.ctx = ctx
        shared: dict[str, torch.Tensor] = {}   # absolute names: one device tensor for all
        for prefix, part in self._named_parts:
            mine = {}
            for name, p in part.param_specs().items():
                full = _tensor_name(prefix, name)
                if name.startswith("/"):
                    if full not in shared:
                        dt = ctx.dtype if p.kind == "matrix" else \
                            torch.float32 if p.kind == "gain" else torch.int32
                        shared[full] = tensors[full].to(device=ctx.device, dtype=dt).contiguous()
                    mine[name] = shared[full]
                else:
                    mine[name] = tensors[full]
            part.load(mine, ctx)
        for pos in self._positions:
            pos.load({}, ctx)
        self.embedding = tensors[s.embed_name].to(device=ctx.device, dtype=ctx.dtype).contiguous()
        head = self.embedding if s.tie_embeddings else \
            tensors[s.lm_head_name].to(device=ctx.device, dtype=ctx.dtype).contiguous()
        self.lm_head = Linear(head)
        if s.position_sinusoid_base > 0:
            # base^(-2i / d) in 64-bit, rounded once; the angle p * inv_freq is 32-bit arithmetic
            pairs = (s.hidden_size + 1) // 2
            inv = torch.tensor([s.position_sinusoid_base ** (-2.0 * i / s.hidden_size)
                                for i in range(pairs)], dtype=torch.float64)
            self._inv_freq = inv.to(torch.float32).to(ctx.device)

    # ----------------------------------------------------------------------------- cache

    def cache_specs(self) -> tuple[list[KVSpec | None], list[StateSpec | None]]:
        """What each cache entry needs: the spec of the run that writes it."""
        n = self.spec.n_cache_entries
        ids = sorted({r.cache for r in self.spec.order})
        if ids != list(range(n)):
            raise ValueError(f"cache entries must be numbered 0..{n - 1}, got {ids}")
        kv: list[KVSpec | None] = [None] * n
        st: list = [None] * n
        # per cache entry: how many of its state tensors are the mixer's (the rest, after
        # them, are the block's own), and whether each side holds one tensor or a tuple
        self._state_split: dict[int, tuple[int, bool, int, bool]] = {}
        for run in self.spec.order:
            if run.write:
                block = self.blocks[run.layer]
                mixer = block.cache_owner
                mine = mixer.state_spec() if mixer is not None else None
                own = block.state_spec() if hasattr(block, "state_spec") else None
                if mixer is not None:
                    kv[run.cache] = mixer.kv_spec()
                if own is None:
                    st[run.cache] = mine
                    continue
                as_tuple = lambda v: () if v is None else tuple(v) if isinstance(v, (tuple, list)) else (v,)  # noqa: E731
                a, b = as_tuple(mine), as_tuple(own)
                st[run.cache] = a + b
                self._state_split[run.cache] = (len(a), isinstance(mine, (tuple, list)),
                                                len(b), isinstance(own, (tuple, list)))
        # a run that only READS an entry may look further back than the run that writes it (a
        # wider window, or no window at all): the entry then keeps what its farthest reader needs
        for run in self.spec.order:
            mixer = self.blocks[run.layer].cache_owner
            need = mixer.kv_spec() if (not run.write and mixer is not None) else None
            have = kv[run.cache]
            if need is None or have is None:
                continue
            if (need.n_kv_heads, need.head_dim, need.planes) != \
                    (have.n_kv_heads, have.head_dim, have.planes):
                raise ValueError(f"layer {run.layer} reads cache entry {run.cache}, whose keys "
                                 f"have another shape ({have} against {need})")
            if have.window is not None and (need.window is None or need.window > have.window):
                kv[run.cache] = KVSpec(have.n_kv_heads, have.head_dim, need.window, have.planes)
        return kv, st

    def _states_of(self, cache, entry: int):
        """(the mixer's state, the block's state) of a cache entry, each as its part declared
        it (one tensor, a tuple, or None)."""
        state = cache.states[entry]
        split = getattr(self, "_state_split", {}).get(entry)
        if split is None:
            return state, None
        n_a, a_tuple, n_b, b_tuple = split
        a, b = state[:n_a], state[n_a:n_a + n_b]
        return ((a if a_tuple else a[0]) if n_a else None), (b if b_tuple else b[0])

    def kernel_jobs(self, dtype: torch.dtype):
        """The CUDA libraries this model's steps use in ``dtype``, as jobs for
        :func:`scratch_llm_b200.kernels.ops.prepare_jobs`, if its parts say what they need
        (``kernel_jobs(dtype)``); None if none does (everything is then prepared by head size)."""
        said = [p.kernel_jobs(dtype) for p in self.all_parts() if hasattr(p, "kernel_jobs")]
        said = [jobs for jobs in said if jobs is not None]
        if not said:
            return None
        names = ["sllm_elementwise", "sllm_sampling", "sllm_stream_ops"]
        names += ["sllm_gemm_simt"] if dtype == torch.float32 else ["sllm_gemv_mma", "sllm_gemv_tma"]
        return [ops.core_job(n) for n in names] + [job for jobs in said for job in jobs]

    def head_dims(self) -> list[int]:
        return sorted({p.head_dim for p in self.all_parts()
                       if isinstance(getattr(p, "head_dim", None), int)})

    # --------------------------------------------------------------------------- forward

    def _embed(self, batch, resid: torch.Tensor):
        """The tokens' embeddings into the stream.  In steps of a few tokens the first run's
        norm is prepared for the product after it on the way (returned as what is pending),
        where that norm and that product can (scratch_llm_b200.parts.stream)."""
        s = self.spec
        n, d = batch.n_tokens, s.hidden_size
        if s.position_sinusoid_base > 0 or self._first_wants_current:
            # the stream, and its copy in the compute dtype for a first block whose branches
            # read the stream as it is
            x = resid
            if self._first_wants_current and self.embedding.dtype != torch.float32:
                x = torch.empty((n, d), dtype=self.embedding.dtype, device=resid.device)
            ops.embed_positional(batch.token_ids, batch.positions, self.embedding, resid,
                                 None if x is resid else x, batch.pending_tokens,
                                 s.embedding_multiplier, self._inv_freq)
            return Current(x) if self._first_wants_current else None
        entry = self._first_entry
        if (entry is not None and n <= StreamSink.MAX_TOKENS and d % 8 == 0
                and self.embedding.dtype == torch.bfloat16 and entry[1].accepts_normed(n)):
            norm = entry[0]
            x_out = torch.empty((n, d), dtype=torch.bfloat16, device=resid.device)
            shares = torch.empty((d // 8, 8), dtype=torch.float32, device=resid.device)
            ops.embed_prepare(batch.token_ids, self.embedding, resid, batch.pending_tokens,
                              s.embedding_multiplier, norm.weight, x_out, shares)
            return Normed(x_out, shares, d, norm.eps, norm)
        ops.embed(batch.token_ids, self.embedding, resid, batch.pending_tokens,
                  scale=s.embedding_multiplier)
        return None

    def forward(self, batch, cache) -> torch.Tensor | None:
        """Run the batch's tokens from the cache; returns logits [n_out, vocab] in 32-bit, or
        None when no logits are wanted."""
        s = self.spec
        resid = torch.empty((batch.n_tokens, s.hidden_size), dtype=torch.float32,
                            device=self.ctx.device)
        pending = self._embed(batch, resid)
        if self.embed_norm is not None:
            if pending is not None:
                raise ValueError("a norm after the embedding needs an embedding that leaves "
                                 "nothing pending")
            self.embed_norm.in_place(resid)
        first = None
        if self._keeps_first:
            if pending is not None:
                raise ValueError("a model that joins the stream with the embedding output needs "
                                 "an embedding that leaves nothing pending")
            first = resid.clone()
        for i, run in enumerate(s.order):
            if run.join is not None:
                if pending is not None:
                    raise ValueError("a join takes a stream with nothing pending")
                resid = self.joins[run.join].forward(resid, first)
            pages, group = cache.entry_pages(run.cache)
            state, block_state = self._states_of(cache, run.cache)
            view = CacheView(pages=pages,
                             block_table=batch.block_tables[group] if group is not None else None,
                             page_size=cache.page_size, state=state, block_state=block_state)
            block = self.blocks[run.layer]
            if i == len(s.order) - 1 and self._final_entry is not None and batch.wants_every_token:
                pending = block.forward(resid, pending, batch, view, run.write,
                                        next_entry=self._final_entry)
            elif self._next_entry[i] is not None:
                # what the next run starts with, so that this block's last product may prepare
                # it (the final norm works on gathered rows: nothing is prepared for it)
                pending = block.forward(resid, pending, batch, view, run.write,
                                        next_entry=self._next_entry[i])
            else:
                pending = block.forward(resid, pending, batch, view, run.write)
            if self.stream_probe is not None:
                self.stream_probe(i, resid, pending)
        if batch.n_out == 0:
            return None
        if isinstance(pending, Normed):      # prepared by the last run: every row, in order
            h = self.final_norm.forward(resid, pending)
        else:
            h = self.final_norm.forward(resid, pending, out_rows=batch.logit_index)
        logits = self.lm_head(h, out_dtype=torch.float32)
        if s.logit_scale != 1.0 or s.logit_softcap > 0:
            ops.logit_cap(logits, s.logit_scale, s.logit_softcap)
        return logits


def build_model(config) -> DecoderModel:
    """The model of a typed configuration, without weights and without touching a device."""
    from ..config import get_architecture

    arch = get_architecture(config.architecture)
    spec = config.model_spec()
    return arch.model_factory(spec) if arch.model_factory else DecoderModel(spec)
