"""Arrangements of a layer's parts around the residual stream.

``pre_norm``: ``x + Mixer(Norm(x))`` then ``x + FeedForward(Norm(x))``
(src/scratch_llm/model.py:423-436 of the reference).  The residual stream is a 32-bit tensor
that every norm call updates in place: a block returns its last delta as *pending*, and the
next norm (the next block's, or the model's final norm) adds it while it reads the stream, so
the sum costs no pass of its own.
"""

from __future__ import annotations

import torch

from .base import Block, CacheView, FeedForward, Mixer, Norm, PositionEncoding
from .linear import Linear
from .registry import register_block
from .stream import Current, StreamSink, Terms


@register_block("pre_norm")
class PreNormBlock(Block):
    ROLES = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm",
             "feed_forward_norm": "norm", "position": "position"}
    pad_safe = True   # the arrangement itself touches no token: its parts decide

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm,
                 feed_forward_norm: Norm, position: PositionEncoding) -> None:
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm
        self.position = position

    #: forward() takes next_entry=: what follows this block in the run order
    takes_next_entry = True

    def entry(self):
        """(the norm that takes the pending delta, the part that takes the norm's output)."""
        return self.mixer_norm, self.mixer

    @staticmethod
    def _sink(resid: torch.Tensor, producer, norm, consumer, n_tokens: int):
        """A sink for ``producer``'s output if it, the norm after it and the part after that
        all can hand the norm over (scratch_llm_b200.parts.stream), else None."""
        if n_tokens > StreamSink.MAX_TOKENS:    # (first: larger steps should pay nothing here)
            return None
        if norm is None or consumer is None or not getattr(producer, "accepts_sink", False) \
                or not getattr(norm, "deferrable", False):
            return None
        can = getattr(consumer, "accepts_normed", None)
        return StreamSink(resid, norm) if can is not None and can(n_tokens) else None

    def forward(self, resid: torch.Tensor, pending, batch, cache: CacheView, write: bool,
                next_entry=None):
        n = resid.shape[0]
        h = self.mixer_norm.forward(resid, pending)
        sink = self._sink(resid, self.mixer, self.feed_forward_norm, self.feed_forward, n)
        if sink is None:
            a = self.mixer.forward(h, batch, cache, write, self.position)
        else:
            a = self.mixer.forward(h, batch, cache, write, self.position, sink=sink)
        h = self.feed_forward_norm.forward(resid, a)
        norm, consumer = next_entry if next_entry is not None else (None, None)
        sink = self._sink(resid, self.feed_forward, norm, consumer, n)
        if sink is None:
            return self.feed_forward.forward(h)
        return self.feed_forward.forward(h, sink=sink)


@register_block("branch_norm")
class BranchNormBlock(Block):
    """Norm on a branch's OUTPUT only: ``x <- x + norm(Mixer(x))``, then (if the layer has one)
    ``x <- x + norm(FeedForward(x))``, then (if it has one) ``x <- x + norm(Side(x, tokens))``.
    The branches read the stream as it is.  The stream is 32-bit; every add hands on a copy in
    the compute dtype for the next branch to read, so that no cast kernel runs (in 32-bit the
    stream itself is that copy)."""

    ROLES = {"mixer": "mixer", "mixer_norm": "norm", "feed_forward": "feed_forward",
             "feed_forward_norm": "norm", "side": "side", "side_norm": "norm",
             "position": "position"}
    OPTIONAL_ROLES = frozenset({"feed_forward", "feed_forward_norm", "side", "side_norm"})
    pad_safe = True   # the arrangement itself touches no token: its parts decide
    #: the block before this one (or the embedding) should hand on a :class:`~.stream.Current`
    wants_current = True

    def __init__(self, mixer: Mixer, mixer_norm: Norm, position: PositionEncoding,
                 feed_forward: FeedForward | None = None, feed_forward_norm: Norm | None = None,
                 side=None, side_norm: Norm | None = None) -> None:
        if (feed_forward is None) != (feed_forward_norm is None) or \
                (side is None) != (side_norm is None):
            raise ValueError("a branch and the norm of its output come together")
        self.mixer, self.mixer_norm, self.position = mixer, mixer_norm, position
        self.feed_forward, self.feed_forward_norm = feed_forward, feed_forward_norm
        self.side, self.side_norm = side, side_norm

    @staticmethod
    def _join(resid: torch.Tensor, norm: Norm, delta: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
        """resid += norm(delta); returns the stream in the compute dtype."""
        if x.dtype == torch.float32:
            norm.add_normed(resid, delta)
            return resid
        norm.add_normed(resid, delta, cast_out=x)   # the old copy is no longer needed
        return x

    def forward(self, resid: torch.Tensor, pending, batch, cache: CacheView, write: bool):
        if isinstance(pending, Current):
            x = pending.x
        else:
            if pending is not None:
                raise ValueError("a branch_norm block takes a stream with nothing pending")
            x = resid   # (a 32-bit model; a block before it that hands on nothing)
        x = self._join(resid, self.mixer_norm,
                       self.mixer.forward(x, batch, cache, write, self.position), x)
        if self.feed_forward is not None:
            x = self._join(resid, self.feed_forward_norm, self.feed_forward.forward(x), x)
        if self.side is not None:
            x = self._join(resid, self.side_norm, self.side.forward(x, batch), x)
        return Current(x)


@register_block("sandwich")
class SandwichBlock(Block):
    """A norm before AND after each branch: ``x <- x + norm_b(Mixer(mix(norm_a(x))))``, then (if
    the layer has a feed-forward) ``x <- x + norm_d(FeedForward(norm_c(x)))``.  ``mix`` is an
    optional token mix (a token shift) on what the mixer reads; its state is the block's own
    (``state_spec``), one per cache entry, so a layer that runs twice carries two.

    The stream is 32-bit and every add happens at once: nothing is pending between blocks.
    Where the norm after the mixer chains with the norm in front of the feed-forward
    (``chains_with``), one kernel does both."""

    ROLES = {"mixer": "mixer", "mixer_norm": "norm", "mixer_out_norm": "norm",
             "feed_forward": "feed_forward", "feed_forward_norm": "norm",
             "feed_forward_out_norm": "norm", "token_mix": "token_mix", "position": "position"}
    OPTIONAL_ROLES = frozenset({"feed_forward", "feed_forward_norm", "feed_forward_out_norm",
                                "token_mix"})
    pad_safe = True   # the arrangement itself touches no token: its parts decide

    def __init__(self, mixer: Mixer, mixer_norm: Norm, mixer_out_norm: Norm,
                 position: PositionEncoding, feed_forward: FeedForward | None = None,
                 feed_forward_norm: Norm | None = None,
                 feed_forward_out_norm: Norm | None = None, token_mix=None) -> None:
        if len({feed_forward is None, feed_forward_norm is None,
                feed_forward_out_norm is None}) != 1:
            raise ValueError("a feed-forward comes with the norms before and after it")
        if token_mix is not None and not getattr(mixer_norm, "fuses_token_mix", False):
            raise ValueError("the norm in front of the mixer cannot mix tokens: a token mix "
                             "needs a norm that says fuses_token_mix")
        self.mixer, self.mixer_norm, self.mixer_out_norm = mixer, mixer_norm, mixer_out_norm
        self.position, self.token_mix = position, token_mix
        self.feed_forward, self.feed_forward_norm = feed_forward, feed_forward_norm
        self.feed_forward_out_norm = feed_forward_out_norm

    def state_spec(self):
        return self.token_mix.state_spec() if self.token_mix is not None else None

    def forward(self, resid: torch.Tensor, pending, batch, cache: CacheView, write: bool):
        if isinstance(pending, Current):
            pending = None
        if pending is not None:
            raise ValueError("a sandwich block takes a stream with nothing pending")
        if self.token_mix is None:
            h = self.mixer_norm.forward(resid, None)
        else:
            h = self.mixer_norm.forward(resid, None, token_mix=(
                self.token_mix.mu, cache.block_state, batch, write))
        y = self.mixer.forward(h, batch, cache, write, self.position)
        if self.feed_forward is None:
            self.mixer_out_norm.add_normed(resid, y)
            return None
        chains = getattr(self.mixer_out_norm, "chains_with", None)
        if chains is not None and chains(self.feed_forward_norm):
            h = self.mixer_out_norm.add_normed(resid, y, then=self.feed_forward_norm)
        else:
            self.mixer_out_norm.add_normed(resid, y)
            h = self.feed_forward_norm.forward(resid, None)
        self.feed_forward_out_norm.add_normed(resid, self.feed_forward.forward(h))
        return None


@register_block("shared_norm")
class SharedNormBlock(Block):
    """ONE norm in front of a layer whose branches run side by side on its output:
    ``h = norm(x)``, ``x <- x + mult * (Mixer(h) + FeedForward(h))`` (the feed-forward is
    optional).  Nothing is added here: the block hands the branches' outputs on as a weighted sum
    (:class:`~.stream.Terms`), which the next norm (the next layer's, or the model's last) forms
    in 32-bit while it reads the stream; so the norm must say ``takes_terms``.  A mixer may
    itself return such a sum (two mixers side by side, each with a weight)."""

    ROLES = {"mixer": "mixer", "feed_forward": "feed_forward", "norm": "norm",
             "position": "position"}
    OPTIONAL_ROLES = frozenset({"feed_forward"})
    pad_safe = True   # the arrangement itself touches no token: its parts decide

    def __init__(self, mixer: Mixer, norm: Norm, position: PositionEncoding,
                 feed_forward: FeedForward | None = None, residual_mult: float = 1.0) -> None:
        if not getattr(norm, "takes_terms", False):
            raise ValueError("a shared_norm block needs a norm that takes a sum of terms as what "
                             "is pending (takes_terms)")
        self.mixer, self.norm, self.position = mixer, norm, position
        self.feed_forward, self.residual_mult = feed_forward, float(residual_mult)
        #: the branches' output matrices joined into one [hidden, sum of their inputs], once the
        #: weights are there: None = not tried yet, False = a branch cannot hand out its activations
        self._joint = None
        self._widths: list[tuple[int, int]] = []     # per segment: (first column, width)
        self._zero_fill = False

    def _join_outputs(self) -> None:
        """Both branches end with a matrix product into the stream, weighted by constants:
        ``sum_i c_i W_i a_i = [c_1 W_1 | c_2 W_2 | ...] [a_1; a_2; ...]``, one product over the
        concatenated activations, which the branches write side by side into one buffer.  The
        constants go into the joined matrix (formed in 32-bit, rounded once)."""
        branches = [self.mixer] + ([self.feed_forward] if self.feed_forward is not None else [])
        segments = []
        for part in branches:
            mine = part.out_segments() if hasattr(part, "out_segments") else None
            if mine is None:
                self._joint = False
                return
            segments += mine
        blocks, at = [], 0
        for w, coef in segments:
            width = w.shape[1]
            padded = -(-width // 8) * 8        # every segment starts on a 16-byte boundary
            block = w.new_zeros((w.shape[0], padded))
            block[:, :width] = (w.float() * coef).to(w.dtype) if coef != 1.0 else w
            blocks.append(block)
            self._widths.append((at, width))
            self._zero_fill |= padded != width
            at += padded
        self._n_mixer = len(segments) - (1 if self.feed_forward is not None else 0)
        self._joint = Linear(torch.cat(blocks, 1).contiguous())
        for part in branches:
            part.release_out()

    def forward(self, resid: torch.Tensor, pending, batch, cache: CacheView, write: bool):
        h = self.norm.forward(resid, pending)
        if self._joint is None:
            self._join_outputs()
        if self._joint is not False:
            w = self._joint.weight
            # (zeros where segments are padded up to 16 bytes, and in padded steps, whose padding
            # tokens some branches leave unwritten)
            cat = (torch.zeros if self._zero_fill or batch.padded else torch.empty)(
                (h.shape[0], w.shape[1]), dtype=w.dtype, device=w.device)
            outs = [cat[:, a:a + n] for a, n in self._widths]
            self.mixer.activations_into(h, batch, cache, write, self.position,
                                        outs[:self._n_mixer])
            if self.feed_forward is not None:
                self.feed_forward.activations_into(h, outs[self._n_mixer:])
            return Terms.of(self._joint(cat), self.residual_mult)
        out = Terms.of(self.mixer.forward(h, batch, cache, write, self.position),
                       self.residual_mult)
        if self.feed_forward is not None:
            out = out + Terms.of(self.feed_forward.forward(h), self.residual_mult)
        return out
