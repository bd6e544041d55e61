"""Arrangements: how a layer's mixer, feed-forward and norms are wired.

``prenorm_residual`` is the layout of crates/coheryn-engine/src/inference.rs:440-540:
x += mixer(norm(x)); x += feed_forward(norm(x)).  The residual stream is float32; each
sub-layer's output is handed on as a pending ``delta`` that the NEXT norm adds to the
stream while it normalises, so the sum and the norm cost one pass over the row.
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from .base import Arrangement, Part, PostNormed, StreamCopy, register_arrangement
from .native_block import NativeBlock


class PreNormResidual(Arrangement):
    """x += mixer(mixer_norm(x)); x += feed_forward(feed_forward_norm(x)); the feed-forward with its norm may be absent."""

    SLOTS = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "feed_forward_norm": "norm"}
    OPTIONAL = ("feed_forward", "feed_forward_norm")
    NAMES = {"mixer_norm": "input_layernorm", "mixer": "self_attn", "feed_forward_norm": "post_attention_layernorm",
             "feed_forward": "mlp"}

    def __init__(self, parts):
        super().__init__(parts)
        if (self.slots.get("feed_forward") is None) != (self.slots.get("feed_forward_norm") is None):
            raise ValueError("prenorm_residual: a feed-forward comes with its norm or not at all")

    def parts(self) -> Dict[str, Part]:
        names = self.names or self.NAMES
        return {names[slot]: part for slot, part in self.slots.items() if part is not None}

    _native = None     # None: not looked at yet; False: not made of the built-in parts

    def _native_block(self):
        nb = self._native
        if nb is None or (nb is not False and not nb.current(self)):
            nb = self._native = NativeBlock.build(self) or False
        return nb

    def forward(self, residual, delta, step, cache):
        if ops.NATIVE_BLOCK:
            nb = self._native_block()
            if nb:
                out = nb.run(residual, delta, step, cache)   # the whole block from one call into the library
                if out is not None:
                    return residual, out
        mixed = self.mixer.forward(self.mixer_norm.forward(residual, delta), step, cache)
        if self.feed_forward is None:
            return residual, mixed
        out = self.feed_forward.forward(self.feed_forward_norm.forward(residual, mixed), step)
        return residual, out

    @property
    def supports_tail(self):
        return self.mixer.supports_tail

    def forward_tail(self, residual, delta, step, cache):
        mixed = self.mixer.forward_tail(self.mixer_norm.forward(residual, delta), step, cache)
        if mixed is None:
            return None, None
        kept = ops.gather_rows(residual, step.tail_rows)
        if self.feed_forward is None:
            return kept, mixed
        out = self.feed_forward.forward(self.feed_forward_norm.forward(kept, mixed), step.tail)
        return kept, out


class ParallelResidual(Arrangement):
    """x += mixer(h) + feed_forward(h) with ONE norm h = norm(x) that both read; the feed-forward may be absent.
    The summands are not added here: each part writes its own (a mixer made of several writes several) into a
    float32 stack that the NEXT norm adds to the stream in order while it normalises, so the block needs parts
    that offer ``output_parts`` and ``forward_into`` and a model whose norms all take partial sums."""

    SLOTS = {"norm": "norm", "mixer": "mixer", "feed_forward": "feed_forward"}
    OPTIONAL = ("feed_forward",)
    NAMES = {"norm": "input_layernorm", "mixer": "mixer", "feed_forward": "mlp"}

    def __init__(self, parts):
        super().__init__(parts)
        for part in self.producers():
            if not hasattr(part, "forward_into"):
                raise ValueError(f"parallel_residual: {type(part).__name__} cannot write its output into a stack of summands")

    def parts(self) -> Dict[str, Part]:
        names = self.names or self.NAMES
        return {names[slot]: part for slot, part in self.slots.items()}

    _joined = None     # None: not looked at yet; False: the producers write their own summands

    def _joined_output(self):
        """[o_1 | o_2 | ..] times the output matrices stacked side by side is the sum of the producers' outputs: ONE
        product instead of one per producer, when every producer hands its activations over and every piece starts on
        a 16-byte boundary in bfloat16 (eight elements).  Returns (stacked matrix, column ranges) or False."""
        if self._joined is None:
            self._joined = False
            producers = self.producers()
            if all(hasattr(p, "forward_open") and hasattr(p, "output_weights") for p in producers):
                weights = [p.output_weights() for p in producers]
                if all(w is not None for w in weights):
                    flat = [w for ws in weights for w in ws]
                    if all(w.dim() == 2 and w.shape[1] % 8 == 0 and w.dtype == flat[0].dtype for w in flat):
                        ranges, at = [], 0
                        for w in flat:
                            ranges.append((at, at + w.shape[1]))
                            at += w.shape[1]
                        self._joined = (torch.cat(flat, dim=1).contiguous(), ranges, [len(ws) for ws in weights])
        return self._joined

    def forward(self, residual, delta, step, cache):
        if not self.mixer.partial_output:
            raise ValueError("parallel_residual needs a model whose norms all take partial sums")
        h = self.norm.forward(residual, delta)
        joined = self._joined_output() if ops.JOINED_OUTPUT else False
        if joined:
            w_out, ranges, counts = joined
            T = residual.shape[0]
            acts = torch.empty((T, w_out.shape[1]), dtype=w_out.dtype, device=residual.device)
            views = [acts[:, a:b] for a, b in ranges]
            self.mixer.forward_open(h, step, cache, views[:counts[0]])
            if self.feed_forward is not None:
                self.feed_forward.forward_open(h, step, None, views[counts[0]:])
            # a long K: the product may leave its K slices to the next norm (a float32 stack), as the down projection does
            out = ops.linear(acts, w_out, out_dtype=torch.float32, partial_ok=True)
            return residual, out if out.dim() == 3 else out.unsqueeze(0)
        n_mix = self.mixer.output_parts
        n = n_mix + (self.feed_forward.output_parts if self.feed_forward is not None else 0)
        out = torch.empty((n, residual.shape[0], residual.shape[1]), dtype=torch.float32, device=residual.device)
        self.mixer.forward_into(h, step, cache, out[:n_mix])
        if self.feed_forward is not None:
            self.feed_forward.forward_into(h, step, out[n_mix:])
        return residual, out


class SandwichResidual(Arrangement):
    """A norm before and after each sub-layer: x += mixer_post_norm(mixer(mixer_norm(x))), then
    x += feed_forward_post_norm(feed_forward(feed_forward_norm(x))); the feed-forward with its two norms may be absent.
    A sub-layer's output is handed on as a pending :class:`PostNormed` delta, and the NEXT norm (this block's, the
    following block's or the model's last) normalises it, adds it to the float32 stream and normalises the sum in one
    kernel, so the block costs one norm kernel per sub-layer like the pre-norm block."""

    SLOTS = {"mixer_norm": "norm", "mixer": "mixer", "mixer_post_norm": "norm", "feed_forward_norm": "norm",
             "feed_forward": "feed_forward", "feed_forward_post_norm": "norm"}
    OPTIONAL = ("feed_forward_norm", "feed_forward", "feed_forward_post_norm")
    NAMES = {"mixer_norm": "pre_mixer_norm", "mixer": "mixer", "mixer_post_norm": "post_mixer_norm",
             "feed_forward_norm": "pre_feed_forward_norm", "feed_forward": "feed_forward",
             "feed_forward_post_norm": "post_feed_forward_norm"}

    def __init__(self, parts):
        super().__init__(parts)
        ff = [self.slots.get(n) is not None for n in ("feed_forward_norm", "feed_forward", "feed_forward_post_norm")]
        if any(ff) and not all(ff):
            raise ValueError("sandwich_residual: a feed-forward comes with both of its norms or not at all")

    def parts(self) -> Dict[str, Part]:
        names = self.names or self.NAMES
        return {names[slot]: part for slot, part in self.slots.items()}

    def forward(self, residual, delta, step, cache):
        h = self.mixer_norm.forward(residual, delta)
        post = self.mixer_post_norm
        delta = PostNormed(self.mixer.forward(h, step, cache), post.weight, post.eps)
        if self.feed_forward is not None:
            h = self.feed_forward_norm.forward(residual, delta)
            post = self.feed_forward_post_norm
            delta = PostNormed(self.feed_forward.forward(h, step), post.weight, post.eps)
        return residual, delta

    @property
    def supports_tail(self):
        return self.mixer.supports_tail

    def forward_tail(self, residual, delta, step, cache):
        """The mixer updates its cache for all rows; its output, the feed-forward and both following norms run for the
        wanted rows only."""
        h = self.mixer_norm.forward(residual, delta)
        post = self.mixer_post_norm
        mixed = self.mixer.forward_tail(h, step, cache)
        if mixed is None:
            return None, None
        kept = ops.gather_rows(residual, step.tail_rows)
        delta = PostNormed(mixed, post.weight, post.eps)
        if self.feed_forward is not None:
            h = self.feed_forward_norm.forward(kept, delta)
            post = self.feed_forward_post_norm
            delta = PostNormed(self.feed_forward.forward(h, step.tail), post.weight, post.eps)
        return kept, delta


class PostNormResidual(Arrangement):
    """The norm AFTER the sum: x <- mixer_norm(alpha x + mixer(x)), then x <- feed_forward_norm(alpha x + feed_forward(x));
    the sub-layers read the stream itself.  Optionally a third sub-layer ``side`` whose output is normalised by itself and
    added: x <- x + side_norm(side(x)).  The feed-forward (with its norm) and the side (with its norm) may be absent.

    The float32 stream is rewritten in place by the kernel that normalises a row, which also writes the row in the compute
    dtype for the next matrix products; between blocks that copy travels in the pending delta's place as a
    :class:`StreamCopy`."""

    SLOTS = {"mixer": "mixer", "mixer_norm": "norm", "feed_forward": "feed_forward", "feed_forward_norm": "norm",
             "side": "feed_forward", "side_norm": "norm"}
    OPTIONAL = ("feed_forward", "feed_forward_norm", "side", "side_norm")
    NAMES = {"mixer": "mixer", "mixer_norm": "post_mixer_norm", "feed_forward": "feed_forward",
             "feed_forward_norm": "post_feed_forward_norm", "side": "side", "side_norm": "side_norm"}

    def __init__(self, parts, alpha: float = 1.0):
        super().__init__(parts)
        self.alpha = float(alpha)
        for a, b in (("feed_forward", "feed_forward_norm"), ("side", "side_norm")):
            if (self.slots.get(a) is None) != (self.slots.get(b) is None):
                raise ValueError(f"postnorm_residual: {a} comes with {b} or not at all")

    def parts(self) -> Dict[str, Part]:
        names = self.names or self.NAMES
        return {names[slot]: part for slot, part in self.slots.items()}

    def cache_owner(self):
        return self.mixer

    def producers(self):
        return [p for p in (self.mixer, self.feed_forward) if p is not None]     # the side's product is short: never split

    def _input(self, residual, delta):
        if isinstance(delta, StreamCopy):
            return delta.value
        if delta is not None:
            raise ValueError("postnorm_residual follows blocks that leave nothing pending")
        dtype = self.mixer.runtime.dtype
        return residual if dtype == torch.float32 else residual.to(dtype)

    def _rest(self, residual, h, step):
        if self.feed_forward is not None:
            h = self.feed_forward_norm.post(residual, self.feed_forward.forward(h, step), self.alpha)
        if self.side is not None:
            h = self.side_norm.post(residual, self.side.forward(h, step), normed_summand=True)
        return residual, StreamCopy(h)

    def forward(self, residual, delta, step, cache):
        h = self._input(residual, delta)
        h = self.mixer_norm.post(residual, self.mixer.forward(h, step, cache), self.alpha)
        return self._rest(residual, h, step)

    @property
    def supports_tail(self):
        return self.mixer.supports_tail

    def forward_tail(self, residual, delta, step, cache):
        """The mixer updates its cache for all rows; everything behind it runs for the wanted rows only."""
        mixed = self.mixer.forward_tail(self._input(residual, delta), step, cache)
        if mixed is None:
            return None, None
        kept = ops.gather_rows(residual, step.tail_rows)
        h = self.mixer_norm.post(kept, mixed, self.alpha)
        return self._rest(kept, h, step.tail)


register_arrangement("postnorm_residual", PostNormResidual)
register_arrangement("sandwich_residual", SandwichResidual)
register_arrangement("prenorm_residual", PreNormResidual)
register_arrangement("parallel_residual", ParallelResidual)
