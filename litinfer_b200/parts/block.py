"""Arrangement of a layer's parts.  ``prenorm``: x += Mixer(norm(x));
x += FeedForward(norm(x)) (src/llaisys/models/qwen2.cpp:272-316).

The residual stream x is float32.  A block does not add the output of its
last part itself: told the next block's entry (its first norm), it lets that part
add, and normalise for the next block, in the tail of its last product
(``Carry.normed``); otherwise it hands the output on (``Carry.delta``) and the next
block, or the model's tail, adds it inside its first norm kernel.  Either way
add and norm are one pass over x.

A block takes its parts from the roles of its :class:`~litinfer_b200.config.spec.BlockSpec`
(:meth:`Block.build`); ``prenorm`` wants ``mixer`` and ``mixer_norm`` and, unless the layer has
no feed-forward, ``feed_forward`` and ``feed_forward_norm``.
"""

from __future__ import annotations

from typing import List

from dataclasses import dataclass
from typing import Dict, Optional

import torch

from .. import kernels as K
from ..weights.loader import ParamSpec
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, Carry, Tail


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    def __init__(self, spec, prefix, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        self.mixer_norm = self.build(NORMS, "mixer_norm")
        self.mixer = self.build(MIXERS, "mixer")
        self.feed_forward = self.build(FEED_FORWARDS, "feed_forward", required=False)
        self.feed_forward_norm = self.build(NORMS, "feed_forward_norm", required=self.feed_forward is not None)

    def parts(self) -> List:
        return [p for p in (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward) if p is not None]

    def entry(self):
        return Tail(None, self.mixer_norm, self.mixer.takes_deferred)

    def fused_decode(self):
        if type(self) is not PreNormBlock or self.feed_forward is None:
            return None
        mixer, ff = self.mixer.fused_decode(), self.feed_forward.fused_decode()
        n1, n2 = self.mixer_norm.fused_decode(), self.feed_forward_norm.fused_decode()
        if None in (mixer, ff, n1, n2) or mixer["hidden"] != ff["hidden"] or n1["size"] != mixer["hidden"] or n2["size"] != mixer["hidden"]:
            return None
        return dict(mixer, **ff, norm_first=n1, norm_ffn=n2)

    def forward(self, x32, ctx, cache, carry, next_entry=None):
        if carry is None:
            h = self.mixer_norm.forward(x32)
        elif carry.normed is not None:
            h = carry.normed                               # the block before applied this block's first norm
        else:
            h = self.mixer_norm.add_forward(x32, carry.delta)
        if self.feed_forward is None:
            if next_entry is None:
                return x32, Carry(delta=self.mixer.forward(h, ctx, cache))
            return x32, Carry(normed=self.mixer.forward_into(h, ctx, cache, Tail(x32, next_entry.norm, next_entry.defer)))
        h = self.mixer.forward_into(h, ctx, cache, Tail(x32, self.feed_forward_norm, self.feed_forward.takes_deferred))
        if next_entry is None:
            return x32, Carry(delta=self.feed_forward.forward(h, ctx))
        return x32, Carry(normed=self.feed_forward.forward_into(h, ctx, Tail(x32, next_entry.norm, next_entry.defer)))


@dataclass
class StreamsEntry(Tail):
    """The entry of a block that keeps several residual streams: its first norm and the weights with which its first
    sublayer reads the streams, so that the block before can do that read in the pass that writes its own output back."""

    read: Optional[torch.Tensor] = None


class _Connection:
    """The tensors that tie one sublayer to the streams: read weights [s], write weights [s], mix [s, s] (from, to)."""

    def __init__(self, prefix: str, streams: int, names: Dict[str, str]) -> None:
        self.streams = streams
        self.names = {k: prefix + names.get(k, k) for k in ("in", "out", "mix")}
        self.read = self.write = self.mix = None

    def params(self):
        s = self.streams
        return [ParamSpec(self.names["in"], (s,), role="vector", mean=1.0 / s, std=0.05),
                ParamSpec(self.names["out"], (s,), role="vector", init="ones_normal"),
                ParamSpec(self.names["mix"], (s, s), role="vector", init="eye_normal", std=0.05)]

    def bind(self, tensors) -> None:
        self.read, self.write, self.mix = (tensors.pop(self.names[k]) for k in ("in", "out", "mix"))


@BLOCKS.register("hyper_prenorm")
class HyperPreNormBlock(Block):
    """Pre-norm sublayers over several residual streams (hyper-connections).  Instead of one stream x there are s
    copies, ``xs [tokens, s, width]``, all equal to the embedding at the start and summed at the end.  A sublayer
    (the mixer, then the feed-forward if the layer has one) reads ``u = sum_s in[s] xs[s]``, runs on ``norm(u)``, and its
    output y goes back as ``xs'[r] = sum_s mix[s, r] xs[s] + out[r] y``, every stream from the old ones.  Each sublayer has
    its own in / out / mix tensors (roles ``mixer_connection`` and ``feed_forward_connection`` give their prefixes).

    The write-back of a sublayer and the read and norm of the next one are one kernel (as add + norm is for a single
    stream); told the next block's entry, the last sublayer of this block does the next block's first read."""

    def __init__(self, spec, prefix, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        self.mixer_norm = self.build(NORMS, "mixer_norm")
        self.mixer = self.build(MIXERS, "mixer")
        self.feed_forward = self.build(FEED_FORWARDS, "feed_forward", required=False)
        self.feed_forward_norm = self.build(NORMS, "feed_forward_norm", required=self.feed_forward is not None)
        conn = spec.part("connections")
        if conn is None:
            raise ValueError(f"block 'hyper_prenorm' at {spec.prefix!r} needs a part 'connections' with the number of streams")
        self.streams = int(conn["streams"])
        names = conn.get("names", {})
        self.mixer_connection = _Connection(spec.prefix_of("mixer_connection"), self.streams, names)
        self.feed_forward_connection = (_Connection(spec.prefix_of("feed_forward_connection"), self.streams, names)
                                        if self.feed_forward is not None else None)

    def parts(self) -> List:
        return [p for p in (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward) if p is not None]

    def params(self):
        out = self.mixer_connection.params()
        if self.feed_forward_connection is not None:
            out += self.feed_forward_connection.params()
        return out

    def bind(self, tensors) -> None:
        self.mixer_connection.bind(tensors)
        if self.feed_forward_connection is not None:
            self.feed_forward_connection.bind(tensors)

    def entry(self):
        return StreamsEntry(None, self.mixer_norm, False, read=self.mixer_connection.read)

    @staticmethod
    def _write_back(xs, y, conn, next_norm, next_read):
        """The sublayer's output into the streams; the next sublayer's input if its norm and read weights are known."""
        if next_norm is None:
            K.hc_update(xs, y, conn.mix, conn.write)
            return None
        return next_norm.streams_update_forward(xs, y, conn.mix, conn.write, next_read)

    def forward(self, xs, ctx, cache, carry, next_entry=None):
        if xs.dim() != 3 or xs.shape[1] != self.streams:
            raise ValueError(f"a block over {self.streams} streams was handed a residual of shape {tuple(xs.shape)}")
        if carry is not None and carry.delta is not None:
            raise ValueError("a block over several streams cannot take an output that is still to be added")
        h = carry.normed if carry is not None and carry.normed is not None else self.mixer_norm.streams_forward(xs, self.mixer_connection.read)
        nxt = next_entry if isinstance(next_entry, StreamsEntry) else None
        # (a mixer of two side by side hands both outputs over: the write-back adds them up)
        y = self.mixer.forward_pair(h, ctx, cache) if getattr(self.mixer, "produces_pairs", False) else self.mixer.forward(h, ctx, cache)
        if self.feed_forward is None:
            h = self._write_back(xs, y, self.mixer_connection, nxt.norm if nxt else None, nxt.read if nxt else None)
            return xs, (Carry(normed=h) if h is not None else None)
        h = self._write_back(xs, y, self.mixer_connection, self.feed_forward_norm, self.feed_forward_connection.read)
        y = self.feed_forward.forward(h, ctx)
        h = self._write_back(xs, y, self.feed_forward_connection, nxt.norm if nxt else None, nxt.read if nxt else None)
        return xs, (Carry(normed=h) if h is not None else None)


@BLOCKS.register("sandwich")
class SandwichBlock(Block):
    """A norm before and a norm after each sublayer: ``x += post(Mixer(pre(x)))``, then ``x += post'(FeedForward(pre'(x)))``.
    Roles: ``mixer_norm``, ``mixer_post_norm``, and with a feed-forward ``feed_forward_norm``, ``feed_forward_post_norm``;
    any registered norm that says what it is through ``statistics()`` (weight, centered or not, eps) serves in any role.

    The norm after a sublayer, the addition to the stream and the norm before the next sublayer are one kernel and one
    pass over the stream (``kernels.norm_add_norm``); told the next block's entry, the last sublayer's pass already
    applies that block's first norm."""

    def __init__(self, spec, prefix, dtype, device):
        super().__init__(spec, prefix, dtype, device)
        self.mixer_norm = self.build(NORMS, "mixer_norm")
        self.mixer = self.build(MIXERS, "mixer")
        self.mixer_post_norm = self.build(NORMS, "mixer_post_norm")
        self.feed_forward = self.build(FEED_FORWARDS, "feed_forward", required=False)
        self.feed_forward_norm = self.build(NORMS, "feed_forward_norm", required=self.feed_forward is not None)
        self.feed_forward_post_norm = self.build(NORMS, "feed_forward_post_norm", required=self.feed_forward is not None)
        for n in (self.mixer_norm, self.mixer_post_norm, self.feed_forward_norm, self.feed_forward_post_norm):
            if n is not None and not hasattr(n, "statistics"):
                raise ValueError(f"block 'sandwich' at {spec.prefix!r}: norm '{n.spec.kind}' does not say what it is (statistics())")

    def parts(self) -> List:
        return [p for p in (self.mixer_norm, self.mixer, self.mixer_post_norm, self.feed_forward_norm, self.feed_forward,
                            self.feed_forward_post_norm) if p is not None]

    def entry(self):
        return Tail(None, self.mixer_norm, False)

    def _close(self, x32, y, post, nxt):
        """x32 += post(y); the next norm of the sum if that norm is known and of a kind the kernel takes."""
        if nxt is not None and hasattr(nxt, "statistics"):
            out = torch.empty(x32.shape, dtype=self.dtype, device=x32.device)
            K.norm_add_norm(x32, y, post.statistics(), nxt.statistics(), out)
            return out
        K.norm_add_norm(x32, y, post.statistics(), None, None)
        return nxt.forward(x32) if nxt is not None else None

    def forward(self, x32, ctx, cache, carry, next_entry=None):
        if carry is None:
            h = self.mixer_norm.forward(x32)
        elif carry.normed is not None:
            h = carry.normed
        else:
            h = self.mixer_norm.add_forward(x32, carry.delta)
        nxt = next_entry.norm if next_entry is not None and type(next_entry) is Tail else None
        y = self.mixer.forward(h, ctx, cache)
        if self.feed_forward is None:
            h = self._close(x32, y, self.mixer_post_norm, nxt)
            return x32, (Carry(normed=h) if h is not None else None)
        h = self._close(x32, y, self.mixer_post_norm, self.feed_forward_norm)
        # (a mixture of experts hands its rows over as they are: the pass over the stream sums a token's rows itself)
        y = self.feed_forward.forward_rows(h, ctx) if getattr(self.feed_forward, "produces_row_sums", False) else self.feed_forward.forward(h, ctx)
        h = self._close(x32, y, self.feed_forward_post_norm, nxt)
        return x32, (Carry(normed=h) if h is not None else None)
