"""Arrangements of a block's parts around the residual stream.

``pre_norm``:  x += mixer(norm1(x));  x += feed_forward(norm2(x)); a norm whose consumer can fold it into
its first matrix product is handed over unevaluated (``norm.DeferredNorm``)
(berniehans/titan: engine/engine-core/src/forward_cpu.rs:281-386).  The
residual stream ``x`` is float32 and is updated in place: mixer and
feed-forward add into it in the epilogue of their last matrix product.  The other arrangements (``pre_norm_scaled``,
``output_norm``, ``hyper``, ``parallel``) are described at their classes.
"""
from __future__ import annotations

from typing import List

import torch

from ..weights.loader import WeightSpec
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Part


class PreNormBlock(Part):
    def __init__(self, spec):
        if spec.feed_forward is None or spec.mixer_norm is None or spec.feed_forward_norm is None or spec.norms:
            raise ValueError("the pre_norm arrangement takes a mixer, a feed-forward and exactly the two norms before them")
        self.spec = spec
        self.mixer_norm = NORMS.build(spec.mixer_norm)
        self.mixer = MIXERS.build(spec.mixer)
        self.feed_forward_norm = NORMS.build(spec.feed_forward_norm)
        self.feed_forward = FEED_FORWARDS.build(spec.feed_forward)

    def parts(self):
        return (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward)

    def weight_specs(self, prefix: str = "") -> List[WeightSpec]:
        out: List[WeightSpec] = []
        for part in self.parts():
            out += part.weight_specs(self.spec.prefix)
        return out

    def bind(self, get) -> None:
        for part in self.parts():
            part.bind(lambda name: get(self.spec.prefix + name))

    @staticmethod
    def _normed(norm, consumer, x, ctx):
        """The norm's rows for the part that consumes them; not yet computed (a DeferredNorm) if the norm can be
        deferred and the part can fold it into its first product."""
        # up to 16 rows: measured after 2,048-token prompts, folding gains 3 % of the step at 12 and 16 sequences and
        # loses 1 to 3 % at 20 to 32 (the kernels take up to 32 rows: twice the float32 rows per weight tile through L2)
        if (getattr(consumer, "folds_norm", False) and hasattr(norm, "deferred") and getattr(norm, "groups", 1) == 1 and ctx.options.get("fold_norms", True)
                and x.shape[0] <= int(ctx.options.get("fold_norms_rows", 16))):
            return norm.deferred(x, ctx)
        return norm.forward(x, ctx)

    def forward(self, x: torch.Tensor, ctx, cache) -> None:
        self.mixer.forward(self._normed(self.mixer_norm, self.mixer, x, ctx), ctx, cache, x)
        self.feed_forward.forward(self._normed(self.feed_forward_norm, self.feed_forward, x, ctx), ctx, x)


BLOCKS.register("pre_norm", PreNormBlock)


class ScaledPreNormBlock(Part):
    """``pre_norm_scaled``: pre-norm with a learned scale on every sublayer's output ("layer scale"):

        x += s1 * mixer(norm1(x));   x += s2 * feed_forward(norm2(x))

    s1 and s2 are vectors as wide as the residual stream, named in ``LayerSpec.extra`` under "scales" (two tensor names
    relative to the layer's prefix).  The feed-forward, with its norm and scale, may be absent.  A sublayer adds into a
    zeroed float32 buffer of the step; one kernel then scales that buffer, adds it to the residual stream and leaves it
    zeroed.  Where the norm that follows is a ``dyt`` norm (its result depends on the element alone), the same kernel
    also writes the normed rows that the next sublayer reads: the feed-forward's input here, or the next block's
    mixer input, which the next block then finds in ``ctx.carried`` (the model names the block that runs next)."""

    def __init__(self, spec):
        if spec.mixer_norm is None or (spec.feed_forward is None) != (spec.feed_forward_norm is None) or spec.norms:
            raise ValueError("the pre_norm_scaled arrangement takes a mixer with its norm, and a feed-forward with its norm or neither")
        names = tuple(spec.option("scales", ()))
        if len(names) != (1 if spec.feed_forward is None else 2):
            raise ValueError("the pre_norm_scaled arrangement needs the name of one scale vector for each sublayer")
        self.spec, self.scale_names = spec, names
        self.mixer_norm = NORMS.build(spec.mixer_norm)
        self.mixer = MIXERS.build(spec.mixer)
        self.feed_forward_norm = None if spec.feed_forward_norm is None else NORMS.build(spec.feed_forward_norm)
        self.feed_forward = None if spec.feed_forward is None else FEED_FORWARDS.build(spec.feed_forward)
        self.scales: List[torch.Tensor] = []

    def parts(self):
        return (self.mixer_norm, self.mixer) + (() if self.feed_forward is None else (self.feed_forward_norm, self.feed_forward))

    def weight_specs(self, prefix: str = "") -> List[WeightSpec]:
        out: List[WeightSpec] = []
        for part in self.parts():
            out += part.weight_specs(self.spec.prefix)
        width = self.spec.mixer.hidden_size
        return out + [WeightSpec(self.spec.prefix + n, (width,), "vector", ("one_plus_normal", 0.1)) for n in self.scale_names]

    def bind(self, get) -> None:
        for part in self.parts():
            part.bind(lambda name: get(self.spec.prefix + name))
        self.scales = [get(self.spec.prefix + n) for n in self.scale_names]

    def _join(self, y, scale, x, ctx, next_norm):
        """x += scale * y, y zeroed; the rows of ``next_norm`` over the new x if that norm can ride along, else None."""
        from .. import kernels as K
        if next_norm is not None and hasattr(next_norm, "triple") and ctx.options.get("fuse_scaled_norm", True):
            h = ctx.empty(tuple(x.shape))
            K.scale_add(y, scale, x, ctx.stream, zero_y=True, norm=next_norm.triple(), h=h)
            return h
        K.scale_add(y, scale, x, ctx.stream, zero_y=True)
        return None

    def forward(self, x: torch.Tensor, ctx, cache) -> None:
        y = ctx.carried.get("sublayer_sum")
        if y is None or y.shape != x.shape:
            y = ctx.carried["sublayer_sum"] = torch.zeros_like(x)         # zeroed once a step; the joining kernel leaves it zeroed
        kept = ctx.carried.pop("normed_rows", None)
        h = kept[0] if kept is not None and kept[1] == ctx.run and kept[0].shape == x.shape else self.mixer_norm.forward(x, ctx)
        self.mixer.forward(h, ctx, cache, y)
        following = getattr(ctx.next_block, "mixer_norm", None) if isinstance(ctx.next_block, ScaledPreNormBlock) else None
        if self.feed_forward is None:
            h = self._join(y, self.scales[0], x, ctx, following)
        else:
            h = self._join(y, self.scales[0], x, ctx, self.feed_forward_norm)
            self.feed_forward.forward(h if h is not None else self.feed_forward_norm.forward(x, ctx), ctx, y)
            h = self._join(y, self.scales[1], x, ctx, following)
        if h is not None:
            ctx.carried["normed_rows"] = (h, ctx.run + 1)


BLOCKS.register("pre_norm_scaled", ScaledPreNormBlock)


class OutputNormBlock(Part):
    """``output_norm``: every sublayer reads the residual stream itself and its OUTPUT is normed before it is added:

        x += norm1(mixer(x));  x += norm2(feed_forward(x));  x += norm_k(extra_k(x)) for every further sublayer

    The feed-forward (with its norm) may be absent.  Further sublayers are feed-forward parts named in
    ``LayerSpec.extra`` under "sublayers" (a tuple of FeedForwardSpec), their norms are ``LayerSpec.norms`` in the same
    order.  A sublayer adds into a zeroed float32 buffer of the step; one kernel then norms that buffer's rows, adds them
    to the residual stream, leaves the buffer zeroed for the next sublayer and, in bfloat16, writes the new rows rounded
    for the next sublayer's first product (in float32 the sublayers read the residual stream in place)."""

    def __init__(self, spec):
        if spec.mixer_norm is None or (spec.feed_forward is None) != (spec.feed_forward_norm is None):
            raise ValueError("the output_norm arrangement takes a mixer with its norm, and a feed-forward with its norm or neither")
        self.spec = spec
        self.mixer = MIXERS.build(spec.mixer)
        self.mixer_norm = NORMS.build(spec.mixer_norm)
        self.feed_forward = None if spec.feed_forward is None else FEED_FORWARDS.build(spec.feed_forward)
        self.feed_forward_norm = None if spec.feed_forward_norm is None else NORMS.build(spec.feed_forward_norm)
        for n in (spec.mixer_norm, spec.feed_forward_norm) + tuple(spec.norms):
            if n is not None and (n.kind != "rmsnorm" or getattr(n, "groups", 1) != 1):
                raise ValueError("the output_norm arrangement folds a plain RMS norm (one group) into the kernel that adds a sublayer's output")
        more = tuple(spec.option("sublayers", ()))
        if len(more) != len(spec.norms):
            raise ValueError(f"{len(more)} further sublayers with {len(spec.norms)} norms")
        self.more = [(FEED_FORWARDS.build(f), NORMS.build(n)) for f, n in zip(more, spec.norms)]

    def parts(self):
        first = (self.mixer, self.mixer_norm) + (() if self.feed_forward is None else (self.feed_forward, self.feed_forward_norm))
        return first + tuple(p for pair in self.more for p in pair)

    def weight_specs(self, prefix: str = "") -> List[WeightSpec]:
        out: List[WeightSpec] = []
        for part in self.parts():
            out += part.weight_specs(self.spec.prefix)
        return out

    def bind(self, get) -> None:
        for part in self.parts():
            part.bind(lambda name: get(self.spec.prefix + name))

    def bind_shared(self, shared) -> None:
        for part in self.parts():
            if hasattr(part, "bind_shared"):
                part.bind_shared(shared)

    def _input(self, x, ctx):
        """The residual rows as a sublayer's first product reads them: x itself in float32; in bfloat16 the rounded copy
        that the kernel before left (if it was made for exactly this state of x), else one made now."""
        if ctx.dtype == torch.float32:
            return x, None
        kept = ctx.carried.pop("rounded_rows", None)
        if kept is not None and kept[1] == ctx.run and kept[0].shape == x.shape:
            return kept[0], kept[0]
        from .. import kernels as K
        h = ctx.empty(tuple(x.shape))
        K.round_rows(x, h, ctx.stream)
        return h, h

    def forward(self, x: torch.Tensor, ctx, cache) -> None:
        from .. import kernels as K
        y = ctx.carried.get("sublayer_sum")
        if y is None or y.shape != x.shape:
            y = ctx.carried["sublayer_sum"] = torch.zeros_like(x)         # zeroed once a step; the norm kernel leaves it zeroed
        h, lowp = self._input(x, ctx)
        steps = [(lambda: self.mixer.forward(h, ctx, cache, y), self.mixer_norm)]
        if self.feed_forward is not None:
            steps.append((lambda: self.feed_forward.forward(h, ctx, y), self.feed_forward_norm))
        steps += [((lambda part=part: part.forward(h, ctx, y)), norm) for part, norm in self.more]
        for run_sublayer, norm in steps:
            run_sublayer()
            K.rmsnorm_add(y, norm.weight, x, norm.spec.eps, ctx.stream, lowp=lowp, zero_y=True)
        if lowp is not None:
            ctx.carried["rounded_rows"] = (lowp, ctx.run + 1)             # valid for the next run of the order, if nothing else touches x


BLOCKS.register("output_norm", OutputNormBlock)


class HyperConnectionBlock(Part):
    """``hyper``: a pre-norm block over several residual streams ("hyper-connections").  The model keeps S copies of the
    residual stream side by side, [T, S * H].  For each sublayer, with three small tensors ``in`` [S], ``out`` [S] and
    ``mix`` [S, S] (indexed [from, to]):

        u = sum_s in[s] x_s;   y = sublayer(norm(u));   x_r <- sum_s mix[s, r] x_s + out[r] * y   (all r from the old streams)

    The tensors' names are ``<name>.in|out|mix`` with one name per sublayer in ``LayerSpec.extra["connections"]``; the number
    of streams is ``LayerSpec.extra["streams"]``.  The feed-forward, with its norm and connection, may be absent.  A sublayer
    adds into a zeroed float32 buffer of the step; ONE kernel then writes it into the streams, mixes them, leaves the buffer
    zeroed and reads the blend for the sublayer that follows, normed (the feed-forward's input here, or the next block's
    mixer input, which that block finds in ``ctx.carried``; after the last block the plain sum of the streams, which the
    model takes as the residual stream that goes to the final norm)."""

    def __init__(self, spec):
        if spec.mixer_norm is None or (spec.feed_forward is None) != (spec.feed_forward_norm is None) or spec.norms:
            raise ValueError("the hyper arrangement takes a mixer with its norm, and a feed-forward with its norm or neither")
        names = tuple(spec.option("connections", ()))
        if len(names) != (1 if spec.feed_forward is None else 2):
            raise ValueError("the hyper arrangement needs the name of one connection for each sublayer")
        self.streams = int(spec.option("streams", 0))
        if self.streams < 1:
            raise ValueError("the hyper arrangement needs the number of streams")
        for n in (spec.mixer_norm, spec.feed_forward_norm):
            if n is not None and (n.kind != "rmsnorm" or getattr(n, "groups", 1) != 1):
                raise ValueError("the hyper arrangement folds a plain RMS norm (one group) into the kernel that reads the streams")
        self.spec, self.names = spec, names
        self.mixer_norm = NORMS.build(spec.mixer_norm)
        self.mixer = MIXERS.build(spec.mixer)
        self.feed_forward_norm = None if spec.feed_forward_norm is None else NORMS.build(spec.feed_forward_norm)
        self.feed_forward = None if spec.feed_forward is None else FEED_FORWARDS.build(spec.feed_forward)
        self.connections: List[tuple] = []          # per sublayer: (in, out, mix)

    def parts(self):
        return (self.mixer_norm, self.mixer) + (() if self.feed_forward is None else (self.feed_forward_norm, self.feed_forward))

    def weight_specs(self, prefix: str = "") -> List[WeightSpec]:
        out: List[WeightSpec] = []
        for part in self.parts():
            out += part.weight_specs(self.spec.prefix)
        S = self.streams
        for n in self.names:
            p = self.spec.prefix + n
            out += [WeightSpec(p + ".in", (S,), "vector", ("normal_around", 0.2, 1.0 / S)),
                    WeightSpec(p + ".out", (S,), "vector", ("one_plus_normal", 0.2)),
                    WeightSpec(p + ".mix", (S, S), "vector", ("normal_around", 0.2, 1.0 / S))]
        return out

    def bind(self, get) -> None:
        for part in self.parts():
            part.bind(lambda name: get(self.spec.prefix + name))
        self.connections = [tuple(get(self.spec.prefix + n + s).contiguous() for s in (".in", ".out", ".mix")) for n in self.names]

    def _read(self, x, ctx, which: int, norm):
        from .. import kernels as K
        h = ctx.empty((x.shape[0], self.spec.mixer.hidden_size))
        K.hyper(x, self.streams, ctx.stream, in_w=self.connections[which][0], norm_w=norm.weight, eps=norm.spec.eps, h=h)
        return h

    def _join(self, y, which: int, x, ctx, following):
        """Sublayer ``which`` has left its result in y: write it into the streams, and read for what follows.  ``following``:
        (in, norm) of the next sublayer, or "sum" after the last block of the model, or None."""
        from .. import kernels as K
        _, out_w, mix = self.connections[which]
        W = self.spec.mixer.hidden_size
        if following == "sum":
            ones = ctx.scratch.get("stream_ones")
            if ones is None or ones.numel() != self.streams:
                ones = ctx.scratch["stream_ones"] = torch.ones(self.streams, dtype=torch.float32, device=ctx.device)
            total = ctx.empty((x.shape[0], W), torch.float32)
            K.hyper(x, self.streams, ctx.stream, y=y, mix=mix, out_w=out_w, in_w=ones, h=total)
            ctx.carried["stream_sum"] = (total, ctx.run + 1)
            return None
        if following is None:
            K.hyper(x, self.streams, ctx.stream, y=y, mix=mix, out_w=out_w)
            return None
        in_w, norm = following
        h = ctx.empty((x.shape[0], W))
        K.hyper(x, self.streams, ctx.stream, y=y, mix=mix, out_w=out_w, in_w=in_w, norm_w=norm.weight, eps=norm.spec.eps, h=h)
        return h

    def forward(self, x: torch.Tensor, ctx, cache) -> None:
        W = self.spec.mixer.hidden_size
        if x.shape[1] != self.streams * W:
            raise ValueError(f"the hyper arrangement of {self.streams} streams was given rows of {x.shape[1]} elements, not {self.streams * W}")
        y = ctx.carried.get("sublayer_sum")
        if y is None or y.shape != (x.shape[0], W):
            y = ctx.carried["sublayer_sum"] = torch.zeros((x.shape[0], W), dtype=torch.float32, device=ctx.device)   # zeroed once a step; the joining kernel leaves it zeroed
        kept = ctx.carried.pop("normed_rows", None)
        h = kept[0] if kept is not None and kept[1] == ctx.run and kept[0].shape == (x.shape[0], W) else self._read(x, ctx, 0, self.mixer_norm)
        self.mixer.forward(h, ctx, cache, y)
        nxt = ctx.next_block
        if nxt is None:
            following = "sum"
        elif isinstance(nxt, HyperConnectionBlock) and nxt.streams == self.streams and ctx.options.get("fuse_hyper", True):
            following = (nxt.connections[0][0], nxt.mixer_norm)
        else:
            following = None
        if self.feed_forward is None:
            h = self._join(y, 0, x, ctx, following)
        else:
            h = self._join(y, 0, x, ctx, (self.connections[1][0], self.feed_forward_norm))
            self.feed_forward.forward(h, ctx, y)
            h = self._join(y, 1, x, ctx, following)
        if h is not None:
            ctx.carried["normed_rows"] = (h, ctx.run + 1)


BLOCKS.register("hyper", HyperConnectionBlock)


class ParallelBlock(Part):
    """``parallel``: ONE norm, and both sublayers read its output:

        h = norm(x);   x += mult * (mixer(h) + feed_forward(h))

    ``mult`` is ``LayerSpec.extra["residual_mult"]`` (1 if absent); the feed-forward may be absent.  Mixer and feed-forward
    add into a zeroed float32 buffer of the step; one kernel then adds that buffer, times ``mult``, to the residual stream,
    leaves it zeroed and, where the block that runs next is of this arrangement with an RMS norm (in groups or not), writes
    that norm's rows, which the next block finds in ``ctx.carried``.  A layer runs one such kernel and, but for the first
    layer of a step, no norm kernel of its own."""

    def __init__(self, spec):
        if spec.mixer_norm is None or spec.feed_forward_norm is not None or spec.norms:
            raise ValueError("the parallel arrangement takes one norm (the mixer's), a mixer, and a feed-forward or none")
        self.spec = spec
        self.mult = float(spec.option("residual_mult", 1.0))
        self.mixer_norm = NORMS.build(spec.mixer_norm)
        self.mixer = MIXERS.build(spec.mixer)
        self.feed_forward = None if spec.feed_forward is None else FEED_FORWARDS.build(spec.feed_forward)

    def parts(self):
        return (self.mixer_norm, self.mixer) + (() if self.feed_forward is None else (self.feed_forward,))

    def weight_specs(self, prefix: str = "") -> List[WeightSpec]:
        out: List[WeightSpec] = []
        for part in self.parts():
            out += part.weight_specs(self.spec.prefix)
        return out

    def bind(self, get) -> None:
        for part in self.parts():
            part.bind(lambda name: get(self.spec.prefix + name))

    def forward(self, x: torch.Tensor, ctx, cache) -> None:
        from .. import kernels as K
        y = ctx.carried.get("sublayer_sum")
        if y is None or y.shape != x.shape:
            y = ctx.carried["sublayer_sum"] = torch.zeros_like(x)         # zeroed once a step; the joining kernel leaves it zeroed
        kept = ctx.carried.pop("normed_rows", None)
        h = kept[0] if kept is not None and kept[1] == ctx.run and kept[0].shape == x.shape else self.mixer_norm.forward(x, ctx)
        self.mixer.forward(h, ctx, cache, y)
        if self.feed_forward is not None:
            self.feed_forward.forward(h, ctx, y)
        nxt = ctx.next_block
        following = nxt.mixer_norm if isinstance(nxt, ParallelBlock) and hasattr(nxt.mixer_norm, "groups") and ctx.options.get("fuse_parallel_norm", True) else None
        if following is None:
            K.residual_group_norm(y, self.mult, x, ctx.stream)
            return
        h = ctx.empty(tuple(x.shape))
        K.residual_group_norm(y, self.mult, x, ctx.stream, norm_w=following.weight, groups=following.groups, eps=following.spec.eps, h=h)
        ctx.carried["normed_rows"] = (h, ctx.run + 1)


BLOCKS.register("parallel", ParallelBlock)
