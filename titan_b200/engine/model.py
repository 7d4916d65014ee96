"""A decoder assembled from a ``ModelSpec``: embedding, blocks in their running order,
final norm and LM head.

The running order is data (``ModelSpec.order``): it may name a layer twice, and
a layer's mixer may read another layer's cache (``MixerSpec.cache_from``).
berniehans/titan hard-codes ``for layer in 0..L`` (engine/engine-core/src/
forward_driver.rs:988, 2149-2334) and computes logits for the last position
only (:1215-1238); here the wanted rows are gathered before the final norm, so
the LM head runs on those rows alone.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import kernels as K
from ..cache.groups import CacheNeed
from ..parts import NORMS, build_block, declare_weights, linear
from ..weights.loader import WeightSource, WeightSpec


class DecoderModel:
    def __init__(self, spec):
        spec.validate()
        self.spec = spec
        self.blocks = [build_block(layer) for layer in spec.layers]
        self.final_norm = NORMS.build(spec.final_norm)
        self.embedding_norm = None if spec.embedding_norm is None else NORMS.build(spec.embedding_norm)
        self.embedding: Optional[torch.Tensor] = None
        self.shared = {}
        self.lm_head: Optional[torch.Tensor] = None

    def declared_weights(self) -> List[WeightSpec]:
        return declare_weights(self.spec)

    def cache_needs(self) -> List[Optional[CacheNeed]]:
        """One entry per RUN of the order, so a layer that runs twice keeps two caches."""
        return [self.blocks[i].mixer.cache_need() for i in self.spec.order]

    def cache_run_of(self, run: int) -> int:
        """The run whose cache the ``run``-th block of the order uses."""
        src = self.spec.layers[self.spec.order[run]].mixer.cache_from
        return run if src is None else self.spec.order.index(src)

    def load(self, source: WeightSource) -> None:
        by_name = {w.name: w for w in self.declared_weights()}
        get = lambda name: source.get(by_name[name])
        self.embedding = get(self.spec.embedding)
        self.shared = {name: get(name) for name, _ in self.spec.shared_tensors}
        for b in self.blocks:
            b.bind(get)
            if hasattr(b, "bind_shared"):
                b.bind_shared(self.shared)
        self.final_norm.bind(get)
        if self.embedding_norm is not None:
            self.embedding_norm.bind(get)
        self.lm_head = self.embedding if self.spec.lm_head is None else get(self.spec.lm_head)

    def weight_bytes(self) -> int:
        """Bytes a decode step reads: every matrix once (the embedding table only as LM head when tied)."""
        seen, total = set(), 0
        def add(t):
            nonlocal total
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        for i in set(self.spec.order):
            for part in self.blocks[i].parts():
                for v in vars(part).values():
                    if isinstance(v, torch.Tensor):
                        add(v)
        add(self.lm_head)
        add(self.final_norm.weight)
        return total

    # ------------------------------------------------------------------ #
    def forward_hidden(self, ctx, cache) -> torch.Tensor:
        """The residual stream [T, H] (float32) after the last block."""
        lay = ctx.layout
        x = torch.empty((lay.T, self.spec.hidden_size), dtype=torch.float32, device=ctx.device)
        K.embed(self.embedding, lay.tokens, x, ctx.stream)
        if self.spec.embedding_scale is not None:
            K.scale_f32(x, float(self.spec.embedding_scale), ctx.stream)
        if self.embedding_norm is not None:    # a norm on the embedded rows; the residual stream stays float32
            x = self.embedding_norm.forward(x, ctx, out_dtype=torch.float32)
        streams = self.spec.streams
        if streams > 1:                        # every stream starts as the embedded rows: [T, streams * H], stream s at columns s * H
            x = x.repeat(1, streams)
        if "row_sums" not in ctx.scratch:      # places where folded norms leave sums of squares: one per run of a layer
            ctx.scratch["row_sums"] = torch.zeros((len(self.spec.order), 16, 32), dtype=torch.float32, device=ctx.device)
        for run, i in enumerate(self.spec.order):
            ctx.run = run
            ctx.next_block = self.blocks[self.spec.order[run + 1]] if run + 1 < len(self.spec.order) else None
            self.blocks[i].forward(x, ctx, cache.view_for_layer(self.cache_run_of(run)))
            if ctx.after_layer is not None:    # an observer of the residual stream after every run of a layer (tests, debugging)
                ctx.after_layer(run, self._stream_sum(x, ctx, peek=True))
        for late in ctx.after_blocks:          # cache rows that a later layer of the step still had to read as they were
            late()
        ctx.after_blocks.clear()
        return self._stream_sum(x, ctx)

    def _stream_sum(self, x: torch.Tensor, ctx, peek: bool = False) -> torch.Tensor:
        """The residual stream that leaves the blocks: x itself, or the sum of the streams (which the last block may have
        left in ``ctx.carried`` already)."""
        streams = self.spec.streams
        if streams == 1:
            return x
        kept = ctx.carried.get("stream_sum") if peek else ctx.carried.pop("stream_sum", None)
        if kept is not None and kept[1] == ctx.run + 1:
            return kept[0]
        total = torch.empty((x.shape[0], self.spec.hidden_size), dtype=torch.float32, device=ctx.device)
        ones = ctx.scratch.get("stream_ones")
        if ones is None or ones.numel() != streams:
            ones = ctx.scratch["stream_ones"] = torch.ones(streams, dtype=torch.float32, device=ctx.device)
        K.hyper(x, streams, ctx.stream, in_w=ones, h=total)
        return total

    def logits(self, x: torch.Tensor, ctx, rows: torch.Tensor) -> torch.Tensor:
        """float32 logits [len(rows), vocab] at the given rows of the residual stream."""
        hn = self.final_norm.forward(x, ctx, rows)
        out = torch.empty((rows.numel(), self.spec.vocab_size), dtype=torch.float32, device=ctx.device)
        linear.matmul(hn, self.lm_head, out, linear.EPI_F32, ctx)
        if self.spec.logit_scale is not None:
            K.scale_f32(out, float(self.spec.logit_scale), ctx.stream)
        return out
