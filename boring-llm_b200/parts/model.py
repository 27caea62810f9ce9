"""A decoder put together from parts, with the order of its layers as data."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from ..weights import TensorSpec
from .base import Part, takes_pending_norm


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order: run block `block` on cache layer `cache`. A block may be named
    by several entries (its weights run twice), and an entry with `write_cache` false reads the
    cache layer that an earlier entry wrote instead of writing one of its own. A block whose mixer
    keeps several caches (pages AND a state slot: its `cache_spec()` is a tuple) names as many cache
    layers, as a tuple."""
    block: int
    cache: Optional[object]          # int, or a tuple of ints for a block with several caches
    write_cache: bool = True

    def cache_layers(self) -> tuple:
        if self.cache is None:
            return ()
        return tuple(self.cache) if isinstance(self.cache, (tuple, list)) else (self.cache,)


class DecoderModel(Part):
    """embedding -> blocks in `schedule` order -> final norm -> output head.

    The reference runs its layers in a fixed loop (src/model.br:1297-1358); here the loop's order is
    a list so that models which repeat layers or share caches need no new code.
    """

    def __init__(self, embedding, blocks: Sequence[Part], final_norm, head,
                 schedule: Optional[Sequence[LayerCall]] = None, ignorable_tensors: Sequence[str] = (),
                 depth_mix: Optional[Sequence[Part]] = None):
        """`depth_mix`: one part per entry of the run order (`parts.depth.DepthWeightedAverage`); entry i's part turns the
        streams X_0 .. X_(i+1) (the embedding rows and what each entry so far left) into what the next entry, or the
        final norm, reads. Without it every entry reads what the one before left."""
        super().__init__()
        self.embedding, self.blocks, self.final_norm, self.head = embedding, list(blocks), final_norm, head
        self.depth_mix = list(depth_mix) if depth_mix is not None else None
        self.schedule: List[LayerCall] = list(schedule) if schedule is not None else self._default_order()
        self.keep_streams = None                # a list: every forward pass appends a copy of the stream behind each entry (tests)
        self.ignorable_tensors = tuple(ignorable_tensors)
        written = set()
        for call in self.schedule:
            if not 0 <= call.block < len(self.blocks):
                raise ValueError(f"run order names block {call.block}, but there are {len(self.blocks)}")
            for c in call.cache_layers():
                if call.write_cache:
                    if c in written:
                        raise ValueError(f"cache layer {c} is written by two entries of the run order")
                    written.add(c)
                elif c not in written:
                    raise ValueError(f"an entry reads cache layer {c} before any entry writes it")
        if self.depth_mix is not None and len(self.depth_mix) != len(self.schedule):
            raise ValueError(f"{len(self.depth_mix)} depth-mix parts for {len(self.schedule)} entries of the run order")

    def _default_order(self) -> List[LayerCall]:
        """Every block once, in order, each with cache layers of its own: cache layer i for block i, or, in a model with
        blocks that keep several caches, numbered through (one per cache)."""
        specs = [b.cache_spec() for b in self.blocks]
        if not any(isinstance(sp, tuple) for sp in specs):
            return [LayerCall(i, i if sp is not None else None) for i, sp in enumerate(specs)]
        order, nxt = [], 0
        for i, spec in enumerate(specs):
            if spec is None:
                order.append(LayerCall(i, None))
            elif isinstance(spec, tuple):
                order.append(LayerCall(i, tuple(range(nxt, nxt + len(spec)))))
                nxt += len(spec)
            else:
                order.append(LayerCall(i, nxt))
                nxt += 1
        return order

    def children(self):
        return (self.embedding, *self.blocks, *(self.depth_mix or ()), self.final_norm, self.head)

    @property
    def vocab_size(self) -> int:
        return self.head.vocab

    @property
    def graph_safe(self) -> bool:
        """Whether a decode step of this model may be captured in a CUDA graph and replayed."""
        return all(getattr(b, "graph_safe", False) for b in self.blocks)

    def cache_specs(self) -> list:
        """What each cache layer needs, indexed by cache layer (None where unused)."""
        n = 1 + max([c for call in self.schedule for c in call.cache_layers()], default=-1)
        specs = [None] * n
        for call in self.schedule:
            layers = call.cache_layers()
            if not layers:
                continue
            spec = self.blocks[call.block].cache_spec()
            each = spec if isinstance(spec, tuple) else (spec,)
            if len(each) != len(layers):
                raise ValueError(f"block {call.block} keeps {len(each)} caches, its entry of the run order names {len(layers)} cache layers")
            for c, sp in zip(layers, each):
                if specs[c] is not None and specs[c] != sp:
                    raise ValueError(f"cache layer {c} is shared by layers with different needs")
                specs[c] = sp
        return specs

    def forward(self, ctx) -> torch.Tensor:
        """Runs the tokens of `ctx` through every layer and returns 32-bit logits at `ctx.logit_rows`."""
        ctx.memo.clear()                        # a context may be run again (before a capture, at a replay's capture): nothing is carried over
        if self.depth_mix is not None:
            x = self._forward_depth_mixed(ctx)
            return self._logits(ctx, x)
        x = self.embedding.forward(ctx)
        for i, call in enumerate(self.schedule):
            # the norm that reads the stream after this block: the next block's first (the final norm reads a few rows only)
            after = self.blocks[self.schedule[i + 1].block] if i + 1 < len(self.schedule) else None
            reader = getattr(after, "mixer", None)
            ctx.norm_after_block = getattr(after, "mixer_norm", None) if takes_pending_norm(reader, x.shape[0]) else None
            self.blocks[call.block].forward(ctx, x, call.cache, call.write_cache)
            if self.keep_streams is not None:
                self.keep_streams.append(x.clone())
        ctx.norm_after_block = None
        return self._logits(ctx, x)

    def _forward_depth_mixed(self, ctx) -> torch.Tensor:
        """All streams live in one buffer [entries + 2, T, dim]: stream 0 the embedding rows; entry i works in place in
        stream i + 1, which its predecessor's mix has filled with what it reads, and leaves X_(i+1) there; its own mix
        writes stream i + 2. Nothing is copied but the embedding rows, once."""
        n = len(self.schedule)
        streams = ctx.empty((n + 2, ctx.T, self.embedding.dim), torch.float32)
        self.embedding.forward(ctx, out=streams[0])
        streams[1].copy_(streams[0])
        ctx.norm_after_block = None
        from .depth import AfterBlock
        for i, call in enumerate(self.schedule):
            nxt = self.blocks[self.schedule[i + 1].block] if i + 1 < n else None
            after = AfterBlock(self.depth_mix[i], streams, streams[i + 2], getattr(nxt, "mixer_norm", None))
            ctx.after_block = after                  # a block may fold the average (and the next block's first norm) into its last kernel
            self.blocks[call.block].forward(ctx, streams[i + 1], call.cache, call.write_cache)
            ctx.after_block = None
            after.run_unfused(ctx)
        ctx.memo["streams"] = streams            # for whoever wants to look at the stream after each entry (tests)
        return streams[n + 1]

    def _logits(self, ctx, x) -> torch.Tensor:
        if ctx.logit_rows.shape[0] == 0:
            return ctx.empty((0, self.vocab_size), torch.float32)
        fused = getattr(self.head, "forward_fused_norm", None)
        logits = fused(ctx, x, self.final_norm, ctx.logit_rows) if fused is not None else None
        if logits is None:
            logits = self.head.forward(ctx, self.final_norm.forward(ctx, x, ctx.logit_rows))
        return logits
