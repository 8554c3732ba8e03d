"""A decoder put together from a ModelSpec: embedding, blocks in schedule order, final norm, head.

This class is architecture-neutral: which mixer, feed-forward, norm and position encoding each layer
has, under which names its tensors are stored and in which order layers run is all in the ModelSpec.
Flow as in libmir's metal/src/engine/dense/swiglu/model.rs:117-131 and
cuda/src/backend/model/session/prefill/packed.rs:23-89 (packed rows, final norm and head only on the
rows whose logits are wanted).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from .. import kernels
from ..config.spec import FixedState, ModelSpec, PagedKv, ParamSpec
from ..parts.base import BuildEnv, Part
from ..parts.block import build_block
from ..registry import build_part


@dataclass(frozen=True)
class CacheEntryPlan:
    """What schedule entry `entry` needs from the cache manager."""

    entry: int
    requirement: object            # PagedKv | FixedState | None
    source: int                    # the entry whose storage it uses (itself unless cache_of)
    writes: bool


class DecoderModel:
    def __init__(self, spec: ModelSpec, env: BuildEnv):
        spec.validate()
        self.spec = spec
        self.env = env
        self.blocks = [build_block(layer, env) for layer in spec.layers]
        self.final_norm = build_part(spec.final_norm, env)
        self.embedding_norm = build_part(spec.embedding.norm, env) if spec.embedding.norm is not None else None
        self.embedding: Optional[torch.Tensor] = None
        self.pair_embedding: Optional[torch.Tensor] = None      # the table of token pairs, if the model has one
        self.loop_steps: Optional[torch.Tensor] = None          # [passes, hidden] 32-bit: what each pass of a loop adds
        self.head: Optional[torch.Tensor] = None
        self._runs_key, self._runs_list, self._native = None, [], {}
        self.after_entry = None      # for inspection: called with (schedule index, streams) after every run of a layer

    # -- what the cache manager must provide ------------------------------------
    def cache_plan(self) -> List[CacheEntryPlan]:
        """An entry that reads another's cache must ask for the same shape; its window may differ, and the entry that
        owns the pages then keeps what the widest of them sees (every token, if one of them has no window)."""
        from dataclasses import replace
        schedule = self.spec.schedule
        needs = [self.blocks[entry.layer].cache_requirement() for entry in schedule]
        for index, entry in enumerate(schedule):
            if entry.cache_of is None:
                continue
            mine, other = needs[index], needs[entry.cache_of]
            if isinstance(mine, PagedKv) and isinstance(other, PagedKv):
                if replace(mine, window=None, keep_first=0) != replace(other, window=None, keep_first=0):
                    raise ValueError(f"schedule entry {index} reads the cache of entry {entry.cache_of}, whose shape "
                                     f"{other} differs from its own {mine}")
                if mine.window != other.window or mine.keep_first != other.keep_first:
                    widest = None if None in (mine.window, other.window) else max(mine.window, other.window)
                    kept = max(mine.keep_first, other.keep_first) if widest is not None else 0
                    needs[entry.cache_of] = replace(other, window=widest, keep_first=kept)
            elif other != mine:
                raise ValueError(f"schedule entry {index} reads the cache of entry {entry.cache_of}, whose shape "
                                 f"{other} differs from its own {mine}")
        plan = []
        for index, entry in enumerate(schedule):
            if entry.cache_of is not None:
                plan.append(CacheEntryPlan(index, needs[entry.cache_of], entry.cache_of, False))
            else:
                plan.append(CacheEntryPlan(index, needs[index], index, True))
        return plan

    # -- parameters ---------------------------------------------------------------
    def parameter_table(self) -> Dict[str, Tuple[object, str, ParamSpec]]:
        """Checkpoint name -> (owner, local name, ParamSpec) for every tensor of the model."""
        spec = self.spec
        table: Dict[str, Tuple[object, str, ParamSpec]] = {}
        table[spec.embedding.name] = (self, "embedding", ParamSpec((spec.embedding.vocab_size, spec.embedding.hidden_size)))
        if spec.embedding.pairs is not None:
            pairs = spec.embedding.pairs
            table[pairs.name] = (self, "pair_embedding", ParamSpec((pairs.buckets + 1, spec.embedding.hidden_size)))
        if spec.loop is not None and spec.loop.step_tensor:
            table[spec.loop.step_tensor] = (self, "loop_steps", ParamSpec((spec.loop.passes, spec.hidden_size), init="zeros",
                                                                          store="float32", accept_transposed=False))
        for layer_spec, block in zip(spec.layers, self.blocks):
            for slot, part in block.parts():
                for local, param in part.parameters().items():
                    table[layer_spec.prefix + layer_spec.names[slot] + local] = (part, local, param)
        for local, param in self.final_norm.parameters().items():
            table[spec.final_norm_name + local] = (self.final_norm, local, param)
        if self.embedding_norm is not None:
            for local, param in self.embedding_norm.parameters().items():
                table[spec.embedding.norm_name + local] = (self.embedding_norm, local, param)
        if not spec.head.tied:
            table[spec.head.name] = (self, "head", ParamSpec((spec.head.vocab_size, spec.head.hidden_size)))
        return table

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Hand every loaded tensor (by checkpoint name) to the part that owns it."""
        per_owner: Dict[int, Tuple[object, Dict[str, torch.Tensor]]] = {}
        for name, (owner, local, _) in self.parameter_table().items():
            if name in tensors:
                per_owner.setdefault(id(owner), (owner, {}))[1][local] = tensors[name]
        for owner, local_tensors in per_owner.values():
            if owner is self:
                self.embedding = local_tensors["embedding"].contiguous()
                if "pair_embedding" in local_tensors:
                    self.pair_embedding = local_tensors["pair_embedding"].contiguous()
                self.head = local_tensors.get("head")
                if "loop_steps" in local_tensors:
                    self.loop_steps = local_tensors["loop_steps"].contiguous()
            else:
                owner.bind(local_tensors)
        if self.spec.head.tied:
            self.head = self.embedding
        self.head = self.head.contiguous()
        if self.spec.head.scale != 1.0:
            # logits = scale * head . norm(x): the factor goes into the final norm's 32-bit weight, once
            if not getattr(self.final_norm, "foldable", False):
                raise ValueError("a head with a logit scale needs a final norm with a 32-bit weight to carry it")
            self.final_norm.scale_weight(self.spec.head.scale)
        self._runs_key = None                       # descriptors of the layers hold pointers to the old tensors

    def parts(self) -> List[Part]:
        out: List[Part] = []
        for block in self.blocks:
            out.extend(part for _, part in block.parts())
        out.append(self.final_norm)
        if self.embedding_norm is not None:
            out.append(self.embedding_norm)
        return out

    def portion_multiple(self) -> int:
        """The least common multiple of what the parts ask of the scheduler's cuts (Part.portion_multiple)."""
        import math
        return math.lcm(*[max(1, int(part.portion_multiple)) for part in self.parts()])

    def weight_bytes_per_step(self) -> int:
        """Bytes of weights one step reads: every layer of the schedule once, the final norm and the
        head; the embedding table is only gathered from."""
        total = 0
        for entry in self.spec.schedule:
            total += sum(part.weight_bytes() for _, part in self.blocks[entry.layer].parts())
        total += self.final_norm.weight_bytes() + self.head.numel() * self.head.element_size()
        return total

    def open_pass(self, ctx, entry, residual: torch.Tensor, embedded: Optional[torch.Tensor]) -> None:
        """What a pass of the model's loop starts with: every pass but the first adds the embedding's output to the
        residual, every pass adds its row of the step tensor."""
        loop = self.spec.loop
        rows = embedded if (loop.add_embedding and entry.opens_pass > 0) else None
        vector = self.loop_steps[entry.opens_pass] if self.loop_steps is not None else None
        kernels.add_rows(residual, rows, vector)
        ctx.residual_stats = None

    # -- running --------------------------------------------------------------------
    def forward(self, ctx) -> torch.Tensor:
        """Run the tokens of the step; returns the 32-bit residual [T, H] after the last layer."""
        spec = self.spec
        if spec.streams:
            return self.forward_streams(ctx)
        residual = ctx.alloc((ctx.num_tokens, spec.hidden_size), torch.float32)
        if spec.embedding.pairs is not None:
            pairs = spec.embedding.pairs
            kernels.embed_pairs(self.embedding, self.pair_embedding, ctx.tokens, ctx.previous_tokens, residual,
                                pairs.mul_previous, pairs.mul_current, spec.embedding.multiplier)
        else:
            kernels.embed(self.embedding, ctx.tokens, residual, spec.embedding.multiplier)
        if self.embedding_norm is not None:                  # the stream starts from the normed rows, in 32-bit
            self.embedding_norm.forward(ctx, residual, out=residual)
        embedded = None
        if spec.loop is not None and spec.loop.add_embedding and any((e.opens_pass or 0) > 0 for e in spec.schedule):
            embedded = ctx.alloc(tuple(residual.shape), torch.float32)       # later passes add the embedding's output again
            embedded.copy_(residual)
        ctx.rounded_residual = None          # (a block leaves one only for the block right behind it, which takes it)
        for run in self._runs(ctx):
            if run.layers is not None:
                run.execute(ctx, residual)
                continue
            index = run.first
            entry = spec.schedule[index]
            if entry.opens_pass is not None:
                self.open_pass(ctx, entry, residual, embedded)
            # the norm that the next block in the schedule starts with: this block's last product may prepare it
            following = self.blocks[spec.schedule[index + 1].layer] if index + 1 < len(spec.schedule) else None
            ctx.norm_after_block = following.first_norm() if following is not None else None
            if index + 1 < len(spec.schedule) and (self._native.get(index + 1) is not None
                                                   or spec.schedule[index + 1].opens_pass is not None):
                ctx.norm_after_block = None          # the next block starts from a residual that this one has not seen
            ctx.next_reads_residual = (following is not None and getattr(following, "reads_residual_itself", False)
                                       and self._native.get(index + 1) is None
                                       and spec.schedule[index + 1].opens_pass is None)
            self.blocks[entry.layer].forward(ctx, ctx.cache_view(index), residual)
        return residual

    def forward_streams(self, ctx) -> torch.Tensor:
        """A residual kept as several streams [T, S, H]: every stream starts as the embedding's output, the blocks (of
        the "streams" arrangement, run part by part) read and write all of them, and what the final norm gets is
        their sum."""
        spec = self.spec
        if spec.embedding.pairs is not None or spec.loop is not None:
            raise ValueError("a residual of several streams goes with a plain embedding and a loop without additions")
        embedded = ctx.alloc((ctx.num_tokens, spec.hidden_size), torch.float32)
        kernels.embed(self.embedding, ctx.tokens, embedded, spec.embedding.multiplier)
        if self.embedding_norm is not None:
            self.embedding_norm.forward(ctx, embedded, out=embedded)
        streams = ctx.alloc((ctx.num_tokens, spec.streams, spec.hidden_size), torch.float32)
        kernels.streams_spread(embedded, streams)
        ctx.rounded_residual = None
        ctx.norm_after_block = None
        ctx.next_reads_residual = False
        ctx.normed_streams = None
        for index, entry in enumerate(spec.schedule):
            # who reads the streams first in the next block: this block's last update norms their mix on the way out
            following = self.blocks[spec.schedule[index + 1].layer] if index + 1 < len(spec.schedule) else None
            ctx.streams_reader_after_block = following.first_reader() if following is not None else "sum"
            self.blocks[entry.layer].forward(ctx, ctx.cache_view(index), streams)
            if self.after_entry is not None:
                self.after_entry(index, streams)
        total, ctx.streams_reader_after_block, ctx.normed_streams = ctx.normed_streams, None, None
        if total is not None and total.dtype == torch.float32 and total.shape == embedded.shape:
            return total                     # the last update left the streams' sum
        kernels.streams_sum(streams, embedded)
        return embedded

    def _runs(self, ctx) -> list:
        """The schedule cut into runs: consecutive entries whose blocks the native executor takes form one run (one
        native call), every other entry runs part by part from Python.  Built once per cache storage, since the
        descriptors hold pointers to its pages."""
        key = id(ctx.views)
        if self._runs_key == key:
            return self._runs_list
        from ..kernels.executor import LayerRun
        self._native = {}
        if kernels.NATIVE_LAYERS:
            for index, entry in enumerate(self.spec.schedule):
                self._native[index] = self.blocks[entry.layer].native_descriptor(ctx.cache_view(index)) \
                    if entry.opens_pass is None else None        # (a pass opens from Python, before its first block)
        runs, index = [], 0
        while index < len(self.spec.schedule):
            if self._native.get(index) is None:
                runs.append(LayerRun(index, None, self.env.dtype))
                index += 1
                continue
            last = index
            while last + 1 < len(self.spec.schedule) and self._native.get(last + 1) is not None:
                last += 1
            runs.append(LayerRun(index, [self._native[i] for i in range(index, last + 1)], self.env.dtype))
            index = last + 1
        self._runs_key, self._runs_list = key, runs
        return runs

    def logits(self, ctx, residual: torch.Tensor, rows: torch.Tensor, out: Optional[torch.Tensor] = None,
               candidates=None) -> torch.Tensor:
        """32-bit logits [len(rows), V] at the packed rows `rows` (an int32 device tensor).  `candidates`
        (kernels.HeadCandidates): filled by the head's kernel where it can, for the sampling that follows."""
        normed = self.final_norm.forward(ctx, residual, rows=rows)
        if out is None:
            out = ctx.alloc((rows.numel(), self.spec.vocab_size), torch.float32)
        kernels.head_logits(normed, self.head, out, candidates)
        if self.spec.head.softcap:
            kernels.softcap(out, self.spec.head.softcap)
            if candidates is not None:
                candidates.valid = False             # (they hold the logits as they were before the cap)
        return out
