"""Grouped-query softmax attention over the paged cache.

input [T, H] -> one packed projection [T, (Hq + 2 Hkv) D] (weights row-stacked [Wq; Wk; Wv] as libmir's
CUDA loader packs them, cuda/src/backend/linear/pack.rs:35-76) -> per-head q/k RMSNorm and rotary,
K and V written to their pages (one kernel) -> attention over the request's pages -> output projection
accumulated into the 32-bit residual.  Formulas: metal/src/engine/dense/swiglu/attention.rs:14-112.
Options, all from the spec: q/k-norm, q/k/v bias and output bias, window, scale, position encoding, a value width
of its own (value_head_dim), first tokens that a window keeps visible (keep_first), stored names of the tensors,
one sink per query head in the softmax's denominator (sinks), a sigmoid gate on the concatenated heads from a
projection of the mixer's input (gate: its weight is one more segment of the packed projection, behind q, k and v),
and no keys and values of its own (own_kv False: the packed projection is [Wq; Wg] and the mixer attends over the
cache of the schedule entry that its own entry names).  Further forms, also from the spec: a sink that is a constant of
the design (fixed_sink), a gate with one number per head (gate_per_head), a q/k norm over all heads of the projection
at once, a norm without weights or one that follows the rotation (these run the kernel of csrc/qk_prepare.cu), scores
capped by softcap * tanh(score / softcap), and a stored bias by the bucket of the distance between query and key (the
table is spread out to one row per distance when the weights are bound).
"""

from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from ..config.spec import PagedKv, ParamSpec, TensorSource
from ..registry import build_part
from .base import Mixer


class SoftmaxAttention(Mixer):
    takes_normed_residual = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        s = spec
        if s.heads % s.kv_heads:
            raise ValueError("heads must be divisible by kv_heads")
        self.q_width = s.heads * s.head_dim
        self.kv_width = s.kv_heads * s.head_dim
        self.v_width = s.kv_heads * s.value_dim
        self.out_width = s.heads * s.value_dim
        self.stored = dict(s.names)              # local name -> the name the checkpoint uses
        self.position = build_part(s.position, env) if s.position is not None else None
        self.gate_width = (s.heads if s.gate_per_head else self.out_width) if s.gate else 0
        self.kv_columns = self.kv_width + self.v_width if s.own_kv else 0       # columns of k and v in a packed row
        self.packed_width = self.q_width + self.kv_columns + self.gate_width
        if s.gate_per_head:
            self.packed_width += -self.packed_width % 8     # (a gate of one column per head: the rows still end on 16 bytes)
        if s.qk_norm_span not in ("head", "projection"):
            raise ValueError(f"unknown q/k norm span {s.qk_norm_span!r}")
        if s.qk_norm_after_rotation and s.qk_norm_span != "head":
            raise ValueError("only the per-head q/k norm can follow the rotation")
        if s.gate_per_head and not s.gate:
            raise ValueError("gate_per_head describes a gate")
        if s.fixed_sink is not None and s.sinks:
            raise ValueError("a sink is stored or a constant, not both")
        # the q/k treatments that the kernel of csrc/qk_prepare.cu runs (the older kernel knows the per-head norm
        # with a weight, before the rotation)
        self.other_norm = s.qk_norm and (s.qk_norm_span != "head" or not s.qk_norm_weight or s.qk_norm_after_rotation)
        if self.other_norm and not s.own_kv:
            raise ValueError("these q/k norms need keys of the mixer's own")
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = self.q_norm = self.k_norm = self.sinks = None
        self.distance_bias = None
        if s.fixed_sink is not None:
            self.sinks = torch.full((s.heads,), float(s.fixed_sink), dtype=torch.float32, device=env.device)

    @property
    def graph_safe(self):
        return self.position is None or self.position.graph_safe

    def cache_requirement(self):
        s = self.spec
        return PagedKv(s.kv_heads, s.head_dim, s.window, s.value_head_dim if s.value_dim != s.head_dim else None,
                       s.keep_first if s.window is not None else 0)

    # names under which checkpoints store query, key and value as one row-stacked tensor [Wq; Wk; Wv]
    # (models/src/weights/binding/roles/parse.rs: "self_attn.qkv_proj.weight" | "self_attn.query_key_value.weight")
    FUSED_NAMES = ("qkv_proj", "query_key_value")

    def parameters(self):
        s = self.spec
        total = self.q_width + self.kv_width + self.v_width
        ranges = {"q_proj": (0, self.q_width), "k_proj": (self.q_width, self.q_width + self.kv_width),
                  "v_proj": (self.q_width + self.kv_width, total)}

        def fused(projection, suffix):
            if self.stored:                      # a checkpoint with names of its own stores the three separately
                return ()
            return tuple(TensorSource(f"{name}.{suffix}", ranges[projection], total) for name in self.FUSED_NAMES)

        if not s.own_kv:                         # queries alone: keys and values are another entry's
            ranges = {"q_proj": ranges["q_proj"]}
        table = {f"{projection}.weight": ParamSpec((end - begin, s.hidden_size), sources=fused(projection, "weight"))
                 for projection, (begin, end) in ranges.items()}
        table["o_proj.weight"] = ParamSpec((s.hidden_size, self.out_width))
        if s.qkv_bias:
            for projection, (begin, end) in ranges.items():
                table[f"{projection}.bias"] = ParamSpec((end - begin,), sources=fused(projection, "bias"))
        if s.out_bias:
            table["o_proj.bias"] = ParamSpec((s.hidden_size,))
        if s.qk_norm and s.qk_norm_weight:
            whole = s.qk_norm_span == "projection"
            table["q_norm.weight"] = ParamSpec((self.q_width if whole else s.head_dim,), init="ones", store="float32")
            if s.own_kv:
                table["k_norm.weight"] = ParamSpec((self.kv_width if whole else s.head_dim,), init="ones", store="float32")
        if s.gate:
            table["g_proj.weight"] = ParamSpec((self.gate_width, s.hidden_size), accept_transposed=not s.gate_per_head)
        if s.distance_bias is not None:
            table["rel_bias"] = ParamSpec((s.distance_bias.rows, s.heads), init="normal", store="float32",
                                          accept_transposed=False)
        if s.sinks:
            table["sinks"] = ParamSpec((s.heads,), init="zeros", store="float32")
        return {self.stored.get(local, local): param for local, param in table.items()}

    def bind(self, tensors):
        local_of = {stored: local for local, stored in self.stored.items()}
        tensors = {local_of.get(name, name): tensor for name, tensor in tensors.items()}
        projections = ("q_proj", "k_proj", "v_proj") if self.spec.own_kv else ("q_proj",)
        weights = [tensors[f"{name}.weight"] for name in projections]
        if self.spec.gate:
            weights.append(tensors["g_proj.weight"])
        rows = sum(w.shape[0] for w in weights)
        if rows < self.packed_width:              # the packed rows end on a 16-byte boundary
            weights.append(torch.zeros((self.packed_width - rows, weights[0].shape[1]), dtype=weights[0].dtype,
                                       device=weights[0].device))
        self.w_qkv = torch.cat(weights, dim=0)
        self.w_o = tensors["o_proj.weight"].contiguous()
        if self.spec.qkv_bias:
            biases = [tensors[f"{name}.bias"] for name in projections]
            rows = sum(b.numel() for b in biases)
            if rows < self.packed_width:          # the gate's projection has no bias, the padding neither
                biases.append(torch.zeros(self.packed_width - rows, dtype=biases[0].dtype, device=biases[0].device))
            self.b_qkv = torch.cat(biases, dim=0)
        if self.spec.out_bias:
            self.b_o = tensors["o_proj.bias"].contiguous()
        if self.spec.qk_norm and self.spec.qk_norm_weight:
            self.q_norm = tensors["q_norm.weight"].contiguous()
            self.k_norm = tensors["k_norm.weight"].contiguous() if self.spec.own_kv else None
        if self.spec.sinks:
            self.sinks = tensors["sinks"].contiguous()
        if self.spec.fixed_sink is not None:
            self.sinks = torch.full((self.spec.heads,), float(self.spec.fixed_sink), dtype=torch.float32,
                                    device=self.w_o.device)
        if self.spec.distance_bias is not None:
            self.distance_bias = self.bias_by_distance(tensors["rel_bias"].float())

    def bias_by_distance(self, table: torch.Tensor) -> torch.Tensor:
        """The stored table [buckets, heads] spread out to one entry per distance n = 0, 1, ... and laid out [heads,
        distances] for the kernels: entry n is the table's row bucket(n).  It ends where nothing changes any more (the
        last bucket is reached, or the window ends); the kernels use its last entry for every greater distance."""
        import math
        bias = self.spec.distance_bias
        rows, exact = bias.rows, bias.rows // 2

        def bucket(n: int) -> int:
            if n < exact:
                return n
            return min(rows - 1, exact + int(math.floor(math.log(n / exact) / math.log(bias.farthest / exact)
                                                        * (rows - exact))))
        buckets, n = [], 0
        while True:
            buckets.append(bucket(n))
            n += 1
            if buckets[-1] == rows - 1 or (self.spec.window is not None and n >= self.spec.window):
                break
        index = torch.tensor(buckets, dtype=torch.long, device=table.device)
        return table[index].t().contiguous()

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_qkv, self.w_o, self.b_qkv, self.b_o, self.sinks,
                                                          self.distance_bias) if t is not None)

    def forward(self, ctx, cache, x, residual, overwrite=False):
        """residual += attention(x) W_o^T; with `overwrite` the result replaces `residual` (a 32-bit buffer of a
        mixer that combines several branches) instead of being added to it."""
        s = self.spec
        tokens = residual.shape[0]
        if not s.own_kv and cache.writes:
            raise ValueError("an attention mixer without keys and values of its own needs another entry's cache")
        qkv = ctx.alloc((tokens, self.packed_width), self.env.dtype)
        group = ctx.groups[cache.group]
        rotation = self.position.rotation() if self.position is not None else (None, 0)
        interleaved = False
        if rotation is None and getattr(self.position, "interleaved", False) and self.position.magnitude == 1.0:
            # the other pairing of the same rotation: the kernel that norms q and k and writes the cache knows it too
            rotation, interleaved = (self.position.table, self.position.rotary_dim), True
        if self.other_norm and (rotation is None or interleaved):
            raise ValueError("these q/k norms go with the half-split rotation or none")
        if self.other_norm:
            self.project_with_other_norm(ctx, cache, group, x, qkv, *rotation)
        elif rotation is None:
            self.project_with_other_position(ctx, cache, group, x, qkv)
        else:
            self.project(ctx, cache, group, x, qkv, *rotation, interleaved=interleaved)
        mixed = ctx.alloc((tokens, self.out_width), self.env.dtype)
        self.attend(ctx, group, cache, qkv, mixed)
        if overwrite:
            kernels.linear(mixed, self.w_o, residual, self.b_o, alloc=ctx.alloc)
        else:
            ctx.accumulate(mixed, self.w_o, residual, self.b_o)      # may also prepare the norm that follows

    def project(self, ctx, cache, group, x, qkv, table, rotary_dim, interleaved=False):
        """Projection, then per-head norm, rotation and cache write in one kernel."""
        s = self.spec
        kernels.linear(x, self.w_qkv, qkv, self.b_qkv, alloc=ctx.alloc)
        kernels.qk_rope_store(qkv, ctx.positions, group.slot_mapping, table, self.q_norm, self.k_norm,
                              cache.k_pages, cache.v_pages, s.heads, s.kv_heads, s.head_dim, rotary_dim,
                              s.qk_norm_eps, write_kv=cache.writes and s.own_kv, value_dim=s.value_dim,
                              interleaved=interleaved, queries_only=not s.own_kv)

    def project_with_other_norm(self, ctx, cache, group, x, qkv, table, rotary_dim):
        """Projection, then the kernel that knows the norm over a whole projection, the norm without weights and the
        norm behind the rotation; it rotates and writes the cache as well."""
        s = self.spec
        kernels.linear(x, self.w_qkv, qkv, self.b_qkv, alloc=ctx.alloc)
        kernels.qk_prepare(qkv, ctx.positions, group.slot_mapping, table, self.q_norm, self.k_norm, cache.k_pages,
                           cache.v_pages, s.heads, s.kv_heads, s.head_dim, s.value_dim, rotary_dim, s.qk_norm_eps,
                           s.qk_norm_span, after_rotation=s.qk_norm_after_rotation, write_kv=cache.writes)

    def project_with_other_position(self, ctx, cache, group, x, qkv):
        """A position encoding that is no rotation of the kernel's: projection, then the per-head norms alone, then
        the encoding's own `apply` on the q and k views, then keys and values into their pages."""
        s = self.spec
        if not s.own_kv:
            raise ValueError("a position encoding of another kind needs keys of the mixer's own")
        kernels.linear(x, self.w_qkv, qkv, self.b_qkv, alloc=ctx.alloc)
        if s.qk_norm:
            kernels.qk_rope_store(qkv, ctx.positions, None, None, self.q_norm, self.k_norm, None, None, s.heads,
                                  s.kv_heads, s.head_dim, 0, s.qk_norm_eps, keys_in_place=True, value_dim=s.value_dim)
        tokens = qkv.shape[0]
        queries = qkv[:, :self.q_width].view(tokens, s.heads, s.head_dim)
        keys = qkv[:, self.q_width:self.q_width + self.kv_width].view(tokens, s.kv_heads, s.head_dim)
        self.position.apply(ctx, queries, keys)
        if cache.writes:
            kernels.qk_rope_store(qkv, ctx.positions, group.slot_mapping, None, None, None, cache.k_pages,
                                  cache.v_pages, s.heads, s.kv_heads, s.head_dim, 0, s.qk_norm_eps, write_kv=True,
                                  value_dim=s.value_dim)

    def attend(self, ctx, group, cache, qkv, out):
        """Attention of every packed row over its request's pages; the kernel is chosen by dtype and size:
        bfloat16 with head_dim 64 or 128 runs on tensor cores (split over the keys when every row is a
        single decoded token), everything else runs the reference kernel."""
        s = self.spec
        kept = s.keep_first if s.window is not None else 0
        first = self.q_width + self.kv_columns
        gate = qkv[:, first:first + self.gate_width] if s.gate else None        # [tokens, heads * value_dim] or [tokens, heads]
        scored = s.softcap is not None or self.distance_bias is not None or s.gate_per_head
        fast = self.env.dtype == torch.bfloat16 and s.head_dim in kernels.FAST_HEAD_DIMS and s.value_dim == s.head_dim
        if fast and scored and not kept:
            # capped or biased scores, or a gate per head: single tokens split over the keys, portions as tiles of
            # queries, each on the tcgen05 or the mma.sync kernel by size
            extras = dict(sinks=self.sinks, gate_per_head=s.gate_per_head, softcap=s.softcap,
                          distance_bias=self.distance_bias)
            singles = ctx.num_rows if ctx.decode_only else ctx.single_rows
            if singles:
                longest = ctx.max_context if ctx.decode_only else ctx.single_context
                partition, count, floats = kernels.decode_attention_plan(singles, s.heads, s.kv_heads, s.head_dim,
                                                                         cache.page_size, longest)
                scratch = ctx.alloc((floats,), torch.float32) if floats else None
                kernels.decode_attention(qkv[:singles], out[:singles], cache.k_pages, cache.v_pages,
                                         group.block_table[:singles], ctx.positions, cache.page_size, s.heads,
                                         s.kv_heads, s.head_dim, s.scale, s.window, partition, count, scratch,
                                         gate=gate[:singles] if gate is not None else None, **extras)
            if singles < ctx.num_rows:
                kernels.prefill_attention(qkv, out, cache.k_pages, cache.v_pages, group.block_table[singles:],
                                          ctx.query_starts[singles:], ctx.context_lens[singles:], cache.page_size,
                                          s.heads, s.kv_heads, s.head_dim, s.scale, s.window,
                                          portion_tokens=out.shape[0] - singles, gate=gate, **extras)
            return
        fast = fast and not scored
        if fast and kept:
            # kept first keys: single tokens run the mma.sync kernel split over the keys, which walks the kept keys
            # and then the window's (the tcgen05 decode kernel does not know kept keys); portions run as tiles of
            # queries on either tile kernel
            singles = ctx.num_rows if ctx.decode_only else ctx.single_rows
            if singles:
                longest = ctx.max_context if ctx.decode_only else ctx.single_context
                partition, count, floats = kernels.decode_attention_kept_plan(singles, s.heads, s.head_dim, longest)
                scratch = ctx.alloc((floats,), torch.float32) if floats else None
                kernels.decode_attention(qkv[:singles], out[:singles], cache.k_pages, cache.v_pages,
                                         group.block_table[:singles], ctx.positions, cache.page_size, s.heads,
                                         s.kv_heads, s.head_dim, s.scale, s.window, partition, count, scratch,
                                         keep_first=kept, numbering=ctx.alloc((singles,), torch.int32),
                                         sinks=self.sinks, gate=gate[:singles] if gate is not None else None)
            if singles < ctx.num_rows:
                kernels.prefill_attention(qkv, out, cache.k_pages, cache.v_pages, group.block_table[singles:],
                                          ctx.query_starts[singles:], ctx.context_lens[singles:], cache.page_size,
                                          s.heads, s.kv_heads, s.head_dim, s.scale, s.window,
                                          portion_tokens=out.shape[0] - singles, keep_first=kept, sinks=self.sinks,
                                          gate=gate)
            return
        if fast:
            # the single-token rows come first in the batch: they run as decoded tokens (keys split over CTAs, the
            # heads of a KV group in one CTA), the prompt portions after them as tiles of queries
            singles = ctx.num_rows if ctx.decode_only else ctx.single_rows
            if singles:
                longest = ctx.max_context if ctx.decode_only else ctx.single_context
                partition, count, floats = kernels.decode_attention_plan(singles, s.heads, s.kv_heads, s.head_dim,
                                                                         cache.page_size, longest)
                scratch = ctx.alloc((floats,), torch.float32) if floats else None
                kernels.decode_attention(qkv[:singles], out[:singles], cache.k_pages, cache.v_pages,
                                         group.block_table[:singles], ctx.positions, cache.page_size, s.heads,
                                         s.kv_heads, s.head_dim, s.scale, s.window, partition, count, scratch,
                                         sinks=self.sinks, gate=gate[:singles] if gate is not None else None)
            if singles < ctx.num_rows:
                kernels.prefill_attention(qkv, out, cache.k_pages, cache.v_pages, group.block_table[singles:],
                                          ctx.query_starts[singles:], ctx.context_lens[singles:], cache.page_size,
                                          s.heads, s.kv_heads, s.head_dim, s.scale, s.window,
                                          portion_tokens=out.shape[0] - singles, sinks=self.sinks, gate=gate)
            return
        kernels.paged_attention_generic(qkv, out, cache.k_pages, cache.v_pages, group.block_table, ctx.row_of_token,
                                        ctx.positions, cache.page_size, s.heads, s.kv_heads, s.head_dim, s.scale,
                                        s.window, value_dim=s.value_dim,
                                        keep_first=s.keep_first if s.window is not None else 0, sinks=self.sinks,
                                        gate=gate, gate_per_head=s.gate_per_head, softcap=s.softcap,
                                        distance_bias=self.distance_bias)
