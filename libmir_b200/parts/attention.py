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
cache of the schedule entry that its own entry names).
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
        self.gate_width = self.out_width if s.gate else 0
        self.kv_columns = self.kv_width + self.v_width if s.own_kv else 0       # columns of k and v in a packed row
        self.packed_width = self.q_width + self.kv_columns + self.gate_width
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = self.q_norm = self.k_norm = self.sinks = None

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
        if s.qk_norm:
            table["q_norm.weight"] = ParamSpec((s.head_dim,), init="ones", store="float32")
            if s.own_kv:
                table["k_norm.weight"] = ParamSpec((s.head_dim,), init="ones", store="float32")
        if s.gate:
            table["g_proj.weight"] = ParamSpec((self.out_width, s.hidden_size))
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
        self.w_qkv = torch.cat(weights, dim=0)
        self.w_o = tensors["o_proj.weight"].contiguous()
        if self.spec.qkv_bias:
            biases = [tensors[f"{name}.bias"] for name in projections]
            if self.spec.gate:                    # the gate's projection has no bias
                biases.append(torch.zeros(self.gate_width, dtype=biases[0].dtype, device=biases[0].device))
            self.b_qkv = torch.cat(biases, dim=0)
        if self.spec.out_bias:
            self.b_o = tensors["o_proj.bias"].contiguous()
        if self.spec.qk_norm:
            self.q_norm = tensors["q_norm.weight"].contiguous()
            self.k_norm = tensors["k_norm.weight"].contiguous() if self.spec.own_kv else None
        if self.spec.sinks:
            self.sinks = tensors["sinks"].contiguous()

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_qkv, self.w_o, self.b_qkv, self.b_o, self.sinks)
                   if t is not None)

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
        if rotation is None:
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
        gate = qkv[:, self.q_width + self.kv_columns:] if s.gate else None      # [tokens, heads * value_dim] view
        fast = self.env.dtype == torch.bfloat16 and s.head_dim in kernels.FAST_HEAD_DIMS and s.value_dim == s.head_dim
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
                                        gate=gate)
