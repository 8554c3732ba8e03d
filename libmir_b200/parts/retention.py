"""Retention: linear attention with one fixed decay per head, no softmax and no denominator.

With h the mixer's input, H heads, key width D and value width V:
    q, k, v = W_q h, W_k h, W_v h                 per head [D], [D], [V]; no biases
    q, k    = rotated by the token's position     (the position encoding of the spec), then k times D^-1/2
    S_t     = decay_h S_t-1 + k_t v_t^T           per head, S [D, V], zeros at a request's start
    o_t     = S_t^T q_t
    y       = o / rms(o) per head * silu(W_g h)   no weight in the norm
    out     = W_o y
Per request the mixer keeps S of every head (32-bit) in the request's state slot.  The rotation, the decay, the state
and the recurrence are 32-bit (csrc/retention.cu rotates while it stages the projections' results, or for prompts'
portions in a kernel of its own into 32-bit scratch, so nothing rotated is rounded to the engine's dtype); the
projections run in the engine's dtype.  All four projections that read h are one product on row-stacked weights
[Wq; Wk; Wv; Wg], each segment padded to a multiple of eight rows so that the views into the packed result stay
16-byte aligned.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..config.spec import FixedState, ParamSpec
from ..registry import build_part
from .base import Mixer


def _pad8(n: int) -> int:
    return -(-n // 8) * 8


class Retention(Mixer):
    graph_safe = True          # the batch is read from device tensors only; padding rows (position < 0) are skipped
    takes_normed_residual = True   # x is used by one product only, which can take a folded norm over

    def __init__(self, spec, env):
        super().__init__(spec, env)
        s = spec
        if min(s.heads, s.key_dim, s.value_dim) <= 0 or len(s.decays) != s.heads:
            raise ValueError("retention needs heads, key_dim and value_dim above zero and one decay per head")
        if s.key_dim > 256:
            raise ValueError("the recurrence kernel takes key heads up to 256 wide")
        self.qk_width = s.heads * s.key_dim
        self.v_width = s.heads * s.value_dim
        self.position = build_part(s.position, env) if s.position is not None else None
        if self.position is not None and (getattr(self.position, "interleaved", False)
                                          or getattr(self.position, "magnitude", 1.0) != 1.0
                                          or not hasattr(self.position, "table")):
            raise ValueError("retention rotates half-split pairs with plain cos and sin only")
        # segments of the packed projection: name -> first column
        self.offsets, cursor = {}, 0
        for name, width in (("q", self.qk_width), ("k", self.qk_width), ("v", self.v_width), ("g", self.v_width)):
            self.offsets[name] = cursor
            cursor = _pad8(cursor + width)
        self.packed_width = cursor
        self.decays = torch.tensor(list(s.decays), dtype=torch.float32, device=env.device)
        self.ones = torch.ones(s.value_dim, dtype=torch.float32, device=env.device)
        self.w_in = self.w_o = None

    def cache_requirement(self):
        s = self.spec
        return FixedState((s.heads, s.value_dim, s.key_dim), "float32")

    def parameters(self):
        s = self.spec
        matrix = lambda rows, columns: ParamSpec((rows, columns), accept_transposed=False)
        return {"q": matrix(self.qk_width, s.hidden_size), "k": matrix(self.qk_width, s.hidden_size),
                "v": matrix(self.v_width, s.hidden_size), "g": matrix(self.v_width, s.hidden_size),
                "o": matrix(s.hidden_size, self.v_width)}

    def bind(self, tensors):
        s = self.spec
        sample = tensors["q"]
        w_in = torch.zeros((self.packed_width, s.hidden_size), dtype=sample.dtype, device=sample.device)
        for name, first in self.offsets.items():
            w_in[first:first + tensors[name].shape[0]] = tensors[name]
        self.w_in = w_in
        self.w_o = tensors["o"].contiguous()

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_o))

    def forward(self, ctx, cache, x, residual, overwrite=False):
        """residual += W_o y (or residual = W_o y with `overwrite`, for an arrangement that norms the result)."""
        s = self.spec
        tokens = residual.shape[0]
        state = cache.states[0] if getattr(cache, "states", None) else cache.state
        packed = ctx.alloc((tokens, self.packed_width), self.env.dtype)
        kernels.linear(x, self.w_in, packed, alloc=ctx.alloc)
        view = lambda name, width: packed[:, self.offsets[name]:self.offsets[name] + width]
        read = ctx.alloc((tokens, self.v_width), torch.float32)
        # a step with portions of prompts rotates once per token and head in a kernel of its own
        prepared = None if ctx.decode_only else ctx.alloc(
            (kernels.retention_prepared_floats(tokens, s.heads, s.key_dim),), torch.float32)
        kernels.retention_scan(view("q", self.qk_width), view("k", self.qk_width), view("v", self.v_width),
                               self.position.table if self.position is not None else None, self.decays,
                               float(s.key_dim) ** -0.5, state, ctx.query_starts, ctx.state_slots, ctx.positions, read,
                               s.heads, s.key_dim, s.value_dim, prepared=prepared)
        mixed = ctx.alloc((tokens, self.v_width), self.env.dtype)
        kernels.gated_head_norm(read, view("g", self.v_width), self.ones, mixed, s.heads, s.value_dim, s.norm_eps, False)
        if overwrite:
            kernels.linear(mixed, self.w_o, residual, alloc=ctx.alloc)
        else:
            ctx.accumulate(mixed, self.w_o, residual)
