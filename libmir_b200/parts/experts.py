"""A mixture of gated experts with a routed choice per token, and an optional shared expert.

With h the feed-forward's input, E experts of which each token uses `top`:
    s = sigmoid(W_router h)                        32-bit: the product accumulates and leaves its result in 32-bit (the
                                                   weights are the stored 16-bit values, h its 16-bit rounding)
    choice = s + correction                        the correction steers the choice only
    a group = E / groups neighbouring experts; its score = the sum of its two largest choice scores; only experts
    of the `keep_groups` best groups can be chosen (the others count as minus infinity)
    chosen = the `top` experts with the largest choice scores;  weight = s[chosen] / (sum of them + 1e-20) * scale
    out = sum over chosen of weight * expert(h)    expert(h) = W_down (silu(W_gate h) * (W_up h))
        + sigmoid(w_sg . h) * shared(h)            one number per token gates the shared expert, if there is one
Other forms from the spec: s = softmax(W_router h) over all the router's outputs; a group's score = its largest choice
score; the last `identity` outputs of the router are identity experts, which have no tensors and whose result is h
itself (they take part in scores, groups and choice; the ordered pairs leave them out, and the kernel that adds the
weighted rows reads h for them); a shared expert without a gate.
Everything runs on the device without a count ever being read back (csrc/moe.cu): the (token, expert) pairs are
ordered by expert, two grouped products run over the ordered pairs with each pair's expert's weights (in bfloat16 on
tensor cores: the tcgen05 product of csrc/gemm_tc.cu on row tiles from a list on the device; in float32 as 32-bit
multiply-adds), and one kernel adds the weighted rows, and the shared
expert's, into the 32-bit residual.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..config.spec import ParamSpec
from .base import FeedForward


class RoutedExperts(FeedForward):
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        s = spec
        self.routed = s.experts + s.identity          # the router's outputs: experts with weights, then identity experts
        if s.experts <= 0 or s.identity < 0 or not 0 < s.top <= self.routed or s.groups <= 0 or self.routed % s.groups \
                or not 0 < s.keep_groups <= s.groups or s.keep_groups * (self.routed // s.groups) < s.top:
            raise ValueError(f"routed experts: {s.top} of {self.routed} experts cannot be chosen from {s.keep_groups} of "
                             f"{s.groups} groups")
        if s.score not in ("sigmoid", "softmax") or s.group_score not in ("top2", "max"):
            raise ValueError(f"routed experts: unknown score rule {s.score!r} / {s.group_score!r}")
        self.router = self.correction = self.w_gate = self.w_up = self.w_down = None
        self.shared_gate_up = self.shared_down = None
        self.shared_gate = False

    def parameters(self):
        s = self.spec
        matrix = lambda rows, columns: ParamSpec((rows, columns), accept_transposed=False)
        table = {"router": matrix(self.routed, s.hidden_size)}
        if s.correction:
            table["correction"] = ParamSpec((self.routed,), init="zeros", store="float32")
        for expert in range(s.experts):
            table[f"e{expert}.gate"] = matrix(s.expert_size, s.hidden_size)
            table[f"e{expert}.up"] = matrix(s.expert_size, s.hidden_size)
            table[f"e{expert}.down"] = matrix(s.hidden_size, s.expert_size)
        if s.shared_size:
            table["shared.gate"] = matrix(s.shared_size, s.hidden_size)
            table["shared.up"] = matrix(s.shared_size, s.hidden_size)
            table["shared.down"] = matrix(s.hidden_size, s.shared_size)
            if s.shared_gate:
                table["shared.sg"] = matrix(1, s.hidden_size)
        return table

    def bind(self, tensors):
        s = self.spec
        # the router's rows and, behind them, the shared expert's gate row: one product gives every 32-bit logit
        rows = [tensors["router"]] + ([tensors["shared.sg"].reshape(1, -1)] if s.shared_size and s.shared_gate else [])
        padding = -(self.routed + len(rows) - 1) % 8
        if padding:
            rows.append(torch.zeros((padding, s.hidden_size), dtype=tensors["router"].dtype, device=tensors["router"].device))
        self.router = torch.cat(rows, dim=0).contiguous()
        self.correction = tensors["correction"].contiguous() if s.correction else None
        stack = lambda name: torch.stack([tensors[f"e{expert}.{name}"] for expert in range(s.experts)]).contiguous()
        # gate and up rows of all experts in one tensor, the up rows behind the gate rows: the tcgen05 grouped product
        # reads an expert's two slices through one tensor map
        gate_up = torch.cat([stack("gate"), stack("up")], dim=0).contiguous()
        self.w_gate, self.w_up, self.w_down = gate_up[:s.experts], gate_up[s.experts:], stack("down")
        if s.shared_size:
            self.shared_gate_up = torch.cat([tensors["shared.gate"], tensors["shared.up"]], dim=0)
            self.shared_down = tensors["shared.down"].contiguous()
            self.shared_gate = bool(s.shared_gate)

    def weight_bytes(self):
        """What a step reads at most: the router, the shared expert, and `top` experts per token would be the least; a
        large batch reads every expert."""
        tensors = (self.router, self.w_gate, self.w_up, self.w_down, self.shared_gate_up, self.shared_down)
        return sum(t.numel() * t.element_size() for t in tensors if t is not None)

    def forward(self, ctx, x, residual, overwrite=False):
        """residual += the experts' weighted results; with `overwrite` they replace `residual` (a 32-bit buffer of an
        arrangement that takes the branch's result by itself)."""
        s = self.spec
        tokens = x.shape[0]
        dtype = self.env.dtype
        ids = ctx.alloc((tokens, s.top), torch.int32)
        weights = ctx.alloc((tokens, s.top), torch.float32)
        gate = ctx.alloc((tokens,), torch.float32) if self.shared_gate else None
        logits = ctx.alloc((tokens, self.router.shape[0]), torch.float32)
        kernels.linear(x, self.router, logits, alloc=ctx.alloc)       # 32-bit accumulation and result
        kernels.moe_route(logits, self.correction, self.shared_gate, ids, weights, gate, self.routed, s.top, s.groups,
                          s.keep_groups, s.scale, score=s.score, group_score=s.group_score)
        found = kernels.moe_sort(ids, s.experts, ctx.alloc, kernels.expert_tile_pairs(dtype, s.hidden_size, s.expert_size))
        hidden = ctx.alloc((tokens * s.top, s.expert_size), dtype)
        kernels.moe_gate_up(x, found, s.top, self.w_gate, self.w_up, hidden, ctx.alloc)
        pair_rows = ctx.alloc((tokens * s.top, s.hidden_size), torch.float32)
        kernels.moe_down(hidden, found, self.w_down, pair_rows)
        shared_rows = None
        if s.shared_size:
            shared_hidden = ctx.alloc((tokens, s.shared_size), dtype)
            kernels.gate_up_silu(x, self.shared_gate_up, shared_hidden, ctx.alloc)
            shared_rows = ctx.alloc((tokens, s.hidden_size), torch.float32)
            kernels.linear(shared_hidden, self.shared_down, shared_rows, alloc=ctx.alloc)
        kernels.moe_combine(residual, pair_rows, weights, shared_rows, gate, overwrite=overwrite,
                            ids=ids if s.identity else None, real_experts=s.experts,
                            identity_rows=x if s.identity else None)
        ctx.residual_stats = None
