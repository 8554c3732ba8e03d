"""Norms of the 32-bit residual.  RMSNorm: y = x * rsqrt(mean(x^2) + eps) * (offset + w); offset 0 is the plain form, offset 1 the form whose
weight is stored around zero (the sum is formed once, in 32-bit, when the weight is bound).

libmir cuda/kernels/rms_norm_bf16.cu:3-36; eps key and aliases models/src/layout/decoder/parse/mod.rs:82-86.
The input is the 32-bit residual stream; the weight is kept in 32-bit (exact for every stored dtype).

LayerNorm (at the end of the file): y = (x - mean) / sqrt(variance + eps) * w + b with the variance as the mean of the
squared deviations; weight and bias 32-bit.  It can form its input on the way in as a mix of the streams of a residual
that is kept as several copies (`read`).
"""

from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from ..config.spec import ParamSpec
from .base import Norm


class RmsNorm(Norm):
    graph_safe = True
    foldable = True       # y = x * s * w with one s per row: the products around it can take it over

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.weight: Optional[torch.Tensor] = None

    def parameters(self):
        init = "zeros" if self.spec.offset else "ones"
        return {self.spec.tensor: ParamSpec((self.spec.size,), init=init, store="float32")}

    def bind(self, tensors):
        weight = tensors[self.spec.tensor].contiguous()
        self.weight = weight + self.spec.offset if self.spec.offset else weight

    def scale_weight(self, factor: float) -> None:
        """Multiply the bound weight by a constant (a model's logit scale carried by its final norm)."""
        self.weight = (self.weight * factor).contiguous()

    def weight_bytes(self):
        return self.weight.numel() * 4

    def forward(self, ctx, x, out=None, rows=None, lazy=False):
        """`lazy`: the caller's next product can take over this norm; if what it needs is at hand (the sums of
        squares of x and its rows times this norm's weight, written by the product that last added into x),
        return a NormedResidual instead of running a kernel."""
        if (lazy and kernels.FUSE_NORM_INTO_PRODUCT and out is None and rows is None
                and self.env.dtype == torch.bfloat16):
            stats = ctx.stats_for(x, self.weight)
            if stats is not None:
                return kernels.NormedResidual(x, self.weight, self.spec.eps, stats[0], stats[1], self.env.dtype,
                                              stats[2])
        n_rows = x.shape[0] if rows is None else rows.numel()
        if out is None:
            out = ctx.alloc((n_rows, self.spec.size), self.env.dtype)
        kernels.rms_norm(x, self.weight, self.spec.eps, out, rows)
        return out


class LayerNorm(Norm):
    graph_safe = True
    foldable = False      # (the mean and the bias keep it out of the products around it)

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def parameters(self):
        return {self.spec.tensor: ParamSpec((self.spec.size,), init="ones", store="float32"),
                self.spec.bias_tensor: ParamSpec((self.spec.size,), init="zeros", store="float32")}

    def bind(self, tensors):
        self.weight = tensors[self.spec.tensor].contiguous()
        self.bias = tensors[self.spec.bias_tensor].contiguous()

    def weight_bytes(self):
        return (self.weight.numel() + self.bias.numel()) * 4

    def forward(self, ctx, x, out=None, rows=None, lazy=False, read=None):
        """`read` (float32 [S]): x is a residual of S streams [tokens, S, width] and the norm's input is their mix
        sum_s read[s] x_s, formed in the same kernel."""
        n_rows = x.shape[0] if rows is None else rows.numel()
        if out is None:
            out = ctx.alloc((n_rows, self.spec.size), self.env.dtype)
        kernels.layer_norm(x, self.weight, self.bias, self.spec.eps, out, rows, read)
        return out
