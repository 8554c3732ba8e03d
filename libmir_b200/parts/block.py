"""Arrangements of a mixer and a feed-forward in one layer.

pre_norm:  x += mixer(norm_1(x));  x += feed_forward(norm_2(x))
(metal/src/engine/dense/swiglu/layer.rs:123-166).  The residual stream x is 32-bit; each branch adds
its result into it (the matrix product's accumulate epilogue), so no separate add kernel runs.
A layer without feed-forward, or without one of the norms, leaves that step out.

parallel:  h = norm_1(x);  x += mixer(h) + feed_forward(h)
One norm, and both branches read its output; each adds its result into the 32-bit residual, so the sum
x + mixer(h) + feed_forward(h) is formed in 32-bit whatever the engine's dtype.
With a second norm (`feed_forward_norm`): x += mixer(norm_1(x)) + feed_forward(norm_2(x)), both norms of the same x:
both are computed before either branch adds into the residual, by one kernel where they are RMS norms with one eps
(one root mean square, two weights).

output_norm:  x += m * norm_1(mixer(x));  x += m * norm_2(feed_forward(x))
Each branch reads the residual itself (cast to the engine's dtype) and its RESULT goes through the norm: the branch
writes its result into a 32-bit buffer, and one kernel norms that buffer and adds m times it into the residual, so
the norm and the residual sum are 32-bit.  m is LayerSpec.residual_scale.

streams:  the residual is S copies x_1 .. x_S per token (hyper-connections).  For each of the two sublayers, with its
stored mixing tensors in [S], mix [S, S] and out [S]:  u = sum_s in[s] x_s;  y = sublayer(norm(u));  then all streams
at once from the old ones, x_t <- sum_s mix[s, t] x_s + out[t] y.  Everything outside the sublayer is 32-bit: the
norm's kernel forms u on the way in, the sublayer leaves y in a 32-bit buffer, one kernel updates the streams and, in the
same pass, forms and norms the mix that the next sublayer (of this block or the next) reads.
"""

from __future__ import annotations

import torch

from ..registry import build_part
from .base import Block, Part


class PreNormBlock(Block):
    SLOTS = ("mixer_norm", "mixer", "feed_forward_norm", "feed_forward")

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.mixer_norm = build_part(spec.mixer_norm, env)
        self.mixer = build_part(spec.mixer, env)
        self.feed_forward_norm = build_part(spec.feed_forward_norm, env)
        self.feed_forward = build_part(spec.feed_forward, env)

    def parts(self):
        """(slot name, part) of every part this block holds."""
        return [(slot, getattr(self, slot)) for slot in self.SLOTS if getattr(self, slot) is not None]

    def cache_requirement(self):
        return self.mixer.cache_requirement()

    def first_norm(self):
        """The norm this block applies to the incoming residual before anything else, or None."""
        return self.mixer_norm

    def native_descriptor(self, cache):
        """The layer as the native executor wants it (kernels.executor.LayerDesc), if every part of it is of the
        built-in kind that the executor runs (RMSNorm, softmax attention with the kernel's rotation or no position
        encoding, SwiGLU or no feed-forward) and its weights are bound; else None, and the parts run one by one."""
        from ..kernels.executor import LayerDesc, NormDesc
        from .attention import SoftmaxAttention
        from .feed_forward import SwiGlu
        from .norm import RmsNorm
        mixer, ff = self.mixer, self.feed_forward
        if type(mixer) is not SoftmaxAttention or type(self.mixer_norm) is not RmsNorm or cache is None \
                or cache.k_pages is None or mixer.w_qkv is None:
            return None
        if ff is not None and (type(ff) is not SwiGlu or type(self.feed_forward_norm) is not RmsNorm):
            return None
        if mixer.spec.value_dim != mixer.spec.head_dim or (mixer.spec.window is not None and mixer.spec.keep_first):
            return None                      # the executor knows neither a value width of its own nor kept first tokens
        rotation = mixer.position.rotation() if mixer.position is not None else (None, 0)
        if rotation is None or self.env.dtype not in (torch.bfloat16, torch.float32):
            return None
        s = mixer.spec
        if cache.k_pages.shape[1:] != (s.kv_heads, s.head_dim) or cache.v_pages.shape != cache.k_pages.shape \
                or not cache.k_pages.is_contiguous() or not cache.v_pages.is_contiguous():
            return None
        pointer = lambda tensor: None if tensor is None else tensor.data_ptr()
        norm = lambda part: NormDesc(part.weight.data_ptr(), part.spec.eps, part.spec.size)
        table, rotary_dim = rotation
        desc = LayerDesc()
        desc.mixer_norm = norm(self.mixer_norm)
        desc.w_qkv, desc.b_qkv, desc.w_o, desc.b_o = (pointer(mixer.w_qkv), pointer(mixer.b_qkv), pointer(mixer.w_o),
                                                      pointer(mixer.b_o))
        desc.q_norm, desc.k_norm, desc.inv_freq = pointer(mixer.q_norm), pointer(mixer.k_norm), pointer(table)
        desc.heads, desc.kv_heads, desc.head_dim, desc.rotary_dim = s.heads, s.kv_heads, s.head_dim, rotary_dim
        desc.window, desc.group, desc.writes_cache, desc.page_size = (int(s.window or 0), cache.group, int(cache.writes),
                                                                      cache.page_size)
        desc.scale, desc.qk_eps = s.scale, s.qk_norm_eps
        desc.k_pages, desc.v_pages, desc.cache_rows = cache.k_pages.data_ptr(), cache.v_pages.data_ptr(), cache.k_pages.shape[0]
        if ff is not None:
            desc.ff_norm = norm(self.feed_forward_norm)
            desc.w_gate_up, desc.w_down, desc.inter = ff.w_gate_up.data_ptr(), ff.w_down.data_ptr(), ff.spec.intermediate_size
        return desc

    def forward(self, ctx, cache, residual):
        # Before a part runs, the context is told which norm follows it, so that its last product can prepare
        # that norm (parts.base.PartContext).
        after = ctx.norm_after_block
        x = (self._norm(self.mixer_norm, self.mixer, ctx, residual) if self.mixer_norm is not None
             else ctx.cast_residual(residual))
        ctx.residual_stats = None            # the mixer changes the residual; it may note new sums of squares
        ctx.upcoming_norm = self.feed_forward_norm if self.feed_forward is not None else after
        self.mixer.forward(ctx, cache, x, residual)
        if self.feed_forward is not None:
            x = (self._norm(self.feed_forward_norm, self.feed_forward, ctx, residual)
                 if self.feed_forward_norm is not None else ctx.cast_residual(residual))
            ctx.residual_stats = None
            ctx.upcoming_norm = after
            self.feed_forward.forward(ctx, x, residual)
        ctx.upcoming_norm = None

    @staticmethod
    def _norm(norm, consumer, ctx, residual):
        if consumer.takes_normed_residual and norm.foldable:
            return norm.forward(ctx, residual, lazy=True)
        return norm.forward(ctx, residual)


class ParallelBlock(Block):
    """x += mixer(norm(x)) + feed_forward(norm(x)): the norm runs once and both branches read its output; or, with a
    second norm, x += mixer(norm_1(x)) + feed_forward(norm_2(x)) with both norms taken of the same x."""

    SLOTS = ("mixer_norm", "mixer", "feed_forward_norm", "feed_forward")

    def __init__(self, spec, env):
        super().__init__(spec, env)
        if spec.feed_forward_norm is not None and (spec.feed_forward is None or spec.mixer_norm is None):
            raise ValueError("a second norm in the parallel arrangement needs a feed-forward and a first norm")
        self.mixer_norm = build_part(spec.mixer_norm, env)
        self.mixer = build_part(spec.mixer, env)
        self.feed_forward_norm = build_part(spec.feed_forward_norm, env)
        self.feed_forward = build_part(spec.feed_forward, env)

    def parts(self):
        return [(slot, getattr(self, slot)) for slot in self.SLOTS if getattr(self, slot) is not None]

    def cache_requirement(self):
        return self.mixer.cache_requirement()

    def first_norm(self):
        return self.mixer_norm if self.feed_forward_norm is None else None    # (two norms run as one kernel of their own)

    def forward(self, ctx, cache, residual):
        # Both branches read the same normed rows.  If the product that last added into the residual left what this
        # norm needs (sums of squares and weighted rows: a few-rows step), and both branches can take the norm over
        # into their first products, no norm kernel runs; else the norm runs once as a kernel.
        after = ctx.norm_after_block
        if self.feed_forward_norm is not None:
            self._forward_two_norms(ctx, cache, residual, after)
            return
        consumers = [part for part in (self.mixer, self.feed_forward) if part is not None]
        foldable = self.mixer_norm is not None and self.mixer_norm.foldable and \
            all(part.takes_normed_residual for part in consumers)
        if self.mixer_norm is None:
            x = ctx.cast_residual(residual)
        else:
            x = self.mixer_norm.forward(ctx, residual, lazy=True) if foldable else self.mixer_norm.forward(ctx, residual)
        # the branch that adds into the residual last may prepare the norm the next block starts with
        ctx.residual_stats = None
        ctx.upcoming_norm = after if self.feed_forward is None else None
        self.mixer.forward(ctx, cache, x, residual)
        if self.feed_forward is not None:
            ctx.residual_stats = None
            ctx.upcoming_norm = after
            self.feed_forward.forward(ctx, x, residual)
        ctx.upcoming_norm = None


    def _forward_two_norms(self, ctx, cache, residual, after):
        """Both norms read the residual as it is now, so both run before either branch adds into it."""
        from .norm import RmsNorm
        first, second = self.mixer_norm, self.feed_forward_norm
        if type(first) is RmsNorm and type(second) is RmsNorm and first.spec.eps == second.spec.eps \
                and first.spec.size == second.spec.size:
            from .. import kernels
            shape = (residual.shape[0], first.spec.size)
            x_mixer, x_feed = ctx.alloc(shape, self.env.dtype), ctx.alloc(shape, self.env.dtype)
            kernels.rms_norm_pair(residual, first.weight, second.weight, first.spec.eps, x_mixer, x_feed)
        else:
            x_mixer, x_feed = first.forward(ctx, residual), second.forward(ctx, residual)
        ctx.residual_stats = None
        ctx.upcoming_norm = None
        self.mixer.forward(ctx, cache, x_mixer, residual)
        ctx.residual_stats = None
        ctx.upcoming_norm = after
        self.feed_forward.forward(ctx, x_feed, residual)
        ctx.upcoming_norm = None


class OutputNormBlock(Block):
    """x += m * norm_1(mixer(x)), then x += m * norm_2(feed_forward(x)): the norms stand on the branches' results."""

    reads_residual_itself = True         # it starts by reading the residual in the engine dtype

    SLOTS = ("mixer_norm", "mixer", "feed_forward_norm", "feed_forward")

    def __init__(self, spec, env):
        super().__init__(spec, env)
        from .norm import RmsNorm
        self.mixer_norm = build_part(spec.mixer_norm, env)
        self.mixer = build_part(spec.mixer, env)
        self.feed_forward_norm = build_part(spec.feed_forward_norm, env)
        self.feed_forward = build_part(spec.feed_forward, env)
        for norm, branch in ((self.mixer_norm, self.mixer), (self.feed_forward_norm, self.feed_forward)):
            if branch is not None and type(norm) is not RmsNorm:
                raise ValueError("the output_norm arrangement takes an RMS norm behind every branch")
        self.scale = float(spec.residual_scale)

    def parts(self):
        return [(slot, getattr(self, slot)) for slot in self.SLOTS if getattr(self, slot) is not None]

    def cache_requirement(self):
        return self.mixer.cache_requirement()

    def forward(self, ctx, cache, residual):
        from .. import kernels
        ctx.upcoming_norm = None             # no norm reads the residual: nothing for a product to prepare
        ctx.residual_stats = None
        hand_on = ctx.next_reads_residual
        x = ctx.take_rounded(residual)
        result = ctx.alloc(tuple(residual.shape), torch.float32)
        self.mixer.forward(ctx, cache, x, result, overwrite=True)
        # the kernel that adds the normed branch also writes the new residual in the engine dtype for whoever reads it next
        rounded = ctx.rounded_buffer(residual) if self.feed_forward is not None or hand_on else None
        kernels.add_normed_branches([result], [self.mixer_norm.weight], residual, self.mixer_norm.spec.eps, self.scale,
                                    rounded=rounded)
        if self.feed_forward is not None:
            x = rounded if rounded is not None else ctx.cast_residual(residual)
            self.feed_forward.forward(ctx, x, result, overwrite=True)
            rounded = ctx.rounded_buffer(residual) if hand_on else None
            kernels.add_normed_branches([result], [self.feed_forward_norm.weight], residual,
                                        self.feed_forward_norm.spec.eps, self.scale, rounded=rounded)
        ctx.rounded_residual = rounded if hand_on else None
        ctx.residual_stats = None


class StreamMix(Part):
    """The three small tensors by which one sublayer reads and writes a residual of several streams."""

    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.read = self.write = self.mix = self.ones = None

    def parameters(self):
        from ..config.spec import ParamSpec
        s = self.spec.streams
        return {"in": ParamSpec((s,), init="ones", store="float32"),
                "out": ParamSpec((s,), init="ones", store="float32"),
                "mix": ParamSpec((s, s), init="normal", store="float32", accept_transposed=False)}

    def bind(self, tensors):
        self.read, self.write, self.mix = (tensors[name].contiguous() for name in ("in", "out", "mix"))
        self.ones = torch.ones_like(self.read)          # the factors of a reader that takes the streams' plain sum

    def weight_bytes(self):
        return sum(t.numel() * 4 for t in (self.read, self.write, self.mix))


class StreamsBlock(Block):
    """Pre-norm sublayers on a residual of several streams [tokens, S, width]: each reads a mix of the streams through
    its norm and writes its result into all of them."""

    SLOTS = ("mixer_norm", "mixer", "feed_forward_norm", "feed_forward", "mixer_streams", "feed_forward_streams")

    def __init__(self, spec, env):
        super().__init__(spec, env)
        for slot in self.SLOTS:
            setattr(self, slot, build_part(getattr(spec, slot), env))
        if self.mixer_norm is None or self.mixer_streams is None or \
                (self.feed_forward is not None and (self.feed_forward_norm is None or self.feed_forward_streams is None)):
            raise ValueError("the streams arrangement takes a norm and mixing tensors for every sublayer")
        from .norm import LayerNorm
        if any(norm is not None and type(norm) is not LayerNorm for norm in (self.mixer_norm, self.feed_forward_norm)):
            raise ValueError("the streams arrangement reads through a layer norm (the norm whose kernel mixes the streams)")

    def parts(self):
        return [(slot, getattr(self, slot)) for slot in self.SLOTS if getattr(self, slot) is not None]

    def cache_requirement(self):
        return self.mixer.cache_requirement()

    def first_reader(self):
        """(norm, mixing tensors) of the sublayer that reads the streams first."""
        return self.mixer_norm, self.mixer_streams

    def forward(self, ctx, cache, residual):
        ctx.upcoming_norm = None             # the products' results go through the streams' update, not into a norm
        ctx.residual_stats = None
        tokens, _, width = residual.shape
        result = ctx.alloc((tokens, width), torch.float32)
        x, ctx.normed_streams = ctx.normed_streams, None       # what the update before this block left, if it did
        if x is None or x.shape[0] != tokens:
            x = self.mixer_norm.forward(ctx, residual, read=self.mixer_streams.read)
        after = ctx.streams_reader_after_block
        self.mixer.forward(ctx, cache, x, result, overwrite=True)
        if self.feed_forward is not None:
            x = self._write(ctx, residual, result, self.mixer_streams, (self.feed_forward_norm, self.feed_forward_streams))
            self.feed_forward.forward(ctx, x, result, overwrite=True)
            ctx.normed_streams = self._write(ctx, residual, result, self.feed_forward_streams, after)
        else:
            ctx.normed_streams = self._write(ctx, residual, result, self.mixer_streams, after)
        ctx.residual_stats = None

    def _write(self, ctx, residual, result, streams, reader):
        """The streams take a sublayer's result; with a reader (norm, mixing tensors) the same kernel leaves the normed
        mix of the new streams that this reader starts from, which is returned; the reader "sum" gets their 32-bit sum."""
        from .. import kernels
        if reader is None:
            kernels.streams_write(residual, result, streams.mix, streams.write)
            return None
        if reader == "sum":                  # the model's last update: the streams' sum, 32-bit, on the way out
            total = ctx.alloc((residual.shape[0], residual.shape[2]), torch.float32)
            kernels.streams_write_norm(residual, result, streams.mix, streams.write, streams.ones, None, None, 0.0, total)
            return total
        norm, following = reader
        out = ctx.alloc((residual.shape[0], residual.shape[2]), self.env.dtype)
        kernels.streams_write_norm(residual, result, streams.mix, streams.write, following.read, norm.weight, norm.bias,
                                   norm.spec.eps, out)
        return out


ARRANGEMENTS = {"pre_norm": PreNormBlock, "parallel": ParallelBlock, "output_norm": OutputNormBlock,
                "streams": StreamsBlock}


def build_block(layer_spec, env):
    from ..errors import RegistryError
    cls = ARRANGEMENTS.get(layer_spec.arrangement)
    if cls is None:
        raise RegistryError(f"unknown arrangement {layer_spec.arrangement!r}; known: {', '.join(sorted(ARRANGEMENTS))}")
    return cls(layer_spec, env)
