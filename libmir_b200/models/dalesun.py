"""Dalesun: a decoder whose sublayers read the residual itself and whose norms stand on the sublayers' OUTPUT,
x += m * norm(mixer(x)), then x += m * norm(feed_forward(x)), with softmax-attention and retention mixers:
config.json -> ModelSpec.

config.json:
    architecture  "Dalesun"
    vocab, width, norm.eps, residual_mult (m)
    layers[i]     {type, mixer, mlp}; tensors of layer i start with "l<i>."
        type "attention"  mixer {heads, kv_heads, dim, vdim, scale, rot {dims, base}, mask {size}, kv_from}: grouped
                          softmax attention with q/k/v biases, a per-head RMS norm of q and k (one weight for all
                          heads), interleaved rotation of the first rot.dims dims, a sliding window, one sink per query
                          head in the softmax's denominator, and a sigmoid gate on the concatenated heads; with
                          `kv_from: j` the layer has no key / value tensors and attends over layer j's cache
        type "retention"  mixer {heads, dim, vdim, decay [one per head], rot {dims, base}}: a matrix state per head
                          with a fixed decay, half-split rotation of q and k, per-head unit norm, silu gate
        mlp       {kind "dense", ff} (up, squared relu, down) or null
Norm weights are stored around zero (the norm multiplies by 1 + w); the q/k norms have plain weights.  The embedded
rows go through a norm of the same kind (`embed.norm`) before the first layer.
Tensor names: embed, embed.norm, l<i>.norm1, l<i>.norm2, l<i>.mix.*, l<i>.mlp.{up,down}, final.norm, head.
"""

from __future__ import annotations

from typing import Mapping, Optional

from ..config.spec import (EmbeddingSpec, GeluMlpSpec, HeadSpec, LayerSpec, ModelSpec, RetentionSpec, RmsNormSpec,
                           RotarySpec, ScheduleEntry, SoftmaxAttentionSpec)
from ..errors import ConfigError
from ..registry import register_architecture

LAYER_NAMES = {"mixer_norm": "norm1", "feed_forward_norm": "norm2", "mixer": "mix.", "feed_forward": "mlp."}
ATTENTION_NAMES = (("q_proj.weight", "q"), ("k_proj.weight", "k"), ("v_proj.weight", "v"), ("o_proj.weight", "o"),
                   ("q_proj.bias", "q.b"), ("k_proj.bias", "k.b"), ("v_proj.bias", "v.b"),
                   ("q_norm.weight", "q.norm"), ("k_norm.weight", "k.norm"), ("g_proj.weight", "g"), ("sinks", "sink"))


def _need(table, key: str, where: str):
    if not isinstance(table, Mapping) or key not in table:
        raise ConfigError(f"Dalesun config: {where} needs `{key}`")
    return table[key]


def _rotation(mixer: Mapping, dim: int, layout: str, where: str) -> Optional[RotarySpec]:
    rot = mixer.get("rot")
    if not rot:
        return None
    dims = int(_need(rot, "dims", where + ".rot"))
    if dims == 0:
        return None
    if dims % 2 or not 0 < dims <= dim:
        raise ConfigError(f"Dalesun config: {where}.rot.dims {dims} must be even and at most dim {dim}")
    return RotarySpec(head_dim=dim, rotary_dim=dims, theta=float(_need(rot, "base", where + ".rot")), layout=layout)


def _attention(mixer: Mapping, width: int, eps: float, where: str) -> SoftmaxAttentionSpec:
    heads, kv_heads, dim = (int(_need(mixer, key, where)) for key in ("heads", "kv_heads", "dim"))
    if heads % kv_heads:
        raise ConfigError(f"Dalesun config: {where}: heads must be a multiple of kv_heads")
    mask = mixer.get("mask") or {}
    return SoftmaxAttentionSpec(
        hidden_size=width, heads=heads, kv_heads=kv_heads, head_dim=dim, scale=float(_need(mixer, "scale", where)),
        qk_norm=True, qk_norm_eps=eps, qkv_bias=True, window=int(mask["size"]) if mask.get("size") else None,
        position=_rotation(mixer, dim, "interleaved", where), value_head_dim=int(mixer.get("vdim", dim)),
        names=ATTENTION_NAMES, sinks=True, gate=True, own_kv=mixer.get("kv_from") is None)


def _retention(mixer: Mapping, width: int, eps: float, where: str) -> RetentionSpec:
    heads, dim = int(_need(mixer, "heads", where)), int(_need(mixer, "dim", where))
    decays = tuple(float(d) for d in _need(mixer, "decay", where))
    if len(decays) != heads:
        raise ConfigError(f"Dalesun config: {where}.decay lists {len(decays)} numbers for {heads} heads")
    return RetentionSpec(hidden_size=width, heads=heads, key_dim=dim, value_dim=int(mixer.get("vdim", dim)),
                         decays=decays, norm_eps=eps, position=_rotation(mixer, dim, "half", where))


def build(config: Mapping, catalog: Optional[Mapping[str, tuple]] = None) -> ModelSpec:
    width, vocab = int(_need(config, "width", "the model")), int(_need(config, "vocab", "the model"))
    eps = float(_need(_need(config, "norm", "the model"), "eps", "norm"))
    scale = float(config.get("residual_mult", 1.0))
    norm = RmsNormSpec(size=width, eps=eps, offset=1.0, tensor="")
    layers, schedule = [], []
    for index, layer in enumerate(_need(config, "layers", "the model")):
        where = f"layers[{index}]"
        kind, mixer = _need(layer, "type", where), _need(layer, "mixer", where)
        source = None
        if kind == "attention":
            mixer_spec = _attention(mixer, width, eps, where)
            if mixer.get("kv_from") is not None:
                source = int(mixer["kv_from"])
                lender = layers[source].mixer if 0 <= source < index else None
                if not isinstance(lender, SoftmaxAttentionSpec) or not lender.own_kv:
                    raise ConfigError(f"Dalesun config: {where}.kv_from {source} must name an earlier attention layer "
                                      "with keys and values of its own")
                same = ("heads", "kv_heads", "head_dim", "value_dim", "position")
                if any(getattr(lender, key) != getattr(mixer_spec, key) for key in same):
                    raise ConfigError(f"Dalesun config: {where} reads the keys and values of layer {source}, whose "
                                      "head counts, sizes and rotation must equal its own")
        elif kind == "retention":
            mixer_spec = _retention(mixer, width, eps, where)
        else:
            raise ConfigError(f"Dalesun config: {where} has type {kind!r}; known: attention, retention")
        mlp = layer.get("mlp")
        feed_forward = None
        if mlp is not None:
            if mlp.get("kind") != "dense":
                raise ConfigError(f"Dalesun config: {where}.mlp has kind {mlp.get('kind')!r}; known: dense")
            feed_forward = GeluMlpSpec(hidden_size=width, intermediate_size=int(_need(mlp, "ff", where + ".mlp")),
                                       activation="relu2")
        layers.append(LayerSpec(prefix=f"l{index}.", mixer=mixer_spec, feed_forward=feed_forward, mixer_norm=norm,
                                feed_forward_norm=norm if feed_forward is not None else None, names=LAYER_NAMES,
                                arrangement="output_norm", residual_scale=scale))
        schedule.append(ScheduleEntry(layer=index, cache_of=source))
    return ModelSpec(
        architecture="Dalesun", hidden_size=width, vocab_size=vocab,
        max_positions=int(config.get("max_positions", 1 << 30)),
        embedding=EmbeddingSpec("embed", vocab, width, 1.0, norm=norm, norm_name="embed.norm"),
        layers=tuple(layers), schedule=tuple(schedule),
        final_norm=norm, final_norm_name="final.norm", head=HeadSpec("head", vocab, width, tied=False),
    )


register_architecture("Dalesun", build)
