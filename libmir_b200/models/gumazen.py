"""Gumazen: a pre-norm decoder with layer norms, a residual kept as several streams (hyper-connections), three kinds of
softmax attention, dense and routed feed-forwards with identity experts, and a run of layers that repeats:
config.json -> ModelSpec.

config.json:
    architecture  "Gumazen"
    vocab, width, norm.eps
    streams       how many copies of the residual there are (absent: one plain residual, no stream tensors)
    loop          {start, stop, times}: layers start .. stop - 1 run `times` times in a row with the same weights, every
                  pass with a cache of its own; nothing else happens between passes
    layers[i]     {type, mixer, mlp}; tensors of layer i start with "l<i>."
        type "attention"    {heads, kv_heads, dim, vdim, scale, rot {dims, base}}: rotation of q and k (half-split
                            pairs of the first rot.dims channels), then every head divided by its root mean square
                            (no weights); causal; one is added to the softmax's denominator
        type "attention_2"  {heads, kv_heads, dim, vdim, scale, softcap, bias_max, mask {size}}: an RMS norm of q and
                            of k over all heads at once (weights q.norm, k.norm); no rotation; scores capped by
                            softcap * tanh(score / softcap), then a stored bias by the bucket of the distance (rel
                            [buckets, heads]); a sliding window; one sigmoid gate per head from a projection (g) of the
                            mixer's input
        type "attention_3"  {heads, kv_heads, dim, vdim, scale, rot {dims, base, scaling {factor, low, high,
                            original}}}: biases on q, k, v and the output projection; the norm over all heads at once,
                            then the rotation with frequencies remapped by wavelength; causal
        mlp       {kind "dense", ff}: down(relu(up x)^2);  {kind "moe", expert {ff}, router {experts, top, scale,
                  identity, groups {count, keep}}, shared {ff}}: gated experts chosen by softmax scores plus a stored
                  correction within the best groups (a group judged by its largest choice score), the last
                  router.identity router outputs being identity experts, and a shared expert;  or null
Every norm is a layer norm with weight and bias (eps = norm.eps).
Tensor names: embed, l<i>.norm1(.b), l<i>.norm2(.b), l<i>.hc1.{in,out,mix}, l<i>.hc2.{in,out,mix}, l<i>.mix.*,
l<i>.mlp.*, final.norm(.b), head.
"""

from __future__ import annotations

from typing import Mapping, Optional

from ..config.decoder import RopeScaling
from ..config.spec import (DistanceBiasSpec, EmbeddingSpec, GeluMlpSpec, HeadSpec, LayerNormSpec, LayerSpec, ModelSpec,
                           RotarySpec, RoutedExpertsSpec, ScheduleEntry, SoftmaxAttentionSpec, StreamMixSpec)
from ..errors import ConfigError
from ..registry import register_architecture

LAYER_NAMES = {"mixer_norm": "norm1", "feed_forward_norm": "norm2", "mixer": "mix.", "feed_forward": "mlp.",
               "mixer_streams": "hc1.", "feed_forward_streams": "hc2."}
ATTENTION_NAMES = (("q_proj.weight", "q"), ("k_proj.weight", "k"), ("v_proj.weight", "v"), ("o_proj.weight", "o"),
                   ("q_proj.bias", "q.b"), ("k_proj.bias", "k.b"), ("v_proj.bias", "v.b"), ("o_proj.bias", "o.b"),
                   ("q_norm.weight", "q.norm"), ("k_norm.weight", "k.norm"), ("g_proj.weight", "g"), ("rel_bias", "rel"))


def _need(table, key: str, where: str):
    if not isinstance(table, Mapping) or key not in table:
        raise ConfigError(f"Gumazen config: {where} needs `{key}`")
    return table[key]


def _rotation(mixer: Mapping, dim: int, where: str) -> Optional[RotarySpec]:
    rot = mixer.get("rot")
    if not rot:
        return None
    dims = int(_need(rot, "dims", where + ".rot"))
    if dims == 0:
        return None
    if dims % 2 or not 0 < dims <= dim:
        raise ConfigError(f"Gumazen config: {where}.rot.dims {dims} must be even and at most dim {dim}")
    scaling = None
    if rot.get("scaling"):
        table = rot["scaling"]
        factor, low, high, original = (float(_need(table, key, where + ".rot.scaling"))
                                       for key in ("factor", "low", "high", "original"))
        scaling = RopeScaling(factor=factor, low_freq_factor=low, high_freq_factor=high,
                              original_max_position_embeddings=original)
    return RotarySpec(head_dim=dim, rotary_dim=dims, theta=float(_need(rot, "base", where + ".rot")), scaling=scaling,
                      layout="half")


def _attention(kind: str, mixer: Mapping, width: int, eps: float, where: str, catalog, prefix: str) -> SoftmaxAttentionSpec:
    heads, kv_heads, dim = (int(_need(mixer, key, where)) for key in ("heads", "kv_heads", "dim"))
    if kv_heads <= 0 or heads % kv_heads:
        raise ConfigError(f"Gumazen config: {where}: heads must be a multiple of kv_heads")
    common = dict(hidden_size=width, heads=heads, kv_heads=kv_heads, head_dim=dim, value_head_dim=int(mixer.get("vdim", dim)),
                  scale=float(_need(mixer, "scale", where)), qk_norm=True, qk_norm_eps=eps, names=ATTENTION_NAMES)
    if kind == "attention":
        return SoftmaxAttentionSpec(**common, position=_rotation(mixer, dim, where), qk_norm_span="head",
                                    qk_norm_weight=False, qk_norm_after_rotation=True, fixed_sink=0.0)
    if kind == "attention_2":
        name = prefix + "rel"
        rows = int(catalog[name][0]) if catalog is not None and name in catalog else int(mixer.get("bias_rows", 32))
        farthest = float(_need(mixer, "bias_max", where))
        if rows < 2 or farthest <= rows // 2:
            raise ConfigError(f"Gumazen config: {where}: a bias table of {rows} rows needs bias_max above {rows // 2}")
        return SoftmaxAttentionSpec(**common, position=None, qk_norm_span="projection",
                                    window=int(_need(_need(mixer, "mask", where), "size", where + ".mask")),
                                    softcap=float(_need(mixer, "softcap", where)),
                                    distance_bias=DistanceBiasSpec(rows=rows, farthest=farthest), gate=True,
                                    gate_per_head=True)
    return SoftmaxAttentionSpec(**common, position=_rotation(mixer, dim, where), qk_norm_span="projection", qkv_bias=True,
                                out_bias=True)


def _feed_forward(mlp: Mapping, width: int, where: str):
    kind = mlp.get("kind")
    if kind == "dense":
        return GeluMlpSpec(hidden_size=width, intermediate_size=int(_need(mlp, "ff", where)), activation="relu2")
    if kind == "moe":
        router = _need(mlp, "router", where)
        groups = router.get("groups") or {}
        shared = mlp.get("shared") or {}
        count = int(groups.get("count", 1))
        return RoutedExpertsSpec(
            hidden_size=width, expert_size=int(_need(_need(mlp, "expert", where), "ff", where + ".expert")),
            experts=int(_need(router, "experts", where + ".router")), top=int(_need(router, "top", where + ".router")),
            groups=count, keep_groups=int(groups.get("keep", count)), scale=float(router.get("scale", 1.0)),
            correction=True, shared_size=int(shared.get("ff", 0)), shared_gate=False, score="softmax", group_score="max",
            identity=int(router.get("identity", 0)))
    raise ConfigError(f"Gumazen config: {where} has kind {kind!r}; known: dense, moe")


def build(config: Mapping, catalog: Optional[Mapping[str, tuple]] = None) -> ModelSpec:
    width, vocab = int(_need(config, "width", "the model")), int(_need(config, "vocab", "the model"))
    eps = float(_need(_need(config, "norm", "the model"), "eps", "norm"))
    streams = int(config.get("streams") or 0)
    norm = LayerNormSpec(size=width, eps=eps, tensor="", bias_tensor=".b")
    mix = StreamMixSpec(streams=streams) if streams else None
    layers = []
    for index, layer in enumerate(_need(config, "layers", "the model")):
        where = f"layers[{index}]"
        prefix = f"l{index}."
        kind, mixer = _need(layer, "type", where), _need(layer, "mixer", where)
        if kind not in ("attention", "attention_2", "attention_3"):
            raise ConfigError(f"Gumazen config: {where} has type {kind!r}; known: attention, attention_2, attention_3")
        mixer_spec = _attention(kind, mixer, width, eps, where, catalog, prefix + "mix.")
        mlp = layer.get("mlp")
        feed_forward = _feed_forward(mlp, width, where + ".mlp") if mlp is not None else None
        layers.append(LayerSpec(prefix=prefix, mixer=mixer_spec, feed_forward=feed_forward, mixer_norm=norm,
                                feed_forward_norm=norm if feed_forward is not None else None, names=LAYER_NAMES,
                                arrangement="streams" if streams else "pre_norm", mixer_streams=mix,
                                feed_forward_streams=mix if feed_forward is not None else None))
    count = len(layers)
    loop = config.get("loop")
    if loop:
        start, stop, times = (int(_need(loop, key, "loop")) for key in ("start", "stop", "times"))
        if not 0 <= start <= stop <= count or times < 1:
            raise ConfigError(f"Gumazen config: loop {start}..{stop} x {times} does not fit {count} layers")
        order = list(range(start)) + list(range(start, stop)) * times + list(range(stop, count))
    else:
        order = list(range(count))
    return ModelSpec(
        architecture="Gumazen", hidden_size=width, vocab_size=vocab,
        max_positions=int(config.get("max_positions", 1 << 30)),
        embedding=EmbeddingSpec("embed", vocab, width, 1.0),
        layers=tuple(layers), schedule=tuple(ScheduleEntry(layer=i) for i in order),
        final_norm=norm, final_norm_name="final.norm", head=HeadSpec("head", vocab, width, tied=False), streams=streams,
    )


register_architecture("Gumazen", build)
