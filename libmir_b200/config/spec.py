"""The description a model is built from: data only, no tensors and no kernels.

An architecture's builder (libmir_b200/models) turns its config.json into a ModelSpec:
a list of LayerSpec, each naming the kind and the numbers of its mixer, feed-forward,
norms and position encoding, and a schedule, the order in which the layers run.
Parts are looked up by `kind` in the part registry, so a layer may use any registered
mixer or feed-forward, and different layers may use different ones.

The seams follow libmir's semantic model: MixerSpec / FeedForwardSpec /
PositionEncodingSpec / NormalizationKind (models/src/semantic/attention.rs:5-9,111-124,
feed_forward.rs:5-30, model.rs:110-115).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Union

from ..errors import ConfigError


# --------------------------------------------------------------------------- parameters
@dataclass(frozen=True)
class TensorSource:
    """Another way a checkpoint may store a wanted tensor: as rows [rows[0], rows[1]) of the stored tensor
    `name` (a name local to the part, like the key of the ParamSpec that lists this source), which has
    `total_rows` rows in all.  libmir splits a fused `self_attn.qkv_proj.weight` / `query_key_value.weight`
    into query, key and value rows this way (models/src/weights/binding/shapes/transforms.rs:22-35)."""

    name: str
    rows: tuple
    total_rows: int


@dataclass(frozen=True)
class ParamSpec:
    """One tensor that a part wants from the checkpoint.

    `store` says how it is kept on the device: "compute" follows the engine's dtype
    (bfloat16 or float32), "float32" is kept in 32-bit whatever the engine's dtype
    (norm weights and biases: small, and exact for every stored dtype), "int32" is an
    integer table.  `init` is what the random-weights writer fills it with.
    """

    shape: tuple
    init: str = "normal"          # "normal" N(0, 0.02), "ones", "zeros"
    store: str = "compute"        # "compute" | "float32" | "int32"
    optional: bool = False        # absent from the checkpoint is fine (bias, q/k-norm discovery)
    sources: tuple = ()           # TensorSource: other stored tensors this one may be cut from
    # A 2-d tensor stored with its two dimensions swapped ([in, out] for [out, in]) is recognised by its shape
    # and transposed while loading (transforms.rs:52-58); a square tensor is always taken as stored.
    accept_transposed: bool = True


# --------------------------------------------------------------------------- cache needs
@dataclass(frozen=True)
class PagedKv:
    """Keys and values of every token in pages; with a window only the last `window` are kept.  Keys are
    `head_dim` wide; values too unless `value_head_dim` says otherwise (libmir's KvStorageSpec has both widths,
    cuda/src/backend/kv/storage/mod.rs:17-25)."""

    kv_heads: int
    head_dim: int
    window: Optional[int] = None
    value_head_dim: Optional[int] = None     # 0: one vector per token and kv head only (a latent read as key and as value)
    keep_first: int = 0           # with a window: the request's first tokens whose pages are never given back

    @property
    def value_dim(self) -> int:
        return self.head_dim if self.value_head_dim is None else self.value_head_dim

    @property
    def elements_per_token(self) -> int:
        """Cached elements per token and schedule entry: keys and values of every kv head."""
        return self.kv_heads * (self.head_dim + self.value_dim)


@dataclass(frozen=True)
class FixedState:
    """State of fixed size per request, kept in the request's state slot."""

    shape: tuple
    dtype: str = "float32"


@dataclass(frozen=True)
class CacheBundle:
    """What a mixer made of several mechanisms asks for one schedule entry: at most one set of pages and any number
    of fixed-size states, in the order its parts will find them in CacheView.states."""

    paged: Optional[PagedKv] = None
    states: tuple = ()


CacheRequirement = Union[PagedKv, FixedState, CacheBundle, None]


def split_requirement(requirement) -> tuple:
    """(PagedKv or None, tuple of FixedState) of any cache requirement."""
    if requirement is None:
        return None, ()
    if isinstance(requirement, PagedKv):
        return requirement, ()
    if isinstance(requirement, FixedState):
        return None, (requirement,)
    if isinstance(requirement, CacheBundle):
        return requirement.paged, tuple(requirement.states)
    raise ConfigError(f"unknown cache requirement {requirement!r}")


def bundle_requirements(requirements) -> CacheRequirement:
    """One requirement for several parts that share a schedule entry (None if none of them asks for anything)."""
    paged, states = None, []
    for requirement in requirements:
        pages, fixed = split_requirement(requirement)
        if pages is not None:
            if paged is not None:
                raise ConfigError("one schedule entry holds at most one set of cache pages")
            paged = pages
        states.extend(fixed)
    if paged is None and not states:
        return None
    if paged is not None and not states:
        return paged
    if paged is None and len(states) == 1:
        return states[0]
    return CacheBundle(paged, tuple(states))


# --------------------------------------------------------------------------- parts
@dataclass(frozen=True)
class PartSpec:
    """Base of every part description; `kind` selects the implementation in the registry."""

    kind: str = field(init=False, default="")


@dataclass(frozen=True)
class RmsNormSpec(PartSpec):
    """y = x / sqrt(mean(x^2) + eps) * (offset + w).  `offset` 1 is the form whose weight is stored around zero;
    `tensor` is the local name of the weight ("" where the checkpoint names the norm itself)."""

    size: int = 0
    eps: float = 1e-5
    offset: float = 0.0
    tensor: str = "weight"
    kind: str = field(init=False, default="rms_norm")


@dataclass(frozen=True)
class LayerNormSpec(PartSpec):
    """y = (x - mean) / sqrt(variance + eps) * w + b, the variance being the mean of the squared deviations.  `tensor`
    and `bias_tensor` are the local names of weight and bias ("" where the checkpoint names the norm itself)."""

    size: int = 0
    eps: float = 1e-5
    tensor: str = "weight"
    bias_tensor: str = "bias"
    kind: str = field(init=False, default="layer_norm")


@dataclass(frozen=True)
class StreamMixSpec(PartSpec):
    """How one sublayer reads and writes a residual kept as `streams` copies (hyper-connections): three stored 32-bit
    tensors, `in` [S] (the sublayer's input is sum_s in[s] x_s), `mix` [S, S] indexed [from, to] and `out` [S]
    (x_t <- sum_s mix[s, t] x_s + out[t] * the sublayer's result, all streams at once from the old ones)."""

    streams: int = 0
    kind: str = field(init=False, default="stream_mix")


@dataclass(frozen=True)
class DistanceBiasSpec:
    """A learned bias on attention scores by the distance n = query position - key position: the stored table has
    `rows` buckets (one column per query head); bucket(n) = n below rows // 2, and from there on
    min(rows - 1, rows // 2 + floor(ln(n / (rows // 2)) / ln(farthest / (rows // 2)) * (rows - rows // 2)))."""

    rows: int
    farthest: float


@dataclass(frozen=True)
class YarnScaling:
    """Frequencies stretched by `factor` where a pair turns fewer than `slow` times over `original` positions, kept
    where it turns more than `fast` times, blended linearly (by pair index) in between; cos and sin are multiplied by
    0.1 ln(factor) + 1."""

    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class RotarySpec(PartSpec):
    """Rotary position encoding of the first `rotary_dim` dims of a head.  `layout` "half": dims i and i + r/2 form a
    pair; "interleaved": dims 2i and 2i + 1.  `scaling`: config.RopeScaling (the llama3 rule), YarnScaling or None."""

    head_dim: int = 0
    rotary_dim: int = 0
    theta: float = 10000.0
    scaling: Any = None
    layout: str = "half"
    kind: str = field(init=False, default="rotary")


@dataclass(frozen=True)
class SoftmaxAttentionSpec(PartSpec):
    hidden_size: int = 0
    heads: int = 0
    kv_heads: int = 0
    head_dim: int = 0
    scale: float = 1.0
    qk_norm: bool = False
    qk_norm_eps: float = 1e-6
    qkv_bias: bool = False
    out_bias: bool = False
    window: Optional[int] = None
    position: Optional[PartSpec] = None
    value_head_dim: Optional[int] = None     # width of a value head where it differs from head_dim
    keep_first: int = 0                      # with a window: the first tokens every later query still sees
    names: tuple = ()                        # (local name, stored name) pairs for checkpoints with names of their own
    # sinks: the softmax's denominator also holds exp(s_h) of one stored number per query head (tensor `sink`), which
    # has no key and no value and is not scaled.  gate: the concatenated heads are multiplied by the sigmoid of a
    # projection (tensor `g`) of the mixer's input before the output projection.  own_kv False: the mixer has no key
    # and value tensors; it attends with its own queries over the cache of the schedule entry that its entry names
    # (ScheduleEntry.cache_of), whose head counts, widths and rotation must equal its own.
    sinks: bool = False
    gate: bool = False
    own_kv: bool = True
    # fixed_sink: every head's sink is this constant of the design instead of a stored number (0: one is added to the
    # softmax's denominator).  gate_per_head: the gate's projection has one row per query head, whose sigmoid
    # multiplies the whole head.  qk_norm_span: "head" norms every head by itself with one weight [head_dim] for all
    # heads; "projection" norms q as a whole and k as a whole over all their heads, with weights of that width.
    # qk_norm_weight False: the norm has no weights.  qk_norm_after_rotation: the per-head norm follows the rotation.
    # softcap: score <- softcap * tanh(score / softcap) after the scale.  distance_bias: a stored table (tensor
    # `rel_bias` [rows, heads]) added to the scores after the cap, by the bucket of the distance; `scale` does not
    # multiply it.
    fixed_sink: Optional[float] = None
    gate_per_head: bool = False
    qk_norm_span: str = "head"
    qk_norm_weight: bool = True
    qk_norm_after_rotation: bool = False
    softcap: Optional[float] = None
    distance_bias: Optional[DistanceBiasSpec] = None
    kind: str = field(init=False, default="softmax_attention")

    @property
    def value_dim(self) -> int:
        return self.head_dim if self.value_head_dim is None else self.value_head_dim


@dataclass(frozen=True)
class SwiGluSpec(PartSpec):
    hidden_size: int = 0
    intermediate_size: int = 0
    kind: str = field(init=False, default="swiglu")


@dataclass(frozen=True)
class GeluMlpSpec(PartSpec):
    """down(act(up(x))): a dense feed-forward without a gate.  `activation`: "gelu_tanh" (the tanh form), "gelu_erf"
    (the exact form) or "relu2" (the square of relu)."""

    hidden_size: int = 0
    intermediate_size: int = 0
    activation: str = "gelu_tanh"
    kind: str = field(init=False, default="gelu_mlp")


@dataclass(frozen=True)
class LatentAttentionSpec(PartSpec):
    """Softmax attention whose keys and values are up-projections of one cached latent per token, beside one rotated
    key part shared by all heads (parts/latent_attention.py).  Per head `head_dim` unrotated and `rotary_dim` rotated
    query / key dims and `value_dim` value dims; `q_rank` and `kv_rank` are the widths of the two latents.
    `gate`: the concatenated heads are multiplied by the sigmoid of a projection of the mixer's input."""

    hidden_size: int = 0
    heads: int = 0
    head_dim: int = 0
    rotary_dim: int = 0
    value_dim: int = 0
    q_rank: int = 0
    kv_rank: int = 0
    scale: float = 1.0
    norm_eps: float = 1e-5
    gate: bool = True
    position: Optional[PartSpec] = None
    kind: str = field(init=False, default="latent_attention")


@dataclass(frozen=True)
class WkvSpec(PartSpec):
    """Time mixing with a matrix state per head, a decay per head and key channel from a low-rank pair with tanh
    between (rank `decay_rank`), a bonus for the current token, and inputs blended with the token before
    (parts/wkv.py)."""

    hidden_size: int = 0
    heads: int = 0
    head_dim: int = 0
    decay_rank: int = 0
    norm_eps: float = 1e-5
    kind: str = field(init=False, default="wkv")


@dataclass(frozen=True)
class RoutedExpertsSpec(PartSpec):
    """A mixture of gated experts (down(silu(gate x) * up x)), `top` of `experts` per token (parts/experts.py).
    Router: 32-bit logits, `score` "sigmoid" or "softmax" (over all the router's outputs); with `correction` a stored
    bias is added to the scores for the choice only; experts lie in `groups` equal groups of neighbours of which the
    `keep_groups` best (`group_score` "top2": by the sum of a group's two largest choice scores, "max": by its largest)
    may be chosen from; the chosen scores are divided by their sum and multiplied by `scale`.  `identity` > 0: the
    router has that many more outputs behind the experts', identity experts without tensors whose result is the
    feed-forward's input itself; they take part in scores, groups and choice like the others (`experts` counts only
    the experts with weights).  `shared_size` > 0: an expert of that width runs for every token, times the sigmoid of
    one number per token if `shared_gate`."""

    hidden_size: int = 0
    expert_size: int = 0
    experts: int = 0
    top: int = 0
    groups: int = 1
    keep_groups: int = 1
    scale: float = 1.0
    correction: bool = True
    shared_size: int = 0
    shared_gate: bool = True
    score: str = "sigmoid"
    group_score: str = "top2"
    identity: int = 0
    kind: str = field(init=False, default="routed_experts")


@dataclass(frozen=True)
class RetentionSpec(PartSpec):
    """Linear attention with one fixed decay per head and no softmax (parts/retention.py): per head a matrix state
    S <- decay_h S + k v^T, read out as S^T q, with k scaled by key_dim^-1/2 after the rotation; the read-out of each
    head is divided by its root mean square and multiplied by silu of a projection of the mixer's input.  `decays`
    holds one number per head."""

    hidden_size: int = 0
    heads: int = 0
    key_dim: int = 0
    value_dim: int = 0
    decays: tuple = ()
    norm_eps: float = 1e-5
    position: Optional[PartSpec] = None
    kind: str = field(init=False, default="retention")


@dataclass(frozen=True)
class GatedDeltaRuleSpec(PartSpec):
    """The gated delta rule (parts/delta_rule.py).  `decay`: "head" one decay per head from a full projection `a`,
    "channel" one per head and key channel from a low-rank pair `a1`, `a2` of rank `decay_rank`.  `gate`: "silu" of
    a full projection `g`, or "sigmoid" of a low-rank pair `g1`, `g2` of rank `gate_rank`."""

    hidden_size: int = 0
    heads: int = 0
    kv_heads: int = 0
    key_dim: int = 0
    value_dim: int = 0
    conv_taps: int = 4
    decay: str = "head"
    decay_rank: int = 0
    gate: str = "silu"
    gate_rank: int = 0
    norm_eps: float = 1e-5
    kind: str = field(init=False, default="gated_delta_rule")


@dataclass(frozen=True)
class SideBySideSpec(PartSpec):
    """Several mixers that read the same input; the result is `scale` times the sum of their outputs, each first
    RMS-normed over the model width with a plain weight `<branch name>.<out_tensor>`."""

    hidden_size: int = 0
    branches: tuple = ()                     # (name, PartSpec) pairs; a branch's tensors lie under "<name>."
    eps: float = 1e-5
    scale: float = 0.5
    out_tensor: str = "out"
    kind: str = field(init=False, default="side_by_side")


@dataclass(frozen=True)
class TokenPairsSpec:
    """A second embedding table added to the first, indexed by a hash of a token and the one before it:
    row (previous * mul_previous + token * mul_current) mod buckets; a request's first token takes row `buckets`."""

    name: str
    buckets: int
    mul_previous: int
    mul_current: int


# --------------------------------------------------------------------------- layers and model
@dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement of a mixer and a feed-forward with their norms.

    `prefix` is the checkpoint prefix of the layer; `names` maps each slot of the
    arrangement to the sub-prefix of its tensors, so names are data of the architecture.
    Arrangements: "pre_norm" (a norm before each of the two branches, one after the other), "parallel" (both
    branches read the same residual and their results are added to it together: through one norm, `mixer_norm`, if
    `feed_forward_norm` is None, else each through a norm of its own), "output_norm" (each branch reads the
    residual itself and its RESULT goes through the norm: x += residual_scale * norm(branch(x)), one after the other)
    and "streams" (the residual is ModelSpec.streams copies; each branch reads a mix of them through its norm and
    writes into all of them as `mixer_streams` / `feed_forward_streams`, StreamMixSpec, say).
    """

    prefix: str
    mixer: PartSpec
    feed_forward: Optional[PartSpec]
    mixer_norm: Optional[PartSpec]
    feed_forward_norm: Optional[PartSpec]
    names: Mapping[str, str]
    arrangement: str = "pre_norm"
    residual_scale: float = 1.0           # what a branch's (normed) result is multiplied by ("output_norm" only)
    mixer_streams: Optional[PartSpec] = None          # ("streams" only) how the mixer reads and writes the streams
    feed_forward_streams: Optional[PartSpec] = None   # the same for the feed-forward


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  `layer` indexes ModelSpec.layers and may repeat.

    Every entry has a cache of its own unless `cache_of` names an earlier entry (by its
    index in the schedule) whose cache it reads without writing to it.
    """

    layer: int
    cache_of: Optional[int] = None
    opens_pass: Optional[int] = None      # the number of the pass of ModelSpec.loop that starts with this entry


@dataclass(frozen=True)
class LoopSpec:
    """A run of layers that is repeated with the same weights (every repeat is a schedule entry of its own, so it has
    a cache or state of its own).  Before each pass the row `pass` of the tensor `step_tensor` [passes, hidden] is
    added to the residual, and before each pass but the first, ahead of that, the embedding's output."""

    passes: int
    step_tensor: Optional[str] = None
    add_embedding: bool = True


@dataclass(frozen=True)
class EmbeddingSpec:
    name: str
    vocab_size: int
    hidden_size: int
    multiplier: float = 1.0
    pairs: Optional[TokenPairsSpec] = None
    norm: Optional[PartSpec] = None       # a norm applied to the embedded rows before the first layer,
    norm_name: str = ""                   # stored under this name


@dataclass(frozen=True)
class HeadSpec:
    """Output projection; `tied_to` names the embedding tensor it shares, else `name` is its own.  `scale`
    multiplies the logits."""

    name: str
    vocab_size: int
    hidden_size: int
    tied: bool = False
    scale: float = 1.0
    softcap: Optional[float] = None       # logits <- softcap * tanh(logits / softcap)


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: EmbeddingSpec
    layers: tuple
    schedule: tuple
    final_norm: PartSpec
    final_norm_name: str
    head: HeadSpec
    strip_prefixes: tuple = ()      # checkpoint prefixes that may wrap every name
    loop: Optional[LoopSpec] = None
    # streams > 0: the residual is that many copies per token, all equal to the embedding's output at the start and
    # summed before the final norm; every layer then has the "streams" arrangement
    streams: int = 0

    def validate(self) -> None:
        if not self.layers:
            raise ConfigError("a model needs at least one layer")
        for index, layer in enumerate(self.layers):
            if (layer.arrangement == "streams") != (self.streams > 0):
                raise ConfigError(f"layer {index}: the \"streams\" arrangement and a residual of several streams "
                                  "(ModelSpec.streams) go together")
        for index, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise ConfigError(f"schedule entry {index} names layer {entry.layer}, the model has {len(self.layers)}")
            if entry.cache_of is not None:
                if not 0 <= entry.cache_of < index:
                    raise ConfigError(f"schedule entry {index} reads the cache of entry {entry.cache_of}, "
                                      "which must be an earlier entry")
                if self.schedule[entry.cache_of].cache_of is not None:
                    raise ConfigError(f"schedule entry {index} reads the cache of entry {entry.cache_of}, "
                                      "which has no cache of its own")
            if entry.opens_pass is not None and (self.loop is None or not 0 <= entry.opens_pass < self.loop.passes):
                raise ConfigError(f"schedule entry {index} opens pass {entry.opens_pass} of a loop the model does not have")
