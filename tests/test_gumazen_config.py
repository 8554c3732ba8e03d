"""Gumazen without a GPU: configuration -> model description, tensor names and shapes, the schedule of a repeated run
of layers, what the cache manager is asked for, configuration errors; the spread of the bias table by distance; fixed
points of the plain implementation itself."""

import copy
import math

import pytest
import torch

import plain_gumazen as plain
from gumazen_configs import ALL, GUMAZEN_A, GUMAZEN_B, GUMAZEN_C, GUMAZEN_D, make_folder

from libmir_b200.config.spec import DistanceBiasSpec, SoftmaxAttentionSpec
from libmir_b200.errors import ConfigError
from libmir_b200.parts import BuildEnv, SoftmaxAttention
from libmir_b200.registry import architecture_of, build_spec
from libmir_b200.weights import parameter_specs

F64 = torch.float64


def test_the_class_is_chosen_by_the_configuration():
    assert architecture_of(GUMAZEN_A) == "Gumazen"
    assert build_spec(GUMAZEN_A, None).architecture == "Gumazen"


def test_description_of_the_three_kinds_of_attention():
    spec = build_spec(GUMAZEN_A, None)
    assert spec.streams == 3 and all(layer.arrangement == "streams" for layer in spec.layers)
    assert all(layer.mixer_norm.kind == "layer_norm" and layer.mixer_norm.eps == 1e-6 for layer in spec.layers)
    scaled, sink, biased, bare = (layer.mixer for layer in spec.layers)
    assert (scaled.heads, scaled.kv_heads, scaled.head_dim, scaled.value_dim, scaled.scale) == (4, 2, 32, 16, 0.21)
    assert scaled.qkv_bias and scaled.out_bias and scaled.qk_norm_span == "projection" and scaled.qk_norm_weight
    assert not scaled.qk_norm_after_rotation and scaled.fixed_sink is None and scaled.window is None
    assert scaled.position.layout == "half" and scaled.position.rotary_dim == 16 and scaled.position.scaling.factor == 4.0
    assert sink.fixed_sink == 0.0 and sink.qk_norm_span == "head" and not sink.qk_norm_weight
    assert sink.qk_norm_after_rotation and not sink.qkv_bias and sink.position.rotary_dim == 8
    assert sink.position.theta == 300.0 and sink.position.scaling is None
    assert biased.position is None and biased.window == 20 and biased.softcap == 5.0 and biased.gate and biased.gate_per_head
    assert (biased.distance_bias.rows, biased.distance_bias.farthest) == (12, 40.0)
    assert biased.qk_norm_span == "projection" and not biased.qkv_bias
    assert bare.position is None and bare.qkv_bias                       # the third kind without a rotation
    assert spec.layers[3].feed_forward is None and spec.layers[3].feed_forward_norm is None
    assert spec.layers[3].feed_forward_streams is None


def test_description_of_the_feed_forwards():
    spec = build_spec(GUMAZEN_A, None)
    dense, routed = spec.layers[0].feed_forward, spec.layers[1].feed_forward
    assert dense.activation == "relu2" and dense.intermediate_size == 72
    assert (routed.experts, routed.identity, routed.top, routed.groups, routed.keep_groups) == (6, 2, 3, 4, 2)
    assert routed.score == "softmax" and routed.group_score == "max" and routed.correction and not routed.shared_gate
    assert routed.scale == 1.7 and routed.shared_size == 40 and routed.expert_size == 24
    lone = build_spec(GUMAZEN_B, None).layers[0].feed_forward       # keys that may be left out
    assert (lone.experts, lone.identity, lone.top, lone.groups, lone.keep_groups, lone.scale, lone.shared_size) == \
        (1, 0, 1, 1, 1, 1.0, 0)


def test_a_repeated_run_of_layers_is_a_schedule_with_an_entry_per_run():
    assert [entry.layer for entry in build_spec(GUMAZEN_A, None).schedule] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert [entry.layer for entry in build_spec(GUMAZEN_B, None).schedule] == [0, 1, 2, 3]
    assert [entry.layer for entry in build_spec(GUMAZEN_C, None).schedule] == [0, 1, 2, 1, 2]
    assert [entry.layer for entry in build_spec(GUMAZEN_D, None).schedule] == [0, 1, 2, 0, 1, 2]
    once = dict(GUMAZEN_A, loop={"start": 2, "stop": 2, "times": 3})         # an empty run
    assert [entry.layer for entry in build_spec(once, None).schedule] == [0, 1, 2, 3]


def test_a_single_residual_when_the_configuration_names_no_streams():
    spec = build_spec(GUMAZEN_C, None)
    assert spec.streams == 0 and all(layer.arrangement == "pre_norm" and layer.mixer_streams is None for layer in spec.layers)
    names = parameter_specs(GUMAZEN_C)
    assert not any(".hc1." in name or ".hc2." in name for name in names)


def test_tensor_names_and_shapes():
    shapes = {name: tuple(param.shape) for name, param in parameter_specs(GUMAZEN_A).items()}
    assert shapes["embed"] == (211, 96) and shapes["head"] == (211, 96)
    assert shapes["final.norm"] == (96,) and shapes["final.norm.b"] == (96,)
    assert shapes["l0.norm1"] == (96,) and shapes["l0.norm1.b"] == (96,) and shapes["l0.norm2.b"] == (96,)
    assert "l3.norm2" not in shapes and "l3.hc2.in" not in shapes
    for part in ("hc1", "hc2"):
        assert shapes[f"l0.{part}.in"] == (3,) and shapes[f"l0.{part}.out"] == (3,) and shapes[f"l0.{part}.mix"] == (3, 3)
    assert shapes["l0.mix.q"] == (128, 96) and shapes["l0.mix.k"] == (64, 96) and shapes["l0.mix.v"] == (32, 96)
    assert shapes["l0.mix.q.b"] == (128,) and shapes["l0.mix.k.b"] == (64,) and shapes["l0.mix.v.b"] == (32,)
    assert shapes["l0.mix.q.norm"] == (128,) and shapes["l0.mix.k.norm"] == (64,)
    assert shapes["l0.mix.o"] == (96, 64) and shapes["l0.mix.o.b"] == (96,)
    assert shapes["l1.mix.q"] == (144, 96) and "l1.mix.q.norm" not in shapes and "l1.mix.q.b" not in shapes
    assert shapes["l2.mix.q.norm"] == (64,) and shapes["l2.mix.k.norm"] == (16,)
    assert shapes["l2.mix.g"] == (4, 96) and shapes["l2.mix.rel"] == (12, 4) and shapes["l2.mix.o"] == (96, 128)
    assert shapes["l0.mlp.up"] == (72, 96) and shapes["l0.mlp.down"] == (96, 72)
    assert shapes["l1.mlp.router"] == (8, 96) and shapes["l1.mlp.correction"] == (8,)       # experts and identity experts
    assert shapes["l1.mlp.e5.gate"] == (24, 96) and shapes["l1.mlp.e5.down"] == (96, 24) and "l1.mlp.e6.gate" not in shapes
    assert shapes["l1.mlp.shared.up"] == (40, 96) and "l2.mlp.shared.up" not in shapes


def test_the_bias_tables_rows_come_from_the_stored_tensor():
    catalog = {"l2.mix.rel": (20, 4)}
    assert build_spec(GUMAZEN_A, catalog).layers[2].mixer.distance_bias.rows == 20


@pytest.mark.parametrize("change,needle", [
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c["layers"][0].update(type="attention_9"), "attention_9"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=34), "rot.dims"),
    (lambda c: c["layers"][2]["mixer"].pop("mask"), "mask"),
    (lambda c: c["layers"][2]["mixer"].update(bias_max=5), "bias_max"),
    (lambda c: c["layers"][1]["mlp"].update(kind="other"), "other"),
    (lambda c: c["layers"][1]["mlp"]["router"].pop("top"), "top"),
    (lambda c: c["loop"].update(stop=9), "loop"),
])
def test_configuration_errors_name_what_is_wrong(change, needle):
    config = copy.deepcopy(GUMAZEN_A)
    change(config)
    with pytest.raises(ConfigError) as error:
        build_spec(config, None)
    assert needle in str(error.value)


def test_the_bias_table_is_spread_to_one_entry_per_distance():
    """What the attention part hands to the kernels: [heads, distances], ending where the last bucket or the window's
    end is reached; constants whose buckets fall on exact powers too."""
    for rows, farthest, window in ((24, 150.0, 80), (12, 40.0, 20), (2, 5.0, 3), (8, 64.0, None), (5, 3.0, 200), (16, 70.0, 1)):
        spec = SoftmaxAttentionSpec(hidden_size=16, heads=3, kv_heads=1, head_dim=8, window=window,
                                    distance_bias=DistanceBiasSpec(rows=rows, farthest=farthest))
        part = SoftmaxAttention(spec, BuildEnv(torch.float32, torch.device("cpu")))
        table = torch.arange(rows * 3, dtype=torch.float32).view(rows, 3)
        got = part.bias_by_distance(table)
        assert got.shape[0] == 3 and got.is_contiguous()
        for n in range(got.shape[1]):
            assert torch.equal(got[:, n], table[plain.distance_bucket(n, rows, farthest)])
        last = got.shape[1] - 1
        assert (window is not None and last == window - 1) or plain.distance_bucket(last, rows, farthest) == rows - 1


def test_buckets_are_exact_below_half_the_table_and_logarithmic_above():
    rows, farthest = 16, 128.0
    assert [plain.distance_bucket(n, rows, farthest) for n in range(8)] == list(range(8))
    assert plain.distance_bucket(8, rows, farthest) == 8
    assert plain.distance_bucket(127, rows, farthest) == 15 and plain.distance_bucket(10 ** 6, rows, farthest) == 15
    buckets = [plain.distance_bucket(n, rows, farthest) for n in range(200)]
    assert buckets == sorted(buckets) and set(buckets) == set(range(16))
    # the k-th logarithmic bucket begins where n / 8 reaches (128 / 8) ^ (k / 8)
    for k in range(1, 8):
        edge = 8 * 16.0 ** (k / 8)
        assert plain.distance_bucket(math.ceil(edge + 1e-9), rows, farthest) == 8 + k
        assert plain.distance_bucket(math.floor(edge - 1e-9), rows, farthest) == 8 + k - 1


def test_fixed_points_of_the_plain_implementation():
    x = torch.randn(5, 12, dtype=F64)
    ones, zeros = torch.ones(12, dtype=F64), torch.zeros(12, dtype=F64)
    normed = plain.layer_norm(x, ones, zeros, 0.0)
    assert torch.allclose(normed.mean(-1), torch.zeros(5, dtype=F64), atol=1e-12)
    assert torch.allclose((normed ** 2).mean(-1), torch.ones(5, dtype=F64), atol=1e-12)
    assert torch.allclose((plain.unit_rms(x, 0.0) ** 2).mean(-1), torch.ones(5, dtype=F64), atol=1e-12)
    # one key, no sink: the value itself; with the sink of zero and a score of zero: half of it
    q, k, v = torch.zeros(1, 2, 4, dtype=F64), torch.randn(1, 1, 4, dtype=F64), torch.randn(1, 1, 6, dtype=F64)
    assert torch.allclose(plain.attend(q, k, v, 1.0)[0, 0], v[0, 0])
    assert torch.allclose(plain.attend(q, k, v, 1.0, sink=True)[0, 1], 0.5 * v[0, 0])
    # a cap far above the scores changes nothing; a window of one sees the token itself
    q, k, v = (torch.randn(9, 2, 4, dtype=F64) for _ in range(3))
    assert torch.allclose(plain.attend(q, k, v, 0.3, softcap=1e9), plain.attend(q, k, v, 0.3), atol=1e-9)
    assert torch.allclose(plain.attend(q, k, v, 0.3, window=1), v)


def test_model_folders_hold_what_the_description_asks_for(tmp_path):
    from libmir_b200.weights import read_catalog
    for name, config in ALL.items():
        folder = make_folder(tmp_path / name, config, seed=1, dtype="bfloat16")
        stored = {key: tuple(entry.shape) for key, entry in read_catalog(folder).items()}
        wanted = {key: tuple(param.shape) for key, param in parameter_specs(config).items()}
        assert stored == wanted
        config_read, weights = plain.read_model(folder)
        logits = plain.forward(config_read, weights, [1, 2, 3, 4, 5])
        assert tuple(logits.shape) == (5, config["vocab"]) and bool(torch.isfinite(logits).all())
