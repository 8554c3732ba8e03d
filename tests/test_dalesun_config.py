"""Dalesun without a GPU: configuration -> model description, tensor names and shapes, what the cache manager is asked
for (borrowed keys and values share the lender's pages; the lender keeps what the widest window sees), configuration
errors; fixed points of the plain implementation itself."""

import copy
import math

import numpy as np
import pytest
import torch

import plain_dalesun as plain
from dalesun_configs import ALL, DALESUN_A, DALESUN_B, DALESUN_C, DALESUN_D, make_folder, random_config

from libmir_b200.cache import CacheManager
from libmir_b200.config.spec import FixedState, PagedKv
from libmir_b200.errors import ConfigError
from libmir_b200.models.decoder import DecoderModel
from libmir_b200.parts.base import BuildEnv
from libmir_b200.registry import architecture_of, build_spec
from libmir_b200.weights import catalog_shapes, parameter_specs

F64 = torch.float64


def test_the_class_is_chosen_by_the_configuration():
    assert architecture_of(DALESUN_A) == "Dalesun"
    assert build_spec(DALESUN_A, None).architecture == "Dalesun"


def test_description_and_tensor_names():
    spec = build_spec(DALESUN_A, None)
    assert [layer.mixer.kind for layer in spec.layers] == ["retention", "softmax_attention", "softmax_attention", "retention"]
    assert all(layer.arrangement == "output_norm" and layer.residual_scale == 0.5 for layer in spec.layers)
    assert spec.layers[2].feed_forward is None and spec.layers[2].feed_forward_norm is None
    assert spec.layers[1].feed_forward.activation == "relu2" and spec.layers[1].feed_forward.intermediate_size == 72
    retention = spec.layers[0].mixer
    assert (retention.heads, retention.key_dim, retention.value_dim, retention.decays) == (3, 24, 40, (0.9, 0.97, 0.995))
    assert retention.position.layout == "half" and retention.position.rotary_dim == 16
    attention, borrower = spec.layers[1].mixer, spec.layers[2].mixer
    assert (attention.heads, attention.kv_heads, attention.head_dim, attention.value_dim, attention.window,
            attention.scale) == (6, 2, 32, 16, 24, 0.21)
    assert attention.position.layout == "interleaved" and attention.position.theta == 500.0
    assert attention.sinks and attention.gate and attention.qk_norm and attention.qkv_bias and attention.own_kv
    assert not borrower.own_kv and borrower.window == 40
    assert [(entry.layer, entry.cache_of) for entry in spec.schedule] == [(0, None), (1, None), (2, 1), (3, None)]
    assert build_spec(DALESUN_B, None).layers[0].residual_scale == 1.0
    assert build_spec(DALESUN_B, None).layers[1].mixer.position is None
    assert build_spec(DALESUN_B, None).layers[0].mixer.window is None
    shapes = {name: tuple(param.shape) for name, param in parameter_specs(DALESUN_A).items()}
    assert shapes["embed"] == (211, 96) and shapes["embed.norm"] == (96,) and shapes["final.norm"] == (96,)
    assert shapes["head"] == (211, 96)
    assert shapes["l0.norm1"] == (96,) and shapes["l0.norm2"] == (96,) and "l2.norm2" not in shapes
    assert shapes["l0.mix.q"] == (72, 96) and shapes["l0.mix.k"] == (72, 96) and shapes["l0.mix.v"] == (120, 96)
    assert shapes["l0.mix.g"] == (120, 96) and shapes["l0.mix.o"] == (96, 120)
    assert shapes["l1.mix.q"] == (192, 96) and shapes["l1.mix.k"] == (64, 96) and shapes["l1.mix.v"] == (32, 96)
    assert shapes["l1.mix.q.b"] == (192,) and shapes["l1.mix.k.b"] == (64,) and shapes["l1.mix.v.b"] == (32,)
    assert shapes["l1.mix.q.norm"] == (32,) and shapes["l1.mix.k.norm"] == (32,) and shapes["l1.mix.sink"] == (6,)
    assert shapes["l1.mix.g"] == (96, 96) and shapes["l1.mix.o"] == (96, 96)
    assert shapes["l1.mlp.up"] == (72, 96) and shapes["l1.mlp.down"] == (96, 72)
    # a borrower has queries, gate, sink and output, and nothing of keys and values
    assert shapes["l2.mix.q"] == (192, 96) and shapes["l2.mix.q.norm"] == (32,) and shapes["l2.mix.sink"] == (6,)
    assert not any(name.startswith("l2.mix.k") or name.startswith("l2.mix.v") for name in shapes)
    assert "l2.mlp.up" not in shapes


def test_what_the_cache_manager_is_asked_for():
    model = DecoderModel(build_spec(DALESUN_A, None), BuildEnv(torch.float32, torch.device("cpu")))
    plan = model.cache_plan()
    assert [item.source for item in plan] == [0, 1, 1, 3] and [item.writes for item in plan] == [True, True, False, True]
    assert plan[0].requirement == FixedState((3, 40, 24), "float32") and plan[3].requirement == FixedState((2, 16, 16), "float32")
    # the lender keeps what the widest of the windows that read its pages sees
    assert plan[1].requirement == PagedKv(2, 32, 40, 16, 0)
    manager = CacheManager(plan, page_size=8, num_pages=10, max_requests=2)
    assert len(manager.groups) == 1 and sorted(manager.state_entries) == [0, 3]
    # a lender without a window keeps every token although its borrower has one; and the other way round
    plan = DecoderModel(build_spec(DALESUN_D, None), BuildEnv(torch.float32, torch.device("cpu"))).cache_plan()
    assert plan[1].requirement.window is None
    widened = copy.deepcopy(DALESUN_D)
    widened["layers"][1]["mixer"]["mask"] = {"size": 9}
    del widened["layers"][2]["mixer"]["mask"]
    plan = DecoderModel(build_spec(widened, None), BuildEnv(torch.float32, torch.device("cpu"))).cache_plan()
    assert plan[1].requirement.window is None


def test_random_weights_have_the_configurations_names(tmp_path):
    folder = make_folder(tmp_path, DALESUN_C, seed=1, dtype="bfloat16")
    catalog = dict(catalog_shapes(folder))
    assert set(catalog) == set(parameter_specs(DALESUN_C))
    assert catalog["l1.mix.q"] == (100, 100) and catalog["l1.mix.v"] == (60, 100) and catalog["l2.mix.sink"] == (4,)
    config, weights = plain.read_model(folder)
    logits = plain.forward(config, weights, [1, 2, 3, 4, 5])
    assert logits.shape == (5, 150) and torch.isfinite(logits).all()


def test_configurations_drawn_at_random_are_described():
    rng = np.random.default_rng(3)
    for _ in range(30):
        config = random_config(rng)
        spec = build_spec(config, None)
        assert len(spec.layers) == len(config["layers"])
        for entry, layer in zip(spec.schedule, config["layers"]):
            assert entry.cache_of == layer["mixer"].get("kv_from")


@pytest.mark.parametrize("change,text", [
    (lambda c: c["layers"][0].update(type="mamba"), "type"),
    (lambda c: c["layers"][1]["mlp"].update(kind="routed"), "kind"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_heads"), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=34), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=0), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=3), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(heads=4), "layer 1"),
    (lambda c: c["layers"][1]["mixer"].update(heads=5), "kv_heads"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_configuration_errors_name_what_is_wrong(change, text):
    config = copy.deepcopy(DALESUN_A)
    change(config)
    with pytest.raises(ConfigError) as error:
        build_spec(config, None)
    assert text in str(error.value)


def test_plain_implementation_fixed_points():
    # interleaved pairs: position 0 turns nothing; at position 1 the first pair (frequency 1) turns by one radian
    x = torch.tensor([[3.0, 4.0, 5.0]], dtype=F64)
    assert torch.equal(plain.rotate_interleaved(x, torch.tensor([0]), {"dims": 2, "base": 7.0}), x)
    turned = plain.rotate_interleaved(x, torch.tensor([1]), {"dims": 2, "base": 7.0})[0]
    assert math.isclose(float(turned[0]), 3.0 * math.cos(1.0) - 4.0 * math.sin(1.0), rel_tol=1e-12)
    assert math.isclose(float(turned[1]), 4.0 * math.cos(1.0) + 3.0 * math.sin(1.0), rel_tol=1e-12) and turned[2] == 5.0
    # half-split pairs: channel 0 goes with channel 2 (frequency 1), channel 1 with 3 (frequency 1 / 4)
    y = torch.tensor([[1.0, 2.0, 3.0, 4.0, 9.0]], dtype=F64)
    turned = plain.rotate_half(y, torch.tensor([2]), {"dims": 4, "base": 16.0})[0]
    assert math.isclose(float(turned[0]), math.cos(2.0) - 3.0 * math.sin(2.0), rel_tol=1e-12)
    assert math.isclose(float(turned[3]), 4.0 * math.cos(0.5) + 2.0 * math.sin(0.5), rel_tol=1e-12) and turned[4] == 9.0
    assert torch.allclose(plain.frequencies({"dims": 4, "base": 100.0}), torch.tensor([1.0, 0.1], dtype=F64))
    # the norms: a constant vector has root mean square |c|
    assert torch.allclose(plain.unit_rms(torch.full((1, 4), -3.0, dtype=F64), 0.0), torch.full((1, 4), -1.0, dtype=F64))
    assert torch.allclose(plain.norm_one_plus(torch.full((1, 4), 2.0, dtype=F64), torch.full((4,), 0.5, dtype=F64), 0.0),
                          torch.full((1, 4), 1.5, dtype=F64))
    assert torch.equal(plain.relu_squared(torch.tensor([-2.0, 3.0], dtype=F64)), torch.tensor([0.0, 9.0], dtype=F64))
    # attention: one token, one head: the sink takes its share although it has no value
    eye = torch.eye(2, dtype=F64)
    zero = torch.zeros(2, dtype=F64)
    w = {"p.q": eye, "p.k": eye, "p.v": eye, "p.g": eye * 50.0, "p.o": eye, "p.q.b": zero, "p.k.b": zero, "p.v.b": zero,
         "p.q.norm": torch.ones(2, dtype=F64), "p.k.norm": torch.ones(2, dtype=F64), "p.sink": torch.tensor([0.3], dtype=F64)}
    mixer = {"heads": 1, "kv_heads": 1, "dim": 2, "scale": 0.5}
    h = torch.tensor([[1.0, 3.0]], dtype=F64)
    keys, values = plain.attention_keys_values(h, w, "p.", mixer, 0.0)
    out = plain.attention(h, w, "p.", mixer, 0.0, keys, values)[0]
    score = 0.5 * 2.0                                             # unit-rms q . k = dim; times scale
    share = math.exp(score) / (math.exp(score) + math.exp(0.3))
    assert torch.allclose(out, share * h[0])                      # (the gate's sigmoid(50 h) is 1)
    # a window of one: every token sees itself alone
    h3 = torch.tensor([[1.0, 3.0], [2.0, -1.0], [0.5, 0.25]], dtype=F64)
    mixer1 = dict(mixer, mask={"size": 1})
    keys, values = plain.attention_keys_values(h3, w, "p.", mixer1, 0.0)
    w_open = dict(w, **{"p.g": eye * 0.0})
    out = plain.attention(h3, w_open, "p.", mixer1, 0.0, keys, values)
    assert torch.allclose(out, 0.5 * share * h3)                  # sigmoid(0) = 1/2
    # retention: two tokens of one head, no rotation
    wr = {"r.q": eye, "r.k": eye, "r.v": eye, "r.g": eye, "r.o": eye}
    hr = torch.tensor([[1.0, 0.0], [1.0, 1.0]], dtype=F64)
    out, state = plain.retention(hr, wr, "r.", {"heads": 1, "dim": 2, "decay": [0.5]}, 0.0)
    s1 = torch.outer(hr[0], hr[0]) * 2 ** -0.5
    s2 = 0.5 * s1 + torch.outer(hr[1], hr[1]) * 2 ** -0.5
    assert torch.allclose(state[0], s2)
    o2 = s2.T @ hr[1]
    assert torch.allclose(out[1], o2 / torch.sqrt((o2 * o2).mean()) * plain.silu(hr[1]))
    # a state carried over a cut gives what the whole sequence gives
    first, carried = plain.retention(hr[:1], wr, "r.", {"heads": 1, "dim": 2, "decay": [0.5]}, 0.0)
    second, _ = plain.retention(hr[1:], wr, "r.", {"heads": 1, "dim": 2, "decay": [0.5]}, 0.0, carried, 1)
    assert torch.allclose(torch.cat([first, second]), out)
