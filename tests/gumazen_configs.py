"""Tiny Gumazen configurations for the tests, and model folders with weights that make every mechanism matter.
The configurations differ from one another in every size, in the kinds and order of layers, in the loop, the number of
streams, windows, rotations, caps, bias tables and router constants; some take values that make two sizes equal or 1,
some leave optional keys out, two have heads that the tensor-core attention kernels take (64 and 128 channels)."""

from __future__ import annotations

from pathlib import Path

import torch


def _rot(dims, base, scaling=None):
    rot = {"dims": dims, "base": base}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return rot


def sink_attention(heads, kv_heads, dim, vdim, scale, rot=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        mixer["rot"] = _rot(*rot)
    return {"type": "attention", "mixer": mixer}


def biased_attention(heads, kv_heads, dim, vdim, scale, window, softcap, bias_rows, bias_max):
    return {"type": "attention_2", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
                                             "mask": {"size": window}, "softcap": softcap, "bias_max": bias_max,
                                             "bias_rows": bias_rows}}


def scaled_attention(heads, kv_heads, dim, vdim, scale, rot=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        mixer["rot"] = _rot(*rot)
    return {"type": "attention_3", "mixer": mixer}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def experts(count, top, ff, identity=0, groups=None, scale=1.0, shared=0):
    router = {"experts": count, "top": top, "scale": scale}
    if identity:
        router["identity"] = identity
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared:
        mlp["shared"] = {"ff": shared}
    return mlp


def _layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


GUMAZEN_A = {   # three streams, a loop in the middle, value heads narrower and wider than key heads, identity experts
    "architecture": "Gumazen", "vocab": 211, "width": 96, "norm": {"eps": 1e-6}, "streams": 3,
    "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        _layer(scaled_attention(4, 2, 32, 16, 0.21, rot=(16, 10000.0, (4.0, 1.0, 4.0, 64))), dense(72)),
        _layer(sink_attention(6, 2, 24, 24, 0.3, rot=(8, 300.0)), experts(6, 3, 24, identity=2, groups=(4, 2), scale=1.7, shared=40)),
        _layer(biased_attention(4, 1, 16, 32, 0.25, window=20, softcap=5.0, bias_rows=12, bias_max=40), experts(5, 2, 32, identity=1, groups=(3, 2), scale=0.8)),
        _layer(scaled_attention(3, 3, 20, 12, 0.2), None),
    ],
}

GUMAZEN_B = {   # sizes that are equal or 1: one stream, one head, a window of one token, one expert of one, no loop
    "architecture": "Gumazen", "vocab": 130, "width": 64, "norm": {"eps": 1e-5}, "streams": 1,
    "layers": [
        _layer(biased_attention(1, 1, 16, 16, 0.25, window=1, softcap=2.0, bias_rows=4, bias_max=9), experts(1, 1, 64)),
        _layer(sink_attention(1, 1, 16, 16, 0.5, rot=(16, 100.0)), dense(64)),
        _layer(scaled_attention(2, 2, 8, 8, 0.4, rot=(8, 50.0)), experts(3, 3, 16, identity=3, groups=(6, 6), shared=16)),
        _layer(biased_attention(2, 1, 8, 8, 1.0, window=3, softcap=50.0, bias_rows=2, bias_max=5), None),
    ],
}

GUMAZEN_C = {   # heads of 64 channels (tensor cores in bfloat16); a single residual (no `streams`); the loop at the end
    "architecture": "Gumazen", "vocab": 150, "width": 104, "norm": {"eps": 1e-5},
    "loop": {"start": 1, "stop": 3, "times": 2},
    "layers": [
        _layer(sink_attention(4, 1, 64, 64, 0.11, rot=(24, 250000.0)), dense(52)),
        _layer(biased_attention(4, 2, 64, 64, 0.14, window=50, softcap=12.0, bias_rows=16, bias_max=70), experts(8, 2, 24, identity=4, groups=(3, 2), scale=2.0, shared=24)),
        _layer(scaled_attention(2, 1, 64, 64, 0.125, rot=(64, 5000.0, (8.0, 1.0, 4.0, 96))), dense(40)),
    ],
}

GUMAZEN_D = {   # heads of 128 channels; two streams; the whole model repeated
    "architecture": "Gumazen", "vocab": 97, "width": 128, "norm": {"eps": 1e-6}, "streams": 2,
    "loop": {"start": 0, "stop": 3, "times": 2},
    "layers": [
        _layer(scaled_attention(2, 1, 128, 128, 0.09, rot=(32, 10000.0, (2.0, 1.0, 2.0, 32))), experts(4, 2, 48, identity=4, groups=(2, 1), scale=1.2)),
        _layer(sink_attention(4, 2, 128, 128, 0.07, rot=(128, 500000.0)), dense(96)),
        _layer(biased_attention(2, 2, 128, 128, 0.08, window=70, softcap=20.0, bias_rows=10, bias_max=64), None),
    ],
}

ALL = {"A": GUMAZEN_A, "B": GUMAZEN_B, "C": GUMAZEN_C, "D": GUMAZEN_D}
PAGE_SIZES = {"A": 8, "B": 16, "C": 4, "D": 16}


def make_folder(tmp_path, config: dict, seed: int, dtype: str, sharpen: float = 2.0, edit=None) -> Path:
    """config.json + model.safetensors.  The random weights of the package's writer are rescaled so that norm weights
    and biases, the streams' mixing tensors, gates, the bias by distance, the router and its correction and the
    attention scores are far from their neutral values: a missed or extra key at a window's edge, a sink left out, a
    wrong bucket, a dropped stream or expert then changes the logits well beyond the tolerances.  `sharpen` multiplies
    the scores (through the q and k norm weights, or the projections where the norm has none); `edit(tensors)` may
    change the table of tensors before it is written."""
    from libmir_b200.weights import load_tensor, read_catalog, write_file, write_model_folder
    folder = write_model_folder(Path(tmp_path), config, seed=seed, dtype=dtype)
    tensors = {name: load_tensor(entry) for name, entry in read_catalog(folder).items()}
    generator = torch.Generator().manual_seed(seed + 1000)
    normal = lambda shape, deviation: torch.randn(shape, generator=generator) * deviation
    streams = config.get("streams") or 1
    for name, tensor in list(tensors.items()):
        kind = tensor.dtype
        parts = name.split(".")
        last = parts[-1]
        if last in ("norm1", "norm2") or name == "final.norm" or name.endswith("q.norm") or name.endswith("k.norm"):
            new = 1.0 + normal(tensor.shape, 0.25)
            if name.endswith("q.norm") or name.endswith("k.norm"):
                new = new * sharpen ** 0.5
        elif last == "b":
            new = normal(tensor.shape, 0.5)
        elif len(parts) == 3 and parts[1] in ("hc1", "hc2"):
            if last == "in":
                new = 1.0 / streams + normal(tensor.shape, 0.3)
            elif last == "out":
                new = 1.0 + normal(tensor.shape, 0.3)
            else:
                new = torch.eye(streams) + normal(tensor.shape, 0.3)
        elif last == "rel":
            new = normal(tensor.shape, 1.5)
        elif last == "correction":
            new = normal(tensor.shape, 0.08)
        elif last == "router":
            new = tensor.float() * 10.0
        elif name == "embed":
            new = tensor.float() * 10.0
        elif ".mix." in name and last == "g":
            new = tensor.float() * 10.0
        elif ".mix." in name and last in ("q", "k", "v"):
            new = tensor.float() * 5.0
        elif last == "up":
            new = tensor.float() * 5.0
        else:
            continue
        tensors[name] = new.to(kind)
    if edit is not None:
        edit(tensors)
    write_file(folder / "model.safetensors", tensors)
    return folder


def random_config(rng) -> dict:
    """A configuration drawn at random: any layer order, head counts and widths that are no multiples of 8 (or of 4),
    with and without rotation, scaling, streams, loop, identity experts, groups and shared expert."""
    def rotation(dim, scaled):
        if rng.random() < 0.2:
            return None
        dims = int(rng.choice([d for d in (2, 4, 6, 8, 16, 32, 64, 128) if d <= dim]))
        scaling = (float(rng.choice([2.0, 8.0])), 1.0, float(rng.choice([2.0, 4.0])), int(rng.choice([16, 64, 256]))) \
            if scaled and rng.random() < 0.7 else None
        return (dims, float(rng.choice([50.0, 10000.0, 500000.0])), scaling)

    def mixer():
        dim = int(rng.choice([4, 12, 16, 20, 24, 40, 64, 96, 128]))
        kv_heads = int(rng.integers(1, 4))
        heads = kv_heads * int(rng.integers(1, 5))
        vdim = dim if rng.random() < 0.5 else int(rng.choice([4, 6, 8, 12, 24, 40, 96]))
        scale = float(rng.uniform(0.05, 0.4))
        kind = rng.integers(0, 3)
        if kind == 0:
            return sink_attention(heads, kv_heads, dim, vdim, scale, rotation(dim, False))
        if kind == 1:
            rows = int(rng.choice([2, 5, 8, 12, 32]))
            return biased_attention(heads, kv_heads, dim, vdim, scale, int(rng.integers(1, 90)),
                                    float(rng.choice([2.0, 10.0, 30.0])), rows, float(rows // 2 + rng.integers(1, 100)))
        return scaled_attention(heads, kv_heads, dim, vdim, scale, rotation(dim, True))

    def feed_forward():
        draw = rng.random()
        if draw < 0.2:
            return None
        if draw < 0.5:
            return dense(int(rng.choice([40, 64, 100, 130])))
        count, identity = int(rng.integers(1, 9)), int(rng.integers(0, 4))
        total = count + identity
        group_count = int(rng.choice([g for g in range(1, total + 1) if total % g == 0]))
        keep = int(rng.integers(1, group_count + 1))
        top = int(rng.integers(1, keep * (total // group_count) + 1))
        return experts(count, top, int(rng.choice([8, 20, 24, 48])), identity, (group_count, keep),
                       float(rng.uniform(0.5, 3.0)), int(rng.choice([0, 16, 36])))

    layers = [_layer(mixer(), feed_forward()) for _ in range(int(rng.integers(1, 5)))]
    config = {"architecture": "Gumazen", "vocab": int(rng.integers(30, 300)),
              "width": int(rng.choice([48, 52, 64, 72, 100, 136, 50])),
              "norm": {"eps": float(rng.choice([1e-5, 1e-6, 1e-4]))}, "layers": layers}
    if rng.random() < 0.75:
        config["streams"] = int(rng.integers(1, 6))
    if rng.random() < 0.6:
        start = int(rng.integers(0, len(layers)))
        config["loop"] = {"start": start, "stop": int(rng.integers(start, len(layers) + 1)), "times": int(rng.integers(1, 4))}
    return config
