"""Tiny Dalesun configurations for the tests, and model folders with weights that make every mechanism matter.
The configurations differ from one another in every size, in the order and kinds of layers, in windows, rotations,
decays and the residual's multiplier; some take values that make two sizes equal or 1, some leave optional keys out,
two have heads that the tensor-core attention kernels take (64 and 128 channels)."""

from __future__ import annotations

from pathlib import Path

import torch


def _rot(dims, base):
    return {"dims": dims, "base": base}


def _attention(heads, kv_heads, dim, vdim, scale, window=None, rot=None, kv_from=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        mixer["mask"] = {"size": window}
    if rot is not None:
        mixer["rot"] = _rot(*rot)
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "attention", "mixer": mixer}


def _retention(dim, vdim, decays, rot=None):
    mixer = {"heads": len(decays), "dim": dim, "vdim": vdim, "decay": list(decays)}
    if rot is not None:
        mixer["rot"] = _rot(*rot)
    return {"type": "retention", "mixer": mixer}


def _layer(mixer, ff):
    return dict(mixer, mlp={"kind": "dense", "ff": ff} if ff else None)


DALESUN_A = {   # value heads of another width than key heads; a borrower whose window is wider than its lender's
    "architecture": "Dalesun", "vocab": 211, "width": 96, "norm": {"eps": 1e-6}, "residual_mult": 0.5,
    "layers": [
        _layer(_retention(24, 40, (0.9, 0.97, 0.995), rot=(16, 10000.0)), 160),
        _layer(_attention(6, 2, 32, 16, 0.21, window=24, rot=(16, 500.0)), 72),
        _layer(_attention(6, 2, 32, 16, 0.3, window=40, rot=(16, 500.0), kv_from=1), None),
        _layer(_retention(16, 16, (0.8, 0.99), rot=(16, 100.0)), 40),
    ],
}

DALESUN_B = {   # sizes that are equal or 1: one head, a window of one token and none at all, no rotation, no multiplier
    "architecture": "Dalesun", "vocab": 130, "width": 64, "norm": {"eps": 1e-5},
    "layers": [
        _layer(_attention(1, 1, 16, 16, 0.25, rot=(16, 100.0)), 64),
        _layer(_retention(64, 64, (0.9375,)), 64),
        _layer(_attention(2, 2, 8, 8, 0.4, window=1), None),
        _layer(_attention(1, 1, 16, 16, 0.5, window=3, rot=(16, 100.0), kv_from=0), 32),
    ],
}

DALESUN_C = {   # heads of 64 channels (tensor cores in bfloat16), widths that are no multiples of 8 in retention
    "architecture": "Dalesun", "vocab": 150, "width": 100, "norm": {"eps": 1e-5}, "residual_mult": 1.3,
    "layers": [
        _layer(_attention(4, 1, 64, 64, 0.11, window=50, rot=(24, 250000.0)), 52),
        _layer(_retention(20, 12, (0.5, 0.9, 0.99, 0.999, 1.0), rot=(6, 1000.0)), None),
        _layer(_attention(4, 1, 64, 64, 0.16, window=17, rot=(24, 250000.0), kv_from=0), 36),
        _layer(_attention(3, 3, 64, 64, 0.125, rot=(64, 50.0)), 44),
    ],
}

DALESUN_D = {   # heads of 128 channels; a borrower with a narrower window behind a lender without one
    "architecture": "Dalesun", "vocab": 97, "width": 128, "norm": {"eps": 1e-6}, "residual_mult": 0.25,
    "layers": [
        _layer(_retention(128, 64, (0.99, 0.9), rot=(128, 500000.0)), 200),
        _layer(_attention(4, 2, 128, 128, 0.09, rot=(32, 10000.0)), None),
        _layer(_attention(4, 2, 128, 128, 0.07, window=70, rot=(32, 10000.0), kv_from=1), 48),
    ],
}

ALL = {"A": DALESUN_A, "B": DALESUN_B, "C": DALESUN_C, "D": DALESUN_D}
PAGE_SIZES = {"A": 8, "B": 16, "C": 4, "D": 16}


def make_folder(tmp_path, config: dict, seed: int, dtype: str, sharpen: float = 2.0) -> Path:
    """config.json + model.safetensors.  The random weights of the package's writer are rescaled so that norm
    weights, sinks, gates, biases and attention scores are far from their neutral values: a lost state, a missed or
    extra key at a window's edge, a sink left out, a gate or a bias dropped then changes the logits well beyond the
    tolerances.  `sharpen` multiplies the scores (through the q and k norm weights)."""
    from libmir_b200.weights import load_tensor, read_catalog, write_file, write_model_folder
    folder = write_model_folder(Path(tmp_path), config, seed=seed, dtype=dtype)
    tensors = {name: load_tensor(entry) for name, entry in read_catalog(folder).items()}
    generator = torch.Generator().manual_seed(seed + 1000)
    normal = lambda shape, deviation: torch.randn(shape, generator=generator) * deviation
    for name, tensor in list(tensors.items()):
        kind = tensor.dtype
        last = name.split(".")[-1]
        if last in ("norm1", "norm2") or name in ("final.norm", "embed.norm"):
            new = normal(tensor.shape, 0.25)                      # stored around zero
        elif name.endswith("q.norm") or name.endswith("k.norm"):
            new = (1.0 + normal(tensor.shape, 0.25)) * sharpen ** 0.5
        elif last == "sink":
            new = 1.0 + normal(tensor.shape, 1.0)
        elif last == "b":
            new = normal(tensor.shape, 0.5)
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
    write_file(folder / "model.safetensors", tensors)
    return folder


def random_config(rng) -> dict:
    """A configuration drawn at random: any layer order, head counts and widths that are no multiples of 8 (or of 4),
    with and without rotation, window, multiplier and feed-forward; borrowers of an earlier layer's keys."""
    def rotation(dim):
        if rng.random() < 0.2:
            return None
        dims = int(rng.choice([d for d in (2, 4, 6, 8, 16, 32, 64, 128) if d <= dim]))
        return (dims, float(rng.choice([50.0, 10000.0, 500000.0])))

    def attention(lenders):
        if lenders and rng.random() < 0.4:
            source = int(rng.choice(sorted(lenders)))
            lent = lenders[source]["mixer"]
            rot = (lent["rot"]["dims"], lent["rot"]["base"]) if "rot" in lent else None
            window = int(rng.integers(1, 90)) if rng.random() < 0.7 else None
            return _attention(lent["heads"], lent["kv_heads"], lent["dim"], lent["vdim"], float(rng.uniform(0.05, 0.4)),
                              window, rot, kv_from=source)
        dim = int(rng.choice([4, 12, 16, 20, 24, 40, 64, 96, 128]))
        kv_heads = int(rng.integers(1, 4))
        heads = kv_heads * int(rng.integers(1, 5))
        vdim = dim if rng.random() < 0.5 else int(rng.choice([4, 6, 8, 12, 24, 40, 96]))
        window = int(rng.integers(1, 90)) if rng.random() < 0.7 else None
        return _attention(heads, kv_heads, dim, vdim, float(rng.uniform(0.05, 0.4)), window, rotation(dim))

    def retention():
        dim = int(rng.choice([4, 12, 20, 32, 36, 64, 100, 128]))
        heads = int(rng.integers(1, 6))
        decays = [float(1.0 - 2.0 ** -rng.uniform(1.0, 11.0)) for _ in range(heads)]
        return _retention(dim, int(rng.choice([4, 6, 12, 20, 32, 64])), decays, rotation(dim))

    layers, lenders = [], {}
    for index in range(int(rng.integers(1, 6))):
        if rng.random() < 0.55:
            mixer = attention(lenders)
            if "kv_from" not in mixer["mixer"]:
                lenders[index] = mixer
        else:
            mixer = retention()
        layers.append(_layer(mixer, int(rng.choice([0, 40, 64, 100, 130]))))
    config = {"architecture": "Dalesun", "vocab": int(rng.integers(30, 300)),
              "width": int(rng.choice([48, 52, 64, 72, 100, 136, 50])),
              "norm": {"eps": float(rng.choice([1e-5, 1e-6, 1e-4]))}, "layers": layers}
    if rng.random() < 0.8:
        config["residual_mult"] = float(rng.uniform(0.2, 1.5))
    return config
