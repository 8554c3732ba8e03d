"""A plain, slow implementation of the Dalesun design in float64: whole sequences, no cache, no batching, one
function per mechanism.  It shares no code with the package and is what the engine is compared with.

Notation: n tokens, width w.  Weights are stored [out, in]; a token's row vector x is multiplied as x @ W.T.

The design: x = norm(embed[token]); every layer adds its two sublayers through a norm on the sublayer's OUTPUT,
x <- x + m * norm(mixer(x)), x <- x + m * norm(ff(x)), with the sublayers reading x itself; mixers are softmax
attention (biases, per-head q/k norm, interleaved partial rotation, sliding window, a sink in the softmax's
denominator, a sigmoid output gate, optionally the keys and values of an earlier layer) and retention (a matrix state
per head with a fixed decay, rotate-half rotation, per-head unit norm, a silu gate); the feed-forward is
down(relu(up x)^2).
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import numpy as np
import torch

F64 = torch.float64


# ------------------------------------------------------------------------------ reading a model folder
def read_model(folder):
    """(config, {name: float64 tensor}) of a folder with config.json and model.safetensors."""
    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    raw = (folder / "model.safetensors").read_bytes()
    size = int.from_bytes(raw[:8], "little")
    header = json.loads(raw[8:8 + size])
    body = raw[8 + size:]
    weights = {}
    for name, entry in header.items():
        if name == "__metadata__":
            continue
        begin, end = entry["data_offsets"]
        data = body[begin:end]
        if entry["dtype"] == "BF16":
            bits = np.frombuffer(data, dtype=np.uint16).astype(np.uint32) << 16
            values = torch.from_numpy(bits.view(np.float32).copy())
        elif entry["dtype"] == "F32":
            values = torch.from_numpy(np.frombuffer(data, dtype=np.float32).copy())
        elif entry["dtype"] == "I32":
            values = torch.from_numpy(np.frombuffer(data, dtype=np.int32).copy())
        else:
            raise ValueError(f"{name}: dtype {entry['dtype']}")
        weights[name] = values.reshape(entry["shape"]).to(F64)
    return config, weights


# ------------------------------------------------------------------------------ small pieces
def unit_rms(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_one_plus(x, weight, eps):
    """The model's norm: the weight is stored around zero."""
    return unit_rms(x, eps) * (1.0 + weight)


def silu(z):
    return z / (1.0 + torch.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def relu_squared(z):
    return torch.clamp(z, min=0.0) ** 2


# ------------------------------------------------------------------------------ rotation
def frequencies(rot):
    dims, base = int(rot["dims"]), float(rot["base"])
    return torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)


def _cos_sin(x, positions, rot):
    # the design computes the angle as a 32-bit product of the position and a 32-bit frequency
    angles = (positions.to(torch.float32)[:, None] * frequencies(rot).to(torch.float32)[None, :]).to(F64)
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [angles.shape[1]]
    return torch.cos(angles).reshape(shape), torch.sin(angles).reshape(shape)


def rotate_interleaved(x, positions, rot):
    """x [n, ..., d]: dims 2i and 2i + 1 of the first rot.dims form a pair."""
    dims = int(rot["dims"])
    cos, sin = _cos_sin(x, positions, rot)
    out = x.clone()
    first, second = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = first * cos - second * sin
    out[..., 1:dims:2] = second * cos + first * sin
    return out


def rotate_half(x, positions, rot):
    """x [n, ..., d]: dims i and i + rot.dims / 2 of the first rot.dims form a pair."""
    dims = int(rot["dims"])
    half = dims // 2
    cos, sin = _cos_sin(x, positions, rot)
    out = x.clone()
    first, second = x[..., :half], x[..., half:dims]
    out[..., :half] = first * cos - second * sin
    out[..., half:dims] = second * cos + first * sin
    return out


# ------------------------------------------------------------------------------ mixers
def attention_keys_values(h, weights, prefix, mixer, eps):
    """Keys (after norm and rotation) [n, G, dim] and values [n, G, vdim] of a layer that has projections of its own."""
    n = h.shape[0]
    groups, dim, vdim = int(mixer["kv_heads"]), int(mixer["dim"]), int(mixer.get("vdim", mixer["dim"]))
    w = lambda name: weights[prefix + name]
    k = (h @ w("k").T + w("k.b")).reshape(n, groups, dim)
    v = (h @ w("v").T + w("v.b")).reshape(n, groups, vdim)
    k = unit_rms(k, eps) * w("k.norm")
    if mixer.get("rot"):
        k = rotate_interleaved(k, torch.arange(n), mixer["rot"])
    return k, v


def attention(h, weights, prefix, mixer, eps, keys, values):
    """Softmax attention of h [n, w] over the given keys and values, with a window and a sink."""
    n = h.shape[0]
    heads, groups, dim = int(mixer["heads"]), int(mixer["kv_heads"]), int(mixer["dim"])
    vdim = int(mixer.get("vdim", dim))
    w = lambda name: weights[prefix + name]
    q = (h @ w("q").T + w("q.b")).reshape(n, heads, dim)
    q = unit_rms(q, eps) * w("q.norm")
    if mixer.get("rot"):
        q = rotate_interleaved(q, torch.arange(n), mixer["rot"])
    window = (mixer.get("mask") or {}).get("size")
    sink = w("sink")
    out = torch.zeros(n, heads, vdim, dtype=F64)
    for head in range(heads):
        group = head // (heads // groups)
        scores = (q[:, head] @ keys[:, group].T) * float(mixer["scale"])      # [query, key]
        i, j = torch.arange(n)[:, None], torch.arange(n)[None, :]
        hidden = j > i
        if window:
            hidden = hidden | (i - j >= int(window))
        scores = scores.masked_fill(hidden, float("-inf"))
        top = torch.maximum(scores.max(dim=1, keepdim=True).values, sink[head])
        weights_ = torch.exp(scores - top)
        total = weights_.sum(dim=1, keepdim=True) + torch.exp(sink[head] - top)     # the sink: no key, no value
        out[:, head] = (weights_ / total) @ values[:, group]
    mixed = out.reshape(n, heads * vdim) * sigmoid(h @ w("g").T)
    return mixed @ w("o").T


def retention(h, weights, prefix, mixer, eps, state=None, first_position=0):
    """Linear attention with a fixed decay per head; h [n, w].  Returns (output, state [heads, dim, vdim])."""
    n = h.shape[0]
    heads, dim = int(mixer["heads"]), int(mixer["dim"])
    vdim = int(mixer.get("vdim", dim))
    w = lambda name: weights[prefix + name]
    positions = torch.arange(first_position, first_position + n)
    q = (h @ w("q").T).reshape(n, heads, dim)
    k = (h @ w("k").T).reshape(n, heads, dim)
    v = (h @ w("v").T).reshape(n, heads, vdim)
    if mixer.get("rot"):
        q, k = rotate_half(q, positions, mixer["rot"]), rotate_half(k, positions, mixer["rot"])
    k = k * dim ** -0.5
    decay = torch.tensor([float(d) for d in mixer["decay"]], dtype=F64)
    if state is None:
        state = torch.zeros(heads, dim, vdim, dtype=F64)
    out = torch.zeros(n, heads, vdim, dtype=F64)
    for t in range(n):
        state = decay[:, None, None] * state + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hkv,hk->hv", state, q[t])
    mixed = unit_rms(out, eps).reshape(n, heads * vdim) * silu(h @ w("g").T)
    return mixed @ w("o").T, state


# ------------------------------------------------------------------------------ feed-forward
def feed_forward(h, weights, prefix):
    return relu_squared(h @ weights[prefix + "up"].T) @ weights[prefix + "down"].T


# ------------------------------------------------------------------------------ the model
def forward(config, weights, tokens, layers_out=None):
    """Logits [n, vocab] of one sequence.  `layers_out`: a list that receives the residual after every layer."""
    eps = float(config["norm"]["eps"])
    m = float(config.get("residual_mult", 1.0))
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x = norm_one_plus(weights["embed"][ids], weights["embed.norm"], eps)
    kept = {}                                              # layer -> (keys, values) for layers that lend theirs
    for index, layer in enumerate(config["layers"]):
        prefix = f"l{index}."
        mixer = layer["mixer"]
        if layer["type"] == "attention":
            source = mixer.get("kv_from")
            if source is None:
                kept[index] = attention_keys_values(x, weights, prefix + "mix.", mixer, eps)
                keys, values = kept[index]
            else:
                keys, values = kept[int(source)]
            y = attention(x, weights, prefix + "mix.", mixer, eps, keys, values)
        elif layer["type"] == "retention":
            y, _ = retention(x, weights, prefix + "mix.", mixer, eps)
        else:
            raise ValueError(layer["type"])
        x = x + m * norm_one_plus(y, weights[prefix + "norm1"], eps)
        if layer.get("mlp") is not None:
            y = feed_forward(x, weights, prefix + "mlp.")
            x = x + m * norm_one_plus(y, weights[prefix + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return norm_one_plus(x, weights["final.norm"], eps) @ weights["head"].T
