"""Gumazen, plain and slow: whole sequences, no cache, float64, one function per mechanism.

Written from the design's equations alone; it shares no code with the package.  `weights` maps stored tensor names to
tensors, `config` is the model's config.json as a dict.  Angles are formed as the design forms them: the 32-bit
product of a position and a 32-bit frequency.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import numpy as np
import torch

F = torch.float64


def read_model(folder):
    """(config, {name: tensor}) of a folder with config.json and model.safetensors (an 8-byte length, a JSON table of
    names, then the data)."""
    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    raw = (folder / "model.safetensors").read_bytes()
    size = int.from_bytes(raw[:8], "little")
    table = json.loads(raw[8:8 + size])
    body = raw[8 + size:]
    weights = {}
    for name, entry in table.items():
        if name == "__metadata__":
            continue
        begin, end = entry["data_offsets"]
        data = body[begin:end]
        if entry["dtype"] == "BF16":
            bits = np.frombuffer(data, dtype=np.uint16).astype(np.uint32) << 16
            values = torch.from_numpy(bits.view(np.float32).copy())
        elif entry["dtype"] == "F32":
            values = torch.from_numpy(np.frombuffer(data, dtype=np.float32).copy())
        else:
            raise ValueError(f"{name}: dtype {entry['dtype']}")
        weights[name] = values.reshape(entry["shape"]).to(F)
    return config, weights


def layer_norm(x, weight, bias, eps):
    mean = x.mean(-1, keepdim=True)
    centred = x - mean
    variance = (centred * centred).mean(-1, keepdim=True)
    return centred / torch.sqrt(variance + eps) * weight.to(F) + bias.to(F)


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def frequencies(rot):
    """f_i = base^(-2i / dims), remapped where the rotation names a scaling: kept for wavelengths below
    original / high, divided by factor above original / low, blended in between."""
    dims = int(rot["dims"])
    out = []
    for i in range(dims // 2):
        f = float(rot["base"]) ** (-2.0 * i / dims)
        scaling = rot.get("scaling")
        if scaling:
            factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            wavelength = 2.0 * math.pi / f
            if wavelength > original / low:
                f = f / factor
            elif wavelength >= original / high:
                s = (original / wavelength - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=torch.float32)


def rotate(x, rot):
    """x [T, heads, dim]: pairs (i, i + dims/2) of the first dims channels turn by position * f_i."""
    dims = int(rot["dims"])
    half = dims // 2
    positions = torch.arange(x.shape[0], dtype=torch.float32)
    angles = (positions[:, None] * frequencies(rot)[None, :]).to(F)          # a 32-bit product, then exact
    cos, sin = torch.cos(angles)[:, None, :], torch.sin(angles)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


def distance_bucket(n, rows, farthest):
    exact = rows // 2
    if n < exact:
        return n
    return min(rows - 1, exact + int(math.floor(math.log(n / exact) / math.log(farthest / exact) * (rows - exact))))


def attend(q, k, v, scale, window=None, sink=False, softcap=None, rel=None, farthest=None):
    """q [T, H, D], k [T, G, D], v [T, G, V] -> [T, H, V].  Causal; `window`: only the last `window` keys (the token
    itself among them); `sink`: one is added to the softmax's denominator; `softcap`: c tanh(score / c) after the
    scale; `rel` [rows, H]: a bias by the bucket of the distance, added after the cap."""
    tokens, heads, _ = q.shape
    per_group = heads // k.shape[1]
    out = torch.zeros(tokens, heads, v.shape[2], dtype=F)
    for h in range(heads):
        g = h // per_group
        for i in range(tokens):
            first = 0 if window is None else max(0, i - window + 1)
            scores = (k[first:i + 1, g] @ q[i, h]) * scale
            if softcap is not None:
                scores = softcap * torch.tanh(scores / softcap)
            if rel is not None:
                buckets = [distance_bucket(i - j, rel.shape[0], farthest) for j in range(first, i + 1)]
                scores = scores + rel[buckets, h].to(F)
            top = max(float(scores.max()), 0.0) if sink else float(scores.max())
            weights = torch.exp(scores - top)
            denominator = weights.sum() + (math.exp(-top) if sink else 0.0)
            out[i, h] = (weights / denominator) @ v[first:i + 1, g]
    return out


def project(h, weights, name):
    y = h @ weights[name].to(F).T
    if name + ".b" in weights:
        y = y + weights[name + ".b"].to(F)
    return y


def mixer_attention(h, weights, p, m, eps):
    """Rotation of q and k, then each head divided by its root mean square; a sink of score 0."""
    tokens = h.shape[0]
    q = project(h, weights, p + "q").view(tokens, m["heads"], m["dim"])
    k = project(h, weights, p + "k").view(tokens, m["kv_heads"], m["dim"])
    v = project(h, weights, p + "v").view(tokens, m["kv_heads"], m["vdim"])
    if m.get("rot"):
        q, k = rotate(q, m["rot"]), rotate(k, m["rot"])
    q, k = unit_rms(q, eps), unit_rms(k, eps)
    mixed = attend(q, k, v, m["scale"], sink=True)
    return project(mixed.reshape(tokens, -1), weights, p + "o")


def mixer_attention_2(h, weights, p, m, eps):
    """Norm of q and k over all heads at once, no rotation, capped scores plus a bias by distance, a window, one
    sigmoid gate per head."""
    tokens = h.shape[0]
    q = unit_rms(project(h, weights, p + "q"), eps) * weights[p + "q.norm"].to(F)
    k = unit_rms(project(h, weights, p + "k"), eps) * weights[p + "k.norm"].to(F)
    q = q.view(tokens, m["heads"], m["dim"])
    k = k.view(tokens, m["kv_heads"], m["dim"])
    v = project(h, weights, p + "v").view(tokens, m["kv_heads"], m["vdim"])
    mixed = attend(q, k, v, m["scale"], window=m["mask"]["size"], softcap=m["softcap"], rel=weights[p + "rel"],
                   farthest=m["bias_max"])
    gate = torch.sigmoid(h @ weights[p + "g"].to(F).T)                      # [T, heads]
    mixed = mixed * gate[:, :, None]
    return project(mixed.reshape(tokens, -1), weights, p + "o")


def mixer_attention_3(h, weights, p, m, eps):
    """Biases, norm of q and k over all heads at once, then the rotation with remapped frequencies."""
    tokens = h.shape[0]
    q = unit_rms(project(h, weights, p + "q"), eps) * weights[p + "q.norm"].to(F)
    k = unit_rms(project(h, weights, p + "k"), eps) * weights[p + "k.norm"].to(F)
    q = q.view(tokens, m["heads"], m["dim"])
    k = k.view(tokens, m["kv_heads"], m["dim"])
    v = project(h, weights, p + "v").view(tokens, m["kv_heads"], m["vdim"])
    if m.get("rot"):
        q, k = rotate(q, m["rot"]), rotate(k, m["rot"])
    mixed = attend(q, k, v, m["scale"])
    return project(mixed.reshape(tokens, -1), weights, p + "o")


MIXERS = {"attention": mixer_attention, "attention_2": mixer_attention_2, "attention_3": mixer_attention_3}


def dense(h, weights, p):
    hidden = torch.relu(h @ weights[p + "up"].to(F).T)
    return (hidden * hidden) @ weights[p + "down"].to(F).T


def gated_expert(h, weights, p):
    gate = h @ weights[p + "gate"].to(F).T
    return (gate * torch.sigmoid(gate) * (h @ weights[p + "up"].to(F).T)) @ weights[p + "down"].to(F).T


def route(h, weights, p, router):
    """(chosen [T, top], weight [T, top]): softmax scores over experts and identity experts, the correction added for
    the choice only, groups judged by their largest choice score, weights renormalised and scaled."""
    scores = torch.softmax(h @ weights[p + "router"].to(F).T, dim=-1)
    choice = scores + weights[p + "correction"].to(F) if p + "correction" in weights else scores.clone()
    total = scores.shape[1]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    size = total // groups["count"]
    chosen, amounts = [], []
    for t in range(scores.shape[0]):
        best = choice[t].view(groups["count"], size).max(dim=1).values
        order = sorted(range(groups["count"]), key=lambda g: (-float(best[g]), g))[:groups["keep"]]
        allowed = [e for e in range(total) if e // size in order]
        picked = sorted(allowed, key=lambda e: (-float(choice[t, e]), e))[:router["top"]]
        w = scores[t, picked]
        chosen.append(picked)
        amounts.append(w / (w.sum() + 1e-20) * router["scale"])
    return chosen, amounts


def experts(h, weights, p, mlp):
    router = mlp["router"]
    real = router["experts"]
    chosen, amounts = route(h, weights, p, router)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t], amounts[t]):
            row = h[t:t + 1]
            out[t] += w * (gated_expert(row, weights, f"{p}e{e}.")[0] if e < real else row[0])
    if mlp.get("shared"):
        out = out + gated_expert(h, weights, p + "shared.")
    return out


def feed_forward(h, weights, p, mlp):
    return dense(h, weights, p) if mlp["kind"] == "dense" else experts(h, weights, p, mlp)


def layer_order(config):
    count = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return list(range(count))
    inside = list(range(loop["start"], loop["stop"]))
    return list(range(loop["start"])) + inside * loop["times"] + list(range(loop["stop"], count))


def sublayer(streams, weights, hc, norm, eps, run):
    """One sublayer on the streams [S, T, W] (or on the single residual [T, W] if `hc` is None)."""
    if hc is None:
        return streams + run(layer_norm(streams, weights[norm], weights[norm + ".b"], eps))
    read = (weights[hc + "in"].to(F)[:, None, None] * streams).sum(0)
    y = run(layer_norm(read, weights[norm], weights[norm + ".b"], eps))
    mix, out = weights[hc + "mix"].to(F), weights[hc + "out"].to(F)
    return torch.einsum("st,sxw->txw", mix, streams) + out[:, None, None] * y[None]


def forward(config, weights, tokens, want_layers=False):
    """Logits [T, vocab] of one whole sequence (and the residual after every layer run, if asked for)."""
    eps = float(config["norm"]["eps"])
    x = weights["embed"].to(F)[torch.as_tensor(tokens, dtype=torch.long)]
    count = config.get("streams")
    state = x[None].repeat(count, 1, 1) if count else x
    after = []
    for index in layer_order(config):
        layer = config["layers"][index]
        p = f"l{index}."
        mixer = lambda h: MIXERS[layer["type"]](h, weights, p + "mix.", layer["mixer"], eps)
        state = sublayer(state, weights, p + "hc1." if count else None, p + "norm1", eps, mixer)
        if layer.get("mlp"):
            ff = lambda h: feed_forward(h, weights, p + "mlp.", layer["mlp"])
            state = sublayer(state, weights, p + "hc2." if count else None, p + "norm2", eps, ff)
        after.append(state.sum(0) if count else state)
    x = state.sum(0) if count else state
    logits = layer_norm(x, weights["final.norm"], weights["final.norm.b"], eps) @ weights["head"].to(F).T
    return (logits, torch.stack(after)) if want_layers else logits
