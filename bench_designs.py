"""`bench.py --design doderax | zufotar | dalesun | gumazen`: prefill and decode throughput of a design at layer sizes that resemble a
real model's (random weights), beside the dense SwiGLU decoder of equal width, depth and parameter count (and, for
Zufotar, beside Doderax, the closest model of the framework: recurrent mixers and attention in parallel layers), and
every kernel the design adds alone, with the fraction of its roofline, beside the like kernel of the closest model.

A kernel alone is launched 24 times inside one CUDA graph on rotating copies of its operands (together more than the
L2 holds); the graph is replayed five times and the median time per launch is taken from CUDA events.
"""

from __future__ import annotations

import gc
import statistics

PROMPT = 2048
BATCH = 8
PAGE = 16

# width, feed-forward, layers (three recurrent layers, then one with attention beside the recurrence), heads
DESIGN_SIZES = {
    "w2048": dict(width=2048, ff=8192, layers=12, heads=16, kv_heads=4, dim=128, window=1024, keep_first=4, vocab=65536),
    "w4096": dict(width=4096, ff=14336, layers=8, heads=32, kv_heads=8, dim=128, window=2048, keep_first=4, vocab=65536),
}


# Zufotar: latent attention and wkv layers in turn; the first feed-forward dense, the others routed experts; layers
# 2 and 3 run twice.  `runs` is the number of layer runs of a step, the depth of the models it is put beside.
ZUFOTAR_SIZES = {
    "w2048": dict(width=2048, layers=8, runs=10, heads=16, dim=128, rot=64, vdim=128, q_rank=768, kv_rank=512,
                  wkv_heads=32, wkv_dim=64, decay_rank=64, ff=8192, experts=64, top=6, expert_ff=1024, groups=(8, 4),
                  shared_ff=2048, vocab=65536, kv_heads=4, window=1024, keep_first=4),
    "w4096": dict(width=4096, layers=6, runs=8, heads=32, dim=128, rot=64, vdim=128, q_rank=1536, kv_rank=512,
                  wkv_heads=64, wkv_dim=64, decay_rank=64, ff=14336, experts=64, top=6, expert_ff=2048, groups=(8, 4),
                  shared_ff=4096, vocab=65536, kv_heads=8, window=2048, keep_first=4),
}


def zufotar_config(s: dict) -> dict:
    latent = {"heads": s["heads"], "dim": s["dim"], "rot_dim": s["rot"], "vdim": s["vdim"], "q_rank": s["q_rank"],
              "kv_rank": s["kv_rank"], "scale": (s["dim"] + s["rot"]) ** -0.5,
              "rot": {"dims": s["rot"], "base": 1000000.0,
                      "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    wkv = {"heads": s["wkv_heads"], "dim": s["wkv_dim"], "decay_rank": s["decay_rank"]}
    moe = {"kind": "moe", "expert": {"ff": s["expert_ff"]}, "shared": {"ff": s["shared_ff"]},
           "router": {"experts": s["experts"], "top": s["top"], "scale": 2.5,
                      "groups": {"count": s["groups"][0], "keep": s["groups"][1]}}}
    layers = []
    for index in range(s["layers"]):
        mixer = {"type": "latent_attention", "mixer": latent} if index % 2 == 0 else {"type": "wkv", "mixer": wkv}
        layers.append(dict(mixer, mlp={"kind": "dense", "ff": s["ff"]} if index == 0 else moe))
    return {"architecture": "Zufotar", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6},
            "embedding": {"scale": 1.0}, "logit_softcap": 30.0, "loop": {"start": 2, "stop": 4, "times": 2},
            "layers": layers}


def zufotar_kernel_table(s, tools) -> dict:
    """Every kernel the design adds, alone, at the sizes of a 2,048-token prompt and of a step of 8 decoded tokens:
    [microseconds, fraction of its roofline], beside the like kernel of the closest model."""
    import torch
    from libmir_b200 import kernels
    timed, copies, rand, device, hbm, flops_peak = (tools[k] for k in ("timed", "copies", "rand", "device", "hbm", "flops_peak"))
    bf16, f32, i32 = torch.bfloat16, torch.float32, torch.int32
    width, heads, dim, rot, vdim, rank = s["width"], s["heads"], s["dim"], s["rot"], s["vdim"], s["kv_rank"]
    key_width = rank + rot
    table = {}
    alloc = lambda shape, kind: torch.empty(shape, dtype=kind, device=device)
    for label, rows, portion in ((f"prefill_{PROMPT}", 1, PROMPT), (f"decode_b{BATCH}", BATCH, 1)):
        tokens = rows * portion
        starts = torch.arange(0, tokens + 1, portion, dtype=i32, device=device)
        row_of = torch.arange(tokens, dtype=i32, device=device) // portion
        slots = torch.arange(rows, dtype=i32, device=device)
        context = PROMPT if portion > 1 else PROMPT + 1
        positions = (torch.arange(tokens, dtype=i32, device=device) % portion) + (context - portion)
        prompt = portion > 1
        # ---- attention over cached latents, beside the dense decoder's attention over all keys
        pages_per_row = -(-(context + PAGE) // PAGE)
        cache_rows = rows * pages_per_row * PAGE
        caches = [rand(cache_rows, 1, key_width, scale=0.5)
                  for _ in range(max(2, min(24, -(-(300 << 20) // (cache_rows * key_width * 2)))))]
        block_table = torch.arange(rows * pages_per_row, dtype=i32, device=device).view(rows, pages_per_row).contiguous()
        contexts = torch.full((rows,), context, dtype=i32, device=device)
        folded = rand(tokens, heads * key_width, scale=0.3)
        attended = torch.empty(tokens, heads * rank, device=device, dtype=bf16)
        per_partition, partitions = kernels.latent_attention_plan(rows, portion * heads, context)
        scale = (dim + rot) ** -0.5
        calls = [lambda c=c: kernels.latent_attention(folded, attended, c, block_table, starts, contexts, PAGE, heads,
                                                      key_width, rank, scale, portion * heads, per_partition, partitions,
                                                      alloc) for c in caches]
        if prompt:
            flops = 2.0 * (PROMPT * (PROMPT + 1) / 2) * heads * (key_width + rank)
            table[f"{label}_latent_attention"] = timed(calls, flops, flops_peak)
        else:
            table[f"{label}_latent_attention"] = timed(calls, rows * context * key_width * 2, hbm)
        kv_heads = s["kv_heads"]
        k_cache = [rand(cache_rows, kv_heads, dim, scale=0.5) for _ in range(max(2, min(24, -(-(300 << 20) // (cache_rows * kv_heads * dim * 4)))))]
        v_cache = [rand(cache_rows, kv_heads, dim, scale=0.5) for _ in k_cache]
        qkv = rand(tokens, (heads + 2 * kv_heads) * dim, scale=0.3)
        mixed = torch.empty(tokens, heads * dim, device=device, dtype=bf16)
        if prompt:
            calls = [lambda k=k, v=v: kernels.prefill_attention(qkv, mixed, k, v, block_table, starts, contexts, PAGE, heads,
                                                                 kv_heads, dim, dim ** -0.5, None) for k, v in zip(k_cache, v_cache)]
            table[f"{label}_dense_attention_full"] = timed(calls, 4.0 * (PROMPT * (PROMPT + 1) / 2) * dim * heads, flops_peak)
        else:
            q_positions = torch.full((tokens,), context - 1, dtype=i32, device=device)
            partition, count, floats = kernels.decode_attention_plan(rows, heads, kv_heads, dim, PAGE, context)
            scratch = torch.empty(max(floats, 1), device=device, dtype=f32)
            calls = [lambda k=k, v=v: kernels.decode_attention(qkv, mixed, k, v, block_table, q_positions, PAGE, heads, kv_heads,
                                                                dim, dim ** -0.5, None, partition, count,
                                                                scratch if floats else None) for k, v in zip(k_cache, v_cache)]
            table[f"{label}_dense_attention_full"] = timed(calls, rows * context * kv_heads * dim * 2 * 2, hbm)
        # ---- the products per head around it, the latents' norms and the rotation
        q = rand(tokens, heads, dim + rot, scale=0.3)
        w_uk = rand(heads, dim, rank, scale=0.05)
        folded3 = folded.view(tokens, heads, key_width)
        calls = [lambda: kernels.head_linear(q[:, :, :dim], w_uk, folded3[:, :, :rank])]
        work = 2.0 * tokens * heads * dim * rank
        table[f"{label}_head_linear_keys_into_queries"] = timed(calls, work, flops_peak) if prompt else \
            timed(calls, heads * dim * rank * 2, hbm)
        w_uv = rand(heads, rank, vdim, scale=0.05)
        gate = rand(tokens, heads * vdim)
        values = torch.empty(tokens, heads, vdim, device=device, dtype=bf16)
        calls = [lambda: kernels.head_linear(attended.view(tokens, heads, rank), w_uv, values, gate)]
        table[f"{label}_head_linear_values_gated"] = timed(calls, 2.0 * tokens * heads * rank * vdim, flops_peak) if prompt else \
            timed(calls, heads * rank * vdim * 2, hbm)
        packed = rand(tokens, s["q_rank"] + key_width + 8)
        inv_freq = torch.rand(rot // 2, device=device, dtype=f32)
        latent_q = torch.empty(tokens, s["q_rank"], device=device, dtype=bf16)
        slot_map = torch.arange(tokens, dtype=i32, device=device)
        ones_q, ones_kv = torch.ones(s["q_rank"], device=device), torch.ones(rank, device=device)
        calls = [lambda c=c: kernels.latent_prepare(packed, 0, s["q_rank"], s["q_rank"], rank, rot, ones_q, ones_kv, 1e-6,
                                                    positions, slot_map, inv_freq, 1.1, True, latent_q, c) for c in caches]
        table[f"{label}_latent_prepare"] = timed(calls, tokens * (s["q_rank"] + key_width) * 4, hbm)
        calls = [lambda: kernels.rope_rows(q[:, :, dim:], folded3[:, :, rank:], positions, inv_freq, 1.1, True)]
        table[f"{label}_rope_rows"] = timed(calls, tokens * heads * rot * 4, hbm)
        # ---- wkv, beside the gated delta rule with one decay per key channel at the same heads
        wh, wd = s["wkv_heads"], s["wkv_dim"]
        wwidth = wh * wd
        packs = copies(lambda: (torch.zeros(rows, wh, wd, wd, device=device, dtype=f32), rand(3, tokens, wwidth, scale=0.3),
                                rand(tokens, wwidth, dtype=f32)), rows * wh * wd * wd * 4)
        bias, bonus = rand(wwidth, dtype=f32), rand(wwidth, dtype=f32, scale=0.3)
        out = torch.empty(tokens, wwidth, device=device, dtype=f32)
        calls = [lambda p=p: kernels.wkv_scan(p[1][0], p[1][1], p[1][2], p[2], bias, bonus, p[0], starts, slots, positions, out,
                                              wh, wd) for p in packs]
        state_bytes = rows * wh * wd * wd * 4 * 2 + tokens * wwidth * (3 * 2 + 4 + 4)
        note = ["of the bf16 tensor peak; the kernel is 32-bit FMA, one token after the other"]
        table[f"{label}_wkv_scan"] = timed(calls, 4.0 * tokens * wh * wd * wd, flops_peak) + note if prompt else timed(calls, state_bytes, hbm)
        packs = copies(lambda: (torch.zeros(rows, wh, wd, wd, device=device, dtype=f32), rand(tokens, 3 * wwidth, dtype=f32, scale=0.1)),
                       rows * wh * wd * wd * 4)
        beta = torch.rand(tokens, wh, device=device, dtype=f32)
        decay = torch.rand(tokens, wwidth, device=device, dtype=f32) * 0.5 + 0.5
        calls = [lambda p=p: kernels.delta_rule_scan(p[1], beta, decay, p[0], starts, slots, positions, out, wh, wh, wd, wd)
                 for p in packs]
        table[f"{label}_doderax_delta_rule_channel"] = timed(calls, 8.0 * tokens * wh * wd * wd, flops_peak) + note if prompt else \
            timed(calls, rows * wh * wd * wd * 8 + tokens * wwidth * 24, hbm)
        h = rand(tokens, width)
        tail = torch.zeros(rows, width, device=device, dtype=f32)
        mu = torch.rand(5, width, device=device, dtype=f32)
        mixes = [torch.empty(5, tokens, width, device=device, dtype=bf16) for _ in range(2)]
        calls = [lambda m=m: kernels.wkv_mix(h, tail, mu, row_of, starts, slots, positions, m, single_tokens_only=not prompt)
                 for m in mixes]
        table[f"{label}_wkv_mix"] = timed(calls, tokens * width * 12, hbm)
        read = rand(tokens, wwidth, dtype=f32)
        norm_weight = rand(wwidth, dtype=f32)
        gated = torch.empty(tokens, wwidth, device=device, dtype=bf16)
        calls = [lambda: kernels.gated_head_norm(read, h[:, :wwidth], norm_weight, gated, wh, wd, 1e-6, False)]
        table[f"{label}_gated_head_norm"] = timed(calls, tokens * wwidth * 8, hbm)
        # ---- two norms in one kernel beside one norm; the exact GELU beside the tanh form
        residual = rand(tokens, width, dtype=f32)
        w_a, w_b = rand(width, dtype=f32), rand(width, dtype=f32)
        out_a, out_b = (torch.empty(tokens, width, device=device, dtype=bf16) for _ in range(2))
        table[f"{label}_rms_norm_pair"] = timed([lambda: kernels.rms_norm_pair(residual, w_a, w_b, 1e-6, out_a, out_b)],
                                                tokens * width * 8, hbm)
        table[f"{label}_dense_rms_norm"] = timed([lambda: kernels.rms_norm(residual, w_a, 1e-6, out_a)], tokens * width * 6, hbm)
        packs = copies(lambda: rand(tokens, s["ff"]), tokens * s["ff"] * 2)
        table[f"{label}_gelu_erf"] = timed([lambda p=p: kernels.gelu_erf(p) for p in packs], tokens * s["ff"] * 4, hbm)
        table[f"{label}_doderax_gelu_tanh"] = timed([lambda p=p: kernels.gelu_tanh(p) for p in packs], tokens * s["ff"] * 4, hbm)
        # ---- routed experts, beside the dense decoder's products of the same work
        experts, top, ff = s["experts"], s["top"], s["expert_ff"]
        pairs = tokens * top
        router = rand(experts + 8, width, scale=0.05)            # the router's rows, the shared gate's row, padding
        correction = rand(experts, dtype=f32, scale=0.1)
        logits = torch.empty(tokens, experts + 8, device=device, dtype=f32)
        ids = torch.empty(tokens, top, device=device, dtype=i32)
        weights = torch.empty(tokens, top, device=device, dtype=f32)
        shared_gate = torch.empty(tokens, device=device, dtype=f32)
        calls = [lambda: kernels.linear(h, router, logits, alloc=alloc)]
        table[f"{label}_moe_router_logits"] = timed(calls, tokens * width * 2 + (experts + 8) * width * 2, hbm)
        calls = [lambda: kernels.moe_route(logits, correction, True, ids, weights, shared_gate, experts, top,
                                           s["groups"][0], s["groups"][1], 2.5)]
        table[f"{label}_moe_route"] = timed(calls, tokens * (experts + 8) * 4, hbm)
        tile = kernels.expert_tile_pairs(bf16, width, ff)
        found = kernels.moe_sort(ids, experts, alloc, tile)
        table[f"{label}_moe_sort"] = timed([lambda: kernels.moe_sort(ids, experts, alloc, tile)], pairs * 8, hbm)
        torch.cuda.synchronize()
        used = int(torch.unique(ids).numel())
        banks = max(2, min(8, -(-(300 << 20) // (experts * ff * width * 6))))
        both = [rand(2 * experts, ff, width, scale=0.03) for _ in range(banks)]        # gate rows, the up rows behind them
        gates, ups = [b[:experts] for b in both], [b[experts:] for b in both]
        downs = [rand(experts, width, ff, scale=0.03) for _ in range(banks)]
        hidden = torch.empty(pairs, ff, device=device, dtype=bf16)
        calls = [lambda g=g, u=u: kernels.moe_gate_up(h, found, top, g, u, hidden, alloc) for g, u in zip(gates, ups)]
        table[f"{label}_moe_gate_up"] = timed(calls, 4.0 * pairs * ff * width, flops_peak) if prompt else \
            timed(calls, used * 2 * ff * width * 2, hbm)
        pair_rows = torch.empty(pairs, width, device=device, dtype=f32)
        calls = [lambda d=d: kernels.moe_down(hidden, found, d, pair_rows) for d in downs]
        table[f"{label}_moe_down"] = timed(calls, 2.0 * pairs * ff * width, flops_peak) if prompt else \
            timed(calls, used * ff * width * 2, hbm)
        shared_rows = rand(tokens, width, dtype=f32)
        calls = [lambda: kernels.moe_combine(residual, pair_rows, weights, shared_rows, shared_gate)]
        table[f"{label}_moe_combine"] = timed(calls, pairs * width * 4 + tokens * width * 12, hbm)
        # the same work as dense products: a prompt's pairs as rows of one product; a step's experts as one wide matrix
        dense_rows, dense_inter = (pairs, ff) if prompt else (tokens, ff * used)
        x_dense = rand(dense_rows, width)
        w_gu = [rand(2 * dense_inter, width, scale=0.03) for _ in range(max(2, min(8, -(-(300 << 20) // (dense_inter * width * 4)))))]
        hidden_dense = torch.empty(dense_rows, dense_inter, device=device, dtype=bf16)
        calls = [lambda w=w: kernels.gate_up_silu(x_dense, w, hidden_dense, alloc) for w in w_gu]
        table[f"{label}_dense_gate_up_same_work"] = timed(calls, 4.0 * dense_rows * dense_inter * width, flops_peak) if prompt else \
            timed(calls, 2 * dense_inter * width * 2, hbm)
        w_d = [rand(width, dense_inter, scale=0.03) for _ in w_gu]
        out_dense = torch.zeros(dense_rows, width, device=device, dtype=f32)
        calls = [lambda w=w: kernels.linear(hidden_dense, w, out_dense, accumulate=True) for w in w_d]
        table[f"{label}_dense_down_same_work"] = timed(calls, 2.0 * dense_rows * dense_inter * width, flops_peak) if prompt else \
            timed(calls, dense_inter * width * 2, hbm)
    return table


# Dalesun: two retention layers, an attention layer with keys of its own and one that borrows them, in turn.
DALESUN_SIZES = {
    "w2048": dict(width=2048, ff=8192, layers=12, heads=16, kv_heads=4, dim=128, window=1024, keep_first=4, vocab=65536,
                  retention_heads=16, retention_dim=128),
    "w4096": dict(width=4096, ff=14336, layers=8, heads=32, kv_heads=8, dim=128, window=2048, keep_first=4, vocab=65536,
                  retention_heads=32, retention_dim=128),
}


def dalesun_config(s: dict) -> dict:
    heads, dim = s["retention_heads"], s["retention_dim"]
    retention = {"heads": heads, "dim": dim, "vdim": dim, "rot": {"dims": dim, "base": 500000.0},
                 "decay": [1.0 - 2.0 ** (-4.0 - 8.0 * h / heads) for h in range(heads)]}
    attention = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"],
                 "scale": s["dim"] ** -0.5, "rot": {"dims": s["dim"] // 2, "base": 10000.0}, "mask": {"size": s["window"]}}
    mlp = {"kind": "dense", "ff": s["ff"]}
    layers = []
    for index in range(s["layers"]):
        if index % 4 < 2:
            layers.append({"type": "retention", "mixer": retention, "mlp": mlp})
        elif index % 4 == 2:
            layers.append({"type": "attention", "mixer": attention, "mlp": mlp})
        else:
            layers.append({"type": "attention", "mixer": dict(attention, kv_from=index - 1), "mlp": mlp})
    return {"architecture": "Dalesun", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-5},
            "residual_mult": 0.5, "layers": layers}


def dalesun_kernel_table(s, tools) -> dict:
    """Every kernel the design adds or extends, alone, at the sizes of a 2,048-token prompt and of a step of 8 decoded
    tokens: [microseconds, fraction of its roofline], beside the like kernel of the closest models (Doderax's delta
    rule with one decay per head; the dense decoder's attention, rotation and feed-forward products)."""
    import torch
    from libmir_b200 import kernels
    timed, copies, rand, device, hbm, flops_peak = (tools[k] for k in ("timed", "copies", "rand", "device", "hbm", "flops_peak"))
    bf16, f32, i32 = torch.bfloat16, torch.float32, torch.int32
    width, heads, kv_heads, dim, ff, window = s["width"], s["heads"], s["kv_heads"], s["dim"], s["ff"], s["window"]
    rh, rd = s["retention_heads"], s["retention_dim"]
    table = {}
    alloc = lambda shape, kind: torch.empty(shape, dtype=kind, device=device)
    note = ["of the bf16 tensor peak; the kernel is 32-bit FMA, one token after the other"]
    for label, rows, portion in ((f"prefill_{PROMPT}", 1, PROMPT), (f"decode_b{BATCH}", BATCH, 1)):
        tokens = rows * portion
        prompt = portion > 1
        starts = torch.arange(0, tokens + 1, portion, dtype=i32, device=device)
        slots = torch.arange(rows, dtype=i32, device=device)
        context = PROMPT if prompt else PROMPT + 1
        positions = (torch.arange(tokens, dtype=i32, device=device) % portion) + (context - portion)
        # ---- the retention recurrence (rotation inside), beside the delta rule with one decay per head
        rwidth = rh * rd
        packs = copies(lambda: (torch.zeros(rows, rh, rd, rd, device=device, dtype=f32), rand(tokens, 4 * rwidth, scale=0.3)),
                       rows * rh * rd * rd * 4)
        inv_freq = torch.rand(rd // 2, device=device, dtype=f32)
        decays = torch.rand(rh, device=device, dtype=f32) * 0.1 + 0.9
        read = torch.empty(tokens, rwidth, device=device, dtype=f32)
        # (a prompt's portion: the rotation's kernel and the walk over what it left, as the mixer runs them)
        scratch = torch.empty(kernels.retention_prepared_floats(tokens, rh, rd), device=device, dtype=f32) if prompt else None
        calls = [lambda p=p: kernels.retention_scan(p[1][:, :rwidth], p[1][:, rwidth:2 * rwidth], p[1][:, 2 * rwidth:3 * rwidth],
                                                    inv_freq, decays, rd ** -0.5, p[0], starts, slots, positions, read,
                                                    rh, rd, rd, prepared=scratch) for p in packs]
        state_bytes = rows * rh * rd * rd * 8 + tokens * rwidth * (3 * 2 + 4)
        table[f"{label}_retention_scan"] = timed(calls, 4.0 * tokens * rh * rd * rd, flops_peak) + note if prompt else \
            timed(calls, state_bytes, hbm)
        packs = copies(lambda: (torch.zeros(rows, rh, rd, rd, device=device, dtype=f32), rand(tokens, 3 * rwidth, dtype=f32, scale=0.1)),
                       rows * rh * rd * rd * 4)
        beta = torch.rand(tokens, rh, device=device, dtype=f32)
        decay = torch.rand(tokens, rh, device=device, dtype=f32) * 0.5 + 0.5
        calls = [lambda p=p: kernels.delta_rule_scan(p[1], beta, decay, p[0], starts, slots, positions, read, rh, rh, rd, rd)
                 for p in packs]
        table[f"{label}_doderax_delta_rule_head"] = timed(calls, 8.0 * tokens * rh * rd * rd, flops_peak) + note if prompt else \
            timed(calls, rows * rh * rd * rd * 8 + tokens * rwidth * 20, hbm)
        # ---- unit norm per head with a silu gate; the branch's norm into the residual (Doderax's kernels, one branch)
        packs = copies(lambda: (rand(tokens, rwidth, dtype=f32), rand(tokens, rwidth)), tokens * rwidth * 6)
        ones = torch.ones(rd, device=device, dtype=f32)
        gated = torch.empty(tokens, rwidth, device=device, dtype=bf16)
        calls = [lambda p=p: kernels.gated_head_norm(p[0], p[1], ones, gated, rh, rd, 1e-6, False) for p in packs]
        table[f"{label}_gated_head_norm"] = timed(calls, tokens * rwidth * 8, hbm)
        packs = copies(lambda: (rand(tokens, width, dtype=f32), rand(tokens, width, dtype=f32)), tokens * width * 8)
        w_a, w_b = rand(width, dtype=f32), rand(width, dtype=f32)
        calls = [lambda p=p: kernels.add_normed_branches([p[0]], [w_a], p[1], 1e-6, 0.6) for p in packs]
        table[f"{label}_add_normed_branch"] = timed(calls, tokens * width * 12, hbm)
        calls = [lambda p=p: kernels.add_normed_branches([p[0], p[0]], [w_a, w_b], p[1], 1e-6, 0.5) for p in packs]
        table[f"{label}_doderax_add_normed_branches"] = timed(calls, tokens * width * 12, hbm)
        out_w = torch.empty(tokens, width, device=device, dtype=bf16)
        calls = [lambda p=p: kernels.rms_norm(p[0], w_a, 1e-6, out_w) for p in packs]
        table[f"{label}_dense_rms_norm"] = timed(calls, tokens * width * 6, hbm)
        # ---- q/k norm, rotation of interleaved pairs, keys and values into pages; rows [q | k | v | gate]
        pages_per_row = -(-(context + PAGE) // PAGE)
        cache_rows = rows * pages_per_row * PAGE
        count = max(2, min(24, -(-(300 << 20) // (cache_rows * kv_heads * dim * 4))))
        k_cache = [rand(cache_rows, kv_heads, dim, scale=0.5) for _ in range(count)]
        v_cache = [rand(cache_rows, kv_heads, dim, scale=0.5) for _ in range(count)]
        block_table = torch.arange(rows * pages_per_row, dtype=i32, device=device).view(rows, pages_per_row).contiguous()
        contexts = torch.full((rows,), context, dtype=i32, device=device)
        slot_map = (torch.arange(tokens, dtype=i32, device=device) // portion) * (pages_per_row * PAGE) + positions
        packed_width = (heads + 2 * kv_heads) * dim
        rows_gated = rand(tokens, packed_width + heads * dim, scale=0.3)
        rows_plain = rand(tokens, packed_width, scale=0.3)
        norm_q, norm_k = torch.ones(dim, device=device), torch.ones(dim, device=device)
        freq = torch.rand(dim // 4, device=device, dtype=f32)
        moved = tokens * (heads + kv_heads) * dim * 4 + tokens * kv_heads * dim * 4
        calls = [lambda k=k, v=v: kernels.qk_rope_store(rows_gated, positions, slot_map, freq, norm_q, norm_k, k, v, heads,
                                                        kv_heads, dim, dim // 2, 1e-6, value_dim=dim, interleaved=True)
                 for k, v in zip(k_cache, v_cache)]
        table[f"{label}_qk_rope_store_interleaved"] = timed(calls, moved, hbm)
        freq_half = torch.rand(dim // 2, device=device, dtype=f32)
        calls = [lambda k=k, v=v: kernels.qk_rope_store(rows_plain, positions, slot_map, freq_half, norm_q, norm_k, k, v, heads,
                                                        kv_heads, dim, dim, 1e-6) for k, v in zip(k_cache, v_cache)]
        table[f"{label}_dense_qk_rope_store"] = timed(calls, moved, hbm)
        # ---- attention in a window with a sink per head and a sigmoid gate, beside the dense decoder's in the same window
        qkv = rand(tokens, packed_width + heads * dim, scale=0.3)
        gate = qkv[:, packed_width:]
        sinks = rand(heads, dtype=f32)
        mixed = torch.empty(tokens, heads * dim, device=device, dtype=bf16)
        scale = dim ** -0.5
        if prompt:
            visible = sum(min(p + 1, window) for p in range(PROMPT))
            flops = 4.0 * visible * dim * heads
            for extras, name in (({"sinks": sinks, "gate": gate}, "attention_window_sink_gate"), ({}, "dense_attention_window")):
                calls = [lambda k=k, v=v, e=extras: kernels.prefill_attention(qkv, mixed, k, v, block_table, starts, contexts,
                                                                               PAGE, heads, kv_heads, dim, scale, window, **e)
                         for k, v in zip(k_cache, v_cache)]
                table[f"{label}_{name}"] = timed(calls, flops, flops_peak)
        else:
            q_positions = torch.full((tokens,), context - 1, dtype=i32, device=device)
            partition, parts, floats = kernels.decode_attention_plan(rows, heads, kv_heads, dim, PAGE, context)
            scratch = torch.empty(max(floats, 1), device=device, dtype=f32)
            key_bytes = rows * min(window, context) * kv_heads * dim * 2 * 2
            for extras, name in (({"sinks": sinks, "gate": gate}, "attention_window_sink_gate"), ({}, "dense_attention_window")):
                calls = [lambda k=k, v=v, e=extras: kernels.decode_attention(qkv, mixed, k, v, block_table, q_positions, PAGE,
                                                                              heads, kv_heads, dim, scale, window, partition,
                                                                              parts, scratch if floats else None, **e)
                         for k, v in zip(k_cache, v_cache)]
                table[f"{label}_{name}"] = timed(calls, key_bytes, hbm)
        # ---- the feed-forward's first product with the squared relu in its epilogue, beside the dense decoder's
        # gate and up product with its silu, at the same multiply-adds
        x = rand(tokens, width)
        banks = max(2, min(8, -(-(300 << 20) // (ff * width * 2))))
        ups = [rand(ff, width, scale=0.03) for _ in range(banks)]
        hidden = torch.empty(tokens, ff, device=device, dtype=bf16)
        calls = [lambda w=w: kernels.linear_act(x, w, hidden, "relu2", alloc=alloc) for w in ups]
        table[f"{label}_up_relu_squared"] = timed(calls, 2.0 * tokens * ff * width, flops_peak) if prompt else \
            timed(calls, ff * width * 2, hbm)
        hidden_half = torch.empty(tokens, ff // 2, device=device, dtype=bf16)
        calls = [lambda w=w: kernels.gate_up_silu(x, w, hidden_half, alloc) for w in ups]
        table[f"{label}_dense_gate_up_silu_same_work"] = timed(calls, 2.0 * tokens * ff * width, flops_peak) if prompt else \
            timed(calls, ff * width * 2, hbm)
    return table


# Gumazen: a residual of four streams, layer norms, three kinds of attention in turn (rotated with remapped frequencies
# and biases; capped scores with a bias by distance in a window and a gate per head; rotated, normed behind the rotation,
# with a sink), the first feed-forward dense with a squared relu, the others routed experts of which some are identity
# experts; the middle layers run twice.  `runs` is the number of layer runs of a step.
GUMAZEN_SIZES = {
    "w2048": dict(width=2048, streams=4, layers=8, loop=(2, 6, 2), runs=12, heads=16, kv_heads=4, dim=128, window=1024,
                  softcap=50.0, bias_rows=32, bias_max=512.0, ff=8192, experts=56, identity=8, top=6, expert_ff=1024,
                  groups=(8, 4), shared_ff=2048, vocab=65536),
    "w4096": dict(width=4096, streams=4, layers=6, loop=(2, 4, 2), runs=8, heads=32, kv_heads=8, dim=128, window=2048,
                  softcap=50.0, bias_rows=32, bias_max=1024.0, ff=14336, experts=56, identity=8, top=6, expert_ff=2048,
                  groups=(8, 4), shared_ff=4096, vocab=65536),
}


def gumazen_config(s: dict) -> dict:
    heads = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"], "scale": s["dim"] ** -0.5}
    scaled = {"type": "attention_3", "mixer": dict(heads, rot={"dims": s["dim"] // 2, "base": 1000000.0, "scaling": {
        "factor": 4.0, "low": 1.0, "high": 4.0, "original": 4096}})}
    biased = {"type": "attention_2", "mixer": dict(heads, softcap=s["softcap"], bias_max=s["bias_max"],
                                                   bias_rows=s["bias_rows"], mask={"size": s["window"]})}
    sink = {"type": "attention", "mixer": dict(heads, rot={"dims": s["dim"], "base": 10000.0})}
    moe = {"kind": "moe", "expert": {"ff": s["expert_ff"]}, "shared": {"ff": s["shared_ff"]},
           "router": {"experts": s["experts"], "identity": s["identity"], "top": s["top"], "scale": 2.0,
                      "groups": {"count": s["groups"][0], "keep": s["groups"][1]}}}
    kinds = (scaled, biased, sink)
    layers = [dict(kinds[index % 3], mlp={"kind": "dense", "ff": s["ff"]} if index == 0 else moe)
              for index in range(s["layers"])]
    start, stop, times = s["loop"]
    return {"architecture": "Gumazen", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-5},
            "streams": s["streams"], "loop": {"start": start, "stop": stop, "times": times}, "layers": layers}


def gumazen_kernel_table(s, tools) -> dict:
    """Every kernel the design adds or extends, alone, at the sizes of a 2,048-token prompt and of a step of 8 decoded
    tokens: [microseconds, fraction of its roofline], beside the like kernel of the closest models (the dense decoder's
    norm, q/k kernel and attention; Zufotar's router and the sum of its experts' rows)."""
    import torch
    from libmir_b200 import kernels
    timed, copies, rand, device, hbm, flops_peak = (tools[k] for k in ("timed", "copies", "rand", "device", "hbm", "flops_peak"))
    bf16, f32, i32 = torch.bfloat16, torch.float32, torch.int32
    width, heads, kv_heads, dim, window, count = s["width"], s["heads"], s["kv_heads"], s["dim"], s["window"], s["streams"]
    table = {}
    for label, rows, portion in ((f"prefill_{PROMPT}", 1, PROMPT), (f"decode_b{BATCH}", BATCH, 1)):
        tokens = rows * portion
        prompt = portion > 1
        starts = torch.arange(0, tokens + 1, portion, dtype=i32, device=device)
        context = PROMPT if prompt else PROMPT + 1
        positions = (torch.arange(tokens, dtype=i32, device=device) % portion) + (context - portion)
        # ---- the residual's streams: the layer norm that reads their mix, the update that writes all of them
        packs = copies(lambda: (rand(tokens, count, width, dtype=f32), rand(tokens, width, dtype=f32)), tokens * width * 4 * (count + 1))
        w_a, w_b = rand(width, dtype=f32), rand(width, dtype=f32)
        read, write = rand(count, dtype=f32), rand(count, dtype=f32)
        mix = rand(count, count, dtype=f32)
        out_w = torch.empty(tokens, width, device=device, dtype=bf16)
        calls = [lambda p=p: kernels.layer_norm(p[0], w_a, w_b, 1e-5, out_w, None, read) for p in packs]
        table[f"{label}_layer_norm_of_streams"] = timed(calls, tokens * width * (4 * count + 2), hbm)
        calls = [lambda p=p: kernels.layer_norm(p[1], w_a, w_b, 1e-5, out_w) for p in packs]
        table[f"{label}_layer_norm"] = timed(calls, tokens * width * 6, hbm)
        calls = [lambda p=p: kernels.rms_norm(p[1], w_a, 1e-6, out_w) for p in packs]
        table[f"{label}_dense_rms_norm"] = timed(calls, tokens * width * 6, hbm)
        calls = [lambda p=p: kernels.streams_write(p[0], p[1], mix, write) for p in packs]
        table[f"{label}_streams_write"] = timed(calls, tokens * width * 4 * (2 * count + 1), hbm)
        if hasattr(kernels, "streams_write_norm"):
            calls = [lambda p=p: kernels.streams_write_norm(p[0], p[1], mix, write, read, w_a, w_b, 1e-5, out_w) for p in packs]
            table[f"{label}_streams_write_and_next_norm"] = timed(calls, tokens * width * (4 * (2 * count + 1) + 2), hbm)
        # ---- q and k: the norm over a whole projection (with and without the rotation behind it), the rotation with the
        # unweighted norm per head behind it; keys and values into pages; beside the dense decoder's kernel
        pages_per_row = -(-(context + PAGE) // PAGE)
        cache_rows = rows * pages_per_row * PAGE
        banks = max(2, min(24, -(-(300 << 20) // (cache_rows * kv_heads * dim * 4))))
        k_cache = [rand(cache_rows, kv_heads, dim, scale=0.5) for _ in range(banks)]
        v_cache = [rand(cache_rows, kv_heads, dim, scale=0.5) for _ in range(banks)]
        block_table = torch.arange(rows * pages_per_row, dtype=i32, device=device).view(rows, pages_per_row).contiguous()
        contexts = torch.full((rows,), context, dtype=i32, device=device)
        slot_map = (torch.arange(tokens, dtype=i32, device=device) // portion) * (pages_per_row * PAGE) + positions
        packed_width = (heads + 2 * kv_heads) * dim
        qkv = rand(tokens, packed_width + 8 * (-(-heads // 8)), scale=0.3)
        plain_rows = rand(tokens, packed_width, scale=0.3)
        q_whole, k_whole = torch.ones(heads * dim, device=device), torch.ones(kv_heads * dim, device=device)
        norm_q, norm_k = torch.ones(dim, device=device), torch.ones(dim, device=device)
        freq_half, freq_quarter = torch.rand(dim // 2, device=device, dtype=f32), torch.rand(dim // 4, device=device, dtype=f32)
        moved = tokens * (heads + kv_heads) * dim * 4 + tokens * kv_heads * dim * 4
        for name, args in (("qk_prepare_projection_norm_then_rotation", (freq_quarter, q_whole, k_whole, dim // 2, "projection", False)),
                           ("qk_prepare_projection_norm", (None, q_whole, k_whole, 0, "projection", False)),
                           ("qk_prepare_rotation_then_head_norm", (freq_half, None, None, dim, "head", True))):
            freq, qw, kw, rotary, span, after = args
            calls = [lambda k=k, v=v: kernels.qk_prepare(qkv, positions, slot_map, freq, qw, kw, k, v, heads, kv_heads, dim, dim,
                                                         rotary, 1e-5, span, after_rotation=after) for k, v in zip(k_cache, v_cache)]
            table[f"{label}_{name}"] = timed(calls, moved, hbm)
        calls = [lambda k=k, v=v: kernels.qk_rope_store(plain_rows, positions, slot_map, freq_half, norm_q, norm_k, k, v, heads,
                                                        kv_heads, dim, dim, 1e-6) for k, v in zip(k_cache, v_cache)]
        table[f"{label}_dense_qk_rope_store"] = timed(calls, moved, hbm)
        # ---- attention: capped scores with a bias by distance in a window and a gate per head; all keys with a sink;
        # beside the dense decoder's in the same window and over all keys
        gate = qkv[:, packed_width:packed_width + heads]
        bias = rand(heads, min(window, int(s["bias_max"]) + 1), dtype=f32)
        sinks = torch.zeros(heads, device=device, dtype=f32)
        mixed = torch.empty(tokens, heads * dim, device=device, dtype=bf16)
        scale = dim ** -0.5
        scored = dict(gate=gate, gate_per_head=True, softcap=s["softcap"], distance_bias=bias)
        if prompt:
            in_window = 4.0 * sum(min(p + 1, window) for p in range(PROMPT)) * dim * heads
            everything = 4.0 * (PROMPT * (PROMPT + 1) / 2) * dim * heads
            for extras, span, flops, name in ((scored, window, in_window, "attention_window_capped_biased_gated"),
                                              ({}, window, in_window, "dense_attention_window"),
                                              ({"sinks": sinks}, None, everything, "attention_full_sink"),
                                              ({}, None, everything, "dense_attention_full")):
                calls = [lambda k=k, v=v, e=extras, w=span: kernels.prefill_attention(qkv, mixed, k, v, block_table, starts, contexts,
                                                                                       PAGE, heads, kv_heads, dim, scale, w, **e)
                         for k, v in zip(k_cache, v_cache)]
                table[f"{label}_{name}"] = timed(calls, flops, flops_peak)
        else:
            q_positions = torch.full((tokens,), context - 1, dtype=i32, device=device)
            for extras, span, name in ((scored, window, "attention_window_capped_biased_gated"), ({}, window, "dense_attention_window"),
                                       ({"sinks": sinks}, None, "attention_full_sink"), ({}, None, "dense_attention_full")):
                plan = kernels.decode_attention_plan
                partition, parts, floats = plan(rows, heads, kv_heads, dim, PAGE, context)
                scratch = torch.empty(max(floats, 1), device=device, dtype=f32)
                key_bytes = rows * (min(span, context) if span else context) * kv_heads * dim * 2 * 2
                calls = [lambda k=k, v=v, e=extras, w=span: kernels.decode_attention(qkv, mixed, k, v, block_table, q_positions, PAGE,
                                                                                      heads, kv_heads, dim, scale, w, partition, parts,
                                                                                      scratch if floats else None, **e)
                         for k, v in zip(k_cache, v_cache)]
                table[f"{label}_{name}"] = timed(calls, key_bytes, hbm)
        # ---- the router (softmax scores, a group judged by its best, identity experts among the outputs) and the sum of
        # the chosen experts' rows (identity experts add the input's row), beside Zufotar's
        total, top = s["experts"] + s["identity"], s["top"]
        logits = [rand(tokens, total + 8, dtype=f32) for _ in range(4)]
        correction = rand(total, dtype=f32, scale=0.05)
        ids = torch.empty(tokens, top, device=device, dtype=i32)
        weights = torch.empty(tokens, top, device=device, dtype=f32)
        route_bytes = tokens * (total * 4 + top * 8)
        for kind, groups, name in (("softmax", "max", "moe_route_softmax_best_of_group"), ("sigmoid", "top2", "zufotar_moe_route")):
            calls = [lambda l=l: kernels.moe_route(l, correction, False, ids, weights, None, total, top, s["groups"][0],
                                                   s["groups"][1], 2.5, score=kind, group_score=groups) for l in logits]
            table[f"{label}_{name}"] = timed(calls, route_bytes, hbm)
        packs = copies(lambda: (rand(tokens * top, width, dtype=f32), rand(tokens, width, dtype=f32), rand(tokens, width, dtype=f32)),
                       tokens * width * 4 * (top + 2))
        x = rand(tokens, width)
        combine_bytes = tokens * width * 4 * (top + 3)
        calls = [lambda p=p: kernels.moe_combine(p[1], p[0], weights, p[2], None, overwrite=True, ids=ids,
                                                 real_experts=s["experts"], identity_rows=x) for p in packs]
        table[f"{label}_moe_combine_with_identity_experts"] = timed(calls, combine_bytes - tokens * width * 4, hbm)
        calls = [lambda p=p: kernels.moe_combine(p[1], p[0], weights, p[2], None) for p in packs]
        table[f"{label}_zufotar_moe_combine"] = timed(calls, combine_bytes, hbm)
    return table


def doderax_config(s: dict) -> dict:
    delta = {"heads": s["heads"], "kv_heads": s["heads"], "dim": s["dim"], "vdim": s["dim"], "conv": 4,
             "decay_rank": 64, "gate_rank": 64}
    left = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"], "scale": s["dim"] ** -0.5,
            "rot": {"dims": s["dim"] // 2, "base": 1000000.0}, "mask": {"size": s["window"], "keep_first": s["keep_first"]}}
    right = {"heads": s["heads"], "kv_heads": s["heads"] // 2, "dim": s["dim"], "vdim": s["dim"], "conv": 4}
    mlp = {"kind": "dense", "ff": s["ff"]}
    layers = [{"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp} if index % 4 == 3 else
              {"type": "channel_delta", "mixer": delta, "mlp": mlp} for index in range(s["layers"])]
    return {"architecture": "Doderax", "vocab": s["vocab"], "width": s["width"], "logit_scale": 1.0,
            "norm": {"eps": 1e-6}, "embedding": {"bigram": {"buckets": 65521, "mul_prev": 8191, "mul_cur": 131}},
            "layers": layers}


def dense_config(s: dict) -> dict:
    """The dense SwiGLU decoder of the same width, depth and heads; its three feed-forward matrices hold what the
    design's two hold."""
    inter = -(-(2 * s["ff"] // 3) // 128) * 128
    return {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": s["width"],
            "intermediate_size": inter, "num_hidden_layers": s["layers"], "num_attention_heads": s["heads"],
            "num_key_value_heads": s["kv_heads"], "head_dim": s["dim"], "vocab_size": s["vocab"],
            "max_position_embeddings": 16384, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
            "tie_word_embeddings": False, "hidden_act": "silu"}


def run(args, peaks: dict) -> dict:
    import numpy as np
    import torch

    from libmir_b200 import CacheConfig, CudaConfig, Library, RuntimeConfig, SchedulerConfig, StepEntry, kernels
    from libmir_b200.sampling import RequestSampler

    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    rng = np.random.default_rng(0)
    hbm, flops_peak = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    steps, warmup = args.steps, max(args.warmup, 3)
    bf16, f32, i32 = torch.bfloat16, torch.float32, torch.int32

    def events():
        return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def model_numbers(config, vocab):
        pages = BATCH * (-(-(PROMPT + steps + warmup + 64) // PAGE)) + 64
        runtime = RuntimeConfig(kv_cache=CacheConfig(block_size=PAGE, block_count=pages),
                                scheduler=SchedulerConfig(max_batch_requests=BATCH, max_batch_tokens=8192,
                                                          prefill_chunk_tokens=4096),
                                cuda=CudaConfig(decode_graphs=True), dtype="bfloat16")
        model = Library(runtime).load_random(config, seed=0)
        for buffer in model.storage.buffers:
            buffer.normal_(0.0, 0.5)
        times = []
        tokens = rng.integers(0, vocab, size=PROMPT).tolist()
        for index in range(7):
            model.admit(f"p{index}")
            start, stop = events()
            torch.cuda.synchronize()
            start.record()
            result = model.step([StepEntry(f"p{index}", tokens, [PROMPT - 1])], [RequestSampler()])
            stop.record()
            torch.cuda.synchronize()
            result.tokens.cpu()
            model.release(f"p{index}")
            if index >= 2:
                times.append(start.elapsed_time(stop))
        prefill_ms = statistics.median(times)
        regions = []
        for _ in range(3):
            ids = []
            for index in range(BATCH):
                sequence = model.cache.admit(f"d{index}")
                model.cache.grow(sequence, PROMPT)
                model.cache.commit(sequence, PROMPT)
                sequence.last_token = 1                        # (the cache is synthetic: any token stands before)
                ids.append(f"d{index}")
            samplers = [RequestSampler() for _ in ids]
            entries = [StepEntry(i, [int(t)], [0]) for i, t in zip(ids, rng.integers(0, vocab, size=BATCH))]
            out = model.decode_many(entries, samplers, warmup)
            entries = [StepEntry(i, [int(t)], [0]) for i, t in zip(ids, out[-1].tolist())]
            torch.cuda.synchronize()
            start, stop = events()
            start.record()
            model.decode_many(entries, samplers, steps)
            stop.record()
            torch.cuda.synchronize()
            regions.append(start.elapsed_time(stop) / steps)
            for request_id in ids:
                model.release(request_id)
        decode_ms = statistics.median(regions)
        weight_bytes = model.decoder.weight_bytes_per_step()
        state_bytes = sum(t.numel() * t.element_size() // t.shape[0]
                          for held in model.storage.states.values()
                          for t in (held if isinstance(held, tuple) else (held,)))
        numbers = {"prefill_ms": round(prefill_ms, 3), "prefill_tokens_per_s": round(PROMPT * 1e3 / prefill_ms),
                   "decode_ms_per_step": round(decode_ms, 4), "decode_tokens_per_s": round(BATCH * 1e3 / decode_ms),
                   "weight_gb": round(weight_bytes / 1e9, 3), "state_mb_per_request": round(state_bytes / 1e6, 2)}
        model.unload()
        return numbers

    def timed(calls, work, peak, launches=24, repeats=5):
        for call in calls[:2]:
            call()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for index in range(launches):
                calls[index % len(calls)]()
        graph.replay()
        torch.cuda.synchronize()
        times = []
        for _ in range(repeats):
            start, stop = events()
            start.record()
            graph.replay()
            stop.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(stop) * 1e3 / launches)
        us = statistics.median(times)
        del graph                                   # (freed here, not by the collector during some later capture)
        gc.collect()
        return [round(us, 2), round(work / (us * 1e-6) / peak, 4)]

    def copies(make, bytes_each):
        return [make() for _ in range(max(2, min(24, -(-(300 << 20) // max(bytes_each, 1)))))]

    def kernel_table(s):
        heads, kv_heads, dim, width, ff = s["heads"], s["kv_heads"], s["dim"], s["width"], s["ff"]
        table = {}
        rand = lambda *shape, dtype=bf16, scale=1.0: (torch.randn(*shape, device=device, dtype=f32) * scale).to(dtype)
        for label, rows, portion in ((f"prefill_{PROMPT}", 1, PROMPT), (f"decode_b{BATCH}", BATCH, 1)):
            tokens = rows * portion
            starts = torch.arange(0, tokens + 1, portion, dtype=i32, device=device)
            row_of = torch.arange(tokens, dtype=i32, device=device) // portion
            positions = torch.full((tokens,), PROMPT, dtype=i32, device=device)
            # the recurrence: state [slots, H, V, D] read and written once per step; 4 D V multiply-adds per token and head
            for per_channel, name in ((True, "delta_rule_channel"), (False, "delta_rule_head")):
                decay_width = heads * dim if per_channel else heads
                packs = copies(lambda: (torch.zeros(rows, heads, dim, dim, device=device, dtype=f32),
                                        rand(tokens, 3 * heads * dim, dtype=f32, scale=0.1)),
                               rows * heads * dim * dim * 4)
                beta = torch.rand(tokens, heads, device=device, dtype=f32)
                decay = torch.rand(tokens, decay_width, device=device, dtype=f32) * 0.5 + 0.5
                out = torch.empty(tokens, heads * dim, device=device, dtype=f32)
                slots = torch.arange(rows, dtype=i32, device=device)
                calls = [lambda p=p: kernels.delta_rule_scan(p[1], beta, decay, p[0], starts, slots, positions, out, heads,
                                                             heads, dim, dim) for p in packs]
                state_bytes = rows * heads * dim * dim * 4 * 2 + tokens * (3 * heads * dim + decay_width + heads * dim) * 4
                if portion == 1:
                    table[f"{label}_{name}"] = timed(calls, state_bytes, hbm)
                else:   # a prompt: the state stays in registers; the work is 32-bit multiply-adds, no tensor cores
                    table[f"{label}_{name}"] = timed(calls, 8.0 * tokens * heads * dim * dim, flops_peak) + ["of the bf16 tensor peak; the kernel is 32-bit FMA, one token after the other"]
                # the parallel pass before it: convolution, unit vectors, gates
                raw = rand(tokens, 3 * heads * dim + 64)
                conv_w = rand(3 * heads * dim, 4)
                conv_tail = torch.zeros(rows, 3, 3 * heads * dim, device=device, dtype=f32)
                beta_raw = rand(tokens, heads)
                decay_raw = rand(tokens, decay_width, dtype=f32 if per_channel else bf16)
                bias, a_log = rand(decay_width, dtype=f32), rand(heads, dtype=f32, scale=0.3)
                prepared = [torch.empty(tokens, 3 * heads * dim, device=device, dtype=f32) for _ in range(4)]
                decay_out = torch.empty(tokens, decay_width, device=device, dtype=f32)
                calls = [lambda o=o: kernels.delta_rule_prepare(raw[:, :3 * heads * dim], conv_w, conv_tail, beta_raw, decay_raw,
                                                                bias, a_log, row_of, starts, slots, positions, o, beta,
                                                                decay_out, heads, heads, dim, dim) for o in prepared]
                moved = tokens * (3 * heads * dim * 6 + decay_width * 8)
                table[f"{label}_{name}_prepare"] = timed(calls, moved, hbm)
            channels = 3 * heads * dim
            packs = copies(lambda: rand(tokens, channels + 64), tokens * channels * 2)
            weight = rand(channels, 4)
            tail = torch.zeros(rows, 3, channels, device=device, dtype=f32)
            out = torch.empty(tokens, channels, device=device, dtype=f32)
            slots = torch.arange(rows, dtype=i32, device=device)
            calls = [lambda p=p: kernels.short_conv_silu(p[:, :channels], weight, tail, row_of, starts, slots, positions, out)
                     for p in packs]
            table[f"{label}_short_conv_silu"] = timed(calls, tokens * channels * 6 + rows * 3 * channels * 8, hbm)
            packs = copies(lambda: (rand(tokens, heads * dim, dtype=f32), rand(tokens, heads * dim)), tokens * heads * dim * 6)
            norm_weight = rand(dim, dtype=f32)
            out16 = torch.empty(tokens, heads * dim, device=device, dtype=bf16)
            calls = [lambda p=p: kernels.gated_head_norm(p[0], p[1], norm_weight, out16, heads, dim, 1e-6, True) for p in packs]
            table[f"{label}_gated_head_norm"] = timed(calls, tokens * heads * dim * 8, hbm)
            packs = copies(lambda: (rand(tokens, width, dtype=f32), rand(tokens, width, dtype=f32), rand(tokens, width, dtype=f32)),
                           tokens * width * 12)
            w_a, w_b = rand(width, dtype=f32), rand(width, dtype=f32)
            calls = [lambda p=p: kernels.add_normed_branches([p[0], p[1]], [w_a, w_b], p[2], 1e-6, 0.5) for p in packs]
            table[f"{label}_add_normed_branches"] = timed(calls, tokens * width * 16, hbm)
            packs = copies(lambda: rand(tokens, ff), tokens * ff * 2)
            calls = [lambda p=p: kernels.gelu_tanh(p) for p in packs]
            table[f"{label}_gelu_tanh"] = timed(calls, tokens * ff * 4, hbm)
            # the dense decoder's elementwise kernels for comparison
            packs = copies(lambda: rand(tokens, width, dtype=f32), tokens * width * 4)
            out_w = torch.empty(tokens, width, device=device, dtype=bf16)
            calls = [lambda p=p: kernels.rms_norm(p, w_a, 1e-6, out_w) for p in packs]
            table[f"{label}_dense_rms_norm"] = timed(calls, tokens * width * 6, hbm)
            inter = ff * 2 // 3 // 128 * 128
            packs = copies(lambda: rand(tokens, 2 * inter), tokens * inter * 4)
            out_i = torch.empty(tokens, inter, device=device, dtype=bf16)
            calls = [lambda p=p: kernels.silu_mul(p, out_i) for p in packs]
            table[f"{label}_dense_silu_mul"] = timed(calls, tokens * inter * 6, hbm)
            # attention: a window with kept first keys (the tile kernel) beside the dense decoder's kernels, same sizes
            context = PROMPT if portion > 1 else PROMPT + 1
            pages_per_row = -(-(context + PAGE) // PAGE)
            cache_rows = rows * pages_per_row * PAGE
            layers = max(2, min(24, -(-(300 << 20) // (cache_rows * kv_heads * dim * 4))))
            k_cache = [rand(cache_rows, kv_heads, dim, scale=0.5) for _ in range(layers)]
            v_cache = [rand(cache_rows, kv_heads, dim, scale=0.5) for _ in range(layers)]
            block_table = torch.arange(rows * pages_per_row, dtype=i32, device=device).view(rows, pages_per_row).contiguous()
            contexts = torch.full((rows,), context, dtype=i32, device=device)
            q_positions = torch.full((tokens,), context - 1, dtype=i32, device=device)
            qkv = rand(tokens, (heads + 2 * kv_heads) * dim, scale=0.3)
            mixed = torch.empty(tokens, heads * dim, device=device, dtype=bf16)
            window = s["window"]
            scale = dim ** -0.5
            calls = [lambda k=k, v=v: kernels.prefill_attention(qkv, mixed, k, v, block_table, starts, contexts, PAGE, heads,
                                                                 kv_heads, dim, scale, window,
                                                                 keep_first=s["keep_first"]) for k, v in zip(k_cache, v_cache)]
            if portion > 1:
                visible = sum(min(p + 1, window) for p in range(PROMPT))
                flops = 4.0 * visible * dim * heads
                table[f"{label}_attention_window_kept"] = timed(calls, flops, flops_peak)
                calls = [lambda k=k, v=v: kernels.prefill_attention(qkv, mixed, k, v, block_table, starts, contexts, PAGE,
                                                                     heads, kv_heads, dim, scale, window) for k, v in zip(k_cache, v_cache)]
                table[f"{label}_dense_attention_window"] = timed(calls, flops, flops_peak)
                calls = [lambda k=k, v=v: kernels.prefill_attention(qkv, mixed, k, v, block_table, starts, contexts, PAGE,
                                                                     heads, kv_heads, dim, scale, None) for k, v in zip(k_cache, v_cache)]
                table[f"{label}_dense_attention_full"] = timed(calls, 4.0 * (PROMPT * (PROMPT + 1) / 2) * dim * heads, flops_peak)
            else:
                key_bytes = rows * min(window, context) * kv_heads * dim * 2 * 2
                partition, count, floats = kernels.decode_attention_kept_plan(rows, heads, dim, context)
                scratch = torch.empty(max(floats, 1), device=device, dtype=f32)
                numbering = torch.empty(rows, device=device, dtype=i32)
                calls = [lambda k=k, v=v: kernels.decode_attention(qkv, mixed, k, v, block_table, q_positions, PAGE, heads,
                                                                    kv_heads, dim, scale, window, partition, count, scratch,
                                                                    keep_first=s["keep_first"], numbering=numbering)
                         for k, v in zip(k_cache, v_cache)]
                table[f"{label}_attention_window_kept"] = timed(calls, key_bytes, hbm)
                for span, name in ((window, "dense_attention_window"), (None, "dense_attention_full")):
                    partition, count, floats = kernels.decode_attention_plan(rows, heads, kv_heads, dim, PAGE, context)
                    scratch = torch.empty(max(floats, 1), device=device, dtype=f32)
                    calls = [lambda k=k, v=v: kernels.decode_attention(qkv, mixed, k, v, block_table, q_positions, PAGE, heads,
                                                                        kv_heads, dim, scale, span, partition, count,
                                                                        scratch if floats else None)
                             for k, v in zip(k_cache, v_cache)]
                    read = rows * (min(span, context) if span else context) * kv_heads * dim * 2 * 2
                    table[f"{label}_{name}"] = timed(calls, read, hbm)
        return table

    if args.design == "zufotar":
        rand = lambda *shape, dtype=bf16, scale=1.0: (torch.randn(*shape, device=device, dtype=f32) * scale).to(dtype)
        tools = {"timed": timed, "copies": copies, "rand": rand, "device": device, "hbm": hbm, "flops_peak": flops_peak}
        report = {}
        for name in [n for n in ZUFOTAR_SIZES if args.design_sizes in ("all", n)]:
            s = ZUFOTAR_SIZES[name]
            entry = {"sizes": s}
            if not args.skip_points:
                entry["kernels_us_and_fraction_of_roofline"] = zufotar_kernel_table(s, tools)
                torch.cuda.empty_cache()
            beside = dict(s, layers=s["runs"])
            entry["zufotar"] = model_numbers(zufotar_config(s), s["vocab"])
            entry["doderax"] = model_numbers(doderax_config(beside), s["vocab"])
            entry["dense_swiglu"] = model_numbers(dense_config(beside), s["vocab"])
            report[name] = entry
        return report
    if args.design == "gumazen":
        rand = lambda *shape, dtype=bf16, scale=1.0: (torch.randn(*shape, device=device, dtype=f32) * scale).to(dtype)
        tools = {"timed": timed, "copies": copies, "rand": rand, "device": device, "hbm": hbm, "flops_peak": flops_peak}
        report = {}
        for name in [n for n in GUMAZEN_SIZES if args.design_sizes in ("all", n)]:
            s = GUMAZEN_SIZES[name]
            entry = {"sizes": s}
            if not args.skip_points:
                entry["kernels_us_and_fraction_of_roofline"] = gumazen_kernel_table(s, tools)
                torch.cuda.empty_cache()
            entry["gumazen"] = model_numbers(gumazen_config(s), s["vocab"])
            entry["zufotar"] = model_numbers(zufotar_config(ZUFOTAR_SIZES[name]), s["vocab"])
            entry["dense_swiglu"] = model_numbers(dense_config(dict(DESIGN_SIZES[name], layers=s["runs"])), s["vocab"])
            report[name] = entry
        return report
    if args.design == "dalesun":
        rand = lambda *shape, dtype=bf16, scale=1.0: (torch.randn(*shape, device=device, dtype=f32) * scale).to(dtype)
        tools = {"timed": timed, "copies": copies, "rand": rand, "device": device, "hbm": hbm, "flops_peak": flops_peak}
        report = {}
        for name in [n for n in DALESUN_SIZES if args.design_sizes in ("all", n)]:
            s = DALESUN_SIZES[name]
            entry = {"sizes": s}
            if not args.skip_points:
                entry["kernels_us_and_fraction_of_roofline"] = dalesun_kernel_table(s, tools)
                torch.cuda.empty_cache()
            entry["dalesun"] = model_numbers(dalesun_config(s), s["vocab"])
            entry["doderax"] = model_numbers(doderax_config(s), s["vocab"])
            entry["dense_swiglu"] = model_numbers(dense_config(s), s["vocab"])
            report[name] = entry
        return report
    chosen = [name for name in DESIGN_SIZES if args.design_sizes in ("all", name)]
    report = {}
    for name in chosen:
        s = DESIGN_SIZES[name]
        entry = {"sizes": s}
        if not args.skip_points:
            entry["kernels_us_and_fraction_of_roofline"] = kernel_table(s)
        entry["doderax"] = model_numbers(doderax_config(s), s["vocab"])
        entry["dense_swiglu"] = model_numbers(dense_config(s), s["vocab"])
        report[name] = entry
    return report
