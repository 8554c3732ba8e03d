"""Gumazen on the GPU against the plain implementation (tests/plain_gumazen.py): every mechanism's kernel alone, then
whole models through the engine's step function, cache manager and scheduler: prompts whole, token by token, in
portions down to two tokens, in batches of unequal requests, with pages and slots that change hands, with keys far
away, at page borders and on either side of a window's edge, in long decoding, and greedy generation through the
entry point."""

import json
import math

import numpy as np
import pytest
import torch

import plain_gumazen as plain
from gumazen_configs import ALL, PAGE_SIZES, make_folder, random_config
from helpers import TOL, Trace, random_ids, run_trace

pytestmark = pytest.mark.gpu
F64 = torch.float64
BF16 = torch.bfloat16
DTYPES = [(torch.float32, 2e-6), (torch.bfloat16, 8e-3)]


def device():
    return torch.device("cuda", 0)


def close(got, want, tol, what=""):
    got = got.detach().double().cpu() if isinstance(got, torch.Tensor) else torch.as_tensor(got, dtype=F64)
    want = want.detach().double().cpu() if isinstance(want, torch.Tensor) else torch.as_tensor(want, dtype=F64)
    error = (got - want).abs().max().item()
    bound = tol * max(1.0, want.abs().max().item())
    assert math.isfinite(error) and error <= bound, f"{what}: max |diff| {error:.3e} > {bound:.3e}"


def relative_error(got, want):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    return np.sqrt(((got - want) ** 2).mean(-1)) / np.sqrt((want ** 2).mean(-1))


def close_logits(got, want, dtype, what=""):
    """Logits [positions, vocab] of a whole model, judged by each position's relative root-mean-square error.
    float32: every position within 2e-4.  bfloat16: nine in ten within the tolerance and all but three in a hundred
    within five times it: two experts whose choice scores lie closer together than the rounding of the router's input
    may be chosen differently by the engine and the 64-bit implementation at that one token.  A key missed or seen at
    a window's edge, a sink, a stream, a bucket or an expert left out is an error of order one at most positions."""
    relative = relative_error(got, want)
    assert np.isfinite(relative).all(), f"{what}: not finite"
    if dtype == "float32":
        assert relative.max() <= 2e-4, f"{what}: {relative.max():.3e} at position {int(relative.argmax())}"
    else:
        assert np.quantile(relative, 0.9) <= TOL[dtype] and (relative <= 5 * TOL[dtype]).mean() >= 0.97, \
            f"{what}: relative error of positions: 90% {np.quantile(relative, 0.9):.3e}, max {relative.max():.3e}"


def on_device(tensor, dtype=None):
    return tensor.to(device=device(), dtype=dtype or tensor.dtype).contiguous()


def ints(values):
    return torch.as_tensor(np.asarray(values, dtype=np.int32), device=device())


# ------------------------------------------------------------------------------ norms and streams
@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("width", [50, 96, 2304])
def test_layer_norm_plain_gathered_and_over_a_mix_of_streams(dtype, tol, width):
    from libmir_b200 import kernels
    generator = torch.Generator().manual_seed(width)
    x = torch.randn(9, 3, width, generator=generator, dtype=F64) * 3.0 + 1.5
    weight, bias = torch.randn(width, generator=generator, dtype=F64), torch.randn(width, generator=generator, dtype=F64)
    read = torch.tensor([0.7, -1.2, 0.4], dtype=F64)
    rows = [7, 0, 3, 3]
    single = on_device(x[:, 0].float())
    out = torch.empty(9, width, dtype=dtype, device=device())
    kernels.layer_norm(single, on_device(weight.float()), on_device(bias.float()), 1e-5, out)
    close(out, plain.layer_norm(single.double().cpu(), weight.float(), bias.float(), 1e-5), tol, "plain rows")
    out = torch.empty(len(rows), width, dtype=dtype, device=device())
    kernels.layer_norm(single, on_device(weight.float()), on_device(bias.float()), 1e-5, out, rows=ints(rows))
    close(out, plain.layer_norm(single.double().cpu()[rows], weight.float(), bias.float(), 1e-5), tol, "gathered rows")
    streams = on_device(x.float())
    mixed = (read.float().double()[None, :, None] * streams.double().cpu()).sum(1)
    out = torch.empty(9, width, dtype=dtype, device=device())
    kernels.layer_norm(streams, on_device(weight.float()), on_device(bias.float()), 1e-5, out, read=on_device(read.float()))
    close(out, plain.layer_norm(mixed, weight.float(), bias.float(), 1e-5), 4 * tol, "a mix of streams")


@pytest.mark.parametrize("count", [1, 2, 4, 7])
def test_streams_are_spread_updated_all_at_once_and_summed(count):
    from libmir_b200 import kernels
    generator = torch.Generator().manual_seed(count)
    tokens, width = 11, 52
    x = torch.randn(tokens, width, generator=generator)
    mix, write = torch.randn(count, count, generator=generator), torch.randn(count, generator=generator)
    branch = torch.randn(tokens, width, generator=generator)
    streams = torch.empty(tokens, count, width, device=device())
    kernels.streams_spread(on_device(x), streams)
    assert torch.equal(streams.cpu(), x[:, None, :].expand(tokens, count, width))
    start = torch.randn(tokens, count, width, generator=generator)
    streams = on_device(start)
    kernels.streams_write(streams, on_device(branch), on_device(mix), on_device(write))
    want = torch.einsum("st,xsw->xtw", mix.double(), start.double()) + write.double()[None, :, None] * branch.double()[:, None, :]
    close(streams, want, 2e-6, "streams after a sublayer")
    total = torch.empty(tokens, width, device=device())
    kernels.streams_sum(streams, total)
    close(total, streams.double().cpu().sum(1), 2e-6, "sum of the streams")


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("count,width", [(1, 52), (2, 96), (3, 50), (4, 2304), (5, 64), (7, 33), (8, 128), (16, 40)])
def test_the_update_of_the_streams_also_norms_the_next_readers_mix(dtype, tol, count, width):
    """One kernel: the streams after a sublayer as streams_write leaves them, and the layer norm of the next reader's
    mix of them; every count with a kernel of its own and the general one, widths with and without 16-byte rows."""
    from libmir_b200 import kernels
    generator = torch.Generator().manual_seed(count * 1000 + width)
    tokens = 10
    start = torch.randn(tokens, count, width, generator=generator) * 2.0 + 0.5
    branch = torch.randn(tokens, width, generator=generator)
    mix, write = torch.eye(count) + 0.4 * torch.randn(count, count, generator=generator), torch.randn(count, generator=generator)
    read = torch.randn(count, generator=generator)
    weight, bias = torch.randn(width, generator=generator), torch.randn(width, generator=generator)
    streams = on_device(start)
    out = torch.empty(tokens, width, dtype=dtype, device=device())
    kernels.streams_write_norm(streams, on_device(branch), on_device(mix), on_device(write), on_device(read),
                               on_device(weight), on_device(bias), 1e-5, out)
    want = torch.einsum("st,xsw->xtw", mix.double(), start.double()) + write.double()[None, :, None] * branch.double()[:, None, :]
    close(streams, want, 2e-6, "streams after a sublayer")
    mixed = (read.double()[None, :, None] * want).sum(1)
    close(out, plain.layer_norm(mixed, weight, bias, 1e-5), 8 * tol, "the next reader's normed mix")
    twice = on_device(start)
    kernels.streams_write(twice, on_device(branch), on_device(mix), on_device(write))
    assert torch.equal(twice, streams), "the same streams as the update alone leaves"
    # without a norm: the mix itself; with factors of one, the sum that streams_sum gives, bit for bit
    again, total, summed = on_device(start), torch.empty(tokens, width, device=device()), torch.empty(tokens, width, device=device())
    kernels.streams_write_norm(again, on_device(branch), on_device(mix), on_device(write), torch.ones(count, device=device()),
                               None, None, 0.0, total)
    kernels.streams_sum(again, summed)
    assert torch.equal(again, streams) and torch.equal(total, summed)


# ------------------------------------------------------------------------------ q/k treatment
@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,rotary,span,weighted,after", [
    (6, 2, 32, 16, 16, "projection", True, False), (4, 1, 64, 64, 24, "head", False, True),
    (3, 3, 20, 12, 0, "projection", True, False), (2, 1, 128, 128, 128, "head", False, True),
    (1, 1, 16, 16, 16, "head", True, False), (2, 2, 8, 24, 8, None, False, False),
    (4, 1, 64, 64, 32, "projection", True, False), (4, 2, 64, 64, 0, "projection", True, False),
    (3, 1, 128, 128, 48, "head", True, False), (5, 5, 32, 32, 16, "head", False, True),
    (9, 3, 128, 128, 64, "projection", True, False), (2, 1, 256, 256, 256, "head", True, True)])
@pytest.mark.parametrize("tokens", [13, 300])
def test_queries_and_keys_are_normed_rotated_and_stored(dtype, tol, tokens, heads, kv_heads, dim, vdim, rotary, span, weighted, after):
    """The norm over a whole projection, per head without weights behind the rotation, per head with weights before
    it, and none; rows with columns behind q, k and v that must stay as they are; a slot of -1 writes nothing.  Few
    and many tokens; heads of 16-byte pieces in bfloat16 (the kernel with wide accesses: the whole head rotated, at
    most half of it, none) and other sizes."""
    from libmir_b200 import kernels
    generator = torch.Generator().manual_seed(dim + heads)
    extra, eps = 8, 1e-5
    q_width, k_width, v_width = heads * dim, kv_heads * dim, kv_heads * vdim
    packed = torch.randn(tokens, q_width + k_width + v_width + extra, generator=generator) * 2.0
    rows = on_device(packed, dtype)
    before = rows.clone()
    positions = [40, 41, 42, 0, 1, 2, 3, 999, 7, 8, 9, 10, 11] + list(range(100, 87 + tokens))
    slots = [5, 6, 7, 20, 21, 22, 23, 2, -1, 30, 31, 32, 33] + list(range(40, 27 + tokens))
    pages = 40 + tokens
    rot = {"dims": rotary, "base": 700.0, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 32}}
    table = on_device(plain.frequencies(rot)) if rotary else None
    per = dim if span == "head" else None
    q_weight = 1.0 + 0.3 * torch.randn(per or q_width, generator=generator) if weighted else None
    k_weight = 1.0 + 0.3 * torch.randn(per or k_width, generator=generator) if weighted else None
    k_pages = torch.full((pages, kv_heads, dim), 77.0, dtype=dtype, device=device())
    v_pages = torch.full((pages, kv_heads, vdim), 77.0, dtype=dtype, device=device())
    kernels.qk_prepare(rows, ints(positions), ints(slots), table, on_device(q_weight) if weighted else None,
                       on_device(k_weight) if weighted else None, k_pages, v_pages, heads, kv_heads, dim, vdim, rotary, eps,
                       span, after_rotation=after)
    source = before.double().cpu()

    def treated(x, count, weight):
        if span == "projection":
            x = plain.unit_rms(x, eps) * weight.double()
        x = x.view(tokens, count, dim)
        if span == "head" and not after:
            x = plain.unit_rms(x, eps) * (weight.double() if weight is not None else 1.0)
        if rotary:
            angles = torch.tensor(positions, dtype=torch.float32)[:, None] * plain.frequencies(rot)[None, :]
            cos, sin = torch.cos(angles.double())[:, None, :], torch.sin(angles.double())[:, None, :]
            half = rotary // 2
            u, v = x[..., :half], x[..., half:rotary]
            x = torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., rotary:]], dim=-1)
        if span == "head" and after:
            x = plain.unit_rms(x, eps) * (weight.double() if weight is not None else 1.0)
        return x
    want_q = treated(source[:, :q_width], heads, q_weight).reshape(tokens, q_width)
    want_k = treated(source[:, q_width:q_width + k_width], kv_heads, k_weight)
    want_v = source[:, q_width + k_width:q_width + k_width + v_width].view(tokens, kv_heads, vdim)
    close(rows[:, :q_width], want_q, tol, "queries in place")
    assert torch.equal(rows[:, q_width:], before[:, q_width:]), "what lies behind the queries is left alone"
    written = [t for t in range(tokens) if slots[t] >= 0]
    close(k_pages[[slots[t] for t in written]], want_k[written], tol, "keys in their pages")
    close(v_pages[[slots[t] for t in written]], want_v[written], tol, "values in their pages")
    untouched = [s for s in range(pages) if s not in slots]
    assert (k_pages[untouched] == 77.0).all() and (v_pages[untouched] == 77.0).all()


# ------------------------------------------------------------------------------ attention
def spread_bias(table, window, farthest):
    """One entry per distance from the bucket rule, a head's entries side by side (the test's own restatement of what
    the part hands to the kernels)."""
    rows, out, n = table.shape[0], [], 0
    while True:
        out.append(plain.distance_bucket(n, rows, farthest))
        n += 1
        if out[-1] == rows - 1 or (window is not None and n >= window):
            break
    return table[out].t().contiguous()          # [heads, distances]


def pool_of(keys, values, page, rng, dtype):
    """Scatter each request's keys and values into a shuffled pool of pages; garbage elsewhere.  Returns the pool
    tensors and the block table [requests, width]."""
    needs = [-(-k.shape[0] // page) for k in keys]
    total = sum(needs) + 5
    order = rng.permutation(total)
    width = max(needs)
    table = np.full((len(keys), width), -1, dtype=np.int32)
    k_pool = torch.full((total * page, keys[0].shape[1], keys[0].shape[2]), 1e4, dtype=torch.float32)
    v_pool = torch.full((total * page, values[0].shape[1], values[0].shape[2]), 1e4, dtype=torch.float32)
    at = 0
    for r, (k, v) in enumerate(zip(keys, values)):
        for p in range(needs[r]):
            page_id = int(order[at]); at += 1
            table[r, p] = page_id
            n = min(page, k.shape[0] - p * page)
            k_pool[page_id * page:page_id * page + n] = k[p * page:p * page + n]
            v_pool[page_id * page:page_id * page + n] = v[p * page:p * page + n]
    return on_device(k_pool, dtype), on_device(v_pool, dtype), ints(table)


ATTENTION_CASES = [
    # dtype, heads, kv_heads, dim, vdim, page, window, softcap, bias rows and farthest, gate per head, sink, path
    (torch.float32, 4, 2, 24, 40, 8, 37, 6.0, (12, 50.0), True, False, "reference"),
    (torch.float32, 3, 1, 16, 16, 16, None, None, None, False, True, "reference"),
    (BF16, 6, 2, 64, 64, 16, 90, 25.0, (28, 110.0), True, False, "reference"),
    (BF16, 4, 2, 64, 64, 4, 50, 8.0, (16, 70.0), True, False, "tiles"),
    (BF16, 2, 2, 128, 128, 16, 70, 20.0, (10, 64.0), True, False, "tiles"),
    (BF16, 8, 1, 64, 64, 8, 33, None, (6, 9.0), False, False, "tiles"),
    (BF16, 4, 4, 128, 128, 32, 200, 3.0, None, True, True, "tiles"),
    (BF16, 4, 2, 128, 128, 16, 160, 12.0, (20, 300.0), True, False, "tiles"),
    (BF16, 2, 1, 128, 128, 8, None, 40.0, (8, 400.0), False, False, "tiles"),
]


@pytest.mark.parametrize("dtype,heads,kv_heads,dim,vdim,page,window,softcap,bias,per_head,sink,path", ATTENTION_CASES)
def test_attention_with_capped_biased_scores_where_keys_at_the_edges_stand_out(dtype, heads, kv_heads, dim, vdim, page,
                                                                              window, softcap, bias, per_head, sink, path):
    """Three requests of unequal lengths in a shuffled pool.  In each, the keys just inside and just outside the last
    queries' windows (or the first token, without a window), and the keys on either side of a page border, are made to
    stand out for their query, the one outside more than the one inside: a window that is one token off, or a page
    read from the wrong place, changes the result entirely.  Prompt portions that start in mid-request and single
    tokens, through the reference kernel and the tensor-core kernels (one and several partitions of the keys)."""
    from libmir_b200 import kernels
    rng = np.random.default_rng(dim + page)
    generator = torch.Generator().manual_seed(dim * 3 + page)
    lengths = [300, 19, 131]
    scale = 1.0 / math.sqrt(dim)
    rel = torch.randn(bias[0], heads, generator=generator) * 1.5 if bias else None
    qs, ks, vs, gates, wants = [], [], [], [], []
    for n in lengths:
        q = torch.randn(n, heads, dim, generator=generator)
        k = torch.randn(n, kv_heads, dim, generator=generator)
        v = torch.randn(n, kv_heads, vdim, generator=generator)
        for query in (n - 1, n - 2, n // 2):
            direction = q[query, 0] / q[query, 0].norm()
            inside = query - (window - 1) if window else 0
            if inside >= 0:
                k[inside, 0] = direction * 9.0
            if window and inside - 1 >= 0:
                k[inside - 1, 0] = direction * 18.0            # just outside: must not be seen
            border = (query // page) * page
            if 0 < border and (not window or query - border < window - 1):
                k[border, 0] += direction * 5.0
                k[border - 1, 0] += direction * 4.0
        q, k, v = (t.to(dtype).double() for t in (q, k, v))
        gate = torch.randn(n, heads if per_head else heads * vdim, generator=generator).to(dtype).double()
        want = plain.attend(q, k, v, scale, window=window, sink=sink, softcap=softcap, rel=rel,
                            farthest=bias[1] if bias else None)
        factor = torch.sigmoid(gate)
        want = want * (factor[:, :, None] if per_head else factor.view(n, heads, vdim))
        qs.append(q); ks.append(k); vs.append(v); gates.append(gate); wants.append(want.reshape(n, heads * vdim))
    k_pool, v_pool, table = pool_of(ks, vs, page, rng, dtype)
    sinks = torch.zeros(heads, device=device()) if sink else None
    spread = on_device(spread_bias(rel, window, bias[1])) if bias else None
    extras = dict(sinks=sinks, gate_per_head=per_head, softcap=softcap, distance_bias=spread)
    tol = 2e-5 if dtype == torch.float32 else 2e-2

    def packed(rows_of):
        """The rows' queries and gates as packed projection rows [q | k v left out: zeros | gate]."""
        q = torch.cat([qs[r][a:b].reshape(b - a, -1) for r, a, b in rows_of])
        gate = torch.cat([gates[r][a:b] for r, a, b in rows_of])
        filler = torch.zeros(q.shape[0], 8, dtype=F64)
        tail = torch.zeros(q.shape[0], -(q.shape[1] + 8 + gate.shape[1]) % 8, dtype=F64)      # rows of 16-byte pieces
        rows = on_device(torch.cat([q, filler, gate, tail], dim=1), dtype)
        return rows, rows[:, q.shape[1] + 8:q.shape[1] + 8 + gate.shape[1]]
    # portions that start in mid-request: the last tokens of every request
    portions = [(0, 150, 300), (1, 0, 19), (2, 64, 131)]
    rows, gate = packed(portions)
    want = torch.cat([wants[r][a:b] for r, a, b in portions])
    counts = [b - a for _, a, b in portions]
    starts = ints(np.concatenate([[0], np.cumsum(counts)]))
    out = torch.zeros(sum(counts), heads * vdim, dtype=dtype, device=device())
    if path == "reference":
        row_of = ints(np.repeat(np.arange(3), counts))
        positions = ints(np.concatenate([np.arange(a, b) for _, a, b in portions]))
        kernels.paged_attention_generic(rows, out, k_pool, v_pool, table, row_of, positions, page, heads, kv_heads, dim,
                                        scale, window, value_dim=vdim, gate=gate, **extras)
    else:
        kernels.prefill_attention(rows, out, k_pool, v_pool, table, starts, ints(lengths), page, heads, kv_heads, dim, scale,
                                  window, tensor_cores=False, gate=gate, **extras)
        if dim == 128 and page % 8 == 0:                        # the tcgen05 kernel takes these sizes
            close(out, want, tol, f"{path}: prompt portions, mma.sync")
            out.zero_()
            kernels.launch_counts(reset=True)
            kernels.prefill_attention(rows, out, k_pool, v_pool, table, starts, ints(lengths), page, heads, kv_heads, dim,
                                      scale, window, tensor_cores=True, gate=gate, **extras)
            assert kernels.launch_counts().get("prefill_attention_tc", 0) == 1
    close(out, want, tol, f"{path}: prompt portions")
    if path == "reference":
        return
    # single tokens: the last token of every request, keys in one partition and in several
    singles = [(r, n - 1, n) for r, n in enumerate(lengths)]
    rows, gate = packed(singles)
    want = torch.cat([wants[r][a:b] for r, a, b in singles])
    positions = ints([n - 1 for n in lengths])
    # (partitions of 512 and 128 keys run the tcgen05 kernel where it takes the sizes, of 64 keys the mma.sync kernel)
    for keys_per_partition in (512, 128, 64):
        with kernels.option("decode_partition_keys", keys_per_partition):
            partition, count, floats = kernels.decode_attention_kept_plan(3, heads, dim, max(lengths))
            scratch = torch.empty(floats, dtype=torch.float32, device=device()) if floats else None
            out = torch.zeros(3, heads * vdim, dtype=dtype, device=device())
            kernels.launch_counts(reset=True)
            kernels.decode_attention(rows, out, k_pool, v_pool, table, positions, page, heads, kv_heads, dim, scale, window,
                                     partition, count, scratch, gate=gate, **extras)
            on_tcgen05 = dim == 128 and page % 8 == 0 and keys_per_partition % 128 == 0
            assert (kernels.launch_counts().get("decode_attention_tc", 0) == 1) == on_tcgen05, kernels.launch_counts()
        close(out, want, tol, f"single tokens, partitions of {keys_per_partition} keys")


# ------------------------------------------------------------------------------ experts
@pytest.mark.parametrize("experts,identity,top,groups,keep", [(10, 6, 5, 4, 3), (6, 2, 3, 4, 2), (1, 0, 1, 1, 1), (3, 3, 3, 6, 6),
                                                              (4, 4, 2, 2, 1), (5, 1, 2, 3, 2), (7, 0, 7, 1, 1)])
def test_router_with_softmax_scores_groups_by_their_best_and_identity_experts(experts, identity, top, groups, keep):
    from libmir_b200 import kernels
    total = experts + identity
    generator = torch.Generator().manual_seed(total * 7 + top)
    tokens = 37
    logits = torch.randn(tokens, total + 3, generator=generator) * 2.0
    correction = torch.randn(total, generator=generator) * 0.3 - 0.2          # choice scores below zero too
    ids = torch.empty(tokens, top, dtype=torch.int32, device=device())
    weights = torch.empty(tokens, top, dtype=torch.float32, device=device())
    kernels.moe_route(on_device(logits), on_device(correction), False, ids, weights, None, total, top, groups, keep, 2.5,
                      score="softmax", group_score="max")
    router = {"top": top, "scale": 2.5, "groups": {"count": groups, "keep": keep}}
    fake = {"p.router": torch.eye(total + 3, dtype=F64)[:total], "p.correction": correction.double()}
    chosen, amounts = plain.route(logits.double(), fake, "p.", router)
    for t in range(tokens):
        assert sorted(ids[t].tolist()) == sorted(chosen[t]), f"token {t}"
        by_id = dict(zip(ids[t].tolist(), weights[t].tolist()))
        for e, w in zip(chosen[t], amounts[t].tolist()):
            assert abs(by_id[e] - w) <= 2e-6 * max(1.0, abs(w))


@pytest.mark.parametrize("dtype,tol", DTYPES)
def test_identity_experts_add_the_input_itself_and_results_can_replace_the_buffer(dtype, tol):
    from libmir_b200 import kernels
    generator = torch.Generator().manual_seed(5)
    tokens, width, top, real = 9, 40, 3, 4
    ids = torch.randint(0, 7, (tokens, top), generator=generator, dtype=torch.int32)
    weights = torch.rand(tokens, top, generator=generator)
    rows = torch.randn(tokens * top, width, generator=generator)
    x = torch.randn(tokens, width, generator=generator).to(dtype)
    shared = torch.randn(tokens, width, generator=generator)
    rows_dev = on_device(rows)
    rows_dev[(ids.view(-1) >= real).to(device())] = float("nan")          # identity slots have no row: never read
    want = torch.zeros(tokens, width, dtype=F64)
    for t in range(tokens):
        for s in range(top):
            source = rows[t * top + s].double() if ids[t, s] < real else x[t].double()
            want[t] += weights[t, s].double() * source
    want += shared.double()
    start = torch.randn(tokens, width, generator=generator)
    for overwrite in (False, True):
        residual = on_device(start)
        kernels.moe_combine(residual, rows_dev, on_device(weights), on_device(shared), None, overwrite=overwrite,
                            ids=on_device(ids), real_experts=real, identity_rows=on_device(x))
        close(residual, want if overwrite else want + start.double(), 2e-6, f"overwrite {overwrite}")


# ------------------------------------------------------------------------------ whole models
def load(folder, dtype, page_size, pages, requests=4, graphs=False):
    from libmir_b200 import CacheConfig, CudaConfig, Library, RuntimeConfig, SchedulerConfig
    runtime = RuntimeConfig(kv_cache=CacheConfig(block_size=page_size, block_count=pages),
                            scheduler=SchedulerConfig(max_batch_requests=requests),
                            cuda=CudaConfig(decode_graphs=graphs), dtype=dtype)
    return Library(runtime).load(folder)


def reference(folder, ids):
    config, weights = plain.read_model(folder)
    return plain.forward(config, weights, list(ids)).numpy()


def feed(model, name, ids, cuts):
    """Feed `ids` in portions of the given sizes (the last repeated), wanting every position; returns logits [n, V]."""
    from libmir_b200 import StepEntry
    model.admit(name)
    out, cursor, turn = [], 0, 0
    while cursor < len(ids):
        size = min(cuts[min(turn, len(cuts) - 1)], len(ids) - cursor)
        result = model.step([StepEntry(name, ids[cursor:cursor + size], range(size))])
        out.append(result.logits.float().cpu().numpy().copy())
        cursor += size
        turn += 1
    model.release(name)
    return np.concatenate(out)


@pytest.mark.parametrize("name", ["A", "D"])
def test_the_residual_after_every_run_of_a_layer(tmp_path, name):
    """One prompt in 32-bit: the sum of the streams after each run of a layer (a repeated layer counts every time)
    against the plain implementation's, so that a fault shows at the run that has it."""
    from libmir_b200 import StepEntry
    config = ALL[name]
    folder = make_folder(tmp_path, config, seed=2, dtype="float32")
    ids = random_ids(np.random.default_rng(1), config["vocab"], 60)
    plain_config, weights = plain.read_model(folder)
    _, want = plain.forward(plain_config, weights, ids, want_layers=True)
    model = load(folder, "float32", PAGE_SIZES[name], 40)
    seen = []
    model.decoder.after_entry = lambda index, streams: seen.append(streams.sum(1).cpu())
    model.admit("x")
    model.step([StepEntry("x", ids, [0])])
    model.decoder.after_entry = None
    assert len(seen) == want.shape[0] == len(plain.layer_order(config))
    for run, (got, expected) in enumerate(zip(seen, want)):
        close(got, expected, 2e-5, f"after layer run {run}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ALL))
def test_whole_prompts_token_by_token_and_portions(tmp_path, name, dtype):
    """A prompt whole; the same token by token from its first token (150 single steps: long decoding, windows that
    pass over decoded tokens, the first tokens of a sequence); in portions of changing size down to two tokens; and
    most of it whole with the rest decoded."""
    config = ALL[name]
    folder = make_folder(tmp_path, config, seed=3, dtype=dtype)
    ids = random_ids(np.random.default_rng(7), config["vocab"], 150)
    want = reference(folder, ids)
    model = load(folder, dtype, PAGE_SIZES[name], 60)
    whole = feed(model, "whole", ids, [len(ids)])
    close_logits(whole, want, dtype, f"{name}/{dtype} whole")
    single = feed(model, "single", ids, [1])
    close_logits(single, want, dtype, f"{name}/{dtype} token by token")
    portions = feed(model, "portions", ids, [2, 3, 1, 7, 2, 16, 5, 2, 33, 1, 2, 9])
    close_logits(portions, want, dtype, f"{name}/{dtype} portions")
    late = feed(model, "late", ids, [118, 1])
    close_logits(late, want, dtype, f"{name}/{dtype} prompt then decoding")
    if dtype == "float32":
        # 32-bit results do not depend on the cut at all: attention reduces a query's keys in an order that depends on
        # its position alone, products and norms reduce in one fixed order, an expert pair's row does not depend on
        # which tile it shares with whom
        assert np.array_equal(whole, single) and np.array_equal(whole, portions) and np.array_equal(whole, late)
    for group in model.cache_stats()["groups"]:
        assert group["free"] == group["pages"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C", "D"])
def test_batches_of_unequal_requests_with_pages_and_slots_that_change_hands(tmp_path, name, dtype):
    """Up to three live requests of unequal lengths, portions of some beside single tokens of others, requests that
    sit a step out, in a pool so small that pages and slots are used again; every request against itself alone."""
    from libmir_b200 import StepEntry
    config = ALL[name]
    folder = make_folder(tmp_path, config, seed=5, dtype=dtype)
    rng = np.random.default_rng(11)
    lengths = [70, 31, 96, 18, 55, 40, 77]
    requests = [random_ids(rng, config["vocab"], n) for n in lengths]
    want = [reference(folder, ids) for ids in requests]
    page = PAGE_SIZES[name]
    model = load(folder, dtype, page, 3 * (-(-96 // page)) + 2, requests=3)
    queue, live, got = list(range(len(requests))), {}, {i: [] for i in range(len(requests))}
    while queue or live:
        while queue and len(live) < 3:
            index = queue.pop(0)
            model.admit(f"r{index}")
            live[index] = 0
        entries, ended = [], []
        for index in list(live):
            cursor, ids = live[index], requests[index]
            if len(live) > 1 and rng.random() < 0.25:
                continue
            decode_from = max(2, len(ids) - 20)
            size = 1 if cursor >= decode_from else min(int(rng.integers(2, 19)), decode_from - cursor)
            entries.append(StepEntry(f"r{index}", ids[cursor:cursor + size], range(size)))
            live[index] = cursor + size
            if live[index] == len(ids):
                ended.append(index)
        if not entries:
            continue
        result = model.step(entries)
        logits, at = result.logits.float().cpu().numpy(), 0
        for entry in entries:
            got[int(entry.request_id[1:])].append(logits[at:at + len(entry.tokens)].copy())
            at += len(entry.tokens)
        for index in ended:
            model.release(f"r{index}")
            del live[index]
        model.cache.check()
    if dtype == "float32":
        for index in range(len(requests)):
            close_logits(np.concatenate(got[index]), want[index], dtype, f"{name}/{dtype} request {index} in a mixed batch")
    else:       # (the share of positions is taken over all requests: the shortest has eighteen)
        close_logits(np.concatenate([np.concatenate(got[index]) for index in range(len(requests))]), np.concatenate(want),
                     dtype, f"{name}/{dtype} requests in mixed batches")
    stats = model.cache_stats()
    for group in stats["groups"]:
        assert group["free"] == group["pages"] and group["reused"] > 0


def test_far_tokens_decide_the_logits_in_prompt_and_in_decoding(tmp_path):
    """Sharp attention without a window (the sink's and the rotated, scaled kind): the last positions depend on keys
    hundreds of tokens back, over many pages; whole, with the last tokens decoded one by one, and in portions."""
    layers = [{"type": "attention", "mlp": None,
               "mixer": {"heads": 2, "kv_heads": 1, "dim": 16, "vdim": 24, "scale": 0.25, "rot": {"dims": 8, "base": 10000.0}}},
              {"type": "attention_3", "mlp": None,
               "mixer": {"heads": 2, "kv_heads": 2, "dim": 16, "vdim": 8, "scale": 0.25,
                         "rot": {"dims": 16, "base": 10000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 128}}}}]
    config = {"architecture": "Gumazen", "vocab": 90, "width": 64, "norm": {"eps": 1e-5}, "streams": 2, "layers": layers}
    ids = random_ids(np.random.default_rng(4), 90, 700)
    for dtype in ("float32", "bfloat16"):
        folder = make_folder(tmp_path / dtype, config, seed=6, dtype=dtype, sharpen=12.0)
        plain_config, weights = plain.read_model(folder)
        want = plain.forward(plain_config, weights, ids).numpy()
        shorter = plain.forward(plain_config, weights, ids[300:]).numpy()
        assert np.abs(shorter[-20:] - want[-20:]).max() > 0.1          # the early tokens matter
        model = load(folder, dtype, 16, 50)
        close_logits(feed(model, "whole", ids, [700]), want, dtype, f"far tokens, whole, {dtype}")
        close_logits(feed(model, "late", ids, [650, 1]), want, dtype, f"far tokens, decoded, {dtype}")
        close_logits(feed(model, "cut", ids, [15, 17, 300, 2, 31]), want, dtype, f"far tokens, portions, {dtype}")


@pytest.mark.parametrize("dim,page", [(24, 8), (64, 4), (128, 16)])
def test_the_windows_edge_and_the_buckets_show_in_the_logits(tmp_path, dim, page):
    """Two windowed layers with capped, biased scores: the plain implementation with a window one token wider or
    narrower, or with another farthest distance of the buckets, gives other logits, and the engine gives the
    configured ones, in a prompt and in decoding (heads of 24 channels run the reference kernel, of 64 and 128 the
    tensor-core kernels in bfloat16)."""
    def model_config(first, second, farthest=(69.0, 30.0)):
        mixer = {"heads": 2, "kv_heads": 1, "dim": dim, "vdim": dim, "scale": 0.5 / math.sqrt(dim), "softcap": 15.0,
                 "bias_rows": 8}
        return {"architecture": "Gumazen", "vocab": 80, "width": 64, "norm": {"eps": 1e-5}, "layers": [
            {"type": "attention_2", "mlp": None, "mixer": dict(mixer, mask={"size": first}, bias_max=farthest[0])},
            {"type": "attention_2", "mlp": None, "mixer": dict(mixer, mask={"size": second}, bias_max=farthest[1])}]}

    def raise_the_last_bucket(tensors):
        # the last bucket of either layer begins two or three keys before its window ends (distances 34.. of 37 and
        # 19.. of 21), and its bias puts most of the weight there: the key at the edge carries a third or a half of it
        for name in ("l0.mix.rel", "l1.mix.rel"):
            table = tensors[name].float()
            table[-1] += 6.0
            tensors[name] = table.to(tensors[name].dtype)
    config = model_config(37, 21)
    ids = random_ids(np.random.default_rng(dim), 80, 120)
    for dtype in ("float32", "bfloat16"):
        folder = make_folder(tmp_path / dtype, config, seed=8, dtype=dtype, sharpen=6.0, edit=raise_the_last_bucket)
        _, weights = plain.read_model(folder)
        want = plain.forward(config, weights, ids).numpy()
        seen = []
        for other in (model_config(38, 21), model_config(36, 21), model_config(37, 22), model_config(37, 20),
                      model_config(37, 21, farthest=(60.0, 30.0)), model_config(37, 21, farthest=(69.0, 24.0))):
            moved = plain.forward(other, weights, ids).numpy()
            seen.append(np.median(relative_error(moved, want)[45:]))
            assert seen[-1] > 0.01                                  # a window one token off, or other buckets, are seen
        model = load(folder, dtype, page, 80)
        for label, cuts in (("whole", [120]), ("decoded", [30, 1]), ("portions", [36, 2, 19, 2, 1, 22])):
            relative = relative_error(feed(model, label, ids, cuts), want)
            if dtype == "float32":
                assert relative.max() <= 2e-4, f"{label}: {relative.max():.3e} at position {int(relative.argmax())}"
            else:
                assert np.median(relative[45:]) <= 0.5 * min(seen) and relative.max() <= 1.5 * TOL[dtype], \
                    f"{label}/{dtype}: median {np.median(relative[45:]):.3e}, max {relative.max():.3e}"


def test_the_tensor_core_kernels_run_the_designs_attention_in_bfloat16(tmp_path):
    """Heads of 64 and 128 channels: prompts and single tokens of all three kinds of attention run the tile kernels
    (heads of 128 channels on tcgen05, of 64 on mma.sync), not the reference kernel."""
    from libmir_b200 import kernels
    for name in ("C", "D"):
        config = ALL[name]
        folder = make_folder(tmp_path / name, config, seed=3, dtype="bfloat16")
        ids = random_ids(np.random.default_rng(2), config["vocab"], 90)
        model = load(folder, "bfloat16", 16, 40)
        kernels.launch_counts(reset=True)
        feed(model, "x", ids, [70, 1])
        counts = kernels.launch_counts()
        assert counts.get("paged_attention_generic", 0) == 0, counts
        tiles, split = ("prefill_attention_tc", "decode_attention_tc") if name == "D" else \
            ("prefill_attention", "decode_attention")                              # heads of 128 channels: tcgen05
        assert counts.get(tiles, 0) > 0 and counts.get(split, 0) > 0, counts
        assert counts.get("qk_prepare", 0) > 0 and counts.get("layer_norm", 0) > 0


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_scheduler(tmp_path, name, graphs):
    """Model.generate_batch (scheduler, sampler, decode steps as captured graphs or not) against the plain
    implementation choosing greedily; float32, so that equal choices are expected wherever the best two logits are
    not closer than the tolerance."""
    from libmir_b200 import GenerationOverrides, GenerationRequest
    config = ALL[name]
    folder = make_folder(tmp_path, config, seed=9, dtype="float32")
    plain_config, weights = plain.read_model(folder)
    rng = np.random.default_rng(2)
    prompts = [random_ids(rng, config["vocab"], n) for n in (5, 23, 1)]
    model = load(folder, "float32", PAGE_SIZES[name], 48, graphs=graphs)
    outputs = model.generate_batch([GenerationRequest(p, GenerationOverrides(max_tokens=12, ignore_eos=True))
                                    for p in prompts])
    for prompt, output in zip(prompts, outputs):
        assert len(output.token_ids) == 12
        ids = list(prompt)
        for token in output.token_ids:
            logits = plain.forward(plain_config, weights, ids)[-1]
            best = int(torch.argmax(logits))
            assert token == best or float(logits[best] - logits[token]) < 1e-4, \
                f"{name}: the engine chose {token}, the plain implementation {best}"
            ids.append(token)
    if graphs:
        assert model.runner._graphs is not None and len(model.runner._graphs.graphs) > 0


@pytest.mark.parametrize("name", ["C", "D"])
def test_decode_steps_replayed_from_captured_graphs_in_bfloat16(tmp_path, name):
    """Two requests decoded together through captured graphs in bfloat16 (heads of 64 and 128 channels, a window that
    passes over the decoded tokens, the experts' grouped products inside a replayed graph): the teacher-forced logits
    of every step against the plain implementation."""
    from libmir_b200 import StepEntry, kernels
    from libmir_b200.sampling import RequestSampler
    config = ALL[name]
    folder = make_folder(tmp_path, config, seed=8, dtype="bfloat16")
    rng = np.random.default_rng(5)
    requests = {"a": random_ids(rng, config["vocab"], 100), "b": random_ids(rng, config["vocab"], 87)}
    want = {key: reference(folder, ids) for key, ids in requests.items()}
    prompt = {"a": 21, "b": 8}
    model = load(folder, "bfloat16", PAGE_SIZES[name], 80, graphs=True)
    got = {key: [] for key in requests}
    for key, ids in requests.items():
        model.admit(key)
        result = model.step([StepEntry(key, ids[:prompt[key]], range(prompt[key]))])
        got[key].append(result.logits.float().cpu().numpy().copy())
    for step in range(79):
        entries = [StepEntry(key, [ids[prompt[key] + step]], [0]) for key, ids in requests.items()]
        result = model.step(entries, [RequestSampler() for _ in entries])
        logits = result.logits.float().cpu().numpy()
        for row, key in enumerate(requests):
            got[key].append(logits[row:row + 1].copy())
    assert model.runner._graphs is not None and len(model.runner._graphs.graphs) > 0
    everything = np.concatenate([np.concatenate(got[key]) for key in requests])
    wanted = np.concatenate([want[key][:prompt[key] + 79] for key in requests])
    close_logits(everything, wanted, "bfloat16", "decode steps from captured graphs")
    assert kernels.tensor_core_linear_error() == 0 and kernels.decode_attention_error() == 0


def test_trace_runner_picks_the_design_by_its_configuration(tmp_path):
    """bin/trace_run as a user runs it: the model class comes from config.json; prompts in portions, decoded tokens,
    a pool that holds less than all requests together."""
    config = ALL["A"]
    folder = make_folder(tmp_path / "model", config, seed=4, dtype="bfloat16")
    (folder / "config.json").write_text(json.dumps(dict(config, vocab_size=config["vocab"])))   # (helpers read this key)
    rng = np.random.default_rng(3)
    requests = {f"q{i}": random_ids(rng, config["vocab"], n) for i, n in enumerate((100, 64, 37))}
    want = {name: reference(folder, ids) for name, ids in requests.items()}
    for dtype, extra in (("bfloat16", []), ("float32", []), ("bfloat16", ["--decode-graphs"])):
        trace = Trace()
        for name, ids in requests.items():
            trace.step([(name, ids[:len(ids) - 10], [0, len(ids) - 11])])
            for position in range(len(ids) - 10, len(ids)):
                trace.step([(name, ids[position:position + 1], [0])], end=[name] if position == len(ids) - 1 else [])
        results = run_trace(folder, dtype, trace, tmp_path / f"out-{dtype}-{len(extra)}", max_tokens=128,
                            extra_args=["--page-size", "8"] + extra)
        got = np.stack([results[index][row] for index, rows in enumerate(trace.expect) for row in range(len(rows))])
        wanted = np.stack([want[name][position] for rows in trace.expect for name, position in rows])
        close_logits(got, wanted, dtype, f"trace {dtype} {extra}")


def test_generate_command_line(tmp_path):
    """bin/generate on a model folder of the design: two prompts as one batch, greedy, against the plain
    implementation."""
    import subprocess
    import sys
    from helpers import ROOT
    config = ALL["D"]
    folder = make_folder(tmp_path / "model", config, seed=12, dtype="float32")
    plain_config, weights = plain.read_model(folder)
    command = [sys.executable, str(ROOT / "bin" / "generate"), str(folder), "--dtype", "float32", "--block-size", "8",
               "--block-count", "64", "--max-tokens", "6", "--ignore-eos"]
    done = subprocess.run(command + ["--prompt-ids", "5,9,80,33;7", "--json"], capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-3000:]
    outputs = [json.loads(line) for line in done.stdout.splitlines() if line.startswith("{")]
    assert len(outputs) == 2
    for prompt, output in zip(([5, 9, 80, 33], [7]), outputs):
        ids = list(prompt)
        for token in output["token_ids"]:
            logits = plain.forward(plain_config, weights, ids)[-1]
            best = int(torch.argmax(logits))
            assert token == best or float(logits[best] - logits[token]) < 1e-4
            ids.append(token)


@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_at_random(tmp_path, seed):
    """Sizes nobody chose: a prompt whole, token by token, in portions and as a prompt followed by decoding, in both
    dtypes, against the plain implementation (32-bit: every position within 2e-4 of its logits' root mean square and
    the same bits under every cut; bfloat16: nine positions in ten within the tolerance)."""
    rng = np.random.default_rng(900 + seed)
    config = random_config(rng)
    page = int(rng.choice([4, 8, 16]))
    ids = random_ids(rng, config["vocab"], 100)
    for dtype in ("float32", "bfloat16"):
        folder = make_folder(tmp_path / dtype, config, seed=seed, dtype=dtype)
        want = reference(folder, ids)
        model = load(folder, dtype, page, 80)
        outputs = [feed(model, "whole", ids, [len(ids)]), feed(model, "single", ids, [1]),
                   feed(model, "portions", ids, [2, 5, 1, 33, 3, 16, 2, 7]), feed(model, "late", ids, [80, 1])]
        for got in outputs:
            relative = relative_error(got, want)
            assert np.isfinite(relative).all(), json.dumps(config)
            if dtype == "float32":
                assert relative.max() <= 2e-4, f"{relative.max():.3e} at {int(relative.argmax())}: {json.dumps(config)}"
            else:
                assert np.quantile(relative, 0.9) <= TOL[dtype], f"{np.quantile(relative, 0.9):.3e}: {json.dumps(config)}"
        if dtype == "float32":
            assert all(np.array_equal(outputs[0], other) for other in outputs[1:]), json.dumps(config)
        model.unload()
