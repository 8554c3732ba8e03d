"""Dalesun on the GPU against the plain implementation (tests/plain_dalesun.py): every mechanism's kernel alone, then
whole models through the engine's step function, cache manager and scheduler: prompts whole, token by token, in
portions down to two tokens, in batches of unequal requests, with pages and state slots that change hands, with keys
far away, at page borders and on either side of a window's edge, in long decoding, and greedy generation through the
entry point."""

import json
import math

import numpy as np
import pytest
import torch

import plain_dalesun as plain
from dalesun_configs import ALL, PAGE_SIZES, make_folder, random_config
from helpers import TOL, Trace, random_ids, run_trace

pytestmark = pytest.mark.gpu
F64 = torch.float64
BF16 = torch.bfloat16


def device():
    return torch.device("cuda", 0)


def close(got, want, tol, what=""):
    got = got.detach().double().cpu() if isinstance(got, torch.Tensor) else torch.as_tensor(got, dtype=F64)
    want = want.detach().double().cpu() if isinstance(want, torch.Tensor) else torch.as_tensor(want, dtype=F64)
    error = (got - want).abs().max().item()
    bound = tol * max(1.0, want.abs().max().item())
    assert math.isfinite(error) and error <= bound, f"{what}: max |diff| {error:.3e} > {bound:.3e}"


def close_logits(got, want, dtype, what=""):
    """Logits [positions, vocab] of a whole model.  float32: every value within the tolerance.  bfloat16: positions
    are judged by their relative root-mean-square error, nine in ten within the tolerance and all but three in a
    hundred within five times it: where a recurrent head reads almost nothing out of a young state, or a branch's
    result is small, the norm on the branch's result magnifies the projections' rounding.  A lost state, a key missed
    or seen at a window's edge, a sink or a gate left out is an error of order one at most positions."""
    if dtype == "float32":
        return close(got, want, TOL[dtype], what)
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    relative = np.sqrt(((got - want) ** 2).mean(-1)) / np.sqrt((want ** 2).mean(-1))
    assert np.isfinite(relative).all(), f"{what}: not finite"
    assert np.quantile(relative, 0.9) <= TOL[dtype] and (relative <= 5 * TOL[dtype]).mean() >= 0.97, \
        f"{what}: relative error of positions: 90% {np.quantile(relative, 0.9):.3e}, max {relative.max():.3e}"


def on_device(tensor, dtype=None):
    return tensor.to(device=device(), dtype=dtype or tensor.dtype).contiguous()


def batch_description(portions, slots, starts_at=None):
    """Device tensors describing packed rows: portions = tokens per request row; positions count from starts_at."""
    starts = np.concatenate([[0], np.cumsum(portions)]).astype(np.int32)
    row_of_token = np.repeat(np.arange(len(portions)), portions).astype(np.int32)
    first = starts_at or [0] * len(portions)
    positions = np.concatenate([np.arange(f, f + n) for f, n in zip(first, portions)]) if len(portions) else []
    to = lambda a: torch.as_tensor(np.asarray(a, dtype=np.int32), device=device())
    return to(row_of_token), to(starts), to(slots), to(positions)


DTYPES = [(torch.float32, 2e-6), (torch.bfloat16, 8e-3)]


# ------------------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("rows", [1, 8, 32, 33, 127, 128, 300])
def test_up_projection_with_the_squared_relu_in_its_epilogue(rows):
    """relu(x W^T)^2 through every product the row count selects (the weight-streaming kernel, the library product
    with the activation's kernel, the many-rows tcgen05 kernel), and in 32-bit."""
    from libmir_b200 import kernels
    torch.manual_seed(rows)
    x, w = torch.randn(rows, 136), torch.randn(200, 136) * 0.2
    for dtype, tol in ((torch.float32, 1e-5), (BF16, 2e-2)):
        xs, ws = x.to(dtype), w.to(dtype)
        want = plain.relu_squared(xs.double() @ ws.double().T)
        out = torch.full((rows, 200), 7.0, dtype=dtype, device=device())
        kernels.linear_act(on_device(xs), on_device(ws), out, "relu2")
        close(out, want, tol, f"relu2, {rows} rows, {dtype}")
    assert kernels.tensor_core_linear_error() == 0 and kernels.stream_linear_error() == 0


@pytest.mark.parametrize("dtype,tol", DTYPES)
def test_branch_norm_into_the_residual(dtype, tol):
    """x += m * y / rms(y) * w: the norm that stands on a sublayer's result, every tensor 32-bit."""
    from libmir_b200 import kernels
    torch.manual_seed(3)
    for rows, width in ((1, 8), (5, 100), (130, 192), (3, 2050)):
        residual, branch, weight = torch.randn(rows, width), torch.randn(rows, width) * 30.0, 1.0 + torch.randn(width) * 0.3
        want = residual.double() + 0.6 * plain.unit_rms(branch.double(), 1e-6) * weight.double()
        got = on_device(residual)
        kernels.add_normed_branches([on_device(branch)], [on_device(weight)], got, 1e-6, 0.6)
        close(got, want, 2e-6, f"{rows} x {width}")
        # the same kernel also leaves the new residual rounded to bfloat16 for the next reader: the same bits as a cast
        again = on_device(residual)
        rounded = torch.full((rows, width), 7.0, dtype=BF16, device=device())
        kernels.add_normed_branches([on_device(branch)], [on_device(weight)], again, 1e-6, 0.6, rounded=rounded)
        assert torch.equal(again, got) and torch.equal(rounded, got.to(BF16)), f"{rows} x {width}: rounded copy"


def plain_recurrence(q, k, v, decays, state):
    """q, k [n, heads, dim] (rotated, k scaled), v [n, heads, vdim], state [heads, dim, vdim] float64: the read-outs."""
    out = torch.zeros(v.shape, dtype=F64)
    for t in range(q.shape[0]):
        state = decays[:, None, None] * state + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hkv,hk->hv", state, q[t])
    return out, state


@pytest.mark.parametrize("dtype", [torch.float32, BF16])
@pytest.mark.parametrize("heads,dim,vdim,rotary", [(2, 64, 64, 64), (3, 20, 12, 6), (1, 128, 40, 32), (4, 6, 6, 0),
                                                   (2, 100, 64, 100), (5, 32, 20, 16), (1, 160, 8, 2), (2, 256, 96, 64)])
def test_retention_recurrence_against_the_plain_one(dtype, heads, dim, vdim, rotary):
    """Three requests in one batch: a whole prompt, a portion that goes on from a carried state in mid-sequence, a
    single token; then the same requests continued with single tokens (the variant for steps of single tokens).
    Slots that no row names stay as they were."""
    from libmir_b200 import kernels
    torch.manual_seed(heads * dim)
    rot = {"dims": rotary, "base": 5000.0} if rotary else None
    decays = torch.tensor([1.0 - 2.0 ** -(2 + 2 * h) for h in range(heads)], dtype=F64)
    slots, lengths, starts = [4, 0, 2], [70, 33, 1], [0, 517, 9]
    ld = heads * (2 * dim + vdim) + 8
    state0 = torch.randn(6, heads, vdim, dim) * 0.5
    state0[4] = 0.0                                              # the whole prompt starts from nothing
    state = on_device(state0)
    inv_freq = on_device(plain.frequencies(rot).float()) if rot else None
    for phase in range(2):
        if phase == 1:
            starts = [s + n for s, n in zip(starts, lengths)]
            lengths = [1, 1, 1]
        tokens = sum(lengths)
        packed = (torch.randn(tokens, ld) * 0.7).to(dtype)
        q, k, v = (packed[:, :heads * dim], packed[:, heads * dim:2 * heads * dim],
                   packed[:, 2 * heads * dim:2 * heads * dim + heads * vdim])
        row_of_token, query_starts, slot_tensor, positions = batch_description(lengths, slots, starts)
        before = state.cpu().double()
        want, want_state, cursor = [], before.clone(), 0
        for slot, n, first in zip(slots, lengths, starts):
            rows = slice(cursor, cursor + n)
            place = torch.arange(first, first + n)
            qh, kh = q[rows].double().reshape(n, heads, dim), k[rows].double().reshape(n, heads, dim)
            if rot:
                qh, kh = plain.rotate_half(qh, place, rot), plain.rotate_half(kh, place, rot)
            o, s = plain_recurrence(qh, kh * dim ** -0.5, v[rows].double().reshape(n, heads, vdim), decays,
                                    before[slot].transpose(1, 2))
            want.append(o.reshape(n, heads * vdim))
            want_state[slot] = s.transpose(1, 2)
            cursor += n
        packed_gpu = on_device(packed)
        out = torch.full((tokens, heads * vdim), 5.0, dtype=torch.float32, device=device())
        # the same step once more with the rotation in a kernel of its own (scratch full of NaN): the same bits
        scratch = torch.full((kernels.retention_prepared_floats(tokens, heads, dim),), float("nan"), device=device())
        other_state, other_out = state.clone(), torch.full_like(out, 6.0)
        kernels.retention_scan(packed_gpu[:, :heads * dim], packed_gpu[:, heads * dim:2 * heads * dim],
                               packed_gpu[:, 2 * heads * dim:2 * heads * dim + heads * vdim], inv_freq,
                               on_device(decays.float()), float(dim) ** -0.5, other_state, query_starts, slot_tensor,
                               positions, other_out, heads, dim, vdim, prepared=scratch)
        kernels.retention_scan(packed_gpu[:, :heads * dim], packed_gpu[:, heads * dim:2 * heads * dim],
                               packed_gpu[:, 2 * heads * dim:2 * heads * dim + heads * vdim], inv_freq,
                               on_device(decays.float()), float(dim) ** -0.5, state, query_starts, slot_tensor, positions,
                               out, heads, dim, vdim)
        assert torch.equal(out, other_out) and torch.equal(state, other_state), f"prepared rows, phase {phase}"
        close(out, torch.cat(want), 3e-5, f"read-outs, phase {phase}")
        close(state, want_state, 3e-5, f"states, phase {phase}")
        for untouched in (1, 3, 5):
            assert torch.equal(state[untouched].cpu(), before[untouched].float())


def test_a_steps_cut_does_not_change_the_recurrence_at_all():
    """32-bit read-outs and states of a request are the same bits whether its tokens come whole, in portions or one
    by one: one order of sums for every shape of step."""
    from libmir_b200 import kernels
    torch.manual_seed(1)
    heads, dim, vdim, n = 3, 48, 24, 90
    packed = on_device(torch.randn(n, heads * (2 * dim + vdim)))
    inv_freq = on_device(plain.frequencies({"dims": 32, "base": 100.0}).float())
    decays = on_device(torch.tensor([0.9, 0.99, 0.999]))

    def run(cuts, separate_rotation=False):
        state = torch.zeros(1, heads, vdim, dim, device=device())
        out = torch.zeros(n, heads * vdim, device=device())
        cursor = 0
        while cursor < n:
            size = min(cuts[0], n - cursor)
            cuts = cuts[1:] + cuts[:1]
            rows = packed[cursor:cursor + size]
            _, starts, slots, positions = batch_description([size], [0], [cursor])
            scratch = torch.empty(kernels.retention_prepared_floats(size, heads, dim), device=device()) \
                if separate_rotation else None
            kernels.retention_scan(rows[:, :heads * dim], rows[:, heads * dim:2 * heads * dim], rows[:, 2 * heads * dim:],
                                   inv_freq, decays, dim ** -0.5, state, starts, slots, positions, out[cursor:cursor + size],
                                   heads, dim, vdim, prepared=scratch)
            cursor += size
        return out.cpu(), state.cpu()
    whole = run([n])
    for cuts in ([1], [2, 3, 1, 7, 33], [31, 2]):
        for separate_rotation in (False, True):
            other = run(cuts, separate_rotation)
            assert torch.equal(whole[0], other[0]) and torch.equal(whole[1], other[1]), (cuts, separate_rotation)


@pytest.mark.parametrize("dtype,tol", DTYPES)
def test_head_unit_norm_with_a_silu_gate(dtype, tol):
    from libmir_b200 import kernels
    torch.manual_seed(2)
    for tokens, heads, vdim in ((1, 1, 8), (9, 3, 20), (70, 5, 64), (4, 2, 130)):
        o = torch.randn(tokens, heads * vdim) * 3.0
        packed = torch.randn(tokens, heads * vdim + 24).to(dtype)
        gate = packed[:, 16:16 + heads * vdim]
        want = plain.unit_rms(o.double().reshape(tokens, heads, vdim), 1e-5).reshape(tokens, -1) * plain.silu(gate.double())
        out = torch.zeros(tokens, heads * vdim, dtype=dtype, device=device())
        kernels.gated_head_norm(on_device(o), on_device(packed)[:, 16:16 + heads * vdim],
                                torch.ones(vdim, device=device()), out, heads, vdim, 1e-5, False)
        close(out, want, tol, f"{tokens} x {heads} x {vdim}")


@pytest.mark.parametrize("dtype,tol", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,rotary,borrower", [(6, 2, 32, 16, 16, False), (1, 1, 16, 16, 16, False),
                                                                     (4, 1, 64, 64, 24, True), (3, 3, 20, 12, 0, False),
                                                                     (4, 2, 128, 128, 32, True), (6, 1, 80, 40, 40, False)])
def test_queries_and_keys_are_normed_rotated_in_interleaved_pairs_and_stored(dtype, tol, heads, kv_heads, dim, vdim,
                                                                            rotary, borrower):
    """Packed rows [q | k | v | gate] (a borrower: [q | gate]): per-head RMS norm with one plain weight for all heads,
    rotation of the pairs (2i, 2i + 1) of the first channels, keys and values into their places of the pool; the gate's
    columns are left alone."""
    from libmir_b200 import kernels
    torch.manual_seed(dim + heads)
    tokens, eps = 11, 1e-5
    rot = {"dims": rotary, "base": 700.0} if rotary else None
    positions = torch.tensor([0, 1, 2, 3, 500, 501, 77, 9, 10, 11, 4096], dtype=torch.int32)
    kv_columns = 0 if borrower else kv_heads * (dim + vdim)
    gate_columns = heads * vdim
    packed = torch.randn(tokens, heads * dim + kv_columns + gate_columns).to(dtype)
    q_norm, k_norm = 1.0 + torch.randn(dim) * 0.3, 1.0 + torch.randn(dim) * 0.3
    q = plain.unit_rms(packed[:, :heads * dim].double().reshape(tokens, heads, dim), eps) * q_norm.double()
    if rot:
        q = plain.rotate_interleaved(q, positions, rot)
    k_pool = torch.zeros(64, kv_heads, dim, dtype=dtype, device=device())
    v_pool = torch.zeros(64, kv_heads, vdim, dtype=dtype, device=device())
    slots = torch.tensor([5, 6, 7, 40, 41, 63, 0, 1, 2, 33, 20], dtype=torch.int32)
    rows = on_device(packed)
    kernels.qk_rope_store(rows, on_device(positions), None if borrower else on_device(slots),
                          on_device(plain.frequencies(rot).float()) if rot else None, on_device(q_norm),
                          None if borrower else on_device(k_norm), None if borrower else k_pool,
                          None if borrower else v_pool, heads, kv_heads, dim, rotary, eps, write_kv=not borrower,
                          value_dim=vdim, interleaved=True, queries_only=borrower)
    close(rows[:, :heads * dim], q.reshape(tokens, -1), tol, "queries")
    assert torch.equal(rows[:, heads * dim + kv_columns:].cpu(), packed[:, heads * dim + kv_columns:])      # the gate
    if not borrower:
        k = packed[:, heads * dim:heads * dim + kv_heads * dim].double().reshape(tokens, kv_heads, dim)
        k = plain.unit_rms(k, eps) * k_norm.double()
        if rot:
            k = plain.rotate_interleaved(k, positions, rot)
        v = packed[:, heads * dim + kv_heads * dim:heads * dim + kv_columns].reshape(tokens, kv_heads, vdim)
        close(k_pool[slots.long()], k, tol, "keys in the pool")
        assert torch.equal(v_pool[slots.long()].cpu(), v)
        mask = torch.ones(64, dtype=torch.bool)
        mask[slots.long()] = False
        assert float(k_pool[mask].abs().max()) == 0.0 and float(v_pool[mask].abs().max()) == 0.0


def plain_attention(q, k, v, scale, window, sinks, gate, first):
    """q [n, H, d] at positions first .. first + n - 1 over keys k [m, G, d] and values [m, G, e]: float64, with a
    window, a sink per head in the denominator and a sigmoid gate [n, H * e] on the result."""
    n, heads, _ = q.shape
    keys, groups, _ = k.shape
    out = torch.zeros(n, heads, v.shape[2], dtype=F64)
    i, j = torch.arange(first, first + n)[:, None], torch.arange(keys)[None, :]
    hidden = j > i
    if window:
        hidden = hidden | (i - j >= window)
    for head in range(heads):
        group = head // (heads // groups)
        scores = ((q[:, head].double() @ k[:, group].double().T) * scale).masked_fill(hidden, float("-inf"))
        top = scores.max(dim=1, keepdim=True).values
        if sinks is not None:
            top = torch.maximum(top, sinks[head].double())
        weights = torch.exp(scores - top)
        total = weights.sum(dim=1, keepdim=True)
        if sinks is not None:
            total = total + torch.exp(sinks[head].double() - top)
        out[:, head] = (weights / total) @ v[:, group].double()
    out = out.reshape(n, -1)
    return out * plain.sigmoid(gate.double()) if gate is not None else out


def scatter_into_pool(ks, vs, page, rng, dtype):
    """Each request's keys and values into shuffled pages of one pool (garbage elsewhere); the pools and the table."""
    blocks = [-(-k.shape[0] // page) for k in ks]
    total = sum(blocks) + 3
    order = rng.permutation(total)
    k_pool = (torch.randn(total * page, *ks[0].shape[1:]) * 40.0).to(dtype)
    v_pool = (torch.randn(total * page, *vs[0].shape[1:]) * 40.0).to(dtype)
    table = torch.full((len(ks), max(blocks)), -1, dtype=torch.int32)
    cursor = 0
    for r, (k, v) in enumerate(zip(ks, vs)):
        for block in range(blocks[r]):
            physical = int(order[cursor]); cursor += 1
            table[r, block] = physical
            rows = slice(block * page, min(k.shape[0], (block + 1) * page))
            k_pool[physical * page: physical * page + rows.stop - rows.start] = k[rows]
            v_pool[physical * page: physical * page + rows.stop - rows.start] = v[rows]
    return k_pool, v_pool, table


# which kernel a case runs: the reference kernel, the mma.sync kernels, the tcgen05 kernels
ATTENTION_CASES = [
    # dtype, heads, kv_heads, dim, vdim, page, window, path
    (torch.float32, 6, 2, 32, 16, 8, 24, "reference"), (BF16, 6, 1, 80, 80, 16, 40, "reference"),
    (torch.float32, 1, 1, 16, 16, 4, 1, "reference"), (BF16, 3, 3, 20, 12, 4, None, "reference"),
    (BF16, 4, 1, 64, 64, 8, 50, "mma"), (BF16, 6, 3, 64, 64, 16, None, "mma"), (BF16, 4, 2, 128, 128, 16, 70, "mma"),
    (BF16, 4, 2, 128, 128, 16, 70, "tcgen05"), (BF16, 8, 1, 128, 128, 32, None, "tcgen05"),
    (BF16, 5, 5, 128, 128, 8, 129, "tcgen05"),
]


@pytest.mark.parametrize("dtype,heads,kv_heads,dim,vdim,page,window,path", ATTENTION_CASES)
def test_attention_with_sink_gate_and_window_where_one_key_stands_out(dtype, heads, kv_heads, dim, vdim, page, window, path):
    """Per request one query is made to look at one chosen key (its query and that key scaled so that this score
    stands out): the first token, either side of a page border, hundreds of tokens back, the oldest key the window
    still shows and the newest it hides (the hidden one must NOT show: the query then sees its other keys and the
    sink).  Requests run as a whole prompt, a portion that starts in mid-request, a two-token portion and single
    decoded tokens, in one batch through the kernels the engine would choose, with sinks and gate in their epilogues."""
    from libmir_b200 import kernels
    rng = np.random.default_rng(dim + heads)
    torch.manual_seed(dim * heads)
    scale = 0.9 / math.sqrt(dim)
    w = window or 10 ** 9
    # (context length, first token of the step's portion, the key the last query looks at)
    plans = [(300, 0, 0 if not window else 300 - window), (300, 283, 299 - w if window else 7),
             (97, 95, 96 - (w - 1) if window and w <= 97 else 2 * page - 1), (130, 129, 2 * page if not window else 130 - w),
             (260, 259, 259 - (w - 1) if window else 3), (64, 63, 63), (1, 0, 0)]
    singles_first = sorted(plans, key=lambda plan: plan[0] - plan[1] != 1)       # single tokens lead the batch
    qs, ks, vs = [], [], []
    for length, first, target in singles_first:
        q = torch.randn(length, heads, dim)
        k = torch.randn(length, kv_heads, dim)
        target = max(0, min(length - 1, target))
        direction = torch.randn(dim)
        direction /= direction.norm()
        k[target] = direction * 6.0
        q[-1] = direction * 6.0 / scale + torch.randn(heads, dim) * 0.1
        qs.append(q.to(dtype)); ks.append(k.to(dtype)); vs.append(torch.randn(length, kv_heads, vdim).to(dtype))
    sinks = torch.randn(heads) * 1.5 + 1.0
    k_pool, v_pool, table = scatter_into_pool(ks, vs, page, rng, dtype)
    q_rows = torch.cat([q[first:].reshape(length - first, -1) for q, (length, first, _) in zip(qs, singles_first)])
    tokens = q_rows.shape[0]
    gate = (torch.randn(tokens, heads * vdim) * 2.0).to(dtype)
    packed = torch.cat([q_rows, torch.randn(tokens, 24).to(dtype), gate], dim=1)
    portions = [length - first for length, first, _ in singles_first]
    row_of_token, starts, _, positions = batch_description(portions, [0] * len(portions), [first for _, first, _ in singles_first])
    contexts = torch.tensor([length for length, _, _ in singles_first], dtype=torch.int32, device=device())
    want = torch.cat([plain_attention(q[first:], k, v, scale, window, sinks, gate[a:b], first)
                      for q, k, v, (length, first, _), a, b in zip(qs, ks, vs, singles_first, starts.tolist(), starts.tolist()[1:])])
    # the sinks matter to ordinary queries (the query that looks at its chosen key hardly feels them)
    assert (plain_attention(qs[-1], ks[-1], vs[-1], scale, window, None, None, 0)
            - plain_attention(qs[-1], ks[-1], vs[-1], scale, window, sinks, None, 0)).abs().max() > 1e-2
    rows = on_device(packed)
    gate_view = rows[:, heads * dim + 24:]
    out = torch.full((tokens, heads * vdim), 9.0, dtype=dtype, device=device())
    pools = (on_device(k_pool), on_device(v_pool))
    table, sinks_gpu = on_device(table), on_device(sinks)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    if path == "reference":
        kernels.paged_attention_generic(rows, out, *pools, table, row_of_token, positions, page, heads, kv_heads, dim,
                                        scale, window, value_dim=vdim, sinks=sinks_gpu, gate=gate_view)
        close(out, want, tol, "reference kernel")
        return
    singles = sum(1 for n in portions if n == 1)
    for partition in (64, 128) if path == "mma" else (128, 256):
        out.fill_(9.0)
        count = -(-300 // partition)
        floats = kernels.decode_attention_scratch_floats(singles, heads, dim, count)
        scratch = torch.full((max(floats, 1),), float("nan"), device=device())
        with kernels.option("decode_tensor_cores", int(path == "tcgen05")):
            kernels.decode_attention(rows[:singles], out[:singles], *pools, table[:singles], positions, page, heads,
                                     kv_heads, dim, scale, window, partition, count, scratch if floats else None,
                                     sinks=sinks_gpu, gate=gate_view[:singles])
        kernels.prefill_attention(rows, out, *pools, table[singles:], starts[singles:], contexts[singles:], page, heads,
                                  kv_heads, dim, scale, window, tensor_cores=path == "tcgen05", sinks=sinks_gpu,
                                  gate=gate_view)
        close(out, want, tol, f"{path} kernels, partitions of {partition} keys")
    # a context short enough for one partition: the attention kernel itself writes the final rows
    with kernels.option("decode_tensor_cores", int(path == "tcgen05")):
        out.fill_(9.0)
        kernels.decode_attention(rows[:singles], out[:singles], *pools, table[:singles], positions, page, heads, kv_heads,
                                 dim, scale, window, 384, 1, None, sinks=sinks_gpu, gate=gate_view[:singles])
    close(out[:singles], want[:singles], tol, f"{path} decode kernel, one partition")
    assert kernels.decode_attention_error() == 0 and kernels.prefill_attention_error() == 0


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


@pytest.mark.parametrize("name", ["A", "C"])
def test_the_residual_stream_after_every_layer(tmp_path, name):
    """One prompt in 32-bit: the residual after each layer against the plain implementation's, so that a fault shows
    at the layer that has it."""
    from libmir_b200 import StepEntry
    from libmir_b200.parts.block import OutputNormBlock
    config = ALL[name]
    folder = make_folder(tmp_path, config, seed=2, dtype="float32")
    ids = random_ids(np.random.default_rng(1), config["vocab"], 60)
    plain_config, weights = plain.read_model(folder)
    want = []
    plain.forward(plain_config, weights, ids, want)
    model = load(folder, "float32", PAGE_SIZES[name], 40)
    seen, original = [], OutputNormBlock.forward

    def recording(self, ctx, cache, residual):
        original(self, ctx, cache, residual)
        seen.append(residual.clone())
    OutputNormBlock.forward = recording
    try:
        model.admit("x")
        model.step([StepEntry("x", ids, [0])])
    finally:
        OutputNormBlock.forward = original
    assert len(seen) == len(want) == len(config["layers"])
    for layer, (got, expected) in enumerate(zip(seen, want)):
        close(got, expected, 2e-5, f"after layer {layer}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ALL))
def test_whole_prompts_token_by_token_and_portions(tmp_path, name, dtype):
    """A prompt whole; the same token by token from its first token (150 single steps: long decoding, windows that
    pass over decoded tokens, the first tokens of a sequence); in portions of changing size down to two tokens; and
    most of it whole with the rest decoded."""
    config = ALL[name]
    folder = make_folder(tmp_path, config, seed=3, dtype=dtype)
    rng = np.random.default_rng(7)
    ids = random_ids(rng, config["vocab"], 150)
    want = reference(folder, ids)
    model = load(folder, dtype, PAGE_SIZES[name], 60)
    whole = feed(model, "whole", ids, [len(ids)])
    close_logits(whole, want, dtype, f"{name}/{dtype} whole")
    single = feed(model, "single", ids, [1])
    close_logits(single, want, dtype, f"{name}/{dtype} token by token")
    portions = feed(model, "portions", ids, [2, 3, 1, 7, 2, 16, 5, 2, 33, 1, 2, 9])
    close_logits(portions, want, dtype, f"{name}/{dtype} portions")
    late = feed(model, "late", ids, [118, 1])                      # most of it whole, the last 32 one by one
    close_logits(late, want, dtype, f"{name}/{dtype} prompt then decoding")
    if dtype == "float32":
        # 32-bit results do not depend on the cut at all: the recurrence walks a request's tokens in order, attention
        # reduces a query's keys in an order that depends on its position alone, products reduce in one fixed order
        assert np.array_equal(whole, single) and np.array_equal(whole, portions) and np.array_equal(whole, late)
    for group in model.cache_stats()["groups"]:
        assert group["free"] == group["pages"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C", "D"])
def test_batches_of_unequal_requests_with_pages_and_slots_that_change_hands(tmp_path, name, dtype):
    """Up to three live requests of unequal lengths, portions of some beside single tokens of others, requests that
    sit a step out, in a pool so small that pages and state slots are used again; every request against itself
    alone (the plain implementation)."""
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
    assert stats["free_slots"] == 3
    for group in stats["groups"]:
        assert group["free"] == group["pages"] and group["reused"] > 0


@pytest.mark.parametrize("kind", ["attention", "retention"])
def test_far_tokens_decide_the_logits_in_prompt_and_in_decoding(tmp_path, kind):
    """One mixer whose memory reaches far: sharp attention without a window (the last positions depend on keys
    hundreds of tokens back, over many pages), a wide window that the prompt outgrows, and retention with decays near
    one; whole, with the last tokens decoded one by one, and in portions."""
    if kind == "attention":
        layers = [{"type": "attention", "mlp": None,
                   "mixer": {"heads": 2, "kv_heads": 1, "dim": 16, "vdim": 24, "scale": 0.25, "rot": {"dims": 8, "base": 10000.0}}},
                  {"type": "attention", "mlp": None,
                   "mixer": {"heads": 2, "kv_heads": 1, "dim": 16, "vdim": 24, "scale": 0.25, "mask": {"size": 450},
                             "rot": {"dims": 8, "base": 10000.0}, "kv_from": 0}}]
    else:
        layers = [{"type": "retention", "mlp": None,
                   "mixer": {"heads": 2, "dim": 16, "vdim": 24, "decay": [0.998, 0.9995], "rot": {"dims": 16, "base": 10000.0}}}]
    config = {"architecture": "Dalesun", "vocab": 90, "width": 64, "norm": {"eps": 1e-5}, "layers": layers}
    rng = np.random.default_rng(4)
    ids = random_ids(rng, 90, 700)
    for dtype in ("float32", "bfloat16"):
        folder = make_folder(tmp_path / dtype, config, seed=6, dtype=dtype, sharpen=12.0)
        plain_config, weights = plain.read_model(folder)
        want = plain.forward(plain_config, weights, ids).numpy()
        shorter = plain.forward(plain_config, weights, ids[300:]).numpy()
        # the early tokens matter: without the first 300 the last logits are others
        assert np.abs(shorter[-20:] - want[-20:]).max() > 0.1
        model = load(folder, dtype, 16, 50)
        close_logits(feed(model, "whole", ids, [700]), want, dtype, f"far tokens, whole, {dtype}")
        close_logits(feed(model, "late", ids, [650, 1]), want, dtype, f"far tokens, decoded, {dtype}")
        close_logits(feed(model, "cut", ids, [15, 17, 300, 2, 31]), want, dtype, f"far tokens, portions, {dtype}")


@pytest.mark.parametrize("dim,page", [(24, 8), (64, 4), (128, 16)])
def test_the_windows_edge_shows_in_the_logits(tmp_path, dim, page):
    """One attention layer and a borrower with another window, sharp scores: the plain implementation with a window one
    token wider or narrower gives other logits, and the engine gives the configured window's, in a prompt and in
    decoding (heads of 24 channels run the reference kernel, of 64 and 128 the tensor-core kernels in bfloat16)."""
    def model_config(first, second):
        mixer = {"heads": 2, "kv_heads": 1, "dim": dim, "vdim": dim, "scale": 0.5 / math.sqrt(dim), "rot": {"dims": 8, "base": 100.0}}
        return {"architecture": "Dalesun", "vocab": 80, "width": 64, "norm": {"eps": 1e-5}, "residual_mult": 1.0, "layers": [
            {"type": "attention", "mlp": None, "mixer": dict(mixer, mask={"size": first})},
            {"type": "attention", "mlp": None, "mixer": dict(mixer, mask={"size": second}, kv_from=0)}]}
    config = model_config(37, 21)
    ids = random_ids(np.random.default_rng(dim), 80, 120)
    for dtype in ("float32", "bfloat16"):
        folder = make_folder(tmp_path / dtype, config, seed=8, dtype=dtype, sharpen=1.0)
        _, weights = plain.read_model(folder)
        want = plain.forward(config, weights, ids).numpy()
        seen = []
        for other in (model_config(38, 21), model_config(36, 21), model_config(37, 22), model_config(37, 20)):
            moved = plain.forward(other, weights, ids).numpy()
            relative = np.sqrt(((moved - want) ** 2).mean(-1)) / np.sqrt((want ** 2).mean(-1))
            seen.append(np.median(relative[45:]))
            assert seen[-1] > 0.015 and relative[45:].min() > 2e-3             # a window one token off is seen
        model = load(folder, dtype, page, 80)
        for label, cuts in (("whole", [120]), ("decoded", [30, 1]), ("portions", [36, 2, 19, 2, 1, 22])):
            got = feed(model, label, ids, cuts)
            relative = np.sqrt(((got - want) ** 2).mean(-1)) / np.sqrt((want ** 2).mean(-1))
            if dtype == "float32":
                assert relative.max() <= 2e-4, f"{label}: {relative.max():.3e} at position {int(relative.argmax())}"
            else:
                assert np.median(relative[45:]) <= 0.5 * min(seen) and relative.max() <= 1.5 * TOL[dtype], \
                    f"{label}/{dtype}: median {np.median(relative[45:]):.3e}, max {relative.max():.3e}"


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
    """Two requests decoded together through captured graphs in bfloat16 (heads of 64 and 128 channels: the tensor-core
    attention kernels with sinks and gate in their epilogues, a window that passes over the decoded tokens): the
    teacher-forced logits of every step against the plain implementation."""
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
    # (the third run replays every single-token step from a captured graph, as generation does)
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
            relative = np.sqrt(((got - want) ** 2).mean(-1)) / np.sqrt((want ** 2).mean(-1))
            assert np.isfinite(relative).all(), json.dumps(config)
            if dtype == "float32":
                assert relative.max() <= 2e-4, f"{relative.max():.3e} at {int(relative.argmax())}: {json.dumps(config)}"
            else:
                assert np.quantile(relative, 0.9) <= TOL[dtype], f"{np.quantile(relative, 0.9):.3e}: {json.dumps(config)}"
        if dtype == "float32":
            assert all(np.array_equal(outputs[0], other) for other in outputs[1:]), json.dumps(config)
        model.unload()
