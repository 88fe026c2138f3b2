"""The kernels behind the Medolorn mechanisms, one at a time, against the plain functions of
``plain_medolorn`` (NumPy, double): the matrix-state recurrences in both rules (whole
sequences, and cut into portions that carry their state, down to single tokens), the router
and the experts, the gated residual sum, the joined rows in front of a pass, the input filter
with one and with several taps, the latent attention's norms and rotations and its products
per head.  Sizes are ones the models of the other tests do not have.
"""
from __future__ import annotations

import math

import numpy as np
import pytest
import torch

import plain_medolorn as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def device_tensor(array, dtype=torch.float32):
    return torch.tensor(np.asarray(array), dtype=torch.float32).to(dtype).cuda().contiguous()


def as_double(tensor):
    return tensor.float().cpu().numpy().astype(np.float64)


def rounded(array, dtype):
    """What the device holds of ``array`` in ``dtype``, as double."""
    return as_double(torch.tensor(np.asarray(array), dtype=torch.float32).to(dtype))


def batch(lengths, slots):
    """Device description of one step: request r brings lengths[r] tokens and owns slots[r]."""
    starts = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    token_request = np.concatenate([np.full(n, r) for r, n in enumerate(lengths)]).astype(np.int32)
    make = lambda a: torch.tensor(np.asarray(a, dtype=np.int32)).cuda()
    return make(token_request), make(slots), make(starts)


def close(got, want, atol, rtol=0.0):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape
    assert np.isfinite(got).all()
    error = np.abs(got - want)
    assert (error <= atol + rtol * np.abs(want)).all(), \
        f"worst error {error.max():.3e} at {np.unravel_index(error.argmax(), error.shape)}"


# ------------------------------------------------------ recurrences with a matrix state

def run_scan(ops, lengths_per_step, slots, q, k, v, heads, qk_heads, dim, vdim, dtype, **kwargs):
    """Feeds every request's rows (``q[r]`` and so on, whole sequences) in steps: step ``s``
    brings ``lengths_per_step[s][r]`` tokens of request ``r``.  Returns ``o`` per request."""
    requests = len(q)
    state = torch.full((max(slots) + 2, heads * ops.scan_state_floats(vdim, dim) + 3), 7.0,
                       dtype=torch.float32, device="cuda")
    state[slots] = 0.0                       # admission zeroes a request's row
    cursor = [0] * requests
    outputs = [[] for _ in range(requests)]
    gates = {name: kwargs.pop(name) for name in ("decay_in", "beta_in") if name in kwargs}
    for lengths in lengths_per_step:
        live = [r for r in range(requests) if lengths[r] > 0]
        _, d_slots, d_starts = batch([lengths[r] for r in live], [slots[r] for r in live])
        take = lambda rows: device_tensor(np.concatenate(
            [rows[r][cursor[r]:cursor[r] + lengths[r]] for r in live]), dtype)
        n = sum(lengths)
        positions = torch.tensor(np.concatenate(
            [np.arange(cursor[r], cursor[r] + lengths[r]) for r in live]).astype(np.int32)).cuda()
        o = torch.full((n, heads * vdim), float("nan"), dtype=torch.float32, device="cuda")
        step_gates = {}
        if gates:
            joined = take([np.concatenate([gates[name][r] for name in sorted(gates)], axis=1)
                           for r in range(requests)])
            for index, name in enumerate(sorted(gates)):
                step_gates[name] = joined[:, index * heads:(index + 1) * heads]
        ops.linear_state_scan(take(q), take(k), take(v), state, o, d_starts, d_slots, len(live),
                              heads, qk_heads, dim, vdim,
                              positions=positions if kwargs.get("rotary_dim") else None,
                              **step_gates, **kwargs)
        at = 0
        for r in live:
            outputs[r].append(as_double(o[at:at + lengths[r]]))
            at += lengths[r]
            cursor[r] += lengths[r]
    assert float(state[max(slots) + 1].min()) == 7.0          # rows of other slots are not touched
    return [np.concatenate(rows) for rows in outputs]


def cuts(total, sizes):
    """``total`` tokens cut into portions of the given sizes, repeated; the rest one by one."""
    out, left, index = [], total, 0
    while left > 0 and index < len(sizes):
        out.append(min(sizes[index], left))
        left -= out[-1]
        index += 1
    return out + [1] * left


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,qk_heads,dim,vdim", [(3, 3, 20, 12), (4, 2, 48, 40), (2, 1, 8, 136)])
def test_delta_rule_whole_and_in_portions(heads, qk_heads, dim, vdim, dtype):
    from helix_runtime_b200.ops import library as ops
    rng = np.random.default_rng(heads * dim)
    lengths = (70, 1, 37)
    q = [rounded(rng.normal(size=(n, qk_heads * dim)), dtype) for n in lengths]
    k = [rounded(rng.normal(size=(n, qk_heads * dim)), dtype) for n in lengths]
    v = [rounded(rng.normal(size=(n, heads * vdim)), dtype) for n in lengths]
    a = [rounded(rng.normal(size=(n, heads)) * 2.0, dtype) for n in lengths]
    b = [rounded(rng.normal(size=(n, heads)) * 2.0, dtype) for n in lengths]
    a_log = rng.uniform(math.log(0.01), math.log(2.0), size=heads)
    dt_bias = rng.uniform(-3.0, 0.5, size=heads)
    share = heads // qk_heads
    want = []
    for r, n in enumerate(lengths):
        qh = q[r].reshape(n, qk_heads, dim)
        kh = k[r].reshape(n, qk_heads, dim)
        qh = qh / np.sqrt((qh * qh).sum(-1, keepdims=True) + 1e-6) * dim ** -0.5
        kh = kh / np.sqrt((kh * kh).sum(-1, keepdims=True) + 1e-6)
        decay = np.exp(-np.exp(a_log) * plain.softplus(a[r] + dt_bias))
        want.append(plain.delta_rule_scan(np.repeat(qh, share, 1), np.repeat(kh, share, 1),
                                          v[r].reshape(n, heads, vdim), plain.sigmoid(b[r]), decay)
                    .reshape(n, heads * vdim))
    kwargs = dict(delta=True, decay_in=a, beta_in=b, a_log=device_tensor(a_log),
                  dt_bias=device_tensor(dt_bias), unit_norm=True, unit_eps=1e-6,
                  q_scale=dim ** -0.5)
    slots = [2, 0, 3]
    whole = run_scan(ops, [lengths], slots, q, k, v, heads, qk_heads, dim, vdim, dtype, **kwargs)
    portions = [cuts(n, [5, 2, 33, 2, 9]) for n in lengths]
    steps = [[p[s] if s < len(p) else 0 for p in portions] for s in range(max(map(len, portions)))]
    cut = run_scan(ops, steps, slots, q, k, v, heads, qk_heads, dim, vdim, dtype, **kwargs)
    alone = run_scan(ops, [[1 if s < n else 0 for n in lengths] for s in range(max(lengths))],
                     slots, q, k, v, heads, qk_heads, dim, vdim, dtype, **kwargs)
    for r in range(len(lengths)):
        close(whole[r], want[r], 5e-5, 1e-4)
        close(cut[r], want[r], 5e-5, 1e-4)
        close(alone[r], want[r], 5e-5, 1e-4)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("layout", ["halves", "interleaved"])
@pytest.mark.parametrize("heads,dim,vdim,dims", [(3, 24, 10, 24), (1, 40, 72, 12), (2, 16, 16, 0)])
def test_constant_decay_with_rotation(heads, dim, vdim, dims, layout, dtype):
    from helix_runtime_b200.ops import library as ops
    rng = np.random.default_rng(heads + dim + dims)
    lengths = (3, 90)
    base = 700.0
    decay = np.asarray([0.9, 0.999, 0.97][:heads])
    q = [rounded(rng.normal(size=(n, heads * dim)), dtype) for n in lengths]
    k = [rounded(rng.normal(size=(n, heads * dim)), dtype) for n in lengths]
    v = [rounded(rng.normal(size=(n, heads * vdim)), dtype) for n in lengths]
    want = []
    for r, n in enumerate(lengths):
        positions = np.arange(n)
        qh, kh = q[r].reshape(n, heads, dim), k[r].reshape(n, heads, dim)
        if dims:
            qh = plain.rotate_pairs(qh, positions, base, dims, layout)
            kh = plain.rotate_pairs(kh, positions, base, dims, layout)
        want.append(plain.retention_scan(qh, kh * dim ** -0.5, v[r].reshape(n, heads, vdim), decay)
                    .reshape(n, heads * vdim))
    exact = np.power(base, -2.0 * np.arange(max(dims, 2) // 2) / max(dims, 2))
    kwargs = dict(delta=False, fixed_decay=device_tensor(decay),
                  fixed_decay_m1=device_tensor(decay - 1.0), k_scale=dim ** -0.5, rotary_dim=dims,
                  rotary_layout=ops.ROTARY_LAYOUTS[layout], freq=device_tensor(exact),
                  freq_exact=torch.tensor(exact, dtype=torch.float64).cuda())
    slots = [1, 0]
    whole = run_scan(ops, [lengths], slots, q, k, v, heads, heads, dim, vdim, dtype, **kwargs)
    portions = [cuts(n, [2, 31, 2, 7, 40]) for n in lengths]
    steps = [[p[s] if s < len(p) else 0 for p in portions] for s in range(max(map(len, portions)))]
    cut = run_scan(ops, steps, slots, q, k, v, heads, heads, dim, vdim, dtype, **kwargs)
    scale = max(float(np.abs(w).max()) for w in want)
    # bfloat16 engine: angles in float32 at positions below 100, sums in float32
    tolerance = 3e-6 * scale if dtype == torch.float32 else 2e-4 * scale
    for r in range(len(lengths)):
        close(whole[r], want[r], tolerance, 1e-5)
        close(cut[r], want[r], tolerance, 1e-5)


def test_a_far_token_stays_in_a_slowly_decaying_state():
    """One early key is made to match the last query (both scaled up); with a decay of 0.9995 it
    dominates the read-out 600 tokens later, 400 of them decoded one by one, and its value comes
    back: a state that is lost, reset or mixed up on the way cannot produce it."""
    from helix_runtime_b200.ops import library as ops
    rng = np.random.default_rng(3)
    heads, dim, vdim, n = 2, 32, 24, 640
    decay = np.asarray([0.9995, 0.5])
    q = rng.normal(size=(n, heads, dim)) * 0.1
    k = rng.normal(size=(n, heads, dim)) * 0.01
    v = rng.normal(size=(n, heads, vdim))
    mark = rng.normal(size=dim)
    mark /= np.linalg.norm(mark)
    k[30, 0], q[n - 1, 0] = 6.0 * mark, 6.0 * mark
    v[30, 0] = np.arange(vdim) - 10.0
    want = plain.retention_scan(q, k, v, decay).reshape(n, heads * vdim)
    signal = 36.0 * 0.9995 ** (n - 31) * v[30, 0]
    assert np.abs(want[n - 1, :vdim] - signal).max() < 0.02 * np.abs(signal).max()
    rows = lambda x: [x.reshape(n, -1)]
    kwargs = dict(delta=False, fixed_decay=device_tensor(decay),
                  fixed_decay_m1=device_tensor(decay - 1.0))
    steps = [[m] for m in cuts(n, [100, 37, 2, 101])]
    got = run_scan(ops, steps, [1], rows(q), rows(k), rows(v), heads, heads, dim, vdim,
                   torch.float32, **kwargs)[0]
    close(got, want, 2e-4, 2e-5)


# ------------------------------------------------------------------------ routed experts

@pytest.mark.parametrize("experts,top", [(1, 1), (7, 7), (12, 3), (40, 6), (70, 1)])
def test_router_scores_choices_and_weights(experts, top):
    from helix_runtime_b200.ops import library as ops
    rng = np.random.default_rng(experts)
    tokens, scale = 9, 1.75
    sums = rng.normal(size=(tokens, experts + 2)) * 2.0
    if experts > 2:
        sums[1, :experts] = sums[1, 0]           # all equal: the lowest indices win
        sums[2, experts - 1] = sums[2, 0] = 9.0  # two equal at the top
    sums = rounded(sums, torch.float32)
    chosen = torch.full((tokens, top), -1, dtype=torch.int32, device="cuda")
    weights = torch.zeros((tokens, top), dtype=torch.float32, device="cuda")
    ops.route_top(device_tensor(sums), chosen, weights, tokens, experts, top, scale)
    scores = plain.sigmoid(sums[:, :experts])
    for t in range(tokens):
        want = np.argsort(-scores[t], kind="stable")[:top]
        assert chosen[t].cpu().tolist() == want.tolist(), f"token {t}"
        close(as_double(weights[t]), scores[t, want] / (scores[t, want].sum() + 1e-20) * scale, 1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,ff,experts,top,tokens", [(40, 24, 5, 2, 11), (72, 9, 3, 3, 1),
                                                         (136, 64, 9, 1, 70)])
def test_experts_against_the_plain_sum(width, ff, experts, top, tokens, dtype):
    from helix_runtime_b200.ops import library as ops
    rng = np.random.default_rng(width)
    h = rounded(rng.normal(size=(tokens, width)), dtype)
    router = rounded(rng.normal(size=(experts, width)) * 2.0 / math.sqrt(width), dtype)
    weights_plain = [{"gate": rounded(rng.normal(size=(ff, width)) / math.sqrt(width), dtype),
                      "up": rounded(rng.normal(size=(ff, width)) / math.sqrt(width), dtype),
                      "down": rounded(rng.normal(size=(width, ff)) / math.sqrt(ff), dtype)}
                     for _ in range(experts)]
    rnd = plain.to_bfloat16 if dtype == torch.bfloat16 else plain.identity
    want = plain.routed_experts(h, router, weights_plain, top, 1.5, rnd)
    gate_up = device_tensor(np.stack([np.concatenate([e["gate"], e["up"]]) for e in weights_plain]), dtype)
    down = device_tensor(np.stack([e["down"] for e in weights_plain]), dtype)
    sums = device_tensor(h @ router.T)
    chosen = torch.empty((tokens, top), dtype=torch.int32, device="cuda")
    weights = torch.empty((tokens, top), dtype=torch.float32, device="cuda")
    act = torch.empty((tokens * top, ff), dtype=dtype, device="cuda")
    start = rng.normal(size=(tokens, width))
    out = device_tensor(start)
    ops.route_top(sums, chosen, weights, tokens, experts, top, 1.5)
    ops.expert_gate_up(device_tensor(h, dtype), gate_up, chosen, act, tokens, top)
    ops.expert_down(act, down, chosen, weights, out, tokens, top)
    close(as_double(out) - rounded(start, torch.float32), want,
          2e-5 if dtype == torch.float32 else 2e-2, 1e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("width,ff,experts,top,tokens", [(40, 24, 5, 2, 37), (136, 64, 9, 1, 70),
                                                         (256, 136, 7, 3, 300), (64, 200, 3, 3, 11),
                                                         (128, 128, 20, 2, 1500)])
def test_experts_sorted_for_grouped_products(width, ff, experts, top, tokens):
    """The same sum through the pairs sorted by expert and two grouped tensor-core products:
    experts with no token, with less than a tile and with several tiles; the sorted order
    holds every pair once and every tile names its rows' expert."""
    from helix_runtime_b200.ops import library as ops
    dtype = torch.bfloat16
    rng = np.random.default_rng(ff)
    h = rounded(rng.normal(size=(tokens, width)), dtype)
    router = rounded(rng.normal(size=(experts, width)) * 2.0 / math.sqrt(width), dtype)
    router[experts // 2] = 0.0
    router[experts // 2, 0] = -50.0 * np.sign(h[:, 0]).mean()       # an expert almost nobody takes
    weights_plain = [{"gate": rounded(rng.normal(size=(ff, width)) / math.sqrt(width), dtype),
                      "up": rounded(rng.normal(size=(ff, width)) / math.sqrt(width), dtype),
                      "down": rounded(rng.normal(size=(width, ff)) / math.sqrt(ff), dtype)}
                     for _ in range(experts)]
    want = plain.routed_experts(h, router, weights_plain, top, 0.75, plain.to_bfloat16)
    gate_up = device_tensor(np.stack([np.concatenate([e["gate"], e["up"]]) for e in weights_plain]), dtype)
    down = device_tensor(np.stack([e["down"] for e in weights_plain]), dtype)
    sums = device_tensor(h @ router.T)
    chosen = torch.empty((tokens, top), dtype=torch.int32, device="cuda")
    weights = torch.empty((tokens, top), dtype=torch.float32, device="cuda")
    ops.route_top(sums, chosen, weights, tokens, experts, top, 0.75)
    pairs = tokens * top
    tile = ops.expert_tile(pairs, experts)
    tiles = ops.expert_tile_bound(pairs, experts, tile)
    pair_row = torch.full((pairs,), -7, dtype=torch.int32, device="cuda")
    tile_group = torch.full((tiles,), -7, dtype=torch.int32, device="cuda")
    ops.expert_rows(chosen, pair_row, tile_group, pairs, experts, tile, tiles)
    rows, groups, picks = pair_row.cpu().numpy(), tile_group.cpu().numpy(), chosen.cpu().numpy().ravel()
    assert len(set(rows.tolist())) == pairs and rows.min() >= 0 and rows.max() < tiles * tile
    assert (groups[rows // tile] == picks).all(), "a pair lies in a tile of another expert"
    used = np.zeros(tiles, dtype=bool)
    used[rows // tile] = True
    assert (groups[~used] == -1).all() and (groups[used] >= 0).all()
    poison = float("nan")
    rows_in = torch.full((tiles * tile, width), poison, dtype=dtype, device="cuda")
    rows_act = torch.full((tiles * tile, ff), poison, dtype=dtype, device="cuda")
    rows_out = torch.full((tiles * tile, width), poison, dtype=torch.float32, device="cuda")
    status = torch.zeros((1,), dtype=torch.int32, device="cuda")
    ops.expert_gather(device_tensor(h, dtype), pair_row, rows_in, tokens, top)
    ops.gemm_tc_grouped(rows_in, gate_up, rows_act, tiles * tile, ff, ops.EPI_SWIGLU, ff, tile,
                        tile_group, status)
    ops.gemm_tc_grouped(rows_act, down, rows_out, tiles * tile, width, ops.EPI_STORE_F32, 0, tile,
                        tile_group, status)
    start = rng.normal(size=(tokens, width))
    out = device_tensor(start)
    ops.expert_combine(rows_out, pair_row, weights, out, tokens, top, width)
    assert int(status.item()) == 0
    close(as_double(out) - rounded(start, torch.float32), want, 2e-2, 1e-2)


# ------------------------------------------------- gated connection, rows joined for a pass

def test_gated_residual_sum_and_joined_rows():
    from helix_runtime_b200.ops import library as ops
    rng = np.random.default_rng(8)
    tokens, width = 6, 50
    x, y = rng.normal(size=(8, width)), rng.normal(size=(8, width)) * 3.0
    sums, bias = rng.normal(size=(8, width + 6)) * 4.0, rng.normal(size=width)
    residual = device_tensor(x)
    ops.gated_residual_add(residual, device_tensor(y), device_tensor(sums), device_tensor(bias), tokens)
    want = rounded(x, torch.float32)
    want[:tokens] += rounded(y, torch.float32)[:tokens] * plain.sigmoid(
        rounded(sums, torch.float32)[:tokens, :width] + rounded(bias, torch.float32))
    close(as_double(residual), want, 2e-6, 1e-6)          # rows beyond the step stay as they were
    for dtype in DTYPES:
        joined = torch.full((8, 2 * width + 8), 5.0, dtype=dtype, device="cuda")
        ops.join_rows(device_tensor(x), device_tensor(y), joined, tokens)
        close(as_double(joined[:tokens, :width]), rounded(x[:tokens], dtype), 0.0)
        close(as_double(joined[:tokens, width:2 * width]), rounded(y[:tokens], dtype), 0.0)
        assert float(joined[tokens:].min()) == 5.0 and float(joined[:, 2 * width:].min()) == 5.0


# ---------------------------------------------------------------------------- input filter

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps,silu", [(1, True), (1, False), (2, False), (6, True)])
def test_causal_filter_in_portions_down_to_one_token(taps, silu, dtype):
    """A filter of one tap keeps no history and still multiplies by its tap (and applies silu)."""
    from helix_runtime_b200.ops import library as ops
    rng = np.random.default_rng(taps)
    channels, lengths, slots = 37, (23, 2, 9), [1, 3, 0]
    weight = rounded(rng.normal(size=(channels, taps)), torch.float32)
    rows = [rounded(rng.normal(size=(n, channels)), dtype) for n in lengths]
    want = [plain.causal_filter(r, weight) for r in rows]
    if silu:
        want = [plain.silu(w) for w in want]
    state = None
    if taps > 1:
        state = torch.zeros((4, (taps - 1) * channels + 5), dtype=torch.float32, device="cuda")
    portions = [cuts(n, [1, 1, 3, 2, 1, 7]) for n in lengths]
    cursor = [0] * len(lengths)
    for s in range(max(map(len, portions))):
        live = [r for r in range(len(lengths)) if s < len(portions[r])]
        sizes = [portions[r][s] for r in live]
        token_request, d_slots, d_starts = batch(sizes, [slots[r] for r in live])
        raw = device_tensor(np.concatenate([rows[r][cursor[r]:cursor[r] + n]
                                            for r, n in zip(live, sizes)]), dtype)
        out = torch.empty_like(raw)
        ops.causal_filter(raw, out, device_tensor(weight), None, state, sum(sizes), silu,
                          token_request, d_slots, d_starts)
        at = 0
        for r, n in zip(live, sizes):
            close(as_double(out[at:at + n]), want[r][cursor[r]:cursor[r] + n],
                  3e-6 if dtype == torch.float32 else 3e-2, 1e-6 if dtype == torch.float32 else 8e-3)
            at += n
            cursor[r] += n


# ------------------------------------------------------------------------ latent attention

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("layout", ["interleaved", "halves"])
@pytest.mark.parametrize("q_rank,kv_rank,rot,dims,heads", [(24, 40, 8, 8, 3), (50, 18, 12, 6, 2),
                                                           (16, 32, 0, 0, 4)])
def test_latent_norms_rows_and_rotations(q_rank, kv_rank, rot, dims, heads, layout, dtype):
    from helix_runtime_b200.ops import library as ops
    rng = np.random.default_rng(q_rank + rot)
    tokens, eps, base = 7, 1e-5, 333.0
    row_dim = -(-(kv_rank + rot) // 16) * 16
    positions = np.asarray([0, 1, 2, 50, 51, 997, 3], dtype=np.int32)
    down = rounded(rng.normal(size=(tokens, q_rank + kv_rank + rot + 3)) * 2.0, torch.float32)
    q_weight, kv_weight = rng.normal(size=q_rank) + 1.0, rng.normal(size=kv_rank) + 1.0
    q_weight, kv_weight = rounded(q_weight, torch.float32), rounded(kv_weight, torch.float32)
    exact = np.power(base, -2.0 * np.arange(max(dims, 2) // 2) / max(dims, 2))
    freq = device_tensor(exact) if dims else None
    freq_exact = torch.tensor(exact, dtype=torch.float64).cuda() if dims else None
    code = ops.ROTARY_LAYOUTS[layout]
    d_positions = torch.tensor(positions).cuda()
    latent = torch.empty((tokens, q_rank), dtype=dtype, device="cuda")
    rows = torch.full((tokens, (heads + 2) * row_dim), float("nan"), dtype=dtype, device="cuda")
    ops.latent_prepare(device_tensor(down), device_tensor(q_weight), device_tensor(kv_weight), eps,
                       d_positions, freq, freq_exact, dims, code, latent, rows, heads * row_dim,
                       tokens, q_rank, kv_rank, rot, row_dim)
    loose = dtype == torch.bfloat16
    close(as_double(latent), plain.norm_plain(down[:, :q_rank], q_weight, eps),
          3e-6 if not loose else 3e-2, 1e-6 if not loose else 8e-3)
    c = plain.norm_plain(down[:, q_rank:q_rank + kv_rank], kv_weight, eps)
    key = as_double(rows[:, heads * row_dim:(heads + 1) * row_dim])
    value = as_double(rows[:, (heads + 1) * row_dim:])
    close(key[:, :kv_rank], c, 3e-6 if not loose else 3e-2, 1e-6 if not loose else 8e-3)
    assert (value[:, :kv_rank] == key[:, :kv_rank]).all()
    assert (value[:, kv_rank:] == 0.0).all() and (key[:, kv_rank + rot:] == 0.0).all()
    if rot:
        shared = down[:, q_rank + kv_rank:q_rank + kv_rank + rot].reshape(tokens, 1, rot)
        turned = plain.rotate_pairs(shared, positions, base, dims, layout).reshape(tokens, rot)
        close(key[:, kv_rank:kv_rank + rot], turned, 6e-6 if not loose else 4e-2,
              1e-6 if not loose else 8e-3)
        # the queries' rotated parts, behind `offset` other columns of their buffer
        offset = 5
        q = rounded(rng.normal(size=(tokens, offset + heads * rot)), dtype)
        ops.latent_queries(device_tensor(q, dtype), offset, rows, d_positions, freq, freq_exact,
                           dims, code, tokens, heads, kv_rank, rot, row_dim)
        got = as_double(rows[:, :heads * row_dim]).reshape(tokens, heads, row_dim)
        turned = plain.rotate_pairs(q[:, offset:].reshape(tokens, heads, rot), positions, base, dims,
                                    layout)
        close(got[:, :, kv_rank:kv_rank + rot], turned, 6e-6 if not loose else 4e-2,
              1e-6 if not loose else 8e-3)
        assert (got[:, :, kv_rank + rot:] == 0.0).all()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens,heads,out_dim,in_dim", [(5, 3, 40, 16), (130, 2, 70, 33), (1, 5, 8, 96)])
def test_one_small_product_per_head(tokens, heads, out_dim, in_dim, dtype):
    from helix_runtime_b200.ops import library as ops
    rng = np.random.default_rng(tokens)
    x_stride, out_stride = in_dim + 3, out_dim + 8
    x = rounded(rng.normal(size=(tokens, heads * x_stride)), dtype)
    w = rounded(rng.normal(size=(heads, out_dim, in_dim)) / math.sqrt(in_dim), dtype)
    out = torch.full((tokens, heads * out_stride), 9.0, dtype=dtype, device="cuda")
    ops.head_products(device_tensor(x, dtype), x_stride, device_tensor(w, dtype), out, out_stride,
                      tokens)
    got = as_double(out).reshape(tokens, heads, out_stride)
    want = np.einsum("hoi,thi->tho", w, x.reshape(tokens, heads, x_stride)[:, :, :in_dim])
    close(got[:, :, :out_dim], want, 3e-6 if dtype == torch.float32 else 2e-2,
          1e-6 if dtype == torch.float32 else 8e-3)
    assert (got[:, :, out_dim:] == 9.0).all()


# ------------------------------ attention with a token's heads side by side in a tile's rows

@pytest.mark.parametrize("heads,kv_heads", [(6, 1), (32, 1), (8, 2), (3, 1), (64, 1), (10, 5)])
@pytest.mark.parametrize("window,keep", [(0, 0), (1, 0), (19, 0), (64, 0), (70, 6)])
def test_heads_that_share_a_cached_row_side_by_side(heads, kv_heads, window, keep):
    """Prompt portions and single decoded tokens, with and without a window, pages that the
    window has given back taken out of the table; group sizes that divide a tile's 64 rows and
    that do not."""
    from test_rekasun_kernels_gpu import assert_close as close_rows, tolerance, windowed_case
    rng = np.random.default_rng(heads)
    for context, new in [(0, 150), (37, 90), (210, 17), (129, 1), (15, 1), (0, 1), (100, 23)]:
        head_dim, page = ((48, 16) if heads % 2 else (32, 8))
        out, expected, _ = windowed_case(rng, torch.bfloat16, heads, kv_heads, head_dim, page,
                                         context, new, window, keep, tensor_cores="packed",
                                         free_dead_pages=window > 0)
        close_rows(out, expected, f"{heads} heads, window {window} keep {keep}, context "
                   f"{context}, {new} new", **tolerance(torch.bfloat16, 2e-5))


def test_a_key_at_the_windows_edge_for_every_head_of_a_token():
    from test_rekasun_kernels_gpu import edge_keys, windowed_case
    rng = np.random.default_rng(32)
    window, keep = 48, 0
    for new in (1, 80):
        for key, _ in edge_keys(299, window, keep):
            seen = 299 - key < window
            out, expected, values = windowed_case(rng, torch.bfloat16, 6, 1, 32, 16, 300 - new, new,
                                                  window, keep, dominant=(new - 1, key),
                                                  tensor_cores="packed")
            wanted = np.repeat(values[:, key], 6, axis=0).reshape(-1)
            distance = float(np.abs(out[-1] - wanted).max())
            assert (distance < 3e-2) == seen, f"key {key} seen={seen}: distance {distance}"
