"""The kernels behind the Rorovik mechanisms, one at a time, against the plain functions of
``plain_rorovik`` (NumPy, double): the attention kernels with sinks, distance slopes and a
window (CUDA cores, the streaming kernel, the ``mma.sync`` kernel with a head or a token's heads
per tile, the tcgen05 kernel), what sits between the fused projection and the cache, the norm behind a sublayer,
the per-token gate, the router's rules, identity outputs and clamped experts in both forms, the
biased gated activation, and the stretched rotary frequencies.  Sizes are ones the models of the
other tests do not have.
"""
from __future__ import annotations

import math

import numpy as np
import pytest
import torch

import plain_rorovik as plain
from test_rekasun_kernels_gpu import dev, host, rounded, status_word, to_cache_layout

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def device_tensor(array, dtype=torch.float32):
    return torch.tensor(np.asarray(array), dtype=torch.float32).to(dtype).cuda().contiguous()


def as_double(tensor):
    return tensor.float().cpu().numpy().astype(np.float64)


def held(array, dtype):
    """What the device holds of ``array`` in ``dtype``, as double."""
    return as_double(torch.tensor(np.asarray(array), dtype=torch.float32).to(dtype))


def close(got, want, atol, rtol=0.0, what=""):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: {got.shape} vs {want.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite values"
    error = np.abs(got - want)
    assert (error <= atol + rtol * np.abs(want)).all(), \
        f"{what}: worst error {error.max():.3e} at {np.unravel_index(error.argmax(), error.shape)}"


# ------------------------------------------------ attention with sinks, slopes and a window

def attention_case(rng, dtype, kernel, heads, kv_heads, head_dim, page_size, context, new, window,
                   sinks, slopes, dominant=None, split_keys=32):
    """One request with ``context`` cached keys and ``new`` query tokens through one kernel.
    ``dominant=(row, key)`` scales the key at that position along that row's query.  Pages that
    the window has passed are taken out of the block table, as the cache manager does."""
    from helix_runtime_b200.ops import library as ops
    total = context + new
    keys = held(rng.normal(size=(total, kv_heads, head_dim)), dtype)
    values = held(rng.normal(size=(total, kv_heads, head_dim)), dtype)
    queries = held(rng.normal(size=(new, heads, head_dim)), dtype)
    share = heads // kv_heads
    if dominant is not None:
        row, position = dominant
        for kv in range(kv_heads):
            direction = queries[row, kv * share]
            keys[position, kv] = held(direction / np.linalg.norm(direction) * 60.0, dtype)
            queries[row, kv * share:(kv + 1) * share] = direction
    pages = -(-total // page_size)
    num_pages = pages + 3
    order = rng.permutation(num_pages)
    tables = np.full((2, pages + 1), -1, dtype=np.int32)
    k_cache = np.full((num_pages, kv_heads, page_size, head_dim), np.nan, dtype=np.float32)
    v_cache = np.full_like(k_cache, np.nan)
    first_seen = max(0, context - window + 1) if window else 0
    for p in range(pages):
        lo, hi = p * page_size, min((p + 1) * page_size, total)
        if hi <= first_seen:
            continue                                    # given back: nobody reads it again
        tables[1, p] = order[p]
        k_cache[order[p], :, :hi - lo] = keys[lo:hi].transpose(1, 0, 2)
        v_cache[order[p], :, :hi - lo] = values[lo:hi].transpose(1, 0, 2)
    q = queries.reshape(new, heads * head_dim)
    out = torch.full((new, heads * head_dim), float("nan"), dtype=dtype, device="cuda")
    status = status_word()
    scale = 1.3 / math.sqrt(head_dim)
    sink_t = None if sinks is None else device_tensor(sinks)
    slope_t = None if slopes is None else device_tensor(slopes)
    common = (dev(q, dtype), dev(to_cache_layout(k_cache, dtype), dtype),
              dev(to_cache_layout(v_cache, dtype), dtype))
    starts, slots = dev([0, new], torch.int32), dev([1], torch.int32)
    if kernel in ("mma", "packed", "tcgen05"):
        ops.prefill_attention(*common, starts, dev([context], torch.int32), slots,
                              dev(tables, torch.int32), out, 1, new, heads, kv_heads, head_dim,
                              page_size, num_pages, scale, 1, status, window=window or 0,
                              tensor_memory=kernel == "tcgen05", packed=kernel == "packed",
                              sinks=sink_t, slopes=slope_t)
    else:
        longest = min(total, window) if window else total
        max_splits = max(1, -(-longest // split_keys))
        ops.paged_attention(*common, dev(np.arange(context, total), torch.int32),
                            dev(np.zeros(new), torch.int32), slots, dev(tables, torch.int32), out,
                            None, new, heads, kv_heads, head_dim, page_size, num_pages,
                            window or 0, scale, split_keys, max_splits, status, sinks=sink_t,
                            slopes=slope_t)
    assert int(status.item()) == 0
    spread = np.arange(heads) // share
    expected = plain.sink_softmax_attention(
        queries, keys[:, spread], values[:, spread], scale,
        np.full(heads, -np.inf) if sinks is None else held(sinks, torch.float32), window,
        None if slopes is None else held(slopes, torch.float32), first=context)
    return host(out).reshape(new, heads, head_dim), expected, values


# CUDA cores (float32), the streaming kernel (bfloat16), the ``mma.sync`` kernel with a head per
# tile and with a token's heads per tile, the tcgen05 kernel (prompt portions only)
KERNELS = [(torch.float32, "paged"), (torch.bfloat16, "paged"), (torch.bfloat16, "mma"),
           (torch.bfloat16, "packed"), (torch.bfloat16, "tcgen05")]


def sizes_for(kernel):
    """Head size and page size: the tcgen05 kernel takes heads from 64 and pages from 16."""
    return (64, 16) if kernel == "tcgen05" else (32, 8)


def bounds(dtype):
    return dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=8e-3)


@pytest.mark.parametrize("dtype,kernel", KERNELS)
@pytest.mark.parametrize("window", [None, 1, 19, 64, 70])
@pytest.mark.parametrize("terms", ["sinks", "slopes", "both"])
def test_sinks_and_slopes_in_portions_and_decoding(dtype, kernel, window, terms):
    rng = np.random.default_rng(17)
    heads, kv_heads = (6, 2) if kernel != "packed" else (6, 1)
    sinks = rng.normal(size=heads) * 2.0 + 1.0 if terms != "slopes" else None
    slopes = 2.0 ** (-6.0 * (np.arange(heads) + 1) / heads) if terms != "sinks" else None
    for context, new in [(0, 150), (37, 90), (210, 17), (129, 1), (15, 1), (0, 1), (100, 23),
                         (300, 600)]:
        if kernel == "tcgen05" and new == 1:
            continue
        got, want, _ = attention_case(rng, dtype, kernel, heads, kv_heads, *sizes_for(kernel),
                                      context, new, window, sinks, slopes)
        close(got, want, what=f"window {window} context {context} new {new}", **bounds(dtype))


@pytest.mark.parametrize("dtype,kernel", KERNELS)
def test_a_sink_far_above_the_scores_takes_the_weight(dtype, kernel):
    """A sink of 40 leaves the keys next to nothing: the result is close to zero, and with a
    sink of -40 it is the plain softmax's."""
    rng = np.random.default_rng(18)
    heads = 4
    head_dim = sizes_for(kernel)[0]
    for new in (1, 70):
        if kernel == "tcgen05" and new == 1:
            continue
        got, want, _ = attention_case(rng, dtype, kernel, heads, 1, head_dim, 16, 90 - new, new, 50,
                                      np.full(heads, 40.0), None)
        assert np.abs(got).max() < 1e-6 and np.abs(want).max() < 1e-6
        got, want, _ = attention_case(rng, dtype, kernel, heads, 1, head_dim, 16, 90 - new, new, 50,
                                      np.full(heads, -40.0), None)
        assert np.abs(want).max() > 0.1
        close(got, want, what=f"{new} new tokens", **bounds(dtype))


@pytest.mark.parametrize("dtype,kernel", KERNELS)
@pytest.mark.parametrize("new", [1, 80])
def test_a_key_at_the_windows_edge_with_sinks_and_slopes(dtype, kernel, new):
    """One key is scaled so that it takes nearly all the weight of the last query: just inside
    the window the result is that key's value, just outside it is not."""
    if kernel == "tcgen05" and new == 1:
        pytest.skip("single tokens are not the tcgen05 kernel's")
    rng = np.random.default_rng(19)
    window, total, heads = 48, 300, 4
    sinks = np.array([0.5, -1.0, 2.0, 0.0])
    slopes = np.array([0.02, 0.01, 0.005, 0.0025])
    for key in (total - window, total - window - 1, total - 1, total - window + 1):
        seen = total - 1 - key < window
        got, want, values = attention_case(rng, dtype, kernel, heads, 1, sizes_for(kernel)[0], 16,
                                           total - new, new, window, sinks, slopes,
                                           dominant=(new - 1, key))
        close(got, want, what=f"key {key}", **bounds(dtype))
        distance = float(np.abs(got[-1] - values[key, 0][None, :]).max())
        assert (distance < 3e-2) == seen, f"key {key} seen={seen}: distance {distance}"


def test_a_far_key_among_hundreds_without_a_window():
    """No window: a key 700 positions back that stands out is found, in a prompt and decoded;
    with a slope the same key counts for less by exp(-slope * distance)."""
    rng = np.random.default_rng(20)
    for dtype, kernel in KERNELS:
        for new in (1, 40):
            if kernel == "tcgen05" and new == 1:
                continue
            head_dim = sizes_for(kernel)[0]
            got, want, values = attention_case(rng, dtype, kernel, 4, 1, head_dim, 16, 720 - new,
                                               new, None, np.zeros(4), None,
                                               dominant=(new - 1, 19))
            close(got, want, what="far key", **bounds(dtype))
            assert np.abs(got[-1] - values[19, 0][None, :]).max() < 3e-2
            got, want, _ = attention_case(rng, dtype, kernel, 4, 1, head_dim, 16, 720 - new, new,
                                          None, np.zeros(4), np.full(4, 0.5),
                                          dominant=(new - 1, 19))
            close(got, want, what="far key under a slope", **bounds(dtype))


# --------------------------------------- between the fused projection and the cache append

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,row", [(3, 1, 10, 6, 16), (4, 2, 24, 32, 32),
                                                         (2, 2, 16, 16, 16)])
def test_biases_whole_norms_temperature_value_mix_and_gates(heads, kv_heads, dim, vdim, row, dtype):
    from helix_runtime_b200.ops import library as ops
    rng = np.random.default_rng(heads * dim)
    tokens, eps, coef, every, lam = 9, 1e-4, 0.6, 4, 0.35
    q_size, k_size, v_size = heads * dim, kv_heads * dim, kv_heads * vdim
    width = q_size + k_size + v_size + heads
    # a row stride that is a multiple of four where the sizes allow: the kernel then takes four
    # numbers at a time (the heads of 10 never do)
    sums = held(rng.normal(size=(tokens, width + 4 - width % 4)) * 2.0, torch.float32)
    positions = np.array([0, 2, 3, 4, 7, 11, 12, 40, 1000])
    qb, kb, vb = (held(rng.normal(size=n) * 0.5, torch.float32) for n in (q_size, k_size, v_size))
    qw, kw = (held(1.0 + 0.3 * rng.normal(size=n), torch.float32) for n in (q_size, k_size))
    first = held(rng.normal(size=(tokens, v_size)), torch.float32)
    rnd = plain.to_bfloat16 if dtype == torch.bfloat16 else plain.identity
    q = plain.rms_norm(sums[:, :q_size] + qb, qw, eps) \
        * plain.query_temperature(positions.astype(np.float64), coef, every)[:, None]
    k = plain.rms_norm(sums[:, q_size:q_size + k_size] + kb, kw, eps)
    v = sums[:, q_size + k_size:q_size + k_size + v_size] + vb
    gates = plain.sigmoid(sums[:, q_size + k_size + v_size:width])
    for mode, want_v in ((0, v), (1, v), (2, (1.0 - lam) * v + lam * first)):
        projected = device_tensor(sums)
        rows = torch.full((tokens, (heads + 2 * kv_heads) * row + 5), 7.0, dtype=dtype, device="cuda")
        source = device_tensor(first)
        gate_out = torch.zeros((tokens, heads), dtype=torch.float32, device="cuda")
        ops.biased_normed_rows(projected, mode == 2, rows, tokens, heads, kv_heads, dim, vdim, row,
                               dev(positions, torch.int32), q_bias=device_tensor(qb),
                               k_bias=device_tensor(kb), v_bias=device_tensor(vb),
                               q_weight=device_tensor(qw), k_weight=device_tensor(kw), eps=eps,
                               temp_coef=coef, temp_every=every, value_mix=mode, mix=lam,
                               value_source=source, gates=gate_out)
        got = as_double(rows)
        tight = dict(atol=3e-6, rtol=3e-6) if dtype == torch.float32 else dict(atol=1e-6, rtol=4e-3)
        got_q = got[:, :heads * row].reshape(tokens, heads, row)
        got_k = got[:, heads * row:(heads + kv_heads) * row].reshape(tokens, kv_heads, row)
        got_v = got[:, (heads + kv_heads) * row:(heads + 2 * kv_heads) * row] \
            .reshape(tokens, kv_heads, row)
        close(got_q[:, :, :dim], rnd(q).reshape(tokens, heads, dim), what="queries", **tight)
        close(got_k[:, :, :dim], rnd(k).reshape(tokens, kv_heads, dim), what="keys", **tight)
        close(got_v[:, :, :vdim], rnd(want_v).reshape(tokens, kv_heads, vdim), what="values", **tight)
        assert (got_q[:, :, dim:] == 0).all() and (got_k[:, :, dim:] == 0).all()
        assert (got_v[:, :, vdim:] == 0).all() and (got[:, (heads + 2 * kv_heads) * row:] == 7).all()
        close(as_double(gate_out), gates, 2e-6, what="gates")
        if mode == 1:
            close(as_double(source), v, 2e-6, what="kept values")
        if mode == 2:       # an accumulator is left clear, what lies behind it untouched
            left = as_double(projected)
            assert (left[:, :width] == 0).all() and (left[:, width:] == sums[:, width:]).all()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dim,vdim", [(6, 10), (8, 12)])
def test_keys_and_values_go_straight_into_the_pages(dim, vdim, dtype):
    """With the cache given, two requests' tokens land in the slots their block tables name (a
    page's last slot, the next page's first), in the cache's own layout, padded coordinates as
    zeros; slots of other tokens keep what they held, and the rows get the queries only."""
    from helix_runtime_b200.ops import library as ops
    from test_kernels_gpu import from_cache_layout
    rng = np.random.default_rng(11)
    heads, kv_heads, row, page, pages = 2, 2, 16, 4, 7
    positions = np.array([2, 3, 4, 9, 0])                  # three requests: 2, 3, 4; 9; 0
    token_request = np.array([0, 0, 0, 1, 2])
    slots = np.array([3, 1, 2])                             # block table rows of the requests
    tables = np.full((4, 4), -1, dtype=np.int32)
    tables[3, :2] = [5, 0]
    tables[1, :3] = [6, 2, 4]
    tables[2, :1] = [1]
    width = heads * dim + kv_heads * (dim + vdim)
    sums = held(rng.normal(size=(5, width)), torch.float32)
    k_cache = torch.full((pages, kv_heads, page, row), 3.0, dtype=dtype, device="cuda")
    v_cache = torch.full((pages, kv_heads, page, row), 4.0, dtype=dtype, device="cuda")
    rows = torch.full((5, heads * row + 2), 7.0, dtype=dtype, device="cuda")
    status = status_word()
    ops.biased_normed_rows(device_tensor(sums), False, rows, 5, heads, kv_heads, dim, vdim, row,
                           dev(positions, torch.int32), token_request=dev(token_request, torch.int32),
                           request_table_row=dev(slots, torch.int32),
                           block_tables=dev(tables, torch.int32), k_cache=k_cache, v_cache=v_cache,
                           page_size=page, num_pages=pages, status=status)
    assert int(status.item()) == 0
    got_k = from_cache_layout(host(k_cache), dtype)
    got_v = from_cache_layout(host(v_cache), dtype)
    want_k = np.full((pages, kv_heads, page, row), 3.0)
    want_v = np.full((pages, kv_heads, page, row), 4.0)
    k = sums[:, heads * dim:(heads + kv_heads) * dim].reshape(5, kv_heads, dim)
    v = sums[:, (heads + kv_heads) * dim:].reshape(5, kv_heads, vdim)
    for token in range(5):
        table_page = tables[slots[token_request[token]], positions[token] // page]
        slot = positions[token] % page
        want_k[table_page, :, slot] = 0.0
        want_v[table_page, :, slot] = 0.0
        want_k[table_page, :, slot, :dim] = held(k[token], dtype)
        want_v[table_page, :, slot, :vdim] = held(v[token], dtype)
    close(got_k, want_k, 0.0, what="keys in the pages")
    close(got_v, want_v, 0.0, what="values in the pages")
    got = as_double(rows)
    assert (got[:, heads * row:] == 7.0).all(), "nothing is written behind the queries"
    close(got[:, :heads * row].reshape(5, heads, row)[:, :, :dim],
          held(sums[:, :heads * dim], dtype).reshape(5, heads, dim), 0.0, what="queries")


def test_parts_of_the_projection_rule_may_be_absent():
    """No biases, no norm, no temperature, no gates: the rows are the sums, cut into heads."""
    from helix_runtime_b200.ops import library as ops
    rng = np.random.default_rng(5)
    tokens, heads, kv_heads, dim, vdim, row = 4, 2, 1, 6, 8, 16
    sums = held(rng.normal(size=(tokens, heads * dim + kv_heads * (dim + vdim))), torch.float32)
    rows = torch.zeros((tokens, (heads + 2 * kv_heads) * row), dtype=torch.float32, device="cuda")
    ops.biased_normed_rows(device_tensor(sums), False, rows, tokens, heads, kv_heads, dim, vdim, row,
                           dev(np.arange(tokens), torch.int32))
    got = as_double(rows).reshape(tokens, heads + 2 * kv_heads, row)
    close(got[:, :heads, :dim].reshape(tokens, -1), sums[:, :heads * dim], 0.0)
    close(got[:, heads, :dim], sums[:, heads * dim:(heads + 1) * dim], 0.0)
    close(got[:, heads + 1, :vdim], sums[:, (heads + 1) * dim:], 0.0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_head_gate_norm_behind_a_sublayer_and_token_gate(dtype):
    from helix_runtime_b200.ops import library as ops
    rng = np.random.default_rng(6)
    tokens, heads, row, width = 7, 3, 16, 50
    loose = dict(atol=3e-6, rtol=3e-6) if dtype == torch.float32 else dict(atol=1e-6, rtol=4e-3)
    context = held(rng.normal(size=(tokens, heads * row)), dtype)
    gates = held(rng.uniform(size=(tokens, heads)), torch.float32)
    buffer = device_tensor(context, dtype)
    ops.head_gate(buffer, device_tensor(gates), tokens, heads, row)
    close(as_double(buffer), held(context * np.repeat(gates, row, axis=1), dtype), what="head gate",
          **loose)
    # x += m * norm(y) * w, and the updated rows in the compute type
    x, y = held(rng.normal(size=(tokens + 1, width)), torch.float32), \
        held(rng.normal(size=(tokens + 1, width)) * 5.0, torch.float32)
    w = held(1.0 + 0.3 * rng.normal(size=width), torch.float32)
    residual, cast = device_tensor(x), torch.zeros((tokens + 1, width), dtype=dtype, device="cuda")
    ops.norm_residual_add(residual, device_tensor(y), device_tensor(w), 1e-3, -0.7, tokens,
                          cast_out=cast)
    want = x[:tokens] - 0.7 * plain.rms_norm(y[:tokens], w, 1e-3)
    close(as_double(residual)[:tokens], want, 3e-6, 3e-6, "normed residual sum")
    close(as_double(residual)[tokens], x[tokens], 0.0, what="the row behind the step")
    close(as_double(cast)[:tokens], held(want, dtype), what="rows in the compute type", **loose)
    # g = gelu_tanh(s) * table[token, offset:offset + dim]
    vocab, columns, offset, dim = 13, 20, 6, 5
    table = held(rng.normal(size=(vocab, columns)), dtype)
    sums = held(rng.normal(size=(tokens, dim + 2)) * 2.0, torch.float32)
    ids = rng.integers(0, vocab, size=tokens)
    out = torch.zeros((tokens, dim), dtype=dtype, device="cuda")
    status = status_word()
    ops.token_gate(device_tensor(sums), False, device_tensor(table, dtype), offset,
                   dev(ids, torch.int32), out, tokens, dim, status)
    close(as_double(out), held(plain.gelu_tanh(sums[:, :dim]) * table[ids, offset:offset + dim], dtype),
          what="token gate", **loose)
    assert int(status.item()) == 0


# ------------------------------------------------------------------------ routed experts

@pytest.mark.parametrize("outputs,top", [(1, 1), (7, 7), (12, 3), (40, 6), (70, 1)])
def test_softmax_router_with_corrections(outputs, top):
    """Scores are the softmax over all outputs; the correction moves choices, not weights; the
    weights are not renormed; among equal choice scores the lowest index wins."""
    from helix_runtime_b200.ops import library as ops
    rng = np.random.default_rng(outputs)
    tokens = 9
    sums = rng.normal(size=(tokens, outputs + 2)) * 2.0
    correction = rng.normal(size=outputs) * 0.2
    if outputs > 2:
        sums[1, :outputs] = sums[1, 0]
        correction[:] = np.where(np.arange(outputs) % 2, 0.25, 0.0)      # ties among the odd ones
    sums, correction = held(sums, torch.float32), held(correction, torch.float32)
    chosen = torch.full((tokens, top), -1, dtype=torch.int32, device="cuda")
    weights = torch.zeros((tokens, top), dtype=torch.float32, device="cuda")
    ops.route_top(device_tensor(sums), chosen, weights, tokens, outputs, top, 1.0, softmax=True,
                  correction=device_tensor(correction), normalize=False)
    z = sums[:, :outputs] - sums[:, :outputs].max(axis=1, keepdims=True)
    scores = np.exp(z) / np.exp(z).sum(axis=1, keepdims=True)
    moved = 0
    for t in range(tokens):
        choice = scores[t] + correction
        order = np.argsort(-choice, kind="stable")
        margin = np.inf if outputs == top else choice[order[top - 1]] - choice[order[top]]
        if t != 1 and margin < 1e-6:
            continue                      # a close call: float32 against double may differ
        got = chosen[t].cpu().tolist()
        if t == 1 and outputs > 2:        # equal scores: odd outputs first, each in ascending order
            assert got == order[:top].tolist(), f"token {t}"
        else:
            assert sorted(got) == sorted(order[:top].tolist()), f"token {t}"
        close(as_double(weights[t]), scores[t, got], 1e-6, what=f"weights of token {t}")
        moved += sorted(got) != sorted(np.argsort(-scores[t], kind="stable")[:top].tolist())
    if outputs == 12:
        assert moved > 0, "the correction changed no choice: the test shows nothing"


def plain_experts(h, router, correction, experts, identity, top, limit, rnd):
    weights = {"x.mlp.router": router, "x.mlp.correction": correction}
    for index, expert in enumerate(experts):
        for name, value in expert.items():
            weights[f"x.mlp.e{index}.{name}"] = value
    mlp = {"expert": {"limit": limit},
           "router": {"experts": len(experts), "identity": identity, "top": top}}
    margins = []
    return plain.routed_feed_forward(h, weights, "x", mlp, rnd, margins), margins[0]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,ff,experts,identity,top,tokens,limit",
                         [(40, 24, 5, 2, 3, 11, 0.8), (72, 9, 1, 3, 4, 1, 0.3),
                          (136, 64, 9, 0, 1, 70, 1.5), (64, 16, 2, 6, 2, 30, 2.0)])
def test_identity_outputs_and_clamped_experts(width, ff, experts, identity, top, tokens, limit,
                                              dtype):
    """One product per (token, choice) pair; and, in bfloat16 with enough pairs, the pairs sorted
    by expert for grouped tensor-core products with the clamped gate as the epilogue."""
    from helix_runtime_b200.ops import library as ops
    rng = np.random.default_rng(width + identity)
    outputs = experts + identity
    h = held(rng.normal(size=(tokens, width)), dtype)
    router = held(rng.normal(size=(outputs, width)) * 2.0 / math.sqrt(width), dtype)
    correction = held(rng.normal(size=outputs) * 0.1, torch.float32)
    plain_weights = [{"gate": held(rng.normal(size=(ff, width)) * 2.0 / math.sqrt(width), dtype),
                      "up": held(rng.normal(size=(ff, width)) * 2.0 / math.sqrt(width), dtype),
                      "down": held(rng.normal(size=(width, ff)) / math.sqrt(ff), dtype)}
                     for _ in range(experts)]
    rnd = plain.to_bfloat16 if dtype == torch.bfloat16 else plain.identity
    want, margin = plain_experts(h, router, correction, plain_weights, identity, top, limit, rnd)
    gate_up = device_tensor(np.stack([np.concatenate([e["gate"], e["up"]]) for e in plain_weights]), dtype)
    down = device_tensor(np.stack([e["down"] for e in plain_weights]), dtype)
    sums = device_tensor(h @ router.T)
    x = device_tensor(h, dtype)
    chosen = torch.empty((tokens, top), dtype=torch.int32, device="cuda")
    weights = torch.empty((tokens, top), dtype=torch.float32, device="cuda")
    ops.route_top(sums, chosen, weights, tokens, outputs, top, 1.0, softmax=True,
                  correction=device_tensor(correction), normalize=False)
    sure = margin > 1e-5
    tolerance = dict(atol=3e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=1e-2)
    start = rng.normal(size=(tokens, width))

    out = device_tensor(start)
    act = torch.full((tokens * top, ff), float("nan"), dtype=dtype, device="cuda")
    ops.expert_identity_add(x, chosen, weights, out, tokens, top, experts)
    ops.expert_gate_up(x, gate_up, chosen, act, tokens, top, ops.GATE_CLAMPED_SIGMOID, limit)
    ops.expert_down(act, down, chosen, weights, out, tokens, top)
    close((as_double(out) - held(start, torch.float32))[sure], want[sure], what="pair by pair",
          **tolerance)
    if dtype != torch.bfloat16 or width % 8 or ff % 8:
        return
    pairs = tokens * top
    tile = ops.expert_tile(pairs, experts)
    tiles = ops.expert_tile_bound(pairs, experts, tile)
    pair_row = torch.full((pairs,), -7, dtype=torch.int32, device="cuda")
    tile_group = torch.full((tiles,), -7, dtype=torch.int32, device="cuda")
    ops.expert_rows(chosen, pair_row, tile_group, pairs, experts, tile, tiles)
    rows, picks = pair_row.cpu().numpy(), chosen.cpu().numpy().ravel()
    assert ((rows < 0) == (picks >= experts)).all(), "identity choices take no row"
    rows_in = torch.full((tiles * tile, width), float("nan"), dtype=dtype, device="cuda")
    rows_act = torch.full((tiles * tile, ff), float("nan"), dtype=dtype, device="cuda")
    rows_out = torch.full((tiles * tile, width), float("nan"), dtype=torch.float32, device="cuda")
    status = status_word()
    ops.expert_gather(x, pair_row, rows_in, tokens, top)
    ops.gemm_tc_grouped(rows_in, gate_up, rows_act, tiles * tile, ff, ops.EPI_SWIGLU, ff, tile,
                        tile_group, status, gate_activation=ops.GATE_CLAMPED_SIGMOID,
                        gate_limit=limit)
    ops.gemm_tc_grouped(rows_act, down, rows_out, tiles * tile, width, ops.EPI_STORE_F32, 0, tile,
                        tile_group, status)
    out = device_tensor(start)
    ops.expert_identity_add(x, chosen, weights, out, tokens, top, experts)
    ops.expert_combine(rows_out, pair_row, weights, out, tokens, top, width)
    assert int(status.item()) == 0
    close((as_double(out) - held(start, torch.float32))[sure], want[sure], what="sorted by expert",
          **tolerance)


def test_the_clamp_binds():
    """Sums far beyond the limit: the gate stops at the limit from above only, the other factor
    from both sides."""
    from helix_runtime_b200.ops import library as ops
    limit = 0.75
    gate = np.array([[-9.0, -0.2, 0.3, 0.75, 5.0, 100.0]])
    up = np.array([[-50.0, -0.75, 0.1, 0.5, 0.76, 30.0]])
    sums = device_tensor(np.concatenate([gate, up], axis=1))
    act = torch.zeros((1, 6), dtype=torch.float32, device="cuda")
    ops.swiglu(sums, act, activation=ops.GATE_CLAMPED_SIGMOID, limit=limit)
    g, u = np.minimum(gate, limit), np.clip(up, -limit, limit)
    close(as_double(act), g * plain.sigmoid(1.702 * g) * (u + 1.0), 1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
def test_gate_and_up_with_biases_through_relu(dtype):
    from helix_runtime_b200.ops import library as ops
    rng = np.random.default_rng(9)
    tokens, ff = 5, 37
    sums = held(rng.normal(size=(tokens, 2 * ff)), torch.float32)
    gate_bias, up_bias = (held(rng.normal(size=ff), torch.float32) for _ in range(2))
    buffer = device_tensor(sums)
    act = torch.zeros((tokens, ff), dtype=dtype, device="cuda")
    ops.swiglu(buffer, act, zero_input=True, activation=ops.GATE_RELU,
               gate_bias=device_tensor(gate_bias), up_bias=device_tensor(up_bias))
    want = np.maximum(sums[:, :ff] + gate_bias, 0.0) * (sums[:, ff:] + up_bias)
    close(as_double(act), held(want, dtype), 1e-6, 4e-3 if dtype == torch.bfloat16 else 1e-6)
    assert (as_double(buffer) == 0).all()


@pytest.mark.parametrize("tokens,width,ff,tiled", [(200, 64, 136, False), (300, 128, 256, True),
                                                   (2100, 256, 384, True), (129, 72, 40, False)])
@pytest.mark.parametrize("activation,limit", [("relu", 0.0), ("clamped_sigmoid", 0.9), ("silu", 0.0)])
def test_biases_and_gate_as_the_epilogue_of_the_product(tokens, width, ff, tiled, activation, limit):
    """Prompt portions on the tensor cores: ``f(x Wg' + bg, x Wu' + bu)`` leaves the product's
    epilogue in bfloat16, with the weights row-major and as tiles."""
    from helix_runtime_b200.ops import library as ops
    rng = np.random.default_rng(tokens + ff)
    x = held(rng.normal(size=(tokens, width)), torch.bfloat16)
    w = held(rng.normal(size=(2 * ff, width)) * 1.5 / math.sqrt(width), torch.bfloat16)
    gate_bias, up_bias = (held(rng.normal(size=ff) * 0.5, torch.float32) for _ in range(2))
    gate, up = x @ w[:ff].T + gate_bias, x @ w[ff:].T + up_bias
    if activation == "relu":
        want = np.maximum(gate, 0.0) * up
    elif activation == "silu":
        want = gate * plain.sigmoid(gate) * up
    else:
        g, u = np.minimum(gate, limit), np.clip(up, -limit, limit)
        want = g * plain.sigmoid(1.702 * g) * (u + 1.0)
    out = torch.full((tokens + 3, ff), 9.0, dtype=torch.bfloat16, device="cuda")
    status = status_word()
    matrix = device_tensor(w, torch.bfloat16)
    held_w = ops.tile_weights(matrix) if tiled else matrix
    ops.gemm_tc(device_tensor(x, torch.bfloat16), held_w, out, tokens, ff, ops.EPI_SWIGLU, status,
                up_row_offset=ff, weight_shape=(2 * ff, width) if tiled else None,
                gate_activation=ops.GATE_ACTIVATIONS[activation], gate_limit=limit,
                gate_bias=device_tensor(gate_bias), up_bias=device_tensor(up_bias))
    assert int(status.item()) == 0
    close(as_double(out)[:tokens], want, 2e-2, 1e-2, what=f"{activation} of {tokens} tokens")
    assert (as_double(out)[tokens:] == 9.0).all()


# ------------------------------------------------------------- stretched rotary frequencies

@pytest.mark.parametrize("dims,base,scaling", [
    (32, 250000.0, {"factor": 8.0, "original": 512, "fast": 32.0, "slow": 1.0}),
    (8, 300.0, {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 0.5}),
    (6, 77.0, {"factor": 3.0, "original": 10, "fast": 2.0, "slow": 0.25}),
    (16, 10000.0, {"factor": 4.0, "original": 4096, "fast": 1.0, "slow": 1.0}),
    (12, 50.0, None)])
def test_stretched_frequencies_and_the_rotation_with_an_amplitude(dims, base, scaling):
    from helix_runtime_b200.ops import library as ops
    from helix_runtime_b200.parts.attention import stretched_frequencies
    want, amplitude = plain.stretched_frequencies(dims, base, scaling)
    got, got_amplitude = stretched_frequencies(dims, base, scaling)
    close(got.numpy(), want, 0.0, 1e-14)
    assert abs(got_amplitude - amplitude) < 1e-15
    if scaling is not None:
        assert amplitude > 1.0 and (want <= base ** (-2.0 * np.arange(dims // 2) / dims)).all()
    # the shared key part through the kernel, with rot = dims + 2 (two coordinates not turned)
    rng = np.random.default_rng(dims)
    tokens, q_rank, kv_rank, rot = 6, 8, 10, dims + 2
    row = kv_rank + rot + (kv_rank + rot) % 2
    positions = np.array([0, 1, 17, 300, 999, 5000])
    down = held(rng.normal(size=(tokens, q_rank + kv_rank + rot)), torch.float32)
    for dtype in DTYPES:
        latent = torch.zeros((tokens, q_rank), dtype=dtype, device="cuda")
        rows = torch.zeros((tokens, 2 * row), dtype=dtype, device="cuda")
        ops.latent_prepare(device_tensor(down), device_tensor(np.ones(q_rank)),
                           device_tensor(np.ones(kv_rank)), 1e-5, dev(positions, torch.int32),
                           got.float().cuda(), got.cuda(), dims, 0, latent, rows, 0, tokens, q_rank,
                           kv_rank, rot, row, amplitude=got_amplitude)
        turned = plain.rotate_interleaved(down[:, q_rank + kv_rank:], positions.astype(np.float64),
                                          want, amplitude)
        # float32 angles at position 5,000 are good to about 5000 * 2^-24
        close(as_double(rows)[:, kv_rank:kv_rank + rot], held(turned, dtype),
              2e-5 if dtype == torch.float32 else 2e-3, 8e-3 if dtype == torch.bfloat16 else 0.0,
              what=f"rotated key part in {dtype}")
