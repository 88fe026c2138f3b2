"""The kernels behind the Rekasun decoder's mechanisms, each alone against the plain form:
LayerNorm, the gelu_tanh gate (kernel and product epilogue), the scaled embedding, the short
causal filter with its state and cache append, the sigmoid output gate, and attention over a
window with kept first keys (CUDA-core kernel for decode tokens and float32, the tensor-core
kernel for prompt portions)."""
from __future__ import annotations

import math

import numpy as np
import pytest
import torch

import plain_rekasun as plain
from engine_harness import assert_close
from helix_runtime_b200.ops import library as ops
from test_kernels_gpu import (DEVICE, DTYPES, dev, from_cache_layout, host, rounded, status_word,
                              to_cache_layout)

pytestmark = pytest.mark.gpu


def tolerance(dtype, tight=1e-5):
    return dict(atol=tight, rtol=tight) if dtype == torch.float32 else dict(atol=2e-2, rtol=8e-3)


# ------------------------------------------------------------- norm, gate, embedding

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,eps,with_bias", [(24, 1e-3, True), (200, 1e-5, True),
                                                  (1000, 1e-6, False), (4096, 1e-5, True),
                                                  (5000, 1e-6, True)])
def test_layernorm(dtype, hidden, eps, with_bias):
    rng = np.random.default_rng(1)
    # a mean far from zero: the variance must be taken of the deviations
    x = (rng.normal(size=(7, hidden)) * 2.0 + 30.0).astype(np.float32)
    w = (1.0 + 0.3 * rng.normal(size=hidden)).astype(np.float32)
    b = (0.5 * rng.normal(size=hidden)).astype(np.float32) if with_bias else None
    out = torch.empty((7, hidden), dtype=dtype, device=DEVICE)
    ops.layernorm(dev(x), dev(w), None if b is None else dev(b), out, eps)
    expected = plain.layer_norm(x.astype(np.float64), w, b, eps).astype(np.float32)
    assert_close(host(out), expected, "layernorm", **tolerance(dtype, 2e-5))
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEVICE)
    out = torch.empty((3, hidden), dtype=dtype, device=DEVICE)
    ops.layernorm(dev(x), dev(w), None if b is None else dev(b), out, eps, rows)
    assert_close(host(out), expected[[6, 0, 3]], "layernorm gathered", **tolerance(dtype, 2e-5))


@pytest.mark.parametrize("dtype", DTYPES)
def test_gelu_tanh_gate(dtype):
    rng = np.random.default_rng(2)
    tokens, inter = 9, 176
    gate_up = (rng.normal(size=(tokens, 2 * inter)) * 3.0).astype(np.float32)
    gate_up[0, :5] = [-100.0, 100.0, 0.0, -20.0, -3.0]
    buffer = dev(gate_up)
    act = torch.empty((tokens, inter), dtype=dtype, device=DEVICE)
    ops.swiglu(buffer, act, zero_input=True, activation=ops.GATE_GELU_TANH)
    expected = plain.gelu_tanh(gate_up[:, :inter].astype(np.float64)) * gate_up[:, inter:]
    assert_close(host(act), expected.astype(np.float32), "gelu_tanh gate", **tolerance(dtype))
    assert float(buffer.abs().sum()) == 0.0


@pytest.mark.parametrize("tokens,inter,depth", [(3, 176, 64), (33, 320, 120), (200, 1000, 264),
                                                (300, 512, 256)])
def test_product_with_gelu_tanh_gate_epilogue(tokens, inter, depth):
    rng = np.random.default_rng(3)
    x = rounded(rng.normal(size=(tokens, depth)), torch.bfloat16)
    w = rounded(rng.normal(size=(2 * inter, depth)) / math.sqrt(depth) * 2.0, torch.bfloat16)
    act = torch.empty((tokens, inter), dtype=torch.bfloat16, device=DEVICE)
    status = status_word()
    ops.gemm_tc(dev(x, torch.bfloat16), dev(w, torch.bfloat16), act, tokens, inter,
                ops.EPI_GEGLU_TANH, status, up_row_offset=inter)
    assert int(status.item()) == 0
    sums = x.astype(np.float64) @ w.astype(np.float64).T
    expected = plain.gelu_tanh(sums[:, :inter]) * sums[:, inter:]
    assert_close(host(act), expected.astype(np.float32), "gated product", atol=2e-2, rtol=1e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_times_a_constant_and_rows_added_back(dtype):
    rng = np.random.default_rng(4)
    table = rounded(rng.normal(size=(50, 72)), dtype)
    ids = np.array([3, 49, 0, 3], dtype=np.int32)
    out = torch.empty((4, 72), dtype=torch.float32, device=DEVICE)
    ops.embed(dev(table, dtype), dev(ids, torch.int32), out, status_word(), 2.5)
    np.testing.assert_array_equal(host(out), (table[ids] * np.float32(2.5)).astype(np.float32))
    other = rng.normal(size=(6, 72)).astype(np.float32)
    kept = dev(other)
    ops.add_rows(kept, out, 4)
    np.testing.assert_array_equal(host(kept)[:4], other[:4] + host(out))
    np.testing.assert_array_equal(host(kept)[4:], other[4:])


# ------------------------------------------------------------------ causal filter

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps", [2, 3, 4])
@pytest.mark.parametrize("own_cache", [True, False])
def test_causal_filter_over_portions_with_state_and_append(dtype, taps, own_cache):
    """Three requests fed in portions of changing size (1, 2, fewer than the filter reaches,
    many), in one batch per round; the state rows carry the filter across the cuts; keys and
    values land in their pages; passthrough columns are copied."""
    rng = np.random.default_rng(10 + taps)
    heads, kv_heads, head_dim, extra = 3, 1, 8, 24
    channels = (heads + 2 * kv_heads) * head_dim
    total = channels + extra
    page_size, num_pages = 4, 40
    lengths = [23, 9, 14]
    cuts = [[1, 2, 1, 7, 2, 10], [2, 1, 1, 5], [5, 1, 1, 1, 6]]
    u = [rounded(rng.normal(size=(n, total)), dtype) for n in lengths]
    filt = rng.normal(size=(channels, taps)).astype(np.float32)
    expected = [plain.causal_filter(x[:, :channels].astype(np.float64), filt.astype(np.float64))
                for x in u]
    slots = np.array([2, 0, 3], dtype=np.int32)
    tables = np.full((4, 8), -1, dtype=np.int32)
    order = rng.permutation(num_pages)
    cursor = 0
    for r, n in enumerate(lengths):
        for p in range(-(-n // page_size)):
            tables[slots[r], p] = order[cursor]
            cursor += 1
    state = torch.zeros((4, taps - 1, channels), dtype=dtype, device=DEVICE)
    k_cache = torch.full((num_pages, kv_heads, page_size, head_dim), float("nan"), dtype=dtype,
                         device=DEVICE)
    v_cache = torch.full_like(k_cache, float("nan"))
    done = [0, 0, 0]
    q_size, kv_size = heads * head_dim, kv_heads * head_dim
    got = [np.zeros((n, total), dtype=np.float32) for n in lengths]
    for round_index in range(max(len(c) for c in cuts)):
        batch = [(r, cuts[r][round_index]) for r in range(3) if round_index < len(cuts[r])]
        rows = np.concatenate([u[r][done[r]:done[r] + n] for r, n in batch])
        positions = np.concatenate([np.arange(done[r], done[r] + n) for r, n in batch])
        token_request = np.concatenate([[i] * n for i, (r, n) in enumerate(batch)])
        starts = np.concatenate([[0], np.cumsum([n for _, n in batch])])
        request_slots = np.array([slots[r] for r, _ in batch], dtype=np.int32)
        tokens = len(rows)
        out = torch.full((tokens, total), float("nan"), dtype=dtype, device=DEVICE)
        status = status_word()
        ops.short_conv_append(dev(rows, dtype), None, out, dev(filt), state,
                              dev(positions, torch.int32), dev(token_request, torch.int32),
                              dev(request_slots, torch.int32), dev(starts, torch.int32),
                              dev(tables, torch.int32) if own_cache else None,
                              k_cache if own_cache else None, v_cache if own_cache else None,
                              tokens, heads, kv_heads, head_dim, total, page_size, num_pages, status)
        assert int(status.item()) == 0
        result = host(out)
        for i, (r, n) in enumerate(batch):
            got[r][done[r]:done[r] + n] = result[starts[i]:starts[i] + n]
            done[r] += n
    keys, values = from_cache_layout(host(k_cache), dtype), from_cache_layout(host(v_cache), dtype)
    tol = tolerance(dtype, 1e-5)
    for r, n in enumerate(lengths):
        assert done[r] == n
        assert_close(got[r][:, :q_size], expected[r][:, :q_size].astype(np.float32),
                     f"filtered queries of request {r}", **tol)
        np.testing.assert_array_equal(got[r][:, channels:], u[r][:, channels:])
        for t in range(n):
            if own_cache:
                page, slot = tables[slots[r], t // page_size], t % page_size
                assert_close(keys[page, :, slot].reshape(-1), expected[r][t, q_size:q_size + kv_size]
                             .astype(np.float32), f"key {t} of request {r}", **tol)
                assert_close(values[page, :, slot].reshape(-1), expected[r][t, q_size + kv_size:]
                             .astype(np.float32), f"value {t} of request {r}", **tol)
        if not own_cache:
            assert_close(got[r][:, q_size:channels], expected[r][:, q_size:].astype(np.float32),
                         f"filtered keys and values of request {r}", **tol)
        # the state is the last projected values
        np.testing.assert_array_equal(host(state)[slots[r]], u[r][n - (taps - 1):, :channels])
    if not own_cache:
        assert torch.isnan(k_cache).all()


def test_causal_filter_reads_sums_and_rounds_them_as_a_store_would():
    rng = np.random.default_rng(20)
    heads, kv_heads, head_dim, taps = 2, 2, 16, 3
    channels = (heads + 2 * kv_heads) * head_dim
    total = channels + 32
    sums = rng.normal(size=(8, total)).astype(np.float32)
    filt = rng.normal(size=(channels, taps)).astype(np.float32)
    state_rows = rounded(rng.normal(size=(1, taps - 1, channels)), torch.bfloat16)
    accum, state = dev(sums), dev(state_rows, torch.bfloat16)
    out = torch.empty((5, total), dtype=torch.bfloat16, device=DEVICE)
    ops.short_conv_append(None, accum, out, dev(filt), state, dev(np.arange(7, 12), torch.int32),
                          dev(np.zeros(5), torch.int32), dev([0], torch.int32),
                          dev([0, 5], torch.int32), None, None, None, 5, heads, kv_heads, head_dim,
                          total, 8, 4, status_word())
    stored = rounded(sums[:5], torch.bfloat16)
    expected = plain.causal_filter(stored[:, :channels].astype(np.float64), filt.astype(np.float64),
                                   history=state_rows[0].astype(np.float64))
    assert_close(host(out)[:, :channels], expected.astype(np.float32), "filtered sums",
                 atol=2e-2, rtol=8e-3)
    np.testing.assert_array_equal(host(out)[:, channels:], stored[:, channels:])
    np.testing.assert_array_equal(host(accum), sums)            # left for the gate to clear
    np.testing.assert_array_equal(host(state)[0], stored[3:5, :channels])


@pytest.mark.parametrize("dtype", DTYPES)
def test_sigmoid_gate_and_the_accumulator_it_clears(dtype):
    rng = np.random.default_rng(21)
    tokens, width = 6, 80
    context = rounded(rng.normal(size=(tokens, width)), dtype)
    gate = rounded(rng.normal(size=(tokens, width + 16)) * 4.0, dtype)
    gate[0, :3] = [-90.0, 90.0, 0.0]
    accum = dev(rng.normal(size=(9, 200)).astype(np.float32))
    before = host(accum).copy()
    buffer = dev(context, dtype)
    ops.sigmoid_gate(buffer, dev(gate, dtype)[:, 16:], tokens, width, clear=accum)
    expected = context * plain.sigmoid(gate[:, 16:].astype(np.float64))
    assert_close(host(buffer), expected.astype(np.float32), "gated heads", **tolerance(dtype))
    assert float(accum[:tokens].abs().sum()) == 0.0
    np.testing.assert_array_equal(host(accum)[tokens:], before[tokens:])


# ------------------------------------------------- attention: window with kept first keys

def windowed_case(rng, dtype, heads, kv_heads, head_dim, page_size, context, new, window, keep,
                  dominant=None, tensor_cores=False, split_keys=32, free_dead_pages=True):
    tensor_memory = tensor_cores == "tcgen05"
    """One request with ``context`` cached keys and ``new`` query tokens.  ``dominant=(row, key)``
    scales the key at that position along the query of that row.  Pages that no query of the
    step can see are taken out of the block table, as the cache manager does."""
    total = context + new
    keys = rounded(rng.normal(size=(kv_heads, total, head_dim)), dtype)
    values = rounded(rng.normal(size=(kv_heads, total, head_dim)), dtype)
    queries = rounded(rng.normal(size=(heads, new, head_dim)), dtype)
    if dominant is not None:
        row, position = dominant
        for kv in range(kv_heads):
            direction = queries[kv * (heads // kv_heads), row]
            keys[kv, position] = rounded(direction / np.linalg.norm(direction) * 60.0, dtype)
            for head in range(kv * (heads // kv_heads), (kv + 1) * (heads // kv_heads)):
                queries[head, row] = queries[kv * (heads // kv_heads), row]
    pages = -(-total // page_size)
    num_pages = pages + 3
    order = rng.permutation(num_pages)
    tables = np.full((2, pages + 1), -1, dtype=np.int32)
    k_cache = np.full((num_pages, kv_heads, page_size, head_dim), np.nan, dtype=np.float32)
    v_cache = np.full_like(k_cache, np.nan)
    first_seen = max(0, context - window + 1)
    for p in range(pages):
        lo, hi = p * page_size, min((p + 1) * page_size, total)
        if free_dead_pages and hi <= first_seen and lo >= keep:
            continue                                    # given back: nobody reads it again
        tables[1, p] = order[p]
        k_cache[order[p], :, :hi - lo] = keys[:, lo:hi]
        v_cache[order[p], :, :hi - lo] = values[:, lo:hi]
    q = queries.transpose(1, 0, 2).reshape(new, heads * head_dim)
    out = torch.full((new, heads * head_dim), float("nan"), dtype=dtype, device=DEVICE)
    status = status_word()
    scale = 1.0 / math.sqrt(head_dim)
    common = (dev(q, dtype), dev(to_cache_layout(k_cache, dtype), dtype),
              dev(to_cache_layout(v_cache, dtype), dtype))
    starts, slots = dev([0, new], torch.int32), dev([1], torch.int32)
    if tensor_cores:
        ops.prefill_attention(*common, starts, dev([context], torch.int32), slots,
                              dev(tables, torch.int32), out, 1, new, heads, kv_heads,
                              head_dim, page_size, num_pages, scale, 1, status, window=window,
                              keep_first=keep, tensor_memory=tensor_memory,
                              packed=tensor_cores == "packed")
    else:
        longest = min(total, window + keep)
        max_splits = max(1, -(-longest // split_keys))
        ops.paged_attention(*common, dev(np.arange(context, total), torch.int32),
                            dev(np.zeros(new), torch.int32), slots, dev(tables, torch.int32), out,
                            None, new, heads, kv_heads, head_dim, page_size, num_pages, window,
                            scale, split_keys, max_splits, status, keep_first=keep)
    assert int(status.item()) == 0
    expected = plain.attention(queries.astype(np.float64), keys.astype(np.float64),
                               values.astype(np.float64), scale, window, keep, query_offset=context)
    return host(out), expected.transpose(1, 0, 2).reshape(new, -1).astype(np.float32), values


# CUDA cores (float32), the streaming kernel (bfloat16 decode tokens and short portions), and
# the two tensor-core kernels for prompt portions
KERNELS = [(torch.float32, False), (torch.bfloat16, False), (torch.bfloat16, "mma"),
           (torch.bfloat16, "tcgen05")]


@pytest.mark.parametrize("dtype,tensor_cores", KERNELS)
@pytest.mark.parametrize("window,keep", [(1, 0), (7, 3), (16, 16), (33, 5), (40, 20), (64, 0),
                                         (65, 64), (200, 1)])
def test_window_with_kept_keys_in_portions_and_decoding(dtype, tensor_cores, window, keep):
    rng = np.random.default_rng(30)
    for context, new in [(0, 150), (37, 90), (210, 17), (100, 300)] + \
            ([] if tensor_cores else [(129, 1), (15, 1)]):
        head_dim, page = (64, 16) if tensor_cores == "tcgen05" else (32, 8)
        out, expected, _ = windowed_case(rng, dtype, 4, 2, head_dim, page, context, new, window,
                                         keep, tensor_cores=tensor_cores)
        assert_close(out, expected, f"window {window} keep {keep} context {context} new {new}",
                     **tolerance(dtype, 2e-5))


def edge_keys(position, window, keep):
    """(key, seen?) just inside and outside the window and the kept keys of a query."""
    cases = {(position - window + 1, True), (position - window, position - window < keep),
             (keep - 1, True), (keep, position - keep < window), (0, True), (position, True)}
    return sorted((key, seen) for key, seen in cases if 0 <= key <= position)


@pytest.mark.parametrize("dtype,tensor_cores", KERNELS)
@pytest.mark.parametrize("new", [1, 80, 200])
def test_one_key_at_every_edge_stands_out_or_is_not_seen(dtype, tensor_cores, new):
    """One key is scaled so that it would take all the weight of the last query: just inside
    the window or among the kept keys the output is that key's value, just outside it is what
    the other keys give; in decoding (one new token) and in a prompt portion."""
    if tensor_cores and new == 1:
        pytest.skip("single tokens are the CUDA-core kernel's")
    rng = np.random.default_rng(31)
    window, keep, context = 48, 5, 300 - new
    for key, seen in edge_keys(299, window, keep):
        head_dim = 64 if tensor_cores == "tcgen05" else 32
        out, expected, values = windowed_case(rng, dtype, 4, 2, head_dim, 16, context, new, window,
                                              keep, dominant=(new - 1, key),
                                              tensor_cores=tensor_cores)
        assert_close(out, expected, f"key {key}", **tolerance(dtype, 2e-5))
        wanted = np.repeat(values[:, key], 2, axis=0).reshape(-1)
        distance = float(np.abs(out[-1] - wanted).max())
        assert (distance < 3e-2) == seen, f"key {key} seen={seen}: distance {distance}"
