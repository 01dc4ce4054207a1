"""Routing, sort, tile table and combine of the oracle against numpy restatements."""
import numpy as np

from oracle import oracle as O


def test_route_topk_softmax():
    rng = np.random.default_rng(0)
    logits = rng.normal(size=(33, 128)).astype(np.float32)
    logits[0, 5] = logits[0, 9] = 10.0  # tie: lowest index first
    idx, w = O.moe_route(logits, 8)
    for t in range(logits.shape[0]):
        order = np.lexsort((np.arange(128), -logits[t]))[:8]
        assert np.array_equal(idx[t], order)
        sel = logits[t, order].astype(np.float64)
        sm = np.exp(sel - sel.max())
        assert np.allclose(w[t], sm / sm.sum(), rtol=1e-6)
    assert idx[0, 0] == 5 and idx[0, 1] == 9


def test_sort_is_stable_argsort():
    rng = np.random.default_rng(1)
    idx = rng.integers(0, 16, size=(40, 4)).astype(np.int32)
    sorted_ids, token_rows, inverse = O.moe_sort(idx, 16, 4)
    order = np.argsort(idx.reshape(-1), kind="stable")
    assert np.array_equal(sorted_ids, idx.reshape(-1)[order])
    assert np.array_equal(token_rows, order // 4)
    assert np.array_equal(inverse, np.argsort(order, kind="stable"))


def test_tile_table_restarts_at_expert_runs():
    ids = np.array([0] * 40 + [2] * 3 + [5] * 33, dtype=np.int32)
    tiles, count = O.moe_tile_table(ids, 8, 32)
    assert tiles.shape[0] == (ids.size + 31) // 32 + 8  # prefill_indirect.rs:16-18
    assert [tuple(t) for t in tiles[:count]] == [(0, 32), (32, 40), (40, 43), (43, 75), (75, 76)]
    assert np.all(tiles[count:] == 0)


def test_combine_left_to_right_fold():
    rng = np.random.default_rng(2)
    tokens, k, hidden = 5, 8, 16
    down = O.f32_to_bf16(rng.normal(size=(tokens * k, hidden)).astype(np.float32))
    w = rng.random(size=(tokens, k)).astype(np.float32)
    inverse = rng.permutation(tokens * k).astype(np.int32)
    out = O.moe_combine(down, w, inverse, k)
    d = O.bf16_to_f32(down)
    for t in range(tokens):
        acc = np.zeros(hidden, dtype=np.float32)
        for j in range(k):
            prod = d[inverse[t * k + j]] * w[t, j]
            acc = prod if j == 0 else (prod + acc).astype(np.float32)
        assert np.array_equal(out[t], O.f32_to_bf16(acc))


def test_swiglu_rounding_points():
    g = O.f32_to_bf16(np.array([-3.0, -0.5, 0.0, 0.7, 4.0], dtype=np.float32))
    u = O.f32_to_bf16(np.array([1.5, -2.0, 3.0, 0.25, -1.0], dtype=np.float32))
    act = O.bf16_to_f32(O.swiglu_bf16(g, u))
    gf, uf = O.bf16_to_f32(g).astype(np.float64), O.bf16_to_f32(u).astype(np.float64)
    ref = gf / (1 + np.exp(-gf)) * uf
    assert np.allclose(act, ref, rtol=2e-2, atol=1e-3)
