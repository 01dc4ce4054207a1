"""GPU parity of routing, sort, gather_qmm and the whole routed-expert block (hidden 2048, intermediate
768, top-8 geometry at a reduced expert count for the oracle's sake, and at full size through
properties)."""
import numpy as np
import pytest
import torch

from lisa_b200 import ops
from lisa_b200.quant import QuantizedLinear, SwitchGlu
from oracle import oracle as O
from tests import util
from tests.gpu_util import dev_bf16, dev_f32, dev_i32, dev_u32, host_bf16_bits

pytestmark = pytest.mark.gpu


def test_route_matches_oracle(cuda):
    rng = np.random.default_rng(0)
    logits = rng.normal(size=(257, 128)).astype(np.float32)
    logits[3, 40] = logits[3, 7] = 9.0
    idx, w = ops.moe_route(dev_f32(logits, cuda), 8)
    ridx, rw = O.moe_route(logits, 8)
    assert np.array_equal(idx.cpu().numpy(), ridx)
    assert np.allclose(w.cpu().numpy(), rw, rtol=2e-6, atol=1e-7)


@pytest.mark.parametrize("tokens,experts,top_k", [(1, 128, 8), (64, 128, 8), (4096, 128, 8), (33, 512, 10), (5, 16, 1)])
def test_sort_is_stable(cuda, tokens, experts, top_k):
    rng = np.random.default_rng(tokens)
    idx = rng.integers(0, experts, size=(tokens, top_k)).astype(np.int32)
    s, t, inv = ops.moe_sort(dev_i32(idx, cuda), experts, top_k)
    rs, rt, rinv = O.moe_sort(idx, experts, top_k)
    assert np.array_equal(s.cpu().numpy(), rs)
    assert np.array_equal(t.cpu().numpy(), rt)
    assert np.array_equal(inv.cpu().numpy(), rinv)


def test_swiglu_and_combine_bit_exact(cuda):
    rng = np.random.default_rng(1)
    g = O.f32_to_bf16(rng.normal(0, 2, size=(40, 96)).astype(np.float32))
    u = O.f32_to_bf16(rng.normal(0, 2, size=(40, 96)).astype(np.float32))
    act = host_bf16_bits(ops.swiglu(dev_bf16(g, cuda), dev_bf16(u, cuda)))
    ref = O.swiglu_bf16(g, u)
    # expf may differ in the last ulp between host libm and the device; allow one bf16 ulp
    assert util.bf16_ulp_distance(act, ref) <= 1
    tokens, k, hidden = 5, 8, 96
    w = rng.random(size=(tokens, k)).astype(np.float32)
    inverse = rng.permutation(tokens * k).astype(np.int32)
    out = host_bf16_bits(ops.moe_combine(dev_bf16(g, cuda), dev_f32(w, cuda), dev_i32(inverse, cuda), k))
    assert np.array_equal(out, O.moe_combine(g, w, inverse, k))


@pytest.mark.parametrize("bits", [4, 2])
@pytest.mark.parametrize("n,k", [(768, 2048), (2048, 768)])
@pytest.mark.parametrize("rows", [3, 12, 40, 48, 300])
def test_gather_qmm_matches_oracle(cuda, bits, n, k, rows):
    """Up to eight rows per expert on average: the matvec kernel over a table of (expert, <= 8 rows) entries (GEMV
    law, f32 weights); more: the grouped tensor-core GEMM over a table of taller tiles (tile-loader law, weights
    rounded to bf16).  Expert runs longer than eight rows (several entries) occur in both."""
    rng = np.random.default_rng(2 + rows)
    experts = 6
    w, s, b = util.affine_weights(rng, n, k, bits, 64, experts=experts)
    ids = np.sort(rng.integers(0, experts, size=rows)).astype(np.int32)
    ids[ids == 2] = 3   # an expert with no rows
    ids[0] = -1         # ids outside the table, at both ends of the sorted order: zeros, no weight access
    ids[-1] = experts
    x = util.activations(rng, ids.size, k)
    y = ops.gather_qmm(dev_bf16(x, cuda).reshape(ids.size, 1, k), dev_u32(w, cuda), dev_bf16(s, cuda),
                       dev_bf16(b, cuda), None, dev_i32(ids, cuda), True, 64, bits, True)
    assert y.shape == (ids.size, 1, n)
    got = O.bf16_to_f32(host_bf16_bits(y).reshape(ids.size, n))
    ref = O.bf16_to_f32(O.gather_qmm(x, w, s, b, ids, 64, bits, round_weight_bf16=rows > 8 * experts))
    assert util.parity(got, ref)[0] <= 1e-2
    assert np.all(got[-1] == 0) and np.all(got[0] == 0)


def test_grouped_gather_qmm_equals_dense_gemm_per_expert(cuda):
    """The routed-expert geometry at full size (128 experts, 4096 tokens x top-8 = 32768 sorted rows, 2048 -> 768):
    every expert run of the grouped GEMM must equal the dense tensor-core GEMM on that expert's rows and
    weights: the same kernel and products; the dense call may add its k-blocks as two slices, so the f32
    sum can differ in its last bits (one bf16 ulp of the output at most)."""
    from lisa_b200 import _cabi

    rng = np.random.default_rng(7)
    experts, n, k, rows = 128, 768, 2048, 32768
    g = torch.Generator(device=cuda)
    g.manual_seed(5)
    w = torch.randint(-2 ** 31, 2 ** 31 - 1, (experts, n, k // 8), dtype=torch.int32, device=cuda, generator=g)
    s = (torch.randn((experts, n, k // 64), device=cuda, generator=g) * 0.02).abs().to(torch.bfloat16)
    b = (torch.randn((experts, n, k // 64), device=cuda, generator=g) * 0.01).to(torch.bfloat16)
    x = torch.randn((rows, k), device=cuda, generator=g).to(torch.bfloat16)
    ids = np.sort(rng.integers(0, experts, size=rows)).astype(np.int32)
    y = ops.gather_qmm(x.reshape(rows, 1, k), w, s, b, None, dev_i32(ids, cuda), True, 64, 4, True).reshape(rows, n)
    for e in (0, 1, 17, 64, 127):
        sel = np.nonzero(ids == e)[0]
        lo, hi = int(sel[0]), int(sel[-1]) + 1
        dense = ops.quantized_matmul(x[lo:hi].contiguous(), w[e], s[e], b[e], True, 64, 4, flags=_cabi.FLAG_FORCE_QMM)
        d, yy = dense.float(), y[lo:hi].float()
        assert (d - yy).abs().max() <= 2.0 ** -7 * d.abs().max(), e
        assert (d != yy).float().mean() < 0.2, e


@pytest.mark.parametrize("tokens", [1, 64])
def test_switch_glu_block_matches_oracle(cuda, tokens):
    """Config 4 geometry (hidden 2048, intermediate 768, top-8, group 64, 4-bit) with 16 experts."""
    rng = np.random.default_rng(3 + tokens)
    experts, hidden, inter, top_k = 16, 2048, 768, 8
    gate = util.affine_weights(rng, inter, hidden, 4, 64, experts=experts)
    up = util.affine_weights(rng, inter, hidden, 4, 64, experts=experts)
    down = util.affine_weights(rng, hidden, inter, 4, 64, experts=experts)
    x = util.activations(rng, tokens, hidden)
    logits = rng.normal(size=(tokens, experts)).astype(np.float32)

    def lin(t):
        return QuantizedLinear(dev_u32(t[0], cuda), dev_bf16(t[1], cuda), dev_bf16(t[2], cuda), 64, 4)

    block = SwitchGlu(lin(gate), lin(up), lin(down), top_k)
    y = block.forward(dev_bf16(x, cuda), dev_f32(logits, cuda))
    # more than eight sorted rows per expert run as the grouped GEMM (weights rounded to bf16 once), fewer as matvecs
    ref, _ = O.moe_forward(x, logits, gate, up, down, top_k, 64, 4, round_weight_bf16=tokens * top_k > 8 * experts)
    got = O.bf16_to_f32(host_bf16_bits(y))
    err, l2 = util.parity(got, O.bf16_to_f32(ref))
    # three bf16 rounding points sit between input and output; the block output still holds 1e-2
    assert err <= 1e-2 and l2 <= 1e-2, (err, l2)


def _lin_triplet(t, cuda):
    return dev_u32(t[0], cuda), dev_bf16(t[1], cuda), dev_bf16(t[2], cuda)


@pytest.mark.parametrize("bits,gs", [(4, 64), (2, 64), (4, 32), (4, 128)])
@pytest.mark.parametrize("tokens", [1, 2])
def test_decode_path_stages_match_oracle(cuda, tokens, bits, gs):
    """The per-slot path for a handful of tokens: gate|up + SwiGLU per slot against the oracle's matvecs on the
    same rows, then down + fold per token against the oracle's matvec on the activations the GPU produced and its
    fold on those results."""
    rng = np.random.default_rng(40 + tokens + bits + gs)
    experts, hidden, inter, top_k = 12, 1024, 384, 8
    gate = util.affine_weights(rng, inter, hidden, bits, gs, experts=experts)
    up = util.affine_weights(rng, inter, hidden, bits, gs, experts=experts)
    down = util.affine_weights(rng, hidden, inter, bits, gs, experts=experts)
    x = util.activations(rng, tokens, hidden)
    idx = np.stack([rng.choice(experts, size=top_k, replace=False) for _ in range(tokens)]).astype(np.int32)
    wts = rng.random(size=(tokens, top_k)).astype(np.float32)
    tidx = dev_i32(idx, cuda)
    act = ops.moe_gate_up_act(dev_bf16(x, cuda), tidx, _lin_triplet(gate, cuda), _lin_triplet(up, cuda), gs, bits)
    ab = host_bf16_bits(act)
    slots = idx.reshape(-1)
    order = np.argsort(slots, kind="stable")          # the oracle wants sorted ids
    xs = np.repeat(x, top_k, axis=0)[order]
    og = O.gather_qmm(xs, *gate, slots[order], gs, bits, round_weight_bf16=False)
    ou = O.gather_qmm(xs, *up, slots[order], gs, bits, round_weight_bf16=False)
    ref = np.empty_like(ab)
    ref[order] = O.swiglu_bf16(og, ou)
    err, l2 = util.parity(O.bf16_to_f32(ab), O.bf16_to_f32(ref))
    assert err <= 1e-2 and l2 <= 1e-2, (err, l2)
    y = ops.moe_down_combine(act, tidx, dev_f32(wts, cuda), _lin_triplet(down, cuda), gs, bits)
    od = np.empty((slots.size, hidden), dtype=np.uint16)
    od[order] = O.gather_qmm(ab[order], *down, slots[order], gs, bits, round_weight_bf16=False)
    inverse = np.arange(slots.size, dtype=np.int32)   # rows already in slot order
    want = O.moe_combine(od, wts, inverse, top_k)
    err, l2 = util.parity(O.bf16_to_f32(host_bf16_bits(y)), O.bf16_to_f32(want))
    assert err <= 1e-2 and l2 <= 1e-2, (err, l2)
    assert ops.device_status() == 0


def test_decode_path_skips_ids_outside_the_table_and_honours_xrow(cuda):
    rng = np.random.default_rng(77)
    experts, hidden, inter, top_k, tokens = 6, 512, 256, 4, 3
    gate = util.affine_weights(rng, inter, hidden, 4, 64, experts=experts)
    up = util.affine_weights(rng, inter, hidden, 4, 64, experts=experts)
    down = util.affine_weights(rng, hidden, inter, 4, 64, experts=experts)
    x = util.activations(rng, tokens, hidden)
    idx = rng.integers(0, experts, size=(tokens, top_k)).astype(np.int32)
    idx[0, 1], idx[2, 3] = -1, experts
    wts = rng.random(size=(tokens, top_k)).astype(np.float32)
    g, u, d = (_lin_triplet(t, cuda) for t in (gate, up, down))
    tx, tidx = dev_bf16(x, cuda), dev_i32(idx, cuda)
    act = ops.moe_gate_up_act(tx, tidx, g, u, 64, 4)
    ab = host_bf16_bits(act)
    assert np.all(ab[1] == 0) and np.all(ab[11] == 0) and np.any(ab[0] != 0)
    # an explicit row map equal to slot / top_k changes nothing; a permuted one reads the other token's row
    rows = (np.arange(tokens * top_k) // top_k).astype(np.int32)
    assert torch.equal(ops.moe_gate_up_act(tx, tidx, g, u, 64, 4, xrow=dev_i32(rows, cuda)), act)
    swapped = host_bf16_bits(ops.moe_gate_up_act(tx, tidx, g, u, 64, 4, xrow=dev_i32((tokens - 1 - rows).astype(np.int32), cuda)))
    flipped = host_bf16_bits(ops.moe_gate_up_act(dev_bf16(x[::-1].copy(), cuda), tidx, g, u, 64, 4))
    assert np.array_equal(swapped, flipped)
    # the fold: slots outside the table add zero, the others as if the bad ones had weight zero
    y = host_bf16_bits(ops.moe_down_combine(act, tidx, dev_f32(wts, cuda), d, 64, 4))
    idx2, w2 = idx.copy(), wts.copy()
    idx2[0, 1], idx2[2, 3] = 0, 0
    act2 = act.clone()
    act2[1], act2[11] = 0, 0
    y2 = host_bf16_bits(ops.moe_down_combine(act2, dev_i32(idx2, cuda), dev_f32(w2, cuda), d, 64, 4))
    # expert 0 on a zero row gives bias * 0 = 0 as well
    assert np.array_equal(y, y2)


@pytest.mark.parametrize("tokens", [1, 2])
def test_decode_path_agrees_with_the_sorted_path(cuda, tokens):
    """128 experts, top-8, 2048 / 768: the three-launch path against the sorted chain on the same device (both
    follow the matvec law; sums differ in order only)."""
    rng = np.random.default_rng(300 + tokens)
    experts, hidden, inter, top_k = 128, 2048, 768, 8
    gate = util.affine_weights(rng, inter, hidden, 4, 64, experts=experts)
    up = util.affine_weights(rng, inter, hidden, 4, 64, experts=experts)
    down = util.affine_weights(rng, hidden, inter, 4, 64, experts=experts)

    def lin(t):
        return QuantizedLinear(dev_u32(t[0], cuda), dev_bf16(t[1], cuda), dev_bf16(t[2], cuda), 64, 4)

    block = SwitchGlu(lin(gate), lin(up), lin(down), top_k)
    tx = dev_bf16(util.activations(rng, tokens, hidden), cuda)
    tl = dev_f32(rng.normal(size=(tokens, experts)).astype(np.float32), cuda)
    before = ops.launch_count()
    fast = block.forward(tx, tl)
    assert ops.launch_count() - before == 3
    old = SwitchGlu.DECODE_SLOTS
    try:
        SwitchGlu.DECODE_SLOTS = 0
        chain = block.forward(tx, tl)
    finally:
        SwitchGlu.DECODE_SLOTS = old
    f, c = fast.float(), chain.float()
    assert float((f - c).abs().max()) <= 2.0 ** -6 * float(c.abs().max())


@pytest.mark.parametrize("rows", [8, 40, 300, 2000])
def test_gather_qmm_siblings_equals_the_separate_calls(cuda, rows):
    """gate | up through one table and one grouped launch (the warp-per-output kernel below 24 rows, the grouped
    matvec up to eight rows per expert, the grouped GEMM beyond) against two gather_qmm calls: the same kernels on
    the same tiles, ids outside the table included."""
    rng = np.random.default_rng(60 + rows)
    experts, n, k = 12, 768, 2048
    gate = util.affine_weights(rng, n, k, 4, 64, experts=experts)
    up = util.affine_weights(rng, n, k, 4, 64, experts=experts)
    ids = np.sort(rng.integers(0, experts, size=rows)).astype(np.int32)
    ids[0], ids[-1] = -1, experts
    x = dev_bf16(util.activations(rng, rows, k), cuda)
    tg = tuple(f(a, cuda) for f, a in zip((dev_u32, dev_bf16, dev_bf16), gate))
    tu = tuple(f(a, cuda) for f, a in zip((dev_u32, dev_bf16, dev_bf16), up))
    tid = dev_i32(ids, cuda)
    before = ops.launch_count()
    g, u = ops.gather_qmm_siblings(x, [tg, tu], tid)
    fused_launches = ops.launch_count() - before
    g2 = ops.gather_qmm(x, *tg, None, tid, True, 64, 4, True)
    u2 = ops.gather_qmm(x, *tu, None, tid, True, 64, 4, True)
    # the same products; the matvec form may cut k into other slices for twice the tiles (another f32 summation
    # order: a bf16 rounding step of the output at most, measured against max(|y|, rms) because sums near zero
    # have no meaningful ulp), the other two forms give the same bits
    for a, b in ((g, g2), (u, u2)):
        if 24 <= rows <= 8 * experts:
            err, _ = util.parity(a.float().cpu().numpy(), b.float().cpu().numpy())
            assert err <= 2.0 ** -7, err
        else:
            assert torch.equal(a, b)
    assert torch.all(g[0] == 0) and torch.all(u[-1] == 0)
    if rows >= 24:
        assert fused_launches == 2   # one table (it zeroes both outputs' out-of-table rows) and one grouped launch
    assert ops.device_status() == 0
