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
