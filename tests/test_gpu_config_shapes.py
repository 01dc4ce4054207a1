"""GPU parity at the full sizes of the benchmark workloads, through the dispatch a caller gets without flags:
the 2-bit 27B-class stack at eight rows, the routed-expert block with 128 experts and top-8 routing, the GGUF
K-quant matrices at 512 tokens, and the decode shapes of the 4-bit stack.  Where the CPU oracle would take
minutes, output rows or tokens are sampled."""
import numpy as np
import pytest
import torch

from lisa_b200 import _cabi, ops
from lisa_b200.quant import QuantizedLinear, SwitchGlu
from oracle import oracle as O
from tests import util
from tests.gpu_util import dev_bf16, dev_f32, dev_i32, dev_u32, dev_u8, host_bf16_bits

pytestmark = pytest.mark.gpu
TOL = 1e-2  # max over elements of |y - ref| / max(|ref|, rms(ref)), f32 accumulate, bf16 out


@pytest.mark.parametrize("n,k", [(17408, 5120), (5120, 17408)])
@pytest.mark.parametrize("m", [1, 8])
def test_two_bit_stack_shapes_default_dispatch(cuda, n, k, m):
    """gate/up (5120 -> 17408) and down (17408 -> 5120) of the 2-bit stack, one and eight rows, no flags: at
    k = 17408 the eight rows do not fit one pass of the streaming kernel and run as several launches."""
    rng = np.random.default_rng(n + m)
    w, s, b = util.affine_weights(rng, n, k, 2, 64)
    x = util.activations(rng, m, k)
    y = ops.quantized_matmul(dev_bf16(x, cuda), dev_u32(w, cuda), dev_bf16(s, cuda), dev_bf16(b, cuda), True, 64, 2)
    got = O.bf16_to_f32(host_bf16_bits(y))
    truth = O.affine_matmul(x, w, s, b, 64, 2, round_weight_bf16=False, f64=True)
    err, l2 = util.parity(got, truth)
    assert err <= TOL, (err, l2)
    assert ops.device_status() == 0


@pytest.mark.parametrize("n,k", [(9728, 2560), (4096, 2560), (1024, 2560), (2560, 4096), (2560, 9728)])
def test_four_bit_decode_shapes_default_dispatch(cuda, n, k):
    """The five distinct linears of the 4-bit stack at one row, no flags (the kernel a decode call takes)."""
    rng = np.random.default_rng(n + k)
    w, s, b = util.affine_weights(rng, n, k, 4, 64)
    x = util.activations(rng, 1, k)
    y = ops.quantized_matmul(dev_bf16(x, cuda), dev_u32(w, cuda), dev_bf16(s, cuda), dev_bf16(b, cuda), True, 64, 4)
    err, l2 = util.parity(O.bf16_to_f32(host_bf16_bits(y)), O.affine_matmul(x, w, s, b, 64, 4, round_weight_bf16=False, f64=True))
    assert err <= TOL, (err, l2)
    assert ops.device_status() == 0


@pytest.mark.parametrize("n,k", [(9728, 2560), (4096, 2560), (1024, 2560), (2560, 4096), (2560, 9728)])
def test_four_bit_prefill_shapes_sampled_rows(cuda, n, k):
    """The same five linears at 2048 rows through the tensor-core GEMM; 64 output columns and 96 rows of x are
    checked against the tile-loader law (weights rounded to bf16 once)."""
    rng = np.random.default_rng(n * 3 + k)
    m = 2048
    w, s, b = util.affine_weights(rng, n, k, 4, 64)
    x = util.activations(rng, m, k)
    y = ops.quantized_matmul(dev_bf16(x, cuda), dev_u32(w, cuda), dev_bf16(s, cuda), dev_bf16(b, cuda), True, 64, 4)
    cols = np.sort(rng.choice(n, size=64, replace=False))
    rows = np.sort(rng.choice(m, size=96, replace=False))
    got = O.bf16_to_f32(host_bf16_bits(y))[np.ix_(rows, cols)]
    truth = O.affine_matmul(x[rows], w[cols], s[cols], b[cols], 64, 4, round_weight_bf16=True, f64=True)
    err, l2 = util.parity(got, truth)
    assert err <= TOL, (err, l2)


@pytest.mark.parametrize("n,k,m,bits", [(17408, 5120, 512, 2), (5120, 17408, 512, 2), (1024, 8192, 256, 4), (2560, 9728, 640, 4),
                                        (1024, 4096, 300, 4)])
def test_gemm_launch_forms_sampled_rows(cuda, n, k, m, bits):
    """The launch forms the host chooses between, each on a shape that takes it: one k-slice (17408 x 5120 at 512
    rows), three (5120 x 17408 at 512 rows: 80 CTAs of 272 k-blocks), four (1024 x 8192 at 256 rows), and the
    384-token tile with a ragged last tile (640 and 300 rows).  64 output columns and 96 rows of x against the
    tile-loader law."""
    rng = np.random.default_rng(n + k + m)
    w, s, b = util.affine_weights(rng, n, k, bits, 64)
    x = util.activations(rng, m, k)
    y = ops.quantized_matmul(dev_bf16(x, cuda), dev_u32(w, cuda), dev_bf16(s, cuda), dev_bf16(b, cuda), True, 64, bits)
    cols = np.sort(rng.choice(n, size=64, replace=False))
    rows = np.sort(rng.choice(m, size=96, replace=False))
    rows[-1] = m - 1
    got = O.bf16_to_f32(host_bf16_bits(y))[np.ix_(rows, cols)]
    truth = O.affine_matmul(x[rows], w[cols], s[cols], b[cols], 64, bits, round_weight_bf16=True, f64=True)
    err, l2 = util.parity(got, truth)
    assert err <= TOL, (err, l2)
    assert ops.device_status() == 0


@pytest.mark.parametrize("fmt,name", [(O.Q4_K, "Q4K"), (O.Q2_K, "Q2K")])
@pytest.mark.parametrize("rows,k", [(18432, 7168), (7168, 18432)])
def test_gguf_512_tokens_full_shapes_sampled_rows(cuda, fmt, name, rows, k):
    """The GGUF matrices at 512 tokens through the tensor-core product (workspace given); 48 weight rows are
    checked for every token against the f64 product of the decoded blocks."""
    rng = np.random.default_rng(rows + fmt)
    tokens = 512
    w = util.gguf_weights(rng, fmt, rows, k)
    x = rng.normal(0, 1, size=(tokens, k)).astype(np.float32)
    y = ops.packed_matmul(name, dev_u8(w, cuda), dev_f32(x, cuda)).cpu().numpy()
    sel = np.sort(rng.choice(rows, size=48, replace=False))
    dec = O.gguf_decode(fmt, w[sel]).reshape(sel.size, k).astype(np.float64)
    truth = x.astype(np.float64) @ dec.T
    err, l2 = util.parity(y[:, sel], truth)
    assert err <= 2e-4 and l2 <= 1e-4, (err, l2)  # two bf16 planes per operand: 16 significant bits
    assert ops.device_status() == 0


def _experts(rng, experts, hidden, inter):
    gate = util.affine_weights(rng, inter, hidden, 4, 64, experts=experts)
    up = util.affine_weights(rng, inter, hidden, 4, 64, experts=experts)
    down = util.affine_weights(rng, hidden, inter, 4, 64, experts=experts)
    return gate, up, down


@pytest.mark.parametrize("tokens", [1, 64, 4096])
def test_routed_block_128_experts_top8(cuda, tokens):
    """The routed-expert block at its full geometry: 128 experts, top-8, hidden 2048, intermediate 768, 4-bit
    group 64.  Routing, sort and the weighted fold are compared exactly; each GEMM stage is compared with the
    oracle ON THE SAME INPUT BITS (the stage before, as the GPU produced it) at 1e-2, SwiGLU within one bf16
    ulp; then the block output against the oracle's own chain.  At 4096 tokens the oracle runs on the sorted
    rows of 64 sampled tokens."""
    rng = np.random.default_rng(100 + tokens)
    experts, hidden, inter, top_k = 128, 2048, 768, 8
    gate, up, down = _experts(rng, experts, hidden, inter)
    x = util.activations(rng, tokens, hidden)
    logits = rng.normal(size=(tokens, experts)).astype(np.float32)

    def lin(t):
        return QuantizedLinear(dev_u32(t[0], cuda), dev_bf16(t[1], cuda), dev_bf16(t[2], cuda), 64, 4)

    block = SwitchGlu(lin(gate), lin(up), lin(down), top_k)
    tx, tl = dev_bf16(x, cuda), dev_f32(logits, cuda)
    # the stages, as SwitchGlu.forward chains them
    idx, wts = ops.moe_route(tl, top_k)
    ridx, rw = O.moe_route(logits, top_k)
    assert np.array_equal(idx.cpu().numpy(), ridx)
    assert np.allclose(wts.cpu().numpy(), rw, rtol=2e-6, atol=1e-7)
    sorted_ids, token_rows, inverse = ops.moe_sort(idx, experts, top_k)
    rs, rt, rinv = O.moe_sort(ridx, experts, top_k)
    assert np.array_equal(sorted_ids.cpu().numpy(), rs) and np.array_equal(token_rows.cpu().numpy(), rt)
    assert np.array_equal(inverse.cpu().numpy(), rinv)
    xs = ops.gather_rows(tx, token_rows)
    assert np.array_equal(host_bf16_bits(xs), x[rt])
    g = ops.gather_qmm(xs, block.gate.weight, block.gate.scales, block.gate.biases, None, sorted_ids, True, 64, 4, True)
    u = ops.gather_qmm(xs, block.up.weight, block.up.scales, block.up.biases, None, sorted_ids, True, 64, 4, True)
    act = ops.swiglu(g, u)
    d = ops.gather_qmm(act, block.down.weight, block.down.scales, block.down.biases, None, sorted_ids, True, 64, 4, True)
    y = ops.moe_combine(d, wts, inverse, top_k)
    gb, ub, ab, db, yb = (host_bf16_bits(t) for t in (g, u, act, d, y))

    # sorted rows the oracle recomputes: all of them, or those of 64 sampled tokens
    toks = np.arange(tokens) if tokens <= 64 else np.sort(rng.choice(tokens, size=64, replace=False))
    rows = np.sort(rinv.reshape(tokens, top_k)[toks].reshape(-1))
    ids = rs[rows]
    # more than eight sorted rows per expert run as the grouped tensor-core GEMM (weights rounded to bf16), fewer
    # through the matvec kernel (f32 weights)
    rounded = rs.size > 8 * experts  # (fewer than 24 rows: the warp-per-output kernel, f32 weights as well)
    for name, got, inp, wt in (("gate", gb, x[rt][rows], gate), ("up", ub, x[rt][rows], up), ("down", db, ab[rows], down)):
        ref = O.bf16_to_f32(O.gather_qmm(inp, *wt, ids, 64, 4, round_weight_bf16=rounded))
        err, l2 = util.parity(O.bf16_to_f32(got[rows]), ref)
        assert err <= TOL, (name, err, l2)
    assert util.bf16_ulp_distance(ab[rows], O.swiglu_bf16(gb[rows], ub[rows])) <= 1
    # the fold over the GPU's own down rows and route weights (expf can differ in the last ulp between host and
    # device), for the sampled tokens: exact
    fold = O.moe_combine(db, wts.cpu().numpy(), rinv, top_k)
    assert np.array_equal(yb[toks], fold[toks])
    # the whole block against the oracle's chain (three bf16 rounding points between input and output)
    sub_inv = np.searchsorted(rows, rinv.reshape(tokens, top_k)[toks]).astype(np.int32)
    og = O.gather_qmm(x[rt][rows], *gate, ids, 64, 4, round_weight_bf16=rounded)
    ou = O.gather_qmm(x[rt][rows], *up, ids, 64, 4, round_weight_bf16=rounded)
    od = O.gather_qmm(O.swiglu_bf16(og, ou), *down, ids, 64, 4, round_weight_bf16=rounded)
    oy = O.moe_combine(od, rw[toks], sub_inv, top_k)
    err, l2 = util.parity(O.bf16_to_f32(yb[toks]), O.bf16_to_f32(oy))
    assert err <= TOL and l2 <= TOL, (err, l2)
    # and SwitchGlu.forward is that chain; below 24 slots it takes the per-slot path (three launches), whose
    # dot products sum in another order: the same 1e-2 against the oracle's chain
    fwd = host_bf16_bits(block.forward(tx, tl))
    if tokens * top_k >= SwitchGlu.DECODE_SLOTS:
        assert np.array_equal(fwd, yb)
    else:
        err, l2 = util.parity(O.bf16_to_f32(fwd[toks]), O.bf16_to_f32(oy))
        assert err <= TOL and l2 <= TOL, (err, l2)
    assert ops.device_status() == 0


def test_sort_and_combine_with_an_id_outside_the_table(cuda):
    """A slot whose expert id is outside [0, experts) -- an expert this rank does not own -- is not sorted:
    inverse = -1, the tail of the sorted arrays is filled (id = experts, token row 0), gather_qmm writes zeros
    for the tail and the fold adds nothing for the slot.  Only outputs are checked."""
    rng = np.random.default_rng(9)
    tokens, experts, top_k, hidden, inter = 5, 6, 3, 128, 64
    idx = rng.integers(0, experts, size=(tokens, top_k)).astype(np.int32)
    idx[1, 2] = experts + 3
    idx[4, 0] = -2
    flat = idx.reshape(-1)
    valid = np.nonzero((flat >= 0) & (flat < experts))[0]
    order = valid[np.argsort(flat[valid], kind="stable")]
    s, t, inv = ops.moe_sort(dev_i32(idx, cuda), experts, top_k)
    s, t, inv = s.cpu().numpy(), t.cpu().numpy(), inv.cpu().numpy()
    nv = order.size
    assert np.array_equal(s[:nv], flat[order]) and np.array_equal(t[:nv], order // top_k)
    assert np.all(s[nv:] == experts) and np.all(t[nv:] == 0)
    exp_inv = np.full(flat.size, -1, dtype=np.int32)
    exp_inv[order] = np.arange(nv, dtype=np.int32)
    assert np.array_equal(inv, exp_inv)
    # the static entry agrees
    s2, t2, inv2 = ops.moe_sort_static(dev_i32(idx, cuda), experts, top_k)
    assert np.array_equal(s2.cpu().numpy(), s) and np.array_equal(t2.cpu().numpy(), t) and np.array_equal(inv2.cpu().numpy(), inv)
    # fold: the two slots add nothing
    down_rows = O.f32_to_bf16(rng.normal(0, 1, size=(flat.size, hidden)).astype(np.float32))
    w = rng.random(size=(tokens, top_k)).astype(np.float32)
    out = host_bf16_bits(ops.moe_combine(dev_bf16(down_rows, cuda), dev_f32(w, cuda), dev_i32(inv, cuda), top_k))
    w0 = w.copy().reshape(-1)
    w0[exp_inv < 0] = 0.0
    ref = O.moe_combine(down_rows, w0.reshape(tokens, top_k), np.maximum(exp_inv, 0), top_k)
    assert np.array_equal(out, ref)
    # gather_qmm over the sorted ids: zeros in the tail
    wq, sq, bq = util.affine_weights(rng, inter, hidden, 4, 64, experts=experts)
    xs = ops.gather_rows(dev_bf16(util.activations(rng, tokens, hidden), cuda), dev_i32(t, cuda))
    yq = ops.gather_qmm(xs, dev_u32(wq, cuda), dev_bf16(sq, cuda), dev_bf16(bq, cuda), None, dev_i32(s, cuda), True, 64, 4, True)
    assert torch.all(yq[nv:] == 0)


def test_a_wait_that_runs_out_is_reported_and_can_be_cleared(cuda):
    """The barrier between GPUs with a peer that never arrives: rank 0 of a world of two on ONE device, the
    other rank's flag is never written.  The kernel gives up after its bounded wait (about a second), the
    status word says so, the context stays usable, and the word can be reset."""
    import ctypes as C

    assert ops.device_status() == 0
    flags = [torch.zeros(16, dtype=torch.int64, device=cuda) for _ in range(2)]
    arr = (C.c_void_p * 2)(flags[0].data_ptr(), flags[1].data_ptr())
    _cabi.check(_cabi.lib().lisa_cuda_peer_barrier(torch.cuda.current_stream().cuda_stream, 0, 2, arr, 1))
    torch.cuda.synchronize()
    status = ops.device_status()
    assert status != 0 and (status >> 24) != 0, status
    assert int(flags[1][0]) == 1  # rank 0 did announce itself to the peer
    # the device still works
    assert float((torch.ones(8, device=cuda) * 2).sum()) == 16.0
    ops.clear_device_status()
    assert ops.device_status() == 0
