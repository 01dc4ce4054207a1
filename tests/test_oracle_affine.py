"""The affine half of the oracle against the laws and relations the reference states."""
import numpy as np
import pytest

from oracle import oracle as O
from tests import util


@pytest.mark.parametrize("bits", [2, 4, 8])
@pytest.mark.parametrize("gs", [32, 64, 128])
def test_dequantize_law(bits, gs):
    """array_ops.rs:56-83: low code first, one scale/bias per group, q*s+b in f32, one cast."""
    rng = np.random.default_rng(bits * 100 + gs)
    n, k = 5, 256
    w, s, b = util.affine_weights(rng, n, k, bits, gs)
    got = O.affine_dequantize(w, s, b, gs, bits, out_f32=True)
    per = 32 // bits
    sf, bf = O.bf16_to_f32(s), O.bf16_to_f32(b)
    for r in range(n):
        for c in range(0, k, 7):
            q = (int(w[r, c // per]) >> ((c % per) * bits)) & ((1 << bits) - 1)
            want = np.float32(np.float32(q) * sf[r, c // gs]) + bf[r, c // gs]
            assert got[r, c] == np.float32(want)
    bf16 = O.affine_dequantize(w, s, b, gs, bits)
    assert np.array_equal(bf16, O.f32_to_bf16(got))


def test_lcg_matches_reference_formula():
    """array_ops.rs:659-662."""
    vals, seed = O.lcg_fill(0x1234, 4)
    s = 0x1234
    for v in vals:
        s = (s * 6364136223846793005 + 1) % (1 << 64)
        assert v == np.float32((s >> 40) / float(1 << 23) - 1.0)
    assert seed == s


@pytest.mark.parametrize("bits", [2, 4, 8])
def test_quantize_roundtrip_and_smoke_relation(bits):
    """ops::quantize then dequantize stays within one step; quantized_matmul vs
    dequantize+matmul max-abs < 0.1 (crates/lisa-engine/src/models/qwen4/smoke.rs:19-42)."""
    vals, _ = O.lcg_fill(7, 8 * 256)
    w = vals.reshape(8, 256)
    wq, sc, bi = O.affine_quantize(w, 64, bits)
    s16, b16 = O.f32_to_bf16(sc), O.f32_to_bf16(bi)
    deq = O.affine_dequantize(wq, O.f32_to_bf16(sc), O.f32_to_bf16(bi), 64, bits, out_f32=True)
    step = np.abs(O.bf16_to_f32(s16)).repeat(64, axis=1)
    # the far edge of a group can clip by up to one step (q is clamped to 2^bits-1)
    assert np.all(np.abs(deq - w) <= 1.01 * step + 0.02)
    x = O.f32_to_bf16(O.lcg_fill(9, 3 * 256)[0].reshape(3, 256))
    y = O.bf16_to_f32(O.affine_matmul(x, wq, s16, b16, 64, bits, threads=2))
    ref = O.bf16_to_f32(x) @ O.bf16_to_f32(O.affine_dequantize(wq, s16, b16, 64, bits)).T
    assert np.max(np.abs(y - ref)) < 0.1


@pytest.mark.parametrize("bits", [2, 4])
def test_factored_qmv_agrees_with_dequant_matmul(bits):
    """The reference has two laws for the same contraction: its qmv kernels never round the
    weight (quantized.metal:196-295) while its GEMM tiles and ops::dequantize round it to bf16
    first.  Each stays within 1e-2 of its own f64 value; across the two laws the bf16 weight
    rounding alone moves an output by up to about 1e-2 of the output rms."""
    rng = np.random.default_rng(3)
    n, k = 64, 1024
    w, s, b = util.affine_weights(rng, n, k, bits)
    x = util.activations(rng, 2, k)
    exact = O.affine_matmul(x, w, s, b, 64, bits, round_weight_bf16=False, f64=True, threads=2)
    rounded = O.affine_matmul(x, w, s, b, 64, bits, round_weight_bf16=True, f64=True, threads=2)
    for y in (O.affine_qmv_factored(x, w, s, b, 64, bits),
              O.affine_matmul(x, w, s, b, 64, bits, round_weight_bf16=False, threads=1)):
        assert util.parity(O.bf16_to_f32(y), exact)[0] <= 5e-3
    y = O.affine_matmul(x, w, s, b, 64, bits, round_weight_bf16=True, threads=2)
    assert util.parity(O.bf16_to_f32(y), rounded)[0] <= 5e-3
    assert util.parity(rounded, exact)[0] <= 2e-2


def test_threads_do_not_change_results():
    rng = np.random.default_rng(4)
    w, s, b = util.affine_weights(rng, 40, 512, 4)
    x = util.activations(rng, 3, 512)
    assert np.array_equal(O.affine_matmul(x, w, s, b, 64, 4, threads=1), O.affine_matmul(x, w, s, b, 64, 4, threads=5))


def test_gather_qmm_equals_per_run_matmul():
    """array_ops.rs:591-630: sorted rows, one quantized_matmul per expert run."""
    rng = np.random.default_rng(5)
    e, n, k = 4, 16, 256
    w, s, b = util.affine_weights(rng, n, k, 4, experts=e)
    ids = np.array([0, 0, 1, 3, 3, 3], dtype=np.int32)
    x = util.activations(rng, ids.size, k)
    y = O.gather_qmm(x, w, s, b, ids, 64, 4, threads=2)
    for r, ex in enumerate(ids):
        assert np.array_equal(y[r], O.affine_matmul(x[r:r + 1], w[ex], s[ex], b[ex], 64, 4, threads=1)[0])


def test_add_rmsnorm_restatement():
    """The add + RMSNorm restatement: unit weight and zero residual give x / rms(x) up to the two bf16 roundings;
    the sum is the bf16 rounding of the exact f32 sum; a weight scales the normed row before the last rounding."""
    rng = np.random.default_rng(9)
    m, k = 3, 512
    x = O.f32_to_bf16(rng.normal(0, 3, size=(m, k)).astype(np.float32))
    zero = np.zeros((m, k), dtype=np.uint16)
    one = O.f32_to_bf16(np.ones(k, dtype=np.float32))
    total, normed = O.add_rmsnorm(x, zero, one, 0.0)
    assert np.array_equal(total, x)
    xf = O.bf16_to_f32(x).astype(np.float64)
    want = xf / np.sqrt(np.mean(xf * xf, axis=1, keepdims=True))
    got = O.bf16_to_f32(normed).astype(np.float64)
    assert np.max(np.abs(got - want) / np.maximum(np.abs(want), 1e-3)) <= 2.0 ** -8
    r = O.f32_to_bf16(rng.normal(0, 1, size=(m, k)).astype(np.float32))
    total, _ = O.add_rmsnorm(x, r, one, 1e-6)
    assert np.array_equal(total, O.f32_to_bf16((O.bf16_to_f32(x) + O.bf16_to_f32(r)).astype(np.float32)))
    two = O.f32_to_bf16(np.full(k, 2.0, dtype=np.float32))
    _, n2 = O.add_rmsnorm(x, zero, two, 0.0)
    assert np.array_equal(O.bf16_to_f32(n2), 2.0 * O.bf16_to_f32(normed))   # a power of two commutes with the rounding
