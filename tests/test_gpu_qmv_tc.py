"""GPU parity of the tensor-memory GEMV (qmv_tc.cu) against the oracle's qmv law, through the C ABI."""
import numpy as np
import pytest
import torch

from lisa_b200 import _cabi, ops
from oracle import oracle as O
from tests import util
from tests.gpu_util import dev_bf16, dev_u32, host_bf16_bits

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _run(cuda, n, k, m, bits, seed=0, flags=_cabi.FLAG_FORCE_QMV_TC):
    rng = np.random.default_rng(seed + n + k + m)
    w, s, b = util.affine_weights(rng, n, k, bits, 64)
    x = util.activations(rng, m, k)
    y = ops.quantized_matmul(dev_bf16(x, cuda), dev_u32(w, cuda), dev_bf16(s, cuda), dev_bf16(b, cuda), True, 64, bits,
                             flags=flags)
    got = O.bf16_to_f32(host_bf16_bits(y))
    truth = O.affine_matmul(x, w, s, b, 64, bits, round_weight_bf16=False, f64=True)
    return got, truth


# config shapes (some with a cluster of k-slices and a packed ring that wraps), ragged n, short k, m up to 8 and beyond
@pytest.mark.parametrize("n,k,m,bits", [
    (128, 256, 1, 4), (256, 512, 3, 4), (1024, 2560, 1, 4), (9728, 2560, 1, 4), (2560, 9728, 4, 4), (4096, 2560, 8, 4),
    (2560, 4096, 2, 4), (200, 320, 2, 4), (8, 64, 1, 4), (768, 2048, 1, 4), (2048, 768, 11, 4),
    (128, 512, 1, 2), (17408, 5120, 1, 2), (5120, 17408, 2, 2), (136, 1088, 5, 2)])
def test_matches_oracle(cuda, n, k, m, bits):
    got, truth = _run(cuda, n, k, m, bits)
    err, l2 = util.parity(got, truth)
    assert err <= TOL, (err, l2)
    assert ops.device_status() == 0


def test_repeated_cold_launches_are_stable(cuda):
    """A ring that wraps, two CTAs per SM, weights that are not in L2: twelve different matrices in turn."""
    g = torch.Generator(device=cuda)
    g.manual_seed(0)
    n, k = 2560, 9728
    x = torch.randn((1, k), device=cuda, generator=g).to(torch.bfloat16)
    for _ in range(12):
        w = torch.randint(-2 ** 31, 2 ** 31 - 1, (n, k // 8), dtype=torch.int32, device=cuda, generator=g)
        s = (torch.randn((n, k // 64), device=cuda, generator=g) * 0.02).abs().to(torch.bfloat16)
        b = (torch.randn((n, k // 64), device=cuda, generator=g) * 0.01).to(torch.bfloat16)
        ref = ops.quantized_matmul(x, w, s, b, True, 64, 4, flags=_cabi.FLAG_FORCE_QMV).float()
        y = ops.quantized_matmul(x, w, s, b, True, 64, 4, flags=_cabi.FLAG_FORCE_QMV_TC).float()
        assert (y - ref).abs().max() <= 0.02 * ref.abs().max()


def test_rows_do_not_depend_on_m(cuda):
    """Row r of an m-row call equals the m=1 call on that row, bit for bit (array_ops.rs:500-555 contract)."""
    rng = np.random.default_rng(5)
    n, k, m = 1024, 2560, 6
    w, s, b = util.affine_weights(rng, n, k, 4, 64)
    x = util.activations(rng, m, k)
    tw, ts, tb = dev_u32(w, cuda), dev_bf16(s, cuda), dev_bf16(b, cuda)
    full = host_bf16_bits(ops.quantized_matmul(dev_bf16(x, cuda), tw, ts, tb, True, 64, 4, flags=_cabi.FLAG_FORCE_QMV_TC))
    for r in (0, 3, 5):
        one = host_bf16_bits(ops.quantized_matmul(dev_bf16(x[r:r + 1], cuda), tw, ts, tb, True, 64, 4,
                                                  flags=_cabi.FLAG_FORCE_QMV_TC))
        assert np.array_equal(one[0], full[r])


def test_unsupported_group_size_is_refused(cuda):
    rng = np.random.default_rng(1)
    w, s, b = util.affine_weights(rng, 128, 256, 4, 128)
    x = util.activations(rng, 1, 256)
    with pytest.raises(_cabi.LisaError):
        ops.quantized_matmul(dev_bf16(x, cuda), dev_u32(w, cuda), dev_bf16(s, cuda), dev_bf16(b, cuda), True, 128, 4,
                             flags=_cabi.FLAG_FORCE_QMV_TC)


# q|k|v and gate|up of configs[1]; ragged row counts; three linears; m up to 8 and beyond; 2-bit
@pytest.mark.parametrize("ns,k,m,bits", [
    ((4096, 1024, 1024), 2560, 1, 4), ((9728, 9728), 2560, 1, 4), ((200, 72), 320, 2, 4), ((128, 128, 128), 512, 8, 4),
    ((1024, 520), 2048, 11, 4), ((17408, 17408), 5120, 1, 2), ((136, 264, 8), 1088, 3, 2)])
def test_sibling_linears_in_one_launch_match_oracle_and_separate_calls(cuda, ns, k, m, bits):
    """lisa_cuda_quantized_matmul_siblings: every linear's output against the oracle (the qmv bar) and against
    its own quantized_matmul call (the same products; only the number of k-slices, hence the f32 summation
    order, may differ: one bf16 ulp)."""
    rng = np.random.default_rng(sum(ns) + k + m)
    x = util.activations(rng, m, k)
    tx = dev_bf16(x, cuda)
    host, dev = [], []
    for n in ns:
        w, s, b = util.affine_weights(rng, n, k, bits, 64)
        host.append((w, s, b))
        dev.append((dev_u32(w, cuda), dev_bf16(s, cuda), dev_bf16(b, cuda)))
    launches = ops.launch_count()
    ys = ops.quantized_matmul_siblings(tx, dev, True, 64, bits)
    assert ops.launch_count() - launches == 1  # all the linears in one launch (more than 8 rows: one GEMM launch)
    for (w, s, b), (tw, ts, tb), y in zip(host, dev, ys):
        got = O.bf16_to_f32(host_bf16_bits(y))
        truth = O.affine_matmul(x, w, s, b, 64, bits, round_weight_bf16=m > 8, f64=True)
        assert util.parity(got, truth)[0] <= TOL
        single = O.bf16_to_f32(host_bf16_bits(ops.quantized_matmul(tx, tw, ts, tb, True, 64, bits)))
        assert np.max(np.abs(got - single)) <= 2.0 ** -7 * np.max(np.abs(single))
    assert ops.device_status() == 0


def test_sibling_linears_with_many_rows_equal_separate_calls(cuda):
    rng = np.random.default_rng(77)
    ns, k, m = (256, 128), 512, 40
    x = util.activations(rng, m, k)
    tx = dev_bf16(x, cuda)
    dev = []
    for n in ns:
        w, s, b = util.affine_weights(rng, n, k, 4, 64)
        dev.append((dev_u32(w, cuda), dev_bf16(s, cuda), dev_bf16(b, cuda)))
    ys = ops.quantized_matmul_siblings(tx, dev, True, 64, 4)
    for (tw, ts, tb), y in zip(dev, ys):
        assert torch.equal(y, ops.quantized_matmul(tx, tw, ts, tb, True, 64, 4))


@pytest.mark.parametrize("ratio", [2.0 ** 6, 2.0 ** 10])
def test_heavy_tailed_activations_stay_inside_the_stated_bound(cuda, ratio):
    """The tensor-memory kernel puts the activations of a (token, 64-k group) on an integer grid of 2^-13 of the
    group's largest power of two, so an element is off by at most 2^(E-14).  With one channel per group `ratio`
    times the rest and weight rows that are zero on that channel, the row error must stay below
    sum_k |w_k| * 2^(E_g(k) - 14) plus the bf16 rounding of the output."""
    rng = np.random.default_rng(21)
    n, k, m = 512, 2560, 2
    w, s, b = util.affine_weights(rng, n, k, 4, 64)
    x = O.bf16_to_f32(util.activations(rng, m, k))
    hot = np.arange(0, k, 64) + rng.integers(0, 64, size=k // 64)
    x[:, hot] *= ratio
    xb = O.f32_to_bf16(x.astype(np.float32))
    wq = w.copy()
    for c in hot:
        wq[:, c // 8] &= ~np.uint32(0xF << (4 * (c % 8)))
    b0 = np.zeros_like(b)
    y = ops.quantized_matmul(dev_bf16(xb, cuda), dev_u32(wq, cuda), dev_bf16(s, cuda), dev_bf16(b0, cuda), True, 64, 4,
                             flags=_cabi.FLAG_FORCE_QMV_TC)
    got = O.bf16_to_f32(host_bf16_bits(y)).astype(np.float64)
    truth = O.affine_matmul(xb, wq, s, b0, 64, 4, round_weight_bf16=False, f64=True).astype(np.float64)
    wabs = np.abs(O.affine_dequantize(wq, s, b0, 64, 4, out_f32=True).astype(np.float64))          # [n, k]
    xf = O.bf16_to_f32(xb).astype(np.float64).reshape(m, k // 64, 64)
    step = 2.0 ** (np.floor(np.log2(np.abs(xf).max(axis=2))) - 14)                                  # [m, groups]
    bound = np.einsum("ngk,mg->mn", wabs.reshape(n, k // 64, 64), step) + 2.0 ** -8 * np.abs(truth) + 1e-6
    assert np.all(np.abs(got - truth) <= bound)
