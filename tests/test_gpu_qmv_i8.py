"""GPU parity of the integer mma.sync GEMV (qmv_i8.cu) against the oracle's qmv law, through the C ABI."""
import numpy as np
import pytest
import torch

from lisa_b200 import _cabi, ops
from oracle import oracle as O
from tests import util
from tests.gpu_util import dev_bf16, dev_u32, host_bf16_bits

pytestmark = pytest.mark.gpu
TOL = 1e-2
I8 = _cabi.FLAG_FORCE_QMV_I8


def _run(cuda, n, k, m, bits, seed=0, flags=I8):
    rng = np.random.default_rng(seed + n + k + m)
    w, s, b = util.affine_weights(rng, n, k, bits, 64)
    x = util.activations(rng, m, k)
    y = ops.quantized_matmul(dev_bf16(x, cuda), dev_u32(w, cuda), dev_bf16(s, cuda), dev_bf16(b, cuda), True, 64, bits,
                             flags=flags)
    got = O.bf16_to_f32(host_bf16_bits(y))
    truth = O.affine_matmul(x, w, s, b, 64, bits, round_weight_bf16=False, f64=True)
    return got, truth


# the decode shapes of the 4-bit stack (q, o, gate, down) and of the 2-bit stack (gate, down), ragged row counts
# (a 16-row box plus single-row boxes, fewer rows than a tile), a k of one ring stage, 1..8 rows and more
@pytest.mark.parametrize("n,k,m,bits", [
    (128, 512, 1, 4), (256, 512, 3, 4), (1024, 2560, 1, 4), (9728, 2560, 1, 4), (2560, 9728, 1, 4), (2560, 9728, 4, 4),
    (4096, 2560, 8, 4), (2560, 4096, 2, 4), (200, 1024, 2, 4), (8, 512, 1, 4), (768, 2048, 5, 4), (2048, 1536, 11, 4),
    (4728, 2560, 7, 4), (17, 512, 6, 4),
    (128, 512, 1, 2), (17408, 5120, 1, 2), (136, 1024, 5, 2), (1000, 2560, 8, 2)])
def test_matches_oracle(cuda, n, k, m, bits):
    got, truth = _run(cuda, n, k, m, bits)
    err, l2 = util.parity(got, truth)
    assert err <= TOL, (err, l2)
    assert ops.device_status() == 0


def test_default_dispatch_takes_the_decode_shapes(cuda):
    """No flag: the dispatch of quantized_matmul on the decode shapes of the 4-bit stack (one row)."""
    for n, k in ((4096, 2560), (1024, 2560), (2560, 4096), (9728, 2560), (2560, 9728)):
        got, truth = _run(cuda, n, k, 1, 4, seed=3, flags=0)
        err, l2 = util.parity(got, truth)
        assert err <= TOL, (n, k, err, l2)


def test_repeated_cold_launches_are_stable(cuda):
    """A ring that wraps many times, weights that are not in L2: twelve different matrices in turn, compared
    with the bf16 mma.sync kernel."""
    g = torch.Generator(device=cuda)
    g.manual_seed(0)
    n, k = 2560, 9728
    x = torch.randn((1, k), device=cuda, generator=g).to(torch.bfloat16)
    for _ in range(12):
        w = torch.randint(-2 ** 31, 2 ** 31 - 1, (n, k // 8), dtype=torch.int32, device=cuda, generator=g)
        s = (torch.randn((n, k // 64), device=cuda, generator=g) * 0.02).abs().to(torch.bfloat16)
        b = (torch.randn((n, k // 64), device=cuda, generator=g) * 0.01).to(torch.bfloat16)
        ref = ops.quantized_matmul(x, w, s, b, True, 64, 4, flags=_cabi.FLAG_FORCE_QMV).float()
        y = ops.quantized_matmul(x, w, s, b, True, 64, 4, flags=I8).float()
        assert (y - ref).abs().max() <= 0.02 * ref.abs().max()


def test_rows_do_not_depend_on_m(cuda):
    """Row r of an m-row call equals the m=1 call on that row, bit for bit (array_ops.rs:500-555 contract)."""
    rng = np.random.default_rng(5)
    n, k, m = 1024, 2560, 7
    w, s, b = util.affine_weights(rng, n, k, 4, 64)
    x = util.activations(rng, m, k)
    tw, ts, tb = dev_u32(w, cuda), dev_bf16(s, cuda), dev_bf16(b, cuda)
    full = host_bf16_bits(ops.quantized_matmul(dev_bf16(x, cuda), tw, ts, tb, True, 64, 4, flags=I8))
    for r in (0, 3, 4, 6):
        one = host_bf16_bits(ops.quantized_matmul(dev_bf16(x[r:r + 1], cuda), tw, ts, tb, True, 64, 4, flags=I8))
        assert np.array_equal(one[0], full[r])


def test_row_permutation_permutes_outputs(cuda):
    """Permuting the rows of W permutes y bit for bit (array_ops.rs:1243-1323): a row's sum does not depend on
    where the row sits in the matrix or in the grid."""
    rng = np.random.default_rng(11)
    n, k = 2560, 4096
    w, s, b = util.affine_weights(rng, n, k, 4, 64)
    x = util.activations(rng, 1, k)
    perm = rng.permutation(n)
    y = host_bf16_bits(ops.quantized_matmul(dev_bf16(x, cuda), dev_u32(w, cuda), dev_bf16(s, cuda), dev_bf16(b, cuda),
                                            True, 64, 4, flags=I8))
    yp = host_bf16_bits(ops.quantized_matmul(dev_bf16(x, cuda), dev_u32(w[perm], cuda), dev_bf16(s[perm], cuda),
                                             dev_bf16(b[perm], cuda), True, 64, 4, flags=I8))
    assert np.array_equal(yp[0], y[0][perm])


def test_unsupported_shapes_are_refused(cuda):
    rng = np.random.default_rng(1)
    for n, k, gs in ((128, 256, 128), (128, 768, 64)):
        w, s, b = util.affine_weights(rng, n, k, 4, gs)
        x = util.activations(rng, 1, k)
        with pytest.raises(_cabi.LisaError):
            ops.quantized_matmul(dev_bf16(x, cuda), dev_u32(w, cuda), dev_bf16(s, cuda), dev_bf16(b, cuda), True, gs, 4,
                                 flags=I8)


# q|k|v and gate|up of the 4-bit stack; ragged row counts; three linears; up to 8 rows and beyond; 2-bit
@pytest.mark.parametrize("ns,k,m,bits", [
    ((4096, 1024, 1024), 2560, 1, 4), ((9728, 9728), 2560, 1, 4), ((200, 72), 512, 2, 4), ((128, 128, 128), 512, 8, 4),
    ((1024, 520), 2048, 11, 4), ((17408, 17408), 5120, 1, 2), ((136, 264, 8), 1024, 3, 2)])
def test_sibling_linears_in_one_launch_match_oracle_and_separate_calls(cuda, ns, k, m, bits):
    rng = np.random.default_rng(sum(ns) + k + m)
    x = util.activations(rng, m, k)
    tx = dev_bf16(x, cuda)
    host, devs = [], []
    for n in ns:
        w, s, b = util.affine_weights(rng, n, k, bits, 64)
        host.append((w, s, b))
        devs.append((dev_u32(w, cuda), dev_bf16(s, cuda), dev_bf16(b, cuda)))
    before = ops.launch_count()
    ys = ops.quantized_matmul_siblings(tx, devs, True, 64, bits, flags=I8)
    if m <= 8:  # (more rows go to one call per linear)
        assert ops.launch_count() - before == 1
    for y, (w, s, b), d in zip(ys, host, devs):
        got_bits = host_bf16_bits(y)
        err, l2 = util.parity(O.bf16_to_f32(got_bits), O.affine_matmul(x, w, s, b, 64, bits, round_weight_bf16=False, f64=True))
        assert err <= TOL, (err, l2)
        # the same rows through a call of their own: the same sums up to the order of the warps' partial sums
        alone = host_bf16_bits(ops.quantized_matmul(tx, *d, True, 64, bits, flags=I8))
        assert util.bf16_ulp_distance(alone, got_bits) <= 1
    assert ops.device_status() == 0


@pytest.mark.parametrize("ratio", [2.0 ** 10, 2.0 ** 12])
def test_heavy_tailed_activations(cuda, ratio):
    """One channel per 64-k group carries an activation `ratio` times the others, and the weight rows carry code
    0 and bias 0 on that channel's group... the remaining elements of the group are then represented on the
    integer grid of the outlier (2^-14 of it).  The result is compared with the f64 contraction of the
    unrounded activations at the tolerance of every other test."""
    rng = np.random.default_rng(21)
    n, k, m = 512, 2560, 2
    w, s, b = util.affine_weights(rng, n, k, 4, 64)
    x = O.bf16_to_f32(util.activations(rng, m, k))
    hot = np.arange(0, k, 64) + rng.integers(0, 64, size=k // 64)  # one channel per group
    x[:, hot] *= ratio
    xb = O.f32_to_bf16(x.astype(np.float32))
    # the rows see nothing of the hot channels: their codes are 0 there, and every bias is 0
    wq = w.copy()
    for c in hot:
        wq[:, c // 8] &= ~np.uint32(0xF << (4 * (c % 8)))
    b0 = np.zeros_like(b)
    y = ops.quantized_matmul(dev_bf16(xb, cuda), dev_u32(wq, cuda), dev_bf16(s, cuda), dev_bf16(b0, cuda), True, 64, 4,
                             flags=I8)
    got = O.bf16_to_f32(host_bf16_bits(y))
    truth = O.affine_matmul(xb, wq, s, b0, 64, 4, round_weight_bf16=False, f64=True)
    err, l2 = util.parity(got, truth)
    assert err <= TOL, (ratio, err, l2)
