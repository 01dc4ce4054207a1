"""GPU parity of the affine path (dequantize, qmv, serial rows) against the CPU oracle,
through the C ABI.  Tolerance on outputs: |y - ref| <= 1e-2 * max(|ref|, rms(ref)) against
the f64 contraction (max-relative 1e-2, fp32 accumulate, bf16 out); dequantized weights
bit-exact."""
import numpy as np
import pytest
import torch

from lisa_b200 import _cabi, ops
from oracle import oracle as O
from tests import util
from tests.gpu_util import dev_bf16, dev_u32, host_bf16_bits

pytestmark = pytest.mark.gpu

TOL = 1e-2


def _upload(dev, w, s, b, x=None):
    out = [dev_u32(w, dev), dev_bf16(s, dev), dev_bf16(b, dev)]
    if x is not None:
        out.append(dev_bf16(x, dev))
    return out


@pytest.mark.parametrize("bits", [2, 4, 8])
@pytest.mark.parametrize("gs", [32, 64, 128])
def test_dequantize_bit_exact(cuda, bits, gs):
    rng = np.random.default_rng(bits * 1000 + gs)
    n, k = 37, 768
    w, s, b = util.affine_weights(rng, n, k, bits, gs)
    tw, ts, tb = _upload(cuda, w, s, b)
    got = host_bf16_bits(ops.dequantize(tw, ts, tb, gs, bits))
    assert np.array_equal(got, O.affine_dequantize(w, s, b, gs, bits))


def test_dequantize_leading_axes_and_large(cuda):
    rng = np.random.default_rng(11)
    w, s, b = util.affine_weights(rng, 64, 2560, 4, 64, experts=3)
    tw, ts, tb = _upload(cuda, w, s, b)
    got = host_bf16_bits(ops.dequantize(tw, ts, tb, 64, 4))
    assert got.shape == (3, 64, 2560)
    assert np.array_equal(got, O.affine_dequantize(w, s, b, 64, 4))


def _check_qmm(cuda, n, k, m, bits, gs, flags, seed=0):
    rng = np.random.default_rng(seed + n + k + m)
    w, s, b = util.affine_weights(rng, n, k, bits, gs)
    x = util.activations(rng, m, k)
    tw, ts, tb, tx = _upload(cuda, w, s, b, x)
    y = ops.quantized_matmul(tx, tw, ts, tb, True, gs, bits, flags=flags)
    torch.cuda.synchronize()
    got_bits = host_bf16_bits(y)
    assert got_bits.shape == (m, n)
    truth = O.affine_matmul(x, w, s, b, gs, bits, round_weight_bf16=False, f64=True)
    err, l2 = util.parity(O.bf16_to_f32(got_bits), truth)
    assert err <= TOL, f"n={n} k={k} m={m} bits={bits} gs={gs} flags={flags}: err {err:.3e} l2 {l2:.3e}"
    # against the reference-shaped CPU result as well (bf16 on both sides): a few ULPs at most
    ref_bits = O.affine_matmul(x, w, s, b, gs, bits, round_weight_bf16=False)
    err2, _ = util.parity(O.bf16_to_f32(got_bits), O.bf16_to_f32(ref_bits))
    assert err2 <= TOL
    return got_bits


QMV_SHAPES = [
    # (n, k) — 9728 x 2560 and the other Qwen3-4B-shaped projections, then ragged cases
    (9728, 2560), (1024, 2560), (2560, 4096), (2560, 9728),
    (2048, 768), (768, 2048),       # config 4 expert shapes; K=768 is not a multiple of 512
    (8, 64), (1, 128), (13, 192), (1001, 512), (300, 5120),
]


@pytest.mark.parametrize("n,k", QMV_SHAPES)
@pytest.mark.parametrize("bits", [4, 2])
def test_qmv_stream_m1(cuda, n, k, bits):
    _check_qmm(cuda, n, k, 1, bits, 64, _cabi.FLAG_FORCE_QMV)
    assert ops.device_status() == 0


@pytest.mark.parametrize("n,k", [(9728, 2560), (13, 192), (2048, 768)])
@pytest.mark.parametrize("bits", [4, 2])
def test_qmv_simple_m1(cuda, n, k, bits):
    _check_qmm(cuda, n, k, 1, bits, 64, _cabi.FLAG_FORCE_QMV_SIMPLE)


@pytest.mark.parametrize("gs", [32, 128])
@pytest.mark.parametrize("bits", [4, 2])
def test_qmv_other_group_sizes(cuda, gs, bits):
    _check_qmm(cuda, 520, 1024, 1, bits, gs, _cabi.FLAG_FORCE_QMV)
    _check_qmm(cuda, 520, 1024, 3, bits, gs, _cabi.FLAG_FORCE_QMV_SIMPLE)


@pytest.mark.parametrize("m", [2, 3, 4, 5, 8])
@pytest.mark.parametrize("bits", [4, 2])
def test_qmv_small_batches(cuda, m, bits):
    _check_qmm(cuda, 1536, 2560, m, bits, 64, _cabi.FLAG_FORCE_QMV)
    _check_qmm(cuda, 24, 768, m, bits, 64, _cabi.FLAG_FORCE_QMV)
    assert ops.device_status() == 0


def test_qmv_with_programmatic_launch_chain(cuda):
    """Back-to-back launches with programmatic stream serialization give the same bits as
    ordinary launches (each kernel prefetches weights while the previous one drains)."""
    rng = np.random.default_rng(5)
    k = 2560
    layers = [util.affine_weights(rng, n, k, 4, 64) for n in (4096, 1024, 1024, 9728)]
    x = util.activations(rng, 1, k)
    tx = dev_bf16(x, cuda)
    dev_layers = [_upload(cuda, *l) for l in layers]
    plain = [ops.quantized_matmul(tx, *dl, True, 64, 4, flags=_cabi.FLAG_FORCE_QMV) for dl in dev_layers]
    torch.cuda.synchronize()
    for _ in range(3):
        chained = [ops.quantized_matmul(tx, *dl, True, 64, 4, flags=_cabi.FLAG_FORCE_QMV | _cabi.FLAG_PDL)
                   for dl in dev_layers]
    torch.cuda.synchronize()
    for a, c in zip(plain, chained):
        assert torch.equal(a.view(torch.int16), c.view(torch.int16))
    assert ops.device_status() == 0


@pytest.mark.parametrize("bits", [4, 2])
def test_serial_rows_bit_identical_to_single_rows(cuda, bits):
    """array_ops.rs:650-710: a row batch equals independent serial calls bit for bit."""
    rng = np.random.default_rng(6)
    n, k, rows = 512, 1024, 7
    w, s, b = util.affine_weights(rng, n, k, bits, 64)
    x = util.activations(rng, rows, k)
    tw, ts, tb, tx = _upload(cuda, w, s, b, x)
    batch = ops.quantized_matmul_serial_rows(tx.reshape(rows, 1, k), tw, ts, tb, True, 64, bits)
    assert batch.shape == (rows, 1, n)
    for r in range(rows):
        one = ops.quantized_matmul(tx[r:r + 1], tw, ts, tb, True, 64, bits)
        assert torch.equal(batch[r, 0].view(torch.int16), one[0].view(torch.int16))


def test_row_permutation_is_bit_exact(cuda):
    """array_ops.rs:1243-1323: permuting weight rows permutes outputs, nothing else."""
    rng = np.random.default_rng(7)
    n, k = 1024, 2560
    w, s, b = util.affine_weights(rng, n, k, 4, 64)
    x = util.activations(rng, 1, k)
    perm = rng.permutation(n)
    tw, ts, tb, tx = _upload(cuda, w, s, b, x)
    pw, ps, pb = _upload(cuda, w[perm], s[perm], b[perm])
    y = host_bf16_bits(ops.quantized_matmul(tx, tw, ts, tb, True, 64, 4))
    yp = host_bf16_bits(ops.quantized_matmul(tx, pw, ps, pb, True, 64, 4))
    assert np.array_equal(yp[0], y[0][perm])


def test_run_twice_same_bits(cuda):
    got1 = _check_qmm(cuda, 4096, 2560, 1, 4, 64, 0, seed=3)
    got2 = _check_qmm(cuda, 4096, 2560, 1, 4, 64, 0, seed=3)
    assert np.array_equal(got1, got2)


def test_full_size_linearity_config1(cuda):
    """Size-independent property at 9728 x 2560, one row: y(x1 + x2) == y(x1) + y(x2) up to
    rounding when x1, x2 and their sum are bf16-exact, and y(0) == 0."""
    rng = np.random.default_rng(8)
    n, k = 9728, 2560
    w, s, b = util.affine_weights(rng, n, k, 4, 64)
    x1 = (rng.integers(-8, 9, size=(1, k)) / 4.0).astype(np.float32)
    x2 = (rng.integers(-8, 9, size=(1, k)) / 4.0).astype(np.float32)
    tw, ts, tb = _upload(cuda, w, s, b)
    ys = []
    for xv in (x1, x2, x1 + x2, np.zeros_like(x1)):
        tx = dev_bf16(O.f32_to_bf16(xv), cuda)
        ys.append(ops.quantized_matmul(tx, tw, ts, tb, True, 64, 4).float().cpu().numpy())
    assert np.all(ys[3] == 0)
    err, _ = util.parity(ys[2], ys[0] + ys[1])
    assert err <= TOL


def test_non_cuda_tensor_is_refused():
    w = torch.zeros((8, 8), dtype=torch.int32)
    s = torch.zeros((8, 1), dtype=torch.bfloat16)
    x = torch.zeros((1, 64), dtype=torch.bfloat16)
    with pytest.raises(_cabi.LisaError):
        ops.quantized_matmul(x, w, s, s, True, 64, 4)


@pytest.mark.parametrize("ns,k,m,bits", [((200, 1024, 72), 2048, 300, 4), ((4096, 1024, 1024), 2560, 512, 4),
                                          ((136, 264), 1088, 40, 2), ((256, 128), 512, 40, 4)])
def test_sibling_linears_as_one_gemm_launch(cuda, ns, k, m, bits):
    """lisa_cuda_quantized_matmul_siblings with many rows: one tensor-core GEMM launch for all the linears;
    every output against the oracle's GEMM law (weights rounded to bf16) and against its own
    quantized_matmul call (same products; the number of k-slices may differ: one bf16 ulp)."""
    from lisa_b200 import _cabi

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
    assert ops.launch_count() - launches == 1
    for (w, s, b), (tw, ts, tb), y in zip(host, dev, ys):
        got = O.bf16_to_f32(host_bf16_bits(y))
        truth = O.affine_matmul(x, w, s, b, 64, bits, round_weight_bf16=True, f64=True)
        assert util.parity(got, truth)[0] <= 1e-2
        single = O.bf16_to_f32(host_bf16_bits(ops.quantized_matmul(tx, tw, ts, tb, True, 64, bits, flags=_cabi.FLAG_FORCE_QMM)))
        assert np.max(np.abs(got - single)) <= 2.0 ** -7 * np.max(np.abs(single))
    assert ops.device_status() == 0
