"""GPU parity of the tcgen05 prefill GEMM against the CPU oracle (rounded-weight law:
w = bf16(f32(q)*scale + bias), f32 accumulate, bf16 out), through the C ABI."""
import numpy as np
import pytest
import torch

from lisa_b200 import _cabi, ops
from oracle import oracle as O
from tests import util
from tests.gpu_util import dev_bf16, dev_u32, host_bf16_bits

pytestmark = pytest.mark.gpu

TOL = 1e-2


def _run(cuda, n, k, m, bits, gs, seed=0, rows=None, flags=_cabi.FLAG_FORCE_QMM):
    rng = np.random.default_rng(seed + n * 7 + k * 3 + m)
    w, s, b = util.affine_weights(rng, n, k, bits, gs)
    x = util.activations(rng, m, k)
    y = ops.quantized_matmul(dev_bf16(x, cuda), dev_u32(w, cuda), dev_bf16(s, cuda), dev_bf16(b, cuda), True, gs, bits,
                             flags=flags)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    got = O.bf16_to_f32(host_bf16_bits(y))
    assert got.shape == (m, n)
    pick = np.arange(n) if rows is None else rows
    truth = O.affine_matmul(x, np.ascontiguousarray(w[pick]), np.ascontiguousarray(s[pick]),
                            np.ascontiguousarray(b[pick]), gs, bits, round_weight_bf16=True, f64=True)
    err, l2 = util.parity(got[:, pick], truth)
    assert err <= TOL and l2 <= 3e-3, f"n={n} k={k} m={m} bits={bits} gs={gs}: err {err:.3e} l2 {l2:.3e}"
    return got


@pytest.mark.parametrize("bits", [4, 2])
@pytest.mark.parametrize("n,k,m", [(128, 64, 16), (128, 256, 16), (256, 512, 48), (128, 1024, 256)])
def test_qmm_single_tiles(cuda, bits, n, k, m):
    _run(cuda, n, k, m, bits, 64)


@pytest.mark.parametrize("bits", [4, 2])
@pytest.mark.parametrize("n,k,m", [(200, 320, 33), (1000, 768, 5), (136, 2048, 300), (72, 192, 513)])
def test_qmm_ragged_shapes(cuda, bits, n, k, m):
    """Row, column and k tails: n % 128, m % 16 and k % 256 all non-zero."""
    _run(cuda, n, k, m, bits, 64)


@pytest.mark.parametrize("gs", [32, 128])
@pytest.mark.parametrize("bits", [4, 2])
def test_qmm_group_sizes(cuda, gs, bits):
    _run(cuda, 256, 1024, 64, bits, gs)
    if gs == 32:
        if bits == 4:
            _run(cuda, 128, 96, 16, bits, gs)  # k not a multiple of 64 (2-bit rows would be 24 bytes: refused)


@pytest.mark.parametrize("n,k", [(4096, 2560), (2560, 9728)])
def test_qmm_prefill_config2(cuda, n, k):
    """The Qwen3-4B-shaped prefill, M = 2048; the oracle checks 48 weight rows spread over the
    tiles (every token), row independence covers the rest."""
    rows = np.unique(np.concatenate([np.arange(0, n, n // 40), [n - 1, 127, 128]]))
    _run(cuda, n, k, 2048, 4, 64, rows=rows)


def test_qmm_config3_2bit_m512(cuda):
    n, k = 5120, 17408
    rows = np.arange(0, n, 160)
    _run(cuda, n, k, 512, 2, 64, rows=rows)


def test_qmm_default_dispatch_uses_gemm_for_large_m(cuda):
    before = ops.launch_count()
    a = _run(cuda, 512, 1024, 64, 4, 64, flags=0)
    assert ops.launch_count() - before == 1
    b = _run(cuda, 512, 1024, 64, 4, 64, flags=_cabi.FLAG_FORCE_QMM)
    assert np.array_equal(a, b)


def test_qmm_matches_dequantize_then_dense_matmul(cuda):
    """quantized_matmul vs dequantize + matmul (crates/lisa-engine/src/models/qwen4/smoke.rs:19-42);
    torch's bf16 GEMM is the dense reference here."""
    rng = np.random.default_rng(9)
    n, k, m = 768, 2048, 192
    w, s, b = util.affine_weights(rng, n, k, 4, 64)
    x = util.activations(rng, m, k)
    tw, ts, tb, tx = dev_u32(w, cuda), dev_bf16(s, cuda), dev_bf16(b, cuda), dev_bf16(x, cuda)
    y = ops.quantized_matmul(tx, tw, ts, tb, True, 64, 4, flags=_cabi.FLAG_FORCE_QMM).float()
    dense = (tx.float() @ ops.dequantize(tw, ts, tb, 64, 4).float().T)
    err, _ = util.parity(y.cpu().numpy(), dense.cpu().numpy())
    assert err <= TOL
