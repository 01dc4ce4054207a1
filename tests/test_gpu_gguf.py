"""GPU parity of the GGUF Q2_K / Q4_K matvecs against the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch

from lisa_b200 import _cabi, ops
from oracle import oracle as O
from tests import util
from tests.gpu_util import dev_f32, dev_i32, dev_u8

pytestmark = pytest.mark.gpu

FORMATS = [("Q2K", O.Q2_K), ("Q4K", O.Q4_K)]


@pytest.mark.parametrize("name,fmt", FORMATS)
@pytest.mark.parametrize("width", [256, 1280, 2304, 5120, 8192])
def test_dense_matches_exact_dyadic_dot(cuda, name, fmt, width):
    """kernel_tests.rs:178-210: equality, not tolerance."""
    rows, tokens = 16, 3
    blocks = O.gguf_dyadic_blocks(fmt, width * rows // 256)
    w = blocks.reshape(rows, -1)
    x = O.gguf_dyadic_inputs(tokens * width).reshape(tokens, width)
    y = ops.packed_matvec(name, dev_u8(w, cuda), dev_f32(x, cuda)).cpu().numpy()
    assert np.array_equal(y, O.gguf_matvec(fmt, w, x))


@pytest.mark.parametrize("name,fmt", FORMATS)
@pytest.mark.parametrize("experts", [192, 384])
def test_expert_ids_and_broadcast_match_dense(cuda, name, fmt, experts):
    """kernel_tests.rs:212-263, including ids -1 and `experts` (exactly 0.0)."""
    width, rows, tokens, top_k = 256, 8, 3, 6
    blocks = O.gguf_dyadic_blocks(fmt, width * rows * experts // 256)
    w = blocks.reshape(experts, rows, -1)
    sel = np.array([(i * 79 + 1) % experts for i in range(tokens * top_k)], dtype=np.int32)
    sel[0], sel[1], sel[2] = experts - 1, -1, experts
    ids = sel.reshape(tokens, top_k)
    tw = dev_u8(w, cuda)
    for slots in (1, top_k):
        x = O.gguf_dyadic_inputs(tokens * slots * width).reshape(tokens, slots, width)
        y = ops.expert_matvec(name, tw, dev_f32(x, cuda), dev_i32(ids, cuda)).cpu().numpy()
        assert np.array_equal(y, O.gguf_expert_matvec(fmt, w, x, ids))
        assert np.all(y[0, 1] == 0.0) and np.all(y[0, 2] == 0.0)


@pytest.mark.parametrize("name,fmt", FORMATS)
@pytest.mark.parametrize("rows,k,tokens", [(64, 7168, 1), (72, 18432, 1), (64, 7168, 5), (8, 256, 9)])
def test_random_blocks_within_tolerance(cuda, name, fmt, rows, k, tokens):
    """Uniform random code bytes, d and dmin ~ |N(0, 0.01)|; f32 accumulate, so the bar is far below 1e-2."""
    rng = np.random.default_rng(rows + k + tokens)
    w = util.gguf_weights(rng, fmt, rows, k)
    x = rng.normal(0, 1, size=(tokens, k)).astype(np.float32)
    y = ops.packed_matvec(name, dev_u8(w, cuda), dev_f32(x, cuda)).cpu().numpy()
    dec = O.gguf_decode(fmt, w).reshape(rows, k).astype(np.float64)
    truth = x.astype(np.float64) @ dec.T
    err, l2 = util.parity(y, truth)
    assert err <= 1e-4 and l2 <= 1e-5, (err, l2)
    ref = O.gguf_matvec(fmt, w, x)
    assert util.parity(y, ref)[0] <= 1e-4


@pytest.mark.parametrize("name,fmt", FORMATS)
def test_full_size_row_slices_config5(cuda, name, fmt):
    """K=7168, N=18432 at full size: the oracle checks a strided sample of rows; the rest is
    covered by row independence (a row's result does not depend on which rows surround it)."""
    rng = np.random.default_rng(12)
    rows, k = 18432, 7168
    w = util.gguf_weights(rng, fmt, rows, k)
    x = rng.normal(0, 1, size=(1, k)).astype(np.float32)
    tw, tx = dev_u8(w, cuda), dev_f32(x, cuda)
    y = ops.packed_matvec(name, tw, tx).cpu().numpy()
    pick = np.arange(0, rows, 97)
    ref = O.gguf_matvec(fmt, np.ascontiguousarray(w[pick]), x)
    assert util.parity(y[:, pick], ref)[0] <= 1e-4
    sub = ops.packed_matvec(name, dev_u8(np.ascontiguousarray(w[1024:1024 + 64]), cuda), tx).cpu().numpy()
    # one token takes the tensor-memory kernel, whose number of k-slices follows the row count (64 rows: 8
    # slices, 18432 rows: 1): the same products in another f32 summation order
    assert util.parity(sub, y[:, 1024:1024 + 64])[0] <= 1e-5


def test_layout_rejections(cuda):
    w = torch.zeros((12, 84), dtype=torch.uint8, device=cuda)
    x = torch.zeros((1, 256), dtype=torch.float32, device=cuda)
    with pytest.raises(_cabi.LisaError, match="unsupported GGUF quantized matvec layout"):
        ops.packed_matvec("Q2K", w, x)


@pytest.mark.parametrize("name,fmt", FORMATS)
@pytest.mark.parametrize("rows,k,tokens", [(128, 1024, 32), (200, 2048, 77), (1024, 7168, 512), (256, 1024, 40)])
def test_tensor_core_matmul_within_tolerance(cuda, name, fmt, rows, k, tokens):
    """packed_matmul with a workspace and 32 tokens or more -> tcgen05 GEMM; activations and decoded
    weights each enter as two bf16 planes (hi + lo, 16 significant bits): 5e-4 max-relative and 1e-4
    relative L2 against the f64 product of the decoded blocks (observed 2e-5 .. 1.1e-4 and 5e-6 .. 2.5e-5),
    far inside the 1e-2 of the path."""
    rng = np.random.default_rng(rows + k + tokens)
    w = util.gguf_weights(rng, fmt, rows, k)
    x = rng.normal(0, 1, size=(tokens, k)).astype(np.float32)
    y = ops.packed_matmul(name, dev_u8(w, cuda), dev_f32(x, cuda)).cpu().numpy()
    dec = O.gguf_decode(fmt, w).reshape(rows, k).astype(np.float64)
    truth = x.astype(np.float64) @ dec.T
    err, l2 = util.parity(y, truth)
    assert err <= 5e-4 and l2 <= 1e-4, (err, l2)
    assert ops.device_status() == 0


@pytest.mark.parametrize("name,fmt", FORMATS)
def test_tensor_core_matmul_on_dyadic_inputs_is_exact(cuda, name, fmt):
    """The reference's dyadic construction (kernel_tests.rs:178-210) through the GEMM: weights and
    activations are exact in bf16 hi + lo planes, so the product equals the f64 dot."""
    rows, width, tokens = 128, 1024, 48
    blocks = O.gguf_dyadic_blocks(fmt, width * rows // 256)
    w = blocks.reshape(rows, -1)
    x = O.gguf_dyadic_inputs(tokens * width).reshape(tokens, width)
    y = ops.packed_matmul(name, dev_u8(w, cuda), dev_f32(x, cuda)).cpu().numpy()
    dec = O.gguf_decode(fmt, blocks).reshape(rows, width).astype(np.float64)
    assert np.array_equal(y.astype(np.float64), x.astype(np.float64) @ dec.T)


@pytest.mark.parametrize("name,fmt", FORMATS)
def test_packed_matmul_small_is_the_exact_matvec(cuda, name, fmt):
    rng = np.random.default_rng(3)
    rows, k, tokens = 64, 1024, 8
    w = util.gguf_weights(rng, fmt, rows, k)
    x = rng.normal(0, 1, size=(tokens, k)).astype(np.float32)
    a = ops.packed_matmul(name, dev_u8(w, cuda), dev_f32(x, cuda))
    b = ops.packed_matvec(name, dev_u8(w, cuda), dev_f32(x, cuda))
    assert torch.equal(a, b)


@pytest.mark.parametrize("tokens", [1, 2])
@pytest.mark.parametrize("rows,width", [(16, 256), (128, 1280), (200, 5120), (1024, 8192)])
def test_q4k_one_or_two_tokens_tensor_memory_kernel_is_exact_on_dyadic_inputs(cuda, tokens, rows, width):
    """One or two tokens of a Q4_K matrix take the tensor-memory kernel (activations as three signed
    bytes, tcgen05.mma.kind::i8): the reference's dyadic construction must still come out exactly."""
    blocks = O.gguf_dyadic_blocks(O.Q4_K, width * rows // 256)
    w = blocks.reshape(rows, -1)
    x = O.gguf_dyadic_inputs(tokens * width).reshape(tokens, width)
    y = ops.packed_matvec("Q4K", dev_u8(w, cuda), dev_f32(x, cuda)).cpu().numpy()
    assert np.array_equal(y, O.gguf_matvec(O.Q4_K, w, x))
    assert ops.device_status() == 0


@pytest.mark.parametrize("rows,k,tokens", [(18432, 7168, 1), (7168, 18432, 2), (136, 2048, 1)])
def test_q4k_one_or_two_tokens_random_blocks(cuda, rows, k, tokens):
    """K=7168 N=18432 and K=18432 N=7168 at M=1 (and 2) through the tensor-memory kernel: the matvec bar."""
    rng = np.random.default_rng(rows + k + tokens)
    w = util.gguf_weights(rng, O.Q4_K, rows, k)
    x = rng.normal(0, 1, size=(tokens, k)).astype(np.float32)
    x[0, 5] = 300.0   # an outlier: the exponent is per 32-element sub-block
    x[0, 40:72] = 0.0  # and an all-zero sub-block
    y = ops.packed_matvec("Q4K", dev_u8(w, cuda), dev_f32(x, cuda)).cpu().numpy()
    dec = O.gguf_decode(O.Q4_K, w).reshape(rows, k).astype(np.float64)
    truth = x.astype(np.float64) @ dec.T
    err, l2 = util.parity(y, truth)
    assert err <= 1e-4 and l2 <= 1e-5, (err, l2)


@pytest.mark.parametrize("rows,width", [(16, 1024), (128, 5120), (200, 8192), (1024, 2048)])
def test_q2k_one_token_tensor_memory_kernel_is_exact_on_dyadic_inputs(cuda, rows, width):
    """One token of a Q2_K matrix whose rows are whole groups of four blocks takes the tensor-memory kernel
    (2-bit codes as bytes, one accumulator column per 16-element sub-block): exact on the dyadic construction."""
    blocks = O.gguf_dyadic_blocks(O.Q2_K, width * rows // 256)
    w = blocks.reshape(rows, -1)
    x = O.gguf_dyadic_inputs(width).reshape(1, width)
    y = ops.packed_matvec("Q2K", dev_u8(w, cuda), dev_f32(x, cuda)).cpu().numpy()
    assert np.array_equal(y, O.gguf_matvec(O.Q2_K, w, x))
    assert ops.device_status() == 0


@pytest.mark.parametrize("rows,k", [(18432, 7168), (7168, 18432), (136, 2048), (64, 1024)])
def test_q2k_one_token_random_blocks(cuda, rows, k):
    rng = np.random.default_rng(rows + k)
    w = util.gguf_weights(rng, O.Q2_K, rows, k)
    x = rng.normal(0, 1, size=(1, k)).astype(np.float32)
    x[0, 5] = 300.0    # an outlier: the exponent is per 16-element sub-block
    x[0, 32:48] = 0.0  # and an all-zero sub-block
    y = ops.packed_matvec("Q2K", dev_u8(w, cuda), dev_f32(x, cuda)).cpu().numpy()
    dec = O.gguf_decode(O.Q2_K, w).reshape(rows, k).astype(np.float64)
    truth = x.astype(np.float64) @ dec.T
    err, l2 = util.parity(y, truth)
    assert err <= 1e-4 and l2 <= 1e-5, (err, l2)
    assert ops.device_status() == 0


@pytest.mark.parametrize("name,fmt", FORMATS)
@pytest.mark.parametrize("slots_shared", [True, False])
def test_expert_form_decode_sized_through_the_tensor_memory_kernel(cuda, name, fmt, slots_shared):
    """Decode-sized id tables (tokens * top_k up to 256) run every slot as a one-token tile of the tensor-memory
    kernel: exact on the dyadic construction (rows of whole 336-byte groups for Q2_K), zeros for ids outside the
    table, both input forms (one row per token, or one per slot)."""
    experts, rows, width, tokens, top_k = 24, 200, 2048, 3, 8
    blocks = O.gguf_dyadic_blocks(fmt, width * rows * experts // 256)
    w = blocks.reshape(experts, rows, -1)
    sel = np.array([(i * 7 + 1) % experts for i in range(tokens * top_k)], dtype=np.int32)
    sel[3], sel[10] = -1, experts
    ids = sel.reshape(tokens, top_k)
    slots = 1 if slots_shared else top_k
    x = O.gguf_dyadic_inputs(tokens * slots * width).reshape(tokens, slots, width)
    before = ops.launch_count()
    y = ops.expert_matvec(name, dev_u8(w, cuda), dev_f32(x, cuda), dev_i32(ids, cuda)).cpu().numpy()
    assert ops.launch_count() - before == 1
    assert np.array_equal(y, O.gguf_expert_matvec(fmt, w, x, ids))
    assert np.all(y[0, 3] == 0.0) and np.all(y[1, 2] == 0.0)
    assert ops.device_status() == 0


@pytest.mark.parametrize("name,fmt", FORMATS)
def test_expert_form_random_blocks(cuda, name, fmt):
    """The routed down projection of the GGUF checkpoints' geometry (2048 -> 4096, top-8, one token) on random
    blocks against the f64 product of the decoded rows."""
    rng = np.random.default_rng(11 + fmt)
    experts, rows, k, top_k = 12, 4096, 2048, 8
    w = util.gguf_weights(rng, fmt, rows, k, experts=experts)
    x = rng.normal(0, 1, size=(1, top_k, k)).astype(np.float32)
    ids = rng.choice(experts, size=(1, top_k), replace=False).astype(np.int32)
    y = ops.expert_matvec(name, dev_u8(w.reshape(experts, rows, -1), cuda), dev_f32(x, cuda), dev_i32(ids, cuda)).cpu().numpy()
    for j in range(top_k):
        dec = O.gguf_decode(fmt, w[ids[0, j]].reshape(rows, -1)).reshape(rows, k).astype(np.float64)
        truth = dec @ x[0, j].astype(np.float64)
        err, l2 = util.parity(y[0, j], truth)
        assert err <= 1e-4 and l2 <= 1e-5, (j, err, l2)
    assert ops.device_status() == 0


@pytest.mark.parametrize("width", [256, 1280, 5120])
def test_q5k_dense_and_expert_forms_are_exact_on_dyadic_inputs(cuda, width):
    """Q5_K (quant.rs:161-182): the warp-per-row kernel on the reference's dyadic construction, dense with 1 and 3
    tokens and the expert form with ids outside the table."""
    fmt, name = O.Q5_K, "Q5K"
    rows = 16
    blocks = O.gguf_dyadic_blocks(fmt, width * rows // 256)
    w = blocks.reshape(rows, -1)
    for tokens in (1, 3):
        x = O.gguf_dyadic_inputs(tokens * width).reshape(tokens, width)
        y = ops.packed_matvec(name, dev_u8(w, cuda), dev_f32(x, cuda)).cpu().numpy()
        assert np.array_equal(y, O.gguf_matvec(fmt, w, x))
    experts, tokens, top_k = 12, 2, 4
    eb = O.gguf_dyadic_blocks(fmt, width * 8 * experts // 256).reshape(experts, 8, -1)
    ids = np.array([[0, 5, -1, 11], [experts, 3, 3, 7]], dtype=np.int32)
    x = O.gguf_dyadic_inputs(tokens * top_k * width).reshape(tokens, top_k, width)
    y = ops.expert_matvec(name, dev_u8(eb, cuda), dev_f32(x, cuda), dev_i32(ids, cuda)).cpu().numpy()
    assert np.array_equal(y, O.gguf_expert_matvec(fmt, eb, x, ids))
    assert np.all(y[0, 2] == 0.0) and np.all(y[1, 0] == 0.0)


def test_q5k_random_blocks(cuda):
    rng = np.random.default_rng(21)
    rows, k, tokens = 72, 7168, 5
    w = rng.integers(0, 256, size=(rows, k // 256, 176), dtype=np.uint8)
    d = O.f32_to_f16_bits(np.abs(rng.normal(0, 0.01, size=(rows, k // 256, 2))).astype(np.float32))
    w[..., 0], w[..., 1] = d[..., 0] & 0xFF, d[..., 0] >> 8
    w[..., 2], w[..., 3] = d[..., 1] & 0xFF, d[..., 1] >> 8
    w = np.ascontiguousarray(w.reshape(rows, -1))
    x = rng.normal(0, 1, size=(tokens, k)).astype(np.float32)
    y = ops.packed_matvec("Q5K", dev_u8(w, cuda), dev_f32(x, cuda)).cpu().numpy()
    dec = O.gguf_decode(O.Q5_K, w).reshape(rows, k).astype(np.float64)
    err, l2 = util.parity(y, x.astype(np.float64) @ dec.T)
    assert err <= 1e-4 and l2 <= 1e-5, (err, l2)
    # the tensor-core product has no Q5_K decoder: many tokens run as matvecs and give the same law
    xm = rng.normal(0, 1, size=(40, k)).astype(np.float32)
    ym = ops.packed_matmul("Q5K", dev_u8(w, cuda), dev_f32(xm, cuda)).cpu().numpy()
    err, l2 = util.parity(ym, xm.astype(np.float64) @ dec.T)
    assert err <= 1e-4 and l2 <= 1e-5, (err, l2)
