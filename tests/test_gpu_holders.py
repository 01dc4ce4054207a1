"""GPU tests of the holders and loaders around the kernels: ops.quantize against the oracle's restatement of the
reference's host loop (bit for bit), QuantizedEmbedding (row-indexed dequantize, tied head), 8-bit weights, and
real files: a safetensors triplet and a GGUF tensor read by the C++ readers and run through the kernels."""
import json
import struct

import numpy as np
import pytest
import torch

from lisa_b200 import ops
from lisa_b200.files import GgufPackage, Shard, TensorType
from lisa_b200.quant import QuantizedEmbedding, QuantizedLinear
from oracle import oracle as O
from tests import util
from tests.gpu_util import dev_bf16, dev_f32, dev_u32, host_bf16_bits
from tests.test_files import gguf_bytes, st_bytes

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("bits,gs", [(4, 64), (2, 64), (8, 64), (4, 32), (4, 128)])
def test_quantize_is_the_reference_host_loop_bit_for_bit(cuda, bits, gs):
    rng = np.random.default_rng(bits * 100 + gs)
    rows, k = 37, 512
    w = O.f32_to_bf16(rng.normal(0, 0.05, size=(rows, k)).astype(np.float32))
    w[3, :gs] = 0               # an all-zero group: scale eps, bias 0
    w[5, 64:128] = w[5, 64]     # a constant group
    wq, s, b = ops.quantize(dev_bf16(w, cuda), gs, bits)
    rq, rs, rb = O.affine_quantize(O.bf16_to_f32(w), gs, bits)
    assert np.array_equal(wq.cpu().numpy().view(np.uint32), rq)
    assert np.array_equal(host_bf16_bits(s), O.f32_to_bf16(rs)) and np.array_equal(host_bf16_bits(b), O.f32_to_bf16(rb))
    # and the round trip: dequantize(quantize(w)) stays within half a step of w, plus the bf16 rounding of the
    # scale (times the largest code) and of the bias
    back = O.bf16_to_f32(host_bf16_bits(ops.dequantize(wq, s, b, gs, bits)))
    step = np.repeat(np.abs(O.bf16_to_f32(host_bf16_bits(s))), gs, axis=1)
    wf = O.bf16_to_f32(w)
    edge = np.repeat(np.abs(wf).reshape(rows, k // gs, gs).max(axis=2), gs, axis=1)
    # (the far edge of a group can sit up to a step outside the grid: the scale is re-fitted to the near edge)
    assert np.all(np.abs(back - wf) <= 1.01 * step + 2.0 ** -6 * edge + 1e-6)
    with pytest.raises(ops.LisaError, match="incompatible with K"):
        ops.quantize(dev_bf16(w, cuda), 48, bits)


def test_quantized_embedding_forward_and_tied_head(cuda):
    rng = np.random.default_rng(4)
    vocab, k = 1000, 1024
    w, s, b = util.affine_weights(rng, vocab, k, 4, 64)
    emb = QuantizedEmbedding(dev_u32(w, cuda), dev_bf16(s, cuda), dev_bf16(b, cuda), 64, 4)
    ids = np.array([[0, 999, 17], [17, 500, 3]], dtype=np.int64)
    rows = emb.forward(torch.from_numpy(ids).to(cuda))
    assert rows.shape == (2, 3, k)
    table = O.affine_dequantize(w, s, b, 64, 4)
    assert np.array_equal(host_bf16_bits(rows).reshape(6, k), table[ids.reshape(-1)])
    bad = emb.forward(torch.tensor([vocab, -1], device=cuda))
    assert torch.all(bad == 0)
    x = util.activations(rng, 2, k)
    y = emb.as_linear(dev_bf16(x, cuda))
    err, l2 = util.parity(O.bf16_to_f32(host_bf16_bits(y)), O.affine_matmul(x, w, s, b, 64, 4, round_weight_bf16=False, f64=True))
    assert err <= 1e-2, (err, l2)


@pytest.mark.parametrize("m", [1, 5, 40])
@pytest.mark.parametrize("gs", [64, 32])
def test_eight_bit_weights(cuda, m, gs):
    """8-bit affine weights (the lm-head case of the reference's test loop over bits 2, 4, 8)."""
    rng = np.random.default_rng(m + gs)
    n, k = 264, 1024
    w, s, b = util.affine_weights(rng, n, k, 8, gs)
    x = util.activations(rng, m, k)
    y = ops.quantized_matmul(dev_bf16(x, cuda), dev_u32(w, cuda), dev_bf16(s, cuda), dev_bf16(b, cuda), True, gs, 8)
    err, l2 = util.parity(O.bf16_to_f32(host_bf16_bits(y)), O.affine_matmul(x, w, s, b, gs, 8, round_weight_bf16=False, f64=True))
    assert err <= 1e-2, (err, l2)


def test_safetensors_triplet_to_linear(cuda, tmp_path):
    rng = np.random.default_rng(8)
    n, k = 256, 2560
    w, s, b = util.affine_weights(rng, n, k, 4, 32)   # group 32: detected from the shapes, not taken from a config
    path = tmp_path / "model.safetensors"
    path.write_bytes(st_bytes({"layers.0.mlp.gate_proj.weight": ("U32", w), "layers.0.mlp.gate_proj.scales": ("BF16", s),
                               "layers.0.mlp.gate_proj.biases": ("BF16", b)}))
    shard = Shard.open(str(path))
    lin = QuantizedLinear.load(shard, "layers.0.mlp", "gate_proj", device=cuda)
    assert lin.group_size == 32 and lin.bits == 4 and lin.dims_out() == n
    x = util.activations(rng, 3, k)
    y = lin.forward(dev_bf16(x, cuda))
    err, l2 = util.parity(O.bf16_to_f32(host_bf16_bits(y)), O.affine_matmul(x, w, s, b, 32, 4, round_weight_bf16=False, f64=True))
    assert err <= 1e-2, (err, l2)
    shard.close()


@pytest.mark.parametrize("fmt,kind,name", [(O.Q4_K, TensorType.Q4_K, "Q4K"), (O.Q2_K, TensorType.Q2_K, "Q2K")])
def test_gguf_file_to_matvec(cuda, tmp_path, fmt, kind, name):
    """A .gguf file on disk -> header parse -> mapping -> [rows, row_bytes] view on the device -> packed_matvec,
    and the expert form from a rank-3 tensor."""
    rng = np.random.default_rng(fmt)
    rows, k, experts = 64, 1024, 3
    dense = util.gguf_weights(rng, fmt, rows, k)
    stack = util.gguf_weights(rng, fmt, rows, k, experts=experts)
    pad = -dense.nbytes % 32
    payload = dense.tobytes() + bytes(pad) + stack.tobytes()
    path = tmp_path / "w.gguf"
    path.write_bytes(gguf_bytes([("blk.0.ffn_down.weight", [k, rows], kind, 0),
                                 ("blk.0.ffn_down_exps.weight", [k, rows, experts], kind, dense.nbytes + pad)], payload))
    pkg = GgufPackage.open(str(path))
    wd = pkg.device_weights("blk.0.ffn_down.weight", cuda)
    assert tuple(wd.shape) == (rows, dense.shape[1])
    x = rng.normal(0, 1, size=(2, k)).astype(np.float32)
    y = ops.packed_matvec(name, wd, dev_f32(x, cuda)).cpu().numpy()
    assert util.parity(y, O.gguf_matvec(fmt, dense, x))[0] <= 1e-4
    we = pkg.device_weights("blk.0.ffn_down_exps.weight", cuda)
    assert tuple(we.shape) == (experts, rows, dense.shape[1])
    ids = np.array([[2, 0], [1, 5]], dtype=np.int32)  # 5 is outside the table: zeros
    xe = rng.normal(0, 1, size=(2, 1, k)).astype(np.float32)
    ye = ops.expert_matvec(name, we, dev_f32(xe, cuda), torch.from_numpy(ids).to(cuda)).cpu().numpy()
    assert util.parity(ye, O.gguf_expert_matvec(fmt, stack, xe, ids))[0] <= 1e-4
    assert np.all(ye[1, 1] == 0)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("bits,gs,m", [(4, 64, 1), (2, 64, 5), (8, 32, 2), (4, 128, 40)])
def test_f16_and_f32_compute_dtypes(cuda, dtype, bits, gs, m):
    """ops::quantized_matmul casts x, scales and biases to the promoted dtype (array_ops.rs:398-404) and dequantize
    returns the scales' dtype: f16 and f32 through the generic kernels, against the f64 contraction of
    q * s + b (the matvec law) and the one-rounding dequantize law."""
    rng = np.random.default_rng(bits + gs + m)
    n, k = 136, 512
    w = rng.integers(0, 1 << 32, size=(n, k * bits // 32), dtype=np.uint32)
    s = np.abs(rng.normal(0, 0.02, size=(n, k // gs))).astype(np.float32)
    b = rng.normal(0, 0.01, size=(n, k // gs)).astype(np.float32)
    x = rng.normal(0, 1, size=(m, k)).astype(np.float32)
    ts, tb, tx = (torch.from_numpy(a).to(cuda).to(dtype) for a in (s, b, x))
    tw = dev_u32(w, cuda)
    y = ops.quantized_matmul(tx, tw, ts, tb, True, gs, bits)
    assert y.dtype == dtype and y.shape == (m, n)
    # codes, and the values the kernel actually saw (rounded to the dtype)
    codes = np.stack([(w >> (bits * j)) & ((1 << bits) - 1) for j in range(32 // bits)], axis=-1).reshape(n, k).astype(np.float64)
    sf, bf, xf = (t.float().cpu().numpy().astype(np.float64) for t in (ts, tb, tx))
    dense = codes * np.repeat(sf, gs, axis=1) + np.repeat(bf, gs, axis=1)
    truth = xf @ dense.T
    err, l2 = util.parity(y.float().cpu().numpy(), truth)
    assert err <= (2e-3 if dtype == torch.float16 else 2e-5), (err, l2)
    d = ops.dequantize(tw, ts, tb, gs, bits)
    assert d.dtype == dtype
    want = (codes.astype(np.float32) * np.repeat(sf, gs, axis=1).astype(np.float32)).astype(np.float32) + np.repeat(bf, gs, axis=1).astype(np.float32)
    want_t = torch.from_numpy(want.astype(np.float32)).to(dtype)
    assert torch.equal(d.cpu(), want_t)   # f32(q) * s rounded, + b rounded, then one cast: bit for bit
