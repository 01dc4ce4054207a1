"""Residual add + RMSNorm in front of the quantized linears: the fused form inside the decode kernel's activation
staging, the kernel of its own, and the entry point that picks between them, against the oracle."""
import numpy as np
import pytest
import torch

from lisa_b200 import _cabi, ops
from oracle import oracle as O
from tests import util
from tests.gpu_util import dev_bf16, dev_u32, host_bf16_bits

pytestmark = pytest.mark.gpu
EPS = 1e-6


def _inputs(rng, m, k):
    x = util.activations(rng, m, k)
    r = O.f32_to_bf16(rng.normal(0, 2, size=(m, k)).astype(np.float32))
    w = O.f32_to_bf16((1.0 + rng.normal(0, 0.1, size=(k,))).astype(np.float32))
    return x, r, w


@pytest.mark.parametrize("m,k", [(1, 2560), (3, 1024), (8, 5120), (40, 768)])
def test_add_rmsnorm_kernel(cuda, m, k):
    rng = np.random.default_rng(m + k)
    x, r, w = _inputs(rng, m, k)
    total, normed = ops.add_rmsnorm(dev_bf16(x, cuda), dev_bf16(r, cuda), dev_bf16(w, cuda), EPS)
    ot, on = O.add_rmsnorm(x, r, w, EPS)
    assert np.array_equal(host_bf16_bits(total), ot)              # one rounding of an exact sum: bit for bit
    assert util.bf16_ulp_distance(host_bf16_bits(normed), on) <= 2  # inv may differ in its last bits


@pytest.mark.parametrize("bits", [4, 2])
@pytest.mark.parametrize("m,k,ns", [(1, 2560, (4096, 1024, 1024)), (1, 5120, (9728, 9728)), (4, 2560, (2560,)), (8, 5120, (1024, 1024)),
                                     (1, 17408, (5120,))])
def test_fused_addnorm_decode_rows(cuda, m, k, ns, bits):
    """One launch: sum bit for bit, normed within a bf16 ulp of the oracle's, every linear against the oracle's
    matvec on the normed rows the GPU wrote (same input bits) at 1e-2, and against the oracle's whole chain."""
    rng = np.random.default_rng(m * 7 + k + len(ns) + bits)
    x, r, w = _inputs(rng, m, k)
    lins = [util.affine_weights(rng, n, k, bits, 64) for n in ns]
    dl = [(dev_u32(a, cuda), dev_bf16(b, cuda), dev_bf16(c, cuda)) for a, b, c in lins]
    before = ops.launch_count()
    ys, total, normed = ops.quantized_matmul_addnorm(dev_bf16(x, cuda), dev_bf16(r, cuda), dev_bf16(w, cuda), EPS, dl, 64, bits)
    launches = ops.launch_count() - before
    ot, on = O.add_rmsnorm(x, r, w, EPS)
    assert np.array_equal(host_bf16_bits(total), ot)
    nb = host_bf16_bits(normed)
    assert util.bf16_ulp_distance(nb, on) <= 2  # inv may differ in its last bits
    for y, (a, b, c) in zip(ys, lins):
        got = O.bf16_to_f32(host_bf16_bits(y))
        err, l2 = util.parity(got, O.affine_matmul(nb, a, b, c, 64, bits, round_weight_bf16=False, f64=True))
        assert err <= 1e-2, (err, l2)
        err, l2 = util.parity(got, O.affine_matmul(on, a, b, c, 64, bits, round_weight_bf16=False, f64=True))
        assert err <= 1e-2, (err, l2)
    if k != 17408 or m <= 4:
        assert launches == 1, launches
    # without the normed output the linears give the same bits
    ys2, total2, none = ops.quantized_matmul_addnorm(dev_bf16(x, cuda), dev_bf16(r, cuda), dev_bf16(w, cuda), EPS, dl, 64, bits,
                                                      write_norm=False)
    assert none is None and torch.equal(total2, total)
    for a, b in zip(ys, ys2):
        assert torch.equal(a, b)
    assert ops.device_status() == 0


def test_addnorm_equals_the_separate_calls(cuda):
    """The fused launch against add_rmsnorm followed by the sibling matmul on the same device: the normed rows may
    differ by a bf16 ulp where the two sums of squares round differently; the outputs stay within 2^-6."""
    rng = np.random.default_rng(5)
    m, k, ns = 2, 2560, (4096, 1024)
    x, r, w = _inputs(rng, m, k)
    lins = [util.affine_weights(rng, n, k, 4, 64) for n in ns]
    dl = [(dev_u32(a, cuda), dev_bf16(b, cuda), dev_bf16(c, cuda)) for a, b, c in lins]
    tx, tr, tw = dev_bf16(x, cuda), dev_bf16(r, cuda), dev_bf16(w, cuda)
    ys, total, normed = ops.quantized_matmul_addnorm(tx, tr, tw, EPS, dl)
    t2, n2 = ops.add_rmsnorm(tx, tr, tw, EPS)
    ref = ops.quantized_matmul_siblings(n2, dl)
    assert torch.equal(total, t2)
    assert util.bf16_ulp_distance(host_bf16_bits(normed), host_bf16_bits(n2)) <= 2
    for a, b in zip(ys, ref):
        assert float((a.float() - b.float()).abs().max()) <= 2.0 ** -6 * float(b.float().abs().max())


def test_addnorm_unfused_shapes(cuda):
    """Many rows, and a group size the decode kernel does not take: the norm runs as its own kernel and the entry
    point wants the normed buffer."""
    rng = np.random.default_rng(6)
    for m, k, n, gs in ((300, 1024, 512, 64), (2, 1024, 256, 32)):
        x, r, w = _inputs(rng, m, k)
        a, b, c = util.affine_weights(rng, n, k, 4, gs)
        dl = [(dev_u32(a, cuda), dev_bf16(b, cuda), dev_bf16(c, cuda))]
        tx, tr, tw = dev_bf16(x, cuda), dev_bf16(r, cuda), dev_bf16(w, cuda)
        ys, total, normed = ops.quantized_matmul_addnorm(tx, tr, tw, EPS, dl, gs, 4)
        ot, on = O.add_rmsnorm(x, r, w, EPS)
        assert np.array_equal(host_bf16_bits(total), ot)
        nb = host_bf16_bits(normed)
        assert util.bf16_ulp_distance(nb, on) <= 2  # inv may differ in its last bits
        law = m > 8
        err, l2 = util.parity(O.bf16_to_f32(host_bf16_bits(ys[0])), O.affine_matmul(nb, a, b, c, gs, 4, round_weight_bf16=law, f64=True))
        assert err <= 1e-2, (err, l2)
        with pytest.raises(_cabi.LisaError) as e:
            ops.quantized_matmul_addnorm(tx, tr, tw, EPS, dl, gs, 4, write_norm=False)
        assert e.value.code == _cabi.ERR_WORKSPACE


@pytest.mark.parametrize("bits", [4, 2])
@pytest.mark.parametrize("m,k,n", [(1, 9728, 2560), (3, 1024, 512), (8, 17408, 5120), (1, 768, 2048)])
def test_fused_swiglu_in_front_of_the_down_projection(cuda, m, k, n, bits):
    """One launch for SwiGLU + linear on decode rows: the activation rows it writes equal the swiglu kernel's bit for
    bit, and the output equals the plain matmul on them (same kernel, same activation bits)."""
    rng = np.random.default_rng(m + k + n + bits)
    g = O.f32_to_bf16(rng.normal(0, 2, size=(m, k)).astype(np.float32))
    u = O.f32_to_bf16(rng.normal(0, 2, size=(m, k)).astype(np.float32))
    a, b, c = util.affine_weights(rng, n, k, bits, 64)
    tw, ts, tb = dev_u32(a, cuda), dev_bf16(b, cuda), dev_bf16(c, cuda)
    tg, tu = dev_bf16(g, cuda), dev_bf16(u, cuda)
    y, act = ops.quantized_matmul_swiglu(tg, tu, tw, ts, tb, 64, bits, write_act=True)
    ref_act = ops.swiglu(tg, tu)
    assert torch.equal(act, ref_act)
    assert util.bf16_ulp_distance(host_bf16_bits(act), O.swiglu_bf16(g, u)) <= 1   # expf: host libm against the device
    assert torch.equal(y, ops.quantized_matmul(ref_act, tw, ts, tb, True, 64, bits))
    err, l2 = util.parity(O.bf16_to_f32(host_bf16_bits(y)),
                          O.affine_matmul(host_bf16_bits(act), a, b, c, 64, bits, round_weight_bf16=False, f64=True))
    assert err <= 1e-2, (err, l2)
    y2, none = ops.quantized_matmul_swiglu(tg, tu, tw, ts, tb, 64, bits)
    assert none is None and torch.equal(y2, y)
    assert ops.device_status() == 0


def test_swiglu_unfused_shapes(cuda):
    rng = np.random.default_rng(3)
    m, k, n = 100, 1024, 256
    g = O.f32_to_bf16(rng.normal(0, 2, size=(m, k)).astype(np.float32))
    u = O.f32_to_bf16(rng.normal(0, 2, size=(m, k)).astype(np.float32))
    a, b, c = util.affine_weights(rng, n, k, 4, 64)
    tw, ts, tb = dev_u32(a, cuda), dev_bf16(b, cuda), dev_bf16(c, cuda)
    tg, tu = dev_bf16(g, cuda), dev_bf16(u, cuda)
    y, act = ops.quantized_matmul_swiglu(tg, tu, tw, ts, tb, write_act=True)
    assert torch.equal(act, ops.swiglu(tg, tu))
    assert torch.equal(y, ops.quantized_matmul(act, tw, ts, tb, True, 64, 4))
    with pytest.raises(_cabi.LisaError) as e:
        ops.quantized_matmul_swiglu(tg, tu, tw, ts, tb)
    assert e.value.code == _cabi.ERR_WORKSPACE
