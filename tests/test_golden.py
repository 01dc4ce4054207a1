"""The committed fixtures of tests/golden/: the oracle reproduces them (CPU), and the CUDA path
matches them without the oracle in the loop (GPU)."""
import glob
import json
import os

import numpy as np
import pytest

from oracle import oracle as O
from tests import util

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    return dict(np.load(os.path.join(GOLDEN, name + ".npz")))


def names(prefix):
    return sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN, prefix + "*.npz")))


# ------------------------------------------------------------------ CPU: oracle vs fixtures
def test_reference_constants_are_the_ones_the_oracle_reproduces():
    with open(os.path.join(GOLDEN, "reference_constants.json")) as f:
        c = json.load(f)
    assert O.gguf_reference_hash(O.Q2_K) == int(c["gguf_fnv1a64"]["Q2_K"], 16)
    assert O.gguf_reference_hash(O.Q4_K) == int(c["gguf_fnv1a64"]["Q4_K"], 16)
    assert O.BLOCK_BYTES[O.Q2_K] == c["block_bytes"]["Q2_K"] and O.BLOCK_BYTES[O.Q4_K] == c["block_bytes"]["Q4_K"]


@pytest.mark.parametrize("name", names("affine_"))
def test_oracle_reproduces_affine_fixture(name):
    g = load(name)
    bits, gs = int(g["bits"]), int(g["group_size"])
    assert np.array_equal(O.affine_dequantize(g["w"], g["scales"], g["biases"], gs, bits), g["dequant_bf16"])
    y = O.affine_matmul(g["x"], g["w"], g["scales"], g["biases"], gs, bits, round_weight_bf16=True, threads=2)
    assert np.array_equal(y, g["y_rounded_weight_bf16"])
    assert np.array_equal(O.affine_qmv_factored(g["x"], g["w"], g["scales"], g["biases"], gs, bits), g["y_factored_bf16"])


@pytest.mark.parametrize("name", names("gguf_"))
def test_oracle_reproduces_gguf_fixture(name):
    g = load(name)
    fmt = int(g["fmt"])
    assert np.array_equal(O.gguf_decode(fmt, g["w"]).reshape(g["decoded"].shape), g["decoded"])
    assert np.array_equal(O.gguf_matvec(fmt, g["w"], g["x"], threads=2), g["y"])


@pytest.mark.parametrize("name", names("moe_"))
def test_oracle_reproduces_moe_fixture(name):
    g = load(name)
    top_k, experts = int(g["top_k"]), g["gate_w"].shape[0]
    idx, wts = O.moe_route(g["logits"], top_k)
    assert np.array_equal(idx, g["idx"]) and np.array_equal(wts, g["weights"])
    s, t, inv = O.moe_sort(idx, experts, top_k)
    assert np.array_equal(s, g["sorted_ids"]) and np.array_equal(t, g["token_rows"]) and np.array_equal(inv, g["inverse"])
    y, _ = O.moe_forward(g["x"], g["logits"], *[(g[n + "_w"], g[n + "_s"], g[n + "_b"]) for n in ("gate", "up", "down")],
                         top_k, round_weight_bf16=False)
    assert np.array_equal(y, g["y_bf16"])


# ------------------------------------------------------------------ GPU: CUDA path vs fixtures
@pytest.mark.gpu
@pytest.mark.parametrize("name", names("affine_"))
def test_cuda_matches_affine_fixture(cuda, name):
    from lisa_b200 import _cabi, ops
    from tests.gpu_util import dev_bf16, dev_u32, host_bf16_bits

    g = load(name)
    bits, gs = int(g["bits"]), int(g["group_size"])
    w, s, b = dev_u32(g["w"], cuda), dev_bf16(g["scales"], cuda), dev_bf16(g["biases"], cuda)
    # unpacked weights: bit-exact
    assert np.array_equal(host_bf16_bits(ops.dequantize(w, s, b, gs, bits)), g["dequant_bf16"])
    if bits == 8:
        return  # the matmul kernels cover the 2- and 4-bit formats of the path
    x = dev_bf16(g["x"], cuda)
    want_f = O.bf16_to_f32(g["y_factored_bf16"])
    want_r = O.bf16_to_f32(g["y_rounded_weight_bf16"])
    # GEMV follows the factored law, the tensor-core GEMM the rounded-weight law; 1e-2 max-relative
    y = O.bf16_to_f32(host_bf16_bits(ops.quantized_matmul(x, w, s, b, True, gs, bits, flags=_cabi.FLAG_FORCE_QMV)))
    assert util.parity(y, want_f)[0] <= 1e-2
    y = O.bf16_to_f32(host_bf16_bits(ops.quantized_matmul(x, w, s, b, True, gs, bits, flags=_cabi.FLAG_FORCE_QMM)))
    assert util.parity(y, want_r)[0] <= 1e-2


@pytest.mark.gpu
@pytest.mark.parametrize("name", names("gguf_"))
def test_cuda_matches_gguf_fixture(cuda, name):
    from lisa_b200 import ops
    from tests.gpu_util import dev_f32, dev_u8

    g = load(name)
    fmt = "Q2K" if int(g["fmt"]) == O.Q2_K else "Q4K"
    y = ops.packed_matvec(fmt, dev_u8(g["w"], cuda), dev_f32(g["x"], cuda)).cpu().numpy()
    assert util.parity(y, g["y"])[0] <= 1e-4


@pytest.mark.gpu
@pytest.mark.parametrize("name", names("moe_"))
def test_cuda_matches_moe_fixture(cuda, name):
    from lisa_b200 import ops
    from lisa_b200.quant import QuantizedLinear, SwitchGlu
    from tests.gpu_util import dev_bf16, dev_f32, dev_u32, host_bf16_bits

    g = load(name)
    top_k, experts = int(g["top_k"]), g["gate_w"].shape[0]
    idx, wts = ops.moe_route(dev_f32(g["logits"], cuda), top_k)
    assert np.array_equal(idx.cpu().numpy(), g["idx"])
    assert np.allclose(wts.cpu().numpy(), g["weights"], rtol=2e-6, atol=1e-7)
    s, t, inv = ops.moe_sort(idx, experts, top_k)
    assert np.array_equal(s.cpu().numpy(), g["sorted_ids"])
    assert np.array_equal(t.cpu().numpy(), g["token_rows"])
    assert np.array_equal(inv.cpu().numpy(), g["inverse"])

    def lin(n):
        return QuantizedLinear(dev_u32(g[n + "_w"], cuda), dev_bf16(g[n + "_s"], cuda), dev_bf16(g[n + "_b"], cuda), 64, 4)

    y = SwitchGlu(lin("gate"), lin("up"), lin("down"), top_k).forward(dev_bf16(g["x"], cuda), dev_f32(g["logits"], cuda))
    err, l2 = util.parity(O.bf16_to_f32(host_bf16_bits(y)), O.bf16_to_f32(g["y_bf16"]))
    assert err <= 1e-2 and l2 <= 1e-2, (err, l2)
