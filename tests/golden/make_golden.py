"""Regenerates the fixtures in this directory:  python tests/golden/make_golden.py

Two kinds of fixture live here.

* ``reference_constants.json`` -- known answers copied (as numbers, by reading) from the
  reference's own tests: the FNV-1a-64 hashes of the GGUF block decoders over its LCG input
  (crates/lisa-gguf/src/quant.rs:197-198) and the geometry of its dyadic exact-dot tests
  (crates/lisa-engine/src/models/deepseek41/kernel_tests.rs:178-263).  The reference's affine
  tests compare one Metal kernel with another and hold no vectors, so there are none to copy.
* ``*.npz`` -- seeded inputs with the outputs of the CPU oracle (``oracle/``), which restates
  the reference's algorithms and reproduces the constants above.  They freeze the oracle's
  answers: a change of the oracle, of numpy's generators or of the CUDA path shows up as a diff
  against these files, on machines that have neither the reference nor the oracle's history.

The reference itself (Rust + Metal) cannot be built or run in this environment, so no fixture is
an output of the reference binary.
"""
from __future__ import annotations

import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import oracle as O  # noqa: E402
from tests import util  # noqa: E402

REFERENCE_CONSTANTS = {
    "gguf_fnv1a64": {
        "source": "crates/lisa-gguf/src/quant.rs:197-198",
        "Q2_K": "0x92f0e7a5daf379e9",
        "Q4_K": "0xa8fd5258d144add5",
    },
    "gguf_dyadic": {
        "source": "crates/lisa-engine/src/models/deepseek41/kernel_tests.rs:178-263",
        "d_bits": "0x1800",
        "dmin_bits": "0x1400",
        "inputs": [-0.125, 0.0, 0.125],
        "widths": [256, 1280, 2304, 5120, 8192],
        "rows": 16,
        "tokens": 3,
        "expert_counts": [192, 384],
        "top_k": 6,
    },
    "block_bytes": {"source": "crates/lisa-gguf/src/quant.rs:64-101", "Q2_K": 84, "Q4_K": 144},
}


def affine_case(seed: int, n: int, k: int, m: int, bits: int, group_size: int):
    rng = np.random.default_rng(seed)
    w, s, b = util.affine_weights(rng, n, k, bits, group_size)
    x = util.activations(rng, m, k)
    return {
        "w": w, "scales": s, "biases": b, "x": x,
        "bits": np.int32(bits), "group_size": np.int32(group_size),
        "dequant_bf16": O.affine_dequantize(w, s, b, group_size, bits),
        # the two summation laws of the reference (tile loaders round the weight to bf16, the
        # GEMV keeps scale * sum(q x) + bias * sum(x) in f32); each GPU kernel follows one of them
        "y_rounded_weight_bf16": O.affine_matmul(x, w, s, b, group_size, bits, round_weight_bf16=True, threads=1),
        "y_factored_bf16": O.affine_qmv_factored(x, w, s, b, group_size, bits),
    }


def gguf_case(seed: int, fmt: int, rows: int, k: int, tokens: int):
    rng = np.random.default_rng(seed)
    w = util.gguf_weights(rng, fmt, rows, k)
    x = rng.normal(0, 1, size=(tokens, k)).astype(np.float32)
    return {"fmt": np.int32(fmt), "w": w, "x": x, "decoded": O.gguf_decode(fmt, w).reshape(rows, k),
            "y": O.gguf_matvec(fmt, w, x, threads=1)}


def moe_case(seed: int, tokens: int, experts: int, top_k: int, hidden: int, inter: int):
    rng = np.random.default_rng(seed)
    logits = rng.normal(0, 1, size=(tokens, experts)).astype(np.float32)
    idx, wts = O.moe_route(logits, top_k)
    sorted_ids, token_rows, inverse = O.moe_sort(idx, experts, top_k)
    gate = util.affine_weights(rng, inter, hidden, 4, 64, experts)
    up = util.affine_weights(rng, inter, hidden, 4, 64, experts)
    down = util.affine_weights(rng, hidden, inter, 4, 64, experts)
    x = util.activations(rng, tokens, hidden)
    # ten sorted rows: the reference runs such a block as per-run matvecs (unrounded weights, array_ops.rs:591-630)
    y, _ = O.moe_forward(x, logits, gate, up, down, top_k, round_weight_bf16=False)
    out = {"logits": logits, "idx": idx, "weights": wts, "sorted_ids": sorted_ids, "token_rows": token_rows,
           "inverse": inverse, "x": x, "y_bf16": y, "top_k": np.int32(top_k)}
    for name, (w, s, b) in (("gate", gate), ("up", up), ("down", down)):
        out[f"{name}_w"], out[f"{name}_s"], out[f"{name}_b"] = w, s, b
    return out


def main() -> None:
    with open(os.path.join(HERE, "reference_constants.json"), "w") as f:
        json.dump(REFERENCE_CONSTANTS, f, indent=1)
        f.write("\n")
    cases = {
        "affine_4bit_n48_k256_m1": affine_case(11, 48, 256, 1, 4, 64),
        "affine_4bit_n40_k320_m5": affine_case(12, 40, 320, 5, 4, 64),
        "affine_2bit_n32_k512_m3": affine_case(13, 32, 512, 3, 2, 64),
        "affine_4bit_g32_n16_k96_m2": affine_case(14, 16, 96, 2, 4, 32),
        "affine_8bit_n8_k128_m1": affine_case(15, 8, 128, 1, 8, 64),
        "gguf_q2k_r8_k512_t2": gguf_case(21, O.Q2_K, 8, 512, 2),
        "gguf_q4k_r8_k512_t2": gguf_case(22, O.Q4_K, 8, 512, 2),
        "moe_t5_e8_k2_h128_i64": moe_case(31, 5, 8, 2, 128, 64),
    }
    for name, arrays in cases.items():
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **arrays)
        print(name, sum(a.nbytes for a in arrays.values()), "bytes of arrays")


if __name__ == "__main__":
    main()
