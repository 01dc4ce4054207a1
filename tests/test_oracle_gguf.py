"""Pins the GGUF half of the oracle to the reference's own known answers."""
import numpy as np
import pytest

from oracle import oracle as O


# Frozen in crates/lisa-gguf/src/quant.rs:195-198 from the unmodified GGML C dequantizers.
REFERENCE_HASHES = {O.Q2_K: 0x92F0E7A5DAF379E9, O.Q4_K: 0xA8FD5258D144ADD5, O.Q5_K: 0xF8A0E7F3F1B1AEE0,
                    O.Q8_0: 0xC0087397958E8331}


@pytest.mark.parametrize("fmt", [O.Q2_K, O.Q4_K, O.Q5_K, O.Q8_0])
def test_block_decoders_match_reference_hashes(fmt):
    assert O.gguf_reference_hash(fmt) == REFERENCE_HASHES[fmt]


@pytest.mark.parametrize("fmt", [O.Q2_K, O.Q4_K, O.Q5_K])
@pytest.mark.parametrize("width", [256, 1280, 2304, 5120, 8192])
def test_dyadic_dot_is_exact(fmt, width):
    """kernel_tests.rs:178-210: with d=0x1800, dmin=0x1400 and x in {-1/8,0,1/8} every partial sum
    is exact in f32, so the sequential f32 dot equals the f64 dot."""
    rows, tokens = 16, 3
    blocks = O.gguf_dyadic_blocks(fmt, width * rows // 256)
    w = blocks.reshape(rows, -1)
    x = O.gguf_dyadic_inputs(tokens * width).reshape(tokens, width)
    assert set(np.unique(x)) <= {-0.125, 0.0, 0.125}
    y = O.gguf_matvec(fmt, w, x, threads=2)
    dec = O.gguf_decode(fmt, blocks).reshape(rows, width).astype(np.float64)
    assert np.array_equal(y.astype(np.float64), x.astype(np.float64) @ dec.T)


@pytest.mark.parametrize("fmt", [O.Q2_K, O.Q4_K])
def test_expert_ids_and_broadcast(fmt):
    """kernel_tests.rs:212-263: ids -1 and `experts` give exactly 0.0; slots in {1, top_k}."""
    experts, width, rows, tokens, top_k = 192, 256, 8, 3, 6
    blocks = O.gguf_dyadic_blocks(fmt, width * rows * experts // 256)
    w = blocks.reshape(experts, rows, -1)
    sel = np.array([(i * 79 + 1) % experts for i in range(tokens * top_k)], dtype=np.int32)
    sel[0], sel[1], sel[2] = experts - 1, -1, experts
    ids = sel.reshape(tokens, top_k)
    dec = O.gguf_decode(fmt, blocks).reshape(experts, rows, width).astype(np.float64)
    for slots in (1, top_k):
        x = O.gguf_dyadic_inputs(tokens * slots * width).reshape(tokens, slots, width)
        y = O.gguf_expert_matvec(fmt, w, x, ids, threads=2)
        for t in range(tokens):
            for s in range(top_k):
                e = ids[t, s]
                want = np.zeros(rows) if (e < 0 or e >= experts) else dec[e] @ x[t, s % slots].astype(np.float64)
                assert np.array_equal(y[t, s].astype(np.float64), want)


def test_decode_matches_formula_q4k():
    rng = np.random.default_rng(1)
    blk = rng.integers(0, 256, size=144, dtype=np.uint8)
    blk[0:2] = np.frombuffer(np.float16(0.01).tobytes(), dtype=np.uint8)
    blk[2:4] = np.frombuffer(np.float16(0.02).tobytes(), dtype=np.uint8)
    out = O.gguf_decode(O.Q4_K, blk)
    d, dmin = np.float32(np.float16(0.01)), np.float32(np.float16(0.02))
    b = blk.astype(np.int64)
    for g in range(8):
        if g < 4:
            sc, m = b[4 + g] & 63, b[8 + g] & 63
        else:
            sc = (b[8 + g] & 15) | ((b[g] >> 6) << 4)
            m = (b[8 + g] >> 4) | ((b[4 + g] >> 6) << 4)
        for l in range(32):
            q = (b[16 + (g // 2) * 32 + l] >> (4 * (g % 2))) & 15
            want = np.float32(np.float32(d * np.float32(sc)) * np.float32(q)) - np.float32(dmin * np.float32(m))
            assert out[g * 32 + l] == np.float32(want)
