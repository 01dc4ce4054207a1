"""ctypes front end of the CPU oracle (``liblisa_oracle.so``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()``
and by ``bench.py``'s CPU-baseline legs, never by the ``lisa_b200`` package.
Arrays are numpy; bf16/f16 tensors travel as ``uint16`` bit patterns.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liblisa_oracle.so")

Q8_0 = 8
Q2_K = 10
Q4_K = 12
Q5_K = 13
BLOCK_BYTES = {Q8_0: 34, Q2_K: 84, Q4_K: 144, Q5_K: 176}
BLOCK_WIDTH = {Q8_0: 32, Q2_K: 256, Q4_K: 256, Q5_K: 256}


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside this file."""
    src = os.path.join(_HERE, "lisa_oracle.c")
    hdr = os.path.join(_HERE, "lisa_oracle.h")
    stale = (not os.path.exists(_LIB_PATH)) or any(
        os.path.getmtime(p) > os.path.getmtime(_LIB_PATH) for p in (src, hdr)
    )
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B", "liblisa_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.oracle_gguf_reference_hash.restype = C.c_uint64
        _lib.oracle_moe_tile_table.restype = C.c_int64
        _lib.oracle_f32_to_bf16.restype = C.c_uint16
        _lib.oracle_f32_to_bf16.argtypes = [C.c_float]
        _lib.oracle_f32_to_f16.restype = C.c_uint16
        _lib.oracle_f32_to_f16.argtypes = [C.c_float]
        _lib.oracle_f16_to_f32.restype = C.c_float
        _lib.oracle_f16_to_f32.argtypes = [C.c_uint16]
    return _lib


def _p(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.c_void_p)


def _i64(v) -> C.c_int64:
    return C.c_int64(int(v))


def _chk(rc: int, what: str) -> None:
    if rc != 0:
        raise ValueError(f"oracle: {what} rejected its arguments (rc={rc})")


# ---------------------------------------------------------------- conversions
def f32_to_bf16(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 bit patterns (vectorised; equals
    oracle_f32_to_bf16 element for element, checked in tests)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = ((u.astype(np.uint64) + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    r[nan] = ((u[nan] >> 16) | 0x40).astype(np.uint16)
    return r


def bf16_to_f32(a: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(a, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_f16_bits(a: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32).astype(np.float16).view(np.uint16)


# ---------------------------------------------------------------- affine
def affine_dequantize(w, scales, biases, group_size: int, bits: int, out_f32: bool = False):
    """ops::dequantize: w uint32 [..., K*bits/32], scales/biases bf16 bits [..., K/gs]."""
    w = np.ascontiguousarray(w, dtype=np.uint32)
    kq = w.shape[-1]
    k = kq * 32 // bits
    rows = w.size // kq
    s = np.ascontiguousarray(scales, dtype=np.uint16)
    b = np.ascontiguousarray(biases, dtype=np.uint16)
    if out_f32:
        out = np.empty(w.shape[:-1] + (k,), dtype=np.float32)
        rc = lib().oracle_affine_dequantize_f32(_p(w), _p(s), _p(b), _i64(rows), _i64(k),
                                                group_size, bits, _p(out))
    else:
        out = np.empty(w.shape[:-1] + (k,), dtype=np.uint16)
        rc = lib().oracle_affine_dequantize_bf16(_p(w), _p(s), _p(b), _i64(rows), _i64(k),
                                                 group_size, bits, _p(out))
    _chk(rc, "affine_dequantize")
    return out


def affine_matmul(x, w, scales, biases, group_size: int, bits: int, round_weight_bf16: bool = True,
                  threads: int = 0, f64: bool = False):
    """y = x . dequant(W)^T; x bf16 bits [M,K]; returns bf16 bits [M,N] (or f64)."""
    x = np.ascontiguousarray(x, dtype=np.uint16)
    w = np.ascontiguousarray(w, dtype=np.uint32)
    s = np.ascontiguousarray(scales, dtype=np.uint16)
    b = np.ascontiguousarray(biases, dtype=np.uint16)
    m, k = x.shape
    n = w.shape[0]
    threads = threads or (os.cpu_count() or 1)
    if f64:
        y = np.empty((m, n), dtype=np.float64)
        rc = lib().oracle_affine_matmul_f64(_p(x), _i64(m), _i64(k), _p(w), _p(s), _p(b), _i64(n),
                                            group_size, bits, int(round_weight_bf16), threads, _p(y))
    else:
        y = np.empty((m, n), dtype=np.uint16)
        rc = lib().oracle_affine_matmul(_p(x), _i64(m), _i64(k), _p(w), _p(s), _p(b), _i64(n),
                                        group_size, bits, int(round_weight_bf16), threads, _p(y))
    _chk(rc, "affine_matmul")
    return y


def affine_qmv_factored(x, w, scales, biases, group_size: int, bits: int):
    x = np.ascontiguousarray(x, dtype=np.uint16)
    w = np.ascontiguousarray(w, dtype=np.uint32)
    s = np.ascontiguousarray(scales, dtype=np.uint16)
    b = np.ascontiguousarray(biases, dtype=np.uint16)
    m, k = x.shape
    n = w.shape[0]
    y = np.empty((m, n), dtype=np.uint16)
    _chk(lib().oracle_affine_qmv_factored(_p(x), _i64(m), _i64(k), _p(w), _p(s), _p(b), _i64(n),
                                          group_size, bits, _p(y)), "affine_qmv_factored")
    return y


def affine_quantize(w_f32, group_size: int = 64, bits: int = 4):
    """ops::quantize: returns (wq uint32, scales f32, biases f32)."""
    w = np.ascontiguousarray(w_f32, dtype=np.float32)
    rows, k = w.shape
    wq = np.zeros((rows, k * bits // 32), dtype=np.uint32)
    sc = np.empty((rows, k // group_size), dtype=np.float32)
    bi = np.empty((rows, k // group_size), dtype=np.float32)
    _chk(lib().oracle_affine_quantize(_p(w), _i64(rows), _i64(k), group_size, bits, _p(wq), _p(sc),
                                      _p(bi)), "affine_quantize")
    return wq, sc, bi


def lcg_fill(seed: int, count: int):
    s = C.c_uint64(seed)
    out = np.empty(count, dtype=np.float32)
    lib().oracle_lcg_fill(C.byref(s), _p(out), _i64(count))
    return out, s.value


def gather_qmm(x, w, scales, biases, ids, group_size: int, bits: int,
               round_weight_bf16: bool = True, threads: int = 0):
    x = np.ascontiguousarray(x, dtype=np.uint16)
    w = np.ascontiguousarray(w, dtype=np.uint32)
    s = np.ascontiguousarray(scales, dtype=np.uint16)
    b = np.ascontiguousarray(biases, dtype=np.uint16)
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    rows, k = x.shape
    experts, n = w.shape[0], w.shape[1]
    y = np.empty((rows, n), dtype=np.uint16)
    threads = threads or (os.cpu_count() or 1)
    _chk(lib().oracle_gather_qmm(_p(x), _i64(rows), _i64(k), _p(w), _p(s), _p(b), _p(ids),
                                 _i64(experts), _i64(n), group_size, bits, int(round_weight_bf16),
                                 threads, _p(y)), "gather_qmm")
    return y


# ---------------------------------------------------------------- GGUF
def gguf_decode(fmt: int, packed) -> np.ndarray:
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    blocks = packed.size // BLOCK_BYTES[fmt]
    out = np.empty(blocks * BLOCK_WIDTH[fmt], dtype=np.float32)
    _chk(lib().oracle_gguf_decode(fmt, _p(packed), _i64(blocks), _p(out)), "gguf_decode")
    return out


def gguf_reference_hash(fmt: int) -> int:
    return int(lib().oracle_gguf_reference_hash(fmt))


def gguf_dyadic_blocks(fmt: int, count: int) -> np.ndarray:
    out = np.empty(count * BLOCK_BYTES[fmt], dtype=np.uint8)
    _chk(lib().oracle_gguf_dyadic_blocks(fmt, _i64(count), _p(out)), "gguf_dyadic_blocks")
    return out


def gguf_dyadic_inputs(count: int) -> np.ndarray:
    out = np.empty(count, dtype=np.float32)
    lib().oracle_gguf_dyadic_inputs(_i64(count), _p(out))
    return out


def gguf_matvec(fmt: int, w, x, threads: int = 0) -> np.ndarray:
    """w uint8 [rows,row_bytes], x f32 [tokens,K] -> f32 [tokens,rows]."""
    w = np.ascontiguousarray(w, dtype=np.uint8)
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, row_bytes = w.shape
    tokens = x.shape[0]
    y = np.empty((tokens, rows), dtype=np.float32)
    threads = threads or (os.cpu_count() or 1)
    _chk(lib().oracle_gguf_matvec(fmt, _p(w), _i64(rows), _i64(row_bytes), _p(x), _i64(tokens),
                                  threads, _p(y)), "gguf_matvec")
    return y


def gguf_expert_matvec(fmt: int, w, x, ids, threads: int = 0) -> np.ndarray:
    """w uint8 [E,rows,row_bytes], x f32 [tokens,slots,K], ids i32 [tokens,top_k]."""
    w = np.ascontiguousarray(w, dtype=np.uint8)
    x = np.ascontiguousarray(x, dtype=np.float32)
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    experts, rows, row_bytes = w.shape
    tokens, slots = x.shape[0], x.shape[1]
    top_k = ids.shape[1]
    y = np.empty((tokens, top_k, rows), dtype=np.float32)
    threads = threads or (os.cpu_count() or 1)
    _chk(lib().oracle_gguf_expert_matvec(fmt, _p(w), _i64(experts), _i64(rows), _i64(row_bytes),
                                         _p(x), _i64(tokens), _i64(slots), _p(ids), _i64(top_k),
                                         threads, _p(y)), "gguf_expert_matvec")
    return y


# ---------------------------------------------------------------- MoE
def moe_route(logits, top_k: int):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    tokens, experts = logits.shape
    idx = np.empty((tokens, top_k), dtype=np.int32)
    wts = np.empty((tokens, top_k), dtype=np.float32)
    _chk(lib().oracle_moe_route(_p(logits), _i64(tokens), _i64(experts), top_k, _p(idx), _p(wts)),
         "moe_route")
    return idx, wts


def moe_sort(idx, experts: int, top_k: int):
    idx = np.ascontiguousarray(idx, dtype=np.int32).reshape(-1)
    n = idx.size
    sorted_ids = np.empty(n, dtype=np.int32)
    token_rows = np.empty(n, dtype=np.int32)
    inverse = np.empty(n, dtype=np.int32)
    _chk(lib().oracle_moe_sort(_p(idx), _i64(n), _i64(experts), top_k, _p(sorted_ids),
                               _p(token_rows), _p(inverse)), "moe_sort")
    return sorted_ids, token_rows, inverse


def moe_tile_table(sorted_ids, experts: int, tile_rows: int = 32):
    sorted_ids = np.ascontiguousarray(sorted_ids, dtype=np.int32)
    rows = sorted_ids.size
    cap = (rows + tile_rows - 1) // tile_rows + experts
    tiles = np.zeros((cap, 2), dtype=np.int32)
    count = lib().oracle_moe_tile_table(_p(sorted_ids), _i64(rows), _i64(experts), tile_rows,
                                        _p(tiles), _i64(cap))
    if count < 0:
        raise ValueError("oracle: tile table overflow")
    return tiles, int(count)


def swiglu_bf16(gate, up):
    gate = np.ascontiguousarray(gate, dtype=np.uint16)
    up = np.ascontiguousarray(up, dtype=np.uint16)
    act = np.empty_like(gate)
    lib().oracle_swiglu_bf16(_p(gate), _p(up), _i64(gate.size), _p(act))
    return act


def moe_combine(down_sorted, weights, inverse, top_k: int):
    down_sorted = np.ascontiguousarray(down_sorted, dtype=np.uint16)
    weights = np.ascontiguousarray(weights, dtype=np.float32)
    inverse = np.ascontiguousarray(inverse, dtype=np.int32).reshape(-1)
    hidden = down_sorted.shape[1]
    tokens = inverse.size // top_k
    out = np.empty((tokens, hidden), dtype=np.uint16)
    _chk(lib().oracle_moe_combine(_p(down_sorted), _p(weights), _p(inverse), _i64(tokens), top_k,
                                  _i64(hidden), _p(out)), "moe_combine")
    return out


def moe_forward(x, logits, gate, up, down, top_k: int, group_size: int = 64, bits: int = 4,
                round_weight_bf16: bool = True):
    """The generic SparseMoeBlock path without the shared expert
    (crates/lisa-engine/src/models/qwen4/moe.rs:352-481): route, stable sort,
    three gather_qmm calls with SwiGLU between, weighted un-sort.
    gate/up/down are (w, scales, biases) triples with a leading expert axis."""
    x = np.ascontiguousarray(x, dtype=np.uint16)
    experts = gate[0].shape[0]
    idx, wts = moe_route(logits, top_k)
    sorted_ids, token_rows, inverse = moe_sort(idx, experts, top_k)
    xs = x[token_rows]
    g = gather_qmm(xs, *gate, sorted_ids, group_size, bits, round_weight_bf16)
    u = gather_qmm(xs, *up, sorted_ids, group_size, bits, round_weight_bf16)
    act = swiglu_bf16(g, u)
    d = gather_qmm(act, *down, sorted_ids, group_size, bits, round_weight_bf16)
    return moe_combine(d, wts, inverse, top_k), dict(idx=idx, weights=wts, sorted_ids=sorted_ids,
                                                      token_rows=token_rows, inverse=inverse,
                                                      gate=g, up=u, act=act, down=d)


def add_rmsnorm(x, residual, weight, eps: float):
    """Residual add + RMSNorm with the rounding points of the reference's fused chain
    (crates/lisa-mlx/src/jit/matmul.rs:304-316; crates/lisa-mlx/src/shaders/common/matmul/norm_qmv.metal:159-185):
    sum = bf16(f32(x) + f32(r)); inv = 1 / sqrt(mean(sum^2) + eps); normed = bf16(w * bf16(f32(sum) * inv)).
    bf16 bit arrays [m, k] (weight [k]) in and out.  The mean is taken in f64 and inv rounded to f32 once (the
    reference accumulates in f32 in an order of its own; a kernel's inv may differ from this one in its last bits,
    which can move a normed element by one bf16 ulp)."""
    xs = bf16_to_f32(np.ascontiguousarray(x, dtype=np.uint16))
    rs = bf16_to_f32(np.ascontiguousarray(residual, dtype=np.uint16))
    ws = bf16_to_f32(np.ascontiguousarray(weight, dtype=np.uint16))
    total = f32_to_bf16((xs + rs).astype(np.float32))
    sf = bf16_to_f32(total)
    mean = np.mean(sf.astype(np.float64) ** 2, axis=-1, keepdims=True)
    inv = (1.0 / np.sqrt(mean + np.float64(np.float32(eps)))).astype(np.float32)
    inner = bf16_to_f32(f32_to_bf16((sf * inv).astype(np.float32)))
    normed = f32_to_bf16((ws[None, :] * inner).astype(np.float32))
    return total, normed
