"""The C-ABI library loads without a GPU, exports every symbol the header declares, and
rejects bad arguments on the host before touching CUDA."""
import ctypes
import os
import re

import pytest

import __graft_entry__ as entry
from lisa_b200 import _cabi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(_cabi.LIB_PATH):
        entry.build()
    return _cabi.lib()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "lisa_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lisa_cuda_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = declared_symbols()
    assert len(names) >= 18
    for name in names:
        assert hasattr(lib, name), name
    assert set(names) == set(_cabi.SIGNATURES), "ctypes table and header disagree"


def test_rust_binding_names_every_export():
    """rust/lisa-cuda-sys (source only, never compiled here) declares every function of both headers."""
    rust = open(os.path.join(ROOT, "rust", "lisa-cuda-sys", "src", "lib.rs")).read()
    declared = set(re.findall(r"\bpub fn (lisa_\w+)\s*\(", rust))
    wanted = set(declared_symbols())
    files = re.sub(r"/\*.*?\*/", "", open(os.path.join(ROOT, "include", "lisa_files.h")).read(), flags=re.S)
    wanted |= set(re.findall(r"\b(lisa_(?:gguf|safetensors|detect)\w*)\s*\(", files))
    assert wanted and wanted <= declared, sorted(wanted - declared)


def test_version(lib):
    assert lib.lisa_cuda_version() >= 100


def _qmm(lib, **kw):
    a = dict(stream=None, x=16, m=1, k=64, w=16, scales=16, biases=16, n=8, transpose=1, gs=64, bits=4, dtype=0, y=16)
    a.update(kw)
    return lib.lisa_cuda_quantized_matmul(a["stream"], a["x"], a["m"], a["k"], a["w"], a["scales"], a["biases"],
                                          a["n"], a["transpose"], a["gs"], a["bits"], a["dtype"], a["y"])


def test_quantized_matmul_rejections_mirror_the_reference(lib):
    # array_ops.rs:387-392: transpose=false and missing biases are refused
    assert _qmm(lib, transpose=0) == _cabi.ERR_UNSUPPORTED
    assert "only transpose=true supported" in _cabi.last_error()
    assert _qmm(lib, biases=None) == _cabi.ERR_BAD_ARG
    assert "affine biases required" in _cabi.last_error()
    assert _qmm(lib, bits=3) == _cabi.ERR_UNSUPPORTED
    assert _qmm(lib, gs=48) == _cabi.ERR_UNSUPPORTED
    assert _qmm(lib, dtype=3) == _cabi.ERR_UNSUPPORTED   # bf16, f16 and f32 are the compute dtypes
    assert _qmm(lib, k=96) == _cabi.ERR_BAD_ARG  # not a multiple of the group size
    assert _qmm(lib, m=0) == _cabi.ERR_BAD_ARG
    assert _qmm(lib, x=8) == _cabi.ERR_MISALIGNED
    assert _qmm(lib, k=1 << 31) == _cabi.ERR_OVERFLOW


def test_gather_qmm_rejections(lib):
    def call(**kw):
        a = dict(x=16, rows=4, k=64, w=16, s=16, b=16, lhs=None, rhs=16, e=2, n=8, t=1, gs=64, bits=4, sorted=1,
                 dtype=0, y=16, ws=None, wsb=0)
        a.update(kw)
        return lib.lisa_cuda_gather_qmm(None, a["x"], a["rows"], a["k"], a["w"], a["s"], a["b"], a["lhs"], a["rhs"],
                                        a["e"], a["n"], a["t"], a["gs"], a["bits"], a["sorted"], a["dtype"], a["y"],
                                        a["ws"], a["wsb"])
    # array_ops.rs:573-585
    assert call(t=0) == _cabi.ERR_UNSUPPORTED
    assert call(lhs=16) == _cabi.ERR_UNSUPPORTED and "lhs_indices path not ported" in _cabi.last_error()
    assert call(sorted=0) == _cabi.ERR_UNSUPPORTED
    assert call(rhs=None) == _cabi.ERR_BAD_ARG and "rhs_indices required" in _cabi.last_error()
    assert call(b=None) == _cabi.ERR_BAD_ARG
    assert call() == _cabi.ERR_WORKSPACE  # no workspace given
    assert lib.lisa_cuda_gather_qmm_workspace_bytes(512, 128) > 0


def test_decode_block_rejections(lib):
    def gate(**kw):
        a = dict(x=16, idx=16, xrow=None, slots=8, top_k=8, e=4, hidden=256, inter=128, wg=16, sg=16, bg=16, wu=16, su=16,
                 bu=16, gs=64, bits=4, dtype=0, act=16)
        a.update(kw)
        return lib.lisa_cuda_moe_gate_up_act(None, a["x"], a["idx"], a["xrow"], a["slots"], a["top_k"], a["e"], a["hidden"],
                                             a["inter"], a["wg"], a["sg"], a["bg"], a["wu"], a["su"], a["bu"], a["gs"],
                                             a["bits"], a["dtype"], a["act"])

    def down(**kw):
        a = dict(act=16, idx=16, w=16, tokens=1, top_k=8, e=4, inter=128, hidden=256, wd=16, sd=16, bd=16, gs=64, bits=4,
                 dtype=0, out=16)
        a.update(kw)
        return lib.lisa_cuda_moe_down_combine(None, a["act"], a["idx"], a["w"], a["tokens"], a["top_k"], a["e"], a["inter"],
                                              a["hidden"], a["wd"], a["sd"], a["bd"], a["gs"], a["bits"], a["dtype"], a["out"])
    for call in (gate, down):
        assert call(idx=None) == _cabi.ERR_BAD_ARG
        assert call(bits=3) == _cabi.ERR_UNSUPPORTED
        assert call(bits=8) == _cabi.ERR_UNSUPPORTED
        assert call(gs=48) == _cabi.ERR_UNSUPPORTED
        assert call(top_k=33) == _cabi.ERR_LIMIT
        assert call(dtype=2) == _cabi.ERR_UNSUPPORTED
        assert call(e=0) == _cabi.ERR_BAD_ARG
    assert gate(x=8) == _cabi.ERR_MISALIGNED
    assert gate(hidden=72) == _cabi.ERR_UNSUPPORTED      # packed rows that are not whole 16-byte chunks
    assert gate(slots=0) == _cabi.ERR_BAD_ARG and down(tokens=0) == _cabi.ERR_BAD_ARG


def test_addnorm_rejections(lib):
    import ctypes as C
    one = (C.c_void_p * 1)(16)
    ns = (C.c_int64 * 1)(128)

    def call(x=16, r=16, nw=16, eps=1e-6, m=1, k=256, count=1, w=one, tr=1, gs=64, bits=4, dtype=0, y=one, total=16, normed=16):
        return lib.lisa_cuda_quantized_matmul_addnorm(None, x, r, nw, eps, m, k, count, w, one, one, ns, tr, gs, bits, dtype, y, total,
                                                      normed, 0)
    assert call(r=None) == _cabi.ERR_BAD_ARG
    assert call(total=None) == _cabi.ERR_BAD_ARG
    assert call(tr=0) == _cabi.ERR_UNSUPPORTED
    assert call(count=4) == _cabi.ERR_BAD_ARG
    assert call(eps=-1.0) == _cabi.ERR_BAD_ARG
    assert call(dtype=2) == _cabi.ERR_UNSUPPORTED
    assert call(nw=8) == _cabi.ERR_MISALIGNED
    sw = lib.lisa_cuda_quantized_matmul_swiglu
    assert sw(None, 16, None, 1, 256, 16, 16, 16, 128, 1, 64, 4, 0, 16, None, 0) == _cabi.ERR_BAD_ARG       # no up
    assert sw(None, 16, 16, 1, 256, 16, 16, 16, 128, 0, 64, 4, 0, 16, None, 0) == _cabi.ERR_UNSUPPORTED   # transpose
    assert sw(None, 16, 24, 1, 256, 16, 16, 16, 128, 1, 64, 4, 0, 16, None, 0) == _cabi.ERR_MISALIGNED
    assert sw(None, 16, 16, 1, 256, 16, 16, None, 128, 1, 64, 4, 0, 16, None, 0) == _cabi.ERR_BAD_ARG     # affine biases required
    f = lib.lisa_cuda_add_rmsnorm
    assert f(None, 16, 16, 16, 1e-6, 1, 12, 0, 16, 16) == _cabi.ERR_BAD_ARG        # k % 8
    assert f(None, 16, 16, 16, 1e-6, 1, 64, 0, 16, None) == _cabi.ERR_BAD_ARG
    assert f(None, 16, 16, 16, 1e-6, 1, 64, 1, 16, 16) == _cabi.ERR_UNSUPPORTED    # bf16 only
    assert f(None, 16, 24, 16, 1e-6, 1, 64, 0, 16, 16) == _cabi.ERR_MISALIGNED


def test_gguf_rejections(lib):
    f = lib.lisa_cuda_gguf_packed_matvec
    # deepseek41.rs:50-65,100-101
    assert f(None, 10, 16, 12, 84, 16, 1, 16) == _cabi.ERR_BAD_ARG      # rows % 8
    assert f(None, 10, 16, 16, 85, 16, 1, 16) == _cabi.ERR_BAD_ARG      # row_bytes % block
    assert f(None, 10, 16, 16, 84, 16, 0, 16) == _cabi.ERR_BAD_ARG      # tokens < 1
    assert f(None, 10, 16, 16, 84, 16, 65536, 16) == _cabi.ERR_BAD_ARG  # tokens > 65535
    assert f(None, 11, 16, 16, 84, 16, 1, 16) == _cabi.ERR_UNSUPPORTED  # Q3_K is not on the path
    g = lib.lisa_cuda_gguf_expert_matvec
    assert g(None, 12, 16, 4, 8, 144, 16, 2, 3, 16, 6, 16) == _cabi.ERR_BAD_ARG   # slots not in {1, top_k}
    assert g(None, 12, 16, 4, 8, 144, 16, 2, 1, 16, 33, 16) == _cabi.ERR_BAD_ARG  # top_k > 32


def test_allgather_and_peer_barrier_rejections(lib):
    import ctypes as C

    ag, pb = lib.lisa_cuda_quantized_matmul_allgather, lib.lisa_cuda_peer_barrier
    table = (C.c_void_p * 8)(*([0x1000] * 8))  # never dereferenced: every call below is refused on the host
    def call(world=2, n_local=128, n_total=256, col0=0, m=1, gs=64, tr=1, tbl=table):
        return ag(None, 0x1000, m, 256, 0x1000, 0x1000, 0x1000, n_local, tr, gs, 4, _cabi.BF16, tbl, world, n_total, col0, 0)
    assert call(world=0) == _cabi.ERR_BAD_ARG and call(world=9) == _cabi.ERR_BAD_ARG
    assert call(tbl=None) == _cabi.ERR_BAD_ARG
    assert call(tr=0) == _cabi.ERR_UNSUPPORTED
    assert call(col0=200) == _cabi.ERR_BAD_ARG          # block past the end of the output
    assert call(gs=128) == _cabi.ERR_UNSUPPORTED         # the tensor-memory GEMV is group size 64
    assert pb(None, 2, 2, table, 1) == _cabi.ERR_BAD_ARG  # rank outside the world
    assert pb(None, 0, 0, table, 1) == _cabi.ERR_BAD_ARG
    assert pb(None, 0, 2, None, 1) == _cabi.ERR_BAD_ARG


def test_sibling_linears_rejections(lib):
    import ctypes as C

    f = lib.lisa_cuda_quantized_matmul_siblings
    ptrs = (C.c_void_p * 3)(*([0x1000] * 3))  # never dereferenced: every call below is refused on the host
    ns = (C.c_int64 * 3)(128, 128, 128)
    def call(count=2, w=ptrs, n=ns, tr=1, bits=4, k=256):
        return f(None, 0x1000, 1, k, count, w, ptrs, ptrs, n, tr, 64, bits, _cabi.BF16, ptrs, 0)
    assert call(count=0) == _cabi.ERR_BAD_ARG and call(count=4) == _cabi.ERR_BAD_ARG
    assert call(w=None) == _cabi.ERR_BAD_ARG and call(n=None) == _cabi.ERR_BAD_ARG
    assert call(tr=0) == _cabi.ERR_UNSUPPORTED
    assert call(bits=3) == _cabi.ERR_UNSUPPORTED
    assert call(k=250) == _cabi.ERR_BAD_ARG               # k not a multiple of the group size
    assert call(n=(C.c_int64 * 3)(128, 0, 128)) == _cabi.ERR_BAD_ARG


def test_gguf_matmul_workspace_and_rejections(lib):
    ws = lib.lisa_cuda_gguf_packed_matmul_workspace_bytes
    assert ws(512, 28 * 144, _cabi.GGUF_Q4_K) >= 2 * 512 * 7168 * 2
    assert ws(0, 144, _cabi.GGUF_Q4_K) == 0
    f = lib.lisa_cuda_gguf_packed_matmul
    assert f(None, 12, 16, 12, 144, 16, 64, 16, None, 0) == _cabi.ERR_BAD_ARG      # rows % 8
    assert f(None, 11, 16, 16, 144, 16, 64, 16, None, 0) == _cabi.ERR_UNSUPPORTED  # Q3_K is not on the path


def test_product_package_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "lisa_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".hpp")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower() or f == "__never__", f"{f} mentions the oracle"
