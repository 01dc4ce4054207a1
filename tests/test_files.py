"""The host-side weight-file readers (include/lisa_files.h) against the cases the reference's own tests hold
(crates/lisa-gguf/src/tests.rs, crates/lisa-engine/src/core/quant.rs tests): GGUF header geometry and range
checks, rejections, truncation, bounded ordered disk reads, mapping offsets; safetensors shards and the
{weight, scales, biases} triplet with group-size detection.  CPU only."""
import json
import mmap
import os
import struct

import numpy as np
import pytest

import __graft_entry__ as entry
from lisa_b200 import _cabi, files
from lisa_b200.files import GgufPackage, Shard, TensorType
from lisa_b200._cabi import LisaError


@pytest.fixture(scope="module", autouse=True)
def built():
    if not os.path.exists(_cabi.LIB_PATH):
        entry.build()


def gstring(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def gguf_bytes(tensors, payload: bytes, metadata=None, alignment=32) -> bytes:
    """A GGUF v3 file: `tensors` = (name, dims, type id, offset); metadata = list of (key, type id, encoded value)."""
    metadata = metadata if metadata is not None else [("general.architecture", 8, gstring("deepseek41"))]
    out = b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(metadata))
    for key, kind, enc in metadata:
        out += gstring(key) + struct.pack("<I", kind) + enc
    for name, dims, kind, offset in tensors:
        out += gstring(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        out += struct.pack("<IQ", kind, offset)
    out += b"\0" * (-len(out) % alignment)
    return out + payload


def test_type_geometry():
    assert TensorType.layout(TensorType.Q2_K) == ("Q2_K", 256, 84)
    assert TensorType.layout(TensorType.Q4_K) == ("Q4_K", 256, 144)
    assert TensorType.layout(TensorType.IQ4_NL) == ("IQ4_NL", 32, 18)
    assert TensorType.layout(39) == ("MXFP4", 32, 17)
    assert TensorType.row_bytes(TensorType.Q2_K, 7168) == 2352 and TensorType.row_bytes(TensorType.Q4_K, 18432) == 10368
    with pytest.raises(LisaError, match="not a positive multiple"):
        TensorType.row_bytes(TensorType.Q4_K, 100)
    with pytest.raises(LisaError, match="unsupported GGUF tensor type"):
        TensorType.layout(999)


def test_header_geometry_and_range_checks():
    tensors = [("a", [256, 2], TensorType.IQ1_M, 0), ("b", [32, 4], TensorType.IQ4_NL, 128)]
    data = gguf_bytes(tensors, bytes(200))
    h = GgufPackage.read(data)
    assert h.tensors["a"].bytes == 112 and h.tensors["b"].bytes == 72
    assert h.tensors["b"].offset == h.data_offset + 128
    assert h.architecture() == "deepseek41"
    with pytest.raises(LisaError):
        GgufPackage.read(data, len(data) - 1)
    overlap = gguf_bytes([("a", [32, 2], TensorType.Q8_0, 0), ("b", [32, 2], TensorType.Q8_0, 32)], bytes(100))
    with pytest.raises(LisaError, match="overlapping GGUF tensors a and b"):
        GgufPackage.read(overlap)


def test_header_rejects_invalid_types_dimensions_and_duplicates():
    for tensor in [("a", [31], TensorType.IQ4_NL, 0), ("a", [0], TensorType.F32, 0), ("a", [2 ** 64 - 1, 2], TensorType.F32, 0),
                   ("a", [32], 999, 0), ("a", [32], TensorType.Q8_0, 1)]:
        with pytest.raises(LisaError):
            GgufPackage.read(gguf_bytes([tensor], bytes(128)))
    dup = gguf_bytes([("a", [1], TensorType.F32, 0), ("a", [1], TensorType.F32, 32)], bytes(36))
    with pytest.raises(LisaError, match="duplicate GGUF tensor a"):
        GgufPackage.read(dup)
    with pytest.raises(LisaError, match="invalid GGUF magic"):
        GgufPackage.read(b"GGML" + bytes(60))
    with pytest.raises(LisaError, match="only GGUF version 3"):
        GgufPackage.read(b"GGUF" + struct.pack("<IQQ", 2, 0, 0) + bytes(40))


def test_header_truncation_is_an_error():
    data = gguf_bytes([("a", [32], TensorType.Q8_0, 0)], bytes(34))
    h = GgufPackage.read(data)
    # a header-only download may omit tensor payloads, never part of the metadata or of the tensor descriptors
    for length in range(h.data_offset - 31):
        with pytest.raises(LisaError):
            GgufPackage.read(data[:length], len(data))
    assert GgufPackage.read(data[:h.data_offset], len(data)).tensors["a"].bytes == 34


def test_metadata_values():
    meta = [("general.architecture", 8, gstring("glm")), ("general.alignment", 4, struct.pack("<I", 64)),
            ("x.count", 10, struct.pack("<Q", 2 ** 40)), ("x.neg", 5, struct.pack("<i", -7)), ("x.f", 6, struct.pack("<f", 1.5)),
            ("x.flag", 7, b"\x01"), ("x.names", 9, struct.pack("<IQ", 8, 2) + gstring("q") + gstring("k")),
            ("x.sizes", 9, struct.pack("<IQ", 4, 3) + struct.pack("<III", 1, 2, 3))]
    data = gguf_bytes([("a", [32], TensorType.Q8_0, 64)], bytes(128), metadata=meta, alignment=64)
    h = GgufPackage.read(data)
    assert h.architecture() == "glm" and h.integer("x.count") == 2 ** 40 and h.number("x.f") == 1.5
    assert h.array("x.names") == ["q", "k"] and h.array("x.sizes") == [1, 2, 3]
    assert h.tensors["a"].offset == h.data_offset + 64 and h.data_offset % 64 == 0
    with pytest.raises(LisaError, match="missing or invalid GGUF integer x.neg"):
        h.integer("x.neg")
    assert h.metadata_kind("x.flag") == 3 and h.metadata_kind("nope") == -1
    nested = [("general.architecture", 8, gstring("glm")), ("bad", 9, struct.pack("<IQ", 9, 1))]
    with pytest.raises(LisaError, match="invalid GGUF array element type"):
        GgufPackage.read(gguf_bytes([], b"", metadata=nested))
    with pytest.raises(LisaError, match="duplicate GGUF key"):
        GgufPackage.read(gguf_bytes([], b"", metadata=[meta[0], meta[0]]))


def test_disk_reads_are_bounded_and_ordered(tmp_path):
    values = np.arange(16, dtype="<f4").tobytes()
    path = tmp_path / "a.gguf"
    path.write_bytes(gguf_bytes([("a", [4, 4], TensorType.F32, 0)], values))
    pkg = GgufPackage.open(str(path))
    got = pkg.read_rows("a", [3, 0, 3])
    assert got[:16] == values[48:64] and got[16:32] == values[:16] and got[32:48] == values[48:64]
    with pytest.raises(LisaError, match="GGUF row index out of range"):
        pkg.read_rows("a", [4])
    with pytest.raises(LisaError, match="read outside GGUF tensor a"):
        pkg.read_bytes("a", 63, 2)
    with pytest.raises(LisaError, match="invalid or oversized GGUF row output buffer"):
        pkg.read_rows("a", [0], out_bytes=8)
    with pytest.raises(LisaError, match="missing GGUF tensor b"):
        pkg.tensor("b")


def test_mapping_preserves_payload_offset_and_lifetime(tmp_path):
    values = np.arange(16, dtype="<f4").tobytes()
    path = tmp_path / "m.gguf"
    path.write_bytes(gguf_bytes([("a", [4, 4], TensorType.F32, 0)], values))
    pkg = GgufPackage.open(str(path))
    page = mmap.PAGESIZE
    m = pkg.mapped_region("a")
    assert m.length == pkg.mapped_region_bytes("a") and m.length % page == 0 and m.ptr % page == 0
    assert m.inner == pkg.tensor("a").offset % page and m.inner != 0
    assert m.inner + len(values) <= m.length
    assert pkg.weight_view_shape("a") == (1, 4, 16)
    pkg.close()  # the mapping outlives the package
    assert m.array().tobytes() == values
    m.close()


def _split_meta(no, count, total, arch="glm"):
    return [("general.architecture", 8, gstring(arch)), ("split.no", 2, struct.pack("<H", no)),
            ("split.count", 2, struct.pack("<H", count)), ("split.tensors.count", 5, struct.pack("<i", total))]


def test_split_package(tmp_path):
    a = gguf_bytes([("blk.0.w", [256, 8], TensorType.Q4_K, 0)], bytes(8 * 144), metadata=_split_meta(0, 2, 2))
    b = gguf_bytes([("blk.1.w", [256, 8, 3], TensorType.Q2_K, 0)], bytes(24 * 84), metadata=_split_meta(1, 2, 2))
    (tmp_path / "m-00001-of-00002.gguf").write_bytes(a)
    (tmp_path / "m-00002-of-00002.gguf").write_bytes(b)
    pkg = GgufPackage.open(str(tmp_path / "m-00001-of-00002.gguf"))
    assert len(pkg.shards) == 2 and sorted(pkg.tensors) == ["blk.0.w", "blk.1.w"]
    assert pkg.tensor("blk.1.w").shard == 1 and pkg.weight_view_shape("blk.1.w") == (3, 8, 84)
    assert pkg.weight_view_shape("blk.0.w") == (1, 8, 144)
    with pytest.raises(LisaError, match="pass the first GGUF shard"):
        GgufPackage.open(str(tmp_path / "m-00002-of-00002.gguf"))
    with pytest.raises(LisaError, match="GGUF shard count mismatch"):
        GgufPackage.open_paths([str(tmp_path / "m-00001-of-00002.gguf")])
    (tmp_path / "n-00001-of-00002.gguf").write_bytes(a)
    with pytest.raises(LisaError, match="missing GGUF shard"):
        GgufPackage.open(str(tmp_path / "n-00001-of-00002.gguf"))
    (tmp_path / "n-00002-of-00002.gguf").write_bytes(gguf_bytes([("blk.0.w", [256, 8], TensorType.Q4_K, 0)], bytes(8 * 144),
                                                                metadata=_split_meta(1, 2, 2)))
    with pytest.raises(LisaError, match="duplicate GGUF tensor blk.0.w across shards"):
        GgufPackage.open(str(tmp_path / "n-00001-of-00002.gguf"))


# ------------------------------------------------------------------------------------------ safetensors
def st_bytes(tensors, metadata=None) -> bytes:
    """tensors: name -> (dtype name, numpy array as stored)."""
    header, payload = {}, b""
    if metadata:
        header["__metadata__"] = metadata
    for name, (dtype, arr) in tensors.items():
        raw = np.ascontiguousarray(arr).tobytes()
        header[name] = {"dtype": dtype, "shape": list(arr.shape), "data_offsets": [len(payload), len(payload) + len(raw)]}
        payload += raw
    h = json.dumps(header, separators=(",", ":")).encode()
    h += b" " * (-len(h) % 8)
    return struct.pack("<Q", len(h)) + h + payload


def test_detect_group_size():
    # K = 2560: 4-bit weights have 320 columns; 40 scale columns are group 64, 80 are group 32
    assert files.detect_group_size(320, 40, 4) == 64 and files.detect_group_size(320, 80, 4) == 32
    assert files.detect_group_size(160, 40, 2) == 64 and files.detect_group_size(640, 20, 8) == 128
    assert files.detect_group_size(320, 7, 4) is None and files.detect_group_size(0, 40, 4) is None
    assert files.detect_group_size(320, 40, 3) is None and files.detect_group_size(320, 40, 0) is None
    assert files.detect_group_size(2 ** 30, 1, 4) is None  # k overflows 32 bits
    from lisa_b200 import quant
    for args in [(320, 40, 4), (320, 80, 4), (320, 7, 4), (160, 40, 2), (0, 1, 4), (2 ** 20, 1, 4)]:
        assert quant.detect_group_size(*args) == files.detect_group_size(*args)


def test_shard_and_quantized_triplet(tmp_path):
    rng = np.random.default_rng(0)
    w = rng.integers(0, 2 ** 32, size=(16, 40), dtype=np.uint32)      # K = 320 at 4 bits
    s = rng.integers(0, 2 ** 16, size=(16, 10), dtype=np.uint16)      # group 32
    b = rng.integers(0, 2 ** 16, size=(16, 10), dtype=np.uint16)
    e = rng.integers(0, 2 ** 32, size=(8, 16, 40), dtype=np.uint32)   # experts
    es = rng.integers(0, 2 ** 16, size=(8, 16, 5), dtype=np.uint16)   # group 64
    path = tmp_path / "model.safetensors"
    path.write_bytes(st_bytes({"m.q_proj.weight": ("U32", w), "m.q_proj.scales": ("BF16", s), "m.q_proj.biases": ("BF16", b),
                               "m.experts.weight": ("U32", e), "m.experts.scales": ("BF16", es), "m.experts.biases": ("BF16", es),
                               "m.norm.weight": ("F32", np.ones(4, dtype=np.float32))}, metadata={"format": "mlx"}))
    sh = Shard.open(str(path))
    assert sh.tensor_names() == sorted(["m.q_proj.weight", "m.q_proj.scales", "m.q_proj.biases", "m.experts.weight",
                                        "m.experts.scales", "m.experts.biases", "m.norm.weight"])
    arr, dt = sh.tensor("m.norm.weight")
    assert dt == "F32" and np.array_equal(arr, np.ones(4, dtype=np.float32))
    tw, ts, tb, gs, bits = sh.quantized_triplet("m", "q_proj", bits=4, group_size_hint=64)
    assert gs == 32 and bits == 4 and np.array_equal(tw, w) and np.array_equal(ts, s) and np.array_equal(tb, b)
    tw, ts, tb, gs, bits = sh.quantized_triplet("m.experts", "", bits=4)
    assert gs == 64 and tw.shape == (8, 16, 40) and np.array_equal(ts, es)
    with pytest.raises(LisaError, match="tensor m.k_proj.weight missing from shard"):
        sh.quantized_triplet("m", "k_proj")
    with pytest.raises(LisaError, match="tensor m.norm.scales missing from shard"):
        sh.quantized_triplet("m", "norm")
    sh.close()


def test_shard_rejections(tmp_path):
    def write(raw):
        p = tmp_path / "bad.safetensors"
        p.write_bytes(raw)
        return str(p)

    good = st_bytes({"a": ("F32", np.zeros((2, 2), dtype=np.float32))})
    with pytest.raises(LisaError, match="too small"):
        Shard.open(write(b"abc"))
    with pytest.raises(LisaError, match="invalid or oversized header"):
        Shard.open(write(struct.pack("<Q", 10 ** 9) + b"{}"))
    with pytest.raises(LisaError, match="parsing shard header"):
        Shard.open(write(struct.pack("<Q", 4) + b"{,,}"))
    with pytest.raises(LisaError, match="must be an object"):
        Shard.open(write(struct.pack("<Q", 2) + b"[]"))

    def header(obj, payload=b""):
        h = json.dumps(obj).encode()
        return struct.pack("<Q", len(h)) + h + payload

    with pytest.raises(LisaError, match="unsupported dtype F64 for a"):
        Shard.open(write(header({"a": {"dtype": "F64", "shape": [1], "data_offsets": [0, 8]}}, bytes(8))))
    with pytest.raises(LisaError, match="exceeds shard payload bounds"):
        Shard.open(write(header({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}, bytes(8))))
    with pytest.raises(LisaError, match="tensor byte size differs from shape for a"):
        Shard.open(write(header({"a": {"dtype": "F32", "shape": [3], "data_offsets": [0, 16]}}, bytes(16))))
    with pytest.raises(LisaError, match="missing shape for a"):
        Shard.open(write(header({"a": {"dtype": "F32", "data_offsets": [0, 16]}}, bytes(16))))
    with pytest.raises(LisaError, match="data_offsets must have two entries for a"):
        Shard.open(write(header({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0]}}, bytes(16))))
    with pytest.raises(LisaError, match="invalid dimension for a"):
        Shard.open(write(header({"a": {"dtype": "F32", "shape": [-1], "data_offsets": [0, 0]}}, b"")))
    assert Shard.open(write(good)).tensor("a")[0].shape == (2, 2)


def test_header_declares_what_the_library_exports():
    import re
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    text = re.sub(r"/\*.*?\*/", "", open(os.path.join(root, "include", "lisa_files.h")).read(), flags=re.S)
    names = sorted(set(re.findall(r"\b(lisa_(?:gguf|safetensors|detect)_\w+)\s*\(", text)))
    assert set(names) == set(files.SIGNATURES)
    lib = _cabi.lib()
    for name in names:
        assert hasattr(lib, name), name
