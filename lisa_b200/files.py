"""Host-side mirror of the reference's weight-file readers over the C ABI of ``include/lisa_files.h``.

``TensorType`` / ``GgufPackage`` follow ``lisa_gguf::{TensorType, Header, Package, Tensor}``
(crates/lisa-gguf/src/{lib,header,package}.rs); ``Shard`` follows ``lisa_engine::core::loader::Shard``
(crates/lisa-engine/src/core/loader.rs:50-160).  The parsing, range checks and reads happen in the C++
library; this module only marshals.  Failures raise ``LisaError`` with the reference's messages.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Optional, Sequence

import numpy as np

from . import _cabi
from ._cabi import LisaError


class _GgufTensor(C.Structure):
    _fields_ = [("name", C.c_char_p), ("rank", C.c_uint32), ("dimensions", C.c_uint64 * 4), ("type", C.c_uint32),
                ("offset", C.c_uint64), ("bytes", C.c_uint64), ("rows", C.c_uint64), ("row_bytes", C.c_uint64),
                ("shard", C.c_int32)]


class _StTensor(C.Structure):
    _fields_ = [("name", C.c_char_p), ("dtype", C.c_int32), ("rank", C.c_int32), ("shape", C.c_int64 * 8),
                ("data", C.c_void_p), ("bytes", C.c_uint64)]


class _Triplet(C.Structure):
    _fields_ = [("weight", _StTensor), ("scales", _StTensor), ("biases", _StTensor), ("group_size", C.c_int32),
                ("bits", C.c_int32), ("n", C.c_int64), ("k", C.c_int64)]


_vp, _u64, _i64, _int = C.c_void_p, C.c_uint64, C.c_int64, C.c_int
_P = C.POINTER

# name -> (restype, argtypes); mirrors include/lisa_files.h declaration by declaration.
SIGNATURES = {
    "lisa_gguf_type_layout": (_int, [C.c_uint32, _P(C.c_char_p), _P(_u64), _P(_u64)]),
    "lisa_gguf_row_bytes": (_int, [C.c_uint32, _u64, _P(_u64)]),
    "lisa_gguf_parse": (_int, [_vp, _u64, _u64, _P(_vp)]),
    "lisa_gguf_open": (_int, [C.c_char_p, _P(_vp)]),
    "lisa_gguf_open_paths": (_int, [_P(C.c_char_p), _int, _P(_vp)]),
    "lisa_gguf_close": (None, [_vp]),
    "lisa_gguf_data_offset": (_u64, [_vp]),
    "lisa_gguf_file_bytes": (_u64, [_vp]),
    "lisa_gguf_shard_count": (_int, [_vp]),
    "lisa_gguf_shard_path": (C.c_char_p, [_vp, _int]),
    "lisa_gguf_tensor_count": (_i64, [_vp]),
    "lisa_gguf_tensor_at": (_int, [_vp, _i64, _P(_GgufTensor)]),
    "lisa_gguf_find_tensor": (_i64, [_vp, C.c_char_p]),
    "lisa_gguf_metadata_kind": (_int, [_vp, C.c_char_p]),
    "lisa_gguf_metadata_u64": (_int, [_vp, C.c_char_p, _P(_u64)]),
    "lisa_gguf_metadata_f64": (_int, [_vp, C.c_char_p, _P(C.c_double)]),
    "lisa_gguf_metadata_str": (C.c_char_p, [_vp, C.c_char_p]),
    "lisa_gguf_metadata_array_len": (_i64, [_vp, C.c_char_p]),
    "lisa_gguf_metadata_array_u64": (_int, [_vp, C.c_char_p, _i64, _P(_u64)]),
    "lisa_gguf_metadata_array_str": (C.c_char_p, [_vp, C.c_char_p, _i64]),
    "lisa_gguf_read_bytes": (_int, [_vp, _i64, _u64, _vp, _u64]),
    "lisa_gguf_read_rows": (_int, [_vp, _i64, _P(_u64), _u64, _vp, _u64]),
    "lisa_gguf_mapped_region_bytes": (_int, [_vp, _i64, _P(_u64)]),
    "lisa_gguf_map_region": (_int, [_vp, _i64, _P(_vp), _P(_u64), _P(_u64)]),
    "lisa_gguf_unmap": (_int, [_vp, _u64]),
    "lisa_gguf_weight_view": (_int, [_vp, _i64, _P(_i64), _P(_i64), _P(_i64)]),
    "lisa_safetensors_open": (_int, [C.c_char_p, _P(_vp)]),
    "lisa_safetensors_close": (None, [_vp]),
    "lisa_safetensors_tensor_count": (_i64, [_vp]),
    "lisa_safetensors_tensor_at": (_int, [_vp, _i64, _P(_StTensor)]),
    "lisa_safetensors_find": (_int, [_vp, C.c_char_p, _P(_StTensor)]),
    "lisa_detect_group_size": (C.c_int32, [C.c_int32, C.c_int32, C.c_int32]),
    "lisa_safetensors_quantized_triplet": (_int, [_vp, C.c_char_p, C.c_char_p, C.c_int32, C.c_int32, _P(_Triplet)]),
}

_bound = False


def _lib():
    global _bound
    handle = _cabi.lib()
    if not _bound:
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _bound = True
    return handle


def _check(rc: int) -> None:
    if rc != 0:
        raise LisaError(rc, _cabi.last_error())


class TensorType:
    """GGML block geometry (crates/lisa-gguf/src/lib.rs:22-83)."""
    F32, F16, Q8_0, Q2_K, Q4_K, Q5_K, IQ2_XXS, IQ2_XS, IQ4_NL, IQ1_M, BF16 = 0, 1, 8, 10, 12, 13, 16, 17, 20, 29, 30

    @staticmethod
    def layout(kind: int):
        name, block, size = C.c_char_p(), _u64(), _u64()
        _check(_lib().lisa_gguf_type_layout(kind, C.byref(name), C.byref(block), C.byref(size)))
        return name.value.decode(), block.value, size.value

    @staticmethod
    def row_bytes(kind: int, columns: int) -> int:
        out = _u64()
        _check(_lib().lisa_gguf_row_bytes(kind, columns, C.byref(out)))
        return out.value


class TensorInfo:
    """One tensor record (header.rs:58-78); ``offset`` is absolute in its shard file."""

    def __init__(self, rec: _GgufTensor, index: int):
        self.index = index
        self.name = rec.name.decode()
        self.dimensions = [int(rec.dimensions[i]) for i in range(rec.rank)]
        self.kind = int(rec.type)
        self.offset, self.bytes = int(rec.offset), int(rec.bytes)
        self._rows, self._row_bytes, self.shard = int(rec.rows), int(rec.row_bytes), int(rec.shard)

    def rows(self) -> int:
        return self._rows

    def row_bytes(self) -> int:
        return self._row_bytes


class Mapping:
    """A page-aligned read-only mapping that holds one tensor (package.rs:26-66); it outlives the package."""

    def __init__(self, ptr: int, length: int, inner: int, nbytes: int):
        self.ptr, self.length, self.inner, self.nbytes = ptr, length, inner, nbytes

    def array(self) -> np.ndarray:
        """The tensor's own bytes (never the padding around them)."""
        buf = (C.c_uint8 * self.nbytes).from_address(self.ptr + self.inner)
        a = np.frombuffer(buf, dtype=np.uint8)
        a.flags.writeable = False
        return a

    def close(self) -> None:
        if self.ptr:
            _check(_lib().lisa_gguf_unmap(self.ptr, self.length))
            self.ptr = 0

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class GgufPackage:
    """``Package`` / ``Header`` of crates/lisa-gguf/src/{package,header}.rs: header metadata of the first shard,
    the tensors of every shard, bounded disk reads and mappings."""

    def __init__(self, handle: int):
        self._h = handle
        lib = _lib()
        self.tensors: Dict[str, TensorInfo] = {}
        rec = _GgufTensor()
        for i in range(lib.lisa_gguf_tensor_count(handle)):
            _check(lib.lisa_gguf_tensor_at(handle, i, C.byref(rec)))
            info = TensorInfo(rec, i)
            self.tensors[info.name] = info
        self.data_offset = int(lib.lisa_gguf_data_offset(handle))
        self.file_bytes = int(lib.lisa_gguf_file_bytes(handle))
        self.shards = [lib.lisa_gguf_shard_path(handle, i).decode() for i in range(lib.lisa_gguf_shard_count(handle))]

    # ---- constructors
    @classmethod
    def open(cls, path: str) -> "GgufPackage":
        h = _vp()
        _check(_lib().lisa_gguf_open(str(path).encode(), C.byref(h)))
        return cls(h.value)

    @classmethod
    def open_paths(cls, paths: Sequence[str]) -> "GgufPackage":
        arr = (C.c_char_p * len(paths))(*[str(p).encode() for p in paths])
        h = _vp()
        _check(_lib().lisa_gguf_open_paths(arr, len(paths), C.byref(h)))
        return cls(h.value)

    @classmethod
    def read(cls, data: bytes, file_bytes: Optional[int] = None) -> "GgufPackage":
        """``Header::read`` on bytes in memory; `file_bytes` is the complete file's length."""
        h = _vp()
        buf = (C.c_uint8 * max(len(data), 1)).from_buffer_copy(data.ljust(1, b"\0"))
        _check(_lib().lisa_gguf_parse(buf, len(data), len(data) if file_bytes is None else file_bytes, C.byref(h)))
        return cls(h.value)

    def close(self) -> None:
        if self._h:
            _lib().lisa_gguf_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- metadata (header.rs:216-229)
    def metadata_kind(self, key: str) -> int:
        return _lib().lisa_gguf_metadata_kind(self._h, key.encode())

    def integer(self, key: str) -> int:
        out = _u64()
        _check(_lib().lisa_gguf_metadata_u64(self._h, key.encode(), C.byref(out)))
        return out.value

    def number(self, key: str) -> float:
        out = C.c_double()
        _check(_lib().lisa_gguf_metadata_f64(self._h, key.encode(), C.byref(out)))
        return out.value

    def string(self, key: str) -> Optional[str]:
        s = _lib().lisa_gguf_metadata_str(self._h, key.encode())
        return s.decode() if s is not None else None

    def architecture(self) -> str:
        s = self.string("general.architecture")
        if s is None:
            raise LisaError(_cabi.ERR_BAD_ARG, "GGUF has no general.architecture")
        return s

    def array(self, key: str) -> Optional[list]:
        n = _lib().lisa_gguf_metadata_array_len(self._h, key.encode())
        if n < 0:
            return None
        out = []
        for i in range(n):
            s = _lib().lisa_gguf_metadata_array_str(self._h, key.encode(), i)
            if s is not None:
                out.append(s.decode())
                continue
            v = _u64()
            out.append(v.value if _lib().lisa_gguf_metadata_array_u64(self._h, key.encode(), i, C.byref(v)) == 0 else None)
        return out

    # ---- tensors
    def tensor(self, name: str) -> TensorInfo:
        idx = _lib().lisa_gguf_find_tensor(self._h, name.encode())
        if idx < 0:
            raise LisaError(int(idx), _cabi.last_error())
        return self.tensors[name]

    def read_bytes(self, name: str, offset: int, length: int) -> bytes:
        info = self.tensor(name)
        buf = (C.c_uint8 * max(length, 1))()
        _check(_lib().lisa_gguf_read_bytes(self._h, info.index, offset, buf, length))
        return bytes(buf[:length])

    def read_rows(self, name: str, rows: Sequence[int], out_bytes: Optional[int] = None) -> bytes:
        info = self.tensor(name)
        n = len(rows)
        total = n * info.row_bytes() if out_bytes is None else out_bytes
        arr = (_u64 * max(n, 1))(*rows)
        buf = (C.c_uint8 * max(total, 1))()
        _check(_lib().lisa_gguf_read_rows(self._h, info.index, arr, n, buf, total))
        return bytes(buf[:total])

    def mapped_region_bytes(self, name: str) -> int:
        out = _u64()
        _check(_lib().lisa_gguf_mapped_region_bytes(self._h, self.tensor(name).index, C.byref(out)))
        return out.value

    def mapped_region(self, name: str) -> Mapping:
        info = self.tensor(name)
        ptr, length, inner = _vp(), _u64(), _u64()
        _check(_lib().lisa_gguf_map_region(self._h, info.index, C.byref(ptr), C.byref(length), C.byref(inner)))
        return Mapping(ptr.value, length.value, inner.value, info.bytes)

    def weight_view_shape(self, name: str):
        """(experts, rows, row_bytes): the uint8 view the engine hands to packed_matvec / expert_matvec
        (crates/lisa-engine/src/core/gguf_resident.rs:95-101)."""
        e, r, b = _i64(), _i64(), _i64()
        _check(_lib().lisa_gguf_weight_view(self._h, self.tensor(name).index, C.byref(e), C.byref(r), C.byref(b)))
        return e.value, r.value, b.value

    def device_weights(self, name: str, device):
        """The tensor's blocks on `device` as uint8 ``[rows, row_bytes]`` (a matrix) or ``[experts, rows,
        row_bytes]``: the `weights` argument of ``ops.packed_matvec`` / ``ops.expert_matvec``."""
        import torch

        e, r, b = self.weight_view_shape(name)
        m = self.mapped_region(name)
        try:
            t = torch.from_numpy(m.array().copy()).to(device)
        finally:
            m.close()
        return t.reshape(r, b) if len(self.tensor(name).dimensions) <= 2 else t.reshape(e, r, b)


_ST_NUMPY = {0: np.uint16, 1: np.float32, 2: np.float16, 3: np.int64, 4: np.int32, 5: np.uint32, 6: np.uint8, 7: np.bool_}
ST_DTYPE_NAMES = {0: "BF16", 1: "F32", 2: "F16", 3: "I64", 4: "I32", 5: "U32", 6: "U8", 7: "BOOL"}


class Shard:
    """An mmap'd safetensors shard (loader.rs:50-160).  Arrays returned by `tensor` are views into the mapping
    (bf16 as uint16 bit patterns) and are valid while the shard is open."""

    def __init__(self, path: str):
        h = _vp()
        _check(_lib().lisa_safetensors_open(str(path).encode(), C.byref(h)))
        self._h = h.value

    @classmethod
    def open(cls, path: str) -> "Shard":
        return cls(path)

    def close(self) -> None:
        if self._h:
            _lib().lisa_safetensors_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _view(self, rec: _StTensor) -> np.ndarray:
        shape = tuple(int(rec.shape[i]) for i in range(rec.rank))
        if rec.bytes == 0:
            return np.zeros(shape, dtype=_ST_NUMPY[rec.dtype])
        buf = (C.c_uint8 * rec.bytes).from_address(rec.data)
        a = np.frombuffer(buf, dtype=_ST_NUMPY[rec.dtype]).reshape(shape)
        a.flags.writeable = False
        return a

    def tensor_names(self) -> List[str]:
        rec = _StTensor()
        names = []
        for i in range(_lib().lisa_safetensors_tensor_count(self._h)):
            _check(_lib().lisa_safetensors_tensor_at(self._h, i, C.byref(rec)))
            names.append(rec.name.decode())
        return names

    def tensor(self, name: str):
        """(array, dtype name): ``tensor_bytes`` of loader.rs:151-155 with the shape applied."""
        rec = _StTensor()
        _check(_lib().lisa_safetensors_find(self._h, name.encode(), C.byref(rec)))
        return self._view(rec), ST_DTYPE_NAMES[rec.dtype]

    def quantized_triplet(self, prefix: str, key: str = "", bits: int = 4, group_size_hint: int = 64):
        """``{prefix}.{key}.weight/.scales/.biases`` with the group size detected from the shapes
        (quant.rs:408-432).  Returns (weight u32, scales bits, biases bits, group_size, bits)."""
        t = _Triplet()
        _check(_lib().lisa_safetensors_quantized_triplet(self._h, prefix.encode(), key.encode(), bits, group_size_hint, C.byref(t)))
        return self._view(t.weight), self._view(t.scales), self._view(t.biases), int(t.group_size), int(t.bits)


def detect_group_size(weight_cols: int, scales_cols: int, bits: int) -> Optional[int]:
    """``detect_group_size`` (quant.rs:273-287) through the library; None when the shapes are inconsistent."""
    g = _lib().lisa_detect_group_size(weight_cols, scales_cols, bits)
    return int(g) if g else None
