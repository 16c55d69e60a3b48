"""GGUF files in front of the backend: `GgufFile` mirrors src/gguf/mod.rs (open, metadata, tensors,
tensor_view) and `Loader` mirrors the upload helper of src/arch/mod.rs:40-68, over the C ABI
(`llmrs_gguf_*`, `llmrs_cuda_upload_gguf_tensor` in include/llmrs_cuda.h).

The directory is parsed by the native library; tensor bytes are only read when asked for, and
`Loader.opt` moves them file -> pinned staging -> device without a host copy of the tensor."""
from __future__ import annotations

import ctypes as C
import dataclasses
import os
import sys
import time
from typing import Dict, List, Optional, Sequence

import numpy as np

from .backend import BackendError, CudaBackend, CudaBuffer, DType, TensorView, _Buf, _GgufTensor, load_library

# llmrs_gguf_type -> numpy dtype of packed array elements
_NP = {0: np.uint8, 1: np.int8, 2: np.uint16, 3: np.int16, 4: np.uint32, 5: np.int32, 6: np.float32, 7: np.bool_,
       10: np.uint64, 11: np.int64, 12: np.float64}
_STRING, _ARRAY = 8, 9


class GgufError(RuntimeError):
    """A `llmrs_gguf_*` call failed (GgufError, src/gguf/mod.rs:88-115)."""

    def __init__(self, code: int, message: str):
        super().__init__(message)
        self.code = code


@dataclasses.dataclass(frozen=True)
class TensorInfo:
    """src/gguf/mod.rs:14-24, with the name and shape resolved."""
    name: str
    dtype: int                    # GGUF type id; DType(dtype) for the ones the backend holds
    shape: Sequence[int]
    offset: int
    nbytes: int


class GgufFile:
    """src/gguf/mod.rs:80-86."""

    def __init__(self, path: str):
        self._lib = load_library()
        self._h = C.c_void_p()
        rc = self._lib.llmrs_gguf_open(os.fsencode(path), C.byref(self._h))
        if rc != 0:
            self._h = None
            raise GgufError(rc, self._err())
        self.path = path
        self.version = int(self._lib.llmrs_gguf_version(self._h))
        self.data_offset = int(self._lib.llmrs_gguf_data_offset(self._h))
        self.tensors: List[TensorInfo] = []
        info = _GgufTensor()
        for i in range(self._lib.llmrs_gguf_tensor_count(self._h)):
            self._ok(self._lib.llmrs_gguf_tensor_at(self._h, i, C.byref(info)))
            self.tensors.append(self._info(info))
        self.metadata: Dict[str, object] = self._read_metadata()

    @classmethod
    def open(cls, path: str) -> "GgufFile":
        """src/gguf/mod.rs:167."""
        return cls(path)

    def close(self) -> None:
        if self._h:
            self._lib.llmrs_gguf_close(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _err(self) -> str:
        return (self._lib.llmrs_gguf_last_error() or b"").decode(errors="replace")

    def _ok(self, rc: int) -> None:
        if rc != 0:
            raise GgufError(rc, self._err())

    @staticmethod
    def _info(t: _GgufTensor) -> TensorInfo:
        return TensorInfo(t.name.decode(), int(t.dtype), tuple(int(t.shape[d]) for d in range(t.n_dims)),
                          int(t.offset), int(t.nbytes))

    def _read_metadata(self) -> Dict[str, object]:
        out: Dict[str, object] = {}
        key, typ, et, cnt = C.c_char_p(), C.c_uint32(), C.c_uint32(), C.c_uint64()
        for i in range(self._lib.llmrs_gguf_metadata_count(self._h)):
            self._ok(self._lib.llmrs_gguf_metadata_at(self._h, i, C.byref(key), C.byref(typ), C.byref(et), C.byref(cnt)))
            k = key.value
            out[k.decode()] = self._value(k, typ.value, et.value, cnt.value)
        return out

    def _value(self, k: bytes, typ: int, et: int, cnt: int):
        if typ == _STRING:
            p, n = C.c_void_p(), C.c_uint64()
            self._ok(self._lib.llmrs_gguf_get_str(self._h, k, C.byref(p), C.byref(n)))
            return C.string_at(p, n.value).decode()
        if typ == _ARRAY:
            if et == _STRING:
                p, n = C.c_void_p(), C.c_uint64()
                vals = []
                for j in range(cnt):
                    self._ok(self._lib.llmrs_gguf_get_array_str(self._h, k, j, C.byref(p), C.byref(n)))
                    vals.append(C.string_at(p, n.value).decode())
                return vals
            p = C.c_void_p()
            self._ok(self._lib.llmrs_gguf_get_array(self._h, k, None, None, C.byref(p)))
            dt = np.dtype(_NP[et])
            if cnt == 0:
                return np.empty(0, dt)
            return np.frombuffer(C.string_at(p, cnt * dt.itemsize), dtype=dt).copy()
        if typ in (6, 12):
            v = C.c_double()
            self._ok(self._lib.llmrs_gguf_get_f64(self._h, k, C.byref(v)))
            return float(v.value)
        v = C.c_uint64()
        self._ok(self._lib.llmrs_gguf_get_u64(self._h, k, C.byref(v)))
        if typ == 7:
            return bool(v.value)
        if typ in (1, 3, 5, 11):                  # signed: the library sign-extends to 64 bits
            return int(C.c_int64(v.value).value)
        return int(v.value)

    def file_size(self) -> int:
        """src/gguf/mod.rs:224-226."""
        return int(self._lib.llmrs_gguf_file_size(self._h))

    def as_u32(self, key: str) -> Optional[int]:
        """MetadataValue::as_u32 on `metadata.get(key)` (src/gguf/metadata.rs:38-46)."""
        v = C.c_uint32()
        return int(v.value) if self._lib.llmrs_gguf_get_u32(self._h, key.encode(), C.byref(v)) == 0 else None

    def tensor_info(self, name: str) -> TensorInfo:
        info = _GgufTensor()
        self._ok(self._lib.llmrs_gguf_find_tensor(self._h, name.encode(), C.byref(info)))
        return self._info(info)

    def tensor_view(self, name: str) -> TensorView:
        """src/gguf/mod.rs:242-254: name, dtype, shape and the tensor's bytes (read from the file now)."""
        info = self.tensor_info(name)
        data = np.empty(info.nbytes, dtype=np.uint8)
        self._ok(self._lib.llmrs_gguf_read_tensor(self._h, name.encode(), data.ctypes.data_as(C.c_void_p), data.nbytes))
        try:
            dt = DType(info.dtype)
        except ValueError:
            dt = info.dtype                       # a dtype the backend does not hold: the id itself
        return TensorView(info.name, dt, list(info.shape), data)


def arch_name(gguf: GgufFile) -> str:
    """src/arch/mod.rs:33-37."""
    v = gguf.metadata.get("general.architecture")
    if not isinstance(v, str):
        raise KeyError("missing metadata key: general.architecture")
    return v


class Loader:
    """Tensor upload helper (src/arch/mod.rs:40-68)."""

    def __init__(self, gguf: GgufFile, backend: CudaBackend):
        self.gguf, self.backend = gguf, backend
        self.bytes = 0
        self.start = time.perf_counter()

    def opt(self, name: str, rows: Optional[Sequence[int]] = None) -> Optional[CudaBuffer]:
        """src/arch/mod.rs:52-57: None when the file has no such tensor.  `rows=(first, end)` uploads only
        that slice of the outer dimension (one rank's part of an N-sharded weight, see shard.row_range)."""
        raw = _Buf()
        be = self.backend
        if rows is None:
            rc = be._lib.llmrs_cuda_upload_gguf_tensor(be._ctx, self.gguf._h, name.encode(), C.byref(raw))
        else:
            rc = be._lib.llmrs_cuda_upload_gguf_tensor_rows(be._ctx, self.gguf._h, name.encode(), int(rows[0]),
                                                            int(rows[1]) - int(rows[0]), C.byref(raw))
        if rc == -9:
            return None
        be._check(rc)
        info = self.gguf.tensor_info(name)
        outer = int(info.shape[1]) if len(info.shape) > 1 else 1
        self.bytes += info.nbytes if rows is None else info.nbytes // outer * (int(rows[1]) - int(rows[0]))
        return CudaBuffer(be, raw)

    def req(self, name: str, rows: Optional[Sequence[int]] = None) -> CudaBuffer:
        """src/arch/mod.rs:59-61 (a panic there)."""
        buf = self.opt(name, rows)
        if buf is None:
            raise KeyError(f"missing tensor: {name}")
        return buf

    def print_stats(self) -> None:
        """src/arch/mod.rs:63-67."""
        elapsed = time.perf_counter() - self.start
        gb = self.bytes / (1024.0 ** 3)
        print(f"Uploaded model weights: {gb:.2f} GB in {elapsed:.3f}s ({gb / max(elapsed, 1e-9):.1f} GB/s)", file=sys.stderr)


__all__ = ["GgufFile", "GgufError", "TensorInfo", "Loader", "arch_name", "BackendError"]
