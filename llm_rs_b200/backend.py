"""Host-side mirror of llm-rs's `Backend` trait for the Q4_K / Q6_K matmul path.

Same names, argument meaning and error behaviour as the reference interface
(src/backend/mod.rs:15-89) so that code written against `MetalBackend` reads the
same here: `upload_tensor`, `alloc`, `matmul`, `read_to_vec_f32`, `sync`,
`gpu_secs_total`, `reset_gpu_secs`.  Every call goes through the C ABI of
include/llmrs_cuda.h (ctypes); there is no CPU path, and importing the library
on a machine without the built .so, or creating a backend without a B200,
raises.  Every method of the trait is present; dtypes a method does not handle are
refused with an error, as the reference does with `unimplemented!` for what a backend lacks
(src/backend/metal/mod.rs:511).
"""
from __future__ import annotations

import ctypes as C
import enum
import os
from dataclasses import dataclass
from typing import Sequence

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libllmrs_cuda.so")


class DType(enum.IntEnum):
    """GGUF dtype ids (src/tensor/mod.rs:3-33); only the ones this path handles."""
    F32 = 0
    F16 = 1
    Q4_0 = 2
    Q8_0 = 8
    Q4K = 12
    Q6K = 14
    I32 = 26
    BF16 = 30

    def block_elems(self) -> int:                     # src/tensor/mod.rs:37-50
        return 256 if self in (DType.Q4K, DType.Q6K) else 32 if self in (DType.Q4_0, DType.Q8_0) else 1

    def block_size_bytes(self) -> int:                # src/tensor/mod.rs:52-86
        return {DType.F32: 4, DType.I32: 4, DType.BF16: 2, DType.F16: 2, DType.Q4_0: 18, DType.Q8_0: 34,
                DType.Q4K: 144, DType.Q6K: 210}[self]

    def storage_size(self, n_elements: int) -> int:   # src/tensor/mod.rs:89-93
        be = self.block_elems()
        if n_elements % be:
            raise ValueError(f"element count {n_elements} not divisible by block size {be}")
        return n_elements // be * self.block_size_bytes()


@dataclass
class TensorView:
    """Borrowed tensor bytes as they sit in a GGUF file (src/tensor/mod.rs:142-154)."""
    name: str
    dtype: DType
    shape: Sequence[int]
    data: np.ndarray            # uint8 (or any dtype; its bytes are used)

    def n_elements(self) -> int:
        n = 1
        for d in self.shape:
            n *= int(d)
        return n


class BackendError(RuntimeError):
    """A C-ABI call returned a non-zero status (the Rust binding would panic here)."""

    def __init__(self, code: int, message: str):
        super().__init__(f"llmrs_cuda error {code}: {message}")
        self.code = code


class _GgufTensor(C.Structure):
    """llmrs_gguf_tensor: one entry of a GGUF file's tensor table."""
    _fields_ = [("name", C.c_char_p), ("dtype", C.c_uint32), ("n_dims", C.c_uint32), ("shape", C.c_uint64 * 4),
                ("offset", C.c_uint64), ("nbytes", C.c_uint64)]


class _Buf(C.Structure):
    _fields_ = [("dptr", C.c_void_p), ("nbytes", C.c_uint64), ("dtype", C.c_uint32), ("dim0", C.c_uint32),
                ("dim1", C.c_uint32), ("layout", C.c_uint32), ("owned", C.c_uint32), ("device", C.c_uint32)]


# Every symbol include/llmrs_cuda.h declares: (restype, argtypes).
_VP, _U64P = C.c_void_p, C.POINTER(C.c_uint64)
_BUFP = C.POINTER(_Buf)
ABI = {
    "llmrs_cuda_create": (C.c_int, [C.c_int, _VP, C.POINTER(_VP)]),
    "llmrs_cuda_destroy": (C.c_int, [_VP]),
    "llmrs_cuda_upload_tensor": (C.c_int, [_VP, C.c_uint32, _U64P, C.c_int, _VP, C.c_size_t, _BUFP]),
    "llmrs_cuda_alloc": (C.c_int, [_VP, C.c_uint32, _U64P, C.c_int, _BUFP]),
    "llmrs_cuda_wrap": (C.c_int, [_VP, _VP, C.c_uint32, _U64P, C.c_int, _BUFP]),
    "llmrs_cuda_free": (C.c_int, [_VP, _BUFP]),
    "llmrs_cuda_matmul": (C.c_int, [_VP, _BUFP, _BUFP, _BUFP]),
    "llmrs_cuda_matmul_static_scratch": (C.c_int, [_VP, _BUFP, _BUFP, _BUFP]),
    "llmrs_cuda_silu": (C.c_int, [_VP, _BUFP]),
    "llmrs_cuda_mul": (C.c_int, [_VP, _BUFP, _BUFP, _BUFP]),
    "llmrs_cuda_add": (C.c_int, [_VP, _BUFP, _BUFP, _BUFP]),
    "llmrs_cuda_rms_norm": (C.c_int, [_VP, _BUFP, _BUFP, _BUFP, C.c_float]),
    "llmrs_cuda_argmax": (C.c_int, [_VP, _BUFP, C.POINTER(C.c_uint32)]),
    "llmrs_cuda_rms_norm_heads": (C.c_int, [_VP, _BUFP, _BUFP, C.c_float]),
    "llmrs_cuda_rope": (C.c_int, [_VP, _BUFP, _BUFP, _BUFP, C.c_uint32, C.c_float, C.c_uint32]),
    "llmrs_cuda_rope_scatter_kv": (C.c_int, [_VP, _BUFP, _BUFP, _BUFP, _BUFP, C.c_uint32, C.c_float, C.c_uint32,
                                             _BUFP, _BUFP, _BUFP]),
    "llmrs_cuda_scatter_kv": (C.c_int, [_VP, _BUFP, _BUFP, _BUFP, C.c_uint32, C.c_uint32]),
    "llmrs_cuda_gather": (C.c_int, [_VP, _BUFP, _BUFP, _BUFP, C.c_uint32]),
    "llmrs_cuda_attention": (C.c_int, [_VP] + [_BUFP] * 7 + [C.c_uint32] * 5),
    "llmrs_cuda_rms_norm_matmul": (C.c_int, [_VP, _BUFP, _BUFP, _BUFP, _BUFP, C.c_float]),
    "llmrs_cuda_rms_norm_matmul_gate_up": (C.c_int, [_VP, _BUFP, _BUFP, _BUFP, _BUFP, _BUFP, C.c_float]),
    "llmrs_cuda_rms_norm_matmul_qkv": (C.c_int, [_VP] + [_BUFP] * 8 + [C.c_float]),
    "llmrs_cuda_matmul_add": (C.c_int, [_VP, _BUFP, _BUFP, _BUFP, _BUFP]),
    "llmrs_cuda_matmul_gate_up": (C.c_int, [_VP, _BUFP, _BUFP, _BUFP, _BUFP]),
    "llmrs_cuda_embed": (C.c_int, [_VP, _BUFP, _BUFP, C.POINTER(C.c_uint32), C.c_uint32]),
    "llmrs_cuda_matmul_allgather": (C.c_int, [_VP, _BUFP, _BUFP, _BUFP, C.c_uint32, C.c_uint32, C.POINTER(_VP), _VP]),
    "llmrs_cuda_allgather_mailbox_bytes": (C.c_size_t, [C.c_uint32, C.c_uint32]),
    "llmrs_cuda_matmul_allgather_max_tokens": (C.c_int, [C.c_uint32, C.c_uint32]),
    "llmrs_cuda_dequantize": (C.c_int, [_VP, _BUFP, _VP]),
    "llmrs_cuda_write": (C.c_int, [_VP, _BUFP, _VP, C.c_size_t]),
    "llmrs_cuda_read_f32": (C.c_int, [_VP, _BUFP, C.POINTER(C.c_float), C.c_size_t]),
    "llmrs_cuda_sync": (C.c_int, [_VP]),
    "llmrs_cuda_gpu_secs_total": (C.c_int, [_VP, C.POINTER(C.c_double)]),
    "llmrs_cuda_reset_gpu_secs": (C.c_int, [_VP]),
    "llmrs_cuda_launch_count": (C.c_int, [_VP, _U64P]),
    "llmrs_cuda_perf_table": (C.c_size_t, [_VP, C.c_char_p, C.c_size_t]),
    "llmrs_cuda_last_error": (C.c_char_p, [_VP]),
    "llmrs_cuda_upload_gguf_tensor": (C.c_int, [_VP, _VP, C.c_char_p, _BUFP]),
    "llmrs_cuda_upload_gguf_tensor_rows": (C.c_int, [_VP, _VP, C.c_char_p, C.c_uint64, C.c_uint64, _BUFP]),
    "llmrs_gguf_open": (C.c_int, [C.c_char_p, C.POINTER(_VP)]),
    "llmrs_gguf_close": (None, [_VP]),
    "llmrs_gguf_last_error": (C.c_char_p, []),
    "llmrs_gguf_version": (C.c_uint32, [_VP]),
    "llmrs_gguf_file_size": (C.c_uint64, [_VP]),
    "llmrs_gguf_data_offset": (C.c_uint64, [_VP]),
    "llmrs_gguf_tensor_count": (C.c_uint64, [_VP]),
    "llmrs_gguf_metadata_count": (C.c_uint64, [_VP]),
    "llmrs_gguf_tensor_at": (C.c_int, [_VP, C.c_uint64, C.POINTER(_GgufTensor)]),
    "llmrs_gguf_find_tensor": (C.c_int, [_VP, C.c_char_p, C.POINTER(_GgufTensor)]),
    "llmrs_gguf_read_tensor": (C.c_int, [_VP, C.c_char_p, _VP, C.c_size_t]),
    "llmrs_gguf_metadata_at": (C.c_int, [_VP, C.c_uint64, C.POINTER(C.c_char_p), C.POINTER(C.c_uint32),
                                         C.POINTER(C.c_uint32), _U64P]),
    "llmrs_gguf_get_u32": (C.c_int, [_VP, C.c_char_p, C.POINTER(C.c_uint32)]),
    "llmrs_gguf_get_u64": (C.c_int, [_VP, C.c_char_p, _U64P]),
    "llmrs_gguf_get_f64": (C.c_int, [_VP, C.c_char_p, C.POINTER(C.c_double)]),
    "llmrs_gguf_get_str": (C.c_int, [_VP, C.c_char_p, C.POINTER(_VP), _U64P]),
    "llmrs_gguf_get_array": (C.c_int, [_VP, C.c_char_p, C.POINTER(C.c_uint32), _U64P, C.POINTER(_VP)]),
    "llmrs_gguf_get_array_str": (C.c_int, [_VP, C.c_char_p, C.c_uint64, C.POINTER(_VP), _U64P]),
}

_lib = None


def load_library() -> C.CDLL:
    """dlopen the in-tree CUDA library and bind every declared symbol.  Fails loudly when
    the library has not been built (`python -m llm_rs_b200.build`): there is no fallback."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m llm_rs_b200.build`")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in ABI.items():
            fn = getattr(lib, name)          # AttributeError if the symbol is not exported
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


class CudaBuffer:
    """Device buffer + dtype + dims: the counterpart of MetalBuffer (metal/mod.rs:13-34)."""

    def __init__(self, backend: "CudaBackend", raw: _Buf, keepalive=None):
        self._backend = backend
        self._raw = raw
        self._keepalive = keepalive       # e.g. the torch tensor whose memory is wrapped

    dtype = property(lambda self: DType(self._raw.dtype))
    dim0 = property(lambda self: int(self._raw.dim0))
    dim1 = property(lambda self: int(self._raw.dim1))
    layout = property(lambda self: int(self._raw.layout))
    nbytes = property(lambda self: int(self._raw.nbytes))
    data_ptr = property(lambda self: int(self._raw.dptr or 0))

    def n_elements(self) -> int:
        return self.dim0 * max(self.dim1, 1)

    def seq_len(self) -> int:
        return max(self.dim1, 1)

    def free(self) -> None:
        if self._raw.dptr and self._backend._ctx:
            self._backend._check(self._backend._lib.llmrs_cuda_free(self._backend._ctx, C.byref(self._raw)))
        self._keepalive = None

    def __del__(self):                    # Drop
        try:
            self.free()
        except Exception:
            pass


class CudaBackend:
    """The B200 backend.  One instance = one device + one stream; not thread-safe."""

    Buffer = CudaBuffer

    def __init__(self, device: int = 0, stream: int | None = None):
        self._lib = load_library()
        self._ctx = None
        ctx = C.c_void_p()
        rc = self._lib.llmrs_cuda_create(device, C.c_void_p(stream) if stream else None, C.byref(ctx))
        if rc != 0:
            raise BackendError(rc, (self._lib.llmrs_cuda_last_error(None) or b"").decode())
        self._ctx = ctx
        self.device = device

    # -- plumbing --
    def _check(self, rc: int) -> None:
        if rc != 0:
            raise BackendError(rc, (self._lib.llmrs_cuda_last_error(self._ctx) or b"").decode())

    @staticmethod
    def _shape(shape: Sequence[int]):
        arr = (C.c_uint64 * len(shape))(*[int(d) for d in shape])
        return arr, len(shape)

    def close(self) -> None:
        if self._ctx:
            self._lib.llmrs_cuda_destroy(self._ctx)
            self._ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- Backend trait, matmul path --
    def upload_tensor(self, tv: TensorView) -> CudaBuffer:
        """src/backend/mod.rs:18."""
        data = np.ascontiguousarray(tv.data)
        shp, nd = self._shape(tv.shape)
        raw = _Buf()
        self._check(self._lib.llmrs_cuda_upload_tensor(self._ctx, int(tv.dtype), shp, nd,
                                                       data.ctypes.data_as(C.c_void_p), data.nbytes, C.byref(raw)))
        return CudaBuffer(self, raw)

    def alloc(self, shape: Sequence[int], dtype: DType) -> CudaBuffer:
        """src/backend/mod.rs:19."""
        shp, nd = self._shape(shape)
        raw = _Buf()
        self._check(self._lib.llmrs_cuda_alloc(self._ctx, int(dtype), shp, nd, C.byref(raw)))
        return CudaBuffer(self, raw)

    def matmul(self, out: CudaBuffer, weight: CudaBuffer, input: CudaBuffer) -> None:
        """`out = matmul(weight, input)`; src/backend/mod.rs:29-34."""
        self._check(self._lib.llmrs_cuda_matmul(self._ctx, C.byref(out._raw), C.byref(weight._raw),
                                                C.byref(input._raw)))

    def read_to_vec_f32(self, buf: CudaBuffer) -> np.ndarray:
        """src/backend/mod.rs:80."""
        out = np.empty(buf.n_elements(), dtype=np.float32)
        self._check(self._lib.llmrs_cuda_read_f32(self._ctx, C.byref(buf._raw),
                                                  out.ctypes.data_as(C.POINTER(C.c_float)), out.size))
        return out

    def gpu_secs_total(self) -> float:
        """src/backend/mod.rs:84."""
        v = C.c_double()
        self._check(self._lib.llmrs_cuda_gpu_secs_total(self._ctx, C.byref(v)))
        return float(v.value)

    def reset_gpu_secs(self) -> None:
        """src/backend/mod.rs:85."""
        self._check(self._lib.llmrs_cuda_reset_gpu_secs(self._ctx))

    def sync(self) -> None:
        """src/backend/mod.rs:88."""
        self._check(self._lib.llmrs_cuda_sync(self._ctx))

    # -- additions of this backend (no trait counterpart) --
    def wrap(self, data_ptr: int, shape: Sequence[int], dtype: DType, keepalive=None) -> CudaBuffer:
        """Describe caller-owned device memory (e.g. `tensor.data_ptr()`) as a buffer."""
        shp, nd = self._shape(shape)
        raw = _Buf()
        self._check(self._lib.llmrs_cuda_wrap(self._ctx, C.c_void_p(data_ptr), int(dtype), shp, nd, C.byref(raw)))
        return CudaBuffer(self, raw, keepalive)

    def write(self, dst: CudaBuffer, host: np.ndarray) -> None:
        """Enqueue a host->device copy of `host`'s bytes into `dst` (activations of a step)."""
        self._check(self._lib.llmrs_cuda_write(self._ctx, C.byref(dst._raw), host.ctypes.data_as(C.c_void_p),
                                               host.nbytes))

    def dequantize(self, weight: CudaBuffer) -> np.ndarray:
        """Weight -> float32 [N, K] on the device, copied back (testing aid)."""
        K, N = weight.dim0, max(weight.dim1, 1)
        tmp = self.alloc([K, N], DType.F32)
        self._check(self._lib.llmrs_cuda_dequantize(self._ctx, C.byref(weight._raw), C.c_void_p(tmp.data_ptr)))
        out = self.read_to_vec_f32(tmp).reshape(N, K)
        tmp.free()
        return out

    def matmul_static_scratch(self, out: CudaBuffer, weight: CudaBuffer, input: CudaBuffer) -> None:
        """`matmul` through the tensor-core kernel with its scratch in the 8 MiB device array built
        into the library: for hosts that must not allocate device memory while running.  Raises
        BackendError (-2) when 2*K*M + 4*M bytes (twice the first term up to 64 tokens) do not fit; calls that may overlap on the GPU race
        on the shared array."""
        self._check(self._lib.llmrs_cuda_matmul_static_scratch(self._ctx, C.byref(out._raw), C.byref(weight._raw),
                                                               C.byref(input._raw)))

    def silu(self, x: CudaBuffer) -> None:
        """Backend::silu (src/backend/mod.rs:76): in place."""
        self._check(self._lib.llmrs_cuda_silu(self._ctx, C.byref(x._raw)))

    def mul(self, out: CudaBuffer, a: CudaBuffer, b: CudaBuffer) -> None:
        self._check(self._lib.llmrs_cuda_mul(self._ctx, C.byref(out._raw), C.byref(a._raw), C.byref(b._raw)))

    def add(self, out: CudaBuffer, a: CudaBuffer, b: CudaBuffer) -> None:
        self._check(self._lib.llmrs_cuda_add(self._ctx, C.byref(out._raw), C.byref(a._raw), C.byref(b._raw)))

    def rms_norm(self, out: CudaBuffer, input: CudaBuffer, weight: CudaBuffer, eps: float) -> None:
        """Backend::rms_norm (src/backend/mod.rs:36-38); `weight` is an F32 buffer of dim values."""
        self._check(self._lib.llmrs_cuda_rms_norm(self._ctx, C.byref(out._raw), C.byref(input._raw),
                                                  C.byref(weight._raw), float(eps)))

    def argmax(self, logits: CudaBuffer) -> int:
        """Backend::argmax (src/backend/mod.rs:21-23): computed on the device, four bytes come back."""
        v = C.c_uint32()
        self._check(self._lib.llmrs_cuda_argmax(self._ctx, C.byref(logits._raw), C.byref(v)))
        return int(v.value)

    def rms_norm_heads(self, x: CudaBuffer, weight: CudaBuffer, eps: float) -> None:
        """Backend::rms_norm_heads (src/backend/mod.rs:40-43): in place, per chunk of weight.dim0 values."""
        self._check(self._lib.llmrs_cuda_rms_norm_heads(self._ctx, C.byref(x._raw), C.byref(weight._raw), float(eps)))

    def upload_u32(self, data: Sequence[int]) -> CudaBuffer:
        """Backend::upload_u32 (src/backend/mod.rs:74-75): a small index array as an I32 buffer."""
        arr = np.ascontiguousarray(data, dtype=np.uint32).reshape(-1)
        return self.upload_tensor(TensorView("u32", DType.I32, [max(arr.size, 1)], arr if arr.size else np.zeros(1, np.uint32)))

    def rope(self, q: CudaBuffer, k: CudaBuffer, positions: CudaBuffer, head_dim: int, rope_theta: float,
             split_half: bool = False) -> None:
        """Backend::rope (src/backend/mod.rs:45-47); split_half=False is RopeLayout::Interleaved."""
        self._check(self._lib.llmrs_cuda_rope(self._ctx, C.byref(q._raw), C.byref(k._raw), C.byref(positions._raw),
                                              head_dim, float(rope_theta), 1 if split_half else 0))

    def rope_scatter_kv(self, q: CudaBuffer, k: CudaBuffer, v: CudaBuffer, positions: CudaBuffer, head_dim: int,
                        rope_theta: float, k_pool: CudaBuffer, v_pool: CudaBuffer, slot_mapping: CudaBuffer,
                        split_half: bool = False) -> None:
        """rope(q, k) + scatter_kv(k_pool, k) + scatter_kv(v_pool, v) (src/arch/llama.rs:156-158) as one call."""
        self._check(self._lib.llmrs_cuda_rope_scatter_kv(self._ctx, C.byref(q._raw), C.byref(k._raw), C.byref(v._raw),
                                                         C.byref(positions._raw), head_dim, float(rope_theta),
                                                         1 if split_half else 0, C.byref(k_pool._raw),
                                                         C.byref(v_pool._raw), C.byref(slot_mapping._raw)))

    def scatter_kv(self, pool: CudaBuffer, src: CudaBuffer, slot_mapping: CudaBuffer, kv_dim: int, num_tokens: int) -> None:
        self._check(self._lib.llmrs_cuda_scatter_kv(self._ctx, C.byref(pool._raw), C.byref(src._raw),
                                                    C.byref(slot_mapping._raw), kv_dim, num_tokens))

    def gather(self, out: CudaBuffer, src: CudaBuffer, indices: CudaBuffer, num_indices: int) -> None:
        self._check(self._lib.llmrs_cuda_gather(self._ctx, C.byref(out._raw), C.byref(src._raw), C.byref(indices._raw),
                                                num_indices))

    def attention(self, out: CudaBuffer, q: CudaBuffer, k_pool: CudaBuffer, v_pool: CudaBuffer, block_table: CudaBuffer,
                  query_starts: CudaBuffer, seq_lens: CudaBuffer, n_heads: int, n_kv_heads: int, head_dim: int,
                  block_size: int, max_blocks_per_seq: int) -> None:
        """Backend::attention (src/backend/mod.rs:49-66): paged varlen causal grouped-query attention."""
        self._check(self._lib.llmrs_cuda_attention(self._ctx, C.byref(out._raw), C.byref(q._raw), C.byref(k_pool._raw),
                                                   C.byref(v_pool._raw), C.byref(block_table._raw),
                                                   C.byref(query_starts._raw), C.byref(seq_lens._raw), n_heads,
                                                   n_kv_heads, head_dim, block_size, max_blocks_per_seq))

    def rms_norm_matmul(self, out: CudaBuffer, weight: CudaBuffer, input: CudaBuffer, norm_weight: CudaBuffer,
                        eps: float) -> None:
        """out = matmul(weight, rms_norm(input, norm_weight, eps)): rms_norm + matmul (src/arch/llama.rs:152-155)."""
        self._check(self._lib.llmrs_cuda_rms_norm_matmul(self._ctx, C.byref(out._raw), C.byref(weight._raw),
                                                         C.byref(input._raw), C.byref(norm_weight._raw), float(eps)))

    def rms_norm_matmul_gate_up(self, out: CudaBuffer, w_gate: CudaBuffer, w_up: CudaBuffer, input: CudaBuffer,
                                norm_weight: CudaBuffer, eps: float) -> None:
        """rms_norm + matmul, matmul, silu, mul (src/arch/llama.rs:164-168) as one call."""
        self._check(self._lib.llmrs_cuda_rms_norm_matmul_gate_up(self._ctx, C.byref(out._raw), C.byref(w_gate._raw),
                                                                 C.byref(w_up._raw), C.byref(input._raw),
                                                                 C.byref(norm_weight._raw), float(eps)))

    def rms_norm_matmul_qkv(self, out_q: CudaBuffer, out_k: CudaBuffer, out_v: CudaBuffer, wq: CudaBuffer, wk: CudaBuffer,
                            wv: CudaBuffer, input: CudaBuffer, norm_weight: CudaBuffer, eps: float) -> None:
        """rms_norm + the q, k and v projections (src/arch/llama.rs:152-155) as one call."""
        self._check(self._lib.llmrs_cuda_rms_norm_matmul_qkv(
            self._ctx, C.byref(out_q._raw), C.byref(out_k._raw), C.byref(out_v._raw), C.byref(wq._raw), C.byref(wk._raw),
            C.byref(wv._raw), C.byref(input._raw), C.byref(norm_weight._raw), float(eps)))

    def matmul_add(self, out: CudaBuffer, weight: CudaBuffer, input: CudaBuffer, residual: CudaBuffer) -> None:
        """out = residual + matmul(weight, input): matmul followed by add (src/arch/llama.rs:162-163) as one call."""
        self._check(self._lib.llmrs_cuda_matmul_add(self._ctx, C.byref(out._raw), C.byref(weight._raw),
                                                    C.byref(input._raw), C.byref(residual._raw)))

    def matmul_gate_up(self, out: CudaBuffer, w_gate: CudaBuffer, w_up: CudaBuffer, input: CudaBuffer) -> None:
        """out = silu(matmul(w_gate, input)) * matmul(w_up, input): the calls matmul, matmul, silu, mul
        of the reference's feed-forward block (src/arch/llama.rs:165-168) as one."""
        self._check(self._lib.llmrs_cuda_matmul_gate_up(self._ctx, C.byref(out._raw), C.byref(w_gate._raw),
                                                        C.byref(w_up._raw), C.byref(input._raw)))

    def embed(self, out: CudaBuffer, table: CudaBuffer, tokens: Sequence[int]) -> None:
        """Backend::embed (src/backend/mod.rs:25-27): out[:, i] = dequantised row tokens[i] of the
        Q4_K / Q6_K table; `out` is [dim] for one token, else [dim, len(tokens)]."""
        ids = np.ascontiguousarray(tokens, dtype=np.uint32).reshape(-1)
        self._check(self._lib.llmrs_cuda_embed(self._ctx, C.byref(out._raw), C.byref(table._raw),
                                               ids.ctypes.data_as(C.POINTER(C.c_uint32)), ids.size))

    def matmul_allgather(self, out: CudaBuffer, weight_shard: CudaBuffer, input: CudaBuffer, rank: int, world: int,
                         peer_mailbox: Sequence[int], step_word: int) -> None:
        """Decode matmul of this rank's weight rows with the all-gather fused into the kernel: every
        result goes into `out` ([N_local * world] or [N_local * world, M], local memory) and, as one
        8-byte {value, call number} store, into the other ranks' mailboxes (`peer_mailbox`, device
        pointers this GPU can store through); the kernel finishes when it has copied what the
        others posted into `out`.  step_word = address of a local uint32 the kernel counts calls in."""
        pm = (C.c_void_p * world)(*[C.c_void_p(int(p)) for p in peer_mailbox])
        self._check(self._lib.llmrs_cuda_matmul_allgather(self._ctx, C.byref(out._raw), C.byref(weight_shard._raw),
                                                          C.byref(input._raw), rank, world, pm,
                                                          C.c_void_p(int(step_word))))

    def allgather_mailbox_bytes(self, n_total: int, tokens: int) -> int:
        return int(self._lib.llmrs_cuda_allgather_mailbox_bytes(n_total, tokens))

    def allgather_max_tokens(self, weight_dtype: DType, in_features: int) -> int:
        """Largest token count matmul_allgather accepts for this weight type and in_features."""
        return int(self._lib.llmrs_cuda_matmul_allgather_max_tokens(int(weight_dtype), in_features))

    def launch_count(self) -> int:
        v = C.c_uint64()
        self._check(self._lib.llmrs_cuda_launch_count(self._ctx, C.byref(v)))
        return int(v.value)


    def perf_table(self) -> str:
        """The per-kernel table of the last sync (LLMRS_PERF=1 at creation; the reference's LLM_PERF
        output, src/backend/metal/mod.rs:323-400).  Empty when nothing was recorded."""
        n = int(self._lib.llmrs_cuda_perf_table(self._ctx, None, 0))
        if n == 0:
            return ""
        buf = C.create_string_buffer(n + 1)
        self._lib.llmrs_cuda_perf_table(self._ctx, buf, n + 1)
        return buf.value.decode()
