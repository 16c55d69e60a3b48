"""The C-ABI library loads and exports exactly what include/llmrs_cuda.h declares.
No compute calls: this runs without a GPU."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "llmrs_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(llmrs_(?:cuda|gguf)_\w+)\s*\(", text)))


def test_header_and_binding_agree():
    from llm_rs_b200.backend import ABI
    assert declared_symbols() == sorted(ABI), "ctypes table and header must list the same entry points"


def test_library_exports_every_declared_symbol(cuda_lib):
    for name in declared_symbols():
        assert hasattr(cuda_lib, name), f"{name} is declared in the header but not exported"


def test_buffer_struct_matches_header():
    from llm_rs_b200.backend import _Buf
    # void* + u64 + 6 * u32, no padding surprises
    assert C.sizeof(_Buf) == 8 + 8 + 6 * 4
    assert [f[0] for f in _Buf._fields_] == ["dptr", "nbytes", "dtype", "dim0", "dim1", "layout", "owned", "device"]


def test_no_fallback_without_device(cuda_lib):
    """Without a usable B200 the backend refuses to come up; it never computes on the CPU."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present; the no-device path cannot be shown here")
    from llm_rs_b200 import BackendError, CudaBackend
    with pytest.raises(BackendError) as e:
        CudaBackend(0)
    assert e.value.code == -5


def test_product_does_not_import_oracle():
    """The package and the CUDA sources never reference the test oracle."""
    pkg = os.path.join(ROOT, "llm_rs_b200")
    for dirpath, _dirs, files in os.walk(pkg):
        if os.path.basename(dirpath) == "build":
            continue
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src.lower(), f"{f} mentions the oracle"


def test_integration_rust_binding_is_consistent():
    """The Rust text of INTEGRATION.md cannot be compiled here, so it is held to what can be checked by
    reading: every llmrs_* function a Rust block calls is declared in an `extern "C"` block of the page
    (in a code block or in the prose that says what to add), and every declared name exists in the header."""
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    blocks = re.findall(r"```rust\n(.*?)```", text, flags=re.S)
    assert blocks, "no Rust blocks found"
    declared = set(re.findall(r"\bfn\s+(llmrs_(?:cuda|gguf)_\w+)\s*\(", text))
    called = set()
    for b in blocks:
        for name in re.findall(r"\b(llmrs_(?:cuda|gguf)_\w+)\s*\(", b):
            called.add(name)
    header = set(declared_symbols())
    assert called <= declared, f"called in the Rust text but never declared extern: {sorted(called - declared)}"
    assert declared <= header, f"declared extern in INTEGRATION.md but not in the header: {sorted(declared - header)}"
    # the Rust struct derives only Clone and Copy: nothing may ask it for a Default
    assert "LlmrsBuf::default()" not in text
    # the build step compiles every kernel file of the package
    csrc = os.path.join(ROOT, "llm_rs_b200", "csrc")
    assert "read_dir(\"cuda/csrc\")" in text and all(f.endswith((".cu", ".cuh", ".h")) for f in os.listdir(csrc))
