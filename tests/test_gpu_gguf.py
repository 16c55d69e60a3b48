"""GGUF file -> device (`Loader`, llmrs_cuda_upload_gguf_tensor): what arrives in device memory is what
upload_tensor stores for the same bytes, for the gguf-py fixture and for tensors of several staging pieces."""
import json
import os

import numpy as np
import pytest

from llm_rs_b200 import DType, TensorView, synth
from oracle import gguf as OG
from oracle import oracle as O

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
TINY = os.path.join(HERE, "golden", "tiny.gguf")


@pytest.fixture(scope="module")
def G(cuda_lib):
    from llm_rs_b200 import gguf
    return gguf


def test_loader_uploads_the_fixture(backend, G):
    buf = open(TINY, "rb").read()
    p = OG.parse(buf)
    with G.GgufFile.open(TINY) as g:
        ld = G.Loader(g, backend)
        total = 0
        for t in p["tensors"]:
            dev = ld.req(t["name"])
            raw = np.frombuffer(OG.tensor_bytes(buf, p, t["name"]), dtype=np.uint8)
            total += raw.nbytes
            K = t["shape"][0]
            N = t["shape"][1] if len(t["shape"]) > 1 else 1
            assert (dev.dtype, dev.dim0, dev.dim1) == (DType(t["dtype"]), K, N if len(t["shape"]) > 1 else 0)
            if t["dtype"] in (O.Q4K, O.Q6K):
                got = backend.dequantize(dev)
                want = O.dequant(t["dtype"], raw, K, N)
                assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), t["name"]
            else:
                backend.sync()
                assert np.array_equal(backend.read_to_vec_f32(dev), raw.view(np.float32)), t["name"]
        assert ld.bytes == total
        assert ld.opt("blk.7.attn_q.weight") is None
        with pytest.raises(KeyError, match="missing tensor: blk.7.attn_q.weight"):
            ld.req("blk.7.attn_q.weight")
        ld.print_stats()
        # the uploaded weights work as any other: one decode matmul on the output projection
        w = ld.req("output.weight")
        x = synth.activations(1, 256, tid=5)
        xb = backend.upload_tensor(TensorView("x", DType.F32, [256], x))
        out = backend.alloc([130], DType.F32)
        backend.matmul(out, w, xb)
        backend.sync()
        raw = np.frombuffer(OG.tensor_bytes(buf, p, "output.weight"), dtype=np.uint8)
        assert O.rel_l2(backend.read_to_vec_f32(out).reshape(1, 130), O.matmul(O.Q6K, raw, 256, 130, x, acc="f64")) <= 1e-4


@pytest.mark.parametrize("dt,K,N", [(O.Q6K, 4096, 30001), (O.Q4K, 4096, 32000), (O.Q6K, 768, 129)])
def test_streamed_upload_equals_upload_tensor(backend, G, tmp_path, dt, K, N):
    """Tensors of 101 MB (four staging pieces, the ring reused), 74 MB (three) and a ragged small one, behind
    an unrelated tensor so that the file offset is not piece-aligned: same device bytes as upload_tensor."""
    w = synth.weight(dt, K, N, tid=77)
    pad = bytes(range(200)) + bytes(56)
    path = str(tmp_path / "big.gguf")
    with open(path, "wb") as f:
        f.write(OG.build([("general.architecture", 8, "llama", None)],
                         [("pad", [256], 24, pad), ("w", [K, N], dt, np.ascontiguousarray(w).tobytes()), ("tail", [4], 0, bytes(16))]))
    with G.GgufFile(path) as g:
        ld = G.Loader(g, backend)
        a = ld.req("w")
        b = backend.upload_tensor(TensorView("w", DType(dt), [K, N], w))
        assert (a.dtype, a.dim0, a.dim1, a.layout, a.nbytes) == (b.dtype, b.dim0, b.dim1, b.layout, b.nbytes)
        da, db = backend.dequantize(a), backend.dequantize(b)
        assert np.array_equal(da.view(np.uint32), db.view(np.uint32))
        rows = np.r_[0:3, N // 2:N // 2 + 3, N - 3:N]
        want = O.dequant(dt, np.ascontiguousarray(w).reshape(N, -1)[rows].reshape(-1), K, len(rows))
        assert np.array_equal(da[rows].view(np.uint32), want.view(np.uint32))
        assert ld.bytes == w.nbytes


@pytest.mark.parametrize("dt", [O.Q4K, O.Q6K])
def test_row_slices_for_sharded_weights(backend, G, tmp_path, dt):
    """Each rank of an N-sharded matmul uploads its rows only (shard.row_range): the slices dequantise to the
    rows of the whole tensor, in every split, and bad ranges are refused before anything is read."""
    from llm_rs_b200 import BackendError
    from llm_rs_b200.shard import row_range
    K, N = 768, 1008
    w = synth.weight(dt, K, N, tid=88)
    path = str(tmp_path / "shard.gguf")
    with open(path, "wb") as f:
        f.write(OG.build([], [("w", [K, N], dt, np.ascontiguousarray(w).tobytes()), ("v", [K], 0, bytes(4 * K))]))
    want = O.dequant(dt, w, K, N)
    with G.GgufFile(path) as g:
        ld = G.Loader(g, backend)
        for world in (2, 3, 8):
            for rank in range(world):
                a, b = row_range(N, rank, world)
                part = ld.req("w", rows=(a, b))
                assert (part.dim0, part.dim1) == (K, b - a)
                assert np.array_equal(backend.dequantize(part).view(np.uint32), want[a:b].view(np.uint32)), (world, rank)
        for bad in ((0, 0), (5, 4), (1007, 1009), (1008, 1009)):
            with pytest.raises(BackendError) as e:
                ld.req("w", rows=bad)
            assert e.value.code == -2
        assert ld.req("v", rows=(0, 1)).dim1 == 0          # a 1-D tensor is one row: only the whole of it
        with pytest.raises(BackendError):
            ld.req("v", rows=(0, 2))
        assert ld.opt("nope", rows=(0, 1)) is None
