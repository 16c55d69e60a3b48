"""Behaviour around the kernels, on a B200 through the C ABI: a bounded wait that runs out, CUDA graphs
that outlive a growth of the context's scratch, the residual that is the output itself, the per-kernel
timing table.  Nothing here faults or hangs the GPU: the one failure is a wait with a short limit on a
mailbox word that nothing writes, after which the kernel returns and the host reads an error code."""
import os

import numpy as np
import pytest

from llm_rs_b200 import BackendError, CudaBackend, DType, TensorView, synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _ctx_with_env(env, **kw):
    old = {k: os.environ.get(k) for k in env}
    os.environ.update(env)
    try:
        return CudaBackend(0, **kw)
    finally:
        for k, v in old.items():
            if v is None:
                del os.environ[k]
            else:
                os.environ[k] = v


def _w(be, dt, K, N, tid):
    w = synth.weight(dt, K, N, tid=tid)
    return w, be.upload_tensor(TensorView("w", DType(dt), [K, N], w))


def _x(be, x, M, K):
    return be.upload_tensor(TensorView("x", DType.F32, [K] if M == 1 else [K, M], np.ascontiguousarray(x, np.float32)))


@pytest.mark.parametrize("M", [1, 16])
def test_abandoned_peer_wait_is_reported_and_the_context_survives(cuda_lib, M):
    """The fused all-gather waits, with a limit, for the words its peers post.  Here rank 0 of a
    pretended two-rank group runs alone and the "peer's" mailbox is a second local buffer nobody writes:
    the wait runs out (LLMRS_WAIT_POLLS=1024: about 30 us), the kernel finishes, sync reports
    LLMRS_ERR_KERNEL, and the next matmul on the same context is correct.  M=1: the decode kernel's
    exchange; M=16: the tensor-core kernel's."""
    import torch
    be = _ctx_with_env({"LLMRS_WAIT_POLLS": "1024", "LLMRS_GEMV_MAX_M": "4"})
    try:
        dt, K, n_local, world = O.Q4K, 1024, 64, 2
        w, wbuf = _w(be, dt, K, n_local, tid=901)
        x = synth.activations(M, K, tid=902)
        xbuf = _x(be, x, M, K)
        nbytes = be.allgather_mailbox_bytes(n_local * world, M)
        boxes = [torch.zeros(nbytes // 8, dtype=torch.int64, device="cuda:0") for _ in range(world)]
        step = torch.zeros(1, dtype=torch.int32, device="cuda:0")
        out = be.alloc([n_local * world] if M == 1 else [n_local * world, M], DType.F32)
        torch.cuda.synchronize()
        be.matmul_allgather(out, wbuf, xbuf, 0, world, [b.data_ptr() for b in boxes], step.data_ptr())
        with pytest.raises(BackendError) as e:
            be.sync()
        assert e.value.code == -6 and "bounded wait" in str(e.value)
        # rank 0's own rows are there all the same; the peer's half was never delivered
        got = be.read_to_vec_f32(out).reshape(M, n_local * world)
        truth = O.matmul(dt, w, K, n_local, x, acc="f64")
        assert O.rel_l2(got[:, :n_local], truth) <= 1e-4
        # what rank 0 posted for its peer sits in the peer's mailbox, tagged with call number 1
        words = boxes[1].cpu().numpy().view(np.uint32).reshape(-1, 2)
        posted = words[words[:, 1] == 1]
        assert posted.shape[0] == M * n_local
        assert np.array_equal(np.sort(posted[:, 0].view(np.float32)), np.sort(got[:, :n_local].reshape(-1)))
        # the context is still good
        out2 = be.alloc([n_local] if M == 1 else [n_local, M], DType.F32)
        be.matmul(out2, wbuf, xbuf)
        be.sync()
        assert O.rel_l2(be.read_to_vec_f32(out2).reshape(M, n_local), truth) <= 1e-4
    finally:
        be.close()


def test_graph_captured_before_the_scratch_grew_still_replays(cuda_lib):
    """A CUDA graph holds the addresses of the context's scratch at capture time.  A later, larger call
    makes the scratch grow; the outgrown buffer is kept, so the old graph still computes the right thing."""
    import torch
    stream = torch.cuda.Stream(device=0)
    with torch.cuda.stream(stream):
        be = _ctx_with_env({"LLMRS_GEMV_MAX_M": "4"}, stream=stream.cuda_stream)
        try:
            dt, K, N = O.Q6K, 2048, 384
            w, wbuf = _w(be, dt, K, N, tid=911)
            x16 = synth.activations(16, K, tid=912)
            xb16 = _x(be, x16, 16, K)
            out16 = be.alloc([N, 16], DType.F32)
            be.matmul(out16, wbuf, xb16)                 # warm call: the scratch reaches its 16-token size
            be.sync()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                be.matmul(out16, wbuf, xb16)
            # a much larger call: new scratch
            x512 = synth.activations(512, K, tid=913)
            out512 = be.alloc([N, 512], DType.F32)
            be.matmul(out512, wbuf, _x(be, x512, 512, K))
            be.sync()
            assert O.rel_l2(be.read_to_vec_f32(out512).reshape(512, N), O.matmul(dt, w, K, N, x512, acc="f64")) <= 2e-3
            truth = O.matmul(dt, w, K, N, x16, acc="f64")
            for _ in range(2):
                be.write(out16, np.zeros(16 * N, np.float32))
                be.sync()
                g.replay()
                stream.synchronize()
                assert O.rel_l2(be.read_to_vec_f32(out16).reshape(16, N), truth) <= 1e-4
        finally:
            be.close()


@pytest.mark.parametrize("dt", [O.Q4K, O.Q6K])
@pytest.mark.parametrize("M,bf16", [(1, False), (9, False), (9, True), (40, False), (128, False), (128, True)])
def test_matmul_add_with_the_residual_as_output(backend, dt, M, bf16):
    """x = x + matmul(w, h), residual and output the same buffer, at token counts that reach each kernel."""
    K, N = 1024, 320
    w, wbuf = _w(backend, dt, K, N, tid=921)
    h = synth.activations(M, K, tid=922 + M)
    res = synth.activations(M, N, tid=923 + M) * np.float32(30.0)
    if bf16:
        res = O.bf16_bits_to_f32(synth.bf16_bits(res)).reshape(M, N)
        xb = backend.upload_tensor(TensorView("x", DType.BF16, [N] if M == 1 else [N, M], synth.bf16_bits(res)))
    else:
        xb = _x(backend, res, M, N)
    backend.matmul_add(xb, wbuf, _x(backend, h, M, K), xb)
    backend.sync()
    got = backend.read_to_vec_f32(xb).reshape(M, N)
    truth = O.matmul(dt, w, K, N, h, acc="f64").astype(np.float64) + res
    assert O.rel_l2(got, truth) <= (1e-4 if M <= 64 else 2e-3) + (2.0 ** -8 if bf16 else 0.0)


def test_perf_table(cuda_lib):
    """LLMRS_PERF=1: each sync yields one line per kind of operation, with calls, time and rates."""
    be = _ctx_with_env({"LLMRS_PERF": "1", "LLMRS_PEAK_HBM_GBS": "6464.9", "LLMRS_PEAK_TFLOPS": "1658.7"})
    try:
        K, N = 4096, 4096
        _, wbuf = _w(be, O.Q4K, K, N, tid=931)
        xb = _x(be, synth.activations(1, K, tid=932), 1, K)
        out = be.alloc([N], DType.F32)
        for _ in range(3):
            be.matmul(out, wbuf, xb)
        be.add(out, out, out)
        xb70 = _x(be, synth.activations(70, K, tid=933), 70, K)
        out70 = be.alloc([N, 70], DType.F32)
        be.matmul(out70, wbuf, xb70)
        assert be.perf_table() == ""
        be.sync()
        table = be.perf_table()
        rows = {ln[:34].strip(): ln[34:].split() for ln in table.splitlines()[1:-1]}
        assert set(rows) == {"matmul q4_k decode kernel", "add", "matmul q4_k tensor cores"}, table
        assert rows["matmul q4_k decode kernel"][0] == "3" and rows["add"][0] == "1"
        us, gbs = float(rows["matmul q4_k decode kernel"][1]), float(rows["matmul q4_k decode kernel"][3])
        assert 3.0 < us < 300.0 and abs(gbs - 3 * 9469952 / us * 1e-3) <= 0.02 * gbs, table
        assert float(rows["matmul q4_k tensor cores"][5]) > 1.0       # TFLOP/s
        assert "6465 GB/s" in table and "1659 TFLOP/s" in table
        be.sync()                                                     # nothing new: the table stays
        assert be.perf_table() == table
    finally:
        be.close()
