"""Two-GPU test of the N-sharded decode matmul with the all-gather fused into the kernel.
Needs two B200s on one node; skipped on a single-GPU box."""
import os
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from llm_rs_b200 import CudaBackend, DType, TensorView, synth
    from llm_rs_b200.shard import FusedGather, row_range
    from oracle import oracle as O
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    ok, msg = True, ""
    try:
        stream = torch.cuda.Stream(device=rank)
        with torch.cuda.stream(stream):
            be = CudaBackend(rank, stream=stream.cuda_stream)
            # (the last two run the tensor-core kernel, whose epilogue does the same exchange)
            # (N = 1000: row tiles that end inside a rank's slice)
            for dt, K, N, M in ((O.Q6K, 4096, 4096, 1), (O.Q4K, 2048, 1024, 3), (O.Q4K, 1024, 1000, 2),
                                (O.Q4K, 1024, 2048, 16), (O.Q6K, 8192, 512, 70)):
                tol = 1e-4 if M <= 4 else 2e-3
                a, b = row_range(N, rank, world)
                w_full = synth.weight(dt, K, N, tid=dt)
                w_loc = synth.weight(dt, K, N, tid=dt, rows=(a, b))
                wbuf = be.upload_tensor(TensorView("w", DType(dt), [K, b - a], w_loc))
                fused = FusedGather(be, N, M)
                for call in range(3):                      # flags and buffers are reused across steps
                    x = synth.activations(M, K, tid=50 + call)
                    xbuf = be.upload_tensor(TensorView("x", DType.F32, [K] if M == 1 else [K, M], x))
                    out = fused(wbuf, xbuf)
                    be.sync()
                    got = out.cpu().numpy()
                    err = O.rel_l2(got, O.matmul(dt, w_full, K, N, x, acc="f64"))
                    if not err <= tol:
                        ok, msg = False, f"dtype {dt} M {M} call {call}: rel_l2 {err}"
                    dist.barrier()
                # the same call captured once in a CUDA graph and replayed: the kernel keeps its own count
                x = synth.activations(M, K, tid=60)
                xbuf = be.upload_tensor(TensorView("x", DType.F32, [K] if M == 1 else [K, M], x))
                fused(wbuf, xbuf)                          # warm call outside capture
                be.sync()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    fused(wbuf, xbuf)
                truth = O.matmul(dt, w_full, K, N, x, acc="f64")
                for _ in range(3):
                    fused.out.zero_()
                    g.replay()
                    stream.synchronize()
                    got = fused.out.cpu().numpy()
                    err = O.rel_l2(got, truth)
                    if not err <= tol:
                        ok, msg = False, f"dtype {dt} M {M} graph replay: rel_l2 {err}"
                dist.barrier()
            be.close()
    except Exception as e:  # noqa: BLE001
        ok, msg = False, repr(e)
    finally:
        q.put((rank, ok, msg))
        dist.destroy_process_group()


def test_fused_allgather_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + os.getpid() % 1000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=300) for _ in procs)
    for p in procs:
        p.join(60)
    assert all(r[1] for r in res), res
