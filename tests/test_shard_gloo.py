"""The N-sharding host logic on CPU: two gloo ranks, a float64 stand-in for the local matmul."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, K, N, Ms, q):
    sys.path.insert(0, ROOT)
    from llm_rs_b200.shard import ShardedMatmul, row_range
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(1)
        W = torch.randn(N, K, generator=g, dtype=torch.float64)
        a, b = row_range(N, rank, world)
        Wl = W[a:b]

        def local_matmul(out, x):
            out.copy_((x.reshape(-1, K).double() @ Wl.T).to(out.dtype))

        sm = ShardedMatmul(N, local_matmul)
        ok = True
        for M in Ms:
            x = torch.randn(M, K, generator=g, dtype=torch.float64)
            got = sm(x if M > 1 else x[0], out_dtype=torch.float64)
            ok = ok and got.shape == (M, N) and torch.allclose(got, x @ W.T, rtol=1e-12, atol=1e-12)
            got2 = sm(x if M > 1 else x[0], out_dtype=torch.float64)      # buffers are reused
            ok = ok and torch.allclose(got2, x @ W.T, rtol=1e-12, atol=1e-12)
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_row_range():
    from llm_rs_b200.shard import row_range
    for N in (1024, 4096, 14336, 128256):
        for G in (1, 2, 4, 8):
            rs = [row_range(N, r, G) for r in range(G)]
            assert rs[0][0] == 0 and rs[-1][1] == N
            assert all(rs[i][1] == rs[i + 1][0] for i in range(G - 1))
            assert len({b - a for a, b in rs}) == 1
    import pytest
    with pytest.raises(ValueError):
        row_range(10, 0, 4)


def test_sharded_matmul_two_gloo_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, 64, 48, (1, 3), q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(60)
    assert res == [(0, True), (1, True)]
