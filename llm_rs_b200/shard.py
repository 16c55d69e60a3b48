"""Output-row (N) sharding of the matmul across the GPUs of one node.

Every output row of `out = matmul(weight, input)` reads only its own weight row
(shaders/ops.metal:249-289 in the reference), so rank g of G keeps rows
[g*N/G, (g+1)*N/G) of every weight, computes its slice of the output with the same kernels, and
the slices are all-gathered (the one exchange step of this path).  Activations are replicated.

The gather/reorder logic is plain torch.distributed and runs on CPU tensors with the gloo backend
too, which is how it is tested without GPUs; `local_matmul` is then any callable.
"""
from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist


def row_range(N: int, rank: int, world: int) -> tuple[int, int]:
    """Rows [a, b) of an N-row weight owned by `rank`.  N must divide evenly: equal slices are
    what lets the all-gather write straight into the final buffer."""
    if N % world:
        raise ValueError(f"out_features {N} is not divisible by {world} ranks")
    per = N // world
    return rank * per, (rank + 1) * per


class ShardedMatmul:
    """out[M, N] = x[M, K] . W[N, K]^T with W's rows split across the process group.

    local_matmul(out_slice, x) must fill out_slice ([M, N/G], contiguous) with this rank's rows.
    For M == 1 the slice is a view into the final [1, N] buffer and the all-gather is in place;
    for M > 1 slices are gathered as [G, M, N/G] and transposed into [M, N].
    """

    def __init__(self, N: int, local_matmul: Callable[[torch.Tensor, torch.Tensor], None],
                 group: dist.ProcessGroup | None = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.N = N
        self.rows = row_range(N, self.rank, self.world)
        self.local_matmul = local_matmul
        self._bufs: dict = {}

    def _buffers(self, M: int, like: torch.Tensor):
        key = (M, like.device, like.dtype)
        if key not in self._bufs:
            per = self.N // self.world
            full = torch.empty(M, self.N, device=like.device, dtype=like.dtype)
            if M == 1 or self.world == 1:
                a, b = self.rows
                local = full[:, a:b] if M == 1 else torch.empty(M, per, device=like.device, dtype=like.dtype)
                gathered = None
                if self.world == 1:
                    local = full
            else:
                local = torch.empty(M, per, device=like.device, dtype=like.dtype)
                gathered = torch.empty(self.world, M, per, device=like.device, dtype=like.dtype)
            self._bufs[key] = (full, local, gathered)
        return self._bufs[key]

    def __call__(self, x: torch.Tensor, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
        M = x.shape[0] if x.dim() == 2 else 1
        full, local, gathered = self._buffers(M, torch.empty(0, device=x.device, dtype=out_dtype))
        self.local_matmul(local, x)
        if self.world == 1:
            return full
        if M == 1:
            dist.all_gather_into_tensor(full.view(-1), local.reshape(-1), group=self.group)
            return full
        dist.all_gather_into_tensor(gathered.view(-1), local.reshape(-1), group=self.group)
        full.view(M, self.world, -1).copy_(gathered.permute(1, 0, 2))
        return full


class FusedGather:
    """Decode matmuls (M <= 4) of N-sharded weights whose all-gather runs inside the kernel.

    One object serves every weight with the same total N and token count.  It owns this rank's
    [M, N] output (ordinary device memory), its mailbox in symmetric memory
    (torch.distributed._symmetric_memory), so that every rank can hand the kernel device pointers
    to every other rank's mailbox, and a device word in which the kernel counts the calls.  The
    kernel (llmrs_cuda_matmul_allgather) posts each result to the other ranks as one 8-byte
    {value, call number} store over NVLink and copies what the others posted into `out` before
    it finishes: no NCCL call, no fence, no separate flag.  Nothing that changes per call is a
    launch argument, so a step captured in a CUDA graph can be replayed.  `out` is complete when
    the call's kernel has finished (stream order).
    """

    def __init__(self, backend, N: int, M: int, out_dtype=torch.float32, group: dist.ProcessGroup | None = None):
        import torch.distributed._symmetric_memory as symm
        from .backend import DType
        self.be = backend
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.N, self.M = N, M
        row_range(N, self.rank, self.world)                       # checks divisibility
        dev = torch.device("cuda", backend.device)
        self.out = torch.zeros(M, N, dtype=out_dtype, device=dev)
        self.out_buf = backend.wrap(self.out.data_ptr(), [N] if M == 1 else [N, M],
                                    DType.F32 if out_dtype == torch.float32 else DType.BF16, keepalive=self.out)
        self.mailbox = symm.empty((backend.allgather_mailbox_bytes(N, M) // 8,), dtype=torch.int64, device=dev)
        self.step_word = torch.zeros(1, dtype=torch.int32, device=dev)
        self.mailbox.zero_()
        torch.cuda.synchronize(dev)
        handle = symm.rendezvous(self.mailbox, self.group)
        self.peer_mailbox = [int(p) for p in handle.buffer_ptrs]
        dist.barrier(self.group)                                   # every mailbox is zeroed before any call

    def __call__(self, weight_shard, input_buf) -> torch.Tensor:
        self.be.matmul_allgather(self.out_buf, weight_shard, input_buf, self.rank, self.world, self.peer_mailbox,
                                 self.step_word.data_ptr())
        return self.out
