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


def gather_pointers(out_ptrs, flag_ptrs, rank: int, M: int, N: int, elt: int):
    """Device addresses the fused all-gather kernel needs, from the per-rank base addresses of the
    symmetric [2, M, N] output and the [world] uint32 flag array: (peer_out[2][world],
    peer_flags[world], my_flags).  Rank r publishes its step in slot r of every rank's flag array."""
    half = M * N * elt
    peer_out = [[int(p) + b * half for p in out_ptrs] for b in (0, 1)]
    peer_flags = [int(p) + 4 * rank for p in flag_ptrs]
    return peer_out, peer_flags, int(flag_ptrs[rank])


class FusedGatherMatmul:
    """Decode matmul (M <= 4) of an N-sharded weight whose all-gather runs inside the kernel.

    Output buffers and flag arrays live in symmetric memory (torch.distributed._symmetric_memory),
    so every rank can hand the kernel device pointers to every other rank's buffer.  The kernel
    (llmrs_cuda_matmul_allgather) stores its slice into all buffers over NVLink with plain stores,
    publishes a step number in the peers' flag arrays and returns when all slices have arrived in
    its own buffer.  No NCCL call per step.  The call returns this rank's [M, N] tensor, complete
    once the call's kernel has finished (stream order).

    Two output buffers alternate by step.  A peer can start step s+1 as soon as its own step s is
    complete, and would then store into the buffer this rank may still be reading; with two
    buffers the one returned by step s is not written again before step s+2, which no peer can
    reach until this rank's step s+1 kernel has run -- and that kernel is ordered, on this rank's
    stream, after whatever consumed step s.  Consumers on other streams must order themselves
    against the next-but-one call.
    """

    def __init__(self, backend, weight_shard, N: int, M: int, out_dtype=torch.float32,
                 group: dist.ProcessGroup | None = None):
        import torch.distributed._symmetric_memory as symm
        from .backend import DType
        if M > 4:
            raise ValueError("the fused all-gather serves the decode kernel only (M <= 4)")
        self.be, self.w = backend, weight_shard
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.N, self.M = N, M
        row_range(N, self.rank, self.world)                       # checks divisibility
        dev = torch.device("cuda", backend.device)
        self.out = symm.empty((2, M, N), dtype=out_dtype, device=dev)
        self.flags = symm.empty((self.world,), dtype=torch.int32, device=dev)
        self.out.zero_()
        self.flags.zero_()
        torch.cuda.synchronize(dev)
        oh = symm.rendezvous(self.out, self.group)
        fh = symm.rendezvous(self.flags, self.group)
        self.peer_out, self.peer_flags, self.my_flags = gather_pointers(
            oh.buffer_ptrs, fh.buffer_ptrs, self.rank, M, N, self.out.element_size())
        self.out_dtype = DType.F32 if out_dtype == torch.float32 else DType.BF16
        self.step = 0
        dist.barrier(self.group)                                   # all flag arrays are zeroed before any step

    def __call__(self, input_buf) -> torch.Tensor:
        self.step += 1
        b = self.step & 1
        self.be.matmul_allgather(self.w, input_buf, self.out_dtype, self.N, self.rank, self.world,
                                 self.peer_out[b], self.peer_flags, self.my_flags, self.step)
        return self.out[b]
