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
