"""Token-row data parallelism for the INT8 Linear path.

Every output row depends only on its own input row (per-token scales are row-local,
deploy/int8_exec.py:83-101) and on the weights, so the path shards by contiguous row blocks over the
ranks of one node with replicated weights and no collective on the data path.  The only exchange is
the OPTIONAL all-gather of the 16-bit outputs (NCCL over NVLink on GPUs, gloo on CPU in the tests).
One process per GPU; rendezvous comes from the torchrun environment.
"""
from __future__ import annotations

import os
from typing import Optional, Tuple

import torch
import torch.distributed as dist


def rows_per_rank(M: int, world: int) -> int:
    return (int(M) + int(world) - 1) // int(world)


def shard_rows(M: int, world: int, rank: int) -> Tuple[int, int]:
    """Half-open row range [start, stop) of `rank`: blocks of ceil(M / world) rows, the last ones short or empty."""
    per = rows_per_rank(M, world)
    start = min(int(M), int(rank) * per)
    return start, min(int(M), start + per)


def init_from_env(device_type: str = "cuda") -> Tuple[int, int, int]:
    """(rank, local_rank, world) from RANK / LOCAL_RANK / WORLD_SIZE; initialises the default process
    group (nccl for cuda, gloo otherwise) when WORLD_SIZE > 1."""
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if device_type == "cuda":
        torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        kw = {}
        if device_type == "cuda":
            kw["device_id"] = torch.device("cuda", local)
        dist.init_process_group(backend="nccl" if device_type == "cuda" else "gloo", rank=rank, world_size=world, **kw)
    return rank, local, world


def all_gather_rows(y_local: torch.Tensor, M: int, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Concatenates the ranks' row blocks into the full [M, N] output.  Row-major blocks make the gather
    a pure concatenation; short last blocks are padded to the common block height and trimmed after."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return y_local
    world = dist.get_world_size(group)
    per = rows_per_rank(M, world)
    N = y_local.shape[1]
    if y_local.shape[0] != per:
        pad = y_local.new_zeros((per, N))
        pad[: y_local.shape[0]] = y_local
        y_local = pad
    full = y_local.new_empty((world * per, N))
    dist.all_gather_into_tensor(full, y_local.contiguous(), group=group)
    return full[:M]


class RowShardedLinear(torch.nn.Module):
    """Runs `linear` on this rank's row block of a full-size input; `gather=True` returns the full output."""

    def __init__(self, linear: torch.nn.Module, gather: bool = False, group: Optional[dist.ProcessGroup] = None):
        super().__init__()
        self.linear = linear
        self.gather = gather
        self.group = group

    def forward(self, x_full: torch.Tensor) -> torch.Tensor:
        M = x_full.shape[0]
        world = dist.get_world_size(self.group) if dist.is_initialized() else 1
        rank = dist.get_rank(self.group) if dist.is_initialized() else 0
        a, b = shard_rows(M, world, rank)
        y = self.linear(x_full[a:b])
        return all_gather_rows(y, M, self.group) if self.gather else y
