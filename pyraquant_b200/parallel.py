"""Token-row data parallelism for the INT8 Linear path.

Every output row depends only on its own input row (per-token scales are row-local,
deploy/int8_exec.py:83-101) and on the weights, so the path shards by contiguous row blocks over the
ranks of one node with replicated weights and no collective on the data path.  The only exchange is
the OPTIONAL all-gather of the 16-bit outputs (NCCL over NVLink on GPUs, gloo on CPU in the tests), either after
the layer (`all_gather_rows`) or hidden behind it chunk by chunk (`OverlappedRowGather` with NCCL / gloo,
`PeerPushGather` with the copy engines).  One process per GPU; rendezvous comes from the torchrun environment.
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


# ------------------------------------------------------------------------------------------------ overlapped gather
def cyclic_block_rows(M: int, world: int, chunks: int) -> int:
    """Rows per block when the M rows are dealt out block-cyclically: `chunks * world` blocks of equal height c (the
    last ones short or empty), block j = rows [j c, (j + 1) c), owned by rank j % world."""
    n = int(world) * int(chunks)
    return (int(M) + n - 1) // n


def cyclic_local_blocks(M: int, world: int, rank: int, chunks: int):
    """[(start, stop)] of this rank's `chunks` blocks, in the order it processes them (block i of the rank is global
    block i * world + rank); stops are clipped to M."""
    c = cyclic_block_rows(M, world, chunks)
    out = []
    for i in range(chunks):
        a = min(int(M), (i * world + rank) * c)
        out.append((a, min(int(M), a + c)))
    return out


class OverlappedRowGather:
    """All-gather of a row-parallel layer's outputs hidden behind its computation.

    With contiguous row blocks per rank the gather can only start when the whole layer is done.  Here the rows are dealt
    out block-cyclically instead (rows are independent, so any assignment is valid): the rank computes its block of chunk
    i, hands it to an asynchronous all-gather (NCCL runs it on its own stream), and computes its block of chunk i + 1
    meanwhile.  Chunk i of all ranks is the contiguous row range [i * world * c, (i + 1) * world * c) of the full output,
    so every gather writes straight into its place and the result is in natural row order.

    `forward(x_block) -> y_block` is the local layer; `run` takes either the full input (every rank slices its blocks as
    views) or, with `local=True`, this rank's rows already laid out block after block ([chunks * c, K])."""

    def __init__(self, M: int, N: int, dtype: torch.dtype, device, chunks: int = 4, group: Optional[dist.ProcessGroup] = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.M, self.N, self.chunks = int(M), int(N), int(chunks)
        self.c = cyclic_block_rows(M, self.world, chunks)
        self.full = torch.empty((self.chunks * self.world * self.c, N), dtype=dtype, device=device)

    def run(self, forward, x: torch.Tensor, local: bool = False, wait: bool = True) -> torch.Tensor:
        """Computes and gathers; with wait=False the last gathers may still be in flight on return (the next layer then
        computes behind them) and `finish()` must be called before the result is read."""
        c, W = self.c, self.world
        works = self._works = []
        for i, (a, b) in enumerate(cyclic_local_blocks(self.M, W, self.rank, self.chunks)):
            xb = x[i * c: i * c + (b - a)] if local else x[a:b]
            dst = self.full[i * W * c: (i + 1) * W * c]
            if b - a == c:
                y = forward(xb)
            else:                                   # short or empty block at the end of M: pad to the common height
                y = self.full.new_zeros((c, self.N))
                if b > a:
                    y[: b - a] = forward(xb)
            if W == 1:
                dst.copy_(y)
            else:
                works.append(dist.all_gather_into_tensor(dst, y.contiguous(), group=self.group, async_op=True))
        if wait:
            self.finish()
        return self.full[: self.M]

    def finish(self) -> None:
        for w in getattr(self, "_works", []):
            w.wait()
        self._works = []


class PeerPushGather(OverlappedRowGather):
    """The same overlapped gather with the GPUs' copy engines instead of NCCL kernels (CUDA, one node).

    Every rank's full-size output buffer lives in torch's symmetric memory (`torch.distributed._symmetric_memory`: the
    same allocation on every rank, each mapped into every peer's address space); a finished chunk is then WRITTEN into
    every peer's buffer by plain device-to-device copies on side streams.  Copies between peer GPUs run on the DMA engines over NVLink, need no SM
    and therefore overlap with the persistent GEMM, which NCCL's copy kernels cannot (they wait for SMs the GEMM holds
    until it ends).  No kernel of this library ever reads a peer's memory.
    Ordering: `run` ends with a stream-ordered all-reduce of one element after this rank's copies, so when it completes
    on a rank, every peer's writes into that rank's buffer have completed; it starts with one as well, so that no peer
    overwrites a buffer its owner may still be reading from the previous call."""

    def __init__(self, M: int, N: int, dtype: torch.dtype, device, chunks: int = 4, group: Optional[dist.ProcessGroup] = None,
                 copy_streams: int = 1, direct: bool = True):
        super().__init__(M, N, dtype, device, chunks, group)
        self.device = torch.device(device)
        self.direct = direct           # the layer writes its rows of this rank's buffer itself (no local copy)
        self.peers = [self.full] * self.world
        if self.world > 1:
            import torch.distributed._symmetric_memory as symm_mem
            shape = tuple(self.full.shape)
            self.full = symm_mem.empty(shape, dtype=dtype, device=self.device)
            self._handle = symm_mem.rendezvous(self.full, group=group if group is not None else dist.group.WORLD)
            self.peers = [self.full if r == self.rank else self._handle.get_buffer(r, shape, dtype) for r in range(self.world)]
        # One copy stream by default: a single device-to-device copy already runs at the link rate (742 GB/s out of a GPU
        # with the seven copies of a block one after the other; every GPU then also receives from one sender at a time),
        # while concurrent copies on several streams share it badly (716 GB/s with one stream per peer at 355 MB per copy,
        # 390-580 GB/s when the copies are 44-180 MB).
        n_streams = max(1, copy_streams)
        self.streams = [torch.cuda.Stream(self.device) for _ in range(n_streams)]
        self._token = torch.zeros(1, device=self.device)

    def run(self, forward, x: torch.Tensor, local: bool = False, wait: bool = True) -> torch.Tensor:
        c, W, r = self.c, self.world, self.rank
        cur = torch.cuda.current_stream(self.device)
        if W > 1:
            dist.all_reduce(self._token, group=self.group)           # peers are done reading what the last call delivered
        for st in self.streams:
            st.wait_stream(cur)
        for i, (a, b) in enumerate(cyclic_local_blocks(self.M, W, r, self.chunks)):
            if b <= a:
                continue
            xb = x[i * c: i * c + (b - a)] if local else x[a:b]
            row = (i * W + r) * c
            mine = self.full[row: row + (b - a)]
            if self.direct and hasattr(forward, "forward_into"):
                forward.forward_into(xb, mine)
                srcrows = mine
            else:
                srcrows = forward(xb)
                mine.copy_(srcrows)
            done = torch.cuda.Event(); done.record(cur)
            for k in range(1, W):                                    # every peer is one hop away on a switch: round robin
                st = self.streams[k % len(self.streams)]
                st.wait_event(done)
                with torch.cuda.stream(st):
                    self.peers[(r + k) % W][row: row + (b - a)].copy_(srcrows, non_blocking=True)
            if srcrows is not mine:
                for st in self.streams:
                    srcrows.record_stream(st)
        if wait:
            self.finish()
        return self.full[: self.M]

    def finish(self) -> None:
        cur = torch.cuda.current_stream(self.device)
        for st in self.streams:
            cur.wait_stream(st)
        if self.world > 1:
            dist.all_reduce(self._token, group=self.group)           # every rank's copies are behind its all-reduce


class PeerStoreGather(PeerPushGather):
    """Row-sharded layer whose GEMM epilogue performs the all-gather (CUDA, one node).

    The full-size output buffers live in symmetric memory as in `PeerPushGather`; here the GEMM kernel itself stores
    every output tile to this GPU's buffer and to each peer's (`Int8Linear.forward_into` -> `pq_int8_gemm_bcast`, plain
    vector stores to peer memory from the epilogue warps), so tiles cross NVLink while the tensor cores work on the next
    ones and no copy or collective kernel follows the layer.  The kernel waits on nobody: ordering between ranks is the
    stream-ordered one-element all-reduce before (peers have finished reading the previous result) and after (every
    rank's kernel, and with it its stores, is complete) the layer.  Rows are dealt out as one contiguous block per rank
    and chunk (`chunks` = 1 unless a later layer wants to start on early rows)."""

    def __init__(self, M: int, N: int, dtype: torch.dtype, device, chunks: int = 1, group: Optional[dist.ProcessGroup] = None):
        super().__init__(M, N, dtype, device, chunks, group, copy_streams=1)

    def run(self, linear, x: torch.Tensor, local: bool = False, wait: bool = True) -> torch.Tensor:
        c, W, r = self.c, self.world, self.rank
        if W > 1:
            dist.all_reduce(self._token, group=self.group)
        for i, (a, b) in enumerate(cyclic_local_blocks(self.M, W, r, self.chunks)):
            if b <= a:
                continue
            xb = x[i * c: i * c + (b - a)] if local else x[a:b]
            row = (i * W + r) * c
            more = [self.peers[(r + k) % W][row: row + (b - a)] for k in range(1, W)]
            linear.forward_into(xb, self.full[row: row + (b - a)], more)
        if wait:
            self.finish()
        return self.full[: self.M]

    def finish(self) -> None:
        if self.world > 1:
            dist.all_reduce(self._token, group=self.group)


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
