"""Row sharding and the optional output all-gather on two gloo ranks (CPU): the compute inside each
rank is the CPU oracle, so only the host-side partitioning and the collective are under test."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle
from pyraquant_b200 import parallel


def test_shard_rows_cover_and_disjoint():
    for M in (0, 1, 7, 8, 66048, 66049):
        for world in (1, 2, 4, 8):
            spans = [parallel.shard_rows(M, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == M
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            assert all(b - a <= parallel.rows_per_rank(M, world) for a, b in spans)
    assert parallel.shard_rows(66048, 8, 7) == (57792, 66048)


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _worker(rank, world, port, M, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    torch.set_num_threads(1)
    r, _l, w = parallel.init_from_env(device_type="cpu")
    assert (r, w) == (rank, world)
    L = oracle.make_layer(3, M, 128, 64)
    wq, ws = oracle.quant_weight(L["w"])

    class Lin(torch.nn.Module):
        def forward(self, x):
            return oracle.int8_linear_forward(x, wq, ws, L["bias"], L["lr_A"], L["lr_B"])

    # chunked, overlapped gather over block-cyclic rows: same result, natural row order
    for chunks in (1, 3, 4):
        og = parallel.OverlappedRowGather(M, 64, L["x"].dtype, "cpu", chunks=chunks)
        got = og.run(Lin(), L["x"])
        assert torch.equal(got, Lin()(L["x"])), chunks
        blocks = parallel.cyclic_local_blocks(M, world, rank, chunks)
        xl = torch.cat([L["x"][a:b] for a, b in blocks] + [L["x"][:0]])
        c = parallel.cyclic_block_rows(M, world, chunks)
        xpad = torch.zeros(chunks * c, xl.shape[1], dtype=xl.dtype)
        off = 0
        for i, (a, b) in enumerate(blocks):
            xpad[i * c: i * c + (b - a)] = L["x"][a:b]
        assert torch.equal(og.run(Lin(), xpad, local=True), Lin()(L["x"])), chunks
    full = parallel.RowShardedLinear(Lin(), gather=True)(L["x"])
    local = parallel.RowShardedLinear(Lin(), gather=False)(L["x"])
    want = Lin()(L["x"])
    a, b = parallel.shard_rows(M, world, rank)
    ok = torch.equal(full, want) and torch.equal(local, want[a:b])
    t = torch.tensor([1.0 if ok else 0.0])
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    if rank == 0:
        ret.put(float(t.item()))
    dist.barrier()
    dist.destroy_process_group()


def test_cyclic_blocks_cover_rows_once():
    for M in (0, 1, 7, 66, 67, 66048, 66049):
        for world in (1, 2, 4, 8):
            for chunks in (1, 3, 4):
                c = parallel.cyclic_block_rows(M, world, chunks)
                seen = []
                for r in range(world):
                    blocks = parallel.cyclic_local_blocks(M, world, r, chunks)
                    assert len(blocks) == chunks and all(0 <= b - a <= c for a, b in blocks)
                    seen += [(a, b) for a, b in blocks if b > a]
                seen.sort()
                assert (not seen and M == 0) or (seen[0][0] == 0 and seen[-1][1] == M)
                assert all(seen[i][1] == seen[i + 1][0] for i in range(len(seen) - 1))
    assert parallel.cyclic_block_rows(66048, 8, 4) == 2064


def test_two_rank_gloo_sharded_forward_and_gather():
    ctx = mp.get_context("spawn")
    for M in (66, 67):                       # even and ragged split
        ret = ctx.SimpleQueue()
        port = _free_port()
        procs = [ctx.Process(target=_worker, args=(r, 2, port, M, ret)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0
        assert ret.get() == 1.0
