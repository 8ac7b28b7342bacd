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
