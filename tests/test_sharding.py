"""Host-side slot sharding (no collective on the data path): partition properties, and a world-size-2 gloo run in
which two CPU ranks step disjoint shards of the same batch through the oracle and together reproduce the
single-process result."""
import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from statequant_b200 import sharding


def test_partition_is_exact():
    g = torch.Generator().manual_seed(0)
    idx = torch.randint(-1, 50, (200,), generator=g).to(torch.int32)
    for world in (1, 2, 4, 8):
        seen = torch.zeros_like(idx)
        for r in range(world):
            loc = sharding.to_local(idx, r, world)
            assert int(loc.max()) < sharding.local_slots(50, r, world)
            own = loc > 0
            assert torch.equal(own.nonzero().flatten(), sharding.rows_of(idx, r, world))
            # local -> global is the inverse map
            assert torch.equal(((loc[own] - 1) * world + r + 1), idx[own])
            seen += own.to(torch.int32)
        assert torch.equal(seen, (idx > 0).to(torch.int32))          # every live row served exactly once


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path[:0] = [here, os.path.dirname(here)]
    from oracle import oracle
    import statequant_b200 as sq
    from statequant_b200.kernels import SlotLayout
    hv, hk, D, m, slots, rows = 4, 2, 64, 4, 9, 6
    lay = SlotLayout(sq.Quantizer(4, 'k', 32), hv, hk, D, D, m=m)
    g = torch.Generator().manual_seed(1)
    S = torch.randn(slots - 1, hv, D, D, generator=g) * 0.4
    # this rank's shard of the slot table
    n_loc = sharding.local_slots(slots, rank, world)
    blob = lay.alloc(n_loc, 'cpu')
    V = lay.views(blob)
    mine = [s for s in range(1, slots) if sharding.owner(s, world) == rank]
    lay.write(V, torch.tensor([(s - 1) // world + 1 for s in mine]), S[[s - 1 for s in mine]])
    outs = []
    for t in range(2 * m + 1):
        idx = (torch.randperm(slots - 1, generator=g)[:rows] + 1).to(torch.int32)
        idx[t % rows] = 0
        q, k = torch.randn(rows, hk, D, generator=g), torch.randn(rows, hk, D, generator=g)
        v = torch.randn(rows, hv, D, generator=g)
        gg, be = -torch.rand(rows, hv, generator=g) * 0.1, torch.rand(rows, hv, generator=g)
        out = torch.full((rows, hv, D), 7.)
        oracle.gdn_step(lay, V, sharding.to_local(idx, rank, world), q, k, v, out, D ** -0.5, g=gg, beta=be)
        dist.barrier()                                   # timing fence only: no data is exchanged on the path
        total = out.clone()
        dist.all_reduce(total)                           # test-side gather: rows of other ranks are zero
        outs.append(total)
    if rank == 0:
        ret.put(torch.stack(outs).numpy())               # plain bytes: no shared-memory handle that dies with the rank
    dist.destroy_process_group()


def test_two_ranks_reproduce_one(tmp_path):
    import random
    port = random.randint(20000, 40000)
    ctx = mp.get_context('spawn')
    ret = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    two = ret.get(timeout=120)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    ret1 = ctx.Queue()
    p = ctx.Process(target=_worker, args=(0, 1, port + 1, ret1))
    p.start()
    one = ret1.get(timeout=120)
    p.join(60)
    assert (two == one).all() and two.shape == one.shape
