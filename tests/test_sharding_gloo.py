"""The N>1 path on CPU: two gloo ranks build their shards of one global workload the way bench.py does, parse them
with the host emulation of the pipeline, and agree on the whole-job figures (no collective on the data path: only
the barrier, the max over ranks of the time and the sum of the bytes)."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _rank_main(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, HERE)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import bench
    import emu_lib
    import oracle_lib
    from zluda_b200 import corpus
    n_modules, total_bytes = 6, 96 << 10          # per rank, as bench.py's --modules / --bytes
    mods = bench.make_workload(rank, world, n_modules, total_bytes)
    sizes = corpus.config1_sizes(1001, n_modules * world, total_bytes * world)
    mine = corpus.greedy_partition(sizes, world)[rank]
    # planned sizes steer the partition; a module's text ends at a statement boundary, so it is close to its plan
    assert len(mods) == len(mine)
    assert all(abs(len(m) - int(sizes[i])) <= 1024 for m, i in zip(mods, mine))
    # every rank parses only its own modules; results must equal the oracle's
    emu = emu_lib.load()
    oracle = oracle_lib.load()
    dumps, stats = emu.parse(mods, 0)
    for m, d in zip(mods, dumps):
        assert oracle.parse(m, 0)[1] == d
    # the shards are disjoint and cover the global list
    gathered = [None] * world
    dist.all_gather_object(gathered, mine)
    flat = sorted(i for part in gathered for i in part)
    assert flat == list(range(n_modules * world))
    # whole-job figures as bench.py forms them: sum of bytes, max of time
    t = torch.tensor([float(10 + rank), float(sum(len(m) for m in mods))], dtype=torch.float64)
    tmax, tsum = t.clone(), t.clone()
    dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
    assert float(tmax[0]) == 10 + world - 1
    assert abs(int(tsum[1]) - int(sum(int(s) for s in sizes))) <= 1024 * n_modules * world
    # byte balance of the greedy partition: no rank is more than one module above the mean
    loads = [sum(int(sizes[i]) for i in part) for part in gathered]
    assert max(loads) - min(loads) <= max(int(s) for s in sizes)
    dist.barrier()
    dist.destroy_process_group()
    open(os.path.join(out_dir, "rank%d.ok" % rank), "w").write("ok")


def test_two_ranks_shard_by_module(tmp_path):
    world = 2
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_rank_main, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all(os.path.exists(os.path.join(str(tmp_path), "rank%d.ok" % r)) for r in range(world))
