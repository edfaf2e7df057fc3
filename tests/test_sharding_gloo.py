"""Multi-rank host logic on CPU (gloo, world_size 2): units are partitioned with no overlap,
every rank's accounting adds up to the whole cache, and the max-over-ranks reduction that
bench.py uses for its timing works.  No data-path collective exists to test: shards are
independent by construction."""

import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    import sys
    sys.path.insert(0, os.path.join(ROOT, "turboquant-pytorch_b200"))
    from turboquant import batched
    import turboquant as tq
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    layers, heads, seq = 36, 2, 8192
    units = batched.shard_units(layers, heads, rank, world)
    # per-rank accounting of its shard (pure arithmetic, same code path as memory_bytes)
    packed = 0
    for layer, _head in units:
        codec = tq.TurboQuantV3(128, key_bits=4, value_bits=2, residual_window=0, layer_idx=layer, n_layers=layers,
                                protected_layers=0)
        packed += codec.memory_bytes(1, 1, seq)["compressed_bytes"]
    gathered = [None] * world
    dist.all_gather_object(gathered, (units, packed))
    t = torch.tensor([1.0 + rank], dtype=torch.float64)        # stand-in for a per-rank elapsed time
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        out.put((gathered, float(t.item())))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_partition_the_cache_and_reduce_timings():
    world = 2
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    gathered, tmax = out.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    all_units = [u for units, _ in gathered for u in units]
    assert sorted(all_units) == [(l, h) for l in range(36) for h in range(2)]
    assert len(set(all_units)) == 72
    assert sum(packed for _, packed in gathered) == 58982400         # the whole configs[1] cache
    assert tmax == 2.0
