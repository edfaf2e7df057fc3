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
    # the Llama-shaped cache the benchmark splits over the ranks: whole (layer, head-range) blocks per rank
    sys.path.insert(0, ROOT)
    import bench
    cfg = bench.CACHES["kv"]
    blocks = bench.rank_layers(cfg, rank, world)
    llama_packed = 0
    for layer, hrange in blocks:
        codec = tq.TurboQuantV3(128, key_bits=cfg["key_bits"], value_bits=cfg["value_bits"],
                                residual_window=cfg["window"], layer_idx=layer, n_layers=cfg["layers"],
                                protected_layers=cfg["protected"])
        assert (codec.key_bits, codec.value_bits) == bench.layer_bits(cfg, layer)
        llama_packed += codec.memory_bytes(cfg["batch"], len(hrange), cfg["seq"])["compressed_bytes"]
    gathered = [None] * world
    dist.all_gather_object(gathered, (units, packed, [(l, list(h)) for l, h in blocks], llama_packed))
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
    all_units = [u for units, *_ in gathered for u in units]
    assert sorted(all_units) == [(l, h) for l in range(36) for h in range(2)]
    assert len(set(all_units)) == 72
    assert sum(g[1] for g in gathered) == 58982400                   # the whole configs[1] cache
    llama_units = [(l, h) for g in gathered for l, hs in g[2] for h in hs]
    assert sorted(llama_units) == [(l, h) for l in range(32) for h in range(8)] and len(set(llama_units)) == 256
    assert sum(g[3] for g in gathered) == 14305722368                # the whole configs[2] cache, packed + window
    assert tmax == 2.0


def test_rank_blocks_cover_the_cache_for_every_world_size():
    import sys
    sys.path.insert(0, ROOT)
    import bench
    for name in ("kv", "qwen"):
        cfg = bench.CACHES[name]
        for world in (1, 2, 3, 4, 8):
            seen = []
            for r in range(world):
                for layer, heads in bench.rank_layers(cfg, r, world):
                    assert heads.step == 1 and 0 <= heads.start < heads.stop <= cfg["kv_heads"]
                    seen += [(layer, h) for h in heads]
            assert sorted(seen) == [(l, h) for l in range(cfg["layers"]) for h in range(cfg["kv_heads"])]


def test_cost_balanced_shards_cover_the_units_and_equalise_the_cost():
    import sys
    sys.path.insert(0, os.path.join(ROOT, "turboquant-pytorch_b200"))
    from turboquant import batched
    layers, heads = 32, 8
    costs = [batched.tile_cost(8, 8) if l < 4 or l >= 28 else batched.tile_cost(6, 4) for l in range(layers)]
    assert batched.tile_cost(8, 8) > batched.tile_cost(6, 4) > batched.tile_cost(4, 2)
    for world in (1, 2, 3, 4, 8, 16):
        shards = [batched.shard_units(layers, heads, r, world, layer_costs=costs) for r in range(world)]
        flat = [u for sh in shards for u in sh]
        assert flat == [(l, h) for l in range(layers) for h in range(heads)]          # contiguous, complete, in order
        load = [sum(costs[l] for l, _h in sh) for sh in shards]
        assert max(load) - min(load) <= 1.5 * max(costs)                               # within a unit and a half
        plain = [len(batched.shard_units(layers, heads, r, world)) for r in range(world)]
        assert sum(plain) == layers * heads and max(plain) - min(plain) <= 1
    # the protected layers make the end shards shorter
    eight = [len(batched.shard_units(layers, heads, r, 8, layer_costs=costs)) for r in range(8)]
    assert eight[0] < 32 < eight[3] and eight[0] == eight[-1]
