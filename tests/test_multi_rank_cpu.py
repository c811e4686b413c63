"""World-size-2 gloo test of the multi-device protocol for the sharded sum (config 2a with dim 0
split over ranks): each rank reduces its shard to unrounded f32 partials, the partials are
all-reduced, and the sum is rounded to f16 once, so any number of ranks gives the 1-rank answer.
The per-rank partial comes from the CPU oracle here (no GPU in this container); on the GPU box the
same protocol runs with b200_reduce_sum_to_f32 / NCCL / b200_cast_from_f32 (bench.py --gpus N)."""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "tests"))


def _worker(rank, world, port, q):
    import oracle_lib as O
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(99)  # every rank builds the same global tensor, then takes its shard
        x = rng.standard_normal((8, 64, 256), dtype=np.float32).astype(np.float16)
        per = x.shape[0] // world
        shard = x[rank * per:(rank + 1) * per]
        part = torch.from_numpy(O.reduce_sum_f64(shard, 1, per * 64, 256).astype(np.float32))
        dist.all_reduce(part)  # the only data-path collective of the hot path
        total = part.numpy().astype(np.float16)
        # rows of the max reduction are sharded without any exchange: gather them only to check
        m = torch.from_numpy(O.reduce("max", shard, per * 64, 256, 1).view(np.uint16).astype(np.int32))
        gathered = [torch.empty_like(m) for _ in range(world)]
        dist.all_gather(gathered, m)
        if rank == 0:
            want = O.reduce("sum", x, 1, 8 * 64, 256)
            wmax = O.reduce("max", x, 8 * 64, 256, 1)
            ok_sum = np.allclose(total.astype(np.float64), want.astype(np.float64), rtol=2e-3, atol=1e-3)
            ok_max = np.array_equal(torch.cat(gathered).numpy().astype(np.uint16), wmax.view(np.uint16))
            q.put((bool(ok_sum), bool(ok_max)))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_sharded_sum_protocol_world_size_2():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert q.get(timeout=5) == (True, True)
