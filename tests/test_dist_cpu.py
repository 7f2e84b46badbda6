"""Host-side logic of the data-parallel path with two gloo ranks on the CPU: shards are a disjoint
cover, every rank takes the same number of steps (short ranks join with zero gradients), and the
gradient collective is a SUM."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from neutronbench_b200.toolkit import batches_of, epoch_steps, shard_for_rank, sum_gradients


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n_ids, batch, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ids = np.random.RandomState(2000).permutation(n_ids).astype(np.uint32)   # same shuffle on every rank
    mine = shard_for_rank(ids, rank, world)
    steps = epoch_steps(n_ids, batch, world)
    my_batches = batches_of(len(mine), batch)
    assert my_batches <= steps
    total = torch.zeros(4)
    for step in range(steps):
        if step < my_batches:
            seeds = mine[step * batch:(step + 1) * batch]
            grad = torch.full((4,), float(len(seeds)))          # stand-in gradient: the batch's size
        else:
            grad = torch.zeros(4)                               # UpdateZero: still joins the collective
        sum_gradients(grad, world)
        total += grad
    gathered = [None] * world
    dist.all_gather_object(gathered, mine.tolist())
    if rank == 0:
        flat = sorted(x for part in gathered for x in part)
        assert flat == list(range(n_ids)), "shards must be a disjoint cover of the train list"
        assert total[0].item() == float(n_ids), "summed stand-in gradients must count every seed once"
        out.put("ok")
    dist.destroy_process_group()


def test_two_rank_sharding_and_gradient_sum():
    world, n_ids, batch = 2, 1001, 128      # 501 / 500 ids -> 4 batches each; try uneven below
    ctx = mp.get_context("spawn")
    for n, b in [(n_ids, batch), (129, 128)]:   # second case: rank 0 has 2 batches, rank 1 has 1
        out = ctx.Queue()
        port = _free_port()
        procs = [ctx.Process(target=_worker, args=(r, world, port, n, b, out)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0
        assert out.get(timeout=5) == "ok"


def test_epoch_steps_arithmetic():
    assert epoch_steps(151427, 1024, 1) == 148
    assert epoch_steps(151427, 1024, 8) == 19
    assert epoch_steps(129, 128, 2) == 1 and batches_of(65, 128) == 1
    assert epoch_steps(130, 64, 2) == 2
