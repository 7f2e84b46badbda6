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


# ---------------------------------------------------------------------------------------------------------
# The product's own epoch loop (GCN_GPU_NEIGHBOR_impl.Forward) under world_size 2, with the GPU step stubbed:
# ranks whose shards differ by one batch must still issue the same number of gradient collectives.
# ---------------------------------------------------------------------------------------------------------
def _loop_worker(rank, world, port, n_ids, batch, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from types import SimpleNamespace

    from neutronbench_b200.toolkit import GCN_GPU_NEIGHBOR_impl, GCNConfig

    class StubbedStep(GCN_GPU_NEIGHBOR_impl):
        """Everything that touches the GPU replaced: a batch's 'gradient' is its seed count."""

        def __init__(self, cfg):
            self.cfg, self.rank, self.world_size = cfg, rank, world
            self.device = torch.device("cpu")
            self.layers, self.multi_label, self.use_engine = 2, False, True
            self.overlap_update, self._update_stream = False, None
            self.P = SimpleNamespace(grad=torch.zeros(4))
            self.step_count, self.collectives, self.total = 0, 0, torch.zeros(4)
            self._last = (0.0, 0)

        def engine_step(self, sampler, train=True):
            _, lo, n = sampler._next_seed_ids()
            self.P.grad.fill_(float(n))
            self._last = (1.0, n)              # loss 1 per batch, every seed a hit
            return SimpleNamespace(v=[0, n])

        def _apply_adam(self):
            self.collectives += 1
            self.total += self.P.grad

        def read_stats(self):
            return self._last

        def check_device_errors(self):
            pass

        def _join_update_stream(self):
            pass

    class Seeds:                                # the sampler's seed bookkeeping, nothing on the device
        def __init__(self, ids):
            self.sample_nids, self.batch_size, self.fanout = ids, batch, [10, 5]
            self.sample_rate, self.lower_fanout, self.random_batches, self._dev_nids = 0.0, 0, False, None
            self.work_range, self.work_offset = [0, len(ids)], 0
            self.batch_nums = batches_of(len(ids), batch)
        sample_not_finished = lambda self: self.work_offset < self.work_range[1]
        restart = lambda self: setattr(self, "work_offset", 0)
        from neutronbench_b200.graph import Sampler as _S
        _next_seed_ids = _S._next_seed_ids

    ids = np.random.RandomState(2000).permutation(n_ids).astype(np.uint32)
    mine = shard_for_rank(ids, rank, world)
    tk = StubbedStep(GCNConfig(layers=(8, 4, 2), fanout=(10, 5), batch_size=batch, pipelines=1))
    acc, loss, batches = tk.Forward(Seeds(mine), train=True)
    steps = epoch_steps(n_ids, batch, world)
    assert tk.collectives == steps == tk.step_count, (tk.collectives, steps, tk.step_count)
    assert tk.total[0].item() == float(n_ids)          # every seed counted once; padded steps added zeros
    assert acc == 1.0 and batches == sum(batches_of(len(shard_for_rank(ids, r, world)), batch) for r in range(world))
    assert abs(loss - 1.0) < 1e-12
    if rank == 0:
        out.put("ok")
    dist.destroy_process_group()


def test_product_epoch_loop_pads_short_ranks_with_zero_updates():
    ctx = mp.get_context("spawn")
    for n, b in [(129, 64), (1001, 128), (3, 64)]:     # 65 / 64 ids at batch 64: 2 batches against 1; 3 ids: one short batch each
        out = ctx.Queue()
        port = _free_port()
        procs = [ctx.Process(target=_loop_worker, args=(r, 2, port, n, b, out)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0, "a rank failed or never returned from the epoch loop"
        assert out.get(timeout=5) == "ok"
