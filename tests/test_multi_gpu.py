"""Two real ranks on two GPUs (skipped where fewer are visible): the product's data-parallel loop and the
node-id-sharded feature table over mapped peer memory.  NCCL's in-switch reduction is off and peers are read with
plain loads; a rank leaves only between steps, after its work has drained."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _setup_rank(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0", NCCL_DEBUG="WARN", NCCL_MAX_CTAS="4")
    for p in (ROOT, os.path.join(ROOT, "tests")):
        if p not in sys.path:
            sys.path.insert(0, p)
    import datetime
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank), timeout=datetime.timedelta(seconds=120))
    return torch.device("cuda", rank)


def _problem(dev, V=5000, F=96, classes=7, sharded=False, rank=0, world=1, pipelines=1, batch=200):
    from helpers import small_graph
    from neutronbench_b200 import FullyRepGraph, GCN_GPU_NEIGHBOR_impl, GCNConfig, GNNDatum, Workspace
    from neutronbench_b200.peer import ShardedFeatureTable, shard_rows_for
    edges, co, ri = small_graph(V, 70000, seed=8)
    rng = np.random.RandomState(1)
    feat = rng.randn(V, F).astype(np.float32)
    label = rng.randint(0, classes, size=V).astype(np.int64)
    cfg = GCNConfig(layers=[F, 64, classes], fanout=(6, 4), batch_size=batch, drop_rate=0.0, seed=2000, pipelines=pipelines)
    g = FullyRepGraph.from_edges(torch.from_numpy(edges).to(dev), V, Workspace(64 << 20))
    lab = torch.from_numpy(label).to(dev)
    if sharded:
        rows = shard_rows_for(V, world)
        mine = torch.from_numpy(np.ascontiguousarray(feat[rank * rows: (rank + 1) * rows]))
        table = ShardedFeatureTable.from_rank_shard(mine, V, rank, world, dev)
        datum = GNNDatum(None, lab, np.zeros(V, np.int32), shards=table)
    else:
        datum = GNNDatum(torch.from_numpy(feat).to(dev), lab, np.zeros(V, np.int32))
    tk = GCN_GPU_NEIGHBOR_impl(g, datum, cfg, rank=rank, world_size=world)
    return g, tk, cfg


def _dp_worker(rank, world, port, out):
    import torch.distributed as dist
    dev = _setup_rank(rank, world, port)
    from neutronbench_b200 import Sampler
    from neutronbench_b200.toolkit import shard_for_rank
    # 500 ids dealt to 2 ranks = 250 each at batch 200: two batches per rank; 700 ids: 350 each, two batches;
    # 500 ids at batch 200 with rank 1 given fewer ids below: 2 batches against 1 (zero-gradient padding).
    ids = np.arange(100, 600, dtype=np.uint32)
    mine = shard_for_rank(ids, rank, world)
    if rank == 1:
        mine = mine[:150]                       # one batch only: the second step is an UpdateZero
    for pipelines in (1, 3):
        g, tk, cfg = _problem(dev, rank=rank, world=world, pipelines=pipelines)
        smp = Sampler(g, mine, cfg.fanout, cfg.batch_size, tk.ws, seed=cfg.seed, with_edge_weights=False)
        acc, loss, batches = tk.Forward(smp, train=True)
        torch.cuda.synchronize()
        assert tk.step_count == 2 and batches == 3, (tk.step_count, batches)     # 2 + 1 batches summed over ranks
        w = tk.P.W.clone()
        other = [torch.empty_like(w) for _ in range(world)]
        dist.all_gather(other, w)
        assert torch.equal(other[0], other[1]), "ranks hold different weights after the epoch"
        if rank == 0:
            out.put((pipelines, w.cpu().numpy()))
    dist.barrier()
    dist.destroy_process_group()


def _single_rank_equivalent(dev):
    """One rank that sums, per step, the gradients of the batches the two ranks trained on."""
    from neutronbench_b200 import Sampler
    from neutronbench_b200.toolkit import shard_for_rank
    ids = np.arange(100, 600, dtype=np.uint32)
    shards = [shard_for_rank(ids, 0, 2), shard_for_rank(ids, 1, 2)[:150]]
    g, tk, cfg = _problem(dev)
    samplers = [Sampler(g, s, cfg.fanout, cfg.batch_size, tk.ws, seed=cfg.seed, with_edge_weights=False) for s in shards]
    for step in range(2):
        total = torch.zeros_like(tk.P.grad)
        for smp in samplers:
            if smp.sample_not_finished():
                tk.forward_backward(smp.sample_one(), train=True)
                total += tk.P.grad
        tk.P.grad.copy_(total)
        tk._apply_adam()
        tk.step_count += 1
    torch.cuda.synchronize()
    return tk.P.W.cpu().numpy()


def _run(worker, world=2):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    results = []
    try:
        while len(results) < 2:
            results.append(out.get(timeout=300))
    finally:
        for p in procs:
            p.join(300)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    return results


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_equal_one_rank_summing_both_batches(cuda_device):
    """2 ranks x batch B give the weights of 1 rank that sums the two batches' gradients (the sum is MPI_SUM, not a
    mean), also when one rank runs out of batches a step early, for the plain and the pipelined loop.  Each rank's
    sampler stream differs from the single-rank replay's, so the replay uses the Python step on the same seeds with
    draws keyed the same way (draw 0, 1 per sampler)."""
    results = dict(_run(_dp_worker))
    expect = _single_rank_equivalent(cuda_device)
    for pipelines in (1, 3):
        assert np.abs(results[pipelines] - expect).max() <= 1e-6, pipelines
    np.testing.assert_array_equal(results[1].view(np.uint32), results[3].view(np.uint32))


def _shard_worker(rank, world, port, out):
    import torch.distributed as dist
    dev = _setup_rank(rank, world, port)
    from neutronbench_b200 import Sampler
    ws = []
    for sharded in (False, True):
        g, tk, cfg = _problem(dev, sharded=sharded, rank=rank, world=world, pipelines=3)
        tk.world_size = 1                       # same batches on both ranks: only the feature path differs
        smp = Sampler(g, np.arange(800, dtype=np.uint32), cfg.fanout, cfg.batch_size, tk.ws, seed=cfg.seed,
                      with_edge_weights=False)
        tk.Forward(smp, train=True)
        torch.cuda.synchronize()
        ws.append(tk.P.W.cpu().numpy().copy())
        if sharded:
            dist.barrier()
            tk.datum.shards.close()
    assert np.array_equal(ws[0].view(np.uint32), ws[1].view(np.uint32)), "sharded table changed the training result"
    out.put((rank, True))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_feature_shards_on_a_peer_gpu_equal_the_whole_table(cuda_device):
    """Half of the rows live on the other GPU and are read over NVLink with plain loads while the batch is staged:
    training is bit-identical to the run with the whole table in local memory."""
    results = dict(_run(_shard_worker))
    assert results == {0: True, 1: True}


def _comm_worker(rank, world, port, out):
    """libnb_b200_comm.so without torch.distributed: the unique id travels through a file, as a C++ host would pass it
    with MPI_Bcast."""
    import ctypes as C
    import time
    for p in (ROOT, os.path.join(ROOT, "tests")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(NCCL_NVLS_ENABLE="0", NCCL_DEBUG="WARN")
    from neutronbench_b200 import _lib
    torch.cuda.set_device(rank)
    path = f"/tmp/nb_comm_id_{port}"
    if rank == 0:
        uid = C.create_string_buffer(128)
        _lib.call_comm("nb_comm_unique_id", uid)
        with open(path + ".tmp", "wb") as f:
            f.write(uid.raw)
        os.replace(path + ".tmp", path)
    else:
        for _ in range(600):
            if os.path.exists(path):
                break
            time.sleep(0.05)
    uid = open(path, "rb").read()
    assert len(uid) == 128
    comm = C.c_void_p()
    _lib.call_comm("nb_comm_create", C.byref(comm), uid, world, rank)
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.arange(1000, dtype=torch.float32, device=f"cuda:{rank}") * (rank + 1)
    _lib.call_comm("nb_allreduce_sum_f32", comm, g.data_ptr(), g.numel(), stream)
    w = torch.full((257,), float(rank + 5), device=f"cuda:{rank}")
    _lib.call_comm("nb_broadcast_f32", comm, w.data_ptr(), w.numel(), 0, stream)
    torch.cuda.synchronize()
    expect = torch.arange(1000, dtype=torch.float32) * sum(r + 1 for r in range(world))
    ok = bool(torch.equal(g.cpu(), expect)) and bool((w.cpu() == 5.0).all())
    _lib.call_comm("nb_comm_destroy", comm)
    out.put((rank, ok))
    if rank == 0:
        time.sleep(0.5)
        try:
            os.remove(path)
        except OSError:
            pass


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_nb_allreduce_and_broadcast_over_nccl(cuda_device):
    """nb_allreduce_sum_f32 is a SUM (MPI_SUM in the reference, comm/network.h:189-193), in place on the device buffer;
    nb_broadcast_f32 hands rank 0's weights to everyone (Parameter::init_parameter)."""
    results = dict(_run(_comm_worker))
    assert results == {0: True, 1: True}
