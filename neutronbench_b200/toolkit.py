"""Sampled mini-batch GCN trainer: the host-side mirror of GCN_GPU_NEIGHBOR_impl
(toolkits/GCN_GPU_NEIGHBOR.hpp:7-1556) on top of the C ABI.

One training step = sample_one -> feature/label gather -> per layer (aggregate, X*W, relu+dropout) ->
loss -> backward (dW = Y^T dZ, dY = dZ W^T, transposed-CSR aggregate fused with the relu/dropout
gradient) -> gradient sum over ranks -> Adam.  Like the reference (core/ntsContext.hpp:292) the
input-side block is never back-propagated, so an L-layer step runs L forward and L-1 backward
aggregations.  Every kernel is from libnb_b200.so; torch provides device memory, streams and
torch.distributed only.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch

from . import _lib
from .cuda_stream import Cuda_Stream, Workspace, ptr
from .graph import FullyRepGraph, SampledSubgraph, Sampler


@dataclass
class GCNConfig:
    """The .cfg keys the sampled GCN path reads (core/GraphSegment.cpp:196-405)."""
    layers: Sequence[int] = (128, 128, 40)        # LAYERS a-b-c
    fanout: Sequence[int] = (25, 10)              # hop order: seeds first (cfg FANOUT lists the reverse)
    val_fanout: Optional[Sequence[int]] = None
    batch_size: int = 1024
    learn_rate: float = 0.01
    weight_decay: float = 0.0001
    drop_rate: float = 0.5
    classes: int = 1
    cache_type: str = "none"                      # none | rate | gpu_memory
    cache_rate: float = 0.0
    cache_policy: str = "degree"
    seed: int = 2000
    fuse_gather: bool = True                      # layer-0 aggregation reads the feature store directly
    beta1: float = 0.9
    beta2: float = 0.999
    epsilon: float = 1e-9                         # toolkits/GCN_GPU_NEIGHBOR.hpp:217
    pipelines: int = 1                            # PIPELINES > 1: sampling of batch i+1 overlaps training of batch i
    sample_rate: float = 0.0                      # SAMPLE_RATE > 0: degree-proportional fan-out for training batches
    lower_fanout: int = 0                         # LOWER_FANOUT of that mode
    # rows that are not cached are copied once per distinct source into a staging table by the sampling half
    # (None: for a table sharded over GPUs, which is read no other way, and for a host table when world_size > 1)
    stage_misses: Optional[bool] = None
    reserve_sms: Optional[int] = None             # SMs left to the gradient all-reduce (None: 4 when world_size > 1)
    cache_row_pitch: int = 0                      # floats between rows of the GPU feature cache (0: chosen from the width)


class Parameter:
    """All layer weights in one flat bucket so that the gradient sum and Adam are one call each.
    Per layer: xavier-uniform W[row x col] (core/NtsScheduler.hpp:641-643), zero M and V, and the
    running beta powers of Parameter::next (core/NtsScheduler.hpp:700-711)."""

    def __init__(self, layer_sizes: Sequence[int], cfg: GCNConfig, device, generator: Optional[torch.Generator] = None):
        self.shapes = [(layer_sizes[i], layer_sizes[i + 1]) for i in range(len(layer_sizes) - 1)]
        self.offsets = [0]
        for r, c in self.shapes:
            self.offsets.append(self.offsets[-1] + r * c)
        n = self.offsets[-1]
        host = torch.empty(n, dtype=torch.float32)
        for i, (r, c) in enumerate(self.shapes):
            bound = math.sqrt(6.0 / (r + c))
            w = torch.empty(r, c).uniform_(-bound, bound, generator=generator)
            host[self.offsets[i]: self.offsets[i + 1]] = w.reshape(-1)
        self.W = host.to(device)
        self.grad = torch.zeros(n, dtype=torch.float32, device=device)
        self.M = torch.zeros(n, dtype=torch.float32, device=device)
        self.V = torch.zeros(n, dtype=torch.float32, device=device)
        self.cfg = cfg
        self.beta1_t = np.float32(cfg.beta1)
        self.beta2_t = np.float32(cfg.beta2)

    def w(self, l: int) -> torch.Tensor:
        r, c = self.shapes[l]
        return self.W[self.offsets[l]: self.offsets[l + 1]].view(r, c)

    def g(self, l: int) -> torch.Tensor:
        r, c = self.shapes[l]
        return self.grad[self.offsets[l]: self.offsets[l + 1]].view(r, c)

    def learn_with_decay_Adam(self, stream: int):
        """learnC2G_with_decay_Adam + next (core/NtsScheduler.hpp:794-811, 700-711)."""
        c = self.cfg
        _lib.call("nb_adam", ptr(self.W), ptr(self.grad), ptr(self.M), ptr(self.V), self.W.numel(), c.learn_rate,
                  c.beta1, c.beta2, c.epsilon, c.weight_decay, float(self.beta1_t), float(self.beta2_t), stream)
        self.beta1_t = np.float32(self.beta1_t * np.float32(c.beta1))
        self.beta2_t = np.float32(self.beta2_t * np.float32(c.beta2))


class GNNDatum:
    """Feature table, labels and split mask (core/ntsDataloador.hpp:32-476).  Features stay where the
    caller put them: a CUDA tensor, a pinned host tensor that the gather kernel reads zero-copy, or
    (`shards`) a table sharded by node-id range over the GPUs of the job."""

    def __init__(self, feature: Optional[torch.Tensor], label: torch.Tensor, mask: np.ndarray, shards=None):
        assert shards is not None or (feature.dtype == torch.float32 and feature.dim() == 2)
        self.local_feature = feature
        self.local_label = label      # int64 on the GPU
        self.local_mask = mask        # 0 train, 1 val, 2 test (core/ntsDataloador.hpp:318-330)
        self.shards = shards          # a peer.ShardedFeatureTable, or None


def cache_slots_by_key(key: np.ndarray, cache_num: int) -> np.ndarray:
    """mark_cache_node after a descending sort by `key` (toolkits/GCN_GPU_NEIGHBOR.hpp:930-943): the first
    cache_num nodes of the order take slots 0..cache_num-1, all others 0xFFFFFFFF.  The reference's
    std::sort leaves equal keys in unspecified order; here ties go by ascending id."""
    V = len(key)
    order = np.lexsort((np.arange(V, dtype=np.int64), -key.astype(np.int64)))
    hashmap = np.full(V, 0xFFFFFFFF, dtype=np.uint32)
    cache_num = min(int(cache_num), V)
    hashmap[order[:cache_num]] = np.arange(cache_num, dtype=np.uint32)
    return hashmap


def cache_slots_by_degree(out_degree: np.ndarray, cache_num: int) -> np.ndarray:
    """CACHE_POLICY:degree — cache_high_degree (toolkits/GCN_GPU_NEIGHBOR.hpp:958-967)."""
    return cache_slots_by_key(out_degree, cache_num)


def cache_slots_by_sample_count(sample_count: np.ndarray, cache_num: int) -> np.ndarray:
    """CACHE_POLICY:sample — cache_sample (toolkits/GCN_GPU_NEIGHBOR.hpp:974-999): nodes ordered by how often
    they appeared as a block source during one dry-run epoch of the training sampler."""
    return cache_slots_by_key(sample_count, cache_num)


def cache_slots_random(num_vertices: int, cache_num: int, seed: int) -> np.ndarray:
    """CACHE_POLICY:random — cache_random_node (toolkits/GCN_GPU_NEIGHBOR.hpp:969-972): a seeded shuffle of
    the node ids; the first cache_num take the slots.  (The reference shuffles with its own seeded
    generator; only the distribution, a uniform random subset, is matched.)"""
    order = np.random.RandomState(seed).permutation(num_vertices)
    hashmap = np.full(num_vertices, 0xFFFFFFFF, dtype=np.uint32)
    cache_num = min(int(cache_num), num_vertices)
    hashmap[order[:cache_num]] = np.arange(cache_num, dtype=np.uint32)
    return hashmap


def cache_nodes_for_memory(free_bytes: int, feature_size: int, num_vertices: int, reserve_mb: int = 100) -> int:
    """CACHE_TYPE:gpu_memory sizing (toolkits/GCN_GPU_NEIGHBOR.hpp:1427-1441): the memory left after a dry
    run, minus 100 MB, divided by the bytes of one feature row."""
    free_mb = free_bytes / (1024.0 * 1024.0) - reserve_mb
    if free_mb <= 0:
        return 0
    return int(min(num_vertices, free_mb * 1024 * 1024 / 4 / feature_size))


class GCN_GPU_NEIGHBOR_impl:
    """Trainer with the reference toolkit's structure (init_nn / Forward / Update / run)."""

    def __init__(self, graph: FullyRepGraph, datum: GNNDatum, cfg: GCNConfig, ws: Optional[Workspace] = None,
                 rank: int = 0, world_size: int = 1, use_engine: bool = True):
        self.graph = graph
        self.datum = datum
        self.cfg = cfg
        self.device = graph.device
        self.rank, self.world_size = rank, world_size
        self.layers = len(cfg.layers) - 1
        assert len(cfg.fanout) == self.layers
        self.ws = ws if ws is not None else Workspace(default_workspace_bytes(graph.global_vertices, cfg))
        self.cuda_stream = Cuda_Stream()
        gen = torch.Generator().manual_seed(cfg.seed)
        self.P = Parameter(cfg.layers, cfg, self.device, gen)
        if world_size > 1:
            # every rank starts from rank 0's weights (Parameter::init_parameter, core/NtsScheduler.hpp:691)
            torch.distributed.broadcast(self.P.W, src=0)
        self.step_count = 0
        # (loss, hits) for one label per node; (loss, predicted-and-true, predicted, true) with CLASSES > 1
        self.stats = torch.zeros(4, dtype=torch.float32, device=self.device)
        self._stats_host = torch.zeros(4, dtype=torch.float32).pin_memory()
        self.multi_label = int(cfg.classes) > 1
        # Gradient sum + Adam on a (high-priority) stream of their own when there is an all-reduce to hide: they
        # overlap the next batch's layer-0 aggregation, which does not read the weights.  Measured on 2 GPUs:
        # 0.234 against 0.254 ms/step end to end.  NB_OVERLAP_UPDATE=0 / 1 overrides.
        self.overlap_update = os.environ.get("NB_OVERLAP_UPDATE", "1" if world_size > 1 else "0") == "1"
        self._update_stream = None
        # The per-step gradient sum goes through the library's own NCCL communicator (nb_allreduce_sum_f32): three
        # C calls per step on the update stream instead of a torch.distributed collective, whose host-side cost per call
        # is a visible share of a 0.23 ms step (4 GPUs, Reddit-shaped: 0.215 against 0.229 ms per step end to end).
        # torch.distributed stays for set-up, per-epoch scalars and as the fallback (NB_NATIVE_ALLREDUCE=0, a backend
        # other than NCCL, or the communication library not built).
        self._native_comm = None
        if world_size > 1 and use_engine and os.environ.get("NB_NATIVE_ALLREDUCE", "1") == "1" and \
                torch.distributed.get_backend() == "nccl":
            self._native_comm = _open_native_comm(rank, world_size, self.device)
        self.fuse_output_layer = True   # last layer + loss + its gradients in two launches (nb_output_layer)
        if self.multi_label:
            assert int(cfg.classes) == int(cfg.layers[-1]), "CLASSES > 1 needs one output per class"
            assert datum.local_label.dim() == 2 and datum.local_label.size(1) == int(cfg.classes)
        self.dev_cache_feature = None
        self.dev_cache_node_hashmap = None
        self.cache_node_num = 0
        self.feature_on_device = datum.shards is None and datum.local_feature.is_cuda
        # Staging is needed for a sharded table.  For a table in mapped host memory it measured no gain on one GPU
        # (Products-shaped: 0.72 against 0.70 ms per step: repeated reads of a host row inside one launch already hit
        # L2, and the staging copy slows the dense kernels that run beside it), but with several ranks reading the
        # same host memory it takes the host reads out of the training stream (4 ranks: 0.70 against 0.75 ms), so
        # it is the default when world_size > 1 and some rows are not cached.
        self.stage_misses = default_stage_misses(cfg, datum.shards is not None, self.feature_on_device, world_size)
        self.reserve_sms = (4 if world_size > 1 else 0) if cfg.reserve_sms is None else int(cfg.reserve_sms)
        self.device_errors_checked = 0
        self.agg_edges_fwd = 0
        self.agg_edges_bwd = 0
        self.events = None  # when a list: (name, algorithmic bytes, start event, end event) per aggregation
        # use_engine: a batch is one native call (nb_gcn_step) instead of one Python call per kernel family;
        # both issue the same kernels in the same order and give identical results.
        self.use_engine = use_engine
        self._engine = None
        self._engine_cfg = None
        self.last_info = None
        # pipelined batch loop (pipeline_version, toolkits/GCN_GPU_NEIGHBOR.hpp:399-505): two sampled
        # subgraphs in flight, sampling on a stream of its own
        self._batches = None
        self._batch_ws = None
        self._sample_streams = None
        self._compute_stream = None

    def _timed(self, name: str, nbytes: int, fn):
        """Runs fn(); with self.events set, brackets it with CUDA events on the current stream."""
        if self.events is None:
            fn()
            return
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        self.events.append((name, nbytes, s, e))

    @staticmethod
    def agg_bytes_fwd(blk, F: int, gather_fused: bool = False, cached: bool = False) -> int:
        """Compulsory traffic of one forward aggregation: every source row read once, every destination
        row written once, row indices, column offsets, the two sqrt-degree vectors; the gather-fused
        form also reads the global ids (and cache slots) of the sources."""
        s, v, e = blk.src_size, blk.v_size, blk.e_size
        b = 4 * F * (s + v) + 4 * e + 4 * (v + 1) + 4 * (s + v)
        if gather_fused:
            b += 4 * s + (4 * s if cached else 0)
        return b

    @staticmethod
    def agg_bytes_bwd(blk, F: int, masked: bool = True) -> int:
        s, v, e = blk.src_size, blk.v_size, blk.e_size
        return 4 * F * (v + s) + 4 * e + 4 * (s + 1) + 4 * (s + v) + (4 * F * s if masked else 0)

    # ------------------------------------------------------------------ cache (toolkits/...:899-999, 1214-1243)
    def sample_counts(self, train_sampler: Sampler) -> np.ndarray:
        """Dry-run epoch of cache_sample (toolkits/GCN_GPU_NEIGHBOR.hpp:974-999): how often every node is a
        source of a sampled block.  The sampler is restarted afterwards; the draws are not replayed by
        training (the reference also trains on fresh draws)."""
        V = self.graph.global_vertices
        counts = torch.zeros(V, dtype=torch.int32, device=self.device)
        stream = torch.cuda.current_stream().cuda_stream
        while train_sampler.sample_not_finished():
            ssg = train_sampler.sample_one()
            for blk in ssg.sampled_sgs:
                _lib.call("nb_count_ids", ptr(blk.source), blk.src_size, V, ptr(counts), stream)
        train_sampler.restart()
        return counts.cpu().numpy().view(np.uint32)

    def determine_cache_node_idx(self, node_nums: int, train_sampler: Optional[Sampler] = None):
        V = self.graph.global_vertices
        node_nums = min(int(node_nums), V)
        self.cache_node_num = node_nums
        if node_nums == 0:
            return
        policy = self.cfg.cache_policy
        if policy == "degree":
            out_deg = self.graph.out_degree.cpu().numpy().astype(np.uint32)
            out_deg = np.maximum(out_deg, 1)  # generate_backward_structure clamp, core/graph.hpp:3983-3986
            hashmap = cache_slots_by_degree(out_deg, node_nums)
        elif policy == "sample":
            assert train_sampler is not None, "CACHE_POLICY:sample needs the training sampler for its dry run"
            hashmap = cache_slots_by_sample_count(self.sample_counts(train_sampler), node_nums)
        elif policy == "random":
            hashmap = cache_slots_random(V, node_nums, self.cfg.seed)
        else:
            raise ValueError(f"cache_policy {policy!r} is not one of degree | sample | random")
        self.dev_cache_node_hashmap = torch.from_numpy(hashmap.view(np.int32)).to(self.device)
        F = self.cfg.layers[0]
        # private layout: rows padded to 16 bytes so that 128-bit loads and bulk copies apply; wide rows (the ones the
        # aggregation stages through shared memory) start on a 128-byte line, which saves a partly used line per row read
        ld = (F + 31) // 32 * 32 if F >= 256 else (F + 3) // 4 * 4
        if self.cfg.cache_row_pitch:
            assert self.cfg.cache_row_pitch >= F and self.cfg.cache_row_pitch % 4 == 0
            ld = int(self.cfg.cache_row_pitch)
        self.dev_cache_feature = torch.zeros((node_nums, ld), dtype=torch.float32, device=self.device)
        feat = self.datum.local_feature
        _lib.call("nb_cache_fill", ptr(self.dev_cache_feature), ld, ptr(feat), feat.stride(0),
                  ptr(self.dev_cache_node_hashmap), V, F, torch.cuda.current_stream().cuda_stream)
        assert self._engine is None, "the feature cache must be set up before the first native step"

    def init_cache(self, train_sampler: Optional[Sampler] = None):
        """CACHE_TYPE handling of run() (toolkits/GCN_GPU_NEIGHBOR.hpp:1426-1454)."""
        c = self.cfg
        V = self.graph.global_vertices
        if c.cache_type in ("rate", "random"):
            assert 0.0 <= c.cache_rate <= 1.0
            self.determine_cache_node_idx(int(V * c.cache_rate), train_sampler)
        elif c.cache_type == "gpu_memory":
            # The reference trains one dry-run epoch to learn libtorch's peak memory.  Here every per-step
            # buffer comes from arenas of fixed size, so it is enough to create them (and the sampling
            # slots of the pipelined loop) before asking the driver how much memory is left.
            reserve = [Workspace(default_workspace_bytes(V, c)) for _ in range(max(2, c.pipelines) if c.pipelines > 1 else 0)]
            torch.cuda.synchronize()
            free_bytes, _total = torch.cuda.mem_get_info(self.device)
            del reserve
            self.determine_cache_node_idx(cache_nodes_for_memory(free_bytes, c.layers[0], V), train_sampler)
        elif c.cache_type != "none":
            raise ValueError(f"cache_type {c.cache_type!r} is not one of none | rate | random | gpu_memory")

    # ------------------------------------------------------------------ one step
    def _rows(self, shape) -> torch.Tensor:
        """Uninitialised fp32 buffer of at least [rows x cols] on the device, handed to the library by address only.
        A block without edges or vertices gives zero rows; one row is allocated then, so that the address is a valid
        (never dereferenced) non-null pointer — torch reports a null address for an empty tensor."""
        rows, cols = shape
        return torch.empty((max(int(rows), 1), int(cols)), dtype=torch.float32, device=self.device)

    def _aggregate0(self, ssg: SampledSubgraph, stream: int) -> torch.Tensor:
        blk = ssg.sampled_sgs[0]
        F = self.cfg.layers[0]
        feat = self.datum.local_feature
        Y = self._rows((blk.v_size, F))
        cache, hm = self.dev_cache_feature, self.dev_cache_node_hashmap
        if self.cfg.fuse_gather:
            self._timed("fwd0_gather_fused", self.agg_bytes_fwd(blk, F, True, hm is not None), lambda: _lib.call(
                "nb_spmm_csc_fwd_gather_fused", self.ws.handle, ptr(feat), feat.stride(0), ptr(cache),
                cache.stride(0) if cache is not None else 0, ptr(hm), ptr(blk.source), ptr(Y), ptr(blk.row_indices),
                ptr(blk.column_offset), ptr(blk.src_norm), ptr(blk.dst_norm), blk.v_size, blk.src_size, blk.e_size, F, stream))
        else:
            X0 = self._rows((blk.src_size, F))
            _lib.call("nb_feature_gather", ptr(X0), ptr(feat), feat.stride(0), None, 0, 0, ptr(cache),
                      cache.stride(0) if cache is not None else 0, ptr(hm), ptr(blk.source), blk.src_size, F, stream)
            self._timed("fwd0", self.agg_bytes_fwd(blk, F), lambda: _lib.call(
                "nb_spmm_csc_fwd_fused", ptr(X0), ptr(Y), ptr(blk.row_indices), ptr(blk.column_offset),
                ptr(blk.src_norm), ptr(blk.dst_norm), blk.v_size, F, stream))
        return Y

    def forward_backward(self, ssg: SampledSubgraph, train: bool = True):
        """Runs one batch; leaves loss and hit count in self.stats (device) and dW in P.grad."""
        c, L = self.cfg, self.layers
        stream = torch.cuda.current_stream().cuda_stream
        wsh = self.ws.handle
        p = c.drop_rate if train else 0.0
        scale = 1.0 / (1.0 - p) if p > 0 else 1.0
        Y: List[torch.Tensor] = []
        X: List[Optional[torch.Tensor]] = [None]
        # the last layer with one label per vertex runs fused with its loss and gradients, as in the native step
        fused_out = (self.fuse_output_layer and not self.multi_label
                     and bool(_lib.load().nb_output_layer_supported(int(c.layers[L - 1]), int(c.layers[L]))))
        for l in range(L):
            blk = ssg.sampled_sgs[l]
            if l == 0:
                y = self._aggregate0(ssg, stream)
            else:
                y = self._rows((blk.v_size, c.layers[l]))
                self._timed(f"fwd{l}", self.agg_bytes_fwd(blk, c.layers[l]), lambda: _lib.call(
                    "nb_spmm_csc_fwd_fused", ptr(X[l]), ptr(y), ptr(blk.row_indices), ptr(blk.column_offset),
                    ptr(blk.src_norm), ptr(blk.dst_norm), blk.v_size, c.layers[l], stream))
            Y.append(y)
            if l == L - 1 and fused_out:
                break
            z = self._rows((blk.v_size, c.layers[l + 1]))
            _lib.call("nb_gemm", wsh, ptr(y), ptr(self.P.w(l)), ptr(z), blk.v_size, c.layers[l + 1], c.layers[l], 0,
                      0, stream)
            if l < L - 1:
                _lib.call("nb_relu_dropout", ptr(z), blk.v_size * c.layers[l + 1], p, c.seed, l, self.step_count, stream)
            X.append(z)
        last = ssg.sampled_sgs[L - 1]
        B, C = last.v_size, c.layers[L]
        dZ = torch.empty((B, C), dtype=torch.float32, device=self.device) if (train and not fused_out) else None
        dY_out = None
        if fused_out:
            H = c.layers[L - 1]
            if train and L > 1:
                dY_out = torch.empty((B, H), dtype=torch.float32, device=self.device)
            _lib.call("nb_output_layer", wsh, ptr(Y[L - 1]), ptr(self.P.w(L - 1)), ptr(self.datum.local_label),
                      ptr(last.destination), B, H, C, 1 if train else 0, ptr(self.P.g(L - 1)), ptr(dY_out),
                      ptr(self.stats), stream)
        elif self.multi_label:   # Loss(..., onelabel=false), utils/torch_func.hpp:67-75
            lab = torch.empty((B, C), dtype=torch.int64, device=self.device)
            _lib.call("nb_label_gather", ptr(lab), ptr(self.datum.local_label), ptr(last.destination), B, C, stream)
            _lib.call("nb_sigmoid_bce", wsh, ptr(X[L]), ptr(lab), B, C, ptr(dZ), ptr(self.stats), stream)
        else:
            lab = torch.empty(B, dtype=torch.int64, device=self.device)
            _lib.call("nb_label_gather", ptr(lab), ptr(self.datum.local_label), ptr(last.destination), B, 1, stream)
            _lib.call("nb_softmax_nll", wsh, ptr(X[L]), ptr(lab), B, C, ptr(dZ), ptr(self.stats), stream)
        self.agg_edges_fwd += sum(b.e_size for b in ssg.sampled_sgs)
        if not train:
            return
        for l in range(L - 1, -1, -1):
            blk = ssg.sampled_sgs[l]
            Fi, Fo = c.layers[l], c.layers[l + 1]
            from_fused = fused_out and l == L - 1     # dW and dY of the last layer are already there
            if not from_fused:
                _lib.call("nb_gemm", wsh, ptr(Y[l]), ptr(dZ), ptr(self.P.g(l)), Fi, Fo, blk.v_size, 1, 0, stream)
            if l == 0:
                break  # the input-side block is never back-propagated (core/ntsContext.hpp:292)
            if from_fused:
                dY = dY_out
            else:
                dY = self._rows((blk.v_size, Fi))
                _lib.call("nb_gemm", wsh, ptr(dZ), ptr(self.P.w(l)), ptr(dY), blk.v_size, Fi, Fo, 0, 1, stream)
            dX = self._rows((blk.src_size, Fi))
            self._timed(f"bwd{l}", self.agg_bytes_bwd(blk, Fi), lambda: _lib.call(
                "nb_spmm_csr_bwd_fused", ptr(dY), ptr(dX), ptr(blk.row_offset), ptr(blk.column_indices),
                ptr(blk.src_norm), ptr(blk.dst_norm), ptr(X[l]), scale, blk.src_size, Fi, stream))
            self.agg_edges_bwd += blk.e_size
            dZ = dX

    # ------------------------------------------------------------------ native step (nb_gcn_*)
    def _ensure_engine(self):
        if self._engine is not None:
            return self._engine
        import ctypes as C
        c = self.cfg
        ec = _lib.GcnConfig()
        ec.num_layers = self.layers
        for i, w in enumerate(c.layers):
            ec.layer_size[i] = int(w)
        for i, f in enumerate(c.fanout):
            ec.fanout[i] = int(f)
        ec.num_vertices = self.graph.global_vertices
        ec.learn_rate, ec.weight_decay, ec.drop_rate = c.learn_rate, c.weight_decay, c.drop_rate
        ec.beta1, ec.beta2, ec.epsilon = c.beta1, c.beta2, c.epsilon
        ec.seed = c.seed
        ec.fuse_gather = 1 if c.fuse_gather else 0
        ec.sample_rate, ec.lower_fanout = float(c.sample_rate), int(c.lower_fanout)
        ec.classes = int(c.classes)
        ec.d_graph_column_offset = ptr(self.graph.column_offset)
        ec.d_graph_row_indices = ptr(self.graph.row_indices)
        if self.datum.shards is not None:
            sh = self.datum.shards
            ec.d_feat_shards, ec.num_shards, ec.shard_rows = ptr(sh.table), sh.num_shards, sh.shard_rows
            ec.feat, ec.feat_ld = None, sh.ld
        else:
            feat = self.datum.local_feature
            ec.feat, ec.feat_ld = ptr(feat), feat.stride(0)
        ec.stage_misses = 1 if self.stage_misses else 0
        if self.dev_cache_feature is not None:
            ec.d_cache, ec.cache_ld = ptr(self.dev_cache_feature), self.dev_cache_feature.stride(0)
            ec.d_hashmap = ptr(self.dev_cache_node_hashmap)
        ec.d_label = ptr(self.datum.local_label)
        ec.d_W, ec.d_grad, ec.d_M, ec.d_V = ptr(self.P.W), ptr(self.P.grad), ptr(self.P.M), ptr(self.P.V)
        handle = C.c_void_p()
        _lib.load().nb_set_fused_output_layer(1 if self.fuse_output_layer else 0)
        _lib.call("nb_gcn_create", C.byref(handle), C.byref(ec), self.ws.handle)
        self._engine, self._engine_cfg = handle, ec
        if self.reserve_sms:
            _lib.call("nb_gcn_set_option", handle, b"reserve_sms", self.reserve_sms)
        return handle

    def engine_step(self, sampler: Sampler, train: bool = True):
        """One batch through nb_gcn_step; leaves loss/hits in self.stats and dW in P.grad."""
        import ctypes as C
        eng = self._ensure_engine()
        seeds, n = sampler.next_seeds()
        info = _lib.GcnStepInfo()
        _lib.call("nb_gcn_step", eng, ptr(seeds), n, 1 if train else 0, ptr(self.stats), C.byref(info),
                  torch.cuda.current_stream().cuda_stream)
        L = self.layers
        self.agg_edges_fwd += sum(info.e[l] for l in range(L))
        if train:
            self.agg_edges_bwd += sum(info.e[l] for l in range(1, L))
        self.last_info = info
        return info

    # ------------------------------------------------------------------ pipelined halves of the native step
    def _ensure_pipeline(self):
        """PIPELINES = P keeps P sampled subgraphs in flight: one training, P-1 being drawn, each by a
        library thread on a stream of its own."""
        if self._batches is not None:
            return
        import ctypes as C
        slots = max(2, int(self.cfg.pipelines))
        self._sample_streams = [torch.cuda.Stream(device=self.device) for _ in range(slots)]
        self._batch_ws = [Workspace(default_workspace_bytes(self.graph.global_vertices, self.cfg)) for _ in range(slots)]
        self._slot_seeds = [torch.empty(self.cfg.batch_size, dtype=torch.int32).pin_memory() for _ in range(slots)]
        self._slot_refs = [None] * slots
        self._stats_ring = [torch.zeros(4, dtype=torch.float32).pin_memory() for _ in range(2)]
        self._stats_dev_ring = [torch.zeros(4, dtype=torch.float32, device=self.device) for _ in range(2)]
        self._readback_stream = torch.cuda.Stream(device=self.device)
        self._readback_on_side_stream = os.environ.get("NB_READBACK_STREAM", "1") == "1"
        self._batches = []
        for w in self._batch_ws:
            h = C.c_void_p()
            _lib.call("nb_gcn_batch_create", C.byref(h), w.handle)
            self._batches.append(h)
        _lib.call("nb_gcn_set_sampler_threads", self._ensure_engine(), slots - 1)

    def sample_batch(self, sampler: Sampler, slot: int, train: bool = True):
        """Asks the library's sampler thread (nb_gcn_sample_async) to draw the sampler's next batch into
        subgraph `slot` on the sampling stream; returns at once.  compute_batch(slot) waits for it."""
        self._ensure_pipeline()
        seeds, n = sampler.next_seeds_into(self._slot_seeds[slot])
        self._slot_refs[slot] = seeds   # keeps a staged device slice alive until the batch is computed
        _lib.call("nb_gcn_sample_async", self._ensure_engine(), self._batches[slot], ptr(seeds), n, 1 if train else 0,
                  self._sample_streams[slot].cuda_stream)
        return n

    def sample_from_edges(self, seeds: torch.Tensor, raw_edges: Sequence[torch.Tensor], slot: int = 0):
        """nb_gcn_sample_from_edges: builds subgraph `slot` from externally sampled edge lists (one int32 device
        tensor of global source ids per hop, seeds first) instead of drawing it; compute_batch(slot) trains on it.
        This is how a run of the reference's trainer is replayed through the native step."""
        import ctypes as C
        self._ensure_pipeline()
        L = self.layers
        assert len(raw_edges) == L
        ptrs = (C.c_void_p * L)(*[r.data_ptr() if r.numel() else None for r in raw_edges])
        counts = (C.c_uint32 * L)(*[int(r.numel()) for r in raw_edges])
        self._slot_refs[slot] = (seeds, list(raw_edges))
        _lib.call("nb_gcn_sample_from_edges", self._ensure_engine(), self._batches[slot], ptr(seeds), int(seeds.numel()),
                  ptrs, counts, self._sample_streams[slot].cuda_stream)

    def compute_batch(self, slot: int, train: bool = True, stats: Optional[torch.Tensor] = None):
        """nb_gcn_compute on subgraph `slot`, on the current stream; never blocks the host.  Loss and hits go to
        `stats` (default: self.stats)."""
        import ctypes as C
        info = _lib.GcnStepInfo()
        _lib.call("nb_gcn_compute", self._ensure_engine(), self._batches[slot], 1 if train else 0,
                  ptr(self.stats if stats is None else stats), C.byref(info), torch.cuda.current_stream().cuda_stream)
        L = self.layers
        self.agg_edges_fwd += sum(info.e[l] for l in range(L))
        if train:
            self.agg_edges_bwd += sum(info.e[l] for l in range(1, L))
        self.last_info = info
        return info

    def run_pipelined(self, sampler: Sampler, max_batches: Optional[int] = None, train: bool = True,
                      on_batch=None, read_back: bool = True, pad_to_steps: int = 0):
        """Batch loop with the next batch's sampling issued while the current batch trains.  The order of
        batches, sampler draws and optimizer steps is that of the plain loop, so results are identical.
        Returns (correct, nodes, loss sum, batches); with read_back False no statistics are read.
        pad_to_steps: when this rank has fewer batches than that, it joins the remaining gradient sums with
        zeros (UpdateZero), so that every rank of a data-parallel job issues the same number of collectives."""
        assert self.use_engine, "the pipelined loop runs on the native step"
        correct = nodes = batches = 0
        loss_sum = 0.0
        if not sampler.sample_not_finished() or (max_batches is not None and max_batches <= 0):
            if train:
                self._pad_steps(pad_to_steps - batches)
            return correct, nodes, loss_sum, batches
        self._ensure_pipeline()
        slots = len(self._batches)
        # The training half runs on a high-priority stream: when an SM frees up, its kernels are placed before the
        # short sampling kernels of the batches drawn ahead, which have slack.
        if self._compute_stream is None:
            self._compute_stream = torch.cuda.Stream(device=self.device, priority=-1)
        outer = torch.cuda.current_stream()
        self._compute_stream.wait_stream(outer)
        with torch.cuda.stream(self._compute_stream):
            result = self._run_pipelined_on_current_stream(sampler, max_batches, train, on_batch, read_back, slots)
            if train:
                self._pad_steps(pad_to_steps - result[3])
        outer.wait_stream(self._compute_stream)
        return result

    def _pad_steps(self, n: int):
        for _ in range(max(0, n)):
            self.UpdateZero()
            self.step_count += 1
        if n > 0:
            self._join_update_stream()

    def _run_pipelined_on_current_stream(self, sampler, max_batches, train, on_batch, read_back, slots):
        correct = nodes = batches = 0
        loss_sum = 0.0

        def more_to_issue():
            return sampler.sample_not_finished() and (max_batches is None or issued < max_batches)

        issued = 0
        while issued < slots - 1 and more_to_issue():   # fill the pipeline
            self.sample_batch(sampler, issued % slots, train)
            issued += 1
        slot = 0
        pending_read = None
        while True:
            if more_to_issue():   # the sampler threads draw ahead while this thread enqueues batch i
                self.sample_batch(sampler, issued % slots, train)
                issued += 1
            dev_stats = self._stats_dev_ring[batches & 1] if read_back else None
            info = self.compute_batch(slot, train=train, stats=dev_stats)
            if train:
                self.Update()
                self.step_count += 1
            if read_back:   # copy now, read one batch later: the host never waits for the batch it just enqueued
                if pending_read is not None:
                    pending_read[1].synchronize()
                    loss, score = self._loss_and_score(pending_read[0])
                    loss_sum += loss
                    correct += score
                # The copy runs on a stream of its own, behind an event of the training stream, and each of two
                # device buffers is written by every other step: a copy enqueued on the training stream itself would
                # put a DMA operation, and the switch back from it, in front of the next step's first kernel.
                host = self._stats_ring[batches & 1]
                if self._readback_on_side_stream:
                    done = torch.cuda.Event()
                    done.record()
                    rb = self._readback_stream
                    rb.wait_event(done)
                    with torch.cuda.stream(rb):
                        host.copy_(dev_stats, non_blocking=True)
                        ev = torch.cuda.Event()
                        ev.record()
                else:
                    host.copy_(dev_stats, non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record()
                pending_read = (host, ev)
            batches += 1
            nodes += info.v[self.layers - 1]
            if on_batch is not None:
                on_batch(batches)
            if batches >= issued:
                break
            slot = (slot + 1) % slots
        if pending_read is not None:
            pending_read[1].synchronize()
            loss, score = self._loss_and_score(pending_read[0])
            loss_sum += loss
            correct += score
        self._join_update_stream()
        return correct, nodes, loss_sum, batches

    def Update(self):
        """Gradient SUM over ranks (MPI_SUM in the reference, comm/network.h:189-193) then Adam."""
        if self.use_engine and self.overlap_update:
            # on a stream of their own, the gradient sum and Adam overlap the next batch's layer-0 aggregation
            if self._update_stream is None:
                self._update_stream = torch.cuda.Stream(device=self.device, priority=-1)
            us = self._update_stream
            if self._native_comm is not None:
                eng = self._ensure_engine()
                _lib.call("nb_gcn_wait_gradients", eng, us.cuda_stream)
                _lib.call_comm("nb_allreduce_sum_f32", self._native_comm, self.P.grad.data_ptr(), self.P.grad.numel(),
                               us.cuda_stream)
                _lib.call("nb_gcn_update", eng, us.cuda_stream)
                return
            with torch.cuda.stream(us):
                _lib.call("nb_gcn_wait_gradients", self._ensure_engine(), us.cuda_stream)
                sum_gradients(self.P.grad, self.world_size)
                _lib.call("nb_gcn_update", self._ensure_engine(), us.cuda_stream)
            return
        sum_gradients(self.P.grad, self.world_size)
        self._apply_adam()

    def _apply_adam(self):
        if self.use_engine:
            _lib.call("nb_gcn_update", self._ensure_engine(), torch.cuda.current_stream().cuda_stream)
        else:
            self.P.learn_with_decay_Adam(torch.cuda.current_stream().cuda_stream)

    def _join_update_stream(self):
        """Later work on the current stream (reading the weights, evaluation) sees the last update."""
        if self._update_stream is not None:
            torch.cuda.current_stream().wait_stream(self._update_stream)

    def UpdateZero(self):
        """A rank that ran out of batches still joins the collective with zeros
        (toolkits/GCN_GPU_NEIGHBOR.hpp:309-313).  The zeroing is ordered after every earlier reader of the
        gradient bucket (the previous step's sum and Adam) and before this step's sum: with the update on a
        stream of its own it runs on that stream, behind the previous update."""
        if self.use_engine and self.overlap_update:
            if self._update_stream is None:
                self._update_stream = torch.cuda.Stream(device=self.device, priority=-1)
            us = self._update_stream
            with torch.cuda.stream(us):
                _lib.call("nb_gcn_wait_gradients", self._ensure_engine(), us.cuda_stream)
                self.P.grad.zero_()
                if self._native_comm is not None:
                    _lib.call_comm("nb_allreduce_sum_f32", self._native_comm, self.P.grad.data_ptr(),
                                   self.P.grad.numel(), us.cuda_stream)
                else:
                    sum_gradients(self.P.grad, self.world_size)
                _lib.call("nb_gcn_update", self._ensure_engine(), us.cuda_stream)
            return
        self.P.grad.zero_()      # same stream as the previous update: stream order is enough
        self.Update()

    def check_device_errors(self):
        """Reads the library's device-side error word (bounded waits that gave up, ids or labels outside their
        tables) and raises if it is set: a step that met one has left rows unwritten or skipped.  Synchronises;
        called at epoch ends, outside timed regions."""
        import ctypes as C
        flags = C.c_uint32(0)
        _lib.call("nb_device_error_flags", C.byref(flags))
        self.device_errors_checked += 1
        if flags.value:
            raise RuntimeError(f"libnb_b200 device error word is {flags.value:#x} (1: copy wait gave up, 2: tensor-core "
                               "wait gave up, 4: vertex id outside every feature table, 8: label outside [0, C))")

    def epoch_steps(self, sampler: Sampler) -> int:
        """Optimizer steps of one epoch of a data-parallel job: the largest batch count over the ranks (one
        scalar MAX-reduce per epoch).  Ranks with fewer batches pad with UpdateZero."""
        n = int(sampler.batch_nums)
        if self.world_size > 1:
            t = torch.tensor([n], dtype=torch.int64, device=self.device)
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            n = int(t.item())
        return n

    def _sum_epoch_stats(self, correct, nodes, loss_sum, batches):
        """correct / nodes / loss / batch count summed over the ranks, as the reference all-reduces its epoch
        statistics (toolkits/GCN_GPU_NEIGHBOR.hpp:785-790)."""
        if self.world_size == 1:
            return correct, nodes, loss_sum, batches
        t = torch.tensor([float(correct), float(nodes), float(loss_sum), float(batches)], dtype=torch.float64,
                         device=self.device)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.SUM)
        c, n, l, b = t.tolist()
        return (c if self.multi_label else int(round(c))), int(round(n)), l, int(round(b))

    def train_step(self, sampler: Sampler):
        if self.use_engine:
            self.engine_step(sampler, train=True)
        else:
            self.forward_backward(sampler.sample_one(), train=True)
        self.Update()
        self.step_count += 1
        self._join_update_stream()

    def _loss_and_score(self, host: torch.Tensor):
        """(loss, hits) of a batch, or with CLASSES > 1 (loss, F1 of the batch) as f1_score computes it
        (utils/torch_func.hpp:31-60)."""
        loss = float(host[0])
        if not self.multi_label:
            return loss, int(host[1])
        true_p, all_pre, all_true = float(host[1]), float(host[2]), float(host[3])
        if true_p == 0 or all_pre == 0:
            return loss, 0.0
        precision, recall = np.float32(true_p) / np.float32(all_pre), np.float32(true_p) / np.float32(all_true)
        return loss, float(np.float32(2) * precision * recall / (precision + recall))

    def read_stats(self):
        """Device -> host read of (loss, hits) — (loss, F1) with CLASSES > 1 — of the last batch; the only
        host sync of a step besides the size read-backs of the block builder."""
        self._stats_host.copy_(self.stats, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self._loss_and_score(self._stats_host)

    def Forward(self, sampler: Sampler, rng: Optional[np.random.RandomState] = None, train: bool = True,
                max_batches: Optional[int] = None):
        """One epoch over the sampler's seeds (Forward + zerocopy_version,
        toolkits/GCN_GPU_NEIGHBOR.hpp:604-800).  Returns (accuracy, mean loss, batches)."""
        if rng is not None:
            sampler.shuffle(rng)
        # the native step samples with the training fan-out and sizes its arenas for the training batch
        native = (self.use_engine and list(sampler.fanout) == list(self.cfg.fanout)
                  and sampler.batch_size <= self.cfg.batch_size
                  and (not train or (sampler.sample_rate, sampler.lower_fanout) == (self.cfg.sample_rate, self.cfg.lower_fanout)))
        # data parallel: every rank takes the same number of optimizer steps (the largest shard's batch count)
        steps = self.epoch_steps(sampler) if (train and self.world_size > 1) else 0
        if max_batches is not None:
            steps = min(steps, max_batches)
        if native and self.cfg.pipelines > 1:
            correct, nodes, loss_epoch, batches = self.run_pipelined(sampler, max_batches, train=train, pad_to_steps=steps)
            sampler.restart()
            self.check_device_errors()
            correct, nodes, loss_epoch, batches = self._sum_epoch_stats(correct, nodes, loss_epoch, batches)
            return self._epoch_accuracy(correct, nodes, batches), loss_epoch / max(batches, 1), batches
        correct = nodes = batches = 0
        loss_epoch = 0.0
        while sampler.sample_not_finished():
            if max_batches is not None and batches >= max_batches:
                break
            if native:
                info = self.engine_step(sampler, train=train)
                batch_nodes = info.v[self.layers - 1]
            else:
                ssg = sampler.sample_one(phase=train)
                self.forward_backward(ssg, train=train)
                batch_nodes = ssg.sampled_sgs[self.layers - 1].v_size
            if train:
                self.Update()
                self.step_count += 1
            loss, hits = self.read_stats()
            loss_epoch += loss
            correct += hits
            nodes += batch_nodes
            batches += 1
        if train:
            self._pad_steps(steps - batches)
        self._join_update_stream()
        sampler.restart()
        self.check_device_errors()
        correct, nodes, loss_epoch, batches = self._sum_epoch_stats(correct, nodes, loss_epoch, batches)
        return self._epoch_accuracy(correct, nodes, batches), loss_epoch / max(batches, 1), batches

    def _epoch_accuracy(self, score_sum, nodes: int, batches: int) -> float:
        """correct / nodes, or the mean of the batches' F1 with CLASSES > 1
        (toolkits/GCN_GPU_NEIGHBOR.hpp:783-793)."""
        if self.multi_label:
            return score_sum / max(batches, 1)
        return score_sum / max(nodes, 1)


def drop_train_ids_by_degree(train_ids: np.ndarray, in_degree: np.ndarray, batch_type: str, del_frac: float) -> np.ndarray:
    """BATCH_TYPE:dellow | delhigh with DEL_FRAC (toolkits/GCN_GPU_NEIGHBOR.hpp:1365-1377): the training ids are
    sorted by in-degree — descending for delhigh, ascending for dellow — and the last DEL_FRAC of that order
    is dropped, so delhigh keeps the high-degree end and dellow the low-degree end, as the reference's code
    does.  Equal degrees are ordered by id (std::sort leaves them unspecified)."""
    if batch_type not in ("dellow", "delhigh"):
        return train_ids
    deg = in_degree[train_ids].astype(np.int64)
    key = -deg if batch_type == "delhigh" else deg
    order = np.lexsort((train_ids.astype(np.int64), key))
    keep = int(len(train_ids) * (1 - del_frac))
    return train_ids[order[:keep]]


def shard_for_rank(ids: np.ndarray, rank: int, world_size: int) -> np.ndarray:
    """Data parallelism over mini-batches: the (already shuffled) train list is dealt round-robin, so
    every id belongs to exactly one rank and shard sizes differ by at most one.  (The reference gives
    each MPI rank the train nodes of its own vertex range, toolkits/GCN_GPU_NEIGHBOR.hpp:1339-1348; with
    a replicated topology any disjoint cover is equivalent.)"""
    return ids[rank::world_size]


def batches_of(n_ids: int, batch_size: int) -> int:
    return (n_ids + batch_size - 1) // batch_size


def epoch_steps(n_ids_total: int, batch_size: int, world_size: int) -> int:
    """Steps every rank takes per epoch: the largest shard's batch count.  Ranks whose shard is
    exhausted earlier still join each step's gradient sum with zeros (UpdateZero,
    toolkits/GCN_GPU_NEIGHBOR.hpp:309-313), so all ranks issue the same number of collectives."""
    largest = (n_ids_total + world_size - 1) // world_size
    return batches_of(largest, batch_size)


def default_stage_misses(cfg: GCNConfig, sharded: bool, feature_on_device: bool, world_size: int) -> bool:
    """Whether the sampling half copies a batch's uncached rows into a staging table.  An explicit setting wins; a
    sharded table is read no other way; a table in host memory is staged when several ranks share that memory and some
    rows are not cached."""
    if cfg.stage_misses is not None:
        return bool(cfg.stage_misses)
    all_cached = cfg.cache_type == "rate" and cfg.cache_rate >= 1.0
    return bool(sharded or (not feature_on_device and world_size > 1 and not all_cached))


def _open_native_comm(rank: int, world_size: int, device):
    """A communicator of libnb_b200_comm.so over the ranks of the default process group: rank 0 draws the NCCL id and
    torch.distributed carries it to the others (what a C++ host does with MPI_Bcast).  None where the library was not
    built."""
    import ctypes as C
    try:
        _lib.load_comm()
    except (ImportError, OSError):
        return None
    uid = torch.zeros(128, dtype=torch.uint8, device=device)
    if rank == 0:
        buf = C.create_string_buffer(128)
        _lib.call_comm("nb_comm_unique_id", buf)
        uid.copy_(torch.frombuffer(bytearray(buf.raw), dtype=torch.uint8))
    torch.distributed.broadcast(uid, src=0)
    comm = C.c_void_p()
    _lib.call_comm("nb_comm_create", C.byref(comm), bytes(uid.cpu().numpy().tobytes()), world_size, rank)
    return comm


def sum_gradients(grad: torch.Tensor, world_size: int):
    """Gradient SUM over ranks (MPI_SUM, comm/network.h:189-193), in place."""
    if world_size > 1:
        torch.distributed.all_reduce(grad, op=torch.distributed.ReduceOp.SUM)
    return grad


def default_workspace_bytes(num_vertices: int, cfg: GCNConfig) -> int:
    """Arena size for the block builder and split-K partials at this configuration's upper bounds."""
    v = cfg.batch_size
    e_max = 0
    for f in cfg.fanout:
        if cfg.sample_rate > 0:   # degree-proportional counts have no fan-out bound: allow for hub-heavy batches
            f = max(f if f > 0 else 64, 4 * cfg.lower_fanout, 64)
        e = v * (f if f > 0 else 64)
        e_max = max(e_max, e)
        v = min(num_vertices, e)
    words = (num_vertices + 31) // 32
    block = 8 * words + 16 * min(num_vertices, e_max) + 8 * e_max
    widest = max(cfg.layers[i] * cfg.layers[i + 1] for i in range(len(cfg.layers) - 1))
    splitk = 4 * widest * 320
    # per-step activations and gradients when a whole step lives in the arena (nb_gcn_step)
    v, acts = cfg.batch_size, 0
    for i, f in enumerate(cfg.fanout):
        layer = len(cfg.fanout) - 1 - i                      # hop i feeds GCN layer L-1-i
        width = max(cfg.layers[layer], cfg.layers[layer + 1])
        acts += 6 * 4 * v * width
        v = min(num_vertices, v * (f if f > 0 else 64))
    acts += 4 * v * ((cfg.layers[0] + 3) // 4 * 4)           # gathered input rows (gather not fused) / staged misses
    return int(block + splitk + acts + (64 << 20))


class GCN_GPU_impl:
    """Full-graph GCN on one GPU, the reference's non-sampled trainer (toolkits/GCN.hpp:140-260 with its single-GPU
    operator, core/ntsSingleGPUFusedGraphOp.hpp:49-70): per layer X_{l+1} = relu(A X_l W_l) with dropout on the
    inputs of layers l >= 1, last layer without relu, mean NLL of log_softmax over the TRAIN vertices, Adam with weight
    decay.  Like NtsContext::self_backward the first graph operator is not back-propagated.  Every kernel is from
    libnb_b200; the aggregation forms 1 / (sqrt(out_deg[src]) * sqrt(in_deg[dst])) from the whole graph's degrees."""

    def __init__(self, partitioned_graph, datum: GNNDatum, cfg: GCNConfig, ws: Optional[Workspace] = None):
        self.pg, self.datum, self.cfg = partitioned_graph, datum, cfg
        self.device = partitioned_graph.graph.device
        self.layers = len(cfg.layers) - 1
        V = partitioned_graph.vertices
        assert datum.local_feature.is_cuda and datum.local_feature.size(0) == V
        widest = max(cfg.layers)
        self.ws = ws if ws is not None else Workspace(int(4 * V * widest * 2 + 4 * max(cfg.layers[i] * cfg.layers[i + 1]
                                                          for i in range(self.layers)) * 640 + (64 << 20)))
        self.P = Parameter(cfg.layers, cfg, self.device, torch.Generator().manual_seed(cfg.seed))
        self.step_count = 0
        self.stats = torch.zeros(4, dtype=torch.float32, device=self.device)
        mask = np.asarray(datum.local_mask)
        self.ids = [torch.from_numpy(np.nonzero(mask == k)[0].astype(np.int32)).to(self.device) for k in (0, 1, 2)]
        # position of every train vertex inside the train list, for scattering the loss gradient back to full rows
        pos = np.zeros(V, dtype=np.int32)
        train = np.nonzero(mask == 0)[0]
        pos[train] = np.arange(len(train), dtype=np.int32)
        self.train_pos = torch.from_numpy(pos).to(self.device)
        self.agg_edges_fwd = self.agg_edges_bwd = 0

    def _buf(self, rows, cols):
        return torch.empty((max(int(rows), 1), int(cols)), dtype=torch.float32, device=self.device)

    def _loss_on(self, logits: torch.Tensor, ids: torch.Tensor, dlogits_full: Optional[torch.Tensor]):
        """Mean NLL and hits over the vertices `ids`; with dlogits_full the gradient rows are written there (other
        rows of it must already be zero)."""
        stream = torch.cuda.current_stream().cuda_stream
        n, C = int(ids.numel()), logits.size(1)
        rows = self._buf(n, C)
        _lib.call("nb_feature_gather", ptr(rows), ptr(logits), C, None, 0, 0, None, 0, None, ptr(ids), n, C, stream)
        lab = torch.empty(max(n, 1), dtype=torch.int64, device=self.device)
        _lib.call("nb_label_gather", ptr(lab), ptr(self.datum.local_label), ptr(ids), n, 1, stream)
        drows = self._buf(n, C) if dlogits_full is not None else None
        _lib.call("nb_softmax_nll", self.ws.handle, ptr(rows), ptr(lab), n, C, ptr(drows), ptr(self.stats), stream)
        if dlogits_full is not None:
            _lib.call("nb_feature_gather_indexed", ptr(dlogits_full), C, ptr(drows), C, ptr(self.train_pos), ptr(ids),
                      None, n, C, stream)

    def epoch(self, train: bool = True):
        """One full-graph step (Forward, Loss, self_backward, Update of toolkits/GCN.hpp).  Returns the logits."""
        c, L, pg = self.cfg, self.layers, self.pg
        V = pg.vertices
        stream = torch.cuda.current_stream().cuda_stream
        wsh = self.ws.handle
        p = c.drop_rate if train else 0.0
        scale = 1.0 / (1.0 - p) if p > 0 else 1.0
        X = [self.datum.local_feature]
        Y = []
        for l in range(L):
            Fi, Fo = c.layers[l], c.layers[l + 1]
            y = self._buf(V, Fi)
            _lib.call("nb_spmm_csc_fwd_fused", ptr(X[l]), ptr(y), ptr(pg.row_indices), ptr(pg.column_offset),
                      ptr(pg.src_norm), ptr(pg.dst_norm), V, Fi, stream)
            Y.append(y)
            z = self._buf(V, Fo)
            _lib.call("nb_gemm", wsh, ptr(y), ptr(self.P.w(l)), ptr(z), V, Fo, Fi, 0, 0, stream)
            if l < L - 1:   # relu, then the dropout that the next layer applies to its input
                _lib.call("nb_relu_dropout", ptr(z), V * Fo, p, c.seed, l, self.step_count, stream)
            X.append(z)
        self.agg_edges_fwd += L * pg.edges
        if not train:
            return X[L]
        C = c.layers[L]
        dZ = torch.zeros((V, C), dtype=torch.float32, device=self.device)
        self._loss_on(X[L], self.ids[0], dZ)
        for l in range(L - 1, -1, -1):
            Fi, Fo = c.layers[l], c.layers[l + 1]
            _lib.call("nb_gemm", wsh, ptr(Y[l]), ptr(dZ), ptr(self.P.g(l)), Fi, Fo, V, 1, 0, stream)
            if l == 0:
                break   # the first graph operator is not back-propagated (core/ntsContext.hpp:292)
            dY = self._buf(V, Fi)
            _lib.call("nb_gemm", wsh, ptr(dZ), ptr(self.P.w(l)), ptr(dY), V, Fi, Fo, 0, 1, stream)
            dX = self._buf(V, Fi)
            _lib.call("nb_spmm_csr_bwd_fused", ptr(dY), ptr(dX), ptr(pg.row_offset), ptr(pg.column_indices),
                      ptr(pg.src_norm), ptr(pg.dst_norm), ptr(X[l]), scale, V, Fi, stream)
            self.agg_edges_bwd += pg.edges
            dZ = dX
        self.P.learn_with_decay_Adam(stream)
        self.step_count += 1
        return X[L]

    def read_stats(self):
        host = self.stats.cpu()
        return float(host[0]), int(host[1])

    def Test(self, which: int, logits: torch.Tensor) -> float:
        """Accuracy over the vertices of one split (0 train, 1 val, 2 test)."""
        ids = self.ids[which]
        if ids.numel() == 0:
            return 0.0
        self._loss_on(logits, ids, None)
        return self.read_stats()[1] / int(ids.numel())
