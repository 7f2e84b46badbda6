"""Device-resident mirrors of the reference's graph containers and sampler.

Names follow the reference: ``FullyRepGraph`` (core/FullyRepGraph.hpp:406-561), ``sampCSC``
(core/coocsc.hpp:27-831), ``SampledSubgraph`` (core/FullyRepGraph.hpp:30-405) and ``Sampler``
(core/ntsSampler.hpp:29-1519).  All block arrays live in HBM and are produced by kernels of
libnb_b200.so; the host only sees sizes.  Index arrays are stored as torch.int32 tensors that carry
the reference's uint32 bit patterns.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import numpy as np
import torch

from . import _lib
from .cuda_stream import Cuda_Stream, Workspace, ptr


def _i32(n, device):
    return torch.empty(int(n), dtype=torch.int32, device=device)


def _f32(n, device):
    return torch.empty(int(n), dtype=torch.float32, device=device)


class FullyRepGraph:
    """Whole-graph CSC by destination, replicated on the GPU (core/FullyRepGraph.hpp:406-451).

    column_offset is int64 on the device (the reference keeps uint32 and truncates the edge count,
    core/FullyRepGraph.hpp:417,434); row_indices is int32.
    """

    def __init__(self, column_offset: torch.Tensor, row_indices: torch.Tensor, vertices: int,
                 out_degree: Optional[torch.Tensor] = None, in_degree: Optional[torch.Tensor] = None):
        assert column_offset.dtype == torch.int64 and row_indices.dtype == torch.int32
        self.column_offset = column_offset
        self.row_indices = row_indices
        self.global_vertices = int(vertices)
        self.global_edges = int(row_indices.numel())
        self.out_degree = out_degree
        self.in_degree = in_degree
        self.device = column_offset.device

    @classmethod
    def from_edges(cls, edges: torch.Tensor, vertices: int, ws: Workspace) -> "FullyRepGraph":
        """ReadRepGraphFromRawFile (core/FullyRepGraph.hpp:485-560) on the device.  ``edges`` is an
        int32 tensor [E, 2] of (src, dst) pairs in file order, already on the GPU."""
        assert edges.dtype == torch.int32 and edges.dim() == 2 and edges.size(1) == 2 and edges.is_cuda
        edges = edges.contiguous()
        E = edges.size(0)
        dev = edges.device
        co = torch.empty(vertices + 1, dtype=torch.int64, device=dev)
        ri = _i32(E, dev)
        out_deg = _i32(vertices, dev)
        in_deg = _i32(vertices, dev)
        _lib.call("nb_graph_build_csc", ws.handle, ptr(edges), E, vertices, ptr(co), ptr(ri), ptr(out_deg),
                  ptr(in_deg), torch.cuda.current_stream().cuda_stream)
        return cls(co, ri, vertices, out_deg, in_deg)

    @classmethod
    def from_edge_file(cls, path: str, vertices: int, ws: Workspace, device="cuda") -> "FullyRepGraph":
        """Reads the reference's binary .edge format: little-endian (u32 src, u32 dst) pairs, edge count
        = file size / 8 (core/graph.hpp:1059-1060)."""
        raw = np.fromfile(path, dtype="<u4").reshape(-1, 2)
        edges = torch.from_numpy(raw.view(np.int32)).to(device)
        return cls.from_edges(edges, vertices, ws)


class sampCSC:
    """One sampled block (core/coocsc.hpp:792-813).  Arrays may be longer than the logical sizes."""

    def __init__(self):
        self.v_size = 0
        self.e_size = 0
        self.src_size = 0
        self.destination = None       # [v]   global ids of outputs
        self.source = None            # [s]   distinct global ids of inputs, ascending
        self.column_offset = None     # [v+1] CSC by destination
        self.row_indices = None       # [e]   local source ranks
        self.row_offset = None        # [s+1] CSR by source
        self.column_indices = None    # [e]   local destinations, ascending inside a row
        self.edge_weight_forward = None   # [e] CSC order
        self.edge_weight_backward = None  # [e] CSR order
        self.src_norm = None          # [s] (float)sqrt(out degree in the block)
        self.dst_norm = None          # [v] (float)sqrt(in degree in the block)

    # accessors named like the reference's (core/coocsc.hpp:532-555)
    def dst(self):
        return self.destination[: self.v_size]

    def src(self):
        return self.source[: self.src_size]

    def c_o(self):
        return self.column_offset[: self.v_size + 1]

    def r_i(self):
        return self.row_indices[: self.e_size]

    def r_o(self):
        return self.row_offset[: self.src_size + 1]

    def c_i(self):
        return self.column_indices[: self.e_size]

    def dev_ewf(self):
        return self.edge_weight_forward

    def dev_ewb(self):
        return self.edge_weight_backward


def build_block(ws: Workspace, num_vertices: int, destination: torch.Tensor, column_offset: torch.Tensor,
                row_indices_global: torch.Tensor, v: int, e: int, with_edge_weights: bool = True,
                stream: Optional[int] = None) -> sampCSC:
    """nb_block_build on one hop's raw edge list (global source ids in CSC order).  row_indices_global
    is overwritten with local ranks (like sampCSC::postprocessing does, core/coocsc.hpp:417-424)."""
    dev = column_offset.device
    cap = max(1, min(num_vertices, e))
    blk = sampCSC()
    blk.v_size, blk.e_size = int(v), int(e)
    blk.destination = destination
    blk.column_offset = column_offset
    blk.row_indices = row_indices_global
    blk.source = _i32(cap, dev)
    blk.row_offset = _i32(cap + 1, dev)
    blk.column_indices = _i32(max(e, 1), dev)
    blk.src_norm = _f32(cap, dev)
    blk.dst_norm = _f32(max(v, 1), dev)
    if with_edge_weights:
        blk.edge_weight_forward = _f32(max(e, 1), dev)
        blk.edge_weight_backward = _f32(max(e, 1), dev)
    s = C.c_uint32(0)
    _lib.call("nb_block_build", ws.handle, num_vertices, ptr(row_indices_global), ptr(column_offset), v, e,
              ptr(blk.source), C.byref(s), ptr(blk.row_offset), ptr(blk.column_indices), ptr(blk.src_norm),
              ptr(blk.dst_norm), ptr(blk.edge_weight_forward), ptr(blk.edge_weight_backward),
              torch.cuda.current_stream().cuda_stream if stream is None else stream)
    blk.src_size = int(s.value)
    return blk


class SampledSubgraph:
    """Per-batch list of blocks; index 0 is the input-side block after sample_one
    (core/ntsSampler.hpp:1088)."""

    def __init__(self, layers: int, fanout: Sequence[int]):
        self.layers = int(layers)
        self.fanout = list(fanout)
        self.sampled_sgs: List[sampCSC] = []

    def update_fanout(self, fanout):
        if isinstance(fanout, int):
            self.fanout = [fanout] * len(self.fanout)
        else:
            assert len(fanout) == len(self.fanout)
            self.fanout = list(fanout)


class Sampler:
    """Fan-out neighbour sampler over a FullyRepGraph (core/ntsSampler.hpp:29-1106), on the GPU.

    ``fanout`` is in hop order (seeds first) — the order the reference holds after reversing the cfg
    list (toolkits/GCN_GPU_NEIGHBOR.hpp:126-130).
    """

    def __init__(self, whole_graph: FullyRepGraph, index: Sequence[int], fanout: Sequence[int], batch_size: int,
                 ws: Workspace, full_batch: bool = False, seed: int = 2000, with_edge_weights: bool = True,
                 sample_rate: float = 0.0, lower_fanout: int = 0):
        self.whole_graph = whole_graph
        # SAMPLE_RATE > 0: the training sampler takes max(int(deg * rate), min(lower_fanout, deg)) neighbours
        # per destination instead of min(deg, fanout) (core/ntsSampler.hpp:901-912)
        self.sample_rate = float(sample_rate)
        self.lower_fanout = int(lower_fanout)
        # BATCH_TYPE:random — every training batch is a fresh uniform subset of the seed list instead of
        # the next slice of it (sampCSC::random_batch, core/coocsc.hpp:488-499)
        self.random_batches = False
        self._batch_rng = np.random.RandomState(int(seed))
        self.sample_nids = np.asarray(index, dtype=np.uint32).copy()
        self.fanout = list(fanout)
        self.layers = len(self.fanout)
        self.full_batch = full_batch
        self.work_range = [0, len(self.sample_nids)]
        self.work_offset = 0
        self.ws = ws
        self.seed = int(seed)
        self.draws = 0  # number of sample_one calls so far; part of the Philox key
        self.with_edge_weights = with_edge_weights
        self.subgraph = SampledSubgraph(self.layers, self.fanout)
        self.cs = Cuda_Stream()
        self.update_batch_size(batch_size)
        self._pinned_seeds = None
        self._dev_nids = None

    # core/ntsSampler.hpp:259-265
    def update_batch_size(self, batch_size: int):
        self.batch_size = int(batch_size)
        if self.work_range[1] < self.batch_size or self.full_batch:
            self.batch_size = self.work_range[1]
        self.batch_nums = (self.work_range[1] + self.batch_size - 1) // self.batch_size if self.batch_size else 0

    def update_fanout(self, fanout):
        self.fanout = [fanout] * self.layers if isinstance(fanout, int) else list(fanout)
        self.subgraph.update_fanout(self.fanout)

    def sample_not_finished(self) -> bool:
        return self.work_offset < self.work_range[1]

    def restart(self):
        self.work_offset = self.work_range[0]

    def shuffle(self, rng: np.random.RandomState):
        """Per-epoch reshuffle of the seed list (toolkits/GCN_GPU_NEIGHBOR.hpp:742-745)."""
        rng.shuffle(self.sample_nids)
        self._dev_nids = None

    def stage_seeds_on_device(self):
        """Upload the whole (shuffled) seed list once; later batches slice it on the device instead of
        copying their seeds from pinned host memory every step."""
        self._dev_nids = torch.from_numpy(self.sample_nids.view(np.int32).copy()).to(self.whole_graph.device)

    def unstage_seeds(self):
        self._dev_nids = None

    def get_compute_cnt(self) -> int:
        """Sum of e_size over the blocks (core/ntsSampler.hpp:629-635)."""
        return sum(b.e_size for b in self.subgraph.sampled_sgs)

    def _seeds_to_device(self, seeds: np.ndarray) -> torch.Tensor:
        n = len(seeds)
        if self._pinned_seeds is None or self._pinned_seeds.numel() < n:
            self._pinned_seeds = torch.empty(max(n, self.batch_size), dtype=torch.int32).pin_memory()
        self._pinned_seeds[:n].copy_(torch.from_numpy(seeds.view(np.int32)))
        return self._pinned_seeds[:n].to(self.whole_graph.device, non_blocking=True)

    def _next_seed_ids(self):
        """Host view of the next batch's seeds (None when they are a slice of the staged device list);
        advances work_offset (the last batch of an epoch is short, core/ntsSampler.hpp:846)."""
        assert self.work_offset < self.work_range[1]
        actl = min(self.batch_size, self.work_range[1] - self.work_offset)
        lo = self.work_offset
        self.work_offset += actl
        if self.random_batches:
            pick = self._batch_rng.choice(len(self.sample_nids), size=actl, replace=False)
            return self.sample_nids[pick], lo, actl
        if self._dev_nids is not None:
            return None, lo, actl
        return self.sample_nids[lo: lo + actl], lo, actl

    def next_seeds(self):
        """Seeds of the next batch as a device tensor, and their number."""
        host, lo, actl = self._next_seed_ids()
        if host is None:
            return self._dev_nids[lo: lo + actl], actl
        return self._seeds_to_device(host), actl

    def next_seeds_into(self, pinned: torch.Tensor):
        """Like next_seeds, for a caller that hands the seeds to a library thread: a slice of the staged
        device list, or (host seeds) a copy in the caller's pinned int32 buffer, which the library reads
        itself.  Returns (tensor whose data_ptr() holds the seeds, count)."""
        host, lo, actl = self._next_seed_ids()
        if host is None:
            return self._dev_nids[lo: lo + actl], actl
        pinned[:actl].copy_(torch.from_numpy(np.ascontiguousarray(host).view(np.int32)))
        return pinned[:actl], actl

    def sample_one(self, ssg: Optional[SampledSubgraph] = None, raw_edges: Optional[list] = None,
                   phase: bool = True) -> SampledSubgraph:
        """One batch: per hop, column offsets, sampling, dedup/reindex, CSR, weights
        (core/ntsSampler.hpp:843-1106).  ``raw_edges`` (list per hop of device int32 tensors of global
        source ids laid out by the hop's column offsets) replaces the Philox sampler with an externally
        supplied edge list — the form in which parity with the reference is defined."""
        ssg = self.subgraph if ssg is None else ssg
        dst, actl = self.next_seeds()
        g = self.whole_graph
        stream = torch.cuda.current_stream().cuda_stream
        v = actl
        blocks = []
        for hop in range(self.layers):
            co = _i32(v + 1, g.device)
            e = C.c_uint32(0)
            by_rate = phase and self.sample_rate > 0
            if by_rate:
                _lib.call("nb_sample_hop_offsets_rate", self.ws.handle, ptr(g.column_offset), ptr(dst), v,
                          self.sample_rate, self.lower_fanout, ptr(co), C.byref(e), stream)
            else:
                _lib.call("nb_sample_hop_offsets", self.ws.handle, ptr(g.column_offset), ptr(dst), v,
                          int(self.fanout[hop]), ptr(co), C.byref(e), stream)
            e = int(e.value)
            if raw_edges is not None:
                ri = raw_edges[hop].clone()
                assert ri.numel() == e, "supplied edge list does not match the hop's column offsets"
            else:
                ri = _i32(max(e, 1), g.device)
                hop_key = (self.draws << 8) | hop
                _lib.call("nb_sample_hop", ptr(g.column_offset), ptr(g.row_indices), ptr(dst), v,
                          -1 if by_rate else int(self.fanout[hop]), ptr(co), self.seed, hop_key, ptr(ri), stream)
            blk = build_block(self.ws, g.global_vertices, dst, co, ri, v, e, self.with_edge_weights, stream)
            blocks.append(blk)
            dst = blk.source
            v = blk.src_size
        self.draws += 1
        blocks.reverse()  # index 0 = input-side block (core/ntsSampler.hpp:1088)
        ssg.sampled_sgs = blocks
        return ssg

    # -- feature / label loading (core/ntsSampler.hpp:364-376, 424-469, 501-529)
    def load_feature_gpu(self, cuda_stream: Cuda_Stream, ssg: SampledSubgraph, local_feature: torch.Tensor,
                         global_feature: torch.Tensor) -> torch.Tensor:
        blk = ssg.sampled_sgs[0]
        if local_feature.size(0) < blk.src_size:
            local_feature.resize_(blk.src_size, local_feature.size(1))
        cuda_stream.zero_copy_feature_move_gpu(ptr(local_feature), ptr(global_feature), ptr(blk.source),
                                               local_feature.size(1), blk.src_size)
        return local_feature

    def load_feature_gpu_cache(self, cuda_stream: Cuda_Stream, ssg: SampledSubgraph, local_feature: torch.Tensor,
                               global_feature: Optional[torch.Tensor], dev_cache_feature: torch.Tensor,
                               dev_cache_node_hashmap: torch.Tensor) -> torch.Tensor:
        blk = ssg.sampled_sgs[0]
        if local_feature.size(0) < blk.src_size:
            local_feature.resize_(blk.src_size, local_feature.size(1))
        cuda_stream.gather_feature_cached(ptr(local_feature), ptr(global_feature), ptr(dev_cache_feature),
                                          ptr(blk.source), local_feature.size(1), blk.src_size,
                                          ptr(dev_cache_node_hashmap), dev_cache_feature.stride(0))
        return local_feature

    def load_label_gpu(self, cuda_stream: Cuda_Stream, ssg: SampledSubgraph, local_label: torch.Tensor,
                       global_label: torch.Tensor, classes: int = 1) -> torch.Tensor:
        blk = ssg.sampled_sgs[self.layers - 1]
        if classes > 1:
            if local_label.dim() != 2 or local_label.size(0) != blk.v_size or local_label.size(1) != classes:
                local_label.resize_(blk.v_size, classes)
            cuda_stream.global_copy_mulilabel_move_gpu(ptr(local_label), ptr(global_label), ptr(blk.destination),
                                                       blk.v_size, classes)
        else:
            if local_label.size(0) != blk.v_size:
                local_label.resize_(blk.v_size)
            cuda_stream.global_copy_label_move_gpu(ptr(local_label), ptr(global_label), ptr(blk.destination),
                                                   blk.v_size)
        return local_label


class PartitionedGraph:
    """The whole graph as one chunk with precomputed GCN edge weights — what the reference's full-graph operators
    read (PartitionedGraph::graph_chunks of CSC_segment_pinned, core/PartitionedGraph.hpp; the weights are
    nts_norm_degree = 1 / ((float)sqrt(out_degree[src]) * (float)sqrt(in_degree[dst])) over the WHOLE graph's
    degrees, clamped to at least 1 as generate_backward_structure does, core/ntsBaseOp.hpp:183-186,
    core/graph.hpp:3983-3986).  Holds the CSC by destination with `edge_weight_forward` in CSC order and its
    transpose (CSR by source, ascending destinations inside a row) with `edge_weight_backward` in CSR order."""

    def __init__(self, graph: FullyRepGraph, ws: Workspace):
        dev = graph.device
        V, E = graph.global_vertices, graph.global_edges
        assert E < 2 ** 32, "block-local offsets are 32-bit"
        self.graph = graph
        self.vertices, self.edges = V, E
        co64 = graph.column_offset
        self.column_offset = co64.to(torch.int32)          # uint32 bit patterns
        self.row_indices = graph.row_indices
        in_deg = (co64[1:] - co64[:-1])
        # transpose: the CSC of the reversed pairs, built by the same kernel (stable in CSC order, hence ascending
        # destinations inside every source's row)
        dst = torch.repeat_interleave(torch.arange(V, device=dev, dtype=torch.int32), in_deg)
        pairs = torch.stack([dst, graph.row_indices], dim=1).contiguous()     # (dst, src): "source" column is dst
        ro64 = torch.empty(V + 1, dtype=torch.int64, device=dev)
        self.column_indices = _i32(max(E, 1), dev)
        _lib.call("nb_graph_build_csc", ws.handle, ptr(pairs), E, V, ptr(ro64), ptr(self.column_indices), None, None,
                  torch.cuda.current_stream().cuda_stream)
        self.row_offset = ro64.to(torch.int32)
        out_deg = (ro64[1:] - ro64[:-1])
        # one-time host work, in the reference's arithmetic: sqrt in double rounded to float, float product, 1/x
        ind = np.maximum(in_deg.cpu().numpy(), 1).astype(np.float64)
        outd = np.maximum(out_deg.cpu().numpy(), 1).astype(np.float64)
        s_in, s_out = np.sqrt(ind).astype(np.float32), np.sqrt(outd).astype(np.float32)
        ri = graph.row_indices.cpu().numpy().view(np.uint32)
        ci = self.column_indices.cpu().numpy().view(np.uint32)[:E]
        dst_h = dst.cpu().numpy()
        src_of_row = np.repeat(np.arange(V, dtype=np.int64), out_deg.cpu().numpy())
        one = np.float32(1.0)
        self.edge_weight_forward = torch.from_numpy(one / (s_out[ri] * s_in[dst_h])).to(dev)
        self.edge_weight_backward = torch.from_numpy(one / (s_out[src_of_row] * s_in[ci])).to(dev)
        # the two factors per vertex, for the aggregation entry points that form the weight per edge themselves
        self.src_norm = torch.from_numpy(s_out).to(dev)
        self.dst_norm = torch.from_numpy(s_in).to(dev)
        self.in_degree, self.out_degree = in_deg, out_deg
        del pairs, dst
