"""Graph operators with the reference's surface (core/ntsBaseOp.hpp:25-48).

``SingleGPUSampleGraphOp`` keeps the constructor arguments and the forward/backward meaning of the
reference class (core/ntsMiniBatchGraphOp.hpp:248-376): forward aggregates X[s x F] of block ``layer``
into a new tensor Y[v x F]; backward maps dY[v x F] to dX[s x F] through the block's CSR.  Tensors are
contiguous fp32 CUDA tensors; the row count comes from the block, never from the tensor (the
reference's X[0] may have more rows than src_size, core/ntsSampler.hpp:369-371).
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from .cuda_stream import Cuda_Stream, ptr
from .graph import SampledSubgraph


class ntsGraphOp:
    """Operator surface (core/ntsBaseOp.hpp:25-48)."""

    def __init__(self, graph=None):
        self.graph_ = graph

    def forward(self, f_input: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def backward(self, output_grad: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class SingleGPUSampleGraphOp(ntsGraphOp):
    def __init__(self, subgraphs: SampledSubgraph, graph=None, layer: int = 0, cs: Optional[Cuda_Stream] = None,
                 fused_weights: bool = False):
        super().__init__(graph)
        self.subgraphs = subgraphs
        self.layer = layer
        self.cuda_stream = cs if cs is not None else Cuda_Stream()
        self.fused_weights = fused_weights

    def forward(self, f_input: torch.Tensor) -> torch.Tensor:
        blk = self.subgraphs.sampled_sgs[self.layer]
        assert f_input.is_cuda and f_input.dtype == torch.float32 and f_input.is_contiguous()
        assert f_input.size(0) >= blk.src_size
        F = f_input.size(1)
        # NewKeyTensor: a new leaf that requires grad (core/NtsScheduler.hpp:351-361); every row is
        # written by the kernel, so no zero fill is needed.
        f_output = torch.empty((blk.v_size, F), dtype=torch.float32, device=f_input.device)
        if self.fused_weights:
            _lib.call("nb_spmm_csc_fwd_fused", ptr(f_input), ptr(f_output), ptr(blk.row_indices),
                      ptr(blk.column_offset), ptr(blk.src_norm), ptr(blk.dst_norm), blk.v_size, F,
                      self.cuda_stream.getStream())
        else:
            self.cuda_stream.Gather_By_Dst_From_Src(ptr(f_input), ptr(f_output), ptr(blk.dev_ewf()),
                                                    ptr(blk.row_indices), ptr(blk.column_offset), 0, 0, 0, 0,
                                                    blk.e_size, blk.v_size, F, True, False)
        return f_output.requires_grad_(True)

    def backward(self, f_output_grad: torch.Tensor) -> torch.Tensor:
        blk = self.subgraphs.sampled_sgs[self.layer]
        assert f_output_grad.is_cuda and f_output_grad.dtype == torch.float32 and f_output_grad.is_contiguous()
        assert f_output_grad.size(0) >= blk.v_size
        F = f_output_grad.size(1)
        f_input_grad = torch.empty((blk.src_size, F), dtype=torch.float32, device=f_output_grad.device)
        if self.fused_weights:
            _lib.call("nb_spmm_csr_bwd_fused", ptr(f_output_grad), ptr(f_input_grad), ptr(blk.row_offset),
                      ptr(blk.column_indices), ptr(blk.src_norm), ptr(blk.dst_norm), None, 1.0, blk.src_size, F,
                      self.cuda_stream.getStream())
        else:
            self.cuda_stream.Gather_By_Src_From_Dst(ptr(f_output_grad), ptr(f_input_grad), ptr(blk.dev_ewb()),
                                                    ptr(blk.row_offset), ptr(blk.column_indices), 0, 0, 0, 0,
                                                    blk.e_size, blk.src_size, F, True, False)
        return f_input_grad


class ForwardSingleGPUfuseOp(ntsGraphOp):
    """The full-graph GCN aggregation on one GPU (core/ntsSingleGPUFusedGraphOp.hpp:49-70 ->
    Graph::forward_single / backward_single, core/graph.hpp:3432-3478 -> GatherByDstFromSrc / GatherBySrcFromDst,
    core/NtsScheduler.hpp:146-178, 239-271): the same two aggregation entry points as the sampled operator, with
    v = s = |V| and the whole-graph edge weights of a PartitionedGraph.  forward returns a new leaf that requires
    grad, like NewKeyTensor; backward maps dY to dX through the transposed structure."""

    def __init__(self, partitioned_graph, active=None, cs: Optional[Cuda_Stream] = None):
        super().__init__(partitioned_graph)
        self.active_ = active
        self.cuda_stream = cs if cs is not None else Cuda_Stream()

    def forward(self, f_input: torch.Tensor) -> torch.Tensor:
        pg = self.graph_
        assert f_input.is_cuda and f_input.dtype == torch.float32 and f_input.is_contiguous()
        assert f_input.size(0) == pg.vertices
        F = f_input.size(1)
        f_output = torch.empty((pg.vertices, F), dtype=torch.float32, device=f_input.device)
        self.cuda_stream.Gather_By_Dst_From_Src(ptr(f_input), ptr(f_output), ptr(pg.edge_weight_forward),
                                                ptr(pg.row_indices), ptr(pg.column_offset), 0, pg.vertices, 0,
                                                pg.vertices, pg.edges, pg.vertices, F, True, False)
        return f_output.requires_grad_(True)

    def backward(self, f_output_grad: torch.Tensor) -> torch.Tensor:
        pg = self.graph_
        assert f_output_grad.is_cuda and f_output_grad.dtype == torch.float32 and f_output_grad.is_contiguous()
        F = f_output_grad.size(1)
        f_input_grad = torch.empty((pg.vertices, F), dtype=torch.float32, device=f_output_grad.device)
        self.cuda_stream.Gather_By_Src_From_Dst(ptr(f_output_grad), ptr(f_input_grad), ptr(pg.edge_weight_backward),
                                                ptr(pg.row_offset), ptr(pg.column_indices), 0, pg.vertices, 0,
                                                pg.vertices, pg.edges, pg.vertices, F, True, False)
        return f_input_grad
