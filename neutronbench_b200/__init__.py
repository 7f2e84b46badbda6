"""B200-native sampled mini-batch GCN path of NeutronBench (ALGORITHM:GCNNEIGHBORGPU).

The compute path is libnb_b200.so (hand-written sm_100a CUDA behind a C ABI, include/nb_b200.h);
this package is the host-side mirror of the reference's operator/toolkit interface.  Importing the
package does not load the library; the first call does, and fails loudly when it is missing.
"""
from . import _lib  # noqa: F401
from .cuda_stream import Cuda_Stream, Workspace  # noqa: F401
from .graph import FullyRepGraph, PartitionedGraph, SampledSubgraph, Sampler, build_block, sampCSC  # noqa: F401
from .ops import ForwardSingleGPUfuseOp, SingleGPUSampleGraphOp, ntsGraphOp  # noqa: F401
from .toolkit import (GCN_GPU_impl, GCN_GPU_NEIGHBOR_impl, GCNConfig, GNNDatum, Parameter, cache_nodes_for_memory,  # noqa: F401
                      cache_slots_by_degree, cache_slots_by_sample_count, cache_slots_random,
                      drop_train_ids_by_degree)

__all__ = [
    "Cuda_Stream", "Workspace", "FullyRepGraph", "SampledSubgraph", "Sampler", "build_block", "sampCSC",
    "SingleGPUSampleGraphOp", "ForwardSingleGPUfuseOp", "PartitionedGraph", "ntsGraphOp", "GCN_GPU_NEIGHBOR_impl", "GCN_GPU_impl", "GCNConfig", "GNNDatum", "Parameter",
    "cache_slots_by_degree", "cache_slots_by_sample_count", "cache_slots_random", "cache_nodes_for_memory", "drop_train_ids_by_degree",
]
