"""Host-side mirror of the reference's CUDA boundary: ``Cuda_Stream`` and the workspace.

``Cuda_Stream`` keeps the method names and argument meaning of the reference class
(cuda/ntsCUDA.hpp:99-211) for the calls on the sampled mini-batch GCN path, and forwards each to the
C ABI of libnb_b200.so.  Arguments are raw device addresses (``tensor.data_ptr()``) exactly like the
reference passes raw pointers.  Unlike the reference the calls do not synchronise the stream
(cuda/ntsCUDAGraphOP.cu:366-373 does after every kernel); ``CUDA_DEVICE_SYNCHRONIZE`` is there for
callers that want the reference's blocking behaviour.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib


def _stream_handle(stream) -> int:
    if stream is None:
        return torch.cuda.current_stream().cuda_stream
    if isinstance(stream, int):
        return stream
    return stream.cuda_stream


def ptr(t) -> int:
    """Device (or mapped host) address of a tensor, 0 for None."""
    return 0 if t is None else t.data_ptr()


class Workspace:
    """Scratch arena for the block builder, scans and split-K partials (nb_ws).

    The arena is a torch uint8 tensor so that device memory stays under torch's allocator; the library
    sub-allocates from it and never frees it.
    """

    def __init__(self, nbytes: int, device=None):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.arena = torch.empty(int(nbytes), dtype=torch.uint8, device=self.device)
        handle = C.c_void_p()
        _lib.call("nb_ws_create", C.byref(handle), self.arena.data_ptr(), int(nbytes))
        self.handle = handle

    def high_water(self) -> int:
        return int(_lib.load().nb_ws_high_water(self.handle))

    def close(self):
        if self.handle:
            _lib.load().nb_ws_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Cuda_Stream:
    """Forwarders with the reference's names (cuda/ntsCUDA.hpp:99-211)."""

    def __init__(self, stream=None):
        self.stream = stream

    # -- stream management (cuda/ntsCUDAGraphOP.cu:340-373)
    def getStream(self):
        return _stream_handle(self.stream)

    def setNewStream(self, stream):
        self.stream = stream

    def CUDA_DEVICE_SYNCHRONIZE(self):
        if self.stream is None or isinstance(self.stream, int):
            torch.cuda.current_stream().synchronize()
        else:
            self.stream.synchronize()

    # -- aggregation (cuda/ntsCUDA.hpp:131-150)
    def Gather_By_Dst_From_Src(self, input, output, weight_forward, row_indices, column_offset, src_start, src_end,
                               dst_start, dst_end, edges, batch_size, feature_size, with_weight=False,
                               tensor_weight=False):
        if not with_weight or tensor_weight:
            raise NotImplementedError("only the scalar-weight variant is on the sampled GCN path")
        if src_start or dst_start:
            raise ValueError("the sampled path always passes 0 offsets (core/ntsMiniBatchGraphOp.hpp:311-313)")
        _lib.call("nb_spmm_csc_fwd", input, output, weight_forward, row_indices, column_offset, batch_size,
                  feature_size, self.getStream())

    def Gather_By_Src_From_Dst(self, input, output, weight_backward, row_offset, column_indices, src_start, src_end,
                               dst_start, dst_end, edges, batch_size, feature_size, with_weight=False,
                               tensor_weight=False):
        if not with_weight or tensor_weight:
            raise NotImplementedError("only the scalar-weight variant is on the sampled GCN path")
        if src_start or dst_start:
            raise ValueError("the sampled path always passes 0 offsets (core/ntsMiniBatchGraphOp.hpp:365-368)")
        _lib.call("nb_spmm_csr_bwd", input, output, weight_backward, row_offset, column_indices, batch_size,
                  feature_size, self.getStream())

    # -- feature / label movement (cuda/ntsCUDA.hpp:190-203)
    def zero_copy_feature_move_gpu(self, dev_feature, pinned_host_feature, src_vertex, feature_size, vertex_size):
        _lib.call("nb_feature_gather", dev_feature, pinned_host_feature, feature_size, None, 0, 0, None, 0, None,
                  src_vertex, vertex_size, feature_size, self.getStream())

    def gather_feature_cached(self, dev_feature, host_pinned_feature, dev_cache_feature, src_vertex, feature_size,
                              vertex_size, cache_node_hashmap, cache_ld=None):
        """zero_copy_feature_move_gpu_cache + gather_feature_from_gpu_cache in one launch: the hit/miss
        split that the reference makes in a serial host loop (core/ntsSampler.hpp:444-456) is resolved
        per row on the device from cache_node_hashmap."""
        _lib.call("nb_feature_gather", dev_feature, host_pinned_feature, feature_size, None, 0, 0, dev_cache_feature,
                  feature_size if cache_ld is None else cache_ld, cache_node_hashmap, src_vertex, vertex_size,
                  feature_size, self.getStream())

    def global_copy_label_move_gpu(self, dev_label, global_dev_label, dst_vertex, vertex_size):
        _lib.call("nb_label_gather", dev_label, global_dev_label, dst_vertex, vertex_size, 1, self.getStream())

    def global_copy_mulilabel_move_gpu(self, dev_label, global_dev_label, dst_vertex, vertex_size, label_size):
        _lib.call("nb_label_gather", dev_label, global_dev_label, dst_vertex, vertex_size, label_size,
                  self.getStream())
