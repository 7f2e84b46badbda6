"""ctypes binding of libnb_b200.so (the C ABI declared in include/nb_b200.h).

The library is the product's compute path; there is no CPU or PyTorch fallback.  Loading fails loudly
when the shared object has not been built (run ``python -c "import __graft_entry__ as g; g.build()"``
or ``make -C neutronbench_b200/csrc``).
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libnb_b200.so")

u32p = C.c_void_p  # device pointers travel as integers (tensor.data_ptr())
f32p = C.c_void_p
u64p = C.c_void_p
i64p = C.c_void_p
ptr = C.c_void_p

NB_MAX_LAYERS = 8


class GcnConfig(C.Structure):
    """struct nb_gcn_config (include/nb_b200.h)."""
    _fields_ = [("num_layers", C.c_uint32), ("layer_size", C.c_uint32 * (NB_MAX_LAYERS + 1)),
                ("fanout", C.c_int32 * NB_MAX_LAYERS), ("num_vertices", C.c_uint32),
                ("learn_rate", C.c_float), ("weight_decay", C.c_float), ("drop_rate", C.c_float),
                ("beta1", C.c_float), ("beta2", C.c_float), ("epsilon", C.c_float), ("seed", C.c_uint64),
                ("fuse_gather", C.c_int), ("d_graph_column_offset", C.c_void_p), ("d_graph_row_indices", C.c_void_p),
                ("feat", C.c_void_p), ("feat_ld", C.c_size_t), ("d_cache", C.c_void_p), ("cache_ld", C.c_size_t),
                ("d_hashmap", C.c_void_p), ("d_label", C.c_void_p), ("d_W", C.c_void_p), ("d_grad", C.c_void_p),
                ("d_M", C.c_void_p), ("d_V", C.c_void_p), ("sample_rate", C.c_float), ("lower_fanout", C.c_int32),
                ("classes", C.c_uint32), ("d_feat_shards", C.c_void_p), ("num_shards", C.c_uint32),
                ("shard_rows", C.c_uint32), ("stage_misses", C.c_int)]


class GcnStepInfo(C.Structure):
    """struct nb_gcn_step_info (include/nb_b200.h)."""
    _fields_ = [("v", C.c_uint32 * NB_MAX_LAYERS), ("s", C.c_uint32 * NB_MAX_LAYERS),
                ("e", C.c_uint32 * NB_MAX_LAYERS), ("agg_bytes", C.c_uint64)]


# name -> (restype, argtypes); mirrors include/nb_b200.h one to one.
SIGNATURES = {
    "nb_last_error": (C.c_char_p, []),
    "nb_version": (C.c_int, []),
    "nb_launch_count": (C.c_uint64, []),
    "nb_ws_create": (C.c_int, [C.POINTER(C.c_void_p), ptr, C.c_size_t]),
    "nb_ws_destroy": (C.c_int, [ptr]),
    "nb_ws_reset": (C.c_int, [ptr]),
    "nb_ws_used": (C.c_size_t, [ptr]),
    "nb_ws_high_water": (C.c_size_t, [ptr]),
    "nb_spmm_csc_fwd": (C.c_int, [f32p, f32p, f32p, u32p, u32p, C.c_uint32, C.c_uint32, ptr]),
    "nb_spmm_csr_bwd": (C.c_int, [f32p, f32p, f32p, u32p, u32p, C.c_uint32, C.c_uint32, ptr]),
    "nb_spmm_csc_fwd_fused": (C.c_int, [f32p, f32p, u32p, u32p, f32p, f32p, C.c_uint32, C.c_uint32, ptr]),
    "nb_spmm_csr_bwd_fused": (C.c_int, [f32p, f32p, u32p, u32p, f32p, f32p, f32p, C.c_float, C.c_uint32,
                                        C.c_uint32, ptr]),
    "nb_spmm_csc_fwd_gather_fused": (C.c_int, [ptr, f32p, C.c_size_t, f32p, C.c_size_t, u32p, u32p, f32p, u32p, u32p,
                                               f32p, f32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, ptr]),
    "nb_set_l2_panel_bytes": (C.c_uint64, [C.c_uint64]),
    "nb_set_staged_spmm": (C.c_int, [C.c_int]),
    "nb_device_error_flags": (C.c_int, [C.POINTER(C.c_uint32)]),
    "nb_device_error_reset": (C.c_int, []),
    "nb_gcn_set_option": (C.c_int, [ptr, C.c_char_p, C.c_int64]),
    "nb_set_option": (C.c_int, [C.c_char_p, C.c_int64]),
    "nb_block_build": (C.c_int, [ptr, C.c_uint32, u32p, u32p, C.c_uint32, C.c_uint32, u32p,
                                 C.POINTER(C.c_uint32), u32p, u32p, f32p, f32p, f32p, f32p, ptr]),
    "nb_sample_hop_offsets": (C.c_int, [ptr, u64p, u32p, C.c_uint32, C.c_int, u32p, C.POINTER(C.c_uint32), ptr]),
    "nb_sample_hop_offsets_rate": (C.c_int, [ptr, u64p, u32p, C.c_uint32, C.c_float, C.c_int, u32p,
                                             C.POINTER(C.c_uint32), ptr]),
    "nb_sample_hop": (C.c_int, [u64p, u32p, u32p, C.c_uint32, C.c_int, u32p, C.c_uint64, C.c_uint32, u32p, ptr]),
    "nb_graph_build_csc": (C.c_int, [ptr, u32p, C.c_uint64, C.c_uint32, u64p, u32p, u32p, u32p, ptr]),
    "nb_feature_gather": (C.c_int, [f32p, f32p, C.c_size_t, ptr, C.c_uint32, C.c_uint32, f32p, C.c_size_t, u32p,
                                    u32p, C.c_uint32, C.c_uint32, ptr]),
    "nb_feature_gather_indexed": (C.c_int, [f32p, C.c_size_t, f32p, C.c_size_t, u32p, u32p, u32p, C.c_uint32,
                                            C.c_uint32, ptr]),
    "nb_shard_alloc": (C.c_int, [C.POINTER(C.c_void_p), C.c_size_t]),
    "nb_shard_free": (C.c_int, [ptr]),
    "nb_shard_upload": (C.c_int, [ptr, ptr, C.c_size_t]),
    "nb_shard_export": (C.c_int, [ptr, C.c_char_p]),
    "nb_shard_open": (C.c_int, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "nb_shard_close": (C.c_int, [ptr]),
    "nb_label_gather": (C.c_int, [i64p, i64p, u32p, C.c_uint32, C.c_uint32, ptr]),
    "nb_cache_fill": (C.c_int, [f32p, C.c_size_t, f32p, C.c_size_t, u32p, C.c_uint32, C.c_uint32, ptr]),
    "nb_count_ids": (C.c_int, [u32p, C.c_uint64, C.c_uint32, u32p, ptr]),
    "nb_set_gemm_mode": (C.c_int, [C.c_int]),
    "nb_gemm": (C.c_int, [ptr, f32p, f32p, f32p, C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_int, ptr]),
    "nb_relu_dropout": (C.c_int, [f32p, C.c_int64, C.c_float, C.c_uint64, C.c_uint32, C.c_uint32, ptr]),
    "nb_softmax_nll": (C.c_int, [ptr, f32p, i64p, C.c_int64, C.c_int64, f32p, f32p, ptr]),
    "nb_softmax_nll_static": (C.c_int, [f32p, i64p, C.c_int64, C.c_int64, f32p, f32p, ptr]),
    "nb_gcn_create": (C.c_int, [C.POINTER(C.c_void_p), C.POINTER(GcnConfig), ptr]),
    "nb_gcn_destroy": (C.c_int, [ptr]),
    "nb_gcn_step": (C.c_int, [ptr, u32p, C.c_uint32, C.c_int, f32p, C.POINTER(GcnStepInfo), ptr]),
    "nb_gcn_update": (C.c_int, [ptr] * 2),
    "nb_gcn_wait_gradients": (C.c_int, [ptr] * 2),
    "nb_gcn_batch_create": (C.c_int, [C.POINTER(C.c_void_p), ptr]),
    "nb_gcn_batch_destroy": (C.c_int, [ptr]),
    "nb_gcn_sample": (C.c_int, [ptr, ptr, u32p, C.c_uint32, C.c_int, ptr]),
    "nb_gcn_sample_async": (C.c_int, [ptr, ptr, u32p, C.c_uint32, C.c_int, ptr]),
    "nb_gcn_sample_from_edges": (C.c_int, [ptr, ptr, u32p, C.c_uint32, C.POINTER(C.c_void_p), C.POINTER(C.c_uint32),
                                           ptr]),
    "nb_gcn_count_sources": (C.c_int, [ptr, ptr, u32p, ptr]),
    "nb_gcn_set_sampler_threads": (C.c_int, [ptr, C.c_int]),
    "nb_gcn_compute": (C.c_int, [ptr, ptr, C.c_int, f32p, C.POINTER(GcnStepInfo), ptr]),
    "nb_gcn_set_timing": (C.c_int, [ptr, C.c_int]),
    "nb_gcn_read_timing": (C.c_int, [ptr, C.POINTER(C.c_double), C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "nb_gcn_read_timing_by_class": (C.c_int, [ptr, C.POINTER(C.c_double), C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "nb_gcn_read_phase_times": (C.c_int, [ptr, C.POINTER(C.c_double)]),
    "nb_set_fused_output_layer": (C.c_int, [C.c_int]),
    "nb_set_pdl": (C.c_int, [C.c_int]),
    "nb_output_layer_supported": (C.c_int, [C.c_uint32, C.c_uint32]),
    "nb_output_layer": (C.c_int, [ptr, f32p, f32p, i64p, u32p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_int, f32p, f32p,
                                  f32p, ptr]),
    "nb_sigmoid_bce": (C.c_int, [ptr, f32p, i64p, C.c_int64, C.c_int64, f32p, f32p, ptr]),
    "nb_adam": (C.c_int, [f32p, f32p, f32p, f32p, C.c_int64, C.c_float, C.c_float, C.c_float, C.c_float,
                          C.c_float, C.c_float, C.c_float, ptr]),
}


# libnb_b200_comm.so: the optional NCCL layer declared at the end of include/nb_b200.h
COMM_LIB_PATH = os.path.join(_HERE, "libnb_b200_comm.so")
COMM_SIGNATURES = {
    "nb_comm_unique_id": (C.c_int, [C.c_char_p]),
    "nb_comm_create": (C.c_int, [C.POINTER(C.c_void_p), C.c_char_p, C.c_int, C.c_int]),
    "nb_comm_destroy": (C.c_int, [ptr]),
    "nb_allreduce_sum_f32": (C.c_int, [ptr, f32p, C.c_size_t, ptr]),
    "nb_broadcast_f32": (C.c_int, [ptr, f32p, C.c_size_t, C.c_int, ptr]),
}
_comm = None


def load_comm():
    """Load libnb_b200_comm.so (needs the NCCL library that PyTorch ships)."""
    global _comm
    if _comm is not None:
        return _comm
    if not os.path.exists(COMM_LIB_PATH):
        raise ImportError(f"{COMM_LIB_PATH} is missing: run `make -C neutronbench_b200/csrc`")
    lib = C.CDLL(COMM_LIB_PATH)
    for name, (res, args) in COMM_SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    lib.nb_last_error.restype = C.c_char_p
    _comm = lib
    return lib


def call_comm(name: str, *args):
    lib = load_comm()
    st = getattr(lib, name)(*args)
    if st != 0:
        raise NbError(name, st, lib.nb_last_error().decode("utf-8", "replace"))
    return st


class NbError(RuntimeError):
    """A libnb_b200 entry point returned a non-zero status."""

    def __init__(self, name: str, status: int, message: str):
        super().__init__(f"{name} failed with status {status}: {message}")
        self.status = status


_lib = None


def load():
    """Load the shared library once and attach the signatures."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: the CUDA extension has not been built. "
            "Run `make -C neutronbench_b200/csrc` (or __graft_entry__.build()). There is no CPU fallback."
        )
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def call(name: str, *args):
    """Call an int-returning entry point and raise NbError on failure."""
    lib = load()
    st = getattr(lib, name)(*args)
    if st != 0:
        raise NbError(name, st, lib.nb_last_error().decode("utf-8", "replace"))
    return st
