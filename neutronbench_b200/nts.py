"""`nts <file.cfg>` for ALGORITHM:GCNNEIGHBORGPU — the cfg-driven entry of the reference
(toolkits/main.cpp:45-58, 116-137) on top of the B200 path.

    python -m neutronbench_b200.nts path/to/file.cfg

The cfg format is the reference's (core/GraphSegment.cpp:196-405): flat KEY:VALUE lines, '#' starts a
comment line, the last occurrence of a key wins, unknown keys are reported and ignored.  Input files
are the reference's: binary .edge (u32 src, u32 dst pairs), text .feat ("id f0 .. fF-1"), .label
("id label"), .mask ("id train|val|eval|test"), or FEATURE_FILE:random
(core/ntsDataloador.hpp:107-156, 264-330).  One line per epoch is logged in the reference's format
(toolkits/GCN_GPU_NEIGHBOR.hpp:1499-1505) so that the reference's log parsers keep working.
"""
from __future__ import annotations

import os
import sys
import time
from dataclasses import dataclass, field
from typing import List

import numpy as np

KNOWN_KEYS = {
    "ALGORITHM", "VERTICES", "EPOCHS", "LAYERS", "FANOUT", "VALFANOUT", "EDGE_FILE", "FEATURE_FILE", "LABEL_FILE",
    "MASK_FILE", "PROC_OVERLAP", "PROC_LOCAL", "PROC_CUDA", "PROC_REP", "LOCK_FREE", "LEARN_RATE", "WEIGHT_DECAY",
    "DECAY_RATE", "DECAY_EPOCH", "DROP_RATE", "BATCH_SIZE", "VALBATCH_SIZE", "OPTIM_KERNEL", "BATCH_NORM",
    "BATCH_SIZE_VEC", "BATCH_SWITCH_ACC", "BATCH_SWITCH_TIME", "BATCH_TYPE", "BEST_PARAMETER", "BLOCK_SIZE",
    "CACHE_EXP", "CACHE_POLICY", "CACHE_RATE", "CACHE_RATE_END", "CACHE_RATE_NUM", "CACHE_RATE_START", "CACHE_TYPE",
    "CLASSES", "DEL_FRAC", "DYNAMIC_SAMPLE", "LOWER_FANOUT", "MINI_PULL", "MODE", "PART_ALGO", "PART_DIM", "PART_NUM",
    "PIPELINES", "RUNS", "RUN_TIME", "SAMPLE_RATE", "SAMPLE_RATE_VEC", "SAMPLE_SWITCH_TIME", "TARGET_DEGREE",
    "THREADS", "THRESHOLD_TRANS", "TIME_SKIP", "TRANS_THRESHOLD_END", "TRANS_THRESHOLD_NUM", "TRANS_THRESHOLD_START",
}


@dataclass
class InputInfo:
    """The fields of the reference's InputInfo (core/GraphSegment.h:142-220) that the sampled GCN path reads."""
    algorithm: str = ""
    vertices: int = 0
    epochs: int = 1
    layer_string: str = ""
    fanout_string: str = ""
    val_fanout_string: str = ""
    edge_file: str = ""
    feature_file: str = ""
    label_file: str = ""
    mask_file: str = ""
    dataset_name: str = ""
    learn_rate: float = 0.01
    weight_decay: float = 0.05
    decay_rate: float = 0.97
    decay_epoch: float = 100
    drop_rate: float = 0.5
    batch_size: int = 0
    val_batch_size: int = 0
    batch_type: str = "shuffle"
    batch_norm: int = 0
    classes: int = 1
    mode: str = "zerocopy"
    cache_type: str = "none"
    cache_policy: str = "degree"
    cache_rate: float = 0.0
    pipelines: int = 1
    sample_rate: float = -1.0
    lower_fanout: int = 0
    del_frac: float = 0.0
    mini_pull: int = 1
    run_time: float = -1.0
    runs: int = 1
    threads: int = -1
    unknown: List[str] = field(default_factory=list)

    def readFromCfgFile(self, path: str) -> "InputInfo":
        conv = {
            "ALGORITHM": ("algorithm", str), "VERTICES": ("vertices", int), "EPOCHS": ("epochs", int),
            "LAYERS": ("layer_string", str), "FANOUT": ("fanout_string", str), "VALFANOUT": ("val_fanout_string", str),
            "FEATURE_FILE": ("feature_file", str), "LABEL_FILE": ("label_file", str), "MASK_FILE": ("mask_file", str),
            "LEARN_RATE": ("learn_rate", float), "WEIGHT_DECAY": ("weight_decay", float),
            "DECAY_RATE": ("decay_rate", float), "DECAY_EPOCH": ("decay_epoch", float),
            "DROP_RATE": ("drop_rate", float), "BATCH_SIZE": ("batch_size", int),
            "VALBATCH_SIZE": ("val_batch_size", int), "BATCH_TYPE": ("batch_type", str),
            "BATCH_NORM": ("batch_norm", int), "CLASSES": ("classes", int), "MODE": ("mode", str),
            "CACHE_TYPE": ("cache_type", str), "CACHE_POLICY": ("cache_policy", str),
            "CACHE_RATE": ("cache_rate", float), "PIPELINES": ("pipelines", int), "MINI_PULL": ("mini_pull", int),
            "RUN_TIME": ("run_time", float), "RUNS": ("runs", int), "THREADS": ("threads", int),
            "SAMPLE_RATE": ("sample_rate", float), "LOWER_FANOUT": ("lower_fanout", int), "DEL_FRAC": ("del_frac", float),
        }
        for line in open(path):
            line = line.rstrip("\n").rstrip("\r")
            if not line or line[0] == "#":
                continue
            k, _, v = line.partition(":")
            if k == "EDGE_FILE":
                self.edge_file = v
                # dataset name = path component after "data/" (core/GraphSegment.cpp:219-223)
                start = v.find("data") + 5
                end = v.find("/", start)
                self.dataset_name = v[start:end] if end >= 0 else v[start:]
            elif k in conv:
                name, typ = conv[k]
                try:
                    setattr(self, name, typ(v.strip()) if typ is not str else v.strip())
                except ValueError:
                    setattr(self, name, typ(0))   # atoi / atof give 0 on garbage
            elif k in KNOWN_KEYS:
                pass                              # accepted, not used by this path
            else:
                self.unknown.append(k)
                print(f"not supported configure {k}")
        return self

    def layers(self) -> List[int]:
        return [int(x) for x in self.layer_string.split("-") if x]

    @staticmethod
    def _fanout(s: str) -> List[int]:
        sep = "," if "," in s else "-"      # core/graph.hpp:286-301
        return [int(x) for x in s.split(sep) if x]

    def fanout_hop_order(self) -> List[int]:
        """FANOUT lists GNN-layer order; the sampler wants seeds first (toolkits/GCN_GPU_NEIGHBOR.hpp:126-130)."""
        return list(reversed(self._fanout(self.fanout_string)))

    def val_fanout_hop_order(self) -> List[int]:
        s = self.val_fanout_string or self.fanout_string
        return list(reversed(self._fanout(s)))


def feature_sidecar_path(feature_file: str, vertices: int, feat_dim: int) -> str:
    return f"{feature_file}.{vertices}x{feat_dim}.f32"


def read_feature(feature_file: str, vertices: int, feat_dim: int, use_sidecar: bool = True) -> np.ndarray:
    """The `.feat` text table ("id v0 v1 ..." per line, core/ntsDataloador.hpp:264-300) as float32
    [vertices x feat_dim].  Parsing the text dominates start-up on large datasets, so the parsed table is
    kept beside the text file as raw little-endian float32 (`<file>.<V>x<F>.f32`) and read from there
    while it is at least as new as the text; a directory that cannot be written is not an error."""
    side = feature_sidecar_path(feature_file, vertices, feat_dim)
    if use_sidecar and os.path.exists(side) and os.path.getmtime(side) >= os.path.getmtime(feature_file) \
            and os.path.getsize(side) == 4 * vertices * feat_dim:
        return np.fromfile(side, dtype="<f4").reshape(vertices, feat_dim)
    feat = np.zeros((vertices, feat_dim), dtype=np.float32)
    with open(feature_file) as ff:
        for line in ff:
            parts = line.split()
            if not parts:
                continue
            vid = int(parts[0])
            if 0 <= vid < vertices:
                feat[vid, :] = np.asarray(parts[1:1 + feat_dim], dtype=np.float32)
    if use_sidecar:
        try:
            tmp = side + ".tmp%d" % os.getpid()
            feat.astype("<f4").tofile(tmp)
            os.replace(tmp, side)
        except OSError:
            pass
    return feat


def read_feature_label_mask(feature_file: str, label_file: str, mask_file: str, vertices: int, feat_dim: int,
                            classes: int = 1):
    """GNNDatum::readFeature_Label_Mask (core/ntsDataloador.hpp:264-330).  Label lines are "id label", or with
    CLASSES > 1 "id count idx_1 ... idx_count" (the set labels of a multi-hot row, :304-312)."""
    feat = read_feature(feature_file, vertices, feat_dim)
    label = np.zeros((vertices, classes), dtype=np.int64) if classes > 1 else np.zeros(vertices, dtype=np.int64)
    mask = np.full(vertices, 3, dtype=np.int32)
    with open(label_file) as lf:
        for line in lf:
            parts = line.split()
            if len(parts) >= 2 and 0 <= int(parts[0]) < vertices:
                if classes > 1:
                    n = int(parts[1])
                    for idx in parts[2: 2 + n]:
                        if 0 <= int(idx) < classes:
                            label[int(parts[0]), int(idx)] = 1
                else:
                    label[int(parts[0])] = int(parts[1])
    code = {"train": 0, "eval": 1, "val": 1, "test": 2}
    with open(mask_file) as mf:
        for line in mf:
            parts = line.split()
            if len(parts) >= 2 and 0 <= int(parts[0]) < vertices:
                mask[int(parts[0])] = code.get(parts[1], 3)
    return feat, label, mask


def random_generate(vertices: int, feat_dim: int, classes: int, seed: int = 2000):
    """GNNDatum::random_generate (core/ntsDataloador.hpp:107-156): features all 1.0, random labels and a
    65 % train / 10 % val / 25 % test split after a seeded shuffle (libc rand() and std::shuffle there;
    numpy's generator here, so the draws differ)."""
    rng = np.random.RandomState(seed)
    feat = np.ones((vertices, feat_dim), dtype=np.float32)
    label = rng.randint(0, classes, size=vertices).astype(np.int64)
    perm = rng.permutation(vertices)
    mask = np.full(vertices, 2, dtype=np.int32)
    mask[perm[: int(vertices * 0.65)]] = 0
    mask[perm[int(vertices * 0.65): int(vertices * 0.75)]] = 1
    return feat, label, mask


def epoch_log_line(epoch, train_loss, train_acc, val_loss, val_acc, test_acc, train_time, sample_t, trans_t, graph_t,
                   nn_t, val_time, run_time, train_bs, val_bs) -> str:
    """The reference's per-epoch LOG_INFO text (toolkits/GCN_GPU_NEIGHBOR.hpp:1499-1505)."""
    return ("Epoch %03d train_loss %.3f train_acc %.3f val_loss %.3f val_acc %.3f test_acc %.3f train_time %.3f(sample "
            "%.3f trans %.3f graph %.3f nn %.3f) val_time %.3f, gcn_run_time %.3f) batch_size (%d, %d)"
            % (epoch, train_loss, train_acc, val_loss, val_acc, test_acc, train_time, sample_t, trans_t, graph_t, nn_t,
               val_time, run_time, train_bs, val_bs))


def run(cfg_path: str, out=sys.stdout) -> float:
    """init_graph + init_nn + run() of GCN_GPU_NEIGHBOR_impl (toolkits/GCN_GPU_NEIGHBOR.hpp:171-288, 1330-1555).
    Returns the best validation accuracy."""
    import torch
    from . import FullyRepGraph, GCN_GPU_NEIGHBOR_impl, GCNConfig, GNNDatum, Sampler, Workspace, _lib
    from .toolkit import drop_train_ids_by_degree, shard_for_rank

    info = InputInfo().readFromCfgFile(cfg_path)
    if info.algorithm != "GCNNEIGHBORGPU":
        raise SystemExit(f"ALGORITHM:{info.algorithm} is not built here; only GCNNEIGHBORGPU is")
    if info.batch_norm:
        raise SystemExit("BATCH_NORM:1 is not supported on the GPU path (the reference keeps its BatchNorm modules on "
                         "the CPU, toolkits/GCN_GPU_NEIGHBOR.hpp:242-246); use BATCH_NORM:0")
    classes = max(1, int(info.classes))
    if classes > 1 and classes != info.layers()[-1]:
        raise SystemExit("CLASSES > 1 needs a last layer with one output per class")
    assert torch.cuda.is_available(), "nts needs a CUDA device; there is no CPU fallback"
    # One process per GPU, started by torchrun (the reference: one MPI rank per GPU, toolkits/main.cpp): every rank
    # holds the whole topology and trains on its own share of the train list.
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        if not torch.distributed.is_initialized():
            # the per-step gradient sum runs beside the next batch's layer-0 aggregation, on the few SMs that kernel
            # leaves free: few channels, and CTAs that do not have to be placed together as one cluster
            os.environ.setdefault("NCCL_MAX_CTAS", "4")
            os.environ.setdefault("NCCL_CGA_CLUSTER_SIZE", "1")
            torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
        if rank != 0:
            out = open(os.devnull, "w")
    dev = torch.device("cuda", torch.cuda.current_device())
    layers = info.layers()
    V = info.vertices
    raw = np.fromfile(info.edge_file, dtype="<u4").reshape(-1, 2)
    edges = torch.from_numpy(raw.view(np.int32)).to(dev)
    graph = FullyRepGraph.from_edges(edges, V, Workspace(int(raw.shape[0]) * 9 + V * 16 + (64 << 20), dev))
    del edges
    if info.feature_file == "random":
        feat, label, mask = random_generate(V, layers[0], layers[-1])
        if classes > 1:   # one random label per node, as a multi-hot row
            label = np.eye(classes, dtype=np.int64)[label]
    else:
        feat, label, mask = read_feature_label_mask(info.feature_file, info.label_file, info.mask_file, V, layers[0],
                                                    classes)
    cache_type = info.cache_type or "none"
    cache_rate = info.cache_rate if cache_type in ("rate", "random") else 0.0
    if cache_type in ("rate", "random") and cache_rate <= 0:
        cache_type = "none"
    cfg = GCNConfig(layers=layers, fanout=info.fanout_hop_order(), val_fanout=info.val_fanout_hop_order(),
                    batch_size=info.batch_size, learn_rate=info.learn_rate, weight_decay=info.weight_decay,
                    drop_rate=info.drop_rate, cache_type=cache_type, cache_rate=cache_rate,
                    cache_policy=info.cache_policy or "degree", pipelines=max(1, int(info.pipelines)),
                    sample_rate=max(0.0, info.sample_rate), lower_fanout=max(0, info.lower_fanout), classes=classes)
    feature = torch.from_numpy(feat)
    # the table stays in pinned host memory (zero-copy misses) unless every row is cached on the GPU anyway
    feature = feature.to(dev) if cache_rate >= 1.0 else feature.pin_memory()
    datum = GNNDatum(feature, torch.from_numpy(label).to(dev), mask)
    tk = GCN_GPU_NEIGHBOR_impl(graph, datum, cfg, rank=rank, world_size=world)
    ids = [np.nonzero(mask == k)[0].astype(np.uint32) for k in (0, 1, 2)]
    print("label rate: %.3f, train/val/test: (%d/%d/%d)" % (sum(map(len, ids)) / V, *map(len, ids)), file=out)
    if info.batch_type == "metis":
        raise ValueError("BATCH_TYPE:metis needs the METIS library, which this build does not link")
    if info.batch_type not in ("shuffle", "sequence", "random", "dellow", "delhigh"):
        raise ValueError(f"BATCH_TYPE {info.batch_type!r} is not one of shuffle | sequence | random | dellow | delhigh")
    in_deg = np.diff(graph.column_offset.cpu().numpy().astype(np.int64))
    train_ids = drop_train_ids_by_degree(ids[0], in_deg, info.batch_type, info.del_frac)
    # this rank's share of every split (the reference: the nodes of the rank's own vertex range,
    # toolkits/GCN_GPU_NEIGHBOR.hpp:1339-1348); statistics are summed over the ranks at every epoch end
    global_sizes = [len(train_ids), len(ids[1]), len(ids[2])]
    train_ids, ids[1], ids[2] = (shard_for_rank(x, rank, world) for x in (train_ids, ids[1], ids[2]))
    train = Sampler(graph, train_ids, cfg.fanout, cfg.batch_size, tk.ws, with_edge_weights=False,
                    sample_rate=cfg.sample_rate, lower_fanout=cfg.lower_fanout)
    train.random_batches = info.batch_type == "random"
    tk.init_cache(train)   # CACHE_POLICY:sample runs its dry-run epoch on the training sampler
    if tk.cache_node_num:
        print("cache_node_num %d (%.3f)" % (tk.cache_node_num, tk.cache_node_num / V), file=out)
    # validation / test: one full batch each with the validation fanout (toolkits/...:1381-1392)
    evals = [Sampler(graph, ids[k], cfg.val_fanout, max(len(ids[k]), 1), tk.ws, full_batch=True,
                     with_edge_weights=False) if global_sizes[k] else None for k in (1, 2)]
    import ctypes
    if tk.use_engine:   # per-phase times of the epoch line come from the library's own clocks
        _lib.call("nb_gcn_set_timing", tk._ensure_engine(), 1)
    rng = np.random.RandomState(2000)
    best_val, run_time = 0.0, 0.0
    for epoch in range(info.epochs):
        if info.run_time > 0 and run_time >= info.run_time:
            break
        t0 = time.time()
        # every batch type but "sequence" reshuffles the seed list per epoch (toolkits/GCN_GPU_NEIGHBOR.hpp:741-745)
        train_acc, train_loss, _ = tk.Forward(train, rng=rng if info.batch_type != "sequence" else None, train=True)
        torch.cuda.synchronize()
        train_time = time.time() - t0
        run_time += train_time
        phase = (ctypes.c_double * 4)()
        if tk.use_engine:
            _lib.call("nb_gcn_read_phase_times", tk._ensure_engine(), phase)
        t1 = time.time()
        val_acc, val_loss = (tk.Forward(evals[0], train=False)[:2] if evals[0] else (0.0, 0.0))
        val_time = time.time() - t1
        test_acc = tk.Forward(evals[1], train=False)[0] if evals[1] else 0.0
        if tk.use_engine:   # evaluation launches are not part of the next epoch's training times
            _lib.call("nb_gcn_read_phase_times", tk._ensure_engine(), (ctypes.c_double * 4)())
        print(epoch_log_line(epoch, train_loss, train_acc, val_loss, val_acc, test_acc, train_time, phase[0] / 1e3,
                             phase[1] / 1e3, phase[2] / 1e3, phase[3] / 1e3, val_time, run_time, train.batch_size, evals[0].batch_size if evals[0] else 0), file=out)
        best_val = max(best_val, val_acc)
    return best_val


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python -m neutronbench_b200.nts <file.cfg>")
    run(sys.argv[1])
