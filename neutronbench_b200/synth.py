"""Seeded synthetic graphs with the shapes of the reference's datasets (Cora, ogbn-arxiv, Reddit,
ogbn-products, ogbn-papers100M stand-ins).  None of those datasets is read; only their published
shapes (node / edge counts, feature width, class count) are used.

Edges come out as an int32 [E, 2] array of (src, dst) pairs — the layout of the reference's binary
.edge file (core/graph.hpp:1059-1060).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

import numpy as np
import torch


@dataclass(frozen=True)
class Shape:
    name: str
    vertices: int
    edges: int
    feature: int
    classes: int
    hidden: int
    fanout: Tuple[int, ...]      # hop order, seeds first
    batch: int
    rmat: Tuple[float, float, float]  # (a, b, c); d = 1 - a - b - c


SHAPES = {
    "arxiv": Shape("arxiv", 169_343, 2_480_000, 128, 40, 128, (25, 10), 1024, (0.57, 0.19, 0.19)),
    "reddit": Shape("reddit", 232_965, 114_850_000, 602, 41, 128, (25, 10), 1024, (0.45, 0.22, 0.22)),
    "products": Shape("products", 2_450_000, 126_170_000, 100, 47, 128, (15, 10, 5), 4096, (0.57, 0.19, 0.19)),
    "papers": Shape("papers", 111_060_000, 1_600_000_000, 128, 172, 128, (15, 10, 5), 8192, (0.57, 0.19, 0.19)),
}


def uniform_undirected_numpy(vertices: int, undirected_edges: int, seed: int, self_loops: bool = True) -> np.ndarray:
    """Cora-shaped graph: uniform random undirected edges, symmetrised, plus self loops."""
    rng = np.random.RandomState(seed)
    a = rng.randint(0, vertices, size=undirected_edges).astype(np.int32)
    b = rng.randint(0, vertices, size=undirected_edges).astype(np.int32)
    src = np.concatenate([a, b])
    dst = np.concatenate([b, a])
    if self_loops:
        loops = np.arange(vertices, dtype=np.int32)
        src = np.concatenate([src, loops])
        dst = np.concatenate([dst, loops])
    return np.stack([src, dst], axis=1).astype(np.int32)


def rmat_numpy(vertices: int, edges: int, abc: Tuple[float, float, float], seed: int,
               self_loops: bool = True) -> np.ndarray:
    """R-MAT edge list on the CPU (small graphs for tests)."""
    rng = np.random.RandomState(seed)
    scale = max(1, int(np.ceil(np.log2(vertices))))
    a, b, c = abc
    out_src = np.empty(0, dtype=np.int64)
    out_dst = np.empty(0, dtype=np.int64)
    while out_src.size < edges:
        n = int((edges - out_src.size) * 1.3) + 16
        src = np.zeros(n, dtype=np.int64)
        dst = np.zeros(n, dtype=np.int64)
        for _ in range(scale):
            r = rng.random_sample(n)
            right = (r >= a) & (r < a + b) | (r >= a + b + c)   # quadrants b and d: column bit set
            down = r >= a + b                                   # quadrants c and d: row bit set
            src = (src << 1) | down
            dst = (dst << 1) | right
        keep = (src < vertices) & (dst < vertices)
        out_src = np.concatenate([out_src, src[keep]])
        out_dst = np.concatenate([out_dst, dst[keep]])
    src, dst = out_src[:edges], out_dst[:edges]
    if self_loops:
        loops = np.arange(vertices, dtype=np.int64)
        src = np.concatenate([src, loops])
        dst = np.concatenate([dst, loops])
    return np.stack([src, dst], axis=1).astype(np.int32)


def rmat_torch(vertices: int, edges: int, abc: Tuple[float, float, float], seed: int, device="cuda",
               self_loops: bool = True, chunk: int = 1 << 25) -> torch.Tensor:
    """R-MAT edge list generated on the GPU in chunks (data preparation; not part of any timed region)."""
    gen = torch.Generator(device=device).manual_seed(seed)
    scale = max(1, int(np.ceil(np.log2(vertices))))
    a, b, c = abc
    parts = []
    have = 0
    while have < edges:
        n = min(chunk, int((edges - have) * 1.3) + 16)
        src = torch.zeros(n, dtype=torch.int64, device=device)
        dst = torch.zeros(n, dtype=torch.int64, device=device)
        for _ in range(scale):
            r = torch.rand(n, generator=gen, device=device)
            right = ((r >= a) & (r < a + b)) | (r >= a + b + c)
            down = r >= a + b
            src = (src << 1) | down
            dst = (dst << 1) | right
        keep = (src < vertices) & (dst < vertices)
        e = torch.stack([src[keep], dst[keep]], dim=1).to(torch.int32)
        e = e[: edges - have]
        parts.append(e)
        have += e.size(0)
    if self_loops:
        loops = torch.arange(vertices, dtype=torch.int32, device=device)
        parts.append(torch.stack([loops, loops], dim=1))
    return torch.cat(parts, dim=0).contiguous()


def split_mask(vertices: int, seed: int, train: float = 0.65, val: float = 0.25) -> np.ndarray:
    """0 train / 1 val / 2 test labels per node after a seeded shuffle (65/25/10 by default)."""
    rng = np.random.RandomState(seed)
    perm = rng.permutation(vertices)
    mask = np.full(vertices, 2, dtype=np.int32)
    n_train = int(vertices * train)
    n_val = int(vertices * val)
    mask[perm[:n_train]] = 0
    mask[perm[n_train:n_train + n_val]] = 1
    return mask
