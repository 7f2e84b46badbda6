"""numpy front end of oracle/liboracle.so (the CPU restatement of the reference).  Test
infrastructure: only tests, __graft_entry__.smoke() and bench.py's CPU-baseline leg import it."""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_SO = os.path.join(ROOT, "oracle", "liboracle.so")
_lib = None


def lib():
    global _lib
    if _lib is None:
        src = os.path.join(ROOT, "oracle", "nts_oracle.c")
        if not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
            subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle"), "liboracle.so"])
        _lib = C.CDLL(_SO)
        _lib.orc_init_co.restype = C.c_uint32
        _lib.orc_init_co_rate.restype = C.c_uint32
        _lib.orc_dedup_reindex.restype = C.c_uint32
        _lib.orc_softmax_nll.restype = C.c_float
        _lib.orc_num_threads.restype = C.c_int
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def build_csc(edges: np.ndarray, V: int):
    edges = np.ascontiguousarray(edges, dtype=np.uint32)
    E = edges.shape[0]
    co = np.zeros(V + 1, dtype=np.uint64)
    ri = np.zeros(max(E, 1), dtype=np.uint32)
    lib().orc_build_csc(_p(edges), C.c_uint64(E), C.c_uint32(V), _p(co), _p(ri))
    return co, ri[:E]


def degrees(edges: np.ndarray, V: int, clamp: bool = True):
    edges = np.ascontiguousarray(edges, dtype=np.uint32)
    out_d = np.zeros(V, dtype=np.uint32)
    in_d = np.zeros(V, dtype=np.uint32)
    lib().orc_degrees(_p(edges), C.c_uint64(edges.shape[0]), C.c_uint32(V), _p(out_d), _p(in_d), C.c_int(int(clamp)))
    return out_d, in_d


def init_co(g_co, dst, fanout):
    dst = np.ascontiguousarray(dst, dtype=np.uint32)
    co = np.zeros(len(dst) + 1, dtype=np.uint32)
    e = lib().orc_init_co(_p(g_co), _p(dst), C.c_uint32(len(dst)), C.c_int(fanout), _p(co))
    return co, int(e)


def init_co_rate(g_co, dst, sample_rate, lower_fanout):
    dst = np.ascontiguousarray(dst, dtype=np.uint32)
    co = np.zeros(len(dst) + 1, dtype=np.uint32)
    e = lib().orc_init_co_rate(_p(g_co), _p(dst), C.c_uint32(len(dst)), C.c_float(sample_rate), C.c_int(lower_fanout),
                               _p(co))
    return co, int(e)


def sample_hop(g_co, g_ri, dst, fanout, co, seed, hop):
    dst = np.ascontiguousarray(dst, dtype=np.uint32)
    e = int(co[-1])
    ri = np.zeros(max(e, 1), dtype=np.uint32)
    lib().orc_sample_hop(_p(g_co), _p(g_ri), _p(dst), C.c_uint32(len(dst)), C.c_int(fanout), _p(co),
                         C.c_uint64(seed), C.c_uint32(hop), _p(ri))
    return ri[:e]


def dedup_reindex(V, row_indices_global):
    ri = np.ascontiguousarray(row_indices_global, dtype=np.uint32).copy()
    e = len(ri)
    src = np.zeros(max(1, min(V, e)), dtype=np.uint32)
    s = lib().orc_dedup_reindex(C.c_uint32(V), _p(ri), C.c_uint32(e), _p(src))
    return src[:s].copy(), ri


def csr_from_csc(co, ri_local, s):
    v = len(co) - 1
    e = int(co[-1])
    ro = np.zeros(s + 1, dtype=np.uint32)
    ci = np.zeros(max(e, 1), dtype=np.uint32)
    lib().orc_csr_from_csc(_p(co), _p(ri_local), C.c_uint32(v), C.c_uint32(s), _p(ro), _p(ci))
    return ro, ci[:e]


def block_weights(co, ri, ro, ci):
    v, s, e = len(co) - 1, len(ro) - 1, int(co[-1])
    sn = np.zeros(max(s, 1), dtype=np.float32)
    dn = np.zeros(max(v, 1), dtype=np.float32)
    wf = np.zeros(max(e, 1), dtype=np.float32)
    wb = np.zeros(max(e, 1), dtype=np.float32)
    lib().orc_block_weights(_p(co), _p(ri), _p(ro), _p(ci), C.c_uint32(v), C.c_uint32(s), _p(sn), _p(dn), _p(wf),
                            _p(wb))
    return sn[:s], dn[:v], wf[:e], wb[:e]


class Block:
    """One sampled block as the reference's sampCSC holds it (core/coocsc.hpp:792-813)."""
    pass


def build_block(V, dst, co, ri_global):
    b = Block()
    b.destination = np.ascontiguousarray(dst, dtype=np.uint32)
    b.column_offset = co
    b.v_size = len(dst)
    b.e_size = int(co[-1])
    b.source, b.row_indices = dedup_reindex(V, ri_global[: b.e_size])
    b.src_size = len(b.source)
    b.row_offset, b.column_indices = csr_from_csc(co, b.row_indices, b.src_size)
    b.src_norm, b.dst_norm, b.edge_weight_forward, b.edge_weight_backward = block_weights(
        co, b.row_indices, b.row_offset, b.column_indices)
    return b


def sample_batch(g_co, g_ri, V, seeds, fanouts, seed, draw=0, raw=None, sample_rate=0.0, lower_fanout=0):
    """Sampler::sample_one (core/ntsSampler.hpp:843-1106): blocks returned input side first.
    ``raw`` (list per hop) injects externally sampled global edge lists; sample_rate > 0 selects the
    degree-proportional counts of the training sampler."""
    dst = np.ascontiguousarray(seeds, dtype=np.uint32)
    blocks, raws = [], []
    for hop, f in enumerate(fanouts):
        co, e = init_co_rate(g_co, dst, sample_rate, lower_fanout) if sample_rate > 0 else init_co(g_co, dst, f)
        rg = raw[hop] if raw is not None else sample_hop(g_co, g_ri, dst, f, co, seed, (draw << 8) | hop)
        raws.append(np.array(rg, dtype=np.uint32, copy=True))
        b = build_block(V, dst, co, rg)
        blocks.append(b)
        dst = b.source
    blocks.reverse()
    return blocks, raws


def spmm_fwd(x, w, ri, co, F=None):
    v = len(co) - 1
    x = np.ascontiguousarray(x, dtype=np.float32)
    F = x.shape[1]
    y = np.zeros((v, F), dtype=np.float32)
    lib().orc_spmm_fwd(_p(x), _p(y), _p(w), _p(ri), _p(co), C.c_uint32(v), C.c_uint32(F))
    return y


def spmm_bwd(gy, w, ro, ci, act=None, scale=1.0):
    s = len(ro) - 1
    gy = np.ascontiguousarray(gy, dtype=np.float32)
    F = gy.shape[1]
    gx = np.zeros((s, F), dtype=np.float32)
    if act is not None:
        act = np.ascontiguousarray(act, dtype=np.float32)
    lib().orc_spmm_bwd(_p(gy), _p(gx), _p(w), _p(ro), _p(ci), C.c_uint32(s), C.c_uint32(F), _p(act),
                       C.c_float(scale))
    return gx


def feature_gather(feat, source, cache=None, hashmap=None):
    feat = np.ascontiguousarray(feat, dtype=np.float32)
    source = np.ascontiguousarray(source, dtype=np.uint32)
    F = feat.shape[1]
    x0 = np.zeros((len(source), F), dtype=np.float32)
    lib().orc_feature_gather(_p(x0), _p(feat), _p(source), C.c_uint32(len(source)), C.c_uint32(F), _p(cache),
                             _p(hashmap))
    return x0


def label_gather(label, dst, label_size=1):
    label = np.ascontiguousarray(label, dtype=np.int64)
    dst = np.ascontiguousarray(dst, dtype=np.uint32)
    out = np.zeros(len(dst) * label_size, dtype=np.int64)
    lib().orc_label_gather(_p(out), _p(label), _p(dst), C.c_uint32(len(dst)), C.c_uint32(label_size))
    return out.reshape(len(dst), label_size) if label_size > 1 else out


def cache_by_degree(out_degree, cache_num):
    out_degree = np.ascontiguousarray(out_degree, dtype=np.uint32)
    V = len(out_degree)
    hm = np.zeros(V, dtype=np.uint32)
    ids = np.zeros(max(cache_num, 1), dtype=np.uint32)
    lib().orc_cache_by_degree(_p(out_degree), C.c_uint32(V), C.c_uint32(cache_num), _p(hm), _p(ids))
    return hm, ids[:cache_num]


def gemm_nn(a, b):
    a = np.ascontiguousarray(a, dtype=np.float32); b = np.ascontiguousarray(b, dtype=np.float32)
    M, K = a.shape; N = b.shape[1]
    c = np.zeros((M, N), dtype=np.float32)
    lib().orc_gemm_nn(_p(a), _p(b), _p(c), C.c_int64(M), C.c_int64(K), C.c_int64(N))
    return c


def gemm_tn(a, b):
    """a: [M x K], b: [M x N] -> a^T b [K x N]."""
    a = np.ascontiguousarray(a, dtype=np.float32); b = np.ascontiguousarray(b, dtype=np.float32)
    M, K = a.shape; N = b.shape[1]
    c = np.zeros((K, N), dtype=np.float32)
    lib().orc_gemm_tn(_p(a), _p(b), _p(c), C.c_int64(M), C.c_int64(K), C.c_int64(N))
    return c


def gemm_nt(a, b):
    """a: [M x N], b: [K x N] -> a b^T [M x K]."""
    a = np.ascontiguousarray(a, dtype=np.float32); b = np.ascontiguousarray(b, dtype=np.float32)
    M, N = a.shape; K = b.shape[0]
    c = np.zeros((M, K), dtype=np.float32)
    lib().orc_gemm_nt(_p(a), _p(b), _p(c), C.c_int64(M), C.c_int64(N), C.c_int64(K))
    return c


def relu_dropout(z, p, seed, layer, step):
    z = np.ascontiguousarray(z, dtype=np.float32).copy()
    lib().orc_relu_dropout(_p(z), C.c_int64(z.size), C.c_float(p), C.c_uint64(seed), C.c_uint32(layer),
                           C.c_uint32(step))
    return z


def softmax_nll(logits, label):
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    label = np.ascontiguousarray(label, dtype=np.int64)
    B, Cn = logits.shape
    d = np.zeros((B, Cn), dtype=np.float32)
    correct = C.c_int64(0)
    loss = lib().orc_softmax_nll(_p(logits), _p(label), C.c_int64(B), C.c_int64(Cn), _p(d), C.byref(correct))
    return float(loss), d, int(correct.value)


def sigmoid_bce(logits, label):
    """Multi-label loss: (mean loss, dlogits, (predicted-and-true, predicted, true))."""
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    label = np.ascontiguousarray(label, dtype=np.int64)
    B, Cn = logits.shape
    d = np.zeros((B, Cn), dtype=np.float32)
    counters = (C.c_int64 * 3)()
    fn = lib().orc_sigmoid_bce
    fn.restype = C.c_float
    loss = fn(_p(logits), _p(label), C.c_int64(B), C.c_int64(Cn), _p(d), counters)
    return float(loss), d, tuple(int(x) for x in counters)


def f1_of(counters):
    """f1_score of one batch (utils/torch_func.hpp:31-60) from its three counters, in float32."""
    tp, pre, tru = counters
    if tp == 0 or pre == 0:
        return 0.0
    precision, recall = np.float32(tp) / np.float32(pre), np.float32(tp) / np.float32(tru)
    return float(np.float32(2) * precision * recall / (precision + recall))


def adam(W, grad, M, V, alpha, b1, b2, eps, wd, b1_t, b2_t):
    lib().orc_adam(_p(W), _p(grad), _p(M), _p(V), C.c_int64(W.size), C.c_float(alpha), C.c_float(b1), C.c_float(b2),
                   C.c_float(eps), C.c_float(wd), C.c_float(b1_t), C.c_float(b2_t))


def philox(c, k):
    out = np.zeros(4, dtype=np.uint32)
    lib().orc_philox(C.c_uint32(c[0]), C.c_uint32(c[1]), C.c_uint32(c[2]), C.c_uint32(c[3]), C.c_uint32(k[0]),
                     C.c_uint32(k[1]), _p(out))
    return out


class GCN:
    """CPU restatement of one GCN_CPU_NEIGHBOR / GCN_GPU_NEIGHBOR training step on given blocks
    (toolkits/GCN_CPU_NEIGHBOR.hpp:225-427): forward, loss, backward, Adam."""

    def __init__(self, layer_sizes, W_flat, lr, wd, drop, seed, b1=0.9, b2=0.999, eps=1e-9, blas=False,
                 multi_label=False):
        self.multi_label = multi_label   # CLASSES > 1: BCE loss; `correct` of train_step is then the batch's F1
        # blas=True routes the dense products through numpy's BLAS (the stand-in for libtorch's CPU mm
        # when the oracle is timed as the host baseline); blas=False uses the plain-C loops.
        self.blas = blas
        self.sizes = list(layer_sizes)
        self.L = len(self.sizes) - 1
        self.offs = [0]
        for i in range(self.L):
            self.offs.append(self.offs[-1] + self.sizes[i] * self.sizes[i + 1])
        self.W = np.array(W_flat, dtype=np.float32, copy=True)
        self.M = np.zeros_like(self.W)
        self.V = np.zeros_like(self.W)
        self.grad = np.zeros_like(self.W)
        self.lr, self.wd, self.drop, self.seed = lr, wd, drop, seed
        self.b1, self.b2, self.eps = b1, b2, eps
        self.b1_t, self.b2_t = np.float32(b1), np.float32(b2)
        self.step = 0

    def w(self, l):
        return self.W[self.offs[l]: self.offs[l + 1]].reshape(self.sizes[l], self.sizes[l + 1])

    def train_step(self, blocks, feat, labels, train=True, cache=None, hashmap=None):
        L = self.L
        p = self.drop if train else 0.0
        scale = 1.0 / (1.0 - p) if p > 0 else 1.0
        X = [feature_gather(feat, blocks[0].source, cache, hashmap)]
        Y = []
        for l in range(L):
            b = blocks[l]
            y = spmm_fwd(X[l], b.edge_weight_forward, b.row_indices, b.column_offset)
            Y.append(y)
            z = (y @ self.w(l)) if self.blas else gemm_nn(y, self.w(l))
            if l < L - 1:
                z = relu_dropout(z, p, self.seed, l, self.step)
            X.append(z)
        if self.multi_label:
            lab = label_gather(labels, blocks[L - 1].destination, label_size=labels.shape[1])
            loss, dZ, counters = sigmoid_bce(X[L], lab.reshape(-1, labels.shape[1]))
            correct = f1_of(counters)
        else:
            lab = label_gather(labels, blocks[L - 1].destination)
            loss, dZ, correct = softmax_nll(X[L], lab)
        if train:
            for l in range(L - 1, -1, -1):
                b = blocks[l]
                self.grad[self.offs[l]: self.offs[l + 1]] = ((Y[l].T @ dZ) if self.blas else gemm_tn(Y[l], dZ)).reshape(-1)
                if l == 0:
                    break
                dY = (dZ @ self.w(l).T) if self.blas else gemm_nt(dZ, self.w(l))
                dZ = spmm_bwd(dY, b.edge_weight_backward, b.row_offset, b.column_indices, act=X[l], scale=scale)
            adam(self.W, self.grad, self.M, self.V, self.lr, self.b1, self.b2, self.eps, self.wd, float(self.b1_t),
                 float(self.b2_t))
            self.b1_t = np.float32(self.b1_t * np.float32(self.b1))
            self.b2_t = np.float32(self.b2_t * np.float32(self.b2))
            self.step += 1
        return loss, correct, Y, X
