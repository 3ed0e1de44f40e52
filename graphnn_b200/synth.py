"""Seeded synthetic inputs with the shapes of the graph-kernel benchmark sets.

The reference evaluates on MUTAG / ENZYMES / NCI1 / NCI109 / D&D text files; these
generators stand in for them (same node-count ranges, degrees, tag counts) so that
every run on every machine sees identical bits.  All randomness comes from
``numpy.random.default_rng(seed)`` (PCG64).

A batch is described the way the reference's batcher builds it
(examples/graph_classification/include/nn_common.h:36-105): graphs are laid out
one after another in a global node numbering, and the directed edge list is in the
order ``GraphStruct::AddEdge`` would see it -- graph by graph, source node
ascending, neighbour ascending.
"""
from __future__ import annotations

import hashlib
import math
from dataclasses import dataclass, field

import numpy as np


@dataclass
class GraphBatch:
    """A block-diagonal batch of small graphs plus the classifier's weights."""

    nodes_per_graph: np.ndarray  # int32 [G]
    edge_src: np.ndarray         # int32 [E]  directed edge x -> y, AddEdge order
    edge_dst: np.ndarray         # int32 [E]
    tags: np.ndarray             # int32 [N]  node type, 0-based
    num_tags: int                # F
    d: int                       # latent dimension
    levels: int                  # L
    hidden: int
    num_class: int
    weights: dict = field(default_factory=dict)  # w_n2l [F,d], p_node_conv [d,d], h1 [d,hidden], h2 [hidden,C]
    name: str = ""

    @property
    def num_graphs(self) -> int:
        return int(self.nodes_per_graph.shape[0])

    @property
    def num_nodes(self) -> int:
        return int(self.nodes_per_graph.sum())

    @property
    def num_edges(self) -> int:
        return int(self.edge_src.shape[0])

    def dense_x(self) -> np.ndarray:
        """One-hot node features [N x F], as GetBatch fills x_cpu (nn_common.h:57-70)."""
        x = np.zeros((self.num_nodes, self.num_tags), dtype=np.float32)
        x[np.arange(self.num_nodes), self.tags] = 1.0
        return x

    def graph_offsets(self) -> np.ndarray:
        """Exclusive prefix sums of the node counts, int32 [G+1]."""
        off = np.zeros(self.num_graphs + 1, dtype=np.int64)
        np.cumsum(self.nodes_per_graph, out=off[1:])
        return off.astype(np.int32)

    def digest(self) -> str:
        h = hashlib.sha256()
        for a in (self.nodes_per_graph, self.edge_src, self.edge_dst, self.tags):
            h.update(np.ascontiguousarray(a).tobytes())
        for k in sorted(self.weights):
            h.update(np.ascontiguousarray(self.weights[k]).tobytes())
        return h.hexdigest()[:16]

    def shard(self, rank: int, world: int) -> "GraphBatch":
        """Contiguous range of graphs for `rank`, balanced by node count; weights are shared."""
        lo, hi = shard_bounds(self.nodes_per_graph, world)[rank]
        off = self.graph_offsets().astype(np.int64)
        n_lo, n_hi = off[lo], off[hi]
        sel = (self.edge_src >= n_lo) & (self.edge_src < n_hi)
        return GraphBatch(
            nodes_per_graph=self.nodes_per_graph[lo:hi].copy(),
            edge_src=(self.edge_src[sel] - n_lo).astype(np.int32),
            edge_dst=(self.edge_dst[sel] - n_lo).astype(np.int32),
            tags=self.tags[n_lo:n_hi].copy(),
            num_tags=self.num_tags, d=self.d, levels=self.levels, hidden=self.hidden,
            num_class=self.num_class, weights=self.weights, name=f"{self.name}[{rank}/{world}]")


def shard_bounds(nodes_per_graph: np.ndarray, world: int) -> list[tuple[int, int]]:
    """Split graphs 0..G into `world` contiguous ranges with near-equal node totals."""
    G = int(nodes_per_graph.shape[0])
    cum = np.cumsum(nodes_per_graph.astype(np.int64))
    total = int(cum[-1]) if G else 0
    cuts = [0]
    for r in range(1, world):
        target = total * r / world
        cuts.append(int(np.searchsorted(cum, target, side="left")) + 1 if G else 0)
    cuts.append(G)
    for i in range(1, len(cuts)):
        cuts[i] = min(max(cuts[i], cuts[i - 1]), G)
    return [(cuts[i], cuts[i + 1]) for i in range(world)]


def _weights(rng, F, d, hidden, C, std):
    def n(*shape):
        return (rng.standard_normal(shape, dtype=np.float32) * np.float32(std)).astype(np.float32)
    return {"w_n2l": n(F, d), "p_node_conv": n(d, d), "h1_weight": n(d, hidden), "h2_weight": n(hidden, C)}


def _finish(name, sizes, und_src, und_dst, tags, F, d, L, hidden, C, rng, std, weight_seed=None):
    """Symmetrise undirected edges (global ids) and order them as GetBatch would add them.
    Weights continue the graph generator's stream unless `weight_seed` names their own."""
    if weight_seed is not None:
        rng = np.random.default_rng(weight_seed)
    s = np.concatenate([und_src, und_dst]).astype(np.int64)
    t = np.concatenate([und_dst, und_src]).astype(np.int64)
    N = int(sizes.sum())
    order = np.argsort(s * N + t, kind="stable")
    return GraphBatch(nodes_per_graph=sizes.astype(np.int32), edge_src=s[order].astype(np.int32),
                      edge_dst=t[order].astype(np.int32), tags=tags.astype(np.int32), num_tags=F, d=d, levels=L,
                      hidden=hidden, num_class=C, weights=_weights(rng, F, d, hidden, C, std), name=name)


def _tree_plus_extra(rng, n: int, extra_frac: float):
    """Random spanning tree (node i>0 attaches to a uniform earlier node) plus
    ceil(extra_frac*(n-1)) distinct random non-tree edges; returns (u, v) with u < v."""
    if n <= 1:
        return np.zeros(0, np.int64), np.zeros(0, np.int64)
    child = np.arange(1, n, dtype=np.int64)
    parent = (rng.random(n - 1) * child).astype(np.int64)  # uniform over 0..i-1
    have = set((int(p) * n + int(c)) for p, c in zip(parent, child))
    want = min(int(math.ceil(extra_frac * (n - 1))), n * (n - 1) // 2 - (n - 1))
    eu, ev = [], []
    while len(eu) < want:
        a, b = rng.integers(0, n, size=2)
        a, b = int(min(a, b)), int(max(a, b))
        if a == b or (a * n + b) in have:
            continue
        have.add(a * n + b)
        eu.append(a)
        ev.append(b)
    return np.concatenate([parent, np.asarray(eu, np.int64)]), np.concatenate([child, np.asarray(ev, np.int64)])


def molecule_like(num_graphs, n_lo, n_hi, num_tags, d, levels, hidden, num_class, weight_std, tag_dist="uniform",
                  seed=0, name="molecule", weight_seed=None) -> GraphBatch:
    rng = np.random.default_rng(seed)
    sizes = rng.integers(n_lo, n_hi + 1, size=num_graphs).astype(np.int64)
    us, vs = [], []
    off = 0
    for n in sizes:
        u, v = _tree_plus_extra(rng, int(n), 0.1)
        us.append(u + off)
        vs.append(v + off)
        off += int(n)
    N = int(sizes.sum())
    if tag_dist == "uniform":
        tags = rng.integers(0, num_tags, size=N)
    else:  # Zipf with exponent tag_dist over ranks 1..num_tags
        p = 1.0 / np.arange(1, num_tags + 1, dtype=np.float64) ** float(tag_dist)
        tags = rng.choice(num_tags, size=N, p=p / p.sum())
    return _finish(name, sizes, np.concatenate(us), np.concatenate(vs), tags, num_tags, d, levels, hidden,
                   num_class, rng, weight_std, weight_seed)


def mutag_like(seed=0, num_graphs=64) -> GraphBatch:
    """64 graphs, 10..28 nodes, tree + 10 % edges, 7 uniform tags, d 64, 3 levels, hidden 128, 2 classes."""
    return molecule_like(num_graphs, 10, 28, 7, 64, 3, 128, 2, 0.1, "uniform", seed, "mutag_like")


def molecules_16k(seed=0, num_graphs=16384, weight_seed=None) -> GraphBatch:
    """16,384 graphs, 20..40 nodes, tree + 10 % edges, 82 tags ~ Zipf(1.2), d 128, 4 levels, hidden 256."""
    return molecule_like(num_graphs, 20, 40, 82, 128, 4, 256, 2, 0.05, 1.2, seed, "molecules_16k", weight_seed)


def proteins_4k(seed=0, num_graphs=4096, n_lo=100, n_hi=620, weight_seed=None) -> GraphBatch:
    """Random geometric graphs in the unit cube, radius for mean degree ~7.4, 3 uniform tags, d 64, 5 levels."""
    rng = np.random.default_rng(seed)
    sizes = rng.integers(n_lo, n_hi + 1, size=num_graphs).astype(np.int64)
    us, vs = [], []
    off = 0
    for n in sizes:
        n = int(n)
        pts = rng.random((n, 3), dtype=np.float32)
        r2 = np.float32((7.4 * 3.0 / (4.0 * math.pi * n)) ** (2.0 / 3.0))
        diff = pts[:, None, :] - pts[None, :, :]
        close = np.triu((diff * diff).sum(-1) < r2, 1)
        u, v = np.nonzero(close)
        us.append(u.astype(np.int64) + off)
        vs.append(v.astype(np.int64) + off)
        off += n
    tags = rng.integers(0, 3, size=int(sizes.sum()))
    return _finish("proteins_4k", sizes, np.concatenate(us), np.concatenate(vs), tags, 3, 64, 5, 128, 2, rng, 0.05,
                   weight_seed)


@dataclass
class LevelProblem:
    """One message-passing level on a single large graph: out = ReLU((A H) W + X)."""

    n_rows: int
    n_src: int
    row_ptr: np.ndarray  # int32 [n_rows+1] (int64 when nnz >= 2^31)
    col_idx: np.ndarray  # int32 [nnz]
    H: np.ndarray        # float32 [n_src, d]
    W: np.ndarray        # float32 [d, d]
    X: np.ndarray | None # float32 [n_rows, d]
    name: str = ""

    @property
    def d(self) -> int:
        return int(self.W.shape[0])

    @property
    def nnz(self) -> int:
        return int(self.col_idx.shape[0])


def csr_from_edges(n_rows: int, src: np.ndarray, dst: np.ndarray):
    """Row `dst` lists `src` in input order (stable), i.e. in-neighbour CSR."""
    order = np.argsort(dst, kind="stable")
    counts = np.bincount(dst, minlength=n_rows)
    row_ptr = np.zeros(n_rows + 1, dtype=np.int64)
    np.cumsum(counts, out=row_ptr[1:])
    return row_ptr.astype(np.int32 if row_ptr[-1] < 2**31 else np.int64), src[order].astype(np.int32)


def erdos_renyi_level(n=1 << 20, nnz=1 << 23, d=64, w_std=0.1, with_x=True, seed=0) -> LevelProblem:
    """Directed G(n, m): `nnz` (src, dst) pairs uniform over n^2, duplicates kept, rows unsorted."""
    rng = np.random.default_rng(seed)
    src = rng.integers(0, n, size=nnz, dtype=np.int64)
    dst = rng.integers(0, n, size=nnz, dtype=np.int64)
    row_ptr, col = csr_from_edges(n, src, dst)
    H = rng.standard_normal((n, d), dtype=np.float32)
    W = (rng.standard_normal((d, d), dtype=np.float32) * np.float32(w_std)).astype(np.float32)
    X = rng.standard_normal((n, d), dtype=np.float32) if with_x else None
    return LevelProblem(n, n, row_ptr, col, H, W, X, f"er_n{n}_m{nnz}_d{d}")


def rmat_edges(scale: int, num_edges: int, a=0.57, b=0.19, c=0.19, seed=0, chunk=1 << 24):
    """R-MAT edge list (src, dst) as int64 arrays; quadrant picked independently per bit."""
    rng = np.random.default_rng(seed)
    src = np.zeros(num_edges, dtype=np.int64)
    dst = np.zeros(num_edges, dtype=np.int64)
    for lo in range(0, num_edges, chunk):
        hi = min(num_edges, lo + chunk)
        s = np.zeros(hi - lo, dtype=np.int64)
        t = np.zeros(hi - lo, dtype=np.int64)
        for _ in range(scale):
            r = rng.random(hi - lo)
            right = ((r >= a) & (r < a + b)) | (r >= a + b + c)   # quadrants b and d set the column bit
            down = r >= a + b                                      # quadrants c and d set the row bit
            s = (s << 1) | down
            t = (t << 1) | right
        src[lo:hi] = s
        dst[lo:hi] = t
    return src, dst


def rmat_level(scale=20, edge_factor=16, d=128, w_std=0.05, seed=0) -> LevelProblem:
    """Symmetrised, deduplicated R-MAT(0.57, 0.19, 0.19, 0.05) graph (self loops kept), no X term."""
    n = 1 << scale
    s, t = rmat_edges(scale, n * edge_factor, seed=seed)
    key = np.unique(np.concatenate([s * n + t, t * n + s]))
    dst, src = key // n, key % n      # sorted by (row, col)
    counts = np.bincount(dst, minlength=n)
    row_ptr = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(counts, out=row_ptr[1:])
    rng = np.random.default_rng(seed + 1)
    H = rng.standard_normal((n, d), dtype=np.float32)
    W = (rng.standard_normal((d, d), dtype=np.float32) * np.float32(w_std)).astype(np.float32)
    rp = row_ptr.astype(np.int32 if row_ptr[-1] < 2**31 else np.int64)
    return LevelProblem(n, n, rp, src.astype(np.int32), H, W, None, f"rmat_s{scale}_d{d}")
