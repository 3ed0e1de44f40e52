"""Files of the reference's graph-classification example: text data sets and checkpoints.

* text data set (examples/graph_classification/data/README.md:1-8): ``N``, then per graph ``n l`` and
  n lines ``t m j_1 .. j_m`` (tag, degree, 0-based neighbour ids).
* checkpoint written by ``ParamSet::Save`` (src/nn/param_set.cpp:28-54): the parameters in
  ``std::map`` (byte-wise name) order, each as ``[rank:u64][dims:u64 x rank][mem_size:u64][fp32 x mem_size]``
  (src/tensor/tensor.cpp:15-29, src/tensor/cpu_dense_tensor.cpp:72-88).
"""
from __future__ import annotations

import struct

import numpy as np

# name in the driver (kernel_mean_field.cpp:14-17) -> key used by this package
MODEL_NAMES = {"input-node-to-latent": "w_n2l", "linear-node-conv": "p_node_conv", "h1_weight": "h1_weight",
               "h2_weight": "h2_weight"}


def write_model(path: str, weights: dict) -> None:
    with open(path, "wb") as f:
        for name in sorted(MODEL_NAMES):                      # std::map order
            w = np.ascontiguousarray(weights[MODEL_NAMES[name]], np.float32)
            f.write(struct.pack("<Q", w.ndim))
            f.write(struct.pack(f"<{w.ndim}Q", *w.shape))
            f.write(struct.pack("<Q", w.size))
            f.write(w.tobytes())


def read_model(path: str) -> dict:
    out = {}
    with open(path, "rb") as f:
        for name in sorted(MODEL_NAMES):
            (rank,) = struct.unpack("<Q", f.read(8))
            dims = struct.unpack(f"<{rank}Q", f.read(8 * rank))
            (mem,) = struct.unpack("<Q", f.read(8))
            data = np.frombuffer(f.read(4 * mem), np.float32)
            n = int(np.prod(dims))
            out[MODEL_NAMES[name]] = data[:n].reshape(dims).copy()
        assert f.read(1) == b"", "trailing bytes in the checkpoint"
    return out


def write_txt_dataset(path: str, graphs: list, labels) -> None:
    """graphs: list of (tags[int], adjacency[list of neighbour lists])."""
    with open(path, "w") as f:
        f.write(f"{len(graphs)}\n")
        for (tags, adj), l in zip(graphs, labels):
            f.write(f"{len(tags)} {int(l)}\n")
            for t, nb in zip(tags, adj):
                f.write(" ".join(str(int(v)) for v in (t, len(nb), *nb)) + "\n")


def read_txt_dataset(path: str):
    """Returns (graphs, labels) with graphs as (tags ndarray, list of neighbour ndarrays)."""
    tok = iter(open(path).read().split())
    n_graphs = int(next(tok))
    graphs, labels = [], []
    for _ in range(n_graphs):
        n, l = int(next(tok)), int(next(tok))
        tags, adj = np.zeros(n, np.int32), []
        for j in range(n):
            tags[j] = int(next(tok))
            m = int(next(tok))
            adj.append(np.fromiter((int(next(tok)) for _ in range(m)), np.int32, m))
        graphs.append((tags, adj))
        labels.append(l)
    return graphs, np.asarray(labels, np.int32)


def graphs_of_batch(batch):
    """GraphBatch -> list of (tags, adjacency) per graph, neighbour lists in AddEdge order."""
    off = batch.graph_offsets().astype(np.int64)
    order_ptr = np.searchsorted(batch.edge_src, np.arange(batch.num_nodes + 1))
    graphs = []
    for g in range(batch.num_graphs):
        lo, hi = off[g], off[g + 1]
        adj = [batch.edge_dst[order_ptr[v]:order_ptr[v + 1]] - lo for v in range(lo, hi)]
        graphs.append((batch.tags[lo:hi], adj))
    return graphs
