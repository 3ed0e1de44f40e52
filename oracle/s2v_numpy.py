"""float64 numpy/scipy restatement of the s2v inference path (TEST INFRASTRUCTURE ONLY).

Used to grade the error of the two fp32 implementations (the CPU checker and the
CUDA library) against a higher-precision answer.  Follows
examples/graph_classification/src/kernel_mean_field.cpp:28-47 (model),
src/nn/msg_pass.cpp:46-67,156-177 (CSR builders) and
src/tensor/cpu_dense_tensor.cpp:177-251 (softmax, argmax).
"""
from __future__ import annotations

import numpy as np
import scipy.sparse as sp


def n2n_csr(num_nodes: int, edge_src, edge_dst):
    """Row y lists the sources x of edges x->y in insertion order, value 1."""
    order = np.argsort(edge_dst, kind="stable")
    row_ptr = np.zeros(num_nodes + 1, np.int64)
    np.cumsum(np.bincount(edge_dst, minlength=num_nodes), out=row_ptr[1:])
    return row_ptr.astype(np.int32), np.asarray(edge_src)[order].astype(np.int32)


def level(row_ptr, col_idx, H, W, X, n_src=None):
    n_rows = len(row_ptr) - 1
    n_src = H.shape[0] if n_src is None else n_src
    A = sp.csr_matrix((np.ones(len(col_idx)), col_idx, row_ptr), shape=(n_rows, n_src))
    z = (A @ H.astype(np.float64)) @ W.astype(np.float64)
    if X is not None:
        z = z + X.astype(np.float64)
    return np.where(z < 0, 0.0, z)


def forward(batch) -> dict:
    N, G = batch.num_nodes, batch.num_graphs
    w = {k: v.astype(np.float64) for k, v in batch.weights.items()}
    row_ptr, col = n2n_csr(N, batch.edge_src, batch.edge_dst)
    A = sp.csr_matrix((np.ones(len(col)), col, row_ptr), shape=(N, N))
    off = batch.graph_offsets()
    S = sp.csr_matrix((np.ones(N), np.arange(N), off), shape=(G, N))
    msg = w["w_n2l"][batch.tags]                       # one-hot X times W_in
    cur = np.where(msg < 0, 0.0, msg)
    levels = [cur]
    for _ in range(batch.levels):
        z = (A @ cur) @ w["p_node_conv"] + msg
        cur = np.where(z < 0, 0.0, z)
        levels.append(cur)
    pooled = S @ cur
    hid = pooled @ w["h1_weight"]
    hid = np.where(hid < 0, 0.0, hid)
    logits = hid @ w["h2_weight"]
    e = np.exp(logits - logits.max(axis=1, keepdims=True))
    probs = e / np.abs(e).sum(axis=1, keepdims=True)
    return {"n2n_row_ptr": row_ptr, "n2n_col_idx": col, "sub_row_ptr": off, "msg": msg,
            "levels": np.stack(levels), "pooled": pooled, "logits": logits, "probs": probs,
            "argmax": logits.argmax(axis=1).astype(np.int32)}
