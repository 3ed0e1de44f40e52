"""Host-side driver of the s2v inference path on one GPU.

Mirrors what the reference's driver does per batch (GetBatch + FeedForward,
examples/graph_classification/include/nn_common.h:36-135): build the node-to-node
CSR and the graph ranges from a batch description, place them on the device and run
the classifier.  All arithmetic happens in libs2v_b200.so; torch only owns memory.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from . import capi


@dataclass
class HostBatch:
    """CSR form of a batch in pinned host memory (what the host-buffer entry point consumes)."""

    num_graphs: int
    num_nodes: int
    row_ptr: torch.Tensor    # int32 [N+1], pinned
    col_idx: torch.Tensor    # int32 [E], pinned
    graph_ptr: torch.Tensor  # int32 [G+1], pinned
    tags: torch.Tensor       # int32 [N], pinned
    max_graph_nodes: int = 0 # node count of the largest graph (0 = unknown)

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.row_ptr, self.col_idx, self.graph_ptr, self.tags))


@dataclass
class DeviceBatch:
    num_graphs: int
    num_nodes: int
    row_ptr: torch.Tensor
    col_idx: torch.Tensor
    graph_ptr: torch.Tensor
    tags: torch.Tensor | None
    x_dense: torch.Tensor | None = None
    val: torch.Tensor | None = None
    max_graph_nodes: int = 0


def _pin(a: np.ndarray) -> torch.Tensor:
    t = torch.from_numpy(np.ascontiguousarray(a))
    return t.pin_memory() if torch.cuda.is_available() else t


def build_host_batch(batch) -> HostBatch:
    """GraphBatch -> CSR arrays, through the library's host builder (bit-identical to
    Node2NodeMsgPass / SubgraphMsgPass::InitCPUWeight, src/nn/msg_pass.cpp:46-67,156-177)."""
    row_ptr, col_idx, _ = capi.build_n2n_csr_host(batch.num_nodes, batch.edge_src, batch.edge_dst, with_val=False)
    return HostBatch(batch.num_graphs, batch.num_nodes, _pin(row_ptr), _pin(col_idx), _pin(batch.graph_offsets()),
                     _pin(batch.tags.astype(np.int32)), int(batch.nodes_per_graph.max()) if batch.num_graphs else 0)


class S2VInference:
    """The classifier of kernel_mean_field.cpp:28-47 with weights resident on one GPU."""

    def __init__(self, weights: dict, levels: int, device: int = 0, pool_average: bool = False):
        self.ctx = capi.Context(device)
        self.device = torch.device("cuda", device)
        self.levels = levels
        self.w = {k: torch.from_numpy(np.ascontiguousarray(v, np.float32)).to(self.device) for k, v in weights.items()}
        self.model = self.ctx.make_model(levels, self.w["w_n2l"], self.w["p_node_conv"], self.w["h1_weight"],
                                         self.w["h2_weight"], pool_average)
        self.d = int(self.w["w_n2l"].shape[1])
        self.num_class = int(self.w["h2_weight"].shape[1])
        self._ws = None

    def to_device(self, hb: HostBatch, dense_x: np.ndarray | None = None) -> DeviceBatch:
        dev = self.device
        x = None if dense_x is None else torch.from_numpy(dense_x).to(dev)
        return DeviceBatch(hb.num_graphs, hb.num_nodes, hb.row_ptr.to(dev), hb.col_idx.to(dev), hb.graph_ptr.to(dev),
                           None if dense_x is not None else hb.tags.to(dev), x, None, hb.max_graph_nodes)

    def _workspace(self, n: int, g: int) -> torch.Tensor:
        need = self.ctx.workspace_bytes(n, g, self.d)
        if self._ws is None or self._ws.numel() < need:
            self._ws = torch.empty(need, dtype=torch.uint8, device=self.device)
        return self._ws

    def forward(self, db: DeviceBatch, want_embed: bool = False, stream=None):
        """Runs on `stream` (raw cudaStream_t; None = the context's stream).  Returns device tensors."""
        G, N = db.num_graphs, db.num_nodes
        logits = torch.empty((G, self.num_class), dtype=torch.float32, device=self.device)
        probs = torch.empty_like(logits)
        pred = torch.empty((G,), dtype=torch.int32, device=self.device)
        embed = torch.empty((N, self.d), dtype=torch.float32, device=self.device) if want_embed else None
        cb = self.ctx.make_batch(G, N, db.row_ptr, db.col_idx, db.val, db.graph_ptr, db.tags, db.x_dense,
                                 db.max_graph_nodes)
        self.ctx.forward(self.model, cb, self._workspace(N, G), logits, probs, pred, embed, stream=stream)
        return logits, probs, pred, embed

    def infer_host(self, hb: HostBatch, logits_out: np.ndarray | None = None, pred_out: np.ndarray | None = None):
        """Host buffers in, host buffers out: uploads, forward, download (one blocking call)."""
        G = hb.num_graphs
        if logits_out is None:
            logits_out = np.empty((G, self.num_class), np.float32)
        if pred_out is None:
            pred_out = np.empty((G,), np.int32)
        cb = self.ctx.make_batch(G, hb.num_nodes, hb.row_ptr, hb.col_idx, None, hb.graph_ptr, hb.tags, None)
        self.ctx.infer_host(self.model, cb, logits_out, pred_out)
        return logits_out, pred_out
