"""Shard-by-graph inference over several ranks: which graphs a rank owns, and the one exchange of the
path -- the final gather of the per-rank logits and predictions.

Graphs of a batch are independent (block-diagonal adjacency), so a batch is split into contiguous
ranges of graphs balanced by node count (`synth.shard_bounds`) and every rank runs the classifier on its
own range with a replica of the weights; no collective runs during levels, pooling or readout.  The
gather is ragged (ranks own different numbers of graphs).  On GPUs it goes through the library's C ABI
(`s2v_gather_logits`, NCCL broadcasts in one group); the torch.distributed form below exists so that the
same logic can run on CPU ranks (gloo) in the tests.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist

from . import synth


def shard_counts(nodes_per_graph: np.ndarray, world: int) -> list[int]:
    """Graphs owned by each rank."""
    return [hi - lo for lo, hi in synth.shard_bounds(nodes_per_graph, world)]


def shard_of(batch, rank: int, world: int):
    """This rank's contiguous range of graphs as a batch of its own (weights shared)."""
    return batch if world == 1 else batch.shard(rank, world)


class ResultGather:
    """Gathers [G_r x C] logits and [G_r] predictions of all ranks, in rank order, onto every rank."""

    def __init__(self, counts: list[int], num_class: int, device, comm=None, group=None):
        self.counts = [int(c) for c in counts]
        self.total = sum(self.counts)
        self.num_class = num_class
        self.comm = comm          # capi.Comm (NCCL through the C ABI) or None (torch.distributed)
        self.group = group
        self.logits_all = torch.empty((self.total, num_class), dtype=torch.float32, device=device)
        self.pred_all = torch.empty((self.total,), dtype=torch.int32, device=device)

    def __call__(self, logits_local: torch.Tensor, pred_local: torch.Tensor, stream=None):
        if self.comm is not None:
            self.comm.gather_logits(self.counts, logits_local, pred_local, self.logits_all, self.pred_all, stream)
            return self.logits_all, self.pred_all
        world = len(self.counts)
        if world == 1:
            self.logits_all.copy_(logits_local)
            self.pred_all.copy_(pred_local)
            return self.logits_all, self.pred_all
        # torch.distributed has no ragged all-gather: pad every rank's rows to the largest shard
        most = max(self.counts)
        lp = torch.zeros((most, self.num_class), dtype=torch.float32, device=logits_local.device)
        pp = torch.zeros((most,), dtype=torch.int32, device=logits_local.device)
        lp[: logits_local.shape[0]] = logits_local
        pp[: pred_local.shape[0]] = pred_local
        lg = [torch.zeros_like(lp) for _ in range(world)]
        pg = [torch.zeros_like(pp) for _ in range(world)]
        dist.all_gather(lg, lp, group=self.group)
        dist.all_gather(pg, pp, group=self.group)
        off = 0
        for r, c in enumerate(self.counts):
            self.logits_all[off:off + c] = lg[r][:c]
            self.pred_all[off:off + c] = pg[r][:c]
            off += c
        return self.logits_all, self.pred_all
