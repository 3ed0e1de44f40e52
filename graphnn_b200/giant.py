"""One giant graph, row-partitioned over the ranks of a job.

Rank p owns rows [p*N/P, (p+1)*N/P) of the CSR matrix A (all columns) and of every
embedding matrix.  A level needs the whole H as its gather source, so each level is

    all-gather of the [N/P x d] slabs  ->  fused level kernel on the local rows (n_src = N)

The only exchange step of the path is that all-gather (NCCL over NVLink; the reference has
no multi-GPU code at all).  It is pipelined against the compute: the local rows are cut
into `chunks` row blocks and block k of level l is all-gathered (on a side stream) while
block k+1 is still being computed, so that level l+1 finds H complete soon after level l's
last block.  Remote rows always land in local HBM first; the kernel never reads peer memory.

The compute step is injectable (`level_fn`) so that the partition / exchange logic can be
exercised on CPU ranks (gloo) with any reference implementation of a level.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch
import torch.distributed as dist


def row_range(n_rows: int, rank: int, world: int) -> tuple[int, int]:
    """Equal row slabs (N must be divisible by the world size; pad the graph otherwise)."""
    if n_rows % world:
        raise ValueError(f"{n_rows} rows do not divide over {world} ranks; pad the graph with isolated nodes")
    per = n_rows // world
    return rank * per, (rank + 1) * per


@dataclass
class CsrShard:
    """Rows [row_lo, row_hi) of a CSR matrix with n_cols columns; row_ptr is rebased to 0."""

    row_lo: int
    row_hi: int
    n_cols: int
    row_ptr: torch.Tensor   # int32 or int64 [rows+1]
    col_idx: torch.Tensor   # int32 [nnz_local]

    @property
    def rows(self) -> int:
        return self.row_hi - self.row_lo

    @property
    def nnz(self) -> int:
        return int(self.col_idx.shape[0])


def shard_csr(row_ptr: np.ndarray, col_idx: np.ndarray, n_cols: int, rank: int, world: int, device=None) -> CsrShard:
    n_rows = len(row_ptr) - 1
    lo, hi = row_range(n_rows, rank, world)
    rp = row_ptr[lo:hi + 1].astype(np.int64)
    base = int(rp[0])
    ci = col_idx[base:int(rp[-1])]
    rp = rp - base
    rp = rp.astype(np.int32 if rp[-1] < 2 ** 31 else np.int64)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device) if device is not None else torch.from_numpy(np.ascontiguousarray(a))
    return CsrShard(lo, hi, n_cols, t(rp), t(ci.astype(np.int32)))


def rmat_shard_on_device(scale: int, num_edges: int, rank: int, world: int, device, a=0.57, b=0.19, c=0.19, seed=0,
                         chunk=1 << 26, relabel: bool = True) -> CsrShard:
    """Symmetrised, deduplicated R-MAT(a,b,c,d) graph with 2^scale nodes, generated on the
    device: every rank draws the same edge stream (counter-based: the generator is re-seeded
    per chunk with (seed, chunk index)) and keeps the directed copies whose row falls in its
    slab, then sorts and deduplicates only those.  Self loops are kept as generated.

    R-MAT puts its heavy rows at the node ids with many zero bits, i.e. mostly in the first row slab.
    With `relabel` every node id v is replaced by (v * 0x9E3779B1) mod 2^scale -- a bijection (the
    multiplier is odd), i.e. the same graph with its nodes renumbered -- which spreads the heavy rows
    evenly over equal row slabs, so that equal row counts are also nearly equal work."""
    n = 1 << scale
    mult = 0x9E3779B1
    lo, hi = row_range(n, rank, world)
    keys = []
    gen = torch.Generator(device=device)
    for ci, start in enumerate(range(0, num_edges, chunk)):
        m = min(chunk, num_edges - start)
        gen.manual_seed(seed * 1000003 + ci)
        s = torch.zeros(m, dtype=torch.int64, device=device)
        t = torch.zeros(m, dtype=torch.int64, device=device)
        for _ in range(scale):
            r = torch.rand(m, device=device, generator=gen)
            right = ((r >= a) & (r < a + b)) | (r >= a + b + c)
            down = r >= a + b
            s = (s << 1) | down
            t = (t << 1) | right
        if relabel:
            s = (s * mult) & (n - 1)
            t = (t * mult) & (n - 1)
        for row, col in ((s, t), (t, s)):
            keep = (row >= lo) & (row < hi)
            keys.append(((row[keep] - lo) << scale) | col[keep])
        del s, t, r, right, down, keep
    key = torch.unique(torch.cat(keys))          # sorted by (local row, column), duplicates removed
    del keys
    rows_local = key >> scale
    col = (key & (n - 1)).to(torch.int32)
    counts = torch.bincount(rows_local, minlength=hi - lo)
    row_ptr = torch.zeros(hi - lo + 1, dtype=torch.int64, device=device)
    torch.cumsum(counts, 0, out=row_ptr[1:])
    if int(row_ptr[-1]) < 2 ** 31:
        row_ptr = row_ptr.to(torch.int32)
    return CsrShard(lo, hi, n, row_ptr, col)


@dataclass
class HubPlan:
    """Rows whose degree exceeds a threshold ("hubs" of a power-law graph) would each be summed
    by a single warp.  They are taken out of the level's CSR: a hub row keeps ONE entry that
    points at an extra source row N + h, and that row is filled, before the level runs, by
    two small launches that sum the hub's neighbours in parallel: partial sums over
    sub-rows of `piece` entries (CSR x dense), then an in-order sum of each hub's partials
    (segmented sum).  Deterministic; no atomics."""

    n_hub: int
    light: CsrShard            # the shard with hub rows collapsed to one entry (columns may be >= n_cols)
    sub_row_ptr: torch.Tensor  # int32 [n_sub+1]  sub-rows of the hubs' entries
    sub_col_idx: torch.Tensor  # int32 [hub nnz]
    hub_seg_ptr: torch.Tensor  # int32 [n_hub+1]  consecutive sub-rows of every hub

    @property
    def n_sub(self) -> int:
        return int(self.sub_row_ptr.shape[0]) - 1


def plan_hubs(shard: CsrShard, threshold: int = 2048, piece: int = 512) -> HubPlan | None:
    rp = shard.row_ptr.to(torch.int64)
    deg = rp[1:] - rp[:-1]
    is_hub = deg > threshold
    n_hub = int(is_hub.sum())
    if n_hub == 0:
        return None
    dev = rp.device
    hub_rows = torch.nonzero(is_hub).flatten()
    hub_deg = deg[hub_rows]
    # entries that belong to hub rows, in CSR order
    row_of_edge = torch.repeat_interleave(torch.arange(shard.rows, device=dev), deg)
    edge_is_hub = is_hub[row_of_edge]
    sub_col = shard.col_idx[edge_is_hub].contiguous()
    # sub-rows: every hub is cut into ceil(deg/piece) consecutive pieces
    pieces = (hub_deg + piece - 1) // piece
    hub_seg = torch.zeros(n_hub + 1, dtype=torch.int64, device=dev)
    torch.cumsum(pieces, 0, out=hub_seg[1:])
    n_sub = int(hub_seg[-1])
    hub_of_sub = torch.repeat_interleave(torch.arange(n_hub, device=dev), pieces)
    idx_in_hub = torch.arange(n_sub, device=dev) - hub_seg[hub_of_sub]
    hub_start = torch.zeros(n_hub + 1, dtype=torch.int64, device=dev)
    torch.cumsum(hub_deg, 0, out=hub_start[1:])
    sub_len = torch.minimum(torch.full_like(idx_in_hub, piece), hub_deg[hub_of_sub] - idx_in_hub * piece)
    sub_rp = torch.zeros(n_sub + 1, dtype=torch.int64, device=dev)
    torch.cumsum(sub_len, 0, out=sub_rp[1:])
    # light CSR: hub rows keep one entry -> extra source row n_cols + h
    new_deg = torch.where(is_hub, torch.ones_like(deg), deg)
    light_rp = torch.zeros(shard.rows + 1, dtype=torch.int64, device=dev)
    torch.cumsum(new_deg, 0, out=light_rp[1:])
    light_col = torch.empty(int(light_rp[-1]), dtype=torch.int32, device=dev)
    keep = ~edge_is_hub
    new_pos_light = light_rp[:-1][row_of_edge[keep]] + (torch.arange(shard.nnz, device=dev)[keep] - rp[:-1][row_of_edge[keep]])
    light_col[new_pos_light] = shard.col_idx[keep]
    light_col[light_rp[:-1][hub_rows]] = (shard.n_cols + torch.arange(n_hub, device=dev)).to(torch.int32)
    rp_dtype = torch.int32 if int(light_rp[-1]) < 2 ** 31 else torch.int64
    light = CsrShard(shard.row_lo, shard.row_hi, shard.n_cols, light_rp.to(rp_dtype), light_col)
    return HubPlan(n_hub, light, sub_rp.to(torch.int32), sub_col, hub_seg.to(torch.int32))


class GiantGraphLevels:
    """L levels  H <- ReLU(A*H*W [+ X])  on a row-partitioned graph.

    Layout of a rank's full copy of H.  The local slab is cut into `chunks` row blocks (the same
    cut on every rank); `full` stores the blocks one after another and, inside block k, the ranks
    one after another:  full = [block 0: rank 0 rows | rank 1 rows | ...][block 1: ...] ... [hub rows].
    Block k of all ranks is therefore ONE contiguous range, and its exchange is a single in-place
    all-gather (send = this rank's piece where it already lies) that can start as soon as the local
    rows of block k are computed, while block k+1 is still being computed.  The column indices of the
    shard are renumbered once, at construction, to positions in this layout.

    `exchange(region, piece, rank)` performs that all-gather: `region` is the [world * rows_k, d]
    range of `full`, `piece` this rank's [rows_k, d] part of it.  It is injectable, like the compute
    step: NCCL through the library's C ABI on the GPU, torch.distributed (gloo) in the CPU tests."""

    def __init__(self, shard: CsrShard, d: int, rank: int, world: int, level_fn, chunks: int = 4, group=None,
                 hub_plan: HubPlan | None = None, spmm_fn=None, segsum_fn=None, exchange=None):
        self.hub = hub_plan
        self.spmm_fn, self.segsum_fn = spmm_fn, segsum_fn
        if hub_plan is not None:
            assert spmm_fn is not None and segsum_fn is not None
            shard = hub_plan.light
        self.d, self.rank, self.world, self.level_fn = d, rank, world, level_fn
        self.chunks = max(1, min(chunks, shard.rows))
        self.group = group
        dev = shard.col_idx.device
        self.device = dev
        rows = shard.rows
        self.rows = rows
        self.n = shard.n_cols
        assert self.n == rows * world, "equal row slabs: the number of columns must be world * rows"
        edges = [rows * k // self.chunks for k in range(self.chunks + 1)]
        self.blocks = [(edges[k], edges[k + 1]) for k in range(self.chunks) if edges[k + 1] > edges[k]]
        # position of global row (r * rows + i) in the block-major layout
        self._edges = torch.tensor([lo for lo, _ in self.blocks] + [rows], dtype=torch.int64, device=dev)
        new_col = torch.empty_like(shard.col_idx)
        piece = 1 << 27                                        # renumber in slices: the int64 temporaries stay small
        for lo in range(0, shard.nnz, piece):
            col = shard.col_idx[lo:lo + piece].to(torch.int64)
            real = col < self.n                                # hub rows (>= n) keep their place behind the blocks
            new_col[lo:lo + piece] = torch.where(real, self.position_of(col.clamp(max=self.n - 1)), col).to(torch.int32)
            del col, real
        self.shard = CsrShard(shard.row_lo, shard.row_hi, shard.n_cols, shard.row_ptr, new_col)
        extra = hub_plan.n_hub if hub_plan is not None else 0       # rank-private source rows N .. N+n_hub
        if hub_plan is not None:                                    # the hubs' own column lists use the same layout
            self.hub_cols = self.position_of(hub_plan.sub_col_idx.to(torch.int64)).to(torch.int32)
        # full[0] holds the input H0 and is never written by run(); the levels alternate between full[1] and full[2]
        self.full = [torch.empty((self.n + extra, d), dtype=torch.float32, device=dev) for _ in range(3)]
        self.partial = torch.empty((hub_plan.n_sub, d), dtype=torch.float32, device=dev) if hub_plan is not None else None
        self.comm_stream = torch.cuda.Stream(device=dev) if dev.type == "cuda" else None
        self.exchange = exchange if exchange is not None else self._exchange_torch
        rp = self.shard.row_ptr
        self._block_rp = []
        for lo, hi in self.blocks:
            seg = rp[lo:hi + 1]
            self._block_rp.append((seg - seg[0]).contiguous())
        self._block_base = [int(rp[lo]) for lo, _ in self.blocks]
        self._block_nnz = [int(rp[hi]) - int(rp[lo]) for lo, hi in self.blocks]
        self.timing = None      # set by run(..., timed=True): per level {"compute_ms", "exchange_ms"}

    def all_gather_bytes_per_level(self) -> int:
        return (self.world - 1) * self.rows * self.d * 4

    def _region(self, full: torch.Tensor, k: int):
        lo, hi = self.blocks[k]
        rk = hi - lo
        region = full[self.world * lo:self.world * hi]
        return region, region[self.rank * rk:(self.rank + 1) * rk]

    def _exchange_torch(self, region, piece, rank):
        if self.world == 1:
            return
        if region.device.type == "cuda":
            dist.all_gather_into_tensor(region, piece, group=self.group)
        else:   # gloo: list form on views of the contiguous region
            rk = piece.shape[0]
            dist.all_gather([region[r * rk:(r + 1) * rk] for r in range(self.world)], piece.clone(), group=self.group)

    def set_input(self, slab: torch.Tensor):
        """Local slab of H0 -> full H0 on every rank (block by block)."""
        for k, (lo, hi) in enumerate(self.blocks):
            region, piece = self._region(self.full[0], k)
            piece.copy_(slab[lo:hi])
            self.exchange(region, piece, self.rank)
        self.cur = 0

    def local_slab(self) -> torch.Tensor:
        """This rank's rows of the current H, in row order (a copy)."""
        return torch.cat([self._region(self.full[self.cur], k)[1] for k in range(len(self.blocks))])

    def gather_rows(self, which: int, positions_of_global_rows: torch.Tensor) -> torch.Tensor:
        return self.full[which][positions_of_global_rows]

    def position_of(self, global_rows: torch.Tensor) -> torch.Tensor:
        """Row index inside `full` of the given global node ids (int64 tensor)."""
        r = torch.div(global_rows, self.rows, rounding_mode="floor")
        i = global_rows - r * self.rows
        k = torch.bucketize(i, self._edges[1:], right=True).clamp(max=len(self.blocks) - 1)
        lo_k = self._edges[k]
        rk = self._edges[k + 1] - lo_k
        return self.world * lo_k + r * rk + (i - lo_k)

    def run(self, W: torch.Tensor, levels: int, X_slab: torch.Tensor | None = None, timed: bool = False,
            return_copy: bool = True) -> torch.Tensor | None:
        """Runs `levels` levels from the input set by set_input (which stays intact, so run() can be repeated);
        returns the local slab of H_L in row order (a copy; None with return_copy=False: the result stays in the
        layout's buffer, see local_slab / level_buffers)."""
        cuda = self.comm_stream is not None
        self.timing = [] if timed and cuda else None
        self.cur = 0
        for _ in range(levels):
            nxt = 1 if self.cur != 1 else 2
            src, dst = self.full[self.cur], self.full[nxt]
            events = []
            marks = []
            if timed and cuda:
                t_begin = torch.cuda.Event(enable_timing=True)
                t_begin.record(torch.cuda.current_stream())
            if self.hub is not None:   # hub sums of this level -> the extra source rows of `src`
                n = self.n
                self.spmm_fn(self.hub.sub_row_ptr, self.hub_cols, src[:n], self.partial)
                self.segsum_fn(self.hub.hub_seg_ptr, self.partial, src[n:])
            for k, (lo, hi) in enumerate(self.blocks):
                region, piece = self._region(dst, k)
                base = self._block_base[k]
                nnz = self._block_nnz[k]
                self.level_fn(self._block_rp[k], self.shard.col_idx[base:base + nnz], src, W,
                              None if X_slab is None else X_slab[lo:hi], piece)
                if self.world > 1:
                    if cuda:
                        ev = torch.cuda.Event()
                        ev.record(torch.cuda.current_stream())
                        with torch.cuda.stream(self.comm_stream):
                            self.comm_stream.wait_event(ev)
                            if timed:
                                x0 = torch.cuda.Event(enable_timing=True)
                                x0.record(self.comm_stream)
                            self.exchange(region, piece, self.rank)
                            done = torch.cuda.Event(enable_timing=timed)
                            done.record(self.comm_stream)
                            if timed:
                                marks.append((x0, done))
                        events.append(done)
                    else:
                        self.exchange(region, piece, self.rank)
            if timed and cuda:
                t_compute = torch.cuda.Event(enable_timing=True)
                t_compute.record(torch.cuda.current_stream())
            for ev in events:          # the next level reads every row of dst
                torch.cuda.current_stream().wait_event(ev)
            if timed and cuda:
                t_end = torch.cuda.Event(enable_timing=True)
                t_end.record(torch.cuda.current_stream())
                self.timing.append((t_begin, t_compute, t_end, marks))
            self.cur = nxt
        return self.local_slab() if return_copy else None

    def level_buffers(self, level: int):
        """(input, output) buffers of level `level` (1-based) of the last run()."""
        out = 1 if level % 2 == 1 else 2
        src = 0 if level == 1 else (2 if out == 1 else 1)
        return self.full[src], self.full[out]

    def timing_summary(self) -> list[dict]:
        """After run(..., timed=True) and a synchronise: per level, compute time, time from the end of the
        compute to the end of the last exchange (the exposed part), and the summed exchange time."""
        out = []
        for t_begin, t_compute, t_end, marks in (self.timing or []):
            out.append({"compute_ms": t_begin.elapsed_time(t_compute), "exposed_exchange_ms": t_compute.elapsed_time(t_end),
                        "exchange_ms_sum": float(sum(a.elapsed_time(b) for a, b in marks))})
        return out


def _exchange_lists(lists, rank: int, world: int, group=None):
    """lists[p] (1-D int32 tensors) go to rank p; returns what every rank sent to this one.  Set-up plumbing on
    torch.distributed point-to-point calls (both gloo and nccl have them)."""
    dev = lists[0].device
    counts = torch.tensor([int(l.numel()) for l in lists], dtype=torch.int64, device=dev)
    all_counts = [torch.zeros(world, dtype=torch.int64, device=dev) for _ in range(world)]
    dist.all_gather(all_counts, counts, group=group)
    got = [torch.empty(int(all_counts[p][rank]), dtype=lists[0].dtype, device=dev) for p in range(world)]
    ops = []
    for p in range(world):
        if p == rank:
            got[p] = lists[p].clone()
            continue
        if lists[p].numel():
            ops.append(dist.P2POp(dist.isend, lists[p].contiguous(), p, group))
        if got[p].numel():
            ops.append(dist.P2POp(dist.irecv, got[p], p, group))
    if ops:
        for req in dist.batch_isend_irecv(ops):
            req.wait()
    return got


class GiantGraphReferenced:
    """The same L levels on a row-partitioned graph, but every rank fetches only the rows of H that its own
    rows reference instead of all of H.  On a power-law graph cut into P slabs a rank references a
    fraction of the remote rows that shrinks with P (a quarter at P = 8 on R-MAT scale 26), so the exchange
    volume and the gather table shrink with it.

    Table of a rank:  [own rows 0 .. rows) | referenced remote rows in ascending global order | hub rows].
    At construction every rank tells each owner which of its rows it needs; per level and row block k the
    owner packs, for every peer, the requested rows of block k (one row-lookup launch) and one group of
    sends / receives moves them straight into place in the peers' tables (`exchange_rows`), while block k+1
    is still being computed.  Column indices are renumbered once to positions in the table.

    `pack_fn(idx, table, out)` : out[i, :] = table[idx[i], :]   (the library's row-lookup kernel on the GPU)
    `exchange_rows(send, send_offsets, table, recv_offsets, recv_rows)` : the pairwise exchange
    (s2v_exchange_rows_f32 on the GPU; torch.distributed point-to-point on CPU ranks)."""

    def __init__(self, shard: CsrShard, d: int, rank: int, world: int, level_fn, pack_fn=None, chunks: int = 8, group=None,
                 hub_plan: HubPlan | None = None, spmm_fn=None, segsum_fn=None, exchange_rows=None):
        self.hub = hub_plan
        self.spmm_fn, self.segsum_fn = spmm_fn, segsum_fn
        if hub_plan is not None:
            assert spmm_fn is not None and segsum_fn is not None
            shard = hub_plan.light
        self.d, self.rank, self.world, self.level_fn, self.group = d, rank, world, level_fn, group
        dev = shard.col_idx.device
        self.device = dev
        rows = shard.rows
        self.rows, self.n = rows, shard.n_cols
        assert self.n == rows * world, "equal row slabs: the number of columns must be world * rows"
        self.row_lo = rank * rows
        self.chunks = max(1, min(chunks, rows))
        edges = [rows * k // self.chunks for k in range(self.chunks + 1)]
        self.blocks = [(edges[k], edges[k + 1]) for k in range(self.chunks) if edges[k + 1] > edges[k]]
        cuts = torch.tensor([lo for lo, _ in self.blocks] + [rows], dtype=torch.int64, device=dev)
        piece = 1 << 27
        # which remote rows do my rows (and my hubs' sub-rows) reference?
        mask = torch.zeros(self.n, dtype=torch.bool, device=dev)
        sources = [shard.col_idx] + ([hub_plan.sub_col_idx] if hub_plan is not None else [])
        for src_cols in sources:
            for lo in range(0, int(src_cols.numel()), piece):
                col = src_cols[lo:lo + piece].to(torch.int64)
                mask[col[col < self.n]] = True
                del col
        self.rows_referenced = int(mask.sum())            # own + remote, for the record
        mask[self.row_lo:self.row_lo + rows] = False
        self.need = torch.nonzero(mask).flatten()         # int64 global ids, ascending
        del mask
        self.n_need = int(self.need.numel())
        self.n_table = rows + self.n_need
        # renumber the columns to table positions (hub rows, >= n, move behind the table)
        new_col = torch.empty_like(shard.col_idx)
        for lo in range(0, shard.nnz, piece):
            col = shard.col_idx[lo:lo + piece].to(torch.int64)
            real = col < self.n
            new_col[lo:lo + piece] = torch.where(real, self.position_of(col.clamp(max=self.n - 1)), col - self.n + self.n_table).to(torch.int32)
            del col, real
        self.shard = CsrShard(shard.row_lo, shard.row_hi, shard.n_cols, shard.row_ptr, new_col)
        extra = hub_plan.n_hub if hub_plan is not None else 0
        if hub_plan is not None:
            self.hub_cols = self.position_of(hub_plan.sub_col_idx.to(torch.int64)).to(torch.int32)
        # receive side: rows needed from owner s in block k are need[nb[s][k] : nb[s][k+1]]
        owner_cut = (torch.arange(world, device=dev, dtype=torch.int64) * rows)[:, None] + cuts[None, :]
        nb = torch.searchsorted(self.need, owner_cut.flatten()).reshape(world, len(self.blocks) + 1).cpu().numpy()
        self._recv_rows = [[int(nb[s][k + 1] - nb[s][k]) for s in range(world)] for k in range(len(self.blocks))]
        self._recv_offsets = [[rows + int(nb[s][k]) for s in range(world)] for k in range(len(self.blocks))]
        # send side: every owner learns which of its rows each peer needs
        requests = [(self.need[int(nb[s][0]):int(nb[s][-1])] - s * rows).to(torch.int32) for s in range(world)]
        give = _exchange_lists(requests, rank, world, group) if world > 1 else [requests[0]]
        self._send_idx, self._send_offsets = [], []
        for k in range(len(self.blocks)):
            parts, offs = [], [0]
            for t in range(world):
                if t == rank or give[t].numel() == 0:
                    offs.append(offs[-1])
                    continue
                a, b = torch.searchsorted(give[t], cuts[k:k + 2].to(give[t].dtype)).tolist()
                parts.append(give[t][a:b])
                offs.append(offs[-1] + (b - a))
            self._send_idx.append(torch.cat(parts).contiguous() if parts else torch.empty(0, dtype=torch.int32, device=dev))
            self._send_offsets.append(offs)
        self.rows_sent_per_level = sum(o[-1] for o in self._send_offsets)
        max_send = max((o[-1] for o in self._send_offsets), default=0)
        self.sendbuf = torch.empty((max(max_send, 1), d), dtype=torch.float32, device=dev)
        # full[0] holds the input H0 and is never written by run(); the levels alternate between full[1] and full[2]
        self.full = [torch.empty((self.n_table + extra, d), dtype=torch.float32, device=dev) for _ in range(3)]
        self.partial = torch.empty((hub_plan.n_sub, d), dtype=torch.float32, device=dev) if hub_plan is not None else None
        self.comm_stream = torch.cuda.Stream(device=dev) if dev.type == "cuda" else None
        self.pack_fn = pack_fn if pack_fn is not None else (lambda idx, table, out: torch.index_select(table, 0, idx.to(torch.int64), out=out))
        self.exchange_rows = exchange_rows if exchange_rows is not None else self._exchange_rows_torch
        rp = self.shard.row_ptr
        self._block_rp = []
        for lo, hi in self.blocks:
            seg = rp[lo:hi + 1]
            self._block_rp.append((seg - seg[0]).contiguous())
        self._block_base = [int(rp[lo]) for lo, _ in self.blocks]
        self._block_nnz = [int(rp[hi]) - int(rp[lo]) for lo, hi in self.blocks]
        self.timing = None

    def exchange_bytes_per_level(self) -> int:
        """Bytes this rank receives per level."""
        return self.n_need * self.d * 4

    def position_of(self, global_rows: torch.Tensor) -> torch.Tensor:
        """Row index inside the table of the given global node ids (own rows, or remote rows this rank references)."""
        own = (global_rows >= self.row_lo) & (global_rows < self.row_lo + self.rows)
        far = torch.searchsorted(self.need, global_rows).clamp(max=max(self.n_need - 1, 0))
        return torch.where(own, global_rows - self.row_lo, self.rows + far)

    def _exchange_rows_torch(self, send, send_offsets, table, recv_offsets, recv_rows):
        ops = []
        for p in range(self.world):
            ns = send_offsets[p + 1] - send_offsets[p]
            if p == self.rank:
                continue
            if ns > 0:
                ops.append(dist.P2POp(dist.isend, send[send_offsets[p]:send_offsets[p + 1]].contiguous(), p, self.group))
            if recv_rows[p] > 0:
                ops.append(dist.P2POp(dist.irecv, table[recv_offsets[p]:recv_offsets[p] + recv_rows[p]], p, self.group))
        if ops:
            for req in dist.batch_isend_irecv(ops):
                req.wait()

    def _ship_block(self, table: torch.Tensor, k: int):
        """Pack the rows of block k that the peers asked for and exchange them into place."""
        n_send = self._send_offsets[k][-1]
        send = self.sendbuf[:max(n_send, 1)]
        if n_send > 0:
            self.pack_fn(self._send_idx[k], table[:self.rows], send[:n_send])
        self.exchange_rows(send, self._send_offsets[k], table, self._recv_offsets[k], self._recv_rows[k])

    def set_input(self, slab: torch.Tensor):
        """Local slab of H0 -> this rank's table of H0 (own rows + the referenced remote rows)."""
        self.full[0][:self.rows].copy_(slab)
        if self.world > 1:
            for k in range(len(self.blocks)):
                self._ship_block(self.full[0], k)
        self.cur = 0

    def local_slab(self) -> torch.Tensor:
        return self.full[self.cur][:self.rows].clone()

    def run(self, W: torch.Tensor, levels: int, X_slab: torch.Tensor | None = None, timed: bool = False,
            return_copy: bool = True) -> torch.Tensor | None:
        """Runs `levels` levels from the input set by set_input (which stays intact); returns the local slab of H_L
        (a copy; None with return_copy=False: the result stays in rows 0 .. rows of the current table)."""
        cuda = self.comm_stream is not None
        self.timing = [] if timed and cuda else None
        self.cur = 0
        for _ in range(levels):
            nxt = 1 if self.cur != 1 else 2
            src, dst = self.full[self.cur], self.full[nxt]
            events, marks = [], []
            if timed and cuda:
                t_begin = torch.cuda.Event(enable_timing=True)
                t_begin.record(torch.cuda.current_stream())
            if self.hub is not None:   # hub sums of this level -> the extra source rows of `src`
                nt = self.n_table
                self.spmm_fn(self.hub.sub_row_ptr, self.hub_cols, src[:nt], self.partial)
                self.segsum_fn(self.hub.hub_seg_ptr, self.partial, src[nt:])
            for k, (lo, hi) in enumerate(self.blocks):
                base, nnz = self._block_base[k], self._block_nnz[k]
                self.level_fn(self._block_rp[k], self.shard.col_idx[base:base + nnz], src, W,
                              None if X_slab is None else X_slab[lo:hi], dst[lo:hi])
                if self.world > 1:
                    if cuda:
                        ev = torch.cuda.Event()
                        ev.record(torch.cuda.current_stream())
                        with torch.cuda.stream(self.comm_stream):
                            self.comm_stream.wait_event(ev)
                            if timed:
                                x0 = torch.cuda.Event(enable_timing=True)
                                x0.record(self.comm_stream)
                            self._ship_block(dst, k)
                            done = torch.cuda.Event(enable_timing=timed)
                            done.record(self.comm_stream)
                            if timed:
                                marks.append((x0, done))
                        events.append(done)
                    else:
                        self._ship_block(dst, k)
            if timed and cuda:
                t_compute = torch.cuda.Event(enable_timing=True)
                t_compute.record(torch.cuda.current_stream())
            for ev in events:          # the next level reads the whole table
                torch.cuda.current_stream().wait_event(ev)
            if timed and cuda:
                t_end = torch.cuda.Event(enable_timing=True)
                t_end.record(torch.cuda.current_stream())
                self.timing.append((t_begin, t_compute, t_end, marks))
            self.cur = nxt
        return self.local_slab() if return_copy else None

    level_buffers = GiantGraphLevels.level_buffers
    timing_summary = GiantGraphLevels.timing_summary


def make_comm_exchange_rows(comm):
    """exchange_rows() for GiantGraphReferenced on the library's NCCL entry point (s2v_exchange_rows_f32), on
    torch's current stream."""

    def exchange_rows(send, send_offsets, table, recv_offsets, recv_rows):
        st = torch.cuda.current_stream().cuda_stream
        comm.exchange_rows(send, send_offsets, table, recv_offsets, recv_rows, st)

    return exchange_rows


def make_gpu_pack_fn(ctx):
    """pack_fn() for GiantGraphReferenced: out[i, :] = table[idx[i], :] with the library's row-lookup kernel
    (s2v_input_proj_onehot_f32 without the ReLU output), on torch's current stream."""

    def pack(idx, table, out):
        st = torch.cuda.current_stream().cuda_stream
        assert st != 0
        ctx.input_proj_onehot(idx, table, out, None, stream=st)

    return pack


def make_comm_exchange(comm, stream_getter=None):
    """exchange() for GiantGraphLevels on the library's NCCL entry point (s2v_allgather_rows_f32): one
    contiguous in-place all-gather per block, on torch's current stream."""

    def exchange(region, piece, rank):
        st = torch.cuda.current_stream().cuda_stream
        comm.allgather_rows(piece, region, st)

    return exchange


def make_gpu_hub_fns(ctx):
    """(spmm_fn, segsum_fn) for HubPlan on the library's kernels, torch's current stream."""

    def spmm_fn(row_ptr, col_idx, H, out):
        st = torch.cuda.current_stream().cuda_stream
        assert st != 0
        ctx.spmm(out.shape[0], H.shape[0], row_ptr, col_idx, None, H, out, stream=st)

    def segsum_fn(seg_ptr, partial, out):
        st = torch.cuda.current_stream().cuda_stream
        assert st != 0
        ctx.segment_sum(seg_ptr, partial, out, stream=st)

    return spmm_fn, segsum_fn


def make_gpu_level_fn(ctx):
    """level_fn running the library's fused level kernel on torch's current stream (which must
    not be the legacy default stream: handle 0 selects the library's own stream)."""

    def level_fn(row_ptr, col_idx, H_full, W, X, out_rows):
        st = torch.cuda.current_stream().cuda_stream
        assert st != 0, "make a torch.cuda.Stream current before running giant-graph levels"
        ctx.level(row_ptr, col_idx, None, H_full, W, X, out_rows, n_src=H_full.shape[0], stream=st)

    return level_fn
