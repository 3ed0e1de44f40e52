"""Row-partitioned giant graph: partition + per-level all-gather logic on CPU ranks (gloo,
world size 2, compute by the CPU oracle), and the same driver on one GPU."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import REPO, assert_close
from graphnn_b200 import giant, synth
from graphnn_b200.synth import LevelProblem


def oracle_levels(oracle_lib, p, levels):
    H = p.H
    for _ in range(levels):
        H, _ = oracle_lib.level(LevelProblem(p.n_rows, p.n_src, p.row_ptr, p.col_idx, H, p.W, None), "oracle")
    return H


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _cpu_rank(rank, world, port, scale, d, levels, chunks, out_dir, referenced=False):
    sys.path.insert(0, REPO)
    sys.path.insert(0, os.path.join(REPO, "tests"))
    from oracle import bindings as ob
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    p = synth.rmat_level(scale=scale, edge_factor=8, d=d, seed=3)
    shard = giant.shard_csr(p.row_ptr, p.col_idx, p.n_src, rank, world)

    def level_fn(row_ptr, col_idx, H_full, W, X, out_rows):
        blk = LevelProblem(len(row_ptr) - 1, H_full.shape[0], row_ptr.numpy(), col_idx.numpy(), H_full.numpy(), W.numpy(),
                           None if X is None else X.numpy())
        res, _ = ob.level(blk, "oracle")
        out_rows.copy_(torch.from_numpy(res))

    def spmm_fn(row_ptr, col_idx, H, out):
        import scipy.sparse as sp
        A = sp.csr_matrix((np.ones(len(col_idx), np.float32), col_idx.numpy(), row_ptr.numpy()), shape=(len(row_ptr) - 1, H.shape[0]))
        out.copy_(torch.from_numpy((A @ H.numpy()).astype(np.float32)))

    def segsum_fn(seg_ptr, partial, out):
        sp_ = seg_ptr.numpy()
        for h in range(len(sp_) - 1):
            out[h] = partial[sp_[h]:sp_[h + 1]].sum(0)

    plan = giant.plan_hubs(shard, threshold=40, piece=16)      # low threshold: several hubs at this scale
    assert plan is not None and plan.n_hub > 0
    if referenced:
        g = giant.GiantGraphReferenced(shard, d, rank, world, level_fn, chunks=chunks, hub_plan=plan, spmm_fn=spmm_fn, segsum_fn=segsum_fn)
        # the table holds my rows plus exactly the remote rows my columns name, and fewer than all of them
        cols = np.unique(np.concatenate([shard.col_idx.numpy()]))
        lo_, hi_ = giant.row_range(p.n_rows, rank, world)
        far = cols[(cols < lo_) | (cols >= hi_)]
        assert g.n_need == len(far) and np.array_equal(g.need.numpy(), far) and g.n_need < p.n_rows - shard.rows
        assert g.exchange_bytes_per_level() == len(far) * d * 4
    else:
        g = giant.GiantGraphLevels(shard, d, rank, world, level_fn, chunks=chunks, hub_plan=plan, spmm_fn=spmm_fn, segsum_fn=segsum_fn)
    lo, hi = giant.row_range(p.n_rows, rank, world)
    g.set_input(torch.from_numpy(p.H[lo:hi]))
    slab = g.run(torch.from_numpy(p.W), levels)
    assert torch.equal(slab, g.local_slab())
    np.save(os.path.join(out_dir, f"slab{rank}.npy"), slab.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_row_partition_with_allgather_two_cpu_ranks(oracle_lib, tmp_path):
    scale, d, levels = 9, 32, 2
    mp.spawn(_cpu_rank, args=(2, _free_port(), scale, d, levels, 3, str(tmp_path)), nprocs=2, join=True)
    p = synth.rmat_level(scale=scale, edge_factor=8, d=d, seed=3)
    want = oracle_levels(oracle_lib, p, levels)
    got = np.concatenate([np.load(tmp_path / "slab0.npy"), np.load(tmp_path / "slab1.npy")])
    assert_close(got, want, "two ranks, hub rows split", scale=max(1.0, float(np.abs(want).max())))


@pytest.mark.parametrize("world,chunks", [(2, 3), (4, 2)])
def test_row_partition_exchanging_only_referenced_rows_cpu_ranks(oracle_lib, tmp_path, world, chunks):
    """Same graph, same levels, but every rank fetches only the rows its columns name (pairwise exchange with
    per-peer counts): the result must equal the single-process oracle, as the all-gather form does."""
    scale, d, levels = 9, 32, 2
    mp.spawn(_cpu_rank, args=(world, _free_port(), scale, d, levels, chunks, str(tmp_path), True), nprocs=world, join=True)
    p = synth.rmat_level(scale=scale, edge_factor=8, d=d, seed=3)
    want = oracle_levels(oracle_lib, p, levels)
    got = np.concatenate([np.load(tmp_path / f"slab{r}.npy") for r in range(world)])
    assert_close(got, want, f"{world} ranks, referenced rows only", scale=max(1.0, float(np.abs(want).max())))


def test_partition_helpers():
    p = synth.rmat_level(scale=8, edge_factor=4, d=32, seed=1)
    shards = [giant.shard_csr(p.row_ptr, p.col_idx, p.n_src, r, 4) for r in range(4)]
    assert sum(s.nnz for s in shards) == p.nnz and all(int(s.row_ptr[0]) == 0 for s in shards)
    assert torch.cat([s.col_idx for s in shards]).numpy().tolist() == p.col_idx.tolist()
    with pytest.raises(ValueError):
        giant.row_range(10, 0, 4)
    g = giant.GiantGraphLevels(shards[1], 32, 1, 4, lambda *a: None, chunks=5)
    assert g.blocks[0][0] == 0 and g.blocks[-1][1] == shards[1].rows and g.all_gather_bytes_per_level() == 3 * 64 * 32 * 4


@pytest.mark.gpu
@pytest.mark.parametrize("scale,d", [(12, 128), (15, 128), (13, 64)])
def test_giant_graph_levels_one_gpu(gpu_ctx, oracle_lib, scale, d):
    p = synth.rmat_level(scale=scale, edge_factor=8, d=d, seed=scale)
    dev = torch.device("cuda", 0)
    stream = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(stream):
        shard = giant.shard_csr(p.row_ptr, p.col_idx, p.n_src, 0, 1, device=dev)
        plan = giant.plan_hubs(shard, threshold=64, piece=32)
        assert plan is not None
        deg = np.diff(p.row_ptr)
        assert plan.n_hub == int((deg > 64).sum()) and int(plan.light.row_ptr[-1]) == int(deg[deg <= 64].sum()) + plan.n_hub
        spmm_fn, segsum_fn = giant.make_gpu_hub_fns(gpu_ctx)
        g = giant.GiantGraphLevels(shard, d, 0, 1, giant.make_gpu_level_fn(gpu_ctx), chunks=2, hub_plan=plan,
                                   spmm_fn=spmm_fn, segsum_fn=segsum_fn)
        g.set_input(torch.from_numpy(p.H).to(dev))
        slab = g.run(torch.from_numpy(p.W).to(dev), 2)
        stream.synchronize()
        got = slab.cpu().numpy()
    want = oracle_levels(oracle_lib, p, 2)
    assert_close(got, want, f"rmat scale {scale} d {d}", scale=max(1.0, float(np.abs(want).max())))
    # the referenced-rows driver on one rank (no exchange; exercises the table layout and the renumbering)
    with torch.cuda.stream(stream):
        g2 = giant.GiantGraphReferenced(shard, d, 0, 1, giant.make_gpu_level_fn(gpu_ctx), pack_fn=giant.make_gpu_pack_fn(gpu_ctx), chunks=3,
                                        hub_plan=plan, spmm_fn=spmm_fn, segsum_fn=segsum_fn)
        assert g2.n_need == 0
        g2.set_input(torch.from_numpy(p.H).to(dev))
        got2 = g2.run(torch.from_numpy(p.W).to(dev), 2)
        # the pack step is the library's row lookup
        idx = torch.tensor([5, 0, 5, shard.rows - 1], dtype=torch.int32, device=dev)
        packed = torch.empty((4, d), dtype=torch.float32, device=dev)
        giant.make_gpu_pack_fn(gpu_ctx)(idx, got2, packed)
        stream.synchronize()
        assert torch.equal(packed, got2[idx.long()])
    # (not bit-equal to `got`: three blocks instead of two fall below the row count at which the library switches kernels)
    assert_close(got2.cpu().numpy(), want, f"referenced-rows driver, rmat scale {scale} d {d}", scale=max(1.0, float(np.abs(want).max())))
    # generated-on-device shard: symmetric, deduplicated, sorted rows
    sh = giant.rmat_shard_on_device(10, 8 << 10, 0, 1, dev, seed=5)
    rp, ci = sh.row_ptr.cpu().numpy().astype(np.int64), sh.col_idx.cpu().numpy()
    rows = np.repeat(np.arange(1 << 10), np.diff(rp))
    pairs = set(zip(rows.tolist(), ci.tolist()))
    assert len(pairs) == len(ci) and all((c, r) in pairs for r, c in pairs)
    assert all(np.all(np.diff(ci[rp[i]:rp[i + 1]]) > 0) for i in range(0, 1 << 10, 37))


def _shard_rank(rank, world, port, out_dir):
    sys.path.insert(0, REPO)
    from oracle import bindings as ob
    from graphnn_b200 import sharding
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    full = synth.molecule_like(37, 5, 30, 9, 32, 2, 24, 3, 0.1, "uniform", seed=11)
    mine = sharding.shard_of(full, rank, world)          # contiguous graphs, balanced by node count
    o = ob.forward(mine, "oracle", want_levels=False)
    gather = sharding.ResultGather(sharding.shard_counts(full.nodes_per_graph, world), full.num_class, torch.device("cpu"))
    logits, pred = gather(torch.from_numpy(o["logits"]), torch.from_numpy(o["argmax"]))
    if rank == 0:
        np.save(os.path.join(out_dir, "logits.npy"), logits.numpy())
        np.save(os.path.join(out_dir, "pred.npy"), pred.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_shard_by_graph_and_logits_gather_two_cpu_ranks(oracle_lib, tmp_path):
    """Batched graphs are independent: sharding by graph and gathering the logits gives exactly
    the single-process result."""
    mp.spawn(_shard_rank, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    full = synth.molecule_like(37, 5, 30, 9, 32, 2, 24, 3, 0.1, "uniform", seed=11)
    want = oracle_lib.forward(full, "oracle", want_levels=False)
    assert np.array_equal(np.load(tmp_path / "logits.npy"), want["logits"])
    assert np.array_equal(np.load(tmp_path / "pred.npy"), want["argmax"])
