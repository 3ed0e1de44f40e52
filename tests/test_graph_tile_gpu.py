"""GPU parity of the whole-classifier tile kernel (batches of graphs of at most 128 nodes, d = 128):
against the CPU oracle, against a float64 restatement for the variants the oracle does not have
(weighted edges, mean pooling), and against the per-level kernels of the same library.  All calls go
through the C ABI (s2v_forward_f32 with s2v_batch.max_graph_nodes set)."""
import numpy as np
import pytest
import scipy.sparse as sp
import torch

from conftest import assert_close
from graphnn_b200 import capi, engine, synth

pytestmark = pytest.mark.gpu


def forward(batch, tiles=True, val=None, pool_average=False, hint=None, levels=None, check_status=True, first_table=True):
    eng = engine.S2VInference(batch.weights, batch.levels if levels is None else levels, pool_average=pool_average)
    eng.ctx.set_option(eng.ctx.OPT_GRAPH_TILES, 1 if tiles else 0)
    eng.ctx.set_option(eng.ctx.OPT_FIRST_LEVEL_TABLE, 1 if first_table else 0)
    hb = engine.build_host_batch(batch)
    db = eng.to_device(hb)
    if val is not None:
        db.val = torch.from_numpy(val).cuda()
    if hint is not None:
        db.max_graph_nodes = hint
    n0 = eng.ctx.launches
    logits, probs, pred, embed = eng.forward(db, want_embed=True)
    if check_status:
        eng.ctx.synchronize()
    return {"logits": logits, "probs": probs, "pred": pred, "embed": embed, "launches": eng.ctx.launches - n0,
            "eng": eng, "hb": hb}


def f64_forward(batch, hb, val=None, pool_average=False, levels=None):
    """kernel_mean_field.cpp:28-47 in float64 (dense/scipy), with optional edge weights and mean pooling."""
    w = {k: v.astype(np.float64) for k, v in batch.weights.items()}
    N = batch.num_nodes
    rp, ci = hb.row_ptr.numpy(), hb.col_idx.numpy()
    A = sp.csr_matrix((np.ones(len(ci)) if val is None else val.astype(np.float64), ci, rp), shape=(N, N))
    msg = w["w_n2l"][batch.tags]
    H = np.maximum(msg, 0)
    for _ in range(batch.levels if levels is None else levels):
        H = np.maximum((A @ H) @ w["p_node_conv"] + msg, 0)
    off = batch.graph_offsets()
    Y = np.stack([H[off[g]:off[g + 1]].sum(0) / (max(off[g + 1] - off[g], 1) if pool_average else 1.0)
                  for g in range(batch.num_graphs)])
    logits = np.maximum(Y @ w["h1_weight"], 0) @ w["h2_weight"]
    return H, logits


def custom_batch(sizes, edge_fn, num_tags=9, levels=3, hidden=64, num_class=2, seed=0, std=0.05):
    """Graphs of the given sizes; edge_fn(rng, n) -> undirected (u, v) pairs with u < v, local ids."""
    rng = np.random.default_rng(seed)
    sizes = np.asarray(sizes, np.int64)
    us, vs, off = [], [], 0
    for n in sizes:
        u, v = edge_fn(rng, int(n))
        us.append(np.asarray(u, np.int64) + off)
        vs.append(np.asarray(v, np.int64) + off)
        off += int(n)
    tags = rng.integers(0, num_tags, int(sizes.sum()))
    return synth._finish("custom", sizes, np.concatenate(us) if us else np.zeros(0, np.int64),
                         np.concatenate(vs) if vs else np.zeros(0, np.int64), tags, num_tags, 128, levels, hidden,
                         num_class, rng, std)


def tree_edges(rng, n):
    return synth._tree_plus_extra(rng, n, 0.1)


def clique_edges(rng, n):
    u, v = np.triu_indices(n, 1)
    return u, v


def ring_chord_edges(rng, n):
    if n < 3:
        return tree_edges(rng, n)
    i = np.arange(n)
    pairs = {(min(a, b), max(a, b)) for a, b in zip(i, (i + 1) % n)} | {(min(a, b), max(a, b)) for a, b in zip(i, (i + 5) % n)} \
        | {(min(a, b), max(a, b)) for a, b in zip(i, (i + 11) % n)}
    pairs = sorted(p for p in pairs if p[0] != p[1])
    return np.array([p[0] for p in pairs]), np.array([p[1] for p in pairs])


def test_tile_kernel_matches_oracle_on_molecules(oracle_lib):
    b = synth.molecules_16k(seed=1, num_graphs=700)
    o = oracle_lib.forward(b, "oracle")
    r = forward(b)
    assert r["launches"] == 4                     # first-level product table, tile plan, tile kernel, readout
    assert_close(r["embed"].cpu().numpy(), o["levels"][-1], "embeddings")
    assert_close(r["logits"].cpu().numpy(), o["logits"], "logits", scale=max(1.0, float(np.abs(o["logits"]).max())))
    assert_close(r["probs"].cpu().numpy(), o["probs"], "probs")
    margin = np.sort(o["logits"], axis=1)
    safe = (margin[:, -1] - margin[:, -2]) > 1e-4 * np.abs(o["logits"]).max()
    assert np.array_equal(r["pred"].cpu().numpy()[safe], o["argmax"][safe]) and safe.mean() > 0.9
    # the same kernel with its first level pushed through the MMA pipeline like the others (S2V_OPT_FIRST_LEVEL_TABLE = 0)
    q = forward(b, first_table=False)
    assert q["launches"] == 3                     # tile plan, tile kernel, readout
    assert_close(q["embed"].cpu().numpy(), o["levels"][-1], "embeddings, first level through the MMAs")
    assert_close(q["logits"].cpu().numpy(), o["logits"], "logits, first level through the MMAs", scale=max(1.0, float(np.abs(o["logits"]).max())))
    # the per-level kernels of the same library agree inside the same bar
    p = forward(b, tiles=False)
    assert p["launches"] > 4
    assert_close(r["embed"].cpu().numpy(), p["embed"].cpu().numpy(), "tile kernel vs per-level kernels")


def test_tile_results_do_not_depend_on_the_packing():
    """A graph's rows never mix with another graph's in the arithmetic, so the same graphs packed into
    different tiles (a sub-batch starts its own packing) give bit-identical embeddings and logits."""
    b = synth.molecules_16k(seed=3, num_graphs=1800)      # (both runs are below the batch size from which the readout
    full = forward(b)                                      # takes its tcgen05 form: the same kernels in both)
    lo, hi = synth.shard_bounds(b.nodes_per_graph, 3)[1]
    part = forward(b.shard(1, 3))
    off = b.graph_offsets()
    assert np.array_equal(part["logits"].cpu().numpy(), full["logits"].cpu().numpy()[lo:hi])
    assert np.array_equal(part["embed"].cpu().numpy(), full["embed"].cpu().numpy()[off[lo]:off[hi]])


@pytest.mark.parametrize("name,sizes,edge_fn", [
    ("one_full_tile", [128], ring_chord_edges),
    ("empty_and_single", [0, 1, 0, 5, 1, 1, 0, 40, 128, 0, 3, 127, 1, 2], tree_edges),
    ("many_single_nodes", [1] * 300 + [2] * 10, tree_edges),
    ("clique_beyond_the_index_cache", [100, 7, 64, 30], clique_edges),
    ("two_planning_passes", None, tree_edges),
])
def test_tile_kernel_edge_cases(name, sizes, edge_fn):
    if sizes is None:
        sizes = np.random.default_rng(5).integers(1, 7, 20000)
    std = 0.004 if edge_fn is clique_edges else 0.05      # keep 4 levels of 100-neighbour sums in range
    b = custom_batch(sizes, edge_fn, seed=len(sizes), std=std)
    r = forward(b)
    assert r["launches"] == 4
    want_h, want_logits = f64_forward(b, r["hb"])
    scale_h = max(1.0, float(np.abs(want_h).max()))
    assert_close(r["embed"].cpu().numpy(), want_h, f"{name}: embeddings", scale=scale_h)
    assert_close(r["logits"].cpu().numpy(), want_logits, f"{name}: logits", scale=max(1.0, float(np.abs(want_logits).max())) * 4)
    p = forward(b, tiles=False)
    assert_close(r["embed"].cpu().numpy(), p["embed"].cpu().numpy(), f"{name}: tile vs per-level", scale=scale_h)


@pytest.mark.parametrize("levels", [1, 2, 6])
def test_tile_kernel_weighted_edges_and_mean_pooling(levels):
    b = synth.molecules_16k(seed=4, num_graphs=300)
    rng = np.random.default_rng(9)
    val = (rng.random(b.num_edges, dtype=np.float32) * 0.6 + 0.2).astype(np.float32)
    r = forward(b, val=val, pool_average=True, levels=levels)
    assert r["launches"] == 4
    want_h, want_logits = f64_forward(b, r["hb"], val=val, pool_average=True, levels=levels)
    assert_close(r["embed"].cpu().numpy(), want_h, "weighted embeddings", scale=max(1.0, float(np.abs(want_h).max())))
    assert_close(r["logits"].cpu().numpy(), want_logits, "mean-pooled logits", scale=max(1.0, float(np.abs(want_logits).max())))
    # averaged messages (Node2NodeMsgPass with average = true): val = 1 / in-degree from the host builder
    rp, ci, avg = capi.build_n2n_csr_host(b.num_nodes, b.edge_src, b.edge_dst, average=True)
    r2 = forward(b, val=avg, levels=levels)
    want2, _ = f64_forward(b, r2["hb"], val=avg, levels=levels)
    assert_close(r2["embed"].cpu().numpy(), want2, "averaged messages")


def test_mean_pooling_per_level_path(gpu_ctx):
    rng = np.random.default_rng(3)
    for d in (32, 64, 128, 48):
        sizes = rng.integers(0, 50, 40)
        seg = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int32)
        H = rng.standard_normal((int(seg[-1]), d), dtype=np.float32)
        Y = torch.full((40, d), float("nan"), device="cuda")
        gpu_ctx.segment_sum(torch.from_numpy(seg).cuda(), torch.from_numpy(H).cuda(), Y, average=True)
        gpu_ctx.synchronize()
        want = np.stack([H[seg[g]:seg[g + 1]].astype(np.float64).sum(0) / max(sizes[g], 1) for g in range(40)])
        assert_close(Y.cpu().numpy(), want, f"segment mean d={d}")


def test_understated_hint_and_bad_tag_are_reported_not_faulted(oracle_lib):
    """A graph larger than the caller promised, and a tag outside the table: the kernels record a status,
    substitute harmless values, return normally, and the context computes correctly afterwards."""
    b = custom_batch([30, 200, 25], tree_edges, seed=2)
    r = forward(b, hint=100, check_status=False)
    with pytest.raises(capi.S2VError) as e:
        r["eng"].ctx.synchronize()
    assert e.value.status in (-2, -4)                  # S2V_ERR_UNSUPPORTED (planner) or S2V_ERR_BAD_CSR (edge leaves its tile)
    r["eng"].ctx.synchronize()                          # cleared
    good = synth.molecules_16k(seed=7, num_graphs=64)
    bad = synth.molecules_16k(seed=7, num_graphs=64)
    bad.tags = bad.tags.copy()
    bad.tags[17] = 999
    for tiles in (True, False):
        rb = forward(bad, tiles=tiles, check_status=False)
        with pytest.raises(capi.S2VError) as e:
            rb["eng"].ctx.synchronize()
        assert e.value.status == -1                     # S2V_ERR_INVALID_ARG
        rg = forward(good, tiles=tiles)
        o = oracle_lib.forward(good, "oracle", want_levels=False)
        assert_close(rg["logits"].cpu().numpy(), o["logits"], "logits after a reported bad tag",
                     scale=max(1.0, float(np.abs(o["logits"]).max())))


def test_host_entry_validates_before_launching():
    b = synth.molecules_16k(seed=8, num_graphs=100)
    eng = engine.S2VInference(b.weights, b.levels)
    hb = engine.build_host_batch(b)
    logits, pred = eng.infer_host(hb)                   # a good batch first (staging allocated)
    n0 = eng.ctx.launches

    def expect(status, mutate, before_launch=True):
        nonlocal n0
        rp, ci, gp, tg = (t.clone() for t in (hb.row_ptr, hb.col_idx, hb.graph_ptr, hb.tags))
        mutate(rp, ci, gp, tg)
        bad = engine.HostBatch(hb.num_graphs, hb.num_nodes, rp, ci, gp, tg, hb.max_graph_nodes)
        with pytest.raises(capi.S2VError) as e:
            eng.infer_host(bad)
        assert e.value.status == status
        if before_launch:
            assert eng.ctx.launches == n0               # nothing was launched
        n0 = eng.ctx.launches

    def set_(t, i, v):
        t[i] = v
    expect(-4, lambda rp, ci, gp, tg: set_(ci, 5, hb.num_nodes))          # column index == N
    expect(-4, lambda rp, ci, gp, tg: set_(ci, 0, -1))
    expect(-4, lambda rp, ci, gp, tg: set_(rp, 10, int(rp[11]) + 1))      # row offsets not monotone
    expect(-4, lambda rp, ci, gp, tg: set_(gp, 3, int(gp[4]) + 1))        # graph offsets not monotone
    # a tag outside the table is clamped by the kernels, so its scan runs beside the device work: still an error, from the host scan
    expect(-1, lambda rp, ci, gp, tg: set_(tg, 7, b.num_tags), before_launch=False)
    assert "tag outside" in eng.ctx.lib.s2v_last_error(eng.ctx.h).decode()
    l1, p1 = eng.infer_host(hb)                                          # and the context carries nothing over
    assert np.array_equal(l1, logits) and np.array_equal(p1, pred)
    # with validation switched off the same good batch still runs
    eng.ctx.set_option(eng.ctx.OPT_VALIDATE_HOST_INPUT, 0)
    l2, p2 = eng.infer_host(hb)
    assert np.array_equal(l2, logits) and np.array_equal(p2, pred)


def test_status_on_a_caller_owned_stream(gpu_ctx):
    s = torch.cuda.Stream()
    gpu_ctx.selftest_wait_timeout(stream=s.cuda_stream)
    with pytest.raises(capi.S2VError) as e:
        gpu_ctx.stream_status(s.cuda_stream)
    assert e.value.status == -7 and "site 99" in str(e.value)
    gpu_ctx.stream_status(s.cuda_stream)               # cleared


@pytest.mark.parametrize("maker", [
    lambda: synth.molecules_16k(seed=11, num_graphs=3000),
    lambda: synth.proteins_4k(seed=11, num_graphs=60),
    lambda: custom_batch([3001, 5, 700], lambda rng, n: (np.zeros(n - 1, np.int64), np.arange(1, n)), seed=1),  # stars: hub rows
], ids=["molecules", "proteins", "hub_rows"])
def test_device_csr_builder_is_bit_identical_to_the_host_builder(gpu_ctx, maker):
    b = maker()
    for average in (False, True):
        rp_h, ci_h, val_h = capi.build_n2n_csr_host(b.num_nodes, b.edge_src, b.edge_dst, average=average)
        N, E = b.num_nodes, b.num_edges
        es = torch.from_numpy(np.ascontiguousarray(b.edge_src, np.int32)).cuda()
        ed = torch.from_numpy(np.ascontiguousarray(b.edge_dst, np.int32)).cuda()
        scratch = torch.empty(gpu_ctx.csr_scratch_bytes(N, E), dtype=torch.uint8, device="cuda")
        rp = torch.full((N + 1,), -1, dtype=torch.int32, device="cuda")
        ci = torch.full((E,), -1, dtype=torch.int32, device="cuda")
        val = torch.full((E,), float("nan"), device="cuda")
        for _ in range(2):                              # twice: the scratch of the first call is stale, not zero
            gpu_ctx.build_n2n_csr(N, es, ed, scratch, rp, ci, val, average=average)
            gpu_ctx.synchronize()
            assert np.array_equal(rp.cpu().numpy(), rp_h)
            assert np.array_equal(ci.cpu().numpy(), ci_h)
            assert np.array_equal(val.cpu().numpy(), val_h)


def test_device_csr_builder_reports_bad_edges(gpu_ctx):
    es = torch.tensor([0, 1, 2, 7], dtype=torch.int32, device="cuda")
    ed = torch.tensor([1, 2, 0, 1], dtype=torch.int32, device="cuda")
    scratch = torch.empty(gpu_ctx.csr_scratch_bytes(3, 4), dtype=torch.uint8, device="cuda")
    rp = torch.zeros(4, dtype=torch.int32, device="cuda")
    ci = torch.zeros(4, dtype=torch.int32, device="cuda")
    gpu_ctx.build_n2n_csr(3, es, ed, scratch, rp, ci)
    with pytest.raises(capi.S2VError) as e:
        gpu_ctx.synchronize()
    assert e.value.status == -4
    assert rp.cpu().tolist() == [0, 1, 2, 3]            # the bad edge was dropped


def test_edge_list_host_entry_matches_csr_host_entry(oracle_lib):
    for b in (synth.molecules_16k(seed=12, num_graphs=900), synth.proteins_4k(seed=12, num_graphs=20), synth.mutag_like(seed=0)):
        eng = engine.S2VInference(b.weights, b.levels)
        hb = engine.build_host_batch(b)
        logits, pred = eng.infer_host(hb)
        es = np.ascontiguousarray(b.edge_src, np.int32)
        ed = np.ascontiguousarray(b.edge_dst, np.int32)
        l2 = np.empty_like(logits)
        p2 = np.empty_like(pred)
        for _ in range(2):
            eng.ctx.infer_edges_host(eng.model, b.num_graphs, b.num_nodes, es, ed, hb.graph_ptr.numpy(), hb.tags.numpy(), l2, p2)
            assert np.array_equal(l2, logits) and np.array_equal(p2, pred)
        o = oracle_lib.forward(b, "oracle", want_levels=False)
        assert_close(l2, o["logits"], "edge-list entry vs oracle", scale=max(1.0, float(np.abs(o["logits"]).max())))


def test_two_batches_in_flight_give_the_synchronous_results():
    """s2v_infer_edges_host_submit / s2v_infer_host_wait: six different batches through the two lanes, the next one
    submitted before the previous one is waited for; every result equals the synchronous entry point's, results
    appear only at the wait, and misuse of a lane is an argument error, not a fault."""
    batches = [synth.molecules_16k(seed=40 + i, num_graphs=300 + 150 * i) for i in range(6)]
    eng = engine.S2VInference(batches[0].weights, batches[0].levels)
    ctx = eng.ctx
    jobs = []
    for b in batches:
        hb = engine.build_host_batch(b)
        es = torch.from_numpy(np.ascontiguousarray(b.edge_src, np.int32)).pin_memory()
        ed = torch.from_numpy(np.ascontiguousarray(b.edge_dst, np.int32)).pin_memory()
        gp, tg = hb.graph_ptr.pin_memory(), hb.tags.pin_memory()
        want_l, want_p = np.empty((b.num_graphs, b.num_class), np.float32), np.empty(b.num_graphs, np.int32)
        ctx.infer_edges_host(eng.model, b.num_graphs, b.num_nodes, es.numpy(), ed.numpy(), gp.numpy(), tg.numpy(), want_l, want_p)
        jobs.append((b, es, ed, gp, tg, want_l, want_p, np.full_like(want_l, np.nan), np.full_like(want_p, -7)))

    def submit(i):
        b, es, ed, gp, tg, _, _, got_l, got_p = jobs[i]
        ctx.infer_edges_host_submit(i % 2, eng.model, b.num_graphs, b.num_nodes, es.numpy(), ed.numpy(), gp.numpy(), tg.numpy(), got_l, got_p)

    submit(0)
    for i in range(len(jobs)):
        if i + 1 < len(jobs):
            submit(i + 1)                              # the other lane, before waiting for this one
        assert np.isnan(jobs[i][7]).all()              # nothing is delivered before the wait
        ctx.infer_host_wait(i % 2)
        assert np.array_equal(jobs[i][7], jobs[i][5]) and np.array_equal(jobs[i][8], jobs[i][6])
    ctx.infer_host_wait(0)                             # idle lane: nothing to do
    # misuse
    submit(0)
    with pytest.raises(capi.S2VError) as e:
        submit(0)                                      # lane 0 still holds a batch
    assert e.value.status == -1
    with pytest.raises(capi.S2VError):
        eng.infer_host(engine.build_host_batch(batches[0]))   # the synchronous entries use lane 0
    ctx.infer_host_wait(0)
    with pytest.raises(capi.S2VError):
        ctx.infer_host_wait(2)
    # a bad tag in a submitted batch is reported at the wait, and the lane is free again afterwards
    b, es, ed, gp, tg, want_l, want_p, got_l, got_p = jobs[1]
    bad = tg.clone()
    bad[3] = b.num_tags
    ctx.infer_edges_host_submit(1, eng.model, b.num_graphs, b.num_nodes, es.numpy(), ed.numpy(), gp.numpy(), bad.numpy(), got_l, got_p)
    with pytest.raises(capi.S2VError) as e:
        ctx.infer_host_wait(1)
    assert e.value.status == -1 and "tag outside" in str(e.value)
    ctx.infer_edges_host_submit(1, eng.model, b.num_graphs, b.num_nodes, es.numpy(), ed.numpy(), gp.numpy(), tg.numpy(), got_l, got_p)
    ctx.infer_host_wait(1)
    assert np.array_equal(got_l, want_l) and np.array_equal(got_p, want_p)
