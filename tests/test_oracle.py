"""CPU tests of the parity checkers themselves: the C restatement against the golden
vectors produced by the reference's own code, against that code when it is built
here, and against the float64 numpy restatement."""
import numpy as np
import pytest

from conftest import assert_close
from graphnn_b200 import synth
from oracle import s2v_numpy


def test_oracle_matches_golden_classifier(oracle_lib, golden):
    g = golden("mutag_like_seed0.npz")
    b = synth.mutag_like(seed=0)
    assert str(g["digest"]) == b.digest(), "generator output changed: regenerate tests/golden"
    o = oracle_lib.forward(b, "oracle")
    for k in ("n2n_row_ptr", "n2n_col_idx", "n2n_val", "sub_row_ptr", "sub_col_idx", "sub_val", "argmax"):
        assert np.array_equal(o[k], g[k]), k
    assert_close(o["levels"][-1], g["last_level"], "last level")
    assert_close(o["pooled"], g["pooled"], "pooled")
    assert_close(o["logits"], g["logits"], "logits")
    assert_close(o["probs"], g["probs"], "probs")


def test_oracle_matches_golden_mixed_classes(oracle_lib, golden):
    g = golden("mutag_like_seed3.npz")
    b = synth.mutag_like(seed=3)
    assert str(g["digest"]) == b.digest()
    o = oracle_lib.forward(b, "oracle", want_levels=False)
    assert np.array_equal(o["n2n_row_ptr"], g["n2n_row_ptr"])
    assert np.array_equal(o["n2n_col_idx"], g["n2n_col_idx"])
    assert np.array_equal(o["argmax"], g["argmax"])
    assert len(np.unique(g["argmax"])) == 2
    assert_close(o["logits"], g["logits"], "logits")


def test_oracle_level_matches_golden(oracle_lib, golden):
    g = golden("er_level_n1000_d64_seed1.npz")
    p = synth.erdos_renyi_level(n=1000, nnz=6000, d=64, seed=1)
    assert np.array_equal(p.row_ptr, g["row_ptr"]) and np.array_equal(p.col_idx, g["col_idx"])
    out, _ = oracle_lib.level(p, "oracle")
    assert_close(out, g["out"], "level output")
    assert (np.diff(p.row_ptr) == 0).any(), "fixture should contain empty rows"


def test_oracle_matches_reference_build(oracle_lib):
    if not oracle_lib.have_reference():
        pytest.skip("reference build not present on this machine")
    for seed in (0, 5):
        b = synth.molecule_like(24, 3, 40, 11, 32, 2, 48, 3, 0.1, "uniform", seed)
        o = oracle_lib.forward(b, "oracle")
        r = oracle_lib.forward(b, "reference")
        for k in ("n2n_row_ptr", "n2n_col_idx", "n2n_val", "sub_row_ptr", "sub_col_idx", "sub_val", "argmax"):
            assert np.array_equal(o[k], r[k]), k
        for k in ("msg", "levels", "pooled", "logits", "probs"):
            assert_close(o[k], r[k], k)
    p = synth.erdos_renyi_level(n=777, nnz=5000, d=128, seed=2, with_x=False)
    a, _ = oracle_lib.level(p, "oracle")
    b_, _ = oracle_lib.level(p, "reference")
    assert_close(a, b_, "level without X")


def test_oracle_threads_do_not_change_results(oracle_lib):
    b = synth.mutag_like(seed=1)
    oracle_lib.set_threads(1, "oracle")
    a = oracle_lib.forward(b, "oracle")
    oracle_lib.set_threads(4, "oracle")
    c = oracle_lib.forward(b, "oracle")
    oracle_lib.set_threads(1, "oracle")
    for k in ("levels", "logits", "probs"):
        assert np.array_equal(a[k], c[k]), k


def test_float64_restatement_agrees(oracle_lib):
    b = synth.mutag_like(seed=0)
    o = oracle_lib.forward(b, "oracle")
    n = s2v_numpy.forward(b)
    assert np.array_equal(o["n2n_row_ptr"], n["n2n_row_ptr"])
    assert np.array_equal(o["n2n_col_idx"], n["n2n_col_idx"])
    assert np.array_equal(o["sub_row_ptr"], n["sub_row_ptr"])
    assert np.array_equal(o["argmax"], n["argmax"])
    assert_close(o["levels"], n["levels"], "levels")
    assert_close(o["logits"], n["logits"], "logits")


def test_level_in_double_agrees_on_short_rows_and_wins_on_long_ones(oracle_lib):
    """oracle_level_f64 (every sum in double) is the yardstick for very long rows: on ordinary rows it agrees with
    the float oracle to the parity bar; on one 300,000-entry row of equal positive values the float sequential sum
    is visibly off while the double one is exact."""
    prob = synth.erdos_renyi_level(n=600, nnz=4800, d=64, seed=3)
    a, _ = oracle_lib.level(prob, "oracle")
    b, _ = oracle_lib.level(prob, "oracle_f64")
    assert_close(a, b, "level f32 vs f64")
    d, n = 8, 300_000
    H = np.full((1, d), 0.1, np.float32)
    W = np.eye(d, dtype=np.float32)
    long_row = synth.LevelProblem(1, 1, np.array([0, n], np.int32), np.zeros(n, np.int32), H, W, None)
    f32, _ = oracle_lib.level(long_row, "oracle")
    f64, _ = oracle_lib.level(long_row, "oracle_f64")
    exact = n * float(np.float32(0.1))
    assert abs(float(f64[0, 0]) - exact) <= 1e-6 * exact
    assert abs(float(f32[0, 0]) - exact) > 1e-5 * exact


def test_generators_shapes():
    b = synth.mutag_like(seed=0)
    assert b.num_graphs == 64 and b.nodes_per_graph.min() >= 10 and b.nodes_per_graph.max() <= 28
    assert b.num_tags == 7 and b.d == 64 and b.levels == 3 and b.hidden == 128 and b.num_class == 2
    # symmetric, ordered as GetBatch adds edges: source ascending, then neighbour ascending
    key = b.edge_src.astype(np.int64) * b.num_nodes + b.edge_dst
    assert (np.diff(key) > 0).all()
    rev = np.sort(b.edge_dst.astype(np.int64) * b.num_nodes + b.edge_src)
    assert np.array_equal(rev, key)
    # tree + ceil(10 %) extra edges per graph, no edge crosses graphs
    off = b.graph_offsets()
    gid = np.searchsorted(off, b.edge_src, side="right") - 1
    assert np.array_equal(gid, np.searchsorted(off, b.edge_dst, side="right") - 1)
    per_graph = np.bincount(gid, minlength=64) // 2
    n = b.nodes_per_graph
    assert np.array_equal(per_graph, (n - 1) + np.ceil(0.1 * (n - 1)).astype(int))
    p = synth.erdos_renyi_level(n=4096, nnz=32768, d=64, seed=0)
    assert p.row_ptr[-1] == 32768 and p.col_idx.max() < 4096 and p.H.dtype == np.float32
    r = synth.rmat_level(scale=10, edge_factor=8, d=32)
    assert r.row_ptr[-1] == r.nnz and r.X is None
    # symmetric after symmetrisation
    rows = np.repeat(np.arange(r.n_rows), np.diff(r.row_ptr))
    a = set(zip(rows.tolist(), r.col_idx.tolist()))
    assert all((c, rr) in a for rr, c in list(a)[:2000])


def test_shard_bounds_cover_and_balance():
    b = synth.molecules_16k(seed=0, num_graphs=512)
    for world in (1, 2, 4, 8):
        bounds = synth.shard_bounds(b.nodes_per_graph, world)
        assert bounds[0][0] == 0 and bounds[-1][1] == b.num_graphs
        assert all(bounds[i][1] == bounds[i + 1][0] for i in range(world - 1))
        nodes = [int(b.nodes_per_graph[lo:hi].sum()) for lo, hi in bounds]
        assert max(nodes) - min(nodes) <= 2 * 40
        shards = [b.shard(r, world) for r in range(world)]
        assert sum(s.num_edges for s in shards) == b.num_edges
        assert sum(s.num_nodes for s in shards) == b.num_nodes


def test_loss_accuracy_tail(oracle_lib, golden):
    g = golden("mutag_like_seed3.npz")
    t = golden("loss_acc_seed3.npz")
    loss, acc, per = oracle_lib.loss_acc(g["logits"], t["labels"], "oracle")
    assert abs(loss - float(t["loss"])) <= 1e-5 * max(1.0, abs(float(t["loss"]))) and acc == float(t["acc"])
    assert_close(per, t["per_graph"], "per-graph cross entropy")
    # clamp: a probability that underflows to 0 is treated as 1e-8
    lg = np.array([[100.0, -100.0], [0.0, 0.0]], np.float32)
    loss2, acc2, per2 = oracle_lib.loss_acc(lg, np.array([1, 0], np.int32), "oracle")
    assert abs(per2[0] - (-np.log(np.float32(1e-8)))) < 1e-4 and abs(per2[1] - np.log(2.0)) < 1e-6 and acc2 == 0.5
    if oracle_lib.have_reference():
        rng = np.random.default_rng(5)
        lgs = (rng.standard_normal((300, 5)) * 10).astype(np.float32)
        lab = rng.integers(0, 5, 300).astype(np.int32)
        a = oracle_lib.loss_acc(lgs, lab, "oracle")
        b = oracle_lib.loss_acc(lgs, lab, "reference")
        assert abs(a[0] - b[0]) <= 1e-5 * abs(b[0]) and a[1] == b[1]
        assert_close(a[2], b[2], "per-graph loss vs reference")


@pytest.mark.parametrize("average", [False, True])
def test_oracle_edge_matrices_match_golden_and_reference(oracle_lib, golden, average):
    """The C restatement of Edge2Node / Node2Edge / Edge2Edge::InitCPUWeight against the committed output of the
    reference's factors, and against the reference build itself when it is present."""
    g = golden("msgpass_matrices_mutag_seed0.npz")
    b = synth.mutag_like(seed=0)
    tag = "avg" if average else "sum"
    for which in ("e2n", "n2e", "e2e"):
        rp, ci, val = oracle_lib.msgpass_matrix(b, which, "oracle", average)
        assert np.array_equal(rp, g[f"{which}_{tag}_row_ptr"]) and np.array_equal(ci, g[f"{which}_{tag}_col_idx"])
        assert np.array_equal(val, g[f"{which}_{tag}_val"])
    if oracle_lib.have_reference():
        b2 = synth.molecule_like(50, 1, 30, 5, 32, 2, 16, 2, 0.1, "uniform", seed=21)
        for which in ("e2n", "n2e", "e2e"):
            want = oracle_lib.msgpass_matrix(b2, which, "reference", average)
            got = oracle_lib.msgpass_matrix(b2, which, "oracle", average)
            assert all(np.array_equal(x, y) for x, y in zip(got, want)), which
