"""GPU parity of the tcgen05 form of the fused level (d = 64 and d = 128) against the CPU
oracle.  The library picks that kernel by batch size; here a context created with
S2V_LEVEL_TC=2 forces it on every shape, so ragged tiles, empty rows, rows longer than the
index window, weighted edges and the table-lookup forms are all covered."""
import os

import numpy as np
import pytest
import torch

from conftest import assert_close
from graphnn_b200 import synth
from graphnn_b200.synth import LevelProblem
from test_level_gpu import dev, oracle_level, run_level

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tc_ctx():
    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    from graphnn_b200 import capi
    old = os.environ.get("S2V_LEVEL_TC")
    os.environ["S2V_LEVEL_TC"] = "2"
    try:
        ctx = capi.Context(0)
    finally:
        if old is None:
            del os.environ["S2V_LEVEL_TC"]
        else:
            os.environ["S2V_LEVEL_TC"] = old
    yield ctx
    ctx.close()


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("n,nnz", [(1, 0), (1, 3), (127, 300), (128, 1000), (129, 5), (1000, 8000), (4099, 60000),
                                   (148 * 128 * 2 + 77, 200000)])
def test_tc_level_shapes(tc_ctx, oracle_lib, d, n, nnz):
    p = synth.erdos_renyi_level(n=n, nnz=nnz, d=d, seed=n + d)
    assert_close(run_level(tc_ctx, p), oracle_level(oracle_lib, p), f"tcgen05 d={d} n={n}")


@pytest.mark.parametrize("d", [64, 128])
def test_tc_level_agrees_with_warp_kernel(tc_ctx, d):
    """Both kernels sum neighbours in CSR order in fp32; the products differ only in how the
    3xTF32 terms are grouped, so the results agree inside the parity bar."""
    p = synth.erdos_renyi_level(n=20000, nnz=150000, d=d, seed=11)
    a = run_level(tc_ctx, p)
    from graphnn_b200 import capi
    os.environ["S2V_LEVEL_TC"] = "0"
    try:
        plain = capi.Context(0)
    finally:
        del os.environ["S2V_LEVEL_TC"]
    b = run_level(plain, p)
    plain.close()
    assert_close(a, b, "tcgen05 vs mma.sync kernel")


@pytest.mark.parametrize("d", [64, 128])
def test_tc_level_without_x_and_with_weights(tc_ctx, oracle_lib, d):
    p = synth.erdos_renyi_level(n=900, nnz=7000, d=d, seed=4, with_x=False)
    assert_close(run_level(tc_ctx, p), oracle_level(oracle_lib, p), "no X")
    rng = np.random.default_rng(0)
    val = rng.random(p.nnz, dtype=np.float32) + 0.5
    p2 = synth.erdos_renyi_level(n=900, nnz=7000, d=d, seed=5)
    assert_close(run_level(tc_ctx, p2, val=val), oracle_level(oracle_lib, p2, val), "weighted edges")
    deg = np.diff(p2.row_ptr)
    avg = np.repeat(1.0 / np.maximum(deg, 1), deg).astype(np.float32)
    assert_close(run_level(tc_ctx, p2, val=avg), oracle_level(oracle_lib, p2, avg), "averaged edges")


@pytest.mark.parametrize("d", [64, 128])
def test_tc_level_heavy_rows_and_rectangular(tc_ctx, oracle_lib, d):
    """Rows longer than one 64-entry index window (and exactly at its edge), empty rows between
    them, and n_src != n_rows."""
    rng = np.random.default_rng(7)
    n_rows, n_src = 300, 5000
    deg = np.zeros(n_rows, np.int64)
    deg[3] = 1500
    deg[4] = 129
    deg[5] = 64
    deg[6] = 65
    deg[7] = 63
    deg[16] = 300
    deg[17] = 257
    deg[40:60] = rng.integers(0, 30, 20)
    deg[130:290] = rng.integers(0, 20, 160)
    row_ptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int32)
    col = rng.integers(0, n_src, int(deg.sum())).astype(np.int32)
    p = LevelProblem(n_rows, n_src, row_ptr, col, rng.standard_normal((n_src, d), dtype=np.float32) * 0.1,
                     (rng.standard_normal((d, d), dtype=np.float32) * 0.1), rng.standard_normal((n_rows, d), dtype=np.float32))
    assert_close(run_level(tc_ctx, p), oracle_level(oracle_lib, p), "heavy rows")
    val = rng.random(p.nnz, dtype=np.float32) + 0.5
    assert_close(run_level(tc_ctx, p, val=val), oracle_level(oracle_lib, p, val), "heavy rows, weighted")


@pytest.mark.parametrize("maker", [
    lambda: synth.molecules_16k(seed=6, num_graphs=200),     # d = 128
    lambda: synth.proteins_4k(seed=6, num_graphs=12),        # d = 64
], ids=["molecules_d128", "proteins_d64"])
def test_tc_lookup_and_first_level_forms(tc_ctx, oracle_lib, maker):
    """X looked up from W_in by tag, and the first level straight from the tags (H0 never in memory)."""
    b = maker()
    o = oracle_lib.forward(b, "oracle")
    rp, ci, tags = dev(o["n2n_row_ptr"]), dev(o["n2n_col_idx"]), dev(b.tags.astype(np.int32))
    W, table = dev(b.weights["p_node_conv"]), dev(b.weights["w_n2l"])
    out = torch.full((b.num_nodes, b.d), float("nan"), device="cuda")
    tc_ctx.level_lookup(rp, ci, None, dev(o["levels"][1]), W, table, tags, out)
    tc_ctx.synchronize()
    assert_close(out.cpu().numpy(), o["levels"][2], "lookup form, level 2")
    fused = torch.full((b.num_nodes, b.d), float("nan"), device="cuda")
    tc_ctx.set_option(tc_ctx.OPT_FIRST_LEVEL_TABLE, 0)      # the tcgen05 kernel's own table-lookup form, not the product table
    try:
        tc_ctx.level_first(rp, ci, None, W, table, tags, fused)
        tc_ctx.synchronize()
    finally:
        tc_ctx.set_option(tc_ctx.OPT_FIRST_LEVEL_TABLE, 1)
    assert_close(fused.cpu().numpy(), o["levels"][1], "first level from tags")


def test_tc_whole_classifier_d64(oracle_lib, monkeypatch):
    """The protein-like configuration end to end with every level on the tcgen05 kernel."""
    from graphnn_b200 import engine
    monkeypatch.setenv("S2V_LEVEL_TC", "2")
    b = synth.proteins_4k(seed=9, num_graphs=24)
    o = oracle_lib.forward(b, "oracle")
    eng = engine.S2VInference(b.weights, b.levels)
    db = eng.to_device(engine.build_host_batch(b))
    logits, probs, pred, embed = eng.forward(db, want_embed=True)
    eng.ctx.synchronize()
    assert_close(embed.cpu().numpy(), o["levels"][-1], "embeddings")
    assert_close(logits.cpu().numpy(), o["logits"], "logits", scale=max(1.0, float(np.abs(o["logits"]).max())))
    assert_close(probs.cpu().numpy(), o["probs"], "probs")


@pytest.mark.parametrize("d", [64, 128])
def test_tc_first_level_with_long_rows(tc_ctx, d):
    """The table form (gather source = ReLU(W_in[tag[col]])) on rows that span several index windows:
    the windows then hold table rows looked up on demand."""
    rng = np.random.default_rng(11)
    n, n_tags = 400, 9
    deg = rng.integers(0, 12, n)
    deg[7], deg[8], deg[200], deg[399] = 700, 64, 129, 65
    row_ptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int32)
    col = rng.integers(0, n, int(deg.sum())).astype(np.int32)
    tags = rng.integers(0, n_tags, n).astype(np.int32)
    table = (rng.standard_normal((n_tags, d)) * 0.3).astype(np.float32)
    W = (rng.standard_normal((d, d)) * 0.1).astype(np.float32)
    fused = torch.full((n, d), float("nan"), device="cuda")
    by_table = torch.full((n, d), float("nan"), device="cuda")
    tc_ctx.level_first(dev(row_ptr), dev(col), None, dev(W), dev(table), dev(tags), by_table)   # product-table form (the default)
    tc_ctx.set_option(tc_ctx.OPT_FIRST_LEVEL_TABLE, 0)
    try:
        tc_ctx.level_first(dev(row_ptr), dev(col), None, dev(W), dev(table), dev(tags), fused)  # the tcgen05 kernel's own form
        tc_ctx.synchronize()
    finally:
        tc_ctx.set_option(tc_ctx.OPT_FIRST_LEVEL_TABLE, 1)
    import scipy.sparse as sp
    h0 = np.maximum(table[tags].astype(np.float64), 0.0)
    A = sp.csr_matrix((np.ones(len(col)), col, row_ptr), shape=(n, n))
    z = (A @ h0) @ W.astype(np.float64) + table[tags]
    got, want = fused.cpu().numpy(), np.where(z < 0, 0.0, z).astype(np.float32)
    long_rows = deg > 100
    assert_close(got[~long_rows], want[~long_rows], f"first level, rows up to 65 non-zeros, d={d}")
    # the 700- and 129-term rows cancel heavily in the product with W: there the absolute bar scales with
    # the size of the terms that cancel (the fp32 reference itself is no closer to this float64 result)
    scale = float(((A @ h0) @ np.abs(W).astype(np.float64))[long_rows].max())
    assert_close(got[long_rows], want[long_rows], f"first level, long rows, d={d}", scale=scale)
    got_t = by_table.cpu().numpy()
    assert_close(got_t[~long_rows], want[~long_rows], f"first level by product table, rows up to 65 non-zeros, d={d}")
    assert_close(got_t[long_rows], want[long_rows], f"first level by product table, long rows, d={d}", scale=scale)


def test_bounded_wait_reports_and_context_survives(gpu_ctx, oracle_lib):
    """The time-out path of the kernels' barrier waits, exercised without any fault: a wait that nothing
    will ever satisfy gives up, the kernel returns, the host reads the status, and the same context then
    runs a level correctly."""
    from graphnn_b200.capi import S2VError
    gpu_ctx.selftest_wait_timeout()
    with pytest.raises(S2VError) as e:
        gpu_ctx.synchronize()
    assert e.value.status == -7 and "site 99" in str(e.value)      # S2V_ERR_DEVICE_TIMEOUT
    gpu_ctx.synchronize()                                           # the status was cleared
    p = synth.erdos_renyi_level(n=20000, nnz=90000, d=128, seed=3)  # large enough for the tcgen05 kernel
    assert_close(run_level(gpu_ctx, p), oracle_level(oracle_lib, p), "level after a reported time-out")


def test_reserved_sms_change_the_grid_not_the_result(tc_ctx):
    """S2V_OPT_RESERVED_SMS shrinks the persistent grid (SMs left to a communication library's kernels); the tiles
    are only dealt differently over the CTAs, so the output is bit-identical."""
    from graphnn_b200 import capi
    p = synth.erdos_renyi_level(n=148 * 128 * 3 + 5, nnz=400000, d=128, seed=5)
    a = run_level(tc_ctx, p)
    tc_ctx.set_option(tc_ctx.OPT_RESERVED_SMS, 20)
    try:
        b = run_level(tc_ctx, p)
        with pytest.raises(capi.S2VError):
            tc_ctx.set_option(tc_ctx.OPT_RESERVED_SMS, 100000)
        with pytest.raises(capi.S2VError):
            tc_ctx.set_option(tc_ctx.OPT_RESERVED_SMS, -1)
    finally:
        tc_ctx.set_option(tc_ctx.OPT_RESERVED_SMS, 0)
    assert np.array_equal(a, b)


@pytest.mark.parametrize("G,d,hidden,C", [(513, 128, 256, 2), (2049, 64, 128, 3), (700, 64, 256, 8)])
def test_tc_readout_small_batches(tc_ctx, G, d, hidden, C):
    """The tcgen05 readout on batches below the size from which the library picks it by itself (the context forces
    the tensor-core kernels): ragged last tile, both hidden widths, both input widths, up to 8 classes."""
    rng = np.random.default_rng(G)
    Y = rng.standard_normal((G, d), dtype=np.float32) * 3.0
    W1 = rng.standard_normal((d, hidden), dtype=np.float32) * 0.1
    W2 = rng.standard_normal((hidden, C), dtype=np.float32) * 0.1
    logits = torch.full((G, C), float("nan"), device="cuda")
    probs = torch.empty((G, C), device="cuda")
    pred = torch.empty(G, dtype=torch.int32, device="cuda")
    tc_ctx.readout(dev(Y), dev(W1), dev(W2), logits, probs, pred)
    tc_ctx.synchronize()
    lg = np.maximum(Y.astype(np.float64) @ W1.astype(np.float64), 0) @ W2.astype(np.float64)
    assert_close(logits.cpu().numpy(), lg, "tcgen05 readout logits", scale=8)
    e = np.exp(lg - lg.max(1, keepdims=True))
    assert_close(probs.cpu().numpy(), e / e.sum(1, keepdims=True), "tcgen05 readout probs", scale=8)
    assert np.array_equal(pred.cpu().numpy(), logits.cpu().numpy().argmax(1))
