"""GPU parity of the fused level kernel and the unfused tensor operations against the
CPU oracle, all through the C ABI."""
import numpy as np
import pytest
import torch

from conftest import assert_close
from graphnn_b200 import synth
from graphnn_b200.synth import LevelProblem

pytestmark = pytest.mark.gpu


def dev(a):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()


def run_level(ctx, p: LevelProblem, val=None, rp64=False, rows=None):
    rp = p.row_ptr.astype(np.int64 if rp64 else np.int32)
    out = torch.full((p.n_rows, p.d), float("nan"), device="cuda")
    ctx.level(dev(rp), dev(p.col_idx), dev(val), dev(p.H), dev(p.W), dev(p.X), out, stream=None)
    ctx.synchronize()
    return out.cpu().numpy()


def oracle_level(oracle_lib, p, val=None):
    if val is None:
        out, _ = oracle_lib.level(p, "oracle")
        return out
    # weighted edges: float64 restatement rounded to fp32 is accurate to well under the bar
    import scipy.sparse as sp
    A = sp.csr_matrix((val.astype(np.float64), p.col_idx, p.row_ptr), shape=(p.n_rows, p.n_src))
    z = (A @ p.H.astype(np.float64)) @ p.W.astype(np.float64)
    if p.X is not None:
        z = z + p.X
    return np.where(z < 0, 0.0, z).astype(np.float32)


def test_level_matches_golden(gpu_ctx, golden):
    g = golden("er_level_n1000_d64_seed1.npz")
    p = synth.erdos_renyi_level(n=1000, nnz=6000, d=64, seed=1)
    assert_close(run_level(gpu_ctx, p), g["out"], "level vs reference golden")


@pytest.mark.parametrize("d", [32, 64, 128])
@pytest.mark.parametrize("n,nnz", [(1, 0), (1, 3), (15, 40), (16, 100), (17, 5), (1000, 8000), (4099, 60000)])
def test_level_shapes(gpu_ctx, oracle_lib, d, n, nnz):
    p = synth.erdos_renyi_level(n=n, nnz=nnz, d=d, seed=n + d)
    assert_close(run_level(gpu_ctx, p), oracle_level(oracle_lib, p), f"d={d} n={n}")


@pytest.mark.parametrize("d", [64, 128])
def test_level_without_x_and_with_weights(gpu_ctx, oracle_lib, d):
    p = synth.erdos_renyi_level(n=900, nnz=7000, d=d, seed=4, with_x=False)
    assert_close(run_level(gpu_ctx, p), oracle_level(oracle_lib, p), "no X")
    rng = np.random.default_rng(0)
    val = rng.random(p.nnz, dtype=np.float32) + 0.5
    p2 = synth.erdos_renyi_level(n=900, nnz=7000, d=d, seed=5)
    assert_close(run_level(gpu_ctx, p2, val=val), oracle_level(oracle_lib, p2, val), "weighted edges")
    # 1/deg averaging as Node2NodeMsgPass(average=true) would produce
    deg = np.diff(p2.row_ptr)
    avg = np.repeat(1.0 / np.maximum(deg, 1), deg).astype(np.float32)
    assert_close(run_level(gpu_ctx, p2, val=avg), oracle_level(oracle_lib, p2, avg), "averaged edges")


def test_level_heavy_rows_and_rectangular(gpu_ctx, oracle_lib):
    """Rows with more non-zeros than the per-warp index buffer, and n_src != n_rows."""
    rng = np.random.default_rng(7)
    n_rows, n_src, d = 70, 5000, 64
    deg = np.zeros(n_rows, np.int64)
    deg[3] = 1500
    deg[16] = 300
    deg[17] = 257
    deg[40:60] = rng.integers(0, 30, 20)
    row_ptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int32)
    col = rng.integers(0, n_src, int(deg.sum())).astype(np.int32)
    p = LevelProblem(n_rows, n_src, row_ptr, col, rng.standard_normal((n_src, d), dtype=np.float32) * 0.1,
                     (rng.standard_normal((d, d), dtype=np.float32) * 0.1), rng.standard_normal((n_rows, d), dtype=np.float32))
    assert_close(run_level(gpu_ctx, p), oracle_level(oracle_lib, p), "heavy rows")
    assert_close(run_level(gpu_ctx, p, rp64=True), oracle_level(oracle_lib, p), "64-bit row offsets")


def test_level_block_diagonal_batch(gpu_ctx, oracle_lib):
    """The layout the classifier actually uses: many small symmetric graphs."""
    b = synth.molecule_like(300, 20, 40, 82, 128, 4, 256, 2, 0.05, 1.2, seed=2)
    o = oracle_lib.forward(b, "oracle")
    p = LevelProblem(b.num_nodes, b.num_nodes, o["n2n_row_ptr"], o["n2n_col_idx"], o["levels"][1],
                     b.weights["p_node_conv"], o["msg"])
    assert_close(run_level(gpu_ctx, p), o["levels"][2], "level 2 of a molecule batch")
    # the same level with the X term looked up from W_in by node tag
    out = torch.empty((b.num_nodes, b.d), device="cuda")
    gpu_ctx.level_lookup(dev(p.row_ptr), dev(p.col_idx), None, dev(p.H), dev(p.W), dev(b.weights["w_n2l"]),
                         dev(b.tags), out)
    gpu_ctx.synchronize()
    assert_close(out.cpu().numpy(), o["levels"][2], "lookup form")


def test_first_level_straight_from_tags(gpu_ctx, oracle_lib):
    """s2v_level_first_f32 (H0 never materialised) against input projection + level, and the oracle: as a gather-sum
    over the product table ReLU(W_in) * W (the default), and in the level kernel's own table-lookup form."""
    from graphnn_b200.capi import S2VError
    b = synth.molecules_16k(seed=4, num_graphs=700)          # ~21k nodes: the tcgen05 kernel takes it too
    o = oracle_lib.forward(b, "oracle")
    rp, ci, tags = dev(o["n2n_row_ptr"]), dev(o["n2n_col_idx"]), dev(b.tags.astype(np.int32))
    W, table = dev(b.weights["p_node_conv"]), dev(b.weights["w_n2l"])
    h0 = torch.empty((b.num_nodes, b.d), device="cuda")
    two_step = torch.empty_like(h0)
    gpu_ctx.input_proj_onehot(tags, table, None, h0)
    gpu_ctx.level_lookup(rp, ci, None, h0, W, table, tags, two_step)
    by_table = torch.full((b.num_nodes, b.d), float("nan"), device="cuda")
    gpu_ctx.level_first(rp, ci, None, W, table, tags, by_table)
    gpu_ctx.set_option(gpu_ctx.OPT_FIRST_LEVEL_TABLE, 0)
    try:
        fused = torch.full((b.num_nodes, b.d), float("nan"), device="cuda")
        gpu_ctx.level_first(rp, ci, None, W, table, tags, fused)
        gpu_ctx.synchronize()
        assert torch.equal(fused, two_step)                   # the level kernel's form: same arithmetic in the same order
        small = synth.mutag_like(seed=0)                      # small batch: not taken by the tcgen05 kernel, the caller must fall back
        with pytest.raises(S2VError) as e:
            gpu_ctx.level_first(dev(np.zeros(small.num_nodes + 1, np.int32)), None, None, dev(small.weights["p_node_conv"]),
                                dev(small.weights["w_n2l"]), dev(small.tags.astype(np.int32)),
                                torch.empty((small.num_nodes, 64), device="cuda"))
        assert e.value.status == -2
    finally:
        gpu_ctx.set_option(gpu_ctx.OPT_FIRST_LEVEL_TABLE, 1)
    assert_close(fused.cpu().numpy(), o["levels"][1], "first level from tags, level-kernel form")
    assert_close(by_table.cpu().numpy(), o["levels"][1], "first level from tags, product-table form")
    # the product-table form takes any batch size and weighted edges; a width whose d/4 is not a power of two is refused
    small = synth.mutag_like(seed=0)
    os_ = oracle_lib.forward(small, "oracle")
    out = torch.full((small.num_nodes, small.d), float("nan"), device="cuda")
    gpu_ctx.level_first(dev(os_["n2n_row_ptr"]), dev(os_["n2n_col_idx"]), None, dev(small.weights["p_node_conv"]),
                        dev(small.weights["w_n2l"]), dev(small.tags.astype(np.int32)), out)
    gpu_ctx.synchronize()
    assert_close(out.cpu().numpy(), os_["levels"][1], "product-table form, 64 small graphs")
    rng = np.random.default_rng(3)
    val = rng.uniform(0.25, 2.0, small.num_edges).astype(np.float32)
    gpu_ctx.level_first(dev(os_["n2n_row_ptr"]), dev(os_["n2n_col_idx"]), dev(val), dev(small.weights["p_node_conv"]),
                        dev(small.weights["w_n2l"]), dev(small.tags.astype(np.int32)), out)
    gpu_ctx.synchronize()
    import scipy.sparse as sp
    tbl = small.weights["w_n2l"].astype(np.float64)
    tg = small.tags.astype(np.int64)
    A = sp.csr_matrix((val.astype(np.float64), os_["n2n_col_idx"], os_["n2n_row_ptr"]), shape=(small.num_nodes, small.num_nodes))
    z = (A @ np.maximum(tbl[tg], 0.0)) @ small.weights["p_node_conv"].astype(np.float64) + tbl[tg]
    assert_close(out.cpu().numpy(), np.where(z < 0, 0.0, z).astype(np.float32), "product-table form, weighted edges")
    with pytest.raises(S2VError) as e:
        gpu_ctx.level_first(dev(np.zeros(11, np.int32)), None, None, dev(np.zeros((12, 12), np.float32)), dev(np.zeros((3, 12), np.float32)),
                            dev(np.zeros(10, np.int32)), torch.empty((10, 12), device="cuda"))
    assert e.value.status == -2


def test_level_relu_keeps_negative_zero_and_nan(gpu_ctx):
    d = 64
    H = np.zeros((16, d), np.float32)
    H[0, 0] = np.nan
    W = np.eye(d, dtype=np.float32)
    X = np.full((16, d), -0.0, np.float32)
    X[2, :] = -3.0
    row_ptr = np.zeros(17, np.int32)
    row_ptr[1:] = 1          # row 0 gathers H[0]
    p = LevelProblem(16, 16, row_ptr, np.array([0], np.int32), H, W, X)
    out = run_level(gpu_ctx, p)
    assert np.isnan(out[0, 0])
    assert (out[1] == 0).all() and not np.signbit(out[1]).any()  # (+0) + (-0) = +0, as in the reference's CopyFrom + Axpy
    assert (out[2] == 0).all() and not np.signbit(out[2]).any()


def test_level_rejects_bad_arguments(gpu_ctx):
    from graphnn_b200.capi import S2VError
    p = synth.erdos_renyi_level(n=64, nnz=100, d=64, seed=0)
    rp, ci, H, W, X = dev(p.row_ptr), dev(p.col_idx), dev(p.H), dev(p.W), dev(p.X)
    out = torch.empty((64, 64), device="cuda")
    with pytest.raises(S2VError) as e:
        gpu_ctx.level(rp, ci, None, H, W, X, H)                     # aliasing
    assert e.value.status == -1
    with pytest.raises(S2VError) as e:
        gpu_ctx.level(rp[:64], ci, None, H, W, X.flatten()[1:1 + 63 * 64].view(63, 64), out[:63])   # X off by 4 bytes
    assert e.value.status == -1
    bad = torch.empty((64, 48), device="cuda")
    with pytest.raises(S2VError) as e:
        gpu_ctx.level(rp, ci, None, torch.empty((64, 48), device="cuda"), W, None, bad)
    assert e.value.status == -2                                      # unsupported d
    with pytest.raises(S2VError):
        gpu_ctx.level(rp, ci, None, H, None, X, out)                # NULL W


# ------------------------------------------------------------------ unfused operations
def test_spmm_alpha_beta(gpu_ctx, oracle_lib):
    p = synth.erdos_renyi_level(n=513, nnz=4000, d=64, seed=9)
    rng = np.random.default_rng(1)
    for n in (64, 7):
        B = rng.standard_normal((513, n), dtype=np.float32)
        C0 = rng.standard_normal((513, n), dtype=np.float32)
        val = rng.random(p.nnz, dtype=np.float32)
        import scipy.sparse as sp
        A = sp.csr_matrix((val.astype(np.float64), p.col_idx, p.row_ptr), shape=(513, 513))
        C = dev(C0.copy())
        gpu_ctx.spmm(513, 513, dev(p.row_ptr), dev(p.col_idx), dev(val), dev(B), C, alpha=0.5, beta=2.0)
        gpu_ctx.synchronize()
        assert_close(C.cpu().numpy(), 0.5 * (A @ B.astype(np.float64)) + 2.0 * C0, f"spmm n={n}")
        C = torch.full((513, n), float("nan"), device="cuda")       # beta = 0 must overwrite, not scale
        gpu_ctx.spmm(513, 513, dev(p.row_ptr), dev(p.col_idx), None, dev(B), C)
        gpu_ctx.synchronize()
        A1 = sp.csr_matrix((np.ones(p.nnz), p.col_idx, p.row_ptr), shape=(513, 513))
        assert_close(C.cpu().numpy(), A1 @ B.astype(np.float64), f"spmm ones n={n}")


@pytest.mark.parametrize("ta,tb", [(False, False), (True, False), (False, True), (True, True)])
def test_gemm(gpu_ctx, ta, tb):
    rng = np.random.default_rng(3)
    m, n, k = 131, 70, 45
    A = rng.standard_normal((k, m) if ta else (m, k), dtype=np.float32)
    B = rng.standard_normal((n, k) if tb else (k, n), dtype=np.float32)
    C0 = rng.standard_normal((m, n), dtype=np.float32)
    C = dev(C0.copy())
    gpu_ctx.gemm(dev(A), dev(B), C, trans_a=ta, trans_b=tb, alpha=1.5, beta=-0.5)
    gpu_ctx.synchronize()
    ref = 1.5 * ((A.T if ta else A).astype(np.float64) @ (B.T if tb else B).astype(np.float64)) - 0.5 * C0
    assert_close(C.cpu().numpy(), ref, "gemm", scale=4)


def test_elementwise_softmax_argmax(gpu_ctx, oracle_lib):
    rng = np.random.default_rng(5)
    x = rng.standard_normal(100003, dtype=np.float32)
    y0 = rng.standard_normal(100003, dtype=np.float32)
    y = dev(y0.copy())
    gpu_ctx.axpy(0.75, dev(x), y)
    r = torch.empty(100003, device="cuda")
    gpu_ctx.relu(dev(x), r)
    s = dev(x.copy())
    gpu_ctx.scale(0.0, s)
    gpu_ctx.synchronize()
    assert_close(y.cpu().numpy(), y0 + np.float32(0.75) * x, "axpy")
    assert np.array_equal(r.cpu().numpy(), np.where(x < 0, np.float32(0), x))
    special = np.array([-0.0, np.nan, -1.0, 2.0], np.float32)     # `if (x < 0) x = 0` keeps -0.0 and NaN
    rs = torch.empty(4, device="cuda")
    gpu_ctx.relu(dev(special), rs)
    gpu_ctx.synchronize()
    rs = rs.cpu().numpy()
    assert rs[0] == 0 and np.signbit(rs[0]) and np.isnan(rs[1]) and rs[2] == 0 and rs[3] == 2
    assert (s.cpu().numpy() == 0).all()
    for cols in (2, 5, 33, 1023):
        l = rng.standard_normal((37, cols), dtype=np.float32) * 3
        l[3, :] = 1.25                     # full tie: first index wins
        if cols > 4:
            l[5, 4] = l[5, 1] = l[5].max() + 1
        P = torch.empty((37, cols), device="cuda")
        I = torch.empty(37, dtype=torch.int32, device="cuda")
        gpu_ctx.softmax(dev(l), P)
        gpu_ctx.argmax(dev(l), I)
        gpu_ctx.synchronize()
        e = np.exp(l.astype(np.float64) - l.max(1, keepdims=True))
        assert_close(P.cpu().numpy(), e / e.sum(1, keepdims=True), f"softmax {cols}")
        assert np.array_equal(I.cpu().numpy(), l.argmax(1).astype(np.int32))
        assert I[3].item() == 0
