"""GPU parity of the whole classifier (input projection, L levels, pooling, readout)
against the reference's golden vectors and the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch

from conftest import assert_close
from graphnn_b200 import engine, synth

pytestmark = pytest.mark.gpu


def run(batch, dense=False, want_embed=True):
    eng = engine.S2VInference(batch.weights, batch.levels)
    hb = engine.build_host_batch(batch)
    db = eng.to_device(hb, batch.dense_x() if dense else None)
    logits, probs, pred, embed = eng.forward(db, want_embed=want_embed)
    eng.ctx.synchronize()
    return eng, hb, logits.cpu().numpy(), probs.cpu().numpy(), pred.cpu().numpy(), (embed.cpu().numpy() if want_embed else None)


@pytest.mark.parametrize("dense", [False, True])
def test_classifier_matches_reference_golden(golden, dense):
    g = golden("mutag_like_seed0.npz")
    b = synth.mutag_like(seed=0)
    eng, hb, logits, probs, pred, embed = run(b, dense)
    assert np.array_equal(hb.row_ptr.numpy(), g["n2n_row_ptr"])        # CSR construction: bit-exact
    assert np.array_equal(hb.col_idx.numpy(), g["n2n_col_idx"])
    assert np.array_equal(hb.graph_ptr.numpy(), g["sub_row_ptr"])      # pooling indices: bit-exact
    assert np.array_equal(pred, g["argmax"])                           # predictions: bit-exact
    assert_close(embed, g["last_level"], "embeddings")
    assert_close(logits, g["logits"], "logits")
    assert_close(probs, g["probs"], "probs")
    # dense X: projection, L levels, pooling, readout; tags: product table, first level (which also range-checks the tags),
    # L - 1 levels, pooling, readout
    assert eng.ctx.launches == 3 + b.levels


def test_classifier_mixed_classes_golden(golden):
    g = golden("mutag_like_seed3.npz")
    b = synth.mutag_like(seed=3)
    _, _, logits, probs, pred, _ = run(b)
    assert np.array_equal(pred, g["argmax"])
    assert_close(logits, g["logits"], "logits")
    assert_close(probs, g["probs"], "probs")


@pytest.mark.parametrize("maker", [
    lambda: synth.molecules_16k(seed=1, num_graphs=700),
    lambda: synth.proteins_4k(seed=1, num_graphs=40),
    lambda: synth.molecule_like(33, 1, 5, 4, 32, 2, 16, 3, 0.3, "uniform", seed=8),   # single-node graphs, 3 classes
])
def test_classifier_matches_oracle(oracle_lib, maker):
    b = maker()
    o = oracle_lib.forward(b, "oracle")
    _, hb, logits, probs, pred, embed = run(b)
    assert np.array_equal(hb.row_ptr.numpy(), o["n2n_row_ptr"])
    assert np.array_equal(hb.col_idx.numpy(), o["n2n_col_idx"])
    # the last level's values reach tens (proteins: 43): like the logits they are held to 1e-5 of their scale; fp32
    # arithmetic in any order is itself 9e-6 away from the float64 restatement on the largest of these batches
    assert_close(embed, o["levels"][-1], "embeddings", scale=max(1.0, float(np.abs(o["levels"][-1]).max())))
    assert_close(logits, o["logits"], "logits", scale=max(1.0, float(np.abs(o["logits"]).max())))
    assert_close(probs, o["probs"], "probs")
    margin = np.sort(o["logits"], axis=1)
    safe = (margin[:, -1] - margin[:, -2]) > 1e-4 * np.abs(o["logits"]).max()
    assert np.array_equal(pred[safe], o["argmax"][safe])
    assert safe.mean() > 0.9


def test_host_buffer_entry_point(oracle_lib):
    b = synth.molecules_16k(seed=2, num_graphs=300)
    o = oracle_lib.forward(b, "oracle", want_levels=False)
    eng = engine.S2VInference(b.weights, b.levels)
    hb = engine.build_host_batch(b)
    for _ in range(2):                      # second call reuses the context's staging buffers
        logits, pred = eng.infer_host(hb)
        assert_close(logits, o["logits"], "logits", scale=max(1.0, float(np.abs(o["logits"]).max())))
        assert np.array_equal(pred, o["argmax"])
    # a smaller batch afterwards must not read stale data
    b2 = synth.mutag_like(seed=0)
    eng2 = engine.S2VInference(b2.weights, b2.levels)
    o2 = oracle_lib.forward(b2, "oracle", want_levels=False)
    logits2, pred2 = eng2.infer_host(engine.build_host_batch(b2))
    assert_close(logits2, o2["logits"], "logits")
    assert np.array_equal(pred2, o2["argmax"])


def test_pooling_and_readout_separately(gpu_ctx, oracle_lib):
    rng = np.random.default_rng(11)
    for d, hidden, C in ((64, 128, 2), (128, 256, 2), (48, 20, 5)):
        sizes = rng.integers(0, 70, 50)          # includes empty graphs
        seg = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int32)
        H = rng.standard_normal((int(seg[-1]), d), dtype=np.float32)
        Y = torch.full((50, d), float("nan"), device="cuda")
        gpu_ctx.segment_sum(torch.from_numpy(seg).cuda(), torch.from_numpy(H).cuda(), Y)
        gpu_ctx.synchronize()
        want = np.stack([H[seg[g]:seg[g + 1]].astype(np.float64).sum(0) for g in range(50)])
        assert_close(Y.cpu().numpy(), want, f"segment sum d={d}", scale=8)
        W1 = rng.standard_normal((d, hidden), dtype=np.float32) * 0.1
        W2 = rng.standard_normal((hidden, C), dtype=np.float32) * 0.1
        logits = torch.empty((50, C), device="cuda")
        probs = torch.empty((50, C), device="cuda")
        pred = torch.empty(50, dtype=torch.int32, device="cuda")
        gpu_ctx.readout(Y, torch.from_numpy(W1).cuda(), torch.from_numpy(W2).cuda(), logits, probs, pred)
        gpu_ctx.synchronize()
        hid = np.maximum(want @ W1.astype(np.float64), 0)
        lg = hid @ W2.astype(np.float64)
        assert_close(logits.cpu().numpy(), lg, "readout logits", scale=8)
        e = np.exp(lg - lg.max(1, keepdims=True))
        assert_close(probs.cpu().numpy(), e / e.sum(1, keepdims=True), "readout probs", scale=8)
        assert np.array_equal(pred.cpu().numpy(), logits.cpu().numpy().argmax(1))


@pytest.mark.parametrize("G,d,hidden,C", [(2048, 128, 256, 2), (5000, 64, 128, 3), (2049, 128, 256, 2),
                                          (148 * 128 * 2 + 77, 128, 256, 8),     # more tiles than SMs: a CTA takes several, 8 classes
                                          (300, 128, 256, 2), (40000, 64, 256, 5), (20011, 128, 128, 3)])
def test_readout_large_batch(gpu_ctx, G, d, hidden, C):
    """Readout on batches of hundreds to tens of thousands of graphs: from 6,144 graphs on the first layer runs on
    the tcgen05 kernel (128-graph tiles, the last one ragged), below that on the mma.sync kernel."""
    rng = np.random.default_rng(G)
    Y = rng.standard_normal((G, d), dtype=np.float32) * 3.0
    W1 = rng.standard_normal((d, hidden), dtype=np.float32) * 0.1
    W2 = rng.standard_normal((hidden, C), dtype=np.float32) * 0.1
    logits = torch.full((G, C), float("nan"), device="cuda")
    probs = torch.empty((G, C), device="cuda")
    pred = torch.empty(G, dtype=torch.int32, device="cuda")
    gpu_ctx.readout(torch.from_numpy(Y).cuda(), torch.from_numpy(W1).cuda(), torch.from_numpy(W2).cuda(), logits, probs, pred)
    gpu_ctx.synchronize()
    hid = np.maximum(Y.astype(np.float64) @ W1.astype(np.float64), 0)
    lg = hid @ W2.astype(np.float64)
    assert_close(logits.cpu().numpy(), lg, "readout logits", scale=8)
    e = np.exp(lg - lg.max(1, keepdims=True))
    assert_close(probs.cpu().numpy(), e / e.sum(1, keepdims=True), "readout probs", scale=8)
    assert np.array_equal(pred.cpu().numpy(), logits.cpu().numpy().argmax(1))


def test_full_size_properties():
    """At the benchmark's full molecule size the oracle is too slow to run per test;
    check size-independent properties instead: a permutation of the graphs permutes
    the predictions, and duplicating a graph duplicates its logits bit for bit."""
    b = synth.molecules_16k(seed=0, num_graphs=4096)
    eng = engine.S2VInference(b.weights, b.levels)
    hb = engine.build_host_batch(b)
    logits, _, pred, _ = eng.forward(eng.to_device(hb))
    eng.ctx.synchronize()
    logits = logits.cpu().numpy()
    half = b.shard(1, 2)                                # graphs of the second half alone
    lo = synth.shard_bounds(b.nodes_per_graph, 2)[1][0]
    l2, _, _, _ = eng.forward(eng.to_device(engine.build_host_batch(half)))
    eng.ctx.synchronize()
    assert np.array_equal(l2.cpu().numpy(), logits[lo:])   # block-diagonal independence, bit-exact
    assert np.isfinite(logits).all()


def test_loss_accuracy_tail_on_device(gpu_ctx, oracle_lib, golden):
    """Fused loss/accuracy launch and the per-factor kernels against the reference's golden tail."""
    g = golden("mutag_like_seed3.npz")
    t = golden("loss_acc_seed3.npz")
    G, C = g["logits"].shape
    logits = torch.from_numpy(g["logits"]).cuda()
    rp = torch.arange(G + 1, dtype=torch.int32, device="cuda")
    ci = torch.from_numpy(t["labels"]).cuda()
    val = torch.ones(G, device="cuda")
    loss = torch.zeros(1, device="cuda")
    acc = torch.zeros(1, device="cuda")
    per = torch.zeros(G, device="cuda")
    gpu_ctx.loss_acc(logits, rp, ci, val, loss, acc, per)
    gpu_ctx.synchronize()
    assert abs(loss.item() - float(t["loss"])) <= 1e-5 * max(1.0, abs(float(t["loss"])))
    assert acc.item() == float(t["acc"])
    assert_close(per.cpu().numpy(), t["per_graph"], "per-graph loss")
    # the same through the one-kernel-per-factor entry points
    ce = torch.zeros(G, device="cuda")
    truth = torch.zeros(G, dtype=torch.int32, device="cuda")
    hit = torch.zeros(G, dtype=torch.int32, device="cuda")
    hitf = torch.zeros(G, device="cuda")
    m = torch.zeros(2, device="cuda")
    gpu_ctx.call("s2v_cross_entropy_f32", None, G, C, logits.data_ptr(), 1, rp.data_ptr(), ci.data_ptr(), val.data_ptr(), ce.data_ptr())
    gpu_ctx.call("s2v_argmax_csr_f32", None, G, rp.data_ptr(), ci.data_ptr(), val.data_ptr(), truth.data_ptr())
    gpu_ctx.call("s2v_in_top_k_f32", None, G, C, logits.data_ptr(), truth.data_ptr(), 1, hit.data_ptr())
    gpu_ctx.call("s2v_cast_i32_f32", None, G, hit.data_ptr(), hitf.data_ptr())
    gpu_ctx.call("s2v_mean_f32", None, G, ce.data_ptr(), m.data_ptr())
    gpu_ctx.call("s2v_mean_f32", None, G, hitf.data_ptr(), m.data_ptr() + 4)
    gpu_ctx.synchronize()
    assert torch.equal(truth.cpu(), ci.cpu()) and torch.equal(ce, per)
    assert abs(m[0].item() - float(t["loss"])) <= 1e-5 * max(1.0, abs(float(t["loss"]))) and m[1].item() == float(t["acc"])
    # large random case against the oracle
    rng = np.random.default_rng(1)
    lg = (rng.standard_normal((5000, 6)) * 8).astype(np.float32)
    lab = rng.integers(0, 6, 5000).astype(np.int32)
    want = oracle_lib.loss_acc(lg, lab, "oracle", topk=2)
    l2, a2 = torch.zeros(1, device="cuda"), torch.zeros(1, device="cuda")
    gpu_ctx.loss_acc(torch.from_numpy(lg).cuda(), torch.arange(5001, dtype=torch.int32, device="cuda"), torch.from_numpy(lab).cuda(),
                     None, l2, a2, None, topk=2)
    gpu_ctx.synchronize()
    assert abs(l2.item() - want[0]) <= 2e-5 * abs(want[0]) and abs(a2.item() - want[1]) <= 1e-6
