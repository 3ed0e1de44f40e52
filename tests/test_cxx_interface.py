"""The host-side C++ mirror of the graphnn operator interface (graphnn_b200/cxx/include):
host-only semantics on CPU, and the inference driver written against it on the GPU, in the
reference's unfused wiring and in the fused wiring, against the reference's golden vectors."""
import os
import struct
import subprocess

import numpy as np
import pytest

from conftest import assert_close
from graphnn_b200 import build as lib_build
from graphnn_b200 import synth


@pytest.fixture(scope="module")
def cxx_bins():
    lib_build.build()
    return lib_build.build_cxx()


def test_host_interface_semantics(cxx_bins):
    r = subprocess.run([cxx_bins["host_interface_test"]], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.split() == ["ok", "schedule", "ok", "msg_pass", "ok", "cpu_tensors"]


def write_batch(path, b):
    with open(path, "wb") as f:
        f.write(struct.pack("8i", b.num_graphs, b.num_nodes, b.num_edges, b.num_tags, b.d, b.levels, b.hidden, b.num_class))
        for a in (b.nodes_per_graph, b.edge_src, b.edge_dst, b.tags):
            f.write(np.ascontiguousarray(a, np.int32).tobytes())
        for k in ("w_n2l", "p_node_conv", "h1_weight", "h2_weight"):
            f.write(np.ascontiguousarray(b.weights[k], np.float32).tobytes())


def read_result(path, b):
    raw = open(path, "rb").read()
    G, N, E, C, d = b.num_graphs, b.num_nodes, b.num_edges, b.num_class, b.d
    off = 0

    def take(n, dt):
        nonlocal off
        a = np.frombuffer(raw, dt, n, off)
        off += n * 4
        return a
    out = {"logits": take(G * C, np.float32).reshape(G, C), "probs": take(G * C, np.float32).reshape(G, C),
           "pred": take(G, np.int32), "embed": take(N * d, np.float32).reshape(N, d),
           "row_ptr": take(N + 1, np.int32), "col_idx": take(E, np.int32)}
    assert off == len(raw)
    return out


@pytest.mark.gpu
@pytest.mark.parametrize("fused", [0, 1])
def test_driver_matches_reference_golden(cxx_bins, golden, tmp_path, fused):
    g = golden("mutag_like_seed0.npz")
    b = synth.mutag_like(seed=0)
    write_batch(tmp_path / "batch.bin", b)
    r = subprocess.run([cxx_bins["s2v_mean_field"], str(tmp_path / "batch.bin"), str(tmp_path / "out.bin"),
                        "--fused", str(fused), "--iters", "2"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    o = read_result(tmp_path / "out.bin", b)
    assert np.array_equal(o["row_ptr"], g["n2n_row_ptr"]) and np.array_equal(o["col_idx"], g["n2n_col_idx"])
    assert np.array_equal(o["pred"], g["argmax"])
    assert_close(o["embed"], g["last_level"], "embeddings")
    assert_close(o["logits"], g["logits"], "logits")
    assert_close(o["probs"], g["probs"], "probs")
    # the unfused wiring runs one kernel per tensor operation, the fused one per level
    factors = int(r.stderr.split(" factors")[0].split()[-1])
    assert factors == (4 + 4 * b.levels + 6 if not fused else 4 + b.levels + 4)


@pytest.mark.gpu
def test_driver_on_a_larger_batch(cxx_bins, oracle_lib, tmp_path):
    b = synth.molecules_16k(seed=3, num_graphs=600)
    o = oracle_lib.forward(b, "oracle")
    write_batch(tmp_path / "batch.bin", b)
    for fused in (0, 1):
        r = subprocess.run([cxx_bins["s2v_mean_field"], str(tmp_path / "batch.bin"), str(tmp_path / "out.bin"),
                            "--fused", str(fused)], capture_output=True, text=True, timeout=120)
        assert r.returncode == 0, r.stdout + r.stderr
        got = read_result(tmp_path / "out.bin", b)
        assert np.array_equal(got["row_ptr"], o["n2n_row_ptr"]) and np.array_equal(got["col_idx"], o["n2n_col_idx"])
        assert_close(got["embed"], o["levels"][-1], f"embeddings fused={fused}")
        assert_close(got["logits"], o["logits"], f"logits fused={fused}", scale=max(1.0, float(np.abs(o["logits"]).max())))
        assert np.array_equal(got["pred"], o["argmax"])


@pytest.mark.gpu
@pytest.mark.parametrize("fused", [0, 1])
def test_driver_loss_and_accuracy_targets(cxx_bins, golden, tmp_path, fused):
    """The reference's TEST-loop targets {loss, acc} through the mirrored factors
    (CrossEntropy, ReduceMean, ArgMax on the CSR labels, InTopK, TypeCast)."""
    t = golden("loss_acc_seed3.npz")
    b = synth.mutag_like(seed=3)
    write_batch(tmp_path / "batch.bin", b)
    np.ascontiguousarray(t["labels"], np.int32).tofile(tmp_path / "labels.bin")
    r = subprocess.run([cxx_bins["s2v_mean_field"], str(tmp_path / "batch.bin"), str(tmp_path / "out.bin"), "--fused", str(fused),
                        "--labels", str(tmp_path / "labels.bin")], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    words = r.stdout.split()
    loss, acc = float(words[1]), float(words[3])
    assert abs(loss - float(t["loss"])) <= 1e-5 * max(1.0, abs(float(t["loss"])))
    assert acc == float(t["acc"])


def test_checkpoint_format_against_reference_written_file(cxx_bins, golden, tmp_path):
    """tests/golden/tiny_reference_saved.model was written by the reference's ParamSet::Save."""
    from conftest import GOLDEN
    from graphnn_b200 import io
    src = os.path.join(GOLDEN, "tiny_reference_saved.model")
    w = golden("tiny_reference_saved_weights.npz")
    got = io.read_model(src)
    for k in ("w_n2l", "p_node_conv", "h1_weight", "h2_weight"):
        assert np.array_equal(got[k], w[k]), k
    io.write_model(str(tmp_path / "py.model"), {k: w[k] for k in w.files})
    assert open(src, "rb").read() == open(tmp_path / "py.model", "rb").read()
    # the C++ mirror: Load the reference's file, Save it again, same bytes
    r = subprocess.run([cxx_bins["host_interface_test"], src, str(tmp_path / "cxx.model")], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0 and "ok checkpoint" in r.stdout, r.stdout + r.stderr
    first = [float(x) for x in r.stdout.splitlines()[0].split()[1:]]
    assert np.allclose(first, [w["w_n2l"][0, 0], w["p_node_conv"][0, 0], w["h1_weight"][0, 0], w["h2_weight"][4, 1]], rtol=1e-7)
    assert open(src, "rb").read() == open(tmp_path / "cxx.model", "rb").read()


def test_txt_dataset_round_trip(tmp_path):
    from graphnn_b200 import io
    b = synth.mutag_like(seed=2, num_graphs=9)
    graphs = io.graphs_of_batch(b)
    labels = np.arange(9) % 2
    io.write_txt_dataset(str(tmp_path / "d.txt"), graphs, labels)
    g2, l2 = io.read_txt_dataset(str(tmp_path / "d.txt"))
    assert np.array_equal(l2, labels) and len(g2) == 9
    for (t1, a1), (t2, a2) in zip(graphs, g2):
        assert np.array_equal(t1, t2) and all(np.array_equal(x, y) for x, y in zip(a1, a2))
    ref_file = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference",
                            "examples", "graph_classification", "data", "MUTAG", "MUTAG.txt")
    if os.path.exists(ref_file):     # the reference's own file, when a checkout is next to this repository
        g, l = io.read_txt_dataset(ref_file)
        assert len(g) == len(l) > 100 and len(set(l.tolist())) == 2
        for tags, adj in g[:20]:          # undirected graphs: every neighbour list is mirrored
            pairs = {(i, int(j)) for i, nb in enumerate(adj) for j in nb}
            assert all((j, i) in pairs for i, j in pairs) and all(0 <= j < len(tags) for _, j in pairs)


@pytest.mark.gpu
def test_serving_driver_on_text_dataset_and_checkpoint(cxx_bins, oracle_lib, tmp_path):
    """s2v_classify: text data set + ParamSet checkpoint -> batched inference, loss and accuracy."""
    from graphnn_b200 import io
    b = synth.mutag_like(seed=3, num_graphs=40)
    labels = np.random.default_rng(1).integers(0, 2, 40).astype(np.int32)
    io.write_txt_dataset(str(tmp_path / "d.txt"), io.graphs_of_batch(b), labels)
    io.write_model(str(tmp_path / "w.model"), b.weights)
    idx = np.arange(39, -1, -1)                 # reversed order: batches differ from the file order
    np.savetxt(tmp_path / "idx.txt", idx, fmt="%d")
    r = subprocess.run([cxx_bins["s2v_classify"], "-graph", str(tmp_path / "d.txt"), "-model", str(tmp_path / "w.model"),
                        "-test_idx", str(tmp_path / "idx.txt"), "-conv", "64", "-hidden", "128", "-lv", "3", "-b", "16",
                        "-node_dim", "7", "-out", str(tmp_path / "pred.txt")], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    o = oracle_lib.forward(b, "oracle", want_levels=False)
    pred = np.loadtxt(tmp_path / "pred.txt", dtype=int)
    assert np.array_equal(pred[:, 0], idx) and np.array_equal(pred[:, 1], o["argmax"][idx]) and np.array_equal(pred[:, 2], labels[idx])
    want_loss, want_acc, _ = oracle_lib.loss_acc(o["logits"], labels, "oracle")
    words = r.stdout.split()
    assert abs(float(words[2]) - want_loss) <= 1e-5 * max(1.0, want_loss) and abs(float(words[4]) - want_acc) < 1e-6


def _gpus_for_test():
    import torch
    return max(1, min(2, torch.cuda.device_count()))


@pytest.mark.gpu
def test_multi_gpu_host_program_shard_by_graph(cxx_bins, oracle_lib, tmp_path):
    """The C++ host that uses only include/s2v_b200.h: graphs sharded over the GPUs present (two if there are two),
    one host thread per GPU, logits gathered with s2v_gather_logits; against the CPU oracle on the whole batch."""
    b = synth.molecules_16k(seed=5, num_graphs=1200)
    write_batch(tmp_path / "batch.bin", b)
    P = _gpus_for_test()
    r = subprocess.run([cxx_bins["s2v_multi_gpu"], "shard", str(tmp_path / "batch.bin"), str(tmp_path / "out.bin"), "--gpus", str(P), "--iters", "2"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert f"shard gpus {P} ms_per_iter" in r.stdout
    raw = open(tmp_path / "out.bin", "rb").read()
    G, C = b.num_graphs, b.num_class
    logits = np.frombuffer(raw, np.float32, G * C, 0).reshape(G, C)
    pred = np.frombuffer(raw, np.int32, G, 4 * G * C)
    o = oracle_lib.forward(b, "oracle", want_levels=False)
    assert_close(logits, o["logits"], "sharded logits", scale=max(1.0, float(np.abs(o["logits"]).max())))
    margin = np.sort(o["logits"], axis=1)
    safe = (margin[:, -1] - margin[:, -2]) > 1e-4 * np.abs(o["logits"]).max()
    assert np.array_equal(pred[safe], o["argmax"][safe]) and safe.mean() > 0.9


@pytest.mark.gpu
@pytest.mark.parametrize("exchange", ["allgather", "referenced"])
@pytest.mark.parametrize("d,chunks", [(64, 3), (128, 1)])
def test_multi_gpu_host_program_giant_graph(cxx_bins, oracle_lib, tmp_path, d, chunks, exchange):
    """Row-partitioned single graph from the same C++ host: block-major H with one in-place all-gather per block and
    level, or (exchange = referenced) every GPU fetching only the rows it references through s2v_exchange_rows_f32."""
    from graphnn_b200.synth import LevelProblem
    p = synth.rmat_level(scale=12, edge_factor=8, d=d, seed=4)
    with open(tmp_path / "graph.bin", "wb") as f:
        f.write(struct.pack("3q", p.n_rows, p.nnz, d))
        f.write(np.ascontiguousarray(p.row_ptr, np.int64).tobytes())
        f.write(np.ascontiguousarray(p.col_idx, np.int32).tobytes())
        f.write(np.ascontiguousarray(p.H, np.float32).tobytes())
        f.write(np.ascontiguousarray(p.W, np.float32).tobytes())
    P = _gpus_for_test()
    r = subprocess.run([cxx_bins["s2v_multi_gpu"], "giant", str(tmp_path / "graph.bin"), str(tmp_path / "out.bin"), "--gpus", str(P),
                        "--levels", "2", "--chunks", str(chunks), "--iters", "2"] + (["--exchange", "referenced"] if exchange == "referenced" else []),
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    got = np.fromfile(tmp_path / "out.bin", np.float32).reshape(p.n_rows, d)
    H = p.H
    for _ in range(2):
        H, _ = oracle_lib.level(LevelProblem(p.n_rows, p.n_src, p.row_ptr, p.col_idx, H, p.W, None), "oracle")
    assert_close(got, H, f"giant graph on {P} GPU(s), exchange {exchange}", scale=max(1.0, float(np.abs(H).max())))
    if exchange == "referenced":
        assert "referenced_remote_rows" in r.stdout
