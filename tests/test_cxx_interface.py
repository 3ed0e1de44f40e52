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
