"""CPU tests of the C-ABI library: it loads, exports every declared entry point, and
its host-only entry points work without a GPU."""
import ctypes
import os
import re

import numpy as np
import pytest

from conftest import REPO
from graphnn_b200 import capi, synth


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(capi.LIB_PATH):
        from graphnn_b200 import build
        build.build()
    return capi.load_library()


def declared_symbols():
    names = set()
    inc = os.path.join(REPO, "include")
    for f in os.listdir(inc):
        if f.endswith(".h"):
            text = open(os.path.join(inc, f)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"\b(s2v_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_every_declared_symbol_is_exported(lib):
    names = declared_symbols()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/ but not exported"
    # and the Python binding knows each of them
    assert set(names) == set(capi.exported_symbols())


def test_status_strings(lib):
    assert lib.s2v_status_str(0) == b"ok"
    assert b"CSR" in lib.s2v_status_str(-4)
    assert lib.s2v_forward_workspace_bytes(1000, 10, 64) >= 3 * 1000 * 64 * 4 + 10 * 64 * 4
    assert lib.s2v_forward_workspace_bytes(-1, 10, 64) == 0


def test_ctx_create_without_gpu_fails_loudly(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = ctypes.c_void_p()
    rc = lib.s2v_ctx_create(0, ctypes.byref(h))
    assert rc == -6 and not h.value          # S2V_ERR_NO_DEVICE, no CPU fallback
    with pytest.raises(capi.S2VError):
        capi.Context(0)


def test_host_csr_builder_matches_oracle_and_golden(lib, oracle_lib, golden):
    g = golden("mutag_like_seed0.npz")
    b = synth.mutag_like(seed=0)
    rp, ci, val = capi.build_n2n_csr_host(b.num_nodes, b.edge_src, b.edge_dst)
    assert np.array_equal(rp, g["n2n_row_ptr"]) and np.array_equal(ci, g["n2n_col_idx"])
    assert np.array_equal(val, g["n2n_val"])
    assert np.array_equal(b.graph_offsets(), g["sub_row_ptr"])
    assert np.array_equal(np.arange(b.num_nodes, dtype=np.int32), g["sub_col_idx"])
    # unsorted insertion order is preserved inside a row (AddEdge order), duplicates kept
    src = np.array([3, 1, 2, 1, 0], np.int32)
    dst = np.array([0, 0, 0, 0, 2], np.int32)
    rp, ci, val = capi.build_n2n_csr_host(4, src, dst, average=True)
    assert rp.tolist() == [0, 4, 4, 5, 5] and ci.tolist() == [3, 1, 2, 1, 0]
    assert np.allclose(val, [0.25, 0.25, 0.25, 0.25, 1.0])
    # empty graph
    rp, ci, _ = capi.build_n2n_csr_host(3, np.zeros(0, np.int32), np.zeros(0, np.int32))
    assert rp.tolist() == [0, 0, 0, 0] and ci.size == 0


def test_host_csr_builder_rejects_bad_edges(lib):
    with pytest.raises(capi.S2VError) as e:
        capi.build_n2n_csr_host(4, np.array([0, 5], np.int32), np.array([1, 2], np.int32))
    assert e.value.status == -4
    with pytest.raises(capi.S2VError):
        capi.build_n2n_csr_host(4, np.array([0, -1], np.int32), np.array([1, 2], np.int32))


def test_validate_csr(lib):
    rp = np.array([0, 2, 2, 3], np.int32)
    ci = np.array([1, 0, 2], np.int32)
    assert capi.validate_csr_host(3, 3, rp, ci) == 0
    assert capi.validate_csr_host(3, 2, rp, ci) == -4            # column out of range
    assert capi.validate_csr_host(3, 3, np.array([0, 2, 1, 3], np.int32), ci) == -4   # not monotone
    assert capi.validate_csr_host(3, 3, np.array([1, 2, 2, 3], np.int32), ci) == -4   # does not start at 0
    assert capi.validate_csr_host(3, 3, np.array([0, 2, 2, 2], np.int32), ci) == -4   # nnz mismatch


@pytest.mark.parametrize("average", [False, True])
def test_edge_level_msgpass_builders_match_reference_golden(lib, golden, average):
    """Edge2Node / Node2Edge / Edge2Edge host builders against the matrices the reference's own factors built
    (tests/golden/msgpass_matrices_mutag_seed0.npz), bit for bit; the n2n average form as well."""
    g = golden("msgpass_matrices_mutag_seed0.npz")
    b = synth.mutag_like(seed=0)
    assert str(g["digest"]) == b.digest()
    tag = "avg" if average else "sum"
    mats = capi.build_edge_csrs_host(b.num_nodes, b.edge_src, b.edge_dst, average=average)
    for which in ("e2n", "n2e", "e2e"):
        rp, ci, val = mats[which]
        assert np.array_equal(rp, g[f"{which}_{tag}_row_ptr"]), which
        assert np.array_equal(ci, g[f"{which}_{tag}_col_idx"]), which
        assert np.array_equal(val, g[f"{which}_{tag}_val"]), which
    rp, ci, val = capi.build_n2n_csr_host(b.num_nodes, b.edge_src, b.edge_dst, average=average)
    assert np.array_equal(rp, g[f"n2n_{tag}_row_ptr"]) and np.array_equal(ci, g[f"n2n_{tag}_col_idx"])
    assert np.array_equal(val, g[f"n2n_{tag}_val"])


def test_edge_level_builders_on_a_large_batch_and_bad_input(lib, oracle_lib):
    b = synth.molecules_16k(seed=4, num_graphs=3000)        # large enough for the OpenMP path of the sort
    mats = capi.build_edge_csrs_host(b.num_nodes, b.edge_src, b.edge_dst, average=True)
    for which in ("e2n", "n2e", "e2e"):
        want = oracle_lib.msgpass_matrix(b, which, "oracle", True)
        assert all(np.array_equal(x, y) for x, y in zip(mats[which], want)), which
    # a small directed graph worked out by hand: 0->1, 1->2, 2->0, 0->2.  Row e = (from -> to) keeps the edges
    # into `from` that do not come from `to`: the last edge (0->2) loses its only candidate 2->0.
    src = np.array([0, 1, 2, 0], np.int32)
    dst = np.array([1, 2, 0, 2], np.int32)
    m = capi.build_edge_csrs_host(3, src, dst)
    assert m["e2e"][0].tolist() == [0, 1, 2, 3, 3] and m["e2e"][1].tolist() == [2, 0, 1]
    assert m["e2n"][0].tolist() == [0, 1, 2, 4] and m["e2n"][1].tolist() == [2, 0, 1, 3]
    assert m["n2e"][1].tolist() == [0, 1, 2, 0]
    with pytest.raises(capi.S2VError):
        capi.build_edge_csrs_host(3, np.array([0, 5], np.int32), np.array([1, 2], np.int32))
