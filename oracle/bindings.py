"""ctypes front-ends of the two compiled checkers (TEST INFRASTRUCTURE ONLY).

``forward(batch, impl)`` runs the whole classifier on a ``GraphBatch``-like object
and returns every intermediate the parity tests compare; ``level(problem, impl)``
runs one message-passing level.  ``impl`` is ``"oracle"`` (s2v_oracle.c) or
``"reference"`` (the reference's C++ behind ref_harness.cpp).
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_ORACLE_SO = os.path.join(HERE, "libs2v_oracle.so")
_REF_SO = os.path.join(HERE, "_ref", "libs2v_ref.so")
_libs: dict = {}

_i32p = C.POINTER(C.c_int32)
_f32p = C.POINTER(C.c_float)
_f64p = C.POINTER(C.c_double)


def have_reference() -> bool:
    return os.path.exists(_REF_SO)


def _lib(impl: str):
    if impl not in _libs:
        path = _ORACLE_SO if impl == "oracle" else _REF_SO
        if not os.path.exists(path):
            raise FileNotFoundError(f"{path} is not built: run `python oracle/build.py`")
        _libs[impl] = C.CDLL(path)
    return _libs[impl]


def _p(a, typ):
    return None if a is None else a.ctypes.data_as(typ)


def set_threads(n: int, impl: str = "oracle") -> None:
    lib = _lib(impl)
    (lib.oracle_set_threads if impl == "oracle" else lib.ref_set_threads)(C.c_int(int(n)))


def forward(batch, impl: str = "oracle", iters: int = 1, want_levels: bool = True) -> dict:
    """Whole classifier on the CPU.  Returns CSR arrays, msg, levels, pooled, logits, probs, argmax (+ seconds)."""
    lib = _lib(impl)
    G, N, E = batch.num_graphs, batch.num_nodes, batch.num_edges
    F, d, L, hid, K = batch.num_tags, batch.d, batch.levels, batch.hidden, batch.num_class
    w = batch.weights
    X = batch.dense_x()
    out = {
        "n2n_row_ptr": np.zeros(N + 1, np.int32), "n2n_col_idx": np.zeros(max(E, 1), np.int32),
        "n2n_val": np.zeros(max(E, 1), np.float32), "sub_row_ptr": np.zeros(G + 1, np.int32),
        "sub_col_idx": np.zeros(max(N, 1), np.int32), "sub_val": np.zeros(max(N, 1), np.float32),
        "msg": np.zeros((N, d), np.float32),
        "levels": np.zeros((L + 1, N, d), np.float32) if want_levels else None,
        "pooled": np.zeros((G, d), np.float32), "logits": np.zeros((G, K), np.float32),
        "probs": np.zeros((G, K), np.float32), "argmax": np.zeros(G, np.int32),
    }
    npg = np.ascontiguousarray(batch.nodes_per_graph, np.int32)
    es = np.ascontiguousarray(batch.edge_src, np.int32)
    ed = np.ascontiguousarray(batch.edge_dst, np.int32)
    args = [C.c_int(G), _p(npg, _i32p), C.c_int(E), _p(es, _i32p), _p(ed, _i32p), C.c_int(F), _p(X, _f32p),
            C.c_int(d), C.c_int(L), C.c_int(hid), C.c_int(K),
            _p(np.ascontiguousarray(w["w_n2l"]), _f32p), _p(np.ascontiguousarray(w["p_node_conv"]), _f32p),
            _p(np.ascontiguousarray(w["h1_weight"]), _f32p), _p(np.ascontiguousarray(w["h2_weight"]), _f32p),
            _p(out["n2n_row_ptr"], _i32p), _p(out["n2n_col_idx"], _i32p), _p(out["n2n_val"], _f32p),
            _p(out["sub_row_ptr"], _i32p), _p(out["sub_col_idx"], _i32p), _p(out["sub_val"], _f32p),
            _p(out["msg"], _f32p), _p(out["levels"], _f32p), _p(out["pooled"], _f32p), _p(out["logits"], _f32p),
            _p(out["probs"], _f32p), _p(out["argmax"], _i32p)]
    if impl == "oracle":
        import time
        secs = []
        for _ in range(max(iters, 1)):
            t0 = time.perf_counter()
            rc = lib.oracle_s2v_forward(*args)
            secs.append(time.perf_counter() - t0)
        out["seconds"] = np.asarray(secs)
    else:
        secs = np.zeros(max(iters, 1), np.float64)
        rc = lib.ref_s2v_forward(*args, C.c_int(iters), _p(secs, _f64p))
        out["seconds"] = secs
    if rc != 0:
        raise RuntimeError(f"{impl} forward failed with status {rc}")
    out["n2n_col_idx"] = out["n2n_col_idx"][:E]
    out["n2n_val"] = out["n2n_val"][:E]
    out["sub_col_idx"] = out["sub_col_idx"][:N]
    out["sub_val"] = out["sub_val"][:N]
    return out


def msgpass_matrix(batch, which: str, impl: str = "oracle", average: bool = False):
    """One of the message-passing matrices of a batch: which in {"n2n", "e2n", "n2e", "e2e", "sub"}.  With
    impl="reference" it is what the reference's own factor builds; with "oracle" the C restatement
    (edge-level matrices only).  Returns (row_ptr, col_idx, val)."""
    lib = _lib(impl)
    code = {"n2n": 0, "e2n": 1, "n2e": 2, "e2e": 3, "sub": 4}[which]
    G, N, E = batch.num_graphs, batch.num_nodes, batch.num_edges
    rows = {"n2n": N, "e2n": N, "n2e": E, "e2e": E, "sub": G}[which]
    npg = np.ascontiguousarray(batch.nodes_per_graph, np.int32)
    es = np.ascontiguousarray(batch.edge_src, np.int32)
    ed = np.ascontiguousarray(batch.edge_dst, np.int32)
    rp = np.zeros(rows + 1, np.int32)
    cap = 1
    for _ in range(2):      # first call sizes the arrays
        ci, val = np.zeros(cap, np.int32), np.zeros(cap, np.float32)
        if impl == "oracle":
            assert which in ("e2n", "n2e", "e2e")
            lib.oracle_build_edge_csr.restype = C.c_int64
            nnz = lib.oracle_build_edge_csr(C.c_int(code), C.c_int64(N), C.c_int64(E), _p(es, _i32p), _p(ed, _i32p), C.c_int(int(average)),
                                            _p(rp, _i32p), _p(ci, _i32p), _p(val, _f32p), C.c_int64(cap))
        else:
            nnz = lib.ref_msgpass_matrix(C.c_int(code), C.c_int(int(average)), C.c_int(G), _p(npg, _i32p), C.c_int(E), _p(es, _i32p),
                                         _p(ed, _i32p), _p(rp, _i32p), _p(ci, _i32p), _p(val, _f32p), C.c_int(cap))
        if nnz < 0:
            raise RuntimeError(f"{impl} msgpass_matrix failed with status {nnz}")
        if nnz <= cap:
            break
        cap = int(nnz)
    return rp, ci[:nnz], val[:nnz]


def level(prob, impl: str = "oracle", iters: int = 1, rows: int | None = None):
    """One level; `rows` limits the computation to the first `rows` output rows (a bounded sample).
    impl: "oracle", "reference", or "oracle_f64" (oracle_level_f64: all sums in double)."""
    lib = _lib("oracle" if impl == "oracle_f64" else impl)
    n_rows = prob.n_rows if rows is None else min(int(rows), prob.n_rows)
    d = prob.d
    rp = np.ascontiguousarray(prob.row_ptr[: n_rows + 1], np.int32)
    nnz = int(rp[-1])
    ci = np.ascontiguousarray(prob.col_idx[:nnz], np.int32)
    H = np.ascontiguousarray(prob.H, np.float32)
    W = np.ascontiguousarray(prob.W, np.float32)
    X = None if prob.X is None else np.ascontiguousarray(prob.X[:n_rows], np.float32)
    out = np.zeros((n_rows, d), np.float32)
    if impl == "oracle_f64":   # every sum in double: the yardstick for very long rows
        lib = _lib("oracle")
        lib.oracle_level_f64.restype = None
        lib.oracle_level_f64(C.c_int64(n_rows), C.c_int64(d), _p(rp, _i32p), _p(ci, _i32p), None, _p(H, _f32p),
                             _p(W, _f32p), _p(X, _f32p), _p(out, _f32p))
        return out, np.zeros(1)
    if impl == "oracle":
        import time
        scratch = np.zeros((2, n_rows, d), np.float32)
        lib.oracle_level.restype = None
        secs = []
        for _ in range(max(iters, 1)):
            t0 = time.perf_counter()
            lib.oracle_level(C.c_int64(n_rows), C.c_int64(d), _p(rp, _i32p), _p(ci, _i32p), None, _p(H, _f32p),
                             _p(W, _f32p), _p(X, _f32p), _p(out, _f32p), _p(scratch, _f32p))
            secs.append(time.perf_counter() - t0)
        return out, np.asarray(secs)
    secs = np.zeros(max(iters, 1), np.float64)
    rc = lib.ref_level_forward(C.c_int(n_rows), C.c_int(prob.n_src), C.c_int(nnz), _p(rp, _i32p), _p(ci, _i32p),
                               None, C.c_int(d), _p(H, _f32p), _p(W, _f32p), _p(X, _f32p), _p(out, _f32p),
                               C.c_int(iters), _p(secs, _f64p))
    if rc != 0:
        raise RuntimeError(f"reference level failed with status {rc}")
    return out, secs


def loss_acc(logits: np.ndarray, labels: np.ndarray, impl: str = "oracle", topk: int = 1):
    """Mean cross entropy (with softmax) and top-k accuracy of logits [G x C] against integer labels [G],
    presented as the one-entry-per-row CSR the reference's batcher builds.  Returns (loss, acc, per_graph)."""
    lib = _lib(impl)
    G, K = logits.shape
    lg = np.ascontiguousarray(logits, np.float32)
    rp = np.arange(G + 1, dtype=np.int32)
    ci = np.ascontiguousarray(labels, np.int32)
    val = np.ones(G, np.float32)
    loss, acc = C.c_float(), C.c_float()
    per = np.zeros(G, np.float32)
    if impl == "oracle":
        lib.oracle_loss_acc.restype = None
        lib.oracle_loss_acc(C.c_int64(G), C.c_int64(K), _p(lg, _f32p), _p(rp, _i32p), _p(ci, _i32p), _p(val, _f32p),
                            C.c_int(topk), C.byref(loss), C.byref(acc), _p(per, _f32p))
    else:
        assert topk == 1
        rc = lib.ref_loss_acc(C.c_int(G), C.c_int(K), _p(lg, _f32p), _p(rp, _i32p), _p(ci, _i32p), _p(val, _f32p),
                              C.byref(loss), C.byref(acc), _p(per, _f32p))
        if rc != 0:
            raise RuntimeError(f"reference loss/acc failed with status {rc}")
    return float(loss.value), float(acc.value), per
