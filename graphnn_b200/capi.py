"""ctypes binding of libs2v_b200.so (the C ABI declared in include/s2v_b200.h).

torch is used only to own device memory and streams; every computation goes through
the shared library.  There is no fallback: if the library is missing, or no B200 is
present, the calls raise.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libs2v_b200.so")

_i32p = C.POINTER(C.c_int32)
_i64p = C.POINTER(C.c_int64)
_f32p = C.POINTER(C.c_float)


class S2VError(RuntimeError):
    def __init__(self, status: int, text: str):
        super().__init__(f"s2v_b200 status {status}: {text}")
        self.status = status


class Model(C.Structure):
    _fields_ = [("num_feat", C.c_int), ("d", C.c_int), ("levels", C.c_int), ("hidden", C.c_int),
                ("num_class", C.c_int), ("w_n2l", C.c_void_p), ("p_node_conv", C.c_void_p),
                ("h1_weight", C.c_void_p), ("h2_weight", C.c_void_p), ("pool_average", C.c_int)]


class Batch(C.Structure):
    _fields_ = [("num_graphs", C.c_int64), ("num_nodes", C.c_int64), ("num_edges", C.c_int64),
                ("n2n_row_ptr", C.c_void_p), ("n2n_col_idx", C.c_void_p), ("n2n_val", C.c_void_p),
                ("graph_ptr", C.c_void_p), ("tags", C.c_void_p), ("x_dense", C.c_void_p),
                ("max_graph_nodes", C.c_int32)]


_lib = None


def load_library():
    """Loads the shared library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise FileNotFoundError(f"{LIB_PATH} not found: build it with `python -m graphnn_b200.build`")
    lib = C.CDLL(LIB_PATH)
    vp, i64, i32, f32 = C.c_void_p, C.c_int64, C.c_int, C.c_float
    sig = {
        "s2v_ctx_create": (i32, [i32, C.POINTER(vp)]),
        "s2v_ctx_destroy": (i32, [vp]),
        "s2v_ctx_device": (i32, [vp]),
        "s2v_ctx_stream": (vp, [vp]),
        "s2v_ctx_synchronize": (i32, [vp]),
        "s2v_stream_status": (i32, [vp, vp]),
        "s2v_ctx_set_option": (i32, [vp, i32, i32]),
        "s2v_status_str": (C.c_char_p, [i32]),
        "s2v_last_error": (C.c_char_p, [vp]),
        "s2v_launch_count": (C.c_uint64, [vp]),
        "s2v_selftest_wait_timeout": (i32, [vp, vp]),
        "s2v_level_f32": (i32, [vp, vp, i64, i64, i32, vp, vp, vp, vp, vp, vp, vp]),
        "s2v_level_rp64_f32": (i32, [vp, vp, i64, i64, i32, vp, vp, vp, vp, vp, vp, vp]),
        "s2v_level_lookup_f32": (i32, [vp, vp, i64, i64, i32, vp, vp, vp, vp, vp, vp, i32, vp, vp]),
        "s2v_level_first_f32": (i32, [vp, vp, i64, i32, vp, vp, vp, vp, vp, i32, vp, vp]),
        "s2v_spmm_csr_f32": (i32, [vp, vp, i64, i64, i32, vp, vp, vp, vp, f32, f32, vp]),
        "s2v_gemm_f32": (i32, [vp, vp, i32, i32, i64, i64, i64, f32, vp, i64, vp, i64, f32, vp, i64]),
        "s2v_axpy_f32": (i32, [vp, vp, i64, f32, vp, vp]),
        "s2v_scale_f32": (i32, [vp, vp, i64, f32, vp]),
        "s2v_relu_f32": (i32, [vp, vp, i64, vp, vp]),
        "s2v_softmax_f32": (i32, [vp, vp, i64, i32, vp, vp]),
        "s2v_argmax_f32": (i32, [vp, vp, i64, i32, vp, vp]),
        "s2v_cross_entropy_f32": (i32, [vp, vp, i64, i32, vp, i32, vp, vp, vp, vp]),
        "s2v_argmax_csr_f32": (i32, [vp, vp, i64, vp, vp, vp, vp]),
        "s2v_in_top_k_f32": (i32, [vp, vp, i64, i32, vp, vp, i32, vp]),
        "s2v_cast_i32_f32": (i32, [vp, vp, i64, vp, vp]),
        "s2v_mean_f32": (i32, [vp, vp, i64, vp, vp]),
        "s2v_loss_acc_f32": (i32, [vp, vp, i64, i32, vp, vp, vp, vp, i32, vp, vp, vp]),
        "s2v_segment_sum_f32": (i32, [vp, vp, i64, i32, vp, vp, vp]),
        "s2v_segment_pool_f32": (i32, [vp, vp, i64, i32, vp, vp, i32, vp]),
        "s2v_readout_f32": (i32, [vp, vp, i64, i32, i32, i32, vp, vp, vp, vp, vp, vp]),
        "s2v_input_proj_onehot_f32": (i32, [vp, vp, i64, i32, i32, vp, vp, vp, vp]),
        "s2v_input_proj_dense_f32": (i32, [vp, vp, i64, i32, i32, vp, vp, vp, vp]),
        "s2v_graph_tiles_workspace_bytes": (C.c_size_t, [i64]),
        "s2v_graph_tiles_f32": (i32, [vp, vp, i64, i32, i32, vp, vp, vp, vp, vp, i32, vp, vp, i32, vp, C.c_size_t, vp, vp]),
        "s2v_forward_workspace_bytes": (C.c_size_t, [i64, i64, i32]),
        "s2v_forward_f32": (i32, [vp, vp, C.POINTER(Model), C.POINTER(Batch), vp, C.c_size_t, vp, vp, vp, vp]),
        "s2v_forward_static_f32": (i32, [vp, vp, C.POINTER(Model), C.POINTER(Batch), vp, vp, vp, vp]),
        "s2v_build_n2n_csr_host": (i32, [i64, i64, vp, vp, i32, vp, vp, vp]),
        "s2v_validate_csr_host": (i32, [i64, i64, i64, vp, vp]),
        "s2v_build_e2n_csr_host": (i32, [i64, i64, vp, vp, i32, vp, vp, vp]),
        "s2v_build_n2e_csr_host": (i32, [i64, i64, vp, vp, vp, vp]),
        "s2v_build_e2e_csr_host": (i32, [i64, i64, vp, vp, vp, vp, vp, i64, C.POINTER(C.c_int64)]),
        "s2v_infer_host_f32": (i32, [vp, C.POINTER(Model), C.POINTER(Batch), vp, vp]),
        "s2v_comm_create": (i32, [i32, vp, vp]),
        "s2v_comm_unique_id": (i32, [vp]),
        "s2v_comm_create_rank": (i32, [i32, vp, i32, i32, C.POINTER(vp)]),
        "s2v_comm_destroy": (i32, [vp]),
        "s2v_comm_rank": (i32, [vp]),
        "s2v_comm_world": (i32, [vp]),
        "s2v_comm_last_error": (C.c_char_p, [vp]),
        "s2v_allgather_rows_f32": (i32, [vp, vp, i64, i32, vp, vp]),
        "s2v_gather_logits": (i32, [vp, vp, vp, i32, vp, vp, vp, vp]),
        "s2v_exchange_rows_f32": (i32, [vp, vp, i32, vp, vp, vp, vp, vp]),
        "s2v_infer_edges_host_f32": (i32, [vp, C.POINTER(Model), i64, i64, i64, vp, vp, vp, vp, vp, vp]),
        "s2v_infer_edges_host_submit": (i32, [vp, i32, C.POINTER(Model), i64, i64, i64, vp, vp, vp, vp, vp, vp]),
        "s2v_infer_host_wait": (i32, [vp, i32]),
        "s2v_build_n2n_csr_scratch_bytes": (C.c_size_t, [i64, i64]),
        "s2v_build_n2n_csr_f32": (i32, [vp, vp, i64, i64, vp, vp, i32, vp, C.c_size_t, vp, vp, vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    lib._s2v_signatures = sig
    _lib = lib
    return lib


def exported_symbols() -> list[str]:
    return sorted(load_library()._s2v_signatures)


def _ptr(t):
    """Device (torch) or host (numpy) address of an array, None -> NULL."""
    if t is None:
        return None
    if isinstance(t, np.ndarray):
        return t.ctypes.data
    return t.data_ptr()


def build_n2n_csr_host(num_nodes: int, edge_src: np.ndarray, edge_dst: np.ndarray, average: bool = False,
                       with_val: bool = True):
    """Host CSR of the node-to-node matrix, bit-identical to the reference's builder."""
    lib = load_library()
    E = int(edge_src.shape[0])
    es = np.ascontiguousarray(edge_src, np.int32)
    ed = np.ascontiguousarray(edge_dst, np.int32)
    row_ptr = np.empty(num_nodes + 1, np.int32)
    col_idx = np.empty(max(E, 1), np.int32)
    val = np.empty(max(E, 1), np.float32) if with_val else None
    rc = lib.s2v_build_n2n_csr_host(num_nodes, E, _ptr(es), _ptr(ed), int(average), _ptr(row_ptr), _ptr(col_idx),
                                    _ptr(val))
    if rc != 0:
        raise S2VError(rc, lib.s2v_status_str(rc).decode())
    return row_ptr, col_idx[:E], (val[:E] if with_val else None)


def build_edge_csrs_host(num_nodes: int, edge_src: np.ndarray, edge_dst: np.ndarray, average: bool = False) -> dict:
    """The edge-level message-passing matrices of the reference (edge-to-node, node-to-edge, edge-to-edge) as
    {"e2n": (row_ptr, col_idx, val), "n2e": ..., "e2e": ...}, built by the library's host builders."""
    lib = load_library()
    E = int(edge_src.shape[0])
    es = np.ascontiguousarray(edge_src, np.int32)
    ed = np.ascontiguousarray(edge_dst, np.int32)

    def check(rc):
        if rc != 0:
            raise S2VError(rc, lib.s2v_status_str(rc).decode())
    out = {}
    rp, ci, val = np.empty(num_nodes + 1, np.int32), np.empty(max(E, 1), np.int32), np.empty(max(E, 1), np.float32)
    check(lib.s2v_build_e2n_csr_host(num_nodes, E, _ptr(es), _ptr(ed), int(average), _ptr(rp), _ptr(ci), _ptr(val)))
    out["e2n"] = (rp, ci[:E], val[:E])
    rp, ci, val = np.empty(E + 1, np.int32), np.empty(max(E, 1), np.int32), np.empty(max(E, 1), np.float32)
    check(lib.s2v_build_n2e_csr_host(num_nodes, E, _ptr(es), _ptr(rp), _ptr(ci), _ptr(val)))
    out["n2e"] = (rp, ci[:E], val[:E])
    nnz = C.c_int64(0)
    rp = np.empty(E + 1, np.int32)
    check(lib.s2v_build_e2e_csr_host(num_nodes, E, _ptr(es), _ptr(ed), _ptr(rp), None, None, 0, C.byref(nnz)))
    ci, val = np.empty(max(nnz.value, 1), np.int32), np.empty(max(nnz.value, 1), np.float32)
    check(lib.s2v_build_e2e_csr_host(num_nodes, E, _ptr(es), _ptr(ed), _ptr(rp), _ptr(ci), _ptr(val), nnz.value, C.byref(nnz)))
    out["e2e"] = (rp, ci[:nnz.value], val[:nnz.value])
    return out


def validate_csr_host(m: int, k: int, row_ptr: np.ndarray, col_idx: np.ndarray) -> int:
    lib = load_library()
    rp = np.ascontiguousarray(row_ptr, np.int32)
    ci = np.ascontiguousarray(col_idx, np.int32)
    return lib.s2v_validate_csr_host(m, k, int(ci.shape[0]), _ptr(rp), _ptr(ci))


COMM_ID_BYTES = 128


def comm_unique_id() -> bytes:
    """s2v_comm_unique_id: the 128-byte id rank 0 hands to the other ranks."""
    lib = load_library()
    buf = C.create_string_buffer(COMM_ID_BYTES)
    rc = lib.s2v_comm_unique_id(buf)
    if rc != 0:
        raise S2VError(rc, f"{lib.s2v_status_str(rc).decode()}: {lib.s2v_comm_last_error(None).decode()}")
    return buf.raw


class Comm:
    """One s2v_comm: this rank's NCCL communicator, created from the id rank 0 distributed."""

    def __init__(self, device: int, unique_id: bytes, world: int, rank: int):
        self.lib = load_library()
        h = C.c_void_p()
        rc = self.lib.s2v_comm_create_rank(int(device), unique_id, int(world), int(rank), C.byref(h))
        if rc != 0:
            raise S2VError(rc, f"{self.lib.s2v_status_str(rc).decode()}: {self.lib.s2v_comm_last_error(None).decode()}")
        self.h, self.world, self.rank = h, world, rank

    def check(self, rc: int):
        if rc != 0:
            raise S2VError(rc, f"{self.lib.s2v_status_str(rc).decode()}: {self.lib.s2v_comm_last_error(self.h).decode()}")

    def allgather_rows(self, slab, full, stream):
        """full[r] = slab of rank r (equal [rows x d] slabs); asynchronous on `stream`."""
        rows, d = slab.shape
        self.check(self.lib.s2v_allgather_rows_f32(self.h, stream, rows, d, _ptr(slab), _ptr(full)))

    def exchange_rows(self, send, send_offsets, recv, recv_offsets, recv_rows, stream):
        """Pairwise exchange of rows: rows [send_offsets[p], send_offsets[p+1]) of `send` go to rank p, recv_rows[p]
        rows from rank p land at row recv_offsets[p] of `recv` (host arrays of counts); asynchronous on `stream`."""
        so = np.ascontiguousarray(send_offsets, np.int64)
        ro = np.ascontiguousarray(recv_offsets, np.int64)
        rr = np.ascontiguousarray(recv_rows, np.int64)
        assert so.shape[0] == self.world + 1 and ro.shape[0] == self.world and rr.shape[0] == self.world
        d = int(recv.shape[1] if recv is not None else send.shape[1])
        self.check(self.lib.s2v_exchange_rows_f32(self.h, stream, d, _ptr(send), so.ctypes.data, _ptr(recv), ro.ctypes.data,
                                                  rr.ctypes.data))

    def gather_logits(self, graphs_per_rank, logits_local, pred_local, logits_all, pred_all, stream):
        counts = np.ascontiguousarray(graphs_per_rank, np.int64)
        num_class = logits_all.shape[1] if logits_all is not None else 1
        self.check(self.lib.s2v_gather_logits(self.h, stream, counts.ctypes.data, num_class, _ptr(logits_local),
                                              _ptr(pred_local), _ptr(logits_all), _ptr(pred_all)))

    def close(self):
        if getattr(self, "h", None):
            self.lib.s2v_comm_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Context:
    """One s2v_ctx: a device, its stream and the library's launch counter."""

    def __init__(self, device: int = 0):
        self.lib = load_library()
        h = C.c_void_p()
        rc = self.lib.s2v_ctx_create(int(device), C.byref(h))
        if rc != 0:
            raise S2VError(rc, self.lib.s2v_status_str(rc).decode())
        self.h = h
        self.device = device

    def close(self):
        if getattr(self, "h", None):
            self.lib.s2v_ctx_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- helpers
    def check(self, rc: int):
        if rc != 0:
            raise S2VError(rc, f"{self.lib.s2v_status_str(rc).decode()}: {self.lib.s2v_last_error(self.h).decode()}")

    def call(self, name: str, *args):
        rc = getattr(self.lib, name)(self.h, *args)
        self.check(rc)

    @property
    def stream(self) -> int:
        return self.lib.s2v_ctx_stream(self.h)

    def synchronize(self):
        self.check(self.lib.s2v_ctx_synchronize(self.h))

    def stream_status(self, stream=None):
        """Synchronises `stream` (None = the context's own) and raises if a kernel recorded a status."""
        self.check(self.lib.s2v_stream_status(self.h, stream))

    OPT_VALIDATE_HOST_INPUT, OPT_LEVEL_TC, OPT_GRAPH_TILES, OPT_RESERVED_SMS, OPT_FIRST_LEVEL_TABLE = 1, 2, 3, 4, 5

    def set_option(self, option: int, value: int):
        self.check(self.lib.s2v_ctx_set_option(self.h, int(option), int(value)))

    @property
    def launches(self) -> int:
        return int(self.lib.s2v_launch_count(self.h))

    def selftest_wait_timeout(self, stream=None):
        """s2v_selftest_wait_timeout: a kernel whose bounded wait runs out on purpose; the next
        synchronize() raises S2VError with the device time-out status."""
        self.call("s2v_selftest_wait_timeout", stream)

    # -- operators (device tensors in, device tensors out; `stream` = raw cudaStream_t or None)
    def level(self, row_ptr, col_idx, val, H, W, X, out, n_src=None, stream=None):
        n_rows, d = out.shape
        n_src = H.shape[0] if n_src is None else n_src
        name = "s2v_level_rp64_f32" if row_ptr.element_size() == 8 else "s2v_level_f32"
        self.call(name, stream, n_rows, n_src, d, _ptr(row_ptr), _ptr(col_idx), _ptr(val), _ptr(H), _ptr(W), _ptr(X),
                  _ptr(out))
        return out

    def level_lookup(self, row_ptr, col_idx, val, H, W, table, x_index, out, stream=None):
        n_rows, d = out.shape
        self.call("s2v_level_lookup_f32", stream, n_rows, H.shape[0], d, _ptr(row_ptr), _ptr(col_idx), _ptr(val),
                  _ptr(H), _ptr(W), _ptr(table), table.shape[0], _ptr(x_index), _ptr(out))
        return out

    def level_first(self, row_ptr, col_idx, val, W, table, tags, out, stream=None):
        n, d = out.shape
        self.call("s2v_level_first_f32", stream, n, d, _ptr(row_ptr), _ptr(col_idx), _ptr(val), _ptr(W), _ptr(table),
                  table.shape[0], _ptr(tags), _ptr(out))
        return out

    def spmm(self, m, k, row_ptr, col_idx, val, B, C_out, alpha=1.0, beta=0.0, stream=None):
        self.call("s2v_spmm_csr_f32", stream, m, k, B.shape[1], _ptr(row_ptr), _ptr(col_idx), _ptr(val), _ptr(B),
                  alpha, beta, _ptr(C_out))
        return C_out

    def gemm(self, A, B, C_out, trans_a=False, trans_b=False, alpha=1.0, beta=0.0, stream=None):
        m = A.shape[1] if trans_a else A.shape[0]
        k = A.shape[0] if trans_a else A.shape[1]
        n = B.shape[0] if trans_b else B.shape[1]
        self.call("s2v_gemm_f32", stream, int(trans_a), int(trans_b), m, n, k, alpha, _ptr(A), A.shape[1], _ptr(B),
                  B.shape[1], beta, _ptr(C_out), C_out.shape[1])
        return C_out

    def axpy(self, a, x, y, stream=None):
        self.call("s2v_axpy_f32", stream, x.numel(), a, _ptr(x), _ptr(y))
        return y

    def scale(self, a, x, stream=None):
        self.call("s2v_scale_f32", stream, x.numel(), a, _ptr(x))
        return x

    def relu(self, x, out, stream=None):
        self.call("s2v_relu_f32", stream, x.numel(), _ptr(x), _ptr(out))
        return out

    def softmax(self, x, out, stream=None):
        self.call("s2v_softmax_f32", stream, x.shape[0], x.shape[1], _ptr(x), _ptr(out))
        return out

    def argmax(self, x, out, stream=None):
        self.call("s2v_argmax_f32", stream, x.shape[0], x.shape[1], _ptr(x), _ptr(out))
        return out

    def loss_acc(self, logits, label_rp, label_ci, label_val, loss, acc, per_graph=None, topk=1, stream=None):
        self.call("s2v_loss_acc_f32", stream, logits.shape[0], logits.shape[1], _ptr(logits), _ptr(label_rp), _ptr(label_ci),
                  _ptr(label_val), topk, _ptr(loss), _ptr(acc), _ptr(per_graph))

    def segment_sum(self, seg_ptr, H, Y, stream=None, average=False):
        self.call("s2v_segment_pool_f32", stream, Y.shape[0], H.shape[1], _ptr(seg_ptr), _ptr(H), int(average), _ptr(Y))
        return Y

    def graph_tiles(self, levels, row_ptr, col_idx, val, graph_ptr, tags, W_in, W, workspace, Y, embed_out=None,
                    pool_average=False, stream=None):
        """s2v_graph_tiles_f32: projection + L levels + pooling of a batch of small graphs in one kernel."""
        self.call("s2v_graph_tiles_f32", stream, Y.shape[0], Y.shape[1], levels, _ptr(row_ptr), _ptr(col_idx), _ptr(val),
                  _ptr(graph_ptr), _ptr(tags), W_in.shape[0], _ptr(W_in), _ptr(W), int(pool_average), _ptr(workspace),
                  workspace.numel() * workspace.element_size(), _ptr(Y), _ptr(embed_out))
        return Y

    def graph_tiles_workspace_bytes(self, num_graphs: int) -> int:
        return int(self.lib.s2v_graph_tiles_workspace_bytes(num_graphs))

    def readout(self, Y, W1, W2, logits, probs=None, pred=None, stream=None):
        self.call("s2v_readout_f32", stream, Y.shape[0], Y.shape[1], W1.shape[1], W2.shape[1], _ptr(Y), _ptr(W1),
                  _ptr(W2), _ptr(logits), _ptr(probs), _ptr(pred))
        return logits

    def input_proj_onehot(self, tags, W_in, msg, h0, stream=None):
        self.call("s2v_input_proj_onehot_f32", stream, tags.shape[0], W_in.shape[0], W_in.shape[1], _ptr(tags),
                  _ptr(W_in), _ptr(msg), _ptr(h0))

    def input_proj_dense(self, X, W_in, msg, h0, stream=None):
        self.call("s2v_input_proj_dense_f32", stream, X.shape[0], X.shape[1], W_in.shape[1], _ptr(X), _ptr(W_in),
                  _ptr(msg), _ptr(h0))

    # -- whole model
    @staticmethod
    def make_model(levels: int, w_n2l, p_node_conv, h1_weight, h2_weight, pool_average: bool = False) -> Model:
        """`w_*` are DEVICE tensors (kept alive by the caller)."""
        return Model(w_n2l.shape[0], w_n2l.shape[1], levels, h1_weight.shape[1], h2_weight.shape[1],
                     _ptr(w_n2l), _ptr(p_node_conv), _ptr(h1_weight), _ptr(h2_weight), int(pool_average))

    @staticmethod
    def make_batch(num_graphs, num_nodes, row_ptr, col_idx, val, graph_ptr, tags=None, x_dense=None,
                   max_graph_nodes: int = 0) -> Batch:
        """Arrays are torch device tensors (device entry) or numpy arrays (host entry).  `max_graph_nodes`:
        node count of the largest graph (0 = unknown: the per-level kernels are used)."""
        return Batch(num_graphs, num_nodes, int(col_idx.shape[0]), _ptr(row_ptr), _ptr(col_idx), _ptr(val),
                     _ptr(graph_ptr), _ptr(tags), _ptr(x_dense), int(max_graph_nodes))

    def workspace_bytes(self, num_nodes, num_graphs, d) -> int:
        return int(self.lib.s2v_forward_workspace_bytes(num_nodes, num_graphs, d))

    def forward(self, model: Model, batch: Batch, workspace, logits, probs=None, pred=None, embed_out=None,
                stream=None):
        self.call("s2v_forward_f32", stream, C.byref(model), C.byref(batch), _ptr(workspace),
                  workspace.numel() * workspace.element_size(), _ptr(logits), _ptr(probs), _ptr(pred),
                  _ptr(embed_out))

    def forward_static(self, model: Model, batch: Batch, logits, probs=None, pred=None, embed_out=None, stream=None):
        """s2v_forward_static_f32: like forward() but with the library's built-in scratch array."""
        self.call("s2v_forward_static_f32", stream, C.byref(model), C.byref(batch), _ptr(logits), _ptr(probs),
                  _ptr(pred), _ptr(embed_out))

    def build_n2n_csr(self, num_nodes: int, edge_src, edge_dst, scratch, row_ptr, col_idx, val=None, average=False,
                      stream=None):
        """s2v_build_n2n_csr_f32: device edge list -> device CSR (all torch int32 device tensors)."""
        self.call("s2v_build_n2n_csr_f32", stream, num_nodes, int(edge_src.shape[0]), _ptr(edge_src), _ptr(edge_dst),
                  int(average), _ptr(scratch), scratch.numel() * scratch.element_size(), _ptr(row_ptr), _ptr(col_idx),
                  _ptr(val))

    def csr_scratch_bytes(self, num_nodes: int, num_edges: int) -> int:
        return int(self.lib.s2v_build_n2n_csr_scratch_bytes(num_nodes, num_edges))

    def infer_edges_host(self, model: Model, num_graphs, num_nodes, edge_src, edge_dst, graph_ptr, tags,
                         logits_host, pred_host):
        """s2v_infer_edges_host_f32: host edge list in, host logits / predictions out."""
        rc = self.lib.s2v_infer_edges_host_f32(self.h, C.byref(model), num_graphs, num_nodes, int(edge_src.shape[0]),
                                               _ptr(edge_src), _ptr(edge_dst), _ptr(graph_ptr), _ptr(tags),
                                               _ptr(logits_host), _ptr(pred_host))
        self.check(rc)

    def infer_edges_host_submit(self, lane: int, model: Model, num_graphs, num_nodes, edge_src, edge_dst, graph_ptr, tags,
                                logits_host, pred_host):
        """s2v_infer_edges_host_submit: the same batch put on lane 0 or 1 without waiting for it; the arrays must
        stay alive and untouched until infer_host_wait(lane) returns."""
        self.check(self.lib.s2v_infer_edges_host_submit(self.h, int(lane), C.byref(model), num_graphs, num_nodes,
                                                        int(edge_src.shape[0]), _ptr(edge_src), _ptr(edge_dst), _ptr(graph_ptr),
                                                        _ptr(tags), _ptr(logits_host), _ptr(pred_host)))

    def infer_host_wait(self, lane: int):
        self.check(self.lib.s2v_infer_host_wait(self.h, int(lane)))

    def infer_host(self, model: Model, batch_host: Batch, logits_host: np.ndarray | None,
                   pred_host: np.ndarray | None):
        rc = self.lib.s2v_infer_host_f32(self.h, C.byref(model), C.byref(batch_host), _ptr(logits_host),
                                         _ptr(pred_host))
        self.check(rc)
