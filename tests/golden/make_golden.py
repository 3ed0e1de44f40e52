"""Generates the committed golden vectors from the reference's own CPU code.

Needs ``oracle/_ref/libs2v_ref.so`` (``python oracle/build.py`` next to a checkout of
the reference).  Inputs come from the seeded generators in ``graphnn_b200.synth``; the
outputs below are what the reference's classes computed for them (MKL replaced by the
plain-loop stand-ins in ``oracle/shim``).

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from graphnn_b200 import synth  # noqa: E402
from oracle import bindings as ob  # noqa: E402


def main():
    assert ob.have_reference(), "build oracle/_ref first"
    # 1. the CPU-runnable classifier config: 64 MUTAG-like graphs
    b = synth.mutag_like(seed=0)
    r = ob.forward(b, "reference")
    np.savez_compressed(
        os.path.join(HERE, "mutag_like_seed0.npz"), digest=b.digest(),
        n2n_row_ptr=r["n2n_row_ptr"], n2n_col_idx=r["n2n_col_idx"], n2n_val=r["n2n_val"],
        sub_row_ptr=r["sub_row_ptr"], sub_col_idx=r["sub_col_idx"], sub_val=r["sub_val"],
        last_level=r["levels"][-1], pooled=r["pooled"], logits=r["logits"], probs=r["probs"], argmax=r["argmax"])
    # 2. same graphs, weights drawn so that both classes occur
    b2 = synth.mutag_like(seed=3)
    r2 = ob.forward(b2, "reference")
    np.savez_compressed(os.path.join(HERE, "mutag_like_seed3.npz"), digest=b2.digest(),
                        n2n_row_ptr=r2["n2n_row_ptr"], n2n_col_idx=r2["n2n_col_idx"], pooled=r2["pooled"],
                        logits=r2["logits"], probs=r2["probs"], argmax=r2["argmax"])
    # 2b. loss / accuracy tail of the driver's TEST loop on those logits, labels drawn from seed 7
    labels = np.random.default_rng(7).integers(0, 2, size=b2.num_graphs).astype(np.int32)
    loss, acc, per_graph = ob.loss_acc(r2["logits"], labels, "reference")
    np.savez_compressed(os.path.join(HERE, "loss_acc_seed3.npz"), labels=labels, loss=np.float32(loss), acc=np.float32(acc),
                        per_graph=per_graph)
    # 3. one fused level on a small directed Erdos-Renyi graph (duplicates, empty rows, unsorted rows)
    p = synth.erdos_renyi_level(n=1000, nnz=6000, d=64, seed=1)
    out, _ = ob.level(p, "reference")
    np.savez_compressed(os.path.join(HERE, "er_level_n1000_d64_seed1.npz"), row_ptr=p.row_ptr, col_idx=p.col_idx,
                        out=out)
    # 4. a checkpoint written by the reference's own ParamSet::Save (byte-format fixture) and its weights
    import ctypes as C
    rng = np.random.default_rng(0)
    F, d, h, K = 3, 4, 5, 2
    w = {"w_n2l": rng.standard_normal((F, d)).astype(np.float32), "p_node_conv": rng.standard_normal((d, d)).astype(np.float32),
         "h1_weight": rng.standard_normal((d, h)).astype(np.float32), "h2_weight": rng.standard_normal((h, K)).astype(np.float32)}
    f32p = C.POINTER(C.c_float)
    ob._lib("reference").ref_save_model(os.path.join(HERE, "tiny_reference_saved.model").encode(), F, d, h, K,
                                        *[w[k].ctypes.data_as(f32p) for k in ("w_n2l", "p_node_conv", "h1_weight", "h2_weight")])
    np.savez(os.path.join(HERE, "tiny_reference_saved_weights.npz"), **w)
    # 5. the message-passing matrices of the reference's own factors (sum and average forms) for the seed-0 batch
    mats = {}
    for which in ("n2n", "e2n", "n2e", "e2e", "sub"):
        for avg in (False, True):
            rp, ci, val = ob.msgpass_matrix(b, which, "reference", avg)
            key = f"{which}_{'avg' if avg else 'sum'}"
            mats[key + "_row_ptr"], mats[key + "_col_idx"], mats[key + "_val"] = rp, ci, val
    np.savez_compressed(os.path.join(HERE, "msgpass_matrices_mutag_seed0.npz"), digest=b.digest(), **mats)
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")
    print("classes seed0:", np.bincount(r["argmax"]), "seed3:", np.bincount(r2["argmax"]))


if __name__ == "__main__":
    main()
