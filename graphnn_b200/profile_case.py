"""Small, self-contained launches of the fused level kernel for profiler captures.

    python -m graphnn_b200.profile_case --case er_d64  [--launches 3]
    python -m graphnn_b200.profile_case --case mol_d128 [--launches 3]

er_d64  : Erdos-Renyi n=524,288, nnz=4,194,304, d=64 with a dense X (half the 1M-node
          benchmark problem: H, X and out are 134 MB each, above the 126 MB L2).
mol_d128: 16,384 molecule-like graphs, d=128, X looked up from W_in by tag
          (the level the classifier benchmark runs; three 252 MB matrices).
Prints the mean CUDA-event time per launch.
"""
from __future__ import annotations

import argparse

import numpy as np
import torch

from . import capi, synth


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="er_d64", choices=["er_d64", "er_d64_full", "mol_d128", "prot_d64"])
    ap.add_argument("--launches", type=int, default=3)
    args = ap.parse_args()
    ctx = capi.Context(0)
    dev = torch.device("cuda", 0)
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    st = stream.cuda_stream

    def up(a):
        return torch.from_numpy(np.ascontiguousarray(a)).to(dev)

    if args.case.startswith("er_d64"):
        full = args.case.endswith("full")
        p = synth.erdos_renyi_level(n=1 << (20 if full else 19), nnz=1 << (23 if full else 22), d=64)
        rp, ci, H, W, X = up(p.row_ptr), up(p.col_idx), up(p.H), up(p.W), up(p.X)
        out = torch.empty_like(X)
        launch = lambda: ctx.level(rp, ci, None, H, W, X, out, stream=st)
        desc = f"{p.name}: n={p.n_rows} nnz={p.nnz}"
    else:
        b = synth.molecules_16k(seed=0) if args.case == "mol_d128" else synth.proteins_4k(seed=0, num_graphs=2048)
        rp_h, ci_h, _ = capi.build_n2n_csr_host(b.num_nodes, b.edge_src, b.edge_dst, with_val=False)
        rp, ci, tags = up(rp_h), up(ci_h), up(b.tags.astype(np.int32))
        W, table = up(b.weights["p_node_conv"]), up(b.weights["w_n2l"])
        H = torch.randn((b.num_nodes, b.d), device=dev).abs_()
        out = torch.empty_like(H)
        launch = lambda: ctx.level_lookup(rp, ci, None, H, W, table, tags, out, stream=st)
        desc = f"{b.name}: N={b.num_nodes} nnz={b.num_edges} d={b.d}"
    launch()
    torch.cuda.synchronize()
    evs = []
    for _ in range(args.launches):
        a, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        launch()
        e.record(stream)
        evs.append((a, e))
    torch.cuda.synchronize()
    ctx.synchronize()
    print(desc, "mean ms/launch:", float(np.mean([a.elapsed_time(e) for a, e in evs])))


if __name__ == "__main__":
    main()
