"""Benchmark of the s2v mean-field inference path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload molecules|proteins|giant] [--case NAME --launches n]

A step is one inference pass over one batch of synthetic graphs that is already resident in HBM:
for the molecule-like default (16,384 graphs IN TOTAL, latent 128, 4 levels) the tile kernel (input
projection, the four levels and the pooling in one launch), the readout, and -- on several GPUs -- the
gather of the logits.  With N ranks the 16,384 graphs are sharded by graph over the ranks (strong
scaling, the configuration as stated); the figure with 16,384 graphs PER rank is reported beside it
under `weak`.  Rank 0 prints ONE JSON line.

`value`      graphs/s over all ranks, inputs on the device, CUDA-event time, max over ranks.
`e2e`        the same metric through the host-buffer entry point the reference's FeedForward
             corresponds to: raw edge list + tags on the host -> upload -> CSR built on the device ->
             forward -> download (s2v_infer_edges_host_f32).  `e2e.from_host_csr` starts from a ready
             host CSR instead, `e2e.host_sorted` sorts the edge list on the host first.
`roofline`   the dominant kernel inside the timed region, timed with CUDA events on its stream.
`level_cfg2` the single fused level on the 1M-node / 8M-edge Erdos-Renyi problem (N = 1 only).
`parity`     the results of this very run checked against the reference's CPU code.
`cpu_baseline`  the reference's own CPU code on this machine's cores, whole batch.

`--impl reference` times the reference's CPU implementation (oracle/_ref, MKL replaced by plain OpenMP
loops) on the whole batch.  `--case` runs one small launch case for profiler captures and prints its time.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

REPO = os.path.dirname(os.path.abspath(__file__))
if REPO not in sys.path:
    sys.path.insert(0, REPO)

from graphnn_b200 import synth  # noqa: E402

WEIGHT_SEED = 20240
WORKLOAD_TEXT = {
    "molecules": "molecules_16k: 16,384 molecule-like graphs (20-40 nodes, tree + 10% edges, 82 Zipf(1.2) tags), "
                 "d=128, L=4, hidden=256, C=2, sum pooling",
    "proteins": "proteins_4k: 4,096 protein-like graphs (100-620 nodes, random geometric, mean degree ~7.4, 3 tags), "
                "d=64, L=5, hidden=128, C=2, sum pooling",
}
METRIC = "s2v_inference_graphs_per_sec"

# DRAM bytes of one launch measured with ncu (dram__bytes_read.sum + dram__bytes_write.sum); each entry names the
# committed summary it was read from.  A kernel without a capture reports traffic = null.
NCU_TRAFFIC = {
    "level_tc_mol_d128": (259830016 + 204611328, "profiles/level_tcgen05.md (mol_d128, 16,384 graphs)"),
    "first_level_mol_d128": (8289024 + 193662464, "profiles/level_first_table.md (mol_first, 16,384 graphs; part of the output is still in L2 when the kernel ends)"),
    "level_tc_er_d64_half": (806403584 + 119012864, "profiles/level_tcgen05.md (er_d64, n=524,288; scaled x2 for the full problem)"),
}


def make_workload(name: str, seed: int):
    if name == "molecules":
        return synth.molecules_16k(seed=seed, weight_seed=WEIGHT_SEED)
    if name == "proteins":
        return synth.proteins_4k(seed=seed, weight_seed=WEIGHT_SEED)
    raise SystemExit(f"unknown workload {name}")


def measured_peaks() -> dict:
    p = os.path.join(REPO, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            j = json.load(f)
        return {"hbm_gbs": float(j["hbm_gbs"]), "bf16_tflops": float(j["bf16_tflops"]), "kind": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "kind": "fallback"}


# ------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU while the timed region runs
    (NVML through pynvml every 20 ms; falls back to polling nvidia-smi)."""

    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, index: int):
        self.index = index
        self.sm = []
        self.sm_max = None
        self.reason_bits = 0
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _run_nvml(self) -> bool:
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            idx = self.index
            if visible:
                ids = [v for v in visible.split(",") if v.strip()]
                if idx < len(ids) and ids[idx].strip().isdigit():
                    idx = int(ids[idx])
            h = pynvml.nvmlDeviceGetHandleByIndex(idx)
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
        except Exception:
            return False
        while not self._stop.is_set():
            try:
                self.sm.append(float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)))
                self.reason_bits |= int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(h))
            except Exception:
                try:
                    self.reason_bits |= int(pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h))
                except Exception:
                    pass
            self._stop.wait(0.02)
        return True

    def _run_smi(self):
        fields = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
                  "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={fields}", "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=5).stdout
                parts = [x.strip() for x in out.strip().split(",")]
                if len(parts) >= 6:
                    self.sm.append(float(parts[0]))
                    self.sm_max = float(parts[1])
                    for i, n in enumerate(names):
                        if parts[2 + i].lower() == "active":
                            self.reason_bits |= self.REASONS[n]
            except Exception:
                pass
            self._stop.wait(0.05)

    def _run(self):
        if not self._run_nvml():
            self._run_smi()

    def __enter__(self):
        self._thread.start()
        time.sleep(0.05)     # let the first sample land before the timed region starts
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self) -> dict:
        if not self.sm:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": ["no samples"]}
        sm = sorted(self.sm)
        reasons = [n for n, bit in self.REASONS.items() if self.reason_bits & bit]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": self.sm_max, "reasons": reasons, "samples": len(sm)}


# ------------------------------------------------------------------ byte / flop models
def level_bytes(n_rows, nnz, d, model: str, x_form: str, h_form: str = "matrix") -> int:
    """Algorithmic bytes of one fused level launch.  `gather`: every neighbour row fetched once per edge;
    `compulsory`: every H row fetched once.  x_form: dense (X read as [N x d]), lookup (tags + table) or
    none.  h_form: matrix (H read from HBM) or table (the first level of the classifier: the gather
    source is ReLU(W_in[tag]), H0 is never in memory, only the tags are read)."""
    b_csr = 4 * (n_rows + 1) + 4 * nnz          # val == NULL form: no value array
    if h_form == "table":
        b_h = 0                                  # the tags are counted under x_form = lookup
    else:
        b_h = 4 * nnz * d if model == "gather" else 4 * n_rows * d
    b_x = {"dense": 4 * n_rows * d, "lookup": 4 * n_rows, "none": 0}[x_form]
    return b_csr + b_h + b_x + 4 * n_rows * d + 4 * d * d


def sampled_level_parity(row_ptr, col_idx, H, W, X, out_dev, n_sample=2048, seed=7):
    """Recomputes a sample of the output rows of one level on the host with the CPU oracle, from the CSR
    slices and H rows of exactly those rows: row 0, the last row, the rows of the last (ragged) 128-row
    tile, the longest rows, and seeded random rows.  Returns the parity block for the bench line."""
    import torch
    from oracle import bindings as ob
    n = len(row_ptr) - 1
    rng = np.random.default_rng(seed)
    deg = np.diff(row_ptr)
    pick = {0, n - 1}
    pick.update(range(max(0, (n - 1) // 128 * 128), n))
    pick.update(np.argsort(deg)[-32:].tolist())
    pick.update(rng.integers(0, n, n_sample).tolist())
    rows = np.array(sorted(pick), np.int64)
    rp = np.zeros(len(rows) + 1, np.int64)
    np.cumsum(deg[rows], out=rp[1:])
    ci = np.concatenate([col_idx[row_ptr[r]:row_ptr[r + 1]] for r in rows]) if len(rows) else np.zeros(0, np.int32)
    prob = synth.LevelProblem(len(rows), H.shape[0], rp.astype(np.int32), ci.astype(np.int32), H, W,
                              None if X is None else np.ascontiguousarray(X[rows]))
    want, _ = ob.level(prob, "oracle")
    got = out_dev[torch.from_numpy(rows).to(out_dev.device)].cpu().numpy()
    err = np.abs(got.astype(np.float64) - want)
    tol = 1e-5 + 1e-5 * np.abs(want)
    return {"rows_checked": int(len(rows)), "max_abs_err": float(err.max()), "max_err_over_tol": float((err / tol).max()),
            "within_rel1e-5_abs1e-5": bool((err <= tol).all()), "longest_row": int(deg[rows].max()),
            "checked_by": "oracle/s2v_oracle.c (oracle_level) on the sampled rows' CSR slices"}


# ------------------------------------------------------------------ reference arm
def reference_forward(full, steps: int, warmup: int, budget_s: float = 100.0):
    """The reference's FactorGraph::FeedForward on the WHOLE batch: warm-up calls (the first call of a batch
    size is many times slower), then up to `steps` timed calls within a time budget."""
    from oracle import bindings as ob
    kind = "reference" if ob.have_reference() else "port"
    impl = "reference" if kind == "reference" else "oracle"
    cores = os.cpu_count() or 1
    ob.set_threads(cores, impl)
    t0 = time.perf_counter()
    out = ob.forward(full, impl, iters=max(warmup, 1) + 1, want_levels=False)
    first_timed = float(out["seconds"][-1])
    spent = time.perf_counter() - t0
    more = int(max(0, min(steps - 1, (budget_s - spent) / max(first_timed, 1e-3))))
    secs = [first_timed]
    if more > 0:
        out2 = ob.forward(full, impl, iters=more + 1, want_levels=False)   # its first call is warm already
        secs += [float(x) for x in out2["seconds"][1:]]
        out = out2
    return out, np.asarray(secs), kind, cores


def run_reference(args, rank: int, world: int):
    if rank != 0:
        return
    full = make_workload(args.workload, 0)
    out, secs, kind, cores = reference_forward(full, args.steps, args.warmup)
    total = float(secs.sum())
    value = full.num_graphs * len(secs) / total
    line = {
        "metric": METRIC, "value": value, "unit": "graphs/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * total / len(secs), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "impl": "reference",
        "config": {"workload": WORKLOAD_TEXT[args.workload], "graphs": full.num_graphs, "nodes": full.num_nodes,
                   "edges": full.num_edges, "input_digest": full.digest(),
                   "sample": f"the whole batch per step; {len(secs)} timed FeedForward calls (time budget) of the {args.steps} asked for"},
        "cpu_baseline": {"value": value, "unit": "graphs/s", "cores": cores, "kind": kind,
                         "sample": f"FactorGraph::FeedForward on all {full.num_graphs} graphs, {len(secs)} timed calls after "
                                   f"{max(args.warmup, 1)} warm-up; MKL replaced by OpenMP plain loops"},
        "e2e": {"value": value, "unit": "graphs/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "steps_run": int(len(secs)), "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ our arm
class ClassifierStep:
    """One inference step on one rank.  Called, it is the library's own forward entry point (s2v_forward_f32) on
    device buffers, followed -- on several GPUs -- by the gather of the logits; `profile()` runs the same kernels
    composed from the library's operators so that each launch can be bracketed by CUDA events on its stream."""

    TILE_AUTO_MAX_NODES = 160000     # the library's automatic mode takes the tile kernel up to this many nodes

    def __init__(self, torch, eng, batch, stream, gather=None, use_tiles=2):
        from graphnn_b200 import engine
        self.torch, self.eng, self.ctx, self.b, self.stream, self.gather = torch, eng, eng.ctx, batch, stream, gather
        dev = eng.device
        self.hb = engine.build_host_batch(batch)
        self.db = eng.to_device(self.hb)
        G, N, d, C = batch.num_graphs, batch.num_nodes, batch.d, batch.num_class
        # use_tiles is the value of S2V_OPT_GRAPH_TILES: 0 never, 1 whenever the batch allows, 2 automatic (the library's default)
        self.mode = int(use_tiles)
        self.tiles = (d == 128 and int(batch.nodes_per_graph.max()) <= 128 and
                      (self.mode == 1 or (self.mode == 2 and N <= self.TILE_AUTO_MAX_NODES)))
        self.Y = torch.empty((G, d), device=dev)
        self.logits = torch.empty((G, C), device=dev)
        self.pred = torch.empty((G,), dtype=torch.int32, device=dev)
        self.cb = self.ctx.make_batch(G, N, self.db.row_ptr, self.db.col_idx, None, self.db.graph_ptr, self.db.tags, None,
                                      self.hb.max_graph_nodes)
        self.ws_fwd = torch.empty(self.ctx.workspace_bytes(N, G, d), dtype=torch.uint8, device=dev)
        if self.tiles:
            self.ws = torch.empty(self.ctx.graph_tiles_workspace_bytes(G), dtype=torch.uint8, device=dev)
        else:
            self.ha = torch.empty((N, d), device=dev)
            self.hbuf = torch.empty((N, d), device=dev)
            self.first_fused = d in (4, 8, 16, 32, 64, 128)      # the library runs level 1 from the tags for these widths
        self.events = []      # (kind, start, end) of the launches bracketed by profile()

    def __call__(self, timed: bool = False):
        st = self.stream.cuda_stream
        self.ctx.set_option(self.ctx.OPT_GRAPH_TILES, self.mode)
        self.ctx.forward(self.eng.model, self.cb, self.ws_fwd, self.logits, None, self.pred, None, stream=st)
        if self.gather is not None:
            self.gather(self.logits, self.pred, st)       # the final gather of the logits (NCCL through the C ABI)

    def _timed(self, kind, fn):
        a, b = self.torch.cuda.Event(enable_timing=True), self.torch.cuda.Event(enable_timing=True)
        a.record(self.stream)
        fn()
        b.record(self.stream)
        self.events.append((kind, a, b))

    def profile(self, iters: int = 10):
        """The kernels of a step, launch by launch, each between two CUDA events."""
        ctx, db, w, st, L = self.ctx, self.db, self.eng.w, self.stream.cuda_stream, self.b.levels
        if self.tiles:                            # untimed first call: the entry point allocates its product table once
            ctx.graph_tiles(L, db.row_ptr, db.col_idx, None, db.graph_ptr, db.tags, w["w_n2l"], w["p_node_conv"], self.ws, self.Y, stream=st)
        if not self.tiles and self.first_fused:   # untimed first call: the entry point allocates its product table once
            ctx.level_first(db.row_ptr, db.col_idx, None, w["p_node_conv"], w["w_n2l"], db.tags, self.hbuf, stream=st)
        for _ in range(iters):
            if self.tiles:
                self._timed("tiles", lambda: ctx.graph_tiles(L, db.row_ptr, db.col_idx, None, db.graph_ptr, db.tags, w["w_n2l"],
                                                             w["p_node_conv"], self.ws, self.Y, stream=st))
            else:
                cur, nxt = self.ha, self.hbuf
                if not self.first_fused:
                    ctx.input_proj_onehot(db.tags, w["w_n2l"], None, self.ha, stream=st)
                for lv in range(L):
                    if lv == 0 and self.first_fused:
                        self._timed("level_first", lambda: ctx.level_first(db.row_ptr, db.col_idx, None, w["p_node_conv"], w["w_n2l"],
                                                                           db.tags, nxt, stream=st))
                    else:
                        self._timed("level", lambda: ctx.level_lookup(db.row_ptr, db.col_idx, None, cur, w["p_node_conv"], w["w_n2l"],
                                                                     db.tags, nxt, stream=st))
                    cur, nxt = nxt, cur
                self._timed("pool", lambda: ctx.segment_sum(db.graph_ptr, cur, self.Y, stream=st))
            self._timed("readout", lambda: ctx.readout(self.Y, w["h1_weight"], w["h2_weight"], self.logits, None, self.pred, stream=st))
        self.torch.cuda.synchronize()

    def kernel_ms(self) -> dict:
        out = {}
        for kind, a, b in self.events:
            out.setdefault(kind, []).append(a.elapsed_time(b))
        return {k: (float(np.mean(v)), len(v)) for k, v in out.items()}


def device_timed(torch, dist, world, stream, step, steps, warmup, local_rank):
    for _ in range(max(warmup, 3)):
        step(False)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        t0.record(stream)
        for _ in range(steps):
            step(True)
        t1.record(stream)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    return t0.elapsed_time(t1), clocks.summary()


def max_over_ranks(torch, dist, world, dev, values):
    t = torch.tensor(values, dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(x) for x in t.cpu()]


def level_cfg2(ctx, torch, peaks):
    """The single fused level on the 1,048,576-node / 8,388,608-edge Erdos-Renyi problem, with a sampled-row
    check of this very output against the CPU oracle."""
    p = synth.erdos_renyi_level()
    dev = torch.device("cuda", torch.cuda.current_device())
    rp = torch.from_numpy(p.row_ptr).to(dev)
    ci = torch.from_numpy(p.col_idx).to(dev)
    H, W, X = (torch.from_numpy(a).to(dev) for a in (p.H, p.W, p.X))
    out = torch.empty_like(X)
    st = torch.cuda.current_stream().cuda_stream
    assert st != 0, "the caller must make a non-default torch stream current (handle 0 selects the context's stream)"
    torch.cuda.synchronize()
    for _ in range(5):
        ctx.level(rp, ci, None, H, W, X, out, stream=st)
    iters = 30
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    torch.cuda.synchronize()
    for a, b in evs:
        a.record()
        ctx.level(rp, ci, None, H, W, X, out, stream=st)
        b.record()
    torch.cuda.synchronize()
    ctx.stream_status(st)
    ms = sorted(a.elapsed_time(b) for a, b in evs)
    mean_ms = float(np.mean(ms))
    gather = level_bytes(p.n_rows, p.nnz, p.d, "gather", "dense")
    comp = level_bytes(p.n_rows, p.nnz, p.d, "compulsory", "dense")
    ach = gather / (mean_ms * 1e-3) / 1e9
    traffic, source = NCU_TRAFFIC["level_tc_er_d64_half"]
    traffic *= 2
    return {"workload": "fused level, Erdos-Renyi n=1048576 nnz=8388608 d=64, ReLU(A*H*W+X)", "ms": mean_ms,
            "ms_min": ms[0], "bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": ach / peaks["hbm_gbs"],
            "peak_kind": peaks["kind"], "bytes_gather_model": gather, "bytes_compulsory_model": comp,
            "edges_per_sec": p.nnz / (mean_ms * 1e-3),
            "traffic": traffic, "traffic_source": source,
            "frac_dram": traffic / (mean_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
            "frac_compulsory": comp / (mean_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
            "launches": iters, "l2_note": "H (268 MB) + X + out exceed the 126 MB L2",
            "parity": sampled_level_parity(p.row_ptr, p.col_idx, p.H, p.W, p.X, out)}


def run_ours(args, rank: int, world: int, local_rank: int):
    # torchrun pins OMP_NUM_THREADS to 1; the host-side scans and the host CSR builder are OpenMP-parallel,
    # so give every rank its share of the host cores before the library loads
    if world > 1:
        os.environ["OMP_NUM_THREADS"] = str(max(1, (os.cpu_count() or 1) // world))
    import torch
    import torch.distributed as dist
    from graphnn_b200 import capi, engine, sharding

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: the CUDA library has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    comm = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        ids = [capi.comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        comm = capi.Comm(local_rank, ids[0], world, rank)

    full = make_workload(args.workload, seed=0)          # the stated job, the same on every rank
    mine = sharding.shard_of(full, rank, world)          # strong scaling: this rank's graphs of the 16,384
    counts = sharding.shard_counts(full.nodes_per_graph, world)
    eng = engine.S2VInference(full.weights, full.levels, device=local_rank)
    ctx = eng.ctx
    # A stream of torch's own (non-zero handle: handle 0 would select the library's context stream, which
    # torch events cannot see), made current for everything below.
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.synchronize()
    torch.cuda.set_stream(stream)
    gather = sharding.ResultGather(counts, full.num_class, dev, comm=comm) if world > 1 else None
    step = ClassifierStep(torch, eng, mine, stream, gather, use_tiles=args.tiles)
    launches0 = ctx.launches
    elapsed_ms, clocks = device_timed(torch, dist, world, stream, step, args.steps, args.warmup, local_rank)
    launches = (ctx.launches - launches0) * args.steps // (args.steps + max(args.warmup, 3))
    ctx.stream_status(stream.cuda_stream)                # a kernel that recorded a status fails the run
    step.profile(10)                                     # the same kernels launch by launch, for the roofline
    ctx.stream_status(stream.cuda_stream)
    kms = step.kernel_ms()
    G, N, E, d, L, C = mine.num_graphs, mine.num_nodes, mine.num_edges, mine.d, mine.levels, mine.num_class

    # ---- end to end through the host-buffer entry points (host buffers in, host buffers out)
    ctx.set_option(ctx.OPT_GRAPH_TILES, int(args.tiles))
    hb = step.hb
    es = torch.from_numpy(np.ascontiguousarray(mine.edge_src, np.int32)).pin_memory()
    ed = torch.from_numpy(np.ascontiguousarray(mine.edge_dst, np.int32)).pin_memory()
    logits_h = np.empty((G, C), np.float32)
    pred_h = np.empty((G,), np.int32)

    def e2e_edges():          # raw edge list -> device CSR build -> forward
        ctx.infer_edges_host(eng.model, G, N, es.numpy(), ed.numpy(), hb.graph_ptr.numpy(), hb.tags.numpy(), logits_h, pred_h)

    def e2e_csr():            # ready host CSR -> forward
        eng.infer_host(hb, logits_h, pred_h)

    def e2e_host_sorted():    # raw edge list -> host sort (s2v_build_n2n_csr_host) -> forward
        rc = ctx.lib.s2v_build_n2n_csr_host(N, E, es.data_ptr(), ed.data_ptr(), 0, hb.row_ptr.data_ptr(), hb.col_idx.data_ptr(), None)
        assert rc == 0
        eng.infer_host(hb, logits_h, pred_h)

    e2e_steps = max(3, min(args.steps, 50))

    def time_e2e(fn) -> float:
        for _ in range(3):
            fn()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        w0 = time.perf_counter()
        for _ in range(e2e_steps):
            fn()
        torch.cuda.synchronize()
        return (time.perf_counter() - w0) * 1e3

    # two batches in flight: every step still uploads its inputs and downloads its results, but step i+1 is
    # submitted (s2v_infer_edges_host_submit, the other lane) before step i is waited for
    pipe_out = [(np.empty((G, C), np.float32), np.empty((G,), np.int32)) for _ in range(2)]

    def submit(i):
        ctx.infer_edges_host_submit(i % 2, eng.model, G, N, es.numpy(), ed.numpy(), hb.graph_ptr.numpy(), hb.tags.numpy(), *pipe_out[i % 2])

    def time_pipelined() -> float:
        for rep in range(2):                                 # first pass: warm-up (the second lane's staging is allocated)
            n = 4 if rep == 0 else e2e_steps
            if rep == 1:
                if world > 1:
                    dist.barrier()
                torch.cuda.synchronize()
                w0 = time.perf_counter()
            submit(0)
            for i in range(n):
                if i + 1 < n:
                    submit(i + 1)
                ctx.infer_host_wait(i % 2)
        return (time.perf_counter() - w0) * 1e3

    e2e_pipe_ms = time_pipelined()
    e2e_csr_ms = time_e2e(e2e_csr)
    e2e_sorted_ms = time_e2e(e2e_host_sorted)
    ctx.set_option(ctx.OPT_VALIDATE_HOST_INPUT, 0)
    e2e_edges_novalidate_ms = time_e2e(e2e_edges)
    ctx.set_option(ctx.OPT_VALIDATE_HOST_INPUT, 1)
    e2e_edges_ms = time_e2e(e2e_edges)                   # last: logits_h / pred_h below come from this entry point
    assert np.array_equal(pred_h, step.pred.cpu().numpy()), "host-buffer path and device path disagree"
    assert all(np.array_equal(p, pred_h) and np.array_equal(l, logits_h) for l, p in pipe_out), "lanes and synchronous entry disagree"

    elapsed_ms, e2e_edges_ms, e2e_csr_ms, e2e_sorted_ms, e2e_edges_novalidate_ms, e2e_pipe_ms = max_over_ranks(
        torch, dist, world, dev, [elapsed_ms, e2e_edges_ms, e2e_csr_ms, e2e_sorted_ms, e2e_edges_novalidate_ms, e2e_pipe_ms])

    # ---- the same with 16,384 graphs PER rank (weak scaling), device-timed only
    weak = None
    if world > 1:
        per_rank = make_workload(args.workload, seed=rank)
        wstep = ClassifierStep(torch, eng, per_rank, stream, sharding.ResultGather([per_rank.num_graphs] * world, C, dev, comm=comm),
                               use_tiles=args.tiles)
        w_ms, _ = device_timed(torch, dist, world, stream, wstep, args.steps, args.warmup, local_rank)
        (w_ms,) = max_over_ranks(torch, dist, world, dev, [w_ms])
        weak = {"value": world * per_rank.num_graphs * args.steps / (w_ms * 1e-3), "unit": "graphs/s", "ms_per_step": w_ms / args.steps,
                "graphs_per_gpu": per_rank.num_graphs, "scaling": "weak", "note": "every rank owns its own 16,384-graph batch (seed = rank)"}
        del wstep, per_rank

    if rank == 0:
        peaks = measured_peaks()
        total_graphs = full.num_graphs
        e2e_bytes_in = int(es.numel() * 4 + ed.numel() * 4 + hb.graph_ptr.numel() * 4 + hb.tags.numel() * 4)
        line = {
            "metric": METRIC, "value": total_graphs * args.steps / (elapsed_ms * 1e-3), "unit": "graphs/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": elapsed_ms / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD_TEXT[args.workload], "graphs_total": total_graphs,
                       "graphs_rank0": G, "nodes_rank0": N, "edges_rank0": E, "parallelism": f"shard-by-graph x{world}, logits gathered with s2v_gather_logits (NCCL)",
                       "l2": ("tile kernel: inputs of a few MB, embeddings never leave shared memory; no flush is done" if step.tiles else
                              ("per-step working set (two [N x d] fp32 matrices + CSR, > 500 MB) exceeds the 126 MB L2; no flush needed"
                               if 2 * N * d * 4 > 126e6 else
                               "rank 0's per-step working set fits the 126 MB L2 at this shard size; the step is launch- and "
                               "latency-bound there, and no flush is done")),
                       "path": "tile kernel" if step.tiles else "per-level kernels",
                       "input_digest": full.digest()},
            "e2e": {"value": total_graphs * e2e_steps / (e2e_edges_ms * 1e-3), "unit": "graphs/s",
                    "h2d_bytes_per_step": e2e_bytes_in, "d2h_bytes_per_step": int(logits_h.nbytes + pred_h.nbytes),
                    "steps": e2e_steps, "ms_per_step": e2e_edges_ms / e2e_steps,
                    "includes": "s2v_infer_edges_host_f32: host validation scan, upload of the raw edge list + tags + graph offsets, CSR built on "
                                "the device, forward, download of logits and predictions (what one FeedForward of the reference covers)",
                    "two_in_flight": {"value": total_graphs * e2e_steps / (e2e_pipe_ms * 1e-3), "ms_per_step": e2e_pipe_ms / e2e_steps,
                                      "includes": "the same work per step (same uploads and downloads), but step i+1 is submitted on the "
                                                  "context's other lane (s2v_infer_edges_host_submit) before step i is waited for "
                                                  "(s2v_infer_host_wait): the transfers of one batch overlap the kernels of the other"},
                    "without_host_validation": {"value": total_graphs * e2e_steps / (e2e_edges_novalidate_ms * 1e-3),
                                                "ms_per_step": e2e_edges_novalidate_ms / e2e_steps},
                    "from_host_csr": {"value": total_graphs * e2e_steps / (e2e_csr_ms * 1e-3), "ms_per_step": e2e_csr_ms / e2e_steps,
                                      "h2d_bytes_per_step": hb.nbytes(), "includes": "s2v_infer_host_f32 on a ready pinned host CSR"},
                    "host_sorted": {"value": total_graphs * e2e_steps / (e2e_sorted_ms * 1e-3), "ms_per_step": e2e_sorted_ms / e2e_steps,
                                    "includes": "s2v_build_n2n_csr_host (OpenMP stable counting sort) + s2v_infer_host_f32"}},
            "gpu_launches": int(launches),
            "kernel_ms": {k: {"mean_ms": v[0], "launches": v[1]} for k, v in kms.items()},
            "kernel_ms_note": "the step's kernels launched one by one from the operator entry points, each between CUDA events (a separate "
                              "pass of 10 steps after the timed region); `value` times s2v_forward_f32 itself",
            "clocks": clocks,
        }
        if step.tiles:
            t_ms = kms["tiles"][0]
            flops_tf32 = 3 * 2 * N * d * d * max(L - 1, 0)      # level 1 is a sum of product-table rows: no MMAs
            flops_fp32 = L * (2 * E * d + 2 * N * d * d + 2 * N * d)
            hbm_bytes = 4 * (N + 1) + 4 * E + 4 * N + 4 * (G + 1) + 4 * G * d + 4 * d * d + 4 * full.num_tags * d
            peak = peaks["bf16_tflops"] / 2
            line["roofline"] = {
                "kernel": "s2v_graph_tile_kernel (tcgen05 3xTF32; its tile-planning launch is inside the bracket)", "bound": "tensor",
                "achieved": flops_tf32 / (t_ms * 1e-3) / 1e12, "peak": peak, "unit": "TFLOP/s",
                "frac": flops_tf32 / (t_ms * 1e-3) / 1e12 / peak,
                "peak_kind": f"{peaks['kind']} dense bf16 cuBLAS burst / 2: TF32 MMAs issue at half the bf16 rate",
                "flops_model": "3 TF32 products (hi*hi, hi*lo, lo*hi) x 2*N*d*d per level x (L - 1) levels (the first level is a gather-sum over the product table)",
                "fp32_equivalent_tflops": flops_fp32 / (t_ms * 1e-3) / 1e12,
                "ms_per_launch": t_ms, "launches": kms["tiles"][1], "traffic": None,
                "hbm_bytes_algorithmic": hbm_bytes, "hbm_gbs": hbm_bytes / (t_ms * 1e-3) / 1e9,
                "hbm_note": "CSR + tags + graph offsets in, pooled [G x d] out: the node embeddings never leave shared memory"}
        else:
            lv_ms, lv_n = kms["level"]
            comp = level_bytes(N, E, d, "compulsory", "lookup")
            ach = comp / (lv_ms * 1e-3) / 1e9
            line["roofline"] = {"kernel": f"s2v_level_tc_kernel (tcgen05, d={d}, X looked up from W_in by tag; levels that read H)",
                                "bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": ach / peaks["hbm_gbs"],
                                "peak_kind": peaks["kind"], "ms_per_launch": lv_ms, "launches": lv_n, "bytes_per_launch": comp,
                                "model": "compulsory (each H row once) + CSR + tags + out + W", "traffic": None}
            if args.workload == "molecules" and world == 1:
                traffic, source = NCU_TRAFFIC["level_tc_mol_d128"]
                line["roofline"].update({"traffic": traffic, "traffic_source": source,
                                         "frac_dram": traffic / (lv_ms * 1e-3) / 1e9 / peaks["hbm_gbs"]})
            if "level_first" in kms:
                f_ms, f_n = kms["level_first"]
                fb = level_bytes(N, E, d, "compulsory", "lookup", h_form="table")
                line["roofline_first_level"] = {"kernel": "first level from the tags: product table ReLU(W_in)*W (tiny launch) + gather-sum over its rows, no per-row product", "bound": "hbm",
                                                "achieved": fb / (f_ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                                "frac": fb / (f_ms * 1e-3) / 1e9 / peaks["hbm_gbs"], "ms_per_launch": f_ms,
                                                "launches": f_n, "bytes_per_launch": fb, "traffic": None,
                                                "time_includes": "the tag range check and the product-table launch of the entry point"}
                if args.workload == "molecules" and world == 1:
                    traffic, source = NCU_TRAFFIC["first_level_mol_d128"]
                    line["roofline_first_level"].update({"traffic": traffic, "traffic_source": source})
        if weak is not None:
            line["weak"] = weak
        if world > 1:
            # the logits of ALL ranks as the timed step gathered them on rank 0, against one call of the reference on the whole batch
            ref_out, _, kind, _ = reference_forward(full, 1, 0, budget_s=0.0)
            got_all, pred_all = gather.logits_all.cpu().numpy(), gather.pred_all.cpu().numpy()
            want = ref_out["logits"]
            err = np.abs(got_all.astype(np.float64) - want)
            scale = max(1.0, float(np.abs(want).max()))
            line["parity"] = {"graphs_checked": int(want.shape[0]), "argmax_equal": bool(np.array_equal(ref_out["argmax"], pred_all)),
                              "max_abs_logit_err": float(err.max()),
                              "within_rel1e-5_abs1e-5xscale": bool((err <= 1e-5 * scale + 1e-5 * np.abs(want)).all()), "logit_scale": scale,
                              "checked_by": f"the reference build (kind={kind}) on the whole batch, against the logits of all {world} shards as "
                                            "s2v_gather_logits assembled them on rank 0 in the timed step"}
        if world == 1:
            ref_out, secs, kind, cores = reference_forward(full, 3, 1, budget_s=60.0)
            line["cpu_baseline"] = {"value": full.num_graphs * len(secs) / float(secs.sum()), "unit": "graphs/s", "cores": cores, "kind": kind,
                                    "sample": f"FactorGraph::FeedForward on all {full.num_graphs} graphs of the batch, {len(secs)} timed calls "
                                              f"after a warm-up; MKL replaced by OpenMP plain loops"}
            want = ref_out["logits"]
            err = np.abs(logits_h.astype(np.float64) - want)
            scale = max(1.0, float(np.abs(want).max()))
            line["parity"] = {"graphs_checked": int(want.shape[0]), "argmax_equal": bool(np.array_equal(ref_out["argmax"], pred_h)),
                              "max_abs_logit_err": float(err.max()),
                              "within_rel1e-5_abs1e-5xscale": bool((err <= 1e-5 * scale + 1e-5 * np.abs(want)).all()), "logit_scale": scale,
                              "checked_by": f"the reference build (kind={kind}) on the whole batch, against the logits the e2e entry point returned"}
            if not args.skip_level:
                line["level_cfg2"] = level_cfg2(ctx, torch, peaks)
            if not step.tiles and d == 128 and int(full.nodes_per_graph.max()) <= 128:
                # the opt-in whole-classifier tile kernel on the same batch, device-timed, checked against the default path
                tstep = ClassifierStep(torch, eng, full, stream, None, use_tiles=1)
                t_ms, _ = device_timed(torch, dist, 1, stream, tstep, min(args.steps, 20), 3, local_rank)
                ctx.stream_status(stream.cuda_stream)
                tstep.profile(10)
                tk = tstep.kernel_ms()
                flops_tf32 = 3 * 2 * N * d * d * max(L - 1, 0)      # level 1 is a sum of product-table rows: no MMAs
                line["tile_kernel"] = {
                    "note": "s2v_graph_tiles_f32 (S2V_OPT_GRAPH_TILES = 1): input projection + all levels + pooling in one kernel, embeddings in shared memory",
                    "value": full.num_graphs * min(args.steps, 20) / (t_ms * 1e-3), "unit": "graphs/s", "ms_per_step": t_ms / min(args.steps, 20),
                    "kernel_ms": tk["tiles"][0], "bound": "tensor", "achieved_tflops_tf32": flops_tf32 / (tk["tiles"][0] * 1e-3) / 1e12,
                    "peak_tflops_tf32": peaks["bf16_tflops"] / 2, "frac": flops_tf32 / (tk["tiles"][0] * 1e-3) / 1e12 / (peaks["bf16_tflops"] / 2),
                    "argmax_equal_to_default_path": bool(np.array_equal(tstep.pred.cpu().numpy(), step.pred.cpu().numpy())),
                    "max_abs_logit_diff_to_default_path": float((tstep.logits - step.logits).abs().max().item())}
    # ---- several GPUs: the row-partitioned giant graph at a scale that runs in seconds
    giant_block = None
    if world > 1 and args.giant_scale > 0 and args.workload == "molecules":
        giant_block = giant_measure(torch, dist, capi, comm, ctx, rank, world, local_rank, dev, stream, args.giant_scale, 3, 2,
                                    args.giant_exchange, args.giant_chunks, args.giant_reserved_sms)
    if rank == 0:
        if giant_block is not None:
            line["giant"] = giant_block
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        comm.close()
        dist.destroy_process_group()


# ------------------------------------------------------------------ giant graph
def giant_measure(torch, dist, capi, comm, ctx, rank, world, local_rank, dev, stream, scale, steps, warmup, exchange_mode="referenced", chunks=0,
                  reserved_sms=0):
    """Single giant R-MAT graph, row-partitioned: 2 levels of ReLU(A*H*W), d = 128.  Per level the ranks exchange
    either only the rows of H each of them references (`referenced`: s2v_exchange_rows_f32, packed by the row-lookup
    kernel) or all of H (`allgather`: s2v_allgather_rows_f32, in place) -- block by block, pipelined against the
    compute.  The timed step starts with H0 already in every rank's table (inputs resident in HBM)."""
    from graphnn_b200 import giant
    d, levels = 128, 2
    shard = giant.rmat_shard_on_device(scale, 16 << scale, rank, world, dev, seed=0)
    n = 1 << scale
    nnz_rank = shard.nnz
    plan = giant.plan_hubs(shard, threshold=2048, piece=512)
    spmm_fn, segsum_fn = giant.make_gpu_hub_fns(ctx)
    if exchange_mode == "referenced":
        chunks = chunks or 8
        g = giant.GiantGraphReferenced(shard, d, rank, world, giant.make_gpu_level_fn(ctx), pack_fn=giant.make_gpu_pack_fn(ctx), chunks=chunks,
                                       hub_plan=plan, spmm_fn=spmm_fn, segsum_fn=segsum_fn,
                                       exchange_rows=giant.make_comm_exchange_rows(comm) if comm is not None else None)
        referenced = g.rows_referenced       # rows of H this rank's shard names at all (own + remote)
        ag_bytes = g.exchange_bytes_per_level()
    else:
        chunks = chunks or 4
        referenced = int(torch.unique(shard.col_idx).numel())
        exchange = giant.make_comm_exchange(comm) if comm is not None else None
        g = giant.GiantGraphLevels(shard, d, rank, world, giant.make_gpu_level_fn(ctx), chunks=chunks, hub_plan=plan,
                                   spmm_fn=spmm_fn, segsum_fn=segsum_fn, exchange=exchange)
        ag_bytes = g.all_gather_bytes_per_level()
    gen = torch.Generator(device=dev)
    gen.manual_seed(1234 + rank)
    slab0 = torch.randn((shard.rows, d), device=dev, generator=gen)
    gen.manual_seed(99)
    W = torch.randn((d, d), device=dev, generator=gen) * 0.05
    stats = torch.tensor([nnz_rank, nnz_rank, referenced], dtype=torch.int64, device=dev)
    nnz_sum = stats[:1].clone()
    if world > 1:
        dist.all_reduce(nnz_sum)
        dist.all_reduce(stats[1:2], op=dist.ReduceOp.MAX)
    nnz_total, nnz_max = int(nnz_sum.item()), int(stats[1].item())
    g.set_input(slab0)               # H0 in every rank's table: the state the timed region starts from
    if world > 1 and reserved_sms > 0:
        ctx.set_option(ctx.OPT_RESERVED_SMS, reserved_sms)
    torch.cuda.synchronize()

    def full_step(timed=False):
        return g.run(W, levels, timed=timed, return_copy=False)   # the result stays in the rank's table

    for _ in range(max(warmup, 1)):
        full_step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    launches0 = ctx.launches
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    step_marks = []
    with ClockSampler(local_rank) as clocks:
        t0.record(stream)
        for _ in range(steps):
            full_step(timed=True)
            step_marks.append(torch.cuda.Event(enable_timing=True))
            step_marks[-1].record(stream)
        t1.record(stream)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    ctx.stream_status(stream.cuda_stream)
    ctx.set_option(ctx.OPT_RESERVED_SMS, 0)
    per_level = g.timing_summary()
    step_ms = [a.elapsed_time(b) for a, b in zip([t0] + step_marks[:-1], step_marks)]
    ms, = max_over_ranks(torch, dist, world, dev, [t0.elapsed_time(t1)])
    # the slowest rank's view of the last step's levels (rank 0's is printed in full)
    lv_mine = per_level[-levels:] if per_level else []
    lv_worst = max_over_ranks(torch, dist, world, dev, [x["compute_ms"] for x in lv_mine] + [x["exposed_exchange_ms"] for x in lv_mine]) if lv_mine else []
    # parity of this very run: sampled output rows of rank 0 recomputed on the host for both levels
    parity = giant_sampled_parity(torch, g, shard, W, levels) if rank == 0 else None
    if rank != 0:
        return None
    peaks = measured_peaks()
    per_level_bytes = 4 * (n + 1) + 4 * nnz_total + 4 * nnz_total * d + 4 * n * d + 4 * d * d   # gather model, all ranks
    sec_per_level = ms * 1e-3 / steps / levels
    lv = per_level[-levels:] if per_level else []
    return {"metric": "s2v_level_edges_per_sec", "value": nnz_total * levels * steps / (ms * 1e-3), "unit": "edges/s",
            "n_gpus": world, "steps": steps, "ms_per_step": ms / steps, "scaling": "strong",
            "config": {"workload": f"giant R-MAT(0.57,0.19,0.19,0.05) scale {scale}, {16 << scale} generated edges, symmetrised + deduplicated "
                                   f"to nnz={nnz_total}, node ids renumbered by an odd multiplier, d=128, 2 levels of ReLU(A*H*W), "
                                   f"row-partitioned x{world}, H0 in every rank's table before the timed region",
                       "exchange": ("referenced rows only (s2v_exchange_rows_f32)" if exchange_mode == "referenced" else "all of H (s2v_allgather_rows_f32)"),
                       "exchange_bytes_received_per_gpu_per_level": ag_bytes, "all_of_H_would_be": (world - 1) * shard.rows * d * 4,
                       "chunks": chunks, "sms_left_to_nccl": reserved_sms if world > 1 else 0,
                       "nnz_max_over_mean": nnz_max / (nnz_total / world), "hub_rows_rank0": 0 if plan is None else plan.n_hub,
                       "rows_of_H_referenced_by_rank0": referenced / n},
            "per_level_rank0": [{**x, "exchange_gbs_per_direction": (ag_bytes / (x["exchange_ms_sum"] * 1e-3) / 1e9) if x["exchange_ms_sum"] > 0 else None}
                                for x in lv],
            "per_level_max_over_ranks": {"compute_ms": lv_worst[:levels], "exposed_exchange_ms": lv_worst[levels:]},
            "step_ms_rank0": step_ms,
            "nvlink_peak_gbs_per_direction": 900, "gpu_launches_per_step": int((ctx.launches - launches0) // steps),
            "roofline": {"kernel": "fused level, gather model, time includes the pipelined exchange", "bound": "hbm",
                         "achieved": per_level_bytes / world / sec_per_level / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": per_level_bytes / world / sec_per_level / 1e9 / peaks["hbm_gbs"], "peak_kind": peaks["kind"], "traffic": None},
            "parity": parity, "clocks": clocks.summary()}


GIANT_LONG_ROW = 4096


def giant_sampled_parity(torch, g, shard, W, levels, n_sample=1024):
    """>= 1,000 output rows of this rank recomputed on the host from the gathered CSR rows.  Level 2 of a sampled row
    needs level 1 of all its neighbours, which are not sampled; so the check is per level: for each level the kernel's
    INPUT matrix (as it lies in device memory after the run) is taken as given and the sampled output rows are
    recomputed from it with the CPU oracle."""
    from oracle import bindings as ob
    rng = np.random.default_rng(11)
    dev = shard.col_idx.device
    rp = shard.row_ptr.to(torch.int64)
    deg = rp[1:] - rp[:-1]
    pick = set(rng.integers(0, g.rows, n_sample).tolist()) | {0, g.rows - 1} | set(torch.topk(deg, 8).indices.cpu().tolist())
    rows = torch.tensor(sorted(pick), dtype=torch.int64, device=dev)
    starts, lens = rp[rows], deg[rows]
    ends_excl = torch.cumsum(lens, 0)
    idx = torch.repeat_interleave(starts - (ends_excl - lens), lens) + torch.arange(int(lens.sum()), device=dev)
    cols = shard.col_idx[idx].to(torch.int64)               # original global column ids of the sampled rows, CSR order
    uniq, inv = torch.unique(cols, return_inverse=True)
    rp_s = torch.cat([torch.zeros(1, dtype=torch.int64, device=dev), ends_excl]).cpu().numpy().astype(np.int32)
    src_pos, out_pos = g.position_of(uniq), g.position_of(shard.row_lo + rows)
    Wh = W.cpu().numpy()
    results = []
    for lvl in range(1, levels + 1):
        src, dst = g.level_buffers(lvl)
        prob = synth.LevelProblem(len(rows), len(uniq), rp_s, inv.cpu().numpy().astype(np.int32), src[src_pos].cpu().numpy(), Wh, None)
        want, _ = ob.level(prob, "oracle")
        want64, _ = ob.level(prob, "oracle_f64")
        got = dst[out_pos].cpu().numpy().astype(np.float64)
        scale = max(1.0, float(np.abs(want).max()))
        lens_h = lens.cpu().numpy()
        short = lens_h <= GIANT_LONG_ROW
        bar32, bar64 = 1e-5 * scale + 1e-5 * np.abs(want), 1e-5 * scale + 1e-5 * np.abs(want64)
        err32, err64 = np.abs(got - want), np.abs(got - want64)
        ok = bool((err32[short] <= bar32[short]).all() and (err64[~short] <= bar64[~short]).all())
        results.append({"level": lvl, "rows_checked": int(len(rows)), "longest_row": int(lens_h.max()),
                        "max_abs_err": float(err32[short].max()) if short.any() else 0.0,
                        "long_rows": int((~short).sum()),
                        "long_rows_max_abs_err_vs_f64": float(err64[~short].max()) if (~short).any() else 0.0,
                        "long_rows_f32_oracle_vs_f64": float(np.abs(want - want64)[~short].max()) if (~short).any() else 0.0,
                        "value_scale": scale, "within_rel1e-5_abs1e-5xscale": ok})
    return {"levels": results,
            "checked_by": "oracle/s2v_oracle.c on the sampled rows' CSR slices and the level's input rows: oracle_level (float sums in CSR "
                          f"order) for rows of at most {GIANT_LONG_ROW} entries; longer rows against oracle_level_f64 (all sums in double), "
                          "because a float sum over 10^5..10^6 entries depends on its order by more than the bar (the float oracle's own "
                          "distance from the double result is printed beside ours)"}


def run_giant(args, rank: int, world: int, local_rank: int):
    import torch
    import torch.distributed as dist
    from graphnn_b200 import capi

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    comm = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        ids = [capi.comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        comm = capi.Comm(local_rank, ids[0], world, rank)
    ctx = capi.Context(local_rank)
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.synchronize()
    torch.cuda.set_stream(stream)
    block = giant_measure(torch, dist, capi, comm, ctx, rank, world, local_rank, dev, stream, args.scale, args.steps, max(args.warmup, 3),
                          args.giant_exchange, args.giant_chunks, args.giant_reserved_sms)
    if rank == 0:
        block.update({"warmup": max(args.warmup, 3), "higher_is_better": True, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                      "gpu_launches": block["gpu_launches_per_step"] * args.steps})
        print(json.dumps(block), flush=True)
    if world > 1:
        dist.barrier()
        comm.close()
        dist.destroy_process_group()


# ------------------------------------------------------------------ profiler cases
def run_case(args):
    """Small, self-contained launches of one kernel for profiler captures; prints the mean CUDA-event time.

    er_d64      fused level, Erdos-Renyi n=524,288, nnz=4,194,304, d=64, dense X (half the 1M-node problem: H, X and
                out are 134 MB each, above the 126 MB L2);  er_d64_full: the full problem
    mol_d128    per-level kernel on 16,384 molecule-like graphs, d=128, X looked up from W_in by tag
    prot_d64    per-level kernel on 2,048 protein-like graphs, d=64
    mol_first   first level straight from the tags (product table + gather-sum) on 16,384 molecule-like graphs, d=128
    prot_first  the same on 2,048 protein-like graphs, d=64
    mol_tiles   tile kernel (projection + 4 levels + pooling) on 16,384 molecule-like graphs;  mol_tiles_small: 4,096 graphs
    readout     readout (two layers + softmax / argmax) of 16,384 pooled embeddings, d=128, hidden=256, 2 classes
    mol_paths   whole forward pass (s2v_forward_f32) on 512 .. 16,384 molecule-like graphs through the per-level kernels
                and through the tile kernel, one line per batch size"""
    import torch
    from graphnn_b200 import capi
    if args.case == "mol_paths":
        from graphnn_b200 import engine
        stream = torch.cuda.Stream()
        torch.cuda.set_stream(stream)
        st = stream.cuda_stream
        for G in (512, 1024, 2048, 4096, 8192, 16384):
            b = synth.molecules_16k(seed=0, weight_seed=WEIGHT_SEED, num_graphs=G)
            eng = engine.S2VInference(b.weights, b.levels)
            db = eng.to_device(engine.build_host_batch(b))
            ms = []
            for mode in (0, 1):
                eng.ctx.set_option(eng.ctx.OPT_GRAPH_TILES, mode)
                for _ in range(5):
                    eng.forward(db, stream=st)
                torch.cuda.synchronize()
                a, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                for _ in range(50):
                    eng.forward(db, stream=st)
                e.record(stream)
                torch.cuda.synchronize()
                eng.ctx.stream_status(st)
                ms.append(a.elapsed_time(e) / 50)
            print(f"G={G} N={b.num_nodes} per-level kernels {ms[0]:.4f} ms  tile kernel {ms[1]:.4f} ms  ratio {ms[0] / ms[1]:.2f}", flush=True)
        return
    ctx = capi.Context(0)
    dev = torch.device("cuda", 0)
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    st = stream.cuda_stream

    def up(a):
        return torch.from_numpy(np.ascontiguousarray(a)).to(dev)

    if args.case == "readout":
        rng = np.random.default_rng(0)
        G, d_, hid, C_ = 16384, 128, 256, 2
        Yd = up(rng.standard_normal((G, d_), dtype=np.float32))
        W1d, W2d = up(rng.standard_normal((d_, hid), dtype=np.float32) * 0.1), up(rng.standard_normal((hid, C_), dtype=np.float32) * 0.1)
        lg, pr = torch.empty((G, C_), device=dev), torch.empty((G, C_), device=dev)
        pd = torch.empty(G, dtype=torch.int32, device=dev)
        launch = lambda: ctx.readout(Yd, W1d, W2d, lg, pr, pd, stream=st)
        desc = f"readout: G={G} d={d_} hidden={hid} C={C_}"
    elif args.case.startswith("er_d64"):
        full = args.case.endswith("full")
        p = synth.erdos_renyi_level(n=1 << (20 if full else 19), nnz=1 << (23 if full else 22), d=64)
        rp, ci, H, W, X = up(p.row_ptr), up(p.col_idx), up(p.H), up(p.W), up(p.X)
        out = torch.empty_like(X)
        launch = lambda: ctx.level(rp, ci, None, H, W, X, out, stream=st)
        desc = f"{p.name}: n={p.n_rows} nnz={p.nnz}"
    else:
        if args.case in ("prot_d64", "prot_first"):
            b = synth.proteins_4k(seed=0, num_graphs=2048)
        else:
            b = synth.molecules_16k(seed=0, num_graphs=4096 if args.case.endswith("small") else 16384)
        rp_h, ci_h, _ = capi.build_n2n_csr_host(b.num_nodes, b.edge_src, b.edge_dst, with_val=False)
        rp, ci, tags, gp = up(rp_h), up(ci_h), up(b.tags.astype(np.int32)), up(b.graph_offsets())
        W, table = up(b.weights["p_node_conv"]), up(b.weights["w_n2l"])
        desc = f"{b.name}: G={b.num_graphs} N={b.num_nodes} nnz={b.num_edges} d={b.d}"
        if args.case in ("mol_first", "prot_first"):
            out = torch.empty((b.num_nodes, b.d), device=dev)
            launch = lambda: ctx.level_first(rp, ci, None, W, table, tags, out, stream=st)
        elif args.case.startswith("mol_tiles"):
            ws = torch.empty(ctx.graph_tiles_workspace_bytes(b.num_graphs), dtype=torch.uint8, device=dev)
            Y = torch.empty((b.num_graphs, b.d), device=dev)
            launch = lambda: ctx.graph_tiles(b.levels, rp, ci, None, gp, tags, table, W, ws, Y, stream=st)
        else:
            H = torch.randn((b.num_nodes, b.d), device=dev).abs_()
            out = torch.empty_like(H)
            launch = lambda: ctx.level_lookup(rp, ci, None, H, W, table, tags, out, stream=st)
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
    ctx.stream_status(st)
    print(desc, "mean ms/launch:", float(np.mean([a.elapsed_time(e) for a, e in evs])))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="molecules", choices=["molecules", "proteins", "giant"])
    ap.add_argument("--scale", type=int, default=24, help="giant workload: log2 of the node count (26 = the full configuration)")
    ap.add_argument("--giant-scale", type=int, default=22,
                    help="default multi-GPU run: log2 node count of the giant-graph block appended to the line (0 = leave it out)")
    ap.add_argument("--giant-exchange", default="referenced", choices=["referenced", "allgather"],
                    help="giant graph: exchange only the rows each rank references, or all of H, per level")
    ap.add_argument("--giant-reserved-sms", type=int, default=0,
                    help="giant graph on several GPUs: SMs the level kernel leaves to NCCL's kernels (S2V_OPT_RESERVED_SMS)")
    ap.add_argument("--giant-chunks", type=int, default=0, help="giant graph: row blocks per rank (0: 8 for referenced, 4 for allgather)")
    ap.add_argument("--skip-level", action="store_true", help="leave out the 1M-node fused-level measurement")
    ap.add_argument("--tiles", type=int, default=2, choices=[0, 1, 2],
                    help="S2V_OPT_GRAPH_TILES: 0 per-level kernels only, 1 whole-classifier tile kernel whenever the batch allows, "
                         "2 the library's default (tile kernel for batches of at most 160,000 nodes)")
    ap.add_argument("--case", default=None, choices=["er_d64", "er_d64_full", "mol_d128", "prot_d64", "mol_first", "prot_first", "readout", "mol_tiles", "mol_tiles_small", "mol_paths"],
                    help="run one small launch case (for profiler captures) instead of the benchmark")
    ap.add_argument("--launches", type=int, default=3)
    args = ap.parse_args()
    if args.case:
        run_case(args)
        return
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world == 1 and args.gpus > 1 and "RANK" not in os.environ:
        # convenience: relaunch under torchrun
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29511", os.path.abspath(__file__)] + sys.argv[1:]
        raise SystemExit(subprocess.call(cmd))
    if args.workload == "giant":
        if args.impl == "reference":
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": "the reference is int32 and single-GPU; the giant-graph "
                                  "configuration has no reference run at this size (parity: sampled rows against the CPU oracle inside the run)"}))
            return
        run_giant(args, rank, world, local_rank)
        return
    if args.impl == "reference":
        args.warmup = max(args.warmup, 1)   # the reference's first FeedForward of a batch size is many times slower
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
