"""Benchmark of the s2v mean-field inference path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload molecules|proteins]

A step is one inference pass (input projection, L fused levels, pooling, readout, logits
gather) over one batch of synthetic graphs that is already resident in HBM.  Default
workload: the batched molecule-like configuration (16,384 graphs per GPU, latent 128,
4 levels), sharded by graph: every rank owns its own 16,384-graph shard of a
16,384 x N-graph job (weak scaling) and the only collective is the final gather of
the logits.  Rank 0 prints ONE JSON line.

`value` is graphs/s over all ranks with inputs on the device; `e2e` is the same metric
through the host-buffer entry point (edge list -> CSR on the host, upload, forward,
download) ; `roofline` describes the fused level kernel inside the timed region;
`level_cfg2` is the single fused level on the 1M-node / 8M-edge Erdos-Renyi problem;
`cpu_baseline` is the reference's own CPU code on this machine's cores.

`--impl reference` times the reference's CPU implementation (oracle/_ref, MKL replaced
by plain OpenMP loops) on a bounded sample of the same workload.
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
    "molecules": "molecules_16k: 16,384 molecule-like graphs per GPU (20-40 nodes, tree + 10% edges, 82 Zipf(1.2) tags), "
                 "d=128, L=4, hidden=256, C=2, sum pooling",
    "proteins": "proteins_4k: 4,096 protein-like graphs per GPU (100-620 nodes, random geometric, mean degree ~7.4, 3 tags), "
                "d=64, L=5, hidden=128, C=2, sum pooling",
}
METRIC = "s2v_inference_graphs_per_sec"


def make_workload(name: str, seed: int):
    if name == "molecules":
        return synth.molecules_16k(seed=seed, weight_seed=WEIGHT_SEED)
    if name == "proteins":
        return synth.proteins_4k(seed=seed, weight_seed=WEIGHT_SEED)
    raise SystemExit(f"unknown workload {name}")


def measured_peaks():
    p = os.path.join(REPO, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


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


# ------------------------------------------------------------------ byte models
def level_bytes(n_rows, nnz, d, model: str, x_form: str) -> int:
    """Algorithmic bytes of one fused level.  `gather`: every neighbour row fetched once
    per edge; `compulsory`: every H row fetched once.  x_form: dense (X read as
    [N x d]), lookup (tags + table) or none."""
    b_csr = 4 * (n_rows + 1) + 4 * nnz          # val == NULL form: no value array
    b_h = 4 * nnz * d if model == "gather" else 4 * n_rows * d
    b_x = {"dense": 4 * n_rows * d, "lookup": 4 * n_rows, "none": 0}[x_form]
    return b_csr + b_h + b_x + 4 * n_rows * d + 4 * d * d


# ------------------------------------------------------------------ reference arm
def run_reference(args, rank: int, world: int):
    if rank != 0:
        return
    from oracle import bindings as ob
    kind = "reference" if ob.have_reference() else "port"
    impl = "reference" if kind == "reference" else "oracle"
    cores = os.cpu_count() or 1
    ob.set_threads(cores, impl)
    sample_graphs = 4096 if args.workload == "molecules" else 512
    full = make_workload(args.workload, 0)
    lo, hi = 0, sample_graphs
    off = full.graph_offsets().astype(np.int64)
    sel = full.edge_src < off[hi]
    sample = synth.GraphBatch(full.nodes_per_graph[lo:hi].copy(), full.edge_src[sel].copy(), full.edge_dst[sel].copy(),
                              full.tags[: off[hi]].copy(), full.num_tags, full.d, full.levels, full.hidden,
                              full.num_class, full.weights, full.name + f"[first {sample_graphs}]")
    iters = args.warmup + args.steps
    out = ob.forward(sample, impl, iters=iters, want_levels=False)
    secs = np.asarray(out["seconds"][args.warmup:])
    total = float(secs.sum())
    value = sample.num_graphs * len(secs) / total
    line = {
        "metric": METRIC, "value": value, "unit": "graphs/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * total / len(secs), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "impl": "reference",
        "config": {"workload": WORKLOAD_TEXT[args.workload],
                   "sample": f"first {sample.num_graphs} graphs ({sample.num_nodes} nodes, {sample.num_edges} edges) per step"},
        "cpu_baseline": {"value": value, "unit": "graphs/s", "cores": cores, "kind": kind,
                         "sample": f"FactorGraph::FeedForward on the first {sample.num_graphs} graphs of the batch, "
                                   f"{len(secs)} timed runs; MKL replaced by OpenMP plain loops"},
        "e2e": {"value": value, "unit": "graphs/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ our arm
def cpu_baseline(args, full):
    """Reference CPU code on a bounded sample (rank 0, N=1 only)."""
    from oracle import bindings as ob
    kind = "reference" if ob.have_reference() else "port"
    impl = "reference" if kind == "reference" else "oracle"
    cores = os.cpu_count() or 1
    ob.set_threads(cores, impl)
    n = 2048 if args.workload == "molecules" else 256
    off = full.graph_offsets().astype(np.int64)
    sel = full.edge_src < off[n]
    sample = synth.GraphBatch(full.nodes_per_graph[:n].copy(), full.edge_src[sel].copy(), full.edge_dst[sel].copy(),
                              full.tags[: off[n]].copy(), full.num_tags, full.d, full.levels, full.hidden,
                              full.num_class, full.weights, "sample")
    out = ob.forward(sample, impl, iters=4, want_levels=False)
    secs = np.asarray(out["seconds"][1:])
    return {"value": sample.num_graphs * len(secs) / float(secs.sum()), "unit": "graphs/s", "cores": cores,
            "kind": kind,
            "sample": f"FactorGraph::FeedForward on the first {n} graphs of the batch ({sample.num_nodes} nodes), "
                      f"3 timed runs after 1 warm-up; MKL replaced by OpenMP plain loops"}, out


def level_cfg2(ctx, torch, peak_gbs, peak_kind):
    """The single fused level on the 1,048,576-node / 8,388,608-edge Erdos-Renyi problem."""
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
    ms = sorted(a.elapsed_time(b) for a, b in evs)
    mean_ms = float(np.mean(ms))
    gather = level_bytes(p.n_rows, p.nnz, p.d, "gather", "dense")
    comp = level_bytes(p.n_rows, p.nnz, p.d, "compulsory", "dense")
    ach = gather / (mean_ms * 1e-3) / 1e9
    return {"workload": "fused level, Erdos-Renyi n=1048576 nnz=8388608 d=64, ReLU(A*H*W+X)", "ms": mean_ms,
            "ms_min": ms[0], "bound": "hbm", "achieved": ach, "peak": peak_gbs, "unit": "GB/s", "frac": ach / peak_gbs,
            "peak_kind": peak_kind, "bytes_gather_model": gather, "bytes_compulsory_model": comp,
            "edges_per_sec": p.nnz / (mean_ms * 1e-3),
            # dram__bytes_read + dram__bytes_write of one launch on the half-size problem
            # (the committed ncu summary of the tcgen05 level kernel: 806.40 MB + 119.01 MB), times two
            "traffic": 2 * (806403584 + 119012864), "traffic_note": "ncu capture at n=524,288, scaled x2",
            "launches": iters,
            "l2_note": "H (268 MB) + X + out exceed the 126 MB L2"}


def run_ours(args, rank: int, world: int, local_rank: int):
    # torchrun pins OMP_NUM_THREADS to 1; the host CSR builder (timed in e2e.from_edge_list) is
    # OpenMP-parallel, so give every rank its share of the host cores before the library loads
    if world > 1:
        os.environ["OMP_NUM_THREADS"] = str(max(1, (os.cpu_count() or 1) // world))
    import torch
    import torch.distributed as dist
    from graphnn_b200 import capi, engine

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: the CUDA library has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    full = make_workload(args.workload, seed=rank)      # this rank's shard of the 16,384 x N-graph job
    eng = engine.S2VInference(full.weights, full.levels, device=local_rank)
    ctx = eng.ctx
    hb = engine.build_host_batch(full)
    db = eng.to_device(hb)
    G, N, E, d, L = full.num_graphs, full.num_nodes, full.num_edges, full.d, full.levels
    C = full.num_class
    w = eng.w
    # the step, composed from the library's operators so that each fused-level launch can
    # be bracketed by CUDA events on the launching stream
    ha = torch.empty((N, d), device=dev)
    hbuf = torch.empty((N, d), device=dev)
    Y = torch.empty((G, d), device=dev)
    logits = torch.empty((G, C), device=dev)
    pred = torch.empty((G,), dtype=torch.int32, device=dev)
    gathered = torch.empty((world * G, C), device=dev) if world > 1 else None
    # A stream of torch's own (non-zero handle: handle 0 would select the library's
    # context stream, which torch events cannot see), made current for everything below.
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.synchronize()
    torch.cuda.set_stream(stream)
    st = stream.cuda_stream
    level_events = []

    # d = 64 / 128: the first level reads ReLU(W_in[tag]) directly (H0 is never written), as s2v_forward_f32 does
    first_fused = d in (64, 128) and N >= 16384

    def step(timed: bool):
        cur, nxt = ha, hbuf
        if not first_fused:
            ctx.input_proj_onehot(db.tags, w["w_n2l"], None, ha, stream=st)
        for lv in range(L):
            if timed:
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
            if lv == 0 and first_fused:
                ctx.level_first(db.row_ptr, db.col_idx, None, w["p_node_conv"], w["w_n2l"], db.tags, nxt, stream=st)
            else:
                ctx.level_lookup(db.row_ptr, db.col_idx, None, cur, w["p_node_conv"], w["w_n2l"], db.tags, nxt, stream=st)
            if timed:
                b.record(stream)
                level_events.append((a, b))
            cur, nxt = nxt, cur
        ctx.segment_sum(db.graph_ptr, cur, Y, stream=st)
        ctx.readout(Y, w["h1_weight"], w["h2_weight"], logits, None, pred, stream=st)
        if world > 1:
            dist.all_gather_into_tensor(gathered, logits)     # the final logits gather

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step(False)
    barrier()
    launches0 = ctx.launches
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        t0.record(stream)
        for _ in range(args.steps):
            step(True)
        t1.record(stream)
        barrier()
    elapsed_ms = t0.elapsed_time(t1)
    launches = ctx.launches - launches0
    level_ms = float(np.mean([a.elapsed_time(b) for a, b in level_events]))

    # ---- end to end through the host-buffer entry point: edge list -> CSR (host) -> upload -> forward -> download
    es = np.ascontiguousarray(full.edge_src, np.int32)
    ed = np.ascontiguousarray(full.edge_dst, np.int32)
    logits_h = np.empty((G, C), np.float32)
    pred_h = np.empty((G,), np.int32)

    def e2e_step(build_csr: bool):
        if build_csr:
            rc = ctx.lib.s2v_build_n2n_csr_host(N, E, es.ctypes.data, ed.ctypes.data, 0, hb.row_ptr.data_ptr(),
                                                hb.col_idx.data_ptr(), None)
            assert rc == 0
        eng.infer_host(hb, logits_h, pred_h)

    e2e_steps = max(3, min(args.steps, 50))

    def time_e2e(build_csr: bool) -> float:
        for _ in range(3):
            e2e_step(build_csr)
        barrier()
        w0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step(build_csr)
        torch.cuda.synchronize()
        return (time.perf_counter() - w0) * 1e3

    # headline e2e: what one FeedForward of the reference times -- adjacency already grouped per node
    # (host CSR here, GraphStruct lists there), uploads, forward, download
    e2e_ms = time_e2e(False)
    e2e_build_ms = time_e2e(True)      # additionally sorting a raw edge list into the CSR on the host
    assert np.array_equal(pred_h, pred.cpu().numpy()), "host-buffer path and device path disagree"

    times = torch.tensor([elapsed_ms, e2e_ms, e2e_build_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms, e2e_build_ms = (float(x) for x in times.cpu())

    if rank == 0:
        peak_gbs, peak_kind = measured_peaks()
        comp = level_bytes(N, E, d, "compulsory", "lookup")
        survey = level_bytes(N, E, d, "compulsory", "dense")
        ach = comp / (level_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": world * G * args.steps / (elapsed_ms * 1e-3), "unit": "graphs/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": elapsed_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD_TEXT[args.workload],
                       "graphs_per_gpu": G, "nodes_per_gpu": N, "edges_per_gpu": E, "parallelism": f"shard-by-graph x{world}",
                       "l2": "per-step working set (3 x [N x d] fp32, > 700 MB) exceeds the 126 MB L2; no flush needed",
                       "input_digest": full.digest()},
            "e2e": {"value": world * G * e2e_steps / (e2e_ms * 1e-3), "unit": "graphs/s",
                    "h2d_bytes_per_step": hb.nbytes(), "d2h_bytes_per_step": int(logits_h.nbytes + pred_h.nbytes),
                    "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps,
                    "includes": "s2v_infer_host_f32 on pinned host CSR + tags: uploads, forward, download of logits and predictions",
                    "from_edge_list": {"value": world * G * e2e_steps / (e2e_build_ms * 1e-3), "ms_per_step": e2e_build_ms / e2e_steps,
                                       "includes": "the same plus s2v_build_n2n_csr_host (stable sort of the raw edge list)"}},
            "gpu_launches": int(launches),
            "roofline": {"kernel": (f"s2v_level_tc_kernel (tcgen05, d={d}, X looked up from W_in by tag)" if d in (64, 128) else
                                    f"s2v_level_kernel<{d}> (X looked up from W_in by tag)"), "bound": "hbm", "achieved": ach,
                         "peak": peak_gbs, "unit": "GB/s", "frac": ach / peak_gbs, "peak_kind": peak_kind,
                         # dram__bytes_read + dram__bytes_write of one launch on this very input
                         # (the committed ncu summary of the tcgen05 level kernel); only known for the default workload
                         "traffic": (259823104 + 205300224) if args.workload == "molecules" else None,
                         "ms_per_launch": level_ms, "launches": len(level_events), "bytes_per_launch": comp,
                         "model": "compulsory (each H row once) + CSR + tags + out + W",
                         "achieved_with_dense_X_model": survey / (level_ms * 1e-3) / 1e9},
            "clocks": clocks.summary(),
        }
        if world == 1:
            base, ref_out = cpu_baseline(args, full)
            line["cpu_baseline"] = base
            n = ref_out["argmax"].shape[0]
            line["parity_vs_cpu_sample"] = {"graphs": int(n), "argmax_equal": bool(np.array_equal(ref_out["argmax"], pred_h[:n])),
                                            "max_abs_logit_diff": float(np.abs(ref_out["logits"] - logits_h[:n]).max())}
            if not args.skip_level:
                line["level_cfg2"] = level_cfg2(ctx, torch, peak_gbs, peak_kind)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_giant(args, rank: int, world: int, local_rank: int):
    """Single giant R-MAT graph, row-partitioned: 2 levels of ReLU(A*H*W), d = 128, one NCCL
    all-gather of the embedding slabs per level, pipelined against the compute."""
    import torch
    import torch.distributed as dist
    from graphnn_b200 import capi, giant

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    ctx = capi.Context(local_rank)
    d, levels, scale = 128, 2, args.scale
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.synchronize()
    torch.cuda.set_stream(stream)
    shard = giant.rmat_shard_on_device(scale, 16 << scale, rank, world, dev, seed=0)
    plan = giant.plan_hubs(shard, threshold=2048, piece=512)
    spmm_fn, segsum_fn = giant.make_gpu_hub_fns(ctx)
    g = giant.GiantGraphLevels(shard, d, rank, world, giant.make_gpu_level_fn(ctx), chunks=4, hub_plan=plan,
                               spmm_fn=spmm_fn, segsum_fn=segsum_fn)
    gen = torch.Generator(device=dev)
    gen.manual_seed(1234 + rank)
    slab0 = torch.randn((shard.rows, d), device=dev, generator=gen)
    gen.manual_seed(99)
    W = torch.randn((d, d), device=dev, generator=gen) * 0.05
    nnz_local = torch.tensor([shard.nnz], dtype=torch.int64, device=dev)
    if world > 1:
        dist.all_reduce(nnz_local)
    nnz_total = int(nnz_local.item())

    def step():
        g.set_input(slab0)
        g.run(W, levels)

    for _ in range(max(args.warmup, 3)):
        step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    launches0 = ctx.launches
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        t0.record(stream)
        for _ in range(args.steps):
            step()
        t1.record(stream)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    times = torch.tensor([t0.elapsed_time(t1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms = float(times.item())
    if rank == 0:
        peak_gbs, peak_kind = measured_peaks()
        n = 1 << scale
        per_level = 4 * (n + 1) + 4 * nnz_total + 4 * nnz_total * d + 4 * n * d + 4 * d * d   # gather model, all ranks
        sec_per_level = ms * 1e-3 / args.steps / levels
        line = {"metric": "s2v_level_edges_per_sec", "value": nnz_total * levels * args.steps / (ms * 1e-3), "unit": "edges/s",
                "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": f"giant R-MAT(0.57,0.19,0.19,0.05) scale {scale}, {16 << scale} generated edges, symmetrised + deduplicated "
                                       f"to nnz={nnz_total}, d=128, 2 levels of ReLU(A*H*W), row-partitioned x{world}",
                           "all_gather_bytes_per_gpu_per_level": g.all_gather_bytes_per_level(), "chunks": 4,
                           "hub_rows_rank0": 0 if plan is None else plan.n_hub,
                           "l2": "H (N x 128 fp32) far exceeds the 126 MB L2"},
                "gpu_launches": int(ctx.launches - launches0),
                "roofline": {"kernel": "fused level, gather model, time includes the pipelined all-gather", "bound": "hbm",
                             "achieved": per_level / world / sec_per_level / 1e9, "peak": peak_gbs, "unit": "GB/s",
                             "frac": per_level / world / sec_per_level / 1e9 / peak_gbs, "peak_kind": peak_kind, "traffic": None},
                "clocks": clocks.summary()}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="molecules", choices=["molecules", "proteins", "giant"])
    ap.add_argument("--scale", type=int, default=24, help="giant workload: log2 of the node count (26 = the full configuration)")
    ap.add_argument("--skip-level", action="store_true", help="leave out the 1M-node fused-level measurement")
    args = ap.parse_args()
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
                                  "configuration has no reference run at this size (scale-20 parity is in tests/test_giant_graph.py)"}))
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
