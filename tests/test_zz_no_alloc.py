"""GPU test of s2v_forward_static_f32, the entry point for callers that cannot
allocate device memory (their memory belongs to another pool, or cudaMalloc's
device-wide synchronisation is not acceptable to them).  It must give the same
results as s2v_forward_f32 with a caller-provided workspace.  Collected last on
purpose: a failure here cannot hide a failure of any other test."""
import numpy as np
import pytest
import torch

from conftest import assert_close
from graphnn_b200 import capi, engine, synth

pytestmark = pytest.mark.gpu

SCRATCH_LIMIT = 16 << 20


def both_ways(eng, batch):
    hb = engine.build_host_batch(batch)
    db = eng.to_device(hb)
    G, N = db.num_graphs, db.num_nodes
    ref = eng.forward(db, want_embed=True)                   # existing entry point, torch-owned workspace
    eng.ctx.synchronize()
    dev = eng.device
    logits = torch.full((G, eng.num_class), float("nan"), device=dev)
    probs = torch.full((G, eng.num_class), float("nan"), device=dev)
    pred = torch.full((G,), -1, dtype=torch.int32, device=dev)
    embed = torch.full((N, eng.d), float("nan"), device=dev)
    cb = eng.ctx.make_batch(G, N, db.row_ptr, db.col_idx, None, db.graph_ptr, db.tags, None)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]               # cudaMemGetInfo: free device memory in bytes
    eng.ctx.forward_static(eng.model, cb, logits, probs, pred, embed)
    eng.ctx.synchronize()
    free_after = torch.cuda.mem_get_info()[0]
    return ref, (logits, probs, pred, embed), free_before - free_after


def check(ref, got, consumed=None, allow_setup=False):
    # Once the first call on the device has resolved the array's address (and the driver has loaded the
    # kernels), a call must leave the amount of free device memory exactly as it found it.
    if consumed is not None and not allow_setup:
        assert consumed == 0, f"the no-allocation entry point consumed {consumed} bytes of device memory"
    for name, a, b in zip(("logits", "probs", "pred", "embed"), ref, got):
        a, b = a.cpu().numpy(), b.cpu().numpy()
        if name == "pred":
            assert np.array_equal(a, b)
        else:
            assert_close(b, a, f"static-scratch {name} vs s2v_forward_f32")


def test_static_scratch_forward_matches_twice_in_a_row():
    first = synth.mutag_like(seed=0)
    eng = engine.S2VInference(first.weights, first.levels)
    assert eng.ctx.workspace_bytes(first.num_nodes, first.num_graphs, first.d) <= SCRATCH_LIMIT
    check(*both_ways(eng, first), allow_setup=True)
    # second call in a row: the array still holds the first call's data, and this batch is
    # larger (different node count), so stale contents would show up as wrong numbers
    second = synth.molecule_like(200, 10, 28, 7, 64, 3, 128, 2, 0.1, "uniform", seed=9)
    second.weights = first.weights
    assert eng.ctx.workspace_bytes(second.num_nodes, second.num_graphs, second.d) <= SCRATCH_LIMIT
    check(*both_ways(eng, second))
    # and the first batch again
    check(*both_ways(eng, first))


def test_static_scratch_rejects_batches_beyond_its_limit():
    b = synth.molecules_16k(seed=0, num_graphs=2048)          # needs ~ 94 MB of scratch
    eng = engine.S2VInference(b.weights, b.levels)
    assert eng.ctx.workspace_bytes(b.num_nodes, b.num_graphs, b.d) > SCRATCH_LIMIT
    db = eng.to_device(engine.build_host_batch(b))
    logits = torch.empty((db.num_graphs, 2), device=eng.device)
    cb = eng.ctx.make_batch(db.num_graphs, db.num_nodes, db.row_ptr, db.col_idx, None, db.graph_ptr, db.tags, None)
    with pytest.raises(capi.S2VError) as e:
        eng.ctx.forward_static(eng.model, cb, logits)
    assert e.value.status == -5 and "built-in array" in str(e.value)
