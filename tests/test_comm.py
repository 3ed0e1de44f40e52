"""CPU tests of the multi-GPU entry points of the C ABI (s2v_comm_*, s2v_allgather_rows_f32,
s2v_gather_logits) against a stand-in NCCL library built from tests/fake_nccl/fake_nccl.c: argument
checking, the ragged packing of the logits gather, and the mapping of failing NCCL calls (injected on
the host through FAKE_NCCL_FAIL) to S2V_ERR_COMM with NCCL's message kept.  No GPU is touched: the
communicators are created with device = -1 and the buffers are host arrays.  Each case runs in a child
process because the library resolves its NCCL once per process."""
import os
import subprocess
import sys
import textwrap

import pytest

from conftest import REPO

FAKE_DIR = os.path.join(REPO, "tests", "fake_nccl")
FAKE_SO = os.path.join(FAKE_DIR, "libfake_nccl.so")


@pytest.fixture(scope="module")
def fake_nccl():
    src = os.path.join(FAKE_DIR, "fake_nccl.c")
    if not os.path.exists(FAKE_SO) or os.path.getmtime(FAKE_SO) < os.path.getmtime(src):
        subprocess.run(["gcc", "-O1", "-shared", "-fPIC", src, "-o", FAKE_SO], check=True)
    return FAKE_SO


def run_child(body: str, env_extra: dict) -> str:
    code = textwrap.dedent("""
        import ctypes, sys, numpy as np
        sys.path.insert(0, %r)
        from graphnn_b200 import capi
        lib = capi.load_library()
    """ % REPO) + textwrap.dedent(body)
    env = dict(os.environ)
    env.update(env_extra)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    return r.stdout


def test_gather_and_allgather_through_the_c_abi(fake_nccl):
    out = run_child("""
        uid = capi.comm_unique_id()
        assert len(uid) == 128
        c = capi.Comm(-1, uid, 1, 0)
        assert lib.s2v_comm_rank(c.h) == 0 and lib.s2v_comm_world(c.h) == 1
        logits = np.arange(10, dtype=np.float32).reshape(5, 2)
        pred = np.arange(5, dtype=np.int32)
        la, pa = np.zeros((5, 2), np.float32), np.zeros(5, np.int32)
        c.gather_logits([5], logits, pred, la, pa, None)
        assert np.array_equal(la, logits) and np.array_equal(pa, pred)
        la[:] = 0
        c.gather_logits([5], logits, None, la, None, None)          # logits only
        assert np.array_equal(la, logits)
        slab = np.arange(12, dtype=np.float32).reshape(3, 4)
        full = np.zeros((3, 4), np.float32)
        c.allgather_rows(slab, full, None)
        assert np.array_equal(full, slab)
        c.allgather_rows(full, full, None)                           # in place
        # pairwise exchange with per-peer counts: with one rank, rows 1..2 of `slab` come back at row 1 of `got`
        got = np.zeros((4, 4), np.float32)
        c.exchange_rows(slab[1:], [0, 2], got, [1], [2], None)
        assert np.array_equal(got[1:3], slab[1:3]) and not got[0].any() and not got[3].any()
        c.exchange_rows(slab, [0, 0], got, [0], [0], None)           # nothing to exchange: no NCCL call
        for bad in (lambda: c.exchange_rows(slab, [2, 0], got, [0], [0], None),
                    lambda: c.exchange_rows(slab, [0, 1], got, [0], [-1], None),
                    lambda: c.exchange_rows(None, [0, 1], got, [0], [1], None)):
            try:
                bad(); raise SystemExit("no error raised")
            except capi.S2VError as e:
                assert e.status == -1, e
        # argument errors are reported before NCCL is reached
        for bad in (lambda: c.gather_logits([-1], logits, pred, la, pa, None),
                    lambda: c.gather_logits([5], logits, pred, None, None, None)):
            try:
                bad(); raise SystemExit("no error raised")
            except capi.S2VError as e:
                assert e.status == -1, e
        assert lib.s2v_comm_create_rank(-1, uid, 2, 2, ctypes.byref(ctypes.c_void_p())) == -1   # rank outside the world
        c.close()
        print("ok")
    """, {"S2V_NCCL_LIBRARY": fake_nccl})
    assert "ok" in out


@pytest.mark.parametrize("call,code,needle", [
    ("ncclGetUniqueId", 2, "unhandled system error"),
    ("ncclCommInitRank", 3, "internal error"),
    ("ncclAllGather", 5, "invalid usage"),
    ("ncclBroadcast", 6, "remote process exited"),
    ("ncclSend", 3, "internal error"),
    ("ncclRecv", 2, "unhandled system error"),
    ("ncclGroupEnd", 1, "unhandled cuda error"),
])
def test_failing_nccl_calls_become_comm_errors(fake_nccl, call, code, needle):
    out = run_child("""
        import os
        fail = os.environ["FAKE_NCCL_FAIL"].split(":")[0]
        def expect(fn):
            try:
                fn()
            except capi.S2VError as e:
                assert e.status == -8 and %r in str(e) and fail in str(e), str(e)      # S2V_ERR_COMM, NCCL's text kept
                return True
            return False
        hit = False
        if fail == "ncclGetUniqueId":
            hit = expect(capi.comm_unique_id)
        else:
            uid = bytes((i * 7 + 1) %% 256 for i in range(128))
            if fail == "ncclCommInitRank":
                hit = expect(lambda: capi.Comm(-1, uid, 1, 0))
            else:
                c = capi.Comm(-1, uid, 1, 0)
                x = np.ones((4, 2), np.float32); y = np.zeros((4, 2), np.float32)
                p = np.ones(4, np.int32); q = np.zeros(4, np.int32)
                if fail == "ncclAllGather":
                    hit = expect(lambda: c.allgather_rows(x, y, None))
                elif fail in ("ncclSend", "ncclRecv"):
                    hit = expect(lambda: c.exchange_rows(x, [0, 4], y, [0], [4], None))
                    fake = ctypes.CDLL(os.environ["S2V_NCCL_LIBRARY"])
                    assert fake.fake_nccl_group_depth() == 0
                else:
                    hit = expect(lambda: c.gather_logits([4], x, p, y, q, None))
                    # the group was closed although a call inside it failed
                    fake = ctypes.CDLL(os.environ["S2V_NCCL_LIBRARY"])
                    assert fake.fake_nccl_group_depth() == 0
                # the communicator stays usable once the injected failure is gone
                del os.environ["FAKE_NCCL_FAIL"]
                c.allgather_rows(x, y, None)
                assert np.array_equal(x, y)
        assert hit
        print("ok")
    """ % needle, {"S2V_NCCL_LIBRARY": fake_nccl, "FAKE_NCCL_FAIL": f"{call}:{code}"})
    assert "ok" in out


def test_missing_nccl_library_is_an_error_not_a_crash():
    out = run_child("""
        try:
            capi.comm_unique_id()
            raise SystemExit("no error raised")
        except capi.S2VError as e:
            assert e.status == -8 and "cannot open" in str(e), str(e)
        print("ok")
    """, {"S2V_NCCL_LIBRARY": "/nonexistent/libnccl.so.2"})
    assert "ok" in out
