"""Host-side request router (ojb200/router.py): shortest-queue assignment and re-queueing after a failed or silent worker.
Failures are made on the host only — a worker that raises, one that never answers — and no GPU is involved."""
import threading
import time

import pytest

from ojb200 import router as R


def _req(n_tokens, tag):
    return [{"kind": "score", "candidates": [[tag] * n_tokens]}]


def test_requests_go_to_the_least_loaded_worker_and_all_complete():
    seen = [[], []]
    gate = threading.Event()

    def mk(w):
        def serve(records):
            gate.wait(2.0)
            seen[w].append(records[0]["candidates"][0][0])
            return ("w%d" % w, records[0]["candidates"][0][0])
        return serve

    rt = R.Router([mk(0), mk(1)])
    try:
        # costs 2400, 410, 410, 410 (rows + the fixed cost of a forward): the heavy one goes to worker 0, the three light
        # ones pile up on worker 1 (410, 820, 1230 < 2400)
        futs = [rt.submit(_req(2000, 0))] + [rt.submit(_req(10, i)) for i in (1, 2, 3)]
        gate.set()
        res = [f.result(timeout=5) for f in futs]
    finally:
        rt.close()
    assert [r[1] for r in res] == [0, 1, 2, 3]
    assert res[0][0] == "w0" and {r[0] for r in res[1:]} == {"w1"}
    assert rt.stats()["served"] == [1, 3] and rt.stats()["requeued"] == 0


def test_a_worker_that_raises_is_retired_and_its_requests_are_served_by_the_others():
    calls = {"bad": 0}

    def bad(records):
        calls["bad"] += 1
        raise RuntimeError("device-side wait ran out")

    def good(records):
        time.sleep(0.01)
        return records[0]["candidates"][0][0]

    rt = R.Router([bad, good, good])
    try:
        res = rt.map([_req(8, i) for i in range(12)])
    finally:
        rt.close()
    assert res == list(range(12))                       # every request answered exactly once, in order
    st = rt.stats()
    assert st["alive"] == [False, True, True] and calls["bad"] == 1 and st["requeued"] >= 1
    assert sum(st["served"]) == 12 and st["served"][0] == 0


def test_a_reply_that_never_comes_is_detected_and_the_request_moves_on():
    never = threading.Event()

    def silent(records):
        never.wait(10.0)                                # the reply is dropped
        return "late"

    def good(records):
        return records[0]["candidates"][0][0]

    rt = R.Router([silent, good], timeout_s=0.2)
    try:
        t0 = time.perf_counter()
        res = rt.map([_req(8, i) for i in range(6)])
        dt = time.perf_counter() - t0
    finally:
        never.set()
        rt.close()
    assert res == list(range(6)) and dt < 5.0
    st = rt.stats()
    assert st["alive"] == [False, True] and st["requeued"] >= 1


def test_a_request_fails_with_the_workers_error_when_every_retry_fails():
    def bad(records):
        raise ValueError("bad request")

    rt = R.Router([bad, bad, bad], max_retries=1)
    try:
        f = rt.submit(_req(4, 0))
        with pytest.raises((ValueError, RuntimeError)):
            f.result(timeout=5)
    finally:
        rt.close()


def test_cost_of_a_request_is_the_size_of_its_prefix_tree():
    root = list(range(3000))
    seqs = [root + [7, 8, 9, i] for i in range(5)]               # 3000 shared + 3 shared stem tokens + one own token each
    assert R.request_cost((seqs, [0] * 5)) == R.FIXED_COST_ROWS + 3004 + 4
    recs = [{"kind": "score", "candidates": seqs[:2]}, {"kind": "score", "candidates": seqs[2:]}]
    assert R.request_cost(recs) == R.request_cost((seqs, [0] * 5))
    assert R._common_prefix([], [1]) == 0 and R._common_prefix([1, 2], [1, 2]) == 2 and R._common_prefix(root, root[:2047] + [0]) == 2047


# ---- workers in processes of their own (the factories below run in the spawned children, which import this module)
def _echo_factory(tag, die_after):
    import os
    served = {"n": 0}

    def serve(records):
        served["n"] += 1
        if die_after and served["n"] > die_after:
            os._exit(3)                                     # the process is gone in the middle of a request
        return (tag, records[0]["candidates"][0][0])
    return serve


def _broken_factory():
    raise RuntimeError("no device")


def test_a_worker_process_that_dies_is_retired_and_its_requests_are_served_by_the_others():
    workers = [R.ProcessWorker(_echo_factory, ("a", 2)), R.ProcessWorker(_echo_factory, ("b", 0))]
    for w in workers:
        w.wait_ready(60)
    rt = R.Router(workers)
    try:
        res = rt.map([_req(8, i) for i in range(10)])
        st = rt.stats()
    finally:
        rt.close()
    assert [r[1] for r in res] == list(range(10))       # every request answered once, in order
    assert st["alive"] == [False, True] and st["requeued"] >= 1 and st["served"][0] == 2 and sum(st["served"]) == 10
    assert "EOFError" in st["errors"][0][1] or "Connection" in st["errors"][0][1]
    assert not workers[0].proc.is_alive()


def test_a_worker_process_that_cannot_start_reports_why():
    w = R.ProcessWorker(_broken_factory)
    with pytest.raises(RuntimeError, match="no device"):
        w.wait_ready(60)
    w.close()
