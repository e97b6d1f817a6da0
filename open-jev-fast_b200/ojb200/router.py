"""Data-parallel request router: one queue in front of one worker per GPU.

open-jev-fast serves one GPU: `_forward` (src/server.py:86-142) takes the model's lock, builds the layout, replays the graph of
the request's key and returns the scores, one request at a time (src/server.py:97). Requests share nothing, so more GPUs
means more of exactly that loop: every worker owns a `server.Scorer` (full weights, its own graph cache and stream) on its
device, and the router only decides which worker gets a request. Nothing crosses between GPUs; there is no collective.

Assignment is shortest queue by outstanding work, where the work of a request is an estimate of its packed rows (what the
prefix tree keeps of the candidates' tokens) plus the fixed cost of a forward: that is what a forward's time follows. A worker that raises on a request, or does not answer
within `timeout_s`, is taken out of rotation and everything it still held is queued again for the others; a request is
retried at most `max_retries` times and then fails with the last error. Failure handling lives on the host only: nothing here
waits on a GPU event of another worker.

A worker is any callable request -> result. Two forms are provided for GPU workers: a `Scorer` called from the router's
worker thread of the same process (all workers then share one Python interpreter, i.e. one interpreter lock for the layout
builds and graph launches of all GPUs), or `ProcessWorker`: the scorer lives in a child process of its own and the router's
thread only ships the request over a pipe and waits for the answer. A child that exits or stops answering looks to the
router like any other failed worker.
"""
import concurrent.futures
import multiprocessing
import queue
import threading
import time


class _Job:
    __slots__ = ("rid", "request", "future", "cost", "tries", "worker", "t_submit", "t_start", "t_done", "error")

    def __init__(self, rid, request, cost):
        self.rid, self.request, self.cost = rid, request, cost
        self.future = concurrent.futures.Future()
        self.tries, self.worker = 0, None
        self.t_submit = time.perf_counter()
        self.t_start = self.t_done = None
        self.error = None


def _common_prefix(a, b):
    """Length of the common prefix of two token lists (slices compare at C speed: 1024 tokens at a time, then bisection)."""
    n, i = min(len(a), len(b)), 0
    while i < n and a[i:i + 1024] == b[i:i + 1024]:
        i += 1024
    if i >= n:
        return n
    lo, hi = i, min(i + 1024, n)                 # a[:lo] == b[:lo]; they differ somewhere before hi
    while lo < hi:
        mid = (lo + hi + 1) // 2
        if a[lo:mid] == b[lo:mid]:
            lo = mid
        else:
            hi = mid - 1
    return lo


FIXED_COST_ROWS = 400        # a forward costs about 15 ms + 0.038 ms per packed row on a B200: the fixed part, in rows


def request_cost(request):
    """Estimated cost of a request in packed rows: the first candidate in full plus, for every further candidate, what it
    does not share with the one before it (candidates of one question are adjacent, so this is the size of the prefix tree
    unless a request interleaves its questions), plus the fixed cost of a forward. Takes the records of `Scorer.forward` or
    a (seqs, groups) pair."""
    seqs = request[0] if isinstance(request, tuple) else [c for r in request for c in r["candidates"]]
    rows, prev = FIXED_COST_ROWS, None
    for s_ in seqs:
        rows += len(s_) - (_common_prefix(prev, s_) if prev is not None else 0)
        prev = s_
    return rows


def _child_main(conn, factory, args):
    """Body of a ProcessWorker's child: build the serve function, say so, then answer requests until told to stop."""
    try:
        fn = factory(*args)
    except BaseException as e:                               # the parent must learn why there is no worker
        conn.send(("failed", repr(e)))
        return
    conn.send(("ready", None))
    while True:
        try:
            kind, payload = conn.recv()
        except EOFError:
            return
        if kind == "stop":
            return
        try:
            conn.send(("ok", fn(payload)))
        except Exception as e:
            conn.send(("err", repr(e)))


class ProcessWorker:
    """A worker in a process of its own. `factory(*args)` runs in the child (started with the `spawn` method, so it must be
    importable there) and returns the serve function; requests and results cross a pipe, so both must pickle (token lists,
    numpy arrays, numbers). Calling the object serves one request; it raises if the child reported an error, has exited, or
    the pipe broke, which is what makes the router retire it."""

    def __init__(self, factory, args=()):
        ctx = multiprocessing.get_context("spawn")
        self.conn, child = ctx.Pipe()
        self.proc = ctx.Process(target=_child_main, args=(child, factory, tuple(args)), daemon=True)
        self.proc.start()
        child.close()
        self.ready = False

    def wait_ready(self, timeout_s=None):
        """Blocks until the child has built its serve function; raises if it could not."""
        if self.ready:
            return
        if not self.conn.poll(timeout_s):
            raise TimeoutError("router: worker process did not come up in time")
        kind, payload = self.conn.recv()
        if kind != "ready":
            raise RuntimeError(f"router: worker process failed to start: {payload}")
        self.ready = True

    def __call__(self, request):
        self.wait_ready()
        self.conn.send(("req", request))
        kind, payload = self.conn.recv()                     # EOFError when the child has died
        if kind != "ok":
            raise RuntimeError(f"router: worker process: {payload}")
        return payload

    def abandon(self):
        """Called by the router when it retires this worker: the child is not asked, it is ended."""
        if self.proc.is_alive():
            self.proc.terminate()

    def close(self):
        try:
            self.conn.send(("stop", None))
        except (OSError, ValueError):
            pass
        self.proc.join(timeout=5.0)
        self.abandon()


class Router:
    """`serve_fns`: one callable per worker, request -> result (for a GPU worker: `lambda records: scorer.forward(records)`,
    which synchronises on its own device-to-host read). Each callable is only ever called from its own worker thread."""

    def __init__(self, serve_fns, timeout_s=None, max_retries=2, cost_fn=request_cost):
        self.fns = list(serve_fns)
        self.timeout_s, self.max_retries, self.cost_fn = timeout_s, max_retries, cost_fn
        self.queues = [queue.Queue() for _ in self.fns]
        self.load = [0] * len(self.fns)              # outstanding cost per worker
        self.inflight = [None] * len(self.fns)       # job a worker is serving right now
        self.alive = [True] * len(self.fns)
        self.served = [0] * len(self.fns)
        self.requeued = 0
        self.errors = []                             # (worker, repr of the error that retired it)
        self.lock = threading.Lock()
        self.stop = False
        self._rid = 0
        self.threads = [threading.Thread(target=self._work, args=(i,), daemon=True) for i in range(len(self.fns))]
        for t in self.threads:
            t.start()
        self.watchdog = None
        if timeout_s is not None:
            self.watchdog = threading.Thread(target=self._watch, daemon=True)
            self.watchdog.start()

    # ------------------------------------------------------------------------------------------------ assignment
    def _assign(self, job, exclude=None):
        """Queue `job` on the live worker with the least outstanding cost. Caller holds the lock."""
        live = [i for i in range(len(self.fns)) if self.alive[i] and i != exclude]
        if not live:
            live = [i for i in range(len(self.fns)) if self.alive[i]]
        if not live:
            job.future.set_exception(RuntimeError("router: no worker left") if job.error is None else job.error)
            return
        w = min(live, key=lambda i: (self.load[i], i))
        job.worker = w
        self.load[w] += job.cost
        self.queues[w].put(job)

    def submit(self, request):
        """Queue one request; returns a concurrent.futures.Future of its result."""
        with self.lock:
            job = _Job(self._rid, request, self.cost_fn(request))
            self._rid += 1
            self._assign(job)
        return job.future

    def map(self, requests):
        """Submit all, wait for all; results in request order."""
        futs = [self.submit(r) for r in requests]
        return [f.result() for f in futs]

    # ------------------------------------------------------------------------------------------------ workers
    def _work(self, w):
        q = self.queues[w]
        while not self.stop:
            try:
                job = q.get(timeout=0.05)
            except queue.Empty:
                continue
            with self.lock:
                if not self.alive[w] or job.future.done() or job.worker != w:
                    continue                               # re-queued elsewhere while it waited here
                self.inflight[w] = job
                job.t_start = time.perf_counter()
            try:
                res = self.fns[w](job.request)
                err = None
            except Exception as e:                         # the worker is presumed broken: its device state is unknown
                res, err = None, e
            with self.lock:
                mine = self.inflight[w] is job
                self.inflight[w] = None
                if not mine:                               # the watchdog gave up on this call and moved the job on
                    continue
                self.load[w] -= job.cost
                if err is None:
                    job.t_done = time.perf_counter()
                    self.served[w] += 1
                    if not job.future.done():
                        job.future.set_result(res)
                    continue
                self._retire(w, err)
                self._retry(job, w, err)

    def _retire(self, w, err):
        """Take worker w out of rotation and hand its queue to the others. Caller holds the lock."""
        if not self.alive[w]:
            return
        self.alive[w] = False
        self.load[w] = 0
        self.errors.append((w, repr(err)))
        abandon = getattr(self.fns[w], "abandon", None)
        if abandon is not None:
            abandon()
        pending = []
        while True:
            try:
                pending.append(self.queues[w].get_nowait())
            except queue.Empty:
                break
        for job in pending:
            if not job.future.done():
                self.requeued += 1
                self._assign(job, exclude=w)

    def _retry(self, job, w, err):
        job.tries += 1
        job.error = err
        if job.tries > self.max_retries:
            if not job.future.done():
                job.future.set_exception(err)
            return
        self.requeued += 1
        self._assign(job, exclude=w)

    def _watch(self):
        """A reply that does not come within timeout_s counts as lost: the worker is retired, the request moves on."""
        while not self.stop:
            time.sleep(min(0.05, self.timeout_s / 4))
            now = time.perf_counter()
            with self.lock:
                for w, job in enumerate(self.inflight):
                    if job is not None and job.t_start is not None and now - job.t_start > self.timeout_s:
                        self.inflight[w] = None
                        err = TimeoutError(f"router: worker {w} did not answer request {job.rid} within {self.timeout_s} s")
                        self._retire(w, err)
                        self._retry(job, w, err)

    def close(self):
        self.stop = True
        for t in self.threads:
            t.join(timeout=1.0)
        for fn in self.fns:
            if isinstance(fn, ProcessWorker):
                fn.close()

    def stats(self):
        with self.lock:
            return dict(alive=list(self.alive), served=list(self.served), requeued=self.requeued, errors=list(self.errors))
