"""Data-parallel request router: one queue in front of one worker per GPU.

open-jev-fast serves one GPU: `_forward` (src/server.py:86-142) takes the model's lock, builds the layout, replays the graph of
the request's key and returns the scores, one request at a time (src/server.py:97). Requests share nothing, so more GPUs
means more of exactly that loop: every worker owns a `server.Scorer` (full weights, its own graph cache and stream) on its
device, and the router only decides which worker gets a request. Nothing crosses between GPUs; there is no collective.

Assignment is shortest queue by outstanding work, where the work of a request is its token count (a forward costs roughly
in proportion to its packed rows, which the token count bounds). A worker that raises on a request, or does not answer
within `timeout_s`, is taken out of rotation and everything it still held is queued again for the others; a request is
retried at most `max_retries` times and then fails with the last error. Failure handling lives on the host only: nothing here
waits on a GPU event of another worker.
"""
import concurrent.futures
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


def request_cost(request):
    """Tokens of a request = sum of its candidates' lengths (records of `Scorer.forward`, or a (seqs, groups) pair)."""
    if isinstance(request, tuple):
        return sum(len(s) for s in request[0])
    return sum(len(c) for r in request for c in r["candidates"])


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

    def stats(self):
        with self.lock:
            return dict(alive=list(self.alive), served=list(self.served), requeued=self.requeued, errors=list(self.errors))
