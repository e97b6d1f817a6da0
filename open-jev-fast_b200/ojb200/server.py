"""Serving shim of the scoring forward: per-shape CUDA graphs, request -> scores, data-parallel sharding of requests.

Follows open-jev-fast's src/server.py: `Entry` (src/server.py:32-49) owns static input buffers and one CUDA graph per
key (N, S, L2); `Scorer.forward(records)` keeps the contract of `_forward(records)` (src/server.py:86-142): one score per
candidate, `noul` questions answered as [0, score], an LRU of at most MAX_GRAPHS graphs, one access-log record per request.
What is outside this repository's scope (HTTP, tokenizer, chat template: the un-vendored `jev` package) is replaced by
token-id lists: a record is {"kind": "noul" | "choice" | "score", "candidates": [[token ids], ...]}. `prompt_ids` is the
tokenisation step of src/server.py:72-85 for callers that bring a Hugging Face tokenizer: the chat template is rendered
once around a marker, split into a fixed head and tail, and all prompts of a request go through one batched encode.
"""
import collections
import json
import os
import threading
import time

import torch

from . import _lib
from . import layout as _layout

NB, PB = int(os.environ.get("ROW_BUCKET", "32")), int(os.environ.get("PATH_BUCKET", "16"))
PRE_B, SUF_B = int(os.environ.get("PRE_BUCKET", "64")), int(os.environ.get("SUF_BUCKET", "16"))
REP_MAX = int(os.environ.get("REP_MAX", "4096"))
STATE_PATH = os.environ.get("OJ_STATE_PATH", "0") == "1"
MAX_GRAPHS = int(os.environ.get("MAX_GRAPHS", "512"))
USE_GRAPH = os.environ.get("USE_GRAPH", "1") == "1"
CAPTURE_AFTER = int(os.environ.get("CAPTURE_AFTER", "1"))


_TEMPLATE_PARTS = {}
_MARK = "\x00OJB\x00"


def prompt_ids(tok, prompts):
    """Token ids of every prompt wrapped in the tokenizer's chat template (one user message, generation prompt, thinking
    off), as src/server.py:72-85 does: the template text is rendered once per tokenizer around a marker and cut at the
    marker; each prompt is then head + prompt + tail and the whole list is encoded by one call of the backend tokenizer.
    A template in which the marker does not appear exactly once falls back to rendering and encoding prompt by prompt."""
    parts = _TEMPLATE_PARTS.get(id(tok))
    if parts is None:
        text = tok.apply_chat_template([{"role": "user", "content": _MARK}], tokenize=False, add_generation_prompt=True,
                                       enable_thinking=False)
        parts = _TEMPLATE_PARTS[id(tok)] = tuple(text.split(_MARK)) if text.count(_MARK) == 1 else ()
    if not parts:
        return [tok(tok.apply_chat_template([{"role": "user", "content": p}], tokenize=False, add_generation_prompt=True,
                                            enable_thinking=False))["input_ids"] for p in prompts]
    enc = tok.backend_tokenizer.encode_batch([parts[0] + p + parts[1] for p in prompts], add_special_tokens=True)
    return [list(e.ids) for e in enc]


def token_records(records, tok, candidate_prompts):
    """Text records -> the token-id records `Scorer.forward` takes. `candidate_prompts(record)` returns the prompt of every
    candidate of a record (the un-vendored jev.candidate_prompts in the reference, src/server.py:91); all prompts of the
    request are tokenised by one `prompt_ids` call."""
    prompts, counts = [], []
    for r in records:
        c = candidate_prompts(r)
        counts.append(len(c))
        prompts += c
    ids = prompt_ids(tok, prompts)
    out, off = [], 0
    for r, c in zip(records, counts):
        out.append({"kind": r.get("kind", "score"), "candidates": ids[off:off + c]})
        off += c
    return out


class Entry:
    """Static buffers + CUDA graph of `score_gtree` for one key (N, S, L2). The tree structure lives in the index tables,
    so every request with the same key replays the same graph after three host-to-device copies. Capture runs in
    thread-local error mode: other threads of the process (the workers of other GPUs behind the router) may allocate and
    launch on their own devices while this one captures."""

    def __init__(self, scorer, dims, host_bufs, capture=True):
        fast = scorer.fast
        dev = scorer.device
        self.scorer = scorer
        self.dims = dict(dims)
        self.g64, self.g32, self.ge = (b.to(dev) for b in host_bufs)
        f = _layout.field_views(dims, self.g64, self.g32, self.ge)
        self.ids = f.pop("ids")
        self.lay = _layout.SimpleNamespace(N=dims["N"], S=dims["S"], L2=dims["L2"], key=(dims["N"], dims["S"], dims["L2"]), **f)
        self.lay.walk_ptr, self.lay.n_walks = self.lay.meta[6:8], 1
        self._body = lambda: fast.score_gtree(self.ids, self.lay, scorer.head_w, scorer.head_b)
        self.g, self.out, self.launches, self.seen = None, None, 0, 0
        if capture:
            self.capture()

    def capture(self):
        """Tune the GEMM choices for this row count, warm up, and (unless the scorer runs without graphs) capture the graph.
        A scorer with capture_after > 1 calls this only when a key comes back; until then the entry runs eagerly with the
        cost model's kernel choices."""
        scorer, dev, body = self.scorer, self.scorer.device, self._body
        scorer.fast.tune(self.dims["N"])    # per-shape choice of GEMM kernel and K split, timed on the model's own weights
        st = torch.cuda.Stream(device=dev)
        st.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(st):
            for _ in range(1):          # warm-up (allocations of every shape happen here, outside the capture)
                body()
        torch.cuda.current_stream(dev).wait_stream(st)
        torch.cuda.synchronize(dev)
        n0 = _lib.launch_count()
        if scorer.use_graph:
            self.g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.g, pool=scorer.pool, stream=scorer.capture_stream, capture_error_mode="thread_local"):
                self.out = body()
            torch.cuda.synchronize(dev)
        else:
            self.out = body()
        self.launches = _lib.launch_count() - n0

    def run(self, host_bufs):
        """Upload one request's tables (pinned host buffers) and replay. Returns the static fp32 [S, A] output."""
        self.g64.copy_(host_bufs[0], non_blocking=True)
        n32 = self.dims.get("n32_used", self.g32.numel())     # without the visibility words when they were not built
        self.g32[:n32].copy_(host_bufs[1][:n32], non_blocking=True)
        self.ge.copy_(host_bufs[2], non_blocking=True)
        return self.replay()

    def replay(self):
        self.seen += 1
        if self.g is not None:
            self.g.replay()
        else:
            n0 = _lib.launch_count()
            self.out = self._body()
            self.launches = _lib.launch_count() - n0
        return self.out


class EntryState:
    """Single-level prefix tree with prefix-state hand-off (long shared context, one question): src/server.py:50-70. Static
    prefix / suffix / mask buffers and one CUDA graph per key (Lp bucket, S, Ls bucket); `run` rebuilds the layout on the
    host (tables padded to the key's capacity) and copies it over the static tables."""
    FIELDS = ("pos32", "rowmask32", "hist", "krange", "chunks", "steps", "walk_ptr", "lastidx")

    def __init__(self, scorer, Lpb, S, Lsb):
        from . import ext as K
        fast, dev = scorer.fast, scorer.device
        self.pre = torch.zeros(Lpb, dtype=torch.long, device=dev)
        self.suf = torch.zeros(S, Lsb, dtype=torch.long, device=dev)
        self.msk = torch.ones(S, Lsb, dtype=torch.long, device=dev)
        self.cap = -(-Lpb // 64) + S * -(-Lsb // 64)
        self.lay = fast.tree_layout(self.pre, self.suf, self.msk, pad=0, dense=False, cap=self.cap)
        fast.tune(self.lay.N32)
        body = lambda: K.score_head(fast.forward_tree(self.pre, self.suf, self.lay, "state", return_all=True), self.lay.lastidx,
                                    scorer.head_w, scorer.head_b)
        st = torch.cuda.Stream(device=dev)
        st.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(st):
            for _ in range(2):
                body()
        torch.cuda.current_stream(dev).wait_stream(st)
        torch.cuda.synchronize(dev)
        self.g = None
        n0 = _lib.launch_count()
        if scorer.use_graph:
            self.g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.g, pool=scorer.pool, stream=scorer.capture_stream, capture_error_mode="thread_local"):
                self.out = body()
            torch.cuda.synchronize(dev)
        else:
            self.out = body()
        self.launches = _lib.launch_count() - n0
        self._body, self._fast = body, fast

    def run(self, pre, suf, msk, pad):
        self.pre.copy_(pre, non_blocking=True)
        self.suf.copy_(suf, non_blocking=True)
        self.msk.copy_(msk, non_blocking=True)
        L = self._fast.tree_layout(pre, suf, msk, pad=pad, dense=False, cap=self.cap)          # host tensors
        for name in self.FIELDS:
            getattr(self.lay, name).copy_(getattr(L, name), non_blocking=True)
        if self.g is not None:
            self.g.replay()
        else:
            self.out = self._body()
        return self.out


class PackedEntry:
    """Static tables + CUDA graph of `score_gtree` for several requests packed into one forward (layout.pack_requests).
    Keyed by the tuple of the requests' (N, S, L2) keys; replay = one small copy per table, then the graph."""

    def __init__(self, scorer, ids, lay):
        fast, dev = scorer.fast, scorer.device
        self.ids, self.lay = ids, lay
        self.tables = dict(ids=ids, **{k: getattr(lay, k) for k in ("pos", "rowmask", "hist", "krange", "chunks", "steps", "walk_ptr",
                                                                   "lastidx")})
        fast.tune(lay.N)
        body = lambda: fast.score_gtree(self.ids, self.lay, scorer.head_w, scorer.head_b)
        st = torch.cuda.Stream(device=dev)
        st.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(st):
            for _ in range(2):
                body()
        torch.cuda.current_stream(dev).wait_stream(st)
        torch.cuda.synchronize(dev)
        self.g = None
        n0 = _lib.launch_count()
        if scorer.use_graph:
            self.g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.g, pool=scorer.pool, stream=scorer.capture_stream, capture_error_mode="thread_local"):
                self.out = body()
            torch.cuda.synchronize(dev)
        else:
            self.out = body()
        self.launches = _lib.launch_count() - n0
        self._body = body

    def run(self, host):
        for k, t in self.tables.items():
            t.copy_(host[k], non_blocking=True)
        if self.g is not None:
            self.g.replay()
        else:
            self.out = self._body()
        return self.out


class Scorer:
    """One GPU's worth of the service: model + head + graph cache + lock (one request at a time per GPU, src/server.py:97)."""

    def __init__(self, fast, head_w, head_b=None, pad_id=0, device=None, use_graph=USE_GRAPH, max_graphs=MAX_GRAPHS,
                 access_log=None, capture_after=CAPTURE_AFTER):
        """capture_after = 1 (the reference's behaviour, src/server.py:118-124): a key's graph is captured the first time the
        key is seen. capture_after = n > 1: the first n - 1 requests of a key run eagerly (no tuning, no warm-up, no capture:
        about the time of one forward instead of three forwards plus the instantiation of a 610-node graph) and the graph is
        captured when the key comes back for the n-th time — for request streams in which most shapes never repeat."""
        self.fast, self.head_w, self.head_b, self.pad_id = fast, head_w, head_b, pad_id
        self.capture_after = max(1, int(capture_after))
        self.device = torch.device(device if device is not None else head_w.device)
        self.use_graph, self.max_graphs = use_graph, max_graphs
        self.graphs = collections.OrderedDict()
        self.pool = torch.cuda.graph_pool_handle() if use_graph else None
        # torch keeps ONE default capture stream per process, on the device that captured first: a scorer on another GPU
        # must bring its own, or its capture would run on the first GPU's stream
        self.capture_stream = torch.cuda.Stream(device=self.device) if use_graph else None
        self.lock = threading.Lock()
        self.nreq = 0
        self.log = open(access_log, "a", buffering=1 << 16) if access_log else None
        self.last = {}

    def entry_for(self, dims, host_bufs):
        key = (dims["N"], dims["S"], dims["L2"])
        ent = self.graphs.get(key)
        captured = False
        if ent is None:
            captured = self.capture_after <= 1
            ent = self.graphs[key] = Entry(self, dims, host_bufs, capture=captured)
            while len(self.graphs) > self.max_graphs:
                self.graphs.popitem(last=False)
        else:
            self.graphs.move_to_end(key)
            if ent.g is None and self.use_graph and ent.seen + 1 >= self.capture_after:
                ent.capture()
                captured = True
        return ent, captured

    def score_tokens(self, seqs, groups, with_info=False):
        """Candidate token lists + question index per candidate -> fp32 [S, A] scores on the GPU (not synchronised; a copy
        owned by the caller). with_info=True also returns this call's record (key, rows, build time, ...), which under
        concurrent callers is not necessarily `self.last`."""
        t0 = time.perf_counter()
        # the kernels read key ranges, not the N x N/32 visibility words: those are neither built nor uploaded
        dims, b64, b32, e32 = _layout.gtree_host(seqs, groups, self.pad_id, NB, PB, pin=True, vbits=False)
        t1 = time.perf_counter()
        with self.lock, torch.cuda.device(self.device):
            ent, captured = self.entry_for(dims, (b64, b32, e32))
            # the graph writes into one static buffer per key: take a private copy before the lock is released, or a second
            # thread with the same key could overwrite it before this caller has read it (src/server.py:129 clones, too)
            out = ent.run((b64, b32, e32)).clone()
            info = self.last = dict(build_ms=(t1 - t0) * 1e3, captured=captured, key=ent.lay.key, rows=dims["Nreal"],
                                    h2d_bytes=b64.numel() * 8 + dims["n32_used"] * 4 + e32.numel() * 4, launches=ent.launches)
        if with_info:
            return out, info
        return out

    def score_state(self, seqs, with_info=False):
        """The reference's route for one question over a long shared context (src/server.py:100-115): the common prefix of
        the candidates is cut off (left-padded to a bucket), the rest of each candidate is one suffix row block. Returns
        fp32 [S, A] (GPU, not synchronised). The general tree route (score_tokens) serves the same requests; this one keeps
        the reference's key (Lp bucket, S, Ls bucket) and its `tree_layout` / `forward_tree` entry points."""
        t0 = time.perf_counter()
        mn = min(len(q) for q in seqs)
        Lp = 0
        while Lp < mn - 1 and all(q[Lp] == seqs[0][Lp] for q in seqs):
            Lp += 1
        S = len(seqs)
        Ls = max(len(q) - Lp for q in seqs)
        ceil_ = lambda x, b: -(-x // b) * b
        Lpb, Lsb = ceil_(Lp, PRE_B), ceil_(Ls, SUF_B)
        pad = Lpb - Lp
        pre = torch.tensor([self.pad_id] * pad + list(seqs[0][:Lp]), dtype=torch.long)
        suf = torch.full((S, Lsb), self.pad_id, dtype=torch.long)
        msk = torch.zeros(S, Lsb, dtype=torch.long)
        for i, q in enumerate(seqs):
            suf[i, :len(q) - Lp] = torch.tensor(q[Lp:])
            msk[i, :len(q) - Lp] = 1
        key = ("state", Lpb, S, Lsb)
        t1 = time.perf_counter()
        with self.lock, torch.cuda.device(self.device):
            ent = self.graphs.get(key)
            captured = ent is None
            if captured:
                ent = self.graphs[key] = EntryState(self, Lpb, S, Lsb)
                while len(self.graphs) > self.max_graphs:
                    self.graphs.popitem(last=False)
            else:
                self.graphs.move_to_end(key)
            out = ent.run(pre, suf, msk, pad).clone()
            info = self.last = dict(build_ms=(t1 - t0) * 1e3, captured=captured, key=key,
                                    rows=Lp + sum(len(q) - Lp for q in seqs), h2d_bytes=0, launches=ent.launches)
        if with_info:
            return out, info
        return out

    def score_packed(self, requests):
        """Several requests in one forward (raises the row count of every GEMM; not in the reference, which scores one
        request at a time). requests = list of (seqs, groups); returns one fp32 [S_r, A] tensor per request (GPU, not
        synchronised). The requests of later calls with the same keys in the same order reuse the captured graph."""
        t0 = time.perf_counter()
        ids, lay, host = _layout.pack_requests(requests, self.pad_id, NB, PB, dev="cpu", pin=True)
        t1 = time.perf_counter()
        key = ("packed",) + lay.key
        with self.lock, torch.cuda.device(self.device):
            ent = self.graphs.get(key)
            captured = ent is None
            if captured:
                dlay = _layout.SimpleNamespace(**{k: (v.to(self.device) if torch.is_tensor(v) else v) for k, v in vars(lay).items()})
                ent = self.graphs[key] = PackedEntry(self, ids.to(self.device), dlay)
                while len(self.graphs) > self.max_graphs:
                    self.graphs.popitem(last=False)
            else:
                self.graphs.move_to_end(key)
            out = ent.run(host).clone()
            self.last = dict(build_ms=(t1 - t0) * 1e3, captured=captured, key=key, rows=lay.N,
                             h2d_bytes=sum(v.numel() * v.element_size() for v in host.values()), launches=ent.launches)
        return list(out.split(lay.counts))

    def forward(self, records):
        """src/server.py:86-142 on token ids: list of per-record score tensors (CPU, fp32)."""
        t0 = time.perf_counter()
        seqs, groups, counts = [], [], []
        for ri, r in enumerate(records):
            c = r["candidates"]
            counts.append(len(c))
            seqs += c
            groups += [ri] * len(c)
        Lp = 0
        if STATE_PATH and len(records) == 1 and len(seqs) > 1:
            mn = min(len(q) for q in seqs)
            while Lp < mn - 1 and all(q[Lp] == seqs[0][Lp] for q in seqs):
                Lp += 1
        if STATE_PATH and len(records) == 1 and (len(seqs) - 1) * Lp > REP_MAX:        # src/server.py:102
            scores, info = self.score_state(seqs, with_info=True)
        else:
            scores, info = self.score_tokens(seqs, groups, with_info=True)
        scores = scores.cpu()                                   # device-to-host read = the synchronisation point
        _lib.check_status(self.device)
        t1 = time.perf_counter()
        with self.lock:
            self.nreq += 1
            nreq = self.nreq
        if self.log:
            rec = dict(ts=time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime()), req=nreq, path="state" if info["key"][0] == "state" else "tree2", gpu=self.device.index,
                       questions=len(records), candidates=len(seqs), tokens=sum(map(len, seqs)), rows=info["rows"],
                       key=info["key"], captured=int(info["captured"]), build_ms=round(info["build_ms"], 3),
                       ms=round((t1 - t0) * 1e3, 3))
            self.log.write(json.dumps(rec) + "\n")
        out, off = [], 0
        for r, c in zip(records, counts):
            v = scores[off:off + c]
            if r.get("kind") == "noul":
                v = torch.stack([torch.zeros_like(v[0]), v[0]])
            out.append(v)
            off += c
        return out


def shard_requests(n_requests, rank, world):
    """Data-parallel split: request i goes to rank i % world (requests are independent; no collective on this path)."""
    return list(range(rank, n_requests, world))
