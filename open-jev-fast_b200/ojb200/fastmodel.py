"""FastQwen35 — the scoring forward of a hybrid Gated-DeltaNet / gated-attention Qwen3.5-style backbone on B200.

Interface of open-jev-fast's src/fastmodel.py: `FastQwen35(core)` reads a Hugging Face Qwen3_5TextModel-shaped module
(src/fastmodel.py:72-112), `gtree_build` packs a request into a two-level prefix tree (src/fastmodel.py:321-398) and
`forward_gtree(ids, lay)` returns the final-norm hidden state of every candidate's last token (src/fastmodel.py:400-482).
Everything below that interface is different: per layer the launches are

    in-proj GEMM (tcgen05)                                        -> proj
    GDN layers : intra-chunk pass (conv+SiLU+L2norm+gates of its rows fused in) -> tree-walking state pass -> gated RMSNorm
    attention  : q/k norm + rotary -> tree attention from three key ranges per row, output gate fused
    out-proj GEMM, split-K fp32 partials -> reduce + residual (fp32 stream) + RMSNorm
    gate/up GEMM with SwiGLU in the epilogue
    down GEMM, split-K                   -> reduce + residual (fp32 stream) + RMSNorm (next layer's input norm)

with no replicated per-candidate layout, no N x N mask and no cuBLAS / Triton / SDPA call. There is no CPU fallback.
"""
import os
from types import SimpleNamespace

import torch

from . import ext as _ext
from . import layout as _layout
from . import lt_ext as _lt

K = _ext.load()
LT = _lt.load()

# Module-level switches with the names open-jev-fast's tests flip (src/fastmodel.py:45-64). Variants that differed only in
# schedule in the reference select the same kernels here.
SK_LIN_OUT = int(os.environ.get("OJ_SK_LIN_OUT", "0"))     # split-K of the GDN out-projection; 0 = choose by timing
SK_FULL_OUT = int(os.environ.get("OJ_SK_FULL_OUT", "0"))   # split-K of the attention o-projection
SK_DOWN = int(os.environ.get("OJ_SK_DOWN", "0"))           # split-K of the MLP down-projection
FATTN = int(os.environ.get("OJ_FATTN", "0"))               # query heads per CTA of the tree attention (3 or 6); 0 = by row count
FATTN_MAX = int(os.environ.get("OJ_FATTN_MAX", "1000000000"))   # kept for compatibility: the kernel serves every N
FATTN_TC = os.environ.get("OJ_FATTN_TC", "1") == "1"            # tcgen05 / TMA attention kernel (head dim 256, key-range mask)
GDN_FUSED, GDN_VER, PREP, GVA, LUT, SK2 = True, 6, "dedup", True, True, True
TREE_NATIVE = os.environ.get("OJ_TREE_NATIVE", "1") == "1"      # 0: replicated per-candidate GDN layout of the reference
# 1: conv + SiLU + L2 norm + gates inside the first Gated DeltaNet launch (same bits, one launch fewer per layer). Measured:
# 32.00 against 31.91 ms on the 539-row tree, 20.86 against 20.19 ms on the 277-row tree — the work lands on the latency chain
# of a kernel that is latency-bound already, so it is off.
FUSE_PREP = os.environ.get("OJ_FUSE_PREP", "0") == "1"

TREE_LEVELS = os.environ.get("OJ_TREE_LEVELS", "0") == "1"      # 1: state pass per tree level (3 launches), 0: one depth-first walk
# (measured on the 539-row tree: depth-first 84 us per layer for intra + state, level-parallel 88 us: the two extra launches
# and the six waves of short single-step CTAs cost more than the shorter dependency chain saves)


class _Layer(SimpleNamespace):
    """Per-layer weights. `w_gu` of the reference ([gate; up] stacked) is rebuilt on demand from the block-interleaved copy
    that the fused SwiGLU GEMM reads, instead of being stored a second time."""

    @property
    def w_gu(self):
        I2, Kd = self.w_gu_blk.shape
        b = self.w_gu_blk.view(I2 // 256, 2, 128, Kd)
        return torch.cat([b[:, 0].reshape(I2 // 2, Kd), b[:, 1].reshape(I2 // 2, Kd)], 0)


class FastQwen35(torch.nn.Module):
    def __init__(self, core, free_original=False, v2=True, fuse_l2=True, fp8=None):
        super().__init__()
        # 8-bit projections (e4m3 operands, per-row scales; README.md:131 of the reference: measured there, not shipped).
        # Off unless asked for: the scores then differ from the bf16 path by more than its tolerance.
        self.fp8 = (os.environ.get("OJ_FP8", "0") == "1") if fp8 is None else bool(fp8)
        self._q8 = {}       # data_ptr of a bf16 weight -> (e4m3 bytes, fp32 row scales)
        cfg = core.config
        self.cfg, self.core = cfg, core
        self.H, self.eps = cfg.hidden_size, cfg.rms_norm_eps
        self.layer_types = list(cfg.layer_types)
        self.embed, self.rotary = core.embed_tokens, core.rotary_emb
        # default rope type on text positions: cos / sin come from ojb_embed_rope together with the embedding rows
        self._own_rope = (getattr(self.rotary, "rope_type", None) == "default" and self.embed.weight.dtype == torch.bfloat16
                          and self.embed.weight.is_contiguous())
        self._inv_freq = self.rotary.inv_freq.detach().float().contiguous()
        self._rope_scale = float(getattr(self.rotary, "attention_scaling", 1.0))
        self.v2, self.fuse_l2 = v2, fuse_l2
        self._bufs = {}
        self._plan, self._tuned = {}, set()     # (op, M, N, K) -> kernel choice, filled by tune()
        # OJ_GEMM_FORCE="gu=8,mm=8,res=8:2" pins the lt_matmul algorithm index (and K ranges) of a projection kind for every
        # shape, like the reference's OJ_SK_* switches (src/fastmodel.py:45-64): for measurements
        self._force = {}
        for item in os.environ.get("OJ_GEMM_FORCE", "").split(","):
            if "=" in item:
                k, v = item.split("=")
                self._force[k.strip()] = tuple(int(t) for t in v.split(":")) if ":" in v else int(v)
        w1 = lambda norm: (1.0 + norm.weight.float()).contiguous()
        self.in_w1 = [w1(L.input_layernorm) for L in core.layers]
        self.post_w1 = [w1(L.post_attention_layernorm) for L in core.layers]
        self.final_w1 = w1(core.norm)
        self.L = []
        with torch.no_grad():
            for i, L in enumerate(core.layers):
                d = _Layer()
                I = L.mlp.gate_proj.weight.shape[0]
                d.fused_mlp = I % 128 == 0
                if d.fused_mlp:
                    d.w_gu_blk = LT.interleave_gate_up(L.mlp.gate_proj.weight, L.mlp.up_proj.weight)
                else:
                    d.w_gu_cat = torch.cat([L.mlp.gate_proj.weight, L.mlp.up_proj.weight], 0).contiguous()
                d.w_down = L.mlp.down_proj.weight
                d.sk_down = SK_DOWN
                if self.layer_types[i] == "linear_attention":
                    la = L.linear_attn
                    d.w_in = torch.cat([la.in_proj_qkv.weight, la.in_proj_z.weight, la.in_proj_b.weight, la.in_proj_a.weight], 0).contiguous()
                    d.w_out, d.sk_out = la.out_proj.weight, SK_LIN_OUT
                    d.convw = la.conv1d.weight.squeeze(1).contiguous()
                    d.A_log, d.dt_bias, d.normw = la.A_log.contiguous(), la.dt_bias.contiguous(), la.norm.weight.contiguous()
                    d.norm_eps = getattr(la.norm, "eps", getattr(la.norm, "variance_epsilon", self.eps))
                    d.KD, d.VD, d.HV, d.HK, d.HD = la.key_dim, la.value_dim, la.num_v_heads, la.num_k_heads, la.head_v_dim
                    if la.head_k_dim != la.head_v_dim or d.HD != 128:
                        raise RuntimeError("FastQwen35: the Gated DeltaNet kernels need key and value head dim 128")
                else:
                    sa = L.self_attn
                    d.w_in = torch.cat([sa.q_proj.weight, sa.k_proj.weight, sa.v_proj.weight], 0).contiguous()
                    d.w_out, d.sk_out = sa.o_proj.weight, SK_FULL_OUT
                    d.qw1, d.kw1 = w1(sa.q_norm), w1(sa.k_norm)
                    d.HQ, d.HKV, d.D, d.scale = cfg.num_attention_heads, cfg.num_key_value_heads, sa.head_dim, sa.scaling
                if self.fp8:
                    for w in ([d.w_gu_blk] if d.fused_mlp else [d.w_gu_cat]) + [d.w_down, d.w_in, d.w_out]:
                        self._q8[w.data_ptr()] = LT.quantize_weight_e4m3(w)
                if free_original:   # the merged copies replace the originals: release q/k/v, in_proj_* and gate/up storage
                    mods = [L.mlp.gate_proj, L.mlp.up_proj]
                    mods += [la.in_proj_qkv, la.in_proj_z, la.in_proj_b, la.in_proj_a] if self.layer_types[i] == "linear_attention" \
                        else [sa.q_proj, sa.k_proj, sa.v_proj]
                    for m in mods:
                        m.weight.data = torch.empty(0, dtype=m.weight.dtype, device=m.weight.device)
                self.L.append(d)

    # ------------------------------------------------------------------------------------------------ GEMM dispatch
    # The reference times every cuBLASLt candidate per shape (src/fastmodel.py:114-156). Here the library's cost model picks
    # kernel, tile width and K split for any shape (lt_ext.gemm_plan); `tune(M)` refines that choice for one row count by
    # timing the candidates on this model's own weights, back to back over all layers (so under the power cap and with the
    # weights coming from HBM, as in the real forward).
    def _mm(self, x, w):
        """out = x @ w^T, bf16 (src/fastmodel.py:168 _mm)."""
        q8 = self._q8.get(w.data_ptr()) if self.fp8 else None
        if q8 is not None:
            xq, sx = LT.quantize_rows_e4m3(x)
            return LT.gemm_e4m3(xq, sx, q8[0], q8[1], 0)
        return LT.lt_matmul(x, w, self._force.get("mm", self._plan.get(("mm", x.shape[0], w.shape[0], w.shape[1]), 0)))

    @staticmethod
    def _split(W, S):
        """src/fastmodel.py:186 _split — kept for callers that want the [S, K/S, N] copy; the GEMM here does not need it."""
        N, Kd = W.shape
        return W.view(N, S, Kd // S).permute(1, 2, 0).contiguous()

    def _res(self, h, y, w, S, w1, mask):
        """Output projection + residual + RMSNorm (src/fastmodel.py:196 _res): fp32 partial products over S ranges of K, then
        one kernel for partial sum + residual + norm. S = 0 lets the plan choose. The residual stream `h` is fp32 [N, H] and is
        updated in place: the partial sums are added in fp32 and the stream is never rounded (the reference rounds the sum
        and the stream to bf16 at every one of its 128 residual adds); only the norm output that feeds the next GEMM is
        bf16. Returns [h, hn] like the reference."""
        M, Kd = y.shape
        idx = 0
        q8 = self._q8.get(w.data_ptr()) if self.fp8 else None
        if q8 is not None:
            yq, sy = LT.quantize_rows_e4m3(y)
            S8 = S if S > 0 else LT.plan_splitk(M, w.shape[0], Kd // 2)      # a 128-byte k-block holds twice the elements
            return [h, K.resnorm_f32(h, None, None, LT.gemm_e4m3(yq, sy, q8[0], q8[1], 2, S8), w1, mask, self.eps)]
        if S == 0:
            idx, S = self._force.get("res", self._plan.get(("res", M, w.shape[0], Kd), (0, 0)))
            if S == 0:
                S = LT.plan_splitk(M, w.shape[0], Kd)
        return [h, K.resnorm_f32(h, None, None, LT.gemm_splitk(y, w, S, idx), w1, mask, self.eps)]

    def _mlp_in(self, hn, d):
        if d.fused_mlp and self.fp8:
            q8 = self._q8[d.w_gu_blk.data_ptr()]
            xq, sx = LT.quantize_rows_e4m3(hn)
            return LT.gemm_e4m3(xq, sx, q8[0], q8[1], 1)
        if d.fused_mlp:
            return LT.gemm_swiglu(hn, d.w_gu_blk, self._force.get("gu", self._plan.get(("gu", hn.shape[0]) + tuple(d.w_gu_blk.shape), 0)))
        return K.silu_mul(self._mm(hn, d.w_gu_cat))

    TUNE_MAX_ROWS = int(os.environ.get("OJ_TUNE_MAX_ROWS", "1024"))
    # OJ_TUNE_EXTRA="8,9": more lt_matmul algorithm indices for tune() to race (the CTA-pair kernels are not raced by default:
    # in isolation they tie with the one-CTA kernels)
    TUNE_EXTRA = [int(v) for v in os.environ.get("OJ_TUNE_EXTRA", "").split(",") if v.strip()]

    def tune(self, M, force=False, report=None):
        """Choose kernel variant (and K split) of every projection for M packed rows by timing (src/fastmodel.py:114-156
        _tune). Each candidate runs over all layers that have the shape, twice, between CUDA events. Above TUNE_MAX_ROWS the
        cost model is kept (every shape then has many units per SM and the 256-row block kernel wins throughout)."""
        if (M in self._tuned or M > self.TUNE_MAX_ROWS or self.fp8) and not force:
            return
        self._tuned.add(M)
        cache = os.environ.get("OJ_TUNE_CACHE")      # optional file that pins the choices across processes (profiling runs)
        if cache and os.path.exists(cache) and not force:
            import json
            saved = json.load(open(cache)).get(str(M))
            if saved is not None:
                for k, v in saved:
                    self._plan[tuple(k)] = tuple(v) if isinstance(v, list) else v
                return
        dev = self.L[0].w_down.device
        g = torch.Generator(device=dev).manual_seed(1234)
        rnd = lambda *shape: (torch.randn(*shape, generator=g, device=dev) * 0.5).to(torch.bfloat16)

        def clock_once(fn, layers):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for d in layers:
                fn(d)
            b.record()
            b.synchronize()
            return a.elapsed_time(b) * 1e3 / len(layers)

        def race(cands, layers):
            """cands: {key: fn(layer)}. Three interleaved rounds over all layers, best round per candidate: a candidate is not
            judged by the clock the GPU happened to run at during its turn."""
            for fn in cands.values():
                for d in layers[:2]:
                    fn(d)
            best = {k: float("inf") for k in cands}
            for _ in range(3):
                for k, fn in cands.items():
                    best[k] = min(best[k], clock_once(fn, layers))
            return best

        def groups(attr):
            out = {}
            for d in self.L:
                w = getattr(d, attr, None)
                if w is not None:
                    out.setdefault(tuple(w.shape), []).append(d)
            return out

        kernels = [1, 3] + ([7] if M <= 2048 else []) + ([10] if M > 256 and M % 256 else []) + self.TUNE_EXTRA
        for (N, Kd), layers in groups("w_in").items():
            x = rnd(M, Kd)
            res = race({i: (lambda d, i=i: LT.lt_matmul(x, d.w_in, i)) for i in kernels + [2]}, layers)
            best = min(res, key=res.get)
            self._plan[("mm", M, N, Kd)] = best
            if report is not None:
                report.append(dict(op="in-proj", M=M, N=N, K=Kd, us=res, best=best))
        for (N, Kd), layers in groups("w_gu_blk").items():
            x = rnd(M, Kd)
            res = race({i: (lambda d, i=i: LT.gemm_swiglu(x, d.w_gu_blk, i)) for i in kernels}, layers)
            best = min(res, key=res.get)
            self._plan[("gu", M, N, Kd)] = best
            if report is not None:
                report.append(dict(op="gate/up", M=M, N=N, K=Kd, us=res, best=best))
        for attr, norms in (("w_out", self.post_w1), ("w_down", self.in_w1)):
            for (N, Kd), layers in groups(attr).items():
                y, h, w1 = rnd(M, Kd), rnd(M, N).float(), norms[0]
                kb = -(-Kd // 64)
                cands = {}
                for S in (1, 2, 3, 4, 6, 8):
                    if (S - 1) * -(-kb // S) >= kb:
                        continue
                    for i in kernels:
                        cands[(i, S)] = lambda d, i=i, S=S: K.resnorm_f32(h, None, None, LT.gemm_splitk(y, getattr(d, attr), S, i),
                                                                          w1, None, self.eps)
                res = race(cands, layers)
                best = min(res, key=res.get)
                self._plan[("res", M, N, Kd)] = best
                if report is not None:
                    report.append(dict(op=attr, M=M, N=N, K=Kd, us={f"v{i} S{S}": round(t, 1) for (i, S), t in res.items()}, best=best))
        torch.cuda.synchronize(dev)
        if cache:
            import json
            allp = json.load(open(cache)) if os.path.exists(cache) else {}
            allp[str(M)] = [[list(k), list(v) if isinstance(v, tuple) else v] for k, v in self._plan.items() if k[1] == M]
            json.dump(allp, open(cache, "w"))

    gtree_build = staticmethod(_layout.gtree_build)

    # ------------------------------------------------------------------------------------------------ tree forward
    def _zero_buf(self, name, shape, device):
        """Persistent zero-initialised buffer: kernels only ever write its real rows, so padding rows stay zero."""
        key = (name,) + tuple(shape)
        b = self._bufs.get(key)
        if b is None:
            b = self._bufs[key] = torch.zeros(shape, dtype=torch.bfloat16, device=device)
        return b

    def _rope(self, x, pos):
        N = x.shape[0]
        cos, sin = self.rotary(x.view(1, N, -1), pos.view(1, 1, N).expand(3, 1, N))
        return cos.reshape(N, -1).contiguous(), sin.reshape(N, -1).contiguous()

    def _linear_tree(self, d, proj, lay):
        N = proj.shape[0]
        if TREE_NATIVE and hasattr(lay, "chunks"):
            o = self._zero_buf("gdn_o", (N, d.HV, d.HD), proj.device)
            if FUSE_PREP and not (hasattr(lay, "lsteps") and TREE_LEVELS):
                K.gdn_chunked_proj(proj, lay.hist, d.convw, d.A_log, d.dt_bias, d.KD, d.VD, d.HV, d.HK, d.HD ** -0.5, lay.chunks,
                                   lay.steps, lay.walk_ptr, lay.n_walks, None, None, o)
                return K.gated_rmsnorm(o, proj, d.normw, d.HV, d.HD, 2 * d.KD + d.VD, d.norm_eps)
            q, k, v, g, beta = K.linattn_prep_rows(proj, lay.hist, d.convw, d.A_log, d.dt_bias, d.KD, d.VD, d.HV, d.HK, d.HD)
            if hasattr(lay, "lsteps") and TREE_LEVELS:
                st = self._bufs.get(("gdn_states", lay.S, d.HV))
                if st is None:
                    st = self._bufs[("gdn_states", lay.S, d.HV)] = torch.empty(1 + lay.S, d.HV, d.HD, d.HD, dtype=torch.float32,
                                                                              device=proj.device)
                K.gdn_tree_levels(q.view(N, d.HK, d.HD), k.view(N, d.HK, d.HD), v.view(N, d.HV, d.HD), g, beta, d.HD ** -0.5,
                                  lay, o, st)
            else:
                K.gdn_chunked(q.view(N, d.HK, d.HD), k.view(N, d.HK, d.HD), v.view(N, d.HV, d.HD), g, beta, d.HD ** -0.5,
                              lay.chunks, lay.steps, lay.walk_ptr, lay.n_walks, None, None, o)
            return K.gated_rmsnorm(o, proj, d.normw, d.HV, d.HD, 2 * d.KD + d.VD, d.norm_eps)
        # the reference's route: every candidate path replicated, one sequence per candidate (src/fastmodel.py:420-454)
        S, L2 = lay.S, lay.L2
        q, k, v, g, beta = K.linattn_prep_dedup2(proj, lay.hist, lay.rep_ptr, lay.rep_pos, L2, d.convw, d.A_log, d.dt_bias,
                                                 d.KD, d.VD, d.HV, d.HK, d.HD, False)
        o_r = K.gdn_fused6(q.view(S, L2, d.HK, d.HD), k.view(S, L2, d.HK, d.HD), v.view(S, L2, d.HV, d.HD),
                           g.view(S, L2, d.HV), beta.view(S, L2, d.HV), d.HD ** -0.5)
        return K.gated_rmsnorm_inv2(o_r, lay.inv, proj, d.normw, None, d.HV, d.HD, 2 * d.KD + d.VD, d.norm_eps)

    def _attn_tree(self, d, proj, lay, cos, sin):
        N = proj.shape[0]
        G = d.HQ // d.HKV
        if FATTN_TC and hasattr(lay, "krange") and d.D == 256 and G <= 6 and N % 32 == 0:
            qt, kt, vt, gate, vt_t = K.fullattn_prep2(proj, d.qw1, d.kw1, cos, sin, 1, N, d.HQ, d.HKV, d.D, self.eps, with_vt_t=True)
            return K.fattn_tree_tc(qt, kt, vt_t, gate, lay.krange, d.scale)
        qt, kt, vt, gate = K.fullattn_prep2(proj, d.qw1, d.kw1, cos, sin, 1, N, d.HQ, d.HKV, d.D, self.eps)
        # measured: 3 heads per CTA (twice the CTAs) is faster up to a few hundred rows (17.7 vs 21.5 us at 288), 6 heads per
        # CTA (each K / V tile loaded once per kv head) above (44 vs 54 us at 544)
        want = FATTN if FATTN else (3 if N <= 384 else 6)
        gq = want if want in (1, 2, 3, 6) and G % want == 0 else 1
        if hasattr(lay, "krange"):
            return K.fattn_tree_ranges(qt, kt, vt, gate, lay.krange, d.scale, gq)
        return K.fattn_tree(qt, kt, vt, gate, None, lay.vbits, d.scale, gq)

    @torch.no_grad()
    def forward_gtree(self, ids, lay, return_all=False):
        """src/fastmodel.py:400-482: ids int64 [N] packed rows, lay from gtree_build -> bf16 [S, H] (final norm applied) of
        every candidate's last row; return_all=True gives all N rows (the scoring head gathers by itself)."""
        if self._own_rope and ids.dtype == torch.int64 and lay.pos.dtype == torch.int64:
            x, cos, sin = K.embed_rope(ids, self.embed.weight, lay.pos, self._inv_freq, self._rope_scale)
        else:                                   # other rope types: the backbone's own module (torch)
            x = self.embed(ids).contiguous()
            cos, sin = self._rope(x, lay.pos)
        lin = [t == "linear_attention" for t in self.layer_types]
        rowmask = lay.rowmask
        h = torch.empty(x.shape, dtype=torch.float32, device=x.device)        # the residual stream, fp32 throughout
        hn = K.resnorm_f32(h, x, None, None, self.in_w1[0], rowmask if lin[0] else None, self.eps)
        nl = len(self.L)
        for i, d in enumerate(self.L):
            proj = self._mm(hn, d.w_in)
            y = self._linear_tree(d, proj, lay) if lin[i] else self._attn_tree(d, proj, lay, cos, sin)
            h, hn = self._res(h, y, d.w_out, d.sk_out, self.post_w1[i], None)
            m = self._mlp_in(hn, d)
            last = i == nl - 1
            h, hn = self._res(h, m, d.w_down, d.sk_down, self.final_w1 if last else self.in_w1[i + 1],
                              None if last or not lin[i + 1] else rowmask)
        return hn if return_all else hn[lay.lastidx]

    @torch.no_grad()
    def score_gtree(self, ids, lay, head_w, head_b=None):
        """Forward + scoring head: fp32 [S, A] (src/server.py:37 `head(forward_gtree(ids, lay).float())`)."""
        hn = self.forward_gtree(ids, lay, return_all=True)
        return K.score_head(hn, lay.lastidx, head_w, head_b)

    # ------------------------------------------------------------------------------------------------ single-level tree
    def tree_layout(self, pre_ids, suf_ids, suf_mask, pad=0, dense=True, cap=None):
        """src/fastmodel.py:247-264: layout of [prefix | S suffixes] with `pad` left-padding rows in the prefix."""
        return _layout.tree_layout(pre_ids, suf_ids, suf_mask, pad, dense, cap)

    @torch.no_grad()
    def forward_tree(self, pre_ids, suf_ids, lay, fla_mode="state", return_all=False):
        """src/fastmodel.py:266-314: long shared prefix, S suffixes -> [S, H]. Both modes of the reference ("replicate" and
        "state") give the same result; here the prefix is always computed once and its Gated DeltaNet state handed to every
        suffix inside the state kernel."""
        ids = torch.zeros(lay.N32, dtype=pre_ids.dtype, device=pre_ids.device)
        ids[:lay.N] = torch.cat([pre_ids, suf_ids.reshape(-1)])
        inner = SimpleNamespace(N=lay.N32, S=lay.S, pos=lay.pos32, rowmask=lay.rowmask32, hist=lay.hist, krange=lay.krange,
                                chunks=lay.chunks, steps=lay.steps, walk_ptr=lay.walk_ptr, n_walks=1, lastidx=lay.lastidx)
        return self.forward_gtree(ids, inner, return_all)

    # ------------------------------------------------------------------------------------------------ batch forward
    @torch.no_grad()
    def forward(self, input_ids=None, attention_mask=None, capture=None, **kw):
        """src/fastmodel.py:205-241: right-padded batch [B, T] of independent sequences -> last_hidden_state [B, T, H].
        Served by the tree machinery: every sequence is a root-less path of its own."""
        B, T = input_ids.shape
        if attention_mask is None:
            attention_mask = torch.ones_like(input_ids)
        lay = _layout.batch_layout(attention_mask, input_ids.device)
        ids = torch.zeros(lay.N, dtype=input_ids.dtype, device=input_ids.device)
        ids[:B * T] = input_ids.reshape(-1)
        hn = self.forward_gtree(ids, lay, return_all=True)
        return SimpleNamespace(last_hidden_state=hn[:B * T].view(B, T, self.H))
