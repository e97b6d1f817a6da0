/* ojb200 — C ABI of the B200-native prefix-tree scoring forward.
 *
 * Every entry point takes plain device (or, where stated, host) pointers and sizes, launches on the given CUDA
 * stream (a cudaStream_t passed as void*), never synchronises, never allocates and never reads results back, so each
 * call can be captured into a CUDA graph. Exceptions, stated at their declarations: the two measurement hooks
 * (ojb_gemm_set_trace, ojb_gdn_set_trace) change process-wide state and the second synchronises; the first call of
 * ojb_gdn_chunked_static on a device does a one-time look-up. Kernel attributes and the SM count are cached per device, so
 * one process may drive several GPUs (make each call with its device current). Return value: OJB_OK or a negative OJB_ERR_* code. Kernels with device-side
 * waits additionally take `status`, a device int32 that stays 0 unless a bounded wait ran out.
 *
 * Each declaration names the interface of lyuyiqi/open-jev-fast that it stands in for (path inside that project).
 * Tensors are row-major and contiguous; "bf16" is __nv_bfloat16; shapes are written [rows, cols].
 */
#ifndef OJB200_H_
#define OJB200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OJB_OK 0
#define OJB_ERR_ARG (-1)      /* shape / alignment / null-pointer precondition violated */
#define OJB_ERR_LAUNCH (-2)   /* CUDA reported a launch or API failure */
#define OJB_ERR_DRIVER (-3)   /* the tensor-map encoder of the CUDA driver could not be obtained */
#define OJB_ERR_LIMIT (-4)    /* size beyond a documented maximum */

/* device-side status codes written into `status` */
#define OJB_DEV_WAIT_TIMEOUT 1

typedef void* ojb_stream_t;

/* Library/ABI version (checked by the Python shim). */
int ojb_abi_version(void);

/* ------------------------------------------------------------------------------------------------------------------
 * GEMM — replaces src/lt.cpp:43 lt_matmul / src/fastmodel.py:168 _mm (cuBLASLt) and src/fastmodel.py:158 _skmm
 * (torch.bmm split-K partials). out[M,N] = x[M,K] · w[N,K]^T, bf16 operands, fp32 accumulation in tensor memory.
 * Requirements: K % 8 == 0, x / w / out 16-byte aligned. variant: 0 = the library chooses (cost model, see ojb_gemm_plan);
 * 1 / 2 = 128-row tile kernel with 128x256 / 128x128 tiles; 3 = 256-row block kernel, automatic w-tile width; 4 = that
 * kernel with all rows of x in swapped-operand units (M <= 2048); a multiple of 16 in [16, 256] = that kernel with this
 * w-tile width; 5 = CTA-pair kernel (tcgen05.mma.cta_group::2) with automatic width; 6 = CTA-pair kernel with all rows of
 * x in swapped-operand units (any M: one pass over w per 512 rows of x, up to 512 accumulator columns per unit);
 * 512 + a multiple of 16 in [16, 256] = the pair kernel with that width; 7 = the block kernel with all but the last full
 * 256-row block of x in block units and the remaining 257..511 rows in two swapped-operand chunks that fit them exactly.
 * ------------------------------------------------------------------------------------------------------------------ */
int ojb_gemm_bf16(const void* x, const void* w, void* out, int64_t M, int64_t N, int64_t K, int variant,
                  int32_t* status, ojb_stream_t stream);

/* Same GEMM with the SwiGLU of src/kernels.cu:1304 silu_mul_lut fused into the epilogue. `w_blk` is the gate/up weight
 * re-laid in blocks of 256 rows: rows [256b, 256b+128) = gate rows [128b, 128b+128), rows [256b+128, 256b+256) = the
 * matching up rows. N = 2*I must be a multiple of 256. out[M, I] = bf16(silu(g) * u) on the fp32 accumulators g, u (the
 * reference rounds g, u and silu(g) to bf16 first; those three roundings are dropped here); the SiLU uses the approximate
 * exponential and reciprocal of the device (about 2 ulp in fp32 before the bf16 rounding). The CTA-pair kernel
 * with block units (variant 5) reads a different interleave: blocks of 64 gate rows followed by their 64 up rows; with all
 * rows swapped (variant 6) it reads the layout above. */
int ojb_gemm_bf16_swiglu(const void* x, const void* w_blk, void* out, int64_t M, int64_t N, int64_t K,
                         int32_t* status, ojb_stream_t stream);
/* The same with the kernel variant forced (0, 1, 3, 4, 5, 6 or 7 as for ojb_gemm_bf16); for tuning. */
int ojb_gemm_bf16_swiglu_v(const void* x, const void* w_blk, void* out, int64_t M, int64_t N, int64_t K, int variant,
                           int32_t* status, ojb_stream_t stream);

/* Split-K partial products, fp32: parts[s, M, N] = x[:, range s] · w[:, range s]^T, S = splits in [1, 16]; range s covers
 * k-blocks (64 columns) [s*c, min((s+1)*c, ceil(K/64))) with c = ceil(ceil(K/64)/S); no range may be empty. Replaces src/fastmodel.py:158-166 (_skmm) — note that `w` stays [N, K] (K-major); the
 * pre-split [S, K/S, N] copy of src/fastmodel.py:186 (_split) is not needed. */
int ojb_gemm_bf16_splitk(const void* x, const void* w, float* parts, int64_t M, int64_t N, int64_t K, int splits,
                         int variant, int32_t* status, ojb_stream_t stream);

/* 8-bit variant of the three GEMM forms (the FP8 path the reference measured, README.md:131 / bench/logs/peak_fp8_bench.log,
 * and did not ship): operands are e4m3 bytes with one fp32 scale per row, out = (xq · wq^T) * sx[m] * sw[n], fp32
 * accumulation in tensor memory (tcgen05.mma.kind::f8f6f4, 256-row block kernel). kind 0: out = bf16 [M, N]; kind 1:
 * SwiGLU as in ojb_gemm_bf16_swiglu (wq = the re-laid gate/up weight, sw in the same row order, N % 256 == 0), out = bf16
 * [M, N/2]; kind 2: fp32 partials [splits, M, N] over K ranges of whole 128-column k-blocks. K % 16 == 0; splits = 1
 * unless kind 2. Off by default in the Python layer (OJ_FP8=1): scores move by more than the bf16 tolerance. */
int ojb_gemm_e4m3(const void* xq, const float* sx, const void* wq, const float* sw, void* out, int64_t M, int64_t N, int64_t K,
                  int32_t kind, int32_t splits, int32_t* status, ojb_stream_t stream);

/* Per-row e4m3 quantisation of a bf16 matrix [rows, K] (K % 8 == 0) for ojb_gemm_e4m3: scale[m] = max|x[m,:]| / 448 (1 for
 * an all-zero row), q[m,k] = e4m3(x[m,k] / scale[m]), round to nearest, saturating. */
int ojb_quantize_rows_e4m3(const void* x, void* q, float* scale, int64_t rows, int64_t K, ojb_stream_t stream);

/* Host-side listing (no GPU work) of the order in which the block GEMM kernels deal out their work units, for a geometry
 * given directly: n_xblk 256-row blocks of x, tail_rows further rows in n_xchunk swapped-operand chunks, weight tiles of BN
 * rows of an N-row weight, `splits` K ranges over kb_total k-blocks, and band_xblk (0 = one band). out int32 [cap, 5] receives
 * (tail, x block, K range, w tile, x chunk) per unit; returns the number of units. Test support: every unit must occur once,
 * and with bands every unit of a band must come before the units of the next band. */
int64_t ojb_gemm_unit_order(int32_t n_xblk, int32_t tail_rows, int32_t n_xchunk, int32_t BN, int64_t N, int32_t splits,
                            int32_t kb_total, int32_t band_xblk, int32_t* out, int64_t cap);

/* Host-side plan (no GPU work): which kernel variant and how many K ranges the library's cost model picks for a shape.
 * kind = 0 bf16 output, 1 SwiGLU-fused, 2 fp32 split-K partials (the only kind that may use more than one range, up to
 * max_splits). *microseconds (optional) receives the modelled time. Takes the place of the algorithm search of
 * src/lt.cpp:93 (lt2_search), which times cuBLASLt candidates on the device. */
int ojb_gemm_plan(int64_t M, int64_t N, int64_t K, int32_t kind, int32_t max_splits, int32_t* variant, int32_t* splits,
                  float* microseconds);

/* Limit of the device-side waits of the GEMM kernels (every mbarrier wait of producer, MMA issuer and epilogue), in
 * milliseconds; 0 restores the default of 2000. When a wait runs out the CTA writes OJB_DEV_WAIT_TIMEOUT to `status`, lets
 * its copies in flight land, frees its tensor memory and returns; the context stays usable and the results of that launch are
 * invalid. Process-wide, read at launch time. No counterpart in the reference, whose one device-side wait
 * (src/kernels.cu:4103, gdn_fused7) is unbounded. */
int ojb_gemm_set_wait_limit_ms(int32_t ms);

/* Failure injection for the tests of that path (host-side switch, off by default): while on, the producer warp of the 128-row
 * tile kernel (variants 1 / 2) announces the bytes of the second k-block it handles but does not issue the copies, so the
 * consumer's bounded wait runs out as described above. Nothing faults, traps or spins without a limit. */
int ojb_gemm_test_drop_copy(int32_t on);

/* Measurement hook of the 256-row block GEMM kernel and the CTA-pair kernel (no counterpart in the reference). `records` =
 * null switches it off; otherwise a device buffer of 1 + 4*capacity uint64 words, word 0 = record counter (zero it before a
 * launch). Every work unit appends {CTA << 32 | tail flag << 31 | unit, ns when its epilogue began to wait, ns when its
 * accumulators were complete, ns when its epilogue ended} (%globaltimer). Results are not affected. Process-wide and not
 * synchronised: set it while no GEMM of this library is being launched from another thread. */
int ojb_gemm_set_trace(uint64_t* records, int32_t capacity);

/* ------------------------------------------------------------------------------------------------------------------
 * Row-wise and element-wise kernels.
 * ------------------------------------------------------------------------------------------------------------------ */

/* src/kernels.cu:41,755 add_rmsnorm. h = bf16(x + delta) (delta may be null: then h_out is not written and h == x);
 * hn = bf16(h * rsqrt(mean(h^2) + eps) * w1) with w1 = 1 + weight in fp32; rows with rowmask[n] == 0 give hn = 0
 * (rowmask may be null). H % 8 == 0. */
int ojb_add_rmsnorm(const void* x, const void* delta, const float* w1, const int32_t* rowmask, void* h_out,
                    void* hn_out, int64_t rows, int64_t H, float eps, ojb_stream_t stream);

/* src/kernels.cu:1444,1488 add_rmsnorm_sk2. delta = bf16(sum_s parts[s]) with parts fp32 [S, rows, H], S in [1, 16];
 * otherwise as ojb_add_rmsnorm (h_out always written). */
int ojb_add_rmsnorm_sk(const void* x, const float* parts, int splits, const float* w1, const int32_t* rowmask,
                       void* h_out, void* hn_out, int64_t rows, int64_t H, float eps, ojb_stream_t stream);

/* src/kernels.cu:41,755 add_rmsnorm and :1444,1488 add_rmsnorm_sk2 with the residual stream held in fp32 (the form the
 * 64-layer forward of this library uses; the two entry points above keep the reference's bf16 stream bit for bit).
 * h fp32 [rows, H] is updated in place: h = float(x_init) when x_init (bf16 [rows, H], the embedding rows) is given, else
 * h += sum_s parts[s] (fp32 [splits, rows, H], splits in [1, 16]) or h += float(delta) (bf16) or h unchanged; exactly one of
 * x_init / parts / delta may be non-null. The sum is formed and added in fp32 and h is never rounded.
 * hn = bf16(h * rsqrt(mean(h^2) + eps) * w1), zero where rowmask[n] == 0 (rowmask may be null). H % 8 == 0, H <= 8192. */
int ojb_resnorm_f32(float* h, const void* x_init, const void* delta, const float* parts, int splits, const float* w1,
                    const int32_t* rowmask, void* hn_out, int64_t rows, int64_t H, float eps, ojb_stream_t stream);

/* src/kernels.cu:1288,1296 act_tables. silu_tab[65536] bf16 and sig_tab[65536] fp32, indexed by the bf16 bit pattern:
 * silu_tab[b] = bf16(x / (1 + expf(-x))), sig_tab[b] = 1 / (1 + expf(-x)). */
int ojb_act_tables(void* silu_tab, float* sig_tab, ojb_stream_t stream);

/* src/kernels.cu:76,769 silu_mul and :1304,1322 silu_mul_lut. gu = [gate | up] of width 2*I per row;
 * out[rows, I] = bf16(bf16(silu(gate)) * up). silu_tab may be null (computed) or the table above (identical bits). */
int ojb_silu_mul(const void* gu, const void* silu_tab, void* out, int64_t rows, int64_t I, ojb_stream_t stream);

/* src/kernels.cu:1416 gate_mul3 (and gate_mul / gate_mul2 through the strides). att element (t, h, d) is read at
 * att[h*att_stride_h + t*att_stride_t + d]; gate is [T, HQ*D]; y[T, HQ*D] = bf16(att * bf16(sigmoid(gate))). */
int ojb_gate_mul(const void* att, int64_t att_stride_t, int64_t att_stride_h, const void* gate, void* y, int64_t T,
                 int64_t HQ, int64_t D, ojb_stream_t stream);

/* The two inputs of the first layer in one launch (src/fastmodel.py:404-405 does both with torch: `self.embed(ids)` and the
 * rotary module of the backbone): x[n, :] = table[ids[n], :] (bf16 [vocab, H]; an id outside the table gives a zero row) and,
 * for the R2 rotary frequencies, cos / sin of pos[n] * inv_freq[j] * 1 written to columns j and j + R2 of cosb / sinb
 * (bf16 [N, 2 * R2]): angle, cos and sin in fp32, times `scaling`, one rounding to bf16 — the default rope type with text
 * positions (the three position rows of the multimodal form are equal). ids, pos int64 [N]; inv_freq fp32 [R2]. */
int ojb_embed_rope(const int64_t* ids, const void* table, int64_t vocab, const int64_t* pos, const float* inv_freq,
                   float scaling, void* x, void* cosb, void* sinb, int64_t N, int64_t H, int64_t R2, ojb_stream_t stream);

/* src/kernels.cu:1381-1392 l2_prefetch: asks the memory system to bring `nbytes` at `data` (16-byte aligned) into L2, one bulk
 * prefetch per `chunk` bytes (a multiple of 16, at most 1 MiB). Returns at once; nothing waits for the prefetch. */
int ojb_l2_prefetch(const void* data, int64_t nbytes, int64_t chunk, ojb_stream_t stream);

/* src/kernels.cu:4759,4767 pack_bits. vis uint8/bool [N, N] -> bits int32 [N, N/32], bit b of word w = key 32w+b. */
int ojb_pack_bits(const uint8_t* vis, int32_t* bits, int64_t N, ojb_stream_t stream);

/* src/kernels.cu:302,843 fullattn_prep2. proj [N, HQ*2D + 2*HKV*D] = per q head [q(D) | gate(D)], then k heads, then
 * v heads. Writes qt [HQ, N, D], kt / vt [HKV, N, D] (head-major), gate [N, HQ*D]. q, k: RMSNorm over D with (1+w)
 * weights qw1 / kw1 (fp32) rounded to bf16, then rotary on the first RD dims (cos / sin bf16 [N, RD], rotate-half
 * pairing d <-> d + RD/2) with a bf16 rounding after each product and the sum. D % 64 == 0, D <= 256. vt_t (may be null)
 * additionally receives V with rows and columns exchanged, [HKV, D, N]: the operand layout of ojb_tree_attn_tc. */
int ojb_fullattn_prep(const void* proj, const float* qw1, const float* kw1, const void* cosb, const void* sinb,
                      void* qt, void* kt, void* vt, void* vt_t, void* gate, int64_t N, int64_t HQ, int64_t HKV, int64_t D,
                      int64_t RD, float eps, ojb_stream_t stream);

/* ------------------------------------------------------------------------------------------------------------------
 * Prefix-tree layout (HOST functions, no CUDA) — replaces src/fastmodel.py:321-398 FastQwen35.gtree_build.
 * Input: S candidate token lists concatenated in `tokens`, candidate c = tokens[seq_off[c] .. seq_off[c+1]); groups[c] =
 * question index of candidate c (every index in 0..max must occur). NB / PB = row / path-length buckets (NB % 32 == 0).
 * ojb_gtree_dims fills dims[10] = {N, S, R, L2, Lr, Nreal, int64 elements of buf64, int32 elements of buf32, int32
 * elements of ext32, chunk-table capacity}. ojb_gtree_fill writes
 *   buf64 = ids[N] | pos[N] | lastidx[S]              (ids / pos padded to a multiple of 4 elements)
 *   buf32 = src[S,L2] | inv[N] | rep_ptr[N+2] | rep_pos[S*L2] | hist[N+1,4] | canon[S*L2] | rowmask[N] | vbits[N,N/32]
 *           (every field padded to a multiple of 8 elements), bit-identical to the reference's tensors, and, if ext32 is
 *   not null, ext32 = krange[N,8] | nodes[1+2S,4] | chunks[cap,4] | steps[cap,4] | meta[8] | lsteps[cap,4] |
 *   lwalks[2+2S, padded to a multiple of 8] (tables of this
 *   implementation only: key ranges for the attention kernel, node / chunk / walk tables for the tree-native
 *   Gated DeltaNet pass). With OJB_LAYOUT_NO_VBITS in `flags` the visibility words are neither computed nor written (the
 *   kernels of this library read the key ranges instead), which makes the build O(N).
 * ------------------------------------------------------------------------------------------------------------------ */
int ojb_gtree_dims(const int64_t* tokens, const int64_t* seq_off, const int32_t* groups, int64_t S, int64_t NB,
                   int64_t PB, int64_t* dims);
#define OJB_LAYOUT_NO_VBITS 1   /* flags: leave vbits (the last field of buf32, the only O(N^2) one) unwritten */
int ojb_gtree_fill(const int64_t* tokens, const int64_t* seq_off, const int32_t* groups, int64_t S, int64_t pad_id,
                   int64_t NB, int64_t PB, int64_t* buf64, int32_t* buf32, int32_t* ext32, int32_t flags);

/* ------------------------------------------------------------------------------------------------------------------
 * Gated DeltaNet (linear attention).
 * ------------------------------------------------------------------------------------------------------------------ */

/* src/kernels.cu:1173-1283 linattn_prep_dedup2 (rep_ptr != null: results scattered to the replicated slots
 * rep_pos[rep_ptr[n] .. rep_ptr[n+1]) of every packed row n, pad slots zeroed; q, k, v, g, beta have n_slots rows) and its
 * unreplicated form (rep_ptr == null: one output row per packed row). proj bf16 [N, 2KD+2VD+2HV] = [q|k|v|z|b|a];
 * hist int32 [N+1, 4] = rows t-3..t on the row's own path (-1 = none); convw bf16 [2KD+VD, 4]; A_log, dt_bias bf16 [HV].
 * Head dim is 128: KD = 128*HK, VD = 128*HV; HV % 4 == 0 (rows of proj are read 16 bytes at a time, so the row length must be
 * a multiple of 8 elements; OJB_ERR_ARG otherwise). q, k bf16 [*, KD]; v bf16 [*, VD]; g fp32 [*, HV]; beta bf16 [*, HV].
 * l2norm = 0 leaves q and k un-normalised (src/kernels.cu:96 linattn_prep and linattn_prep2 with do_l2 = false, whose callers
 * let the attention kernel normalise); every other prep variant of the reference normalises. The same entry point serves
 * the reference's older layouts (per-sequence [B, T], single-level tree, src-mapped slots): they differ only in `hist` and in
 * the slot tables, which the Python layer derives. */
int ojb_gdn_prep(const void* proj, const int32_t* hist, const int32_t* rep_ptr, const int32_t* rep_pos, int64_t n_slots,
                 const void* convw, const void* A_log, const void* dt_bias, void* q, void* k, void* v, float* g,
                 void* beta, int64_t N, int64_t KD, int64_t VD, int64_t HV, int64_t HK, int32_t l2norm, ojb_stream_t stream);

/* Bytes of scratch that ojb_gdn_chunked needs for n_chunks chunk-table entries and HV value heads. */
int64_t ojb_gdn_scratch_bytes(int64_t n_chunks, int64_t HV);

/* src/kernels.cu:4225 gdn_fused6 (and gdn_fused .. gdn_fused9) — chunked gated delta rule, two launches (state-independent
 * pass over all chunks, then the state pass). Rows are addressed through tables so that the same code serves the
 * reference's replicated [B, T] layout and the packed prefix tree:
 *   chunks int32 [n_chunks, 4] = (first row, rows <= 64 (0 = unused entry), -, -)
 *   steps  int32 [*, 4]        = (chunk, load, save, aux) in execution order; load: 0 carry on, 1 zero state, 2 / 3 restore
 *                                parked slot A / B, 4 initial state number (aux >> 16) - 1; save: bit 0 park in slot A,
 *                                bit 1 in slot B; (aux & 0xffff) - 1 = index in final_state written after the step
 *   walk_ptr int32 [n_walks+1] = step ranges that are independent of each other (one CTA column each)
 * q, k bf16 [rows, HK, 128]; v bf16 [rows, HV, 128]; g fp32 (natural-log decay) and beta bf16 [rows, HV];
 * init_state / final_state fp32 [*, HV, 128(dk), 128(dv)] or null; out bf16 [rows, HV, 128], rows not covered by a chunk
 * are left untouched. o = scale * (...). scratch: ojb_gdn_scratch_bytes(n_chunks, HV) bytes, 16-byte aligned.
 * The state pass fetches the operands of each step with bulk copies that complete on an mbarrier; its wait for them is
 * bounded (ojb_gemm_set_wait_limit_ms). `status` (int32 device word, may be null) receives OJB_DEV_WAIT_TIMEOUT if a wait ran
 * out; the walks of that CTA column are then incomplete. The same holds for the three forms below. */
int ojb_gdn_chunked(const void* q, const void* k, const void* v, const float* g, const void* beta, const int32_t* chunks,
                    int64_t n_chunks, const int32_t* steps, const int32_t* walk_ptr, int64_t n_walks,
                    const float* init_state, float* final_state, void* scratch, void* out, int64_t HK, int64_t HV,
                    float scale, int32_t* status, ojb_stream_t stream);

/* ojb_gdn_chunked with ojb_gdn_prep fused into its first launch (src/kernels.cu:1173 linattn_prep_dedup2 + :4225 gdn_fused6 in
 * two launches instead of three): the state-independent pass reads the in-projection output itself — proj bf16
 * [N, 2KD+2VD+2HV] = [q|k|v|z|b|a], hist int32 [N+1, 4], convw bf16 [2KD+VD, 4], A_log / dt_bias bf16 [HV] as for ojb_gdn_prep —
 * and applies conv, SiLU, the L2 norm of q and k and the beta / log-decay formulas per (chunk, head) in shared memory, with
 * the arithmetic of ojb_gdn_prep operation for operation (same bits). Every chunk must be a run of consecutive packed rows of
 * one tree node (what ojb_gtree_fill produces): the rows before a chunk's first row are taken from hist[first row]. Tables,
 * states, scratch and out as for ojb_gdn_chunked. KD = 128*HK, VD = 128*HV, HV % 4 == 0. */
int ojb_gdn_chunked_proj(const void* proj, const int32_t* hist, const void* convw, const void* A_log, const void* dt_bias,
                         const int32_t* chunks, int64_t n_chunks, const int32_t* steps, const int32_t* walk_ptr,
                         int64_t n_walks, const float* init_state, float* final_state, void* scratch, void* out, int64_t KD,
                         int64_t VD, int64_t HK, int64_t HV, float scale, int32_t* status, ojb_stream_t stream);

/* ojb_gdn_chunked with the state pass run level by level (1 + n_levels launches): `levels` is a HOST array of n_levels + 1
 * walk indices; the walks [levels[l], levels[l+1]) of level l run side by side and start from the end states that walks of
 * earlier levels exported to `states` (fp32 [slots, HV, 128, 128]; steps use load = 4 with slot (aux >> 16) - 1 and export
 * to slot (aux & 0xffff) - 1). For a prefix tree: root | question stems | leaves (lsteps / lwalks of ojb_gtree_fill). No
 * counterpart in the reference, whose kernel recomputes the shared nodes once per candidate (src/kernels.cu:4225). */
int ojb_gdn_chunked_levels(const void* q, const void* k, const void* v, const float* g, const void* beta,
                           const int32_t* chunks, int64_t n_chunks, const int32_t* steps, const int32_t* walk_ptr,
                           const int32_t* levels, int64_t n_levels, float* states, void* scratch, void* out, int64_t HK,
                           int64_t HV, float scale, int32_t* status, ojb_stream_t stream);

/* Scratch-free form of ojb_gdn_chunked. It has no counterpart in open-jev-fast. Same arguments without `scratch` (`status`
 * included): the
 * per-(chunk, head) work items live in a fixed 80 MiB array inside the library's device image (every GPU that loads the
 * library holds it until the process exits), so the call needs no device allocation at all. It is meant for callers that
 * cannot allocate around the call — an inference process whose memory plan is frozen after start-up, or host code that has
 * no allocator for device memory. Limits and rules:
 *   - n_chunks * HV <= ojb_gdn_static_max_items() (1024), else OJB_ERR_LIMIT and nothing is launched;
 *   - the first call on each device looks up the array's device address and raises two kernel attributes; make that first
 *     call with the device current and before any stream capture starts. Two host threads that make this first call on the
 *     same device at the same moment both do the look-up and store the same address: harmless, but not synchronised;
 *   - all calls on one GPU share the array: calls that may overlap on the GPU (different streams, no ordering) race;
 *     the array keeps the previous call's contents, and nothing in it needs clearing between calls. */
int64_t ojb_gdn_static_max_items(void);
int ojb_gdn_chunked_static(const void* q, const void* k, const void* v, const float* g, const void* beta,
                           const int32_t* chunks, int64_t n_chunks, const int32_t* steps, const int32_t* walk_ptr,
                           int64_t n_walks, const float* init_state, float* final_state, void* out, int64_t HK, int64_t HV,
                           float scale, int32_t* status, ojb_stream_t stream);

/* Measurement hook of the state pass (no counterpart in the reference): `records` = null switches it off; otherwise a device
 * buffer of 4 + 12 uint64 words per walk step. The CTA of head 0 / column slice 0 / walk 0 stores %globaltimer at kernel entry,
 * when its tables are staged and its first operands requested, and at its exit (words 0-2), then at six points of every step
 * (step begin, operands ready, phase 1 done, v' visible, phase 2 done, step end), words 0-5 of the step's record from its
 * state-chain warp and 6-11 from its output warp. Synchronises the device (it writes a device variable). */
int ojb_gdn_set_trace(uint64_t* records);

/* src/kernels.cu:1333-1374 gated_rmsnorm_inv2 (inv != null) and :143 gated_rmsnorm (inv == null).
 * out[n, h, :] = bf16(((x[r, h, :] * rstd) * w) * z * sigmoid(z)), r = inv[n] or n, z = proj[n, zoff + h*128 ...],
 * rstd = 1/sqrt(mean(x^2) + eps) over the 128 dims. x bf16 [*, HV, 128]; proj bf16 [N, P]; w bf16 [128]. */
int ojb_gated_rmsnorm(const void* x, const int32_t* inv, const void* proj, const void* w, void* out, int64_t N,
                      int64_t HV, int64_t HD, int64_t zoff, int64_t P, float eps, ojb_stream_t stream);

/* ------------------------------------------------------------------------------------------------------------------
 * Tree attention — replaces src/kernels.cu:4287-4458 fattn_tree (and, above 384 rows, the reference's
 * F.scaled_dot_product_attention + gate_mul3 of src/fastmodel.py:470-473).
 * qt bf16 [HQ, N, D], kt / vt bf16 [HKV, N, D] (head-major, from ojb_fullattn_prep), gate bf16 [N, HQ*D].
 * Mask: vbits int32 [N, N/32] (bit b of word w of row n = key 32w+b visible), or, when vbits is null,
 * krange int32 [N, 8] = (e0, a1, e1, a2, e2, a0, -, -): row n sees keys [a0,e0) + [a1,e1) + [a2,e2) (a0 = 0 in the layout of
 * one request; a request packed behind others has its root start there).
 * y[N, HQ*D] = bf16(bf16(softmax(scale * q k^T + mask) v) * bf16(sigmoid(gate))). N % 32 == 0; D in {64, 128, 256};
 * gq = query heads per CTA, a divisor of HQ/HKV, at most 6. Every row must see at least one key.
 * ------------------------------------------------------------------------------------------------------------------ */
int ojb_tree_attn(const void* qt, const void* kt, const void* vt, const void* gate, const int32_t* vbits,
                  const int32_t* krange, void* y, int64_t N, int64_t HQ, int64_t HKV, int64_t D, int64_t gq, float scale,
                  ojb_stream_t stream);

/* The same attention on the tcgen05 tensor cores (head dim 256, key-range mask only): one CTA per (kv head, 16 query rows)
 * stacks the rows of all HQ/HKV <= 6 query heads of the kv head into one operand tile; Q and the visible 64-key blocks of K and
 * V (two per 128-key product, any two visible ones) arrive by TMA, Q K^T and P V are tcgen05.mma with S, P's source and O in tensor memory; two-pass softmax (row maxima first, then
 * P = exp2((s - max) scale log2 e) and O += P V) in the exp2 domain; the gate factor sigmoid(gate) is applied in fp32.
 * vt_t bf16 [HKV, 256, N] is V with keys contiguous (second V output of ojb_fullattn_prep). Same result as ojb_tree_attn up to
 * the rounding of P, of the gate factor and the summation order. `status` receives OJB_DEV_WAIT_TIMEOUT if a bounded
 * device-side wait ran out. N <= 131 072 (OJB_ERR_LIMIT beyond). Replaces the same reference code as ojb_tree_attn (src/kernels.cu:4287-4458; above 384 rows
 * src/fastmodel.py:470-473). */
int ojb_tree_attn_tc(const void* qt, const void* kt, const void* vt_t, const void* gate, const int32_t* krange, void* y,
                     int64_t N, int64_t HQ, int64_t HKV, int64_t D, float scale, int32_t* status, ojb_stream_t stream);

/* Measurement hook of ojb_tree_attn_tc (no counterpart in the reference): `records` = null switches it off; otherwise a device
 * buffer of 16 uint64 words. The CTA of kv head 0 and the last-but-one block of 16 query rows stores %globaltimer at kernel
 * entry [0], after its set-up [1], at the first scores of pass 1 [2] and of pass 2 [3], when the last P tile is handed over
 * [4], when O is complete [5], after its epilogue [6] and at exit [7]; its MMA thread when Q has landed [8] and when every MMA
 * is issued [9]; word 15 = number of key blocks it visits. Synchronises the device (it writes a device variable). */
int ojb_tree_attn_set_trace(uint64_t* records);

/* Scoring head — replaces src/server.py:37 `mdl.head(forward_gtree(...).float())` together with the gather
 * src/fastmodel.py:482 `hn[lay.lastidx]`: out[s, a] = bias[a] + sum_h float(hn[rows[s], h]) * W[a, h], all fp32.
 * hn bf16 [N, H] (final-norm output), rows int64 [S] (last row of each candidate), W fp32 [A, H], bias fp32 [A] or null. */
int ojb_score_head(const void* hn, const int64_t* rows, const float* W, const float* bias, float* out, int64_t S, int64_t A,
                   int64_t H, ojb_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* OJB200_H_ */
