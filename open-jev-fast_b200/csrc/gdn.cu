// Chunked Gated DeltaNet (linear attention) for the scoring forward, tree-native.
//
//   gdn_prep   per packed row: causal depthwise conv (width 4, history taken along the row's own tree path) + SiLU, L2 norm
//              of q and k per head, beta = sigmoid(b), g = -exp(A_log) * softplus(a + dt_bias). Optionally scattered to the
//              replicated per-candidate slots of the reference layout.
//   gdn_intra  per (chunk of <= 64 rows, value head), all chunks in parallel — everything that does not depend on the
//              recurrent state: G = cumsum(g); A = strict_lower((k beta) k^T * exp(G_i - G_j)); T = (I+A)^-1 in fp32 by
//              16 x 16 blocks; u = T (v beta), w = T (k beta e^G) with T as a bf16 value + remainder pair;
//              Aqk = tril(q k^T * exp(G_i - G_j)) * scale; qg = q e^G scale; kg = k e^(G_L - G). K K^T, Q K^T and the two
//              products with T run on the tensor cores (mma.sync bf16, fp32 accumulate).
//              Results go to a scratch item of 40 968 bf16 per (chunk, head), laid out as the state pass reads it.
//   gdn_state  per (value head, 32-column slice of the state, walk): walks the chunks of the tree depth first with the
//              fp32 state slice [128 x 32] in registers; per chunk v' = u - w S, o = qg S + Aqk v', S = S e^(G_L) + kg^T v'
//              (mma.sync). The state at the end of the root and of a question stem is parked in shared memory and restored
//              for every child, so shared prefixes are computed once. The next chunk's operands are prefetched with
//              cp.async while the current one is computed.
//   gated_rmsnorm  per (row, head): RMSNorm over 128 dims times weight times z * sigmoid(z), optional row gather.
#include "common.cuh"

namespace ojb {
namespace {

constexpr int kHD = 128;          // head dim of q, k and v
constexpr int kChunk = 64;
// Shared-memory tile shapes (row lengths padded by 8 bf16 = 16 bytes so that ldmatrix rows fall into distinct banks). The
// scratch item of a (chunk, head) holds its tiles in exactly these padded shapes, so the state pass copies them as flat
// byte ranges: w | qg | kg | u as four 32-column slices | Aqk | float e^(G_L).
constexpr int kLd = kHD + 8;            // [64 x 128] tiles: 272-byte rows
constexpr int kDv = 32;                 // state columns per CTA of the state pass
constexpr int kLdS = kDv + 8;           // [* x 32] tiles: 80-byte rows
constexpr int kLdA = kChunk + 8;        // [64 x 64] tile: 144-byte rows
constexpr int kOffW = 0, kOffQg = kChunk * kLd, kOffKg = 2 * kChunk * kLd, kOffU = 3 * kChunk * kLd,
              kOffA = kOffU + (kHD / kDv) * kChunk * kLdS, kOffGl = kOffA + kChunk * kLdA;
constexpr int kItemElems = kOffGl + 8;  // 40 968 bf16 = 81 936 bytes
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// ------------------------------------------------------------------------------------------------------------ gdn_prep
// grid (ceil(C/8/256), rows [+ pad-slot groups when scattering]); one thread = 8 consecutive channels of one packed row.
// proj [N, P] = [q(KD) | k(KD) | v(VD) | z(VD) | b(HV) | a(HV)].
template <bool SCATTER>
__global__ void __launch_bounds__(256)
gdn_prep_kernel(const bf16_t* __restrict__ proj, const int4* __restrict__ hist, const int32_t* __restrict__ rep_ptr,
                const int32_t* __restrict__ rep_pos, const bf16_t* __restrict__ convw, const bf16_t* __restrict__ A_log,
                const bf16_t* __restrict__ dt_bias, bf16_t* __restrict__ q, bf16_t* __restrict__ k, bf16_t* __restrict__ v,
                float* __restrict__ g, bf16_t* __restrict__ beta, int N, int KD, int VD, int HV, int l2norm) {
  pdl_begin();
  const int C = 2 * KD + VD, P = C + VD + 2 * HV;
  const int n = blockIdx.y;
  int4 hr = make_int4(-1, -1, -1, -1);
  if (n < N) hr = hist[n];
  // padding: blocks past N stand for groups of 16 pad slots (scatter form); packed rows that lie on no path (end padding
  // of the row bucket) have no history entry, not even themselves, and produce zeros
  const bool pad = n >= N || hr.w < 0;
  int p0 = 0, p1 = 1;
  if constexpr (SCATTER) {
    if (n < N) { p0 = rep_ptr[n]; p1 = rep_ptr[n + 1]; }
    else { p0 = rep_ptr[N] + (n - N) * 16; p1 = min(rep_ptr[N + 1], p0 + 16); }
    if (p0 >= p1) return;
  }
  if (blockIdx.x == 0 && threadIdx.x < HV) {
    const int h = threadIdx.x;
    float bv = 0.f, gv = 0.f;
    if (!pad) {
      const bf16_t* pr = proj + static_cast<int64_t>(hr.w) * P + C + VD;
      bv = sigmoid_f(bf2f(pr[h]));
      const float xs = bf2f(pr[HV + h]) + bf2f(dt_bias[h]);
      gv = -expf(bf2f(A_log[h])) * (xs > 20.f ? xs : log1pf(expf(xs)));
    }
    if constexpr (SCATTER) {
      for (int p = p0; p < p1; ++p) {
        const int64_t slot = rep_pos[p];
        beta[slot * HV + h] = f2bf(bv);
        g[slot * HV + h] = gv;
      }
    } else {
      beta[static_cast<int64_t>(n) * HV + h] = f2bf(bv);
      g[static_cast<int64_t>(n) * HV + h] = gv;
    }
  }
  const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c0 >= C) return;
  const bool isqk = c0 < 2 * KD;
  uint4 ov = make_uint4(0u, 0u, 0u, 0u);
  if (!pad) {
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    // taps in the order of the reference: oldest row first, weight column i multiplies history row i
    uint4 wv[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) wv[u] = __ldg(reinterpret_cast<const uint4*>(convw + static_cast<int64_t>(c0) * 4 + u * 8));
    const bf16_t* wb = reinterpret_cast<const bf16_t*>(wv);  // wb[e*4 + tap]
    const int rows[4] = {hr.x, hr.y, hr.z, hr.w};
#pragma unroll
    for (int tap = 0; tap < 4; ++tap) {
      if (rows[tap] >= 0) {
        float xv[8];
        unpack8(*reinterpret_cast<const uint4*>(proj + static_cast<int64_t>(rows[tap]) * P + c0), xv);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] += bf2f(wb[e * 4 + tap]) * xv[e];
      }
    }
    float o[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = round_bf(silu_f(acc[e]));
    if (isqk && l2norm) {  // 16 consecutive threads cover one 128-wide head
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += o[e] * o[e];
#pragma unroll
      for (int off = 8; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
      const float rn = 1.0f / sqrtf(ss + 1e-6f);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] *= rn;
    }
    ov = pack8(o);
  }
  bf16_t* dst;
  int64_t width;
  int col;
  if (c0 < KD) { dst = q; width = KD; col = c0; }
  else if (c0 < 2 * KD) { dst = k; width = KD; col = c0 - KD; }
  else { dst = v; width = VD; col = c0 - 2 * KD; }
  if constexpr (SCATTER) {
    for (int p = p0; p < p1; ++p) *reinterpret_cast<uint4*>(dst + static_cast<int64_t>(rep_pos[p]) * width + col) = ov;
  } else {
    *reinterpret_cast<uint4*>(dst + static_cast<int64_t>(n) * width + col) = ov;
  }
}

// ----------------------------------------------------------------------------------------------------------- gdn_intra
constexpr int kIntraThreads = 256;
constexpr int kLdT = kChunk + 8;  // padded row (bf16) of the [64 x 64] inverse
// K | Q | V tiles (the Q tile holds the fp32 inverse T once q is no longer needed), A (fp32; later the bf16 pair of T) with
// the block scratch P behind it, four vectors: 74 KB, three CTAs per SM
constexpr int kIntraSmem = 3 * kChunk * kLd * 2 + kChunk * kChunk * 4 + 3 * 256 * 4 + 4 * kChunk * 4;
static_assert(kChunk * kChunk * 4 <= kChunk * kLd * 2, "the fp32 inverse must fit over the Q tile");
static_assert(2 * kChunk * kLdT * 2 <= kChunk * kChunk * 4 + 3 * 256 * 4, "the bf16 pair of T must fit over A and P");

// Source of q, k, v, g, beta when the preparation (gdn_prep) is fused into this kernel: the in-projection output itself.
struct PrepSrc {
  const bf16_t* proj;      // [N, P] = [q(KD) | k(KD) | v(VD) | z(VD) | b(HV) | a(HV)]
  const int4* hist;        // [N+1]: rows t-3, t-2, t-1, t on the row's own tree path (-1 = none)
  const bf16_t* convw;     // [2KD+VD, 4]
  const bf16_t* A_log;     // [HV]
  const bf16_t* dt_bias;   // [HV]
  int P;
};

// FUSED: q / k / v / g / beta are not read; the CTA loads the raw in-projection rows of its chunk (plus the three rows that
// precede the chunk on its tree path), applies the causal conv, SiLU and the L2 norm of q and k in shared memory, and derives
// beta and the log-decay from the b / a columns. The arithmetic is that of gdn_prep_kernel, operation for operation, so both
// forms give the same bits; what is saved is a launch and the round trip of q, k, v through global memory.
template <bool FUSED>
__global__ void __launch_bounds__(kIntraThreads, 3)
gdn_intra_kernel(const bf16_t* __restrict__ q, const bf16_t* __restrict__ k, const bf16_t* __restrict__ v,
                 const float* __restrict__ g, const bf16_t* __restrict__ beta, const int32_t* __restrict__ chunks,
                 bf16_t* __restrict__ scratch, int HK, int HV, float scale, int pair, PrepSrc ps) {
  pdl_begin();
  const int4 ch = reinterpret_cast<const int4*>(chunks)[blockIdx.x];
  const int row0 = ch.x, nrows = ch.y;
  if (nrows <= 0) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // Short chunks (at most 32 rows: question stems, candidate tails) are done two to a CTA: the second one occupies local rows
  // 32-63, the cross terms of the two are masked out, so the 64 x 64 algebra is block diagonal and each half is exactly what
  // the chunk alone would give. The short chunks pair up in table order: the even-ranked one takes the next short chunk
  // with it, the odd-ranked CTA has nothing to do. (Any two chunks are independent in this pass.)
  // `pair` = number of CTA slots of the GPU (0 = never pair): chunks are paired only when one CTA per (non-empty chunk, head)
  // would not fit a single wave; with room to spare the short chunks finish sooner side by side. Every CTA reads the same
  // table and reaches the same decision.
  __shared__ int s_rank, s_next, s_real;
  int partner = -1;
  if (pair && nrows <= 32) {
    if (tid == 0) { s_rank = 0; s_next = 0x7fffffff; s_real = 0; }
    __syncthreads();
    int cnt = 0, nxt = 0x7fffffff, real = 0;
    for (int j = tid; j < static_cast<int>(gridDim.x); j += kIntraThreads) {
      const int nj = chunks[j * 4 + 1];
      if (nj > 0) ++real;
      if (nj > 0 && nj <= 32) {
        if (j < static_cast<int>(blockIdx.x)) ++cnt;
        else if (j > static_cast<int>(blockIdx.x)) nxt = min(nxt, j);
      }
    }
    if (cnt) atomicAdd(&s_rank, cnt);
    if (real) atomicAdd(&s_real, real);
    if (nxt != 0x7fffffff) atomicMin(&s_next, nxt);
    __syncthreads();
    if (s_real * HV > pair) {
      if (s_rank & 1) return;
      partner = s_next == 0x7fffffff ? -1 : s_next;
    }
  }
  const bool paired = partner >= 0;
  int rowB0 = 0, nB = 0;
  if (paired) {
    const int4 cb = reinterpret_cast<const int4*>(chunks)[partner];
    rowB0 = cb.x;
    nB = cb.y;
  }
  // global row of local row r, or -1 for padding
  auto grow = [&](int r) -> int64_t {
    if (!paired) return r < nrows ? row0 + r : -1;
    return r < 32 ? (r < nrows ? row0 + r : -1) : (r - 32 < nB ? rowB0 + r - 32 : -1);
  };
  const int h = blockIdx.y, hk = h / (HV / HK);
  extern __shared__ __align__(16) uint8_t smem_raw[];
  bf16_t* Ks = reinterpret_cast<bf16_t*>(smem_raw);
  bf16_t* Qs = Ks + kChunk * kLd;
  bf16_t* Vs = Qs + kChunk * kLd;
  float* As = reinterpret_cast<float*>(Vs + kChunk * kLd);    // [64][64]
  float* Ps = As + kChunk * kChunk;                            // [3][16][16] block products
  float* Gs = Ps + 3 * 256;                                    // G * log2e (inclusive cumsum)
  float* Bs = Gs + kChunk;                                     // beta
  float* EGs = Bs + kChunk;                                    // exp(G)
  float* EKs = EGs + kChunk;                                   // exp(G_L - G)
  float* Tf = reinterpret_cast<float*>(Qs);                    // [64][64] inverse, fp32 (after the elementwise phase)
  const int KD = HK * kHD, VD = HV * kHD;
  bf16_t* item = scratch + (static_cast<int64_t>(blockIdx.x) * HV + h) * kItemElems;
  bf16_t* itemB = paired ? scratch + (static_cast<int64_t>(partner) * HV + h) * kItemElems : item;
  // local row i of the tile -> (item, row inside the item)
  auto out_item = [&](int i) { return (paired && i >= 32) ? itemB : item; };
  auto out_row = [&](int i) { return (paired && i >= 32) ? i - 32 : i; };
  if (paired) {
    // rows 32-63 of both items belong to no chunk row: the state pass multiplies all 64 rows, so they must be zero
    const uint4 z = make_uint4(0u, 0u, 0u, 0u);
    for (int which = 0; which < 2; ++which) {
      bf16_t* it = which ? itemB : item;
      for (int i = tid; i < 3 * 32 * (kLd / 8); i += kIntraThreads) {          // w | qg | kg tiles [64][kLd]
        const int t = i / (32 * (kLd / 8)), rem = i - t * (32 * (kLd / 8));
        *reinterpret_cast<uint4*>(it + t * (kChunk * kLd) + 32 * kLd + rem * 8) = z;
      }
      for (int i = tid; i < 4 * 32 * (kLdS / 8); i += kIntraThreads) {         // four u slices [64][kLdS]
        const int t = i / (32 * (kLdS / 8)), rem = i - t * (32 * (kLdS / 8));
        *reinterpret_cast<uint4*>(it + kOffU + t * (kChunk * kLdS) + 32 * kLdS + rem * 8) = z;
      }
      for (int i = tid; i < 32 * (kLdA / 8); i += kIntraThreads)               // Aqk rows 32-63
        *reinterpret_cast<uint4*>(it + kOffA + 32 * kLdA + i * 8) = z;
    }
  }

  // log-decay and beta of the two rows that each lane of warp 0 sums below: requested before the tiles, so that their
  // latency runs under the tile loads
  float pg0 = 0.f, pg1 = 0.f, pb0 = 0.f, pb1 = 0.f;
  if constexpr (!FUSED) {
    if (warp == 0) {
      const int64_t a0 = grow(lane * 2), a1 = grow(lane * 2 + 1);
      if (a0 >= 0) { pg0 = g[a0 * HV + h]; pb0 = bf2f(beta[a0 * HV + h]); }
      if (a1 >= 0) { pg1 = g[a1 * HV + h]; pb1 = bf2f(beta[a1 * HV + h]); }
    }
  }
  if constexpr (!FUSED) {
  // ---- load K, Q, V rows (zero rows past the end of the chunk): asynchronous 16-byte copies, all twelve of a thread in
  //      flight at once (as plain loads in this loop they went one after the other: 4 to 10 us for 48 KB per CTA)
  for (int i = tid; i < 3 * kChunk * (kHD / 8); i += kIntraThreads) {
    const int which = i / (kChunk * 16), rem = i - which * (kChunk * 16);
    const int r = rem >> 4, cv = (rem & 15) * 8;
    const int64_t row = grow(r);
    bf16_t* dst = which == 0 ? Ks : which == 1 ? Qs : Vs;
    if (row >= 0) {
      const bf16_t* src = which == 0 ? k + row * KD + hk * kHD : which == 1 ? q + row * KD + hk * kHD : v + row * VD + h * kHD;
      cp_async16(smem_u32(dst + r * kLd + cv), src + cv);
    } else {
      *reinterpret_cast<uint4*>(dst + r * kLd + cv) = make_uint4(0u, 0u, 0u, 0u);
    }
  }
  cp_async_commit();
  } else {
  // ---- raw in-projection rows of the chunk into the K / Q / V tiles, and the three rows before each (sub-)chunk on its
  //      tree path into Hs (over A, which is not written before the K K^T phase): [sub-chunk][3 rows][k | q | v][128]
  bf16_t* Hs = reinterpret_cast<bf16_t*>(As);
  const int coff[3] = {KD + hk * kHD, hk * kHD, 2 * KD + h * kHD};   // column of this head's k, q, v inside a proj row
  for (int i = tid; i < 3 * kChunk * (kHD / 8); i += kIntraThreads) {
    const int which = i / (kChunk * 16), rem = i - which * (kChunk * 16);
    const int r = rem >> 4, cv = (rem & 15) * 8;
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    const int64_t row = grow(r);
    if (row >= 0) val = *reinterpret_cast<const uint4*>(ps.proj + row * ps.P + coff[which] + cv);
    bf16_t* dst = which == 0 ? Ks : which == 1 ? Qs : Vs;
    *reinterpret_cast<uint4*>(dst + r * kLd + cv) = val;
  }
  for (int i = tid; i < 2 * 3 * 3 * (kHD / 8); i += kIntraThreads) {
    const int cv = (i & 15) * 8, which = (i >> 4) % 3, j = (i / 48) % 3, sub = i / 144;
    const int64_t first = sub == 0 ? static_cast<int64_t>(row0) : (paired ? static_cast<int64_t>(rowB0) : -1);
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    if (first >= 0) {
      const int4 hr = ps.hist[first];
      const int prow = j == 0 ? hr.x : (j == 1 ? hr.y : hr.z);
      if (prow >= 0) val = *reinterpret_cast<const uint4*>(ps.proj + static_cast<int64_t>(prow) * ps.P + coff[which] + cv);
    }
    *reinterpret_cast<uint4*>(Hs + ((sub * 3 + j) * 3 + which) * kHD + cv) = val;
  }
  __syncthreads();
  // ---- conv (4 taps, oldest first) + SiLU (+ L2 norm of q and k over the 128 dims of the head) in place. One thread = one
  //      8-column vector of one tile over 16 consecutive rows, the last three rows it has seen kept in registers; every
  //      thread fetches the three rows in front of its segment before any row is overwritten.
  const bool worker = tid < 3 * 4 * 16;
  const int c_which = tid / 64, c_seg = (tid >> 4) & 3, c_cv = (tid & 15) * 8;
  bf16_t* tile = c_which == 0 ? Ks : c_which == 1 ? Qs : Vs;
  uint4 win[3], wv[4];
  if (worker) {
    const bool from_hist = c_seg == 0 || (paired && c_seg == 2);      // the segment starts a (sub-)chunk
    const int sub = (paired && c_seg == 2) ? 1 : 0;
#pragma unroll
    for (int j = 0; j < 3; ++j)
      win[j] = from_hist ? *reinterpret_cast<const uint4*>(Hs + ((sub * 3 + j) * 3 + c_which) * kHD + c_cv)
                         : *reinterpret_cast<const uint4*>(tile + (16 * c_seg - 3 + j) * kLd + c_cv);
#pragma unroll
    for (int u = 0; u < 4; ++u)
      wv[u] = __ldg(reinterpret_cast<const uint4*>(ps.convw + static_cast<int64_t>(coff[c_which] + c_cv) * 4 + u * 8));
  }
  __syncthreads();
  if (worker) {
    const bf16_t* wb = reinterpret_cast<const bf16_t*>(wv);  // wb[e * 4 + tap]
    for (int r = 16 * c_seg; r < 16 * c_seg + 16; ++r) {
      const uint4 cur = *reinterpret_cast<const uint4*>(tile + r * kLd + c_cv);
      float x0[8], x1[8], x2[8], x3[8], o[8];
      unpack8(win[0], x0); unpack8(win[1], x1); unpack8(win[2], x2); unpack8(cur, x3);
      const bool real = grow(r) >= 0;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float acc = 0.f;
        acc += bf2f(wb[e * 4 + 0]) * x0[e];
        acc += bf2f(wb[e * 4 + 1]) * x1[e];
        acc += bf2f(wb[e * 4 + 2]) * x2[e];
        acc += bf2f(wb[e * 4 + 3]) * x3[e];
        o[e] = real ? round_bf(silu_f(acc)) : 0.f;
      }
      if (c_which < 2) {      // 16 consecutive lanes hold one row of one head
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += o[e] * o[e];
#pragma unroll
        for (int off = 8; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
        const float rn = 1.0f / sqrtf(ss + 1e-6f);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] *= rn;
      }
      *reinterpret_cast<uint4*>(tile + r * kLd + c_cv) = pack8(o);
      win[0] = win[1]; win[1] = win[2]; win[2] = cur;
    }
  }
  }
  // ---- cumulative log-decay (warp 0): two elements per lane
  if (warp == 0) {
    const int r0 = lane * 2, r1 = r0 + 1;
    // log-decays below -1e4 are clamped: e^-1e4 is zero in fp32 either way, and -inf would turn the differences of the
    // cumulative sums into NaN
    const int64_t gr0 = grow(r0), gr1 = grow(r1);
    float g0 = 0.f, g1 = 0.f, be0 = 0.f, be1 = 0.f;
    if constexpr (FUSED) {
      // beta = bf16(sigmoid(b)), g = -exp(A_log) * softplus(a + dt_bias) from the b / a columns of the row (as gdn_prep)
      const int ba = 2 * KD + 2 * VD;
      const float na = -expf(bf2f(ps.A_log[h])), db = bf2f(ps.dt_bias[h]);
      if (gr0 >= 0) {
        const bf16_t* pr = ps.proj + gr0 * ps.P + ba;
        be0 = round_bf(sigmoid_f(bf2f(pr[h])));
        const float xs = bf2f(pr[HV + h]) + db;
        g0 = fmaxf(na * (xs > 20.f ? xs : log1pf(expf(xs))), -1e4f);
      }
      if (gr1 >= 0) {
        const bf16_t* pr = ps.proj + gr1 * ps.P + ba;
        be1 = round_bf(sigmoid_f(bf2f(pr[h])));
        const float xs = bf2f(pr[HV + h]) + db;
        g1 = fmaxf(na * (xs > 20.f ? xs : log1pf(expf(xs))), -1e4f);
      }
    } else {
      if (gr0 >= 0) { g0 = fmaxf(pg0, -1e4f); be0 = pb0; }
      if (gr1 >= 0) { g1 = fmaxf(pg1, -1e4f); be1 = pb1; }
    }
    Bs[r0] = be0;
    Bs[r1] = be1;
    float s = g0 + g1;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float t = __shfl_up_sync(0xffffffffu, s, o);
      // with two chunks in the tile the sum restarts at local row 32 (lane 16)
      if (lane >= o && (!paired || ((lane ^ (lane - o)) & 16) == 0)) s += t;
    }
    const float c1 = s, c0 = s - g1;      // inclusive sums at r1 and r0
    const float total_hi = __shfl_sync(0xffffffffu, s, 31), total_lo = __shfl_sync(0xffffffffu, s, 15);
    const float total = (paired && lane < 16) ? total_lo : total_hi;     // the sum over this row's own chunk
    Gs[r0] = c0 * kLog2e; Gs[r1] = c1 * kLog2e;
    EGs[r0] = exp2f(c0 * kLog2e); EGs[r1] = exp2f(c1 * kLog2e);
    EKs[r0] = exp2f((total - c0) * kLog2e); EKs[r1] = exp2f((total - c1) * kLog2e);
    if (lane == 0) {
      *reinterpret_cast<float*>(item + kOffGl) = exp2f((paired ? total_lo : total_hi) * kLog2e);
      if (paired) *reinterpret_cast<float*>(itemB + kOffGl) = exp2f(total_hi * kLog2e);
    }
  }
  if constexpr (!FUSED) cp_async_wait<0>();
  __syncthreads();

  // ---- K K^T (warps 0-3) and Q K^T (warps 4-7): 16 rows x 64 columns per warp
  {
    const bool is_qk = warp >= 4;
    const int m0 = (warp & 3) * 16;
    const bf16_t* Am = is_qk ? Qs : Ks;
    float acc[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[nt][e] = 0.f;
    const int a_row = m0 + (lane & 15), a_col = (lane >> 4) * 8;
    const int b_row = (lane & 7) + ((lane >> 4) << 3), b_col = ((lane >> 3) & 1) * 8;
#pragma unroll
    for (int ks = 0; ks < kHD / 16; ++ks) {
      uint32_t a0, a1, a2, a3;
      ldsm_x4(smem_u32(Am + a_row * kLd + ks * 16 + a_col), a0, a1, a2, a3);
#pragma unroll
      for (int np = 0; np < 4; ++np) {  // two 8-column tiles per ldmatrix.x4
        uint32_t b0, b1, b2, b3;
        ldsm_x4(smem_u32(Ks + (np * 16 + b_row) * kLd + ks * 16 + b_col), b0, b1, b2, b3);
        mma_bf16(acc[2 * np], a0, a1, a2, a3, b0, b1);
        mma_bf16(acc[2 * np + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    const int gr = lane >> 2, tc = (lane & 3) * 2;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int i = m0 + gr + half * 8;
        const float gi = Gs[i];
        float o2[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int j = nt * 8 + tc + e;
          const float a = acc[nt][half * 2 + e];
          const bool same = !paired || ((i ^ j) & 32) == 0;      // both rows in the same chunk of the tile
          if (is_qk) o2[e] = (same && j <= i) ? a * exp2f(gi - Gs[j]) * scale : 0.f;
          else o2[e] = (same && j < i) ? a * Bs[i] * exp2f(gi - Gs[j]) : 0.f;
        }
        if (is_qk) {
          // second chunk of a pair: its own block moves to columns 0-31 of its item, the (zero) cross block to 32-63
          const int col = nt * 8 + tc;
          *reinterpret_cast<uint32_t*>(out_item(i) + kOffA + out_row(i) * kLdA + ((paired && i >= 32) ? (col ^ 32) : col)) =
              pack2(o2[0], o2[1]);
        } else {
          As[i * kChunk + nt * 8 + tc] = o2[0];
          As[i * kChunk + nt * 8 + tc + 1] = o2[1];
        }
      }
    }
  }
  __syncthreads();   // all warps are done reading K and Q as MMA operands
  // ---- qg = q e^G scale and kg = k e^(G_L - G) go straight to the item; the right-hand sides v beta and k beta e^G
  //      replace v and k in shared memory
  for (int i = tid; i < kChunk * (kHD / 8); i += kIntraThreads) {
    const int r = i >> 4, cv = (i & 15) * 8;
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(Qs + r * kLd + cv), f);
    const float sq = EGs[r] * scale;
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] *= sq;
    *reinterpret_cast<uint4*>(out_item(r) + kOffQg + out_row(r) * kLd + cv) = pack8(f);
    float kf[8];
    unpack8(*reinterpret_cast<const uint4*>(Ks + r * kLd + cv), kf);
    const float sk = EKs[r], sw = Bs[r] * EGs[r];
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = kf[e] * sk;
    *reinterpret_cast<uint4*>(out_item(r) + kOffKg + out_row(r) * kLd + cv) = pack8(f);
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = kf[e] * sw;
    *reinterpret_cast<uint4*>(Ks + r * kLd + cv) = pack8(f);
    unpack8(*reinterpret_cast<const uint4*>(Vs + r * kLd + cv), f);
    const float sv = Bs[r];
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] *= sv;
    *reinterpret_cast<uint4*>(Vs + r * kLd + cv) = pack8(f);
  }
  __syncthreads();   // q has been consumed: its tile becomes the fp32 inverse
  // ---- T = (I + A)^-1, fp32, by 16 x 16 blocks. First the four diagonal blocks (forward substitution per column) ...
  for (int i = tid; i < kChunk * kChunk; i += kIntraThreads) Tf[i] = 0.f;
  __syncthreads();
  if (tid < kChunk) {
    const int base = (tid >> 4) * 16, c = tid & 15;
    float x[16];
#pragma unroll
    for (int r = 0; r < 16; ++r) {
      float acc = r == c ? 1.f : 0.f;
      const float* arow = As + (base + r) * kChunk + base;
#pragma unroll
      for (int kk = 0; kk < r; ++kk) acc -= arow[kk] * x[kk];
      x[r] = acc;
    }
#pragma unroll
    for (int r = 0; r < 16; ++r) Tf[(base + r) * kChunk + base + c] = x[r];
  }
  __syncthreads();
  // ... then the blocks below the diagonal, one block diagonal at a time: T_ij = -T_ii * sum_{k=j}^{i-1} A_ik T_kj
  {
    const int r = tid >> 4, c = tid & 15;   // one element of a 16 x 16 block per thread
#pragma unroll
    for (int d = 1; d < 4; ++d) {
#pragma unroll
      for (int j = 0; j + d < 4; ++j) {
        const int i = j + d;
        float acc = 0.f;
        for (int kb = j; kb < i; ++kb) {
          const float* arow = As + (16 * i + r) * kChunk + 16 * kb;
          const float* tcol = Tf + (16 * kb) * kChunk + 16 * j + c;
#pragma unroll
          for (int e = 0; e < 16; ++e) acc += arow[e] * tcol[e * kChunk];
        }
        Ps[j * 256 + r * 16 + c] = acc;
      }
      __syncthreads();
#pragma unroll
      for (int j = 0; j + d < 4; ++j) {
        const int i = j + d;
        const float* trow = Tf + (16 * i + r) * kChunk + 16 * i;
        float acc = 0.f;
#pragma unroll
        for (int e = 0; e < 16; ++e) acc += trow[e] * Ps[j * 256 + e * 16 + c];
        Tf[(16 * i + r) * kChunk + 16 * j + c] = -acc;
      }
      __syncthreads();
    }
  }
  // ---- T as a pair of bf16 matrices (value and rounding remainder) over the memory of A, which is no longer needed
  bf16_t* Thi = reinterpret_cast<bf16_t*>(As);
  bf16_t* Tlo = Thi + kChunk * kLdT;
  for (int i = tid; i < kChunk * kChunk; i += kIntraThreads) {
    const int r = i >> 6, c = i & 63;
    const float t = Tf[i];
    const bf16_t hi = f2bf(t);
    Thi[r * kLdT + c] = hi;
    Tlo[r * kLdT + c] = f2bf(t - bf2f(hi));
  }
  __syncthreads();
  // ---- u = T (v beta) (warps 0-3) and w = T (k beta e^G) (warps 4-7) on the tensor cores: 16 rows x 128 columns per warp;
  //      T is lower triangular, so row block m only needs the k-steps 0..m
  {
    const int mt = warp & 3;
    const bool is_w = warp >= 4;
    const bf16_t* Bm = is_w ? Ks : Vs;
    float acc[16][4];
#pragma unroll
    for (int nt = 0; nt < 16; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[nt][e] = 0.f;
    const int a_row = mt * 16 + (lane & 15), a_col = (lane >> 4) * 8;
    const int bt_row = lane & 15, bt_col = (lane >> 4) * 8;
    for (int kk = 0; kk <= mt; ++kk) {
      uint32_t h0, h1, h2, h3, l0, l1, l2, l3;
      ldsm_x4(smem_u32(Thi + a_row * kLdT + kk * 16 + a_col), h0, h1, h2, h3);
      ldsm_x4(smem_u32(Tlo + a_row * kLdT + kk * 16 + a_col), l0, l1, l2, l3);
#pragma unroll
      for (int np = 0; np < 8; ++np) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(smem_u32(Bm + (kk * 16 + bt_row) * kLd + np * 16 + bt_col), b0, b1, b2, b3);
        mma_bf16(acc[2 * np], h0, h1, h2, h3, b0, b1);
        mma_bf16(acc[2 * np + 1], h0, h1, h2, h3, b2, b3);
        mma_bf16(acc[2 * np], l0, l1, l2, l3, b0, b1);
        mma_bf16(acc[2 * np + 1], l0, l1, l2, l3, b2, b3);
      }
    }
    const int gr = lane >> 2, tc = (lane & 3) * 2;
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
      // w keeps its 128 columns in one padded tile, u is stored as four 32-column slices (one per CTA column of the state pass)
      bf16_t* it = out_item(mt * 16);                   // the 16 rows of a warp lie in one chunk of the tile
      bf16_t* dst = is_w ? it + kOffW + nt * 8 + tc : it + kOffU + (nt >> 2) * (kChunk * kLdS) + (nt & 3) * 8 + tc;
      const int ld = is_w ? kLd : kLdS;
      const int orow = out_row(mt * 16) + gr;
      *reinterpret_cast<uint32_t*>(dst + orow * ld) = pack2(acc[nt][0], acc[nt][1]);
      *reinterpret_cast<uint32_t*>(dst + (orow + 8) * ld) = pack2(acc[nt][2], acc[nt][3]);
    }
  }
}

// ----------------------------------------------------------------------------------------------------------- gdn_state
// 8 warps: warps 0-3 carry the state (the sequential chain: w S -> v' -> S update), warps 4-7 compute the outputs
// (qg S + Aqk v') beside them, so the outputs are off the chain that the next step waits for.
constexpr int kStateThreads = 256;
constexpr int kChainThreads = 128;
constexpr int kBufElems = 3 * kChunk * kLd + kChunk * kLdS + kChunk * kLdA;  // w | qg | kg | u-slice | Aqk
constexpr int kStateSmem = 2 * kBufElems * 2 + 2 * kHD * kLdS * 2 + kChunk * kLdS * 2 + 2 * kChainThreads * 32 * 4 + 16;
// lean form for many short walks: one operand buffer, no parking slots -> two CTAs per SM
constexpr int kStateSmemLean = kBufElems * 2 + 2 * kHD * kLdS * 2 + kChunk * kLdS * 2 + 16;

// The operands of one step are three flat byte ranges of the item: w | qg | kg (52 224 B), this CTA's u slice (5 120 B) and
// Aqk (9 216 B), already in the padded shapes the MMA fragments are read from. One thread asks the copy engine for them
// (cp.async.bulk, no tensor map needed for a flat range); the bytes are counted on an mbarrier. As 16-byte cp.async requests
// of all 256 threads the same fetch took longer than a step on part of the SMs (the walk of those CTAs ran at 2.6 us per
// step instead of 1.8), which set the duration of the whole kernel.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void state_prefetch(bf16_t* buf, const bf16_t* item, int dv0, uint32_t bar, bool drop) {
  constexpr uint32_t kB1 = 3 * kChunk * kLd * 2, kB2 = kChunk * kLdS * 2, kB3 = kChunk * kLdA * 2;
  static_assert(kB1 % 16 == 0 && kB2 % 16 == 0 && kB3 % 16 == 0 && (kOffU * 2) % 16 == 0 && (kOffA * 2) % 16 == 0 &&
                (kItemElems * 2) % 16 == 0, "bulk copies need 16-byte aligned ranges");
  const uint32_t dst = smem_u32(buf);
  mbar_expect_tx(bar, kB1 + kB2 + kB3);
  if (drop) return;      // tests only: the announced bytes never arrive, the bounded wait of this step runs out
  bulk_g2s(dst, item, kB1, bar);
  bulk_g2s(dst + kB1, item + kOffU + (dv0 / kDv) * (kChunk * kLdS), kB2, bar);
  bulk_g2s(dst + kB1 + kB2, item + kOffA, kB3, bar);
}

// Measurement hook (ojb_gdn_set_trace): when non-null, the CTA of head 0 / column slice 0 / walk 0 records six %globaltimer
// stamps per step — step begin, operands + state copy ready, phase 1 done, v' visible, phase 2 done, step end — from its
// chain warp 0 (words 0-5 of the step's record) and its output warp 0 (words 6-11).
__device__ unsigned long long* g_state_trace = nullptr;

// steps[s] = (chunk, load, save, aux): load 0 carry on / 1 zero / 2 slot A / 3 slot B / 4 initial state aux>>16 - 1;
// save bit 0 slot A, bit 1 slot B; (aux & 0xffff) - 1 = index of a final-state output written after the step.
template <bool LEAN>
__global__ void __launch_bounds__(kStateThreads)
gdn_state_kernel(const bf16_t* __restrict__ scratch, const int32_t* __restrict__ chunks, const int32_t* __restrict__ steps,
                 const int32_t* __restrict__ walk_ptr, const float* __restrict__ init_state, float* __restrict__ final_state,
                 bf16_t* __restrict__ out, int HV, int32_t* status, int wait_ms, int drop_copy) {
  const unsigned long long t_entry = global_timer_ns();
  pdl_begin();
  const int h = blockIdx.x, dv0 = blockIdx.y * kDv;
  const int s_begin = walk_ptr[blockIdx.z], s_end = walk_ptr[blockIdx.z + 1];
  if (s_begin >= s_end) return;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  bf16_t* bufs = reinterpret_cast<bf16_t*>(smem_raw);
  bf16_t* Sb2 = bufs + (LEAN ? 1 : 2) * kBufElems;  // two bf16 copies of the state slice [128 dk][32 dv], alternating by step
  bf16_t* Vn = Sb2 + 2 * kHD * kLdS;               // v' [64][32]
  float* slots = reinterpret_cast<float*>(Vn + kChunk * kLdS);   // [2][32 regs][128 chain threads]
  const int tid = threadIdx.x, lane = tid & 31;
  const bool chain = tid < kChainThreads;           // warps 0-3: state chain; warps 4-7: outputs
  const int warp = (tid >> 5) & 3;                   // index inside the group: 16 chunk rows / 32 dk rows each
  const int gr = lane >> 2, tc = (lane & 3) * 2;
  const int64_t VD = static_cast<int64_t>(HV) * kHD;

  // state slice in mma accumulator layout: warp owns dk rows [32*warp, 32*warp+32): 2 m-tiles x 4 n-tiles x 4
  float S[2][4][4];
#pragma unroll
  for (int a = 0; a < 2; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b)
#pragma unroll
      for (int e = 0; e < 4; ++e) S[a][b][e] = 0.f;

  // The walk's step, chunk and decay entries are staged in shared memory once: read from global inside the loop they are
  // two dependent L2 round trips on the critical path of every step.
  constexpr int kWin = 128;
  __shared__ int4 sm_step[kWin];
  __shared__ int4 sm_chunk[kWin];
  __shared__ float sm_gl[kWin];
  __shared__ __align__(8) uint64_t sm_bar[2];      // operand buffers full (bytes of the bulk copies)
  __shared__ int sm_abort[2];                      // [0] a bounded wait ran out, [1] the limit in milliseconds
  if (tid == 0) {
    mbar_init(smem_u32(&sm_bar[0]), 1);
    mbar_init(smem_u32(&sm_bar[1]), 1);
    sm_abort[0] = 0;
    sm_abort[1] = wait_ms;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int i = tid; i < min(kWin, s_end - s_begin); i += kStateThreads) {
    const int4 st = reinterpret_cast<const int4*>(steps)[s_begin + i];
    sm_step[i] = st;
    sm_chunk[i] = reinterpret_cast<const int4*>(chunks)[st.x];
    sm_gl[i] = *reinterpret_cast<const float*>(scratch + (static_cast<int64_t>(st.x) * HV + h) * kItemElems + kOffGl);
  }
  __syncthreads();
  auto item_of = [&](int s) {
    const int c = s - s_begin < kWin ? sm_step[s - s_begin].x : steps[s * 4];
    return scratch + (static_cast<int64_t>(c) * HV + h) * kItemElems;
  };
  if constexpr (!LEAN) {
    if (tid == 0) state_prefetch(bufs, item_of(s_begin), dv0, smem_u32(&sm_bar[0]), false);
  }

  unsigned long long* trace = g_state_trace;
  const bool tracer = trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (tid == 0 || tid == kChainThreads);
  if (tracer && tid == 0) { trace[0] = t_entry; trace[1] = global_timer_ns(); }
  for (int s = s_begin; s < s_end; ++s) {
    unsigned long long* rec = tracer ? trace + 4 + (static_cast<size_t>(s - s_begin) * 12 + (tid ? 6 : 0)) : nullptr;
    if (rec) rec[0] = global_timer_ns();
    const bool staged = s - s_begin < kWin;
    const int4 st = staged ? sm_step[s - s_begin] : reinterpret_cast<const int4*>(steps)[s];
    const int4 ch = staged ? sm_chunk[s - s_begin] : reinterpret_cast<const int4*>(chunks)[st.x];
    bf16_t* buf = LEAN ? bufs : bufs + ((s - s_begin) & 1) * kBufElems;
    const bf16_t* item = item_of(s);
    // (the buffer asked for here was last read in the step before this one, which ended with a CTA-wide barrier)
    if (tid == 0) {
      if constexpr (LEAN) {
        state_prefetch(buf, item, dv0, smem_u32(&sm_bar[0]), drop_copy && s == s_begin + 1);
      } else if (s + 1 < s_end) {
        state_prefetch(bufs + ((s + 1 - s_begin) & 1) * kBufElems, item_of(s + 1), dv0, smem_u32(&sm_bar[(s + 1 - s_begin) & 1]),
                       drop_copy && s == s_begin);
      }
    }

    bf16_t* Sb = Sb2 + ((s - s_begin) & 1) * (kHD * kLdS);
    if (chain) {
    // ---- choose the incoming state
    if (st.y == 1 || (st.y == 4 && init_state == nullptr)) {
#pragma unroll
      for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b)
#pragma unroll
          for (int e = 0; e < 4; ++e) S[a][b][e] = 0.f;
    } else if (!LEAN && (st.y == 2 || st.y == 3)) {
      const float* sl = slots + (st.y - 2) * (32 * kChainThreads);
#pragma unroll
      for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b)
#pragma unroll
          for (int e = 0; e < 4; ++e) S[a][b][e] = sl[((a * 4 + b) * 4 + e) * kChainThreads + tid];
    } else if (st.y == 4 && init_state != nullptr) {   // (code 4 without an initial state starts from zero, like code 1)
      const float* is = init_state + (static_cast<int64_t>((st.w >> 16) - 1) * HV + h) * (kHD * kHD);
#pragma unroll
      for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int dk = warp * 32 + a * 16 + gr + (e >> 1) * 8, dv = dv0 + b * 8 + tc + (e & 1);
            S[a][b][e] = is[dk * kHD + dv];
          }
    }
    // ---- bf16 copy of the state for the tensor-core operands
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int dk = warp * 32 + a * 16 + gr + half * 8;
          *reinterpret_cast<uint32_t*>(Sb + dk * kLdS + b * 8 + tc) = pack2(S[a][b][half * 2], S[a][b][half * 2 + 1]);
        }
    }
    // this step's operands have landed (the copies of the next step may still be in flight); the wait is bounded, and a CTA
    // whose wait ran out leaves the walk as a whole
    if constexpr (LEAN) mbar_wait(smem_u32(&sm_bar[0]), static_cast<uint32_t>((s - s_begin) & 1), sm_abort);
    else mbar_wait(smem_u32(&sm_bar[(s - s_begin) & 1]), static_cast<uint32_t>(((s - s_begin) >> 1) & 1), sm_abort);
    __syncthreads();
    if (sm_abort[0]) break;
    if (rec) rec[1] = global_timer_ns();

    const bf16_t* Ws = buf;
    const bf16_t* Qg = buf + kChunk * kLd;
    const bf16_t* Kg = buf + 2 * kChunk * kLd;
    const bf16_t* Us = buf + 3 * kChunk * kLd;
    const bf16_t* Aq = Us + kChunk * kLdS;
    const int m0 = warp * 16;
    const int a_row = m0 + (lane & 15), a_col = (lane >> 4) * 8;
    // B operand from [k][n] storage through ldmatrix.trans: lanes 0-15 rows k0..k0+15 at column n0, lanes 16-31 at n0+8
    const int bt_row = lane & 15, bt_col = (lane >> 4) * 8;

    // ---- (1) chain warps: acc_w = w S, v' = u - acc_w -> shared memory; output warps: acc_o = qg S
    //      (16 rows x 32 columns per warp, K = 128)
    float acc[4][4];
#pragma unroll
    for (int b = 0; b < 4; ++b)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[b][e] = 0.f;
    {
      const bf16_t* Am = chain ? Ws : Qg;
#pragma unroll
      for (int ks = 0; ks < kHD / 16; ++ks) {
        uint32_t w0, w1, w2, w3;
        ldsm_x4(smem_u32(Am + a_row * kLd + ks * 16 + a_col), w0, w1, w2, w3);
#pragma unroll
        for (int np = 0; np < 2; ++np) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4_t(smem_u32(Sb + (ks * 16 + bt_row) * kLdS + np * 16 + bt_col), b0, b1, b2, b3);
          mma_bf16(acc[2 * np], w0, w1, w2, w3, b0, b1);
          mma_bf16(acc[2 * np + 1], w0, w1, w2, w3, b2, b3);
        }
      }
    }
    if (chain) {
#pragma unroll
      for (int b = 0; b < 4; ++b)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int r = m0 + gr + half * 8;
          const __nv_bfloat162 u2 = *reinterpret_cast<const __nv_bfloat162*>(Us + r * kLdS + b * 8 + tc);
          const float2 uf = __bfloat1622float2(u2);
          *reinterpret_cast<uint32_t*>(Vn + r * kLdS + b * 8 + tc) = pack2(uf.x - acc[b][half * 2], uf.y - acc[b][half * 2 + 1]);
        }
    }
    if (rec) rec[2] = global_timer_ns();
    __syncthreads();
    if (rec) rec[3] = global_timer_ns();

    if (!chain) {
    // ---- (2) output warps: o = qg S + Aqk v'   (K = 64)
#pragma unroll
    for (int ks = 0; ks < kChunk / 16; ++ks) {
      uint32_t a0, a1, a2, a3;
      ldsm_x4(smem_u32(Aq + a_row * kLdA + ks * 16 + a_col), a0, a1, a2, a3);
#pragma unroll
      for (int np = 0; np < 2; ++np) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(smem_u32(Vn + (ks * 16 + bt_row) * kLdS + np * 16 + bt_col), b0, b1, b2, b3);
        mma_bf16(acc[2 * np], a0, a1, a2, a3, b0, b1);
        mma_bf16(acc[2 * np + 1], a0, a1, a2, a3, b2, b3);
      }
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = m0 + gr + half * 8;
      if (r < ch.y) {
        bf16_t* orow = out + static_cast<int64_t>(ch.x + r) * VD + h * kHD + dv0;
#pragma unroll
        for (int b = 0; b < 4; ++b)
          *reinterpret_cast<uint32_t*>(orow + b * 8 + tc) = pack2(acc[b][half * 2], acc[b][half * 2 + 1]);
      }
    }
    } else {
    // ---- (3) chain warps: S = S e^(G_L) + kg^T v'   (warp owns dk rows 32*warp.., K = 64 chunk rows)
    {
      const float gl = staged ? sm_gl[s - s_begin] : *reinterpret_cast<const float*>(item + kOffGl);
#pragma unroll
      for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b)
#pragma unroll
          for (int e = 0; e < 4; ++e) S[a][b][e] *= gl;
      // A operand = kg^T: A[m = dk][k = row] = kg[row][dk]; ldmatrix.trans over rows of kg
      const int at_row = (lane & 7) + ((lane >> 4) << 3);   // chunk row (k) inside the 16-row step
      const int at_col = ((lane >> 3) & 1) * 8;             // dk offset (m) inside the 16-row tile
#pragma unroll
      for (int ks = 0; ks < kChunk / 16; ++ks) {
        uint32_t b0[2], b1[2], b2[2], b3[2];
#pragma unroll
        for (int np = 0; np < 2; ++np)
          ldsm_x4_t(smem_u32(Vn + (ks * 16 + bt_row) * kLdS + np * 16 + bt_col), b0[np], b1[np], b2[np], b3[np]);
#pragma unroll
        for (int a = 0; a < 2; ++a) {
          uint32_t a0, a1, a2, a3;
          ldsm_x4_t(smem_u32(Kg + (ks * 16 + at_row) * kLd + warp * 32 + a * 16 + at_col), a0, a1, a2, a3);
#pragma unroll
          for (int np = 0; np < 2; ++np) {
            mma_bf16(S[a][2 * np], a0, a1, a2, a3, b0[np], b1[np]);
            mma_bf16(S[a][2 * np + 1], a0, a1, a2, a3, b2[np], b3[np]);
          }
        }
      }
    }
    // ---- park / export the state
    if (!LEAN && (st.z & 3)) {
#pragma unroll
      for (int sl = 0; sl < 2; ++sl)
        if (st.z & (1 << sl)) {
          float* dst = slots + sl * (32 * kChainThreads);
#pragma unroll
          for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b)
#pragma unroll
              for (int e = 0; e < 4; ++e) dst[((a * 4 + b) * 4 + e) * kChainThreads + tid] = S[a][b][e];
        }
    }
    if ((st.w & 0xffff) != 0 && final_state != nullptr) {
      float* fs = final_state + (static_cast<int64_t>((st.w & 0xffff) - 1) * HV + h) * (kHD * kHD);
#pragma unroll
      for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int dk = warp * 32 + a * 16 + gr + (e >> 1) * 8, dv = dv0 + b * 8 + tc + (e & 1);
            fs[dk * kHD + dv] = S[a][b][e];
          }
    }
    }
    if (rec) rec[4] = global_timer_ns();
    __syncthreads();   // everyone is done with Vn and this operand buffer before they are overwritten
    if (rec) rec[5] = global_timer_ns();
  }
  if (sm_abort[0]) {
    if (tid == 0) report_status(status, OJB_DEV_WAIT_TIMEOUT);
    for (int i = 0; i < 200; ++i) __nanosleep(1000);      // copies that were already issued land before the CTA leaves
    __syncthreads();
  }
  if (tracer && tid == 0) trace[2] = global_timer_ns();
}

// ------------------------------------------------------------------------------------------------------ gated RMSNorm
// one warp per (row, head); 4 dims per lane. x row of packed row n is x[inv[n]] (inv may be null: identity).
__global__ void __launch_bounds__(256)
gated_rmsnorm_kernel(const bf16_t* __restrict__ x, const int32_t* __restrict__ inv, const bf16_t* __restrict__ proj,
                     const bf16_t* __restrict__ w, bf16_t* __restrict__ out, int64_t items, int HV, int zoff, int P, float eps) {
  pdl_begin();
  const int64_t it = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (it >= items) return;
  const int lane = threadIdx.x & 31;
  const int64_t n = it / HV;
  const int h = static_cast<int>(it - n * HV);
  const int64_t srow = inv ? inv[n] : n;
  const int d0 = lane * 4;
  const uint2 xa = *reinterpret_cast<const uint2*>(x + (srow * HV + h) * kHD + d0);
  const uint2 za = *reinterpret_cast<const uint2*>(proj + n * P + zoff + h * kHD + d0);
  const uint2 wa = __ldg(reinterpret_cast<const uint2*>(w + d0));
  const bf16_t* xb = reinterpret_cast<const bf16_t*>(&xa);
  const bf16_t* zb = reinterpret_cast<const bf16_t*>(&za);
  const bf16_t* wb = reinterpret_cast<const bf16_t*>(&wa);
  float xv[4], ss = 0.f;
#pragma unroll
  for (int e = 0; e < 4; ++e) { xv[e] = bf2f(xb[e]); ss += xv[e] * xv[e]; }
  ss = warp_sum(ss);
  const float rstd = 1.0f / sqrtf(ss / static_cast<float>(kHD) + eps);
  uint2 oa;
  bf16_t* ob = reinterpret_cast<bf16_t*>(&oa);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float z = bf2f(zb[e]);
    ob[e] = f2bf(((xv[e] * rstd) * bf2f(wb[e])) * z * sigmoid_f(z));
  }
  *reinterpret_cast<uint2*>(out + n * (static_cast<int64_t>(HV) * kHD) + h * kHD + d0) = oa;
}

}  // namespace
}  // namespace ojb

using namespace ojb;

extern "C" int ojb_gdn_prep(const void* proj, const int32_t* hist, const int32_t* rep_ptr, const int32_t* rep_pos,
                            int64_t n_slots, const void* convw, const void* A_log, const void* dt_bias, void* q, void* k,
                            void* v, float* g, void* beta, int64_t N, int64_t KD, int64_t VD, int64_t HV, int64_t HK,
                            int32_t l2norm, ojb_stream_t stream) {
  if (N == 0) return OJB_OK;
  OJB_REQUIRE(proj && hist && convw && A_log && dt_bias && q && k && v && g && beta && N > 0);
  // every row of proj must start on a 16-byte boundary (the kernel reads 16 bytes at a time): (2KD + 2VD + 2HV) % 8 == 0
  OJB_REQUIRE(HK > 0 && HV > 0 && KD == HK * kHD && VD == HV * kHD && HV <= 256 && HV % 4 == 0);
  const int C = static_cast<int>(2 * KD + VD);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned gx = static_cast<unsigned>(ceil_div(C / 8, 256));
  if (rep_ptr != nullptr) {
    OJB_REQUIRE(rep_pos != nullptr && n_slots > 0);
    dim3 grid(gx, static_cast<unsigned>(N + ceil_div(n_slots, 16)));
    launch_kernel(gdn_prep_kernel<true>, dim3(grid), dim3(256), 0, st, static_cast<const bf16_t*>(proj), reinterpret_cast<const int4*>(hist), rep_ptr, rep_pos,
                                                static_cast<const bf16_t*>(convw), static_cast<const bf16_t*>(A_log),
                                                static_cast<const bf16_t*>(dt_bias), static_cast<bf16_t*>(q), static_cast<bf16_t*>(k),
                                                static_cast<bf16_t*>(v), g, static_cast<bf16_t*>(beta), static_cast<int>(N),
                                                static_cast<int>(KD), static_cast<int>(VD), static_cast<int>(HV), l2norm ? 1 : 0);
  } else {
    dim3 grid(gx, static_cast<unsigned>(N));
    launch_kernel(gdn_prep_kernel<false>, dim3(grid), dim3(256), 0, st, static_cast<const bf16_t*>(proj), reinterpret_cast<const int4*>(hist), nullptr, nullptr,
                                                 static_cast<const bf16_t*>(convw), static_cast<const bf16_t*>(A_log),
                                                 static_cast<const bf16_t*>(dt_bias), static_cast<bf16_t*>(q), static_cast<bf16_t*>(k),
                                                 static_cast<bf16_t*>(v), g, static_cast<bf16_t*>(beta), static_cast<int>(N),
                                                 static_cast<int>(KD), static_cast<int>(VD), static_cast<int>(HV), l2norm ? 1 : 0);
  }
  return launch_status(cudaGetLastError());
}

extern "C" int ojb_gdn_set_trace(uint64_t* records) {
  unsigned long long* p = reinterpret_cast<unsigned long long*>(records);
  return launch_status(cudaMemcpyToSymbol(ojb::g_state_trace, &p, sizeof(p)));
}

namespace ojb {
namespace {
// Two short chunks per CTA only when one CTA per chunk would not fit the GPU in a single wave (three CTAs per SM):
// with room to spare the chunks finish sooner side by side. OJB_GDN_PAIR = 0 / 1 forces the choice (measurements).
int intra_pairing(int64_t n_chunks, int64_t HV) {
  static const int forced = [] { const char* e = getenv("OJB_GDN_PAIR"); return e ? atoi(e) : -1; }();
  if (forced >= 0) return forced != 0 ? 1 : 0;      // 1: pair whenever two short chunks exist; 0: never
  const int sms = device_sm_count();
  const int slots = 3 * (sms > 0 ? sms : 148);
  // the table may have empty slots: the kernel counts the chunks that exist and compares with the CTA slots itself
  return n_chunks * HV > slots ? slots : 0;
}
// Opt-in shared-memory sizes of the two (three with the level form) kernels, once per device.
bool gdn_raise_limits(bool lean_too) {
  static int s_intra[kMaxDevices] = {}, s_intra_f[kMaxDevices] = {}, s_state[kMaxDevices] = {}, s_lean[kMaxDevices] = {};
  return raise_smem_limit(gdn_intra_kernel<false>, static_cast<int>(kIntraSmem), s_intra) &&
         raise_smem_limit(gdn_intra_kernel<true>, static_cast<int>(kIntraSmem), s_intra_f) &&
         raise_smem_limit(gdn_state_kernel<false>, static_cast<int>(kStateSmem), s_state) &&
         (!lean_too || raise_smem_limit(gdn_state_kernel<true>, static_cast<int>(kStateSmemLean), s_lean));
}
}  // namespace
}  // namespace ojb

extern "C" int64_t ojb_gdn_scratch_bytes(int64_t n_chunks, int64_t HV) { return n_chunks * HV * kItemElems * 2; }

extern "C" int ojb_gdn_chunked(const void* q, const void* k, const void* v, const float* g, const void* beta,
                               const int32_t* chunks, int64_t n_chunks, const int32_t* steps, const int32_t* walk_ptr,
                               int64_t n_walks, const float* init_state, float* final_state, void* scratch, void* out,
                               int64_t HK, int64_t HV, float scale, int32_t* status, ojb_stream_t stream) {
  if (n_chunks == 0 || n_walks == 0) return OJB_OK;
  OJB_REQUIRE(q && k && v && g && beta && chunks && steps && walk_ptr && scratch && out);
  OJB_REQUIRE(HK > 0 && HV > 0 && HV % HK == 0 && n_chunks > 0 && n_walks > 0 && n_walks <= 65535 && HV <= 65535);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (!gdn_raise_limits(false)) return OJB_ERR_LAUNCH;
  launch_kernel(gdn_intra_kernel<false>, dim3(dim3(static_cast<unsigned>(n_chunks), static_cast<unsigned>(HV))), dim3(kIntraThreads), kIntraSmem, st, 
      static_cast<const bf16_t*>(q), static_cast<const bf16_t*>(k), static_cast<const bf16_t*>(v), g,
      static_cast<const bf16_t*>(beta), chunks, static_cast<bf16_t*>(scratch), static_cast<int>(HK), static_cast<int>(HV), scale,
      intra_pairing(n_chunks, HV), PrepSrc{});
  if (cudaGetLastError() != cudaSuccess) return OJB_ERR_LAUNCH;
  launch_kernel(gdn_state_kernel<false>, dim3(dim3(static_cast<unsigned>(HV), kHD / kDv, static_cast<unsigned>(n_walks))), dim3(kStateThreads), kStateSmem, st, 
      static_cast<const bf16_t*>(scratch), chunks, steps, walk_ptr, init_state, final_state, static_cast<bf16_t*>(out),
      static_cast<int>(HV), status, gemm_wait_limit_ms(), gemm_drop_copy());
  return launch_status(cudaGetLastError());
}

extern "C" int ojb_gdn_chunked_proj(const void* proj, const int32_t* hist, const void* convw, const void* A_log,
                                    const void* dt_bias, const int32_t* chunks, int64_t n_chunks, const int32_t* steps,
                                    const int32_t* walk_ptr, int64_t n_walks, const float* init_state, float* final_state,
                                    void* scratch, void* out, int64_t KD, int64_t VD, int64_t HK, int64_t HV, float scale,
                                    int32_t* status, ojb_stream_t stream) {
  if (n_chunks == 0 || n_walks == 0) return OJB_OK;
  OJB_REQUIRE(proj && hist && convw && A_log && dt_bias && chunks && steps && walk_ptr && scratch && out);
  OJB_REQUIRE(HK > 0 && HV > 0 && HV % HK == 0 && KD == HK * kHD && VD == HV * kHD && n_chunks > 0 && n_walks > 0 &&
              n_walks <= 65535 && HV <= 65535 && HV % 4 == 0);      // HV % 4: 16-byte aligned rows of proj
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (!gdn_raise_limits(false)) return OJB_ERR_LAUNCH;
  PrepSrc ps{static_cast<const bf16_t*>(proj), reinterpret_cast<const int4*>(hist), static_cast<const bf16_t*>(convw),
             static_cast<const bf16_t*>(A_log), static_cast<const bf16_t*>(dt_bias), static_cast<int>(2 * KD + 2 * VD + 2 * HV)};
  launch_kernel(gdn_intra_kernel<true>, dim3(static_cast<unsigned>(n_chunks), static_cast<unsigned>(HV)), dim3(kIntraThreads),
                kIntraSmem, st, static_cast<const bf16_t*>(nullptr), static_cast<const bf16_t*>(nullptr),
                static_cast<const bf16_t*>(nullptr), static_cast<const float*>(nullptr), static_cast<const bf16_t*>(nullptr), chunks,
                static_cast<bf16_t*>(scratch), static_cast<int>(HK), static_cast<int>(HV), scale, intra_pairing(n_chunks, HV), ps);
  if (cudaGetLastError() != cudaSuccess) return OJB_ERR_LAUNCH;
  launch_kernel(gdn_state_kernel<false>, dim3(static_cast<unsigned>(HV), kHD / kDv, static_cast<unsigned>(n_walks)),
                dim3(kStateThreads), kStateSmem, st, static_cast<const bf16_t*>(scratch), chunks, steps, walk_ptr, init_state,
                final_state, static_cast<bf16_t*>(out), static_cast<int>(HV), status, gemm_wait_limit_ms(), gemm_drop_copy());
  return launch_status(cudaGetLastError());
}

extern "C" int ojb_gated_rmsnorm(const void* x, const int32_t* inv, const void* proj, const void* w, void* out, int64_t N,
                                 int64_t HV, int64_t HD, int64_t zoff, int64_t P, float eps, ojb_stream_t stream) {
  if (N == 0) return OJB_OK;
  OJB_REQUIRE(x && proj && w && out && N > 0 && HV > 0 && HD == kHD && zoff >= 0 && zoff + HV * HD <= P && zoff % 4 == 0 && P % 4 == 0);
  const int64_t items = N * HV;
  launch_kernel(gated_rmsnorm_kernel, dim3(static_cast<unsigned>(ceil_div(items, 8))), dim3(256), 0, static_cast<cudaStream_t>(stream), 
      static_cast<const bf16_t*>(x), inv, static_cast<const bf16_t*>(proj), static_cast<const bf16_t*>(w), static_cast<bf16_t*>(out),
      items, static_cast<int>(HV), static_cast<int>(zoff), static_cast<int>(P), eps);
  return launch_status(cudaGetLastError());
}

// ------------------------------------------------------------------------------------- scratch-free entry point
// Same two kernels as ojb_gdn_chunked, but the (chunk, head) scratch items live in a fixed array inside this library's
// device image instead of a buffer the caller has to allocate. It exists for callers that must not allocate device
// memory around the call: code running under a frozen memory plan (a CUDA-graph memory pool that is already sized, an
// inference server whose allocator is locked after start-up) or host code without access to an allocator at all.
namespace ojb {
namespace {
constexpr int64_t kStaticItems = 1024;   // (chunk-table entries) x (value heads) that fit: 1024 x 81 936 B = 80 MiB per GPU
static __device__ __align__(256) unsigned char g_gdn_static_scratch[kStaticItems * kItemElems * 2];
void* g_static_scratch_addr[kMaxDevices] = {nullptr};
}  // namespace
}  // namespace ojb

extern "C" int64_t ojb_gdn_static_max_items(void) { return ojb::kStaticItems; }

extern "C" int ojb_gdn_chunked_static(const void* q, const void* k, const void* v, const float* g, const void* beta,
                                      const int32_t* chunks, int64_t n_chunks, const int32_t* steps, const int32_t* walk_ptr,
                                      int64_t n_walks, const float* init_state, float* final_state, void* out, int64_t HK,
                                      int64_t HV, float scale, int32_t* status, ojb_stream_t stream) {
  if (n_chunks == 0 || n_walks == 0) return OJB_OK;
  OJB_REQUIRE(q && k && v && g && beta && chunks && steps && walk_ptr && out);
  OJB_REQUIRE(HK > 0 && HV > 0 && HV % HK == 0 && n_chunks > 0 && n_walks > 0 && n_walks <= 65535 && HV <= 65535);
  if (n_chunks * HV > kStaticItems) return OJB_ERR_LIMIT;   // the fixed array holds at most kStaticItems items
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return OJB_ERR_LAUNCH;
  if (g_static_scratch_addr[dev] == nullptr) {
    // Once per device, with that device current: the array's name is only a host-side handle, the kernels need the
    // device address. Also raises the shared-memory limits of the two kernels for this device.
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_gdn_static_scratch) != cudaSuccess || p == nullptr) return OJB_ERR_LAUNCH;
    if (cudaFuncSetAttribute(gdn_intra_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kIntraSmem) != cudaSuccess ||
        cudaFuncSetAttribute(gdn_state_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kStateSmem) != cudaSuccess)
      return OJB_ERR_LAUNCH;
    g_static_scratch_addr[dev] = p;
  }
  bf16_t* scratch = static_cast<bf16_t*>(g_static_scratch_addr[dev]);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // Nothing in the array has to start at zero: the first kernel overwrites every byte of every item that the second one
  // reads (items of unused chunk-table entries are neither written nor read).
  launch_kernel(gdn_intra_kernel<false>, dim3(dim3(static_cast<unsigned>(n_chunks), static_cast<unsigned>(HV))), dim3(kIntraThreads), kIntraSmem, st, 
      static_cast<const bf16_t*>(q), static_cast<const bf16_t*>(k), static_cast<const bf16_t*>(v), g,
      static_cast<const bf16_t*>(beta), chunks, scratch, static_cast<int>(HK), static_cast<int>(HV), scale,
      intra_pairing(n_chunks, HV), PrepSrc{});
  if (cudaGetLastError() != cudaSuccess) return OJB_ERR_LAUNCH;
  launch_kernel(gdn_state_kernel<false>, dim3(dim3(static_cast<unsigned>(HV), kHD / kDv, static_cast<unsigned>(n_walks))), dim3(kStateThreads), kStateSmem, st, 
      scratch, chunks, steps, walk_ptr, init_state, final_state, static_cast<bf16_t*>(out), static_cast<int>(HV), status, gemm_wait_limit_ms(), gemm_drop_copy());
  return launch_status(cudaGetLastError());
}

// --------------------------------------------------------------------------------------------- level-parallel tree pass
// Same kernels, but the state pass runs once per tree level: all walks of a level (one per node of that level) start from
// the end state that their parent's walk exported to `states` in the previous launch, so sibling nodes run side by side
// instead of one after the other inside one CTA column. levels[l] .. levels[l+1] (host array) are the walk indices of level l.
extern "C" int ojb_gdn_chunked_levels(const void* q, const void* k, const void* v, const float* g, const void* beta,
                                      const int32_t* chunks, int64_t n_chunks, const int32_t* steps, const int32_t* walk_ptr,
                                      const int32_t* levels, int64_t n_levels, float* states, void* scratch, void* out,
                                      int64_t HK, int64_t HV, float scale, int32_t* status, ojb_stream_t stream) {
  if (n_chunks == 0 || n_levels == 0) return OJB_OK;
  OJB_REQUIRE(q && k && v && g && beta && chunks && steps && walk_ptr && levels && states && scratch && out);
  OJB_REQUIRE(HK > 0 && HV > 0 && HV % HK == 0 && n_chunks > 0 && n_levels > 0 && n_levels <= 16 && HV <= 65535);
  for (int64_t l = 0; l < n_levels; ++l) OJB_REQUIRE(levels[l + 1] >= levels[l] && levels[l + 1] - levels[l] <= 65535);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (!gdn_raise_limits(true)) return OJB_ERR_LAUNCH;
  launch_kernel(gdn_intra_kernel<false>, dim3(dim3(static_cast<unsigned>(n_chunks), static_cast<unsigned>(HV))), dim3(kIntraThreads), kIntraSmem, st, 
      static_cast<const bf16_t*>(q), static_cast<const bf16_t*>(k), static_cast<const bf16_t*>(v), g,
      static_cast<const bf16_t*>(beta), chunks, static_cast<bf16_t*>(scratch), static_cast<int>(HK), static_cast<int>(HV), scale,
      intra_pairing(n_chunks, HV), PrepSrc{});
  if (cudaGetLastError() != cudaSuccess) return OJB_ERR_LAUNCH;
  for (int64_t l = 0; l < n_levels; ++l) {
    const int nw = levels[l + 1] - levels[l];
    if (nw == 0) continue;
    if (nw > 1) {   // many short walks: the lean form fits two CTAs per SM
      launch_kernel(gdn_state_kernel<true>, dim3(dim3(static_cast<unsigned>(HV), kHD / kDv, static_cast<unsigned>(nw))), dim3(kStateThreads), kStateSmemLean, st, 
          static_cast<const bf16_t*>(scratch), chunks, steps, walk_ptr + levels[l], states, states, static_cast<bf16_t*>(out),
          static_cast<int>(HV), status, gemm_wait_limit_ms(), gemm_drop_copy());
    } else {
      launch_kernel(gdn_state_kernel<false>, dim3(dim3(static_cast<unsigned>(HV), kHD / kDv, 1)), dim3(kStateThreads), kStateSmem, st, 
          static_cast<const bf16_t*>(scratch), chunks, steps, walk_ptr + levels[l], states, states, static_cast<bf16_t*>(out),
          static_cast<int>(HV), status, gemm_wait_limit_ms(), gemm_drop_copy());
    }
    if (cudaGetLastError() != cudaSuccess) return OJB_ERR_LAUNCH;
  }
  return OJB_OK;
}
