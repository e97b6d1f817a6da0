// Ancestor-masked (prefix-tree) GQA flash attention with the sigmoid output gate fused in.
//
// One CTA = (kv head, group of GQ query heads, 16 query rows); two warps per query head, each taking every other visible key
// block (their partial softmax states are merged through shared memory at the end), all warps sharing the K / V tiles of
// their kv head. Keys are visited in blocks of 32; a block is skipped when none of the 16 rows can see any of its keys.
// The mask comes either from the packed visibility words vbits[N, N/32] of the reference layout or from three half-open
// key ranges per row (root, own question stem, own leaf up to the row itself) — the second form needs O(N) memory instead
// of O(N^2). Q K^T and P V run on the tensor cores (mma.sync m16n8k16 bf16, fp32 accumulate), the softmax is the online
// form in the exp2 domain (ex2.approx); K / V tiles are double-buffered with cp.async. OJB_ATTN_SPLIT=1 in the environment
// selects one warp per head (half the shared memory, two CTAs per SM); measured slower than the default of two on both
// benchmark trees (45 vs 44 us at 544 rows with 3 / 6 heads per CTA, 18.6 vs 17.7 us at 288).
#include "common.cuh"

namespace ojb {
namespace {

constexpr int kRows = 16;     // query rows per CTA
constexpr int kKeys = 32;     // keys per block = one visibility word

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
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

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// bits of keys [32*kb, 32*kb+32) that fall in [lo, hi)
__device__ __forceinline__ uint32_t range_word(int lo, int hi, int kb) {
  const int a = max(lo - kb * 32, 0), b = min(hi - kb * 32, 32);
  if (a >= b) return 0u;
  const uint32_t upto_b = b == 32 ? 0xffffffffu : ((1u << b) - 1u);
  return upto_b & ~((1u << a) - 1u);
}

// kSplit = warps per query head, interleaved over the visible key blocks (1 or 2)
template <int D, int kSplit>
__global__ void __launch_bounds__(192 * kSplit)
tree_attn_kernel(const bf16_t* __restrict__ qt, const bf16_t* __restrict__ kt, const bf16_t* __restrict__ vt,
                 const bf16_t* __restrict__ gate, const int32_t* __restrict__ vbits, const int32_t* __restrict__ krange,
                 bf16_t* __restrict__ y, int N, int HQ, int HKV, int GQ, float scale_log2e) {
  pdl_begin();
  constexpr int kLd = D + 8;                    // padded shared-memory row (bf16)
  const int nheads = GQ;                        // query heads of this CTA; warp = split * GQ + head
  const int G = HQ / HKV;                       // query heads per kv head
  const int groups = G / GQ;
  const int kvh = blockIdx.x / groups, grp = blockIdx.x - kvh * groups;
  const int r0 = blockIdx.y * kRows;
  const int NW = N >> 5;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nthreads = nheads * kSplit * 32;
  const int head = warp % nheads, split = warp / nheads;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  bf16_t* Qs = reinterpret_cast<bf16_t*>(smem_raw);          // [GQ][16][kLd]
  bf16_t* KV = Qs + nheads * kRows * kLd;                     // 2 stages x kSplit key blocks x (K [32][kLd] | V [32][kLd])
  uint32_t* words = reinterpret_cast<uint32_t*>(KV + 2 * kSplit * 2 * kKeys * kLd);   // [16][NW] visibility words
  int* vis_list = reinterpret_cast<int*>(words + kRows * NW);            // visible key blocks, then their count at [NW]

  // ---- visibility words of this row block
  for (int i = tid; i < kRows * NW; i += nthreads) {
    const int r = i / NW, kb = i - r * NW;
    uint32_t w;
    if (vbits != nullptr) {
      w = static_cast<uint32_t>(vbits[static_cast<int64_t>(r0 + r) * NW + kb]);
    } else {
      const int* kr = krange + static_cast<int64_t>(r0 + r) * 8;
      w = range_word(kr[5], kr[0], kb) | range_word(kr[1], kr[2], kb) | range_word(kr[3], kr[4], kb);
    }
    words[r * NW + kb] = w;
  }
  // ---- Q rows of the GQ heads -> shared memory
  const int hq0 = kvh * G + grp * GQ;
  for (int i = tid; i < nheads * kRows * (D / 8); i += nthreads) {
    const int w = i / (kRows * (D / 8)), rem = i - w * (kRows * (D / 8));
    const int r = rem / (D / 8), cv = (rem - r * (D / 8)) * 8;
    *reinterpret_cast<uint4*>(Qs + (w * kRows + r) * kLd + cv) =
        *reinterpret_cast<const uint4*>(qt + (static_cast<int64_t>(hq0 + w) * N + r0 + r) * D + cv);
  }
  __syncthreads();
  if (warp == 0) {   // ordered list of key blocks that at least one row sees
    int count = 0;
    for (int base = 0; base < NW; base += 32) {
      const int kb = base + lane;
      uint32_t any = 0;
      if (kb < NW)
        for (int r = 0; r < kRows; ++r) any |= words[r * NW + kb];
      const uint32_t bal = __ballot_sync(0xffffffffu, any != 0);
      if (any != 0) vis_list[count + __popc(bal & ((1u << lane) - 1u))] = kb;
      count += __popc(bal);
    }
    if (lane == 0) vis_list[NW] = count;
  }
  __syncthreads();
  const int nvis = vis_list[NW];

  const bf16_t* kbase = kt + static_cast<int64_t>(kvh) * N * D;
  const bf16_t* vbase = vt + static_cast<int64_t>(kvh) * N * D;
  // stage = kSplit consecutive entries of the visible-block list, one per split
  auto prefetch = [&](int stage, int it) {
    for (int sp = 0; sp < kSplit; ++sp) {
      const int li = it * kSplit + sp;
      if (li >= nvis) break;
      const int kb = vis_list[li];
      bf16_t* ks = KV + (stage * kSplit + sp) * (2 * kKeys * kLd);
      bf16_t* vs = ks + kKeys * kLd;
      const bf16_t* ksrc = kbase + static_cast<int64_t>(kb) * (kKeys * D);
      const bf16_t* vsrc = vbase + static_cast<int64_t>(kb) * (kKeys * D);
      for (int i = tid; i < kKeys * (D / 8); i += nthreads) {      // the K and the V piece at the same (row, column)
        const int r = i / (D / 8), cv = (i - r * (D / 8)) * 8;
        cp_async16(smem_u32(ks + r * kLd + cv), ksrc + r * D + cv);
        cp_async16(smem_u32(vs + r * kLd + cv), vsrc + r * D + cv);
      }
    }
  };
  const int niter = (nvis + kSplit - 1) / kSplit;
  if (niter > 0) prefetch(0, 0);
  cp_async_commit();

  float o[D / 8][4];
#pragma unroll
  for (int nt = 0; nt < D / 8; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[nt][e] = 0.f;
  float m_run[2] = {-1e30f, -1e30f}, l_run[2] = {0.f, 0.f};
  const int gr = lane >> 2, tc = (lane & 3) * 2;
  const bf16_t* Qw = Qs + head * kRows * kLd;
  const int a_row = lane & 15, a_col = (lane >> 4) * 8;
  const int b_row = (lane & 7) + ((lane >> 4) << 3), b_col = ((lane >> 3) & 1) * 8;
  const int bt_row = lane & 15, bt_col = (lane >> 4) * 8;
  // shared-memory byte addresses of this lane's fragment rows, converted once: inside the loops only constants are added
  const uint32_t q_lane = smem_u32(Qw + a_row * kLd + a_col);
  const uint32_t k_lane_off = static_cast<uint32_t>(b_row * kLd + b_col) * 2u, v_lane_off = static_cast<uint32_t>(bt_row * kLd + bt_col) * 2u;

  for (int it = 0; it < niter; ++it) {
    if (it + 1 < niter) prefetch((it + 1) & 1, it + 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const int li = it * kSplit + split;
    if (li < nvis) {
    const int kb = vis_list[li];
    const bf16_t* ks = KV + ((it & 1) * kSplit + split) * (2 * kKeys * kLd);
    const bf16_t* vs = ks + kKeys * kLd;
    const uint32_t k_lane = smem_u32(ks) + k_lane_off, v_lane = smem_u32(vs) + v_lane_off;
    // ---- S = Q K^T  (16 x 32)
    float s[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t a0, a1, a2, a3;     // (keeping the Q fragments in registers across key blocks was measured: no gain)
      ldsm_x4(q_lane + kk * 32, a0, a1, a2, a3);
#pragma unroll
      for (int np = 0; np < 2; ++np) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(k_lane + (np * 16 * kLd + kk * 16) * 2, b0, b1, b2, b3);
        mma_bf16(s[2 * np], a0, a1, a2, a3, b0, b1);
        mma_bf16(s[2 * np + 1], a0, a1, a2, a3, b2, b3);
      }
    }
    // ---- mask, online softmax
    const uint32_t w_lo = words[gr * NW + kb], w_hi = words[(gr + 8) * NW + kb];
    float mx[2] = {m_run[0], m_run[1]};
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int col = nt * 8 + tc + (e & 1);
        const bool vis = ((e < 2 ? w_lo : w_hi) >> col) & 1u;
        s[nt][e] = vis ? s[nt][e] * scale_log2e : -INFINITY;
        mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
      }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
    }
    float alpha[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      alpha[h] = ex2_approx(m_run[h] - mx[h]);
      m_run[h] = mx[h];
      l_run[h] *= alpha[h];          // per-thread partial row sums: the four lanes of a row are added once, at the end
    }
    uint32_t pa[2][4];   // P as A fragments of the two 16-key steps
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      float p[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        p[e] = ex2_approx(s[nt][e] - mx[e >> 1]);
        l_run[e >> 1] += p[e];
      }
      pa[nt >> 1][(nt & 1) * 2 + 0] = pack2(p[0], p[1]);
      pa[nt >> 1][(nt & 1) * 2 + 1] = pack2(p[2], p[3]);
    }
    if (alpha[0] != 1.f || alpha[1] != 1.f) {      // the running maxima settle after the first blocks
#pragma unroll
      for (int nt = 0; nt < D / 8; ++nt) {
        o[nt][0] *= alpha[0]; o[nt][1] *= alpha[0]; o[nt][2] *= alpha[1]; o[nt][3] *= alpha[1];
      }
    }
    // ---- O += P V  (K = 32 keys in two steps, N = D)
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
      for (int np = 0; np < D / 16; ++np) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(v_lane + (kk * 16 * kLd + np * 16) * 2, b0, b1, b2, b3);
        mma_bf16(o[2 * np], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b0, b1);
        mma_bf16(o[2 * np + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b2, b3);
      }
    }
    }
    __syncthreads();   // the stage is free for the prefetch issued in the next iteration
  }
  cp_async_wait<0>();
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
  // ---- merge the partial softmax states of the two splits of a head (split 1 hands over through the K / V buffers)
  if constexpr (kSplit == 2) {
    float* xch = reinterpret_cast<float*>(KV) + static_cast<size_t>(head) * (32 * (D / 2 + 4));
    if (split == 1) {
#pragma unroll
      for (int nt = 0; nt < D / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) xch[(nt * 4 + e) * 32 + lane] = o[nt][e];
      xch[(D / 2 + 0) * 32 + lane] = m_run[0];
      xch[(D / 2 + 1) * 32 + lane] = m_run[1];
      xch[(D / 2 + 2) * 32 + lane] = l_run[0];
      xch[(D / 2 + 3) * 32 + lane] = l_run[1];
    }
    __syncthreads();
    if (split == 1) return;
    float f0[2], f1[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float m1 = xch[(D / 2 + h) * 32 + lane], l1 = xch[(D / 2 + 2 + h) * 32 + lane];
      const float m = fmaxf(m_run[h], m1);
      f0[h] = ex2_approx(m_run[h] - m);
      f1[h] = ex2_approx(m1 - m);
      l_run[h] = l_run[h] * f0[h] + l1 * f1[h];
    }
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[nt][e] = o[nt][e] * f0[e >> 1] + xch[(nt * 4 + e) * 32 + lane] * f1[e >> 1];
  }
  // ---- y = bf16(bf16(O / l) * bf16(sigmoid(gate)))
  const int hq = hq0 + head;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int row = r0 + gr + h * 8;
    const float inv_l = l_run[h] > 0.f ? 1.0f / l_run[h] : 0.f;
    const int64_t off = static_cast<int64_t>(row) * HQ * D + static_cast<int64_t>(hq) * D;
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt) {
      const float2 gv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gate + off + nt * 8 + tc));
      const float a0 = round_bf(o[nt][h * 2] * inv_l), a1 = round_bf(o[nt][h * 2 + 1] * inv_l);
      const float s0 = round_bf(__fdividef(1.0f, 1.0f + __expf(-gv.x))), s1 = round_bf(__fdividef(1.0f, 1.0f + __expf(-gv.y)));
      *reinterpret_cast<uint32_t*>(y + off + nt * 8 + tc) = pack2(a0 * s0, a1 * s1);
    }
  }
}

template <int D, int kSplit>
int launch_attn(const void* qt, const void* kt, const void* vt, const void* gate, const int32_t* vbits, const int32_t* krange,
                void* y, int64_t N, int64_t HQ, int64_t HKV, int64_t GQ, float scale, cudaStream_t st) {
  constexpr int kLd = D + 8;
  const int NW = static_cast<int>(N / 32);
  const size_t smem = (GQ * kRows * kLd + 2 * kSplit * 2 * kKeys * kLd) * 2 + kRows * NW * 4 + (NW + 1) * 4;
  if (smem > 227 * 1024) return OJB_ERR_LIMIT;
  auto kern = tree_attn_kernel<D, kSplit>;
  static int smem_set[kMaxDevices] = {};
  if (!raise_smem_limit(kern, static_cast<int>(smem), smem_set)) return OJB_ERR_LAUNCH;
  const int G = static_cast<int>(HQ / HKV);
  dim3 grid(static_cast<unsigned>(HKV * (G / GQ)), static_cast<unsigned>(N / kRows));
  launch_kernel(kern, dim3(grid), dim3(static_cast<unsigned>(GQ * kSplit * 32)), smem, st, static_cast<const bf16_t*>(qt), static_cast<const bf16_t*>(kt),
                                                          static_cast<const bf16_t*>(vt), static_cast<const bf16_t*>(gate), vbits,
                                                          krange, static_cast<bf16_t*>(y), static_cast<int>(N), static_cast<int>(HQ),
                                                          static_cast<int>(HKV), static_cast<int>(GQ), scale * 1.4426950408889634f);
  return launch_status(cudaGetLastError());
}

}  // namespace
}  // namespace ojb

using namespace ojb;

extern "C" int ojb_tree_attn(const void* qt, const void* kt, const void* vt, const void* gate, const int32_t* vbits,
                             const int32_t* krange, void* y, int64_t N, int64_t HQ, int64_t HKV, int64_t D, int64_t gq,
                             float scale, ojb_stream_t stream) {
  if (N == 0) return OJB_OK;
  OJB_REQUIRE(qt && kt && vt && gate && y && (vbits || krange) && N > 0 && N % 32 == 0);
  OJB_REQUIRE(HQ > 0 && HKV > 0 && HQ % HKV == 0 && gq >= 1 && gq <= 6 && (HQ / HKV) % gq == 0);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  static int split_env = -1;
  if (split_env < 0) {
    const char* e = getenv("OJB_ATTN_SPLIT");
    split_env = e ? atoi(e) : 0;
  }
  const int split = split_env == 1 || split_env == 2 ? split_env : 2;
  if (split == 1) {
    if (D == 256) return launch_attn<256, 1>(qt, kt, vt, gate, vbits, krange, y, N, HQ, HKV, gq, scale, st);
    if (D == 128) return launch_attn<128, 1>(qt, kt, vt, gate, vbits, krange, y, N, HQ, HKV, gq, scale, st);
    if (D == 64) return launch_attn<64, 1>(qt, kt, vt, gate, vbits, krange, y, N, HQ, HKV, gq, scale, st);
    return OJB_ERR_ARG;
  }
  if (D == 256) return launch_attn<256, 2>(qt, kt, vt, gate, vbits, krange, y, N, HQ, HKV, gq, scale, st);
  if (D == 128) return launch_attn<128, 2>(qt, kt, vt, gate, vbits, krange, y, N, HQ, HKV, gq, scale, st);
  if (D == 64) return launch_attn<64, 2>(qt, kt, vt, gate, vbits, krange, y, N, HQ, HKV, gq, scale, st);
  return OJB_ERR_ARG;
}
