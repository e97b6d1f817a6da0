// Prefix-tree GQA attention on the tcgen05 tensor cores (head dim 256), with the sigmoid output gate fused in.
//
// One CTA = one kv head x 16 query rows x ALL query heads of that kv head: the G <= 6 heads share K and V, so their rows are
// stacked into one operand tile (row 16 w + r = head w, query row r; M = 128 in the instruction, the rows past 16 G are never
// looked at) and every K / V tile that reaches the SM is used by all of them. Visibility is decided per 64 keys: a 64-key
// block is skipped when none of the 16 rows sees any of its keys (the mask is three half-open key ranges per row: root, own
// question stem, own leaf up to the row itself). The visible blocks are taken two at a time — any two, they need not be
// neighbours — so every tensor-core product covers 128 keys (an M = 128 instruction costs the same for 64 columns as for 128).
//
//   S = Q K^T   tcgen05.mma, M = 128, N = 128, K = 256: Q and the two K blocks [64 x 256] are K-major 128-byte-swizzled tiles
//               written by TMA (the two blocks land as the two halves of one [128 x 256] operand); S lives in tensor memory
//               (two 128-column buffers, so the product of the next pair runs while the softmax warps work on this one)
//   softmax     two threads per (head, row) = one lane of tensor memory, one per block of the pair: tcgen05.ld of its 64
//               scores, mask, exp2
//   O += P V    P is written as a bf16 K-major swizzled tile [128 x 128] by the softmax threads; V arrives transposed
//               ([256 x N], written by the prep kernel), so a V block [256 d x 64 keys] is K-major too; O [128 x 256] fp32
//               stays in tensor memory for the whole CTA
//
// The softmax is two-pass: pass 1 runs Q K^T over the visible blocks and keeps only the row maxima, pass 2 forms
// P = exp2((s - max) * scale * log2 e) and accumulates O — no rescaling of O ever. With at most two pairs (four visible
// blocks) all scores stay in tensor memory between the passes; with more, pass 2 recomputes the (cheap) Q K^T products.
// Shared memory holds Q (48 KB), two 64 KB regions for K / V pairs and P (32 KB): in pass 1 the regions alternate as K
// stages; in pass 2 region 0 takes the K pair and region 1 the V pair (the natural stagger of Q K^T -> softmax -> P V hides
// their loads). An odd number of visible blocks repeats the last one as the second half of the last pair, masked out.
// Roles: warps 0-7 softmax / epilogue, warp 8 TMA producer, warp 9 MMA issuer; mbarriers between them, every wait bounded (the
// CTA then reports OJB_DEV_WAIT_TIMEOUT through `status`, frees its tensor memory and returns).
#include "gemm_common.cuh"

namespace ojb {
namespace {

constexpr int kD = 256;
constexpr int kQRows = 16;            // query rows per CTA and head
constexpr int kMaxG = 6;              // query heads per kv head that fit the shared-memory plan
constexpr int kTcThreads = 320;       // 8 softmax warps, producer warp, MMA warp
constexpr int kSoftWarps = 8;
constexpr uint32_t kQBytes = kMaxG * kQRows * kD * 2;    // 4 k-blocks of [16 G rows][64]
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColO = 0, kColS = 256;               // O: 256 columns; S: two buffers of 128 columns
constexpr int kStagePitch = kD * 2 + 16;                 // bytes per row of the output staging tile
constexpr int kMaxBlocks = 2048;                         // 64-key blocks a CTA can list (131 072 keys)
constexpr int kSub = 64;               // keys per visibility block
constexpr int kKB = 128;               // keys per product (two blocks)
constexpr uint32_t kRegion = kKB * kD * 2;               // 64 KB: a K pair (4 k-blocks of [128 keys][64]) or a V pair (2 of [256 d][64])
constexpr uint32_t kPBytes = 128 * kKB * 2;              // 2 k-blocks of [128 rows][64 keys]
constexpr int kNS = 2;                                   // S buffers beside O
enum { kBarQ = 0, kBarFull = 1, kBarFree = 3, kBarSFull = 5, kBarSFree = 7, kBarPFull = 9, kBarPFree = 10, kBarO = 11, kBarX = 12,
       kNumBars = 13 };
constexpr size_t kSmemBytes = 1024 + kQBytes + 2 * kRegion + kPBytes + kNumBars * 8 + 16 + kQRows * 8 * 4 + (kMaxBlocks + 1) * 4 +
                              4 * 128 * 4;

// Measurement hook (ojb_tree_attn_set_trace): when non-null, the CTA of kv head 0 and the last-but-one block of query rows
// stores %globaltimer at a few points of its life (see the stamps below).
__device__ unsigned long long* g_attn_trace = nullptr;

struct AttnArgs {
  const bf16_t* gate;
  const int32_t* krange;
  bf16_t* y;
  int32_t* status;
  int N, HQ, HKV, G;
  float scale_log2e;
  int wait_ms;
};

// bits of keys [32 * w, 32 * w + 32) that fall in [lo, hi)
__device__ __forceinline__ uint32_t range_bits(int lo, int hi, int w) {
  const int a = max(lo - w * 32, 0), b = min(hi - w * 32, 32);
  if (a >= b) return 0u;
  const uint32_t upto_b = b == 32 ? 0xffffffffu : ((1u << b) - 1u);
  return upto_b & ~((1u << a) - 1u);
}

__global__ void __launch_bounds__(kTcThreads, 1)
tree_attn_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_vt, AttnArgs g) {
  const unsigned long long t_entry = global_timer_ns();
  pdl_launch_dependents();
  unsigned long long* trace = (blockIdx.x == 0 && blockIdx.y + 2 == gridDim.y) ? g_attn_trace : nullptr;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* Qs = smem;
  constexpr int kStages = 2, kHalf = 1;
  constexpr int kCols = kSub;                  // score columns per softmax thread: one block of the pair
  uint8_t* Rg = Qs + kQBytes;                  // two regions
  uint8_t* Ps = Rg + kStages * kRegion;
  uint64_t* bars = reinterpret_cast<uint64_t*>(Ps + kPBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);      // [0] give-up flag, [1] wait limit in ms
  int* kr = reinterpret_cast<int*>(tmem_slot + 4);                                 // [16 rows][8]
  int* vis_list = kr + kQRows * 8;                                                 // visible key blocks; count at [kMaxBlocks]
  float* xch = reinterpret_cast<float*>(vis_list + kMaxBlocks + 1);                // [maxima, sums][2 column halves][128 rows]

  const uint32_t bar0 = smem_u32(bars);
  auto bar = [&](int i) { return bar0 + 8u * static_cast<uint32_t>(i); };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
  const int kvh = blockIdx.x, r0 = blockIdx.y * kQRows;
  const int G = g.G, N = g.N;
  const int nw = (G * kQRows + 31) / 32;       // softmax warps that own real rows
  const int hq0 = kvh * G;
  const uint32_t qstride = static_cast<uint32_t>(G) * (kQRows * 128);      // bytes of one k-block of the Q tile: [16 G rows][128 B]

  if (tid == 0) {
    for (int i = 0; i < kNumBars; ++i) mbar_init(bar(i), 1);
    mbar_init(bar(kBarSFree), 2 * nw); mbar_init(bar(kBarSFree + 1), 2 * nw);
    mbar_init(bar(kBarPFull), 2 * nw);
    mbar_init(bar(kBarX), 2 * nw);
    abort_flag[0] = 0;
    abort_flag[1] = g.wait_ms;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_vt) : "memory");
  }
  if (warp == kSoftWarps) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  pdl_wait();      // from here on the previous kernel of the stream has completed
  // key ranges of the 16 rows
  if (tid < kQRows * 8) kr[tid] = g.krange[static_cast<int64_t>(r0) * 8 + tid];
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (warp == kSoftWarps && lane == 0) {      // the Q rows do not depend on the list of key blocks: requested while warp 0 builds it
    mbar_expect_tx(bar(kBarQ), static_cast<uint32_t>(G) * 4u * (kQRows * 128u));
    for (int w = 0; w < G; ++w)
      for (int kb4 = 0; kb4 < 4; ++kb4)
        tma_load_2d(smem_u32(Qs) + kb4 * qstride + w * (kQRows * 128), &map_q, bar(kBarQ), kb4 * 64, (hq0 + w) * N + r0);
  }
  // ordered list of the key blocks that at least one of the 16 rows sees
  const int NB = (N + kSub - 1) / kSub;
  if (warp == 0) {
    int count = 0;
    for (int base = 0; base < NB; base += 32) {
      const int kb = base + lane;
      bool any = false;
      if (kb < NB) {
        const int k0 = kb * kSub, k1 = k0 + kSub;
        for (int r = 0; r < kQRows && !any; ++r) {
          const int* q = kr + r * 8;      // (e0, a1, e1, a2, e2, a0)
          any = (q[5] < q[0] && q[5] < k1 && q[0] > k0) || (q[1] < q[2] && q[1] < k1 && q[2] > k0) ||
                (q[3] < q[4] && q[3] < k1 && q[4] > k0);
        }
      }
      const uint32_t bal = __ballot_sync(0xffffffffu, any);
      if (any && count + __popc(bal & ((1u << lane) - 1u)) < kMaxBlocks) vis_list[count + __popc(bal & ((1u << lane) - 1u))] = kb;
      count += __popc(bal);
    }
    if (lane == 0) vis_list[kMaxBlocks] = count < kMaxBlocks ? count : kMaxBlocks;
  }
  __syncthreads();
  const int nblk = vis_list[kMaxBlocks];        // visible 64-key blocks
  const int nvis = (nblk + 1) >> 1;             // pairs of them
  const int T = 2 * nvis;                       // pass 1 (maxima) then pass 2 (P V) over the same blocks
  // Up to kNS pairs: their scores fit in tensor memory beside O, so Q K^T runs once and pass 2 reads the scores again from
  // there. More pairs: the two S buffers rotate and pass 2 recomputes Q K^T.
  const bool one_pass = nvis <= kNS;
  // Gate values of the 16 output pieces this thread multiplies at the very end (consecutive threads take consecutive 16-byte
  // pieces of the [G * 16 rows][256] output tile). Each warp requests them as soon as it has nothing else to wait for, so their
  // latency runs under the last P V products and the staging of O.
  const int pieces = G * kQRows * (kD / 8);
  constexpr int kBatch = (kMaxG * kQRows * (kD / 8) + kTcThreads - 1) / kTcThreads;      // 10
  uint4 gq[kBatch];
  auto prefetch_gates = [&](int base) {
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int i = base + u * kTcThreads;
      gq[u] = make_uint4(0u, 0u, 0u, 0u);
      if (i < pieces) {
        const int row = i >> 5, piece = i & 31;             // tile row = 16 * head + query row
        gq[u] = *reinterpret_cast<const uint4*>(g.gate + (static_cast<int64_t>(r0 + (row & 15)) * g.HQ + (hq0 + (row >> 4))) * kD + piece * 8);
      }
    }
  };
  if (trace && tid == 0) { trace[0] = t_entry; trace[1] = global_timer_ns(); trace[15] = static_cast<unsigned long long>(nblk); }

  if (warp == kSoftWarps) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int use[2] = {0, 0};
      bool ok = true;
      auto load = [&](int R, bool is_v, int p) {      // the K blocks or the V blocks of pair p into region R
        if (!mbar_wait(bar(kBarFree + R), (use[R] & 1) ^ 1, abort_flag)) return false;
        ++use[R];
        mbar_expect_tx(bar(kBarFull + R), kRegion);
        const uint32_t dst = smem_u32(Rg) + R * kRegion;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int kb = vis_list[min(2 * p + h, nblk - 1)];      // an odd count repeats the last block (masked out later)
          if (!is_v) {
            for (int kb4 = 0; kb4 < 4; ++kb4)
              tma_load_2d(dst + kb4 * (kKB * 128) + h * (kSub * 128), &map_k, bar(kBarFull + R), kb4 * 64, kvh * N + kb * kSub);
          } else {
            tma_load_2d(dst + h * (kD * 128), &map_vt, bar(kBarFull + R), kb * kSub, kvh * kD);
          }
        }
        return true;
      };
      if (one_pass) {
        // (a region is free for the next block once the product that read it is done; all Q K^T come before the first P V)
        for (int it = 0; it < nvis && ok; ++it) ok = load(it % kStages, false, it);
        for (int j = 0; j < nvis && ok; ++j) ok = load(j % kStages, true, j);
      } else {
        for (int it = 0; it < nvis && ok; ++it) ok = load(it % kStages, false, it);
        // pass 2: region 0 takes the K pairs (free again when the Q K^T that read it is done), region 1 the V pairs (free when
        // their P V is done); Q K^T (j + 1) is issued before P V (j), so the K pair of j + 1 is asked for before the V pair
        // of j — the order of the requests is the order in which the MMA warp consumes them
        if (ok) ok = load(0, false, 0);
        for (int j = 0; j < nvis && ok; ++j) {
          if (j + 1 < nvis) ok = load((j + 1) % kHalf, false, j + 1);
          if (ok) ok = load(kHalf + j % kHalf, true, j);
        }
      }
    }
  } else if (warp == kSoftWarps + 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc(kKB), idesc_o = umma_idesc(kD);
      int use[2] = {0, 0}, use_s[2] = {0, 0};
      bool ok = mbar_wait(bar(kBarQ), 0, abort_flag);
      if (trace) trace[8] = global_timer_ns();          // Q has landed
      auto qk = [&](int R, int sb) {                    // S[sb] = Q K^T with the K block in region R
        if (!mbar_wait(bar(kBarFull + R), use[R] & 1, abort_flag)) return false;
        ++use[R];
        if (!one_pass && !mbar_wait(bar(kBarSFree + sb), (use_s[sb] & 1) ^ 1, abort_flag)) return false;
        ++use_s[sb];
        tc_fence_after();
        const uint32_t tmem_s = tmem_base + kColS + static_cast<uint32_t>(sb) * kKB;
#pragma unroll
        for (int kb4 = 0; kb4 < 4; ++kb4) {
          const uint64_t qdesc = smem_desc_sw128(smem_u32(Qs) + kb4 * qstride);
          const uint64_t kdesc = smem_desc_sw128(smem_u32(Rg) + R * kRegion + kb4 * (kKB * 128));
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_bf16(tmem_s, qdesc + 2 * k, kdesc + 2 * k, idesc_s, (kb4 > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(bar(kBarFree + R));
        umma_commit(bar(kBarSFull + sb));
        return true;
      };
      auto pv = [&](int j, int R) {                     // O += P V of pass-2 block j, V block in region R
        if (!mbar_wait(bar(kBarPFull), j & 1, abort_flag)) return false;
        if (!mbar_wait(bar(kBarFull + R), use[R] & 1, abort_flag)) return false;
        ++use[R];
        tc_fence_after();
#pragma unroll
        for (int kb2 = 0; kb2 < kKB / 64; ++kb2) {
          const uint64_t pdesc = smem_desc_sw128(smem_u32(Ps) + kb2 * (128 * 128));
          const uint64_t vdesc = smem_desc_sw128(smem_u32(Rg) + R * kRegion + kb2 * (kD * 128));
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16(tmem_base + kColO, pdesc + 2 * k, vdesc + 2 * k, idesc_o, (j > 0 || kb2 > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(bar(kBarFree + R));
        umma_commit(bar(kBarPFree));
        return true;
      };
      if (one_pass) {
        for (int it = 0; it < nvis && ok; ++it) ok = qk(it % kStages, it);
        for (int j = 0; j < nvis && ok; ++j) ok = pv(j, j % kStages);
      } else {
        for (int it = 0; it < nvis && ok; ++it) ok = qk(it % kStages, it & 1);
        for (int j = 0; j < nvis && ok; ++j) {
          ok = qk(j % kHalf, (nvis + j) & 1);
          if (ok && j > 0) ok = pv(j - 1, kHalf + (j - 1) % kHalf);
        }
        if (ok && nvis > 0) ok = pv(nvis - 1, kHalf + (nvis - 1) % kHalf);
      }
      if (ok) umma_commit(bar(kBarO));
      if (trace) trace[9] = global_timer_ns();          // every MMA issued
    }
  } else if (warp < kSoftWarps && (warp & 3) < nw) {
    // ------------------------------------------------------------------ softmax + epilogue: two threads per (head, row).
    // Thread (half, my) takes block `half` of every pair (columns [64 half, +64) of S) and columns [128 half, +128) of O; the two
    // halves exchange their row maxima before pass 2 and their row sums after it through shared memory.
    const int half = warp >> 2;
    const int my = (warp & 3) * 32 + lane;       // tile row = 16 * head + query row = lane of tensor memory
    const int qr = my & 15;
    const int* q = kr + qr * 8;
    const int a0 = q[5], e0 = q[0], a1 = q[1], e1 = q[2], a2 = q[3], e2 = q[4];
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const bool stamp = trace && my == 0 && half == 0;
    constexpr int kLd = kCols / 32;              // 32-column loads per block: 1 or 2
    float m = -INFINITY, l = 0.f;
    int use_s[2] = {0, 0}, xphase = 0;
    bool ok = true;
    auto exchange = [&](float v, int slot) {     // hands v to the thread of the other half, returns that thread's value
      xch[(2 * slot + half) * 128 + my] = v;
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(kBarX));
      if (!mbar_wait(bar(kBarX), xphase & 1, abort_flag)) { ok = false; return v; }
      ++xphase;
      return xch[(2 * slot + (half ^ 1)) * 128 + my];
    };
    for (int it = 0; it < T && ok; ++it) {
      const bool pass2 = it >= nvis;
      const int blk = pass2 ? it - nvis : it;
      const int sub = 2 * blk + half;                    // this thread's block of the pair; past the end: the masked-out repeat
      const int kb = vis_list[min(sub, nblk - 1)];
      const int sb = one_pass ? blk : (it & 1);          // S buffer
      if (it == nvis) {
        m = fmaxf(m, exchange(m, 0));
        if (!ok) break;
      }
      // (pass 2 of the one-pass form reads scores that pass 1 has already waited for)
      if (!(one_pass && pass2)) {
        if (!mbar_wait(bar(kBarSFull + sb), use_s[sb] & 1, abort_flag)) { ok = false; break; }
        ++use_s[sb];
      }
      if (stamp && (it == 0 || it == nvis)) trace[it == 0 ? 2 : 3] = global_timer_ns();   // first S of pass 1 / pass 2
      tc_fence_after();
      const float mc = m * g.scale_log2e;
      uint32_t s[kLd][32];
      const uint32_t taddr = tmem_base + lane_base + kColS + static_cast<uint32_t>(sb * kKB + half * kCols);
#pragma unroll
      for (int i = 0; i < kLd; ++i) tmem_ld32(taddr + 32 * i, s[i]);
      tmem_ld_wait();
      if (!one_pass) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(kBarSFree + sb));          // this warp has consumed its part of the S buffer
      }
      uint32_t bits[kLd];
#pragma unroll
      for (int i = 0; i < kLd; ++i) {
        const int w = kb * (kSub / 32) + i;
        bits[i] = sub < nblk ? (range_bits(a0, e0, w) | range_bits(a1, e1, w) | range_bits(a2, e2, w)) : 0u;
      }
      if (!pass2) {
#pragma unroll
        for (int i = 0; i < kLd; ++i)
#pragma unroll
          for (int c = 0; c < 32; ++c)
            if ((bits[i] >> c) & 1u) m = fmaxf(m, __uint_as_float(s[i][c]));
      } else {
        uint32_t pk[kLd * 16];                            // the probabilities as bf16 pairs
#pragma unroll
        for (int i = 0; i < kLd; ++i)
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            const float p0 = ((bits[i] >> c) & 1u) ? exp2f_fast(__uint_as_float(s[i][c]) * g.scale_log2e - mc) : 0.f;
            const float p1 = ((bits[i] >> (c + 1)) & 1u) ? exp2f_fast(__uint_as_float(s[i][c + 1]) * g.scale_log2e - mc) : 0.f;
            l += p0 + p1;
            pk[i * 16 + (c >> 1)] = pack2(p0, p1);
          }
        // P V of the previous block must have read P before this block's P is written
        if (!mbar_wait(bar(kBarPFree), (blk & 1) ^ 1, abort_flag)) { ok = false; break; }
        // row `my` of the K-major swizzled tile: each 64-key k-block is 128 bytes = 8 chunks of 16, chunk c stored at
        // c ^ (row & 7); this thread's columns start at chunk (half * kCols % 64) / 8 of k-block half * kCols / 64
        uint8_t* prow = Ps + ((half * kCols) / 64) * (128 * 128) + my * 128;
        constexpr int kChunks = kCols / 8;
        const int chunk0 = ((half * kCols) % 64) / 8;
#pragma unroll
        for (int c = 0; c < kChunks; ++c)
          *reinterpret_cast<uint4*>(prow + (((chunk0 + c) ^ (my & 7)) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(kBarPFull));
      }
    }
    if (stamp) trace[4] = global_timer_ns();                  // last P handed over
    if (ok) l += exchange(l, 1);
    // ---- att = bf16(O / l) of this thread's half of its (head, row) into the staging tile [128][kStagePitch] (over Q and
    //      region 0, which no MMA reads any more once O is complete); rows are 16 bytes longer than 512 so that the 32 rows of
    //      a warp spread over the banks
    prefetch_gates(tid);
    if (ok) ok = mbar_wait(bar(kBarO), 0, abort_flag);
    if (stamp) trace[5] = global_timer_ns();                  // O complete
    if (ok) {
      tc_fence_after();
      const float inv_l = l > 0.f ? 1.0f / l : 0.f;
      uint8_t* srow = smem + my * kStagePitch;
#pragma unroll
      for (int cc = 0; cc < kD / 64; ++cc) {
        const int c = half * (kD / 64) + cc;
        uint32_t o[32];
        tmem_ld32(tmem_base + lane_base + kColO + c * 32, o);
        tmem_ld_wait();
#pragma unroll
        for (int v8 = 0; v8 < 4; ++v8) {
          float a[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) a[e] = l > 0.f ? __uint_as_float(o[v8 * 8 + e]) * inv_l : 0.f;   // a row that sees no key: zeros, whatever tensor memory holds
          *reinterpret_cast<uint4*>(srow + c * 64 + v8 * 16) = pack8(a);
        }
      }
    }
  }
  // ---- y = bf16(att * sigmoid(gate)): all ten warps, consecutive threads on consecutive 16-byte pieces of a row, so the
  //      gate is read and y is written in whole 512-byte rows
  if (trace && tid == 0) trace[6] = global_timer_ns();       // staging written (warp 0)
  if (warp >= kSoftWarps || (warp & 3) >= nw) prefetch_gates(tid);
  tc_fence_before();
  __syncthreads();
  if (!abort_flag[0]) {
    // sigmoid(x) = 0.5 tanh(0.5 x) + 0.5: one special-function instruction per value (the exp / reciprocal form needs two, and
    // this loop is bound by them). The gate factor is applied in fp32 and the product rounded once.
    for (int base = tid; base < pieces; base += kBatch * kTcThreads) {
      if (base != tid) prefetch_gates(base);
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        const int i = base + u * kTcThreads;
        if (i < pieces) {
          const int row = i >> 5, piece = i & 31;
          float gv[8], a[8], out[8];
          unpack8(gq[u], gv);
          unpack8(*reinterpret_cast<const uint4*>(smem + row * kStagePitch + piece * 16), a);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            float t;
            asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * gv[e]));
            out[e] = a[e] * fmaf(0.5f, t, 0.5f);
          }
          *reinterpret_cast<uint4*>(g.y + (static_cast<int64_t>(r0 + (row & 15)) * g.HQ + (hq0 + (row >> 4))) * kD + piece * 8) = pack8(out);
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  __syncthreads();
  if (trace && tid == 0) trace[7] = global_timer_ns();
  if (abort_flag[0]) {
    if (tid == 0) report_status(g.status, OJB_DEV_WAIT_TIMEOUT);
    for (int i = 0; i < 200; ++i) __nanosleep(1000);       // copies that were already issued land before the CTA leaves
    __syncthreads();
  }
  if (warp == kSoftWarps) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace
}  // namespace ojb

using namespace ojb;

extern "C" int ojb_tree_attn_set_trace(uint64_t* records) {
  unsigned long long* p = reinterpret_cast<unsigned long long*>(records);
  return launch_status(cudaMemcpyToSymbol(ojb::g_attn_trace, &p, sizeof(p)));
}

extern "C" int ojb_tree_attn_tc(const void* qt, const void* kt, const void* vt_t, const void* gate, const int32_t* krange, void* y,
                                int64_t N, int64_t HQ, int64_t HKV, int64_t D, float scale, int32_t* status,
                                ojb_stream_t stream) {
  if (N == 0) return OJB_OK;
  OJB_REQUIRE(qt && kt && vt_t && gate && krange && y && N > 0 && N % 32 == 0 && D == kD);
  OJB_REQUIRE(HQ > 0 && HKV > 0 && HQ % HKV == 0 && HQ / HKV <= kMaxG);
  OJB_REQUIRE(aligned16(qt) && aligned16(kt) && aligned16(vt_t) && aligned16(gate) && aligned16(y));
  if ((N + kSub - 1) / kSub > kMaxBlocks) return OJB_ERR_LIMIT;
  CUtensorMap map_q, map_k, map_vt;
  int rc = make_map(&map_q, qt, HQ * N, kD, kQRows);
  if (rc == OJB_OK) rc = make_map(&map_k, kt, HKV * N, kD, kSub);
  if (rc == OJB_OK) rc = make_map(&map_vt, vt_t, HKV * kD, N, kD);
  if (rc != OJB_OK) return rc;
  static int smem_set[kMaxDevices] = {};
  if (!raise_smem_limit(tree_attn_tc_kernel, static_cast<int>(kSmemBytes), smem_set)) return OJB_ERR_LAUNCH;
  AttnArgs a{static_cast<const bf16_t*>(gate), krange, static_cast<bf16_t*>(y), status, static_cast<int>(N), static_cast<int>(HQ),
             static_cast<int>(HKV), static_cast<int>(HQ / HKV), scale * 1.4426950408889634f, gemm_wait_limit_ms()};
  launch_kernel(tree_attn_tc_kernel, dim3(static_cast<unsigned>(HKV), static_cast<unsigned>(N / kQRows)), dim3(kTcThreads),
                kSmemBytes, static_cast<cudaStream_t>(stream), map_q, map_k, map_vt, a);
  return launch_status(cudaGetLastError());
}
