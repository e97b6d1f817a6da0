// bf16 GEMM, CTA-pair kernel (third kernel behind ojb_gemm_bf16*), sm_100a:
//   out[M,N] = x[M,K] · w[N,K]^T, both operands K-major, fp32 accumulation in tensor memory (TMEM).
//
// The two CTAs of a cluster (the two SMs of one TPC) work on one unit together with tcgen05.mma.cta_group::2: an MMA of
// M = 256 whose A rows and B rows are split between the shared memories of the two CTAs and whose accumulator rows are split
// between their tensor memories. For a 256 x 256 unit each CTA therefore loads 128 rows of x and 128 rows of w per k-block
// (32 KB instead of the 64 KB a single CTA needs for the same unit), which leaves room for six stages in flight instead
// of three (the main loop of the one-CTA kernel is bound by the latency of these copies), and it keeps only 256 of its 512
// TMEM columns busy, so the epilogue of one unit overlaps the MMAs of the next.
//
// Per CTA, 320 threads:
//   warp 0      TMA producer  — plain (non-multicast) cp.async.bulk.tensor into its own shared memory; the copies of both
//                               CTAs complete on the leader's "full" barrier
//   warp 1      MMA issuer    — one lane of the leader CTA (cluster rank 0) issues the MMAs of the pair; tcgen05.commit
//                               with a CTA mask releases the stage in both CTAs and publishes the accumulator to both
//   warps 2..9  epilogue      — each CTA drains its own 128 accumulator rows through a swizzled shared-memory tile so that
//                               global stores are whole 128-byte rows; then arrives on the leader's "accumulator free" barrier
// Work units, their order and the K ranges are those of the one-CTA block kernel (gemm_units.cuh), dealt to the CTA pairs
// round-robin: block units of 256 rows of x times BN rows of w, and swapped-operand units (256 rows of w as the M side,
// rows of x as the N side) for the last M mod 256 <= 128 rows or, on request, for all of x. In the latter mode a unit
// covers up to 512 rows of x with one pass over its 256 rows of w: its accumulator columns are filled by up to two MMAs per
// k-step (N <= 256 each), so w crosses the memory system once per 512 rows of x; a unit wider than 256 columns uses the
// whole tensor memory and the MMAs of the next unit wait for its epilogue.
//
// Every wait on an mbarrier is bounded (2 s): the CTA then raises its abort flag, records OJB_DEV_WAIT_TIMEOUT, lets copies
// in flight land, and both CTAs still meet at the closing cluster barrier before freeing their TMEM.
#include "gemm_units.cuh"

namespace ojb {
namespace {

constexpr int kPairThreads = 320;
constexpr int kPairEpiWarps = 8;
constexpr int kPairMaxStages = 8;
constexpr uint32_t kHalfABytes = kBM * kBK * 2;      // 16 KB: this CTA's 128 rows of the M-side operand
constexpr uint32_t kStagingBytes = kPairEpiWarps * 4096;   // one [32 rows][128 bytes] tile per epilogue warp
constexpr uint32_t kAccCols = 256;                   // TMEM columns per accumulator buffer (two buffers)

unsigned long long* g_ptrace = nullptr;
int g_ptrace_cap = 0;
#ifdef OJB_GEMM_PROBES
int g_pmma_repeat = 1;
int g_pmax_stages = 0;
#else
constexpr int g_pmma_repeat = 1, g_pmax_stages = 0;
#endif

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same shared-memory location in the CTA of the given cluster rank
__device__ __forceinline__ uint32_t map_to_rank(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// TMA load whose completion bytes are counted on a barrier that may live in the other CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t cluster_bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(cluster_bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t slot_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  const uint32_t z = 0;
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc), "r"(z)
      : "memory");
}
// Arrive on the barrier at this shared-memory offset in every CTA of the mask once all MMAs issued so far have finished.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar, uint16_t cta_mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
               "h"(cta_mask)
               : "memory");
}
__host__ __device__ constexpr uint32_t umma_idesc_m256(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(256 >> 4) << 24);
}

// One [32 rows][128 bytes] tile per epilogue warp: thread `lane` owns row `lane` and writes its eight 16-byte pieces to
// slots (j ^ (lane & 7)), which spreads the eight threads of a quarter-warp over all banks; reading a row back takes the
// same permutation.
__device__ __forceinline__ void stage_put(uint8_t* tile, int lane, int j, const uint4& v) {
  *reinterpret_cast<uint4*>(tile + lane * 128 + ((j ^ (lane & 7)) << 4)) = v;
}
__device__ __forceinline__ uint4 stage_get(const uint8_t* tile, int row, int j) {
  return *reinterpret_cast<const uint4*>(tile + row * 128 + ((j ^ (row & 7)) << 4));
}

// Write the staged tile to out rows [row0, row0+32), tile columns [col0, col0 + 128/sizeof(T)), as 128-byte row segments:
// 8 consecutive lanes cover one row. ncols = columns of the w tile that exist (relative to the tile), tile_off = element
// offset of the tile's column 0 in a row of out.
template <typename T>
__device__ __forceinline__ void stage_flush(const uint8_t* tile, int lane, T* out, int64_t ldo, int64_t tile_off, int row0, int M,
                                            int col0, int ncols, bool vec_ok) {
  constexpr int kVec = 16 / static_cast<int>(sizeof(T));
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = i * 4 + (lane >> 3);
    const int j = lane & 7;
    const uint4 v = stage_get(tile, r, j);
    const int row = row0 + r;
    const int col = col0 + j * kVec;
    if (row < M && col < ncols) {
      T* dst = out + static_cast<int64_t>(row) * ldo + tile_off + col;
      if (vec_ok && col + kVec <= ncols) {
        *reinterpret_cast<uint4*>(dst) = v;
      } else {
        const T* e = reinterpret_cast<const T*>(&v);
        for (int k = 0; k < kVec; ++k)
          if (col + k < ncols) dst[k] = e[k];
      }
    }
  }
}

template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
gemm_pair256_kernel(const __grid_constant__ CUtensorMap map_xh, const __grid_constant__ CUtensorMap map_wh,
                    const __grid_constant__ CUtensorMap map_w128, const __grid_constant__ CUtensorMap map_xt,
                    const __grid_constant__ CUtensorMap map_w64, GemmArgs g) {
  pdl_launch_dependents();
  constexpr uint32_t kTmemCols = 512;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* staging = smem + static_cast<size_t>(g.stages) * g.stage_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + kStagingBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kPairMaxStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const uint32_t tiles0 = smem_u32(smem);
  const uint32_t full0 = smem_u32(bars);
  const uint32_t empty0 = full0 + 8 * kPairMaxStages;
  const uint32_t accfull0 = empty0 + 8 * kPairMaxStages;   // two barriers
  const uint32_t accempty0 = accfull0 + 16;                // two barriers
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int STAGES = g.stages;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair_id = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);     // the leader's arrive.expect_tx (only the leader's full barriers are used)
      mbar_init(empty0 + 8 * s, 1);    // one tcgen05.commit per use, delivered to both CTAs
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(accfull0 + 8 * b, 1);                       // one tcgen05.commit per unit, delivered to both CTAs
      mbar_init(accempty0 + 8 * b, 2 * kPairEpiWarps);      // the epilogue warps of both CTAs (leader's barrier only)
    }
    abort_flag[0] = 0;
    abort_flag[1] = g.wait_ms;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_xh) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_wh) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w128) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_xt) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w64) : "memory");
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();      // the barriers of both CTAs exist before any remote arrive or copy completion reaches them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();      // from here on the previous kernel of the stream has completed

  const int total_block = g.n_xblk * g.n_wtile * g.splits;
  const int total_units = total_block + (g.tail_rows > 0 ? g.n_wtile256 * g.splits * g.n_xchunk : 0);
  const int half_bn = g.BN / 2, half_cw = g.chunk_w / 2;
  // accumulator buffers: two of 256 columns, or, when a swapped unit needs more than 256 columns, one of up to 512 (the
  // MMAs of a unit then wait for the epilogue of the previous one)
  const int nbuf = g.tail_box > static_cast<int>(kAccCols) ? 1 : 2;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int unit = pair_id; unit < total_units && ok; unit += n_pairs) {
        const Unit u = decode_unit(g, unit, total_block);
        const uint32_t my_bytes = kHalfABytes + static_cast<uint32_t>(u.tail ? g.n_chunk * half_cw : half_bn) * (kBK * 2);
        for (int kb = u.kb0; kb < u.kb1; ++kb) {
          if (!mbar_wait(empty0 + 8 * stage, phase ^ 1u, abort_flag)) { ok = false; break; }
          const uint32_t a_dst = tiles0 + stage * g.stage_bytes;
          const uint32_t fb_leader = map_to_rank(full0 + 8 * stage, 0);
          if (leader) mbar_expect_tx(full0 + 8 * stage, 2 * my_bytes);
          if (!u.tail) {
            tma_load_2d_pair(a_dst, &map_xh, fb_leader, kb * kBK, u.xb * kBlockM + static_cast<int>(rank) * kBM);
            tma_load_2d_pair(a_dst + kHalfABytes, &map_wh, fb_leader, kb * kBK, u.wt * g.BN + static_cast<int>(rank) * half_bn);
          } else {
            if (g.w_split64) {
              tma_load_2d_pair(a_dst, &map_w64, fb_leader, kb * kBK, u.wt * 256 + static_cast<int>(rank) * 64);
              tma_load_2d_pair(a_dst + kHalfABytes / 2, &map_w64, fb_leader, kb * kBK, u.wt * 256 + 128 + static_cast<int>(rank) * 64);
            } else {
              tma_load_2d_pair(a_dst, &map_w128, fb_leader, kb * kBK, u.wt * 256 + static_cast<int>(rank) * kBM);
            }
            const int xrow0 = g.n_xblk * kBlockM + u.xc * g.tail_box;
            for (int c = 0; c < g.n_chunk; ++c) {
              const int wc = min(g.chunk_w, g.tail_box - c * g.chunk_w);
              // (the box always has chunk_w / 2 rows: behind a narrower last chunk it fetches rows no MMA reads)
              tma_load_2d_pair(a_dst + kHalfABytes + static_cast<uint32_t>(c * half_cw) * (kBK * 2), &map_xt, fb_leader, kb * kBK,
                               xrow0 + c * g.chunk_w + static_cast<int>(rank) * (wc / 2));
            }
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && leader) {
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int unit = pair_id; unit < total_units && ok; unit += n_pairs, ++it) {
        const Unit u = decode_unit(g, unit, total_block);
        const uint32_t idesc = umma_idesc_m256(g.BN);
        const int buf = nbuf == 2 ? (it & 1) : 0;
        const uint32_t use = static_cast<uint32_t>(nbuf == 2 ? (it >> 1) : it);
        if (!mbar_wait(accempty0 + 8 * buf, (use & 1u) ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t acc = tmem_base + static_cast<uint32_t>(buf) * kAccCols;
        for (int kb = u.kb0; kb < u.kb1; ++kb) {
          if (!mbar_wait(full0 + 8 * stage, phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = tiles0 + stage * g.stage_bytes;
          const uint64_t adesc = smem_desc_sw128(a_addr);
          const uint64_t bdesc = smem_desc_sw128(a_addr + kHalfABytes);
          if (u.tail) {
            for (int rep = 0; rep < OJB_PROBE_REPEAT(g); ++rep) {      // (repeat > 1 in probe builds only)
              for (int c = 0; c < g.n_chunk; ++c) {
                const int wc = min(g.chunk_w, g.tail_box - c * g.chunk_w);
                const uint32_t idesc_c = umma_idesc_m256(wc);
                const uint64_t bdesc_c = smem_desc_sw128(a_addr + kHalfABytes + static_cast<uint32_t>(c * half_cw) * (kBK * 2));
#pragma unroll
                for (int k = 0; k < kBK / kUmmaK; ++k)
                  umma_bf16_pair(acc + static_cast<uint32_t>(c * g.chunk_w), adesc + 2 * k, bdesc_c + 2 * k, idesc_c,
                                 (kb > u.kb0 || k > 0 || rep > 0) ? 1u : 0u);
              }
            }
          } else if (OJB_PROBE_REPEAT(g) == 1) {
#pragma unroll
            for (int k = 0; k < kBK / kUmmaK; ++k)
              umma_bf16_pair(acc, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > u.kb0 || k > 0) ? 1u : 0u);
          } else {                                   // probe builds only
            for (int rep = 0; rep < OJB_PROBE_REPEAT(g); ++rep)
              for (int k = 0; k < kBK / kUmmaK; ++k)
                umma_bf16_pair(acc, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > u.kb0 || k > 0 || rep > 0) ? 1u : 0u);
          }
          umma_commit_pair(empty0 + 8 * stage, 3);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit_pair(accfull0 + 8 * buf, 3);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9 of both CTAs)
    const int quarter = warp & 3;            // TMEM lanes [32*quarter, 32*quarter+32) are the ones this warp may read
    const int half = (warp - 2) >> 2;        // the two warps of a quarter share the columns between them
    uint8_t* tile = staging + (warp - 2) * 4096;
    const uint32_t accempty_leader = map_to_rank(accempty0, 0);
    int it = 0;
    bool ok = true;
    for (int unit = pair_id; unit < total_units && ok; unit += n_pairs, ++it) {
      const Unit u = decode_unit(g, unit, total_block);
      const int buf = nbuf == 2 ? (it & 1) : 0;
      const uint32_t use = static_cast<uint32_t>(nbuf == 2 ? (it >> 1) : it);
      const bool tracing = g.trace != nullptr && warp == 2 && lane == 0 && leader;
      const unsigned long long t_begin = tracing ? global_timer_ns() : 0ull;
      if (!mbar_wait(accfull0 + 8 * buf, use & 1u, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const unsigned long long t_full = tracing ? global_timer_ns() : 0ull;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(buf) * kAccCols;
      if (!u.tail) {
        // ---- block unit: TMEM lane = row of x, TMEM column = column of the w tile
        const int row0 = u.xb * kBlockM + static_cast<int>(rank) * kBM + quarter * 32;
        const int ncols = min(g.N - u.wt * g.BN, g.BN);
        const int64_t tile_off = static_cast<int64_t>(u.wt) * g.BN;
        if constexpr (EPI == kEpiPartialF32) {
          float* out = reinterpret_cast<float*>(g.out) + static_cast<int64_t>(u.split) * g.split_stride;
          const bool vec_ok = (g.ldo % 4) == 0 && (g.BN % 4) == 0;
          const int nfl = (g.BN + 31) / 32;
#pragma unroll 1
          for (int f = half; f < nfl; f += 2) {
            uint32_t r[32];
            tmem_ld32(taddr + f * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 8; ++j) stage_put(tile, lane, j, make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]));
            __syncwarp();
            stage_flush<float>(tile, lane, out, g.ldo, tile_off, row0, g.M, f * 32, ncols, vec_ok);
            __syncwarp();
          }
        } else if constexpr (EPI == kEpiBf16) {
          bf16_t* out = reinterpret_cast<bf16_t*>(g.out);
          const bool vec_ok = (g.ldo % 8) == 0 && (g.BN % 8) == 0;
          const int nfl = (g.BN + 63) / 64;
#pragma unroll 1
          for (int f = half; f < nfl; f += 2) {
            uint32_t ra[32], rb[32];
            tmem_ld32(taddr + f * 64, ra);
            tmem_ld32(taddr + f * 64 + 32, rb);      // may reach past BN into unused columns of this buffer
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float o[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) o[e] = __uint_as_float(ra[8 * j + e]);
              stage_put(tile, lane, j, pack8(o));
#pragma unroll
              for (int e = 0; e < 8; ++e) o[e] = __uint_as_float(rb[8 * j + e]);
              stage_put(tile, lane, j + 4, pack8(o));
            }
            __syncwarp();
            stage_flush<bf16_t>(tile, lane, out, g.ldo, tile_off, row0, g.M, f * 64, ncols, vec_ok);
            __syncwarp();
          }
        } else {
          // SwiGLU: the w tile of 256 rows is [gate 64 | up 64 | gate 64 | up 64]; column c of gate group q pairs with column
          // c of the up group behind it. Each warp of a quarter takes one gate/up group pair = 64 output columns.
          bf16_t* out = reinterpret_cast<bf16_t*>(g.out);
          const bool vec_ok = (g.ldo % 8) == 0;
          const int ncols_o = min(g.N / 2 - u.wt * 128, 128);
          const uint32_t tg = taddr + half * 128;
#pragma unroll 1
          for (int c = 0; c < 2; ++c) {            // two chunks of 32 output columns = four 16-byte pieces each
            uint32_t gr[32], ur[32];
            tmem_ld32(tg + c * 32, gr);
            tmem_ld32(tg + 64 + c * 32, ur);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float o[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const float gv = __uint_as_float(gr[8 * j + e]);
                const float uv = __uint_as_float(ur[8 * j + e]);
                o[e] = silu_f(gv) * uv;
              }
              stage_put(tile, lane, c * 4 + j, pack8(o));
            }
          }
          __syncwarp();
          stage_flush<bf16_t>(tile, lane, out, g.ldo, static_cast<int64_t>(u.wt) * 128, row0, g.M, half * 64, ncols_o, vec_ok);
          __syncwarp();
        }
      } else {
        // ---- swapped unit: TMEM lane = row of w = output column, TMEM column = row of x. A warp writes 32 neighbouring
        //      output columns of one row per store.
        const int m0 = g.n_xblk * kBlockM + u.xc * g.tail_box;
        if constexpr (EPI == kEpiSwiglu) {
          // lanes 0-63 of this CTA hold gate rows, lanes 64-127 the matching up rows: the up warps (quarters 2, 3) pass
          // their values through the staging tiles of the gate warps (quarters 0, 1) of the same column half
          const int nch = g.tail_box / 16;
          // (the tile of the up warp: its owner cannot be in the middle of flushing it)
          float* xch = reinterpret_cast<float*>(staging + (4 * half + (quarter & 1)) * 4096) + lane * 17;
#pragma unroll 1
          for (int c = half; c < nch; c += 2) {
            uint32_t r[16];
            tmem_ld16(taddr + c * 16, r);
            tmem_ld_wait();
            if (quarter >= 2) {
#pragma unroll
              for (int e = 0; e < 16; ++e) xch[e] = __uint_as_float(r[e]);
            }
            asm volatile("bar.sync %0, %1;" ::"r"(1 + half), "r"(128) : "memory");
            if (quarter < 2) {
              const int j = u.wt * 128 + static_cast<int>(rank) * 64 + quarter * 32 + lane;      // output column
              const bool col_ok = j < g.N / 2;
#pragma unroll
              for (int e = 0; e < 16; ++e) {
                const int m = m0 + c * 16 + e;
                if (col_ok && m < g.M) {
                  const float gv = __uint_as_float(r[e]), uv = xch[e];
                  reinterpret_cast<bf16_t*>(g.out)[static_cast<int64_t>(m) * g.ldo + j] = f2bf(silu_f(gv) * uv);
                }
              }
            }
            asm volatile("bar.sync %0, %1;" ::"r"(1 + half), "r"(128) : "memory");
          }
        } else {
          const int col = u.wt * 256 + static_cast<int>(rank) * kBM + quarter * 32 + lane;
          const bool col_ok = col < g.N;
#pragma unroll 1
          for (int c = half; c < g.tail_box / 16; c += 2) {
            uint32_t r[16];
            tmem_ld16(taddr + c * 16, r);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const int m = m0 + c * 16 + e;
              if (col_ok && m < g.M) {
                if constexpr (EPI == kEpiBf16) {
                  reinterpret_cast<bf16_t*>(g.out)[static_cast<int64_t>(m) * g.ldo + col] = f2bf(__uint_as_float(r[e]));
                } else {
                  reinterpret_cast<float*>(g.out)[static_cast<int64_t>(u.split) * g.split_stride + static_cast<int64_t>(m) * g.ldo + col] =
                      __uint_as_float(r[e]);
                }
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(accempty_leader + 8 * buf);
      if (tracing) {
        const unsigned long long slot = atomicAdd(g.trace, 1ull);
        if (slot < static_cast<unsigned long long>(g.trace_cap)) {
          unsigned long long* rec = g.trace + 1 + 4 * slot;
          rec[0] = (static_cast<unsigned long long>(pair_id) << 32) | static_cast<unsigned>(unit) | (u.tail ? 1ull << 31 : 0ull);
          rec[1] = t_begin;
          rec[2] = t_full;
          rec[3] = global_timer_ns();
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) report_status(g.status, OJB_DEV_WAIT_TIMEOUT);
    // copies that were already issued must land before the shared memory of this CTA is handed on
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  cluster_sync_all();      // neither CTA leaves (or frees TMEM) while the other may still signal its barriers
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

constexpr size_t kPairSmemBudget = 227 * 1024;

template <int EPI>
int launch_pair(const void* x, const void* w, void* out, int64_t M, int64_t N, int64_t K, int splits, int bn_req, int64_t ldo,
                int32_t* status, cudaStream_t stream) {
  static int smem_set[kMaxDevices] = {};
  auto kern = gemm_pair256_kernel<EPI>;
  if (!raise_smem_limit(kern, static_cast<int>(kPairSmemBudget), smem_set)) return OJB_ERR_LAUNCH;
  const int pairs = sm_count() / 2;
  if (pairs <= 0) return OJB_ERR_LAUNCH;
  GemmArgs g{};
  g.wait_ms = gemm_wait_limit_ms();
  g.M = static_cast<int>(M);
  g.N = static_cast<int>(N);
  g.K = static_cast<int>(K);
  const bool forced_swapped = bn_req < 0;      // variant 6: the SwiGLU weight is then read in the 128-row interleave
  const bool all_swapped = forced_swapped || M <= kBM;
  if (bn_req < 0) bn_req = 0;
  if (all_swapped) {
    // every row of x through swapped-operand units: passes of at most 512 rows, each the accumulator columns of one unit
    const int64_t m16 = ceil_div(M, 16) * 16;
    g.n_xblk = 0;
    g.tail_rows = static_cast<int>(M);
    g.n_xchunk = static_cast<int>(ceil_div(m16, 512));
    g.tail_box = static_cast<int>(ceil_div(ceil_div(m16, g.n_xchunk), 16) * 16);
  } else {
    g.n_xblk = static_cast<int>(M / kBlockM);
    int r = static_cast<int>(M % kBlockM);
    if (r > kBM) { g.n_xblk += 1; r = 0; }
    g.tail_rows = r;
    g.tail_box = (r + 15) / 16 * 16;
    g.n_xchunk = 1;
  }
  g.n_chunk = g.tail_box > 0 ? static_cast<int>(ceil_div(g.tail_box, 256)) : 1;
  g.chunk_w = g.tail_box > 0 ? static_cast<int>(ceil_div(ceil_div(g.tail_box, g.n_chunk), 16) * 16) : 16;
  g.w_split64 = (EPI == kEpiSwiglu && forced_swapped) ? 1 : 0;
  g.splits = splits;
  g.kb_total = static_cast<int>(ceil_div(K, kBK));
  g.kb_per_split = static_cast<int>(ceil_div(g.kb_total, splits));
  if (static_cast<int64_t>(splits - 1) * g.kb_per_split >= g.kb_total) return OJB_ERR_ARG;   // an empty split
  g.BN = EPI == kEpiSwiglu ? 256 : (bn_req > 0 ? bn_req : choose_bn(N, g.n_xblk, g.tail_box, g.n_xchunk, g.tail_rows > 0, splits, g.kb_total, pairs, EPI));
  g.n_wtile = static_cast<int>(ceil_div(N, g.BN));
  g.n_wtile256 = static_cast<int>(ceil_div(N, 256));
  const int tail_half = g.n_chunk * g.chunk_w / 2;      // rows of x per CTA and stage of a swapped unit
  const int half_b = g.n_xblk > 0 ? (g.BN / 2 > tail_half ? g.BN / 2 : tail_half) : tail_half;
  g.stage_bytes = kHalfABytes + static_cast<uint32_t>(half_b) * (kBK * 2);
  g.stage_bytes = (g.stage_bytes + 1023u) & ~1023u;      // every stage starts on a swizzle-atom boundary
  const size_t fixed = 1024 + kStagingBytes + (2 * kPairMaxStages + 4) * 8 + 16;
  g.stages = static_cast<int>((kPairSmemBudget - fixed) / g.stage_bytes);
  if (g.stages > kPairMaxStages) g.stages = kPairMaxStages;
  if (g_pmax_stages >= 2 && g_pmax_stages <= 12 && g.stages > g_pmax_stages) g.stages = g_pmax_stages;
  if (g.stages < 2) return OJB_ERR_LIMIT;
  g.out = out;
  g.ldo = ldo;
  g.split_stride = M * N;
  g.status = status;
  g.trace = g_ptrace;
  g.trace_cap = g_ptrace_cap;
  g.mma_repeat = g_pmma_repeat;
  g.dbg = 0;
  g.tail_sub = 0;
  g.tma_out = 0;
  CUtensorMap map_xh, map_wh, map_w128, map_xt, map_w64;
  int rc = make_map(&map_xh, x, M, K, kBM);
  if (rc == OJB_OK) rc = make_map(&map_wh, w, N, K, g.BN / 2);
  if (rc == OJB_OK) rc = make_map(&map_w128, w, N, K, kBM);
  if (rc == OJB_OK) rc = make_map(&map_xt, x, M, K, g.tail_box > 0 ? g.chunk_w / 2 : 8);
  if (rc == OJB_OK) rc = make_map(&map_w64, w, N, K, 64);
  if (rc != OJB_OK) return rc;
  const int64_t units = static_cast<int64_t>(g.n_xblk) * g.n_wtile * splits +
                        (g.tail_rows > 0 ? static_cast<int64_t>(g.n_wtile256) * splits * g.n_xchunk : 0);
  int n_pairs = static_cast<int>(units < pairs ? units : pairs);
  if (units > n_pairs && g.tail_rows > 0 && g.n_xblk > 0) {
    const int group = (g.n_xblk + g.n_xchunk) * splits;   // units per w tile when BN = 256
    auto gcd = [](int a, int b) { while (b) { const int t = a % b; a = b; b = t; } return a; };
    while (n_pairs > 1 && gcd(n_pairs, group) != 1) --n_pairs;
  }
  const size_t smem = static_cast<size_t>(g.stages) * g.stage_bytes + fixed;
  launch_kernel(kern, dim3(2 * n_pairs), dim3(kPairThreads), smem, stream, map_xh, map_wh, map_w128, map_xt, map_w64, g);
  return launch_status(cudaGetLastError());
}

}  // namespace

void gemm_pair256_set_trace(unsigned long long* buf, int cap) {
  g_ptrace = buf;
  g_ptrace_cap = buf ? cap : 0;
}
#ifdef OJB_GEMM_PROBES
void gemm_pair256_set_probe(int repeat, int max_stages) {
  g_pmma_repeat = repeat >= 0 ? repeat : 1;
  g_pmax_stages = max_stages;
}
#endif

int gemm_pair256_launch(int epi, int bn_req, const void* x, const void* w, void* out, int64_t M, int64_t N, int64_t K,
                        int splits, int64_t ldo, int32_t* status, cudaStream_t stream) {
  if (epi == kEpiBf16) return launch_pair<kEpiBf16>(x, w, out, M, N, K, splits, bn_req, ldo, status, stream);
  if (epi == kEpiSwiglu) return launch_pair<kEpiSwiglu>(x, w, out, M, N, K, splits, bn_req, ldo, status, stream);
  return launch_pair<kEpiPartialF32>(x, w, out, M, N, K, splits, bn_req, ldo, status, stream);
}

}  // namespace ojb
