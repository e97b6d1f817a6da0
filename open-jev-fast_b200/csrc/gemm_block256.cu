// bf16 GEMM, 256-row block kernel (one of two kernels behind ojb_gemm_bf16*; the other is gemm_tile128.cu), sm_100a:
//   out[M,N] = x[M,K] · w[N,K]^T, both operands K-major, fp32 accumulation in tensor memory (TMEM).
//
// One persistent CTA per SM, 320 threads:
//   warp 0      TMA producer  — cp.async.bulk.tensor (plain, non-multicast), 128-byte swizzle, mbarrier completion
//   warp 1      MMA issuer    — one lane issues tcgen05.mma.cta_group::1.kind::f16; tcgen05.commit releases shared-memory
//                               stages and publishes the accumulators
//   warps 2..9  epilogue      — tcgen05.ld of their 32-lane quarter of one of the two accumulators, conversion, stores
// Two kinds of work unit:
//   block unit  256 rows of x (two 128-row sub-tiles) times BN rows of w. Per 64-wide k-block the two MMAs (M = 128, N = BN)
//               share the w tile, so a CTA pulls (256 + BN) rows from L2 for 256 x BN outputs — one third less than a
//               128 x 256 tile. BN is chosen per shape (multiple of 16, <= 256) so that the units fill the SMs.
//   tail unit   rows of x with the operands swapped: 256 rows of w are the M side (two MMAs with M = 128), up to 256 rows
//               of x are the N side (N = rows rounded up to 16), so these rows cost what they are worth instead of whole
//               128-row tiles of zero padding; the epilogue writes the transposed accumulator. Used for the last
//               M mod 256 (<= 128) rows after the blocks, or — for M <= 2048 on request, always for M <= 128 — for all of
//               x in one or two chunks (a pure swapped-operand GEMM).
// Units are ordered x-block fastest, then k-split, then the tail unit of the w tile, then the next w tile, and dealt to the
// CTAs round-robin: the CTAs that run at the same time work on the same few w tiles, which therefore come from HBM once.
// (Giving each CTA a contiguous run instead was measured 15-20 % slower: 136 CTAs then stream 136 different w tiles at
// once, more than the L2 holds, and every unit reads its tile from HBM again.) The grid size is kept coprime with the
// number of units per w tile so that long block units and short tail units are spread evenly over the CTAs.
//
// Every wait on an mbarrier is bounded: after the wait limit (2 s unless ojb_gemm_set_wait_limit_ms changed it) the kernel raises the CTA's abort flag, records
// OJB_DEV_WAIT_TIMEOUT in the status word, lets copies in flight land, frees its TMEM and returns.
#include "gemm_units.cuh"

namespace ojb {
namespace {

constexpr int kGemmThreads = 320;
constexpr int kEpiWarps = 8;
constexpr int kMaxStages = 12;
constexpr uint32_t kABytes = kBlockM * kBK * 2;   // 32 KB: 256 rows of x (block unit) or 256 rows of w (tail unit)
constexpr uint32_t kSubBytes = kBM * kBK * 2;     // 16 KB: one 128-row sub-tile
constexpr uint32_t kAcc1Col = 256;
constexpr uint32_t kStagingBytes = kEpiWarps * 4096;                // TMEM column of the second accumulator

// Measurement hook (process-wide, set by ojb_gemm_set_trace): where the kernel records unit timelines.
unsigned long long* g_trace = nullptr;
int g_trace_cap = 0;
#ifdef OJB_GEMM_PROBES
int g_mma_repeat = 1;   // MMAs of every stage issued this many times
int g_max_stages = 0;   // 2..12: cap on the number of pipeline stages
int g_dbg = 0;          // 100 / 101: the block epilogue skips its global stores / its TMEM loads; 102: MMAs with M = 64
#else
constexpr int g_mma_repeat = 1, g_max_stages = 0, g_dbg = 0;
#endif

// FP8: the operands are e4m3 bytes (a k-block of 128 bytes is then 128 elements of K and an MMA covers 32 of them); the
// epilogue multiplies the accumulator by the scale of its row of x and of its row of w. Everything counted in bytes (stages,
// swizzle, descriptors) is the same for both operand types.
template <int EPI, bool FP8>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_block256_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    const __grid_constant__ CUtensorMap map_w256, const __grid_constant__ CUtensorMap map_xt,
                    const __grid_constant__ CUtensorMap map_out, const __grid_constant__ CUtensorMap map_w128,
                    const __grid_constant__ CUtensorMap map_tail, GemmArgs g) {
  pdl_launch_dependents();
  constexpr uint32_t kTmemCols = 512;
  constexpr int kKE = FP8 ? 128 : kBK;      // elements of K per k-block (the coordinate step of the copies)
  auto mma = [](uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
    if constexpr (FP8) umma_f8(d, a, b, idesc, acc); else umma_bf16(d, a, b, idesc, acc);
  };
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* staging = smem + static_cast<size_t>(g.stages) * g.stage_bytes;       // [8 warps][32 rows][128 bytes] when tma_out
  // staging: 4 KB per epilogue warp when block units store through it, 2 KB when only swapped units do (a third tile in
  // rotation was measured: no gain, the epilogue of a swapped unit is bound by its 2-byte shared-memory stores)
  const uint32_t stg_warp = g.tma_out ? 4096u : (g.tail_tma ? 2048u : 0u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + kEpiWarps * stg_warp);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kMaxStages + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const uint32_t tiles0 = smem_u32(smem);
  const uint32_t full0 = smem_u32(bars);
  const uint32_t empty0 = full0 + 8 * kMaxStages;
  const uint32_t accfull = empty0 + 8 * kMaxStages;
  const uint32_t accempty = accfull + 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int STAGES = g.stages;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    mbar_init(accfull, 1);
    mbar_init(accempty, kEpiWarps);
    abort_flag[0] = 0;
    abort_flag[1] = g.wait_ms;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w256) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_xt) : "memory");
    if (g.tma_out) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_out) : "memory");
    if (g.tail_sub) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w128) : "memory");
    if (g.tail_tma) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_tail) : "memory");
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();      // from here on the previous kernel of the stream has completed

  const int total_block = g.n_xblk * g.n_wtile * g.splits;
  const int total_units = total_block + (g.tail_rows > 0 ? g.n_wtile256 * g.splits * g.n_xchunk : 0);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
        const Unit u = decode_unit(g, unit, total_block);
        const uint32_t tx = kABytes + static_cast<uint32_t>(u.tail ? g.tail_box : g.BN) * (kBK * 2);
        if (u.tail && g.tail_sub) {
          // A short tail next to full blocks: its own k-block (36 KB) would leave most of the 64 KB stage empty and too few
          // bytes in flight, so a stage carries three sub-stages instead — (k-block, half of the w tile) pairs, each 128 rows
          // of w plus the x rows — in the order gate half, up half, next k-block ...
          const int nh = 2 * (u.kb1 - u.kb0);
          for (int h0 = 0; h0 < nh; h0 += 3) {
            const int cnt = nh - h0 < 3 ? nh - h0 : 3;
            if (!mbar_wait(empty0 + 8 * stage, phase ^ 1u, abort_flag)) { ok = false; break; }
            const uint32_t a_dst = tiles0 + stage * g.stage_bytes;
            const uint32_t fb = full0 + 8 * stage;
            mbar_expect_tx(fb, static_cast<uint32_t>(cnt * g.tail_sub));
            for (int j = 0; j < cnt; ++j) {
              const int h = h0 + j, kb = u.kb0 + (h >> 1);
              tma_load_2d(a_dst + j * g.tail_sub, &map_w128, fb, kb * kKE, u.wt * 256 + (h & 1) * kBM);
              tma_load_2d(a_dst + j * g.tail_sub + kSubBytes, &map_xt, fb, kb * kKE, g.n_xblk * kBlockM + u.xc * g.tail_box);
            }
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          }
          continue;
        }
        for (int kb = u.kb0; kb < u.kb1; ++kb) {
          if (!mbar_wait(empty0 + 8 * stage, phase ^ 1u, abort_flag)) { ok = false; break; }
          const uint32_t a_dst = tiles0 + stage * g.stage_bytes;
          const uint32_t fb = full0 + 8 * stage;
          mbar_expect_tx(fb, tx);
          if (!u.tail) {
            tma_load_2d(a_dst, &map_x, fb, kb * kKE, u.xb * kBlockM);
            tma_load_2d(a_dst + kABytes, &map_w, fb, kb * kKE, u.wt * g.BN);
          } else {
            tma_load_2d(a_dst, &map_w256, fb, kb * kKE, u.wt * 256);
            tma_load_2d(a_dst + kABytes, &map_xt, fb, kb * kKE, g.n_xblk * kBlockM + u.xc * g.tail_box);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
        const Unit u = decode_unit(g, unit, total_block);
        const uint32_t idesc = FP8 ? umma_idesc_e4m3(u.tail ? g.tail_box : g.BN) : umma_idesc(u.tail ? g.tail_box : g.BN);
        if (!mbar_wait(accempty, acc_phase ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        if (u.tail && g.tail_sub) {
          const int nh = 2 * (u.kb1 - u.kb0);
          for (int h0 = 0; h0 < nh; h0 += 3) {
            const int cnt = nh - h0 < 3 ? nh - h0 : 3;
            if (!mbar_wait(full0 + 8 * stage, phase, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint32_t a_addr = tiles0 + stage * g.stage_bytes;
            for (int j = 0; j < cnt; ++j) {
              const int h = h0 + j;
              const uint32_t acc = tmem_base + ((h & 1) ? kAcc1Col : 0u);
              const uint64_t adesc = smem_desc_sw128(a_addr + j * g.tail_sub);
              const uint64_t bdesc = smem_desc_sw128(a_addr + j * g.tail_sub + kSubBytes);
#pragma unroll
              for (int k = 0; k < kBK / kUmmaK; ++k) mma(acc, adesc + 2 * k, bdesc + 2 * k, idesc, (h >= 2 || k > 0) ? 1u : 0u);
            }
            umma_commit(empty0 + 8 * stage);
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          }
          if (!ok) break;
          umma_commit(accfull);
          acc_phase ^= 1u;
          continue;
        }
        for (int kb = u.kb0; kb < u.kb1; ++kb) {
          if (!mbar_wait(full0 + 8 * stage, phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = tiles0 + stage * g.stage_bytes;
          const uint64_t adesc0 = smem_desc_sw128(a_addr);
          const uint64_t adesc1 = smem_desc_sw128(a_addr + kSubBytes);
          const uint64_t bdesc = smem_desc_sw128(a_addr + kABytes);
          if (OJB_PROBE_REPEAT(g) == 1) {
#pragma unroll
            for (int k = 0; k < kBK / kUmmaK; ++k) {
              // advancing K by 16 bf16 = 32 bytes inside the swizzle row: +2 in the (address >> 4) field
              const uint32_t accum = (kb > u.kb0 || k > 0) ? 1u : 0u;
              mma(tmem_base, adesc0 + 2 * k, bdesc + 2 * k, idesc, accum);
              mma(tmem_base + kAcc1Col, adesc1 + 2 * k, bdesc + 2 * k, idesc, accum);
            }
          } else {                                   // probe builds only
            // knob 102: the same MMAs with M = 64 in the instruction descriptor (what does a half-height MMA cost?)
            const uint32_t idesc_m = OJB_PROBE_DBG(g) == 102 ? ((idesc & ~(0x1fu << 24)) | (static_cast<uint32_t>(64 >> 4) << 24)) : idesc;
            for (int rep = 0; rep < OJB_PROBE_REPEAT(g); ++rep)
              for (int k = 0; k < kBK / kUmmaK; ++k) {
                const uint32_t accum = (kb > u.kb0 || k > 0 || rep > 0) ? 1u : 0u;
                mma(tmem_base, adesc0 + 2 * k, bdesc + 2 * k, idesc_m, accum);
                mma(tmem_base + kAcc1Col, adesc1 + 2 * k, bdesc + 2 * k, idesc_m, accum);
              }
          }
          umma_commit(empty0 + 8 * stage);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit(accfull);
        acc_phase ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9)
    const int quarter = warp & 3;           // TMEM lanes [32*quarter, 32*quarter+32) are the ones this warp may read
    const int acc_id = (warp - 2) >> 2;     // warps 2-5 read accumulator 0, warps 6-9 accumulator 1
    // e4m3 operands: scale of row n of w / row m of x (indices clamped: tiles may reach past the matrix)
    auto sw_at = [&](int n) -> float { if constexpr (FP8) return __ldg(g.sw + min(n, g.N - 1)); else return 1.f; };
    auto sx_at = [&](int m) -> float { if constexpr (FP8) return __ldg(g.sx + min(m, g.M - 1)); else return 1.f; };
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
      const Unit u = decode_unit(g, unit, total_block);
      const bool tracing = g.trace != nullptr && warp == 2 && lane == 0;
      const unsigned long long t_begin = tracing ? global_timer_ns() : 0ull;
      if (!mbar_wait(accfull, acc_phase, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const unsigned long long t_full = tracing ? global_timer_ns() : 0ull;
      const uint32_t tlane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
      const uint32_t taddr = tlane + static_cast<uint32_t>(acc_id) * kAcc1Col;
      if (!u.tail) {
        // ---- block unit: this thread owns one row of x, the accumulator columns are output columns
        const int row = u.xb * kBlockM + acc_id * kBM + quarter * 32 + lane;
        const bool row_ok = row < g.M;
        const float rs = sx_at(row);
        if (g.tma_out) {
          // ---- through shared memory: the warp's 32 rows x 128 bytes go into a swizzled tile (16-byte piece j of row r at
          //      slot j ^ (r & 7), the layout of the 128-byte swizzle) and one lane hands the tile to the bulk-copy engine,
          //      which clips it at the edges of out. Stores issued by the threads themselves reach only ~17 GB/s per SM.
          uint8_t* tile = staging + (warp - 2) * 4096;
          const uint32_t tile_s = smem_u32(tile);
          const int row0 = u.xb * kBlockM + acc_id * kBM + quarter * 32;
          auto put = [&](int j, const uint4& v) { *reinterpret_cast<uint4*>(tile + lane * 128 + ((j ^ (lane & 7)) << 4)) = v; };
          auto flush = [&](int col) {     // col = first output column of the tile
            fence_proxy_async();
            __syncwarp();
            if (lane == 0 && row0 < g.M) {
              tma_store_3d(&map_out, tile_s, col, row0, EPI == kEpiPartialF32 ? u.split : 0);
              bulk_commit();
            }
          };
          auto reuse = [&]() {            // the previous store of this warp has read the tile
            if (lane == 0) bulk_wait_read();
            __syncwarp();
          };
          if constexpr (EPI == kEpiSwiglu) {
#pragma unroll 1
            for (int t = 0; t < 2; ++t) {          // two tiles of 64 output columns
              uint32_t gr[32], ur[32];
#pragma unroll 1
              for (int c = 0; c < 2; ++c) {
                tmem_ld32(taddr + t * 64 + c * 32, gr);
                tmem_ld32(taddr + 128 + t * 64 + c * 32, ur);
                tmem_ld_wait();
                if (c == 0) reuse();
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  float o[8];
#pragma unroll
                  for (int e = 0; e < 8; e += 2) {
                    float g0 = __uint_as_float(gr[8 * j + e]), g1 = __uint_as_float(gr[8 * j + e + 1]);
                    float u0 = __uint_as_float(ur[8 * j + e]), u1 = __uint_as_float(ur[8 * j + e + 1]);
                    if constexpr (FP8) {
                      const int wr = u.wt * 256 + t * 64 + c * 32 + 8 * j + e;      // gate row of w; its up row is 128 further
                      g0 *= rs * sw_at(wr); g1 *= rs * sw_at(wr + 1);
                      u0 *= rs * sw_at(wr + 128); u1 *= rs * sw_at(wr + 129);
                    }
                    float s0, s1;
                    silu2_f(g0, g1, s0, s1);
                    o[e] = s0 * u0;
                    o[e + 1] = s1 * u1;
                  }
                  put(c * 4 + j, pack8(o));
                }
              }
              if (u.wt * 128 + t * 64 < g.N / 2) flush(u.wt * 128 + t * 64);
            }
          } else if constexpr (EPI == kEpiBf16) {
            const int nt = g.BN / 64;              // BN is a multiple of 64 on this path
#pragma unroll 1
            for (int t = 0; t < nt; ++t) {
              uint32_t ra[32], rb[32];
              tmem_ld32(taddr + t * 64, ra);
              tmem_ld32(taddr + t * 64 + 32, rb);
              tmem_ld_wait();
              reuse();
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                float o[8];
                const int wr = u.wt * g.BN + t * 64 + 8 * j;
#pragma unroll
                for (int e = 0; e < 8; ++e) o[e] = __uint_as_float(ra[8 * j + e]) * (FP8 ? rs * sw_at(wr + e) : 1.f);
                put(j, pack8(o));
#pragma unroll
                for (int e = 0; e < 8; ++e) o[e] = __uint_as_float(rb[8 * j + e]) * (FP8 ? rs * sw_at(wr + 32 + e) : 1.f);
                put(j + 4, pack8(o));
              }
              if (u.wt * g.BN + t * 64 < g.N) flush(u.wt * g.BN + t * 64);
            }
          } else {
            const int nt = g.BN / 32;              // BN is a multiple of 32 on this path
#pragma unroll 1
            for (int t = 0; t < nt; ++t) {
              uint32_t r[32];
              tmem_ld32(taddr + t * 32, r);
              tmem_ld_wait();
              reuse();
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                if constexpr (FP8) {
                  const int wr = u.wt * g.BN + t * 32 + 4 * j;
#pragma unroll
                  for (int e = 0; e < 4; ++e) r[4 * j + e] = __float_as_uint(__uint_as_float(r[4 * j + e]) * rs * sw_at(wr + e));
                }
                put(j, make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]));
              }
              if (u.wt * g.BN + t * 32 < g.N) flush(u.wt * g.BN + t * 32);
            }
          }
        } else
        // TMEM loads are issued one chunk ahead of the chunk being converted and stored, so their latency overlaps the
        // stores instead of adding up once per chunk.
        if constexpr (EPI == kEpiSwiglu) {
          // BN = 256: columns [0,128) of the tile are gate_j, columns [128,256) the matching up_j
          bf16_t* orow = reinterpret_cast<bf16_t*>(g.out) + static_cast<int64_t>(row) * g.ldo + static_cast<int64_t>(u.wt) * 128;
          const int ncols = g.N / 2 - u.wt * 128;
          auto emit = [&](int c, const uint32_t (&gr)[16], const uint32_t (&ur)[16]) {
            if (!row_ok) return;
#pragma unroll
            for (int j = 0; j < 16; j += 8) {
              if (c * 16 + j < ncols) {
                float o[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                  const float gv = __uint_as_float(gr[j + e]);
                  const float uv = __uint_as_float(ur[j + e]);
                  o[e] = silu_f(gv) * uv;
                }
                *reinterpret_cast<uint4*>(orow + c * 16 + j) = pack8(o);
              }
            }
          };
          uint32_t ga[16], ua[16], gb[16], ub[16];
          tmem_ld16(taddr, ga);
          tmem_ld16(taddr + 128, ua);
          tmem_ld_wait();
#pragma unroll 1
          for (int c = 0; c < 8; c += 2) {
            tmem_ld16(taddr + (c + 1) * 16, gb);
            tmem_ld16(taddr + 128 + (c + 1) * 16, ub);
            emit(c, ga, ua);
            tmem_ld_wait();
            if (c + 2 < 8) {
              tmem_ld16(taddr + (c + 2) * 16, ga);
              tmem_ld16(taddr + 128 + (c + 2) * 16, ua);
            }
            emit(c + 1, gb, ub);
            tmem_ld_wait();
          }
        } else {
          constexpr bool kF32 = EPI == kEpiPartialF32;
          const int64_t off = static_cast<int64_t>(row) * g.ldo + static_cast<int64_t>(u.wt) * g.BN +
                              (kF32 ? static_cast<int64_t>(u.split) * g.split_stride : 0);
          bf16_t* orow_h = reinterpret_cast<bf16_t*>(g.out) + off;
          float* orow_f = reinterpret_cast<float*>(g.out) + off;
          const int ncols = min(g.N - u.wt * g.BN, g.BN);      // columns of this tile that exist
          const bool vec_ok = (g.ldo % 8) == 0 && (g.BN % 8) == 0;
          auto emit = [&](int c, const uint32_t (&r)[32]) {
            if (!row_ok || OJB_PROBE_DBG(g) == 100) return;
            if constexpr (kF32) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                const int col = c * 32 + j;
                if (col + 4 <= ncols && vec_ok) {
                  *reinterpret_cast<uint4*>(orow_f + col) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
                } else {
#pragma unroll
                  for (int e = 0; e < 4; ++e)
                    if (col + e < ncols) orow_f[col + e] = __uint_as_float(r[j + e]);
                }
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                const int col = c * 32 + j;
                if (col + 8 <= ncols && vec_ok) {
                  float o[8];
#pragma unroll
                  for (int e = 0; e < 8; ++e) o[e] = __uint_as_float(r[j + e]);
                  *reinterpret_cast<uint4*>(orow_h + col) = pack8(o);
                } else {
#pragma unroll
                  for (int e = 0; e < 8; ++e)
                    if (col + e < ncols) orow_h[col + e] = f2bf(__uint_as_float(r[j + e]));
                }
              }
            }
          };
          // chunks of 32 columns; the last one may reach past BN into unused columns of this accumulator's 256
          const int nch = (g.BN + 31) / 32;
          uint32_t ra[32], rb[32];
          const bool ld = OJB_PROBE_DBG(g) != 101;
          if (ld) tmem_ld32(taddr, ra);
          tmem_ld_wait();
#pragma unroll 1
          for (int c = 0; c < nch; c += 2) {
            if (c + 1 < nch && ld) tmem_ld32(taddr + (c + 1) * 32, rb);
            emit(c, ra);
            tmem_ld_wait();
            if (c + 1 < nch) {
              if (c + 2 < nch && ld) tmem_ld32(taddr + (c + 2) * 32, ra);
              emit(c + 1, rb);
              tmem_ld_wait();
            }
          }
        }
      } else {
        // ---- tail unit (operands swapped): this thread owns one row of w = one output column, the accumulator columns
        //      are the tail rows of x. A warp writes 32 neighbouring output columns of one row per store.
        const int m0 = g.n_xblk * kBlockM + u.xc * g.tail_box;
        if constexpr (EPI == kEpiSwiglu) {
          // accumulator 0 holds gate rows, accumulator 1 the matching up rows of the same lanes; the two warp sets (both
          // can read these lanes) share the x rows of the chunk between them
          {
            const int j = u.wt * 128 + quarter * 32 + lane;       // output column
            const bool col_ok = j < g.N / 2;
            bf16_t* ocol = reinterpret_cast<bf16_t*>(g.out) + j;
            const int nchunk = g.tail_box / 16;
            const float swg = sw_at(u.wt * 256 + quarter * 32 + lane), swu = sw_at(u.wt * 256 + 128 + quarter * 32 + lane);
            uint8_t* tile0 = staging + (warp - 2) * stg_warp;
            if (g.tail_tma) {          // the stores of this warp's previous unit have read its tiles
              if (lane == 0) bulk_wait_read();
              __syncwarp();
            }
#pragma unroll 1
            for (int c = acc_id; c < nchunk; c += 2) {
              uint32_t gr[16], ur[16];
              tmem_ld16(tlane + c * 16, gr);
              tmem_ld16(tlane + kAcc1Col + c * 16, ur);
              tmem_ld_wait();
              if (g.tail_tma) {
                // [16 rows of x][32 output columns] tile, one bulk tensor store per chunk (clipped at the edges of out)
                bf16_t* t = reinterpret_cast<bf16_t*>(tile0 + ((c >> 1) & 1) * 1024);
                if (c >= acc_id + 4) {
                  if (lane == 0) bulk_wait_read1();
                  __syncwarp();
                }
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                  const float xs = sx_at(m0 + c * 16 + e);
                  const float gv = __uint_as_float(gr[e]) * (FP8 ? xs * swg : 1.f);
                  const float uv = __uint_as_float(ur[e]) * (FP8 ? xs * swu : 1.f);
                  t[e * 32 + lane] = f2bf(silu_f(gv) * uv);
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0 && u.wt * 128 + quarter * 32 < g.N / 2) {
                  tma_store_3d(&map_tail, smem_u32(t), u.wt * 128 + quarter * 32, m0 + c * 16, 0);
                  bulk_commit();
                }
                continue;
              }
#pragma unroll
              for (int e = 0; e < 16; ++e) {
                const int m = m0 + c * 16 + e;
                if (col_ok && m < g.M) {
                  const float xs = sx_at(m);
                  const float gv = __uint_as_float(gr[e]) * (FP8 ? xs * swg : 1.f);
                  const float uv = __uint_as_float(ur[e]) * (FP8 ? xs * swu : 1.f);
                  ocol[static_cast<int64_t>(m) * g.ldo] = f2bf(silu_f(gv) * uv);
                }
              }
            }
          }
        } else {
          const int col = u.wt * 256 + acc_id * kBM + quarter * 32 + lane;
          const bool col_ok = col < g.N;
          const float swc = sw_at(col);
          uint8_t* tile0 = staging + (warp - 2) * stg_warp;
          // bf16: two tiles of 1 KB in turn; fp32: tiles of 2 KB, two of them only beside the 4 KB block-unit tiles
          const bool two = stg_warp == 4096u;
          if (g.tail_tma) {          // the stores of this warp's previous unit have read its tiles
            if (lane == 0) bulk_wait_read();
            __syncwarp();
          }
          // one chunk of 16 accumulator columns (= 16 rows of x); TMEM loads run one chunk ahead of the chunk being stored
          auto emit = [&](int c, const uint32_t (&r)[16]) {
            if (g.tail_tma) {
              uint8_t* t;
              if constexpr (EPI == kEpiPartialF32) {
                t = tile0 + (two ? (c & 1) * 2048 : 0);
                if (two ? c >= 2 : c >= 1) {
                  if (lane == 0) { if (two) bulk_wait_read1(); else bulk_wait_read(); }
                  __syncwarp();
                }
              } else {
                t = tile0 + (c & 1) * 1024;
                if (c >= 2) {
                  if (lane == 0) bulk_wait_read1();
                  __syncwarp();
                }
              }
#pragma unroll
              for (int e = 0; e < 16; ++e) {
                const float v = __uint_as_float(r[e]) * (FP8 ? swc * sx_at(m0 + c * 16 + e) : 1.f);
                if constexpr (EPI == kEpiBf16) reinterpret_cast<bf16_t*>(t)[e * 32 + lane] = f2bf(v);
                else reinterpret_cast<float*>(t)[e * 32 + lane] = v;
              }
              fence_proxy_async();
              __syncwarp();
              const int col0 = u.wt * 256 + acc_id * kBM + quarter * 32;
              if (lane == 0 && col0 < g.N) {
                tma_store_3d(&map_tail, smem_u32(t), col0, m0 + c * 16, EPI == kEpiPartialF32 ? u.split : 0);
                bulk_commit();
              }
              return;
            }
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const int m = m0 + c * 16 + e;
              if (col_ok && m < g.M) {
                const float v = __uint_as_float(r[e]) * (FP8 ? swc * sx_at(m) : 1.f);
                if constexpr (EPI == kEpiBf16) {
                  reinterpret_cast<bf16_t*>(g.out)[static_cast<int64_t>(m) * g.ldo + col] = f2bf(v);
                } else {
                  reinterpret_cast<float*>(g.out)[static_cast<int64_t>(u.split) * g.split_stride + static_cast<int64_t>(m) * g.ldo + col] = v;
                }
              }
            }
          };
          const int nch = g.tail_box / 16;
          uint32_t ra[16], rb[16];
          tmem_ld16(taddr, ra);
          tmem_ld_wait();
#pragma unroll 1
          for (int c = 0; c < nch; c += 2) {
            if (c + 1 < nch) tmem_ld16(taddr + (c + 1) * 16, rb);
            emit(c, ra);
            tmem_ld_wait();
            if (c + 1 < nch) {
              if (c + 2 < nch) tmem_ld16(taddr + (c + 2) * 16, ra);
              emit(c + 1, rb);
              tmem_ld_wait();
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(accempty);
      acc_phase ^= 1u;
      if (tracing) {
        const unsigned long long slot = atomicAdd(g.trace, 1ull);
        if (slot < static_cast<unsigned long long>(g.trace_cap)) {
          unsigned long long* rec = g.trace + 1 + 4 * slot;
          rec[0] = (static_cast<unsigned long long>(blockIdx.x) << 32) | static_cast<unsigned>(unit) | (u.tail ? 1ull << 31 : 0ull);
          rec[1] = t_begin;
          rec[2] = t_full;
          rec[3] = global_timer_ns();
        }
      }
    }
    if ((g.tma_out || g.tail_tma) && lane == 0) bulk_wait_all();     // the shared-memory tiles must outlive the stores that read them
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) report_status(g.status, OJB_DEV_WAIT_TIMEOUT);
    // copies that were already issued must land before the shared memory of this CTA is handed on
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

constexpr size_t kSmemBudget = 227 * 1024;

template <int EPI, bool FP8 = false>
int launch_gemm(const void* x, const void* w, void* out, int64_t M, int64_t N, int64_t K, int splits, int bn_req, int64_t ldo,
                int32_t* status, cudaStream_t stream, const float* sx = nullptr, const float* sw = nullptr) {
  static int smem_set[kMaxDevices] = {};
  auto kern = gemm_block256_kernel<EPI, FP8>;
  if (!raise_smem_limit(kern, static_cast<int>(kSmemBudget), smem_set)) return OJB_ERR_LAUNCH;
  const int sms = sm_count();
  if (sms <= 0) return OJB_ERR_LAUNCH;
  GemmArgs g{};
  g.wait_ms = gemm_wait_limit_ms();
  g.M = static_cast<int>(M);
  g.N = static_cast<int>(N);
  g.K = static_cast<int>(K);
  // bn_req == -1: every row of x goes through swapped-operand units (M <= 2048: chunks of <= 256 rows); bn_req == -2: all
  // but the last full 256-row block go through block units and the remaining 257..511 rows through two swapped-operand
  // chunks that fit them exactly (544 rows = one block + 2 x 144: no MMA runs at the 64-clock floor of a short tail);
  // otherwise full 256-row blocks plus a swapped tail of <= 128 rows (a longer remainder is cheaper as one more zero-padded
  // block)
  const bool hybrid = bn_req == -2 && M > kBlockM;
  const bool all_swapped = (bn_req < 0 && !hybrid) || M <= kBM;
  if (bn_req < 0) bn_req = 0;
  if (all_swapped) {
    if (M > 2048) return OJB_ERR_LIMIT;
    g.n_xblk = 0;
    g.tail_rows = static_cast<int>(M);
    g.n_xchunk = static_cast<int>(ceil_div(M, 256));
    g.tail_box = static_cast<int>(ceil_div(ceil_div(M, g.n_xchunk), 16) * 16);
  } else if (hybrid) {
    g.n_xblk = static_cast<int>(M / kBlockM) - 1;
    g.tail_rows = static_cast<int>(M - static_cast<int64_t>(g.n_xblk) * kBlockM);      // 256 .. 511 rows
    g.n_xchunk = static_cast<int>(ceil_div(g.tail_rows, 256));
    g.tail_box = static_cast<int>(ceil_div(ceil_div(g.tail_rows, g.n_xchunk), 16) * 16);
  } else {
    g.n_xblk = static_cast<int>(M / kBlockM);
    int r = static_cast<int>(M % kBlockM);
    if (r > kBM) { g.n_xblk += 1; r = 0; }
    g.tail_rows = r;
    g.tail_box = (r + 15) / 16 * 16;
    g.n_xchunk = 1;
  }
  g.splits = splits;
  g.kb_total = static_cast<int>(ceil_div(K, FP8 ? 128 : kBK));
  g.kb_per_split = static_cast<int>(ceil_div(g.kb_total, splits));
  if (static_cast<int64_t>(splits - 1) * g.kb_per_split >= g.kb_total) return OJB_ERR_ARG;   // an empty split
  g.BN = EPI == kEpiSwiglu ? 256 : (bn_req > 0 ? bn_req : choose_bn(N, g.n_xblk, g.tail_box, g.n_xchunk, g.tail_rows > 0, splits, g.kb_total, sms, EPI));
  if (FP8 && g.BN % 64 != 0) g.BN = (g.BN + 63) / 64 * 64;      // whole 128-byte store tiles (the scaled epilogue needs them)
  g.n_wtile = static_cast<int>(ceil_div(N, g.BN));
  g.n_wtile256 = static_cast<int>(ceil_div(N, 256));
  {
    // x beyond what the L2 keeps beside the streaming weight (64 MB) and at least 24 x blocks (with fewer, the CTAs that
    // run at the same time already cover several weight tiles per x block, and x is re-read only a few times): bands of about
    // 40 MB of x, equal in size. OJB_GEMM_BAND_MB changes the band size (0 = no bands) for measurements.
    const int64_t xblk_bytes = static_cast<int64_t>(kBlockM) * K * (FP8 ? 1 : 2);
    static const int64_t band_mb = [] { const char* e = getenv("OJB_GEMM_BAND_MB"); return e ? static_cast<int64_t>(atoi(e)) : 40ll; }();
    g.band_xblk = 0;
    if (band_mb > 0 && g.n_xblk >= 24 && static_cast<int64_t>(g.n_xblk) * xblk_bytes > (64ll << 20)) {
      const int64_t per_band = (band_mb << 20) / xblk_bytes > 2 ? (band_mb << 20) / xblk_bytes : 2;
      const int64_t n_bands = ceil_div(g.n_xblk, per_band);
      g.band_xblk = static_cast<int>(ceil_div(g.n_xblk, n_bands));
    }
  }
  const int b_rows = g.n_xblk > 0 ? (g.BN > g.tail_box ? g.BN : g.tail_box) : g.tail_box;
  g.stage_bytes = kABytes + static_cast<uint32_t>(b_rows) * (kBK * 2);
  {
    const uint32_t sub = kSubBytes + static_cast<uint32_t>(g.tail_box) * (kBK * 2);
    g.tail_sub = (g.n_xblk > 0 && g.tail_rows > 0 && g.tail_box <= 32 && 3 * sub <= g.stage_bytes && g_mma_repeat == 1) ? static_cast<int>(sub) : 0;
  }
  // bulk tensor stores need 16-byte aligned rows and whole 128-byte tiles inside every w tile
  const int64_t out_cols = EPI == kEpiSwiglu ? N / 2 : N;
  const int out_elt = EPI == kEpiPartialF32 ? 4 : 2;
  g.tma_out = g.n_xblk > 0 && (ldo * out_elt) % 16 == 0 && g.BN % (128 / out_elt) == 0 ? 1 : 0;
  g.tail_tma = (g.tail_rows > 0 && (ldo * out_elt) % 16 == 0 && (EPI != kEpiPartialF32 || (M * N * 4) % 16 == 0)) ? 1 : 0;
  const size_t fixed = 1024 + (2 * kMaxStages + 2) * 8 + 16 + (g.tma_out ? kStagingBytes : (g.tail_tma ? kEpiWarps * 2048 : 0));
  g.stages = static_cast<int>((kSmemBudget - fixed) / g.stage_bytes);
  if (g.stages > kMaxStages) g.stages = kMaxStages;
  if (g_max_stages >= 2 && g_max_stages <= 12 && g.stages > g_max_stages) g.stages = g_max_stages;
  if (g.stages < 2) return OJB_ERR_LIMIT;
  g.out = out;
  g.ldo = ldo;
  g.split_stride = M * N;
  g.status = status;
  g.trace = g_trace;
  g.trace_cap = g_trace_cap;
  g.mma_repeat = g_mma_repeat;
  g.dbg = g_dbg;
  g.sx = sx;
  g.sw = sw;
  if (FP8 && g.n_xblk > 0 && !g.tma_out) return OJB_ERR_ARG;      // the scaled block epilogue exists on the bulk-store path only
  auto mk = FP8 ? make_map_u8 : make_map;
  CUtensorMap map_x, map_w, map_w256, map_xt;
  int rc = mk(&map_x, x, M, K, kBlockM);
  if (rc == OJB_OK) rc = mk(&map_w, w, N, K, g.BN);
  if (rc == OJB_OK) rc = mk(&map_w256, w, N, K, 256);
  if (rc == OJB_OK) rc = mk(&map_xt, x, M, K, g.tail_box > 0 ? g.tail_box : 16);
  CUtensorMap map_w128;
  if (rc == OJB_OK) rc = mk(&map_w128, w, N, K, kBM);
  CUtensorMap map_out = map_xt;
  if (rc == OJB_OK && g.tma_out)
    rc = make_out_map(&map_out, out, out_elt, M, out_cols, ldo, EPI == kEpiPartialF32 ? splits : 1, g.split_stride);
  CUtensorMap map_tail = map_xt;
  if (rc == OJB_OK && g.tail_tma)
    rc = make_tail_out_map(&map_tail, out, out_elt, M, out_cols, ldo, EPI == kEpiPartialF32 ? splits : 1, g.split_stride);
  if (rc != OJB_OK) return rc;
  const int64_t units = static_cast<int64_t>(g.n_xblk) * g.n_wtile * splits +
                        (g.tail_rows > 0 ? static_cast<int64_t>(g.n_wtile256) * splits * g.n_xchunk : 0);
  int grid = static_cast<int>(units < sms ? units : sms);
  if (units > grid && g.tail_rows > 0) {
    const int group = (g.n_xblk + g.n_xchunk) * splits;   // units per w tile when BN = 256
    auto gcd = [](int a, int b) { while (b) { const int t = a % b; a = b; b = t; } return a; };
    while (grid > 1 && gcd(grid, group) != 1) --grid;
  }
  const size_t smem = static_cast<size_t>(g.stages) * g.stage_bytes + fixed;
  launch_kernel(kern, dim3(grid), dim3(kGemmThreads), smem, stream, map_x, map_w, map_w256, map_xt, map_out, map_w128, map_tail, g);
  return launch_status(cudaGetLastError());
}

}  // namespace

void gemm_block256_set_trace(unsigned long long* buf, int cap) {
  g_trace = buf;
  g_trace_cap = buf ? cap : 0;
}
#ifdef OJB_GEMM_PROBES
void gemm_block256_set_probe(int repeat, int knob) {
  g_mma_repeat = repeat >= 0 ? repeat : 1;
  g_max_stages = knob >= 100 ? 0 : knob;
  g_dbg = knob >= 100 ? knob : 0;
}
#endif

int gemm_block256_launch(int epi, int bn_req, const void* x, const void* w, void* out, int64_t M, int64_t N, int64_t K,
                         int splits, int64_t ldo, int32_t* status, cudaStream_t stream) {
  if (epi == kEpiBf16) return launch_gemm<kEpiBf16>(x, w, out, M, N, K, splits, bn_req, ldo, status, stream);
  if (epi == kEpiSwiglu) return launch_gemm<kEpiSwiglu>(x, w, out, M, N, K, splits, bn_req, ldo, status, stream);
  return launch_gemm<kEpiPartialF32>(x, w, out, M, N, K, splits, bn_req, ldo, status, stream);
}

int gemm_block256_launch_e4m3(int epi, const void* xq, const float* sx, const void* wq, const float* sw, void* out, int64_t M,
                              int64_t N, int64_t K, int splits, int64_t ldo, int32_t* status, cudaStream_t stream) {
  if (epi == kEpiBf16) return launch_gemm<kEpiBf16, true>(xq, wq, out, M, N, K, splits, 0, ldo, status, stream, sx, sw);
  if (epi == kEpiSwiglu) return launch_gemm<kEpiSwiglu, true>(xq, wq, out, M, N, K, splits, 0, ldo, status, stream, sx, sw);
  return launch_gemm<kEpiPartialF32, true>(xq, wq, out, M, N, K, splits, 0, ldo, status, stream, sx, sw);
}

}  // namespace ojb

// Host-side listing of the unit order of the block kernels for a given geometry (no GPU work): out[5 * i .. 5 * i + 4] =
// (tail, x block, k range, w tile, x chunk) of the i-th unit. Returns the number of units, or a negative error code.
extern "C" int64_t ojb_gemm_unit_order(int32_t n_xblk, int32_t tail_rows, int32_t n_xchunk, int32_t BN, int64_t N, int32_t splits,
                                       int32_t kb_total, int32_t band_xblk, int32_t* out, int64_t cap) {
  using namespace ojb;
  if (n_xblk < 0 || tail_rows < 0 || n_xchunk < 1 || BN < 16 || BN > 256 || BN % 16 || N <= 0 || splits < 1 || kb_total < splits ||
      band_xblk < 0 || !out)
    return OJB_ERR_ARG;
  GemmArgs g{};
  g.n_xblk = n_xblk; g.tail_rows = tail_rows; g.n_xchunk = n_xchunk; g.BN = BN; g.N = static_cast<int>(N);
  g.n_wtile = static_cast<int>(ceil_div(N, BN)); g.n_wtile256 = static_cast<int>(ceil_div(N, 256));
  g.splits = splits; g.kb_total = kb_total; g.kb_per_split = static_cast<int>(ceil_div(kb_total, splits));
  g.band_xblk = band_xblk;
  const int64_t units = static_cast<int64_t>(n_xblk) * g.n_wtile * splits +
                        (tail_rows > 0 ? static_cast<int64_t>(g.n_wtile256) * splits * n_xchunk : 0);
  if (units > cap) return OJB_ERR_LIMIT;
  for (int64_t i = 0; i < units; ++i) {
    const Unit u = decode_unit(g, static_cast<int>(i), 0);
    out[5 * i + 0] = u.tail ? 1 : 0; out[5 * i + 1] = u.xb; out[5 * i + 2] = u.split; out[5 * i + 3] = u.wt; out[5 * i + 4] = u.xc;
  }
  return units;
}
