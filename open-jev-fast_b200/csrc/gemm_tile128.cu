// bf16 GEMM, 128-row tile kernel (one of two kernels behind ojb_gemm_bf16*; the other is gemm_block256.cu), sm_100a:
//   out[M,N] = x[M,K] · w[N,K]^T, both operands K-major, fp32 accumulation in tensor memory (TMEM).
//
// One persistent CTA per SM, 192 threads, three roles:
//   warp 0      TMA producer  — cp.async.bulk.tensor (plain, non-multicast) of a 128xBK x-tile and a BNxBK w-tile per stage,
//                               128-byte swizzle, completion on an mbarrier
//   warp 1      MMA issuer    — one lane issues tcgen05.mma (M=128, N=BN, K=16) x4 per stage into one of two TMEM
//                               accumulators; tcgen05.commit releases the stage / publishes the accumulator
//   warps 2..5  epilogue      — tcgen05.ld of their 32-lane quarter, conversion and global stores, while the MMA warp is
//                               already filling the other accumulator
// Work units are (m-block, k-split, n-block) with the m-block varying fastest, so that the CTAs running at the same time
// share one w-tile column (read once from HBM, then from L2) while x (a few MB) stays L2-resident.
//
// Every wait on an mbarrier is bounded: after the wait limit (2 s unless ojb_gemm_set_wait_limit_ms changed it) the kernel raises the CTA's abort flag, records
// OJB_DEV_WAIT_TIMEOUT in the status word, lets copies in flight land, frees its TMEM and returns.
#include "gemm_common.cuh"

namespace ojb {
namespace {

constexpr int kGemmThreads = 192;

struct GemmArgs {
  int M, N, K;
  int num_m, num_n, splits, kb_per_split, kb_total;
  void* out;
  int64_t ldo;          // leading dimension of out in elements
  int64_t split_stride; // elements between consecutive split planes (fp32 partials)
  int32_t* status;
  int wait_ms;          // limit of every mbarrier wait, milliseconds
  int drop_copy;        // failure injection of the tests: the producer leaves out the copies of the second k-block it handles
};

template <int BN, int STAGES>
struct SmemPlan {
  static constexpr uint32_t kABytes = kBM * kBK * 2;
  static constexpr uint32_t kBBytes = BN * kBK * 2;
  static constexpr uint32_t kStageBytes = kABytes + kBBytes;
  static constexpr uint32_t kTileBytes = STAGES * kStageBytes;
  static constexpr uint32_t kBarBytes = (2 * STAGES + 4) * 8 + 16;
  static constexpr uint32_t kTotal = kTileBytes + kBarBytes + 1024;  // + slack for the 1024-byte alignment
};

template <int BN, int STAGES, int EPI>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tile128_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, GemmArgs g) {
  pdl_launch_dependents();
  using Plan = SmemPlan<BN, STAGES>;
  constexpr uint32_t kTmemCols = 2 * BN;  // two accumulators of BN fp32 columns (256 or 512: both powers of two)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Plan::kTileBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const uint32_t tiles0 = smem_u32(smem);
  const uint32_t full0 = smem_u32(bars);
  const uint32_t empty0 = full0 + 8 * STAGES;
  const uint32_t accfull0 = empty0 + 8 * STAGES;
  const uint32_t accempty0 = accfull0 + 16;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(accfull0 + 8 * a, 1);
      mbar_init(accempty0 + 8 * a, 4);
    }
    abort_flag[0] = 0;
    abort_flag[1] = g.wait_ms;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
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

  const int total_units = g.num_m * g.num_n * g.splits;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0, issued = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
        const int m_blk = unit % g.num_m;
        const int rest = unit / g.num_m;
        const int split = rest % g.splits, n_blk = rest / g.splits;
        const int kb0 = split * g.kb_per_split;
        const int kb1 = min(kb0 + g.kb_per_split, g.kb_total);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(empty0 + 8 * stage, phase ^ 1u, abort_flag)) { ok = false; break; }
          const uint32_t a_dst = tiles0 + stage * Plan::kStageBytes;
          const uint32_t fb = full0 + 8 * stage;
          mbar_expect_tx(fb, Plan::kStageBytes);
          if (g.drop_copy && issued++ == 1) {
            // tests only (ojb_gemm_test_drop_copy): the bytes announced for this stage never arrive, the consumer's bounded
            // wait on its barrier runs out, the CTA reports OJB_DEV_WAIT_TIMEOUT and leaves in order
          } else {
            tma_load_2d(a_dst, &map_x, fb, kb * kBK, m_blk * kBM);
            tma_load_2d(a_dst + Plan::kABytes, &map_w, fb, kb * kBK, n_blk * BN);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(BN);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
        const int rest = unit / g.num_m;
        const int split = rest % g.splits;
        const int kb0 = split * g.kb_per_split;
        const int kb1 = min(kb0 + g.kb_per_split, g.kb_total);
        if (!mbar_wait(accempty0 + 8 * acc, acc_phase ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(full0 + 8 * stage, phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = tiles0 + stage * Plan::kStageBytes;
          const uint64_t adesc = smem_desc_sw128(a_addr);
          const uint64_t bdesc = smem_desc_sw128(a_addr + Plan::kABytes);
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            // advancing K by 16 bf16 = 32 bytes inside the swizzle row: +2 in the (address >> 4) field
            umma_bf16(tmem_d, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(empty0 + 8 * stage);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit(accfull0 + 8 * acc);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) are the ones this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int unit = blockIdx.x; unit < total_units && ok; unit += gridDim.x) {
      const int m_blk = unit % g.num_m;
      const int rest = unit / g.num_m;
      const int split = rest % g.splits, n_blk = rest / g.splits;
      if (!mbar_wait(accfull0 + 8 * acc, acc_phase, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int row = m_blk * kBM + quarter * 32 + lane;
      const bool row_ok = row < g.M;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * BN);
      if constexpr (EPI == kEpiSwiglu) {
        // columns [0,128) of the tile are gate_j, columns [128,256) the matching up_j
        static_assert(EPI != kEpiSwiglu || BN == 256, "SwiGLU epilogue needs the 256-wide tile");
        bf16_t* orow = reinterpret_cast<bf16_t*>(g.out) + static_cast<int64_t>(row) * g.ldo + static_cast<int64_t>(n_blk) * 128;
        const int ncols = g.N / 2 - n_blk * 128;  // valid output columns of this tile
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t gr[32], ur[32];
          tmem_ld32(taddr + c * 32, gr);
          tmem_ld32(taddr + 128 + c * 32, ur);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (c * 32 + j < ncols) {
                float o[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                  const float gv = __uint_as_float(gr[j + e]);
                  const float uv = __uint_as_float(ur[j + e]);
                  o[e] = silu_f(gv) * uv;
                }
                *reinterpret_cast<uint4*>(orow + c * 32 + j) = pack8(o);
              }
            }
          }
        }
      } else if constexpr (EPI == kEpiBf16) {
        bf16_t* orow = reinterpret_cast<bf16_t*>(g.out) + static_cast<int64_t>(row) * g.ldo + static_cast<int64_t>(n_blk) * BN;
        const int ncols = g.N - n_blk * BN;
        const bool vec_ok = (g.ldo % 8) == 0;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(taddr + c * 32, r);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              const int col = c * 32 + j;
              if (col + 8 <= ncols && vec_ok) {
                float o[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) o[e] = __uint_as_float(r[j + e]);
                *reinterpret_cast<uint4*>(orow + col) = pack8(o);
              } else {
#pragma unroll
                for (int e = 0; e < 8; ++e)
                  if (col + e < ncols) orow[col + e] = f2bf(__uint_as_float(r[j + e]));
              }
            }
          }
        }
      } else {
        float* orow = reinterpret_cast<float*>(g.out) + static_cast<int64_t>(split) * g.split_stride +
                      static_cast<int64_t>(row) * g.ldo + static_cast<int64_t>(n_blk) * BN;
        const int ncols = g.N - n_blk * BN;
        const bool vec_ok = (g.ldo % 4) == 0;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(taddr + c * 32, r);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              const int col = c * 32 + j;
              if (col + 4 <= ncols && vec_ok) {
                *reinterpret_cast<uint4*>(orow + col) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
              } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                  if (col + e < ncols) orow[col + e] = __uint_as_float(r[j + e]);
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(accempty0 + 8 * acc);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
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

template <int BN, int STAGES, int EPI>
int launch_gemm(const void* x, const void* w, void* out, int64_t M, int64_t N, int64_t K, int splits, int64_t ldo,
                int32_t* status, cudaStream_t stream) {
  using Plan = SmemPlan<BN, STAGES>;
  static int smem_set[kMaxDevices] = {};
  auto kern = gemm_tile128_kernel<BN, STAGES, EPI>;
  if (!raise_smem_limit(kern, static_cast<int>(Plan::kTotal), smem_set)) return OJB_ERR_LAUNCH;
  CUtensorMap map_x, map_w;
  int rc = make_map(&map_x, x, M, K, kBM);
  if (rc != OJB_OK) return rc;
  rc = make_map(&map_w, w, N, K, BN);
  if (rc != OJB_OK) return rc;
  GemmArgs g{};
  g.wait_ms = gemm_wait_limit_ms();
  g.drop_copy = gemm_drop_copy();
  g.M = static_cast<int>(M);
  g.N = static_cast<int>(N);
  g.K = static_cast<int>(K);
  g.num_m = static_cast<int>(ceil_div(M, kBM));
  g.num_n = static_cast<int>(ceil_div(N, BN));
  g.splits = splits;
  g.kb_total = static_cast<int>(ceil_div(K, kBK));
  g.kb_per_split = static_cast<int>(ceil_div(g.kb_total, splits));
  g.out = out;
  g.ldo = ldo;
  g.split_stride = M * N;
  g.status = status;
  const int sms = sm_count();
  if (sms <= 0) return OJB_ERR_LAUNCH;
  const int64_t units = static_cast<int64_t>(g.num_m) * g.num_n * splits;
  const int grid = static_cast<int>(units < sms ? units : sms);
  launch_kernel(kern, dim3(grid), dim3(kGemmThreads), Plan::kTotal, stream, map_x, map_w, g);
  return launch_status(cudaGetLastError());
}

}  // namespace

int gemm_tile128_launch(int epi, int bn, const void* x, const void* w, void* out, int64_t M, int64_t N, int64_t K, int splits,
                        int64_t ldo, int32_t* status, cudaStream_t stream) {
  if (static_cast<int64_t>(splits - 1) * ceil_div(ceil_div(K, kBK), splits) >= ceil_div(K, kBK)) return OJB_ERR_ARG;  // empty split
  if (epi == kEpiSwiglu) return launch_gemm<256, 4, kEpiSwiglu>(x, w, out, M, N, K, 1, ldo, status, stream);
  if (epi == kEpiBf16)
    return bn == 128 ? launch_gemm<128, 6, kEpiBf16>(x, w, out, M, N, K, splits, ldo, status, stream)
                     : launch_gemm<256, 4, kEpiBf16>(x, w, out, M, N, K, splits, ldo, status, stream);
  return bn == 128 ? launch_gemm<128, 6, kEpiPartialF32>(x, w, out, M, N, K, splits, ldo, status, stream)
                   : launch_gemm<256, 4, kEpiPartialF32>(x, w, out, M, N, K, splits, ldo, status, stream);
}

}  // namespace ojb
