// C entry points of the bf16 GEMM and the choice between its kernels.
//
//   tile128   (gemm_tile128.cu)   128 x 256 (or 128 x 128) output tiles, two TMEM accumulators so that the epilogue of one
//             tile overlaps the MMAs of the next. M is padded to a multiple of 128.
//   block256  (gemm_block256.cu)  256 rows of x share each w tile between two MMAs (one third less shared-memory fill per
//             flop), w-tile width chosen per shape, the last M mod 256 <= 128 rows (or all rows when M <= 2048, on request) run with
//             swapped operands at their true cost.
//   pair256   (gemm_pair256.cu)   the same units on CTA pairs with tcgen05.mma.cta_group::2; measured on par with block256
//             (both are bound by shared-memory bandwidth), kept as variants 5 / 6.
// With variant 0 the kernel is the one with the smallest modelled time (plan_kernel): the models replay the round-robin
// deal of units to CTAs with per-unit costs taken from measured unit timelines.
#include "gemm_units.cuh"

using namespace ojb;

namespace {

// variant: 0 = automatic; 1 = tile128 with 128x256 tiles; 2 = tile128 with 128x128 tiles; a multiple of 16 in [16, 256] =
// block256 with that w-tile width; 3 = block256 with automatic width; 4 = block256 with every row of x in swapped-operand
// units (M <= 2048).
// 5 = pair256 (CTA pairs, cta_group::2) with automatic width; 6 = pair256 with every row of x in swapped-operand units
// (any M); 512 + a multiple of 16 in [16, 256] = pair256 with that w-tile width; 7 = block256 with the last 257..511 rows of x in
// two swapped-operand chunks and the rows before them in block units.
bool variant_ok(int v) {
  return (v >= 0 && v <= 7) || (v >= 16 && v <= 256 && v % 16 == 0) || (v >= 528 && v <= 768 && v % 16 == 0);
}

// Modelled SM clocks of the 128-row tile kernel: per k-block a CTA fills (128 + BN) rows and its MMAs read them once,
// 128 bytes per clock; the epilogue overlaps the next tile.
double tile128_clocks(int64_t M, int64_t N, int kb_total, int splits, int bn, int sms) {
  const int64_t units = ceil_div(M, 128) * ceil_div(N, bn) * splits;
  const int64_t grid = units < sms ? units : sms;
  const int per = static_cast<int>(ceil_div(kb_total, splits));
  const double kb = bn == 256 ? 900.0 : 600.0;   // fitted to back-to-back runs against the power cap (133 us at 288 rows, 206 us at 544 for gate/up)
  return static_cast<double>(ceil_div(units, grid)) * (per * kb + 1500.0) + 9000.0;
}

struct Plan {
  int variant;
  double clocks;
};

// Cheapest kernel for this shape and number of K ranges according to the cost models (gemm_units.cuh), never below the
// time HBM needs for the weight.
Plan plan_kernel(int epi, int64_t M, int64_t N, int64_t K, int splits) {
  const int sms = 148;
  const int kb_total = static_cast<int>(ceil_div(K, 64));
  Plan best{3, 1e30};
  auto consider = [&](int variant, double clocks) {
    if (clocks < best.clocks) best = Plan{variant, clocks};
  };
  consider(1, tile128_clocks(M, N, kb_total, splits, 256, sms));
  if (epi != kEpiSwiglu) consider(2, tile128_clocks(M, N, kb_total, splits, 128, sms));
  {  // block256: full blocks + swapped tail
    int n_xblk = static_cast<int>(M / 256), r = static_cast<int>(M % 256);
    if (r > 128) { n_xblk += 1; r = 0; }
    if (n_xblk > 0) {
      const int tail_box = (r + 15) / 16 * 16;
      const int bn = epi == kEpiSwiglu ? 256 : choose_bn(N, n_xblk, tail_box, 1, r > 0, splits, kb_total, sms, epi);
      consider(3, block_kernel_clocks(N, bn, n_xblk, tail_box, 1, r > 0, splits, kb_total, sms, epi));
    }
  }
  if (M <= 2048) {  // block256 with every row in swapped-operand units
    const int n_xchunk = static_cast<int>(ceil_div(M, 256));
    const int tail_box = static_cast<int>(ceil_div(ceil_div(M, n_xchunk), 16) * 16);
    consider(4, block_kernel_clocks(N, 256, 0, tail_box, n_xchunk, true, splits, kb_total, sms, epi));
  }
  const double hbm = (static_cast<double>(N) * K * 2.0) / 3500.0 + 7000.0;     // bytes per clock at 6.3 TB/s and 1.8 GHz
  if (best.clocks < hbm) best.clocks = hbm;
  return best;
}

int dispatch(int epi, int variant, const void* x, const void* w, void* out, int64_t M, int64_t N, int64_t K, int splits,
             int64_t ldo, int32_t* status, cudaStream_t st) {
  if (variant == 0) variant = plan_kernel(epi, M, N, K, splits).variant;
  if (variant == 5 || variant == 6 || variant >= 512)
    return gemm_pair256_launch(epi, variant == 5 ? 0 : (variant == 6 ? -1 : variant - 512), x, w, out, M, N, K, splits, ldo, status, st);
  if (variant == 1 || variant == 2)
    return gemm_tile128_launch(epi, variant == 1 ? 256 : 128, x, w, out, M, N, K, splits, ldo, status, st);
  return gemm_block256_launch(epi, variant == 3 ? 0 : (variant == 4 ? -1 : (variant == 7 ? -2 : variant)), x, w, out, M, N, K, splits, ldo, status, st);
}

}  // namespace

extern "C" int ojb_gemm_bf16(const void* x, const void* w, void* out, int64_t M, int64_t N, int64_t K, int variant,
                             int32_t* status, ojb_stream_t stream) {
  OJB_REQUIRE(x && w && out && M > 0 && N > 0 && K > 0 && K % 8 == 0 && variant_ok(variant));
  OJB_REQUIRE(aligned16(x) && aligned16(w) && aligned16(out));
  return dispatch(kEpiBf16, variant, x, w, out, M, N, K, 1, N, status, static_cast<cudaStream_t>(stream));
}

extern "C" int ojb_gemm_bf16_swiglu_v(const void* x, const void* w_blk, void* out, int64_t M, int64_t N, int64_t K, int variant,
                                      int32_t* status, ojb_stream_t stream) {
  OJB_REQUIRE(x && w_blk && out && M > 0 && N > 0 && K > 0 && K % 8 == 0 && N % 256 == 0);
  OJB_REQUIRE(aligned16(x) && aligned16(w_blk) && aligned16(out) && (variant == 0 || variant == 1 || variant == 3 || variant == 4 || variant == 5 || variant == 6 || variant == 7));
  return dispatch(kEpiSwiglu, variant, x, w_blk, out, M, N, K, 1, N / 2, status, static_cast<cudaStream_t>(stream));
}

extern "C" int ojb_gemm_bf16_swiglu(const void* x, const void* w_blk, void* out, int64_t M, int64_t N, int64_t K,
                                    int32_t* status, ojb_stream_t stream) {
  return ojb_gemm_bf16_swiglu_v(x, w_blk, out, M, N, K, 0, status, stream);
}

extern "C" int ojb_gemm_bf16_splitk(const void* x, const void* w, float* parts, int64_t M, int64_t N, int64_t K,
                                    int splits, int variant, int32_t* status, ojb_stream_t stream) {
  OJB_REQUIRE(x && w && parts && M > 0 && N > 0 && K > 0 && K % 8 == 0 && splits >= 1 && splits <= 16 && variant_ok(variant));
  OJB_REQUIRE(aligned16(x) && aligned16(w) && aligned16(parts));
  return dispatch(kEpiPartialF32, variant, x, w, parts, M, N, K, splits, N, status, static_cast<cudaStream_t>(stream));
}

namespace ojb {
namespace { int g_wait_ms = kDefaultWaitMs, g_drop_copy = 0; }
int gemm_wait_limit_ms() { return g_wait_ms; }
int gemm_drop_copy() { return g_drop_copy; }
}  // namespace ojb

extern "C" int ojb_gemm_set_wait_limit_ms(int32_t ms) {
  OJB_REQUIRE(ms >= 0 && ms <= 60000);
  ojb::g_wait_ms = ms == 0 ? ojb::kDefaultWaitMs : ms;
  return OJB_OK;
}

extern "C" int ojb_gemm_test_drop_copy(int32_t on) {
  ojb::g_drop_copy = on ? 1 : 0;
  return OJB_OK;
}

extern "C" int ojb_gemm_set_trace(uint64_t* records, int32_t capacity) {
  OJB_REQUIRE(capacity >= 0);
  gemm_block256_set_trace(reinterpret_cast<unsigned long long*>(records), capacity);
  gemm_pair256_set_trace(reinterpret_cast<unsigned long long*>(records), capacity);
  return OJB_OK;
}

#ifdef OJB_GEMM_PROBES
// Probe builds only (not declared in the public header): MMA repeat count and pipeline / epilogue knobs.
extern "C" int ojb_gemm_set_probe(int32_t mma_repeat, int32_t knob) {
  OJB_REQUIRE(mma_repeat >= 0 && mma_repeat <= 64 && (knob == 0 || (knob >= 2 && knob <= 12) || knob == 100 || knob == 101 || knob == 102));
  gemm_block256_set_probe(mma_repeat, knob);
  gemm_pair256_set_probe(mma_repeat, knob);
  return OJB_OK;
}
#endif

extern "C" int ojb_gemm_plan(int64_t M, int64_t N, int64_t K, int32_t kind, int32_t max_splits, int32_t* variant, int32_t* splits,
                             float* microseconds) {
  OJB_REQUIRE(M > 0 && N > 0 && K > 0 && kind >= 0 && kind <= 2 && max_splits >= 1 && max_splits <= 16 && variant && splits);
  const int kb_total = static_cast<int>(ceil_div(K, 64));
  Plan best{0, 1e30};
  int best_s = 1;
  for (int s = 1; s <= (kind == kEpiPartialF32 ? max_splits : 1); ++s) {
    const int per = static_cast<int>(ceil_div(kb_total, s));
    if (static_cast<int64_t>(s - 1) * per >= kb_total) continue;
    Plan p = plan_kernel(kind, M, N, K, s);
    // the kernel that sums the partial planes reads S * M * N floats (mostly from L2)
    if (kind == kEpiPartialF32) p.clocks += (s - 1) * static_cast<double>(M) * N * 4.0 / 5000.0;
    if (p.clocks < best.clocks * 0.97) { best = p; best_s = s; }
  }
  *variant = best.variant;
  *splits = best_s;
  if (microseconds) *microseconds = static_cast<float>(best.clocks / 1800.0);
  return OJB_OK;
}

extern "C" int ojb_gemm_e4m3(const void* xq, const float* sx, const void* wq, const float* sw, void* out, int64_t M, int64_t N,
                             int64_t K, int32_t kind, int32_t splits, int32_t* status, ojb_stream_t stream) {
  if (M == 0 || N == 0) return OJB_OK;
  OJB_REQUIRE(xq && sx && wq && sw && out && M > 0 && N > 0 && K > 0 && K % 16 == 0 && kind >= 0 && kind <= 2);
  OJB_REQUIRE(aligned16(xq) && aligned16(wq) && aligned16(out));
  OJB_REQUIRE(kind == 2 ? (splits >= 1 && splits <= 16) : splits == 1);
  OJB_REQUIRE(kind != 1 || N % 256 == 0);
  const int epi = kind == 0 ? kEpiBf16 : (kind == 1 ? kEpiSwiglu : kEpiPartialF32);
  return gemm_block256_launch_e4m3(epi, xq, sx, wq, sw, out, M, N, K, splits, kind == 1 ? N / 2 : N, status,
                                   static_cast<cudaStream_t>(stream));
}
