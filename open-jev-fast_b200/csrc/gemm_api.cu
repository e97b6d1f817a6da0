// C entry points of the bf16 GEMM and the choice between its two kernels.
//
//   tile128   (gemm_tile128.cu)   128 x 256 (or 128 x 128) output tiles, two TMEM accumulators so that the epilogue of one
//             tile overlaps the MMAs of the next. M is padded to a multiple of 128.
//   block256  (gemm_block256.cu)  256 rows of x share each w tile between two MMAs (one third less L2 -> shared-memory
//             traffic per flop: 0.81-0.86 of the measured bf16 peak at M = 512 / 1024 against 0.65 for tile128), w-tile
//             width chosen per shape, and the last M mod 256 <= 128 rows run with swapped operands at their true cost.
// Measured on B200 (python -m ojb200.gemm_sweep): block256 wins when M is a multiple of 256 (or leaves a remainder above
// 128, which it pads into one more block) and when M <= 128 (pure swapped-operand GEMM); when a short tail comes on top of
// full blocks (M = 288, 544) the tail units stream the whole weight once more from L2 and the two kernels tie on the
// gate/up shape while tile128 is ahead on the narrower projections, so tile128 serves those.
#include "gemm_common.cuh"

using namespace ojb;

namespace {

// variant: 0 = automatic; 1 = tile128 with 128x256 tiles; 2 = tile128 with 128x128 tiles; a multiple of 16 in [16, 256] =
// block256 with that w-tile width; 3 = block256 with automatic width; 4 = block256 with every row of x in swapped-operand
// units (M <= 512).
bool variant_ok(int v) { return (v >= 0 && v <= 4) || (v >= 16 && v <= 256 && v % 16 == 0); }

int dispatch(int epi, int variant, const void* x, const void* w, void* out, int64_t M, int64_t N, int64_t K, int splits,
             int64_t ldo, int32_t* status, cudaStream_t st) {
  if (variant == 0) {
    const int sms = 148;
    const int64_t r = M % 256;
    const int64_t tiles256 = ceil_div(M, 128) * ceil_div(N, 256) * splits;     // tile128 work units with 128 x 256 tiles
    if (M <= 128) {
      // few rows: every kernel streams the weight once; what matters is how many CTAs pull on HBM at the same time
      variant = ceil_div(N, 256) * splits >= 100 ? 4 : 2;
    } else if (M <= 512 && r != 0) {
      // one or two swapped-operand chunks cost exactly M rows; tile128 pads to 128 and wins only while its tiles fit one wave
      variant = (tiles256 <= sms && tiles256 >= 100) ? 1 : (tiles256 < 100 && splits == 1 ? 2 : 4);
    } else if (M > 512 && r > 0 && r <= 128 && N < 16384) {
      variant = tiles256 >= 100 ? 1 : 2;
    } else {
      variant = 3;
    }
  }
  if (variant == 1 || variant == 2)
    return gemm_tile128_launch(epi, variant == 1 ? 256 : 128, x, w, out, M, N, K, splits, ldo, status, st);
  return gemm_block256_launch(epi, variant == 3 ? 0 : (variant == 4 ? -1 : variant), x, w, out, M, N, K, splits, ldo, status, st);
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
  OJB_REQUIRE(aligned16(x) && aligned16(w_blk) && aligned16(out) && (variant == 0 || variant == 1 || variant == 3 || variant == 4));
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

extern "C" int ojb_gemm_set_trace(uint64_t* records, int32_t capacity, int32_t mma_repeat, int32_t stage_cols) {
  OJB_REQUIRE(capacity >= 0 && mma_repeat >= 1 && mma_repeat <= 64 && (stage_cols == 0 || stage_cols == 32 || stage_cols == 64));
  gemm_block256_set_trace(reinterpret_cast<unsigned long long*>(records), capacity, mma_repeat, stage_cols);
  return OJB_OK;
}
