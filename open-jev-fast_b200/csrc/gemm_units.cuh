// Work decomposition shared by the block GEMM kernels (gemm_block256.cu: one CTA per unit; gemm_pair256.cu: one CTA pair
// per unit): block units of 256 rows of x times BN rows of w, swapped-operand tail units of 256 rows of w times up to 256
// rows of x, optional K ranges, and the order in which the units are dealt out.
#pragma once
#include "gemm_common.cuh"

namespace ojb {
namespace {

constexpr int kBlockM = 256;       // rows of x per block unit

struct GemmArgs {
  int M, N, K;
  int BN;          // rows of w per block unit: multiple of 16, <= 256
  int n_xblk;      // 256-row blocks of x served by block units
  int tail_rows;   // rows of x served by tail units, starting at row n_xblk * 256 (0 = none)
  int tail_box;    // rows of x per tail unit: multiple of 16, <= 256 = UMMA N of the tail units
  int n_xchunk;    // tail units per w tile and k-split: the tail rows are cut into n_xchunk chunks of tail_box rows
  int n_wtile;     // ceil(N / BN)
  int n_wtile256;  // ceil(N / 256)
  int splits, kb_per_split, kb_total;   // in k-blocks of bk columns
  int bk;                // columns of x and w per shared-memory stage: 64 (128-byte swizzle) or 32 (64-byte swizzle)
  int stages;
  uint32_t stage_bytes;
  uint32_t a_bytes;      // 256 rows x bk columns: the x rows of a block unit or the w rows of a tail unit
  void* out;
  int64_t ldo;           // leading dimension of out in elements
  int64_t split_stride;  // elements between split planes (fp32 partials)
  int32_t* status;
  unsigned long long* trace;   // null, or [0] = record counter followed by records of 4 words (see ojb_gemm_set_trace)
  int trace_cap;
  int mma_repeat;              // 1; > 1 only for measurements: every stage's MMAs are issued this many times
};

struct Unit {
  bool tail;
  int xb, split, wt, kb0, kb1;
  int xc;   // x chunk of a tail unit
};

// Units are ordered by the w rows they read: w tile j contributes its block units (x-block fastest, then k-split) followed
// by the tail units that start inside it, so a tail unit finds its w rows in L2 instead of streaming them from HBM again.
// group_begin(j) = position of the first unit of tile j; tails_before(j) = tail tiles (256 w rows each) that start before
// row j * BN.
__device__ __forceinline__ int tails_before(const GemmArgs& g, int j) {
  if (g.tail_rows == 0) return 0;
  const int t = (j * g.BN + 255) / 256;
  return t < g.n_wtile256 ? t : g.n_wtile256;
}
__device__ __forceinline__ int group_begin(const GemmArgs& g, int j) {
  return (j * g.n_xblk + tails_before(g, j) * g.n_xchunk) * g.splits;
}

__device__ __forceinline__ Unit decode_unit(const GemmArgs& g, int unit, int total_block) {
  (void)total_block;
  Unit u;
  const int nb = g.n_xblk * g.splits;
  int j = static_cast<int>(unit / (nb + g.splits * g.n_xchunk * (g.tail_rows > 0 ? g.BN / 256.0f : 0.0f) + 1e-6f));
  if (j > g.n_wtile - 1) j = g.n_wtile - 1;
  while (j > 0 && group_begin(g, j) > unit) --j;
  while (j + 1 < g.n_wtile && group_begin(g, j + 1) <= unit) ++j;
  const int off = unit - group_begin(g, j);
  u.tail = off >= nb;
  if (!u.tail) {
    u.xb = off % g.n_xblk;
    u.split = off / g.n_xblk;
    u.wt = j;
    u.xc = 0;
  } else {
    const int o2 = off - nb;
    u.xb = g.n_xblk;
    u.xc = o2 % g.n_xchunk;                       // x chunk fastest: the chunks of one w tile run side by side
    u.split = (o2 / g.n_xchunk) % g.splits;
    u.wt = tails_before(g, j) + o2 / (g.n_xchunk * g.splits);
  }
  u.kb0 = u.split * g.kb_per_split;
  u.kb1 = min(u.kb0 + g.kb_per_split, g.kb_total);
  return u;
}

// Width of the w tile of the block units: the multiple of 16 that needs the fewest waves of CTAs, wider tiles preferred
// (they pull less from L2 per flop); tail units are short and fill the gaps.
inline int choose_bn(int64_t N, int n_xblk, int splits, int sms) {
  if (n_xblk == 0) return 256;
  int best = 256;
  double best_cost = 1e30;
  for (int bn = 256; bn >= 64; bn -= 16) {
    const int64_t units = ceil_div(N, bn) * n_xblk * splits;
    const int64_t waves = ceil_div(units, sms);
    const double cost = static_cast<double>(waves) * bn * (1.0 + 0.15 * (256 - bn) / 256.0);
    if (cost < best_cost - 1e-9) { best_cost = cost; best = bn; }
  }
  return best;
}

}  // namespace
}  // namespace ojb
