// Work decomposition shared by the block GEMM kernels (gemm_block256.cu: one CTA per unit; gemm_pair256.cu: one CTA pair
// per unit): block units of 256 rows of x times BN rows of w, swapped-operand tail units of 256 rows of w times up to 256
// rows of x, optional K ranges, and the order in which the units are dealt out.
#pragma once
// Probe builds (-DOJB_GEMM_PROBES, never the shipped library) can repeat the MMAs of a stage, cap the pipeline depth and
// skip parts of the epilogue to separate tensor-pipe, copy and store costs; in the shipped build these read as constants
// and the code behind them is compiled out.
#ifdef OJB_GEMM_PROBES
#define OJB_PROBE_REPEAT(g) ((g).mma_repeat)
#define OJB_PROBE_DBG(g) ((g).dbg)
#else
#define OJB_PROBE_REPEAT(g) 1
#define OJB_PROBE_DBG(g) 0
#endif
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
  int splits, kb_per_split, kb_total;   // in k-blocks of 64 columns
  int stages;
  uint32_t stage_bytes;
  void* out;
  int64_t ldo;           // leading dimension of out in elements
  int64_t split_stride;  // elements between split planes (fp32 partials)
  int32_t* status;
  int wait_ms;                 // limit of every mbarrier wait of the kernel, milliseconds
  unsigned long long* trace;   // null, or [0] = record counter followed by records of 4 words (see ojb_gemm_set_trace)
  int trace_cap;
  int tail_sub;                // bytes of a tail sub-stage (128 rows of w + the x rows), 0 = one k-block per stage
  int tma_out;                 // the block epilogue stores through shared-memory tiles and bulk tensor stores
  int dbg;                     // probe builds only (see below); 0 otherwise
  int mma_repeat;              // probe builds only; 1 otherwise
  // CTA-pair kernel, swapped-operand units: the tail_box accumulator columns (= rows of x) of a unit are produced by
  // n_chunk MMAs per k-step of chunk_w columns each (the last one narrower), so one pass over 256 rows of w serves up to
  // 512 rows of x; w_split64: the 128 rows of w of a CTA are fetched as rows [64r, 64r+64) and [128+64r, 128+64r+64) of the
  // tile (gate and up rows of the same 64 outputs of a SwiGLU weight interleaved in blocks of 128 rows).
  int n_chunk, chunk_w, w_split64;
  // e4m3 operands (block kernel): fp32 scale per row of x and per row of w, applied to the accumulator in the epilogue
  const float* sx;
  const float* sw;
  int tail_tma;                // block kernel: swapped-operand units store through [16][32] shared-memory tiles and bulk tensor stores
  int band_xblk;               // 0, or the x blocks of a band: all units of a band come before those of the next (see decode_unit)
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
// When x is larger than the L2 keeps (tens of thousands of rows), that order would stream all of x from HBM once per w tile:
// the x blocks are then cut into bands of band_xblk blocks, each band small enough to stay in L2, and the whole order above
// runs band after band (w is streamed once per band instead); the tail units belong to the last band.
__host__ __device__ __forceinline__ int tails_before(const GemmArgs& g, int j, bool tails) {
  if (!tails) return 0;
  const int t = (j * g.BN + 255) / 256;
  return t < g.n_wtile256 ? t : g.n_wtile256;
}
__host__ __device__ __forceinline__ int group_begin(const GemmArgs& g, int j, int nx, bool tails) {
  return (j * nx + tails_before(g, j, tails) * g.n_xchunk) * g.splits;
}

// (also compiled for the host: ojb_gemm_unit_order lists the order for the tests)
__host__ __device__ __forceinline__ Unit decode_unit(const GemmArgs& g, int unit, int total_block) {
  (void)total_block;
  Unit u;
  int xb_base = 0, nx = g.n_xblk;
  bool tails = g.tail_rows > 0;
  if (g.band_xblk > 0) {
    const int full = g.band_xblk * g.n_wtile * g.splits;          // units of a band that is not the last one
    const int n_bands = (g.n_xblk + g.band_xblk - 1) / g.band_xblk;
    int b = unit / full;
    if (b > n_bands - 1) b = n_bands - 1;
    unit -= b * full;
    xb_base = b * g.band_xblk;
    nx = g.band_xblk < g.n_xblk - xb_base ? g.band_xblk : g.n_xblk - xb_base;
    tails = tails && b == n_bands - 1;
  }
  const int nb = nx * g.splits;
  int j = static_cast<int>(unit / (nb + g.splits * g.n_xchunk * (tails ? g.BN / 256.0f : 0.0f) + 1e-6f));
  if (j > g.n_wtile - 1) j = g.n_wtile - 1;
  while (j > 0 && group_begin(g, j, nx, tails) > unit) --j;
  while (j + 1 < g.n_wtile && group_begin(g, j + 1, nx, tails) <= unit) ++j;
  const int off = unit - group_begin(g, j, nx, tails);
  u.tail = off >= nb;
  if (!u.tail) {
    u.xb = xb_base + off % nx;
    u.split = off / nx;
    u.wt = j;
    u.xc = 0;
  } else {
    const int o2 = off - nb;
    u.xb = g.n_xblk;
    u.xc = o2 % g.n_xchunk;                       // x chunk fastest: the chunks of one w tile run side by side
    u.split = (o2 / g.n_xchunk) % g.splits;
    u.wt = tails_before(g, j, tails) + o2 / (g.n_xchunk * g.splits);
  }
  u.kb0 = u.split * g.kb_per_split;
  u.kb1 = u.kb0 + g.kb_per_split < g.kb_total ? u.kb0 + g.kb_per_split : g.kb_total;
  return u;
}

// ---- Cost model (host). Times are SM clocks; the constants come from unit timelines measured on B200 (ojb_gemm_set_trace):
// the main loops are bound by shared-memory bandwidth (128 bytes per clock per SM shared between the TMA fill of a stage
// and the operand reads of its MMAs), an MMA with M = 128 never takes less than 64 clocks, a swapped-operand unit keeps
// too few bytes in flight to run faster than about 1200 clocks per k-block, and the epilogue of a block unit costs about 19
// (bf16), 33 (fp32) or 40 (SwiGLU) clocks per accumulator column.
struct UnitCost {
  double block_kb, block_epi, tail_kb, tail_epi;
};
inline UnitCost unit_cost(int bn, int tail_box, int epi) {
  UnitCost c;
  const double smem = 512.0 + 3.0 * bn, mma = 4.0 * bn;
  c.block_kb = smem > mma ? smem : mma;
  c.block_epi = 900.0 + bn * (epi == kEpiPartialF32 ? 33.0 : (epi == kEpiSwiglu ? 40.0 : 19.0));
  const double tsm = 512.0 + 3.0 * tail_box;
  c.tail_kb = tsm > 1200.0 ? tsm : 1200.0;
  c.tail_epi = 3200.0 + 24.0 * tail_box;
  return c;
}

// Longest per-worker sum when the units of the block kernels (order of decode_unit) are dealt round-robin to `workers`
// CTAs (or CTA pairs). n_xblk == 0: swapped-operand units only.
inline double block_kernel_clocks(int64_t N, int bn, int n_xblk, int tail_box, int n_xchunk, bool has_tail, int splits,
                                  int kb_total, int workers, int epi, int* grid_out = nullptr) {
  const int n_wtile = n_xblk > 0 ? static_cast<int>(ceil_div(N, bn)) : static_cast<int>(ceil_div(N, 256));
  const int n_wtile256 = static_cast<int>(ceil_div(N, 256));
  const int per = static_cast<int>(ceil_div(kb_total, splits));
  const UnitCost c = unit_cost(bn, tail_box, epi);
  const int64_t units = static_cast<int64_t>(n_xblk) * n_wtile * splits + (has_tail ? static_cast<int64_t>(n_wtile256) * splits * n_xchunk : 0);
  int grid = static_cast<int>(units < workers ? units : workers);
  if (units > grid && has_tail && n_xblk > 0) {
    const int group = (n_xblk + n_xchunk) * splits;
    auto gcd = [](int a, int b) { while (b) { const int t = a % b; a = b; b = t; } return a; };
    while (grid > 1 && gcd(grid, group) != 1) --grid;
  }
  if (grid_out) *grid_out = grid;
  if (grid <= 0) return 0.0;
  double load[160] = {0.0};
  if (grid > 160) return 1e30;
  int64_t i = 0;
  auto kbs = [&](int s) { const int k1 = (s + 1) * per < kb_total ? (s + 1) * per : kb_total; return k1 - s * per; };
  auto tails_before = [&](int j) {
    if (!has_tail) return 0;
    const int t = n_xblk > 0 ? (j * bn + 255) / 256 : j;
    return t < n_wtile256 ? t : n_wtile256;
  };
  for (int j = 0; j < n_wtile; ++j) {
    for (int s = 0; s < splits; ++s)
      for (int xb = 0; xb < n_xblk; ++xb) load[i++ % grid] += kbs(s) * c.block_kb + c.block_epi;
    const int nt = (j + 1 < n_wtile ? tails_before(j + 1) : (has_tail ? n_wtile256 : 0)) - tails_before(j);
    for (int t = 0; t < nt; ++t)
      for (int s = 0; s < splits; ++s)
        for (int xc = 0; xc < n_xchunk; ++xc) load[i++ % grid] += kbs(s) * c.tail_kb + c.tail_epi;
  }
  double worst = 0.0;
  for (int k = 0; k < grid; ++k) worst = load[k] > worst ? load[k] : worst;
  return worst + 5000.0;      // launch, TMEM allocation, first stages
}

// Width of the w tile of the block units: the multiple of 16 with the smallest modelled time, wider tiles preferred.
inline int choose_bn(int64_t N, int n_xblk, int tail_box, int n_xchunk, bool has_tail, int splits, int kb_total, int workers,
                     int epi) {
  if (n_xblk == 0) return 256;
  int best = 256;
  double best_cost = 1e30;
  for (int bn = 256; bn >= 64; bn -= 16) {
    const double cost = block_kernel_clocks(N, bn, n_xblk, tail_box, n_xchunk, has_tail, splits, kb_total, workers, epi);
    if (cost < best_cost * 0.98) { best_cost = cost; best = bn; }
  }
  return best;
}

}  // namespace
}  // namespace ojb
