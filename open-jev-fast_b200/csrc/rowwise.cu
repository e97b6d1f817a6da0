// Row-wise and element-wise kernels of the scoring forward: residual add + RMSNorm (with or without split-K partial sums),
// SwiGLU product, activation tables, sigmoid gate product, visibility bit packing, attention q/k/v preparation.
// All of them are HBM-bound streaming kernels: 16-byte accesses, one pass over the data, rows held in registers.
#include "common.cuh"
#include <cuda_fp8.h>

namespace ojb {
namespace {

constexpr int kRowThreads = 256;
constexpr int kRowVecs = 4;  // 16-byte vectors per thread held in registers -> H <= 256 * 4 * 8 = 8192

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ float block_sum_256(float v, float* red) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = (lane < kRowThreads / 32) ? red[lane] : 0.f;
  t = warp_sum(t);
  return t;  // every warp reduces the same 8 partials in the same order -> identical value in all threads
}

// One CTA per row. SPLITS == 0: delta is an optional bf16 row; SPLITS > 0: delta = bf16(sum of SPLITS fp32 partial rows).
template <int SPLITS>
__global__ void __launch_bounds__(kRowThreads)
add_rmsnorm_kernel(const bf16_t* __restrict__ x, const bf16_t* __restrict__ delta, const float* __restrict__ parts,
                   int64_t part_stride, const float* __restrict__ w1, const int32_t* __restrict__ rowmask,
                   bf16_t* __restrict__ h_out, bf16_t* __restrict__ hn_out, int H, float eps) {
  pdl_begin();
  __shared__ float red[kRowThreads / 32];
  const int64_t row = blockIdx.x;
  const int nvec = H >> 3;
  float v[kRowVecs][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kRowVecs; ++i) {
    const int vi = threadIdx.x + i * kRowThreads;
    if (vi < nvec) {
      const int64_t off = row * H + static_cast<int64_t>(vi) * 8;
      unpack8(ldg_stream(x + off), v[i]);
      if constexpr (SPLITS > 0) {
        float d[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) d[e] = 0.f;
#pragma unroll
        for (int s = 0; s < SPLITS; ++s) {
          const float* pp = parts + s * part_stride + off;
          const uint4 a = ldg_stream(pp), b = ldg_stream(pp + 4);
          d[0] += __uint_as_float(a.x); d[1] += __uint_as_float(a.y); d[2] += __uint_as_float(a.z); d[3] += __uint_as_float(a.w);
          d[4] += __uint_as_float(b.x); d[5] += __uint_as_float(b.y); d[6] += __uint_as_float(b.z); d[7] += __uint_as_float(b.w);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) v[i][e] = round_bf(v[i][e] + round_bf(d[e]));
        *reinterpret_cast<uint4*>(h_out + off) = pack8(v[i]);
      } else if (delta != nullptr) {
        float d[8];
        unpack8(ldg_stream(delta + off), d);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[i][e] = round_bf(v[i][e] + d[e]);
        *reinterpret_cast<uint4*>(h_out + off) = pack8(v[i]);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += v[i][e] * v[i][e];
    }
  }
  ss = block_sum_256(ss, red);
  const float rstd = rsqrtf(ss / static_cast<float>(H) + eps);
  const bool keep = rowmask ? (rowmask[row] != 0) : true;
#pragma unroll
  for (int i = 0; i < kRowVecs; ++i) {
    const int vi = threadIdx.x + i * kRowThreads;
    if (vi < nvec) {
      const int col = vi * 8;
      const float4 wa = __ldg(reinterpret_cast<const float4*>(w1 + col));
      const float4 wb = __ldg(reinterpret_cast<const float4*>(w1 + col + 4));
      const float w[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = keep ? (v[i][e] * rstd) * w[e] : 0.f;
      *reinterpret_cast<uint4*>(hn_out + row * H + col) = pack8(o);
    }
  }
}

// Residual stream kept in fp32. One CTA per row: h = x_init (bf16, first norm of a forward) or h + delta, where delta is the
// sum of SPLITS fp32 partial rows (SPLITS > 0) or one bf16 row or nothing; the sum is added in fp32 and h is never rounded.
// hn = bf16(h * rstd * w1): the only rounding is the one the consuming GEMM needs for its operand.
template <int SPLITS>
__global__ void __launch_bounds__(kRowThreads)
resnorm_f32_kernel(float* __restrict__ h, const bf16_t* __restrict__ x_init, const bf16_t* __restrict__ delta,
                   const float* __restrict__ parts, int64_t part_stride, const float* __restrict__ w1,
                   const int32_t* __restrict__ rowmask, bf16_t* __restrict__ hn_out, int H, float eps) {
  pdl_begin();
  __shared__ float red[kRowThreads / 32];
  const int64_t row = blockIdx.x;
  const int nvec = H >> 3;
  float v[kRowVecs][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kRowVecs; ++i) {
    const int vi = threadIdx.x + i * kRowThreads;
    if (vi < nvec) {
      const int64_t off = row * H + static_cast<int64_t>(vi) * 8;
      if (x_init != nullptr) {
        unpack8(ldg_stream(x_init + off), v[i]);
      } else {
        const float4 a = *reinterpret_cast<const float4*>(h + off), b = *reinterpret_cast<const float4*>(h + off + 4);
        v[i][0] = a.x; v[i][1] = a.y; v[i][2] = a.z; v[i][3] = a.w;
        v[i][4] = b.x; v[i][5] = b.y; v[i][6] = b.z; v[i][7] = b.w;
      }
      if constexpr (SPLITS > 0) {
        float d[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) d[e] = 0.f;
#pragma unroll
        for (int s = 0; s < SPLITS; ++s) {
          const float* pp = parts + s * part_stride + off;
          const uint4 a = ldg_stream(pp), b = ldg_stream(pp + 4);
          d[0] += __uint_as_float(a.x); d[1] += __uint_as_float(a.y); d[2] += __uint_as_float(a.z); d[3] += __uint_as_float(a.w);
          d[4] += __uint_as_float(b.x); d[5] += __uint_as_float(b.y); d[6] += __uint_as_float(b.z); d[7] += __uint_as_float(b.w);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) v[i][e] += d[e];
      } else if (delta != nullptr) {
        float d[8];
        unpack8(ldg_stream(delta + off), d);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[i][e] += d[e];
      }
      if (x_init != nullptr || SPLITS > 0 || delta != nullptr) {
        *reinterpret_cast<float4*>(h + off) = make_float4(v[i][0], v[i][1], v[i][2], v[i][3]);
        *reinterpret_cast<float4*>(h + off + 4) = make_float4(v[i][4], v[i][5], v[i][6], v[i][7]);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += v[i][e] * v[i][e];
    }
  }
  ss = block_sum_256(ss, red);
  const float rstd = rsqrtf(ss / static_cast<float>(H) + eps);
  const bool keep = rowmask ? (rowmask[row] != 0) : true;
#pragma unroll
  for (int i = 0; i < kRowVecs; ++i) {
    const int vi = threadIdx.x + i * kRowThreads;
    if (vi < nvec) {
      const int col = vi * 8;
      const float4 wa = __ldg(reinterpret_cast<const float4*>(w1 + col));
      const float4 wb = __ldg(reinterpret_cast<const float4*>(w1 + col + 4));
      const float w[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = keep ? (v[i][e] * rstd) * w[e] : 0.f;
      *reinterpret_cast<uint4*>(hn_out + row * H + col) = pack8(o);
    }
  }
}

__global__ void act_tables_kernel(bf16_t* __restrict__ silu_tab, float* __restrict__ sig_tab) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= 65536u) return;
  const float x = __uint_as_float(i << 16);  // bf16 bit pattern widened to fp32
  silu_tab[i] = f2bf(silu_f(x));
  sig_tab[i] = sigmoid_f(x);
}

// 8 outputs per thread; gate at column c, up at column I + c of the same row.
__global__ void __launch_bounds__(256)
silu_mul_kernel(const bf16_t* __restrict__ gu, const bf16_t* __restrict__ tab, bf16_t* __restrict__ out, int I, int64_t nvec) {
  pdl_begin();
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= nvec) return;
  const int vec_per_row = I >> 3;
  const int64_t row = i / vec_per_row;
  const int col = static_cast<int>(i - row * vec_per_row) * 8;
  const bf16_t* gp = gu + row * 2 * I + col;
  const uint4 gv = ldg_stream(gp), uv = ldg_stream(gp + I);
  float u[8], o[8];
  unpack8(uv, u);
  if (tab != nullptr) {
    const uint16_t* gs = reinterpret_cast<const uint16_t*>(&gv);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = bf2f(__ldg(tab + gs[e])) * u[e];
  } else {
    float g[8];
    unpack8(gv, g);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = round_bf(silu_f(g[e])) * u[e];
  }
  *reinterpret_cast<uint4*>(out + row * I + col) = pack8(o);
}

__global__ void __launch_bounds__(256)
gate_mul_kernel(const bf16_t* __restrict__ att, int64_t stride_t, int64_t stride_h, const bf16_t* __restrict__ gate,
                bf16_t* __restrict__ y, int HQ, int D, int64_t nvec) {
  pdl_begin();
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= nvec) return;
  const int64_t e0 = i * 8;
  const int d = static_cast<int>(e0 % D);
  const int64_t th = e0 / D;
  const int h = static_cast<int>(th % HQ);
  const int64_t t = th / HQ;
  float a[8], g[8], o[8];
  unpack8(ldg_stream(att + h * stride_h + t * stride_t + d), a);
  unpack8(ldg_stream(gate + e0), g);
#pragma unroll
  for (int e = 0; e < 8; ++e) o[e] = a[e] * round_bf(sigmoid_f(g[e]));
  *reinterpret_cast<uint4*>(y + e0) = pack8(o);
}

// One warp per 32 keys of one row: ballot of the visibility bytes.
__global__ void __launch_bounds__(256) pack_bits_kernel(const uint8_t* __restrict__ vis, int32_t* __restrict__ bits, int64_t nwords, int N) {
  const int64_t w = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= nwords) return;
  const int lane = threadIdx.x & 31;
  const int words_per_row = N >> 5;
  const int64_t row = w / words_per_row;
  const int wc = static_cast<int>(w - row * words_per_row);
  const uint32_t b = __ballot_sync(0xffffffffu, vis[row * N + wc * 32 + lane] != 0);
  if (lane == 0) bits[w] = static_cast<int32_t>(b);
}

// One warp per (row, task); tasks = HQ query heads, HKV key heads, HKV value heads. Each lane owns D/32 (<= 8) contiguous
// dims. Rotary partner d <-> d + RD/2 lives RD/(2*per) lanes away.
template <int PER>
__global__ void __launch_bounds__(256)
fullattn_prep_kernel(const bf16_t* __restrict__ proj, const float* __restrict__ qw1, const float* __restrict__ kw1,
                     const bf16_t* __restrict__ cosb, const bf16_t* __restrict__ sinb, bf16_t* __restrict__ qt,
                     bf16_t* __restrict__ kt, bf16_t* __restrict__ vt, bf16_t* __restrict__ vt_t, bf16_t* __restrict__ gate,
                     int64_t N, int HQ, int HKV, int D, int RD, float eps) {
  pdl_begin();
  const int ntask = HQ + 2 * HKV;
  const int64_t wid = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (wid >= N * ntask) return;
  const int lane = threadIdx.x & 31;
  const int64_t n = wid / ntask;
  const int task = static_cast<int>(wid - n * ntask);
  const int P = HQ * 2 * D + 2 * HKV * D;
  const int d0 = lane * PER;
  const bf16_t* prow = proj + n * P;
  auto load = [&](const bf16_t* p, float* f) {
    if constexpr (PER == 8) {
      float t[8];
      unpack8(*reinterpret_cast<const uint4*>(p), t);
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = t[e];
    } else {
#pragma unroll
      for (int e = 0; e < PER; ++e) f[e] = bf2f(p[e]);
    }
  };
  auto store = [&](bf16_t* p, const float* f) {
    if constexpr (PER == 8) {
      float t[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) t[e] = f[e];
      *reinterpret_cast<uint4*>(p) = pack8(t);
    } else {
#pragma unroll
      for (int e = 0; e < PER; ++e) p[e] = f2bf(f[e]);
    }
  };
  float xv[PER];
  if (task >= HQ + HKV) {  // value head: plain transpose to head-major
    const int kh = task - HQ - HKV;
    load(prow + HQ * 2 * D + HKV * D + kh * D + d0, xv);
    store(vt + (static_cast<int64_t>(kh) * N + n) * D + d0, xv);
    if (vt_t != nullptr) {      // the same values with rows and columns exchanged: [HKV, D, N] (the tcgen05 attention kernel reads V
#pragma unroll                  // blocks as K-major operand tiles, keys contiguous)
      for (int e = 0; e < PER; ++e) vt_t[(static_cast<int64_t>(kh) * D + d0 + e) * N + n] = f2bf(xv[e]);
    }
    return;
  }
  const bool isq = task < HQ;
  const int hh = isq ? task : task - HQ;
  const bf16_t* src = isq ? prow + static_cast<int64_t>(hh) * 2 * D : prow + HQ * 2 * D + static_cast<int64_t>(hh) * D;
  if (isq) {
    float gv[PER];
    load(src + D + d0, gv);
    store(gate + n * (static_cast<int64_t>(HQ) * D) + hh * D + d0, gv);
  }
  load(src + d0, xv);
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < PER; ++e) ss += xv[e] * xv[e];
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / static_cast<float>(D) + eps);
  const float* w1 = isq ? qw1 : kw1;
  float nv[PER], pv[PER], ov[PER];
#pragma unroll
  for (int e = 0; e < PER; ++e) nv[e] = round_bf((xv[e] * rstd) * __ldg(w1 + d0 + e));
  const int partner = (RD / 2) / PER;  // lane distance of the rotate-half partner
#pragma unroll
  for (int e = 0; e < PER; ++e) pv[e] = __shfl_xor_sync(0xffffffffu, nv[e], partner);
  const bool rope = d0 < RD;
#pragma unroll
  for (int e = 0; e < PER; ++e) {
    if (rope) {
      const float c = bf2f(cosb[n * RD + d0 + e]), s = bf2f(sinb[n * RD + d0 + e]);
      const float rh = (d0 + e < RD / 2) ? -pv[e] : pv[e];
      ov[e] = round_bf(round_bf(nv[e] * c) + round_bf(rh * s));
    } else {
      ov[e] = nv[e];
    }
  }
  bf16_t* dst = isq ? qt : kt;
  store(dst + (static_cast<int64_t>(hh) * N + n) * D + d0, ov);
}

// Per-row e4m3 quantisation for the 8-bit GEMM: scale[m] = max|x[m,:]| / 448 (1 for an all-zero row), q = x / scale rounded
// to e4m3 (saturating). One CTA per row, two passes over the row (the second one hits L1 / L2).
__global__ void __launch_bounds__(kRowThreads)
quantize_rows_e4m3_kernel(const bf16_t* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scale, int K) {
  pdl_begin();
  __shared__ float red[kRowThreads / 32];
  const int64_t row = blockIdx.x;
  const bf16_t* xr = x + row * K;
  float amax = 0.f;
  for (int i = threadIdx.x * 8; i < K; i += kRowThreads * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(xr + i);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(h[e]);
      amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int w = 1; w < kRowThreads / 32; ++w) amax = fmaxf(amax, red[w]);
  const float sc = amax > 0.f ? amax * (1.0f / 448.0f) : 1.0f;
  const float inv = 1.0f / sc;
  if (threadIdx.x == 0) scale[row] = sc;
  uint8_t* qr = q + row * K;
  for (int i = threadIdx.x * 8; i < K; i += kRowThreads * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(xr + i);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
    uint32_t out[2];
#pragma unroll
    for (int e = 0; e < 4; e += 2) {
      const float2 a = __bfloat1622float2(h[e]), b = __bfloat1622float2(h[e + 1]);
      const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a.x * inv, a.y * inv), __NV_SATFINITE, __NV_E4M3);
      const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(b.x * inv, b.y * inv), __NV_SATFINITE, __NV_E4M3);
      out[e >> 1] = lo | (hi << 16);
    }
    *reinterpret_cast<uint2*>(qr + i) = make_uint2(out[0], out[1]);
  }
}

// One thread per slice: a bulk prefetch into L2, nothing is held or waited for.
__global__ void l2_prefetch_kernel(const uint8_t* __restrict__ base, int64_t nbytes, int chunk) {
  const int64_t off = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * chunk;
  if (off >= nbytes) return;
  const uint32_t sz = static_cast<uint32_t>(nbytes - off < chunk ? nbytes - off : chunk);
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(base + off), "r"(sz) : "memory");
}

}  // namespace
}  // namespace ojb

using namespace ojb;

extern "C" int ojb_l2_prefetch(const void* data, int64_t nbytes, int64_t chunk, ojb_stream_t stream) {
  OJB_REQUIRE(data && nbytes >= 0 && chunk >= 16 && chunk % 16 == 0 && chunk <= (1 << 20));
  OJB_REQUIRE((reinterpret_cast<uintptr_t>(data) & 15u) == 0);
  nbytes &= ~static_cast<int64_t>(15);
  if (nbytes == 0) return OJB_OK;
  const int64_t n = ceil_div(nbytes, chunk);
  l2_prefetch_kernel<<<static_cast<unsigned>(ceil_div(n, 128)), 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(data), nbytes, static_cast<int>(chunk));
  return launch_status(cudaGetLastError());
}

extern "C" int ojb_abi_version(void) { return 6; }

extern "C" int ojb_add_rmsnorm(const void* x, const void* delta, const float* w1, const int32_t* rowmask, void* h_out,
                               void* hn_out, int64_t rows, int64_t H, float eps, ojb_stream_t stream) {
  if (rows == 0) return OJB_OK;
  OJB_REQUIRE(x && w1 && hn_out && rows > 0 && H > 0 && H % 8 == 0);
  OJB_REQUIRE(delta == nullptr || h_out != nullptr);
  if (H > kRowThreads * kRowVecs * 8) return OJB_ERR_LIMIT;
  launch_kernel(add_rmsnorm_kernel<0>, dim3(static_cast<unsigned>(rows)), dim3(kRowThreads), 0, static_cast<cudaStream_t>(stream), 
      static_cast<const bf16_t*>(x), static_cast<const bf16_t*>(delta), nullptr, 0, w1, rowmask,
      static_cast<bf16_t*>(h_out), static_cast<bf16_t*>(hn_out), static_cast<int>(H), eps);
  return launch_status(cudaGetLastError());
}

extern "C" int ojb_add_rmsnorm_sk(const void* x, const float* parts, int splits, const float* w1, const int32_t* rowmask,
                                  void* h_out, void* hn_out, int64_t rows, int64_t H, float eps, ojb_stream_t stream) {
  if (rows == 0) return OJB_OK;
  OJB_REQUIRE(x && parts && w1 && h_out && hn_out && rows > 0 && H > 0 && H % 8 == 0 && splits >= 1 && splits <= 16);
  if (H > kRowThreads * kRowVecs * 8) return OJB_ERR_LIMIT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t ps = rows * H;
#define OJB_SK(S)                                                                                                     \
  case S:                                                                                                             \
    launch_kernel(add_rmsnorm_kernel<S>, dim3(static_cast<unsigned>(rows)), dim3(kRowThreads), 0, st,                                        \
        static_cast<const bf16_t*>(x), nullptr, parts, ps, w1, rowmask, static_cast<bf16_t*>(h_out),                  \
        static_cast<bf16_t*>(hn_out), static_cast<int>(H), eps);                                                      \
    break;
  switch (splits) {
    OJB_SK(1) OJB_SK(2) OJB_SK(3) OJB_SK(4) OJB_SK(5) OJB_SK(6) OJB_SK(7) OJB_SK(8)
    OJB_SK(9) OJB_SK(10) OJB_SK(11) OJB_SK(12) OJB_SK(13) OJB_SK(14) OJB_SK(15) OJB_SK(16)
  }
#undef OJB_SK
  return launch_status(cudaGetLastError());
}

extern "C" int ojb_resnorm_f32(float* h, const void* x_init, const void* delta, const float* parts, int splits,
                               const float* w1, const int32_t* rowmask, void* hn_out, int64_t rows, int64_t H, float eps,
                               ojb_stream_t stream) {
  if (rows == 0) return OJB_OK;
  OJB_REQUIRE(h && w1 && hn_out && rows > 0 && H > 0 && H % 8 == 0 && splits >= 0 && splits <= 16);
  OJB_REQUIRE((splits == 0) == (parts == nullptr));
  OJB_REQUIRE(!(parts && delta) && !(x_init && (parts || delta)));
  if (H > kRowThreads * kRowVecs * 8) return OJB_ERR_LIMIT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t ps = rows * H;
#define OJB_RN(S)                                                                                                      \
  case S:                                                                                                              \
    launch_kernel(resnorm_f32_kernel<S>, dim3(static_cast<unsigned>(rows)), dim3(kRowThreads), 0, st, h,               \
                  static_cast<const bf16_t*>(x_init), static_cast<const bf16_t*>(delta), parts, ps, w1, rowmask,        \
                  static_cast<bf16_t*>(hn_out), static_cast<int>(H), eps);                                             \
    break;
  switch (splits) {
    OJB_RN(0) OJB_RN(1) OJB_RN(2) OJB_RN(3) OJB_RN(4) OJB_RN(5) OJB_RN(6) OJB_RN(7) OJB_RN(8)
    OJB_RN(9) OJB_RN(10) OJB_RN(11) OJB_RN(12) OJB_RN(13) OJB_RN(14) OJB_RN(15) OJB_RN(16)
  }
#undef OJB_RN
  return launch_status(cudaGetLastError());
}

// ---- embedding rows + rotary tables of a packed tree: the two things the forward needs before its first layer.
// Block n copies row ids[n] of the embedding table to x[n] (an id outside the table gives a zero row) and writes
// cos / sin of pos[n] * inv_freq[j] for the R2 rotary frequencies, each value twice (columns j and j + R2), as the
// reference's rotary module does for text positions: angle and cos / sin in fp32, one rounding to bf16.
__global__ void __launch_bounds__(256)
embed_rope_kernel(const int64_t* __restrict__ ids, const bf16_t* __restrict__ table, int64_t vocab,
                  const int64_t* __restrict__ pos, const float* __restrict__ inv_freq, float scaling,
                  bf16_t* __restrict__ x, bf16_t* __restrict__ cosb, bf16_t* __restrict__ sinb, int H, int R2) {
  pdl_begin();
  const int64_t n = blockIdx.x;
  const int64_t id = ids[n];
  const bool ok = id >= 0 && id < vocab;
  const uint4* src = reinterpret_cast<const uint4*>(table + (ok ? id : 0) * H);
  uint4* dst = reinterpret_cast<uint4*>(x + n * H);
  for (int i = threadIdx.x; i < (H >> 3); i += blockDim.x) dst[i] = ok ? __ldg(src + i) : make_uint4(0u, 0u, 0u, 0u);
  const float p = static_cast<float>(pos[n]);
  for (int j = threadIdx.x; j < R2; j += blockDim.x) {
    const float a = inv_freq[j] * p;
    const bf16_t c = f2bf(cosf(a) * scaling), sn = f2bf(sinf(a) * scaling);
    cosb[n * 2 * R2 + j] = c; cosb[n * 2 * R2 + R2 + j] = c;
    sinb[n * 2 * R2 + j] = sn; sinb[n * 2 * R2 + R2 + j] = sn;
  }
}

extern "C" int ojb_embed_rope(const int64_t* ids, const void* table, int64_t vocab, const int64_t* pos, const float* inv_freq,
                              float scaling, void* x, void* cosb, void* sinb, int64_t N, int64_t H, int64_t R2,
                              ojb_stream_t stream) {
  if (N == 0) return OJB_OK;
  OJB_REQUIRE(ids && table && pos && inv_freq && x && cosb && sinb && N > 0 && vocab > 0 && H > 0 && H % 8 == 0 && R2 > 0);
  OJB_REQUIRE((reinterpret_cast<uintptr_t>(table) & 15u) == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0);
  launch_kernel(embed_rope_kernel, dim3(static_cast<unsigned>(N)), dim3(256), 0, static_cast<cudaStream_t>(stream), ids,
                static_cast<const bf16_t*>(table), vocab, pos, inv_freq, scaling, static_cast<bf16_t*>(x),
                static_cast<bf16_t*>(cosb), static_cast<bf16_t*>(sinb), static_cast<int>(H), static_cast<int>(R2));
  return launch_status(cudaGetLastError());
}

extern "C" int ojb_act_tables(void* silu_tab, float* sig_tab, ojb_stream_t stream) {
  OJB_REQUIRE(silu_tab && sig_tab);
  act_tables_kernel<<<256, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<bf16_t*>(silu_tab), sig_tab);
  return launch_status(cudaGetLastError());
}

extern "C" int ojb_silu_mul(const void* gu, const void* silu_tab, void* out, int64_t rows, int64_t I, ojb_stream_t stream) {
  OJB_REQUIRE(gu && out && rows >= 0 && I > 0 && I % 8 == 0);
  const int64_t nvec = rows * I / 8;
  if (nvec == 0) return OJB_OK;
  launch_kernel(silu_mul_kernel, dim3(static_cast<unsigned>(ceil_div(nvec, 256))), dim3(256), 0, static_cast<cudaStream_t>(stream), 
      static_cast<const bf16_t*>(gu), static_cast<const bf16_t*>(silu_tab), static_cast<bf16_t*>(out), static_cast<int>(I), nvec);
  return launch_status(cudaGetLastError());
}

extern "C" int ojb_gate_mul(const void* att, int64_t att_stride_t, int64_t att_stride_h, const void* gate, void* y,
                            int64_t T, int64_t HQ, int64_t D, ojb_stream_t stream) {
  OJB_REQUIRE(att && gate && y && T >= 0 && HQ > 0 && D > 0 && D % 8 == 0 && att_stride_t % 8 == 0 && att_stride_h % 8 == 0);
  const int64_t nvec = T * HQ * D / 8;
  if (nvec == 0) return OJB_OK;
  launch_kernel(gate_mul_kernel, dim3(static_cast<unsigned>(ceil_div(nvec, 256))), dim3(256), 0, static_cast<cudaStream_t>(stream), 
      static_cast<const bf16_t*>(att), att_stride_t, att_stride_h, static_cast<const bf16_t*>(gate), static_cast<bf16_t*>(y),
      static_cast<int>(HQ), static_cast<int>(D), nvec);
  return launch_status(cudaGetLastError());
}

extern "C" int ojb_pack_bits(const uint8_t* vis, int32_t* bits, int64_t N, ojb_stream_t stream) {
  OJB_REQUIRE(vis && bits && N > 0 && N % 32 == 0);
  const int64_t nwords = N * (N / 32);
  pack_bits_kernel<<<static_cast<unsigned>(ceil_div(nwords, 8)), 256, 0, static_cast<cudaStream_t>(stream)>>>(vis, bits, nwords,
                                                                                                        static_cast<int>(N));
  return launch_status(cudaGetLastError());
}

extern "C" int ojb_fullattn_prep(const void* proj, const float* qw1, const float* kw1, const void* cosb, const void* sinb,
                                 void* qt, void* kt, void* vt, void* vt_t, void* gate, int64_t N, int64_t HQ, int64_t HKV,
                                 int64_t D, int64_t RD, float eps, ojb_stream_t stream) {
  OJB_REQUIRE(proj && qw1 && kw1 && cosb && sinb && qt && kt && vt && gate && N >= 0 && HQ > 0 && HKV > 0);
  OJB_REQUIRE(D == 256 || D == 128 || D == 64);
  const int per = static_cast<int>(D / 32);
  OJB_REQUIRE(RD > 0 && RD <= D && RD % (2 * per) == 0);
  if (N == 0) return OJB_OK;
  const int64_t warps = N * (HQ + 2 * HKV);
  const unsigned grid = static_cast<unsigned>(ceil_div(warps, 8));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define OJB_PREP(P)                                                                                                     \
  launch_kernel(fullattn_prep_kernel<P>, dim3(grid), dim3(256), 0, st, static_cast<const bf16_t*>(proj), qw1, kw1,                             \
                                                static_cast<const bf16_t*>(cosb), static_cast<const bf16_t*>(sinb),     \
                                                static_cast<bf16_t*>(qt), static_cast<bf16_t*>(kt),                     \
                                                static_cast<bf16_t*>(vt), static_cast<bf16_t*>(vt_t),                   \
                                                static_cast<bf16_t*>(gate), N,                                          \
                                                static_cast<int>(HQ), static_cast<int>(HKV), static_cast<int>(D),       \
                                                static_cast<int>(RD), eps)
  if (per == 8) OJB_PREP(8); else if (per == 4) OJB_PREP(4); else OJB_PREP(2);
#undef OJB_PREP
  return launch_status(cudaGetLastError());
}

// ------------------------------------------------------------------------------------------------------- scoring head
namespace ojb {
namespace {
// one warp per (candidate, output): out[s, a] = bias[a] + sum_h float(hn[rows[s], h]) * W[a, h]
__global__ void __launch_bounds__(256)
score_head_kernel(const bf16_t* __restrict__ hn, const int64_t* __restrict__ rows, const float* __restrict__ W,
                  const float* __restrict__ bias, float* __restrict__ out, int S, int A, int H) {
  pdl_begin();
  const int wid = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (wid >= S * A) return;
  const int lane = threadIdx.x & 31;
  const int s = wid / A, a = wid - s * A;
  const bf16_t* x = hn + rows[s] * static_cast<int64_t>(H);
  const float* w = W + static_cast<int64_t>(a) * H;
  float acc = 0.f;
  for (int c = lane * 8; c < H; c += 256) {
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(x + c), f);
    const float4 w0 = *reinterpret_cast<const float4*>(w + c), w1 = *reinterpret_cast<const float4*>(w + c + 4);
    acc += f[0] * w0.x + f[1] * w0.y + f[2] * w0.z + f[3] * w0.w + f[4] * w1.x + f[5] * w1.y + f[6] * w1.z + f[7] * w1.w;
  }
  acc = warp_sum(acc);
  if (lane == 0) out[wid] = acc + (bias ? bias[a] : 0.f);
}
}  // namespace
}  // namespace ojb

extern "C" int ojb_score_head(const void* hn, const int64_t* rows, const float* W, const float* bias, float* out, int64_t S,
                              int64_t A, int64_t H, ojb_stream_t stream) {
  if (S == 0 || A == 0) return OJB_OK;
  OJB_REQUIRE(hn && rows && W && out && S > 0 && A > 0 && H > 0 && H % 8 == 0);
  const int64_t warps = S * A;
  launch_kernel(ojb::score_head_kernel, dim3(static_cast<unsigned>(ojb::ceil_div(warps, 8))), dim3(256), 0, static_cast<cudaStream_t>(stream), 
      static_cast<const ojb::bf16_t*>(hn), rows, W, bias, out, static_cast<int>(S), static_cast<int>(A), static_cast<int>(H));
  return ojb::launch_status(cudaGetLastError());
}

extern "C" int ojb_quantize_rows_e4m3(const void* x, void* q, float* scale, int64_t rows, int64_t K, ojb_stream_t stream) {
  if (rows == 0) return OJB_OK;
  OJB_REQUIRE(x && q && scale && rows > 0 && K > 0 && K % 8 == 0);
  launch_kernel(quantize_rows_e4m3_kernel, dim3(static_cast<unsigned>(rows)), dim3(kRowThreads), 0, static_cast<cudaStream_t>(stream),
      static_cast<const bf16_t*>(x), static_cast<uint8_t*>(q), scale, static_cast<int>(K));
  return launch_status(cudaGetLastError());
}
