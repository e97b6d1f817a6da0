// Shared device/host helpers for the ojb200 kernels (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "../../include/ojb200.h"

namespace ojb {

typedef __nv_bfloat16 bf16_t;

__device__ __forceinline__ float bf2f(bf16_t v) { return __bfloat162float(v); }
__device__ __forceinline__ bf16_t f2bf(float v) { return __float2bfloat16_rn(v); }
// value of v after one round trip through bf16 (round-to-nearest-even)
__device__ __forceinline__ float round_bf(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// unpack / pack 8 bf16 held in a uint4
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&t);
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Record the first device-side failure code in the caller's status word (may be null).
__device__ __forceinline__ void report_status(int32_t* status, int32_t code) {
  if (status) atomicCAS(status, 0, code);
}

static inline int launch_status(cudaError_t e) { return e == cudaSuccess ? OJB_OK : OJB_ERR_LAUNCH; }

#define OJB_REQUIRE(cond)             \
  do {                                \
    if (!(cond)) return OJB_ERR_ARG;  \
  } while (0)

static inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

}  // namespace ojb
