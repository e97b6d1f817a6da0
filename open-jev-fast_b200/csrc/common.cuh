// Shared device/host helpers for the ojb200 kernels (sm_100a only).
#pragma once
#include <cstdlib>
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

// ---- mbarrier primitives shared by every kernel that waits for asynchronous copies or tensor-core work
constexpr int kDefaultWaitMs = 2000;   // limit of every device-side wait unless ojb_gemm_set_wait_limit_ms changed it

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      " selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait. Returns false when the limit ran out or another role of this CTA already gave up. abort_flag[0] is the
// CTA's give-up flag, abort_flag[1] the limit in milliseconds (both in shared memory, set up by thread 0 of the CTA).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  for (uint32_t it = 1;; ++it) {
    if (mbar_try(bar, parity)) return true;
    if ((it & 63u) == 0) {
      if (*abort_flag) return false;
      if (global_timer_ns() - t0 > static_cast<uint64_t>(abort_flag[1]) * 1000000ull) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}

// Host-settable limit of those waits and the failure switch of the tests (gemm_api.cu: ojb_gemm_set_wait_limit_ms,
// ojb_gemm_test_drop_copy); read by every launcher whose kernel waits on an mbarrier.
int gemm_wait_limit_ms();
int gemm_drop_copy();

static inline int launch_status(cudaError_t e) { return e == cudaSuccess ? OJB_OK : OJB_ERR_LAUNCH; }

// Launch state that CUDA keeps per device (a kernel's opt-in shared-memory size, the SM count) is cached per device, so one
// process can drive several GPUs. Two host threads making the first call on one device at once set the same value twice.
constexpr int kMaxDevices = 64;
inline int current_device() {
  int d = -1;
  return (cudaGetDevice(&d) == cudaSuccess && d >= 0 && d < kMaxDevices) ? d : -1;
}
// Raises the dynamic shared-memory limit of `kern` on the current device to at least `bytes`; `set` remembers, per device,
// what has been granted.
template <typename Kern>
inline bool raise_smem_limit(Kern kern, int bytes, int (&set)[kMaxDevices]) {
  const int d = current_device();
  if (d < 0) return false;
  if (set[d] >= bytes) return true;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return false;
  set[d] = bytes;
  return true;
}
inline int device_sm_count() {
  static int n[kMaxDevices] = {};
  const int d = current_device();
  if (d < 0) return 0;
  if (n[d] == 0 && cudaDeviceGetAttribute(&n[d], cudaDevAttrMultiProcessorCount, d) != cudaSuccess) n[d] = 0;
  return n[d];
}

// ---- Programmatic dependent launch (off unless OJB_PDL=1 is in the environment). Every kernel of the hot loop goes through
// launch_kernel() and begins with pdl_begin(): with the stream-serialisation attribute set, the next kernel of the stream
// may be scheduled as soon as all CTAs of this one have started (its CTAs fill SMs that this grid leaves idle, set up their
// shared memory / barriers / TMEM, and park at their own pdl_wait), and pdl_wait() blocks until the previous kernel has
// completed and its writes are visible. No global memory may be read or written before pdl_wait(). Measured on the 539-row
// tree: 32.9 ms with the attribute against 32.6 ms without, at 1650 against 1695 MHz — the forward runs against the power
// cap, so closing the gaps between kernels only lowers the clock; without the attribute both instructions are no-ops.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_begin() {
  pdl_launch_dependents();
  pdl_wait();
}

inline bool pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("OJB_PDL");
    on = (e && e[0] == '1') ? 1 : 0;
  }
  return on == 1;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

#define OJB_REQUIRE(cond)             \
  do {                                \
    if (!(cond)) return OJB_ERR_ARG;  \
  } while (0)

static inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

}  // namespace ojb
