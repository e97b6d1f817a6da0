// tcgen05 / TMA / mbarrier wrappers and host helpers shared by the two GEMM kernels (sm_100a).
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace ojb {
namespace {


constexpr int kBM = 128;           // UMMA M
constexpr int kBK = 64;            // bf16 elements per stage along K = one 128-byte swizzle row
constexpr int kUmmaK = 16;         // K of one tcgen05.mma.kind::f16
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

// Bulk tensor store of one shared-memory tile (box of the map) to global memory; x = column, y = row, z = plane.
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(map), "r"(src), "r"(x),
               "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all bulk stores of this thread have finished reading their shared-memory source
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// all but the most recent bulk group of this thread have read their shared-memory source
__device__ __forceinline__ void bulk_wait_read1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
// all bulk stores of this thread are complete
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// make shared-memory writes of this thread visible to the bulk-copy engine
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
      : "memory");
}
// The same MMA on 8-bit floating-point operands (kind::f8f6f4; K = 32 elements = 32 bytes per instruction).
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
      : "memory");
}
// Arrive on an mbarrier once every tcgen05.mma issued so far by this thread has finished.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 lanes x 32 consecutive fp32 columns: thread i of the warp receives row (lane base + i).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major bf16 tile whose rows are 128 bytes (64 elements) and which TMA wrote with
// the 128-byte swizzle: 8-row groups are 1024 bytes apart (stride byte offset); the leading byte offset is not used by
// swizzled K-major layouts; bits 46-47 carry the descriptor version of this architecture; bits 61-63 the swizzle mode.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
// Instruction descriptor of tcgen05.mma.kind::f16: fp32 accumulator, bf16 A and B, both K-major, M = 128, N = BN.
__host__ __device__ constexpr uint32_t umma_idesc(int bn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(bn >> 3) << 17) |
         (static_cast<uint32_t>(kBM >> 4) << 24);
}


// Instruction descriptor of tcgen05.mma.kind::f8f6f4: fp32 accumulator, e4m3 A and B (format code 0), both K-major.
__host__ __device__ constexpr uint32_t umma_idesc_e4m3(int bn) {
  return (1u << 4) | (static_cast<uint32_t>(bn >> 3) << 17) | (static_cast<uint32_t>(kBM >> 4) << 24);
}

// 32 lanes x 16 consecutive fp32 columns
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ float exp2f_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// SiLU of the fused epilogues: approximate exponential and division (about 2 ulp in fp32, far below the bf16 rounding that
// follows); the full-precision forms cost more issue slots than the rest of the epilogue together.
__device__ __forceinline__ float silu_f(float x) { return __fdividef(x, 1.0f + __expf(-x)); }
// Two SiLUs with one reciprocal: 1/a = b / (a b). The exponent is capped at 2^60 so that the product of the two
// denominators stays finite; below x = -41.6 the result differs from x e^x by less than 4e-17.
__device__ __forceinline__ void silu2_f(float x0, float x1, float& s0, float& s1) {
  const float d0 = 1.0f + exp2f_fast(fminf(-x0 * 1.4426950408889634f, 60.0f));
  const float d1 = 1.0f + exp2f_fast(fminf(-x1 * 1.4426950408889634f, 60.0f));
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(d0 * d1));
  s0 = x0 * (r * d1);
  s1 = x1 * (r * d0);
}

enum Epilogue { kEpiBf16 = 0, kEpiSwiglu = 1, kEpiPartialF32 = 2 };

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// (a function-local static with an initialiser: several host threads, one per GPU, may make their first call at once)
EncodeTiledFn encode_fn() {
  static const EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      return reinterpret_cast<EncodeTiledFn>(p);
    return static_cast<EncodeTiledFn>(nullptr);
  }();
  return fn;
}

// 2-D bf16 tensor map over a row-major [rows, cols] matrix, box = [box_rows, 64 columns], 128-byte swizzle, zero fill.
// (32-column boxes with the 64-byte swizzle give twice the stages but were measured 30 % slower: the copy engine moves
// whole 128-byte lines.)
int make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return OJB_ERR_DRIVER;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(kBK), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? OJB_OK : OJB_ERR_ARG;
}

// The same for a row-major matrix of bytes (e4m3 operands): a box is box_rows rows of 128 bytes = 128 elements of K.
int make_map_u8(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return OJB_ERR_DRIVER;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols)};
  cuuint32_t box[2] = {128u, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? OJB_OK : OJB_ERR_ARG;
}

// Tensor map of an output matrix for bulk tensor stores from [32 rows][128 bytes] shared-memory tiles written with the
// 128-byte swizzle: rows x cols elements of elt bytes (2 = bf16, 4 = fp32), row pitch ld elements, `planes` matrices
// plane_stride elements apart. Stores are clipped at the matrix edges.
int make_out_map(CUtensorMap* map, void* base, int elt, int64_t rows, int64_t cols, int64_t ld, int64_t planes,
                 int64_t plane_stride) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return OJB_ERR_DRIVER;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(planes)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * elt, static_cast<cuuint64_t>(plane_stride) * elt};
  cuuint32_t box[3] = {static_cast<cuuint32_t>(128 / elt), 32, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, elt == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, base, dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? OJB_OK : OJB_ERR_ARG;
}

// Tensor map of an output matrix for bulk tensor stores of the swapped-operand units: boxes of 16 rows x 32 columns from
// plain (unswizzled) [16][32] shared-memory tiles.
int make_tail_out_map(CUtensorMap* map, void* base, int elt, int64_t rows, int64_t cols, int64_t ld, int64_t planes,
                      int64_t plane_stride) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return OJB_ERR_DRIVER;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(planes)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * elt, static_cast<cuuint64_t>(plane_stride) * elt};
  cuuint32_t box[3] = {32, 16, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, elt == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, base, dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? OJB_OK : OJB_ERR_ARG;
}

inline int sm_count() { return device_sm_count(); }

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

// Launchers of the two kernels (defined in gemm_tile128.cu and gemm_block256.cu). epi is an Epilogue value.
int gemm_tile128_launch(int epi, int bn, const void* x, const void* w, void* out, int64_t M, int64_t N, int64_t K, int splits,
                        int64_t ldo, int32_t* status, cudaStream_t stream);
int gemm_block256_launch(int epi, int bn_req, const void* x, const void* w, void* out, int64_t M, int64_t N, int64_t K,
                         int splits, int64_t ldo, int32_t* status, cudaStream_t stream);
void gemm_block256_set_trace(unsigned long long* buf, int cap);
// process-wide settings kept in gemm_api.cu: limit of the device-side waits (ms) and the failure-injection switch of the tests
// e4m3 operands with one fp32 scale per row of x (sx) and per row of w (sw): out = (xq . wq^T) * sx[m] * sw[n]
int gemm_block256_launch_e4m3(int epi, const void* xq, const float* sx, const void* wq, const float* sw, void* out, int64_t M,
                              int64_t N, int64_t K, int splits, int64_t ldo, int32_t* status, cudaStream_t stream);
int gemm_pair256_launch(int epi, int bn_req, const void* x, const void* w, void* out, int64_t M, int64_t N, int64_t K,
                        int splits, int64_t ldo, int32_t* status, cudaStream_t stream);
void gemm_pair256_set_trace(unsigned long long* buf, int cap);
#ifdef OJB_GEMM_PROBES
void gemm_block256_set_probe(int repeat, int knob);
void gemm_pair256_set_probe(int repeat, int max_stages);
#endif

}  // namespace ojb
