// Asynchronous copies for the sm_100a kernels: mbarriers with BOUNDED waits, TMA tile copies, linear bulk
// copies and the host side of tensor maps.  Included by every kernel that stages operands through shared
// memory with cp.async.bulk.
//
// Bounded waits.  A wait on an mbarrier polls at most NHV_WAIT_LIMIT times (define it before the include to
// change it).  A wait that runs out stores its code in the file's error word and returns false; the kernel then
// leaves through its ordinary exit (give_up_delay() first, so that copies still in flight land while the block's
// shared memory is still its own).  The error word stays set until the host takes it: nhv_wait_error_take()
// reads and clears it, nhv_wait_error_address() gives its device address so that a later kernel of the step
// (the sampler) can fold it into what the host reads anyway.  Every file that includes this header has an error
// word of its own.
#pragma once
#include <cuda.h>
#include <cudaTypedefs.h>

#include "nhv_common.cuh"

#ifndef NHV_WAIT_LIMIT
#define NHV_WAIT_LIMIT (1u << 24)
#endif

static __device__ int g_wait_error = 0;

static __device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
static __device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
static __device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
static __device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
static __device__ __forceinline__ void wait_error_set(int code) { atomicExch(&g_wait_error, code); }
// Bounded wait: false (and the error word set to `code`) if the phase did not complete within the limit.
static __device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int code) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t i = 0; i < (uint32_t)(NHV_WAIT_LIMIT); ++i) {
    uint32_t done;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    if (done) return true;
  }
  wait_error_set(code);
  return false;
}
// One tile of a 2-D tensor map into shared memory; completion is counted in bytes on `bar`.  x (the innermost
// coordinate) times the element size must be a multiple of 16 bytes.  No multicast: every block fetches its own.
static __device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
               ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
// The same of a 3-D tensor map (x innermost).
static __device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n"
               ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar)) : "memory");
}
// The same of a 4-D tensor map (x innermost).
static __device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, int x, int y, int z, int w, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];\n"
               ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(x), "r"(y), "r"(z), "r"(w), "r"(smem_u32(bar)) : "memory");
}
// A linear copy: both addresses 16-byte aligned, the size a multiple of 16 bytes.
static __device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// After a wait ran out: give copies that may still be in flight time to land before the block leaves.
static __device__ __forceinline__ void give_up_delay() {
  for (int i = 0; i < 2000; ++i) __nanosleep(200);
}

// ---------------------------------------------------------------- host side
// Reads and clears the file's error word (0: no bounded wait ran out since the last call; -1: the read failed).
// Synchronises the device.
static inline int nhv_wait_error_take() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_wait_error, sizeof(int)) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(g_wait_error, &zero, sizeof(int));
  return v;
}
// The device address of the file's error word on the current device (nullptr if it cannot be had).
static inline void* nhv_wait_error_address() {
  void* p = nullptr;
  if (cudaGetSymbolAddress(&p, g_wait_error) != cudaSuccess) return nullptr;
  return p;
}

// A tensor map of `rank` (2 to 5) dimensions over bfloat16 elements, innermost first: dims[i] elements that lie
// stride_bytes[i] apart (stride_bytes[0] is 2 and is not passed on; the others must be multiples of 16 and need
// not grow with i), read in boxes of box[i] with the 128-byte swizzle (box[0] * 2 bytes must not exceed 128).  A
// box arrives in shared memory with dimension 0 fastest, then 1, 2, ...
static inline bool nhv_make_map_bf16_nd(CUtensorMap* map, const void* base, int rank, const long long* dims,
                                        const long long* stride_bytes, const int* box) {
  static PFN_cuTensorMapEncodeTiled_v12000 encode = nullptr;
  if (!encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) return false;
    encode = (PFN_cuTensorMapEncodeTiled_v12000)fn;
  }
  if (rank < 2 || rank > 5) return false;
  cuuint64_t d[5], st[4];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) {
    d[i] = (cuuint64_t)dims[i];
    bx[i] = (cuuint32_t)box[i];
    es[i] = 1;
    if (i > 0) st[i - 1] = (cuuint64_t)stride_bytes[i];
  }
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), d, st, bx, es,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// A tensor map over a row-major bfloat16 matrix [rows, cols] whose rows lie `row_stride_elems` apart, read in
// boxes of box_cols x box_rows with the 128-byte swizzle (box_cols * 2 bytes must not exceed 128).
static inline bool nhv_make_map_bf16(CUtensorMap* map, const void* base, long long rows, long long cols,
                                     long long row_stride_elems, int box_cols, int box_rows) {
  static PFN_cuTensorMapEncodeTiled_v12000 encode = nullptr;
  if (!encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) return false;
    encode = (PFN_cuTensorMapEncodeTiled_v12000)fn;
  }
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)row_stride_elems * 2};
  const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  const cuuint32_t elem_strides[2] = {1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
