// Shared device/host helpers of the binade_b200 CUDA library (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/binade_b200.h"

#define BN_TILE 128
#define BN_WARP 32
#define BN_FULL 0xffffffffu

namespace bn {

// Records `msg` as the calling thread's last error and returns `code`.
int fail(int code, const char *msg);
int fail_cuda(cudaError_t e, const char *where);

#define BN_CUDA(call)                                   \
  do {                                                  \
    cudaError_t e_ = (call);                            \
    if (e_ != cudaSuccess) return bn::fail_cuda(e_, #call); \
  } while (0)

// Result of a kernel launch: picks up configuration errors without synchronising.
inline int launched(const char *what) {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? BN_OK : fail_cuda(e, what);
}

// Streaming batch-1 matvec (r4_stream.cu); -1 when the shape is outside its coverage.
int stream_matvec(const bn_r4 *w, const uint16_t *x, int64_t N, int64_t K, uint16_t *y, cudaStream_t s);

int stream_rows(const bn_r4 *w, const uint16_t *x, int64_t x_stride, int64_t M, int64_t N, int64_t K, uint16_t *y, int64_t y_stride, cudaStream_t s);
int stream_gather(const bn_r4 *w, const uint16_t *x, const uint32_t *xi, const uint32_t *ei, int64_t G, int64_t n, int64_t K, int64_t RS, int64_t R0, int64_t split, uint16_t *y, uint16_t *y2, cudaStream_t s);

int stream_gather_grouped(const bn_r4 *w, const uint16_t *x, const uint32_t *xi, const uint32_t *seg, const uint32_t *order, int64_t E, int64_t G, int64_t max_per_expert, int64_t n, int64_t K, int64_t RS, int64_t R0, int64_t split, uint16_t *y, uint16_t *y2, cudaStream_t s);

// Batch-1 matvec with eight (or sixteen, or thirty-two) threads per row, up to four matrices that
// share x in one launch, and the expert gather through the same kernel (r4_oct.cu); -1 when the
// shape is outside its coverage.
int oct_matvec(const bn_r4 *w, const uint16_t *x, int64_t N, int64_t K, uint16_t *y, cudaStream_t s);
int oct_matvec_multi(const bn_r4 *const *w, const int64_t *N, uint16_t *const *y, int nmat, const uint16_t *x, int64_t K, cudaStream_t s);
int oct_gather(const bn_r4 *w, const uint16_t *x, const uint32_t *xi, const uint32_t *ei, int64_t G, int64_t n, int64_t K, int64_t RS, int64_t R0, int64_t split, uint16_t *y, uint16_t *y2, cudaStream_t s);
int oct_status(int *status);

// Register-pipelined batch-1 matvec and expert gather (r4_direct.cu); -1 outside their coverage.
int direct_matvec(const bn_r4 *w, const uint16_t *x, int64_t N, int64_t K, uint16_t *y, cudaStream_t s);
int direct_gather(const bn_r4 *w, const uint16_t *x, const uint32_t *xi, const uint32_t *ei, int64_t G, int64_t n, int64_t K, int64_t RS, int64_t R0, int64_t split, uint16_t *y, uint16_t *y2, cudaStream_t s);

// Tensor-core decode GEMM for up to 128 input rows (r4_mma.cu); -1 outside its coverage.
int mma_rows(const bn_r4 *w, const uint16_t *x, int64_t x_stride, int64_t M, int64_t N, int64_t K, uint16_t *y, int64_t y_stride, int split, cudaStream_t s);
int mma_status(int *status);
int exchange_status(int *status);  // exchange.cu
int exchange_status_reset();
int mma_status_reset();
int stream_status_reset();
int oct_status_reset();

inline int64_t tiles(int64_t K) { return (K + BN_TILE - 1) / BN_TILE; }

// Raises a kernel's dynamic shared memory limit once per (kernel, device).
template <typename Kernel>
inline cudaError_t allow_smem(Kernel k, size_t bytes) {
  return cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

#ifdef __CUDACC__
__device__ __forceinline__ uint32_t lane_id() { return threadIdx.x & 31; }
__device__ __forceinline__ uint32_t lanemask_lt() {
  uint32_t m;
  asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
  return m;
}

// Streaming global loads: read once, keep out of L1.
__device__ __forceinline__ uint32_t ldg_stream_u32(const void *p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ldg_stream_u16(const void *p) {
  uint16_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t smem_addr(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

// fp32 -> BF16 bit pattern, round to nearest even (cvt.rn.bf16.f32; NaN -> 0x7FFF).
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float f) {
  uint16_t r;
  asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(r) : "f"(f));
  return r;
}

// Exclusive prefix (over lanes, in lane order) and warp total of a per-lane count in 0..7,
// from three ballots instead of a five-step shuffle scan. All 32 lanes must call.
__device__ __forceinline__ void warp_scan_small(uint32_t cnt, uint32_t lt, uint32_t &pre, uint32_t &tot) {
  uint32_t b0 = __ballot_sync(BN_FULL, cnt & 1u), b1 = __ballot_sync(BN_FULL, cnt & 2u), b2 = __ballot_sync(BN_FULL, cnt & 4u);
  pre = __popc(b0 & lt) + 2 * __popc(b1 & lt) + 4 * __popc(b2 & lt);
  tot = __popc(b0) + 2 * __popc(b1) + 4 * __popc(b2);
}
#endif

}  // namespace bn
