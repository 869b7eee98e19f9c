// Building-block check: tcgen05.mma with the A operand in tensor memory (the "TS" form).
//   D[128 x 64] (fp32) = A[128 x 64] (bf16, written to TMEM by the threads that own the rows) * B[64 x 64]^T
// A is stored the way the attention kernel stores its probability tile: thread r of the warpgroup owns TMEM
// lane r and writes K/2 32-bit columns, each holding the two consecutive K elements (2c in the low half).
// Kept as a unit-tested building block; not a production op.
#include "host_util.h"
#include "sm100.cuh"

namespace ubm {

__global__ void __launch_bounds__(128, 1)
tsmma_probe_kernel(const __nv_bfloat16* __restrict__ A, const __nv_bfloat16* __restrict__ B, float* __restrict__ D,
                   KernelStatus* status) {
  __shared__ __align__(1024) uint8_t sB[64 * 128];   // [64 n rows][64 k] bf16, 128-byte swizzle
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_slot;
  __shared__ uint32_t abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const WaitScope ws{&abort_flag, status};
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_slot, 128);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tbase = tmem_slot;
  const uint32_t tD = tbase;        // 64 fp32 columns
  const uint32_t tA = tbase + 64;   // 32 columns = 64 bf16 per lane
  const int row = threadIdx.x;
  {
    uint32_t av[32];
    const uint32_t* ap = reinterpret_cast<const uint32_t*>(A + row * 64);
#pragma unroll
    for (int c = 0; c < 32; ++c) av[c] = ap[c];
    tmem_st32(tmem_addr(tA, warp, 0), av);
    tmem_st_wait();
  }
  if (row < 64) {
    const uint4* bp = reinterpret_cast<const uint4*>(B + row * 64);
#pragma unroll
    for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(sB + swz128_offset(row, c)) = bp[c];
  }
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0) {
    tc_fence_after_sync();
    constexpr uint32_t idesc = umma_idesc_bf16(128, 64, 0, 0);
    const uint32_t sb = smem_u32(sB);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint64_t bd = umma_smem_desc(sb + k * 32, 16, 1024, kSwizzle128);
      umma_ts(tD, tA + k * 8, bd, idesc, k != 0 ? 1u : 0u);   // 16 bf16 of K = 8 TMEM columns
    }
    umma_commit(&bar);
  }
  mbar_wait(&bar, 0, ws, 95);
  tc_fence_after_sync();
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    uint32_t v[32];
    tmem_ld32(tmem_addr(tD, warp, c * 32), v);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 32; ++j) D[row * 64 + c * 32 + j] = __uint_as_float(v[j]);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tbase, 128);
  }
}

}  // namespace ubm

extern "C" int ubm_tsmma_probe(const void* A, const void* B, void* D, void* status, void* stream) {
  ubm::tsmma_probe_kernel<<<1, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(A), static_cast<const __nv_bfloat16*>(B), static_cast<float*>(D),
      static_cast<ubm::KernelStatus*>(status));
  UBM_CHECK_LAUNCH("tsmma_probe_kernel");
  return ubm::UBM_OK;
}
