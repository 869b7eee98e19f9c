// Triangle multiplication without any device allocation: the intermediates of the three-kernel
// pipeline live in a fixed array inside the library image instead of caller-provided buffers.
// See ubm_noalloc.h for who this is for and for the contract.
#include "ubm_noalloc.h"

#include <cuda_runtime.h>
#include <stdio.h>

#include "host_util.h"

// The existing entry points (defined in pair_proj_sm100.cu, gemm_sm100.cu, trimul_out_sm100.cu).
extern "C" int ubm_trimul_proj(const void* z, const void* w, const void* colsum, const void* colbias, const void* mask,
                               void* planes, void* stats_out, int N, int Np, void* status, void* stream);
extern "C" int ubm_gemm_bf16(const void* A, const void* B, void* C, const void* bias, const void* residual, int M,
                             int N, int K, int batch, long long lda, long long ldb, long long ldc, long long ldr,
                             long long strideA, long long strideB, long long strideC, long long strideR, int mn_major,
                             int out_fp32, int act, float alpha, void* status, void* stream);
extern "C" int ubm_trimul_out(const void* x, const void* z, const void* wo, const void* wg, const void* o_colsum,
                              const void* o_colbias, const void* g_colsum, const void* g_colbias, void* out, int N,
                              int Np, int add_residual, void* status, void* stream);

// Scratch: operand planes a, b and the contraction result, each [128][MAX_N][MAX_N] bf16.  In host code
// this name is only a handle for cudaGetSymbolAddress; it is not a device address.
static __device__ __align__(256) unsigned char g_trimul_scratch[UBM_TRIMUL_NOALLOC_SCRATCH_BYTES];

namespace {

constexpr int kMaxDevices = 64;
void* g_scratch_ptr[kMaxDevices] = {nullptr};

// Device address of the scratch array on the current device (looked up once per device).
int scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    fprintf(stderr, "[ubm] trimul_noalloc: cudaGetDevice failed: %s\n", cudaGetErrorString(e));
    return ubm::UBM_ERR_DRIVER;
  }
  if (dev < 0 || dev >= kMaxDevices) {
    fprintf(stderr, "[ubm] trimul_noalloc: device ordinal %d is outside the %d devices this entry point tracks\n", dev,
            kMaxDevices);
    return ubm::UBM_ERR_DRIVER;
  }
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_trimul_scratch);
    if (e != cudaSuccess || p == nullptr) {
      fprintf(stderr, "[ubm] trimul_noalloc: cudaGetSymbolAddress failed on device %d: %s\n", dev,
              cudaGetErrorString(e));
      return ubm::UBM_ERR_DRIVER;
    }
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return ubm::UBM_OK;
}

}  // namespace

extern "C" int ubm_trimul_noalloc(const void* z, const void* mask, const void* w_in, const void* in_colsum,
                                  const void* in_colbias, const void* wo, const void* wg, const void* o_colsum,
                                  const void* o_colbias, const void* g_colsum, const void* g_colbias, void* out, int N,
                                  int outgoing, int add_residual, void* status, void* stream) {
  using namespace ubm;
  if (z == nullptr || out == nullptr || w_in == nullptr || wo == nullptr || wg == nullptr || N <= 0 || (N & 7)) {
    fprintf(stderr, "[ubm] trimul_noalloc: bad argument (N must be a positive multiple of 8)\n");
    return UBM_ERR_ARGUMENT;
  }
  if (N > UBM_TRIMUL_NOALLOC_MAX_N) {
    fprintf(stderr,
            "[ubm] trimul_noalloc: N = %d exceeds the built-in scratch array (at most %d tokens); use the "
            "entry points that take caller-provided buffers\n",
            N, UBM_TRIMUL_NOALLOC_MAX_N);
    return UBM_ERR_TOO_LARGE;
  }
  void* base = nullptr;
  int rc = scratch_for_current_device(&base);
  if (rc) return rc;
  const int Np = N;  // N is a multiple of 8, so rows already start on 16-byte boundaries
  const size_t plane_bytes = static_cast<size_t>(128) * N * Np * 2;  // multiple of 256 for N % 8 == 0
  unsigned char* planes = static_cast<unsigned char*>(base);         // a then b
  unsigned char* x = planes + 2 * plane_bytes;
  rc = ubm_trimul_proj(z, w_in, in_colsum, in_colbias, mask, planes, nullptr, N, Np, status, stream);
  if (rc) return rc;
  const long long ld = Np, bs = static_cast<long long>(N) * Np;
  rc = ubm_gemm_bf16(planes, planes + plane_bytes, x, nullptr, nullptr, N, N, N, 128, ld, ld, ld, 0, bs, bs, bs, 0,
                     outgoing ? 0 : 1, 0, 0, 1.0f, status, stream);
  if (rc) return rc;
  return ubm_trimul_out(x, z, wo, wg, o_colsum, o_colbias, g_colsum, g_colbias, out, N, Np, add_residual, status,
                        stream);
}
