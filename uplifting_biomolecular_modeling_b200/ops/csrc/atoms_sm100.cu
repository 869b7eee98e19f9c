// Atom <-> token traffic of the diffusion module: the per-token mean of atom rows (encoder) and the broadcast of
// token rows back to atoms added to the atom stream (decoder).  Both are single-pass gathers with 16-byte
// accesses; the mean adds the atoms of a token in table order, so the result does not depend on scheduling
// (no atomics).  Reference kernel with the same job: _seg_reduce_kernel
// (common/opt_core/opt_core/kernels/dtk_kernels.py) and the deterministic segment reduce of
// precision/det_scatter.py:104.
#include "host_util.h"
#include "sm100.cuh"

namespace ubm {

// t: bf16 [B][A][C]; table: int32 [N][M] atom indices of each token, -1 = no atom; out: bf16 [B][N][C] = mean
__global__ void __launch_bounds__(256) segment_mean_kernel(const __nv_bfloat16* __restrict__ t,
                                                           const int* __restrict__ table,
                                                           __nv_bfloat16* __restrict__ out, int B, int A, int N,
                                                           int M, int C) {
  const int c8 = C / 8;
  const long long total = static_cast<long long>(B) * N * c8;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % c8) * 8;
    const long long bn = i / c8;
    const int n = static_cast<int>(bn % N);
    const int b = static_cast<int>(bn / N);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    int cnt = 0;
    for (int m = 0; m < M; ++m) {
      const int a = __ldg(table + static_cast<long long>(n) * M + m);
      if (a < 0) continue;
      const uint4 u = *reinterpret_cast<const uint4*>(t + (static_cast<long long>(b) * A + a) * C + c);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] += bf16_lo(w[j]);
        acc[2 * j + 1] += bf16_hi(w[j]);
      }
      ++cnt;
    }
    const float inv = 1.0f / static_cast<float>(cnt > 0 ? cnt : 1);
    uint4 o;
    o.x = pack_bf16x2(acc[0] * inv, acc[1] * inv);
    o.y = pack_bf16x2(acc[2] * inv, acc[3] * inv);
    o.z = pack_bf16x2(acc[4] * inv, acc[5] * inv);
    o.w = pack_bf16x2(acc[6] * inv, acc[7] * inv);
    *reinterpret_cast<uint4*>(out + (static_cast<long long>(b) * N + n) * C + c) = o;
  }
}

// out[b][i] = q[b][i] + a[b][a2t[i]]   (q may be null: plain gather); q / out: [B][A][C], a: [B][N][C]
__global__ void __launch_bounds__(256) gather_rows_add_kernel(const __nv_bfloat16* __restrict__ q,
                                                              const __nv_bfloat16* __restrict__ a,
                                                              const int* __restrict__ a2t,
                                                              __nv_bfloat16* __restrict__ out, int B, int A, int N,
                                                              int C) {
  const int c8 = C / 8;
  const long long total = static_cast<long long>(B) * A * c8;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % c8) * 8;
    const long long ba = i / c8;
    const int at = static_cast<int>(ba % A);
    const int b = static_cast<int>(ba / A);
    const int n = __ldg(a2t + at);
    const uint4 ua = *reinterpret_cast<const uint4*>(a + (static_cast<long long>(b) * N + n) * C + c);
    uint4 o = ua;
    if (q != nullptr) {
      const uint4 uq = reinterpret_cast<const uint4*>(q)[i];
      const uint32_t x[4] = {uq.x, uq.y, uq.z, uq.w}, y[4] = {ua.x, ua.y, ua.z, ua.w};
      uint32_t r[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        r[j] = pack_bf16x2(bf16_lo(x[j]) + bf16_lo(y[j]), bf16_hi(x[j]) + bf16_hi(y[j]));
      o = make_uint4(r[0], r[1], r[2], r[3]);
    }
    reinterpret_cast<uint4*>(out)[i] = o;
  }
}

static inline int atoms_grid(long long work) {
  long long b = (work + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 32;
  return static_cast<int>(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace ubm

extern "C" int ubm_segment_mean(const void* t, const void* table, void* out, int B, int A, int N, int M, int C,
                                void* stream) {
  using namespace ubm;
  if (B <= 0 || A <= 0 || N <= 0 || M <= 0 || C <= 0 || (C & 7)) return UBM_ERR_ARGUMENT;
  segment_mean_kernel<<<atoms_grid(static_cast<long long>(B) * N * (C / 8)), 256, 0,
                        static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(t),
                                                             static_cast<const int*>(table),
                                                             static_cast<__nv_bfloat16*>(out), B, A, N, M, C);
  UBM_CHECK_LAUNCH("segment_mean_kernel");
  return UBM_OK;
}

extern "C" int ubm_gather_rows_add(const void* q, const void* a, const void* a2t, void* out, int B, int A, int N,
                                   int C, void* stream) {
  using namespace ubm;
  if (B <= 0 || A <= 0 || N <= 0 || C <= 0 || (C & 7)) return UBM_ERR_ARGUMENT;
  gather_rows_add_kernel<<<atoms_grid(static_cast<long long>(B) * A * (C / 8)), 256, 0,
                           static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(q),
                                                                static_cast<const __nv_bfloat16*>(a),
                                                                static_cast<const int*>(a2t),
                                                                static_cast<__nv_bfloat16*>(out), B, A, N, C);
  UBM_CHECK_LAUNCH("gather_rows_add_kernel");
  return UBM_OK;
}
