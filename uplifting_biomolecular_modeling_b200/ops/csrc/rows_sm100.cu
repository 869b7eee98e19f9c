// Row kernels: memory-bound elementwise / normalisation work that has no GEMM to hide in.
//
//   ubm_layernorm_rows   LayerNorm over the last dimension, one warp per row, 16-byte accesses
//                        (reference rows: fastln / exactln, common/opt_core/opt_core/kernels/ln/DESIGN.md:5-37)
//   ubm_pair_head_bias   bias[h][i][j] = Linear_{c->H}(LN(z[i][j])) as channel-major bf16 planes
//                        (the proj_z of attention with pair bias; reference: _pf_bias_kernel,
//                        common/opt_core/opt_core/kernels/apb/fpf_apb)
//   ubm_adaln_rows       sigmoid(scale[r]) * LN_noaffine(a[r]) + shift[r]   (DiT AdaLN)
//   ubm_gate_residual    out = res + sigmoid(gate) * x
//   ubm_swiglu_rows      out = silu(a) * b for a | b halves of one row
// Reference for the last three: _ln_mod_kernel / _gate_res_kernel / _swiglu_kernel in
// common/opt_core/opt_core/kernels/dtk_kernels.py.
#include "host_util.h"
#include "sm100.cuh"

namespace ubm {

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16(v); }

// One warp per row, two passes over registers-free data (row re-read from L1/L2 on pass two is
// avoided by keeping up to 32 values per lane in registers; wider rows fall back to re-reading).
template <typename TI, typename TO, int MAXPL>
__global__ void __launch_bounds__(256) layernorm_rows_kernel(const TI* __restrict__ x, const float* __restrict__ gamma,
                                                             const float* __restrict__ beta, TO* __restrict__ out,
                                                             long long R, int C, float eps) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (long long r = static_cast<long long>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5); r < R;
       r += static_cast<long long>(gridDim.x) * warps_per_block) {
    const TI* xr = x + r * C;
    float v[MAXPL];
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < MAXPL; ++i) {
      const int c = lane + i * 32;
      v[i] = c < C ? to_f<TI>(xr[c]) : 0.f;
      sum += v[i];
    }
    sum = warp_sum(sum);
    const float mu = sum / C;
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < MAXPL; ++i) {
      const int c = lane + i * 32;
      const float d = c < C ? v[i] - mu : 0.f;
      sq += d * d;
    }
    sq = warp_sum(sq);
    const float rstd = rsqrtf(sq / C + eps);
    TO* orow = out + r * C;
#pragma unroll
    for (int i = 0; i < MAXPL; ++i) {
      const int c = lane + i * 32;
      if (c < C) {
        float y = (v[i] - mu) * rstd;
        if (gamma != nullptr) y *= gamma[c];
        if (beta != nullptr) y += beta[c];
        orow[c] = from_f<TO>(y);
      }
    }
  }
}

// LayerNorm of wide bf16 rows (256 < C <= 2048, C a multiple of 8): one warp per row, 16-byte accesses, the row kept
// in registers (CHUNKS x 8 values per lane).  The single / token tracks and the LM and genomics trunks land here.
template <int CHUNKS>
__global__ void __launch_bounds__(256) layernorm_rows_wide_kernel(const __nv_bfloat16* __restrict__ x,
                                                                  const float* __restrict__ gamma,
                                                                  const float* __restrict__ beta,
                                                                  __nv_bfloat16* __restrict__ out, long long R, int C,
                                                                  float eps) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (long long r = static_cast<long long>(blockIdx.x) * wpb + (threadIdx.x >> 5); r < R;
       r += static_cast<long long>(gridDim.x) * wpb) {
    float v[CHUNKS][8];
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < CHUNKS; ++k) {
      const int c = k * 256 + lane * 8;
      if (c < C) {
        const uint4 u = *reinterpret_cast<const uint4*>(x + r * C + c);
        v[k][0] = bf16_lo(u.x); v[k][1] = bf16_hi(u.x); v[k][2] = bf16_lo(u.y); v[k][3] = bf16_hi(u.y);
        v[k][4] = bf16_lo(u.z); v[k][5] = bf16_hi(u.z); v[k][6] = bf16_lo(u.w); v[k][7] = bf16_hi(u.w);
#pragma unroll
        for (int j = 0; j < 8; ++j) sum += v[k][j];
      }
    }
    const float mu = warp_sum(sum) / C;
    float sq = 0.f;
#pragma unroll
    for (int k = 0; k < CHUNKS; ++k) {
      if (k * 256 + lane * 8 < C) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float d = v[k][j] - mu;
          sq += d * d;
        }
      }
    }
    const float rstd = rsqrtf(warp_sum(sq) / C + eps);
#pragma unroll
    for (int k = 0; k < CHUNKS; ++k) {
      const int c = k * 256 + lane * 8;
      if (c < C) {
        float y[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          y[j] = (v[k][j] - mu) * rstd;
          if (gamma != nullptr) y[j] *= gamma[c + j];
          if (beta != nullptr) y[j] += beta[c + j];
        }
        *reinterpret_cast<uint4*>(out + r * C + c) = make_uint4(pack_bf16x2(y[0], y[1]), pack_bf16x2(y[2], y[3]),
                                                                pack_bf16x2(y[4], y[5]), pack_bf16x2(y[6], y[7]));
      }
    }
  }
}

// LayerNorm of narrow bf16 rows with 16-byte accesses: C = 8 * LPR channels, LPR lanes per row (8, 16 or 32),
// 32 / LPR rows per warp instruction; statistics by xor-shuffles inside the LPR lanes of a row.  The MSA track
// (C = 64, 1.5 M rows per call) spends its LayerNorms here.
template <int LPR>
__global__ void __launch_bounds__(256) layernorm_rows_narrow_kernel(const __nv_bfloat16* __restrict__ x,
                                                                    const float* __restrict__ gamma,
                                                                    const float* __restrict__ beta,
                                                                    __nv_bfloat16* __restrict__ out, long long R,
                                                                    float eps) {
  constexpr int C = 8 * LPR;
  constexpr int RPW = 32 / LPR;
  const int lane = threadIdx.x & 31;
  const int sub = lane / LPR, li = lane % LPR;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  float g[8], b[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    g[j] = gamma != nullptr ? gamma[li * 8 + j] : 1.f;
    b[j] = beta != nullptr ? beta[li * 8 + j] : 0.f;
  }
  for (long long r0 = wid * RPW; r0 < R; r0 += warps * RPW) {
    const long long r = r0 + sub;
    const bool ok = r < R;
    float v[8];
    float sum = 0.f;
    if (ok) {
      const uint4 u = *reinterpret_cast<const uint4*>(x + r * C + li * 8);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[2 * j] = bf16_lo(w[j]);
        v[2 * j + 1] = bf16_hi(w[j]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = 0.f;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) sum += v[j];
#pragma unroll
    for (int s = LPR / 2; s > 0; s >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, s);
    const float mu = sum * (1.0f / C);
    float sq = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) sq += (v[j] - mu) * (v[j] - mu);
#pragma unroll
    for (int s = LPR / 2; s > 0; s >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, s);
    const float rstd = rsqrtf(sq * (1.0f / C) + eps);
    if (ok) {
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        o[j] = pack_bf16x2((v[2 * j] - mu) * rstd * g[2 * j] + b[2 * j],
                           (v[2 * j + 1] - mu) * rstd * g[2 * j + 1] + b[2 * j + 1]);
      *reinterpret_cast<uint4*>(out + r * C + li * 8) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// z rows [R][128] bf16 -> planes out[h][i][j] (bf16, leading dimension Np), LN folded:
//   out = scale_out * (rstd * (w[h] . x - mu * colsum[h]) + colbias[h])
// One thread per row; weights in shared memory (broadcast reads).
template <int H, int RPT>
__global__ void __launch_bounds__(128) pair_head_bias_kernel(const __nv_bfloat16* __restrict__ z,
                                                             const float* __restrict__ w,
                                                             const float* __restrict__ colsum,
                                                             const float* __restrict__ colbias,
                                                             __nv_bfloat16* __restrict__ out, int N, int Np,
                                                             int transpose_out) {
  // Each thread owns RPT consecutive pair rows: a weight vector fetched from shared memory (a broadcast 16-byte
  // load costs four wavefronts) serves RPT rows, which moves the kernel off the shared-memory limit, and the RPT
  // results of a head are consecutive plane elements (one 8-byte store for RPT = 4).
  __shared__ float sw[H * 128];
  for (int i = threadIdx.x; i < H * 128; i += blockDim.x) sw[i] = w[i];
  __syncthreads();
  const long long R = static_cast<long long>(N) * N;
  const long long groups = (R + RPT - 1) / RPT;
  for (long long gq = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; gq < groups;
       gq += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r0 = gq * RPT;
    float acc[RPT][H];
    float sum[RPT], sumsq[RPT];
#pragma unroll
    for (int q = 0; q < RPT; ++q) {
      sum[q] = 0.f;
      sumsq[q] = 0.f;
#pragma unroll
      for (int h = 0; h < H; ++h) acc[q][h] = 0.f;
    }
#pragma unroll 2
    for (int c16 = 0; c16 < 16; ++c16) {
      float e[RPT][8];
#pragma unroll
      for (int q = 0; q < RPT; ++q) {
        const long long r = r0 + q < R ? r0 + q : R - 1;
        const uint4 u = __ldg(reinterpret_cast<const uint4*>(z + r * 128) + c16);
        e[q][0] = bf16_lo(u.x); e[q][1] = bf16_hi(u.x); e[q][2] = bf16_lo(u.y); e[q][3] = bf16_hi(u.y);
        e[q][4] = bf16_lo(u.z); e[q][5] = bf16_hi(u.z); e[q][6] = bf16_lo(u.w); e[q][7] = bf16_hi(u.w);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          sum[q] += e[q][j];
          sumsq[q] = fmaf(e[q][j], e[q][j], sumsq[q]);
        }
      }
#pragma unroll
      for (int h = 0; h < H; ++h) {
        const float4 w0 = *reinterpret_cast<const float4*>(&sw[h * 128 + c16 * 8]);
        const float4 w1 = *reinterpret_cast<const float4*>(&sw[h * 128 + c16 * 8 + 4]);
#pragma unroll
        for (int q = 0; q < RPT; ++q) {
          float a = acc[q][h];
          a = fmaf(e[q][0], w0.x, a); a = fmaf(e[q][1], w0.y, a); a = fmaf(e[q][2], w0.z, a);
          a = fmaf(e[q][3], w0.w, a); a = fmaf(e[q][4], w1.x, a); a = fmaf(e[q][5], w1.y, a);
          a = fmaf(e[q][6], w1.z, a); a = fmaf(e[q][7], w1.w, a);
          acc[q][h] = a;
        }
      }
    }
    float mu[RPT], rstd[RPT];
#pragma unroll
    for (int q = 0; q < RPT; ++q) {
      mu[q] = sum[q] * (1.f / 128.f);
      rstd[q] = rsqrtf(fmaxf(sumsq[q] * (1.f / 128.f) - mu[q] * mu[q], 0.f) + 1e-5f);
    }
    const int i0 = static_cast<int>(r0 / N);
    const int j0 = static_cast<int>(r0 - static_cast<long long>(i0) * N);
    const bool vec = RPT == 4 && !transpose_out && j0 + RPT <= N && ((Np | j0) & 3) == 0;
    if (vec) {
      const long long off = static_cast<long long>(i0) * Np + j0;
#pragma unroll
      for (int h = 0; h < H; ++h) {
        const float cs = colsum[h], cb = colbias[h];
        float v[RPT];
#pragma unroll
        for (int q = 0; q < RPT; ++q) v[q] = fmaf(rstd[q], acc[q][h] - mu[q] * cs, cb);
        *reinterpret_cast<uint2*>(out + static_cast<long long>(h) * N * Np + off) =
            make_uint2(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[RPT - 2], v[RPT - 1]));
      }
    } else {
#pragma unroll
      for (int q = 0; q < RPT; ++q) {
        const long long r = r0 + q;
        if (r < R) {
          const int i = static_cast<int>(r / N);
          const int j = static_cast<int>(r - static_cast<long long>(i) * N);
          const long long off =
              transpose_out ? (static_cast<long long>(j) * Np + i) : (static_cast<long long>(i) * Np + j);
#pragma unroll
          for (int h = 0; h < H; ++h)
            out[static_cast<long long>(h) * N * Np + off] =
                __float2bfloat16(fmaf(rstd[q], acc[q][h] - mu[q] * colsum[h], colbias[h]));
        }
      }
    }
  }
}

// a: [R][C] (bf16), scale/shift: [Rs][C] (bf16) with Rs = R / rows_per_cond (conditioning shared by
// `rows_per_cond`... no: one conditioning row per activation row).  out = sigmoid(scale)*LN(a)+shift.
__global__ void __launch_bounds__(256) adaln_rows_kernel(const __nv_bfloat16* __restrict__ a,
                                                         const __nv_bfloat16* __restrict__ scale,
                                                         const __nv_bfloat16* __restrict__ shift,
                                                         __nv_bfloat16* __restrict__ out, long long R, int C,
                                                         long long cond_rows, long long ld_cond, float eps) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (long long r = static_cast<long long>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5); r < R;
       r += static_cast<long long>(gridDim.x) * warps_per_block) {
    const __nv_bfloat16* ar = a + r * C;
    const long long rc = r % cond_rows;
    float sum = 0.f, sumsq = 0.f;
    for (int c = lane * 2; c < C; c += 64) {
      const __nv_bfloat162 p = *reinterpret_cast<const __nv_bfloat162*>(ar + c);
      const float x0 = __low2float(p), x1 = __high2float(p);
      sum += x0 + x1;
      sumsq += x0 * x0 + x1 * x1;
    }
    sum = warp_sum(sum);
    sumsq = warp_sum(sumsq);
    const float mu = sum / C;
    const float rstd = rsqrtf(fmaxf(sumsq / C - mu * mu, 0.f) + eps);
    for (int c = lane * 2; c < C; c += 64) {
      const __nv_bfloat162 p = *reinterpret_cast<const __nv_bfloat162*>(ar + c);
      const __nv_bfloat162 sc = *reinterpret_cast<const __nv_bfloat162*>(scale + rc * ld_cond + c);
      const __nv_bfloat162 sh = *reinterpret_cast<const __nv_bfloat162*>(shift + rc * ld_cond + c);
      const float y0 = sigmoidf_fast(__low2float(sc)) * ((__low2float(p) - mu) * rstd) + __low2float(sh);
      const float y1 = sigmoidf_fast(__high2float(sc)) * ((__high2float(p) - mu) * rstd) + __high2float(sh);
      *reinterpret_cast<__nv_bfloat162*>(out + r * C + c) = __floats2bfloat162_rn(y0, y1);
    }
  }
}

// The same with 16-byte accesses: a warp per row, the row (up to 1024 channels: four 8-channel chunks per
// lane) stays in registers between the statistics and the output pass, so it is read once.
template <int CHUNKS>
__global__ void __launch_bounds__(256) adaln_rows_vec_kernel(const __nv_bfloat16* __restrict__ a,
                                                             const __nv_bfloat16* __restrict__ scale,
                                                             const __nv_bfloat16* __restrict__ shift,
                                                             __nv_bfloat16* __restrict__ out, long long R, int C,
                                                             long long cond_rows, long long ld_cond, float eps) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (long long r = static_cast<long long>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5); r < R;
       r += static_cast<long long>(gridDim.x) * warps_per_block) {
    const __nv_bfloat16* ar = a + r * C;
    const long long rc = r % cond_rows;
    float x[CHUNKS][8];
    float sum = 0.f, sumsq = 0.f;
#pragma unroll
    for (int k = 0; k < CHUNKS; ++k) {
      const int c = k * 256 + lane * 8;
      if (c < C) {
        const uint4 u = *reinterpret_cast<const uint4*>(ar + c);
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          x[k][2 * j] = bf16_lo(w[j]);
          x[k][2 * j + 1] = bf16_hi(w[j]);
          sum += x[k][2 * j] + x[k][2 * j + 1];
          sumsq += x[k][2 * j] * x[k][2 * j] + x[k][2 * j + 1] * x[k][2 * j + 1];
        }
      }
    }
    sum = warp_sum(sum);
    sumsq = warp_sum(sumsq);
    const float mu = sum / C;
    const float rstd = rsqrtf(fmaxf(sumsq / C - mu * mu, 0.f) + eps);
#pragma unroll
    for (int k = 0; k < CHUNKS; ++k) {
      const int c = k * 256 + lane * 8;
      if (c < C) {
        const uint4 us = __ldg(reinterpret_cast<const uint4*>(scale + rc * ld_cond + c));
        const uint4 uh = __ldg(reinterpret_cast<const uint4*>(shift + rc * ld_cond + c));
        const uint32_t ws[4] = {us.x, us.y, us.z, us.w};
        const uint32_t wh[4] = {uh.x, uh.y, uh.z, uh.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float y0 = sigmoidf_fast(bf16_lo(ws[j])) * ((x[k][2 * j] - mu) * rstd) + bf16_lo(wh[j]);
          const float y1 = sigmoidf_fast(bf16_hi(ws[j])) * ((x[k][2 * j + 1] - mu) * rstd) + bf16_hi(wh[j]);
          o[j] = pack_bf16x2(y0, y1);
        }
        *reinterpret_cast<uint4*>(out + r * C + c) = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  }
}

// Rows of 128 channels (the atom track): half a warp per row, so every lane carries 16 bytes; with a whole warp per
// row half of the lanes sat idle (20.5 us for 63840 rows, 1.6 TB/s).
__global__ void __launch_bounds__(256) adaln_rows_c128_kernel(const __nv_bfloat16* __restrict__ a,
                                                              const __nv_bfloat16* __restrict__ scale,
                                                              const __nv_bfloat16* __restrict__ shift,
                                                              __nv_bfloat16* __restrict__ out, long long R,
                                                              long long cond_rows, long long ld_cond, float eps) {
  constexpr int C = 128;
  const int halves_per_block = blockDim.x >> 4;
  const int l16 = threadIdx.x & 15;
  const int c = l16 * 8;
  for (long long r = static_cast<long long>(blockIdx.x) * halves_per_block + (threadIdx.x >> 4);
       r < ((R + 1) & ~1ll); r += static_cast<long long>(gridDim.x) * halves_per_block) {
    // both halves of a warp run the same number of iterations (R rounded up to even) so the shuffles stay whole
    const bool ok = r < R;
    float x[8];
    float sum = 0.f, sumsq = 0.f;
    if (ok) {
      const uint4 u = *reinterpret_cast<const uint4*>(a + r * C + c);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        x[2 * j] = bf16_lo(w[j]);
        x[2 * j + 1] = bf16_hi(w[j]);
        sum += x[2 * j] + x[2 * j + 1];
        sumsq += x[2 * j] * x[2 * j] + x[2 * j + 1] * x[2 * j + 1];
      }
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) {
      sum += __shfl_xor_sync(0xffffffffu, sum, o);
      sumsq += __shfl_xor_sync(0xffffffffu, sumsq, o);
    }
    if (!ok) continue;
    const float mu = sum * (1.0f / C);
    const float rstd = rsqrtf(fmaxf(sumsq * (1.0f / C) - mu * mu, 0.f) + eps);
    const long long rc = r % cond_rows;
    const uint4 us = __ldg(reinterpret_cast<const uint4*>(scale + rc * ld_cond + c));
    const uint4 uh = __ldg(reinterpret_cast<const uint4*>(shift + rc * ld_cond + c));
    const uint32_t ws[4] = {us.x, us.y, us.z, us.w};
    const uint32_t wh[4] = {uh.x, uh.y, uh.z, uh.w};
    uint32_t o4[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float y0 = sigmoidf_fast(bf16_lo(ws[j])) * ((x[2 * j] - mu) * rstd) + bf16_lo(wh[j]);
      const float y1 = sigmoidf_fast(bf16_hi(ws[j])) * ((x[2 * j + 1] - mu) * rstd) + bf16_hi(wh[j]);
      o4[j] = pack_bf16x2(y0, y1);
    }
    *reinterpret_cast<uint4*>(out + r * C + c) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
  }
}

// out = res + sigmoid(gate[r % cond_rows]) * x   (res may be null)
__global__ void __launch_bounds__(256) gate_residual_kernel(const __nv_bfloat16* __restrict__ x,
                                                            const __nv_bfloat16* __restrict__ gate,
                                                            const __nv_bfloat16* __restrict__ res,
                                                            __nv_bfloat16* __restrict__ out, long long n2, int C2,
                                                            long long cond_rows, long long ld_gate2) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n2;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / C2;
    const int c = static_cast<int>(i - r * C2);
    const long long gi = (r % cond_rows) * ld_gate2 + c;
    const __nv_bfloat162 xv = reinterpret_cast<const __nv_bfloat162*>(x)[i];
    const __nv_bfloat162 gv = reinterpret_cast<const __nv_bfloat162*>(gate)[gi];
    float y0 = sigmoidf_fast(__low2float(gv)) * __low2float(xv);
    float y1 = sigmoidf_fast(__high2float(gv)) * __high2float(xv);
    if (res != nullptr) {
      const __nv_bfloat162 rv = reinterpret_cast<const __nv_bfloat162*>(res)[i];
      y0 += __low2float(rv);
      y1 += __high2float(rv);
    }
    reinterpret_cast<__nv_bfloat162*>(out)[i] = __floats2bfloat162_rn(y0, y1);
  }
}

// ab: [R][2*Hd] -> out [R][Hd] = silu(ab[:, :Hd]) * ab[:, Hd:]
__global__ void __launch_bounds__(256) swiglu_rows_kernel(const __nv_bfloat16* __restrict__ ab,
                                                          __nv_bfloat16* __restrict__ out, long long R, int Hd) {
  const int h2 = Hd >> 1;
  const long long n2 = R * h2;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n2;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / h2;
    const int c = static_cast<int>(i - r * h2);
    const __nv_bfloat162 av = reinterpret_cast<const __nv_bfloat162*>(ab + r * 2 * Hd)[c];
    const __nv_bfloat162 bv = reinterpret_cast<const __nv_bfloat162*>(ab + r * 2 * Hd + Hd)[c];
    reinterpret_cast<__nv_bfloat162*>(out + r * Hd)[c] =
        __floats2bfloat162_rn(siluf_fast(__low2float(av)) * __low2float(bv),
                              siluf_fast(__high2float(av)) * __high2float(bv));
  }
}

// x: [R][3*Hd] = [u | g | w] -> out [R][Hd] = silu(u) * g * w   (16-byte accesses; Hd a multiple of 8)
__global__ void __launch_bounds__(256) swiglu3_rows_kernel(const __nv_bfloat16* __restrict__ x,
                                                           __nv_bfloat16* __restrict__ out, long long R, int Hd) {
  const int h8 = Hd >> 3;
  const long long n8 = R * h8;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / h8;
    const int c = static_cast<int>(i - r * h8) * 8;
    const __nv_bfloat16* row = x + r * 3 * Hd;
    const uint4 uu = *reinterpret_cast<const uint4*>(row + c);
    const uint4 ug = *reinterpret_cast<const uint4*>(row + Hd + c);
    const uint4 uw = *reinterpret_cast<const uint4*>(row + 2 * Hd + c);
    const uint32_t a[4] = {uu.x, uu.y, uu.z, uu.w}, g[4] = {ug.x, ug.y, ug.z, ug.w}, w[4] = {uw.x, uw.y, uw.z, uw.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      o[j] = pack_bf16x2(siluf_fast(bf16_lo(a[j])) * bf16_lo(g[j]) * bf16_lo(w[j]),
                         siluf_fast(bf16_hi(a[j])) * bf16_hi(g[j]) * bf16_hi(w[j]));
    *reinterpret_cast<uint4*>(out + r * Hd + c) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

static inline int grid_for(long long work, int per_block) {
  long long b = (work + per_block - 1) / per_block;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}

}  // namespace ubm

// in_dtype / out_dtype: 0 = bf16, 1 = fp32.  gamma / beta: fp32 [C] or null.  C <= 1024.
extern "C" int ubm_layernorm_rows(const void* x, const void* gamma, const void* beta, void* out, long long R, int C,
                                  float eps, int in_dtype, int out_dtype, void* stream) {
  using namespace ubm;
  if (R <= 0 || C <= 0) return UBM_ERR_ARGUMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (in_dtype == 0 && out_dtype == 0 && C > 256 && C <= 2048 && (C & 7) == 0 &&
      ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
    const __nv_bfloat16* xx = static_cast<const __nv_bfloat16*>(x);
    __nv_bfloat16* oo = static_cast<__nv_bfloat16*>(out);
    const float* gg = static_cast<const float*>(gamma);
    const float* bb = static_cast<const float*>(beta);
    const int gridw = grid_for(R, 8);
    if (C <= 512) layernorm_rows_wide_kernel<2><<<gridw, 256, 0, st>>>(xx, gg, bb, oo, R, C, eps);
    else if (C <= 1024) layernorm_rows_wide_kernel<4><<<gridw, 256, 0, st>>>(xx, gg, bb, oo, R, C, eps);
    else layernorm_rows_wide_kernel<8><<<gridw, 256, 0, st>>>(xx, gg, bb, oo, R, C, eps);
    UBM_CHECK_LAUNCH("layernorm_rows_wide_kernel");
    return UBM_OK;
  }
  if (C > 1024) return UBM_ERR_ARGUMENT;
  if (in_dtype == 0 && out_dtype == 0 && (C == 64 || C == 128 || C == 256) &&
      ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
    const __nv_bfloat16* xx = static_cast<const __nv_bfloat16*>(x);
    __nv_bfloat16* oo = static_cast<__nv_bfloat16*>(out);
    const float* gg = static_cast<const float*>(gamma);
    const float* bb = static_cast<const float*>(beta);
    const int rows_per_block = 8 * (256 / C);
    const int grid2 = grid_for(R, rows_per_block);
    if (C == 64) layernorm_rows_narrow_kernel<8><<<grid2, 256, 0, st>>>(xx, gg, bb, oo, R, eps);
    else if (C == 128) layernorm_rows_narrow_kernel<16><<<grid2, 256, 0, st>>>(xx, gg, bb, oo, R, eps);
    else layernorm_rows_narrow_kernel<32><<<grid2, 256, 0, st>>>(xx, gg, bb, oo, R, eps);
    UBM_CHECK_LAUNCH("layernorm_rows_narrow_kernel");
    return UBM_OK;
  }
  const int grid = grid_for(R, 8);
  const float* g = static_cast<const float*>(gamma);
  const float* b = static_cast<const float*>(beta);
#define UBM_LN_LAUNCH(TI, TO, MP)                                                                          \
  layernorm_rows_kernel<TI, TO, MP><<<grid, 256, 0, st>>>(static_cast<const TI*>(x), g, b, static_cast<TO*>(out), R, \
                                                          C, eps)
#define UBM_LN_BY_WIDTH(TI, TO)      \
  do {                               \
    if (C <= 128) {                  \
      UBM_LN_LAUNCH(TI, TO, 4);      \
    } else if (C <= 256) {           \
      UBM_LN_LAUNCH(TI, TO, 8);      \
    } else if (C <= 512) {           \
      UBM_LN_LAUNCH(TI, TO, 16);     \
    } else {                         \
      UBM_LN_LAUNCH(TI, TO, 32);     \
    }                                \
  } while (0)
  if (in_dtype == 0 && out_dtype == 0) UBM_LN_BY_WIDTH(__nv_bfloat16, __nv_bfloat16);
  else if (in_dtype == 0 && out_dtype == 1) UBM_LN_BY_WIDTH(__nv_bfloat16, float);
  else if (in_dtype == 1 && out_dtype == 0) UBM_LN_BY_WIDTH(float, __nv_bfloat16);
  else UBM_LN_BY_WIDTH(float, float);
#undef UBM_LN_BY_WIDTH
#undef UBM_LN_LAUNCH
  UBM_CHECK_LAUNCH("layernorm_rows_kernel");
  return UBM_OK;
}

extern "C" int ubm_pair_head_bias(const void* z, const void* w, const void* colsum, const void* colbias, void* out,
                                  int N, int Np, int H, int transpose_out, void* stream) {
  using namespace ubm;
  if (N <= 0 || Np < N) return UBM_ERR_ARGUMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = grid_for((static_cast<long long>(N) * N + 1) / 2, 128);     // 2 or 4 rows per thread
  const __nv_bfloat16* zz = static_cast<const __nv_bfloat16*>(z);
  const float* ww = static_cast<const float*>(w);
  const float* cs = static_cast<const float*>(colsum);
  const float* cb = static_cast<const float*>(colbias);
  __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out);
  switch (H) {
    case 4: pair_head_bias_kernel<4, 4><<<grid, 128, 0, st>>>(zz, ww, cs, cb, o, N, Np, transpose_out); break;
    case 8: pair_head_bias_kernel<8, 4><<<grid, 128, 0, st>>>(zz, ww, cs, cb, o, N, Np, transpose_out); break;
    case 16: pair_head_bias_kernel<16, 4><<<grid, 128, 0, st>>>(zz, ww, cs, cb, o, N, Np, transpose_out); break;
    case 32: pair_head_bias_kernel<32, 2><<<grid, 128, 0, st>>>(zz, ww, cs, cb, o, N, Np, transpose_out); break;
    default: return UBM_ERR_ARGUMENT;
  }
  UBM_CHECK_LAUNCH("pair_head_bias_kernel");
  return UBM_OK;
}

// scale / shift: bf16 rows of leading dimension ld_cond (elements), reused cyclically every cond_rows rows.
extern "C" int ubm_adaln_rows(const void* a, const void* scale, const void* shift, void* out, long long R, int C,
                              long long cond_rows, long long ld_cond, float eps, void* stream) {
  using namespace ubm;
  if (R <= 0 || C <= 0 || (C & 1) || cond_rows <= 0 || ld_cond < C) return UBM_ERR_ARGUMENT;
  const __nv_bfloat16* aa = static_cast<const __nv_bfloat16*>(a);
  const __nv_bfloat16* sc = static_cast<const __nv_bfloat16*>(scale);
  const __nv_bfloat16* sh = static_cast<const __nv_bfloat16*>(shift);
  __nv_bfloat16* oo = static_cast<__nv_bfloat16*>(out);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool vec = (C % 8) == 0 && C <= 1024 && (ld_cond % 8) == 0 &&
                   ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(scale) |
                     reinterpret_cast<uintptr_t>(shift) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  const int grid = grid_for(R, 8);
  if (vec && C == 128) {
    adaln_rows_c128_kernel<<<grid_for((R + 1) / 2 * 2, 16), 256, 0, st>>>(aa, sc, sh, oo, R, cond_rows, ld_cond, eps);
  } else if (vec && C <= 256) {
    adaln_rows_vec_kernel<1><<<grid, 256, 0, st>>>(aa, sc, sh, oo, R, C, cond_rows, ld_cond, eps);
  } else if (vec && C <= 512) {
    adaln_rows_vec_kernel<2><<<grid, 256, 0, st>>>(aa, sc, sh, oo, R, C, cond_rows, ld_cond, eps);
  } else if (vec && C <= 768) {
    adaln_rows_vec_kernel<3><<<grid, 256, 0, st>>>(aa, sc, sh, oo, R, C, cond_rows, ld_cond, eps);
  } else if (vec) {
    adaln_rows_vec_kernel<4><<<grid, 256, 0, st>>>(aa, sc, sh, oo, R, C, cond_rows, ld_cond, eps);
  } else {
    adaln_rows_kernel<<<grid, 256, 0, st>>>(aa, sc, sh, oo, R, C, cond_rows, ld_cond, eps);
  }
  UBM_CHECK_LAUNCH("adaln_rows_kernel");
  return UBM_OK;
}

extern "C" int ubm_gate_residual(const void* x, const void* gate, const void* res, void* out, long long R, int C,
                                 long long cond_rows, long long ld_gate, void* stream) {
  using namespace ubm;
  if (R <= 0 || C <= 0 || (C & 1) || cond_rows <= 0 || ld_gate < C || (ld_gate & 1)) return UBM_ERR_ARGUMENT;
  const long long n2 = R * (C / 2);
  gate_residual_kernel<<<grid_for(n2, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(gate),
      static_cast<const __nv_bfloat16*>(res), static_cast<__nv_bfloat16*>(out), n2, C / 2, cond_rows, ld_gate / 2);
  UBM_CHECK_LAUNCH("gate_residual_kernel");
  return UBM_OK;
}

extern "C" int ubm_swiglu3_rows(const void* x, void* out, long long R, int Hd, void* stream) {
  using namespace ubm;
  if (R <= 0 || Hd <= 0 || (Hd & 7) ||
      ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15))
    return UBM_ERR_ARGUMENT;
  swiglu3_rows_kernel<<<grid_for(R * (Hd / 8), 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(out), R, Hd);
  UBM_CHECK_LAUNCH("swiglu3_rows_kernel");
  return UBM_OK;
}

extern "C" int ubm_swiglu_rows(const void* ab, void* out, long long R, int Hd, void* stream) {
  using namespace ubm;
  if (R <= 0 || Hd <= 0 || (Hd & 1)) return UBM_ERR_ARGUMENT;
  swiglu_rows_kernel<<<grid_for(R * (Hd / 2), 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(ab), static_cast<__nv_bfloat16*>(out), R, Hd);
  UBM_CHECK_LAUNCH("swiglu_rows_kernel");
  return UBM_OK;
}
