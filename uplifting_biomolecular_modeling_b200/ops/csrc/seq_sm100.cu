// Row and sequence kernels for the language-model and genomics families (StripedHyena-2 / Evo2, ProGen2, ESM-C,
// Enformer-style towers).  All are memory bound: bf16 (or fp32) rows in, fp32 arithmetic, 16-byte accesses, one
// pass over the data, the neighbouring elementwise steps folded in.
//
//   rmsnorm_rows          y = x * rsqrt(mean(x^2) + eps) * scale                       (Evo2 pre/post norm)
//   fir_gate3             zf = causal_fir3..8(z) over [B, L, 3d]; u = zf_1 * zf_3, x2 = zf_2   (Hyena input stage)
//   fir_inner_gate        out = x2 * (causal_fir(u, h) + D * u)                         (hcs / hcm operators)
//   fftconv_epilogue      out = x2 * (y[b][c][l] + D * u) with y channel-major fp32     (after the inverse FFT)
//   pole_step             s = s * lam + u; out = x2 * (sum_s s * res + D * u)           (hcl decode step)
//   gelu_new, residual_add2, bias_residual, scale_shift_gelu, rotary_split_qkv, add2_softmax_rows, pool2,
//   residual_ln           exact-order elementwise sets of the LM / genomics kits
//
// Reference kernels with the same boundaries: the evo2 Triton set (FIR, RMSNorm tail, FFT-conv epilogue,
// decode-step state), progen2 kits/v0_ew/kernels.cu:37-209 (gelu_new, rotary_split_qkv, residual_add2),
// esmc kits/residual_ln/kernels.cu:28-127, enformer kits/v0_2/enformer_xattn.cu:24-99 (add2 softmax) and
// enformer_fastkit.py:96-157 (bn_gelu, pool, bias_residual).
#include <cuda_fp8.h>

#include "host_util.h"
#include "sm100.cuh"

namespace ubm {

static inline int seq_grid(long long work, int per_block) {
  long long b = (work + per_block - 1) / per_block;
  const long long cap = static_cast<long long>(sm_count()) * 32;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}

__device__ __forceinline__ void unpack8(const uint4& u, float (&e)[8]) {
  e[0] = bf16_lo(u.x); e[1] = bf16_hi(u.x); e[2] = bf16_lo(u.y); e[3] = bf16_hi(u.y);
  e[4] = bf16_lo(u.z); e[5] = bf16_hi(u.z); e[6] = bf16_lo(u.w); e[7] = bf16_hi(u.w);
}
__device__ __forceinline__ uint4 pack8(const float (&e)[8]) {
  return make_uint4(pack_bf16x2(e[0], e[1]), pack_bf16x2(e[2], e[3]), pack_bf16x2(e[4], e[5]),
                    pack_bf16x2(e[6], e[7]));
}

// ------------------------------------------------------------------------------------------ RMSNorm
// one warp per row, the row read once (kept in registers for C <= 8192: up to 32 chunks of 8 per lane)
template <int CHUNKS>
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(const __nv_bfloat16* __restrict__ x,
                                                           const float* __restrict__ scale,
                                                           __nv_bfloat16* __restrict__ out, long long R, int C,
                                                           float eps) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (long long r = static_cast<long long>(blockIdx.x) * wpb + (threadIdx.x >> 5); r < R;
       r += static_cast<long long>(gridDim.x) * wpb) {
    // the row stays packed (16 registers per 128 values): three CTAs per SM keep their loads in flight
    uint4 raw[CHUNKS];
#pragma unroll
    for (int k = 0; k < CHUNKS; ++k) {
      const int c = k * 256 + lane * 8;
      if (c < C) raw[k] = *reinterpret_cast<const uint4*>(x + r * C + c);
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < CHUNKS; ++k) {
      const int c = k * 256 + lane * 8;
      if (c < C) {
        float v[8];
        unpack8(raw[k], v);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += v[j] * v[j];
      }
    }
    ss = warp_sum(ss);
    const float rs = rsqrtf(ss / C + eps);
#pragma unroll
    for (int k = 0; k < CHUNKS; ++k) {
      const int c = k * 256 + lane * 8;
      if (c < C) {
        const float4 s0 = __ldg(reinterpret_cast<const float4*>(scale + c));
        const float4 s1 = __ldg(reinterpret_cast<const float4*>(scale + c + 4));
        const float sc[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
        float v[8], o[8];
        unpack8(raw[k], v);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = v[j] * rs * sc[j];
        *reinterpret_cast<uint4*>(out + r * C + c) = pack8(o);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------ RMSNorm -> e4m3
// The normalised rows as 8-bit floats for an fp8 projection, scaled by the tensor's own maximum ("current
// scaling": no state is carried between calls).  Two launches: the first takes max |y| over the tensor
// (y = x * rsqrt(mean(x^2) + eps) * scale, the bits of a non-negative float order as integers), the second
// writes e4m3(y * 448 / max) and the dequantisation factor max / 448 for the projection's epilogue.
template <int CHUNKS, bool EMIT>
__global__ void __launch_bounds__(256) rmsnorm_fp8_kernel(const __nv_bfloat16* __restrict__ x,
                                                          const float* __restrict__ scale,
                                                          unsigned int* __restrict__ amax_bits,
                                                          uint8_t* __restrict__ out, float* __restrict__ dequant,
                                                          long long R, int C, float eps) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  float q = 0.f;
  if (EMIT) {
    const float amax = fmaxf(__uint_as_float(*amax_bits), 1e-12f);
    q = 448.0f / amax;
    if (blockIdx.x == 0 && threadIdx.x == 0) *dequant = amax / 448.0f;
  }
  float vmax = 0.f;
  for (long long r = static_cast<long long>(blockIdx.x) * wpb + (threadIdx.x >> 5); r < R;
       r += static_cast<long long>(gridDim.x) * wpb) {
    uint4 raw[CHUNKS];
#pragma unroll
    for (int k = 0; k < CHUNKS; ++k) {
      const int c = k * 256 + lane * 8;
      if (c < C) raw[k] = *reinterpret_cast<const uint4*>(x + r * C + c);
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < CHUNKS; ++k) {
      const int c = k * 256 + lane * 8;
      if (c < C) {
        float v[8];
        unpack8(raw[k], v);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += v[j] * v[j];
      }
    }
    ss = warp_sum(ss);
    const float rs = rsqrtf(ss / C + eps);
#pragma unroll
    for (int k = 0; k < CHUNKS; ++k) {
      const int c = k * 256 + lane * 8;
      if (c < C) {
        const float4 s0 = __ldg(reinterpret_cast<const float4*>(scale + c));
        const float4 s1 = __ldg(reinterpret_cast<const float4*>(scale + c + 4));
        const float sc[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
        float v[8], y[8];
        unpack8(raw[k], v);
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] = v[j] * rs * sc[j];
        if (EMIT) {
          uint2 o;
          o.x = static_cast<unsigned int>(__nv_cvt_float2_to_fp8x2(make_float2(y[0] * q, y[1] * q), __NV_SATFINITE, __NV_E4M3)) |
                (static_cast<unsigned int>(__nv_cvt_float2_to_fp8x2(make_float2(y[2] * q, y[3] * q), __NV_SATFINITE, __NV_E4M3)) << 16);
          o.y = static_cast<unsigned int>(__nv_cvt_float2_to_fp8x2(make_float2(y[4] * q, y[5] * q), __NV_SATFINITE, __NV_E4M3)) |
                (static_cast<unsigned int>(__nv_cvt_float2_to_fp8x2(make_float2(y[6] * q, y[7] * q), __NV_SATFINITE, __NV_E4M3)) << 16);
          *reinterpret_cast<uint2*>(out + r * C + c) = o;
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) vmax = fmaxf(vmax, fabsf(y[j]));
        }
      }
    }
  }
  if (!EMIT) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, o));
    if (lane == 0) atomicMax(amax_bits, __float_as_uint(vmax));
  }
}

// rows wider than 4096 channels: two passes over the row (the second one hits L1/L2)
__global__ void __launch_bounds__(256) rmsnorm_rows_wide_kernel(const __nv_bfloat16* __restrict__ x,
                                                                const float* __restrict__ scale,
                                                                __nv_bfloat16* __restrict__ out, long long R, int C,
                                                                float eps) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (long long r = static_cast<long long>(blockIdx.x) * wpb + (threadIdx.x >> 5); r < R;
       r += static_cast<long long>(gridDim.x) * wpb) {
    float ss = 0.f;
    for (int c = lane * 8; c < C; c += 256) {
      float v[8];
      unpack8(*reinterpret_cast<const uint4*>(x + r * C + c), v);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[j] * v[j];
    }
    ss = warp_sum(ss);
    const float rs = rsqrtf(ss / C + eps);
    for (int c = lane * 8; c < C; c += 256) {
      float v[8], o[8];
      unpack8(*reinterpret_cast<const uint4*>(x + r * C + c), v);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = v[j] * rs * scale[c + j];
      *reinterpret_cast<uint4*>(out + r * C + c) = pack8(o);
    }
  }
}

// ------------------------------------------------------------------------------------------ causal FIR
// Depthwise causal FIR over [B][L][C] with taps ht[k][c] (k = 0 multiplies the current sample).  A thread owns 8
// channels and walks TL consecutive positions with the K-1 previous samples in registers, so each input element
// is read once (plus K-1 per run of TL).  tail: [B][K-1][C] samples before position 0, or null (zeros).
template <int K>
struct FirWindow {
  float h[K][8];
  float w[K - 1][8];   // w[j] = sample at distance j+1 behind the current one
  __device__ __forceinline__ void load_taps(const float* __restrict__ ht, int C, int c) {
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const float4 a = __ldg(reinterpret_cast<const float4*>(ht + static_cast<long long>(k) * C + c));
      const float4 b = __ldg(reinterpret_cast<const float4*>(ht + static_cast<long long>(k) * C + c + 4));
      h[k][0] = a.x; h[k][1] = a.y; h[k][2] = a.z; h[k][3] = a.w;
      h[k][4] = b.x; h[k][5] = b.y; h[k][6] = b.z; h[k][7] = b.w;
    }
  }
  __device__ __forceinline__ void prime(const __nv_bfloat16* __restrict__ xb, const __nv_bfloat16* __restrict__ tb,
                                        int l0, int C, int c) {
#pragma unroll
    for (int j = 0; j < K - 1; ++j) {
      const int l = l0 - 1 - j;
      if (l >= 0) {
        unpack8(*reinterpret_cast<const uint4*>(xb + static_cast<long long>(l) * C + c), w[j]);
      } else if (tb != nullptr) {
        unpack8(*reinterpret_cast<const uint4*>(tb + static_cast<long long>(K - 1 + l) * C + c), w[j]);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) w[j][e] = 0.f;
      }
    }
  }
  __device__ __forceinline__ void step(const float (&cur)[8], float (&y)[8]) {
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float a = h[0][e] * cur[e];
#pragma unroll
      for (int j = 0; j < K - 1; ++j) a = fmaf(h[j + 1][e], w[j][e], a);
      y[e] = a;
    }
#pragma unroll
    for (int j = K - 2; j > 0; --j)
#pragma unroll
      for (int e = 0; e < 8; ++e) w[j][e] = w[j - 1][e];
    if (K > 1) {
#pragma unroll
      for (int e = 0; e < 8; ++e) w[0][e] = cur[e];
    }
  }
};

constexpr int kFirTL = 32;   // positions per thread run

// Hyena input stage: z [B][L][3d] -> zf = fir(z) per channel; u = zf[0:d] * zf[2d:3d], x2 = zf[d:2d].
template <int K>
__global__ void __launch_bounds__(128) fir_gate3_kernel(const __nv_bfloat16* __restrict__ z,
                                                        const float* __restrict__ ht,     // [K][3d]
                                                        __nv_bfloat16* tail,  // [B][K-1][3d] or null
                                                        __nv_bfloat16* __restrict__ u, __nv_bfloat16* __restrict__ x2,
                                                        int B, int L, int d, int push) {
  const int c8 = d / 8;
  const int runs = (L + kFirTL - 1) / kFirTL;
  const long long total = static_cast<long long>(B) * runs * c8;
  const int C = 3 * d;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int cc = static_cast<int>(i % c8) * 8;
    const long long br = i / c8;
    const int run = static_cast<int>(br % runs);
    const int b = static_cast<int>(br / runs);
    const __nv_bfloat16* zb = z + static_cast<long long>(b) * L * C;
    __nv_bfloat16* tb = tail == nullptr ? nullptr : tail + static_cast<long long>(b) * (K - 1) * C;
    FirWindow<K> f1, f2, f3;
    f1.load_taps(ht, C, cc);
    f2.load_taps(ht, C, d + cc);
    f3.load_taps(ht, C, 2 * d + cc);
    const int l0 = run * kFirTL;
    f1.prime(zb, tb, l0, C, cc);
    f2.prime(zb, tb, l0, C, d + cc);
    f3.prime(zb, tb, l0, C, 2 * d + cc);
    const int l1 = min(L, l0 + kFirTL);
    for (int l = l0; l < l1; ++l) {
      float a[8], bb[8], cv[8], y1[8], y2[8], y3[8];
      const __nv_bfloat16* row = zb + static_cast<long long>(l) * C;
      unpack8(*reinterpret_cast<const uint4*>(row + cc), a);
      unpack8(*reinterpret_cast<const uint4*>(row + d + cc), bb);
      unpack8(*reinterpret_cast<const uint4*>(row + 2 * d + cc), cv);
      f1.step(a, y1);
      f2.step(bb, y2);
      f3.step(cv, y3);
      // the plain statement rounds zf to the activation type before the gate product
      float uo[8], xo[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        uo[e] = __bfloat162float(__float2bfloat16(y1[e])) * __bfloat162float(__float2bfloat16(y3[e]));
        xo[e] = y2[e];
      }
      const long long o = (static_cast<long long>(b) * L + l) * d + cc;
      *reinterpret_cast<uint4*>(u + o) = pack8(uo);
      *reinterpret_cast<uint4*>(x2 + o) = pack8(xo);
    }
    // decode (one run per row of the batch): the tail is moved on in place - after the last step w[j] is the
    // sample j + 1 positions behind the next one, i.e. row K - 2 - j of the new tail.  This thread is the only
    // one that touches these channels of the tail.
    if (push && K > 1) {
#pragma unroll
      for (int j = 0; j < K - 1; ++j) {
        __nv_bfloat16* row = tb + static_cast<long long>(K - 2 - j) * C;
        *reinterpret_cast<uint4*>(row + cc) = pack8(f1.w[j]);
        *reinterpret_cast<uint4*>(row + d + cc) = pack8(f2.w[j]);
        *reinterpret_cast<uint4*>(row + 2 * d + cc) = pack8(f3.w[j]);
      }
    }
  }
}

// Inner operator of hcs / hcm for ONE new position per row of the batch (decode), with the tail moved on in
// place: out = x2 * (sum_k h[k] s[-k] + D u), s[0] = u, s[-k] = tail[K - 1 - k]; then tail <- (tail[1:], u).
// A CTA owns 64 channels (one 128-byte line of every row); 32 thread rows split the taps, partial sums meet in
// shared memory; every tail row is read into registers before the barrier and written one row up after it.
constexpr int kFirStepMaxTapsPerThread = 8;   // K <= 256

__global__ void __launch_bounds__(256) fir_step_kernel(const __nv_bfloat16* __restrict__ u,     // [B][d]
                                                       const float* __restrict__ ht, int K,     // [K][d]
                                                       const float* __restrict__ D,
                                                       const __nv_bfloat16* __restrict__ x2,    // [B][d] or null
                                                       __nv_bfloat16* tail,                     // [B][K-1][d]
                                                       __nv_bfloat16* __restrict__ out, int d) {
  __shared__ float part[32][8][8];
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the projection behind may prefetch its weights
  const int cg = threadIdx.x & 7;
  const int rg = threadIdx.x >> 3;
  const int b = blockIdx.y;
  const int cc = (blockIdx.x * 8 + cg) * 8;
  const bool live = cc < d;
  __nv_bfloat16* tb = tail + static_cast<long long>(b) * (K - 1) * d;
  uint4 held[kFirStepMaxTapsPerThread];
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (live) {
#pragma unroll
    for (int t = 0; t < kFirStepMaxTapsPerThread; ++t) {
      const int k = rg + 32 * t;
      if (k < K)
        held[t] = k == 0 ? *reinterpret_cast<const uint4*>(u + static_cast<long long>(b) * d + cc)
                         : *reinterpret_cast<const uint4*>(tb + static_cast<long long>(K - 1 - k) * d + cc);
    }
#pragma unroll
    for (int t = 0; t < kFirStepMaxTapsPerThread; ++t) {
      const int k = rg + 32 * t;
      if (k < K) {
        float xv[8];
        unpack8(held[t], xv);
        const float4 h0 = __ldg(reinterpret_cast<const float4*>(ht + static_cast<long long>(k) * d + cc));
        const float4 h1 = __ldg(reinterpret_cast<const float4*>(ht + static_cast<long long>(k) * d + cc + 4));
        const float hv[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = fmaf(hv[e], xv[e], acc[e]);
      }
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) part[rg][cg][e] = acc[e];
  __syncthreads();                                       // every tail row of these channels is in registers
  if (live) {
#pragma unroll
    for (int t = 0; t < kFirStepMaxTapsPerThread; ++t) {
      const int k = rg + 32 * t;                         // the sample k behind becomes the sample k + 1 behind
      if (k < K - 1) *reinterpret_cast<uint4*>(tb + static_cast<long long>(K - 2 - k) * d + cc) = held[t];
    }
    if (rg == 0) {
      float cur[8], g[8];
      unpack8(held[0], cur);
      float sum[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) sum[e] = 0.f;
      for (int r = 0; r < 32; ++r)
#pragma unroll
        for (int e = 0; e < 8; ++e) sum[e] += part[r][cg][e];
      const long long o = static_cast<long long>(b) * d + cc;
      if (x2 != nullptr) {
        unpack8(*reinterpret_cast<const uint4*>(x2 + o), g);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) g[e] = 1.f;
      }
      const float4 d0 = __ldg(reinterpret_cast<const float4*>(D + cc));
      const float4 d1 = __ldg(reinterpret_cast<const float4*>(D + cc + 4));
      const float dv[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
      float r8[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float conv = __bfloat162float(__float2bfloat16(sum[e]));
        r8[e] = g[e] * __bfloat162float(__float2bfloat16(conv + cur[e] * dv[e]));
      }
      *reinterpret_cast<uint4*>(out + o) = pack8(r8);
    }
  }
}

// Inner operator of hcs / hcm: out = x2 * (fir(u, h) + D * u).  Short filters keep the window in registers;
// longer ones (the 128-tap medium filter) re-read the inputs through L1/L2 (generic kernel below).
template <int K>
__global__ void __launch_bounds__(128) fir_inner_gate_kernel(const __nv_bfloat16* __restrict__ u,
                                                             const float* __restrict__ ht,   // [K][d]
                                                             const float* __restrict__ D,
                                                             const __nv_bfloat16* __restrict__ x2,   // or null
                                                             const __nv_bfloat16* __restrict__ tail, // [B][K-1][d]
                                                             __nv_bfloat16* __restrict__ out, int B, int L, int d) {
  const int c8 = d / 8;
  const int runs = (L + kFirTL - 1) / kFirTL;
  const long long total = static_cast<long long>(B) * runs * c8;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int cc = static_cast<int>(i % c8) * 8;
    const long long br = i / c8;
    const int run = static_cast<int>(br % runs);
    const int b = static_cast<int>(br / runs);
    const __nv_bfloat16* ub = u + static_cast<long long>(b) * L * d;
    const __nv_bfloat16* tb = tail == nullptr ? nullptr : tail + static_cast<long long>(b) * (K - 1) * d;
    FirWindow<K> f;
    f.load_taps(ht, d, cc);
    const int l0 = run * kFirTL;
    f.prime(ub, tb, l0, d, cc);
    const float4 d0 = __ldg(reinterpret_cast<const float4*>(D + cc));
    const float4 d1 = __ldg(reinterpret_cast<const float4*>(D + cc + 4));
    const float dv[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
    const int l1 = min(L, l0 + kFirTL);
    for (int l = l0; l < l1; ++l) {
      float cur[8], y[8], g[8];
      const long long o = (static_cast<long long>(b) * L + l) * d + cc;
      unpack8(*reinterpret_cast<const uint4*>(u + o), cur);
      f.step(cur, y);
      if (x2 != nullptr) {
        unpack8(*reinterpret_cast<const uint4*>(x2 + o), g);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) g[e] = 1.f;
      }
      float r[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float conv = __bfloat162float(__float2bfloat16(y[e]));     // the plain statement's bf16 conv output
        r[e] = g[e] * __bfloat162float(__float2bfloat16(conv + cur[e] * dv[e]));
      }
      *reinterpret_cast<uint4*>(out + o) = pack8(r);
    }
  }
}

__global__ void __launch_bounds__(128) fir_inner_gate_long_kernel(const __nv_bfloat16* __restrict__ u,
                                                                  const float* __restrict__ ht, int K,
                                                                  const float* __restrict__ D,
                                                                  const __nv_bfloat16* __restrict__ x2,
                                                                  const __nv_bfloat16* __restrict__ tail,
                                                                  __nv_bfloat16* __restrict__ out, int B, int L,
                                                                  int d) {
  const int c8 = d / 8;
  const long long total = static_cast<long long>(B) * L * c8;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int cc = static_cast<int>(i % c8) * 8;
    const long long bl = i / c8;
    const int l = static_cast<int>(bl % L);
    const int b = static_cast<int>(bl / L);
    const __nv_bfloat16* ub = u + static_cast<long long>(b) * L * d;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float cur[8];
    for (int k = 0; k < K; ++k) {
      const int ls = l - k;
      float xv[8];
      if (ls >= 0) {
        unpack8(*reinterpret_cast<const uint4*>(ub + static_cast<long long>(ls) * d + cc), xv);
      } else if (tail != nullptr) {
        unpack8(*reinterpret_cast<const uint4*>(tail + (static_cast<long long>(b) * (K - 1) + (K - 1 + ls)) * d + cc),
                xv);
      } else {
        break;   // everything further back is zero
      }
      if (k == 0) {
#pragma unroll
        for (int e = 0; e < 8; ++e) cur[e] = xv[e];
      }
      const float4 h0 = __ldg(reinterpret_cast<const float4*>(ht + static_cast<long long>(k) * d + cc));
      const float4 h1 = __ldg(reinterpret_cast<const float4*>(ht + static_cast<long long>(k) * d + cc + 4));
      const float hv[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = fmaf(hv[e], xv[e], acc[e]);
    }
    const long long o = (static_cast<long long>(b) * L + l) * d + cc;
    float g[8];
    if (x2 != nullptr) {
      unpack8(*reinterpret_cast<const uint4*>(x2 + o), g);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) g[e] = 1.f;
    }
    const float4 d0 = __ldg(reinterpret_cast<const float4*>(D + cc));
    const float4 d1 = __ldg(reinterpret_cast<const float4*>(D + cc + 4));
    const float dv[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
    float r[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float conv = __bfloat162float(__float2bfloat16(acc[e]));
      r[e] = g[e] * __bfloat162float(__float2bfloat16(conv + cur[e] * dv[e]));
    }
    *reinterpret_cast<uint4*>(out + o) = pack8(r);
  }
}

// The same operator for filters of tens to hundreds of taps over a long sequence (the 128-tap medium filter of a
// prefill), as a direct convolution on the FMA pipes: 17 G multiply-adds per operator at the 7B shape, against
// three FFT-sized passes over fp32 copies of the sequence.  A CTA owns 32 channels x 512 positions: the input
// tile with its halo (bf16) and the taps (fp32, zero-padded to a multiple of 16) sit in shared memory; a thread
// owns one channel and runs of 16 positions with 16 accumulators, and walks the taps 16 at a time over a
// 31-value register window (out[p] += h[kb + q] * W[p - q + 15], all indices static), so one shared-memory load
// feeds eight multiply-adds.  No tail: positions before the sequence are zero.
constexpr int kFtCh = 32;       // channels per CTA
constexpr int kFtPos = 512;     // positions per CTA
constexpr int kFtRun = 16;      // positions per thread run = taps per block
constexpr int kFtThreads = 256; // eight warps, each a group of position runs

__global__ void __launch_bounds__(kFtThreads, 2) fir_inner_gate_tiled_kernel(const __nv_bfloat16* __restrict__ u,
                                                                   const float* __restrict__ ht, int K, int Kpad,
                                                                   const float* __restrict__ D,
                                                                   const __nv_bfloat16* __restrict__ x2,
                                                                   __nv_bfloat16* __restrict__ out, int L, int d) {
  extern __shared__ __align__(16) unsigned char ft_smem[];
  float* sh = reinterpret_cast<float*>(ft_smem);                                  // [Kpad][32]
  __nv_bfloat16* su = reinterpret_cast<__nv_bfloat16*>(sh + Kpad * kFtCh);        // [Kpad + 512][32], row 0 = t0 - Kpad
  const int c0 = blockIdx.x * kFtCh;
  const int t0 = blockIdx.y * kFtPos;
  const int b = blockIdx.z;
  const __nv_bfloat16* ub = u + static_cast<long long>(b) * L * d;
  for (int i = threadIdx.x; i < Kpad * kFtCh; i += kFtThreads) {
    const int k = i / kFtCh, c = c0 + (i % kFtCh);
    sh[i] = (k < K && c < d) ? ht[static_cast<long long>(k) * d + c] : 0.f;
  }
  // 16-byte loads of 8 channels: four per row of the tile
  for (int i = threadIdx.x; i < (Kpad + kFtPos) * (kFtCh / 8); i += kFtThreads) {
    const int row = i / (kFtCh / 8), c8 = (i % (kFtCh / 8)) * 8;
    const int l = t0 - Kpad + row;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (l >= 0 && l < L && c0 + c8 < d) v = *reinterpret_cast<const uint4*>(ub + static_cast<long long>(l) * d + c0 + c8);
    *reinterpret_cast<uint4*>(su + row * kFtCh + c8) = v;
  }
  __syncthreads();
  const int c = threadIdx.x % kFtCh;
  const int grp = threadIdx.x / kFtCh;                                            // one warp per group of position runs
  if (c0 + c >= d) return;
  const float dv = D[c0 + c];
  for (int run = grp; run < kFtPos / kFtRun; run += kFtThreads / kFtCh) {
    const int l0 = t0 + run * kFtRun;
    if (l0 >= L) break;
    float acc[kFtRun];
#pragma unroll
    for (int p = 0; p < kFtRun; ++p) acc[p] = 0.f;
    // the gate values of this run are requested now and used behind the tap loop
    __nv_bfloat16 gate[kFtRun];
    if (x2 != nullptr) {
#pragma unroll
      for (int p = 0; p < kFtRun; ++p)
        gate[p] = l0 + p < L ? x2[(static_cast<long long>(b) * L + l0 + p) * d + c0 + c] : __float2bfloat16(0.f);
    }
    // W[i] = u[l0 - kb - 15 + i], i = 0..30; tile row of position l is l - t0 + Kpad
    float W[2 * kFtRun - 1];
    const int base = run * kFtRun + Kpad - (kFtRun - 1);                          // row of W[0] at kb = 0
#pragma unroll
    for (int i = 0; i < 2 * kFtRun - 1; ++i) W[i] = __bfloat162float(su[(base + i) * kFtCh + c]);
    for (int kb = 0; kb < Kpad; kb += kFtRun) {
      float h[kFtRun];
#pragma unroll
      for (int q = 0; q < kFtRun; ++q) h[q] = sh[(kb + q) * kFtCh + c];
#pragma unroll
      for (int q = 0; q < kFtRun; ++q)
#pragma unroll
        for (int p = 0; p < kFtRun; ++p) acc[p] = fmaf(h[q], W[p - q + kFtRun - 1], acc[p]);
      if (kb + kFtRun < Kpad) {
        // the next 16 taps look 16 positions further back: the low half of the window moves up, 16 values come in
#pragma unroll
        for (int i = 2 * kFtRun - 2; i >= kFtRun; --i) W[i] = W[i - kFtRun];
        const int nb = base - (kb + kFtRun);
#pragma unroll
        for (int i = 0; i < kFtRun; ++i) W[i] = __bfloat162float(su[(nb + i) * kFtCh + c]);
      }
    }
#pragma unroll
    for (int p = 0; p < kFtRun; ++p) {
      const int l = l0 + p;
      if (l < L) {
        const long long o = (static_cast<long long>(b) * L + l) * d + c0 + c;
        const float cur = __bfloat162float(su[(run * kFtRun + p + Kpad) * kFtCh + c]);
        const float conv = __bfloat162float(__float2bfloat16(acc[p]));
        const float yy = __bfloat162float(__float2bfloat16(conv + cur * dv));
        const float g = x2 == nullptr ? 1.f : __bfloat162float(gate[p]);
        out[o] = __float2bfloat16(g * yy);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------ FFT-conv epilogue
// y: fp32 [B][d][n] (channel-major, the inverse FFT's layout; first L of n samples used), u, x2: bf16 [B][L][d].
// out[b][l][c] = x2 * (bf16(y[b][c][l]) + D[c] * u).  A 32 x 32 tile goes through shared memory so that both the
// fp32 reads (along l) and the bf16 accesses (along c) are coalesced.
__global__ void __launch_bounds__(256) fftconv_epilogue_kernel(const float* __restrict__ y, int n,
                                                               const __nv_bfloat16* __restrict__ u,
                                                               const float* __restrict__ D,
                                                               const __nv_bfloat16* __restrict__ x2,
                                                               __nv_bfloat16* __restrict__ out, int B, int L, int d) {
  __shared__ float tile[32][33];
  const int tl = (L + 31) / 32, tc = (d + 31) / 32;
  const long long tiles = static_cast<long long>(B) * tl * tc;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 8 rows of 32
  for (long long t = blockIdx.x; t < tiles; t += gridDim.x) {
    const int ct = static_cast<int>(t % tc);
    const int lt = static_cast<int>((t / tc) % tl);
    const int b = static_cast<int>(t / (static_cast<long long>(tc) * tl));
    const int l0 = lt * 32, c0 = ct * 32;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int c = c0 + ty + k * 8, l = l0 + tx;
      tile[ty + k * 8][tx] = (c < d && l < L) ? y[(static_cast<long long>(b) * d + c) * n + l] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int l = l0 + ty + k * 8, c = c0 + tx;
      if (l < L && c < d) {
        const long long o = (static_cast<long long>(b) * L + l) * d + c;
        const float conv = __bfloat162float(__float2bfloat16(tile[tx][ty + k * 8]));
        const float yy = __bfloat162float(__float2bfloat16(conv + __bfloat162float(u[o]) * D[c]));
        const float g = x2 == nullptr ? 1.f : __bfloat162float(x2[o]);
        out[o] = __float2bfloat16(g * yy);
      }
    }
    __syncthreads();
  }
}

// ------------------------------------------------------------------------------------------ hcl decode step
// state [B][d][S] fp32 (updated in place), lam / res [d][S] fp32, u / x2 / out [B][d] bf16.
__global__ void __launch_bounds__(256) pole_step_kernel(float* __restrict__ state, const float* __restrict__ lam,
                                                        const float* __restrict__ res,
                                                        const __nv_bfloat16* __restrict__ u,
                                                        const float* __restrict__ D,
                                                        const __nv_bfloat16* __restrict__ x2,
                                                        __nv_bfloat16* __restrict__ out, int B, int d, int S) {
  const long long total = static_cast<long long>(B) * d;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the projection behind may prefetch its weights
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % d);
    const float uv = __bfloat162float(u[i]);
    float* s = state + i * S;
    float acc = 0.f;
    for (int k = 0; k < S; ++k) {
      const float v = s[k] * lam[static_cast<long long>(c) * S + k] + uv;
      s[k] = v;
      acc += v * res[static_cast<long long>(c) * S + k];
    }
    const float yy = __bfloat162float(__float2bfloat16(acc)) + uv * D[c];
    const float g = x2 == nullptr ? 1.f : __bfloat162float(x2[i]);
    out[i] = __float2bfloat16(g * __bfloat162float(__float2bfloat16(yy)));
  }
}

// ------------------------------------------------------------------------------------------ hcl prefill state
// The pole state a prefill of L tokens leaves for decoding: state[b][c][k] = sum_t lam[c][k]^(L-1-t) u[b][t][c].
// The sequence is split into chunks; a thread owns one channel and all S poles of it and runs the recurrence
// s = s * lam + u over its chunk (the u loads of a CTA are 256 contiguous bytes per position); a second kernel
// weights the chunk results by lam^(L - end of chunk) and adds them.  Writing the powers out as a [L][d][S]
// tensor and contracting it - the plain statement - moves 8.6 GB per operator at the 7B shape.
constexpr int kPoleMaxS = 16;

__global__ void __launch_bounds__(128) pole_scan_kernel(const __nv_bfloat16* __restrict__ u,
                                                        const float* __restrict__ lam, float* __restrict__ part,
                                                        int L, int d, int S, int chunk) {
  const int c = blockIdx.x * 128 + threadIdx.x;
  const int ch = blockIdx.y, nch = gridDim.y, b = blockIdx.z;
  if (c >= d) return;
  const int t0 = ch * chunk;
  const int t1 = min(L, t0 + chunk);
  float lm[kPoleMaxS], st[kPoleMaxS];
#pragma unroll
  for (int k = 0; k < kPoleMaxS; ++k) {
    lm[k] = k < S ? lam[static_cast<long long>(c) * S + k] : 0.f;
    st[k] = 0.f;
  }
  const __nv_bfloat16* ub = u + static_cast<long long>(b) * L * d + c;
#pragma unroll 8
  for (int t = t0; t < t1; ++t) {
    const float uv = __bfloat162float(ub[static_cast<long long>(t) * d]);
#pragma unroll
    for (int k = 0; k < kPoleMaxS; ++k) st[k] = fmaf(st[k], lm[k], uv);
  }
  float* o = part + ((static_cast<long long>(b) * nch + ch) * d + c) * S;
#pragma unroll
  for (int k = 0; k < kPoleMaxS; ++k)
    if (k < S) o[k] = st[k];
}

__global__ void __launch_bounds__(256) pole_combine_kernel(const float* __restrict__ part,
                                                           const float* __restrict__ lam, float* __restrict__ state,
                                                           int B, int L, int d, int S, int chunk, int nch) {
  const long long total = static_cast<long long>(B) * d * S;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long cs = i % (static_cast<long long>(d) * S);
    const int b = static_cast<int>(i / (static_cast<long long>(d) * S));
    const float lm = lam[cs];
    float acc = 0.f;
    for (int ch = 0; ch < nch; ++ch) {
      const int t1 = min(L, (ch + 1) * chunk);
      if (t1 <= ch * chunk) break;
      const float w = powf(lm, static_cast<float>(L - t1));           // 1 for the last chunk
      acc = fmaf(w, part[(static_cast<long long>(b) * nch + ch) * d * S + cs], acc);
    }
    state[i] = acc;
  }
}

// ------------------------------------------------------------------------------------------ FFT-conv prologue
// u: bf16 [B][L][d] -> out: fp32 [B][d][n], zero from position L on: the channel-major, zero-padded input the
// real FFT of the long convolution reads (a cast, a strided copy and the transform's own padding otherwise).
__global__ void __launch_bounds__(256) fft_pad_transpose_kernel(const __nv_bfloat16* __restrict__ u,
                                                                float* __restrict__ out, int B, int L, int d, int n) {
  __shared__ float tile[32][33];
  const int tl = (n + 31) / 32, tc = (d + 31) / 32;
  const long long tiles = static_cast<long long>(B) * tl * tc;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (long long t = blockIdx.x; t < tiles; t += gridDim.x) {
    const int lt = static_cast<int>(t % tl);
    const int ct = static_cast<int>((t / tl) % tc);
    const int b = static_cast<int>(t / (static_cast<long long>(tc) * tl));
    const int l0 = lt * 32, c0 = ct * 32;
    if (l0 < L) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int l = l0 + ty + k * 8, c = c0 + tx;
        tile[ty + k * 8][tx] =
            (l < L && c < d) ? __bfloat162float(u[(static_cast<long long>(b) * L + l) * d + c]) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int c = c0 + ty + k * 8, l = l0 + tx;
      if (c < d && l < n) out[(static_cast<long long>(b) * d + c) * n + l] = l0 < L ? tile[tx][ty + k * 8] : 0.f;
    }
    __syncthreads();
  }
}

// X: complex64 [B][d][m], multiplied in place by H: complex64 [d][m] (the filter's spectrum)
__global__ void __launch_bounds__(256) spectrum_mul_kernel(float2* __restrict__ X, const float2* __restrict__ H,
                                                           long long per_batch, long long total) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float2 a = X[i];
    const float2 h = __ldg(H + i % per_batch);
    X[i] = make_float2(a.x * h.x - a.y * h.y, a.x * h.y + a.y * h.x);
  }
}

// ------------------------------------------------------------------------------------------ elementwise sets
enum { EW_GELU_NEW = 0, EW_ADD2 = 1, EW_BIAS_RESIDUAL = 2, EW_SCALE_SHIFT_GELU = 3, EW_SILU_MUL = 4 };

__device__ __forceinline__ float gelu_new_f(float x) {
  // 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))), the "gelu_new" of GPT-J / ProGen2
  const float inner = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.0f + tanhf(inner));
}
__device__ __forceinline__ float gelu_erf_f(float x) { return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f)); }

// x, a, b: bf16 [R][C]; v0 / v1: fp32 [C] per-channel vectors.  C a multiple of 8.
//   GELU_NEW:          out = gelu_new(x)
//   ADD2:              out = x + a + b                      (residual_add2; b may be null)
//   BIAS_RESIDUAL:     out = x + v0[c] + a                  (a may be null)
//   SCALE_SHIFT_GELU:  out = gelu_erf(x * v0[c] + v1[c])    (folded batch norm + GELU)
//   SILU_MUL:          out = silu(x) * a
template <int OP>
__global__ void __launch_bounds__(256) ew_kernel(const __nv_bfloat16* __restrict__ x,
                                                 const __nv_bfloat16* __restrict__ a,
                                                 const __nv_bfloat16* __restrict__ b, const float* __restrict__ v0,
                                                 const float* __restrict__ v1, __nv_bfloat16* __restrict__ out,
                                                 long long R, int C) {
  const int c8 = C / 8;
  const long long total = R * c8;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % c8) * 8;
    float xv[8], av[8], bv[8], o[8];
    unpack8(reinterpret_cast<const uint4*>(x)[i], xv);
    if (a != nullptr) unpack8(reinterpret_cast<const uint4*>(a)[i], av);
    if (b != nullptr) unpack8(reinterpret_cast<const uint4*>(b)[i], bv);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      if (OP == EW_GELU_NEW) {
        o[e] = gelu_new_f(xv[e]);
      } else if (OP == EW_ADD2) {
        o[e] = xv[e] + (a != nullptr ? av[e] : 0.f) + (b != nullptr ? bv[e] : 0.f);
      } else if (OP == EW_BIAS_RESIDUAL) {
        o[e] = xv[e] + v0[c + e] + (a != nullptr ? av[e] : 0.f);
      } else if (OP == EW_SCALE_SHIFT_GELU) {
        o[e] = gelu_erf_f(fmaf(xv[e], v0[c + e], v1[c + e]));
      } else {
        o[e] = (xv[e] / (1.0f + __expf(-xv[e]))) * av[e];
      }
    }
    reinterpret_cast<uint4*>(out)[i] = pack8(o);
  }
}

// rotary_split_qkv: qkv [T][3][H][Dh] bf16 (one fused projection row per token) -> q, k with rotary applied to
// the first `rot` dims of each head (GPT-J interleaved pairs), v copied; outputs [T][H][Dh].  pos: int32 [T].
__global__ void __launch_bounds__(256) rotary_split_qkv_kernel(const __nv_bfloat16* __restrict__ qkv,
                                                               const int* __restrict__ pos,
                                                               __nv_bfloat16* __restrict__ q,
                                                               __nv_bfloat16* __restrict__ k,
                                                               __nv_bfloat16* __restrict__ v, long long T, int H,
                                                               int Dh, int rot, float base) {
  const int half = Dh / 2;
  const long long total = T * H * half;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int p = static_cast<int>(i % half);
    const long long th = i / half;
    const int h = static_cast<int>(th % H);
    const long long t = th / H;
    const long long src = (t * 3 * H + h) * Dh + 2 * p;
    const long long dst = (t * H + h) * Dh + 2 * p;
    const long long hs = static_cast<long long>(H) * Dh;
    float q0 = __bfloat162float(qkv[src]), q1 = __bfloat162float(qkv[src + 1]);
    float k0 = __bfloat162float(qkv[src + hs]), k1 = __bfloat162float(qkv[src + hs + 1]);
    if (2 * p < rot) {
      const float inv = powf(base, -static_cast<float>(2 * p) / static_cast<float>(rot));
      float sn, cs;
      sincosf(static_cast<float>(pos[t]) * inv, &sn, &cs);
      const float a0 = q0 * cs - q1 * sn, a1 = q1 * cs + q0 * sn;
      const float b0 = k0 * cs - k1 * sn, b1 = k1 * cs + k0 * sn;
      q0 = a0; q1 = a1; k0 = b0; k1 = b1;
    }
    *reinterpret_cast<__nv_bfloat162*>(q + dst) = __floats2bfloat162_rn(q0, q1);
    *reinterpret_cast<__nv_bfloat162*>(k + dst) = __floats2bfloat162_rn(k0, k1);
    *reinterpret_cast<__nv_bfloat162*>(v + dst) =
        *reinterpret_cast<const __nv_bfloat162*>(qkv + src + 2 * hs);
  }
}

// softmax over rows of x + a + b (fp32 in and out; a, b may be null); one warp per row, C <= 4096
__global__ void __launch_bounds__(256) add2_softmax_rows_kernel(const float* __restrict__ x,
                                                                const float* __restrict__ a,
                                                                const float* __restrict__ b,
                                                                float* __restrict__ out, long long R, int C) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (long long r = static_cast<long long>(blockIdx.x) * wpb + (threadIdx.x >> 5); r < R;
       r += static_cast<long long>(gridDim.x) * wpb) {
    const long long o = r * C;
    float mx = -3.0e38f;
    for (int c = lane; c < C; c += 32) {
      const float v = x[o + c] + (a ? a[o + c] : 0.f) + (b ? b[o + c] : 0.f);
      mx = fmaxf(mx, v);
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, s));
    float sum = 0.f;
    for (int c = lane; c < C; c += 32) {
      const float v = x[o + c] + (a ? a[o + c] : 0.f) + (b ? b[o + c] : 0.f);
      sum += __expf(v - mx);
    }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    for (int c = lane; c < C; c += 32) {
      const float v = x[o + c] + (a ? a[o + c] : 0.f) + (b ? b[o + c] : 0.f);
      out[o + c] = __expf(v - mx) * inv;
    }
  }
}

// pool2 over the sequence axis of [B][L][C] bf16: mode 0 = max, 1 = mean, 2 = softmax-weighted with logits
// w [B][L][C] (attention pooling of width 2).  L even.
__global__ void __launch_bounds__(256) pool2_kernel(const __nv_bfloat16* __restrict__ x,
                                                    const __nv_bfloat16* __restrict__ w,
                                                    __nv_bfloat16* __restrict__ out, int B, int L, int C, int mode) {
  const int c8 = C / 8;
  const long long total = static_cast<long long>(B) * (L / 2) * c8;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % c8) * 8;
    const long long bl = i / c8;
    const int l2 = static_cast<int>(bl % (L / 2));
    const int b = static_cast<int>(bl / (L / 2));
    const long long s0 = (static_cast<long long>(b) * L + 2 * l2) * C + c;
    float x0[8], x1[8], o[8];
    unpack8(*reinterpret_cast<const uint4*>(x + s0), x0);
    unpack8(*reinterpret_cast<const uint4*>(x + s0 + C), x1);
    if (mode == 2) {
      float w0[8], w1[8];
      unpack8(*reinterpret_cast<const uint4*>(w + s0), w0);
      unpack8(*reinterpret_cast<const uint4*>(w + s0 + C), w1);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float m = fmaxf(w0[e], w1[e]);
        const float e0 = __expf(w0[e] - m), e1 = __expf(w1[e] - m);
        o[e] = (x0[e] * e0 + x1[e] * e1) / (e0 + e1);
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = mode == 0 ? fmaxf(x0[e], x1[e]) : 0.5f * (x0[e] + x1[e]);
    }
    *reinterpret_cast<uint4*>(out + (static_cast<long long>(b) * (L / 2) + l2) * C + c) = pack8(o);
  }
}

// residual + LayerNorm: s = x + res (written to sum_out when not null), out = LN(s) * gamma + beta
template <int CHUNKS>
__global__ void __launch_bounds__(256) residual_ln_kernel(const __nv_bfloat16* __restrict__ x,
                                                          const __nv_bfloat16* __restrict__ res,
                                                          const float* __restrict__ gamma,
                                                          const float* __restrict__ beta,
                                                          __nv_bfloat16* __restrict__ sum_out,
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
        float rr[8];
        unpack8(*reinterpret_cast<const uint4*>(x + r * C + c), v[k]);
        unpack8(*reinterpret_cast<const uint4*>(res + r * C + c), rr);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          // the sum is rounded to the activation type first, as the unfused residual add does
          v[k][j] = __bfloat162float(__float2bfloat16(v[k][j] + rr[j]));
          sum += v[k][j];
        }
        if (sum_out != nullptr) *reinterpret_cast<uint4*>(sum_out + r * C + c) = pack8(v[k]);
      }
    }
    sum = warp_sum(sum);
    const float mu = sum / C;
    float var = 0.f;
#pragma unroll
    for (int k = 0; k < CHUNKS; ++k) {
      const int c = k * 256 + lane * 8;
      if (c < C) {
#pragma unroll
        for (int j = 0; j < 8; ++j) var += (v[k][j] - mu) * (v[k][j] - mu);
      }
    }
    var = warp_sum(var);
    const float rstd = rsqrtf(var / C + eps);
#pragma unroll
    for (int k = 0; k < CHUNKS; ++k) {
      const int c = k * 256 + lane * 8;
      if (c < C) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = (v[k][j] - mu) * rstd * gamma[c + j] + (beta ? beta[c + j] : 0.f);
        *reinterpret_cast<uint4*>(out + r * C + c) = pack8(o);
      }
    }
  }
}

}  // namespace ubm

using namespace ubm;

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

extern "C" int ubm_rmsnorm_rows(const void* x, const void* scale, void* out, long long R, int C, float eps,
                                void* stream) {
  if (R <= 0 || C <= 0 || (C & 7) || !aligned16(x) || !aligned16(out) || !aligned16(scale))
    return UBM_ERR_ARGUMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = seq_grid(R, 8);
  const __nv_bfloat16* xx = static_cast<const __nv_bfloat16*>(x);
  const float* sc = static_cast<const float*>(scale);
  __nv_bfloat16* oo = static_cast<__nv_bfloat16*>(out);
  if (C <= 1024) rmsnorm_rows_kernel<4><<<grid, 256, 0, st>>>(xx, sc, oo, R, C, eps);
  else if (C <= 2048) rmsnorm_rows_kernel<8><<<grid, 256, 0, st>>>(xx, sc, oo, R, C, eps);
  else if (C <= 4096) rmsnorm_rows_kernel<16><<<grid, 256, 0, st>>>(xx, sc, oo, R, C, eps);
  else rmsnorm_rows_wide_kernel<<<grid, 256, 0, st>>>(xx, sc, oo, R, C, eps);
  UBM_CHECK_LAUNCH("rmsnorm_rows_kernel");
  return UBM_OK;
}

// x: bf16 [R][C] (C a multiple of 8, at most 4096); scale: fp32 [C]; amax: uint32 [1] scratch (the bits of the
// maximum); out: e4m3 [R][C]; dequant: fp32 [1] = max / 448
extern "C" int ubm_rmsnorm_fp8(const void* x, const void* scale, void* amax, void* out, void* dequant, long long R,
                               int C, float eps, void* stream) {
  if (R <= 0 || C <= 0 || (C & 7) || C > 4096 || !aligned16(x) || !aligned16(scale) || (reinterpret_cast<uintptr_t>(out) & 7))
    return UBM_ERR_ARGUMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = seq_grid(R, 8);
  const __nv_bfloat16* xx = static_cast<const __nv_bfloat16*>(x);
  const float* sc = static_cast<const float*>(scale);
  unsigned int* am = static_cast<unsigned int*>(amax);
  uint8_t* oo = static_cast<uint8_t*>(out);
  float* dq = static_cast<float*>(dequant);
  if (cudaMemsetAsync(am, 0, sizeof(unsigned int), st) != cudaSuccess) return UBM_ERR_LAUNCH;
#define UBM_RF8(CH)                                                                              \
  do {                                                                                           \
    rmsnorm_fp8_kernel<CH, false><<<grid, 256, 0, st>>>(xx, sc, am, oo, dq, R, C, eps);          \
    rmsnorm_fp8_kernel<CH, true><<<grid, 256, 0, st>>>(xx, sc, am, oo, dq, R, C, eps);           \
  } while (0)
  if (C <= 1024) UBM_RF8(4);
  else if (C <= 2048) UBM_RF8(8);
  else UBM_RF8(16);
#undef UBM_RF8
  UBM_CHECK_LAUNCH("rmsnorm_fp8_kernel");
  return UBM_OK;
}

// z: bf16 [B][L][3d]; ht: fp32 [K][3d] (tap-major); tail: bf16 [B][K-1][3d] or null; u, x2: bf16 [B][L][d].
// push != 0 (decode: L <= 32, tail given): the tail is replaced in place by the last K - 1 samples
extern "C" int ubm_fir_gate3(const void* z, const void* ht, void* tail, void* u, void* x2, int B, int L, int d,
                             int K, int push, void* stream) {
  // three filter windows live in registers at once: up to four taps (the input stage of Hyena uses three)
  if (B <= 0 || L <= 0 || d <= 0 || (d & 7) || K < 1 || K > 4) return UBM_ERR_ARGUMENT;
  if (push && (tail == nullptr || L > kFirTL)) return UBM_ERR_ARGUMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long total = static_cast<long long>(B) * ((L + kFirTL - 1) / kFirTL) * (d / 8);
  const int grid = seq_grid(total, 128);
#define UBM_FG3(KK)                                                                                            \
  fir_gate3_kernel<KK><<<grid, 128, 0, st>>>(static_cast<const __nv_bfloat16*>(z), static_cast<const float*>(ht), \
                                             static_cast<__nv_bfloat16*>(tail),                                 \
                                             static_cast<__nv_bfloat16*>(u), static_cast<__nv_bfloat16*>(x2), B, L, d, \
                                             push)
  switch (K) {
    case 1: UBM_FG3(1); break;
    case 2: UBM_FG3(2); break;
    case 3: UBM_FG3(3); break;
    default: UBM_FG3(4); break;
  }
#undef UBM_FG3
  UBM_CHECK_LAUNCH("fir_gate3_kernel");
  return UBM_OK;
}

// u: bf16 [B][L][d]; ht: fp32 [K][d]; D: fp32 [d]; x2: bf16 [B][L][d] or null; tail: bf16 [B][K-1][d] or null.
extern "C" int ubm_fir_inner_gate(const void* u, const void* ht, const void* D, const void* x2, const void* tail,
                                  void* out, int B, int L, int d, int K, void* stream) {
  if (B <= 0 || L <= 0 || d <= 0 || (d & 7) || K < 1) return UBM_ERR_ARGUMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* uu = static_cast<const __nv_bfloat16*>(u);
  const float* hh = static_cast<const float*>(ht);
  const float* dd = static_cast<const float*>(D);
  const __nv_bfloat16* xx = static_cast<const __nv_bfloat16*>(x2);
  const __nv_bfloat16* tt = static_cast<const __nv_bfloat16*>(tail);
  __nv_bfloat16* oo = static_cast<__nv_bfloat16*>(out);
  if (K <= 8) {
    const long long total = static_cast<long long>(B) * ((L + kFirTL - 1) / kFirTL) * (d / 8);
    const int grid = seq_grid(total, 128);
#define UBM_FIG(KK) fir_inner_gate_kernel<KK><<<grid, 128, 0, st>>>(uu, hh, dd, xx, tt, oo, B, L, d)
    switch (K) {
      case 1: UBM_FIG(1); break;
      case 2: UBM_FIG(2); break;
      case 3: UBM_FIG(3); break;
      case 4: UBM_FIG(4); break;
      case 5: UBM_FIG(5); break;
      case 6: UBM_FIG(6); break;
      case 7: UBM_FIG(7); break;
      default: UBM_FIG(8); break;
    }
#undef UBM_FIG
  } else if (tt == nullptr && L >= 64 && K <= 512 && B <= 65535) {
    const int Kpad = (K + kFtRun - 1) / kFtRun * kFtRun;
    const size_t smem = static_cast<size_t>(Kpad) * kFtCh * sizeof(float) +
                        static_cast<size_t>(Kpad + kFtPos) * kFtCh * sizeof(__nv_bfloat16);
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(fir_inner_gate_tiled_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return UBM_ERR_LAUNCH;
    const dim3 grid((d + kFtCh - 1) / kFtCh, (L + kFtPos - 1) / kFtPos, B);
    fir_inner_gate_tiled_kernel<<<grid, kFtThreads, smem, st>>>(uu, hh, K, Kpad, dd, xx, oo, L, d);
  } else {
    const long long total = static_cast<long long>(B) * L * (d / 8);
    fir_inner_gate_long_kernel<<<seq_grid(total, 128), 128, 0, st>>>(uu, hh, K, dd, xx, tt, oo, B, L, d);
  }
  UBM_CHECK_LAUNCH("fir_inner_gate_kernel");
  return UBM_OK;
}

// u, x2, out: bf16 [B][d]; ht: fp32 [K][d]; tail: bf16 [B][K-1][d], moved on in place.  2 <= K <= 256.
extern "C" int ubm_fir_step(const void* u, const void* ht, const void* D, const void* x2, void* tail, void* out, int B,
                            int d, int K, void* stream) {
  if (B <= 0 || B > 65535 || d <= 0 || (d & 7) || K < 2 || K > 32 * kFirStepMaxTapsPerThread || tail == nullptr)
    return UBM_ERR_ARGUMENT;
  const dim3 grid((d + 63) / 64, B);
  fir_step_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(u), static_cast<const float*>(ht), K, static_cast<const float*>(D),
      static_cast<const __nv_bfloat16*>(x2), static_cast<__nv_bfloat16*>(tail), static_cast<__nv_bfloat16*>(out), d);
  UBM_CHECK_LAUNCH("fir_step_kernel");
  return UBM_OK;
}

extern "C" int ubm_fftconv_epilogue(const void* y, int n, const void* u, const void* D, const void* x2, void* out,
                                    int B, int L, int d, void* stream) {
  if (B <= 0 || L <= 0 || d <= 0 || n < L) return UBM_ERR_ARGUMENT;
  const long long tiles = static_cast<long long>(B) * ((L + 31) / 32) * ((d + 31) / 32);
  fftconv_epilogue_kernel<<<seq_grid(tiles, 1), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float*>(y), n, static_cast<const __nv_bfloat16*>(u), static_cast<const float*>(D),
      static_cast<const __nv_bfloat16*>(x2), static_cast<__nv_bfloat16*>(out), B, L, d);
  UBM_CHECK_LAUNCH("fftconv_epilogue_kernel");
  return UBM_OK;
}

// u: bf16 [B][L][d]; lam: fp32 [d][S] (S <= 16); part: fp32 [B][chunks][d][S] scratch; state: fp32 [B][d][S]
extern "C" int ubm_pole_prefill_state(const void* u, const void* lam, void* part, void* state, int B, int L, int d,
                                      int S, int chunks, void* stream) {
  if (B <= 0 || B > 65535 || L <= 0 || d <= 0 || S <= 0 || S > kPoleMaxS || chunks < 1 || chunks > 65535)
    return UBM_ERR_ARGUMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int chunk = (L + chunks - 1) / chunks;
  pole_scan_kernel<<<dim3((d + 127) / 128, chunks, B), 128, 0, st>>>(
      static_cast<const __nv_bfloat16*>(u), static_cast<const float*>(lam), static_cast<float*>(part), L, d, S, chunk);
  UBM_CHECK_LAUNCH("pole_scan_kernel");
  pole_combine_kernel<<<seq_grid(static_cast<long long>(B) * d * S, 256), 256, 0, st>>>(
      static_cast<const float*>(part), static_cast<const float*>(lam), static_cast<float*>(state), B, L, d, S, chunk,
      chunks);
  UBM_CHECK_LAUNCH("pole_combine_kernel");
  return UBM_OK;
}

// u: bf16 [B][L][d] -> out: fp32 [B][d][n] (n >= L), zero-padded
extern "C" int ubm_fft_pad_transpose(const void* u, void* out, int B, int L, int d, int n, void* stream) {
  if (B <= 0 || L <= 0 || d <= 0 || n < L) return UBM_ERR_ARGUMENT;
  const long long tiles = static_cast<long long>(B) * ((n + 31) / 32) * ((d + 31) / 32);
  fft_pad_transpose_kernel<<<seq_grid(tiles, 1), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(u), static_cast<float*>(out), B, L, d, n);
  UBM_CHECK_LAUNCH("fft_pad_transpose_kernel");
  return UBM_OK;
}

// X: complex64 [B][per_batch] (interleaved re, im), in place; H: complex64 [per_batch]
extern "C" int ubm_spectrum_mul(void* X, const void* H, int B, long long per_batch, void* stream) {
  if (B <= 0 || per_batch <= 0) return UBM_ERR_ARGUMENT;
  const long long total = static_cast<long long>(B) * per_batch;
  spectrum_mul_kernel<<<seq_grid(total, 256 * 4), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<float2*>(X), static_cast<const float2*>(H), per_batch, total);
  UBM_CHECK_LAUNCH("spectrum_mul_kernel");
  return UBM_OK;
}

extern "C" int ubm_pole_step(void* state, const void* lam, const void* res, const void* u, const void* D,
                             const void* x2, void* out, int B, int d, int S, void* stream) {
  if (B <= 0 || d <= 0 || S <= 0) return UBM_ERR_ARGUMENT;
  pole_step_kernel<<<seq_grid(static_cast<long long>(B) * d, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<float*>(state), static_cast<const float*>(lam), static_cast<const float*>(res),
      static_cast<const __nv_bfloat16*>(u), static_cast<const float*>(D), static_cast<const __nv_bfloat16*>(x2),
      static_cast<__nv_bfloat16*>(out), B, d, S);
  UBM_CHECK_LAUNCH("pole_step_kernel");
  return UBM_OK;
}

// op: 0 gelu_new, 1 add2, 2 bias_residual, 3 scale_shift_gelu, 4 silu_mul (see ew_kernel)
extern "C" int ubm_elementwise(int op, const void* x, const void* a, const void* b, const void* v0, const void* v1,
                               void* out, long long R, int C, void* stream) {
  if (R <= 0 || C <= 0 || (C & 7) || !aligned16(x) || !aligned16(out) || !aligned16(a) || !aligned16(b))
    return UBM_ERR_ARGUMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = seq_grid(R * (C / 8), 256);
  const __nv_bfloat16* xx = static_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* aa = static_cast<const __nv_bfloat16*>(a);
  const __nv_bfloat16* bb = static_cast<const __nv_bfloat16*>(b);
  const float* p0 = static_cast<const float*>(v0);
  const float* p1 = static_cast<const float*>(v1);
  __nv_bfloat16* oo = static_cast<__nv_bfloat16*>(out);
  switch (op) {
    case EW_GELU_NEW: ew_kernel<EW_GELU_NEW><<<grid, 256, 0, st>>>(xx, aa, bb, p0, p1, oo, R, C); break;
    case EW_ADD2: ew_kernel<EW_ADD2><<<grid, 256, 0, st>>>(xx, aa, bb, p0, p1, oo, R, C); break;
    case EW_BIAS_RESIDUAL:
      if (v0 == nullptr) return UBM_ERR_ARGUMENT;
      ew_kernel<EW_BIAS_RESIDUAL><<<grid, 256, 0, st>>>(xx, aa, bb, p0, p1, oo, R, C);
      break;
    case EW_SCALE_SHIFT_GELU:
      if (v0 == nullptr || v1 == nullptr) return UBM_ERR_ARGUMENT;
      ew_kernel<EW_SCALE_SHIFT_GELU><<<grid, 256, 0, st>>>(xx, aa, bb, p0, p1, oo, R, C);
      break;
    case EW_SILU_MUL:
      if (a == nullptr) return UBM_ERR_ARGUMENT;
      ew_kernel<EW_SILU_MUL><<<grid, 256, 0, st>>>(xx, aa, bb, p0, p1, oo, R, C);
      break;
    default: return UBM_ERR_ARGUMENT;
  }
  UBM_CHECK_LAUNCH("ew_kernel");
  return UBM_OK;
}

extern "C" int ubm_rotary_split_qkv(const void* qkv, const void* pos, void* q, void* k, void* v, long long T, int H,
                                    int Dh, int rot, float base, void* stream) {
  if (T <= 0 || H <= 0 || Dh <= 0 || (Dh & 1) || rot < 0 || rot > Dh || (rot & 1)) return UBM_ERR_ARGUMENT;
  rotary_split_qkv_kernel<<<seq_grid(T * H * (Dh / 2), 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(qkv), static_cast<const int*>(pos), static_cast<__nv_bfloat16*>(q),
      static_cast<__nv_bfloat16*>(k), static_cast<__nv_bfloat16*>(v), T, H, Dh, rot, base);
  UBM_CHECK_LAUNCH("rotary_split_qkv_kernel");
  return UBM_OK;
}

extern "C" int ubm_add2_softmax_rows(const void* x, const void* a, const void* b, void* out, long long R, int C,
                                     void* stream) {
  if (R <= 0 || C <= 0) return UBM_ERR_ARGUMENT;
  add2_softmax_rows_kernel<<<seq_grid(R, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float*>(x), static_cast<const float*>(a), static_cast<const float*>(b),
      static_cast<float*>(out), R, C);
  UBM_CHECK_LAUNCH("add2_softmax_rows_kernel");
  return UBM_OK;
}

extern "C" int ubm_pool2(const void* x, const void* w, void* out, int B, int L, int C, int mode, void* stream) {
  if (B <= 0 || L <= 0 || (L & 1) || C <= 0 || (C & 7) || mode < 0 || mode > 2 || (mode == 2 && w == nullptr))
    return UBM_ERR_ARGUMENT;
  pool2_kernel<<<seq_grid(static_cast<long long>(B) * (L / 2) * (C / 8), 256), 256, 0,
                 static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(x),
                                                      static_cast<const __nv_bfloat16*>(w),
                                                      static_cast<__nv_bfloat16*>(out), B, L, C, mode);
  UBM_CHECK_LAUNCH("pool2_kernel");
  return UBM_OK;
}

extern "C" int ubm_residual_ln(const void* x, const void* res, const void* gamma, const void* beta, void* sum_out,
                               void* out, long long R, int C, float eps, void* stream) {
  if (R <= 0 || C <= 0 || (C & 7) || C > 4096 || res == nullptr || gamma == nullptr) return UBM_ERR_ARGUMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = seq_grid(R, 8);
  const __nv_bfloat16* xx = static_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* rr = static_cast<const __nv_bfloat16*>(res);
  const float* g = static_cast<const float*>(gamma);
  const float* bt = static_cast<const float*>(beta);
  __nv_bfloat16* so = static_cast<__nv_bfloat16*>(sum_out);
  __nv_bfloat16* oo = static_cast<__nv_bfloat16*>(out);
  if (C <= 1024) residual_ln_kernel<4><<<grid, 256, 0, st>>>(xx, rr, g, bt, so, oo, R, C, eps);
  else if (C <= 2048) residual_ln_kernel<8><<<grid, 256, 0, st>>>(xx, rr, g, bt, so, oo, R, C, eps);
  else residual_ln_kernel<16><<<grid, 256, 0, st>>>(xx, rr, g, bt, so, oo, R, C, eps);
  UBM_CHECK_LAUNCH("residual_ln_kernel");
  return UBM_OK;
}

// ------------------------------------------------------------------------------------------ decode GEMV
// y[b][n] = sum_k W[n][k] x^[b][k] (+ bias[n]) for a handful of rows b (single-token decode): the weight matrix is
// streamed once at memory speed, one warp per output row n, eight independent 16-byte loads per lane in flight,
// fp32 accumulation.  A 128-row MMA tile would use one row of it and, with N / 256 tiles, a fraction of the SMs.
// The rows of a decode block are folded into the same launch:
//   gamma != null : x^ = bf16(x * rsqrt(mean(x^2) + eps) * gamma)   (the block's RMSNorm; else x^ = x)
//   w2 != null    : out = bf16(silu(g) * u), g = bf16(W x^), u = bf16(W2 x^)   (the two halves of SwiGLU)
//   res != null   : out = bf16(res + bf16(y))                                   (the residual stream)
// Every intermediate is rounded to bf16 where the separate kernels round it, so the folded form returns the
// same bits.  x^ is staged once per CTA in shared memory ([MB][K] bf16).
namespace ubm {
constexpr int kGemvThreads = 512;
constexpr int kGemvMaxSmem = 200 * 1024;

__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16(v)); }

__device__ __forceinline__ void unpack16_e4m3(const uint4& u, float (&e)[16]) {
  const unsigned int w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w[i] & 0xffffu), __NV_E4M3);
    const __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w[i] >> 16), __NV_E4M3);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&lo));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&hi));
    e[4 * i] = a.x; e[4 * i + 1] = a.y; e[4 * i + 2] = b.x; e[4 * i + 3] = b.y;
  }
}

// W8: w holds e4m3 bytes ([N][K], K a multiple of 16) and the row sums are multiplied by wscale (the weights'
// dequantisation factor); the activations stay bf16.  Half the bytes of the bf16 form per output row.
template <int MB, bool DUAL, bool W8>
__global__ void __launch_bounds__(kGemvThreads) gemv_rows_kernel(
    const __nv_bfloat16* __restrict__ x, const float* __restrict__ gamma, float eps,
    const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ w2, const float* __restrict__ bias,
    const __nv_bfloat16* __restrict__ res, __nv_bfloat16* __restrict__ out, int M, int N, int K, float wscale) {
  static_assert(!(DUAL && W8), "the two-matrix form reads bf16 weights");
  const int wbytes = W8 ? 1 : 2;                                               // bytes per weight element
  extern __shared__ __align__(16) unsigned char gemv_smem[];
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(gemv_smem);              // [MB][K]
  __shared__ float red[MB][kGemvThreads / 32];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int wpb = kGemvThreads / 32;
  const int nv = K >> 3;                                                       // 16-byte vectors per row
  // rows go to the warps CTA by CTA (dealing them round-robin over the CTAs for an even row count per SM measured
  // slower: 27.5 against 26.7 us for 4096 -> 12288 and 4.2 against 3.5 ms for the whole decode step)
  const int n_first = blockIdx.x * wpb + warp;
  // the first weight row of this warp starts towards L2 while x^ is staged
  if (n_first < N) {
    const char* p0 = reinterpret_cast<const char*>(w) + static_cast<long long>(n_first) * K * wbytes;
    for (int o = lane * 128; o < K * wbytes; o += 32 * 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(p0 + o));
    if (DUAL) {
      const char* p1 = reinterpret_cast<const char*>(w2 + static_cast<long long>(n_first) * K);
      for (int o = lane * 128; o < K * 2; o += 32 * 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(p1 + o));
    }
  }
  // Programmatic dependent launch: the prefetch above read only weights, so this CTA may have started while the
  // previous kernel of the stream drains; x, the residual and the output are touched from here on.  The kernel
  // behind this one may start its own prefetch as soon as every CTA here has passed this point.  Both
  // instructions are no-ops for a launch without the attribute.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // ---- stage x^
  if (gamma != nullptr) {
    float ss[MB];
#pragma unroll
    for (int b = 0; b < MB; ++b) ss[b] = 0.f;
    for (int i = threadIdx.x; i < nv; i += kGemvThreads) {
#pragma unroll
      for (int b = 0; b < MB; ++b) {
        if (b < M) {
          float v[8];
          unpack8(reinterpret_cast<const uint4*>(x + static_cast<long long>(b) * K)[i], v);
#pragma unroll
          for (int e = 0; e < 8; ++e) ss[b] += v[e] * v[e];
        }
      }
    }
#pragma unroll
    for (int b = 0; b < MB; ++b) {
      const float t = warp_sum(ss[b]);
      if (lane == 0) red[b][warp] = t;
    }
    __syncthreads();
    float rs[MB];
#pragma unroll
    for (int b = 0; b < MB; ++b) {
      float t = 0.f;
#pragma unroll
      for (int q = 0; q < wpb; ++q) t += red[b][q];
      rs[b] = rsqrtf(t / K + eps);
    }
    for (int i = threadIdx.x; i < nv; i += kGemvThreads) {
      const float4 s0 = __ldg(reinterpret_cast<const float4*>(gamma) + 2 * i);
      const float4 s1 = __ldg(reinterpret_cast<const float4*>(gamma) + 2 * i + 1);
      const float sc[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
      for (int b = 0; b < MB; ++b) {
        if (b < M) {
          float v[8], o[8];
          unpack8(reinterpret_cast<const uint4*>(x + static_cast<long long>(b) * K)[i], v);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] = v[e] * rs[b] * sc[e];
          reinterpret_cast<uint4*>(xs + static_cast<long long>(b) * K)[i] = pack8(o);
        }
      }
    }
  } else {
    for (int i = threadIdx.x; i < nv; i += kGemvThreads) {
#pragma unroll
      for (int b = 0; b < MB; ++b)
        if (b < M)
          reinterpret_cast<uint4*>(xs + static_cast<long long>(b) * K)[i] =
              reinterpret_cast<const uint4*>(x + static_cast<long long>(b) * K)[i];
    }
  }
  __syncthreads();
  // ---- stream the weights
  for (int n = n_first; n < N; n += gridDim.x * wpb) {
    float acc[MB], acc2[DUAL ? MB : 1];
#pragma unroll
    for (int b = 0; b < MB; ++b) acc[b] = 0.f;
#pragma unroll
    for (int b = 0; b < (DUAL ? MB : 1); ++b) acc2[b] = 0.f;
    if constexpr (W8) {
      const uint4* wr8 = reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(w) + static_cast<long long>(n) * K);
      const int nv8 = K >> 4;                                                  // 16 weights per 16-byte vector
      constexpr int U8 = 4;
      for (int i0 = lane; i0 < nv8; i0 += 32 * U8) {
        uint4 wv[U8];
#pragma unroll
        for (int u = 0; u < U8; ++u) {
          const int i = i0 + 32 * u;
          wv[u] = i < nv8 ? __ldcs(wr8 + i) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < U8; ++u) {
          const int i = i0 + 32 * u;
          if (i < nv8) {
            float wf[16];
            unpack16_e4m3(wv[u], wf);
#pragma unroll
            for (int b = 0; b < MB; ++b) {
              if (b < M) {
                float x0[8], x1[8];
                const uint4* xb = reinterpret_cast<const uint4*>(xs + static_cast<long long>(b) * K);
                unpack8(xb[2 * i], x0);
                unpack8(xb[2 * i + 1], x1);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                  acc[b] = fmaf(wf[e], x0[e], acc[b]);
                  acc[b] = fmaf(wf[8 + e], x1[e], acc[b]);
                }
              }
            }
          }
        }
      }
    }
    const uint4* wr = reinterpret_cast<const uint4*>(w + static_cast<long long>(n) * K);
    const uint4* wr2 = DUAL ? reinterpret_cast<const uint4*>(w2 + static_cast<long long>(n) * K) : nullptr;
    // loads in flight per lane: 8 (two matrices x 4, or one matrix x 8 when few rows leave the registers free)
    constexpr int U = (DUAL || MB > 2) ? 4 : 8;
    for (int i0 = lane; i0 < (W8 ? 0 : nv); i0 += 32 * U) {
      uint4 wv[U], wv2[DUAL ? U : 1];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int i = i0 + 32 * u;
        wv[u] = i < nv ? __ldcs(wr + i) : make_uint4(0u, 0u, 0u, 0u);
        if (DUAL) wv2[u] = i < nv ? __ldcs(wr2 + i) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int i = i0 + 32 * u;
        if (i < nv) {
          float wf[8], wf2[8];
          unpack8(wv[u], wf);
          if (DUAL) unpack8(wv2[u], wf2);
#pragma unroll
          for (int b = 0; b < MB; ++b) {
            if (b < M) {
              float xv[8];
              unpack8(reinterpret_cast<const uint4*>(xs + static_cast<long long>(b) * K)[i], xv);
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                acc[b] = fmaf(wf[e], xv[e], acc[b]);
                if (DUAL) acc2[b] = fmaf(wf2[e], xv[e], acc2[b]);
              }
            }
          }
        }
      }
    }
#pragma unroll
    for (int b = 0; b < MB; ++b) {
      float s = warp_sum(acc[b]);
      float s2 = DUAL ? warp_sum(acc2[b]) : 0.f;
      if (lane == 0 && b < M) {
        const long long o = static_cast<long long>(b) * N + n;
        if (W8) s *= wscale;
        if (bias != nullptr) s += bias[n];
        if (DUAL) {
          const float g = bf16_round(s), up = bf16_round(s2);
          s = (g / (1.0f + __expf(-g))) * up;
        }
        if (res != nullptr) s = bf16_round(s) + __bfloat162float(res[o]);
        out[o] = __float2bfloat16(s);
      }
    }
  }
}

template <bool DUAL, bool W8>
int launch_gemv(const __nv_bfloat16* x, const float* gamma, float eps, const __nv_bfloat16* w, const __nv_bfloat16* w2,
                const float* bias, const __nv_bfloat16* res, __nv_bfloat16* out, int M, int N, int K, float wscale,
                cudaStream_t st) {
  const int MB = M == 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : 8;
  const size_t smem = static_cast<size_t>(MB) * K * sizeof(__nv_bfloat16);
  if (smem > static_cast<size_t>(kGemvMaxSmem)) return UBM_ERR_ARGUMENT;
  const int wpb = kGemvThreads / 32;
  const int per_sm = smem > 100 * 1024 ? 1 : 2;
  int grid = (N + wpb - 1) / wpb;
  if (grid > sm_count() * per_sm) grid = sm_count() * per_sm;
  // launched so that its weight prefetch may overlap the tail of the previous kernel in the stream (see the kernel)
  static const bool pdl = [] {
    const char* e = getenv("UBM_PDL");
    return e == nullptr || e[0] != '0';
  }();
#define UBM_GEMV(MBV)                                                                                          \
  do {                                                                                                         \
    auto kern = gemv_rows_kernel<MBV, DUAL, W8>;                                                               \
    if (smem > 48 * 1024 &&                                                                                    \
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemvMaxSmem) != cudaSuccess)  \
      return UBM_ERR_LAUNCH;                                                                                   \
    cudaLaunchConfig_t cfg = {};                                                                               \
    cfg.gridDim = dim3(grid);                                                                                  \
    cfg.blockDim = dim3(kGemvThreads);                                                                         \
    cfg.dynamicSmemBytes = smem;                                                                               \
    cfg.stream = st;                                                                                           \
    cudaLaunchAttribute attr[1];                                                                               \
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;                                           \
    attr[0].val.programmaticStreamSerializationAllowed = 1;                                                    \
    cfg.attrs = attr;                                                                                          \
    cfg.numAttrs = pdl ? 1 : 0;                                                                                \
    if (cudaLaunchKernelEx(&cfg, kern, x, gamma, eps, w, w2, bias, res, out, M, N, K, wscale) != cudaSuccess)  \
      return UBM_ERR_LAUNCH;                                                                                   \
  } while (0)
  switch (MB) {
    case 1: UBM_GEMV(1); break;
    case 2: UBM_GEMV(2); break;
    case 4: UBM_GEMV(4); break;
    default: UBM_GEMV(8); break;
  }
#undef UBM_GEMV
  UBM_CHECK_LAUNCH("gemv_rows_kernel");
  return UBM_OK;
}
}  // namespace ubm

// x: bf16 [M][K] (M <= 8), w / w2: bf16 [N][K] (rows contiguous, K a multiple of 8; w2 null unless the SwiGLU form
// is asked for), gamma: fp32 [K] or null, bias: fp32 [N] or null, res: bf16 [M][N] or null, out: bf16 [M][N]
extern "C" int ubm_gemv_fused(const void* x, const void* gamma, float eps, const void* w, const void* w2,
                              const void* bias, const void* res, void* out, int M, int N, int K, void* stream) {
  if (M < 1 || M > 8 || N < 1 || K < 8 || (K & 7) || !aligned16(x) || !aligned16(w) ||
      (w2 != nullptr && !aligned16(w2)) || (gamma != nullptr && !aligned16(gamma)))
    return UBM_ERR_ARGUMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* xx = static_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* ww = static_cast<const __nv_bfloat16*>(w);
  const __nv_bfloat16* w22 = static_cast<const __nv_bfloat16*>(w2);
  const __nv_bfloat16* rr = static_cast<const __nv_bfloat16*>(res);
  __nv_bfloat16* oo = static_cast<__nv_bfloat16*>(out);
  const float* gg = static_cast<const float*>(gamma);
  const float* bb = static_cast<const float*>(bias);
  return w2 != nullptr ? ubm::launch_gemv<true, false>(xx, gg, eps, ww, w22, bb, rr, oo, M, N, K, 1.f, st)
                       : ubm::launch_gemv<false, false>(xx, gg, eps, ww, w22, bb, rr, oo, M, N, K, 1.f, st);
}

// The same with the weights in e4m3: w8 [N][K] bytes (K a multiple of 16), wscale their dequantisation factor
extern "C" int ubm_gemv_fused_w8(const void* x, const void* gamma, float eps, const void* w8, float wscale,
                                 const void* bias, const void* res, void* out, int M, int N, int K, void* stream) {
  if (M < 1 || M > 8 || N < 1 || K < 16 || (K & 15) || !aligned16(x) || !aligned16(w8) ||
      (gamma != nullptr && !aligned16(gamma)))
    return UBM_ERR_ARGUMENT;
  return ubm::launch_gemv<false, true>(static_cast<const __nv_bfloat16*>(x), static_cast<const float*>(gamma), eps,
                                       static_cast<const __nv_bfloat16*>(w8), nullptr, static_cast<const float*>(bias),
                                       static_cast<const __nv_bfloat16*>(res), static_cast<__nv_bfloat16*>(out), M, N,
                                       K, wscale, static_cast<cudaStream_t>(stream));
}

extern "C" int ubm_gemv_rows(const void* x, const void* w, const void* bias, void* out, int M, int N, int K,
                             void* stream) {
  return ubm_gemv_fused(x, nullptr, 0.f, w, nullptr, bias, nullptr, out, M, N, K, stream);
}
