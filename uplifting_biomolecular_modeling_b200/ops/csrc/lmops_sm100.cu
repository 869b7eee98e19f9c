// Attention-side kernels of the protein-LM and genomic-track families that are not plain row maps.
//
//   column_attention     per sequence column: one query attends over C clade rows of an alignment whose K / V rows are
//                        stored once per distinct row (clade -> row gather index), optional per-head clade bias
//   relshift_softmax     softmax over keys of content[i][j] + pos[i][j - i + L - 1]: the relative-position logits
//                        are read at their shifted index instead of being materialised as a shifted copy
//
// Reference kernels with the same boundaries: gpnstar accel/fused_col.py:56-195 (column scores / context through a
// gather index), enformer_deepmind ops/edm_softmax.cu.cc:54 (relative shift + softmax),
// enformer kits/v0_2/enformer_xattn.cu:24-45 (content + positional logits softmax).
#include "host_util.h"
#include "sm100.cuh"

namespace ubm {

static inline int lm_grid(long long work, int per_block) {
  long long b = (work + per_block - 1) / per_block;
  const long long cap = static_cast<long long>(sm_count()) * 32;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}

constexpr int kColMaxClades = 256;
static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// q: bf16 [T][H][D]; k, v: bf16 [R][T][H][D]; idx: int32 [C] (clade -> row); bias: fp32 [H][C] or null;
// out: bf16 [T][H][D].  One warp per (t, h): lanes over clades for the scores, lanes over channels for the
// context.  D = 32 or 64, C <= 256.
template <int D>
__global__ void __launch_bounds__(256) column_attention_kernel(const __nv_bfloat16* __restrict__ q,
                                                               const __nv_bfloat16* __restrict__ k,
                                                               const __nv_bfloat16* __restrict__ v,
                                                               const int* __restrict__ idx,
                                                               const float* __restrict__ bias,
                                                               __nv_bfloat16* __restrict__ out, long long T, int H,
                                                               int C, float scale) {
  constexpr int kPer = kColMaxClades / 32;
  constexpr int kDL = D / 32;                     // channels per lane in the context phase
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const long long rows = T * H;
  const long long row_stride = rows * D;          // elements between alignment rows
  for (long long w = static_cast<long long>(blockIdx.x) * wpb + (threadIdx.x >> 5); w < rows;
       w += static_cast<long long>(gridDim.x) * wpb) {
    const int h = static_cast<int>(w % H);
    const long long off = w * D;
    float qf[D];
#pragma unroll
    for (int d = 0; d < D; d += 8) {
      const uint4 u = *reinterpret_cast<const uint4*>(q + off + d);
      qf[d + 0] = bf16_lo(u.x); qf[d + 1] = bf16_hi(u.x); qf[d + 2] = bf16_lo(u.y); qf[d + 3] = bf16_hi(u.y);
      qf[d + 4] = bf16_lo(u.z); qf[d + 5] = bf16_hi(u.z); qf[d + 6] = bf16_lo(u.w); qf[d + 7] = bf16_hi(u.w);
    }
    float s[kPer];
    float mx = -3.0e38f;
#pragma unroll
    for (int ci = 0; ci < kPer; ++ci) {
      const int c = ci * 32 + lane;
      s[ci] = -3.0e38f;
      if (c < C) {
        const __nv_bfloat16* kp = k + static_cast<long long>(idx[c]) * row_stride + off;
        float acc = 0.f;
#pragma unroll
        for (int d = 0; d < D; d += 8) {
          const uint4 u = *reinterpret_cast<const uint4*>(kp + d);
          acc = fmaf(qf[d + 0], bf16_lo(u.x), acc); acc = fmaf(qf[d + 1], bf16_hi(u.x), acc);
          acc = fmaf(qf[d + 2], bf16_lo(u.y), acc); acc = fmaf(qf[d + 3], bf16_hi(u.y), acc);
          acc = fmaf(qf[d + 4], bf16_lo(u.z), acc); acc = fmaf(qf[d + 5], bf16_hi(u.z), acc);
          acc = fmaf(qf[d + 6], bf16_lo(u.w), acc); acc = fmaf(qf[d + 7], bf16_hi(u.w), acc);
        }
        s[ci] = acc * scale + (bias != nullptr ? bias[static_cast<long long>(h) * C + c] : 0.f);
        mx = fmaxf(mx, s[ci]);
      }
    }
#pragma unroll
    for (int sh = 16; sh > 0; sh >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, sh));
    float sum = 0.f;
#pragma unroll
    for (int ci = 0; ci < kPer; ++ci) {
      const int c = ci * 32 + lane;
      s[ci] = c < C ? __expf(s[ci] - mx) : 0.f;
      sum += s[ci];
    }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    float acc[kDL];
#pragma unroll
    for (int j = 0; j < kDL; ++j) acc[j] = 0.f;
#pragma unroll
    for (int ci = 0; ci < kPer; ++ci) {
      if (ci * 32 < C) {
        const int lim = min(32, C - ci * 32);
        for (int cl = 0; cl < lim; ++cl) {
          const float p = __shfl_sync(0xffffffffu, s[ci], cl);
          const __nv_bfloat16* vp = v + static_cast<long long>(idx[ci * 32 + cl]) * row_stride + off + lane * kDL;
          if (kDL == 2) {
            const uint32_t u = *reinterpret_cast<const uint32_t*>(vp);
            acc[0] = fmaf(p, bf16_lo(u), acc[0]);
            acc[kDL - 1] = fmaf(p, bf16_hi(u), acc[kDL - 1]);
          } else {
            acc[0] = fmaf(p, __bfloat162float(vp[0]), acc[0]);
          }
        }
      }
    }
    if (kDL == 2) {
      *reinterpret_cast<uint32_t*>(out + off + lane * 2) = pack_bf16x2(acc[0] * inv, acc[kDL - 1] * inv);
    } else {
      out[off + lane] = __float2bfloat16(acc[0] * inv);
    }
  }
}

// content: fp32 [R][L] with R = batch * heads * L query rows (row r is query i = r % L); pos: fp32 [R][ldp] with
// ldp >= 2L - 1; out: fp32 [R][L] = softmax_j(content[r][j] + pos[r][j - i + L - 1]).  One warp per row.
__global__ void __launch_bounds__(256) relshift_softmax_kernel(const float* __restrict__ content,
                                                               const float* __restrict__ pos,
                                                               float* __restrict__ out, long long R, int L, int ldp) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (long long r = static_cast<long long>(blockIdx.x) * wpb + (threadIdx.x >> 5); r < R;
       r += static_cast<long long>(gridDim.x) * wpb) {
    const int i = static_cast<int>(r % L);
    const float* cp = content + r * L;
    const float* pp = pos + r * ldp + (L - 1 - i);
    float mx = -3.0e38f;
    for (int j = lane; j < L; j += 32) mx = fmaxf(mx, cp[j] + pp[j]);
#pragma unroll
    for (int sh = 16; sh > 0; sh >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, sh));
    float sum = 0.f;
    for (int j = lane; j < L; j += 32) sum += __expf(cp[j] + pp[j] - mx);
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    float* op = out + r * L;
    for (int j = lane; j < L; j += 32) op[j] = __expf(cp[j] + pp[j] - mx) * inv;
  }
}

}  // namespace ubm

using namespace ubm;

extern "C" int ubm_column_attention(const void* q, const void* k, const void* v, const void* idx, const void* bias,
                                    void* out, long long T, int H, int D, int C, float scale, void* stream) {
  if (T <= 0 || H <= 0 || C <= 0 || C > kColMaxClades || (D != 32 && D != 64) || !aligned16(q) || !aligned16(k) ||
      !aligned16(v))
    return UBM_ERR_ARGUMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = lm_grid(T * H, 8);
  const __nv_bfloat16* qq = static_cast<const __nv_bfloat16*>(q);
  const __nv_bfloat16* kk = static_cast<const __nv_bfloat16*>(k);
  const __nv_bfloat16* vv = static_cast<const __nv_bfloat16*>(v);
  if (D == 32)
    column_attention_kernel<32><<<grid, 256, 0, st>>>(qq, kk, vv, static_cast<const int*>(idx),
                                                      static_cast<const float*>(bias),
                                                      static_cast<__nv_bfloat16*>(out), T, H, C, scale);
  else
    column_attention_kernel<64><<<grid, 256, 0, st>>>(qq, kk, vv, static_cast<const int*>(idx),
                                                      static_cast<const float*>(bias),
                                                      static_cast<__nv_bfloat16*>(out), T, H, C, scale);
  UBM_CHECK_LAUNCH("column_attention_kernel");
  return UBM_OK;
}

extern "C" int ubm_relshift_softmax(const void* content, const void* pos, void* out, long long R, int L, int ldp,
                                    void* stream) {
  if (R <= 0 || L <= 0 || R % L != 0 || ldp < 2 * L - 1) return UBM_ERR_ARGUMENT;
  relshift_softmax_kernel<<<lm_grid(R, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float*>(content), static_cast<const float*>(pos), static_cast<float*>(out), R, L, ldp);
  UBM_CHECK_LAUNCH("relshift_softmax_kernel");
  return UBM_OK;
}
