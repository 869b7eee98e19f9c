// Single-query attention over a fixed-size key / value cache (the attention layers of StripedHyena-2 in a captured
// decode step).  Memory bound: every key and value row up to the current position is read once, 16 bytes per
// lane, four keys and four values per half warp in flight; nothing of the step depends on a host value (the
// position is read from device memory), so the launches can sit in a CUDA graph.
//
//   decode_qkv      rotary embedding of the new query and key at the position, key / value rows written into
//                   the cache, rotated query written out                        (one launch)
//   decode_attn     split over the keys: grid (splits, heads, batch); online softmax per half warp, merged per
//                   CTA, one (max, sum, 128 partial outputs) record per split   (one launch)
//   decode_merge    merges the splits and writes the bf16 output row            (one launch)
//
// Head dimension 128.  The plain statement this replaces: two einsums, a mask over the dead part of the cache
// and a softmax (models/evo2.py, AttentionOperator.step); upstream's decode path keeps the same fixed cache
// (evo2 generation with an inference-params cache).
#include <cstdint>

#include "host_util.h"
#include "sm100.cuh"

namespace ubm {

constexpr int kDecHd = 128;
constexpr int kDecThreads = 256;               // 16 half warps, one key each per step
static inline bool dec_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
constexpr int kDecRec = kDecHd + 2;            // partial record: outputs, running max (log2 domain), running sum

__device__ __forceinline__ void dec_unpack8(const uint4& u, float (&e)[8]) {
  e[0] = bf16_lo(u.x); e[1] = bf16_hi(u.x); e[2] = bf16_lo(u.y); e[3] = bf16_hi(u.y);
  e[4] = bf16_lo(u.z); e[5] = bf16_hi(u.z); e[6] = bf16_lo(u.w); e[7] = bf16_hi(u.w);
}

// qkv: bf16 [B][3][H][128]; pos: int64 [1]; q_out: bf16 [B][H][128]; kc / vc: bf16 [B][Lmax][H][128]
__global__ void __launch_bounds__(256) decode_qkv_kernel(const __nv_bfloat16* __restrict__ qkv,
                                                         const long long* __restrict__ pos_ptr,
                                                         __nv_bfloat16* __restrict__ q_out,
                                                         __nv_bfloat16* __restrict__ kc, __nv_bfloat16* __restrict__ vc,
                                                         int B, int H, int Lmax, float base, KernelStatus* status) {
  const long long pos = *pos_ptr;
  if (pos < 0 || pos >= Lmax) {                 // a full cache: nothing is written, the host reads the word
    if (blockIdx.x == 0 && threadIdx.x == 0 && atomicCAS(&status->code, 0u, 3u) == 0u) {
      status->where = 120u;
      status->block = 0u;
      status->aux = static_cast<unsigned int>(pos);
    }
    return;
  }
  const int half = kDecHd / 2;
  const int total = B * H * half;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int p = i % half;
    const int h = (i / half) % H;
    const int b = i / (half * H);
    const long long src = (static_cast<long long>(b) * 3 * H + h) * kDecHd + 2 * p;
    const long long hs = static_cast<long long>(H) * kDecHd;
    const __nv_bfloat162 qv = *reinterpret_cast<const __nv_bfloat162*>(qkv + src);
    const __nv_bfloat162 kv = *reinterpret_cast<const __nv_bfloat162*>(qkv + src + hs);
    const __nv_bfloat162 vv = *reinterpret_cast<const __nv_bfloat162*>(qkv + src + 2 * hs);
    const float inv = 1.0f / powf(base, static_cast<float>(2 * p) / static_cast<float>(kDecHd));
    float sn, cs;
    sincosf(static_cast<float>(pos) * inv, &sn, &cs);
    const float q0 = __bfloat162float(qv.x), q1 = __bfloat162float(qv.y);
    const float k0 = __bfloat162float(kv.x), k1 = __bfloat162float(kv.y);
    const long long row = ((static_cast<long long>(b) * Lmax + pos) * H + h) * kDecHd + 2 * p;
    *reinterpret_cast<__nv_bfloat162*>(q_out + (static_cast<long long>(b) * H + h) * kDecHd + 2 * p) =
        __floats2bfloat162_rn(q0 * cs - q1 * sn, q0 * sn + q1 * cs);
    *reinterpret_cast<__nv_bfloat162*>(kc + row) = __floats2bfloat162_rn(k0 * cs - k1 * sn, k0 * sn + k1 * cs);
    *reinterpret_cast<__nv_bfloat162*>(vc + row) = vv;
  }
}

// q: bf16 [B][H][128]; kc / vc: bf16 [B][Lmax][H][128]; part: fp32 [B][H][S][130]
__global__ void __launch_bounds__(kDecThreads) decode_attn_kernel(const __nv_bfloat16* __restrict__ q,
                                                                  const __nv_bfloat16* __restrict__ kc,
                                                                  const __nv_bfloat16* __restrict__ vc,
                                                                  const long long* __restrict__ pos_ptr,
                                                                  float* __restrict__ part, int H, int Lmax, int chunk,
                                                                  float scale_log2e) {
  __shared__ float s_acc[kDecThreads / 16][kDecHd];
  __shared__ float s_m[kDecThreads / 16], s_l[kDecThreads / 16];
  const int s = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int S = gridDim.x;
  long long n_keys = *pos_ptr + 1;                                   // keys 0 .. pos are alive
  if (n_keys > Lmax) n_keys = Lmax;
  const int k_begin = s * chunk;
  const int k_end = static_cast<int>(min(static_cast<long long>(k_begin) + chunk, n_keys));
  float* rec = part + ((static_cast<long long>(b) * H + h) * S + s) * kDecRec;
  if (k_begin >= k_end) {                                            // nothing alive in this split
    if (threadIdx.x == 0) {
      rec[kDecHd] = -INFINITY;
      rec[kDecHd + 1] = 0.f;
    }
    return;
  }
  const int hw = threadIdx.x >> 4;                                   // half warp
  const unsigned int hmask = (hw & 1) ? 0xffff0000u : 0x0000ffffu;   // the two halves of a warp run different trip counts
  const int l16 = threadIdx.x & 15;                                  // 8 head dimensions each
  float qf[8];
  dec_unpack8(*reinterpret_cast<const uint4*>(q + (static_cast<long long>(b) * H + h) * kDecHd + l16 * 8), qf);
#pragma unroll
  for (int e = 0; e < 8; ++e) qf[e] *= scale_log2e;
  const long long row_stride = static_cast<long long>(H) * kDecHd;
  const __nv_bfloat16* kb = kc + (static_cast<long long>(b) * Lmax * H + h) * kDecHd + l16 * 8;
  const __nv_bfloat16* vb = vc + (static_cast<long long>(b) * Lmax * H + h) * kDecHd + l16 * 8;
  float m = -INFINITY, l = 0.f;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  constexpr int kHw = kDecThreads / 16;
  for (int k0 = k_begin + hw; k0 < k_end; k0 += 4 * kHw) {           // the first key of a batch is alive
    uint4 kv[4], vv[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int k = k0 + u * kHw;
      if (k < k_end) {
        kv[u] = __ldcs(reinterpret_cast<const uint4*>(kb + k * row_stride));
        vv[u] = __ldcs(reinterpret_cast<const uint4*>(vb + k * row_stride));
      }
    }
    float sc[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int k = k0 + u * kHw;
      float d = 0.f;
      if (k < k_end) {
        float kf[8];
        dec_unpack8(kv[u], kf);
#pragma unroll
        for (int e = 0; e < 8; ++e) d = fmaf(qf[e], kf[e], d);
      }
      d += __shfl_xor_sync(hmask, d, 8);
      d += __shfl_xor_sync(hmask, d, 4);
      d += __shfl_xor_sync(hmask, d, 2);
      d += __shfl_xor_sync(hmask, d, 1);
      sc[u] = k < k_end ? d : -INFINITY;
    }
    const float m_new = fmaxf(fmaxf(fmaxf(m, sc[0]), fmaxf(sc[1], sc[2])), sc[3]);   // finite: sc[0] is
    const float corr = exp2f(m - m_new);                                             // 0 on the first batch
    float psum = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] *= corr;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float p = exp2f(sc[u] - m_new);                                          // 0 for a dead key
      psum += p;
      if (k0 + u * kHw < k_end) {
        float vf[8];
        dec_unpack8(vv[u], vf);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = fmaf(p, vf[e], acc[e]);
      }
    }
    l = l * corr + psum;
    m = m_new;
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) s_acc[hw][l16 * 8 + e] = acc[e];
  if (l16 == 0) {
    s_m[hw] = m;
    s_l[hw] = l;
  }
  __syncthreads();
  if (threadIdx.x < kDecHd) {
    float M = -INFINITY;
#pragma unroll
    for (int i = 0; i < kHw; ++i) M = fmaxf(M, s_m[i]);              // finite: half warp 0 saw key k_begin
    float o = 0.f, L = 0.f;
#pragma unroll
    for (int i = 0; i < kHw; ++i) {
      if (s_m[i] > -INFINITY) {
        const float w = exp2f(s_m[i] - M);
        o = fmaf(w, s_acc[i][threadIdx.x], o);
        L = fmaf(w, s_l[i], L);
      }
    }
    rec[threadIdx.x] = o;
    if (threadIdx.x == 0) {
      rec[kDecHd] = M;
      rec[kDecHd + 1] = L;
    }
  }
}

// part: fp32 [B][H][S][130] -> out: bf16 [B][H][128]
__global__ void __launch_bounds__(kDecHd) decode_merge_kernel(const float* __restrict__ part,
                                                              __nv_bfloat16* __restrict__ out, int H, int S) {
  const int h = blockIdx.x, b = blockIdx.y;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the projection behind may prefetch its weights
  const float* rec = part + (static_cast<long long>(b) * H + h) * S * kDecRec;
  float M = -INFINITY;
  for (int s = 0; s < S; ++s) M = fmaxf(M, rec[s * kDecRec + kDecHd]);
  float o = 0.f, L = 0.f;
  for (int s = 0; s < S; ++s) {
    const float ms = rec[s * kDecRec + kDecHd];
    if (ms > -INFINITY) {
      const float w = exp2f(ms - M);
      o = fmaf(w, rec[s * kDecRec + threadIdx.x], o);
      L = fmaf(w, rec[s * kDecRec + kDecHd + 1], L);
    }
  }
  out[(static_cast<long long>(b) * H + h) * kDecHd + threadIdx.x] = __float2bfloat16(L > 0.f ? o / L : 0.f);
}

}  // namespace ubm

// qkv: bf16 [B][3*H*128] (q | k | v of the new token, heads of 128); pos: int64 [1] on the device (the index the
// new key takes; keys 0..pos are attended); kc / vc: bf16 [B][Lmax][H][128] (row pos is written); q_rot: bf16
// [B][H][128] scratch; part: fp32 [B][H][splits][130] scratch; out: bf16 [B][H*128]; status: the device status record: code 3 (bad
// argument), site 120, aux = pos when pos is outside the cache (then nothing is written).
extern "C" int ubm_decode_attention(const void* qkv, const void* pos, void* kc, void* vc, void* q_rot, void* part,
                                    void* out, int B, int H, int Lmax, int splits, float rope_base, float scale,
                                    void* status, void* stream) {
  using namespace ubm;
  if (B < 1 || B > 65535 || H < 1 || H > 65535 || Lmax < 1 || splits < 1 || splits > 1024 || !dec_aligned16(qkv) ||
      !dec_aligned16(kc) || !dec_aligned16(vc) || !dec_aligned16(q_rot) || !dec_aligned16(out) || status == nullptr)
    return UBM_ERR_ARGUMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int chunk = (Lmax + splits - 1) / splits;
  const int total = B * H * (kDecHd / 2);
  decode_qkv_kernel<<<(total + 255) / 256, 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(qkv), static_cast<const long long*>(pos), static_cast<__nv_bfloat16*>(q_rot),
      static_cast<__nv_bfloat16*>(kc), static_cast<__nv_bfloat16*>(vc), B, H, Lmax, rope_base,
      static_cast<KernelStatus*>(status));
  UBM_CHECK_LAUNCH("decode_qkv_kernel");
  decode_attn_kernel<<<dim3(splits, H, B), kDecThreads, 0, st>>>(
      static_cast<const __nv_bfloat16*>(q_rot), static_cast<const __nv_bfloat16*>(kc),
      static_cast<const __nv_bfloat16*>(vc), static_cast<const long long*>(pos), static_cast<float*>(part), H, Lmax,
      chunk, scale * 1.4426950408889634f);
  UBM_CHECK_LAUNCH("decode_attn_kernel");
  decode_merge_kernel<<<dim3(H, B), kDecHd, 0, st>>>(static_cast<const float*>(part), static_cast<__nv_bfloat16*>(out),
                                                     H, splits);
  UBM_CHECK_LAUNCH("decode_merge_kernel");
  return UBM_OK;
}
