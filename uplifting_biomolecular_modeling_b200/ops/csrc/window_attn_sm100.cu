// Atom attention in sequence-local windows: 32 queries attend to the 128 keys centred on them
// (key window of query window w = atoms [32 w - 48, 32 w + 80), clipped to [0, A)), 4 heads x 32, with a
// per-window pair bias and the sigmoid gate fused in.  This op is small (a few GFLOP per diffusion step) and
// memory / launch bound, so it is a plain SIMT kernel: one CTA per (window, head, sample), K and V of the
// window staged in shared memory, four threads per query each owning a quarter of the keys, softmax and the
// P.V reduction finished with shuffles.  q is pre-scaled by log2(e)/sqrt(32) and the bias by log2(e).
// Reference kernels with the same boundary: common/opt_core/opt_core/kernels/atom_window.py
// (_window_attn_kernel), apb/fpf_apb (_atom_fwd).
#include "host_util.h"
#include "sm100.cuh"

namespace ubm {

constexpr int kWQ = 32, kWK = 128, kWD = 32;

struct WindowParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  const __nv_bfloat16* bias;  // [bias_batch][H][nw][32][128] or null
  const __nv_bfloat16* gate;  // [B][A][H*32] (already sigmoid) or null
  __nv_bfloat16* out;         // [B][A][H*32]
  int B, A, H, nw;
  long long ld_in;            // row stride of q / k / v
  int bias_batch;             // 1 = bias shared by all samples
};

__global__ void __launch_bounds__(128) window_attention_kernel(WindowParams p) {
  __shared__ __align__(16) __nv_bfloat16 sK[kWK][kWD + 8];   // +8 bf16 padding: rows 80 bytes apart
  __shared__ __align__(16) __nv_bfloat16 sV[kWK][kWD + 8];
  const int w = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int key0 = w * kWQ - (kWK - kWQ) / 2;
  const long long base = static_cast<long long>(b) * p.A;
  // stage K and V: 128 keys x 64 bytes each = 4 uint4 per key; 128 threads x 4 iterations
  for (int i = threadIdx.x; i < kWK * 4; i += blockDim.x) {
    const int key = i >> 2, c = i & 3;
    const int atom = key0 + key;
    uint4 kv = make_uint4(0, 0, 0, 0), vv = make_uint4(0, 0, 0, 0);
    if (atom >= 0 && atom < p.A) {
      const long long off = (base + atom) * p.ld_in + h * kWD + c * 8;
      kv = __ldg(reinterpret_cast<const uint4*>(p.k + off));
      vv = __ldg(reinterpret_cast<const uint4*>(p.v + off));
    }
    *reinterpret_cast<uint4*>(&sK[key][c * 8]) = kv;
    *reinterpret_cast<uint4*>(&sV[key][c * 8]) = vv;
  }
  const int qi = threadIdx.x >> 2;   // query in window
  const int part = threadIdx.x & 3;  // quarter of the keys
  const int atom_q = w * kWQ + qi;
  float qv[kWD];
  {
    const long long off = (base + atom_q) * p.ld_in + h * kWD;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint4 u = __ldg(reinterpret_cast<const uint4*>(p.q + off) + c);
      const uint32_t ww[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        qv[c * 8 + 2 * e] = bf16_lo(ww[e]);
        qv[c * 8 + 2 * e + 1] = bf16_hi(ww[e]);
      }
    }
  }
  __syncthreads();
  float s[32];
  const __nv_bfloat16* brow = nullptr;
  if (p.bias != nullptr) {
    const int bb = p.bias_batch == 1 ? 0 : b;
    brow = p.bias + ((((static_cast<long long>(bb) * p.H + h) * p.nw + w) * kWQ + qi) * kWK) + part * 32;
  }
  float mx = -1.0e30f;
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    const int key = part * 32 + j;
    const int atom = key0 + key;
    float acc = 0.f;
#pragma unroll
    for (int c = 0; c < kWD; c += 2) {
      const __nv_bfloat162 kk = *reinterpret_cast<const __nv_bfloat162*>(&sK[key][c]);
      acc += qv[c] * __low2float(kk) + qv[c + 1] * __high2float(kk);
    }
    if (brow != nullptr) acc += __bfloat162float(brow[j]);
    if (atom < 0 || atom >= p.A) acc = -1.0e30f;
    s[j] = acc;
    mx = fmaxf(mx, acc);
  }
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
  float l = 0.f;
  float o[kWD];
#pragma unroll
  for (int c = 0; c < kWD; ++c) o[c] = 0.f;
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    const float pj = fast_exp2(s[j] - mx);
    l += pj;
    const int key = part * 32 + j;
#pragma unroll
    for (int c = 0; c < kWD; c += 2) {
      const __nv_bfloat162 vv = *reinterpret_cast<const __nv_bfloat162*>(&sV[key][c]);
      o[c] += pj * __low2float(vv);
      o[c + 1] += pj * __high2float(vv);
    }
  }
  l += __shfl_xor_sync(0xffffffffu, l, 1);
  l += __shfl_xor_sync(0xffffffffu, l, 2);
#pragma unroll
  for (int c = 0; c < kWD; ++c) {
    o[c] += __shfl_xor_sync(0xffffffffu, o[c], 1);
    o[c] += __shfl_xor_sync(0xffffffffu, o[c], 2);
  }
  // each of the four threads of a query writes 8 of the 32 output channels
  const float inv = 1.0f / l;
  const long long orow = (base + atom_q) * (p.H * kWD) + h * kWD + part * 8;
  float f[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) f[e] = o[part * 8 + e] * inv;
  if (p.gate != nullptr) {
    const uint4 u = __ldg(reinterpret_cast<const uint4*>(p.gate + orow));
    const uint32_t ww[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      f[2 * e] *= bf16_lo(ww[e]);
      f[2 * e + 1] *= bf16_hi(ww[e]);
    }
  }
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]);
  u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]);
  u.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p.out + orow) = u;
}

}  // namespace ubm

// q, k, v: bf16 rows [B*A] with row stride ld_in (elements), head h at columns h*32..; A a multiple of 32.
// bias: bf16 [bias_batch][H][A/32][32][128] or null; gate / out: bf16 [B*A][H*32].
extern "C" int ubm_window_attention(const void* q, const void* k, const void* v, const void* bias, const void* gate,
                                    void* out, int B, int A, int H, long long ld_in, int bias_batch, void* stream) {
  using namespace ubm;
  if (B <= 0 || A <= 0 || (A % kWQ) || H <= 0 || ld_in < H * kWD || (ld_in & 7)) return UBM_ERR_ARGUMENT;
  WindowParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k = static_cast<const __nv_bfloat16*>(k);
  p.v = static_cast<const __nv_bfloat16*>(v);
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.gate = static_cast<const __nv_bfloat16*>(gate);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.B = B;
  p.A = A;
  p.H = H;
  p.nw = A / kWQ;
  p.ld_in = ld_in;
  p.bias_batch = bias_batch;
  dim3 grid(p.nw, H, B);
  window_attention_kernel<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(p);
  UBM_CHECK_LAUNCH("window_attention_kernel");
  return UBM_OK;
}
