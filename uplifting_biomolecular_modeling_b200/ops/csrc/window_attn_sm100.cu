// Atom attention in sequence-local windows: 32 queries attend to the 128 keys centred on them
// (key window of query window w = atoms [32 w - 48, 32 w + 80), clipped to [0, A)), 4 heads x 32, with a
// per-window pair bias and the sigmoid gate fused in.  This op is small (a few GFLOP per diffusion step) and
// memory / launch bound, so it is a plain SIMT kernel: one CTA per (window, head, sample), K and V of the
// window staged in shared memory as fp32, four threads per query each owning every fourth key, packed
// two-wide fp32 FMAs for both products, softmax and the P.V reduction finished with shuffles.  q is pre-scaled by log2(e)/sqrt(32) and the bias by log2(e).
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

__device__ __forceinline__ float2 splat2(float x) { return make_float2(x, x); }

// Shared-memory layout: K and V of the window as fp32, 36 floats per key (144 bytes).  The four threads of
// a query take interleaved keys (key = 4 j + part), so the four rows a warp reads in one instruction are
// consecutive: 144 bytes apart = 4 banks apart, and the 16-byte reads do not collide.  (Rows 32 keys apart
// would all start in bank 0.)  The dot products run as packed two-wide fp32 FMAs.
__global__ void __launch_bounds__(128) window_attention_kernel(WindowParams p) {
  constexpr int kLd = kWD + 4;
  __shared__ __align__(16) float sK[kWK][kLd];
  __shared__ __align__(16) float sV[kWK][kLd];
  const int w = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int key0 = w * kWQ - (kWK - kWQ) / 2;
  const long long base = static_cast<long long>(b) * p.A;
  // stage K and V: 128 keys x 4 chunks of 8 bf16, widened to fp32 once here
  for (int i = threadIdx.x; i < kWK * 4; i += blockDim.x) {
    const int key = i >> 2, c = i & 3;
    const int atom = key0 + key;
    uint4 kv = make_uint4(0, 0, 0, 0), vv = make_uint4(0, 0, 0, 0);
    if (atom >= 0 && atom < p.A) {
      const long long off = (base + atom) * p.ld_in + h * kWD + c * 8;
      kv = __ldg(reinterpret_cast<const uint4*>(p.k + off));
      vv = __ldg(reinterpret_cast<const uint4*>(p.v + off));
    }
    float4* dk = reinterpret_cast<float4*>(&sK[key][c * 8]);
    float4* dv = reinterpret_cast<float4*>(&sV[key][c * 8]);
    dk[0] = make_float4(bf16_lo(kv.x), bf16_hi(kv.x), bf16_lo(kv.y), bf16_hi(kv.y));
    dk[1] = make_float4(bf16_lo(kv.z), bf16_hi(kv.z), bf16_lo(kv.w), bf16_hi(kv.w));
    dv[0] = make_float4(bf16_lo(vv.x), bf16_hi(vv.x), bf16_lo(vv.y), bf16_hi(vv.y));
    dv[1] = make_float4(bf16_lo(vv.z), bf16_hi(vv.z), bf16_lo(vv.w), bf16_hi(vv.w));
  }
  const int qi = threadIdx.x >> 2;   // query in window
  const int part = threadIdx.x & 3;  // keys 4 j + part
  const int atom_q = w * kWQ + qi;
  float2 q2[kWD / 2];
  {
    const long long off = (base + atom_q) * p.ld_in + h * kWD;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint4 u = __ldg(reinterpret_cast<const uint4*>(p.q + off) + c);
      q2[c * 4 + 0] = make_float2(bf16_lo(u.x), bf16_hi(u.x));
      q2[c * 4 + 1] = make_float2(bf16_lo(u.y), bf16_hi(u.y));
      q2[c * 4 + 2] = make_float2(bf16_lo(u.z), bf16_hi(u.z));
      q2[c * 4 + 3] = make_float2(bf16_lo(u.w), bf16_hi(u.w));
    }
  }
  const __nv_bfloat16* brow = nullptr;
  if (p.bias != nullptr) {
    const int bb = p.bias_batch == 1 ? 0 : b;
    brow = p.bias + ((((static_cast<long long>(bb) * p.H + h) * p.nw + w) * kWQ + qi) * kWK) + part;
  }
  float bj[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) bj[j] = brow != nullptr ? __bfloat162float(brow[4 * j]) : 0.f;
  __syncthreads();
  float s[32];
  float mx = -1.0e30f;
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    const int key = 4 * j + part;
    const int atom = key0 + key;
    float2 a0 = make_float2(0.f, 0.f), a1 = make_float2(0.f, 0.f);
#pragma unroll
    for (int c = 0; c < kWD / 4; ++c) {
      const float4 kk = *reinterpret_cast<const float4*>(&sK[key][c * 4]);
      a0 = __ffma2_rn(q2[2 * c], make_float2(kk.x, kk.y), a0);
      a1 = __ffma2_rn(q2[2 * c + 1], make_float2(kk.z, kk.w), a1);
    }
    float acc = (a0.x + a0.y) + (a1.x + a1.y) + bj[j];
    if (atom < 0 || atom >= p.A) acc = -1.0e30f;
    s[j] = acc;
    mx = fmaxf(mx, acc);
  }
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
  mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
  float l = 0.f;
  float2 o2[kWD / 2];
#pragma unroll
  for (int c = 0; c < kWD / 2; ++c) o2[c] = make_float2(0.f, 0.f);
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    const float pj = fast_exp2(s[j] - mx);
    l += pj;
    const float2 pp = splat2(pj);
    const int key = 4 * j + part;
#pragma unroll
    for (int c = 0; c < kWD / 4; ++c) {
      const float4 vv = *reinterpret_cast<const float4*>(&sV[key][c * 4]);
      o2[2 * c] = __ffma2_rn(pp, make_float2(vv.x, vv.y), o2[2 * c]);
      o2[2 * c + 1] = __ffma2_rn(pp, make_float2(vv.z, vv.w), o2[2 * c + 1]);
    }
  }
  l += __shfl_xor_sync(0xffffffffu, l, 1);
  l += __shfl_xor_sync(0xffffffffu, l, 2);
  // Sum over the four threads of a query while splitting the channels between them: after the exchange
  // with lane ^ 1 a thread holds 16 channels (the upper half where bit 0 of part is set), after lane ^ 2
  // eight; no register array is indexed by a run-time value.
  const bool b0 = part & 1, b1 = part & 2;
  float r16[16];
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const float2 lo = o2[c], hi = o2[c + 8];
    const float2 send = b0 ? lo : hi;
    const float2 keep = b0 ? hi : lo;
    r16[2 * c] = keep.x + __shfl_xor_sync(0xffffffffu, send.x, 1);
    r16[2 * c + 1] = keep.y + __shfl_xor_sync(0xffffffffu, send.y, 1);
  }
  float f[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const float send = b1 ? r16[c] : r16[c + 8];
    const float keep = b1 ? r16[c + 8] : r16[c];
    f[c] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
  }
  const int ch0 = (b0 ? 16 : 0) + (b1 ? 8 : 0);
  const float inv = 1.0f / l;
  const long long orow = (base + atom_q) * (p.H * kWD) + h * kWD + ch0;
#pragma unroll
  for (int e = 0; e < 8; ++e) f[e] *= inv;
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
