// Template embedder of the AlphaFold3-architecture engines (Algorithm 16) around its pair stack:
//   embed: v[t][i][j][:] = W_dgram dg[t][i][j][0:39] + w_pb (pb[t][i] pb[t][j] same[i][j]) + ri[t][i][:] + rj[t][j][:]
//                          + w_x ux + w_y uy + w_z uz + w_bb (bb[t][i] bb[t][j] same[i][j]) + zp[i][j][:]
//          (eight bias-free Linears of the plain statements, summed in fp32 and rounded to bf16 once; the two
//          residue-type terms arrive as per-token tables ri, rj; zp = linear_z(LayerNorm(z)))
//   tail:  u[i][j][:] = relu(mean_t s[t][i][j][:])            (the output projection W_t is a GEMM on u)
// c_t = 64 channels, 39 distogram bins.  Memory bound (about 210 bytes in, 128 out per pair and template): a thread
// owns 8 channels of one pair, the 39 x 64 distogram weights sit in shared memory.
// Reference kernels with the same boundary: common/opt_core/opt_core/kernels/templ_embed.py (_embed_kernel :58,
// _tail_kernel :99).
#include "host_util.h"
#include "sm100.cuh"

namespace ubm {

constexpr int kTC = 64;      // template pair width
constexpr int kTDG = 39;     // distogram bins

struct TemplParams {
  const __nv_bfloat16* dg;    // [T][N][N][39]
  const __nv_bfloat16* uv;    // [T][N][N][3]
  const float* pbm;           // [T][N] pseudo-beta mask
  const float* bbm;           // [T][N] backbone mask
  const int* asym;            // [N] chain id
  const __nv_bfloat16* ri;    // [T][N][64]
  const __nv_bfloat16* rj;    // [T][N][64]
  const __nv_bfloat16* zp;    // [N][N][64]
  const float* w_dgram;       // [39][64] (transposed)
  const float* w_vec;         // [5][64]: w_pb, w_x, w_y, w_z, w_bb
  __nv_bfloat16* out;         // [T][N][N][64]
  int T, N;
};

__global__ void __launch_bounds__(256) template_embed_kernel(TemplParams p) {
  __shared__ __align__(16) float sW[(kTDG + 5) * kTC];
  for (int i = threadIdx.x; i < kTDG * kTC; i += blockDim.x) sW[i] = p.w_dgram[i];
  for (int i = threadIdx.x; i < 5 * kTC; i += blockDim.x) sW[kTDG * kTC + i] = p.w_vec[i];
  __syncthreads();
  const long long NN = static_cast<long long>(p.N) * p.N;
  const long long total = static_cast<long long>(p.T) * NN * 8;     // 8 channel groups per pair
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int cg = static_cast<int>(idx & 7) * 8;
    const long long pair = idx >> 3;            // t * N * N + i * N + j
    const int t = static_cast<int>(pair / NN);
    const long long ij = pair - static_cast<long long>(t) * NN;
    const int i = static_cast<int>(ij / p.N), j = static_cast<int>(ij - static_cast<long long>(i) * p.N);
    float acc[8];
    {
      const uint4 z = *reinterpret_cast<const uint4*>(p.zp + ij * kTC + cg);
      const uint4 a = *reinterpret_cast<const uint4*>(p.ri + (static_cast<long long>(t) * p.N + i) * kTC + cg);
      const uint4 b = *reinterpret_cast<const uint4*>(p.rj + (static_cast<long long>(t) * p.N + j) * kTC + cg);
      const uint32_t zw[4] = {z.x, z.y, z.z, z.w}, aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        acc[2 * k] = bf16_lo(zw[k]) + bf16_lo(aw[k]) + bf16_lo(bw[k]);
        acc[2 * k + 1] = bf16_hi(zw[k]) + bf16_hi(aw[k]) + bf16_hi(bw[k]);
      }
    }
    const float same = p.asym[i] == p.asym[j] ? 1.0f : 0.0f;
    const float pbp = p.pbm[static_cast<long long>(t) * p.N + i] * p.pbm[static_cast<long long>(t) * p.N + j] * same;
    const float bbp = p.bbm[static_cast<long long>(t) * p.N + i] * p.bbm[static_cast<long long>(t) * p.N + j] * same;
    const __nv_bfloat16* uvp = p.uv + pair * 3;
    const float sc[5] = {pbp, __bfloat162float(uvp[0]), __bfloat162float(uvp[1]), __bfloat162float(uvp[2]), bbp};
#pragma unroll
    for (int s = 0; s < 5; ++s) {
      const float4 w0 = *reinterpret_cast<const float4*>(sW + (kTDG + s) * kTC + cg);
      const float4 w1 = *reinterpret_cast<const float4*>(sW + (kTDG + s) * kTC + cg + 4);
      acc[0] = fmaf(sc[s], w0.x, acc[0]); acc[1] = fmaf(sc[s], w0.y, acc[1]);
      acc[2] = fmaf(sc[s], w0.z, acc[2]); acc[3] = fmaf(sc[s], w0.w, acc[3]);
      acc[4] = fmaf(sc[s], w1.x, acc[4]); acc[5] = fmaf(sc[s], w1.y, acc[5]);
      acc[6] = fmaf(sc[s], w1.z, acc[6]); acc[7] = fmaf(sc[s], w1.w, acc[7]);
    }
    const __nv_bfloat16* dgp = p.dg + pair * kTDG;
#pragma unroll 13
    for (int b = 0; b < kTDG; ++b) {
      const float d = __bfloat162float(dgp[b]);
      const float4 w0 = *reinterpret_cast<const float4*>(sW + b * kTC + cg);
      const float4 w1 = *reinterpret_cast<const float4*>(sW + b * kTC + cg + 4);
      acc[0] = fmaf(d, w0.x, acc[0]); acc[1] = fmaf(d, w0.y, acc[1]);
      acc[2] = fmaf(d, w0.z, acc[2]); acc[3] = fmaf(d, w0.w, acc[3]);
      acc[4] = fmaf(d, w1.x, acc[4]); acc[5] = fmaf(d, w1.y, acc[5]);
      acc[6] = fmaf(d, w1.z, acc[6]); acc[7] = fmaf(d, w1.w, acc[7]);
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(p.out + pair * kTC + cg) = o;
  }
}

// s: bf16 [T][R][C] -> u [R][C] = relu(sum_t s / T), templates added in order in fp32
__global__ void __launch_bounds__(256) template_tail_kernel(const __nv_bfloat16* __restrict__ s,
                                                            __nv_bfloat16* __restrict__ u, int T, long long R, int C) {
  const long long total = R * (C / 8);
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int t = 0; t < T; ++t) {
      const uint4 v = *reinterpret_cast<const uint4*>(s + (static_cast<long long>(t) * R * C) + i * 8);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        acc[2 * k] += bf16_lo(w[k]);
        acc[2 * k + 1] += bf16_hi(w[k]);
      }
    }
    const float inv = 1.0f / static_cast<float>(T);
    uint4 o;
    o.x = pack_bf16x2(fmaxf(acc[0] * inv, 0.f), fmaxf(acc[1] * inv, 0.f));
    o.y = pack_bf16x2(fmaxf(acc[2] * inv, 0.f), fmaxf(acc[3] * inv, 0.f));
    o.z = pack_bf16x2(fmaxf(acc[4] * inv, 0.f), fmaxf(acc[5] * inv, 0.f));
    o.w = pack_bf16x2(fmaxf(acc[6] * inv, 0.f), fmaxf(acc[7] * inv, 0.f));
    *reinterpret_cast<uint4*>(u + i * 8) = o;
  }
}

static inline int templ_grid(long long work) {
  long long b = (work + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  return static_cast<int>(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace ubm

extern "C" int ubm_template_embed(const void* dg, const void* uv, const void* pbm, const void* bbm, const void* asym,
                                  const void* ri, const void* rj, const void* zp, const void* w_dgram,
                                  const void* w_vec, void* out, int T, int N, void* stream) {
  using namespace ubm;
  if (T <= 0 || N <= 0) return UBM_ERR_ARGUMENT;
  TemplParams p;
  p.dg = static_cast<const __nv_bfloat16*>(dg);
  p.uv = static_cast<const __nv_bfloat16*>(uv);
  p.pbm = static_cast<const float*>(pbm);
  p.bbm = static_cast<const float*>(bbm);
  p.asym = static_cast<const int*>(asym);
  p.ri = static_cast<const __nv_bfloat16*>(ri);
  p.rj = static_cast<const __nv_bfloat16*>(rj);
  p.zp = static_cast<const __nv_bfloat16*>(zp);
  p.w_dgram = static_cast<const float*>(w_dgram);
  p.w_vec = static_cast<const float*>(w_vec);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.T = T;
  p.N = N;
  const long long total = static_cast<long long>(T) * N * N * 8;
  template_embed_kernel<<<templ_grid(total), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  UBM_CHECK_LAUNCH("template_embed_kernel");
  return UBM_OK;
}

extern "C" int ubm_template_tail(const void* s, void* u, int T, long long R, int C, void* stream) {
  using namespace ubm;
  if (T <= 0 || R <= 0 || C <= 0 || (C & 7)) return UBM_ERR_ARGUMENT;
  template_tail_kernel<<<templ_grid(R * (C / 8)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(s), static_cast<__nv_bfloat16*>(u), T, R, C);
  UBM_CHECK_LAUNCH("template_tail_kernel");
  return UBM_OK;
}
