// Fused pair transition: y = x + W_o( silu(W_a n) * (W_b n) ), n = LayerNorm(x), c = 128.
//
// One persistent kernel per SM: a 128-row tile of x arrives by TMA and is used three times
// without leaving shared memory - as the A operand of the first GEMM, as the source of the row
// statistics, and as the residual.  LayerNorm is folded into the first GEMM (weights carry
// gamma, the statistics scale the fp32 accumulator).  The hidden dimension is walked in chunks
// of 64: GEMM1 produces [a | b] (128 TMEM columns), the SwiGLU warps turn them into a bf16
// 128 x 64 tile in shared memory, GEMM2 accumulates it into the 128 x 128 output accumulator.
// The hidden activations never touch HBM.  Weight chunks stream from L2 through a 2-stage ring.
//
// Reference kernels with the same fusion boundary: fpf_transition_v2 (Triton, the fastest row on
// B200: common/opt_core/opt_core/kernels/transition/TRANSITION_CELLS.json:2802), flash_sm90a and
// ef2_t16 (wgmma, sm_90a only: common/opt_core/opt_core/kernels/transition/DESIGN.md:24-63).
//
// Warps: 0 = TMA producer, 1 = MMA issuer, 2-5 / 6-9 = two SwiGLU/epilogue groups that take
// alternate hidden chunks.
#include "host_util.h"
#include "sm100.cuh"

namespace ubm {

constexpr int kTRC = 128;
constexpr int kTRXBytes = 128 * 128 * 2;        // 32 KB
constexpr int kTRWabBytes = 128 * 128 * 2;      // 32 KB: [a64|b64 rows][128 k] as two k-blocks
constexpr int kTRWoBytes = 128 * 64 * 2;        // 16 KB: [128 out][64 k]
constexpr int kTRWStage = kTRWabBytes + kTRWoBytes;
constexpr int kTRHBytes = 128 * 64 * 2;         // 16 KB
constexpr int kTRMaxHidden = 1024;

struct TransitionParams {
  long long R;
  int hidden;               // multiple of 64
  const float* ab_colsum;   // [hidden/64][128] in packed order
  const float* ab_colbias;  // [hidden/64][128]
  const float* o_bias;      // [128] or null
  const float* mask;        // [R] or null: multiplies the update
  __nv_bfloat16* out;       // [R][128]
  int add_residual;
  KernelStatus* status;
  int num_tiles;
};

__global__ void __launch_bounds__(320, 1)
transition_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmWab,
                  const __grid_constant__ CUtensorMap tmWo, TransitionParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sX = smem;                       // 2 x 32 KB
  uint8_t* sW = sX + 2 * kTRXBytes;         // 2 x 48 KB
  uint8_t* sH = sW + 2 * kTRWStage;         // 2 x 16 KB
  float* sColsum = reinterpret_cast<float*>(sH + 2 * kTRHBytes);  // [hidden*2]
  float* sColbias = sColsum + 2 * kTRMaxHidden;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sColbias + 2 * kTRMaxHidden);
  uint64_t* x_full = bars;            // [2]
  uint64_t* x_empty = x_full + 2;     // [2] 8 arrivals
  uint64_t* w_full = x_empty + 2;     // [2] first-GEMM weights (a|b rows) landed
  uint64_t* w_empty = w_full + 2;     // [2] commit after the first GEMM: its slot refills while SwiGLU runs
  uint64_t* wo_full = w_empty + 2;    // [2] second-GEMM weights landed
  uint64_t* wo_empty = wo_full + 2;   // [2] commit after the second GEMM
  uint64_t* ab_full = wo_empty + 2;   // [2] commit
  uint64_t* ab_empty = ab_full + 2;   // [2] 4 arrivals
  uint64_t* h_full = ab_empty + 2;    // [2] 4 arrivals
  uint64_t* h_empty = h_full + 2;     // [2] commit
  uint64_t* y_full = h_empty + 2;     // [1] commit
  uint64_t* y_empty = y_full + 1;     // [1] 8 arrivals
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(y_empty + 1);   // 22 barriers before it: 176 of the 256 bytes
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const WaitScope ws{abort_flag, p.status};
  const int nch = p.hidden / 64;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < 2; ++s) {
      mbar_init(&x_full[s], 1);
      mbar_init(&x_empty[s], 8);
      mbar_init(&w_full[s], 1);
      mbar_init(&w_empty[s], 1);
      mbar_init(&wo_full[s], 1);
      mbar_init(&wo_empty[s], 1);
      mbar_init(&ab_full[s], 1);
      mbar_init(&ab_empty[s], 4);
      mbar_init(&h_full[s], 4);
      mbar_init(&h_empty[s], 1);
    }
    mbar_init(y_full, 1);
    mbar_init(y_empty, 8);
    mbar_fence_init();
    tma_prefetch_desc(&tmX);
    tma_prefetch_desc(&tmWab);
    tma_prefetch_desc(&tmWo);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  for (int i = threadIdx.x; i < 2 * p.hidden; i += blockDim.x) {
    sColsum[i] = p.ab_colsum[i];
    sColbias[i] = p.ab_colbias[i];
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tAB = tmem_base;        // two buffers of 128 columns
  const uint32_t tY = tmem_base + 256;   // 128 columns

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t g = 0;   // global chunk counter
      uint32_t xt = 0;  // x tile counter
      auto load_x = [&](int tile, uint32_t cnt) {
        const int xs = cnt & 1;
        mbar_wait(&x_empty[xs], ((cnt >> 1) & 1u) ^ 1u, ws, 31, xs);
        mbar_expect_tx(&x_full[xs], kTRXBytes);
        tma_load_2d(sX + xs * kTRXBytes, &tmX, &x_full[xs], 0, tile * 128);
        tma_load_2d(sX + xs * kTRXBytes + 16384, &tmX, &x_full[xs], 64, tile * 128);
      };
      // The second-GEMM weights of chunk g are requested one chunk late (after the first-GEMM weights of
      // chunk g + 1): their slot frees only when the second GEMM of chunk g - 2 has run, which follows a
      // SwiGLU pass, and waiting for it here must not hold back the first-GEMM weights.
      auto load_wo = [&](uint32_t gc, int hc) {
        const int s = gc & 1;
        mbar_wait(&wo_empty[s], ((gc >> 1) & 1u) ^ 1u, ws, 42, s);
        mbar_expect_tx(&wo_full[s], kTRWoBytes);
        tma_load_2d(sW + s * kTRWStage + kTRWabBytes, &tmWo, &wo_full[s], hc * 64, 0);
      };
      if (blockIdx.x < p.num_tiles) load_x(blockIdx.x, xt++);
      for (int t = blockIdx.x; t < p.num_tiles; t += gridDim.x) {
        for (int h = 0; h < nch; ++h, ++g) {
          const int s = g & 1;
          mbar_wait(&w_empty[s], ((g >> 1) & 1u) ^ 1u, ws, 32, s);
          if (*abort_flag) break;
          uint8_t* dst = sW + s * kTRWStage;
          mbar_expect_tx(&w_full[s], kTRWabBytes);
          tma_load_2d(dst, &tmWab, &w_full[s], 0, h * 128);
          tma_load_2d(dst + 16384, &tmWab, &w_full[s], 64, h * 128);
          if (g > 0) load_wo(g - 1, h == 0 ? nch - 1 : h - 1);
          if (*abort_flag) break;
          if (h == 1 || nch == 1) {
            const int tn = t + gridDim.x;
            if (tn < p.num_tiles) load_x(tn, xt++);
          }
        }
        if (*abort_flag) break;
      }
      if (g > 0 && !*abort_flag) load_wo(g - 1, nch - 1);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (warp-uniform loop, elected lane issues)
    const bool leader = elect_one();
    {
      constexpr uint32_t idesc = umma_idesc_bf16(128, 128);
      // One flat loop over this CTA's chunks (global index G = local tile * nch + chunk).  Step G issues the first
      // GEMM of chunk G and then the second GEMM of chunk G - 2: the accumulator buffer of chunk G is released halfway
      // through the SwiGLU pass of chunk G - 2, so the first GEMM of G runs under the rest of that pass and under
      // the pass of chunk G - 1 on the other group.  (Issuing the second GEMM of G - 1 here instead made every
      // first GEMM wait for the END of a SwiGLU pass, and the group that had just finished idled for its duration.)
      const uint32_t my_tiles =
          static_cast<uint32_t>(p.num_tiles) > blockIdx.x ? (p.num_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0u;
      const uint32_t total = my_tiles * static_cast<uint32_t>(nch);
      auto gemm2 = [&](uint32_t c) {
        const uint32_t tl = c / nch, hh = c - tl * nch;
        const bool first_of_tile = hh == 0;
        const int b = c & 1;
        mbar_wait(&wo_full[b], (c >> 1) & 1u, ws, 43, b);
        mbar_wait(&h_full[b], (c >> 1) & 1u, ws, 33, b);
        if (first_of_tile) mbar_wait(y_empty, (tl & 1u) ^ 1u, ws, 34);
        tc_fence_after_sync();
        const uint32_t ha = smem_u32(sH + b * kTRHBytes);
        const uint32_t wo = smem_u32(sW + b * kTRWStage + kTRWabBytes);
        const uint64_t ad0 = umma_smem_desc(ha, 16, 1024, kSwizzle128);
        const uint64_t bd0 = umma_smem_desc(wo, 16, 1024, kSwizzle128);
        if (leader) {
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_ss(tY, ad0 + static_cast<uint64_t>(k * 2), bd0 + static_cast<uint64_t>(k * 2), idesc,
                    (first_of_tile && k == 0) ? 0u : 1u);
          umma_commit(&h_empty[b]);
          umma_commit(&wo_empty[b]);
          if (hh == static_cast<uint32_t>(nch) - 1) umma_commit(y_full);
        }
        __syncwarp();
      };
      for (uint32_t G = 0; G < total; ++G) {
        const uint32_t tl = G / nch, hh = G - tl * nch;
        const int xs = tl & 1;
        if (hh == 0) mbar_wait(&x_full[xs], (tl >> 1) & 1u, ws, 35, xs);
        const uint32_t xa = smem_u32(sX + xs * kTRXBytes);
        const int b = G & 1;
        mbar_wait(&w_full[b], (G >> 1) & 1u, ws, 36, b);
        mbar_wait(&ab_empty[b], ((G >> 1) & 1u) ^ 1u, ws, 37, b);
        tc_fence_after_sync();
        const uint32_t wa = smem_u32(sW + b * kTRWStage);
        const uint64_t ad0 = umma_smem_desc(xa, 16, 1024, kSwizzle128);
        const uint64_t bd0 = umma_smem_desc(wa, 16, 1024, kSwizzle128);
        if (leader) {
#pragma unroll
          for (int kb = 0; kb < 2; ++kb) {
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma_ss(tAB + b * 128, ad0 + static_cast<uint64_t>(kb * (16384 >> 4) + k * 2),
                      bd0 + static_cast<uint64_t>(kb * (16384 >> 4) + k * 2), idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&w_empty[b]);
          umma_commit(&ab_full[b]);
        }
        __syncwarp();
        if (G >= 2) gemm2(G - 2);
      }
      if (total >= 2) gemm2(total - 2);
      if (total >= 1) gemm2(total - 1);
    }
  } else {
    // ------------------------------------------------------------------ SwiGLU / epilogue groups
    const int grp = (warp - 2) >> 2;
    const int q = warp & 3;
    const int row = q * 32 + lane;
    uint32_t g = 0;
    uint32_t xt = 0;
    uint32_t tile_cnt = 0;
    for (int t = blockIdx.x; t < p.num_tiles; t += gridDim.x, ++xt, ++tile_cnt) {
      const long long r = static_cast<long long>(t) * 128 + row;
      const bool row_ok = r < p.R;
      const int xs = xt & 1;
      mbar_wait(&x_full[xs], (xt >> 1) & 1u, ws, 38, xs);
      const uint8_t* xsm = sX + xs * kTRXBytes;
      float sum = 0.f, sumsq = 0.f;
#pragma unroll 4
      for (int c16 = 0; c16 < 16; ++c16) {
        const uint4 u = *reinterpret_cast<const uint4*>(xsm + (c16 >> 3) * 16384 + swz128_offset(row, c16 & 7));
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          const float a = bf16_lo(w[m]), b = bf16_hi(w[m]);
          sum += a + b;
          sumsq += a * a + b * b;
        }
      }
      const float mu = sum * (1.f / kTRC);
      const float var = fmaxf(sumsq * (1.f / kTRC) - mu * mu, 0.f);
      const float rstd = rsqrtf(var + 1e-5f);
      const float2 a2 = make_float2(rstd, rstd);
      const float2 b2 = make_float2(-mu * rstd, -mu * rstd);

      for (int h = 0; h < nch; ++h, ++g) {
        const int b = g & 1;
        if (b != grp) continue;
        const uint32_t ph = (g >> 1) & 1u;
        mbar_wait(&ab_full[b], ph, ws, 39, b);
        tc_fence_after_sync();
        const uint32_t ta = tmem_addr(tAB, q, b * 128);
        const float* cs = sColsum + h * 128;
        const float* cb = sColbias + h * 128;
        uint32_t packed[32];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t av[32], bv[32];
          tmem_ld32(ta + half * 32, av);
          tmem_ld32(ta + 64 + half * 32, bv);
          tmem_ld_wait();
          if (half == 1) {
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ab_empty[b]);
          }
          float fa[32], fb[32];
          ln_fold32(av, a2, b2, cs + half * 32, cb + half * 32, fa);
          ln_fold32(bv, a2, b2, cs + 64 + half * 32, cb + 64 + half * 32, fb);
#pragma unroll
          for (int m = 0; m < 32; m += 2) {
            const float2 hv = __fmul2_rn(make_float2(siluf_fast(fa[m]), siluf_fast(fa[m + 1])),
                                         make_float2(fb[m], fb[m + 1]));
            packed[half * 16 + (m >> 1)] = pack_bf16x2(hv.x, hv.y);
          }
        }
        mbar_wait(&h_empty[b], ph ^ 1u, ws, 40, b);
        uint8_t* hs = sH + b * kTRHBytes;
#pragma unroll
        for (int c16 = 0; c16 < 8; ++c16) {
          uint4 u = make_uint4(packed[c16 * 4], packed[c16 * 4 + 1], packed[c16 * 4 + 2], packed[c16 * 4 + 3]);
          *reinterpret_cast<uint4*>(hs + swz128_offset(row, c16)) = u;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&h_full[b]);
      }

      // ---- output: columns grp*64 .. +63
      mbar_wait(y_full, tile_cnt & 1u, ws, 41);
      tc_fence_after_sync();
      const float mval = (p.mask != nullptr && row_ok) ? p.mask[r] : 1.0f;
#pragma unroll 1
      for (int c0 = 0; c0 < 64; c0 += 32) {
        uint32_t yv[32];
        tmem_ld32(tmem_addr(tY, q, grp * 64 + c0), yv);
        tmem_ld_wait();
        float f[32];
#pragma unroll
        for (int m = 0; m < 32; ++m) {
          float v = __uint_as_float(yv[m]);
          if (p.o_bias != nullptr) v += __ldg(p.o_bias + grp * 64 + c0 + m);
          f[m] = v * mval;
        }
        if (p.add_residual) {
#pragma unroll
          for (int m8 = 0; m8 < 4; ++m8) {
            const uint4 u = *reinterpret_cast<const uint4*>(xsm + grp * 16384 + swz128_offset(row, (c0 >> 3) + m8));
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int m = 0; m < 4; ++m) {
              f[m8 * 8 + 2 * m] += bf16_lo(w[m]);
              f[m8 * 8 + 2 * m + 1] += bf16_hi(w[m]);
            }
          }
        }
        if (row_ok) {
          __nv_bfloat16* dst = p.out + r * 128 + grp * 64 + c0;
          st_bf16x16(dst, f);
          st_bf16x16(dst + 16, f + 16);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(y_empty);
        mbar_arrive(&x_empty[xs]);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

constexpr int kTRSmemBytes =
    2 * kTRXBytes + 2 * kTRWStage + 2 * kTRHBytes + 4 * kTRMaxHidden * 4 + 256 + 1024;

}  // namespace ubm

// x: bf16 [R][128].  wab: bf16 [(hidden/64)*128][128], chunk h = rows [a(64h..64h+63); b(64h..64h+63)]
// with gamma folded.  wo: bf16 [128][hidden].  ab_colsum / ab_colbias: fp32 [(hidden/64)*128] in the same
// packed order.  o_bias: fp32 [128] or null.  mask: fp32 [R] or null.  out may alias x.
extern "C" int ubm_transition(const void* x, const void* wab, const void* wo, const void* ab_colsum,
                              const void* ab_colbias, const void* o_bias, const void* mask, void* out, long long R,
                              int hidden, int add_residual, void* status, void* stream) {
  using namespace ubm;
  if (R <= 0 || hidden <= 0 || (hidden % 64) || hidden > kTRMaxHidden) return UBM_ERR_ARGUMENT;
  CUtensorMap tmX, tmWab, tmWo;
  {
    uint64_t d[2] = {128, (uint64_t)R};
    uint64_t s[1] = {256};
    uint32_t b[2] = {64, 128};
    int rc = make_tmap(&tmX, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, d, s, b, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  {
    uint64_t d[2] = {128, (uint64_t)(hidden / 64) * 128};
    uint64_t s[1] = {256};
    uint32_t b[2] = {64, 128};
    int rc = make_tmap(&tmWab, wab, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, d, s, b, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  {
    uint64_t d[2] = {(uint64_t)hidden, 128};
    uint64_t s[1] = {(uint64_t)hidden * 2};
    uint32_t b[2] = {64, 128};
    int rc = make_tmap(&tmWo, wo, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, d, s, b, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  TransitionParams p = {};
  p.R = R;
  p.hidden = hidden;
  p.ab_colsum = static_cast<const float*>(ab_colsum);
  p.ab_colbias = static_cast<const float*>(ab_colbias);
  p.o_bias = static_cast<const float*>(o_bias);
  p.mask = static_cast<const float*>(mask);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.add_residual = add_residual;
  p.status = static_cast<KernelStatus*>(status);
  p.num_tiles = static_cast<int>((R + 127) / 128);
  int rc = set_smem(transition_kernel, kTRSmemBytes);
  if (rc) return rc;
  const int grid = p.num_tiles < sm_count() ? p.num_tiles : sm_count();
  transition_kernel<<<grid, 320, kTRSmemBytes, static_cast<cudaStream_t>(stream)>>>(tmX, tmWab, tmWo, p);
  UBM_CHECK_LAUNCH("transition_kernel");
  return UBM_OK;
}
