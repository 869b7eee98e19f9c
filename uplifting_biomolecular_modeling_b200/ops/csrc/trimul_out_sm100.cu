// Triangle multiplication, output stage: z_out = z + sigmoid(g_out(LN_in(z))) * p_out(LN_out(x)),
// where x[c][i][j] are the channel-major planes written by the contraction GEMM.
//
// Both LayerNorms are folded into their GEMMs (W' = W * gamma; the row statistics scale the fp32
// accumulator in the epilogue), so the operands are used as they sit in memory:
//   * the x tile of 128 pairs (i, j0..j0+127) is read from the planes as an MN-major A operand
//     (j contiguous, K = channel) - the transposed copy the reference's K3 reads row by row is
//     never materialised;
//   * the z tile is a K-major A operand of the gate GEMM and also supplies the residual.
// Reference: K3 of common/opt_core/opt_core/kernels/trimul/native/DESIGN.md:21-47
// (LN_in recompute + LN_out + W_o x sigmoid gate + residual) and _k3c/_k3d of
// kernels/fpf_trimul_v4/kernels.py.
//
// Warps: 0 = TMA producer, 1 = MMA issuer, 2-5 / 6-9 = two epilogue groups (output channels
// 0-63 / 64-127).  TMEM: {O, G} x two tiles = 512 columns.
#include "host_util.h"
#include "sm100.cuh"

namespace ubm {

constexpr int kTOStages = 2;
constexpr int kTOTileBytes = 128 * 128 * 2;  // 32 KB per operand tile
constexpr int kTOStageBytes = 2 * kTOTileBytes;

struct TrimulOutParams {
  int rows, N, Np;   // rows = first pair index extent (N, or fewer for a row shard)
  const float* o_colsum;   // [128] rowsum(Wo')
  const float* o_colbias;  // [128] Wo.beta_out
  const float* g_colsum;   // [128]
  const float* g_colbias;  // [128] Wg.beta_in
  const __nv_bfloat16* z;  // [N*N][128] (also residual when add_residual)
  __nv_bfloat16* out;      // [N*N][128]
  int add_residual;
  KernelStatus* status;
  int tiles_per_i, num_tiles;
  // the output rows leave through shared memory: every epilogue warp stages 32 rows x 32 channels (64-byte swizzle)
  // and one lane stores the box with a bulk tensor copy (map tmO over {128, N, rows}; second indices past N are
  // clipped)
  int out_tma;
};
constexpr int kTOOutWarpBytes = 32 * 64;
constexpr int kTOOutBytes = 8 * kTOOutWarpBytes;

__global__ void __launch_bounds__(320, 1)
trimul_out_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmZ,
                  const __grid_constant__ CUtensorMap tmWo, const __grid_constant__ CUtensorMap tmWg,
                  const __grid_constant__ CUtensorMap tmO, TrimulOutParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sWo = smem;                    // 32 KB: two k-blocks [128][64]
  uint8_t* sWg = smem + kTOTileBytes;     // 32 KB
  uint8_t* sSt = smem + 2 * kTOTileBytes; // stages: {x tile 32 KB, z tile 32 KB}
  uint8_t* sOut = sSt + kTOStages * kTOStageBytes;   // 8 warps x 2 KB of output staging
  float* sConst = reinterpret_cast<float*>(sOut + kTOOutBytes);               // 4 x 128
  float* sStats = sConst + 512;                                               // [2 tiles][128 rows][4]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sStats + 2 * 128 * 4);
  uint64_t* full = bars;                 // [stages]
  uint64_t* empty = full + kTOStages;    // [stages]  MMA commit + 8 epilogue warps
  uint64_t* w_full = empty + kTOStages;  // [1]
  uint64_t* acc_full = w_full + 1;       // [2]
  uint64_t* acc_empty = acc_full + 2;    // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const WaitScope ws{abort_flag, p.status};

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kTOStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1 + 8);
    }
    mbar_init(w_full, 1);
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 8);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmX);
    tma_prefetch_desc(&tmZ);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  for (int i = threadIdx.x; i < 128; i += blockDim.x) {
    sConst[i] = p.o_colsum[i];
    sConst[128 + i] = p.o_colbias[i];
    sConst[256 + i] = p.g_colsum[i];
    sConst[384 + i] = p.g_colbias[i];
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(w_full, 2 * kTOTileBytes);
      for (int kb = 0; kb < 2; ++kb) {
        tma_load_2d(sWo + kb * 16384, &tmWo, w_full, kb * 64, 0);
        tma_load_2d(sWg + kb * 16384, &tmWg, w_full, kb * 64, 0);
      }
      int stage = 0;
      uint32_t phase = 0;
      for (int t = blockIdx.x; t < p.num_tiles; t += gridDim.x) {
        const int i = t / p.tiles_per_i;
        const int j0 = (t - i * p.tiles_per_i) * 128;
        mbar_wait(&empty[stage], phase ^ 1u, ws, 21, stage);
        if (*abort_flag) break;
        uint8_t* sx = sSt + stage * kTOStageBytes;
        uint8_t* sz = sx + kTOTileBytes;
        mbar_expect_tx(&full[stage], kTOStageBytes);
        // x tile, MN-major: for channel block kb and j half h a box of [64 c][64 j]
        for (int kb = 0; kb < 2; ++kb)
          for (int h = 0; h < 2; ++h)
            tma_load_3d(sx + (kb * 2 + h) * 8192, &tmX, &full[stage], j0 + h * 64, i, kb * 64);
        // z tile, K-major: rows i*N + j0 .. +127
        const int row0 = i * p.N + j0;  // < 2^31 for N <= 46340
        tma_load_2d(sz, &tmZ, &full[stage], 0, row0);
        tma_load_2d(sz + 16384, &tmZ, &full[stage], 64, row0);
        if (++stage == kTOStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    const bool leader = elect_one();   // warp-uniform loop, the elected lane issues the tcgen05 instructions
    {
      constexpr uint32_t idesc_o = umma_idesc_bf16(128, 128, /*a_mn=*/1, /*b_mn=*/0);
      constexpr uint32_t idesc_g = umma_idesc_bf16(128, 128, 0, 0);
      mbar_wait(w_full, 0, ws, 22);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      for (int t = blockIdx.x; t < p.num_tiles; t += gridDim.x) {
        mbar_wait(&acc_empty[acc], acc_phase ^ 1u, ws, 23, acc);
        mbar_wait(&full[stage], phase, ws, 24, stage);
        tc_fence_after_sync();
        const uint32_t sx = smem_u32(sSt + stage * kTOStageBytes);
        const uint32_t sz = sx + kTOTileBytes;
        const uint32_t wo = smem_u32(sWo), wg = smem_u32(sWg);
        const uint32_t dO = tmem_base + acc * 256;
        const uint32_t dG = dO + 128;
        const uint64_t xd0 = umma_smem_desc(sx, 8192, 1024, kSwizzle128);
        const uint64_t wod0 = umma_smem_desc(wo, 16, 1024, kSwizzle128);
        const uint64_t zd0 = umma_smem_desc(sz, 16, 1024, kSwizzle128);
        const uint64_t wgd0 = umma_smem_desc(wg, 16, 1024, kSwizzle128);
        if (leader) {
#pragma unroll
          for (int kb = 0; kb < 2; ++kb) {
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma_ss(dO, xd0 + static_cast<uint64_t>(kb * (16384 >> 4) + k * (2048 >> 4)),
                      wod0 + static_cast<uint64_t>(kb * (16384 >> 4) + k * 2), idesc_o, (kb | k) != 0 ? 1u : 0u);
          }
#pragma unroll
          for (int kb = 0; kb < 2; ++kb) {
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma_ss(dG, zd0 + static_cast<uint64_t>(kb * (16384 >> 4) + k * 2),
                      wgd0 + static_cast<uint64_t>(kb * (16384 >> 4) + k * 2), idesc_g, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&acc_full[acc]);
          umma_commit(&empty[stage]);
        }
        __syncwarp();
        if (++stage == kTOStages) {
          stage = 0;
          phase ^= 1u;
        }
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
  } else {
    const int grp = (warp - 2) >> 2;
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const bool out_tma = p.out_tma != 0;   // warp-uniform
    uint8_t* stage_w = sOut + (warp - 2) * kTOOutWarpBytes;
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < p.num_tiles; t += gridDim.x) {
      const int i = t / p.tiles_per_i;
      const int j0 = (t - i * p.tiles_per_i) * 128;
      const int j = j0 + row;
      const bool row_ok = j < p.N;
      mbar_wait(&full[stage], phase, ws, 25, stage);
      const uint8_t* sx = sSt + stage * kTOStageBytes;
      const uint8_t* sz = sx + kTOTileBytes;
      float* st = sStats + (acc * 128 + row) * 4;
      if (grp == 0) {
        // statistics over channels of x[:, i, j]: column `row` of the [c][j] tile
        float sum = 0.f, sumsq = 0.f;
        const uint32_t jh = row >> 6, jj = row & 63;
#pragma unroll 8
        for (int c = 0; c < 128; ++c) {
          const uint32_t kb = c >> 6, cc = c & 63;
          const uint8_t* ptr = sx + (kb * 2 + jh) * 8192 + swz128_offset(cc, jj >> 3) + (jj & 7) * 2;
          const float e = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(ptr));
          sum += e;
          sumsq += e * e;
        }
        const float mu = sum * (1.f / 128.f);
        const float var = fmaxf(sumsq * (1.f / 128.f) - mu * mu, 0.f);
        st[0] = mu;
        st[1] = rsqrtf(var + 1e-5f);
      } else {
        float sum = 0.f, sumsq = 0.f;
#pragma unroll 4
        for (int c16 = 0; c16 < 16; ++c16) {
          const uint4 u = *reinterpret_cast<const uint4*>(sz + (c16 >> 3) * 16384 + swz128_offset(row, c16 & 7));
          const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
          for (int m = 0; m < 4; ++m) {
            const float a = bf16_lo(w[m]), b = bf16_hi(w[m]);
            sum += a + b;
            sumsq += a * a + b * b;
          }
        }
        const float mu = sum * (1.f / 128.f);
        const float var = fmaxf(sumsq * (1.f / 128.f) - mu * mu, 0.f);
        st[2] = mu;
        st[3] = rsqrtf(var + 1e-5f);
      }
      // exchange statistics between the two groups (256 epilogue threads)
      asm volatile("bar.sync 1, 256;" ::: "memory");
      const float mux = st[0], rsx = st[1], muz = st[2], rsz = st[3];

      mbar_wait(&acc_full[acc], acc_phase, ws, 26, acc);
      tc_fence_after_sync();
      const uint32_t tO = tmem_addr(tmem_base, q, acc * 256 + grp * 64);
      const uint32_t tG = tO + 128;
      const long long r = static_cast<long long>(i) * p.N + j;
#pragma unroll 1
      for (int c0 = 0; c0 < 64; c0 += 32) {
        uint32_t ov[32], gv[32];
        tmem_ld32(tO + c0, ov);
        tmem_ld32(tG + c0, gv);
        tmem_ld_wait();
        if (out_tma) {
          if (lane == 0) tma_store_wait_read<0>();   // the previous box of this warp has left the staging rows
          __syncwarp();
        }
        if (row_ok) {
          float f[32], fg[32];
          const int cb0 = grp * 64 + c0;
          ln_fold32(ov, make_float2(rsx, rsx), make_float2(-mux * rsx, -mux * rsx), sConst + cb0, sConst + 128 + cb0, f);
          ln_fold32(gv, make_float2(rsz, rsz), make_float2(-muz * rsz, -muz * rsz), sConst + 256 + cb0,
                    sConst + 384 + cb0, fg);
#pragma unroll
          for (int m = 0; m < 32; m += 2) {
            const float2 v = __fmul2_rn(make_float2(f[m], f[m + 1]),
                                        make_float2(sigmoidf_fast(fg[m]), sigmoidf_fast(fg[m + 1])));
            f[m] = v.x;
            f[m + 1] = v.y;
          }
          if (p.add_residual) {
            // residual from the z tile in shared memory: channels grp*64 + c0 .. +31
            const int kb = grp;  // 64 channels per k-block
#pragma unroll
            for (int m8 = 0; m8 < 4; ++m8) {
              const uint4 u =
                  *reinterpret_cast<const uint4*>(sz + kb * 16384 + swz128_offset(row, (c0 >> 3) + m8));
              const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
              for (int m = 0; m < 4; ++m) {
                f[m8 * 8 + 2 * m] += bf16_lo(w[m]);
                f[m8 * 8 + 2 * m + 1] += bf16_hi(w[m]);
              }
            }
          }
          if (out_tma) {
#pragma unroll
            for (int j8 = 0; j8 < 4; ++j8) {
              uint4 u;
              u.x = pack_bf16x2(f[j8 * 8], f[j8 * 8 + 1]);
              u.y = pack_bf16x2(f[j8 * 8 + 2], f[j8 * 8 + 3]);
              u.z = pack_bf16x2(f[j8 * 8 + 4], f[j8 * 8 + 5]);
              u.w = pack_bf16x2(f[j8 * 8 + 6], f[j8 * 8 + 7]);
              *reinterpret_cast<uint4*>(stage_w + swz64_offset(lane, j8)) = u;
            }
          } else {
            __nv_bfloat16* dst = p.out + r * 128 + grp * 64 + c0;
            st_bf16x16(dst, f);
            st_bf16x16(dst + 16, f + 16);
          }
        }
        if (out_tma) {
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_3d(&tmO, stage_w, grp * 64 + c0, j0 + q * 32, i);
            tma_store_commit();
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&acc_empty[acc]);
        mbar_arrive(&empty[stage]);
      }
      if (++stage == kTOStages) {
        stage = 0;
        phase ^= 1u;
      }
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
    if (out_tma && lane == 0) tma_store_wait_all<0>();   // the staging rows are read and the boxes written
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

constexpr int kTOSmemBytes =
    2 * kTOTileBytes + kTOStages * kTOStageBytes + kTOOutBytes + (512 + 2 * 128 * 4) * 4 + 256 + 1024;
static_assert(kTOSmemBytes <= 232448, "shared memory of one CTA");

}  // namespace ubm

// x: bf16 planes [128][N][Np]; z: bf16 [N*N][128]; wo, wg: bf16 [128][128] (gamma folded);
// *_colsum / *_colbias: fp32 [128]; out: bf16 [N*N][128].  out may alias z, with or without the residual: a tile's
// rows of z are copied to shared memory before the same CTA writes those rows, and no other tile touches them.
extern "C" int ubm_trimul_out_rows(const void* x, const void* z, const void* wo, const void* wg, const void* o_colsum,
                                   const void* o_colbias, const void* g_colsum, const void* g_colbias, void* out,
                                   int rows, int N, int Np, int add_residual, void* status, void* stream) {
  using namespace ubm;
  if (N <= 0 || rows <= 0 || Np < N || (Np & 7)) return UBM_ERR_ARGUMENT;
  CUtensorMap tmX, tmZ, tmWo, tmWg;
  {
    uint64_t d[3] = {(uint64_t)N, (uint64_t)rows, 128};
    uint64_t s[2] = {(uint64_t)Np * 2, (uint64_t)rows * Np * 2};
    uint32_t b[3] = {64, 1, 64};
    int rc = make_tmap(&tmX, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, d, s, b, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  {
    uint64_t d[2] = {128, (uint64_t)rows * N};
    uint64_t s[1] = {256};
    uint32_t b[2] = {64, 128};
    int rc = make_tmap(&tmZ, z, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, d, s, b, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  {
    uint64_t d[2] = {128, 128};
    uint64_t s[1] = {256};
    uint32_t b[2] = {64, 128};
    int rc = make_tmap(&tmWo, wo, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, d, s, b, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = make_tmap(&tmWg, wg, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, d, s, b, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  TrimulOutParams p = {};
  p.rows = rows;
  p.N = N;
  p.Np = Np;
  p.o_colsum = static_cast<const float*>(o_colsum);
  p.o_colbias = static_cast<const float*>(o_colbias);
  p.g_colsum = static_cast<const float*>(g_colsum);
  p.g_colbias = static_cast<const float*>(g_colbias);
  p.z = static_cast<const __nv_bfloat16*>(z);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.add_residual = add_residual;
  p.status = static_cast<KernelStatus*>(status);
  p.tiles_per_i = (N + 127) / 128;
  p.num_tiles = p.tiles_per_i * rows;
  CUtensorMap tmO = tmZ;
  p.out_tma = 0;
  {
    static const bool on = [] {
      const char* e = getenv("UBM_PROJ_TMA_STORE");
      return e == nullptr || e[0] != '0';
    }();
    if (on && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
      uint64_t d[3] = {128, (uint64_t)N, (uint64_t)rows};
      uint64_t st[2] = {256, (uint64_t)N * 256};
      uint32_t b[3] = {32, 32, 1};
      int rc2 = make_tmap(&tmO, out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, d, st, b, CU_TENSOR_MAP_SWIZZLE_64B);
      if (rc2) return rc2;
      p.out_tma = 1;
    }
  }
  int rc = set_smem(trimul_out_kernel, kTOSmemBytes);
  if (rc) return rc;
  const int grid = p.num_tiles < sm_count() ? p.num_tiles : sm_count();
  trimul_out_kernel<<<grid, 320, kTOSmemBytes, static_cast<cudaStream_t>(stream)>>>(tmX, tmZ, tmWo, tmWg, tmO, p);
  UBM_CHECK_LAUNCH("trimul_out_kernel");
  return UBM_OK;
}

extern "C" int ubm_trimul_out(const void* x, const void* z, const void* wo, const void* wg, const void* o_colsum,
                              const void* o_colbias, const void* g_colsum, const void* g_colbias, void* out, int N,
                              int Np, int add_residual, void* status, void* stream) {
  return ubm_trimul_out_rows(x, z, wo, wg, o_colsum, o_colbias, g_colsum, g_colbias, out, N, N, Np, add_residual,
                             status, stream);
}
