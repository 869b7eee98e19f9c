// Input projection of the triangle multiplication: a = sigmoid(g_a(n)) * p_a(n) * mask, b likewise,
// n = LayerNorm(z[i][s]), written as channel-major bf16 planes P[2][c][i][s] (the operands of the triangle
// contraction).  Reference: K1 of common/opt_core/opt_core/kernels/trimul/native/DESIGN.md:21-47 and
// _k1c/_k1t of kernels/fpf_trimul_v4/kernels.py.
//
// The projection runs transposed on the tensor cores: D^T[channel][s] = W'[channel][k] . X[s][k]^T, with the
// 512 x 128 weight matrix (gamma folded in) as the resident A operand (four blocks of 128 channels: p_a, g_a,
// p_b, g_b) and a tile of 128 pair entries (one i, 128 consecutive s) as the B operand.  An accumulator
// lane is then one output channel and its 128 columns are consecutive s - exactly the order of a plane
// row - so an epilogue thread writes 256 contiguous bytes with 16-byte stores, instead of 256 two-byte
// stores scattered over 128 planes as in the row-per-lane orientation.  The value and the gate of a channel
// sit in the same lane (columns +0 and +128 of the operand's half), so the gating needs no exchange.
//
// LayerNorm is folded in: out = rstd[s] * (acc - mu[s] * colsum[ch]) + colbias[ch].  The per-s statistics
// are computed thread-per-row from the shared-memory tile (as the row-major kernels do) and passed to all
// threads of the epilogue group through a small shared array; the per-channel constants live in registers.
//
// Warps: 0 = TMA producer, 1 = MMA issuer, 2-5 = epilogue group 0 (operand a), 6-9 = group 1 (operand b).
#include "host_util.h"
#include "sm100.cuh"

namespace ubm {

constexpr int kTPRows = 128;   // pair entries (s) per tile
constexpr int kTPC = 128;      // input channels
constexpr int kTPStages = 2;   // tile ring
constexpr int kTPXBytes = kTPRows * kTPC * 2;   // 32 KB, two k-blocks of [128][64]
constexpr int kTPWBytes = 512 * kTPC * 2;       // 128 KB, two k-blocks of [512][64]

struct TrimulProjParams {
  long long R;          // rows * N
  int rows;             // first pair index extent held here
  int plane_rows;       // rows the planes are allocated for (>= rows)
  int N;                // second pair index extent
  int Np;               // leading dimension of the planes (>= N, multiple of 8)
  int tiles_per_row;    // ceil(N / 128)
  int num_tiles;        // rows * tiles_per_row
  const float* colsum;  // [512] rowsum(W') per output channel
  const float* colbias; // [512]
  const float* mask;    // [R] or null
  __nv_bfloat16* planes;  // [2][128][plane_rows][Np]
  float* stats_out;       // optional [R][2]
  KernelStatus* status;
  PeerSrc src;            // src.n > 0: the input rows are columns of z fetched from their owners (see host_util.h)
  // the planes leave through shared memory: every epilogue warp stages 32 channels x 32 entries (64-byte swizzle)
  // and one lane stores the box {32 entries, 1 row, 32 planes} with a bulk tensor copy (map tmP over
  // {Np, plane_rows, 256})
  int out_tma;
};
constexpr int kTPOutWarpBytes = 32 * 64;
constexpr int kTPOutBytes = 8 * kTPOutWarpBytes;

__global__ void __launch_bounds__(320, 1)
trimul_proj_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
                   const __grid_constant__ PeerSrcMaps peers, const __grid_constant__ CUtensorMap tmP,
                   TrimulProjParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sW = smem;                               // 128 KB
  uint8_t* sX = smem + kTPWBytes;                   // stages * 32 KB
  uint8_t* sOut = sX + kTPStages * kTPXBytes;       // 8 warps x 2 KB of output staging
  float* sStat = reinterpret_cast<float*>(sOut + kTPOutBytes);           // [2 groups][2 parities][3][128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sStat + 2 * 2 * 3 * 128);
  uint64_t* x_full = bars;                 // [stages]
  uint64_t* x_empty = x_full + kTPStages;  // [stages]
  uint64_t* w_full = x_empty + kTPStages;  // [1]
  uint64_t* acc_full = w_full + 1;         // [2]
  uint64_t* acc_empty = acc_full + 2;      // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const WaitScope ws{abort_flag, p.status};

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kTPStages; ++s) {
      mbar_init(&x_full[s], 1);
      mbar_init(&x_empty[s], 1 + 8);  // MMA commit + one arrival per epilogue warp
    }
    mbar_init(w_full, 1);
    for (int h = 0; h < 2; ++h) {
      mbar_init(&acc_full[h], 1);
      mbar_init(&acc_empty[h], 4);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmX);
    tma_prefetch_desc(&tmW);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(w_full, kTPWBytes);
      for (int kb = 0; kb < 2; ++kb)
        for (int h = 0; h < 2; ++h)
          tma_load_2d(sW + kb * 65536 + h * 32768, &tmW, w_full, kb * 64, h * 256);
      int stage = 0;
      uint32_t phase = 0;
      for (int t = blockIdx.x; t < p.num_tiles; t += gridDim.x) {
        const int i = t / p.tiles_per_row;
        const int s0 = (t - i * p.tiles_per_row) * kTPRows;
        const int flat = i * p.N + s0;   // rows past the end of pair row i belong to the next one and are discarded
        mbar_wait(&x_empty[stage], phase ^ 1u, ws, 11, stage);
        if (*abort_flag) break;
        uint8_t* dst = sX + stage * kTPXBytes;
        mbar_expect_tx(&x_full[stage], kTPXBytes);
        if (p.src.n > 0) {
          // transposed source: tile = (column col0 + i of z, rows s0 .. s0 + 127), fetched from the owner of s0
          int q = 0;
#pragma unroll
          for (int j = 1; j < kMaxSrcPeers; ++j)
            if (j < p.src.n && s0 >= p.src.row0[j]) q = j;
          tma_load_3d(dst, &peers.m[q], &x_full[stage], 0, p.src.col0 + i, s0 - p.src.row0[q]);
          tma_load_3d(dst + 16384, &peers.m[q], &x_full[stage], 64, p.src.col0 + i, s0 - p.src.row0[q]);
        } else {
          tma_load_2d(dst, &tmX, &x_full[stage], 0, flat);
          tma_load_2d(dst + 16384, &tmX, &x_full[stage], 64, flat);
        }
        if (++stage == kTPStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (warp-uniform loop, elected lane issues)
    const bool leader = elect_one();
    constexpr uint32_t idesc = umma_idesc_bf16(128, 128);
    mbar_wait(w_full, 0, ws, 12);
    int stage = 0;
    uint32_t phase = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < p.num_tiles; t += gridDim.x) {
      mbar_wait(&x_full[stage], phase, ws, 13, stage);
      tc_fence_after_sync();
      const uint64_t xd0 = umma_smem_desc(smem_u32(sX + stage * kTPXBytes), 16, 1024, kSwizzle128);
      const uint64_t wd0 = umma_smem_desc(smem_u32(sW), 16, 1024, kSwizzle128);
      for (int h = 0; h < 2; ++h) {
        mbar_wait(&acc_empty[h], acc_phase ^ 1u, ws, 14, h);
        tc_fence_after_sync();
        if (leader) {
#pragma unroll
          for (int blk = 0; blk < 2; ++blk) {
            const int mb = h * 2 + blk;   // 128 channels: p_a, g_a, p_b, g_b
#pragma unroll
            for (int kb = 0; kb < 2; ++kb) {
#pragma unroll
              for (int k = 0; k < 4; ++k)
                umma_ss(tmem_base + mb * 128,
                        wd0 + static_cast<uint64_t>(kb * (65536 >> 4) + mb * (16384 >> 4) + k * 2),
                        xd0 + static_cast<uint64_t>(kb * (16384 >> 4) + k * 2), idesc, (kb | k) != 0 ? 1u : 0u);
            }
          }
          umma_commit(&acc_full[h]);
        }
        __syncwarp();
      }
      if (leader) umma_commit(&x_empty[stage]);
      __syncwarp();
      if (++stage == kTPStages) {
        stage = 0;
        phase ^= 1u;
      }
      acc_phase ^= 1u;
    }
  } else {
    // ------------------------------------------------------------------ epilogue groups
    const int grp = (warp - 2) >> 2;  // operand a or b
    const int q = warp & 3;           // TMEM lane quadrant
    const int ch = q * 32 + lane;     // output channel of this thread; also the tile row it takes statistics of
    const float cs_v = p.colsum[grp * 256 + ch], cb_v = p.colbias[grp * 256 + ch];
    const float cs_g = p.colsum[grp * 256 + 128 + ch], cb_g = p.colbias[grp * 256 + 128 + ch];
    const float2 csv2 = make_float2(cs_v, cs_v), cbv2 = make_float2(cb_v, cb_v);
    const float2 csg2 = make_float2(cs_g, cs_g), cbg2 = make_float2(cb_g, cb_g);
    int stage = 0;
    uint32_t phase = 0;
    uint32_t acc_phase = 0;
    uint32_t par = 0;
    const bool wide = (p.Np & 15) == 0;   // plane rows 32-byte aligned: 32-byte stores
    const bool out_tma = p.out_tma != 0;  // warp-uniform
    uint8_t* stage_w = sOut + (warp - 2) * kTPOutWarpBytes;
    for (int t = blockIdx.x; t < p.num_tiles; t += gridDim.x, par ^= 1u) {
      const int i = t / p.tiles_per_row;
      const int s0 = (t - i * p.tiles_per_row) * kTPRows;
      // ---- statistics of tile row `ch` from the shared-memory tile
      mbar_wait(&x_full[stage], phase, ws, 15, stage);
      const uint8_t* xs = sX + stage * kTPXBytes;
      float sum = 0.f, sumsq = 0.f;
#pragma unroll 4
      for (int c16 = 0; c16 < 16; ++c16) {
        const uint4 u = *reinterpret_cast<const uint4*>(xs + (c16 >> 3) * 16384 + swz128_offset(ch, c16 & 7));
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float a = bf16_lo(w[j]), b = bf16_hi(w[j]);
          sum += a + b;
          sumsq += a * a + b * b;
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&x_empty[stage]);
      const float mu = sum * (1.0f / kTPC);
      const float var = fmaxf(sumsq * (1.0f / kTPC) - mu * mu, 0.f);
      const float rstd = rsqrtf(var + 1e-5f);
      const int s = s0 + ch;
      const bool valid = s < p.N;
      const long long r = static_cast<long long>(i) * p.N + s;
      float mval = valid ? 1.0f : 0.0f;            // entries past N are written as zeros (K padding of the contraction)
      if (valid && p.mask != nullptr) mval = p.mask[r];
      if (p.stats_out != nullptr && grp == 0 && valid) {
        p.stats_out[2 * r] = mu;
        p.stats_out[2 * r + 1] = rstd;
      }
      float* st = sStat + (grp * 2 + par) * 3 * 128;
      st[ch] = rstd;
      st[128 + ch] = -mu * rstd;
      st[256 + ch] = mval;
      // the 128 threads of this group exchange statistics; the array of the other parity is still being read
      // by slower warps of the previous tile, which is why there are two
      asm volatile("bar.sync %0, 128;" ::"r"(1 + grp) : "memory");

      // ---- accumulators of this operand: value block at +0, gate block at +128
      mbar_wait(&acc_full[grp], acc_phase, ws, 16, grp);
      tc_fence_after_sync();
      const uint32_t tbase = tmem_addr(tmem_base, q, grp * 256);
      __nv_bfloat16* dst =
          p.planes + ((static_cast<long long>(grp) * 128 + ch) * p.plane_rows + i) * p.Np + s0;
      const float4* st4 = reinterpret_cast<const float4*>(st);
      uint32_t vv[2][16], gv[2][16];
      tmem_ld16(tbase, vv[0]);
      tmem_ld16(tbase + 128, gv[0]);
#pragma unroll
      for (int ci = 0; ci < 8; ++ci) {
        tmem_ld_wait();
        if (ci < 7) {
          tmem_ld16(tbase + (ci + 1) * 16, vv[(ci + 1) & 1]);
          tmem_ld16(tbase + 128 + (ci + 1) * 16, gv[(ci + 1) & 1]);
        }
        const uint32_t* v = vv[ci & 1];
        const uint32_t* g = gv[ci & 1];
        float o[16];
#pragma unroll
        for (int j4 = 0; j4 < 4; ++j4) {
          const float4 rs = st4[ci * 4 + j4];
          const float4 nm = st4[32 + ci * 4 + j4];
          const float4 mk = st4[64 + ci * 4 + j4];
          const float rsv[4] = {rs.x, rs.y, rs.z, rs.w};
          const float nmv[4] = {nm.x, nm.y, nm.z, nm.w};
          const float mkv[4] = {mk.x, mk.y, mk.z, mk.w};
#pragma unroll
          for (int e = 0; e < 4; e += 2) {
            // two adjacent s at a time in packed fp32 instructions
            const int si = j4 * 4 + e;
            const float2 rs2 = make_float2(rsv[e], rsv[e + 1]);
            const float2 nm2 = make_float2(nmv[e], nmv[e + 1]);
            const float2 val = __ffma2_rn(make_float2(__uint_as_float(v[si]), __uint_as_float(v[si + 1])), rs2,
                                          __ffma2_rn(nm2, csv2, cbv2));
            const float2 gt = __ffma2_rn(make_float2(__uint_as_float(g[si]), __uint_as_float(g[si + 1])), rs2,
                                         __ffma2_rn(nm2, csg2, cbg2));
            const float2 sg = make_float2(mkv[e] * sigmoidf_fast(gt.x), mkv[e + 1] * sigmoidf_fast(gt.y));
            const float2 ov = __fmul2_rn(val, sg);
            o[si] = ov.x;
            o[si + 1] = ov.y;
          }
        }
        uint4 u[2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          u[j].x = pack_bf16x2(o[j * 8 + 0], o[j * 8 + 1]);
          u[j].y = pack_bf16x2(o[j * 8 + 2], o[j * 8 + 3]);
          u[j].z = pack_bf16x2(o[j * 8 + 4], o[j * 8 + 5]);
          u[j].w = pack_bf16x2(o[j * 8 + 6], o[j * 8 + 7]);
        }
        const int sc = s0 + ci * 16;
        if (out_tma) {
          if ((ci & 1) == 0) {
            if (lane == 0) tma_store_wait_read<0>();   // the previous box of this warp has left the staging rows
            __syncwarp();
          }
          *reinterpret_cast<uint4*>(stage_w + swz64_offset(lane, (ci & 1) * 2)) = u[0];
          *reinterpret_cast<uint4*>(stage_w + swz64_offset(lane, (ci & 1) * 2 + 1)) = u[1];
          if (ci & 1) {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_store_3d(&tmP, stage_w, s0 + (ci >> 1) * 32, i, grp * 128 + q * 32);   // entries past Np are clipped
              tma_store_commit();
            }
          }
        } else if (wide && sc + 16 <= p.Np) {
          st_global_256(dst + ci * 16, u[0], u[1]);   // a whole 32-byte sector per lane
        } else {
          if (sc < p.Np) *reinterpret_cast<uint4*>(dst + ci * 16) = u[0];
          if (sc + 8 < p.Np) *reinterpret_cast<uint4*>(dst + ci * 16 + 8) = u[1];
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[grp]);
      if (++stage == kTPStages) {
        stage = 0;
        phase ^= 1u;
      }
      acc_phase ^= 1u;
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

constexpr int kTPSmemBytes = kTPWBytes + kTPStages * kTPXBytes + kTPOutBytes + 2 * 2 * 3 * 128 * 4 + 256 + 1024;
static_assert(kTPSmemBytes <= 232448, "shared memory of one CTA");

}  // namespace ubm

// z: [rows*N][128] bf16.  w: [512][128] bf16 = rows [p_a; g_a; p_b; g_b] each already multiplied by
// the LayerNorm gamma.  colsum/colbias: fp32 [512].  mask: fp32 [rows*N] or null.
// planes: bf16 [2][128][plane_rows][Np] (Np multiple of 8, >= N); entries N..Np-1 of a row are written as zeros
// up to the end of the last 128-wide tile.
static int trimul_proj_impl(const void* z, const void* w, const void* colsum, const void* colbias,
                                    const void* mask, void* planes, void* stats_out, int rows, int plane_rows, int N,
                                    int Np, void* status, void* stream, const void* const* z_ptrs,
                                    const int* peer_rows, int npeers, int me) {
  using namespace ubm;
  if (N <= 0 || rows <= 0 || plane_rows < rows || Np < N || (Np & 7)) return UBM_ERR_ARGUMENT;
  TrimulProjParams p = {};
  p.R = static_cast<long long>(rows) * N;
  if (p.R > 0x7fffffffLL) return UBM_ERR_ARGUMENT;   // flat pair index is a 32-bit TMA coordinate
  p.rows = rows;
  p.plane_rows = plane_rows;
  p.N = N;
  p.Np = Np;
  p.tiles_per_row = (N + kTPRows - 1) / kTPRows;
  p.num_tiles = rows * p.tiles_per_row;
  p.colsum = static_cast<const float*>(colsum);
  p.colbias = static_cast<const float*>(colbias);
  p.mask = static_cast<const float*>(mask);
  p.planes = static_cast<__nv_bfloat16*>(planes);
  p.stats_out = static_cast<float*>(stats_out);
  p.status = static_cast<KernelStatus*>(status);
  CUtensorMap tmX, tmW;
  uint64_t dX[2] = {(uint64_t)kTPC, (uint64_t)p.R};
  uint64_t sX[1] = {(uint64_t)kTPC * 2};
  uint32_t bX[2] = {64, kTPRows};
  int rc = make_tmap(&tmX, z, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, dX, sX, bX, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  uint64_t dW[2] = {(uint64_t)kTPC, 512};
  uint64_t sW[1] = {(uint64_t)kTPC * 2};
  uint32_t bW[2] = {64, 256};
  rc = make_tmap(&tmW, w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, dW, sW, bW, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  PeerSrcMaps maps;
  for (int q = 0; q < kMaxSrcPeers; ++q) maps.m[q] = tmX;
  if (npeers > 0) {
    rc = make_peer_src(&maps, &p.src, z_ptrs, peer_rows, npeers, me, N, tmX);
    if (rc) return rc;
  }
  CUtensorMap tmP = tmX;
  p.out_tma = 0;
  {
    static const bool on = [] {
      const char* e = getenv("UBM_PROJ_TMA_STORE");
      return e == nullptr || e[0] != '0';
    }();
    if (on && (reinterpret_cast<uintptr_t>(planes) & 15) == 0) {
      uint64_t dP[3] = {(uint64_t)Np, (uint64_t)plane_rows, 256};
      uint64_t sP[2] = {(uint64_t)Np * 2, (uint64_t)plane_rows * Np * 2};
      uint32_t bP[3] = {32, 1, 32};
      rc = make_tmap(&tmP, planes, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dP, sP, bP, CU_TENSOR_MAP_SWIZZLE_64B);
      if (rc) return rc;
      p.out_tma = 1;
    }
  }
  rc = set_smem(trimul_proj_kernel, kTPSmemBytes);
  if (rc) return rc;
  const int grid = p.num_tiles < sm_count() ? p.num_tiles : sm_count();
  trimul_proj_kernel<<<grid, 320, kTPSmemBytes, static_cast<cudaStream_t>(stream)>>>(tmX, tmW, maps, tmP, p);
  UBM_CHECK_LAUNCH("trimul_proj_kernel");
  return UBM_OK;
}

extern "C" int ubm_trimul_proj_rows(const void* z, const void* w, const void* colsum, const void* colbias,
                                    const void* mask, void* planes, void* stats_out, int rows, int plane_rows, int N,
                                    int Np, void* status, void* stream) {
  return trimul_proj_impl(z, w, colsum, colbias, mask, planes, stats_out, rows, plane_rows, N, Np, status, stream,
                          nullptr, nullptr, 0, 0);
}

// The incoming-edge form on a row-sharded pair tensor: this GPU projects COLUMNS [col0, col0 + rows) of z (col0 =
// first row it owns), reading every 128-entry tile of a column from the GPU that owns those rows with a plain TMA
// load (no multicast): the distributed transpose and the LayerNorm + gated a / b projections are one kernel.
// z_ptrs[q] = GPU q's shard bf16 [peer_rows[q]][N][128] in symmetric memory; N and shard boundaries multiples of
// 128.  mask, if given, is this GPU's fp32 [rows][N] mask of the TRANSPOSED rows.  Outputs as ubm_trimul_proj_rows.
extern "C" int ubm_trimul_proj_rows_peer(const void* const* z_ptrs, const int* peer_rows, int npeers, int me,
                                         const void* w, const void* colsum, const void* colbias, const void* mask,
                                         void* planes, int rows, int plane_rows, int N, int Np, void* status,
                                         void* stream) {
  if (z_ptrs == nullptr || peer_rows == nullptr || npeers < 1 || me < 0 || me >= npeers || rows != peer_rows[me])
    return ubm::UBM_ERR_ARGUMENT;
  return trimul_proj_impl(z_ptrs[me], w, colsum, colbias, mask, planes, nullptr, rows, plane_rows, N, Np, status,
                          stream, z_ptrs, peer_rows, npeers, me);
}

extern "C" int ubm_trimul_proj(const void* z, const void* w, const void* colsum, const void* colbias, const void* mask,
                               void* planes, void* stats_out, int N, int Np, void* status, void* stream) {
  return ubm_trimul_proj_rows(z, w, colsum, colbias, mask, planes, stats_out, N, N, N, Np, status, stream);
}
