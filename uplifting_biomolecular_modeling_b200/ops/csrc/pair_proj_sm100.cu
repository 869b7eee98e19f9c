// Fused LayerNorm -> 512-wide projection of pair rows, with the op-specific epilogue.
//
// Epilogue (MODE_TRIATT): q | k | v | sigmoid(g) rows (bf16, [row][128]) plus the per-head pair bias
// planes bias[h][j][k]; optionally at the transposed pair index (ending node).  Reference: the
// triangle-attention prologue (common/opt_core/opt_core/attn/pair_fused.py:1136, N15
// triatt_procuda_sm90.cu).  (The triangle-multiplication projection, whose planes want the transposed
// accumulator orientation, is a kernel of its own in trimul_proj_sm100.cu.)
//
// LayerNorm is folded into the GEMM: with W' = W * gamma (per input channel),
//   W.LN(x) = rstd * (W'.x - mu * rowsum(W')) + W.beta,
// so the raw bf16 row tile that TMA brings in is the A operand as it stands, and the row
// statistics (computed from the same shared-memory tile while the MMAs run) are applied to the
// fp32 accumulator in the epilogue.  The 512 x 128 weight matrix stays resident in shared memory
// for the life of the persistent CTA; only row tiles stream.
//
// Warps: 0 = TMA producer, 1 = MMA issuer, 2-5 = epilogue group 0 (output half 0),
// 6-9 = epilogue group 1 (output half 1).  Each half is one 128 x 256 accumulator in TMEM, so
// the epilogue of half 0 overlaps the MMAs of half 1 and of the next tile.
#include "host_util.h"
#include "sm100.cuh"

namespace ubm {

constexpr int kPPRows = 128;   // rows per tile
constexpr int kPPC = 128;      // input channels
constexpr int kPPStages = 2;   // row-tile ring
constexpr int kPPXBytes = kPPRows * kPPC * 2;        // 32 KB, two k-blocks of [128][64]
constexpr int kPPWBytes = 512 * kPPC * 2;            // 128 KB, two k-blocks of [512][64]
constexpr int kPPMaxHeads = 8;

enum { MODE_TRIMUL = 0, MODE_TRIATT = 1 };

struct PairProjParams {
  long long R;       // number of pair rows (rows * N)
  int rows;          // first pair index extent (N for a whole pair tensor, fewer for a row shard)
  int plane_rows;    // rows the output planes are allocated for (>= rows; equal-sized symmetric buffers)
  int N;             // tokens (second pair index extent)
  int Np;            // leading dimension of planes (>= N, multiple of 8)
  const float* colsum;   // [512]  rowsum(W') per output column
  const float* colbias;  // [512]  W.beta (+ bias) per output column
  __nv_bfloat16* q;  // each [R][128], row index possibly transposed
  __nv_bfloat16* k;
  __nv_bfloat16* v;
  __nv_bfloat16* g;
  __nv_bfloat16* headbias;   // [H][rows][Np]
  const float* wb;           // [H][128] head-bias weights already multiplied by gamma
  const float* wb_colsum;    // [H]
  const float* wb_colbias;   // [H]
  int H;
  int transpose_out;
  float* stats_out;  // optional [R][2] (mu, rstd) of the input rows, or null
  KernelStatus* status;
  int num_tiles;
  PeerSrc src;       // src.n > 0: the input rows are columns of z fetched from their owners (see host_util.h)
  // q | k | v | gate leave through shared memory: every epilogue warp stages its 32 rows x 32 columns (64-byte
  // swizzle) and one lane stores the box with a bulk tensor copy (maps in PairOutMaps).  Off when a warp's 32 rows
  // could straddle two values of the first pair index under the transposed write (N not a multiple of 32).
  int out_tma;
};

// Output maps, one per q / k / v / gate buffer.  Plain write: {128, R, 1} with boxes {32, 32, 1} at (column, row, 0).
// Transposed write (ending node): {128, N, N} = out[pk][pi][channel] with boxes {32, 1, 32} at (column, pi, pk0):
// 32 consecutive second indices of one first index land on 32 rows that are N * 128 elements apart.
struct PairOutMaps {
  CUtensorMap m[4];
};
constexpr int kPPOutWarpBytes = 32 * 64;
constexpr int kPPOutBytes = 8 * kPPOutWarpBytes;

// Optional timeline (build with -DUBM_PP_TIMELINE): CTA 0 stamps clock64 at fixed points of its first tiles
// into a global buffer [4 roles][kPPTlTiles][8 events] (roles: producer, MMA issuer, epilogue group 0, 1).
#ifdef UBM_PP_TIMELINE
constexpr int kPPTlTiles = 32;
__device__ long long g_pp_timeline[4 * kPPTlTiles * 8];
#define PP_STAMP(role, tile, ev)                                                                              \
  do {                                                                                                        \
    if (blockIdx.x == 0 && (tile) < kPPTlTiles) g_pp_timeline[((role) * kPPTlTiles + (tile)) * 8 + (ev)] = clock64(); \
  } while (0)
#else
#define PP_STAMP(role, tile, ev) do { } while (0)
#endif

template <int MODE>
__global__ void __launch_bounds__(320, 1)
pair_proj_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
                 const __grid_constant__ PeerSrcMaps peers, const __grid_constant__ PairOutMaps outs,
                 PairProjParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sW = smem;                               // 128 KB
  uint8_t* sX = smem + kPPWBytes;                   // stages * 32 KB
  uint8_t* sOut = sX + kPPStages * kPPXBytes;       // 8 warps x 2 KB of output staging
  float* sColsum = reinterpret_cast<float*>(sOut + kPPOutBytes);          // 512
  float* sColbias = sColsum + 512;                                         // 512
  float* sWb = sColbias + 512;                                             // kPPMaxHeads * 128
  uint64_t* bars = reinterpret_cast<uint64_t*>(sWb + kPPMaxHeads * 128);
  uint64_t* x_full = bars;                 // [stages]
  uint64_t* x_empty = x_full + kPPStages;  // [stages]
  uint64_t* w_full = x_empty + kPPStages;  // [1]
  uint64_t* acc_full = w_full + 1;         // [2]
  uint64_t* acc_empty = acc_full + 2;      // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const WaitScope ws{abort_flag, p.status};

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kPPStages; ++s) {
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
  // column constants
  for (int i = threadIdx.x; i < 512; i += blockDim.x) {
    sColsum[i] = p.colsum[i];
    sColbias[i] = p.colbias[i];
  }
  if (MODE == MODE_TRIATT) {
    for (int i = threadIdx.x; i < p.H * 128; i += blockDim.x) sWb[i] = p.wb[i];
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      // resident weights: two k-blocks, each 512 rows loaded as two boxes of 256 rows
      mbar_expect_tx(w_full, kPPWBytes);
      for (int kb = 0; kb < 2; ++kb)
        for (int h = 0; h < 2; ++h)
          tma_load_2d(sW + kb * 65536 + h * 32768, &tmW, w_full, kb * 64, h * 256);
      int stage = 0;
      uint32_t phase = 0;
      int lt = 0;
      for (int t = blockIdx.x; t < p.num_tiles; t += gridDim.x, ++lt) {
        PP_STAMP(0, lt, 0);
        mbar_wait(&x_empty[stage], phase ^ 1u, ws, 11, stage);
        PP_STAMP(0, lt, 1);
        if (*abort_flag) break;
        uint8_t* dst = sX + stage * kPPXBytes;
        mbar_expect_tx(&x_full[stage], kPPXBytes);
        if (p.src.n > 0) {
          // transposed source: tile = (column col0 + i of z, rows k0 .. k0 + 127), fetched from the owner of k0
          const int tiles_per_row = p.N / kPPRows;
          const int i = t / tiles_per_row;
          const int k0 = (t - i * tiles_per_row) * kPPRows;
          int q = 0;
#pragma unroll
          for (int j = 1; j < kMaxSrcPeers; ++j)
            if (j < p.src.n && k0 >= p.src.row0[j]) q = j;
          tma_load_3d(dst, &peers.m[q], &x_full[stage], 0, p.src.col0 + i, k0 - p.src.row0[q]);
          tma_load_3d(dst + 16384, &peers.m[q], &x_full[stage], 64, p.src.col0 + i, k0 - p.src.row0[q]);
        } else {
          tma_load_2d(dst, &tmX, &x_full[stage], 0, t * kPPRows);
          tma_load_2d(dst + 16384, &tmX, &x_full[stage], 64, t * kPPRows);
        }
        if (++stage == kPPStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (warp-uniform loop, elected lane issues)
    const bool leader = elect_one();
    {
      constexpr uint32_t idesc = umma_idesc_bf16(128, 256);
      mbar_wait(w_full, 0, ws, 12);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase = 0;
      int lt = 0;
      for (int t = blockIdx.x; t < p.num_tiles; t += gridDim.x, ++lt) {
        if (lane == 0) PP_STAMP(1, lt, 0);
        mbar_wait(&x_full[stage], phase, ws, 13, stage);
        if (lane == 0) PP_STAMP(1, lt, 1);
        tc_fence_after_sync();
        const uint32_t xa = smem_u32(sX + stage * kPPXBytes);
        const uint32_t wa = smem_u32(sW);
        for (int h = 0; h < 2; ++h) {
          mbar_wait(&acc_empty[h], acc_phase ^ 1u, ws, 14, h);
          if (lane == 0) PP_STAMP(1, lt, 2 + 2 * h);
          tc_fence_after_sync();
          const uint64_t ad0 = umma_smem_desc(xa, 16, 1024, kSwizzle128);
          const uint64_t bd0 = umma_smem_desc(wa + h * 32768, 16, 1024, kSwizzle128);
          if (leader) {
#pragma unroll
            for (int kb = 0; kb < 2; ++kb) {
#pragma unroll
              for (int k = 0; k < 4; ++k)
                umma_ss(tmem_base + h * 256, ad0 + static_cast<uint64_t>(kb * (16384 >> 4) + k * 2),
                        bd0 + static_cast<uint64_t>(kb * (65536 >> 4) + k * 2), idesc, (kb | k) != 0 ? 1u : 0u);
            }
            umma_commit(&acc_full[h]);
          }
          __syncwarp();
          if (lane == 0) PP_STAMP(1, lt, 3 + 2 * h);
        }
        if (leader) umma_commit(&x_empty[stage]);
        __syncwarp();
        if (++stage == kPPStages) {
          stage = 0;
          phase ^= 1u;
        }
        acc_phase ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue groups
    const int grp = (warp - 2) >> 2;  // 0 or 1: which 256-column half
    const int q = warp & 3;           // TMEM lane quadrant
    const int row_in_tile = q * 32 + lane;
    const bool out_tma = p.out_tma != 0;                 // warp-uniform
    uint8_t* stage_w = sOut + (warp - 2) * kPPOutWarpBytes;
    int stage = 0;
    uint32_t phase = 0;
    uint32_t acc_phase = 0;
    int lt = 0;
    for (int t = blockIdx.x; t < p.num_tiles; t += gridDim.x, ++lt) {
      const long long r = static_cast<long long>(t) * kPPRows + row_in_tile;
      const bool row_ok = r < p.R;
      // ---- row statistics (and head bias) from the shared-memory tile
      if (q == 0 && lane == 0) PP_STAMP(2 + grp, lt, 0);
      mbar_wait(&x_full[stage], phase, ws, 15, stage);
      if (q == 0 && lane == 0) PP_STAMP(2 + grp, lt, 1);
      const uint8_t* xs = sX + stage * kPPXBytes;
      float sum = 0.f, sumsq = 0.f;
      float hb[kPPMaxHeads / 2];
#pragma unroll
      for (int h = 0; h < kPPMaxHeads / 2; ++h) hb[h] = 0.f;
      const int hpg = (MODE == MODE_TRIATT) ? (p.H + 1) / 2 : 0;  // heads per group
#pragma unroll 4
      for (int c16 = 0; c16 < 16; ++c16) {
        const int kb = c16 >> 3;
        const uint4 u = *reinterpret_cast<const uint4*>(xs + kb * 16384 + swz128_offset(row_in_tile, c16 & 7));
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
        float e[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          e[2 * j] = bf16_lo(w[j]);
          e[2 * j + 1] = bf16_hi(w[j]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          sum += e[j];
          sumsq += e[j] * e[j];
        }
        if (MODE == MODE_TRIATT) {
#pragma unroll
          for (int h = 0; h < kPPMaxHeads / 2; ++h) {
            if (h < hpg) {
              const float* wrow = sWb + (grp * hpg + h) * 128 + c16 * 8;
              const float4 w0 = *reinterpret_cast<const float4*>(wrow);
              const float4 w1 = *reinterpret_cast<const float4*>(wrow + 4);
              hb[h] += e[0] * w0.x + e[1] * w0.y + e[2] * w0.z + e[3] * w0.w + e[4] * w1.x + e[5] * w1.y +
                       e[6] * w1.z + e[7] * w1.w;
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&x_empty[stage]);
      const float mu = sum * (1.0f / kPPC);
      const float var = fmaxf(sumsq * (1.0f / kPPC) - mu * mu, 0.f);
      const float rstd = rsqrtf(var + 1e-5f);
      if (p.stats_out != nullptr && grp == 0 && row_ok) {
        p.stats_out[2 * r] = mu;
        p.stats_out[2 * r + 1] = rstd;
      }
      // pair index of this row
      int pi = 0, pk = 0;
      if (row_ok) {
        pi = static_cast<int>(r / p.N);
        pk = static_cast<int>(r - static_cast<long long>(pi) * p.N);
      }

      if (MODE == MODE_TRIATT && row_ok) {
        const int oi = p.transpose_out ? pk : pi;
        const int ok = p.transpose_out ? pi : pk;
#pragma unroll
        for (int h = 0; h < kPPMaxHeads / 2; ++h) {
          const int head = grp * hpg + h;
          if (h < hpg && head < p.H) {
            const float val = rstd * (hb[h] - mu * p.wb_colsum[head]) + p.wb_colbias[head];
            p.headbias[(static_cast<long long>(head) * p.plane_rows + oi) * p.Np + ok] = __float2bfloat16(val);
          }
        }
      }

      // ---- accumulator half of this group
      if (q == 0 && lane == 0) PP_STAMP(2 + grp, lt, 2);
      mbar_wait(&acc_full[grp], acc_phase, ws, 16, grp);
      if (q == 0 && lane == 0) PP_STAMP(2 + grp, lt, 3);
      tc_fence_after_sync();
      const uint32_t tbase = tmem_addr(tmem_base, q, grp * 256);
      {
        // half 0 = [q | k], half 1 = [v | g]; rows written at (possibly transposed) pair index
        const long long orow = p.transpose_out ? (static_cast<long long>(pk) * p.N + pi) : r;
        __nv_bfloat16* o0 = (grp == 0 ? p.q : p.v) + orow * 128;
        __nv_bfloat16* o1 = (grp == 0 ? p.k : p.g) + orow * 128;
        const float2 a2 = make_float2(rstd, rstd);
        const float2 b2 = make_float2(-mu * rstd, -mu * rstd);
        // 32-column chunks, the tensor-memory load of the next chunk in flight while this one is processed;
        // the chunk body exists twice (ping-pong registers), not eight times
        // first row of this warp's 32 (a multiple of 32): its pair index places the warp's output box
        const long long r0 = static_cast<long long>(t) * kPPRows + q * 32;
        const int bi = static_cast<int>(r0 / p.N);
        const int bk = static_cast<int>(r0 - static_cast<long long>(bi) * p.N);
        auto chunk = [&](const uint32_t (&av)[32], const int c0) {
          if (out_tma) {
            if (lane == 0) tma_store_wait_read<0>();    // the previous box of this warp has left the staging rows
            __syncwarp();
          }
          if (row_ok) {
            if (q == 0 && lane == 0 && c0 == 32) PP_STAMP(2 + grp, lt, 5);
            float f[32];
            ln_fold32(av, a2, b2, sColsum + grp * 256 + c0, sColbias + grp * 256 + c0, f);
            if (grp == 1 && c0 >= 128) {      // gate columns (warp-uniform)
#pragma unroll
              for (int j = 0; j < 32; ++j) f[j] = sigmoidf_fast(f[j]);
            }
            if (q == 0 && lane == 0 && c0 == 32) PP_STAMP(2 + grp, lt, 6);
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
              __nv_bfloat16* dst = (c0 < 128 ? o0 + c0 : o1 + (c0 - 128));
              st_bf16x16(dst, f);
              st_bf16x16(dst + 16, f + 16);
            }
            if (q == 0 && lane == 0 && c0 == 32) PP_STAMP(2 + grp, lt, 7);
          }
          if (out_tma) {
            // rows past R hold stale bytes: the copy clips them
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              const CUtensorMap* om = &outs.m[grp * 2 + (c0 >> 7)];
              if (p.transpose_out) tma_store_3d(om, stage_w, c0 & 127, bi, bk);
              else tma_store_3d(om, stage_w, c0 & 127, static_cast<int>(r0), 0);
              tma_store_commit();
            }
          }
        };
        uint32_t va[32], vb[32];
        tmem_ld32(tbase, va);
#pragma unroll 1
        for (int c0 = 0; c0 < 256; c0 += 64) {
          tmem_ld_wait();
          tmem_ld32(tbase + c0 + 32, vb);
          chunk(va, c0);
          tmem_ld_wait();
          if (c0 + 64 < 256) tmem_ld32(tbase + c0 + 64, va);
          chunk(vb, c0 + 32);
        }
      }
      if (q == 0 && lane == 0) PP_STAMP(2 + grp, lt, 4);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[grp]);
      if (++stage == kPPStages) {
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

constexpr int kPPSmemBytes =
    kPPWBytes + kPPStages * kPPXBytes + kPPOutBytes + (512 + 512 + kPPMaxHeads * 128) * 4 + 256 + 1024;
static_assert(kPPSmemBytes <= 232448, "shared memory of one CTA");

template <int MODE>
static int launch_pair_proj(const void* x, const void* w, PairProjParams p, cudaStream_t stream,
                            const void* const* z_ptrs = nullptr, const int* peer_rows = nullptr, int npeers = 0,
                            int me = 0) {
  CUtensorMap tmX, tmW;
  uint64_t dX[2] = {(uint64_t)kPPC, (uint64_t)p.R};
  uint64_t sX[1] = {(uint64_t)kPPC * 2};
  uint32_t bX[2] = {64, kPPRows};
  int rc = make_tmap(&tmX, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, dX, sX, bX, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  PeerSrcMaps maps;
  for (int q = 0; q < kMaxSrcPeers; ++q) maps.m[q] = tmX;
  if (npeers > 0) {
    rc = make_peer_src(&maps, &p.src, z_ptrs, peer_rows, npeers, me, p.N, tmX);
    if (rc) return rc;
  }
  uint64_t dW[2] = {(uint64_t)kPPC, 512};
  uint64_t sW[1] = {(uint64_t)kPPC * 2};
  uint32_t bW[2] = {64, 256};
  rc = make_tmap(&tmW, w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, dW, sW, bW, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  p.num_tiles = static_cast<int>((p.R + kPPRows - 1) / kPPRows);
  PairOutMaps outs;
  for (int i = 0; i < 4; ++i) outs.m[i] = tmX;
  p.out_tma = 0;
  {
    static const bool on = [] {
      const char* e = getenv("UBM_PROJ_TMA_STORE");
      return e == nullptr || e[0] != '0';
    }();
    void* bufs[4] = {p.q, p.k, p.v, p.g};
    bool ok = on && MODE == MODE_TRIATT && p.R < (1ll << 31) && (!p.transpose_out || (p.N % 32) == 0);
    for (int i = 0; i < 4; ++i) ok = ok && bufs[i] != nullptr && (reinterpret_cast<uintptr_t>(bufs[i]) & 15) == 0;
    if (ok) {
      for (int i = 0; i < 4; ++i) {
        if (p.transpose_out) {
          uint64_t d[3] = {128, (uint64_t)p.N, (uint64_t)p.N};
          uint64_t st[2] = {128 * 2, (uint64_t)p.N * 128 * 2};
          uint32_t b[3] = {32, 1, 32};
          rc = make_tmap(&outs.m[i], bufs[i], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, d, st, b,
                         CU_TENSOR_MAP_SWIZZLE_64B);
        } else {
          uint64_t d[3] = {128, (uint64_t)p.R, 1};
          uint64_t st[2] = {128 * 2, (uint64_t)p.R * 128 * 2};
          uint32_t b[3] = {32, 32, 1};
          rc = make_tmap(&outs.m[i], bufs[i], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, d, st, b,
                         CU_TENSOR_MAP_SWIZZLE_64B);
        }
        if (rc) return rc;
      }
      p.out_tma = 1;
    }
  }
  auto kern = pair_proj_kernel<MODE>;
  rc = set_smem(kern, kPPSmemBytes);
  if (rc) return rc;
  const int grid = p.num_tiles < sm_count() ? p.num_tiles : sm_count();
  kern<<<grid, 320, kPPSmemBytes, stream>>>(tmX, tmW, maps, outs, p);
  UBM_CHECK_LAUNCH("pair_proj_kernel");
  return UBM_OK;
}

}  // namespace ubm

// w: [512][128] bf16 = rows [q; k; v; g] (gamma folded, q pre-scaled by 1/sqrt(d)).
// wb: fp32 [H][128] head-bias weights (gamma folded); wb_colsum/wb_colbias fp32 [H].
// q,k,v,g: bf16 [N*N][128]; headbias: bf16 [H][N][Np].
static int triatt_proj_impl(const void* z, const void* w, const void* colsum, const void* colbias,
                                    const void* wb, const void* wb_colsum, const void* wb_colbias, void* q, void* k,
                                    void* v, void* g, void* headbias, void* stats_out, int rows, int plane_rows, int N,
                                    int Np, int H, int transpose_out, void* status, void* stream,
                                    const void* const* z_ptrs, const int* peer_rows, int npeers, int me) {
  using namespace ubm;
  if (N <= 0 || rows <= 0 || plane_rows < rows || Np < N || (Np & 7) || H <= 0 || H > kPPMaxHeads)
    return UBM_ERR_ARGUMENT;
  if (transpose_out && rows != N) return UBM_ERR_ARGUMENT;  // the transposed write needs the whole square
  PairProjParams p = {};
  p.R = static_cast<long long>(rows) * N;
  p.rows = rows;
  p.plane_rows = plane_rows;
  p.N = N;
  p.Np = Np;
  p.colsum = static_cast<const float*>(colsum);
  p.colbias = static_cast<const float*>(colbias);
  p.q = static_cast<__nv_bfloat16*>(q);
  p.k = static_cast<__nv_bfloat16*>(k);
  p.v = static_cast<__nv_bfloat16*>(v);
  p.g = static_cast<__nv_bfloat16*>(g);
  p.headbias = static_cast<__nv_bfloat16*>(headbias);
  p.wb = static_cast<const float*>(wb);
  p.wb_colsum = static_cast<const float*>(wb_colsum);
  p.wb_colbias = static_cast<const float*>(wb_colbias);
  p.H = H;
  p.transpose_out = transpose_out;
  p.stats_out = static_cast<float*>(stats_out);
  p.status = static_cast<KernelStatus*>(status);
  return launch_pair_proj<MODE_TRIATT>(z, w, p, static_cast<cudaStream_t>(stream), z_ptrs, peer_rows, npeers, me);
}

extern "C" int ubm_triatt_proj_rows(const void* z, const void* w, const void* colsum, const void* colbias,
                                    const void* wb, const void* wb_colsum, const void* wb_colbias, void* q, void* k,
                                    void* v, void* g, void* headbias, void* stats_out, int rows, int plane_rows, int N,
                                    int Np, int H, int transpose_out, void* status, void* stream) {
  return triatt_proj_impl(z, w, colsum, colbias, wb, wb_colsum, wb_colbias, q, k, v, g, headbias, stats_out, rows,
                          plane_rows, N, Np, H, transpose_out, status, stream, nullptr, nullptr, 0, 0);
}

// The ending-node form on a row-sharded pair tensor: this GPU projects COLUMNS [col0, col0 + rows) of z, where
// col0 is the first row it owns.  z_ptrs[q] = GPU q's shard bf16 [peer_rows[q]][N][128] (symmetric memory, written
// and made visible before this launch); the kernel fetches every 128-entry tile from its owner with a plain TMA
// load (no multicast), so the distributed transpose and the LayerNorm + q|k|v|gate + head-bias projection are one
// kernel.  N and the shard boundaries must be multiples of 128.  Outputs as ubm_triatt_proj_rows.
extern "C" int ubm_triatt_proj_rows_peer(const void* const* z_ptrs, const int* peer_rows, int npeers, int me,
                                         const void* w, const void* colsum, const void* colbias, const void* wb,
                                         const void* wb_colsum, const void* wb_colbias, void* q, void* k, void* v,
                                         void* g, void* headbias, int rows, int plane_rows, int N, int Np, int H,
                                         void* status, void* stream) {
  if (z_ptrs == nullptr || peer_rows == nullptr || npeers < 1 || me < 0 || me >= npeers || rows != peer_rows[me])
    return ubm::UBM_ERR_ARGUMENT;
  return triatt_proj_impl(z_ptrs[me], w, colsum, colbias, wb, wb_colsum, wb_colbias, q, k, v, g, headbias, nullptr,
                          rows, plane_rows, N, Np, H, 0, status, stream, z_ptrs, peer_rows, npeers, me);
}

#ifdef UBM_PP_TIMELINE
extern "C" int ubm_pair_proj_read_timeline(long long* host_out) {
  return cudaMemcpyFromSymbol(host_out, ubm::g_pp_timeline, sizeof(ubm::g_pp_timeline)) == cudaSuccess ? 0 : -1;
}
#endif

extern "C" int ubm_triatt_proj(const void* z, const void* w, const void* colsum, const void* colbias, const void* wb,
                               const void* wb_colsum, const void* wb_colbias, void* q, void* k, void* v, void* g,
                               void* headbias, void* stats_out, int N, int Np, int H, int transpose_out, void* status,
                               void* stream) {
  return ubm_triatt_proj_rows(z, w, colsum, colbias, wb, wb_colsum, wb_colbias, q, k, v, g, headbias, stats_out, N, N,
                              N, Np, H, transpose_out, status, stream);
}
