// Batched bf16 GEMM on tcgen05 tensor cores with TMA-fed operands and TMEM accumulators.
//
//   C[b][m][n] = act(alpha * sum_k A[b][m][k] * B[b][n][k] + bias[n]) + R[b][m][n]
//
// Two operand layouts:
//   K-major  ("TN"): A is [batch][M][K], B is [batch][N][K], K contiguous.
//   MN-major ("NT"): A is [batch][K][M], B is [batch][K][N], M / N contiguous.
// The triangle-multiplication contraction uses both: with channel-major planes
// P[c][r][s] = proj(z[r,s,:])[c] the outgoing update is sum_k Pa[c][i][k] Pb[c][j][k]
// (K-major) and the incoming update is sum_k Pa[c][k][i] Pb[c][k][j] (MN-major), so one
// projection kernel serves both directions and no transposed copy is ever written.
// In the reference this contraction is a cuBLAS strided-batched GEMM
// (common/opt_core/opt_core/kernels/trimul/native/DESIGN.md:21-47).
//
// Kernel shape: persistent CTAs (one per SM), 128 x BN output tile, 64-wide K blocks in a
// multi-stage TMA ring, warp 0 = TMA producer, warp 1 = MMA issuer, warps 2-5 = epilogue.
// Two TMEM accumulator buffers let the epilogue of tile t overlap the MMAs of tile t+1.
#include "host_util.h"
#include "sm100.cuh"

namespace ubm {

struct GemmParams {
  int M, N, K, batch;
  void* C;
  long long ldc, strideC;
  const float* bias;
  const __nv_bfloat16* residual;
  long long ldr, strideR;
  float alpha;
  int out_fp32;
  // 0 none, 1 silu, 2 sigmoid, 3 gelu (erf), 4 relu; 5 = three-way SwiGLU over column triples (192-wide tiles
  // only): the N columns come in groups of 96 = 32 gate | 32 value | 32 second value, and the output, N / 3 columns
  // wide, is silu(gate) * value * second value - the conditioned transition's swish gate and its a_to_b branch
  // from one projection with no [M, N] intermediate; 6 = two-way SwiGLU over column pairs (256-wide tiles): groups
  // of 64 = 32 gate | 32 value, output N / 2 columns wide
  int act;
  // 1: A and B are e4m3 bytes (K-major, one GPU): 128 elements per k-block instead of 64, tcgen05.mma kind::f8f6f4;
  // the accumulator is scaled by alpha * *alpha_dev (the product of the two dequantisation factors)
  int fp8;
  const float* alpha_dev;  // device scalar multiplied into alpha (written by the kernel that quantised A), or null
  int act_col0;  // the activation applies to output columns >= act_col0 (a multiple of 32; 0 = all columns)
  int res_tma;  // residual tiles arrive by TMA (tensor map in the auxiliary map slot 0)
  // bf16 output leaves through shared memory: every epilogue warp stages its 32 rows x 64 columns (128-byte swizzle;
  // 32 columns in the 64-byte swizzle for the SwiGLU form) and one lane stores the box with a bulk tensor copy
  // (tensor map in the auxiliary map slot 1).  A row-per-lane 32-byte global store costs the warp about 375 cycles
  // (32 requests of one sector each); the staged form writes whole 128-byte lines and does not hold the warp.
  int c_tma;
  // blocked output (cblk_col != 0): element (m, n) goes to (m / 32) * cblk_hi + (m % 32) * cblk_lo +
  // (n / 32) * cblk_col + n % 32.  With m = (i, c) and n = (j, d), c, d < 32, this writes the outer-product
  // layout [(i, j)][(c, d)] directly, so no permuted copy of the product is made.
  long long cblk_hi, cblk_lo, cblk_col;
  // multiplicative gate applied after the activation and before the residual: bf16 [gate_rows][ld_gate],
  // row m uses gate row m % gate_rows (conditioning shared by several samples); values are used as they are
  const __nv_bfloat16* gate;
  long long ld_gate;
  int gate_rows;
  // Row-scattered output (the data movement of a reduce-scatter done by the epilogue): output row m belongs to
  // GPU m / c_peer_rows and is stored, with plain peer stores, into that GPU's buffer c_peer[q] at row
  // m % c_peer_rows (leading dimension ldc).  Each GPU passes the address of ITS slot in every peer's slot array,
  // so the partial products of the ranks never overlap; the owner adds the slots afterwards in rank order.
  void* c_peer[8];
  int c_peer_rows;
  KernelStatus* status;
  int tiles_m, tiles_n, num_tiles;
  // peer mode: the N dimension is the concatenation of row shards owned by several GPUs; n-tiles are
  // enumerated shard by shard and each shard's B rows are read through that GPU's tensor map
  int npeers;
  int peer_tile0[9];   // first n-tile of each shard (prefix sums), [npeers] = tiles_n
  int peer_col0[8];    // global column (= row of the gathered operand) where the shard starts
  int peer_cols[8];    // rows in the shard
  // gather-once mode: the last `copy_ctas` CTAs pull the remote shards into a local buffer, tile block by
  // tile block, and publish one flag per (batch, n-tile); compute CTAs read remote shards from that copy
  int my_rank;
  int copy_ctas;
  uint32_t* ready;     // [batch * tiles_n] flags, value >= epoch means "this B block is local now"
  uint32_t epoch;
};

constexpr int kMaxPeers = 8;
struct PeerMaps {
  CUtensorMap m[kMaxPeers];
};

// n-tile -> (shard, first global column, column limit, row offset inside the shard)
template <int BN>
__device__ __forceinline__ void decode_ntile(const GemmParams& p, int nb, int& q, int& n_base, int& n_limit,
                                             int& local_row) {
  if (p.npeers == 0) {
    q = 0;
    n_base = nb * BN;
    n_limit = p.N;
    local_row = n_base;
    return;
  }
  q = 0;
#pragma unroll
  for (int i = 1; i < kMaxPeers; ++i)
    if (i < p.npeers && nb >= p.peer_tile0[i]) q = i;
  local_row = (nb - p.peer_tile0[q]) * BN;
  n_base = p.peer_col0[q] + local_row;
  n_limit = p.peer_col0[q] + p.peer_cols[q];
}

constexpr int kBM = 128;
constexpr int kBK = 64;
// warp 0 = TMA producer, warp 1 = MMA issuer, warps 2..9 = two epilogue groups of four warps: each group covers the
// four TMEM lane quadrants and takes half of the tile's 32-column chunks.  With one group the epilogue of a
// 128 x 256 tile (about 10 us) outlasted its main loop whenever K was below about 1400.
constexpr int kGemmThreads = 320;
constexpr int kEpiGroups = 2;

template <int BN>
struct GemmCfg {
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  // BN = 128 has room for a two-slot ring of residual tiles (128 x 128 bf16 each) that the producer fills by TMA,
  // so the epilogue never waits on a global load
  static constexpr bool kResTma = (BN == 128);
  static constexpr int kStages = 4;   // 128 KB (BN = 128) to 192 KB (BN = 256) of operands in flight
  static constexpr int kResSlotBytes = kBM * 128 * 2;
  static constexpr int kResBytes = kResTma ? 2 * kResSlotBytes : 0;
  // output staging of the eight epilogue warps: 32 rows x 128 bytes each
  static constexpr int kOutWarpBytes = 32 * 128;
  static constexpr int kOutBytes = 8 * kOutWarpBytes;
  static constexpr int kSmemBytes = kStages * kStageBytes + kResBytes + kOutBytes + 1024 /*align*/ + 512 /*barriers*/;
  static_assert(kSmemBytes <= 232448, "shared memory of one CTA");
  // two accumulator buffers; the allocation is a power of two (384 columns of the 192-wide tile take 512)
  static constexpr int kTmemCols = (2 * BN <= 32) ? 32 : (2 * BN <= 64) ? 64 : (2 * BN <= 128) ? 128
                                   : (2 * BN <= 256) ? 256 : 512;
};

// Activation of one 32-column chunk.  The switch sits outside the element loop: with the (warp-uniform) choice
// made per element, every element paid an indirect branch and the 32 activations ran one after another - a
// sigmoid on a quarter of the columns of a 7680 x 768 x 4096 projection cost 33 us on top of 45.
__device__ __forceinline__ void apply_act32(float (&f)[32], int act) {
  switch (act) {
    case 1:
#pragma unroll
      for (int j = 0; j < 32; ++j) f[j] = siluf_fast(f[j]);
      break;
    case 2:
#pragma unroll
      for (int j = 0; j < 32; ++j) f[j] = sigmoidf_fast(f[j]);
      break;
    case 3:
#pragma unroll
      for (int j = 0; j < 32; ++j) f[j] = 0.5f * f[j] * (1.0f + erff(f[j] * 0.70710678118654752f));
      break;
    case 4:
#pragma unroll
      for (int j = 0; j < 32; ++j) f[j] = fmaxf(f[j], 0.0f);
      break;
    default:
      break;
  }
}


// Order of n-tiles in gather-once mode: shards are visited starting with this rank's own (no copy
// needed), then rank+1, rank+2, ... so that the ranks pull from different owners at the same time.
template <int BN>
__device__ __forceinline__ void decode_ntile_rot(const GemmParams& p, int nb_rot, int& q, int& n_base, int& n_limit,
                                                 int& local_row, int& nb_plain) {
  int acc = 0;
  q = p.my_rank;
  for (int i = 0; i < p.npeers; ++i) {
    const int qq = (p.my_rank + i) % p.npeers;
    const int nt = p.peer_tile0[qq + 1] - p.peer_tile0[qq];
    if (nb_rot < acc + nt) {
      q = qq;
      break;
    }
    acc += nt;
  }
  const int lb = nb_rot - acc;
  local_row = lb * BN;
  n_base = p.peer_col0[q] + local_row;
  n_limit = p.peer_col0[q] + p.peer_cols[q];
  nb_plain = p.peer_tile0[q] + lb;
}

// Tile order inside one batch entry.  Plain GEMMs walk the tiles in groups of kGroupM row blocks, row block
// fastest inside a group: the ~148 tiles in flight then cover about 16 x 9 blocks (16 A panels + 9 B panels)
// instead of 148 A panels and one B panel, which is what keeps a large GEMM out of DRAM (A of a 32768 x 4096
// problem does not fit L2).  Peer modes keep the column-block-major order their shard bookkeeping assumes.
constexpr int kGroupM = 16;
template <bool PEER>
__device__ __forceinline__ void decode_tile(const GemmParams& p, int r, int& nb, int& mb) {
  if (PEER) {
    nb = r / p.tiles_m;
    mb = r - nb * p.tiles_m;
    return;
  }
  const int group_size = kGroupM * p.tiles_n;
  const int g = r / group_size;
  const int first_m = g * kGroupM;
  const int gm = min(p.tiles_m - first_m, kGroupM);
  const int rr = r - g * group_size;
  nb = rr / gm;
  mb = first_m + (rr - nb * gm);
}

template <int BN, bool MN_MAJOR, bool PEER>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ PeerMaps peers, const __grid_constant__ PeerMaps gathered, GemmParams p) {
  using Cfg = GemmCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sRes = smem + Cfg::kStages * Cfg::kStageBytes;
  uint8_t* sOut = sRes + Cfg::kResBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(sOut + Cfg::kOutBytes);
  uint64_t* empty_bar = full_bar + Cfg::kStages;
  uint64_t* tfull_bar = empty_bar + Cfg::kStages;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint64_t* rfull_bar = tempty_bar + 2;
  uint64_t* rempty_bar = rfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(rempty_bar + 2);
  const bool res_tma = Cfg::kResTma && !PEER && p.res_tma != 0;
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const WaitScope ws{abort_flag, p.status};

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 4 * kEpiGroups);
      mbar_init(&rfull_bar[a], 1);
      mbar_init(&rempty_bar[a], 4 * kEpiGroups);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // Programmatic dependent launch: the set-up above (barriers, tensor memory, descriptor prefetch) touched nothing
  // that an earlier kernel writes, so it may run while the previous kernel of the stream drains; from here on the
  // kernel reads its operands.  Both instructions are no-ops for a launch without the attribute.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  const int kbk = p.fp8 ? 2 * kBK : kBK;        // elements per k-block: a 128-byte row of either type
  const int num_kb = (p.K + kbk - 1) / kbk;
  const int tiles_per_batch = p.tiles_m * p.tiles_n;
  const int compute_ctas = PEER ? static_cast<int>(gridDim.x) - p.copy_ctas : static_cast<int>(gridDim.x);
  const bool gather_once = PEER && p.copy_ctas > 0;
  // copy CTAs take the lowest block indices so that they are resident before any compute CTA can wait on them
  const int cta_id = PEER ? static_cast<int>(blockIdx.x) - p.copy_ctas : static_cast<int>(blockIdx.x);

  if (PEER && cta_id < 0) {
    // ---------------------------------------------------------------- copy role (gather-once mode)
    // One thread streams remote B blocks [BN rows x 64 k] through the shared-memory ring: TMA load from the
    // owner's memory (plain, no multicast), TMA store into the local gathered buffer; when all k-blocks of an
    // n-tile are local, its flag is published.  Every remote byte crosses NVLink exactly once.
    if (threadIdx.x == 0) {
      constexpr int kSlots = Cfg::kStages * Cfg::kStageBytes / Cfg::kBBytes;   // 32 KB slots in the ring
      static_assert(kSlots <= 2 * Cfg::kStages, "ring barriers");
      uint64_t* slot_bar = full_bar;   // full_bar and empty_bar are contiguous: 2 * kStages barriers of count 1
      const int cid = static_cast<int>(blockIdx.x);
      const int own_tiles = p.peer_tile0[p.my_rank + 1] - p.peer_tile0[p.my_rank];
      const int remote_tiles = p.tiles_n - own_tiles;
      const long long chunks = static_cast<long long>(p.batch) * remote_tiles;
      long long base_it = 0;
      for (long long ch = cid; ch < chunks && !*abort_flag; ch += p.copy_ctas) {
        const int b = static_cast<int>(ch / remote_tiles);
        const int nb_rot = own_tiles + static_cast<int>(ch - static_cast<long long>(b) * remote_tiles);
        int q, n_base, n_limit, lrow, nb_plain;
        decode_ntile_rot<BN>(p, nb_rot, q, n_base, n_limit, lrow, nb_plain);
        int kb_load = 0;
        for (int kb_store = 0; kb_store < num_kb; ++kb_store) {
          while (kb_load < num_kb && kb_load < kb_store + (kSlots - 1)) {
            const long long it = base_it + kb_load;
            const int sl = static_cast<int>(it % kSlots);
            if (it >= kSlots) tma_store_wait_read<0>();   // whatever last used this slot has been read out
            mbar_expect_tx(&slot_bar[sl], Cfg::kBBytes);
            tma_load_3d(smem + sl * Cfg::kBBytes, &peers.m[q], &slot_bar[sl], kb_load * kBK, lrow, b);
            ++kb_load;
          }
          const long long it = base_it + kb_store;
          const int sl = static_cast<int>(it % kSlots);
          mbar_wait(&slot_bar[sl], static_cast<uint32_t>((it / kSlots) & 1), ws, 5, sl);
          if (*abort_flag) break;
          tma_store_3d(&gathered.m[q], smem + sl * Cfg::kBBytes, kb_store * kBK, lrow, b);
          tma_store_commit();
        }
        base_it += num_kb;
        tma_store_wait_all<0>();     // the block is in local memory
        fence_proxy_async_all();
        __threadfence();
        asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.ready + static_cast<long long>(b) * p.tiles_n +
                                                                 nb_plain),
                     "r"(p.epoch)
                     : "memory");
      }
      tma_store_wait_all<0>();
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
      tc_fence_after_sync();
      tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
    return;
  }

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t lt = 0;   // tiles this CTA has started
      for (int t = cta_id; t < p.num_tiles; t += compute_ctas, ++lt) {
        const int b = t / tiles_per_batch;
        const int r = t - b * tiles_per_batch;
        int nb, mb;
        decode_tile<PEER>(p, r, nb, mb);
        if (res_tma) {
          // residual tile of this output tile; its slot was released by the epilogue two tiles ago
          const int rs = lt & 1;
          mbar_wait(&rempty_bar[rs], ((lt >> 1) & 1u) ^ 1u, ws, 7, rs);
          if (*abort_flag) break;
          mbar_expect_tx(&rfull_bar[rs], Cfg::kResSlotBytes);
          tma_load_3d(sRes + rs * Cfg::kResSlotBytes, &gathered.m[0], &rfull_bar[rs], nb * BN, mb * kBM, b);
          tma_load_3d(sRes + rs * Cfg::kResSlotBytes + 16384, &gathered.m[0], &rfull_bar[rs], nb * BN + 64,
                      mb * kBM, b);
        }
        int gq = 0, g_base = 0, g_limit = 0, g_lrow = 0, g_plain = 0;
        if (gather_once) {
          decode_ntile_rot<BN>(p, nb, gq, g_base, g_limit, g_lrow, g_plain);
          if (gq != p.my_rank) {
            // wait (bounded) until the copy CTAs have brought this B block into local memory
            const uint32_t* flag = p.ready + static_cast<long long>(b) * p.tiles_n + g_plain;
            const unsigned long long t0 = globaltimer_ns();
            while (ld_acquire_gpu(flag) < p.epoch) {
              if (*abort_flag) break;
              if (globaltimer_ns() - t0 > kPeerLimitNs) {
                report_failure(ws, kErrPeerTimeout, 6, static_cast<unsigned int>(g_plain));
                break;
              }
              __nanosleep(200);
            }
            fence_proxy_async_all();
          }
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          mbar_wait(&empty_bar[stage], phase ^ 1u, ws, 1, stage);
          if (*abort_flag) break;
          uint8_t* sa = smem + stage * Cfg::kStageBytes;
          uint8_t* sb = sa + Cfg::kABytes;
          mbar_expect_tx(&full_bar[stage], Cfg::kStageBytes);
          if (!MN_MAJOR) {
            tma_load_3d(sa, &tmA, &full_bar[stage], kb * kbk, mb * kBM, b);
            if (PEER && gather_once) {
              // own shard straight from the local planes, remote shards from the gathered local copy
              const CUtensorMap* bm = (gq == p.my_rank) ? &peers.m[gq] : &gathered.m[gq];
              tma_load_3d(sb, bm, &full_bar[stage], kb * kBK, g_lrow, b);
            } else if (PEER) {
              // B rows of this n-tile live on GPU q: plain (non-multicast) TMA load from its memory
              int q, n_base, n_limit, lrow;
              decode_ntile<BN>(p, nb, q, n_base, n_limit, lrow);
              tma_load_3d(sb, &peers.m[q], &full_bar[stage], kb * kBK, lrow, b);
            } else {
              tma_load_3d(sb, &tmB, &full_bar[stage], kb * kbk, nb * BN, b);
            }
          } else {
#pragma unroll
            for (int h = 0; h < kBM / 64; ++h)
              tma_load_3d(sa + h * 8192, &tmA, &full_bar[stage], mb * kBM + h * 64, kb * kBK, b);
#pragma unroll
            for (int h = 0; h < BN / 64; ++h)
              tma_load_3d(sb + h * 8192, &tmB, &full_bar[stage], nb * BN + h * 64, kb * kBK, b);
          }
          if (++stage == Cfg::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (*abort_flag) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // the whole warp runs the loop (warp-uniform operands), one elected lane issues the tcgen05 instructions
    const bool leader = elect_one();
    {
      constexpr uint32_t idesc = umma_idesc_bf16(kBM, BN, MN_MAJOR ? 1 : 0, MN_MAJOR ? 1 : 0);
      constexpr uint32_t idesc_f8 = umma_idesc_e4m3(kBM, BN);
      const bool fp8 = !MN_MAJOR && !PEER && p.fp8 != 0;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      for (int t = cta_id; t < p.num_tiles; t += compute_ctas) {
        mbar_wait(&tempty_bar[acc], acc_phase ^ 1u, ws, 2, acc);
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          mbar_wait(&full_bar[stage], phase, ws, 3, stage);
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint32_t sb = sa + Cfg::kABytes;
          const uint64_t ad0 = MN_MAJOR ? umma_smem_desc(sa, 8192, 1024, kSwizzle128)
                                        : umma_smem_desc(sa, 16, 1024, kSwizzle128);
          const uint64_t bd0 = MN_MAJOR ? umma_smem_desc(sb, 8192, 1024, kSwizzle128)
                                        : umma_smem_desc(sb, 16, 1024, kSwizzle128);
          constexpr uint64_t kStep = MN_MAJOR ? (2048 >> 4) : (32 >> 4);
          if (leader) {
            // four MMAs per 128-byte row: 16 bf16 or 32 e4m3 elements each, 32 bytes apart in both cases
            if (fp8) {
#pragma unroll
              for (int k = 0; k < kBK / 16; ++k)
                umma_ss_f8(d_tmem, ad0 + k * kStep, bd0 + k * kStep, idesc_f8, (kb | k) != 0 ? 1u : 0u);
            } else {
#pragma unroll
              for (int k = 0; k < kBK / 16; ++k)
                umma_ss(d_tmem, ad0 + k * kStep, bd0 + k * kStep, idesc, (kb | k) != 0 ? 1u : 0u);
            }
            umma_commit(&empty_bar[stage]);  // frees the smem stage once these MMAs have read it
          }
          __syncwarp();
          if (++stage == Cfg::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (leader) umma_commit(&tfull_bar[acc]);  // accumulator complete
        __syncwarp();
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9)
    const int q = warp & 3;  // TMEM lane quadrant this warp may read
    const int grp = (warp - 2) >> 2;                       // which half of the tile's column chunks
    const float alpha = p.alpha_dev != nullptr ? p.alpha * __ldg(p.alpha_dev) : p.alpha;
    constexpr int kChunksPerGroup = (BN / 32) / kEpiGroups;
    int acc = 0;
    uint32_t acc_phase = 0;
    const bool vec_ok = p.out_fp32 ? ((p.ldc & 3) == 0 && (p.strideC & 3) == 0 &&
                                      (reinterpret_cast<uintptr_t>(p.C) & 15) == 0)
                                   : ((p.ldc & 7) == 0 && (p.strideC & 7) == 0 &&
                                      (reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
    const bool c_tma = !PEER && p.c_tma != 0;                 // warp-uniform
    uint8_t* stage_w = sOut + (warp - 2) * Cfg::kOutWarpBytes;  // this warp's staging rows (1024-byte aligned)
    const CUtensorMap* tmC = &gathered.m[1];
    uint32_t lt = 0;
    for (int t = cta_id; t < p.num_tiles; t += compute_ctas, ++lt) {
      const int b = t / tiles_per_batch;
      const int r = t - b * tiles_per_batch;
      int nb, mb;
      decode_tile<PEER>(p, r, nb, mb);
      const uint8_t* rsm = sRes + (lt & 1) * Cfg::kResSlotBytes;
      if (res_tma) mbar_wait(&rfull_bar[lt & 1], (lt >> 1) & 1u, ws, 8, lt & 1);
      mbar_wait(&tfull_bar[acc], acc_phase, ws, 4, acc);
      tc_fence_after_sync();
      const int m = mb * kBM + q * 32 + lane;
      const bool row_ok = m < p.M;
      int pq, n_base, n_limit, lrow;
      if (gather_once) {
        int plain;
        decode_ntile_rot<BN>(p, nb, pq, n_base, n_limit, lrow, plain);
      } else {
        decode_ntile<BN>(p, nb, pq, n_base, n_limit, lrow);
      }
      // 32-column chunks; the TMEM load of chunk c + 1 is in flight while chunk c is processed
      const int nchunks = min(BN / 32, (n_limit - n_base + 31) / 32);   // warp-uniform
      // (the chunk body appears twice, not BN/32 times: unrolled over all chunks it outgrew the instruction cache)
      auto process = [&](const uint32_t (&v)[32], const int c) {
        const int n0 = n_base + c * 32;
        if (row_ok) {
          float f[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]) * alpha;
          if (p.bias != nullptr) {
            if (n0 + 32 <= n_limit && (reinterpret_cast<uintptr_t>(p.bias) & 15) == 0) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                const float4 bv = __ldg(reinterpret_cast<const float4*>(p.bias + n0 + j));
                f[j] += bv.x;
                f[j + 1] += bv.y;
                f[j + 2] += bv.z;
                f[j + 3] += bv.w;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (n0 + j < n_limit) f[j] += __ldg(p.bias + n0 + j);
            }
          }
          if (p.act != 0 && n0 >= p.act_col0) apply_act32(f, p.act);
          if (p.gate != nullptr) {
            const __nv_bfloat16* gr = p.gate + static_cast<long long>(m % p.gate_rows) * p.ld_gate + n0;
            if (n0 + 32 <= n_limit && (reinterpret_cast<uintptr_t>(gr) & 31) == 0) {
#pragma unroll
              for (int c2 = 0; c2 < 2; ++c2) {
                float e[16];
                ld_bf16x16(gr + c2 * 16, e);
#pragma unroll
                for (int d = 0; d < 16; ++d) f[c2 * 16 + d] *= e[d];
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (n0 + j < n_limit) f[j] *= __bfloat162float(gr[j]);
            }
          }
          if (res_tma) {
            // 32 columns = four 16-byte units of tile row q*32+lane in the swizzled 64-column block c/2
#pragma unroll
            for (int j8 = 0; j8 < 4; ++j8) {
              const uint4 u = *reinterpret_cast<const uint4*>(rsm + (c >> 1) * 16384 +
                                                              swz128_offset(q * 32 + lane, (c & 1) * 4 + j8));
              const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                f[j8 * 8 + 2 * e] += bf16_lo(w[e]);
                f[j8 * 8 + 2 * e + 1] += bf16_hi(w[e]);
              }
            }
          } else if (p.residual != nullptr) {
            const __nv_bfloat16* rr = p.residual + b * p.strideR + static_cast<long long>(m) * p.ldr + n0;
            if (n0 + 32 <= n_limit && (reinterpret_cast<uintptr_t>(rr) & 31) == 0) {
#pragma unroll
              for (int c = 0; c < 2; ++c) {
                float e[16];
                ld_bf16x16(rr + c * 16, e);
#pragma unroll
                for (int d = 0; d < 16; ++d) f[c * 16 + d] += e[d];
              }
            } else if (n0 + 32 <= n_limit && (p.ldr & 7) == 0 && (p.strideR & 7) == 0 &&
                (reinterpret_cast<uintptr_t>(p.residual) & 15) == 0) {
#pragma unroll
              for (int j8 = 0; j8 < 4; ++j8) {
                const uint4 u = __ldg(reinterpret_cast<const uint4*>(rr) + j8);
                const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  f[j8 * 8 + 2 * e] += bf16_lo(w[e]);
                  f[j8 * 8 + 2 * e + 1] += bf16_hi(w[e]);
                }
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (n0 + j < n_limit) f[j] += __bfloat162float(rr[j]);
            }
          }
          char* c_base = reinterpret_cast<char*>(p.C);
          long long m_out = m;
          if (p.c_peer_rows > 0) {
            const int owner = m / p.c_peer_rows;
            c_base = reinterpret_cast<char*>(p.c_peer[owner]);
            m_out = m - owner * p.c_peer_rows;
          }
          const long long c_off =
              p.cblk_col != 0 ? (static_cast<long long>(m >> 5) * p.cblk_hi + static_cast<long long>(m & 31) * p.cblk_lo +
                                 static_cast<long long>(n0 >> 5) * p.cblk_col)
                              : m_out * p.ldc + n0;
          if (p.out_fp32) {
            float* cp = reinterpret_cast<float*>(c_base) + b * p.strideC + c_off;
            if (n0 + 32 <= n_limit && (reinterpret_cast<uintptr_t>(cp) & 31) == 0) {
#pragma unroll
              for (int j = 0; j < 32; j += 8)
                st_global_256(cp + j,
                              make_uint4(__float_as_uint(f[j]), __float_as_uint(f[j + 1]), __float_as_uint(f[j + 2]),
                                         __float_as_uint(f[j + 3])),
                              make_uint4(__float_as_uint(f[j + 4]), __float_as_uint(f[j + 5]),
                                         __float_as_uint(f[j + 6]), __float_as_uint(f[j + 7])));
            } else if (vec_ok && n0 + 32 <= n_limit) {
#pragma unroll
              for (int j = 0; j < 32; j += 4)
                *reinterpret_cast<float4*>(cp + j) = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (n0 + j < n_limit) cp[j] = f[j];
            }
          } else if (c_tma) {
            // this chunk is one half of the warp's 64-column box: four 16-byte units of staging row `lane`
#pragma unroll
            for (int j8 = 0; j8 < 4; ++j8) {
              uint4 u;
              u.x = pack_bf16x2(f[j8 * 8], f[j8 * 8 + 1]);
              u.y = pack_bf16x2(f[j8 * 8 + 2], f[j8 * 8 + 3]);
              u.z = pack_bf16x2(f[j8 * 8 + 4], f[j8 * 8 + 5]);
              u.w = pack_bf16x2(f[j8 * 8 + 6], f[j8 * 8 + 7]);
              *reinterpret_cast<uint4*>(stage_w + swz128_offset(lane, (c & 1) * 4 + j8)) = u;
            }
          } else {
            __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(c_base) + b * p.strideC + c_off;
            if (n0 + 32 <= n_limit && (reinterpret_cast<uintptr_t>(cp) & 31) == 0) {
              st_bf16x16(cp, f);
              st_bf16x16(cp + 16, f + 16);
            } else if (vec_ok && n0 + 32 <= n_limit) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 u;
                u.x = pack_bf16x2(f[j], f[j + 1]);
                u.y = pack_bf16x2(f[j + 2], f[j + 3]);
                u.z = pack_bf16x2(f[j + 4], f[j + 5]);
                u.w = pack_bf16x2(f[j + 6], f[j + 7]);
                *reinterpret_cast<uint4*>(cp + j) = u;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (n0 + j < n_limit) cp[j] = __float2bfloat16(f[j]);
            }
          }
        }
      };
      uint32_t va[32], vb[32];
      const int c_begin = grp * kChunksPerGroup;
      const int c_end = min(nchunks, c_begin + kChunksPerGroup);
      if constexpr (BN == 192) {
        if (p.act == 5) {
          // this warp's three chunks are one column triple: gate | value | second value of 32 output columns
          if (c_begin + 3 <= c_end) {
            const uint32_t t0 = tmem_addr(tmem_base, q, acc * BN + c_begin * 32);
            tmem_ld32(t0, va);
            tmem_ld_wait();
            tmem_ld32(t0 + 32, vb);
            float f[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] = siluf_fast(__uint_as_float(va[j]) * alpha);
            tmem_ld_wait();
            tmem_ld32(t0 + 64, va);
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] *= __uint_as_float(vb[j]) * alpha;
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] *= __uint_as_float(va[j]) * alpha;
            const int o0 = (n_base + c_begin * 32) / 3;
            if (c_tma) {
              if (lane == 0) tma_store_wait_read<0>();   // the previous box of this warp has left the staging rows
              __syncwarp();
              if (row_ok) {
#pragma unroll
                for (int j8 = 0; j8 < 4; ++j8) {
                  uint4 u;
                  u.x = pack_bf16x2(f[j8 * 8], f[j8 * 8 + 1]);
                  u.y = pack_bf16x2(f[j8 * 8 + 2], f[j8 * 8 + 3]);
                  u.z = pack_bf16x2(f[j8 * 8 + 4], f[j8 * 8 + 5]);
                  u.w = pack_bf16x2(f[j8 * 8 + 6], f[j8 * 8 + 7]);
                  *reinterpret_cast<uint4*>(stage_w + swz64_offset(lane, j8)) = u;
                }
              }
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                tma_store_3d(tmC, stage_w, o0, mb * kBM + q * 32, b);
                tma_store_commit();
              }
            } else if (row_ok) {
              __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(p.C) + b * p.strideC +
                                  static_cast<long long>(m) * p.ldc + o0;
              if ((reinterpret_cast<uintptr_t>(cp) & 31) == 0) {
                st_bf16x16(cp, f);
                st_bf16x16(cp + 16, f + 16);
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) cp[j] = __float2bfloat16(f[j]);
              }
            }
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tempty_bar[acc]);
          if (++acc == 2) {
            acc = 0;
            acc_phase ^= 1u;
          }
          continue;
        }
      }
      if constexpr (BN == 256) {
        if (p.act == 6) {
          // two-way SwiGLU: every 64 accumulator columns are gate | value of 32 output columns
#pragma unroll 1
          for (int c = c_begin; c + 2 <= c_end; c += 2) {
            const uint32_t t0 = tmem_addr(tmem_base, q, acc * BN + c * 32);
            tmem_ld32(t0, va);
            tmem_ld32(t0 + 32, vb);
            tmem_ld_wait();
            float f[32];
#pragma unroll
            for (int j = 0; j < 32; ++j)
              f[j] = siluf_fast(__uint_as_float(va[j]) * alpha) * (__uint_as_float(vb[j]) * alpha);
            const int o0 = (n_base + c * 32) / 2;
            if (c_tma) {
              if (lane == 0) tma_store_wait_read<0>();   // the previous box of this warp has left the staging rows
              __syncwarp();
              if (row_ok) {
#pragma unroll
                for (int j8 = 0; j8 < 4; ++j8) {
                  uint4 u;
                  u.x = pack_bf16x2(f[j8 * 8], f[j8 * 8 + 1]);
                  u.y = pack_bf16x2(f[j8 * 8 + 2], f[j8 * 8 + 3]);
                  u.z = pack_bf16x2(f[j8 * 8 + 4], f[j8 * 8 + 5]);
                  u.w = pack_bf16x2(f[j8 * 8 + 6], f[j8 * 8 + 7]);
                  *reinterpret_cast<uint4*>(stage_w + swz64_offset(lane, j8)) = u;
                }
              }
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                tma_store_3d(tmC, stage_w, o0, mb * kBM + q * 32, b);
                tma_store_commit();
              }
            } else if (row_ok) {
              __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(p.C) + b * p.strideC +
                                  static_cast<long long>(m) * p.ldc + o0;
              if ((reinterpret_cast<uintptr_t>(cp) & 31) == 0) {
                st_bf16x16(cp, f);
                st_bf16x16(cp + 16, f + 16);
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) cp[j] = __float2bfloat16(f[j]);
              }
            }
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tempty_bar[acc]);
          if (++acc == 2) {
            acc = 0;
            acc_phase ^= 1u;
          }
          continue;
        }
      }
      if (c_begin < c_end) tmem_ld32(tmem_addr(tmem_base, q, acc * BN + c_begin * 32), va);
#pragma unroll 1
      for (int c = c_begin; c < c_end; c += 2) {
        tmem_ld_wait();
        if (c + 1 < c_end) tmem_ld32(tmem_addr(tmem_base, q, acc * BN + (c + 1) * 32), vb);
        if (c_tma) {
          if (lane == 0) tma_store_wait_read<0>();   // the previous box of this warp has left the staging rows
          __syncwarp();
        }
        process(va, c);
        if (c + 1 < c_end) {
          tmem_ld_wait();
          if (c + 2 < c_end) tmem_ld32(tmem_addr(tmem_base, q, acc * BN + (c + 2) * 32), va);
          process(vb, c + 1);
        }
        if (c_tma) {
          // columns past N (an odd last chunk) and rows past M hold stale bytes: the copy clips them
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_3d(tmC, stage_w, n_base + c * 32, mb * kBM + q * 32, b);
            tma_store_commit();
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&tempty_bar[acc]);
        if (res_tma) mbar_arrive(&rempty_bar[lt & 1]);
      }
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
    if (c_tma && lane == 0) tma_store_wait_all<0>();   // the staging rows are read and the boxes written
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

template <int BN, bool MN_MAJOR>
static int launch_gemm(const void* A, const void* B, const GemmParams& p0, long long lda, long long ldb,
                       long long strideA, long long strideB, cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  GemmParams p = p0;
  p.npeers = 0;
  p.tiles_m = (p.M + kBM - 1) / kBM;
  p.tiles_n = (p.N + BN - 1) / BN;
  p.num_tiles = p.tiles_m * p.tiles_n * p.batch;
  CUtensorMap tmA, tmB;
  int rc;
  if (!MN_MAJOR) {
    // operands as rows of 128 bytes: 64 bf16 or (fp8) 128 e4m3 elements per k-block
    const uint64_t es = p.fp8 ? 1 : 2;
    const CUtensorMapDataType dt = p.fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    const uint32_t bk = p.fp8 ? 2 * kBK : kBK;
    uint64_t dA[3] = {(uint64_t)p.K, (uint64_t)p.M, (uint64_t)p.batch};
    uint64_t sA[2] = {(uint64_t)lda * es, (uint64_t)strideA * es};
    uint32_t bA[3] = {bk, kBM, 1};
    rc = make_tmap(&tmA, A, dt, 3, dA, sA, bA, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    uint64_t dB[3] = {(uint64_t)p.K, (uint64_t)p.N, (uint64_t)p.batch};
    uint64_t sB[2] = {(uint64_t)ldb * es, (uint64_t)strideB * es};
    uint32_t bB[3] = {bk, (uint32_t)BN, 1};
    rc = make_tmap(&tmB, B, dt, 3, dB, sB, bB, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  } else {
    uint64_t dA[3] = {(uint64_t)p.M, (uint64_t)p.K, (uint64_t)p.batch};
    uint64_t sA[2] = {(uint64_t)lda * 2, (uint64_t)strideA * 2};
    uint32_t bA[3] = {64, kBK, 1};
    rc = make_tmap(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dA, sA, bA, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    uint64_t dB[3] = {(uint64_t)p.N, (uint64_t)p.K, (uint64_t)p.batch};
    uint64_t sB[2] = {(uint64_t)ldb * 2, (uint64_t)strideB * 2};
    uint32_t bB[3] = {64, kBK, 1};
    rc = make_tmap(&tmB, B, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dB, sB, bB, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  auto kern = gemm_bf16_kernel<BN, MN_MAJOR, false>;
  rc = set_smem(kern, Cfg::kSmemBytes);
  if (rc) return rc;
  int grid = p.num_tiles < sm_count() ? p.num_tiles : sm_count();
  PeerMaps none, aux;
  none.m[0] = tmB;
  aux.m[0] = tmB;
  p.res_tma = 0;
  if (Cfg::kResTma && p.residual != nullptr && (p.ldr & 7) == 0 && (p.batch == 1 || (p.strideR & 7) == 0) &&
      (reinterpret_cast<uintptr_t>(p.residual) & 15) == 0) {
    // residual [batch][M][N] as a tensor map: 64-column x 128-row boxes in the 128-byte swizzle
    const long long sr = p.batch == 1 ? (long long)p.M * p.ldr : p.strideR;
    uint64_t dR[3] = {(uint64_t)p.N, (uint64_t)p.M, (uint64_t)p.batch};
    uint64_t sR[2] = {(uint64_t)p.ldr * 2, (uint64_t)sr * 2};
    uint32_t bR[3] = {64, kBM, 1};
    rc = make_tmap(&aux.m[0], p.residual, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dR, sR, bR,
                   CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    p.res_tma = 1;
  }
  p.c_tma = 0;
  {
    static const bool c_tma_on = [] {
      const char* e = getenv("UBM_GEMM_TMA_STORE");
      return e == nullptr || e[0] != '0';
    }();
    const bool swiglu = p.act == 5 || p.act == 6;
    const long long n_out = p.act == 5 ? p.N / 3 : p.act == 6 ? p.N / 2 : p.N;
    if (c_tma_on && !p.out_fp32 && p.cblk_col == 0 && p.c_peer_rows == 0 && (p.ldc & 7) == 0 &&
        (p.batch == 1 || (p.strideC & 7) == 0) && (reinterpret_cast<uintptr_t>(p.C) & 15) == 0 &&
        (swiglu || BN != 192)) {
      const long long sc = p.batch == 1 ? (long long)p.M * p.ldc : p.strideC;
      uint64_t dC[3] = {(uint64_t)n_out, (uint64_t)p.M, (uint64_t)p.batch};
      uint64_t sC[2] = {(uint64_t)p.ldc * 2, (uint64_t)sc * 2};
      uint32_t bC[3] = {swiglu ? 32u : 64u, 32, 1};
      rc = make_tmap(&aux.m[1], p.C, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dC, sC, bC,
                     swiglu ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B);
      if (rc) return rc;
      p.c_tma = 1;
    }
  }
  // launched so that its set-up may overlap the tail of the previous kernel in the stream (see the kernel)
  static const bool pdl = [] {
    const char* e = getenv("UBM_PDL");
    return e == nullptr || e[0] != '0';
  }();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  const cudaError_t le = cudaLaunchKernelEx(&cfg, kern, tmA, tmB, none, aux, p);
  if (le != cudaSuccess) {
    fprintf(stderr, "[ubm] gemm_bf16_kernel: launch failed: %s\n", cudaGetErrorString(le));
    return UBM_ERR_LAUNCH;
  }
  UBM_CHECK_LAUNCH("gemm_bf16_kernel");
  return UBM_OK;
}

}  // namespace ubm

// C ABI ---------------------------------------------------------------------------------
// A, B bf16. ld* and stride* in elements. mn_major: 0 = K contiguous, 1 = M/N contiguous.
// bias: fp32 [N] or null. residual: bf16 with leading dimension ldr / batch stride strideR, or null.
// status: device pointer to a ubm::KernelStatus (16 bytes) or null.
// cblk_*: blocked output addressing (see GemmParams); all zero for the plain [M][N] layout.  The blocked form
// needs N to be a multiple of 32.  gate: optional bf16 [gate_rows][ld_gate] multiplied in before the residual
// (C = act(alpha A.B^T + bias) * gate[m % gate_rows] + residual).  act_col0: the activation applies to columns
// >= act_col0 only (several projections with different activations in one GEMM).
extern "C" int ubm_gemm_bf16_ex(const void* A, const void* B, void* C, const void* bias, const void* residual, int M,
                                int N, int K, int batch, long long lda, long long ldb, long long ldc, long long ldr,
                                long long strideA, long long strideB, long long strideC, long long strideR,
                                int mn_major, int out_fp32, int act, float alpha, long long cblk_hi,
                                long long cblk_lo, long long cblk_col, const void* gate, long long ld_gate,
                                int gate_rows, int act_col0, void* status, void* stream) {
  using namespace ubm;
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return UBM_ERR_ARGUMENT;
  if (cblk_col != 0 && ((N & 31) || residual != nullptr)) return UBM_ERR_ARGUMENT;
  if (act_col0 < 0 || (act_col0 & 31)) return UBM_ERR_ARGUMENT;
  if ((lda & 7) || (ldb & 7) || (batch > 1 && ((strideA & 7) || (strideB & 7)))) {
    fprintf(stderr, "[ubm] gemm: leading dimensions / batch strides must be multiples of 8 elements\n");
    return UBM_ERR_ARGUMENT;
  }
  GemmParams p;
  p.M = M;
  p.N = N;
  p.K = K;
  p.batch = batch;
  p.C = C;
  p.ldc = ldc;
  p.strideC = strideC;
  p.bias = static_cast<const float*>(bias);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.ldr = ldr;
  p.strideR = strideR;
  p.alpha = alpha;
  p.out_fp32 = out_fp32;
  p.act = act;
  p.fp8 = 0;
  p.alpha_dev = nullptr;
  p.act_col0 = act_col0;
  p.cblk_hi = cblk_hi;
  p.cblk_lo = cblk_lo;
  p.cblk_col = cblk_col;
  p.gate = static_cast<const __nv_bfloat16*>(gate);
  p.ld_gate = ld_gate;
  p.gate_rows = gate_rows > 0 ? gate_rows : 1;
  p.c_peer_rows = 0;
  p.status = static_cast<KernelStatus*>(status);
  if (batch == 1) {
    if (strideA == 0) strideA = mn_major ? (long long)K * lda : (long long)M * lda;
    if (strideB == 0) strideB = mn_major ? (long long)K * ldb : (long long)N * ldb;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // Tile width by wave count: 256-wide tiles run the tensor core fastest, but when the 256-wide tiling fills
  // the last wave poorly (e.g. 180 tiles on 148 SMs = 2 waves) 128-wide tiles (3 waves of half the work) finish
  // earlier.  Cost model: waves x tile work, with a 15 % penalty on the narrow tile's main loop.
  bool wide = N > 128;
  if (wide && batch == 1) {
    const long long sms = sm_count();
    const long long tm = (M + kBM - 1) / kBM;
    const long long w256 = (tm * ((N + 255) / 256) + sms - 1) / sms;
    const long long w128 = (tm * ((N + 127) / 128) + sms - 1) / sms;
    if (static_cast<double>(w128) * 0.5 * 1.15 < static_cast<double>(w256)) wide = false;
  }
  if (act == 5) {
    if (mn_major || out_fp32 || bias != nullptr || residual != nullptr || gate != nullptr || cblk_col != 0 ||
        act_col0 != 0 || (N % 96) != 0) {
      fprintf(stderr, "[ubm] gemm: the three-way SwiGLU epilogue takes a K-major bf16 product of 96-column groups "
                      "with no bias, gate or residual\n");
      return UBM_ERR_ARGUMENT;
    }
    return launch_gemm<192, false>(A, B, p, lda, ldb, strideA, strideB, st);
  }
  if (act == 6) {
    if (mn_major || out_fp32 || bias != nullptr || residual != nullptr || gate != nullptr || cblk_col != 0 ||
        act_col0 != 0 || (N % 64) != 0) {
      fprintf(stderr, "[ubm] gemm: the two-way SwiGLU epilogue takes a K-major bf16 product of 64-column groups "
                      "with no bias, gate or residual\n");
      return UBM_ERR_ARGUMENT;
    }
    return launch_gemm<256, false>(A, B, p, lda, ldb, strideA, strideB, st);
  }
  if (mn_major) {
    return wide ? launch_gemm<256, true>(A, B, p, lda, ldb, strideA, strideB, st)
                : launch_gemm<128, true>(A, B, p, lda, ldb, strideA, strideB, st);
  }
  return wide ? launch_gemm<256, false>(A, B, p, lda, ldb, strideA, strideB, st)
              : launch_gemm<128, false>(A, B, p, lda, ldb, strideA, strideB, st);
}

extern "C" int ubm_gemm_bf16(const void* A, const void* B, void* C, const void* bias, const void* residual, int M,
                             int N, int K, int batch, long long lda, long long ldb, long long ldc, long long ldr,
                             long long strideA, long long strideB, long long strideC, long long strideR, int mn_major,
                             int out_fp32, int act, float alpha, void* status, void* stream) {
  return ubm_gemm_bf16_ex(A, B, C, bias, residual, M, N, K, batch, lda, ldb, ldc, ldr, strideA, strideB, strideC,
                          strideR, mn_major, out_fp32, act, alpha, 0, 0, 0, nullptr, 0, 0, 0, status, stream);
}

// C[m][n] = act(alpha * *alpha_dev * sum_k A[m][k] B[n][k] + bias[n]) (+ residual) with A [M][K] and B [N][K] in
// e4m3 (one byte per element, K contiguous; lda / ldb in elements, multiples of 16) and C bf16: tcgen05.mma
// kind::f8f6f4 with fp32 accumulation.  alpha carries the host-known dequantisation factor (the weights'),
// alpha_dev (a device float or null) the one a kernel earlier in the stream wrote for the activations.
extern "C" int ubm_gemm_fp8(const void* A, const void* B, void* C, const void* bias, const void* residual, int M, int N,
                            int K, long long lda, long long ldb, long long ldc, long long ldr, int act, float alpha,
                            const void* alpha_dev, void* status, void* stream) {
  using namespace ubm;
  if (M <= 0 || N <= 0 || K <= 0 || act < 0 || act > 4) return UBM_ERR_ARGUMENT;
  if ((lda & 15) || (ldb & 15) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) {
    fprintf(stderr, "[ubm] gemm_fp8: operands must be 16-byte aligned with leading dimensions in multiples of 16\n");
    return UBM_ERR_ARGUMENT;
  }
  GemmParams p = {};
  p.M = M;
  p.N = N;
  p.K = K;
  p.batch = 1;
  p.C = C;
  p.ldc = ldc;
  p.bias = static_cast<const float*>(bias);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.ldr = ldr;
  p.alpha = alpha;
  p.act = act;
  p.fp8 = 1;
  p.alpha_dev = static_cast<const float*>(alpha_dev);
  p.gate_rows = 1;
  p.status = static_cast<KernelStatus*>(status);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long strideA = static_cast<long long>(M) * lda, strideB = static_cast<long long>(N) * ldb;
  return N > 128 ? launch_gemm<256, false>(A, B, p, lda, ldb, strideA, strideB, st)
                 : launch_gemm<128, false>(A, B, p, lda, ldb, strideA, strideB, st);
}

// GEMM whose epilogue scatters output rows to their owners: the transfer half of a reduce-scatter fused into the
// compute.  C_ptrs[q] = address, in GPU q's memory (mapped here), of the slot this GPU writes: bf16 (or fp32)
// [rows_per_rank][N] with leading dimension ldc.  Output row m goes to C_ptrs[m / rows_per_rank].  K-major only,
// batch 1.  The owners add their slots afterwards (ubm_sum_slots) behind a barrier that orders the stores.
extern "C" int ubm_gemm_bf16_scatter_rows(const void* A, const void* B, void* const* C_ptrs, int npeers,
                                          int rows_per_rank, int M, int N, int K, long long lda, long long ldb,
                                          long long ldc, int out_fp32, float alpha, void* status, void* stream) {
  using namespace ubm;
  if (npeers < 1 || npeers > 8 || M <= 0 || N <= 0 || K <= 0 || rows_per_rank <= 0) return UBM_ERR_ARGUMENT;
  if (static_cast<long long>(rows_per_rank) * npeers < M) return UBM_ERR_ARGUMENT;
  if ((lda & 7) || (ldb & 7)) return UBM_ERR_ARGUMENT;
  GemmParams p = {};
  p.M = M;
  p.N = N;
  p.K = K;
  p.batch = 1;
  p.C = C_ptrs[0];
  p.ldc = ldc;
  p.alpha = alpha;
  p.out_fp32 = out_fp32;
  p.gate_rows = 1;
  p.status = static_cast<KernelStatus*>(status);
  for (int q = 0; q < 8; ++q) p.c_peer[q] = C_ptrs[q < npeers ? q : 0];
  p.c_peer_rows = rows_per_rank;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long strideA = static_cast<long long>(M) * lda, strideB = static_cast<long long>(N) * ldb;
  return N > 128 ? launch_gemm<256, false>(A, B, p, lda, ldb, strideA, strideB, st)
                 : launch_gemm<128, false>(A, B, p, lda, ldb, strideA, strideB, st);
}

// All-gather fused into the GEMM: C[b][m][col0_q + n] = sum_k A[b][m][k] * B_q[b][n][k] where B_q is the
// row shard that GPU q holds (a pointer into its memory, mapped into this process).  Each CTA reads the
// B tiles it needs straight from the owner with ordinary TMA loads (no cluster multicast), so the
// transfer over NVLink overlaps the tensor-core work of the other pipeline stages; nothing is gathered
// into a local buffer first.  The caller orders this launch after the owners have finished writing
// their shards (a stream-ordered barrier over the symmetric buffers).
//   B_ptrs[q]   bf16 [batch][rows_q][K] with leading dimension ldb and batch stride strideB (elements)
//   rows[q]     number of rows of shard q;  the output has sum(rows) columns, shard q starting at the
//               running sum.  K contiguous (K-major) only.
// Gather-once mode (gathered != null, copy_ctas > 0): the last copy_ctas CTAs of the grid copy every remote
// shard block into `gathered` ([batch][sum(rows)][K], leading dimension ldg, batch stride strideG) exactly once
// and publish per-block flags in ready_flags ([batch * n_tiles] uint32, zero at first use; epoch grows by one per
// call); compute CTAs start with the local shard and wait (bounded) for the flag of a remote block before
// loading it from the local copy.  Without it every CTA re-reads remote tiles over NVLink for each m-tile.
extern "C" int ubm_gemm_bf16_allgather_b(const void* A, const void* const* B_ptrs, const int* rows, int npeers,
                                         void* C, int M, int K, int batch, long long lda, long long ldb,
                                         long long ldc, long long strideA, long long strideB, long long strideC,
                                         int out_fp32, float alpha, int my_rank, int copy_ctas, void* gathered,
                                         long long ldg, long long strideG, void* ready_flags, unsigned int epoch,
                                         void* status, void* stream) {
  using namespace ubm;
  constexpr int BN = 256;
  using Cfg = GemmCfg<BN>;
  if (npeers < 1 || npeers > kMaxPeers || M <= 0 || K <= 0 || batch <= 0) return UBM_ERR_ARGUMENT;
  if ((lda & 7) || (ldb & 7) || (strideA & 7) || (strideB & 7)) return UBM_ERR_ARGUMENT;
  GemmParams p = {};
  p.M = M;
  p.K = K;
  p.batch = batch;
  p.C = C;
  p.ldc = ldc;
  p.strideC = strideC;
  p.alpha = alpha;
  p.out_fp32 = out_fp32;
  p.status = static_cast<KernelStatus*>(status);
  p.npeers = npeers;
  p.my_rank = my_rank;
  p.copy_ctas = (gathered != nullptr && ready_flags != nullptr && npeers > 1) ? copy_ctas : 0;
  p.ready = static_cast<uint32_t*>(ready_flags);
  p.epoch = epoch;
  if (my_rank < 0 || my_rank >= npeers) return UBM_ERR_ARGUMENT;
  if (p.copy_ctas > 0 && ((ldg & 7) || (strideG & 7))) return UBM_ERR_ARGUMENT;
  PeerMaps maps, gmaps;
  int col = 0, tile = 0;
  CUtensorMap tmA;
  {
    uint64_t dA[3] = {(uint64_t)K, (uint64_t)M, (uint64_t)batch};
    uint64_t sA[2] = {(uint64_t)lda * 2, (uint64_t)strideA * 2};
    uint32_t bA[3] = {kBK, kBM, 1};
    int rc = make_tmap(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dA, sA, bA, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  for (int q = 0; q < npeers; ++q) {
    p.peer_tile0[q] = tile;
    p.peer_col0[q] = col;
    p.peer_cols[q] = rows[q];
    if (rows[q] > 0) {
      uint64_t dB[3] = {(uint64_t)K, (uint64_t)rows[q], (uint64_t)batch};
      uint64_t sB[2] = {(uint64_t)ldb * 2, (uint64_t)strideB * 2};
      uint32_t bB[3] = {kBK, (uint32_t)BN, 1};
      int rc = make_tmap(&maps.m[q], B_ptrs[q], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dB, sB, bB,
                         CU_TENSOR_MAP_SWIZZLE_128B);
      if (rc) return rc;
      gmaps.m[q] = maps.m[q];
      if (p.copy_ctas > 0) {
        // shard q inside the local gathered buffer [batch][sum(rows)][K]: clipped to the shard's own rows
        uint64_t sG[2] = {(uint64_t)ldg * 2, (uint64_t)strideG * 2};
        const __nv_bfloat16* gbase = static_cast<const __nv_bfloat16*>(gathered) + static_cast<long long>(col) * ldg;
        rc = make_tmap(&gmaps.m[q], gbase, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dB, sG, bB,
                       CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
      }
    } else {
      maps.m[q] = tmA;
      gmaps.m[q] = tmA;
    }
    col += rows[q];
    tile += (rows[q] + BN - 1) / BN;
  }
  for (int q = npeers; q < kMaxPeers; ++q) {
    maps.m[q] = tmA;
    gmaps.m[q] = tmA;
  }
  p.peer_tile0[npeers] = tile;
  p.N = col;
  p.tiles_m = (M + kBM - 1) / kBM;
  p.tiles_n = tile;
  p.num_tiles = p.tiles_m * p.tiles_n * batch;
  if (p.num_tiles == 0) return UBM_OK;
  auto kern = gemm_bf16_kernel<BN, false, true>;
  int rc = set_smem(kern, Cfg::kSmemBytes);
  if (rc) return rc;
  int grid = p.num_tiles < sm_count() ? p.num_tiles : sm_count();
  if (p.copy_ctas > 0) {
    // compute CTAs + copy CTAs must all be resident at once (one CTA per SM): never more than the SM count
    if (p.copy_ctas >= sm_count()) return UBM_ERR_ARGUMENT;
    const int compute = sm_count() - p.copy_ctas;
    grid = (p.num_tiles < compute ? p.num_tiles : compute) + p.copy_ctas;
  }
  kern<<<grid, kGemmThreads, Cfg::kSmemBytes, static_cast<cudaStream_t>(stream)>>>(tmA, tmA, maps, gmaps, p);
  UBM_CHECK_LAUNCH("gemm_bf16_kernel<peer>");
  return UBM_OK;
}
