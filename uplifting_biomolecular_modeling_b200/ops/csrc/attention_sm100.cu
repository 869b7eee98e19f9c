// Attention with a pair bias shared over rows, on tcgen05 / TMEM / TMA (head dimension 32).
//
//   O[r, q, h, :] = softmax_k( Q[r,q,h,:] . K[r,k,h,:] + bias[h, q, k] ) V[r,k,h,:]   (* gate)
//
// r is the "row" of a triangle attention (all rows share the bias of a head), a diffusion
// sample of the token transformer, or a batch entry of single attention with pair bias.  Q is
// pre-scaled by log2(e)/sqrt(d) and the bias by log2(e), so the softmax runs in base 2.
//
// CTA = one query tile (128) x one head x TWO rows.  The two rows share every bias tile that TMA
// brings in (the reason the reference's kernels process several rows per CTA:
// common/opt_core/opt_core/kernels/triattn/triattn_native/DESIGN.md:41-59) and their softmax
// warpgroups ping-pong on the one tensor core.  Per 128-key tile and row:
//   MMA warp  : S = Q K^T            (TMEM, 128 columns per row)
//   softmax WG: S -> registers, S freed at once (the next QK^T overlaps the exponentials),
//               + bias, running max / sum, P (bf16) -> shared memory
//   MMA warp  : O += P V             (TMEM, 32 columns per row; V is an MN-major B operand)
// O is rescaled in TMEM only when a running maximum moved.  No TMA multicast is used: the bias
// tile is loaded once per CTA and reused by both rows from shared memory.
//
// Persistent CTAs walk (head, row group, query tile) with the query tile fastest: CTAs that run together
// work on the same rows, so each K / V tile comes from HBM once and is re-read from L2 by the other query
// tiles; the bias planes of a head (a few MB) stay in L2 throughout.
#include "host_util.h"
#include "sm100.cuh"

namespace ubm {


constexpr int kATile = 128;  // queries per CTA
constexpr float kNegBig = -1.0e30f;

// D = head dimension (32 or 64), TK = keys per step (128 for D = 32, 64 for D = 64 so that two rows,
// two stages and the P tiles still fit in shared memory).
// R2 = rows per CTA (softmax warpgroups sharing each bias tile): 2, or 4 with TK = 64 - four warps per
// scheduler hide the TMEM-load -> bias -> max -> exp latency chain that two cannot.
// TP = the probability tile stays in tensor memory (the P.V product takes its A operand from TMEM) and the pair
// bias is added by the tensor cores: S = bias . I + Q K^T, where the bias tile [128 q][TK keys] is the K-major A
// operand as TMA delivered it and I is a TK x TK identity in shared memory.  The contraction runs over the TK keys
// of the step, so a 64-key step costs four MMAs (an identity on the query side would cost eight).  The softmax
// threads then neither read the bias from shared memory nor write P to it.
// POLY = how many of every four exponentials run as a polynomial on the FMA pipe instead of the special-function
// unit (0 or 1).  Measured and dropped at 1536 tokens, four heads of 32: two of four with packed two-wide fp32
// instructions (5.31 ms against 4.84), exponentials on fp16 or bf16 pairs with two per special-function
// instruction (5.9 ms), three rows per CTA (5.13 ms).
template <int D, int TK, int R2, bool TP = false>
struct AttnCfg {
  static constexpr int kQBytes = kATile * D * 2;
  static constexpr int kKVBytes = TK * D * 2;
  static constexpr int kBiasBytes = kATile * TK * 2;
  static constexpr int kStageBytes = 2 * R2 * kKVBytes + kBiasBytes;  // {K, V} per row, then the bias tile
  static constexpr int kPBytes = kATile * TK * 2;
  // As many stages as fit: the loop is bound by the latency of the tile loads unless they are issued
  // several tiles ahead (with two stages every tile waited a full TMA round trip).
  static constexpr int kPSmem = TP ? 0 : R2 * kPBytes;
  // tensor memory map (512 columns): S[r] at r*TK, O[r] at 256 + r*D, then (TP) P[r] and the identity
  static constexpr int kTmemP = 256 + R2 * D;             // P[r] at kTmemP + r * TK / 2 (two bf16 per column)
  // identity B operand of the bias MMA: TK/64 k-blocks of [TK rows][64 k] bf16, K-major, 128-byte swizzle
  static constexpr int kIdentBlock = TK * 128;
  static constexpr int kIdentBytes = TP ? TK * TK * 2 : 0;
  static constexpr int kStages = (224 * 1024 - R2 * kQBytes - kPSmem - kIdentBytes) / kStageBytes;
  static_assert(kStages >= 2 && kStages <= 8, "stage count");
  static constexpr int kSmemBytes = R2 * kQBytes + kStages * kStageBytes + kPSmem + kIdentBytes + 512 + 1024;
  static_assert(!TP || (R2 * TK <= 256 && kTmemP + R2 * TK / 2 <= 512), "tensor memory budget");
  static constexpr int kThreads = 128 + R2 * 128;
  // setmaxnreg moves registers inside the pool the CTA was launched with (threads x compiled registers):
  //   R2 = 2: 384 x 168 = 64512 = 128 x 56 + 256 x 224;   R2 = 3: 512 x 128 = 65536 = 128 x 56 + 384 x 152;
  //   R2 = 4: 640 x 96 = 61440 >= 128 x 56 + 512 x 104.
  // An increase that does not fit that pool would wait forever, so these pairs are checked below.
  static constexpr int kLaunchRegs = (R2 == 2) ? 168 : (R2 == 3) ? 128 : 96;
  static constexpr int kSoftmaxRegs = (R2 == 2) ? 224 : (R2 == 3) ? 152 : 104;
  static_assert(128 * 56 + R2 * 128 * kSoftmaxRegs <= kThreads * kLaunchRegs, "setmaxnreg budget");
  static constexpr uint64_t kSwz = (D == 32) ? kSwizzle64 : kSwizzle128;  // operand rows are D * 2 bytes
  static constexpr uint32_t kSbo = (D == 32) ? 512 : 1024;               // 8 rows of D * 2 bytes
  static constexpr uint32_t kVStep = 16 * D * 2;                         // 16 keys of V
};

struct AttnParams {
  int rows, Nq, Nk, H;
  const __nv_bfloat16* gate;  // [rows][Nq] rows of H*D gate values (row stride ld_gate) or null
  long long ld_gate;
  __nv_bfloat16* out;         // [rows][Nq][H*32], or transposed [Nq][rows][H*32]
  int transpose_out;
  int has_bias;
  // key mask: additive bf16 rows [rows][ld_mask] (0 = keep, -1e30 = masked) and one flag byte per (row, key step)
  // that is non-zero when the step holds a masked key; steps with a zero flag run the mask-free loop
  const __nv_bfloat16* kmask;
  const uint8_t* kflags;
  long long ld_mask;
  KernelStatus* status;
  int n_qt, n_kt, n_rp, num_items;
  // Pair-bias all-gather inside this launch: the bias planes [H][Nq][ldb] that the tiles read are a buffer of THIS
  // GPU whose rows [g_row0[q], g_row0[q] + g_rows[q]) belong to GPU q.  Before the tile loop every CTA copies its
  // share of the peers' rows from their buffers (g_src[q], same layout, plain peer loads) into the local one, then
  // adds one to g_done; the TMA producers start on bias tiles once g_done has reached g_target (all CTAs of this
  // launch).  The wait is bounded.  g_n == 0: no gather.
  int g_n, g_me;
  const __nv_bfloat16* g_src[8];
  int g_row0[8], g_rows[8];
  __nv_bfloat16* g_dst;
  long long g_ld, g_plane;          // elements per bias row / per head plane
  uint32_t* g_done;
  uint32_t g_target;
  // peer mode: the bias rows (queries) are row shards owned by several GPUs; query tiles are enumerated
  // shard by shard and each tile's bias comes through that GPU's tensor map
  int npeers;
  int peer_tile0[9];
  int peer_row0[8];
  int peer_rows[8];
};

constexpr int kAMaxPeers = 8;
struct BiasPeerMaps {
  CUtensorMap m[kAMaxPeers];
};

// query tile -> (shard, first global query, query limit, row offset inside the shard)
__device__ __forceinline__ void decode_qtile(const AttnParams& p, int qt, int& q, int& q_base, int& q_limit,
                                             int& local_row) {
  if (p.npeers == 0) {
    q = 0;
    q_base = qt * kATile;
    q_limit = p.Nq;
    local_row = q_base;
    return;
  }
  q = 0;
#pragma unroll
  for (int i = 1; i < kAMaxPeers; ++i)
    if (i < p.npeers && qt >= p.peer_tile0[i]) q = i;
  local_row = (qt - p.peer_tile0[q]) * kATile;
  q_base = p.peer_row0[q] + local_row;
  q_limit = p.peer_row0[q] + p.peer_rows[q];
}

// Optional timeline (build with -DUBM_ATTN_TIMELINE): CTA 0 stamps clock64 at fixed points of its first
// tiles into a global buffer [3 roles][kTlTiles][8 events]; used to see which role waits for which.
#ifdef UBM_ATTN_TIMELINE
constexpr int kTlTiles = 48;
__device__ long long g_attn_timeline[3 * kTlTiles * 8];
#define ATT_STAMP(role, tile, ev)                                                        \
  do {                                                                                   \
    if (blockIdx.x == 0 && (tile) < kTlTiles) g_attn_timeline[((role) * kTlTiles + (tile)) * 8 + (ev)] = clock64(); \
  } while (0)
#else
#define ATT_STAMP(role, tile, ev) do { } while (0)
#endif

template <int D, int TK, int R2, bool PEER, bool TP, int POLY>
__global__ void __launch_bounds__(128 + R2 * 128, 1)
attention_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ BiasPeerMaps peers, AttnParams p) {
  using Cfg = AttnCfg<D, TK, R2, TP>;
  constexpr int kAD = D;
  constexpr int kAQBytes = Cfg::kQBytes;
  constexpr int kAKVBytes = Cfg::kKVBytes;
  constexpr int kAStageBytes = Cfg::kStageBytes;
  constexpr int kAPBytes = Cfg::kPBytes;
  constexpr int kAStages = Cfg::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                              // R2 x Q tile
  uint8_t* sSt = sQ + R2 * kAQBytes;               // stages
  uint8_t* sP = sSt + kAStages * kAStageBytes;     // R2 x P tile
  uint8_t* sIdent = sP + (TP ? 0 : R2 * kAPBytes);                               // no P tiles in smem when TP
  uint64_t* bars = reinterpret_cast<uint64_t*>(sIdent + Cfg::kIdentBytes);
  uint64_t* q_full = bars;             // [1]
  uint64_t* q_empty = q_full + 1;      // [1] commit
  uint64_t* kv_full = q_empty + 1;     // [stages]
  uint64_t* kv_empty = kv_full + kAStages;   // [stages] commit + 8 warps
  uint64_t* s_full = kv_empty + kAStages;    // [R2] commit
  uint64_t* s_empty = s_full + R2;     // [R2] 4 warps
  uint64_t* p_full = s_empty + R2;     // [R2] 4 warps
  uint64_t* pv_done = p_full + R2;     // [R2] commit
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + R2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const WaitScope ws{abort_flag, p.status};

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(q_full, 1);
    mbar_init(q_empty, 2);   // the two S issuers
    for (int s = 0; s < kAStages; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], TP ? 3 : 3 + 4 * R2);   // two S issuers, the P.V issuer (+ the softmax warps)
    }
    for (int r = 0; r < R2; ++r) {
      mbar_init(&s_full[r], 1);
      mbar_init(&s_empty[r], 4);
      mbar_init(&p_full[r], 4);
      mbar_init(&pv_done[r], 1);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base;         // S[r] at r * TK
  const uint32_t tO = tmem_base + 256;   // O[r] at r * D
  const uint32_t tP = tmem_base + Cfg::kTmemP;
  const int T = p.n_kt;
  if (p.g_n > 1) {
    // ---- gather prologue: 16-byte units of the peers' bias rows, round-robin over the CTAs of the launch
    for (int q = 0; q < p.g_n; ++q) {
      if (q == p.g_me || p.g_rows[q] <= 0) continue;
      const long long units_per_plane = static_cast<long long>(p.g_rows[q]) * p.g_ld / 8;     // 8 bf16 = 16 bytes
      const long long off0 = static_cast<long long>(p.g_row0[q]) * p.g_ld;
      for (int h = 0; h < p.H; ++h) {
        const uint4* src = reinterpret_cast<const uint4*>(p.g_src[q] + h * p.g_plane + off0);
        uint4* dst = reinterpret_cast<uint4*>(p.g_dst + h * p.g_plane + off0);
        for (long long u = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; u < units_per_plane;
             u += static_cast<long long>(gridDim.x) * blockDim.x) {
          uint4 v;
          asm volatile("ld.global.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                       : "l"(src + u));
          dst[u] = v;
        }
      }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();                   // cumulative: what the CTA's threads wrote is visible before the count
      fence_proxy_async_all();           // the copies are generic-proxy writes that TMA loads will read
      atomicAdd(p.g_done, 1u);
    }
  }
  if (TP) {
    // identity B operand in shared memory: TK/64 k-blocks of [TK rows][64 k], row n has a one at k = n
    constexpr int kChunks = TK / 8;   // 16-byte chunks per row
    for (int i = threadIdx.x; i < TK * kChunks; i += blockDim.x) {
      const int row = i / kChunks, cc = i % kChunks;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if ((row >> 3) == cc) {
        const uint32_t one = (row & 1) ? 0x3F800000u : 0x00003F80u;
        const int w = (row & 7) >> 1;
        v.x = w == 0 ? one : 0u;
        v.y = w == 1 ? one : 0u;
        v.z = w == 2 ? one : 0u;
        v.w = w == 3 ? one : 0u;
      }
      *reinterpret_cast<uint4*>(sIdent + (cc >> 3) * Cfg::kIdentBlock + swz128_offset(row, cc & 7)) = v;
    }
    fence_proxy_async_smem();
    __syncthreads();
  }

  // Register split: warps 0-3 (producer, MMA issuer, two idle warps) give registers up, the softmax
  // warpgroups take them (budget checked in AttnCfg and again on the host before launch).
  if (warp < 4) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t item_cnt = 0, gk = 0;
      if (p.g_n > 1) {
        // every CTA of the launch has finished its share of the gather (bounded wait, as for a peer flag)
        wait_flag_ge(p.g_done, p.g_target, ws, 63, 0);
        fence_proxy_async_all();
      }
      for (int item = blockIdx.x; item < p.num_items; item += gridDim.x, ++item_cnt) {
        const int qt = item % p.n_qt;
        const int tmp = item / p.n_qt;
        const int rp = tmp % p.n_rp;
        const int h = tmp / p.n_rp;
        const int r0 = rp * R2;
        mbar_wait(q_empty, (item_cnt & 1u) ^ 1u, ws, 51);
        if (*abort_flag) break;
        int pq, q_base, q_limit, lrow;
        decode_qtile(p, qt, pq, q_base, q_limit, lrow);
        mbar_expect_tx(q_full, R2 * kAQBytes);
#pragma unroll
        for (int rr = 0; rr < R2; ++rr) tma_load_3d(sQ + rr * kAQBytes, &tmQ, q_full, h * kAD, q_base, r0 + rr);
        for (int j = 0; j < T; ++j, ++gk) {
          const int s = gk % kAStages;
          mbar_wait(&kv_empty[s], ((gk / kAStages) & 1u) ^ 1u, ws, 52, s);
          if (*abort_flag) break;
          uint8_t* st = sSt + s * kAStageBytes;
          mbar_expect_tx(&kv_full[s], p.has_bias ? kAStageBytes : 2 * R2 * kAKVBytes);
#pragma unroll
          for (int rr = 0; rr < R2; ++rr) {
            tma_load_3d(st + (2 * rr) * kAKVBytes, &tmK, &kv_full[s], h * kAD, j * TK, r0 + rr);
            tma_load_3d(st + (2 * rr + 1) * kAKVBytes, &tmV, &kv_full[s], h * kAD, j * TK, r0 + rr);
          }
          if (p.has_bias) {
#pragma unroll
            for (int hb = 0; hb < TK / 64; ++hb) {
              // peer mode: the bias rows of this query tile live on GPU pq (plain TMA load, no multicast)
              const CUtensorMap* bm = PEER ? &peers.m[pq] : &tmB;
              tma_load_3d(st + 2 * R2 * kAKVBytes + hb * 16384, bm, &kv_full[s], j * TK + hb * 64, lrow, h);
            }
          }
        }
        if (*abort_flag) break;
      }
    }
  } else if (warp >= 1 && warp <= 3) {
    // ------------------------------------------------------------------ MMA issuers
    // Issuing one tcgen05.mma costs its thread on the order of a hundred cycles and a key tile needs
    // 18 per row, so the work is spread over three single-thread issuers:
    //   warps 1, 2 : S = I.bias^T + Q K^T for the rows r with r % 2 == warp - 1
    //   warp 3     : O += P V for all rows
    // The whole warp runs the loop with warp-uniform operands; one elected lane issues the tcgen05 instructions.
    const bool leader = elect_one();
    if (warp <= 2) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16(128, TK, 0, 0);   // also the bias MMA: A = bias tile, B = identity
      const int r_first = warp - 1;
      uint32_t item_cnt = 0, gk = 0;
      auto issue_qk = [&](int r, uint32_t g) {
        const uint32_t st = smem_u32(sSt + (g % kAStages) * kAStageBytes);
        const uint32_t qa = smem_u32(sQ + r * kAQBytes);
        const uint32_t ka = st + r * 2 * kAKVBytes;
        const bool with_bias = TP && p.has_bias;
        const uint64_t bd0 = umma_smem_desc(st + 2 * R2 * kAKVBytes, 16, 1024, kSwizzle128);
        const uint64_t ad0 = umma_smem_desc(qa, 16, Cfg::kSbo, Cfg::kSwz);
        const uint64_t kd0 = umma_smem_desc(ka, 16, Cfg::kSbo, Cfg::kSwz);
        const uint64_t id0 = umma_smem_desc(smem_u32(sIdent), 16, 1024, kSwizzle128);
        if (leader) {
          if (with_bias) {
            // S = bias . I: the 128 x TK bias tile sits in shared memory as TK/64 boxes of [128 q][64 k] (K-major A),
            // the identity as TK/64 blocks of [TK n][64 k] (K-major B); 16 keys per MMA
#pragma unroll
            for (int k = 0; k < TK / 16; ++k)
              umma_ss(tS + r * TK, bd0 + static_cast<uint64_t>((k >> 2) * (16384 >> 4) + (k & 3) * 2),
                      id0 + static_cast<uint64_t>((k >> 2) * (Cfg::kIdentBlock >> 4) + (k & 3) * 2), idesc_qk,
                      k != 0 ? 1u : 0u);
          }
#pragma unroll
          for (int k = 0; k < kAD / 16; ++k)
            umma_ss(tS + r * TK, ad0 + static_cast<uint64_t>(k * 2), kd0 + static_cast<uint64_t>(k * 2), idesc_qk,
                    (with_bias || k != 0) ? 1u : 0u);
          umma_commit(&s_full[r]);
        }
        __syncwarp();
      };
      for (int item = blockIdx.x; item < p.num_items; item += gridDim.x, ++item_cnt) {
        mbar_wait(q_full, item_cnt & 1u, ws, 53);
        mbar_wait(&kv_full[gk % kAStages], (gk / kAStages) & 1u, ws, 54, 0);
        tc_fence_after_sync();
        for (int r = r_first; r < R2; r += 2) {
          mbar_wait(&s_empty[r], (gk & 1u) ^ 1u, ws, 55, r);
          tc_fence_after_sync();
          issue_qk(r, gk);
        }
        for (int j = 0; j < T; ++j) {
          const uint32_t g = gk + j;
          if (leader) umma_commit(&kv_empty[g % kAStages]);   // K and bias of tile g: free when the MMAs so far end
          if (j + 1 < T) {
            mbar_wait(&kv_full[(g + 1) % kAStages], ((g + 1) / kAStages) & 1u, ws, 56, 1);
            ATT_STAMP(0, g, 0);
            tc_fence_after_sync();
            for (int r = r_first; r < R2; r += 2) {
              mbar_wait(&s_empty[r], ((g + 1) & 1u) ^ 1u, ws, 57, r);
              tc_fence_after_sync();
              issue_qk(r, g + 1);
              ATT_STAMP(0, g, 1 + r);
            }
          }
        }
        if (leader) umma_commit(q_empty);
        gk += T;
      }
    } else {
      constexpr uint32_t idesc_pv = umma_idesc_bf16(128, kAD, 0, 1);  // B = V is MN-major
      uint32_t gk = 0;
      for (int item = blockIdx.x; item < p.num_items; item += gridDim.x) {
        for (int j = 0; j < T; ++j) {
          const uint32_t g = gk + j;
          mbar_wait(&kv_full[g % kAStages], (g / kAStages) & 1u, ws, 54, 2);
          const uint32_t st = smem_u32(sSt + (g % kAStages) * kAStageBytes);
          for (int r = 0; r < R2; ++r) {
            mbar_wait(&p_full[r], g & 1u, ws, 58, r);
            ATT_STAMP(0, g, 3 + 2 * r);
            tc_fence_after_sync();
            const uint32_t pa = smem_u32(sP + r * kAPBytes);
            const uint64_t vd0 = umma_smem_desc(st + (r * 2 + 1) * kAKVBytes, 16, Cfg::kSbo, Cfg::kSwz);
            const uint64_t pd0 = umma_smem_desc(pa, 16, 1024, kSwizzle128);
            if (leader) {
#pragma unroll
              for (int k = 0; k < TK / 16; ++k) {
                // P: K-major (TMEM, or shared-memory k-blocks of 64 keys); V: MN-major, a step of 16 keys
                const uint64_t bd = vd0 + static_cast<uint64_t>(k * (Cfg::kVStep >> 4));
                if (TP) {
                  umma_ts(tO + r * kAD, tP + r * (TK / 2) + k * 8, bd, idesc_pv, (j | k) != 0 ? 1u : 0u);
                } else {
                  umma_ss(tO + r * kAD, pd0 + static_cast<uint64_t>((k >> 2) * (16384 >> 4) + (k & 3) * 2), bd,
                          idesc_pv, (j | k) != 0 ? 1u : 0u);
                }
              }
              umma_commit(&pv_done[r]);
            }
            __syncwarp();
            ATT_STAMP(0, g, 4 + 2 * r);
          }
          if (leader) umma_commit(&kv_empty[g % kAStages]);   // V of tile g
        }
        gk += T;
      }
    }
  }
  } else {
    if (R2 == 2) {
      asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    } else if (R2 == 3) {
      asm volatile("setmaxnreg.inc.sync.aligned.u32 152;");
    } else {
      asm volatile("setmaxnreg.inc.sync.aligned.u32 104;");
    }
    // ------------------------------------------------------------------ softmax warpgroups
    const int r_in = (warp - 4) >> 2;  // which of the R2 rows
    const int quad = warp & 3;
    const int qrow = quad * 32 + lane;
    uint32_t gk = 0;
    for (int item = blockIdx.x; item < p.num_items; item += gridDim.x) {
      const int qt = item % p.n_qt;
      const int tmp = item / p.n_qt;
      const int rp = tmp % p.n_rp;
      const int h = tmp / p.n_rp;
      const int r = rp * R2 + r_in;
      int pq, q_base, q_limit, lrow;
      decode_qtile(p, qt, pq, q_base, q_limit, lrow);
      const int qi = q_base + qrow;
      float m = kNegBig, l = 0.f;
      for (int j = 0; j < T; ++j) {
        const uint32_t g = gk + j;
        // flag of this (row, key step), fetched ahead of the wait for the score tile
        const uint32_t mflag = (p.kflags != nullptr && r < p.rows) ? p.kflags[static_cast<long long>(r) * T + j] : 0u;
        mbar_wait(&s_full[r_in], g & 1u, ws, 59, r_in);
        if (quad == 0 && lane == 0) ATT_STAMP(1 + r_in, g, 0);
        tc_fence_after_sync();
        float t[TK];
        {
          uint32_t* tu = reinterpret_cast<uint32_t*>(t);
          const uint32_t ta = tmem_addr(tS, quad, r_in * TK);
#pragma unroll
          for (int c = 0; c < TK / 32; ++c) tmem_ld32(ta + c * 32, *reinterpret_cast<uint32_t(*)[32]>(tu + c * 32));
          tmem_ld_wait();
        }
        if (quad == 0 && lane == 0) ATT_STAMP(1 + r_in, g, 1);
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_empty[r_in]);

        if (!TP) mbar_wait(&kv_full[g % kAStages], (g / kAStages) & 1u, ws, 60, r_in);
        if (quad == 0 && lane == 0) ATT_STAMP(1 + r_in, g, 2);
        if (!TP && p.has_bias) {
          const uint8_t* bs = sSt + (g % kAStages) * kAStageBytes + 2 * R2 * kAKVBytes;
#pragma unroll
          for (int c16 = 0; c16 < TK / 8; ++c16) {
            const uint4 u = *reinterpret_cast<const uint4*>(bs + (c16 >> 3) * 16384 + swz128_offset(qrow, c16 & 7));
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              t[c16 * 8 + 2 * e] += bf16_lo(w[e]);
              t[c16 * 8 + 2 * e + 1] += bf16_hi(w[e]);
            }
          }
        }
        if (!TP) {
          __syncwarp();
          if (lane == 0) mbar_arrive(&kv_empty[g % kAStages]);
        }
        if (mflag != 0u) {
          // masked keys in this step: every thread adds the same TK mask values (one broadcast 16-byte load per 8 keys)
          const uint4* mp = reinterpret_cast<const uint4*>(p.kmask + static_cast<long long>(r) * p.ld_mask + j * TK);
#pragma unroll
          for (int c16 = 0; c16 < TK / 8; ++c16) {
            const uint4 u = __ldg(mp + c16);
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              t[c16 * 8 + 2 * e] += bf16_lo(w[e]);
              t[c16 * 8 + 2 * e + 1] += bf16_hi(w[e]);
            }
          }
        }
        if (j == T - 1) {
          const int valid = p.Nk - j * TK;
          if (valid < TK) {
#pragma unroll
            for (int k = 0; k < TK; ++k)
              if (k >= valid) t[k] = kNegBig;
          }
        }
        // four independent chains each for the maximum and the sum: a single chain of TK dependent
        // operations would leave the two warps per scheduler waiting on instruction latency
        float mx[4] = {t[0], t[1], t[2], t[3]};
#pragma unroll
        for (int k = 4; k + 8 <= TK + 4; k += 8) {     // four chains, two new values per step (3-input max)
          mx[0] = max3f(mx[0], t[k], t[k + 4 < TK ? k + 4 : k]);
          mx[1] = max3f(mx[1], t[k + 1], t[k + 5 < TK ? k + 5 : k + 1]);
          mx[2] = max3f(mx[2], t[k + 2], t[k + 6 < TK ? k + 6 : k + 2]);
          mx[3] = max3f(mx[3], t[k + 3], t[k + 7 < TK ? k + 7 : k + 3]);
        }
        const float mt = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
        const float m_new = fmaxf(m, mt);
        const float alpha = fast_exp2(m - m_new);
        if (quad == 0 && lane == 0) ATT_STAMP(1 + r_in, g, 3);
        // differences and partial sums as packed two-wide fp32 operations: one issue slot per two values
        float2 ps01 = make_float2(0.f, 0.f), ps23 = make_float2(0.f, 0.f);
        const float2 neg_m = make_float2(-m_new, -m_new);
        uint32_t pk[TK / 2];
#pragma unroll
        for (int k = 0; k < TK; k += 4) {
          const float2 d01 = __fadd2_rn(make_float2(t[k], t[k + 1]), neg_m);
          const float2 d23 = __fadd2_rn(make_float2(t[k + 2], t[k + 3]), neg_m);
          float2 e01, e23;
          e01.x = fast_exp2(d01.x);
          e01.y = fast_exp2(d01.y);
          e23.x = fast_exp2(d23.x);
          e23.y = (POLY == 1) ? poly_exp2(d23.y) : fast_exp2(d23.y);
          ps01 = __fadd2_rn(ps01, e01);
          ps23 = __fadd2_rn(ps23, e23);
          pk[k >> 1] = pack_bf16x2(e01.x, e01.y);
          pk[(k >> 1) + 1] = pack_bf16x2(e23.x, e23.y);
        }
        const float psum = (ps01.x + ps01.y) + (ps23.x + ps23.y);
        l = l * alpha + psum;
        m = m_new;
        if (quad == 0 && lane == 0) ATT_STAMP(1 + r_in, g, 4);

        // previous P.V of this row must be complete: P buffer free, O stable
        mbar_wait(&pv_done[r_in], (g & 1u) ^ 1u, ws, 61, r_in);
        if (quad == 0 && lane == 0) ATT_STAMP(1 + r_in, g, 5);
        tc_fence_after_sync();
        if (j > 0 && __any_sync(0xffffffffu, alpha < 1.0f)) {
          const uint32_t oa = tmem_addr(tO, quad, r_in * kAD);
#pragma unroll
          for (int dc = 0; dc < kAD / 32; ++dc) {
            uint32_t ov[32];
            tmem_ld32(oa + dc * 32, ov);
            tmem_ld_wait();
#pragma unroll
            for (int d = 0; d < 32; ++d) ov[d] = __float_as_uint(__uint_as_float(ov[d]) * alpha);
            tmem_st32(oa + dc * 32, ov);
          }
          tmem_st_wait();
        }
        if (TP) {
          // P stays in tensor memory: this thread's lane, TK/2 columns of packed bf16 pairs
          const uint32_t pa_t = tmem_addr(tP, quad, r_in * (TK / 2));
#pragma unroll
          for (int c = 0; c < TK / 64; ++c) tmem_st32(pa_t + c * 32, *reinterpret_cast<uint32_t(*)[32]>(pk + c * 32));
          tmem_st_wait();
        } else {
          uint8_t* ps = sP + r_in * kAPBytes;
#pragma unroll
          for (int c16 = 0; c16 < TK / 8; ++c16) {
            const uint4 u = make_uint4(pk[c16 * 4], pk[c16 * 4 + 1], pk[c16 * 4 + 2], pk[c16 * 4 + 3]);
            *reinterpret_cast<uint4*>(ps + (c16 >> 3) * 16384 + swz128_offset(qrow, c16 & 7)) = u;
          }
          fence_proxy_async_smem();
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[r_in]);
        if (quad == 0 && lane == 0) ATT_STAMP(1 + r_in, g, 6);
      }
      // ---- epilogue of this (row, head, query tile)
      mbar_wait(&pv_done[r_in], (gk + T - 1) & 1u, ws, 62, r_in);
      tc_fence_after_sync();
      {
        const bool ok = r < p.rows && qi < q_limit;
        const float inv = 1.0f / l;
        const long long in_row = static_cast<long long>(r) * p.Nq + qi;
        const long long out_row = p.transpose_out ? (static_cast<long long>(qi) * p.rows + r) : in_row;
#pragma unroll
        for (int dc = 0; dc < kAD / 32; ++dc) {
          uint32_t ov[32];
          tmem_ld32(tmem_addr(tO, quad, r_in * kAD + dc * 32), ov);
          tmem_ld_wait();
          if (ok) {
            float f[32];
#pragma unroll
            for (int d = 0; d < 32; ++d) f[d] = __uint_as_float(ov[d]) * inv;
            if (p.gate != nullptr) {
              const __nv_bfloat16* gp = p.gate + in_row * p.ld_gate + h * kAD + dc * 32;
#pragma unroll
              for (int c = 0; c < 2; ++c) {
                float e[16];
                ld_bf16x16(gp + c * 16, e);
#pragma unroll
                for (int d = 0; d < 16; ++d) f[c * 16 + d] *= e[d];
              }
            }
            __nv_bfloat16* op = p.out + out_row * (p.H * kAD) + h * kAD + dc * 32;
            st_bf16x16(op, f);
            st_bf16x16(op + 16, f + 16);
          }
        }
      }
      tc_fence_before_sync();
      gk += T;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

struct AttnGather {
  int n = 0, me = 0;
  const void* const* src = nullptr;   // n device pointers: every GPU's bias buffer [H][Nq][ldb]
  const int* rows = nullptr;          // rows owned by each GPU (sum = Nq)
  void* done = nullptr;               // uint32 counter in this GPU's memory
  unsigned int epoch = 0;             // launches so far with this counter, this one included
};

struct AttnMask {
  const void* kmask = nullptr;   // bf16 [rows][ld_mask], additive (0 / -1e30)
  const void* kflags = nullptr;  // uint8 [rows][ceil(Nk / TK)]
  long long ld_mask = 0;
};

template <int D, int TK, int R2, bool TP, int POLY, bool PEER>
static int launch_attention(const void* q, const void* k, const void* v, const void* bias, const void* gate, void* out,
                            int rows, int Nq, int Nk, int H, long long ldb, long long ld_in, long long ld_gate,
                            int transpose_out, AttnMask mask,
                            void* status, void* stream, int npeers = 0, const void* const* bias_ptrs = nullptr,
                            const int* peer_rows = nullptr, long long peer_head_stride = 0, AttnGather gather = {}) {
  using Cfg = AttnCfg<D, TK, R2, TP>;
  const uint64_t hd = (uint64_t)H * D;
  const uint64_t ldi = ld_in > 0 ? (uint64_t)ld_in : hd;  // row stride of q / k / v in elements
  if (ldi < hd || (ldi & 7)) return UBM_ERR_ARGUMENT;
  if (PEER != (npeers > 0)) return UBM_ERR_ARGUMENT;
  const CUtensorMapSwizzle swz = (D == 32) ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B;
  CUtensorMap tmQ, tmK, tmV, tmB;
  {
    uint64_t d[3] = {hd, (uint64_t)Nq, (uint64_t)rows};
    uint64_t s[2] = {ldi * 2, ldi * 2 * (uint64_t)Nq};
    uint32_t b[3] = {(uint32_t)D, kATile, 1};
    int rc = make_tmap(&tmQ, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, d, s, b, swz);
    if (rc) return rc;
  }
  {
    uint64_t d[3] = {hd, (uint64_t)Nk, (uint64_t)rows};
    uint64_t s[2] = {ldi * 2, ldi * 2 * (uint64_t)Nk};
    uint32_t b[3] = {(uint32_t)D, (uint32_t)TK, 1};
    int rc = make_tmap(&tmK, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, d, s, b, swz);
    if (rc) return rc;
    rc = make_tmap(&tmV, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, d, s, b, swz);
    if (rc) return rc;
  }
  if (bias != nullptr) {
    uint64_t d[3] = {(uint64_t)Nk, (uint64_t)Nq, (uint64_t)H};
    uint64_t s[2] = {(uint64_t)ldb * 2, (uint64_t)ldb * 2 * (uint64_t)Nq};
    uint32_t b[3] = {64, kATile, 1};
    int rc = make_tmap(&tmB, bias, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, d, s, b, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  } else {
    tmB = tmQ;
  }
  AttnParams p = {};
  p.rows = rows;
  p.Nq = Nq;
  p.Nk = Nk;
  p.H = H;
  p.gate = static_cast<const __nv_bfloat16*>(gate);
  p.ld_gate = ld_gate > 0 ? ld_gate : static_cast<long long>(H) * D;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.transpose_out = transpose_out;
  p.has_bias = bias != nullptr ? 1 : 0;
  p.status = static_cast<KernelStatus*>(status);
  p.n_qt = (Nq + kATile - 1) / kATile;
  p.n_kt = (Nk + TK - 1) / TK;
  p.n_rp = (rows + R2 - 1) / R2;
  if (mask.kmask != nullptr) {
    // the mask rows are read in whole key steps with 16-byte loads
    if (mask.kflags == nullptr || mask.ld_mask < (long long)p.n_kt * TK || (mask.ld_mask & 7) ||
        (reinterpret_cast<uintptr_t>(mask.kmask) & 15))
      return UBM_ERR_ARGUMENT;
    p.kmask = static_cast<const __nv_bfloat16*>(mask.kmask);
    p.kflags = static_cast<const uint8_t*>(mask.kflags);
    p.ld_mask = mask.ld_mask;
  }
  BiasPeerMaps maps;
  for (int i = 0; i < kAMaxPeers; ++i) maps.m[i] = tmQ;
  if (PEER) {
    if (npeers > kAMaxPeers || bias_ptrs == nullptr || peer_rows == nullptr) return UBM_ERR_ARGUMENT;
    p.npeers = npeers;
    p.has_bias = 1;
    int row = 0, tile = 0;
    for (int i = 0; i < npeers; ++i) {
      p.peer_tile0[i] = tile;
      p.peer_row0[i] = row;
      p.peer_rows[i] = peer_rows[i];
      if (peer_rows[i] > 0) {
        uint64_t d[3] = {(uint64_t)Nk, (uint64_t)peer_rows[i], (uint64_t)H};
        uint64_t s[2] = {(uint64_t)ldb * 2, (uint64_t)peer_head_stride * 2};
        uint32_t b[3] = {64, kATile, 1};
        int rc = make_tmap(&maps.m[i], bias_ptrs[i], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, d, s, b,
                           CU_TENSOR_MAP_SWIZZLE_128B);
        if (rc) return rc;
      }
      row += peer_rows[i];
      tile += (peer_rows[i] + kATile - 1) / kATile;
    }
    p.peer_tile0[npeers] = tile;
    if (row != Nq) return UBM_ERR_ARGUMENT;
    p.n_qt = tile;
  }
  p.num_items = p.n_qt * p.n_rp * H;
  const int grid = p.num_items < sm_count() ? p.num_items : sm_count();
  if (gather.n > 1) {
    if (PEER || gather.n > 8 || bias == nullptr || gather.src == nullptr || gather.rows == nullptr ||
        gather.done == nullptr || (ldb & 7))
      return UBM_ERR_ARGUMENT;
    p.g_n = gather.n;
    p.g_me = gather.me;
    int row = 0;
    for (int i = 0; i < gather.n; ++i) {
      p.g_src[i] = static_cast<const __nv_bfloat16*>(gather.src[i]);
      p.g_row0[i] = row;
      p.g_rows[i] = gather.rows[i];
      row += gather.rows[i];
    }
    if (row != Nq) return UBM_ERR_ARGUMENT;
    p.g_dst = static_cast<__nv_bfloat16*>(const_cast<void*>(bias));
    p.g_ld = ldb;
    p.g_plane = static_cast<long long>(ldb) * Nq;
    p.g_done = static_cast<uint32_t*>(gather.done);
    p.g_target = gather.epoch * static_cast<uint32_t>(grid);   // the grid size is the same for every launch on a counter
  }
  auto kern = attention_kernel<D, TK, R2, PEER, TP, POLY>;
  {
    // the in-kernel register re-split must fit the pool this build was compiled with, or it would never return
    cudaFuncAttributes fa;
    cudaError_t e = cudaFuncGetAttributes(&fa, kern);
    if (e != cudaSuccess || 128 * 56 + R2 * 128 * Cfg::kSoftmaxRegs > Cfg::kThreads * fa.numRegs) {
      fprintf(stderr, "[ubm] attention: register budget check failed (numRegs=%d)\n", e == cudaSuccess ? fa.numRegs : -1);
      return UBM_ERR_LAUNCH;
    }
  }
  int rc = set_smem(kern, Cfg::kSmemBytes);
  if (rc) return rc;
  kern<<<grid, Cfg::kThreads, Cfg::kSmemBytes, static_cast<cudaStream_t>(stream)>>>(tmQ, tmK, tmV, tmB, maps, p);
  UBM_CHECK_LAUNCH("attention_kernel");
  return UBM_OK;
}

}  // namespace ubm

static int g_attn_variant = 0;
#ifdef UBM_ATTN_TIMELINE
extern "C" int ubm_attention_read_timeline(long long* host_out) {
  return (int)cudaMemcpyFromSymbol(host_out, ubm::g_attn_timeline, sizeof(long long) * 3 * ubm::kTlTiles * 8);
}
#endif

// Low nibble: tile shape for head dimension 32 - 0 = by row count (four rows per CTA with 64-key steps from four
// rows on, else two rows with 64-key steps), 5 = two rows per CTA with 128-key steps, 1 = two rows, 128-key steps,
// P and bias through shared memory.  Bits 4-5: 0 = one exponential in four runs as a polynomial on the FMA pipe
// (four-row form and head dimension 64), 1 = none does.
extern "C" int ubm_attention_set_variant(int v) {
  g_attn_variant = v & 0xff;
  return 0;
}

#define UBM_ATTN_ARGS q, k, v, bias, gate, out, rows, Nq, Nk, H, ldb, ld_in, ld_gate, transpose_out, m, status, stream

// q, k, v, gate, out: bf16 [rows][N*][H*D] (innermost contiguous).  bias: bf16 [H][Nq][ldb] (ldb multiple
// of 8) or null.  q must carry the factor log2(e)/sqrt(d) and bias the factor log2(e).  transpose_out
// writes out[q][r] instead of out[r][q].  ld_in: row stride of q / k / v in elements (0 = H*D), so the
// three may be column slices of one projection output; ld_gate: row stride of the gate (0 = H*D; a multiple of
// 16 elements), so the gate may be a column slice of the same output.  kmask / kflags / ld_mask: optional key
// mask per row (see AttnParams; flags are per 64-key step); null = no mask.  D = 32 (ubm_attention_d32) or 64
// (ubm_attention_d64).
extern "C" int ubm_attention_d32(const void* q, const void* k, const void* v, const void* bias, const void* gate,
                                 void* out, const void* kmask, const void* kflags, int rows, int Nq, int Nk, int H,
                                 long long ldb, long long ld_in, long long ld_gate, long long ld_mask,
                                 int transpose_out, void* status, void* stream) {
  if (rows <= 0 || Nq <= 0 || Nk <= 0 || H <= 0 || (ld_gate & 15)) return ubm::UBM_ERR_ARGUMENT;
  if (bias != nullptr && (ldb < Nk || (ldb & 7))) return ubm::UBM_ERR_ARGUMENT;
  ubm::AttnMask m;
  m.kmask = kmask;
  m.kflags = kflags;
  m.ld_mask = ld_mask;
  const int shape = g_attn_variant & 15, poly = (g_attn_variant >> 4) & 3;
  if (shape == 1) {
    if (kmask != nullptr) return ubm::UBM_ERR_ARGUMENT;   // flags are per 64-key step
    return ubm::launch_attention<32, 128, 2, false, 0, false>(UBM_ATTN_ARGS);
  }
  if (shape == 5) {
    if (kmask != nullptr) return ubm::UBM_ERR_ARGUMENT;
    return ubm::launch_attention<32, 128, 2, true, 0, false>(UBM_ATTN_ARGS);
  }
  if (rows >= 4) {
    // four rows per CTA: one bias tile per four rows keeps the L2 traffic per row low; one exponential in four as a
    // polynomial (4.84 against 5.00 ms at 1536 tokens; two in four cost more issue slots than they free: 5.31 ms)
    if (poly == 1) return ubm::launch_attention<32, 64, 4, true, 0, false>(UBM_ATTN_ARGS);
    return ubm::launch_attention<32, 64, 4, true, 1, false>(UBM_ATTN_ARGS);
  }
  return ubm::launch_attention<32, 64, 2, true, 0, false>(UBM_ATTN_ARGS);
}

extern "C" int ubm_attention_d64(const void* q, const void* k, const void* v, const void* bias, const void* gate,
                                 void* out, const void* kmask, const void* kflags, int rows, int Nq, int Nk, int H,
                                 long long ldb, long long ld_in, long long ld_gate, long long ld_mask,
                                 int transpose_out, void* status, void* stream) {
  if (rows <= 0 || Nq <= 0 || Nk <= 0 || H <= 0 || (ld_gate & 15)) return ubm::UBM_ERR_ARGUMENT;
  if (bias != nullptr && (ldb < Nk || (ldb & 7))) return ubm::UBM_ERR_ARGUMENT;
  ubm::AttnMask m;
  m.kmask = kmask;
  m.kflags = kflags;
  m.ld_mask = ld_mask;
  const int poly = (g_attn_variant >> 4) & 3;
  if (poly == 1) return ubm::launch_attention<64, 64, 2, true, 0, false>(UBM_ATTN_ARGS);
  return ubm::launch_attention<64, 64, 2, true, 1, false>(UBM_ATTN_ARGS);
}

// Pair-bias all-gather inside the attention launch (head dimension 32, four-row form).  Every GPU holds a bias
// buffer bf16 [H][Nq][ldb] in memory its peers have mapped and has written the rows it owns (rows[i] rows for GPU
// i, in rank order); bias_bufs[i] is GPU i's buffer, bias_bufs[me] this GPU's.  The kernel first copies the
// peers' rows into this GPU's buffer - every CTA a share, plain peer loads, no multicast - and then runs the
// attention on the completed planes with the same tile code as ubm_attention_d32; `done` is a uint32 counter on
// this GPU (zero before the first launch) and `epoch` the number of launches that have used it, this one
// included.  All launches that share a counter must have the same rows, Nq and H (same grid).  The caller
// orders the ranks around the launch: a barrier after the owners wrote their rows, one after the launch.
extern "C" int ubm_attention_d32_gather_bias(const void* q, const void* k, const void* v,
                                             const void* const* bias_bufs, const int* rows_per_gpu, int ngpus,
                                             int me, void* done, unsigned int epoch, const void* gate, void* out,
                                             const void* kmask, const void* kflags, int rows, int Nq, int Nk, int H,
                                             long long ldb, long long ld_in, long long ld_gate, long long ld_mask,
                                             int transpose_out, void* status, void* stream) {
  if (rows < 4 || Nq <= 0 || Nk <= 0 || H <= 0 || ngpus < 1 || ngpus > 8 || me < 0 || me >= ngpus ||
      bias_bufs == nullptr || (ld_gate & 15) || ldb < Nk || (ldb & 7))
    return ubm::UBM_ERR_ARGUMENT;
  ubm::AttnMask m;
  m.kmask = kmask;
  m.kflags = kflags;
  m.ld_mask = ld_mask;
  ubm::AttnGather g;
  g.n = ngpus;
  g.me = me;
  g.src = bias_bufs;
  g.rows = rows_per_gpu;
  g.done = done;
  g.epoch = epoch;
  return ubm::launch_attention<32, 64, 4, true, 1, false>(q, k, v, bias_bufs[me], gate, out, rows, Nq, Nk, H, ldb,
                                                          ld_in, ld_gate, transpose_out, m, status, stream, 0, nullptr,
                                                          nullptr, 0, g);
}

// Pair-bias all-gather fused into the attention kernel (head dimension 32): the bias planes are row
// shards, shard i = bf16 [H][peer_rows[i]][ldb] in GPU i's memory with head stride peer_head_stride
// (elements).  Query tiles are enumerated shard by shard and every CTA reads the bias tiles it needs
// from the owner with ordinary TMA loads (no cluster multicast) while its tensor-core work proceeds; the
// gathered [H][N][N] bias never exists in local memory.  sum(peer_rows) must equal Nq.
extern "C" int ubm_attention_d32_peer_bias(const void* q, const void* k, const void* v, const void* const* bias_ptrs,
                                           const int* peer_rows, int npeers, long long peer_head_stride,
                                           const void* gate, void* out, int rows, int Nq, int Nk, int H, long long ldb,
                                           long long ld_in, void* status, void* stream) {
  if (rows <= 0 || Nq <= 0 || Nk <= 0 || H <= 0 || npeers <= 0) return ubm::UBM_ERR_ARGUMENT;
  if (ldb < Nk || (ldb & 7) || (peer_head_stride & 7)) return ubm::UBM_ERR_ARGUMENT;
  return ubm::launch_attention<32, 128, 2, false, 0, true>(q, k, v, nullptr, gate, out, rows, Nq, Nk, H, ldb, ld_in, 0, 0,
                                                           ubm::AttnMask{}, status, stream, npeers, bias_ptrs, peer_rows,
                                                           peer_head_stride);
}
