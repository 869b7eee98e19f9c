// Causal self-attention for head dimension 128 on tcgen05 (the attention layers of the StripedHyena-2 models):
// softmax(scale * Q K^T + causal mask) V, bf16 in / out, fp32 accumulation.
//
// One work item = one (batch, head) and TWO adjacent 128-query tiles, which share every key / value tile that TMA
// brings in (a ring of 64-key stages).  Per tile and key step: S = Q K^T (128 x 64, eight k16 MMAs, accumulator
// in tensor memory), one warpgroup turns S into probabilities in registers (online softmax in the exp2 domain, the
// causal comparison only on the steps that cross the diagonal), writes them back to tensor memory as packed bf16,
// and O += P V runs with P as the tensor-memory A operand (four k16 MMAs of 128 x 128).  Key steps above the
// diagonal of a tile are never issued; the lower tile of a pair simply stops two steps earlier.  Items are
// enumerated longest first.  Queries may be the LAST Nq positions of Nk keys (chunked prefill / continuation).
//
// Tensor memory (512 columns): S[r] at r * 64, P[r] at 128 + r * 32 (two bf16 per column), O[r] at 256 + r * 128.
// Warps: 0 = TMA producer, 1 / 2 = S issuers of tile 0 / 1, 3 = P.V issuer, 4-19 = four softmax warpgroups: two per
// query tile, each taking 32 of the step's 64 key columns (a thread = one query row and 32 logits).  The two halves
// of a tile exchange their row maxima through shared memory once per step (one named barrier of 256 threads) and
// keep separate row sums that are added at the end; with one warpgroup per tile the two softmax warps per scheduler
// left the issue slots half empty (1.0 PFLOP/s at 32768 tokens).
// Every wait is bounded and reports through the status word.
//
// The reference calls a library attention here (evo2/opt/evo2_opt/kit/base.py: flash-attention wrapper of the
// attention blocks); the tcgen05 form has no counterpart there.
#include "host_util.h"
#include "sm100.cuh"

namespace ubm {

constexpr int kCD = 128;        // head dimension
constexpr int kCTile = 128;     // queries per tile
constexpr int kCTK = 64;        // keys per step
constexpr int kCStages = 4;
constexpr int kCQBytes = kCTile * kCD * 2;       // 32 KB: two k-blocks of [128 q][64 d]
constexpr int kCKBytes = kCTK * kCD * 2;         // 16 KB: two k-blocks of [64 keys][64 d]
constexpr int kCStageBytes = 2 * kCKBytes;       // K then V
// row maxima [tile][parity][half][row], then the row sums of an item's end [tile][half][row] (a region of their own:
// a warpgroup that is already in the next item's first step must not overwrite a sum its partner has yet to read)
constexpr int kCXMaxFloats = 2 * 2 * 2 * 128;
constexpr int kCXBytes = (kCXMaxFloats + 2 * 2 * 128) * 4;
constexpr int kCSmemBytes = 2 * kCQBytes + kCStages * kCStageBytes + kCXBytes + 512 + 1024;
constexpr int kCThreads = 640;
constexpr int kCSoftmaxRegs = 104;               // 128 x 56 + 512 x 104 <= 640 x 96
constexpr float kCNegBig = -1.0e30f;

struct CausalParams {
  int B, H, Hkv, Nq, Nk;
  int off;                 // query i sits at key position i + off (off = Nk - Nq >= 0)
  float scale_log2e;       // softmax scale * log2(e)
  __nv_bfloat16* out;      // [B][Nq][ld_out], head h at columns h * 128
  long long ld_out;
  KernelStatus* status;
  int n_qt, n_qp, num_items;
};

__global__ void __launch_bounds__(kCThreads, 1)
causal_attention_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                        const __grid_constant__ CUtensorMap tmV, CausalParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                      // 2 x Q tile
  uint8_t* sSt = sQ + 2 * kCQBytes;        // stages of {K, V}
  float* sX = reinterpret_cast<float*>(sSt + kCStages * kCStageBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sX + kCXBytes / 4);
  uint64_t* q_full = bars;                 // [1]
  uint64_t* q_empty = q_full + 1;          // [1] the two S issuers
  uint64_t* kv_full = q_empty + 1;         // [stages]
  uint64_t* kv_empty = kv_full + kCStages; // [stages] two S issuers + the P.V issuer
  uint64_t* s_full = kv_empty + kCStages;  // [2] commit
  uint64_t* s_empty = s_full + 2;          // [2] 8 warps
  uint64_t* p_full = s_empty + 2;          // [2] 8 warps
  uint64_t* pv_done = p_full + 2;          // [2] commit
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const WaitScope ws{abort_flag, p.status};

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(q_full, 1);
    mbar_init(q_empty, 2);
    for (int s = 0; s < kCStages; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 3);
    }
    for (int r = 0; r < 2; ++r) {
      mbar_init(&s_full[r], 1);
      mbar_init(&s_empty[r], 8);
      mbar_init(&p_full[r], 8);
      mbar_init(&pv_done[r], 1);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base;          // S[r] at r * 64
  const uint32_t tP = tmem_base + 128;    // P[r] at r * 32
  const uint32_t tO = tmem_base + 256;    // O[r] at r * 128
  const int n_kt = (p.Nk + kCTK - 1) / kCTK;
  const int bh = p.B * p.H;

  // item -> (pair of query tiles, batch, head); pairs with the most key steps first
  auto decode = [&](int item, int& qp, int& b, int& h) {
    qp = p.n_qp - 1 - item / bh;
    const int x = item - (item / bh) * bh;
    b = x / p.H;
    h = x - b * p.H;
  };
  // key steps of tile r of pair qp (0 when the tile does not exist)
  auto steps = [&](int qp, int r) -> int {
    const int qt = 2 * qp + r;
    if (qt >= p.n_qt) return 0;
    const int last_key = min(p.Nk, qt * kCTile + kCTile + p.off);   // one past the last visible key
    return min(n_kt, (last_key + kCTK - 1) / kCTK);
  };

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    if (warp == 0) {
      // ------------------------------------------------------------------ TMA producer
      if (lane == 0) {
        uint32_t item_cnt = 0, gk = 0;
        for (int item = blockIdx.x; item < p.num_items; item += gridDim.x, ++item_cnt) {
          int qp, b, h;
          decode(item, qp, b, h);
          const int hk = h / (p.H / p.Hkv);
          const int T = max(steps(qp, 0), steps(qp, 1));
          const int nrow = (2 * qp + 1 < p.n_qt) ? 2 : 1;
          mbar_wait(q_empty, (item_cnt & 1u) ^ 1u, ws, 71);
          if (*abort_flag) break;
          mbar_expect_tx(q_full, nrow * kCQBytes);
          for (int r = 0; r < nrow; ++r)
            for (int kb = 0; kb < 2; ++kb)
              tma_load_3d(sQ + r * kCQBytes + kb * 16384, &tmQ, q_full, h * kCD + kb * 64, (2 * qp + r) * kCTile, b);
          for (int j = 0; j < T; ++j, ++gk) {
            const int s = gk % kCStages;
            mbar_wait(&kv_empty[s], ((gk / kCStages) & 1u) ^ 1u, ws, 72, s);
            if (*abort_flag) break;
            uint8_t* st = sSt + s * kCStageBytes;
            mbar_expect_tx(&kv_full[s], kCStageBytes);
            for (int kb = 0; kb < 2; ++kb) {
              tma_load_3d(st + kb * 8192, &tmK, &kv_full[s], hk * kCD + kb * 64, j * kCTK, b);
              tma_load_3d(st + kCKBytes + kb * 8192, &tmV, &kv_full[s], hk * kCD + kb * 64, j * kCTK, b);
            }
          }
          if (*abort_flag) break;
        }
      }
    } else if (warp <= 2) {
      // ------------------------------------------------------------------ S issuer of tile r = warp - 1
      // (the whole warp runs the loop with warp-uniform operands; one elected lane issues)
      const bool leader = elect_one();
      const int r = warp - 1;
      constexpr uint32_t idesc_qk = umma_idesc_bf16(128, kCTK, 0, 0);
      uint32_t item_cnt = 0, gk = 0, gr = 0;   // gr: steps of this tile so far (parity of its S barriers)
      for (int item = blockIdx.x; item < p.num_items; item += gridDim.x, ++item_cnt) {
        int qp, b, h;
        decode(item, qp, b, h);
        const int Tr = steps(qp, r);
        const int T = max(steps(qp, 0), steps(qp, 1));
        mbar_wait(q_full, item_cnt & 1u, ws, 73);
        for (int j = 0; j < T; ++j) {
          const uint32_t g = gk + j;
          mbar_wait(&kv_full[g % kCStages], (g / kCStages) & 1u, ws, 74, r);
          if (j < Tr) {
            mbar_wait(&s_empty[r], (gr & 1u) ^ 1u, ws, 75, r);
            tc_fence_after_sync();
            const uint32_t qa = smem_u32(sQ + r * kCQBytes);
            const uint32_t ka = smem_u32(sSt + (g % kCStages) * kCStageBytes);
            const uint64_t ad0 = umma_smem_desc(qa, 16, 1024, kSwizzle128);
            const uint64_t kd0 = umma_smem_desc(ka, 16, 1024, kSwizzle128);
            if (leader) {
#pragma unroll
              for (int k = 0; k < kCD / 16; ++k)
                umma_ss(tS + r * kCTK, ad0 + static_cast<uint64_t>((k >> 2) * (16384 >> 4) + (k & 3) * 2),
                        kd0 + static_cast<uint64_t>((k >> 2) * (8192 >> 4) + (k & 3) * 2), idesc_qk, k != 0 ? 1u : 0u);
              umma_commit(&s_full[r]);
            }
            __syncwarp();
            ++gr;
          }
          if (leader) umma_commit(&kv_empty[g % kCStages]);   // K of step g: free when the MMAs issued so far end
          __syncwarp();
        }
        if (leader) umma_commit(q_empty);
        __syncwarp();
        gk += T;
      }
    } else {
      // ------------------------------------------------------------------ P.V issuer (both tiles)
      const bool leader = elect_one();
      constexpr uint32_t idesc_pv = umma_idesc_bf16(128, kCD, 0, 1);   // B = V is MN-major
      uint32_t gk = 0, gr[2] = {0, 0};
      for (int item = blockIdx.x; item < p.num_items; item += gridDim.x) {
        int qp, b, h;
        decode(item, qp, b, h);
        const int T0 = steps(qp, 0), T1 = steps(qp, 1);
        const int T = max(T0, T1);
        for (int j = 0; j < T; ++j) {
          const uint32_t g = gk + j;
          mbar_wait(&kv_full[g % kCStages], (g / kCStages) & 1u, ws, 76, 2);
          const uint32_t va = smem_u32(sSt + (g % kCStages) * kCStageBytes + kCKBytes);
          // V tile: two boxes of [64 keys][64 d] = MN-major B with 64-element runs along d, the second run 8 KB on
          const uint64_t vd0 = umma_smem_desc(va, 8192, 1024, kSwizzle128);
          for (int r = 0; r < 2; ++r) {
            if (j >= (r == 0 ? T0 : T1)) continue;
            mbar_wait(&p_full[r], gr[r] & 1u, ws, 77, r);
            tc_fence_after_sync();
            if (leader) {
#pragma unroll
              for (int k = 0; k < kCTK / 16; ++k)
                umma_ts(tO + r * kCD, tP + r * (kCTK / 2) + k * 8, vd0 + static_cast<uint64_t>(k * (2048 >> 4)),
                        idesc_pv, (j | k) != 0 ? 1u : 0u);
              umma_commit(&pv_done[r]);
            }
            __syncwarp();
            ++gr[r];
          }
          if (leader) umma_commit(&kv_empty[g % kCStages]);   // V of step g
          __syncwarp();
        }
        gk += T;
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 104;");
    // ------------------------------------------------------------------ softmax warpgroups: (tile r, column half)
    const int wg = (warp - 4) >> 2;
    const int r = wg >> 1;
    const int half = wg & 1;
    const int quad = warp & 3;
    const int qrow = quad * 32 + lane;
    const float c = p.scale_log2e;
    constexpr int kHalf = kCTK / 2;              // 32 logits per thread and step
    uint32_t gr = 0;
    for (int item = blockIdx.x; item < p.num_items; item += gridDim.x) {
      int qp, b, h;
      decode(item, qp, b, h);
      const int Tr = steps(qp, r);
      if (Tr == 0) continue;
      const int qb = (2 * qp + r) * kCTile;
      const int qi = qb + qrow;
      const int kmax = qi + p.off;               // last visible key of this query
      float m = kCNegBig, l = 0.f;               // m: maximum over both halves; l: sum over this half only
      for (int j = 0; j < Tr; ++j, ++gr) {
        mbar_wait(&s_full[r], gr & 1u, ws, 78, r);
        tc_fence_after_sync();
        float t[kHalf];
        tmem_ld32(tmem_addr(tS, quad, r * kCTK + half * kHalf), *reinterpret_cast<uint32_t(*)[32]>(t));
        tmem_ld_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_empty[r]);
        // the causal comparison only where the step reaches past the first query of the tile
        if (j * kCTK + kCTK - 1 > qb + p.off) {
          const int k0 = j * kCTK + half * kHalf;
#pragma unroll
          for (int k = 0; k < kHalf; ++k)
            if (k0 + k > kmax) t[k] = kCNegBig;
        }
        float mx[4] = {t[0], t[1], t[2], t[3]};
#pragma unroll
        for (int k = 4; k + 8 <= kHalf + 4; k += 8) {
          mx[0] = max3f(mx[0], t[k], t[k + 4 < kHalf ? k + 4 : k]);
          mx[1] = max3f(mx[1], t[k + 1], t[k + 5 < kHalf ? k + 5 : k + 1]);
          mx[2] = max3f(mx[2], t[k + 2], t[k + 6 < kHalf ? k + 6 : k + 2]);
          mx[3] = max3f(mx[3], t[k + 3], t[k + 7 < kHalf ? k + 7 : k + 3]);
        }
        const float mt = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
        // row maximum of the other half of the columns (buffers alternate by step: a writer two steps ahead would
        // first have to pass the next step's barrier, which the reader reaches only after this read)
        float* xm = sX + ((r * 2 + (gr & 1u)) * 2) * 128;
        xm[half * 128 + qrow] = mt;
        asm volatile("bar.sync %0, 256;" ::"r"(1 + r) : "memory");
        const float m_new = fmaxf(m, fmaxf(mt, xm[(half ^ 1) * 128 + qrow]));
        const float alpha = fast_exp2((m - m_new) * c);
        // exp2(c * (s - m)) with the scale folded into one packed fused multiply-add per two logits
        const float2 c2 = make_float2(c, c);
        const float2 nm2 = make_float2(-m_new * c, -m_new * c);
        float2 ps01 = make_float2(0.f, 0.f), ps23 = make_float2(0.f, 0.f);
        uint32_t pk[kHalf / 2];
#pragma unroll
        for (int k = 0; k < kHalf; k += 4) {
          const float2 d01 = __ffma2_rn(make_float2(t[k], t[k + 1]), c2, nm2);
          const float2 d23 = __ffma2_rn(make_float2(t[k + 2], t[k + 3]), c2, nm2);
          float2 e01, e23;
          e01.x = fast_exp2(d01.x);
          e01.y = fast_exp2(d01.y);
          e23.x = fast_exp2(d23.x);
          e23.y = poly_exp2(d23.y);
          ps01 = __fadd2_rn(ps01, e01);
          ps23 = __fadd2_rn(ps23, e23);
          pk[k >> 1] = pack_bf16x2(e01.x, e01.y);
          pk[(k >> 1) + 1] = pack_bf16x2(e23.x, e23.y);
        }
        l = l * alpha + ((ps01.x + ps01.y) + (ps23.x + ps23.y));
        m = m_new;
        // the previous P.V of this tile must be complete: P buffer free, O stable
        mbar_wait(&pv_done[r], (gr & 1u) ^ 1u, ws, 79, r);
        tc_fence_after_sync();
        if (j > 0 && __any_sync(0xffffffffu, alpha < 1.0f)) {
          // each half rescales its 64 of the 128 output columns
          const uint32_t oa = tmem_addr(tO, quad, r * kCD + half * 64);
#pragma unroll
          for (int dc = 0; dc < 2; ++dc) {
            uint32_t ov[32];
            tmem_ld32(oa + dc * 32, ov);
            tmem_ld_wait();
#pragma unroll
            for (int d = 0; d < 32; ++d) ov[d] = __float_as_uint(__uint_as_float(ov[d]) * alpha);
            tmem_st32(oa + dc * 32, ov);
          }
          tmem_st_wait();
        }
        tmem_st16(tmem_addr(tP, quad, r * (kCTK / 2) + half * (kHalf / 2)), *reinterpret_cast<uint32_t(*)[16]>(pk));
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[r]);
      }
      // ---- epilogue of this tile: O / (l of both halves); this half writes output columns half * 64 .. + 63
      {
        float* xl = sX + kCXMaxFloats + (r * 2) * 128;
        xl[half * 128 + qrow] = l;
        asm volatile("bar.sync %0, 256;" ::"r"(1 + r) : "memory");
        l += xl[(half ^ 1) * 128 + qrow];
      }
      mbar_wait(&pv_done[r], (gr & 1u) ^ 1u, ws, 80, r);
      tc_fence_after_sync();
      {
        const bool ok = qi < p.Nq;
        const float inv = 1.0f / l;
        __nv_bfloat16* op = p.out + (static_cast<long long>(b) * p.Nq + qi) * p.ld_out + h * kCD + half * 64;
#pragma unroll
        for (int dc = 0; dc < 2; ++dc) {
          uint32_t ov[32];
          tmem_ld32(tmem_addr(tO, quad, r * kCD + half * 64 + dc * 32), ov);
          tmem_ld_wait();
          if (ok) {
            float f[32];
#pragma unroll
            for (int d = 0; d < 32; ++d) f[d] = __uint_as_float(ov[d]) * inv;
            st_bf16x16(op + dc * 32, f);
            st_bf16x16(op + dc * 32 + 16, f + 16);
          }
        }
      }
      tc_fence_before_sync();
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace ubm

// q: bf16 [B][Nq][ld] with head h at columns h * 128; k, v: bf16 [B][Nk][ld_kv] with kv head at columns hk * 128
// (Hkv divides H; head h reads kv head h / (H / Hkv)).  out: bf16 [B][Nq][ld_out].  Leading dimensions in elements,
// multiples of 16.  Query i attends to keys 0 .. i + (Nk - Nq).  scale: softmax scale (1 / sqrt(128) when <= 0).
extern "C" int ubm_causal_attention_d128(const void* q, const void* k, const void* v, void* out, int B, int H, int Hkv,
                                         int Nq, int Nk, long long ld_q, long long ld_kv, long long ld_out,
                                         float scale, void* status, void* stream) {
  using namespace ubm;
  if (B <= 0 || H <= 0 || Hkv <= 0 || (H % Hkv) || Nq <= 0 || Nk < Nq) return UBM_ERR_ARGUMENT;
  if (ld_q < (long long)H * kCD || ld_kv < (long long)Hkv * kCD || ld_out < (long long)H * kCD || (ld_q & 15) ||
      (ld_kv & 15) || (ld_out & 15) || (reinterpret_cast<uintptr_t>(out) & 31))
    return UBM_ERR_ARGUMENT;
  CUtensorMap tmQ, tmK, tmV;
  {
    uint64_t d[3] = {(uint64_t)H * kCD, (uint64_t)Nq, (uint64_t)B};
    uint64_t s[2] = {(uint64_t)ld_q * 2, (uint64_t)ld_q * 2 * (uint64_t)Nq};
    uint32_t b[3] = {64, kCTile, 1};
    int rc = make_tmap(&tmQ, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, d, s, b, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  {
    uint64_t d[3] = {(uint64_t)Hkv * kCD, (uint64_t)Nk, (uint64_t)B};
    uint64_t s[2] = {(uint64_t)ld_kv * 2, (uint64_t)ld_kv * 2 * (uint64_t)Nk};
    uint32_t b[3] = {64, kCTK, 1};
    int rc = make_tmap(&tmK, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, d, s, b, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = make_tmap(&tmV, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, d, s, b, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  CausalParams p = {};
  p.B = B;
  p.H = H;
  p.Hkv = Hkv;
  p.Nq = Nq;
  p.Nk = Nk;
  p.off = Nk - Nq;
  p.scale_log2e = (scale > 0.f ? scale : 0.08838834764831845f) * 1.4426950408889634f;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.ld_out = ld_out;
  p.status = static_cast<KernelStatus*>(status);
  p.n_qt = (Nq + kCTile - 1) / kCTile;
  p.n_qp = (p.n_qt + 1) / 2;
  p.num_items = p.n_qp * B * H;
  auto kern = causal_attention_kernel;
  {
    // the in-kernel register re-split must fit the pool this build was compiled with, or it would never return
    cudaFuncAttributes fa;
    cudaError_t e = cudaFuncGetAttributes(&fa, kern);
    if (e != cudaSuccess || 128 * 56 + 512 * kCSoftmaxRegs > kCThreads * fa.numRegs) {
      fprintf(stderr, "[ubm] causal attention: register budget check failed (numRegs=%d)\n",
              e == cudaSuccess ? fa.numRegs : -1);
      return UBM_ERR_LAUNCH;
    }
  }
  int rc = set_smem(kern, kCSmemBytes);
  if (rc) return rc;
  const int grid = p.num_items < sm_count() ? p.num_items : sm_count();
  kern<<<grid, kCThreads, kCSmemBytes, static_cast<cudaStream_t>(stream)>>>(tmQ, tmK, tmV, p);
  UBM_CHECK_LAUNCH("causal_attention_kernel");
  return UBM_OK;
}
