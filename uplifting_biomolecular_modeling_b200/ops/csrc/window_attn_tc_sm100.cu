// Atom attention in sequence-local windows on the tensor cores: one CTA takes four consecutive query
// windows (128 queries) of one head and one sample.  Window w attends to atoms [32 w - 48, 32 w + 80), so
// the four windows together see 224 consecutive atoms; K and V of 256 atoms starting at 128 g - 48 come in
// by TMA (rows before atom 0 or past the last atom are zero-filled and masked), and
//     S[128 x 256] = Q . K^T          (two tcgen05.mma of K = 16, accumulator in tensor memory)
// holds every needed score.  A thread owns one query row and reads only the 128 columns of its own window
// (columns 32 j .. 32 j + 127 for window j of the group), adds the per-window pair bias, takes the softmax in
// base 2 and writes the probabilities back into tensor memory as packed bf16 - zeros outside its window -
// over the score columns it has consumed.  O[128 x 32] = P . V then runs with P as the tensor-memory (TS
// form) operand and V straight from the TMA tile (MN-major), into columns the scores no longer need.  The
// epilogue scales by 1 / sum, applies the gate and stores 64 bytes per row.  Tensor memory per CTA: 256
// columns, so two CTAs share an SM and overlap each other's load and softmax phases.
//
// q is pre-scaled by log2(e)/sqrt(32) and the bias by log2(e).  Reference kernels with the same boundary:
// common/opt_core/opt_core/kernels/atom_window.py (_window_attn_kernel), apb/fpf_apb (_atom_fwd).
#include "host_util.h"
#include "sm100.cuh"

namespace ubm {

constexpr int kWTQ = 128;    // queries per CTA (four windows)
constexpr int kWTK = 256;    // keys held per CTA
constexpr int kWTD = 32;     // head dimension
constexpr int kWTQBytes = kWTQ * kWTD * 2;   // 8 KB
constexpr int kWTKBytes = kWTK * kWTD * 2;   // 16 KB

struct WindowTcParams {
  const __nv_bfloat16* bias;  // [bias_batch][H][nw][32][128] or null
  const __nv_bfloat16* gate;  // [B][A][H*32] (already sigmoid) or null
  __nv_bfloat16* out;         // [B][A][H*32]
  int B, A, H, nw;
  int bias_batch;
  KernelStatus* status;
};

// probabilities of window j of the group -> packed columns 16 j .. 16 j + 63; zeros elsewhere in 0 .. 127
template <int J>
__device__ __forceinline__ void store_probabilities(uint32_t taddr, const uint32_t (&pk)[64]) {
  uint32_t zero[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) zero[i] = 0u;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    if (c >= J && c < J + 4) {
      uint32_t part[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) part[i] = pk[(c - J) * 16 + i];
      tmem_st16(taddr + c * 16, part);
    } else {
      tmem_st16(taddr + c * 16, zero);
    }
  }
}

__global__ void __launch_bounds__(128, 2)
window_attention_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                           const __grid_constant__ CUtensorMap tmV, WindowTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + kWTQBytes;
  uint8_t* sV = sK + kWTKBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + kWTKBytes);
  uint64_t* ld_full = bars;       // TMA tiles landed
  uint64_t* s_full = bars + 1;    // scores complete
  uint64_t* o_full = bars + 2;    // output accumulator complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;   // = window of the group, = tensor-memory lane quadrant
  const int lane = threadIdx.x & 31;
  const int g = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const WaitScope ws{abort_flag, p.status};

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(ld_full, 1);
    mbar_init(s_full, 1);
    mbar_init(o_full, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base;          // 256 fp32 columns; packed P later overlays columns 0..127
  const uint32_t tO = tmem_base + 128;    // 32 columns, written after every thread has read its scores

  const int key0 = g * kWTQ - 48;         // atom of key column 0
  const bool leader = (warp == 0) && elect_one();
  if (leader) {
    mbar_expect_tx(ld_full, kWTQBytes + 2 * kWTKBytes);
    tma_load_3d(sQ, &tmQ, ld_full, h * kWTD, g * kWTQ, b);
    tma_load_3d(sK, &tmK, ld_full, h * kWTD, key0, b);
    tma_load_3d(sV, &tmV, ld_full, h * kWTD, key0, b);
  }
  // the bias row of this query (256 contiguous bytes) travels while the tiles load
  const int w = g * 4 + warp;             // window of this warp
  const int atom_q = w * 32 + lane;
  const bool q_ok = w < p.nw;             // whole window in range (A is a multiple of 32)
  float bj[128];
  if (p.bias != nullptr && q_ok) {
    const int bb = p.bias_batch == 1 ? 0 : b;
    const __nv_bfloat16* brow = p.bias + (((static_cast<long long>(bb) * p.H + h) * p.nw + w) * 32 + lane) * 128;
#pragma unroll
    for (int c = 0; c < 8; ++c) ld_bf16x16(brow + c * 16, bj + c * 16);
  } else {
#pragma unroll
    for (int c = 0; c < 128; ++c) bj[c] = 0.f;
  }

  mbar_wait(ld_full, 0, ws, 71);
  tc_fence_after_sync();
  if (warp == 0) {
    if (leader) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16(128, kWTK, 0, 0);
      const uint64_t qd = umma_smem_desc(smem_u32(sQ), 16, 512, kSwizzle64);
      const uint64_t kd = umma_smem_desc(smem_u32(sK), 16, 512, kSwizzle64);
#pragma unroll
      for (int k = 0; k < kWTD / 16; ++k)
        umma_ss(tS, qd + static_cast<uint64_t>(k * 2), kd + static_cast<uint64_t>(k * 2), idesc_qk, k != 0 ? 1u : 0u);
      umma_commit(s_full);
    }
    __syncwarp();
  }
  mbar_wait(s_full, 0, ws, 72);
  tc_fence_after_sync();

  // ---- softmax over the 128 keys of this query's window: score columns 32 * warp .. + 127
  float s[128];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint32_t v[32];
    tmem_ld32(tmem_addr(tS, warp, 32 * warp + 32 * c), v);
    tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 32; ++i) s[c * 32 + i] = __uint_as_float(v[i]);
  }
  const int katom0 = w * 32 - 48;         // atom of this window's key column 0
  float mx = -1.0e30f;
#pragma unroll
  for (int c = 0; c < 128; ++c) {
    const int atom = katom0 + c;
    const float val = (atom >= 0 && atom < p.A) ? s[c] + bj[c] : -1.0e30f;
    s[c] = val;
    mx = fmaxf(mx, val);
  }
  float l = 0.f;
  uint32_t pk[64];
#pragma unroll
  for (int c = 0; c < 64; ++c) {
    const float p0 = fast_exp2(s[2 * c] - mx);
    const float p1 = fast_exp2(s[2 * c + 1] - mx);
    pk[c] = pack_bf16x2(p0, p1);
    // the sum is taken over the rounded values the tensor core will multiply
    l += bf16_lo(pk[c]) + bf16_hi(pk[c]);
  }
  const uint32_t tP = tmem_addr(tS, warp, 0);
  switch (warp) {
    case 0: store_probabilities<0>(tP, pk); break;
    case 1: store_probabilities<1>(tP, pk); break;
    case 2: store_probabilities<2>(tP, pk); break;
    default: store_probabilities<3>(tP, pk); break;
  }
  tmem_st_wait();
  tc_fence_before_sync();
  __syncthreads();      // every score has been read and every probability written
  tc_fence_after_sync();

  if (warp == 0) {
    if (leader) {
      constexpr uint32_t idesc_pv = umma_idesc_bf16(128, kWTD, 0, 1);   // B = V is MN-major
      const uint64_t vd = umma_smem_desc(smem_u32(sV), 16, 512, kSwizzle64);
#pragma unroll
      for (int k = 0; k < kWTK / 16; ++k)
        umma_ts(tO, tS + k * 8, vd + static_cast<uint64_t>(k * ((16 * kWTD * 2) >> 4)), idesc_pv, k != 0 ? 1u : 0u);
      umma_commit(o_full);
    }
    __syncwarp();
  }
  mbar_wait(o_full, 0, ws, 73);
  tc_fence_after_sync();

  {
    uint32_t ov[32];
    tmem_ld32(tmem_addr(tO, warp, 0), ov);
    tmem_ld_wait();
    if (q_ok && atom_q < p.A) {
      const float inv = 1.0f / l;
      float f[32];
#pragma unroll
      for (int d = 0; d < 32; ++d) f[d] = __uint_as_float(ov[d]) * inv;
      const long long orow = (static_cast<long long>(b) * p.A + atom_q) * (p.H * kWTD) + h * kWTD;
      if (p.gate != nullptr) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          float e[16];
          ld_bf16x16(p.gate + orow + c * 16, e);
#pragma unroll
          for (int d = 0; d < 16; ++d) f[c * 16 + d] *= e[d];
        }
      }
      st_bf16x16(p.out + orow, f);
      st_bf16x16(p.out + orow + 16, f + 16);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 256);
  }
}

constexpr int kWTSmemBytes = kWTQBytes + 2 * kWTKBytes + 64 + 1024;

}  // namespace ubm

// q, k, v: bf16 rows [B*A] with row stride ld_in (elements), head h at columns h*32..; A a multiple of 32.
// bias: bf16 [bias_batch][H][A/32][32][128] or null (32-byte aligned); gate / out: bf16 [B*A][H*32].
// status: device KernelStatus (16 bytes) or null.
extern "C" int ubm_window_attention_tc(const void* q, const void* k, const void* v, const void* bias,
                                       const void* gate, void* out, int B, int A, int H, long long ld_in,
                                       int bias_batch, void* status, void* stream) {
  using namespace ubm;
  if (B <= 0 || A <= 0 || (A % 32) || H <= 0 || ld_in < H * kWTD || (ld_in & 7)) return UBM_ERR_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(bias) & 31) || (reinterpret_cast<uintptr_t>(gate) & 31) ||
      (reinterpret_cast<uintptr_t>(out) & 31))
    return UBM_ERR_ARGUMENT;
  WindowTcParams p = {};
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.gate = static_cast<const __nv_bfloat16*>(gate);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.B = B;
  p.A = A;
  p.H = H;
  p.nw = A / 32;
  p.bias_batch = bias_batch;
  p.status = static_cast<KernelStatus*>(status);
  CUtensorMap tmQ, tmK, tmV;
  uint64_t dims[3] = {(uint64_t)H * kWTD, (uint64_t)A, (uint64_t)B};
  uint64_t strides[2] = {(uint64_t)ld_in * 2, (uint64_t)A * ld_in * 2};
  uint32_t boxq[3] = {kWTD, kWTQ, 1};
  uint32_t boxk[3] = {kWTD, kWTK, 1};
  int rc = make_tmap(&tmQ, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, strides, boxq, CU_TENSOR_MAP_SWIZZLE_64B);
  if (rc) return rc;
  rc = make_tmap(&tmK, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, strides, boxk, CU_TENSOR_MAP_SWIZZLE_64B);
  if (rc) return rc;
  rc = make_tmap(&tmV, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, strides, boxk, CU_TENSOR_MAP_SWIZZLE_64B);
  if (rc) return rc;
  rc = set_smem(window_attention_tc_kernel, kWTSmemBytes);
  if (rc) return rc;
  dim3 grid((p.nw + 3) / 4, H, B);
  window_attention_tc_kernel<<<grid, 128, kWTSmemBytes, static_cast<cudaStream_t>(stream)>>>(tmQ, tmK, tmV, p);
  UBM_CHECK_LAUNCH("window_attention_tc_kernel");
  return UBM_OK;
}
