// Peer-memory primitives over NVLink: a barrier among the GPUs of one host that is launched on the
// stream between two kernels, with a bounded wait.
//
// Each GPU owns an array of flag words in memory that all peers have mapped.  ubm_peer_barrier stores the
// current epoch into every peer's copy of flags[rank] with a system-scope release (after a system fence, so
// everything earlier kernels on this stream wrote - projected operand rows, bias planes - is visible to
// the peer that observes the flag), then spins with acquire loads on its own flags[peer] until every peer
// has reached the same epoch.  The spin is bounded: after the limit the kernel writes a status word
// (code 2, site 90, aux = the peer it waited for) and returns, so a peer that died between steps surfaces
// as an error on the host and never as a hung GPU.  Plain peer loads / stores only (no multimem).
// Reference counterpart: the NCCL collectives and host-side waits of
// common/opt_core/opt_core/mem/rowpair/dist.py:706-709,1566.
#include "host_util.h"
#include "sm100.cuh"

namespace ubm {

struct BarrierParams {
  uint32_t* peer_flags[8];  // peer_flags[q] = base of GPU q's flag array (mapped here)
  int rank, world;
  uint32_t epoch;
  unsigned long long limit_ns;
  KernelStatus* status;
};

__global__ void __launch_bounds__(32) peer_barrier_kernel(BarrierParams p) {
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) abort_flag = 0;
  __syncwarp();
  const WaitScope ws{&abort_flag, p.status};
  const int q = threadIdx.x;
  __threadfence_system();
  if (q < p.world && q != p.rank) st_release_sys(p.peer_flags[q] + p.rank, p.epoch);
  if (q < p.world && q != p.rank)
    wait_flag_ge(p.peer_flags[p.rank] + q, p.epoch, ws, 90, static_cast<unsigned int>(q), p.limit_ns);
  __threadfence_system();
}

// Write `value` into flags[index] of this GPU's own array (used by tests to make a wait run out or pass).
__global__ void set_flag_kernel(uint32_t* flags, int index, uint32_t value) {
  st_release_sys(flags + index, value);
}

}  // namespace ubm

// flag_ptrs: host array of `world` device pointers (each GPU's flag array, >= world uint32, zero-initialised
// once).  epoch must grow by one per barrier and be the same on all ranks.  limit_ms <= 0 selects 4000 ms.
extern "C" int ubm_peer_barrier(const void* const* flag_ptrs, int rank, int world, unsigned int epoch, int limit_ms,
                                void* status, void* stream) {
  using namespace ubm;
  if (world < 1 || world > 8 || rank < 0 || rank >= world) return UBM_ERR_ARGUMENT;
  BarrierParams p = {};
  for (int q = 0; q < world; ++q) p.peer_flags[q] = static_cast<uint32_t*>(const_cast<void*>(flag_ptrs[q]));
  p.rank = rank;
  p.world = world;
  p.epoch = epoch;
  p.limit_ns = limit_ms > 0 ? static_cast<unsigned long long>(limit_ms) * 1000000ull : kPeerLimitNs;
  p.status = static_cast<KernelStatus*>(status);
  peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(p);
  UBM_CHECK_LAUNCH("peer_barrier_kernel");
  return UBM_OK;
}

extern "C" int ubm_set_flag(void* flags, int index, unsigned int value, void* stream) {
  ubm::set_flag_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint32_t*>(flags), index, value);
  UBM_CHECK_LAUNCH("set_flag_kernel");
  return ubm::UBM_OK;
}


// Sum of the slots a reduce-scatter's senders wrote: out[r][c] = sum over p (in rank order) of slots[p][r][c].
// bf16 slots, fp32 accumulation, bf16 (or fp32) output; 16-byte accesses; optional bias [C] and residual [R][C].
namespace ubm {
__global__ void __launch_bounds__(256) sum_slots_kernel(const __nv_bfloat16* __restrict__ slots, long long slot_stride,
                                                        int P, const float* __restrict__ bias,
                                                        const __nv_bfloat16* __restrict__ residual,
                                                        __nv_bfloat16* __restrict__ out, long long R, int C) {
  const int c8 = C / 8;
  const long long total = R * c8;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % c8) * 8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int p = 0; p < P; ++p) {
      const uint4 u = *reinterpret_cast<const uint4*>(slots + p * slot_stride + i * 8);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] += bf16_lo(w[j]);
        acc[2 * j + 1] += bf16_hi(w[j]);
      }
    }
    if (bias != nullptr) {
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += bias[c + j];
    }
    if (residual != nullptr) {
      const uint4 u = *reinterpret_cast<const uint4*>(residual + i * 8);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] += bf16_lo(w[j]);
        acc[2 * j + 1] += bf16_hi(w[j]);
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + i * 8) = o;
  }
}
}  // namespace ubm

// slots: bf16 [P][R][C] contiguous per slot, slot_stride in elements (this GPU's own memory).
extern "C" int ubm_sum_slots(const void* slots, long long slot_stride, int P, const void* bias, const void* residual,
                             void* out, long long R, int C, void* stream) {
  using namespace ubm;
  if (P < 1 || R <= 0 || C <= 0 || (C & 7) || (slot_stride & 7)) return UBM_ERR_ARGUMENT;
  long long blocks = (R * (C / 8) + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 32;
  if (blocks > cap) blocks = cap;
  sum_slots_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(slots), slot_stride, P, static_cast<const float*>(bias),
      static_cast<const __nv_bfloat16*>(residual), static_cast<__nv_bfloat16*>(out), R, C);
  UBM_CHECK_LAUNCH("sum_slots_kernel");
  return UBM_OK;
}
