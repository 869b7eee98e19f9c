// Host-side helpers shared by the kernel entry points: tensor-map encoding through the driver
// entry point (so the library does not link libcuda and still loads on a box without a GPU),
// error codes of the C ABI, and per-device attribute caching.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

namespace ubm {

// Return codes of every extern "C" entry point.
enum : int {
  UBM_OK = 0,
  UBM_ERR_ARGUMENT = -1,   // shape / alignment / size outside what the kernel supports
  UBM_ERR_DRIVER = -2,     // tensor-map encode or driver entry point lookup failed
  UBM_ERR_LAUNCH = -3,     // cudaLaunch / attribute error (see stderr)
  UBM_ERR_TOO_LARGE = -4,  // fixed-size workspace exceeded
};

typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline PFN_encodeTiled get_encode_fn() {
  static PFN_encodeTiled fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr) {
      fprintf(stderr, "[ubm] cuTensorMapEncodeTiled entry point not available (%d)\n", (int)e);
      return nullptr;
    }
    fn = reinterpret_cast<PFN_encodeTiled>(p);
  }
  return fn;
}

// Encode a tiled tensor map of rank `rank` (innermost dimension first).
//   dims[r]     extent in elements
//   strides[r]  byte stride of dimension r+1 (rank-1 entries), multiples of 16
//   box[r]      tile extent in elements
// Returns UBM_OK or an error code; prints the reason.
inline int make_tmap(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int rank, const uint64_t* dims,
                     const uint64_t* strides, const uint32_t* box, CUtensorMapSwizzle swz,
                     CUtensorMapL2promotion l2 = CU_TENSOR_MAP_L2_PROMOTION_L2_128B) {
  PFN_encodeTiled fn = get_encode_fn();
  if (!fn) return UBM_ERR_DRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) {
    fprintf(stderr, "[ubm] tensor map base %p not 16-byte aligned\n", base);
    return UBM_ERR_ARGUMENT;
  }
  cuuint64_t d[5];
  cuuint64_t s[5];
  cuuint32_t b[5];
  cuuint32_t es[5];
  for (int i = 0; i < rank; ++i) {
    d[i] = dims[i];
    b[i] = box[i];
    es[i] = 1;
    if (i + 1 < rank) {
      s[i] = strides[i];
      if (s[i] % 16 != 0) {
        fprintf(stderr, "[ubm] tensor map stride %llu not a multiple of 16 bytes\n", (unsigned long long)s[i]);
        return UBM_ERR_ARGUMENT;
      }
    }
  }
  CUresult r = fn(out, dt, (cuuint32_t)rank, const_cast<void*>(base), d, s, b, es, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                  l2, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "[ubm] cuTensorMapEncodeTiled failed: %d (rank %d dims %llu %llu %llu box %u %u %u)\n", (int)r,
            rank, (unsigned long long)d[0], (unsigned long long)(rank > 1 ? d[1] : 0),
            (unsigned long long)(rank > 2 ? d[2] : 0), b[0], rank > 1 ? b[1] : 0, rank > 2 ? b[2] : 0);
    return UBM_ERR_DRIVER;
  }
  return UBM_OK;
}

inline int sm_count() {
  static int n[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (n[dev] == 0) {
    cudaDeviceGetAttribute(&n[dev], cudaDevAttrMultiProcessorCount, dev);
    if (n[dev] <= 0) n[dev] = 148;
  }
  return n[dev];
}

#define UBM_CHECK_LAUNCH(what)                                                              \
  do {                                                                                      \
    cudaError_t e__ = cudaGetLastError();                                                   \
    if (e__ != cudaSuccess) {                                                               \
      fprintf(stderr, "[ubm] launch of %s failed: %s\n", what, cudaGetErrorString(e__));    \
      return ubm::UBM_ERR_LAUNCH;                                                           \
    }                                                                                       \
  } while (0)

template <typename K>
inline int set_smem(K kernel, int bytes) {
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) {
    fprintf(stderr, "[ubm] cudaFuncSetAttribute(%d bytes) failed: %s\n", bytes, cudaGetErrorString(e));
    return UBM_ERR_LAUNCH;
  }
  return UBM_OK;
}


// Transposed peer source of the projection kernels (row-sharded pair tensor): the rows this GPU projects are
// COLUMNS of z, z^T[i][k] = z[k][i], and z[k] lives on the GPU that owns row k.  m[q] is a 3-d tensor map over GPU
// q's shard bf16 [rows_q][N][128] (box 64 channels x 1 column x 128 rows); a 128-entry tile (fixed column, 128
// consecutive k) is fetched from its owner with a plain TMA load - shard boundaries are multiples of 128, so a tile
// has one owner.  row0[q] = first row of shard q (row0[n] = N); col0 = first column this GPU projects.
constexpr int kMaxSrcPeers = 8;
struct PeerSrcMaps {
  CUtensorMap m[kMaxSrcPeers];
};
struct PeerSrc {
  int n;                        // 0 = local row-major source
  int row0[kMaxSrcPeers + 1];
  int col0;
};

inline int make_peer_src(PeerSrcMaps* maps, PeerSrc* src, const void* const* z_ptrs, const int* rows, int npeers,
                         int me, int N, const CUtensorMap& filler) {
  if (npeers < 1 || npeers > kMaxSrcPeers || me < 0 || me >= npeers || (N & 127)) return UBM_ERR_ARGUMENT;
  src->n = npeers;
  int row = 0;
  for (int q = 0; q < kMaxSrcPeers; ++q) maps->m[q] = filler;
  for (int q = 0; q < npeers; ++q) {
    src->row0[q] = row;
    if (q == me) src->col0 = row;
    if (rows[q] < 0 || (rows[q] & 127 && q + 1 < npeers)) return UBM_ERR_ARGUMENT;
    if (rows[q] > 0) {
      uint64_t d[3] = {128, (uint64_t)N, (uint64_t)rows[q]};
      uint64_t st[2] = {128 * 2, (uint64_t)N * 128 * 2};
      uint32_t b[3] = {64, 1, 128};
      int rc = make_tmap(&maps->m[q], z_ptrs[q], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, d, st, b,
                         CU_TENSOR_MAP_SWIZZLE_128B);
      if (rc) return rc;
    }
    row += rows[q];
  }
  for (int q = npeers; q <= kMaxSrcPeers; ++q) src->row0[q] = row;
  return row == N ? UBM_OK : UBM_ERR_ARGUMENT;
}

}  // namespace ubm
