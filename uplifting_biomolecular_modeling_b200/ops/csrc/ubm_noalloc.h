// Allocation-free entry point of the kernel library.
//
// This entry point has no counterpart in the reference: the reference's triangle multiplication
// always takes its intermediates from the framework's caching allocator.
//
// Who needs it: code that wants the fused triangle multiplication but is not allowed to allocate
// device memory at the moment of the call - a host thread inside a region where the CUDA allocator
// must stay untouched (another library owns the memory pool, or allocation calls would serialise
// against work in flight), a plugin loaded into a process whose memory budget is fixed up front, or a
// C caller that has no tensor library to allocate through.  Such a caller passes only its inputs and
// its output; the intermediates (the two projected operand planes and the contraction result) live in
// a fixed array that is part of the library image.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Largest token count the built-in scratch array holds.
#define UBM_TRIMUL_NOALLOC_MAX_N 160

// Bytes of device memory the scratch array occupies on EVERY GPU that loads the library, from load
// until the process exits: 3 operand planes of [128][MAX_N][MAX_N] bf16.
#define UBM_TRIMUL_NOALLOC_SCRATCH_BYTES (3ull * 128ull * UBM_TRIMUL_NOALLOC_MAX_N * UBM_TRIMUL_NOALLOC_MAX_N * 2ull)

// z_out = [z +] TriangleMultiplication(z) for one [N, N, 128] bf16 pair tensor, same arithmetic and same
// three kernels as ubm_trimul_proj -> ubm_gemm_bf16 -> ubm_trimul_out, without any allocation:
// no cudaMalloc / cudaFree, no allocating library routine.
//
//   z, out            bf16 [N*N][128] device pointers (out may alias z)
//   mask              fp32 [N*N] or null
//   w_in              bf16 [512][128]   rows [p_a; g_a; p_b; g_b], LayerNorm gamma folded in
//   in_colsum/bias    fp32 [512]
//   wo, wg            bf16 [128][128]   output projection / output gate, gamma folded in
//   o_*/g_* colsum/bias  fp32 [128]
//   N                 tokens, 1 <= N <= UBM_TRIMUL_NOALLOC_MAX_N and N a multiple of 8
//   outgoing          1 = outgoing edges, 0 = incoming edges
//   status            device pointer to 4 x uint32 kernel status words, or null
//   stream            cudaStream_t
//
// Returns 0, or a negative code: -1 bad argument, -4 N larger than the scratch array holds (the call
// does nothing), -2 / -3 driver or launch errors.
//
// The first call on each device looks up the device address of the scratch array (with that device
// current) and sets kernel attributes; make that first call before starting any stream capture.
// All calls on a device share the one array and it keeps whatever the last call left in it; nothing in
// it has to start at zero, every element a call reads was written earlier in the same call.  Two calls
// that overlap on the same GPU (different streams, or different host threads) race on the array: issue
// them on one stream, or order them yourself.
int ubm_trimul_noalloc(const void* z, const void* mask, const void* w_in, const void* in_colsum,
                       const void* in_colbias, const void* wo, const void* wg, const void* o_colsum,
                       const void* o_colbias, const void* g_colsum, const void* g_colbias, void* out, int N,
                       int outgoing, int add_residual, void* status, void* stream);

#ifdef __cplusplus
}
#endif
