// LayerNorm backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference (NVIDIA PhysicsNeMo); it exists for
// users of this library whose calling context cannot obtain device memory:
//   * hosts that run under a fixed device-memory budget that is fully handed out before
//     the step loop starts (serving processes, co-located jobs), where a cudaMalloc in the
//     loop can fail or stall;
//   * plug-in style callers (a custom op inside another runtime, a solver callback) that
//     are handed input/output buffers by a foreign allocator and have no allocator of
//     their own to ask for a work buffer;
//   * latency-critical loops in which the implicit device synchronisation of
//     cudaMalloc / cudaFree is not acceptable.
// The regular entry point pnm_layernorm_bwd() needs a caller-provided scratch buffer of
// pnm_layernorm_bwd_scratch_floats() floats for the per-CTA partial sums of dgamma/dbeta.
// The variant below keeps that scratch inside the library image instead: a file-scope
// device array of 160 * 2 * 1024 floats (1.25 MiB) that every GPU loading the library
// holds until the process exits.
//
// Limits and rules
//   * C (the normalised width) must be a multiple of 8 and at most 1024; M >= 1.  Anything
//     else is rejected with PNM_NOALLOC_E_SIZE (-101) and a message on stderr; nothing is
//     launched.
//   * The function never calls cudaMalloc, cudaFree or any allocating library routine.
//   * The first call on each device resolves the device address of the scratch array
//     (cudaGetSymbolAddress with that device current).  Make that first call before any
//     stream capture is started; later calls only launch the two kernels.
//   * All calls on one device share the one scratch array.  The kernels overwrite every
//     scratch element they later read, so nothing has to be cleared between calls, but two
//     calls that overlap on the GPU (different streams without an ordering between them)
//     race on it.  Serialise them, e.g. by using one stream.
//   * Results equal those of pnm_layernorm_bwd() up to the order of the fp32 partial sums
//     (the grid is capped at 160 CTAs here).
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

#define PNM_NOALLOC_E_SIZE (-101)    // M, C outside the supported range
#define PNM_NOALLOC_E_SETUP (-102)   // device query / symbol lookup failed
#define PNM_NOALLOC_E_LAUNCH (-103)  // kernel launch failed

// dy, x, dres (optional), dx: bf16 [M, C]; gamma, dgamma, dbeta: fp32 [C]; mean, rstd: fp32 [M].
// Returns 0 on success.
int pnm_layernorm_bwd_noalloc(const void* dy, const void* x, const float* gamma, const float* mean,
                              const float* rstd, const void* dres, void* dx, float* dgamma, float* dbeta,
                              long long M, int C, void* stream);

#ifdef __cplusplus
}
#endif
