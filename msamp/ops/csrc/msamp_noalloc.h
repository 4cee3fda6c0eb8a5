// Entry point for callers that must not allocate device memory.
//
// This function has no counterpart in the reference; it exists for hosts of this library that
// cannot call cudaMalloc (or any allocating library routine) at the point where they need a
// LayerNorm backward: code running inside a memory-planned region whose device memory was carved up
// ahead of time, plugins loaded into a process whose allocator they are not allowed to touch, or
// steps that must not disturb an allocator's bookkeeping.  msamp_layernorm_bwd needs a scratch
// buffer for the per-CTA partial sums of dgamma/dbeta and leaves its allocation to the caller;
// the variant below keeps that scratch in a file-scope `static __device__` array instead.
//
// Contract
//   * Same arguments and results as msamp_layernorm_bwd, minus the `part` scratch pointer: the caller
//     still passes every input and output (dy, x, gamma, mean, rstd -> dx, dgamma, dbeta).
//   * Limit: cols <= MSAMP_LN_STATIC_MAX_COLS (4096).  Wider rows are rejected with
//     MSAMP_ECAPACITY (6) and a message from msamp_last_error(); nothing is launched.
//   * The scratch is MSAMP_LN_STATIC_PARTS * 2 * MSAMP_LN_STATIC_MAX_COLS floats = 4 MiB, held by
//     every GPU that loads the library until the process exits.
//   * The first call on each device looks up the array's device address with cudaGetSymbolAddress
//     (the array's name is not a device pointer in host code).  That first call should therefore
//     happen before any stream capture begins on that device.
//     The address is remembered per device for the life of the process; after cudaDeviceReset (or
//     any other re-creation of the device's context) it is stale, so reload the library before calling again.
//   * dy, x, dx and gamma must be 16-byte aligned (the kernels use 16-byte accesses); a misaligned
//     pointer is rejected with MSAMP_EINVAL (1) before anything is launched.
//   * The function itself calls no cudaMalloc / cudaFree and no allocating library routine.
//   * All calls share the one array, which keeps the last call's contents.  Nothing in it has to
//     start at zero (every slice that is read was written by the same call), but two calls that
//     overlap on the GPU - different streams, or different host threads - race on it: serialise them.
#pragma once

#define MSAMP_LN_STATIC_PARTS 128
#define MSAMP_LN_STATIC_MAX_COLS 4096

#ifdef __cplusplus
extern "C" {
#endif

int msamp_layernorm_bwd_static(const void* dy, const void* x, const void* gamma, int dtype, int pdtype, const float* mean,
                               const float* rstd, void* dx, void* dgamma, void* dbeta, int rows, int cols, void* stream);

#ifdef __cplusplus
}
#endif
