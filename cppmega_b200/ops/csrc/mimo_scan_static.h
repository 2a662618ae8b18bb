// Allocation-free entry point for the Mamba3 MIMO forward scan.
//
// This function has no counterpart in the reference project; it exists for host programs that drive the scan from
// plain C/C++ (a serving loop, a plug-in inside another runtime) and have no caching allocator of their own to carve
// the kernel's work buffers from.  Such callers cannot afford a device allocation per call (cudaMalloc / cudaFree
// serialise the whole device) and often are not allowed to allocate at all once their memory plan is fixed.
//
// The three work buffers of the scan (per-chunk local states, per-chunk decay totals, per-chunk start states) live in
// one array that is part of the library image on the device, so its storage exists as soon as the module is loaded
// and is never allocated or freed by this call or anything it calls.
//
// Limits:   B * H * (S / 32) <= CM_MIMO_STATIC_MAX_CHUNKS.  The array takes CM_MIMO_STATIC_BYTES (about 12 MiB) of
//           device memory per context that loads the library.  Larger problems are refused with
//           CM_MIMO_STATIC_E_TOO_LARGE and a message on stderr; nothing is launched.
// Set-up:   the first call on each device looks the array's address up (that device must be current, as it must be
//           for the launch anyway).  Make that first call during initialisation, ahead of any stream capture the
//           program does later; later calls on the same device only launch kernels.  The address is cached per device
//           ordinal for the life of the process: a program that destroys a device's primary context (cudaDeviceReset)
//           and creates a new one must not call this entry point again on that device, because the cached address
//           belongs to the module image of the destroyed context.
// Contents: every word the kernels read from the array is written earlier in the same call, so nothing has to be
//           cleared beforehand; the array simply keeps what the last call left in it.
// Sharing:  there is ONE array per device.  Two calls whose kernels may overlap in time (different streams, different
//           host threads) race on it; order them on one stream or with events.
#pragma once
#include <cuda_runtime.h>

#define CM_MIMO_STATIC_MAX_CHUNKS 256
#define CM_MIMO_STATIC_STATE_ELEMS (128 * 64)   /* d_state x headdim */
#define CM_MIMO_STATIC_BYTES \
  ((size_t)CM_MIMO_STATIC_MAX_CHUNKS * CM_MIMO_STATIC_STATE_ELEMS * (4 + 2) + (size_t)CM_MIMO_STATIC_MAX_CHUNKS * 4)

#define CM_MIMO_STATIC_E_TOO_LARGE (-20)   /* B*H*S/32 exceeds CM_MIMO_STATIC_MAX_CHUNKS */
#define CM_MIMO_STATIC_E_SYMBOL (-21)      /* the array's device address could not be obtained */
#define CM_MIMO_STATIC_E_DEVICE (-22)      /* no current device / ordinal out of range */

#ifdef __cplusplus
extern "C" {
#endif

// Same tensors, layouts and return codes as cm_mimo_scan_fwd (N must be 128, S a multiple of 32), without the three
// scratch pointers.  y [B,S,H,64] bf16 and final_state [B,H,128,64] fp32 (may be null) are written by the call.
int cm_mimo_scan_fwd_static(const void* Qn, const void* Kn, const void* V, const void* Z, const float* ADT,
                            const float* DT, const float* Trap, const float* Qb, const float* Kb, const float* Psi,
                            const float* Zeta, const float* Phi, const float* angles, const float* Dskip,
                            float* final_state, void* y, int B, int S, int H, int G, int N, int* err,
                            cudaStream_t stream);

#ifdef __cplusplus
}
#endif
