// Symmetric (peer-mapped) device memory for the fused compute+collective kernels, and the
// small signalling kernels that go with it.
//
// Each rank allocates a buffer with cudaMalloc, exports a CUDA IPC handle, and opens every
// peer's handle; the Python side exchanges the 64-byte handles over the host process group and
// keeps the table of peer pointers.  All cross-GPU waits in kernels are bounded: a flag that is
// never set makes the kernel record ERR_WAIT_PEER and return.
// (The reference has no counterpart: its collectives are NCCL calls issued by Megatron with
// NVLS disabled, cppmega/recipes/nam56r_nemo_recipe.py:429-443.)
#include "common.cuh"

#include <string.h>

extern "C" int cm_symm_alloc(void** ptr, size_t bytes) {
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e != cudaSuccess) return int(e);
  return int(cudaMemset(*ptr, 0, bytes));
}

extern "C" int cm_symm_free(void* ptr) { return int(cudaFree(ptr)); }

extern "C" int cm_ipc_get_handle(void* ptr, void* handle_out64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) return int(e);
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(handle_out64, &h, 64);
  return 0;
}

extern "C" int cm_ipc_open_handle(const void* handle64, void** ptr_out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  return int(cudaIpcOpenMemHandle(ptr_out, h, cudaIpcMemLazyEnablePeerAccess));
}

extern "C" int cm_ipc_close_handle(void* ptr) { return int(cudaIpcCloseMemHandle(ptr)); }

extern "C" int cm_can_access_peer(int dev, int peer) {
  int ok = 0;
  if (cudaDeviceCanAccessPeer(&ok, dev, peer) != cudaSuccess) return 0;
  return ok;
}

namespace cm {

// Store `value` into word `index` of every peer's flag array, after making this GPU's earlier
// writes visible system-wide.
__global__ void signal_peers_kernel(unsigned long long* const* flag_ptrs, int world, int index, unsigned long long value) {
  __threadfence_system();
  const int p = threadIdx.x;
  if (p < world) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(flag_ptrs[p] + index), "l"(value) : "memory");
  }
}

// Copy `n` 8-byte words from `src` to byte offset `dst_off` of every peer's buffer (a tiny all-gather contribution: expert
// counts, a few hundred bytes); the signal that follows on the same stream publishes it.
__global__ void put_words_kernel(const unsigned long long* __restrict__ src, unsigned long long* const* dst_ptrs, int world,
                                 long long dst_off_words, int n) {
  for (int i = threadIdx.x; i < n * world; i += blockDim.x) {
    const int p = i / n, j = i - p * n;
    dst_ptrs[p][dst_off_words + j] = src[j];
  }
}

// Wait until words [first, first+count) of the local flag array are all >= value.
__global__ void wait_flags_kernel(const unsigned long long* flags, int first, int count, unsigned long long value,
                                  unsigned long long timeout_ns, int* err) {
  const int i = threadIdx.x;
  if (i >= count) return;
  if (!wait_flag_ge(flags + first + i, value, timeout_ns) && err) atomicCAS(err, 0, ERR_WAIT_PEER);
}

}  // namespace cm

// flag_ptrs: device array of `world` pointers (each peer's flag array, as mapped in this process).
extern "C" int cm_signal_peers(void* flag_ptrs, int world, int index, unsigned long long value, cudaStream_t s) {
  cm::signal_peers_kernel<<<1, 32, 0, s>>>((unsigned long long* const*)flag_ptrs, world, index, value);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// dst_ptrs: device array of `world` pointers to the same symmetric tensor on every peer; writes src[0..n) at word offset
// dst_off_words of each
extern "C" int cm_put_words(const void* src, void* dst_ptrs, int world, long long dst_off_words, int n, cudaStream_t s) {
  if (n <= 0) return 0;
  cm::put_words_kernel<<<1, 256, 0, s>>>((const unsigned long long*)src, (unsigned long long* const*)dst_ptrs, world, dst_off_words, n);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int cm_wait_flags(const void* flags, int first, int count, unsigned long long value,
                             unsigned long long timeout_ns, int* err, cudaStream_t s) {
  if (count > 1024) return -10;
  cm::wait_flags_kernel<<<1, count < 32 ? 32 : count, 0, s>>>((const unsigned long long*)flags, first, count, value,
                                                             timeout_ns, err);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
