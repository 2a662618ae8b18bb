// Shared device/host helpers for the sm_100a kernels: mbarrier, TMA, tcgen05/TMEM wrappers,
// bounded waits with an error word, and small math utilities.
//
// Every wait in these kernels is bounded.  A wait that runs out stores a code into the
// caller-provided error word (and a CTA-local abort flag) and the kernel unwinds: all
// roles leave their loops, TMEM is released, the CTA returns.  The host reads the error
// word after the stream synchronises and raises.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace cm {

enum ErrorCode : int {
  ERR_NONE = 0,
  ERR_WAIT_FULL = 1,       // consumer never saw a TMA stage arrive
  ERR_WAIT_EMPTY = 2,      // producer never got a stage back
  ERR_WAIT_TMEM_FULL = 3,  // epilogue never saw the accumulator complete
  ERR_WAIT_TMEM_EMPTY = 4, // MMA issuer never got the accumulator back
  ERR_WAIT_PEER = 5,       // a flag owned by another GPU was never set
  ERR_BAD_ARG = 6,
};

#ifndef CM_WAIT_LIMIT
#define CM_WAIT_LIMIT (1u << 24)   // try_wait polls (each suspends up to the HW time slice)
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n"
      ".reg .pred P;\n"
      "elect.sync _|P, 0xffffffff;\n"
      "selp.u32 %0, 1, 0, P;\n"
      "}\n"
      : "=r"(pred));
  return pred;
}

// ---- mbarrier ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok;
}

// Bounded wait.  Returns false (after recording `code`) if the barrier never flips or if
// another role of this CTA has already aborted.
// The bound is wall clock (CM_WAIT_NS, default 2 s): a try_wait poll may itself suspend for an
// implementation-defined time, so counting polls does not bound anything.  A kernel-wide error word that
// is already set (another CTA gave up) ends the wait at once, so a broken launch drains quickly.
#ifndef CM_WAIT_NS
#define CM_WAIT_NS 2000000000ull
#endif
__device__ __forceinline__ unsigned long long cm_globaltimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int* err_word, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = cm_globaltimer();
  for (uint32_t i = 0;; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 63u) == 63u) {
      if (*abort_flag) return false;
      if (err_word && *reinterpret_cast<volatile int*>(err_word) != 0) { *abort_flag = 1; return false; }
      if (cm_globaltimer() - t0 > CM_WAIT_NS) break;
    }
  }
  *abort_flag = 1;
  if (err_word) atomicCAS(err_word, 0, code);
  return false;
}

// ---- cross-GPU flags ------------------------------------------------------------------------
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// Spin until *flag >= value or `timeout_ns` of wall clock has passed (returns false then).
__device__ __forceinline__ bool wait_flag_ge(const unsigned long long* flag, unsigned long long value,
                                             unsigned long long timeout_ns) {
  if (ld_acquire_sys(flag) >= value) return true;
  const unsigned long long t0 = global_timer_ns();
  while (true) {
    if (ld_acquire_sys(flag) >= value) return true;
    if (global_timer_ns() - t0 > timeout_ns) return false;
    __nanosleep(100);
  }
}

// ---- TMA ---------------------------------------------------------------------------------
// Tiled loads into this CTA's shared memory, completion on an mbarrier of this CTA.
// Every load in this library targets exactly one CTA.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1,
                                            int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1),
      "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---- tcgen05 / TMEM ------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {   // one full warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {        // one full warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem], bf16/fp16 inputs, fp32 accumulate.  One thread issues.
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on an mbarrier of this CTA once all previously issued MMAs of this thread retire.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// 32 lanes x 32 consecutive fp32 columns -> 32 registers per thread (thread = TMEM lane).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, 128-byte swizzle.
//   K-major operand: rows of 128 bytes (64 bf16 along K), 8-row groups 1024 bytes apart.
//   MN-major operand: 64-element (128-byte) runs along M/N, k rows 128 bytes apart, 8-row
//   groups `sbo` bytes apart, successive 64-element runs `lbo` bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;                 // descriptor version for this architecture
  d |= 2ull << 61;                 // SWIZZLE_128B
  return d;
}

// Instruction descriptor for kind::f16 with bf16 A/B and fp32 accumulation.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int m, int n, bool a_mn_major, bool b_mn_major) {
  return (1u << 4)                       // D format fp32
         | (1u << 7) | (1u << 10)        // A, B format bf16
         | (uint32_t(a_mn_major) << 15) | (uint32_t(b_mn_major) << 16) | (uint32_t(n >> 3) << 17) |
         (uint32_t(m >> 4) << 24);
}

// ---- misc -----------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Transposing all-reduce: every lane holds 32 values; lane l returns the reduction over the 32 lanes of element l
template <bool IS_MAX>
__device__ __forceinline__ float xreduce32(const float (&v)[32], int lane) {
  float a16[16], a8[8], a4[4], a2[2];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const bool up = lane & 16;
    const float keep = up ? v[i + 16] : v[i], send = up ? v[i] : v[i + 16];
    const float recv = __shfl_xor_sync(0xffffffffu, send, 16);
    a16[i] = IS_MAX ? fmaxf(keep, recv) : keep + recv;
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const bool up = lane & 8;
    const float keep = up ? a16[i + 8] : a16[i], send = up ? a16[i] : a16[i + 8];
    const float recv = __shfl_xor_sync(0xffffffffu, send, 8);
    a8[i] = IS_MAX ? fmaxf(keep, recv) : keep + recv;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const bool up = lane & 4;
    const float keep = up ? a8[i + 4] : a8[i], send = up ? a8[i] : a8[i + 4];
    const float recv = __shfl_xor_sync(0xffffffffu, send, 4);
    a4[i] = IS_MAX ? fmaxf(keep, recv) : keep + recv;
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const bool up = lane & 2;
    const float keep = up ? a4[i + 2] : a4[i], send = up ? a4[i] : a4[i + 2];
    const float recv = __shfl_xor_sync(0xffffffffu, send, 2);
    a2[i] = IS_MAX ? fmaxf(keep, recv) : keep + recv;
  }
  const bool up = lane & 1;
  const float keep = up ? a2[1] : a2[0], send = up ? a2[0] : a2[1];
  const float recv = __shfl_xor_sync(0xffffffffu, send, 1);
  return IS_MAX ? fmaxf(keep, recv) : keep + recv;
}

// ---- host: tensor-map encoding through the runtime's driver entry point -----------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode_tiled();

// 2-D bf16 row-major matrix [rows, cols] (cols contiguous, row pitch `ld` elements), boxes of
// [box_rows, 64] elements with 128-byte swizzle.  Returns 0 on success.
int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                      uint32_t box_rows, uint32_t box_cols = 64);
// 3-D [batch, rows, cols] with dense batch pitch rows*ld.
int make_tmap_3d_bf16(CUtensorMap* out, const void* base, uint64_t batch, uint64_t rows, uint64_t cols, uint64_t ld,
                      uint32_t box_rows, uint32_t box_cols = 64);

int sm_count();

// Function attributes (the dynamic shared-memory limit) are per device: a flag per (call site, device) says whether the
// current device has been configured.  Usage: `static PerDevice cfg; if (cfg.first()) { cudaFuncSetAttribute(...); cfg.done(); }`
struct PerDevice {
  bool set[64] = {};
  int dev = -1;
  bool first() {
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { dev = -1; return true; }
    return !set[dev];
  }
  void done() { if (dev >= 0) set[dev] = true; }
};

}  // namespace cm
