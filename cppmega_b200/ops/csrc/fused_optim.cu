// Distributed-optimizer collectives fused with their arithmetic, over peer-mapped memory.
//
//  reduce_shard:  red[i] = scale * sum_p grad_p[lo + i]          (P2P loads from every rank's
//                 gradient buffer = the reduce-scatter), plus sum(red^2) for the gradient norm.
//  adamw_push:    AdamW on the fp32 master shard with grad = clip * red, then the new low-precision
//                 value is stored into every rank's parameter buffer at [lo + i]  (P2P stores = the
//                 parameter all-gather).
// One pass over the shard each; no staging copies, no separate cast / scale / update kernels.
// Ordering across GPUs is carried by flag words (see symm.cu): gradients-ready before the pull,
// parameters-ready after the push.  Both kernels read the device error word first and do nothing when it is set:
// a flag wait that timed out must not let half-reduced gradients reach the master weights or the peers.
// Baseline being replaced: NCCL reduce-scatter + all-gather around a separate optimizer step
// (87 ms/iter in the reference profile, docs/nam56r_mimo7_nsys_profile_2026_04_11.md:13,39).
#include "common.cuh"

namespace cm {

constexpr int MAX_PEERS = 16;

struct PeerPtrs {
  const void* p[MAX_PEERS];
};
struct PeerPtrsMut {
  void* p[MAX_PEERS];
};

template <typename GradT>
__device__ __forceinline__ void load8(const GradT* p, float (&f)[8]);

template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 t = __bfloat1622float2(b[j]);
    f[2 * j] = t.x;
    f[2 * j + 1] = t.y;
  }
}
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&f)[8]) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

// n must be a multiple of 8; all pointers 32-byte aligned at lo.
template <typename GradT>
__global__ void __launch_bounds__(256) reduce_shard_kernel(PeerPtrs grads, int world, int self, long long lo, long long n,
                                                           float scale, float* __restrict__ red, float* __restrict__ sumsq,
                                                           const int* __restrict__ err) {
  // A bounded wait that ran out earlier on this stream (a peer never signalled) leaves the error word set: the peers'
  // gradients may be incomplete, so this step's reduction and update are skipped on the device, with no host round trip.
  if (err && *reinterpret_cast<const volatile int*>(err) != 0) return;
  float ss = 0.f;
  const long long nv = n / 8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv; i += (long long)gridDim.x * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int q = 0; q < world; ++q) {
      const int p = (self + q) % world;                 // start at self, spread the peers
      float f[8];
      load8<GradT>(reinterpret_cast<const GradT*>(grads.p[p]) + lo + i * 8, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
    float4 o0, o1;
    o0.x = acc[0] * scale; o0.y = acc[1] * scale; o0.z = acc[2] * scale; o0.w = acc[3] * scale;
    o1.x = acc[4] * scale; o1.y = acc[5] * scale; o1.z = acc[6] * scale; o1.w = acc[7] * scale;
    reinterpret_cast<float4*>(red + i * 8)[0] = o0;
    reinterpret_cast<float4*>(red + i * 8)[1] = o1;
    ss += o0.x * o0.x + o0.y * o0.y + o0.z * o0.z + o0.w * o0.w + o1.x * o1.x + o1.y * o1.y + o1.z * o1.z + o1.w * o1.w;
  }
  ss = warp_sum(ss);
  __shared__ float redsm[8];
  if ((threadIdx.x & 31) == 0) redsm[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0 && sumsq) {
    float t = 0.f;
    for (int i = 0; i < 8; ++i) t += redsm[i];
    atomicAdd(sumsq, t);
  }
}

template <typename OutT>
__global__ void __launch_bounds__(256) adamw_push_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                                                         const float* __restrict__ red, const uint8_t* __restrict__ wd_mask,
                                                         const float* __restrict__ clip, PeerPtrsMut params, int world,
                                                         long long lo, long long n, float lr, float b1, float b2, float eps,
                                                         float wd, float inv_bc1, float inv_bc2, const int* __restrict__ err) {
  if (err && *reinterpret_cast<const volatile int*>(err) != 0) return;      // see reduce_shard_kernel: master, moments and peers stay untouched
  const float cs = clip ? *clip : 1.f;
  const long long nv = n / 8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv; i += (long long)gridDim.x * blockDim.x) {
    float out[8];
    const uint2 wm = *reinterpret_cast<const uint2*>(wd_mask + i * 8);
    const uint8_t* wmb = reinterpret_cast<const uint8_t*>(&wm);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const long long e = i * 8 + h * 4;
      float4 g4 = *reinterpret_cast<const float4*>(red + e);
      float4 m4 = *reinterpret_cast<const float4*>(m + e);
      float4 v4 = *reinterpret_cast<const float4*>(v + e);
      float4 p4 = *reinterpret_cast<const float4*>(master + e);
      float* gg = reinterpret_cast<float*>(&g4); float* mm = reinterpret_cast<float*>(&m4);
      float* vv = reinterpret_cast<float*>(&v4); float* pp = reinterpret_cast<float*>(&p4);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float gi = gg[j] * cs;
        mm[j] = b1 * mm[j] + (1.f - b1) * gi;
        vv[j] = b2 * vv[j] + (1.f - b2) * gi * gi;
        float upd = (mm[j] * inv_bc1) / (sqrtf(vv[j] * inv_bc2) + eps);
        if (wmb[h * 4 + j]) upd += wd * pp[j];
        pp[j] -= lr * upd;
        out[h * 4 + j] = pp[j];
      }
      *reinterpret_cast<float4*>(m + e) = m4;
      *reinterpret_cast<float4*>(v + e) = v4;
      *reinterpret_cast<float4*>(master + e) = p4;
    }
    if constexpr (sizeof(OutT) == 2) {
      uint4 o;
      o.x = pack_bf16(out[0], out[1]); o.y = pack_bf16(out[2], out[3]);
      o.z = pack_bf16(out[4], out[5]); o.w = pack_bf16(out[6], out[7]);
      for (int p = 0; p < world; ++p)
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(params.p[p]) + lo + i * 8) = o;
    } else {
      const float4 o0 = make_float4(out[0], out[1], out[2], out[3]), o1 = make_float4(out[4], out[5], out[6], out[7]);
      for (int p = 0; p < world; ++p) {
        float4* d = reinterpret_cast<float4*>(reinterpret_cast<float*>(params.p[p]) + lo + i * 8);
        d[0] = o0;
        d[1] = o1;
      }
    }
  }
}

}  // namespace cm

using namespace cm;

// grad_ptrs / param_ptrs: host arrays of `world` device pointers (peer-mapped buffer bases).
extern "C" int cm_reduce_shard(const void* const* grad_ptrs, int world, int self, long long lo, long long n, float scale,
                               float* red, float* sumsq, int grad_kind, const int* err, cudaStream_t s) {
  if (n <= 0) return 0;
  if (world > MAX_PEERS || (n % 8) || (lo % 8)) return -10;
  PeerPtrs pp;
  for (int i = 0; i < world; ++i) pp.p[i] = grad_ptrs[i];
  long long blocks = (n / 8 + 255) / 256;
  int grid = (int)(blocks < (long long)sm_count() * 8 ? blocks : (long long)sm_count() * 8);
  if (grad_kind == 0) reduce_shard_kernel<float><<<grid, 256, 0, s>>>(pp, world, self, lo, n, scale, red, sumsq, err);
  else reduce_shard_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(pp, world, self, lo, n, scale, red, sumsq, err);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int cm_adamw_push(float* master, float* m, float* v, const float* red, const uint8_t* wd_mask, const float* clip,
                             void* const* param_ptrs, int world, long long lo, long long n, float lr, float b1, float b2,
                             float eps, float wd, float bc1, float bc2, int out_kind, const int* err, cudaStream_t s) {
  if (n <= 0) return 0;
  if (world > MAX_PEERS || (n % 8) || (lo % 8)) return -10;
  PeerPtrsMut pp;
  for (int i = 0; i < world; ++i) pp.p[i] = param_ptrs[i];
  long long blocks = (n / 8 + 255) / 256;
  int grid = (int)(blocks < (long long)sm_count() * 8 ? blocks : (long long)sm_count() * 8);
  if (out_kind == 1)
    adamw_push_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(master, m, v, red, wd_mask, clip, pp, world, lo, n, lr, b1, b2, eps, wd, 1.f / bc1, 1.f / bc2, err);
  else
    adamw_push_kernel<float><<<grid, 256, 0, s>>>(master, m, v, red, wd_mask, clip, pp, world, lo, n, lr, b1, b2, eps, wd, 1.f / bc1, 1.f / bc2, err);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
