// Quantised (int8, 256-element blocks, fp32 absmax) Muon momentum.
//
//   update:  m = beta * q * absmax/127 + (1 - beta) * g ;  absmax' = max|m| ;  q' = round_half_away(m * 127/absmax')
//            g <- m (in place: the gradient buffer becomes the Newton-Schulz input) ;  sumsq[block] = sum m^2,
//            optionally accumulated into a normalisation group (atomicAdd) so fused-QKV slices normalise separately
//   scale:   g *= rsqrt(max(group_sumsq, eps^2))
//   carrier: q8 momentum -> MXFP8 (E4M3 payload + E8M0 scale per 32 values) for a block-scaled Newton-Schulz GEMM
// One warp per 256-element block (8 elements per lane, warp-shuffle reductions); a flat segment table lets one
// launch cover every tensor of a parameter group.
// Same arithmetic as the reference's kernels (cppmega/megatron/cuda_ext/quantized_muon_momentum.cu:152-406; scale
// byte = clamp(ceil(log2(amax/448)) + 127, 1, 254) at :75-91).
#include "common.cuh"

namespace cm {

constexpr int QB = 256;

template <typename GradT>
__global__ void __launch_bounds__(256) qmuon_update_kernel(int8_t* __restrict__ q, float* __restrict__ absmax, GradT* __restrict__ g,
                                                           float* __restrict__ block_sumsq, float* __restrict__ group_sumsq,
                                                           const int* __restrict__ block_group, long long n, long long nblocks,
                                                           float beta) {
  const int lane = threadIdx.x & 31;
  const long long wpb = blockDim.x >> 5;
  for (long long blk = blockIdx.x * wpb + (threadIdx.x >> 5); blk < nblocks; blk += (long long)gridDim.x * wpb) {
    const long long base = blk * QB + lane * 8;
    const float sc = absmax[blk] * (1.f / 127.f);
    float m[8];
    float am = 0.f, ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const long long i = base + j;
      float v = 0.f;
      if (i < n) v = beta * float(q[i]) * sc + (1.f - beta) * float(g[i]);
      m[j] = v;
      am = fmaxf(am, fabsf(v));
      ss += v * v;
    }
    am = warp_max(am);
    ss = warp_sum(ss);
    const float inv = am > 0.f ? 127.f / am : 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const long long i = base + j;
      if (i < n) {
        const float r = m[j] * inv;
        float rr = floorf(fabsf(r) + 0.5f);
        rr = fminf(rr, 127.f);
        q[i] = (int8_t)(r < 0.f ? -rr : rr);
        g[i] = GradT(m[j]);
      }
    }
    if (lane == 0) {
      absmax[blk] = am;
      if (block_sumsq) block_sumsq[blk] = ss;
      if (group_sumsq && block_group) atomicAdd(group_sumsq + block_group[blk], ss);
    }
  }
}

template <typename GradT>
__global__ void __launch_bounds__(256) qmuon_scale_kernel(GradT* __restrict__ g, const float* __restrict__ group_sumsq,
                                                          const int* __restrict__ block_group, long long n, float eps) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float s = group_sumsq[block_group[i / QB]];
    g[i] = GradT(float(g[i]) * rsqrtf(fmaxf(s, eps * eps)));
  }
}

__device__ __forceinline__ uint8_t e8m0_from_amax(float amax) {
  if (!(amax > 0.f)) return 127;
  int e = (int)ceilf(log2f(amax * (1.f / 448.f))) + 127;
  e = e < 1 ? 1 : (e > 254 ? 254 : e);
  return (uint8_t)e;
}

__device__ __forceinline__ uint8_t to_e4m3(float x) {
  // round-to-nearest-even conversion through the hardware cvt
  unsigned short r;
  asm("{\n.reg .b16 t;\ncvt.rn.satfinite.e4m3x2.f32 t, %1, %2;\nmov.b16 %0, t;\n}" : "=h"(r) : "f"(0.f), "f"(x));
  return (uint8_t)(r & 0xff);
}

// one warp per 32-value block of a [rows, cols] matrix (cols % 32 == 0)
__global__ void __launch_bounds__(256) qmuon_emit_mxfp8_kernel(const int8_t* __restrict__ q, const float* __restrict__ absmax,
                                                               const float* __restrict__ inv_norm, uint8_t* __restrict__ payload,
                                                               uint8_t* __restrict__ scales, long long n) {
  const int lane = threadIdx.x & 31;
  const long long wpb = blockDim.x >> 5;
  const long long nb = n / 32;
  const float nrm = inv_norm ? *inv_norm : 1.f;
  for (long long b = blockIdx.x * wpb + (threadIdx.x >> 5); b < nb; b += (long long)gridDim.x * wpb) {
    const long long i = b * 32 + lane;
    const float v = float(q[i]) * absmax[i / QB] * (1.f / 127.f) * nrm;
    const float am = warp_max(fabsf(v));
    const uint8_t sb = e8m0_from_amax(am);
    payload[i] = to_e4m3(v * exp2f(127.f - float(sb)));
    if (lane == 0) scales[b] = sb;
  }
}

}  // namespace cm

using namespace cm;

// grad_kind: 0 fp32, 1 bf16.  block_sumsq / group_sumsq / block_group may be null.
extern "C" int cm_qmuon_update(void* q, float* absmax, void* g, float* block_sumsq, float* group_sumsq,
                               const int* block_group, long long n, float beta, int grad_kind, cudaStream_t s) {
  if (n <= 0) return 0;
  const long long nblocks = (n + QB - 1) / QB;
  long long blocks = (nblocks + 7) / 8;
  int grid = (int)(blocks < (long long)sm_count() * 8 ? blocks : (long long)sm_count() * 8);
  if (grad_kind == 0)
    qmuon_update_kernel<float><<<grid, 256, 0, s>>>((int8_t*)q, absmax, (float*)g, block_sumsq, group_sumsq, block_group, n, nblocks, beta);
  else
    qmuon_update_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((int8_t*)q, absmax, (__nv_bfloat16*)g, block_sumsq, group_sumsq, block_group, n, nblocks, beta);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int cm_qmuon_scale(void* g, const float* group_sumsq, const int* block_group, long long n, float eps, int grad_kind,
                              cudaStream_t s) {
  if (n <= 0) return 0;
  long long blocks = (n + 255) / 256;
  int grid = (int)(blocks < (long long)sm_count() * 8 ? blocks : (long long)sm_count() * 8);
  if (grad_kind == 0) qmuon_scale_kernel<float><<<grid, 256, 0, s>>>((float*)g, group_sumsq, block_group, n, eps);
  else qmuon_scale_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((__nv_bfloat16*)g, group_sumsq, block_group, n, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int cm_qmuon_emit_mxfp8(const void* q, const float* absmax, const float* inv_norm, void* payload, void* scales,
                                   long long n, cudaStream_t s) {
  if (n <= 0) return 0;
  if (n % 32) return -10;
  long long blocks = (n / 32 + 7) / 8;
  int grid = (int)(blocks < (long long)sm_count() * 8 ? blocks : (long long)sm_count() * 8);
  qmuon_emit_mxfp8_kernel<<<grid, 256, 0, s>>>((const int8_t*)q, absmax, inv_norm, (uint8_t*)payload, (uint8_t*)scales, n);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// ---------------------------------------------------------------------------------------------
// AdamW with 8-bit state ("adam8bit"): the scalar / embedding optimizer beside Muon in the reference's small-memory
// lanes (cppmega/recipes/run_profiles.py:181 `muon_scalar_optimizer`).  Per 256-element block, with am_m = max |m| and
// am_v = max sqrt(v) kept in fp32, the codes are companded so that small entries of a block keep relative precision:
//   m8 = round(127 sign(m) sqrt(|m| / am_m))        v8 = round(255 sqrt(sqrt(v) / am_v))
//   m = b1 deq(m8) + (1-b1) g ;  v = b2 deq(v8)^2 + (1-b2) g^2 ;  p -= lr (m^/(sqrt(v^)+eps) + wd p) ;  requantise.
// One warp per block, 8 elements per lane.  `active` (optional, one byte per element): 0 = leave the element alone
// (ranges another optimizer owns).  `gate` as in cm_adamw_gated.
// ---------------------------------------------------------------------------------------------
namespace cm {

template <typename GradT, typename OutT>
__global__ void __launch_bounds__(256) adam8bit_kernel(float* __restrict__ master, int8_t* __restrict__ m8, uint8_t* __restrict__ v8,
                                                       float* __restrict__ am_m, float* __restrict__ am_v, const GradT* __restrict__ g,
                                                       OutT* __restrict__ out, const uint8_t* __restrict__ wd_mask,
                                                       const uint8_t* __restrict__ active, const float* __restrict__ clip,
                                                       long long n, long long nblocks, float lr, float b1, float b2, float eps,
                                                       float wd, float inv_bc1, float inv_bc2, const int* __restrict__ gate) {
  if (gate && *reinterpret_cast<const volatile int*>(gate) != 0) return;
  const float cs = clip ? *clip : 1.f;
  const int lane = threadIdx.x & 31;
  const long long wpb = blockDim.x >> 5;
  for (long long blk = blockIdx.x * wpb + (threadIdx.x >> 5); blk < nblocks; blk += (long long)gridDim.x * wpb) {
    const long long base = blk * QB + lane * 8;
    const float sm = am_m[blk] * (1.f / (127.f * 127.f)), sv = am_v[blk] * (1.f / (255.f * 255.f));
    float m[8], r[8];
    bool on[8];
    float mx_m = 0.f, mx_r = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const long long i = base + j;
      m[j] = r[j] = 0.f;
      on[j] = false;
      if (i < n) {
        const float qm = float(m8[i]), qv = float(v8[i]);
        const float m_old = qm * fabsf(qm) * sm, r_old = qv * qv * sv;
        on[j] = !active || active[i];
        if (on[j]) {
          const float gi = float(g[i]) * cs;
          m[j] = b1 * m_old + (1.f - b1) * gi;
          const float v = b2 * r_old * r_old + (1.f - b2) * gi * gi;
          r[j] = sqrtf(v);
          float p = master[i];
          float upd = (m[j] * inv_bc1) / (sqrtf(v * inv_bc2) + eps);
          if (wd_mask[i]) upd += wd * p;
          p -= lr * upd;
          master[i] = p;
          out[i] = OutT(p);
        } else {
          m[j] = m_old;
          r[j] = r_old;
        }
        mx_m = fmaxf(mx_m, fabsf(m[j]));
        mx_r = fmaxf(mx_r, r[j]);
      }
    }
    mx_m = warp_max(mx_m);
    mx_r = warp_max(mx_r);
    const float im = mx_m > 0.f ? 1.f / mx_m : 0.f, ir = mx_r > 0.f ? 1.f / mx_r : 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const long long i = base + j;
      if (i < n) {
        const float qa = fminf(floorf(127.f * sqrtf(fabsf(m[j]) * im) + 0.5f), 127.f);
        m8[i] = (int8_t)(m[j] < 0.f ? -qa : qa);
        v8[i] = (uint8_t)fminf(floorf(255.f * sqrtf(r[j] * ir) + 0.5f), 255.f);
      }
    }
    if (lane == 0) {
      am_m[blk] = mx_m;
      am_v[blk] = mx_r;
    }
  }
}

}  // namespace cm

// master fp32 [n]; m8 int8 [n], v8 uint8 [n]; am_m, am_v fp32 [ceil(n/256)]; g fp32 (grad_kind 0) or bf16 (1); out bf16
// (out_kind 1) or fp32 (0); wd_mask uint8 [n]; active uint8 [n] or null; clip device scalar or null; gate device word or null
extern "C" int cm_adam8bit(float* master, int8_t* m8, uint8_t* v8, float* am_m, float* am_v, const void* g, void* out,
                           const uint8_t* wd_mask, const uint8_t* active, const float* clip, long long n, float lr, float b1,
                           float b2, float eps, float wd, float bc1, float bc2, int grad_kind, int out_kind, const int* gate,
                           cudaStream_t s) {
  if (n <= 0) return 0;
  const long long nblocks = (n + cm::QB - 1) / cm::QB;
  long long blocks = (nblocks + 7) / 8;
  const int grid = (int)(blocks < (long long)cm::sm_count() * 8 ? blocks : (long long)cm::sm_count() * 8);
  const float i1 = 1.f / bc1, i2 = 1.f / bc2;
#define CM_A8(GT, OT)                                                                                                      \
  cm::adam8bit_kernel<GT, OT><<<grid, 256, 0, s>>>(master, m8, v8, am_m, am_v, (const GT*)g, (OT*)out, wd_mask, active, clip, n, \
                                                   nblocks, lr, b1, b2, eps, wd, i1, i2, gate)
  if (grad_kind == 0 && out_kind == 1) CM_A8(float, __nv_bfloat16);
  else if (grad_kind == 1 && out_kind == 1) CM_A8(__nv_bfloat16, __nv_bfloat16);
  else if (grad_kind == 0 && out_kind == 0) CM_A8(float, float);
  else CM_A8(__nv_bfloat16, float);
#undef CM_A8
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
