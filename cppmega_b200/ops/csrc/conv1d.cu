// Depthwise causal conv1d over the sequence fused with SiLU, channels-last, forward and backward:
//
//   pre[b, s, c] = bias[c] + sum_{j < k} w[c, j] * x[b, s - (k-1) + j, c]        (x = 0 before the sequence start)
//   y[b, s, c]   = silu(pre[b, s, c])
//
// x is read in place from a wider projection (token stride `ldx` elements, channels contiguous), so neither the
// [B,S,C] -> [B,C,S] transposes nor the slice copy of the library convolution exist.  One thread owns 8 adjacent channels
// (one 16-byte vector) and walks a segment of the sequence with the last k-1 inputs in registers: x is read once.
// Backward: kernel 1 recomputes pre, forms g = dy * silu'(pre), writes it, and reduces dw / db per channel over its
// segment (fp32 atomics, one per channel and segment); kernel 2 is the transposed correlation dx[s] = sum_j w[j] g[s+k-1-j].
// Replaces the nn.Conv1d + SiLU of the M2RNN and SSD mixers (reference: cppmega/megatron/m2rnn_spec.py conv path and
// mamba_ssm's causal_conv1d, which its Mamba mixers call).
#include "common.cuh"

namespace cm {
namespace conv {

constexpr int KMAX = 8;
constexpr int SEG = 64;                 // tokens per thread segment

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 t = __bfloat1622float2(b[j]);
    f[2 * j] = t.x;
    f[2 * j + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 o;
  o.x = pack_bf16(f[0], f[1]);
  o.y = pack_bf16(f[2], f[3]);
  o.z = pack_bf16(f[4], f[5]);
  o.w = pack_bf16(f[6], f[7]);
  return o;
}
__device__ __forceinline__ float silu_f(float z) { return z / (1.f + __expf(-z)); }
__device__ __forceinline__ float dsilu_f(float z) {
  const float sg = 1.f / (1.f + __expf(-z));
  return sg * (1.f + z * (1.f - sg));
}

struct Args {
  const __nv_bfloat16* x;      // [B, S, C] with token stride ldx
  const __nv_bfloat16* w;      // [C, k]
  const __nv_bfloat16* bias;   // [C] or null
  long long ldx;
  int B, S, C, k, nseg;
};

// grid: (ceil(C/8 / 128), B * nseg); thread = one channel vector, one segment
template <int K>
__global__ void __launch_bounds__(128) conv_silu_fwd_kernel(const Args a, __nv_bfloat16* __restrict__ y) {
  const int cv = blockIdx.x * blockDim.x + threadIdx.x;
  if (cv * 8 >= a.C) return;
  const int c0 = cv * 8;
  const int b = blockIdx.y / a.nseg, seg = blockIdx.y % a.nseg;
  const int s0 = seg * SEG, s1 = min(a.S, s0 + SEG);
  float w[K][8], bs[8], win[K][8];
#pragma unroll
  for (int j = 0; j < K; ++j)
#pragma unroll
    for (int v = 0; v < 8; ++v) w[j][v] = (j < K) ? __bfloat162float(a.w[(size_t)(c0 + v) * K + j]) : 0.f;
#pragma unroll
  for (int v = 0; v < 8; ++v) bs[v] = a.bias ? __bfloat162float(a.bias[c0 + v]) : 0.f;
  const __nv_bfloat16* xb = a.x + (size_t)b * a.S * a.ldx + c0;
  // window slot j holds x[s - (k-1) + j]; prime it with the k-1 tokens before the segment
#pragma unroll
  for (int j = 0; j < K; ++j) {
    const int s = s0 - (K - 1) + j;
    if (j < K - 1 && s >= 0) load8(xb + (size_t)s * a.ldx, win[j]);
    else
#pragma unroll
      for (int v = 0; v < 8; ++v) win[j][v] = 0.f;
  }
  for (int s = s0; s < s1; ++s) {
    float cur[8];
    load8(xb + (size_t)s * a.ldx, cur);
    float acc[8];
#pragma unroll
    for (int v = 0; v < 8; ++v) acc[v] = bs[v];
#pragma unroll
    for (int j = 0; j < K; ++j) {
      if (j < K - 1) {
#pragma unroll
        for (int v = 0; v < 8; ++v) acc[v] += w[j][v] * win[j][v];
      }
    }
#pragma unroll
    for (int j = 0; j < K; ++j)
      if (j == K - 1) {
#pragma unroll
        for (int v = 0; v < 8; ++v) acc[v] += w[j][v] * cur[v];
      }
    float o[8];
#pragma unroll
    for (int v = 0; v < 8; ++v) o[v] = silu_f(acc[v]);
    *reinterpret_cast<uint4*>(y + ((size_t)b * a.S + s) * a.C + c0) = pack8(o);
    // slide: slot j <- slot j+1, last used slot <- cur
#pragma unroll
    for (int j = 0; j < K - 1; ++j) {
      if (j < K - 2) {
#pragma unroll
        for (int v = 0; v < 8; ++v) win[j][v] = win[j + 1][v];
      } else if (j == K - 2) {
#pragma unroll
        for (int v = 0; v < 8; ++v) win[j][v] = cur[v];
      }
    }
  }
}

// g = dy * silu'(pre) written to `g` [B,S,C]; dw [C,k] / db [C] fp32 accumulated with atomics (zeroed by the caller)
template <int K>
__global__ void __launch_bounds__(128) conv_silu_bwd_g_kernel(const Args a, const __nv_bfloat16* __restrict__ dy,
                                                              __nv_bfloat16* __restrict__ g, float* __restrict__ dw,
                                                              float* __restrict__ db) {
  const int cv = blockIdx.x * blockDim.x + threadIdx.x;
  if (cv * 8 >= a.C) return;
  const int c0 = cv * 8;
  const int b = blockIdx.y / a.nseg, seg = blockIdx.y % a.nseg;
  const int s0 = seg * SEG, s1 = min(a.S, s0 + SEG);
  float w[K][8], bs[8], win[K][8], aw[K][8], ab[8];
#pragma unroll
  for (int j = 0; j < K; ++j)
#pragma unroll
    for (int v = 0; v < 8; ++v) {
      w[j][v] = (j < K) ? __bfloat162float(a.w[(size_t)(c0 + v) * K + j]) : 0.f;
      aw[j][v] = 0.f;
    }
#pragma unroll
  for (int v = 0; v < 8; ++v) { bs[v] = a.bias ? __bfloat162float(a.bias[c0 + v]) : 0.f; ab[v] = 0.f; }
  const __nv_bfloat16* xb = a.x + (size_t)b * a.S * a.ldx + c0;
#pragma unroll
  for (int j = 0; j < K; ++j) {
    const int s = s0 - (K - 1) + j;
    if (j < K - 1 && s >= 0) load8(xb + (size_t)s * a.ldx, win[j]);
    else
#pragma unroll
      for (int v = 0; v < 8; ++v) win[j][v] = 0.f;
  }
  for (int s = s0; s < s1; ++s) {
    float cur[8], dyv[8];
    load8(xb + (size_t)s * a.ldx, cur);
    load8(dy + ((size_t)b * a.S + s) * a.C + c0, dyv);
#pragma unroll
    for (int j = 0; j < K; ++j)
      if (j == K - 1) {
#pragma unroll
        for (int v = 0; v < 8; ++v) win[j][v] = cur[v];
      }
    float gv[8];
#pragma unroll
    for (int v = 0; v < 8; ++v) {
      float acc = bs[v];
#pragma unroll
      for (int j = 0; j < K; ++j)
        if (j < K) acc += w[j][v] * win[j][v];
      gv[v] = dyv[v] * dsilu_f(acc);
      ab[v] += gv[v];
    }
#pragma unroll
    for (int j = 0; j < K; ++j)
      if (j < K) {
#pragma unroll
        for (int v = 0; v < 8; ++v) aw[j][v] += gv[v] * win[j][v];
      }
    *reinterpret_cast<uint4*>(g + ((size_t)b * a.S + s) * a.C + c0) = pack8(gv);
#pragma unroll
    for (int j = 0; j < K - 1; ++j)
      if (j < K - 1) {
#pragma unroll
        for (int v = 0; v < 8; ++v) win[j][v] = win[j + 1][v];
      }
  }
#pragma unroll
  for (int v = 0; v < 8; ++v) {
    atomicAdd(db + c0 + v, ab[v]);
#pragma unroll
    for (int j = 0; j < K; ++j)
      if (j < K) atomicAdd(dw + (size_t)(c0 + v) * K + j, aw[j][v]);
  }
}

// dx[b, s, c] = sum_j w[c, j] * g[b, s + (k-1) - j, c]   (g = 0 past the sequence end); dx has token stride lddx
template <int K>
__global__ void __launch_bounds__(128) conv_silu_bwd_dx_kernel(const Args a, const __nv_bfloat16* __restrict__ g,
                                                               __nv_bfloat16* __restrict__ dx, long long lddx) {
  const int cv = blockIdx.x * blockDim.x + threadIdx.x;
  if (cv * 8 >= a.C) return;
  const int c0 = cv * 8;
  const int b = blockIdx.y / a.nseg, seg = blockIdx.y % a.nseg;
  const int s0 = seg * SEG, s1 = min(a.S, s0 + SEG);
  float w[K][8];
#pragma unroll
  for (int j = 0; j < K; ++j)
#pragma unroll
    for (int v = 0; v < 8; ++v) w[j][v] = (j < K) ? __bfloat162float(a.w[(size_t)(c0 + v) * K + j]) : 0.f;
  const __nv_bfloat16* gb = g + (size_t)b * a.S * a.C + c0;
  for (int s = s0; s < s1; ++s) {
    float acc[8];
#pragma unroll
    for (int v = 0; v < 8; ++v) acc[v] = 0.f;
#pragma unroll
    for (int j = 0; j < K; ++j) {
      const int t = s + (K - 1) - j;
      if (j < K && t < a.S) {
        float gv[8];
        load8(gb + (size_t)t * a.C, gv);          // neighbouring tokens: served by L1 / L2
#pragma unroll
        for (int v = 0; v < 8; ++v) acc[v] += w[j][v] * gv[v];
      }
    }
    *reinterpret_cast<uint4*>(dx + ((size_t)b * a.S + s) * lddx + c0) = pack8(acc);
  }
}

static dim3 grid_of(const Args& a) { return dim3((unsigned)((a.C / 8 + 127) / 128), (unsigned)(a.B * a.nseg)); }

}  // namespace conv
}  // namespace cm

using namespace cm;
using namespace cm::conv;

static int check(const void* x, long long ldx, int C, int k) {
  if (C % 8 || ldx % 8 || (reinterpret_cast<uintptr_t>(x) & 15)) return -10;
  if (k < 1 || k > KMAX) return -10;
  return 0;
}

// x [B,S,C] bf16 (token stride ldx), w [C,k] bf16, bias [C] bf16 or null -> y [B,S,C] bf16 packed
extern "C" int cm_causal_conv1d_silu_fwd(const void* x, const void* w, const void* bias, void* y, int B, int S, int C, int k,
                                         long long ldx, cudaStream_t s) {
  if (B <= 0 || S <= 0 || C <= 0) return 0;
  if (int rc = check(x, ldx, C, k)) return rc;
  Args a{(const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const __nv_bfloat16*)bias, ldx, B, S, C, k, (S + SEG - 1) / SEG};
  switch (k) {
#define CM_CONV_FWD(KK) case KK: conv_silu_fwd_kernel<KK><<<grid_of(a), 128, 0, s>>>(a, (__nv_bfloat16*)y); break;
    CM_CONV_FWD(1) CM_CONV_FWD(2) CM_CONV_FWD(3) CM_CONV_FWD(4) CM_CONV_FWD(5) CM_CONV_FWD(6) CM_CONV_FWD(7) CM_CONV_FWD(8)
#undef CM_CONV_FWD
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// dy [B,S,C] packed; g scratch [B,S,C] bf16; dx [B,S,C] with token stride lddx; dw [C,k], db [C] fp32 ZEROED by the caller
extern "C" int cm_causal_conv1d_silu_bwd(const void* x, const void* w, const void* bias, const void* dy, void* g, void* dx,
                                         float* dw, float* db, int B, int S, int C, int k, long long ldx, long long lddx,
                                         cudaStream_t s) {
  if (B <= 0 || S <= 0 || C <= 0) return 0;
  if (int rc = check(x, ldx, C, k)) return rc;
  if (lddx % 8 || (reinterpret_cast<uintptr_t>(dx) & 15) || (reinterpret_cast<uintptr_t>(dy) & 15)) return -10;
  Args a{(const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const __nv_bfloat16*)bias, ldx, B, S, C, k, (S + SEG - 1) / SEG};
  switch (k) {
#define CM_CONV_BWD(KK)                                                                                             \
  case KK:                                                                                                          \
    conv_silu_bwd_g_kernel<KK><<<grid_of(a), 128, 0, s>>>(a, (const __nv_bfloat16*)dy, (__nv_bfloat16*)g, dw, db);  \
    conv_silu_bwd_dx_kernel<KK><<<grid_of(a), 128, 0, s>>>(a, (const __nv_bfloat16*)g, (__nv_bfloat16*)dx, lddx);   \
    break;
    CM_CONV_BWD(1) CM_CONV_BWD(2) CM_CONV_BWD(3) CM_CONV_BWD(4) CM_CONV_BWD(5) CM_CONV_BWD(6) CM_CONV_BWD(7) CM_CONV_BWD(8)
#undef CM_CONV_BWD
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
