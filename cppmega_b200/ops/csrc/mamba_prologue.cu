// Cumulative rotary angles of the Mamba3 mixer and their backward.
//
//   out[b,t,h,a] = sum_{s<=t} raw[b,s,a] * dt[b,h,s]                      (fp32, a < A <= 32)
//
// The reference builds this with a broadcast multiply and a sequence cumsum in PyTorch
// (cppmega/megatron/noconv_mamba_mixer.py:326-333), i.e. three passes over a [B,S,H,A] fp32 tensor forward and
// five backward.  Here: one pass forward (a warp owns a (b, h, sequence segment); lanes are the angles, so every
// store is one 128-byte line) and two passes backward (suffix sums, then the two reductions over heads / angles).
#include "common.cuh"

namespace cm {

constexpr int ANG_SEG = 512;

// Forward prefix sums in two passes over segments of ANG_FSEG tokens, one warp per (batch, head, segment), lane = angle:
//   pass 1 (WRITE = false)  segment totals -> segsum[b, h, seg, a];
//   pass 2 (WRITE = true)   start from the totals of the earlier segments and write the running sums.
// The dt of a segment sits in registers (lane l holds tokens l, l + 32, ...) and reaches the serial chain by shuffle,
// the raw angles of 32 tokens are requested together, so the chain of 256 dependent FMAs never waits on memory.
constexpr int ANG_FSEG = 256;

template <bool WRITE>
__global__ void __launch_bounds__(128) angle_cumsum_fwd_kernel(const float* __restrict__ raw, const float* __restrict__ dt,
                                                               long long dsb, long long dsh, long long dss,
                                                               float* __restrict__ out, float* __restrict__ segsum, int B, int S, int H,
                                                               int A, int nseg) {
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  const long long BH = (long long)B * H;
  if (w >= BH * nseg) return;
  const int seg = (int)(w / BH);                 // neighbouring warps: neighbouring heads, the same dt cache lines
  const int bh = (int)(w % BH);
  const int b = bh / H, h = bh % H;
  const bool on = lane < A;
  const int t0 = seg * ANG_FSEG;
  const float* rp = raw + ((size_t)b * S + t0) * A + (on ? lane : 0);
  const float* dp = dt + b * dsb + h * dsh + (long long)t0 * dss;
  float dreg[ANG_FSEG / 32];
#pragma unroll
  for (int k = 0; k < ANG_FSEG / 32; ++k) {
    const int t = t0 + k * 32 + lane;
    dreg[k] = t < S ? dp[(long long)(k * 32 + lane) * dss] : 0.f;
  }
  float acc = 0.f;
  if (WRITE && on) {
    const float* sp = segsum + ((size_t)bh * nseg) * A + lane;
    for (int s2 = 0; s2 < seg; ++s2) acc += sp[(size_t)s2 * A];
  }
  float* op = out + (((size_t)b * S + t0) * H + h) * A + lane;
#pragma unroll 1
  for (int k = 0; k < ANG_FSEG / 32; ++k) {
    if (t0 + k * 32 >= S) break;
    float r[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) r[j] = (t0 + k * 32 + j < S) ? rp[(size_t)(k * 32 + j) * A] : 0.f;
    float dk = 0.f;
#pragma unroll
    for (int kk = 0; kk < ANG_FSEG / 32; ++kk) dk = (kk == k) ? dreg[kk] : dk;      // keeps dreg in registers
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      acc = fmaf(r[j], __shfl_sync(0xffffffffu, dk, j), acc);
      if (WRITE && on && t0 + k * 32 + j < S) op[(size_t)(k * 32 + j) * H * A] = acc;
    }
  }
  if (!WRITE && on) segsum[((size_t)bh * nseg + seg) * A + lane] = acc;
}

// segsum[b,h,seg,a] = sum over the segment of g[b,t,h,a]
__global__ void __launch_bounds__(128) angle_segsum_kernel(const float* __restrict__ g, float* __restrict__ segsum, int B, int S, int H,
                                                           int A, int nseg) {
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (w >= (long long)B * H * nseg) return;
  const long long BH = (long long)B * H;
  const int seg = (int)(w / BH);                 // the warps of a CTA take neighbouring heads: neighbouring 128-byte lines
  const int bh = (int)(w % BH);
  const int b = bh / H, h = bh % H;
  if (lane >= A) return;
  const float* gp = g + ((size_t)b * S * H + h) * A + lane;
  const int t0 = seg * ANG_SEG, t1 = min(S, t0 + ANG_SEG);
  float acc = 0.f;
#pragma unroll 16
  for (int t = t0; t < t1; ++t) acc += gp[(size_t)t * H * A];
  segsum[((size_t)bh * nseg + seg) * A + lane] = acc;
}

// suffix sums in place: g[b,t,h,a] <- sum_{s>=t} g[b,s,h,a]
__global__ void __launch_bounds__(128) angle_suffix_kernel(float* __restrict__ g, const float* __restrict__ segsum, int B, int S, int H,
                                                           int A, int nseg) {
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (w >= (long long)B * H * nseg) return;
  const long long BH = (long long)B * H;
  const int seg = (int)(w / BH);
  const int bh = (int)(w % BH);
  const int b = bh / H, h = bh % H;
  if (lane >= A) return;
  float acc = 0.f;
  for (int s2 = nseg - 1; s2 > seg; --s2) acc += segsum[((size_t)bh * nseg + s2) * A + lane];
  float* gp = g + ((size_t)b * S * H + h) * A + lane;
  const int t0 = seg * ANG_SEG, t1 = min(S, t0 + ANG_SEG);
  // 16 independent loads first, then the running sum and the stores: in a plain read-modify-write loop every load waits
  // behind the previous store to the same array
  const size_t st = (size_t)H * A;
  int t = t1 - 1;
  for (; t - 15 >= t0; t -= 16) {
    float v[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = gp[(size_t)(t - j) * st];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      acc += v[j];
      gp[(size_t)(t - j) * st] = acc;
    }
  }
  for (; t >= t0; --t) {
    acc += gp[(size_t)t * st];
    gp[(size_t)t * st] = acc;
  }
}

// Same reduction for A == 32 and S % 32 == 0, one block per 32 consecutive tokens, lane = token: a thread reads the 32
// angles of its (token, head) as one 128-byte run, so ddt needs no shuffle and is written 32 tokens at a time; draw is
// accumulated over a warp's heads in registers and summed over the 8 warps through shared memory.
__global__ void __launch_bounds__(256) angle_reduce32_kernel(const float* __restrict__ g, const float* __restrict__ raw,
                                                             const float* __restrict__ dt, long long dsb, long long dsh, long long dss,
                                                             float* __restrict__ draw, float* __restrict__ ddt, int B, int S, int H) {
  constexpr int A = 32;
  __shared__ float red[8][32][A + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long tile = blockIdx.x;                       // 32 tokens
  const int tiles_per_b = S / 32;
  const int b = (int)(tile / tiles_per_b);
  const int t = (int)(tile % tiles_per_b) * 32 + lane;
  const size_t tok = (size_t)b * S + t;
  float rv[A], acc[A];
  {
    const float4* rp = reinterpret_cast<const float4*>(raw + tok * A);
#pragma unroll
    for (int q = 0; q < A / 4; ++q) {
      const float4 v = rp[q];
      rv[4 * q] = v.x; rv[4 * q + 1] = v.y; rv[4 * q + 2] = v.z; rv[4 * q + 3] = v.w;
      acc[4 * q] = 0.f; acc[4 * q + 1] = 0.f; acc[4 * q + 2] = 0.f; acc[4 * q + 3] = 0.f;
    }
  }
  for (int h = warp; h < H; h += 8) {
    const float4* gp = reinterpret_cast<const float4*>(g + (tok * H + h) * A);
    const float d = dt[b * dsb + h * dsh + (long long)t * dss];
    float s = 0.f;
#pragma unroll
    for (int q = 0; q < A / 4; ++q) {
      const float4 v = gp[q];
      s += v.x * rv[4 * q] + v.y * rv[4 * q + 1] + v.z * rv[4 * q + 2] + v.w * rv[4 * q + 3];
      acc[4 * q] = fmaf(v.x, d, acc[4 * q]);
      acc[4 * q + 1] = fmaf(v.y, d, acc[4 * q + 1]);
      acc[4 * q + 2] = fmaf(v.z, d, acc[4 * q + 2]);
      acc[4 * q + 3] = fmaf(v.w, d, acc[4 * q + 3]);
    }
    ddt[((size_t)b * H + h) * S + t] = s;
  }
#pragma unroll
  for (int a = 0; a < A; ++a) red[warp][lane][a] = acc[a];
  __syncthreads();
  for (int e = threadIdx.x; e < 32 * A; e += 256) {
    const int tt = e / A, a = e % A;
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += red[w][tt][a];
    draw[((size_t)b * S + (tile % tiles_per_b) * 32 + tt) * A + a] = s;
  }
}

// one block per token: draw[b,t,a] = sum_h g*dt ; ddt[b,h,t] = sum_a g*raw     (g holds the suffix sums)
__global__ void __launch_bounds__(256) angle_reduce_kernel(const float* __restrict__ g, const float* __restrict__ raw,
                                                           const float* __restrict__ dt, long long dsb, long long dsh, long long dss,
                                                           float* __restrict__ draw, float* __restrict__ ddt, int B, int S, int H, int A) {
  __shared__ float red[8][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long tok = blockIdx.x;
  const int b = (int)(tok / S), t = (int)(tok % S);
  const bool on = lane < A;
  const float rv = on ? raw[tok * A + lane] : 0.f;
  const float* gp = g + (size_t)tok * H * A;
  float acc = 0.f;
  for (int h = warp; h < H; h += 8) {
    const float gv = on ? gp[(size_t)h * A + lane] : 0.f;
    acc = fmaf(gv, dt[b * dsb + h * dsh + t * dss], acc);
    const float s = warp_sum(gv * rv);
    if (lane == 0) ddt[((size_t)b * H + h) * S + t] = s;
  }
  red[warp][lane] = acc;
  __syncthreads();
  if (warp == 0 && on) {
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += red[i][lane];
    draw[tok * A + lane] = s;
  }
}

// Per-head operand gradients of the scan -> gradients of the group-shared operand and of the per-head bias:
//   dgrp[t, g, c]  = sum_{h in group g} dh[t, h, c]            (bf16 out)
//   dbias[h, c]   += sum_t dh[t, h, c]                          (fp32, atomically accumulated; caller zeroes)
// dh [T, H, C] bf16 with C = R * N columns.  One block covers TT tokens of one group; a thread owns two columns.
constexpr int HR_TT = 64;
template <int HPG>
__global__ void __launch_bounds__(256) head_reduce_kernel(const __nv_bfloat16* __restrict__ dh, __nv_bfloat16* __restrict__ dgrp,
                                                          float* __restrict__ dbias, long long T, int H, int C) {
  const int g = blockIdx.y, G = H / HPG;
  const long long t0 = (long long)blockIdx.x * HR_TT;
  const long long t1 = t0 + HR_TT < T ? t0 + HR_TT : T;
  for (int c2 = threadIdx.x; c2 < C / 2; c2 += blockDim.x) {
    float bx[HPG], by[HPG];
#pragma unroll
    for (int j = 0; j < HPG; ++j) { bx[j] = 0.f; by[j] = 0.f; }
    for (long long t = t0; t < t1; ++t) {
      const __nv_bfloat162* row = reinterpret_cast<const __nv_bfloat162*>(dh + ((size_t)t * H + (size_t)g * HPG) * C) + c2;
      float sx = 0.f, sy = 0.f;
#pragma unroll
      for (int j = 0; j < HPG; ++j) {
        const float2 v = __bfloat1622float2(row[(size_t)j * (C / 2)]);
        bx[j] += v.x; by[j] += v.y;
        sx += v.x; sy += v.y;
      }
      reinterpret_cast<__nv_bfloat162*>(dgrp + ((size_t)t * G + g) * C)[c2] = __floats2bfloat162_rn(sx, sy);
    }
#pragma unroll
    for (int j = 0; j < HPG; ++j) {
      float* d = dbias + ((size_t)g * HPG + j) * C + 2 * c2;
      atomicAdd(d, bx[j]);
      atomicAdd(d + 1, by[j]);
    }
  }
}

}  // namespace cm

using namespace cm;

extern "C" int cm_head_reduce(const void* dh, void* dgrp, float* dbias, long long T, int H, int G, int C, cudaStream_t s) {
  if (T <= 0) return 0;
  if (C % 2 || H % G) return -10;
  dim3 grid((unsigned)((T + HR_TT - 1) / HR_TT), G);
  const int hpg = H / G;
  auto a = (const __nv_bfloat16*)dh;
  auto o = (__nv_bfloat16*)dgrp;
  if (hpg == 16) head_reduce_kernel<16><<<grid, 256, 0, s>>>(a, o, dbias, T, H, C);
  else if (hpg == 8) head_reduce_kernel<8><<<grid, 256, 0, s>>>(a, o, dbias, T, H, C);
  else if (hpg == 4) head_reduce_kernel<4><<<grid, 256, 0, s>>>(a, o, dbias, T, H, C);
  else if (hpg == 2) head_reduce_kernel<2><<<grid, 256, 0, s>>>(a, o, dbias, T, H, C);
  else if (hpg == 1) head_reduce_kernel<1><<<grid, 256, 0, s>>>(a, o, dbias, T, H, C);
  else return -12;
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// raw [B,S,A] fp32 contiguous; dt addressed as dt[b*dsb + h*dsh + t*dss] (element strides); out [B,S,H,A] fp32.
// segsum: [B * H * ceil(S / 256) * A] fp32 scratch
extern "C" int cm_angle_cumsum_fwd(const float* raw, const float* dt, long long dsb, long long dsh, long long dss, float* out,
                                   float* segsum, int B, int S, int H, int A, cudaStream_t s) {
  if (B <= 0 || S <= 0 || H <= 0) return 0;
  if (A <= 0 || A > 32) return -10;
  const int nseg = (S + ANG_FSEG - 1) / ANG_FSEG;
  const long long warps = (long long)B * H * nseg;
  const unsigned grid = (unsigned)((warps + 3) / 4);
  if (nseg > 1) angle_cumsum_fwd_kernel<false><<<grid, 128, 0, s>>>(raw, dt, dsb, dsh, dss, out, segsum, B, S, H, A, nseg);
  angle_cumsum_fwd_kernel<true><<<grid, 128, 0, s>>>(raw, dt, dsb, dsh, dss, out, segsum, B, S, H, A, nseg);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// g [B,S,H,A] fp32: gradient of `out` on entry, overwritten with its suffix sums.  segsum: [B*H*nseg*A] fp32 scratch.
// draw [B,S,A] fp32, ddt [B,H,S] fp32 contiguous.
extern "C" int cm_angle_cumsum_bwd(float* g, const float* raw, const float* dt, long long dsb, long long dsh, long long dss,
                                   float* segsum, float* draw, float* ddt, int B, int S, int H, int A, cudaStream_t s) {
  if (B <= 0 || S <= 0 || H <= 0) return 0;
  if (A <= 0 || A > 32) return -10;
  const int nseg = (S + ANG_SEG - 1) / ANG_SEG;
  const long long warps = (long long)B * H * nseg;
  const unsigned grid = (unsigned)((warps + 3) / 4);
  angle_segsum_kernel<<<grid, 128, 0, s>>>(g, segsum, B, S, H, A, nseg);
  angle_suffix_kernel<<<grid, 128, 0, s>>>(g, segsum, B, S, H, A, nseg);
  if (A == 32 && S % 32 == 0)
    angle_reduce32_kernel<<<(unsigned)((long long)B * S / 32), 256, 0, s>>>(g, raw, dt, dsb, dsh, dss, draw, ddt, B, S, H);
  else
    angle_reduce_kernel<<<(unsigned)((long long)B * S), 256, 0, s>>>(g, raw, dt, dsb, dsh, dss, draw, ddt, B, S, H, A);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// ------------------------------------------------------------------------------------------
// Widening of the state dimension for the 128-wide scan kernels, several tensors in one launch.
//   split job:   in [rows, n] -> out [rows, w]:  out[:, 0:n/2] = in[:, 0:n/2], out[:, w/2 : w/2 + n/2] = in[:, n/2:n], rest 0
//                (each half of the state keeps its place at the start of the wider half, so the rotary pairs (i, n/2 + i)
//                 become (i, w/2 + i));
//   plain job:   out[:, 0:n] = in, rest 0 (the rotary angles).
// inverse = 1 runs the adjoint: in [rows, w] -> out [rows, n] (the gradient of the narrow tensor).
// ------------------------------------------------------------------------------------------
namespace cm {
constexpr int PAD_MAX_JOBS = 8;
struct PadJobs {
  const void* in[PAD_MAX_JOBS];
  void* out[PAD_MAX_JOBS];
  long long rows[PAD_MAX_JOBS];
  int n[PAD_MAX_JOBS], w[PAD_MAX_JOBS], elem[PAD_MAX_JOBS], split[PAD_MAX_JOBS];
  int count;
};

template <typename T>
__device__ __forceinline__ void pad_rows(const T* __restrict__ in, T* __restrict__ out, long long rows, int n, int w, bool split,
                                         bool inverse) {
  const int wide = inverse ? n : w;                      // columns of the tensor this launch writes
  const long long total = rows * wide;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / wide;
    const int c = (int)(i - r * wide);
    if (!inverse) {                                      // c indexes the wide row
      int src = -1;
      if (split) {
        if (c < n / 2) src = c;
        else if (c >= w / 2 && c < w / 2 + n / 2) src = c - w / 2 + n / 2;
      } else if (c < n) {
        src = c;
      }
      out[i] = src >= 0 ? in[r * n + src] : T(0);
    } else {                                             // c indexes the narrow row
      const int src = split ? (c < n / 2 ? c : c - n / 2 + w / 2) : c;
      out[i] = in[r * w + src];
    }
  }
}

__global__ void __launch_bounds__(256) pad_state_kernel(const PadJobs jobs, int inverse) {
  const int j = blockIdx.y;
  if (j >= jobs.count) return;
  if (jobs.elem[j] == 2)
    pad_rows(reinterpret_cast<const uint16_t*>(jobs.in[j]), reinterpret_cast<uint16_t*>(jobs.out[j]), jobs.rows[j], jobs.n[j],
             jobs.w[j], jobs.split[j] != 0, inverse != 0);
  else
    pad_rows(reinterpret_cast<const uint32_t*>(jobs.in[j]), reinterpret_cast<uint32_t*>(jobs.out[j]), jobs.rows[j], jobs.n[j],
             jobs.w[j], jobs.split[j] != 0, inverse != 0);
}
}  // namespace cm

// ins / outs: `count` device pointers; rows / n / w / elem (2 or 4 bytes) / split: per job.  All tensors row-contiguous.
extern "C" int cm_pad_state_dims(const void* const* ins, void* const* outs, const long long* rows, const int* n, const int* w,
                                 const int* elem, const int* split, int count, int inverse, cudaStream_t s) {
  if (count <= 0) return 0;
  if (count > cm::PAD_MAX_JOBS) return -10;
  cm::PadJobs jobs;
  jobs.count = count;
  long long most = 0;
  for (int j = 0; j < count; ++j) {
    if ((elem[j] != 2 && elem[j] != 4) || n[j] <= 0 || w[j] < n[j] || (split[j] && ((n[j] | w[j]) & 1))) return -10;
    jobs.in[j] = ins[j]; jobs.out[j] = outs[j]; jobs.rows[j] = rows[j];
    jobs.n[j] = n[j]; jobs.w[j] = w[j]; jobs.elem[j] = elem[j]; jobs.split[j] = split[j];
    const long long tot = rows[j] * (inverse ? n[j] : w[j]);
    if (tot > most) most = tot;
  }
  long long blocks = (most + 255) / 256;
  const long long cap = (long long)cm::sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  cm::pad_state_kernel<<<dim3((unsigned)blocks, (unsigned)count), 256, 0, s>>>(jobs, inverse);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
