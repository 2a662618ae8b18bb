// Bandwidth-bound kernels: RMSNorm fwd/bwd, SwiGLU fwd/bwd, fused AdamW shard update,
// gradient-buffer sum of squares.  All use 16-byte accesses and keep a row in registers between
// the reduction and the write so each element crosses HBM once per direction.
// (Role of the TE norm / activation kernels the reference links, cppmega/megatron/nam56r_full_spec.py:224-240.)
#include "common.cuh"

namespace cm {

// ---------------------------------------------------------------------------------------------
// RMSNorm.  One CTA of TPB threads per row for wide rows; one warp per row for narrow rows.
// ---------------------------------------------------------------------------------------------
// H = 256 VPL: one warp per row, VPL 16-byte vectors per lane (lane l takes vectors l, l + 32, ...): no block barrier,
// eight independent rows in flight per CTA.
template <int VPL>
__global__ void __launch_bounds__(256, 2) rmsnorm_fwd_warp(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                        __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_out, int rows, float eps) {
  constexpr int H = VPL * 256;
  const int lane = threadIdx.x & 31;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  for (int row = blockIdx.x * 8 + (threadIdx.x >> 5); row < rows; row += gridDim.x * 8) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * H);
    uint4 v[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) v[i] = xr[lane + i * 32];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(b[j]);
        ss += f.x * f.x + f.y * f.y;
      }
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / H + eps);
    if (lane == 0 && rstd_out) rstd_out[row] = rstd;
    uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * H);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const uint4 wv = wr[lane + i * 32];
      const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
      const __nv_bfloat162* wb = reinterpret_cast<const __nv_bfloat162*>(&wv);
      uint4 o;
      uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(b[j]);
        const float2 g = __bfloat1622float2(wb[j]);
        op[j] = pack_bf16(f.x * rstd * g.x, f.y * rstd * g.y);
      }
      yr[lane + i * 32] = o;
    }
  }
}

template <int TPB, int VPT>   // VPT 16-byte vectors per thread; row width <= TPB*VPT*8
__global__ void __launch_bounds__(TPB) rmsnorm_fwd_wide(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                        __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_out,
                                                        int rows, int H, float eps) {
  __shared__ float red[TPB / 32];
  const int nvec = H / 8;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  // the next row is requested before this row's block-wide sum, so the two barriers of a row overlap its loads
  uint4 nxt[VPT];
  auto fetch = [&](int row) {
    if (row < rows) {
      const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * H);
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int idx = threadIdx.x + i * TPB;
        if (idx < nvec) nxt[i] = xr[idx];
      }
    }
  };
  fetch(blockIdx.x);
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    uint4 v[VPT];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * TPB;
      v[i] = nxt[i];
      if (idx < nvec) {
        const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = __bfloat1622float2(b[j]);
          ss += f.x * f.x + f.y * f.y;
        }
      }
    }
    fetch(row + gridDim.x);
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < TPB / 32; ++i) tot += red[i];
    __syncthreads();
    const float rstd = rsqrtf(tot / H + eps);
    if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
    uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * H);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * TPB;
      if (idx < nvec) {
        const uint4 wv = wr[idx];
        const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
        const __nv_bfloat162* wb = reinterpret_cast<const __nv_bfloat162*>(&wv);
        uint4 o;
        uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = __bfloat1622float2(b[j]);
          float2 g = __bfloat1622float2(wb[j]);
          op[j] = pack_bf16(f.x * rstd * g.x, f.y * rstd * g.y);
        }
        yr[idx] = o;
      }
    }
  }
}

// narrow rows: one warp per row, H multiple of 8, H <= 1024
__global__ void __launch_bounds__(256) rmsnorm_fwd_narrow(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                          __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_out,
                                                          int rows, int H, float eps) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int nvec = H / 8;
  for (int row = blockIdx.x * wpb + (threadIdx.x >> 5); row < rows; row += gridDim.x * wpb) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * H);
    uint4 v[4];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = lane + i * 32;
      if (idx < nvec) {
        v[i] = xr[idx];
        const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = __bfloat1622float2(b[j]);
          ss += f.x * f.x + f.y * f.y;
        }
      }
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / H + eps);
    if (lane == 0 && rstd_out) rstd_out[row] = rstd;
    uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * H);
    const uint4* wr = reinterpret_cast<const uint4*>(w);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int idx = lane + i * 32;
      if (idx < nvec) {
        const uint4 wv = wr[idx];
        const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
        const __nv_bfloat162* wb = reinterpret_cast<const __nv_bfloat162*>(&wv);
        uint4 o;
        uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = __bfloat1622float2(b[j]);
          float2 g = __bfloat1622float2(wb[j]);
          op[j] = pack_bf16(f.x * rstd * g.x, f.y * rstd * g.y);
        }
        yr[idx] = o;
      }
    }
  }
}

// backward: dx = rstd * (dy*w - xhat * mean(dy*w*xhat)); dw += sum_rows dy * xhat  (fp32 atomics)
// generic layout: each warp owns a row; lanes stride over 16-byte vectors; dw partials are kept
// per-thread for the columns that thread touches (same columns for every row it visits).
template <int MAXV>   // max vectors per lane (H <= 32*MAXV*8)
__global__ void __launch_bounds__(256) rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                          const __nv_bfloat16* __restrict__ dy, const float* __restrict__ rstd_in,
                                                          __nv_bfloat16* __restrict__ dx, float* __restrict__ dw,
                                                          int rows, int H) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int nvec = H / 8;
  float dwacc[MAXV][8];
#pragma unroll
  for (int i = 0; i < MAXV; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  for (int row = blockIdx.x * wpb + (threadIdx.x >> 5); row < rows; row += gridDim.x * wpb) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * H);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + (size_t)row * H);
    const float rstd = rstd_in[row];
    float xh[MAXV][8], gw[MAXV][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int idx = lane + i * 32;
      if (idx < nvec) {
        const uint4 xv = xr[idx], gv = gr[idx], wv = wr[idx];
        const __nv_bfloat162* xb = reinterpret_cast<const __nv_bfloat162*>(&xv);
        const __nv_bfloat162* gb = reinterpret_cast<const __nv_bfloat162*>(&gv);
        const __nv_bfloat162* wb = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 xf = __bfloat1622float2(xb[j]), gf = __bfloat1622float2(gb[j]), wf = __bfloat1622float2(wb[j]);
          xh[i][2 * j] = xf.x * rstd;       xh[i][2 * j + 1] = xf.y * rstd;
          gw[i][2 * j] = gf.x * wf.x;       gw[i][2 * j + 1] = gf.y * wf.y;
          dwacc[i][2 * j] += gf.x * xh[i][2 * j];
          dwacc[i][2 * j + 1] += gf.y * xh[i][2 * j + 1];
          dot += gw[i][2 * j] * xh[i][2 * j] + gw[i][2 * j + 1] * xh[i][2 * j + 1];
        }
      }
    }
    dot = warp_sum(dot) / H;
    uint4* dxr = reinterpret_cast<uint4*>(dx + (size_t)row * H);
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int idx = lane + i * 32;
      if (idx < nvec) {
        uint4 o;
        uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          op[j] = pack_bf16(rstd * (gw[i][2 * j] - xh[i][2 * j] * dot), rstd * (gw[i][2 * j + 1] - xh[i][2 * j + 1] * dot));
        dxr[idx] = o;
      }
    }
  }
  if (dw) {
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int idx = lane + i * 32;
      if (idx < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) atomicAdd(dw + idx * 8 + j, dwacc[i][j]);
      }
    }
  }
}

// narrow rows (H = 8 * LPR <= 256): LPR lanes per row, 32 / LPR rows per warp and two such groups in flight, so a warp
// keeps 2 * 512 bytes of each operand outstanding instead of one half-used row; dw goes through one shared-memory
// reduction per CTA before the atomics.
template <int LPR>
__global__ void __launch_bounds__(256) rmsnorm_bwd_small(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                         const __nv_bfloat16* __restrict__ dy, const float* __restrict__ rstd_in,
                                                         __nv_bfloat16* __restrict__ dx, float* __restrict__ dw, int rows) {
  constexpr int H = LPR * 8, RPW = 32 / LPR, U = 2;
  __shared__ float red[8][H];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int l = lane % LPR, sub = lane / LPR;
  float wf[8], dwacc[8];
  {
    const uint4 wv = reinterpret_cast<const uint4*>(w)[l];
    const __nv_bfloat162* wb = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 t = __bfloat1622float2(wb[j]);
      wf[2 * j] = t.x; wf[2 * j + 1] = t.y;
      dwacc[2 * j] = 0.f; dwacc[2 * j + 1] = 0.f;
    }
  }
  const long long step = (long long)gridDim.x * 8 * RPW * U;
  for (long long row0 = ((long long)blockIdx.x * 8 + warp) * RPW * U; row0 < rows; row0 += step) {
    uint4 xv[U], gv[U];
    float rs[U];
    bool ok[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long row = row0 + u * RPW + sub;
      ok[u] = row < rows;
      if (ok[u]) {
        xv[u] = reinterpret_cast<const uint4*>(x + row * H)[l];
        gv[u] = reinterpret_cast<const uint4*>(dy + row * H)[l];
        rs[u] = rstd_in[row];
      } else {
        xv[u] = make_uint4(0, 0, 0, 0); gv[u] = xv[u]; rs[u] = 0.f;
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const __nv_bfloat162* xb = reinterpret_cast<const __nv_bfloat162*>(&xv[u]);
      const __nv_bfloat162* gb = reinterpret_cast<const __nv_bfloat162*>(&gv[u]);
      float xh[8], gw[8], dot = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 xf = __bfloat1622float2(xb[j]), gf = __bfloat1622float2(gb[j]);
        xh[2 * j] = xf.x * rs[u];            xh[2 * j + 1] = xf.y * rs[u];
        gw[2 * j] = gf.x * wf[2 * j];        gw[2 * j + 1] = gf.y * wf[2 * j + 1];
        dwacc[2 * j] += gf.x * xh[2 * j];    dwacc[2 * j + 1] += gf.y * xh[2 * j + 1];
        dot += gw[2 * j] * xh[2 * j] + gw[2 * j + 1] * xh[2 * j + 1];
      }
#pragma unroll
      for (int o = LPR / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      dot *= (1.f / H);
      if (ok[u]) {
        uint4 o4;
        uint32_t* op = reinterpret_cast<uint32_t*>(&o4);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          op[j] = pack_bf16(rs[u] * (gw[2 * j] - xh[2 * j] * dot), rs[u] * (gw[2 * j + 1] - xh[2 * j + 1] * dot));
        reinterpret_cast<uint4*>(dx + (row0 + u * RPW + sub) * H)[l] = o4;
      }
    }
  }
  if (dw) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
      for (int o = LPR; o < 32; o <<= 1) dwacc[j] += __shfl_xor_sync(0xffffffffu, dwacc[j], o);
      if (sub == 0) red[warp][l * 8 + j] = dwacc[j];
    }
    __syncthreads();
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
      float t = 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) t += red[k][c];
      atomicAdd(dw + c, t);
    }
  }
}

template <int TPB, int VPT>
__device__ __forceinline__ void rms_fetch_row(uint4 (&xn)[VPT], uint4 (&gn)[VPT], float& rn, const __nv_bfloat16* __restrict__ x,
                                              const __nv_bfloat16* __restrict__ dy, const float* __restrict__ rstd_in, int row, int rows,
                                              int H) {
  if (row >= rows) return;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * H);
  const uint4* gr = reinterpret_cast<const uint4*>(dy + (size_t)row * H);
  rn = rstd_in[row];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * TPB;
    if (idx < H / 8) { xn[i] = xr[idx]; gn[i] = gr[idx]; }
  }
}

// wide rows: one CTA per row (grid-stride), dw partials for this thread's columns stay in registers
template <int TPB, int VPT>
__global__ void __launch_bounds__(TPB) rmsnorm_bwd_wide(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                        const __nv_bfloat16* __restrict__ dy, const float* __restrict__ rstd_in,
                                                        __nv_bfloat16* __restrict__ dx, float* __restrict__ dw,
                                                        int rows, int H) {
  __shared__ float red[TPB / 32];
  const int nvec = H / 8;
  float dwacc[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  // the next row's vectors are requested before this row's reduction, so the block-wide sum and the two barriers
  // of a row overlap the loads of the following one
  uint4 xn[VPT], gn[VPT];
  float rn = 0.f;
  constexpr bool PREFETCH = VPT <= 4;          // wider rows would not fit two rows of operands in registers
  if constexpr (PREFETCH) rms_fetch_row<TPB, VPT>(xn, gn, rn, x, dy, rstd_in, blockIdx.x, rows, H);
  uint4 wv[PREFETCH ? VPT : 1];
  if constexpr (PREFETCH) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * TPB;
      wv[i] = idx < nvec ? wr[idx] : make_uint4(0, 0, 0, 0);
    }
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    if constexpr (!PREFETCH) rms_fetch_row<TPB, VPT>(xn, gn, rn, x, dy, rstd_in, row, rows, H);
    const float rstd = rn;
    uint4 xc[VPT], gc[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) { xc[i] = xn[i]; gc[i] = gn[i]; }
    if constexpr (PREFETCH) rms_fetch_row<TPB, VPT>(xn, gn, rn, x, dy, rstd_in, row + gridDim.x, rows, H);
    float xh[VPT][8], gw[VPT][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * TPB;
      if (idx < nvec) {
        const __nv_bfloat162* xb = reinterpret_cast<const __nv_bfloat162*>(&xc[i]);
        const __nv_bfloat162* gb = reinterpret_cast<const __nv_bfloat162*>(&gc[i]);
        uint4 wcur;
        if constexpr (PREFETCH) wcur = wv[i]; else wcur = wr[idx];
        const __nv_bfloat162* wb = reinterpret_cast<const __nv_bfloat162*>(&wcur);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 xf = __bfloat1622float2(xb[j]), gf = __bfloat1622float2(gb[j]), wf = __bfloat1622float2(wb[j]);
          xh[i][2 * j] = xf.x * rstd;       xh[i][2 * j + 1] = xf.y * rstd;
          gw[i][2 * j] = gf.x * wf.x;       gw[i][2 * j + 1] = gf.y * wf.y;
          dwacc[i][2 * j] += gf.x * xh[i][2 * j];
          dwacc[i][2 * j + 1] += gf.y * xh[i][2 * j + 1];
          dot += gw[i][2 * j] * xh[i][2 * j] + gw[i][2 * j + 1] * xh[i][2 * j + 1];
        }
      }
    }
    dot = warp_sum(dot);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = dot;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < TPB / 32; ++i) tot += red[i];
    __syncthreads();
    dot = tot / H;
    uint4* dxr = reinterpret_cast<uint4*>(dx + (size_t)row * H);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * TPB;
      if (idx < nvec) {
        uint4 o;
        uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          op[j] = pack_bf16(rstd * (gw[i][2 * j] - xh[i][2 * j] * dot), rstd * (gw[i][2 * j + 1] - xh[i][2 * j + 1] * dot));
        dxr[idx] = o;
      }
    }
  }
  if (dw) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * TPB;
      if (idx < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) atomicAdd(dw + idx * 8 + j, dwacc[i][j]);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// SwiGLU: in = [a | b] (width 2F), out = silu(a) * b
// ---------------------------------------------------------------------------------------------
// Rows are walked by (blockIdx.x, threadIdx.y), columns by threadIdx.x: no per-element 64-bit division.  `rows_limit`
// (optional, device): only the first min(rows, *rows_limit) rows are processed - the padded expert-sorted MoE buffers
// are sized for the worst case and the number of rows in use is only known on the device.
constexpr int SWIGLU_TX = 64, SWIGLU_TY = 4;

__global__ void __launch_bounds__(SWIGLU_TX * SWIGLU_TY) swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ in,
                                                                           __nv_bfloat16* __restrict__ out, long long rows, int F,
                                                                           const int* __restrict__ rows_limit) {
  const int fv = F / 8;
  if (rows_limit) rows = min(rows, (long long)*rows_limit);
  for (long long r = blockIdx.x * (long long)SWIGLU_TY + threadIdx.y; r < rows; r += (long long)gridDim.x * SWIGLU_TY) {
    const uint4* pa = reinterpret_cast<const uint4*>(in + r * 2 * F);
    const uint4* pb = reinterpret_cast<const uint4*>(in + r * 2 * F + F);
    uint4* po = reinterpret_cast<uint4*>(out + r * F);
    for (int c = threadIdx.x; c < fv; c += SWIGLU_TX) {
      const uint4 a = pa[c];
      const uint4 b = pb[c];
      const __nv_bfloat162* ab = reinterpret_cast<const __nv_bfloat162*>(&a);
      const __nv_bfloat162* bb = reinterpret_cast<const __nv_bfloat162*>(&b);
      uint4 o;
      uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 af = __bfloat1622float2(ab[j]), bf = __bfloat1622float2(bb[j]);
        op[j] = pack_bf16(af.x / (1.f + __expf(-af.x)) * bf.x, af.y / (1.f + __expf(-af.y)) * bf.y);
      }
      po[c] = o;
    }
  }
}

__global__ void __launch_bounds__(SWIGLU_TX * SWIGLU_TY) swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ in,
                                                                           const __nv_bfloat16* __restrict__ dout,
                                                                           __nv_bfloat16* __restrict__ din, long long rows, int F,
                                                                           const int* __restrict__ rows_limit) {
  const int fv = F / 8;
  if (rows_limit) rows = min(rows, (long long)*rows_limit);
  for (long long r = blockIdx.x * (long long)SWIGLU_TY + threadIdx.y; r < rows; r += (long long)gridDim.x * SWIGLU_TY) {
    const uint4* pa = reinterpret_cast<const uint4*>(in + r * 2 * F);
    const uint4* pb = reinterpret_cast<const uint4*>(in + r * 2 * F + F);
    const uint4* pg = reinterpret_cast<const uint4*>(dout + r * F);
    uint4* qa = reinterpret_cast<uint4*>(din + r * 2 * F);
    uint4* qb = reinterpret_cast<uint4*>(din + r * 2 * F + F);
    for (int c = threadIdx.x; c < fv; c += SWIGLU_TX) {
      const uint4 a = pa[c];
      const uint4 b = pb[c];
      const uint4 g = pg[c];
      const __nv_bfloat162* ab = reinterpret_cast<const __nv_bfloat162*>(&a);
      const __nv_bfloat162* bb = reinterpret_cast<const __nv_bfloat162*>(&b);
      const __nv_bfloat162* gb = reinterpret_cast<const __nv_bfloat162*>(&g);
      uint4 da, db;
      uint32_t* dap = reinterpret_cast<uint32_t*>(&da);
      uint32_t* dbp = reinterpret_cast<uint32_t*>(&db);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 af = __bfloat1622float2(ab[j]), bf = __bfloat1622float2(bb[j]), gf = __bfloat1622float2(gb[j]);
        const float s0 = 1.f / (1.f + __expf(-af.x)), s1 = 1.f / (1.f + __expf(-af.y));
        const float d0 = s0 * (1.f + af.x * (1.f - s0)), d1 = s1 * (1.f + af.y * (1.f - s1));
        dap[j] = pack_bf16(gf.x * bf.x * d0, gf.y * bf.y * d1);
        dbp[j] = pack_bf16(gf.x * af.x * s0, gf.y * af.y * s1);
      }
      qa[c] = da;
      qb[c] = db;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Fused AdamW on a flat fp32 master shard; gradient in fp32 or bf16; writes the bf16/fp32 copy.
// `clip` is a device scalar multiplied into the gradient (gradient clipping without a host sync).
// ---------------------------------------------------------------------------------------------
template <typename GradT, typename OutT>
__global__ void __launch_bounds__(256) adamw_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                                                    const GradT* __restrict__ g, OutT* __restrict__ out,
                                                    const uint8_t* __restrict__ wd_mask, const float* __restrict__ clip,
                                                    long long n, float lr, float b1, float b2, float eps, float wd,
                                                    float inv_bc1, float inv_bc2, const int* __restrict__ gate) {
  if (gate && *reinterpret_cast<const volatile int*>(gate) != 0) return;     // error word set: leave the state untouched
  const float cs = clip ? *clip : 1.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float gi = float(g[i]) * cs;
    const float mi = b1 * m[i] + (1.f - b1) * gi;
    const float vi = b2 * v[i] + (1.f - b2) * gi * gi;
    float p = master[i];
    float upd = (mi * inv_bc1) / (sqrtf(vi * inv_bc2) + eps);
    if (wd_mask[i]) upd += wd * p;
    p -= lr * upd;
    m[i] = mi;
    v[i] = vi;
    master[i] = p;
    out[i] = OutT(p);
  }
}

// four elements per thread: 16-byte accesses to master / m / v, 8- or 16-byte gradient loads, one mask word
template <typename GradT, typename OutT>
__global__ void __launch_bounds__(256) adamw_vec4_kernel(float4* __restrict__ master, float4* __restrict__ m, float4* __restrict__ v,
                                                         const GradT* __restrict__ g, OutT* __restrict__ out,
                                                         const uchar4* __restrict__ wd_mask, const float* __restrict__ clip,
                                                         long long n4, float lr, float b1, float b2, float eps, float wd,
                                                         float inv_bc1, float inv_bc2, const int* __restrict__ gate) {
  if (gate && *reinterpret_cast<const volatile int*>(gate) != 0) return;
  const float cs = clip ? *clip : 1.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float gi[4];
    if constexpr (sizeof(GradT) == 2) {
      const uint2 raw = reinterpret_cast<const uint2*>(g)[i];
      const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
      const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
      gi[0] = a.x; gi[1] = a.y; gi[2] = b.x; gi[3] = b.y;
    } else {
      const float4 raw = reinterpret_cast<const float4*>(g)[i];
      gi[0] = raw.x; gi[1] = raw.y; gi[2] = raw.z; gi[3] = raw.w;
    }
    float4 mm = m[i], vv = v[i], pp = master[i];
    const uchar4 wm = wd_mask[i];
    float* mp = reinterpret_cast<float*>(&mm);
    float* vp = reinterpret_cast<float*>(&vv);
    float* p = reinterpret_cast<float*>(&pp);
    const unsigned char wmask[4] = {wm.x, wm.y, wm.z, wm.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gj = gi[j] * cs;
      mp[j] = b1 * mp[j] + (1.f - b1) * gj;
      vp[j] = b2 * vp[j] + (1.f - b2) * gj * gj;
      float upd = (mp[j] * inv_bc1) / (sqrtf(vp[j] * inv_bc2) + eps);
      if (wmask[j]) upd += wd * p[j];
      p[j] -= lr * upd;
    }
    m[i] = mm;
    v[i] = vv;
    master[i] = pp;
    if constexpr (sizeof(OutT) == 2) {
      uint2 o;
      o.x = pack_bf16(p[0], p[1]);
      o.y = pack_bf16(p[2], p[3]);
      reinterpret_cast<uint2*>(out)[i] = o;
    } else {
      reinterpret_cast<float4*>(out)[i] = pp;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) sumsq_kernel(const T* __restrict__ g, long long n, float* __restrict__ out) {
  float s = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float f = float(g[i]);
    s += f * f;
  }
  s = warp_sum(s);
  __shared__ float red[8];
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < 8; ++i) t += red[i];
    atomicAdd(out, t);
  }
}

// out[i] = sum over slots of stage[slot * n + i]   (bf16 in, fp32 accumulation, bf16 out; 8 values per thread)
__global__ void __launch_bounds__(256) sum_slots_kernel(const __nv_bfloat16* __restrict__ stage, __nv_bfloat16* __restrict__ out,
                                                        int n_slots, long long n) {
  const long long nvec = n / 8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < n_slots; ++s) {
      const uint4 v = reinterpret_cast<const uint4*>(stage + (size_t)s * n)[i];
      const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(b[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]);
    o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out)[i] = o;
  }
}

// Strided copy in 16-byte vectors: a tensor of up to four outer dimensions whose innermost run is contiguous in both
// source and destination.  Sizes d1..d3 (d0 is implied by n_vec), byte strides per outer dimension.
struct StridedCopy {
  long long n_vec;
  int inner_vecs, d1, d2, d3;
  long long ss[4], ds[4];
};
// One work item = U consecutive 16-byte vectors of one inner run (they share the outer indices, so the index arithmetic -
// 32-bit here, the 64-bit divisions of a flat index made this kernel ALU-bound - is paid once per 16 U bytes).
// WS (warp-strided, runs of at least 32 U vectors): a warp moves 32 U consecutive vectors, lane l taking l, l + 32, ...,
// so every load and store instruction covers 512 contiguous bytes; otherwise a thread moves U consecutive vectors.
template <int U, bool WS>
__global__ void __launch_bounds__(256) strided_copy_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, const StridedCopy c) {
  const unsigned groups_per_run = (unsigned)c.inner_vecs / U;          // WS: in units of lanes, i.e. 32 groups per warp item
  const unsigned n_items = (unsigned)(c.n_vec / U);
  for (unsigned idx = blockIdx.x * blockDim.x + threadIdx.x; idx < n_items; idx += gridDim.x * blockDim.x) {
    const unsigned vg = idx % groups_per_run;
    unsigned rest = idx / groups_per_run;
    const unsigned i3 = rest % (unsigned)c.d3; rest /= (unsigned)c.d3;
    const unsigned i2 = rest % (unsigned)c.d2; rest /= (unsigned)c.d2;
    const unsigned i1 = rest % (unsigned)c.d1;
    const unsigned i0 = rest / (unsigned)c.d1;
    // WS: vg = 32 * block + lane within the run; the block's vectors start at 32 U block
    const unsigned first = WS ? (vg >> 5) * (32u * U) + (vg & 31u) : vg * U;
    constexpr unsigned step = WS ? 32u : 1u;
    const uint4* sp = reinterpret_cast<const uint4*>(src + i0 * c.ss[0] + i1 * c.ss[1] + i2 * c.ss[2] + i3 * c.ss[3]) + first;
    uint4* dp = reinterpret_cast<uint4*>(dst + i0 * c.ds[0] + i1 * c.ds[1] + i2 * c.ds[2] + i3 * c.ds[3]) + first;
    uint4 val[U];
#pragma unroll
    for (int u = 0; u < U; ++u) val[u] = sp[u * step];
#pragma unroll
    for (int u = 0; u < U; ++u) dp[u * step] = val[u];
  }
}

}  // namespace cm

using namespace cm;

// sizes [d0,d1,d2,d3] of the outer dimensions, inner run `inner_bytes` (multiple of 16), byte strides; all addresses 16-byte aligned
extern "C" int cm_strided_copy(const void* src, void* dst, const long long* sizes, const long long* sstr, const long long* dstr,
                               long long inner_bytes, cudaStream_t s) {
  if (inner_bytes <= 0 || (inner_bytes % 16)) return -10;
  cm::StridedCopy c;
  c.inner_vecs = (int)(inner_bytes / 16);
  c.d1 = (int)sizes[1]; c.d2 = (int)sizes[2]; c.d3 = (int)sizes[3];
  c.n_vec = sizes[0] * sizes[1] * sizes[2] * sizes[3] * c.inner_vecs;
  if (c.n_vec <= 0) return 0;
  for (int i = 0; i < 4; ++i) { c.ss[i] = sstr[i]; c.ds[i] = dstr[i]; }
  if (c.n_vec >= (1ll << 31)) return -11;                         // 32 GiB in one copy: split it
  const int U = (c.inner_vecs % 4 == 0) ? 4 : (c.inner_vecs % 2 == 0 ? 2 : 1);
  long long blocks = (c.n_vec / U + 255) / 256;
  const long long cap = (long long)cm::sm_count() * 16;
  const int grid = (int)(blocks < cap ? blocks : cap);
  if (c.inner_vecs % 128 == 0) cm::strided_copy_kernel<4, true><<<grid, 256, 0, s>>>((const uint8_t*)src, (uint8_t*)dst, c);
  else if (U == 4) cm::strided_copy_kernel<4, false><<<grid, 256, 0, s>>>((const uint8_t*)src, (uint8_t*)dst, c);
  else if (U == 2) cm::strided_copy_kernel<2, false><<<grid, 256, 0, s>>>((const uint8_t*)src, (uint8_t*)dst, c);
  else cm::strided_copy_kernel<1, false><<<grid, 256, 0, s>>>((const uint8_t*)src, (uint8_t*)dst, c);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int cm_sum_slots(const void* stage, void* out, int n_slots, long long n, cudaStream_t s) {
  if (n <= 0) return 0;
  if (n % 8 || n_slots <= 0) return -10;
  long long blocks = (n / 8 + 255) / 256;
  int grid = (int)(blocks < (long long)sm_count() * 16 ? blocks : (long long)sm_count() * 16);
  sum_slots_kernel<<<grid, 256, 0, s>>>((const __nv_bfloat16*)stage, (__nv_bfloat16*)out, n_slots, n);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int cm_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int rows, int H, float eps,
                              cudaStream_t s) {
  if (rows <= 0) return 0;
  if (H % 8) return -10;
  const __nv_bfloat16* xp = (const __nv_bfloat16*)x;
  const __nv_bfloat16* wp = (const __nv_bfloat16*)w;
  __nv_bfloat16* yp = (__nv_bfloat16*)y;
  if (H <= 1024) {
    const int wpb = 8;
    int grid = (rows + wpb - 1) / wpb;
    grid = grid < sm_count() * 8 ? grid : sm_count() * 8;
    rmsnorm_fwd_narrow<<<grid, 256, 0, s>>>(xp, wp, yp, rstd, rows, H, eps);
  } else if (H == 4096) {
    int grid = (rows + 7) / 8;
    grid = grid < sm_count() * 4 ? grid : sm_count() * 4;
    rmsnorm_fwd_warp<16><<<grid, 256, 0, s>>>(xp, wp, yp, rstd, rows, eps);
  } else if (H <= 128 * 4 * 8) {
    int grid = rows < sm_count() * 8 ? rows : sm_count() * 8;
    rmsnorm_fwd_wide<128, 4><<<grid, 128, 0, s>>>(xp, wp, yp, rstd, rows, H, eps);
  } else if (H <= 256 * 8 * 8) {
    int grid = rows < sm_count() * 4 ? rows : sm_count() * 4;
    rmsnorm_fwd_wide<256, 8><<<grid, 256, 0, s>>>(xp, wp, yp, rstd, rows, H, eps);
  } else {
    return -12;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int cm_rmsnorm_bwd(const void* x, const void* w, const void* dy, const float* rstd, void* dx, float* dw,
                              int rows, int H, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (H % 8) return -10;
  const int wpb = 8;
  int grid = (rows + wpb - 1) / wpb;
  const int cap = sm_count() * 4;
  grid = grid < cap ? grid : cap;
  auto xp = (const __nv_bfloat16*)x; auto wp = (const __nv_bfloat16*)w; auto gp = (const __nv_bfloat16*)dy;
  auto dxp = (__nv_bfloat16*)dx;
  const int cap8 = sm_count() * 8;
  auto small_grid = [&](int rpw) { long long g = ((long long)rows + 8 * rpw * 2 - 1) / (8 * rpw * 2); return (int)(g < cap8 ? g : cap8); };
  if (H == 64) rmsnorm_bwd_small<8><<<small_grid(4), 256, 0, s>>>(xp, wp, gp, rstd, dxp, dw, rows);
  else if (H == 128) rmsnorm_bwd_small<16><<<small_grid(2), 256, 0, s>>>(xp, wp, gp, rstd, dxp, dw, rows);
  else if (H == 256) rmsnorm_bwd_small<32><<<small_grid(1), 256, 0, s>>>(xp, wp, gp, rstd, dxp, dw, rows);
  else if (H <= 32 * 1 * 8) rmsnorm_bwd_kernel<1><<<grid, 256, 0, s>>>(xp, wp, gp, rstd, dxp, dw, rows, H);
  else if (H <= 128 * 1 * 8) rmsnorm_bwd_wide<128, 1><<<(rows < cap ? rows : cap), 128, 0, s>>>(xp, wp, gp, rstd, dxp, dw, rows, H);
  else if (H <= 256 * 2 * 8) rmsnorm_bwd_wide<256, 2><<<(rows < cap ? rows : cap), 256, 0, s>>>(xp, wp, gp, rstd, dxp, dw, rows, H);
  else if (H <= 256 * 8 * 8) rmsnorm_bwd_wide<256, 8><<<(rows < cap ? rows : cap), 256, 0, s>>>(xp, wp, gp, rstd, dxp, dw, rows, H);
  else return -12;
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

static int swiglu_grid(long long rows) {
  const long long blocks = (rows + SWIGLU_TY - 1) / SWIGLU_TY;
  const long long cap = (long long)sm_count() * 16;
  return (int)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

// `rows_limit` (optional device int): process only the first min(rows, *rows_limit) rows
extern "C" int cm_swiglu_fwd_rows(const void* in, void* out, long long rows, int F, const int* rows_limit, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (F % 8) return -10;
  swiglu_fwd_kernel<<<swiglu_grid(rows), dim3(SWIGLU_TX, SWIGLU_TY), 0, s>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, rows, F,
                                                                              rows_limit);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int cm_swiglu_bwd_rows(const void* in, const void* dout, void* din, long long rows, int F, const int* rows_limit,
                                  cudaStream_t s) {
  if (rows <= 0) return 0;
  if (F % 8) return -10;
  swiglu_bwd_kernel<<<swiglu_grid(rows), dim3(SWIGLU_TX, SWIGLU_TY), 0, s>>>((const __nv_bfloat16*)in, (const __nv_bfloat16*)dout,
                                                                              (__nv_bfloat16*)din, rows, F, rows_limit);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int cm_swiglu_fwd(const void* in, void* out, long long rows, int F, cudaStream_t s) {
  return cm_swiglu_fwd_rows(in, out, rows, F, nullptr, s);
}

extern "C" int cm_swiglu_bwd(const void* in, const void* dout, void* din, long long rows, int F, cudaStream_t s) {
  return cm_swiglu_bwd_rows(in, dout, din, rows, F, nullptr, s);
}

// grad_kind: 0 fp32, 1 bf16; out_kind: 0 fp32, 1 bf16.  `gate` (may be null): a device word; when it is non-zero at run
// time the update is skipped (the kernels' error word: a step whose collectives gave up must not reach the weights).
extern "C" int cm_adamw_gated(float* master, float* m, float* v, const void* g, void* out, const uint8_t* wd_mask,
                              const float* clip, long long n, float lr, float b1, float b2, float eps, float wd, float bc1,
                              float bc2, int grad_kind, int out_kind, const int* gate, cudaStream_t s) {
  if (n <= 0) return 0;
  const float i1 = 1.f / bc1, i2 = 1.f / bc2;
  {
    // vector body when every array starts on a 16-byte (mask: 4-byte) boundary; the scalar kernel takes the tail
    const uintptr_t al = reinterpret_cast<uintptr_t>(master) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v) |
                         reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(out);
    const long long n4 = n / 4;
    if (!(al & 15) && !(reinterpret_cast<uintptr_t>(wd_mask) & 3) && n4 > 0) {
      long long vb = (n4 + 255) / 256;
      const int vgrid = (int)(vb < (long long)sm_count() * 16 ? vb : (long long)sm_count() * 16);
#define CM_ADAMW_V4(GT, OT)                                                                                               \
  adamw_vec4_kernel<GT, OT><<<vgrid, 256, 0, s>>>((float4*)master, (float4*)m, (float4*)v, (const GT*)g, (OT*)out,         \
                                                  (const uchar4*)wd_mask, clip, n4, lr, b1, b2, eps, wd, i1, i2, gate)
      if (grad_kind == 0 && out_kind == 1) CM_ADAMW_V4(float, __nv_bfloat16);
      else if (grad_kind == 1 && out_kind == 1) CM_ADAMW_V4(__nv_bfloat16, __nv_bfloat16);
      else if (grad_kind == 0 && out_kind == 0) CM_ADAMW_V4(float, float);
      else CM_ADAMW_V4(__nv_bfloat16, float);
#undef CM_ADAMW_V4
      if (cudaGetLastError() != cudaSuccess) return -3;
      const long long done = n4 * 4;
      if (done == n) return 0;
      const size_t gsz = grad_kind == 0 ? 4 : 2, osz = out_kind == 0 ? 4 : 2;
      master += done; m += done; v += done; wd_mask += done;
      g = (const char*)g + done * gsz;
      out = (char*)out + done * osz;
      n -= done;
    }
  }
  long long blocks = (n + 255) / 256;
  int grid = (int)(blocks < (long long)sm_count() * 16 ? blocks : (long long)sm_count() * 16);
  if (grad_kind == 0 && out_kind == 1)
    adamw_kernel<float, __nv_bfloat16><<<grid, 256, 0, s>>>(master, m, v, (const float*)g, (__nv_bfloat16*)out, wd_mask, clip, n, lr, b1, b2, eps, wd, i1, i2, gate);
  else if (grad_kind == 1 && out_kind == 1)
    adamw_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, s>>>(master, m, v, (const __nv_bfloat16*)g, (__nv_bfloat16*)out, wd_mask, clip, n, lr, b1, b2, eps, wd, i1, i2, gate);
  else if (grad_kind == 0 && out_kind == 0)
    adamw_kernel<float, float><<<grid, 256, 0, s>>>(master, m, v, (const float*)g, (float*)out, wd_mask, clip, n, lr, b1, b2, eps, wd, i1, i2, gate);
  else
    adamw_kernel<__nv_bfloat16, float><<<grid, 256, 0, s>>>(master, m, v, (const __nv_bfloat16*)g, (float*)out, wd_mask, clip, n, lr, b1, b2, eps, wd, i1, i2, gate);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int cm_adamw(float* master, float* m, float* v, const void* g, void* out, const uint8_t* wd_mask,
                        const float* clip, long long n, float lr, float b1, float b2, float eps, float wd, float bc1,
                        float bc2, int grad_kind, int out_kind, cudaStream_t s) {
  return cm_adamw_gated(master, m, v, g, out, wd_mask, clip, n, lr, b1, b2, eps, wd, bc1, bc2, grad_kind, out_kind, nullptr, s);
}

// out (device float, caller zeroes it) += sum of squares of g.  kind: 0 fp32, 1 bf16
extern "C" int cm_sumsq(const void* g, long long n, float* out, int kind, cudaStream_t s) {
  if (n <= 0) return 0;
  long long blocks = (n + 255) / 256;
  int grid = (int)(blocks < (long long)sm_count() * 8 ? blocks : (long long)sm_count() * 8);
  if (kind == 0) sumsq_kernel<float><<<grid, 256, 0, s>>>((const float*)g, n, out);
  else sumsq_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)g, n, out);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
