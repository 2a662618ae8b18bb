// MXFP8 quantisation: E4M3 payload with one E8M0 scale per 32 values.
//
//   scale byte = clamp(ceil(log2(amax / 448)) + 127, 1, 254)   (127 for an all-zero block)
//   payload    = e4m3(x * 2^(127 - scale))
//
//   rowwise      blocks of 32 along the contiguous (last) dimension: the operand layout of a product that reduces
//                over that dimension (forward GEMM: x and W both along K);
//   columnwise   blocks of 32 along the rows, written TRANSPOSED ([cols, rows] payload, [cols, rows/32] scales), so
//                that the result is again a K-major operand for the products that reduce over rows (wgrad over
//                tokens, dgrad over output features);
//   dequantise   payload * 2^(scale - 127) -> bf16;
//   swizzle      row-major [rows, kb] scales -> the 128x4 tile order ([32][4][4] per tile) that block-scaled
//                tensor-core instructions read.
// These replace the reference's cast/transposed-cast kernels and its scale swizzle (Transformer-Engine MXFP8 tensors
// re-used by cppmega/megatron/cutlass_mxfp8_gemm.py:102-506; layout of the swizzle at
// cppmega/megatron/flashinfer_mxfp8_gemm.py:146-160; scale byte at cuda_ext/quantized_muon_momentum.cu:75-91).
#include "common.cuh"

namespace cm {
namespace mx {

__device__ __forceinline__ uint8_t e8m0_from_amax(float amax) {
  if (!(amax > 0.f)) return 127;
  int e = (int)ceilf(log2f(amax * (1.f / 448.f))) + 127;
  e = e < 1 ? 1 : (e > 254 ? 254 : e);
  return (uint8_t)e;
}
// two floats -> two e4m3 bytes (lo in bits 0..7)
__device__ __forceinline__ uint16_t to_e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float e4m3_to_float(uint8_t b) {
  // sign 1, exponent 4 (bias 7), mantissa 3; no infinities, 0x7f / 0xff are NaN
  const uint32_t s = (uint32_t)(b & 0x80) << 24;
  const uint32_t e = (b >> 3) & 0xf, m = b & 7;
  float v;
  if (e == 0) v = (float)m * 0.001953125f;                            // subnormal: m * 2^-9
  else v = __uint_as_float(((e + 120u) << 23) | (m << 20));
  return __uint_as_float(__float_as_uint(v) | s);
}

// position of scale (row, k block) in the 128x4 tile order
__device__ __forceinline__ size_t swizzled_index(long long row, int kb, int kb_tiles) {
  return ((size_t)(row >> 7) * kb_tiles + (kb >> 2)) * 512 + (size_t)(row & 31) * 16 + ((row >> 5) & 3) * 4 + (kb & 3);
}

// one thread = 8 consecutive values; 4 threads = one block of 32
__global__ void __launch_bounds__(256) quantize_rowwise_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ payload,
                                                               uint8_t* __restrict__ scales, uint8_t* __restrict__ sw, long long rows,
                                                               int cols, const float* __restrict__ tamax) {
  const int kb_row = cols / 32, kb_tiles = (kb_row + 3) / 4;
  const long long nvec = rows * (cols / 8);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const uint4 raw = reinterpret_cast<const uint4*>(x)[i];
    const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&raw);
    float f[8];
    float am = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 t = __bfloat1622float2(b[j]);
      f[2 * j] = t.x; f[2 * j + 1] = t.y;
      am = fmaxf(am, fmaxf(fabsf(t.x), fabsf(t.y)));
    }
    const unsigned live = __activemask();          // whole groups of four threads enter or leave the loop together
    am = fmaxf(am, __shfl_xor_sync(live, am, 1));
    am = fmaxf(am, __shfl_xor_sync(live, am, 2));
    const uint8_t sb = e8m0_from_amax(tamax ? *tamax : am);
    const float mult = exp2f(127.f - (float)sb);
    uint2 o;
    o.x = (uint32_t)to_e4m3x2(f[0] * mult, f[1] * mult) | ((uint32_t)to_e4m3x2(f[2] * mult, f[3] * mult) << 16);
    o.y = (uint32_t)to_e4m3x2(f[4] * mult, f[5] * mult) | ((uint32_t)to_e4m3x2(f[6] * mult, f[7] * mult) << 16);
    reinterpret_cast<uint2*>(payload)[i] = o;
    if ((threadIdx.x & 3) == 0) {
      scales[i >> 2] = sb;
      if (sw) {
        const long long blk = i >> 2;
        sw[swizzled_index(blk / kb_row, (int)(blk % kb_row), kb_tiles)] = sb;
      }
    }
  }
}

// CTA = tile of 32 rows x 128 columns; thread c owns one column: 32 values -> one block
__global__ void __launch_bounds__(128) quantize_colwise_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ payload_t,
                                                               uint8_t* __restrict__ scales_t, uint8_t* __restrict__ sw, long long rows,
                                                               int cols, const float* __restrict__ tamax) {
  const long long r0 = (long long)blockIdx.y * 32;
  const int c = blockIdx.x * 128 + threadIdx.x;
  if (c >= cols) return;
  float f[32];
  float am = 0.f;
#pragma unroll
  for (int r = 0; r < 32; ++r) {
    f[r] = (r0 + r < rows) ? __bfloat162float(x[(size_t)(r0 + r) * cols + c]) : 0.f;
    am = fmaxf(am, fabsf(f[r]));
  }
  const uint8_t sb = e8m0_from_amax(tamax ? *tamax : am);
  const float mult = exp2f(127.f - (float)sb);
  uint32_t w[8];
#pragma unroll
  for (int q = 0; q < 8; ++q)
    w[q] = (uint32_t)to_e4m3x2(f[4 * q] * mult, f[4 * q + 1] * mult) | ((uint32_t)to_e4m3x2(f[4 * q + 2] * mult, f[4 * q + 3] * mult) << 16);
  uint4* dst = reinterpret_cast<uint4*>(payload_t + (size_t)c * rows + r0);
  dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
  dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
  scales_t[(size_t)c * (rows / 32) + blockIdx.y] = sb;
  if (sw) sw[swizzled_index(c, (int)blockIdx.y, (int)((rows / 32 + 3) / 4))] = sb;
}

// Both orientations from one read of x: CTA = tile of 32 rows x 256 columns.  Phase 1 is the row-wise kernel (8 values
// per thread, 4 threads per block) and parks the values as fp32 in shared memory; phase 2 walks the columns of the tile.
// The tile is stored column-permuted (logical column 8 v + j at physical column 32 j + v) with a row stride of 257 floats,
// which makes both the phase-1 stores and the phase-2 column reads bank-conflict free.
__global__ void __launch_bounds__(256) quantize_both_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ pay_r,
                                                            uint8_t* __restrict__ sc_r, uint8_t* __restrict__ sw_r,
                                                            uint8_t* __restrict__ pay_t, uint8_t* __restrict__ sc_t,
                                                            uint8_t* __restrict__ sw_t, long long rows, int cols,
                                                            const float* __restrict__ tamax) {
  __shared__ float tile[32][257];
  const long long r0 = (long long)blockIdx.y * 32;
  const int c0 = blockIdx.x * 256;
  const int kb_row = cols / 32, kbt_row = (kb_row + 3) / 4;
  const int kb_col = (int)(rows / 32), kbt_col = (kb_col + 3) / 4;
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int row = it * 8 + (threadIdx.x >> 5);
    const int col = c0 + lane * 8;
    const bool valid = col < cols;
    float f[8];
    float am = 0.f;
    if (valid) {
      const uint4 raw = *reinterpret_cast<const uint4*>(x + (size_t)(r0 + row) * cols + col);
      const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 t = __bfloat1622float2(b[j]);
        f[2 * j] = t.x; f[2 * j + 1] = t.y;
        am = fmaxf(am, fmaxf(fabsf(t.x), fabsf(t.y)));
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = 0.f;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) tile[row][j * 32 + lane] = f[j];
    am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 1));
    am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 2));
    if (valid) {
      const uint8_t sb = e8m0_from_amax(tamax ? *tamax : am);
      const float mult = exp2f(127.f - (float)sb);
      uint2 o;
      o.x = (uint32_t)to_e4m3x2(f[0] * mult, f[1] * mult) | ((uint32_t)to_e4m3x2(f[2] * mult, f[3] * mult) << 16);
      o.y = (uint32_t)to_e4m3x2(f[4] * mult, f[5] * mult) | ((uint32_t)to_e4m3x2(f[6] * mult, f[7] * mult) << 16);
      *reinterpret_cast<uint2*>(pay_r + (size_t)(r0 + row) * cols + col) = o;
      if ((lane & 3) == 0) {
        const int kb = col >> 5;
        sc_r[(size_t)(r0 + row) * kb_row + kb] = sb;
        if (sw_r) sw_r[swizzled_index(r0 + row, kb, kbt_row)] = sb;
      }
    }
  }
  __syncthreads();
  const int p = threadIdx.x;                                // physical column of the tile
  const int col = c0 + (p & 31) * 8 + (p >> 5);             // its logical column
  if (col >= cols) return;
  float f[32];
  float am = 0.f;
#pragma unroll
  for (int r = 0; r < 32; ++r) {
    f[r] = tile[r][p];
    am = fmaxf(am, fabsf(f[r]));
  }
  const uint8_t sb = e8m0_from_amax(tamax ? *tamax : am);
  const float mult = exp2f(127.f - (float)sb);
  uint32_t w[8];
#pragma unroll
  for (int q = 0; q < 8; ++q)
    w[q] = (uint32_t)to_e4m3x2(f[4 * q] * mult, f[4 * q + 1] * mult) | ((uint32_t)to_e4m3x2(f[4 * q + 2] * mult, f[4 * q + 3] * mult) << 16);
  uint4* dst = reinterpret_cast<uint4*>(pay_t + (size_t)col * rows + r0);
  dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
  dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
  sc_t[(size_t)col * kb_col + blockIdx.y] = sb;
  if (sw_t) sw_t[swizzled_index(col, (int)blockIdx.y, kbt_col)] = sb;
}

// absolute maximum of a bf16 tensor: non-negative floats order like their bit patterns, so an integer atomicMax works
__global__ void __launch_bounds__(256) amax_kernel(const __nv_bfloat16* __restrict__ x, long long nvec, float* __restrict__ out) {
  float am = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const uint4 raw = reinterpret_cast<const uint4*>(x)[i];
    const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 t = __bfloat1622float2(b[j]);
      am = fmaxf(am, fmaxf(fabsf(t.x), fabsf(t.y)));
    }
  }
  am = warp_max(am);
  __shared__ float red[8];
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = am;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) am = fmaxf(am, red[w]);
    if (am == am) atomicMax(reinterpret_cast<unsigned int*>(out), __float_as_uint(am));
  }
}

__global__ void __launch_bounds__(256) dequantize_kernel(const uint8_t* __restrict__ payload, const uint8_t* __restrict__ scales,
                                                         __nv_bfloat16* __restrict__ out, long long n) {
  const long long nvec = n / 8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    const uint2 raw = reinterpret_cast<const uint2*>(payload)[i];
    const float mult = exp2f((float)scales[i >> 2] - 127.f);
    const uint8_t* b = reinterpret_cast<const uint8_t*>(&raw);
    uint4 o;
    o.x = pack_bf16(e4m3_to_float(b[0]) * mult, e4m3_to_float(b[1]) * mult);
    o.y = pack_bf16(e4m3_to_float(b[2]) * mult, e4m3_to_float(b[3]) * mult);
    o.z = pack_bf16(e4m3_to_float(b[4]) * mult, e4m3_to_float(b[5]) * mult);
    o.w = pack_bf16(e4m3_to_float(b[6]) * mult, e4m3_to_float(b[7]) * mult);
    reinterpret_cast<uint4*>(out)[i] = o;
  }
}

// out is the flat 128x4-tiled buffer of ceil(rows/128) x ceil(kb/4) tiles of 512 bytes, padded with the neutral scale
__global__ void __launch_bounds__(256) swizzle_scales_kernel(const uint8_t* __restrict__ scales, uint8_t* __restrict__ out, long long rows,
                                                             int kb, int kb_tiles, long long total) {
  for (long long o = blockIdx.x * (long long)blockDim.x + threadIdx.x; o < total; o += (long long)gridDim.x * blockDim.x) {
    const long long tile = o >> 9;
    const int in = (int)(o & 511);
    const int r32 = in >> 4, rg = (in >> 2) & 3, k4 = in & 3;
    const long long row = (tile / kb_tiles) * 128 + rg * 32 + r32;
    const int k = (int)(tile % kb_tiles) * 4 + k4;
    out[o] = (row < rows && k < kb) ? scales[row * kb + k] : (uint8_t)127;
  }
}

}  // namespace mx
}  // namespace cm

using namespace cm;
using namespace cm::mx;

static int grid1d(long long work) {
  long long blocks = (work + 255) / 256;
  long long cap = (long long)sm_count() * 16;
  return (int)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

// x [rows, cols] bf16, cols % 32 == 0 -> payload [rows, cols] u8, scales [rows, cols/32] u8; `swizzled` (optional) also
// receives the scales in the 128x4 tile order (its padding entries must already hold the neutral scale)
// `tensor_amax` (optional, every quantise entry point): a device float holding the absolute maximum of the WHOLE tensor.
// When given, every block uses the one scale derived from it (per-tensor "current scaling" with a power-of-two scale)
// instead of its own: the tensorwise FP8 recipe on the same payload / scale-byte data path.
extern "C" int cm_mxfp8_quantize_rowwise(const void* x, void* payload, void* scales, void* swizzled, long long rows, int cols,
                                         const float* tensor_amax, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (cols % 32) return -10;
  quantize_rowwise_kernel<<<grid1d(rows * (cols / 8)), 256, 0, s>>>((const __nv_bfloat16*)x, (uint8_t*)payload, (uint8_t*)scales,
                                                                  (uint8_t*)swizzled, rows, cols, tensor_amax);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// x [rows, cols] bf16, rows % 32 == 0 -> payload_t [cols, rows] u8, scales_t [cols, rows/32] u8 (+ optional swizzled copy)
extern "C" int cm_mxfp8_quantize_colwise(const void* x, void* payload_t, void* scales_t, void* swizzled, long long rows, int cols,
                                         const float* tensor_amax, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (rows % 32) return -10;
  dim3 grid((cols + 127) / 128, (unsigned)(rows / 32));
  quantize_colwise_kernel<<<grid, 128, 0, s>>>((const __nv_bfloat16*)x, (uint8_t*)payload_t, (uint8_t*)scales_t, (uint8_t*)swizzled, rows, cols, tensor_amax);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// x [rows, cols] bf16 (rows % 32 == 0, cols % 32 == 0) -> row-wise payload / scales and the transposed column-wise pair in
// one pass; the swizzled scale outputs are optional
extern "C" int cm_mxfp8_quantize_both(const void* x, void* pay_r, void* sc_r, void* sw_r, void* pay_t, void* sc_t, void* sw_t,
                                      long long rows, int cols, const float* tensor_amax, cudaStream_t s) {
  if (rows <= 0) return 0;
  if ((rows % 32) || (cols % 32)) return -10;
  dim3 grid((cols + 255) / 256, (unsigned)(rows / 32));
  quantize_both_kernel<<<grid, 256, 0, s>>>((const __nv_bfloat16*)x, (uint8_t*)pay_r, (uint8_t*)sc_r, (uint8_t*)sw_r, (uint8_t*)pay_t,
                                           (uint8_t*)sc_t, (uint8_t*)sw_t, rows, cols, tensor_amax);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// out (device float, zeroed by the caller) = max(out, max |x|) over n bf16 values (n % 8 == 0)
extern "C" int cm_amax_bf16(const void* x, long long n, float* out, cudaStream_t s) {
  if (n <= 0) return 0;
  if (n % 8) return -10;
  amax_kernel<<<grid1d(n / 8), 256, 0, s>>>((const __nv_bfloat16*)x, n / 8, out);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// payload [n] u8 with scales [n/32] (blocks of 32 consecutive values) -> bf16 [n]
extern "C" int cm_mxfp8_dequantize(const void* payload, const void* scales, void* out, long long n, cudaStream_t s) {
  if (n <= 0) return 0;
  if (n % 32) return -10;
  dequantize_kernel<<<grid1d(n / 8), 256, 0, s>>>((const uint8_t*)payload, (const uint8_t*)scales, (__nv_bfloat16*)out, n);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// scales [rows, kb] -> out [ceil(rows/128) * ceil(kb/4) * 512]
extern "C" int cm_mxfp8_swizzle_scales(const void* scales, void* out, long long rows, int kb, cudaStream_t s) {
  if (rows <= 0 || kb <= 0) return 0;
  const int kb_tiles = (kb + 3) / 4;
  const long long total = ((rows + 127) / 128) * (long long)kb_tiles * 512;
  swizzle_scales_kernel<<<grid1d(total), 256, 0, s>>>((const uint8_t*)scales, (uint8_t*)out, rows, kb, kb_tiles, total);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
