// Shared pieces of the Mamba3 MIMO scan kernels (forward and backward).
//
// Work decomposition (chunk-parallel): the sequence is cut into chunks of LT = 32 tokens; with MIMO
// rank R = 4 a chunk is a tile of 128 "fused rows" i = 4*t + r, which is exactly one tcgen05 M=128
// tile.  All heavy kernels run one CTA (128 threads, thread i <-> fused row i <-> TMEM lane i) per
// (batch, head, chunk) with no loop-carried dependency; the only sequential part is an elementwise
// recurrence over chunk states.  Per chunk (N = state dim, P = head dim = 64):
//
//   Qr, Kr [128,N]  = rot(Q + bias), bf16, 128-byte-swizzled shared memory tiles (K-major)
//   PV [128,P]      = V[t] * Psi[r]
//   S1 = Qr Kr^T ;  M[i,j] = ts_tj e^{cs_ti - cs_tj} (tj<ti) | gamma_ti (tj==ti) | 0 ;  Pm = S1 o M
//   O  = Pm PV + e^{cs_ti} (Qr St) + D PV ;   y[t] = sum_r O[4t+r] * Phi[r] * silu(Z[t] Zeta[r])
//   St_end = e^{tot} St + Kr^T (w o PV),  w_j = ts_tj e^{tot - cs_tj}
//
// with cs the inclusive within-chunk cumulative sum of A*dt, tot its last value, gamma/ts the
// trapezoid coefficients.  The reference runs the same mathematics chunk by chunk inside one
// TileLang kernel per (batch, head) (restated at cppmega/megatron/cute_dsl_mimo/cute_dsl_mimo_fwd.py:89-267).
#pragma once
#include "common.cuh"

namespace cm {
namespace mimo {

constexpr int LT = 32;            // tokens per chunk
constexpr int R = 4;              // MIMO rank
constexpr int ROWS = LT * R;      // 128 fused rows
constexpr int P = 64;             // head dim
constexpr int THREADS = 128;
constexpr int SLAB = ROWS * 128;  // bytes of one [128 rows x 64 bf16] swizzled slab
// Row stride of the per-rank [R, P] vectors in shared memory.  The four lanes of a token read four different ranks at
// the same column; with a stride of P (a multiple of 32 banks) those reads collide four ways, with P + 4 they do not.
constexpr int VLD = P + 4;
__device__ __forceinline__ int vec_idx(int x) { return (x / P) * VLD + (x % P); }   // flat [R*P] index -> padded

// byte offset of logical 16-byte chunk `c` (0..7) of row `row` inside a 128B-swizzled slab
__device__ __forceinline__ int sw_off(int row, int c) { return row * 128 + ((c ^ (row & 7)) << 4); }

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 t = __bfloat1622float2(b[j]);
    f[2 * j] = t.x;
    f[2 * j + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 o;
  o.x = pack_bf16(f[0], f[1]); o.y = pack_bf16(f[2], f[3]);
  o.z = pack_bf16(f[4], f[5]); o.w = pack_bf16(f[6], f[7]);
  return o;
}

struct alignas(16) ChunkScalars {   // shared-memory block, one per CTA; the mbarriers are placed right after it,
  float cs[LT];                     // so its size must keep them 8-byte aligned
  float ts[LT];                     // trapezoid coefficient entering the state
  float gam[LT];                    // same-token coefficient
  float tot;                        // cs[LT-1]
  float pad_[3];
};
static_assert(sizeof(ChunkScalars) % 16 == 0, "mbarriers follow this block and need 8-byte alignment");

// Chunk scalars in two steps so that the global loads can be issued at the top of a kernel and consumed later.
// ADT/DT/Trap are [B,H,S] fp32; `base` = (b*H + h)*S + t0.  Only warp 0 takes part.
struct ScalarLoads {
  float a, dt, tr, dt1, tr1;
};
__device__ __forceinline__ ScalarLoads load_chunk_scalars(const float* __restrict__ ADT, const float* __restrict__ DT,
                                                          const float* __restrict__ Trap, size_t base, int t0, int S) {
  ScalarLoads l{0.f, 0.f, 0.f, 0.f, 0.f};
  if ((threadIdx.x >> 5) != 0) return l;
  const int lane = threadIdx.x & 31;
  l.a = ADT[base + lane];
  l.dt = DT[base + lane];
  l.tr = Trap[base + lane];
  if (t0 + lane + 1 < S) {
    l.dt1 = DT[base + lane + 1];
    l.tr1 = Trap[base + lane + 1];
  }
  return l;
}
__device__ __forceinline__ void finish_chunk_scalars(ChunkScalars* sc, const ScalarLoads& l, int t0, int S) {
  const int lane = threadIdx.x & 31;
  if ((threadIdx.x >> 5) != 0) return;
  float a = l.a;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float n = __shfl_up_sync(0xffffffffu, a, o);
    if (lane >= o) a += n;
  }
  const float g = __fdividef(l.dt, 1.f + __expf(-l.tr));
  float nxt = 0.f;
  if (t0 + lane + 1 < S) nxt = __fdividef(l.dt1, 1.f + __expf(l.tr1));            // dt * sigmoid(-trap)
  sc->cs[lane] = a;
  sc->gam[lane] = g;
  sc->ts[lane] = g + nxt;
  if (lane == 31) sc->tot = a;
}
__device__ __forceinline__ void compute_chunk_scalars(ChunkScalars* sc, const float* __restrict__ ADT,
                                                      const float* __restrict__ DT, const float* __restrict__ Trap,
                                                      size_t base, int t0, int S) {
  const ScalarLoads l = load_chunk_scalars(ADT, DT, Trap, base, t0, S);
  finish_chunk_scalars(sc, l, t0, S);
}

// cos/sin of the chunk's rotary angles into shared memory: cs_tab[t][a] (a < NROT).
// angles [B,S,H,NROT] fp32 (already cumulative).  Each thread (t = i/4, r = i%4) fills a quarter row.
// Table rows are NROT + 4 floats apart: 16-byte aligned for vector loads, and the tokens a warp touches at once fall
// into different banks.
// NWG = warpgroups (of 128 threads) in the CTA; the work of a row is split between them.
template <int NROT>
constexpr int tab_stride() { return NROT + 4; }   // 16-byte aligned rows; 4-bank skew per row keeps 128-bit loads conflict-free
template <int NROT>
constexpr int tab_floats() { return LT * (NROT + 4); }   // one table

template <int NROT, int NWG = 1>
__device__ __forceinline__ void fill_sincos(float* cos_tab, float* sin_tab, const float* __restrict__ angles,
                                            size_t b, int t0, int h, int S, int H) {
  const int i = threadIdx.x & 127, wg = threadIdx.x >> 7, t = i >> 2, r = i & 3;
  constexpr int PER = NROT / 4 / NWG;
  constexpr int TS = tab_stride<NROT>();
  const int off = (r * NWG + wg) * PER;
  const float* a = angles + (((size_t)b * S + t0 + t) * H + h) * NROT + off;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    float x = a[j];
    x -= 6.283185307179586f * rintf(x * 0.15915494309189535f);     // range-reduce before the fast path
    float s, c;
    __sincosf(x, &s, &c);
    cos_tab[t * TS + off + j] = c;
    sin_tab[t * TS + off + j] = s;
  }
}

// Two-warpgroup form with the four angles of this thread already in registers (NROT == 32: PER == 4).
template <int NROT>
__device__ __forceinline__ float4 load_angles4(const float* __restrict__ angles, size_t b, int t0, int h, int S, int H) {
  static_assert(NROT == 32, "one float4 per thread");
  const int i = threadIdx.x & 127, wg = threadIdx.x >> 7, t = i >> 2, r = i & 3;
  return *reinterpret_cast<const float4*>(angles + (((size_t)b * S + t0 + t) * H + h) * NROT + (r * 2 + wg) * 4);
}
template <int NROT>
__device__ __forceinline__ void fill_sincos4(float* cos_tab, float* sin_tab, const float4& a4) {
  const int i = threadIdx.x & 127, wg = threadIdx.x >> 7, t = i >> 2, r = i & 3;
  constexpr int TS = tab_stride<NROT>();
  const int off = (r * 2 + wg) * 4;
  const float av[4] = {a4.x, a4.y, a4.z, a4.w};
  float cv[4], sv[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float x = av[j];
    x -= 6.283185307179586f * rintf(x * 0.15915494309189535f);
    __sincosf(x, &sv[j], &cv[j]);
  }
  *reinterpret_cast<float4*>(cos_tab + t * TS + off) = make_float4(cv[0], cv[1], cv[2], cv[3]);
  *reinterpret_cast<float4*>(sin_tab + t * TS + off) = make_float4(sv[0], sv[1], sv[2], sv[3]);
}

__device__ __forceinline__ void ld8(float (&o)[8], const float* p) {        // two 128-bit shared/global loads
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}

// In-place transform of one operand tile (row i of this thread): x <- rot(x + bias[r]).
// Tile = N/64 slabs of [128 x 64] bf16, swizzled.  bias [R,N] fp32 for this head.  Pairs (n, N/2 + n),
// n < NROT, are rotated by the token's angle.
// BLD = floats between the bias rows of consecutive ranks (N when read from global memory; N + 4 in the padded
// shared-memory copy, which puts the four ranks a warp reads at once into different banks).
template <int N, int NROT, int NWG = 1, int BLD = N>
__device__ __forceinline__ void transform_rows(uint8_t* tile, const float* __restrict__ bias, const float* cos_tab,
                                               const float* sin_tab) {
  const int i = threadIdx.x & 127, wg = threadIdx.x >> 7, t = i >> 2, r = i & 3;
  const float* bb = bias + r * BLD;
  constexpr int HALF = N / 2;
  constexpr int TS = tab_stride<NROT>();
  // rotated pairs: chunks [0, NROT/8) of the first half with the same chunks of the second half
#pragma unroll
  for (int c0 = 0; c0 < NROT / 8; c0 += NWG) {
    const int c = c0 + wg;
    const int colA = c * 8, colB = HALF + c * 8;
    uint8_t* pa = tile + (colA / 64) * SLAB + sw_off(i, (colA % 64) / 8);
    uint8_t* pb = tile + (colB / 64) * SLAB + sw_off(i, (colB % 64) / 8);
    float fa[8], fb[8];
    unpack8(*reinterpret_cast<uint4*>(pa), fa);
    unpack8(*reinterpret_cast<uint4*>(pb), fb);
    float ba[8], bbv[8], cs8[8], sn8[8];
    ld8(ba, bb + colA);
    ld8(bbv, bb + colB);
    ld8(cs8, cos_tab + t * TS + colA);
    ld8(sn8, sin_tab + t * TS + colA);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float xa = fa[j] + ba[j], xb = fb[j] + bbv[j];
      fa[j] = cs8[j] * xa - sn8[j] * xb;
      fb[j] = sn8[j] * xa + cs8[j] * xb;
    }
    *reinterpret_cast<uint4*>(pa) = pack8(fa);
    *reinterpret_cast<uint4*>(pb) = pack8(fb);
  }
  // un-rotated remainder of both halves: bias only
#pragma unroll
  for (int hsel = 0; hsel < 2; ++hsel) {
#pragma unroll
    for (int c0 = NROT / 8; c0 < HALF / 8; c0 += NWG) {
      const int c = c0 + wg;
      const int col = hsel * HALF + c * 8;
      uint8_t* p = tile + (col / 64) * SLAB + sw_off(i, (col % 64) / 8);
      float f[8];
      unpack8(*reinterpret_cast<uint4*>(p), f);
      float bv[8];
      ld8(bv, bb + col);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] += bv[j];
      *reinterpret_cast<uint4*>(p) = pack8(f);
    }
  }
}

// PV row of this thread: pv[p] = V[t,p] * Psi[r,p].  V [B,S,H,P] bf16, psi [R,P] fp32 (this head).
__device__ __forceinline__ void load_pv_row(float (&pv)[P], const __nv_bfloat16* __restrict__ V, const float* __restrict__ psi,
                                            size_t b, int t0, int h, int S, int H) {
  const int i = threadIdx.x, t = i >> 2, r = i & 3;
  const uint4* v = reinterpret_cast<const uint4*>(V + (((size_t)b * S + t0 + t) * H + h) * P);
#pragma unroll
  for (int c = 0; c < P / 8; ++c) {
    float f[8];
    unpack8(v[c], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) pv[c * 8 + j] = f[j] * psi[r * P + c * 8 + j];
  }
}

// Two-warpgroup form: this thread owns columns [wg*32, wg*32 + 32) of row i.  `psi` may point to shared memory.
__device__ __forceinline__ void load_pv_half(float (&pv)[P / 2], const __nv_bfloat16* __restrict__ V, const float* psi,
                                             size_t b, int t0, int h, int S, int H) {
  const int i = threadIdx.x & 127, wg = threadIdx.x >> 7, t = i >> 2, r = i & 3;
  const uint4* v = reinterpret_cast<const uint4*>(V + (((size_t)b * S + t0 + t) * H + h) * P + wg * 32);
#pragma unroll
  for (int c = 0; c < P / 16; ++c) {
    float f[8];
    unpack8(v[c], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) pv[c * 8 + j] = f[j] * psi[r * P + wg * 32 + c * 8 + j];
  }
}
// raw 64-byte half row (columns [wg*32, +32)) of a [B,S,H,P] bf16 tensor for this thread's token
struct HalfRowRaw {
  uint4 v[4];
};
// `ld` = elements between consecutive tokens (H*P for a packed tensor; larger for a column slice of a wider matrix)
__device__ __forceinline__ HalfRowRaw load_half_raw(const __nv_bfloat16* __restrict__ X, size_t b, int t0, int h, int S, long long ld) {
  const int i = threadIdx.x & 127, wg = threadIdx.x >> 7, t = i >> 2;
  const uint4* p = reinterpret_cast<const uint4*>(X + ((size_t)b * S + t0 + t) * ld + h * P + wg * 32);
  HalfRowRaw o;
#pragma unroll
  for (int c = 0; c < 4; ++c) o.v[c] = p[c];
  return o;
}
__device__ __forceinline__ void half_raw_to_float(float (&x)[P / 2], const HalfRowRaw& raw) {
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    float f[8];
    unpack8(raw.v[c], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[c * 8 + j] = f[j];
  }
}
// pv = V * psi for this thread's half row; psi -> [R,P] in shared memory
__device__ __forceinline__ void pv_from_raw(float (&pv)[P / 2], const HalfRowRaw& raw, const float* psi) {
  const int i = threadIdx.x & 127, wg = threadIdx.x >> 7, r = i & 3;
  half_raw_to_float(pv, raw);
#pragma unroll
  for (int e = 0; e < P / 2; ++e) pv[e] *= psi[r * VLD + wg * 32 + e];
}
// Sum 32 per-thread values over the four lanes of a token (lanes that differ in their two low bits); lane r ends up
// with the totals of columns [8r, 8r + 8).  24 shuffles instead of 64.
__device__ __forceinline__ void reduce4_keep8(const float (&v)[32], float (&out)[8]) {
  const int lane = threadIdx.x & 31;
  float a16[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const bool up = lane & 2;
    const float keep = up ? v[i + 16] : v[i], send = up ? v[i] : v[i + 16];
    a16[i] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const bool up = lane & 1;
    const float keep = up ? a16[i + 8] : a16[i], send = up ? a16[i] : a16[i + 8];
    out[i] = keep + __shfl_xor_sync(0xffffffffu, send, 1);
  }
}
// Sum 32 per-thread values over the eight lanes of a warp that share a rank (lanes that differ in bits 2..4); the lane
// with bits (b4 b3 b2) ends up with the totals of columns [16 b4 + 8 b3 + 4 b2, +4).  28 shuffles instead of 96.
__device__ __forceinline__ void reduce8_keep4(const float (&v)[32], float (&out)[4]) {
  const int lane = threadIdx.x & 31;
  float a16[16], a8[8];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const bool up = lane & 16;
    const float keep = up ? v[i + 16] : v[i], send = up ? v[i] : v[i + 16];
    a16[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const bool up = lane & 8;
    const float keep = up ? a16[i + 8] : a16[i], send = up ? a16[i] : a16[i + 8];
    a8[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const bool up = lane & 4;
    const float keep = up ? a8[i + 4] : a8[i], send = up ? a8[i] : a8[i + 4];
    out[i] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
  }
}

// 16-value forms of the two reductions above (used where 32-value arrays would not fit the register budget).
// reduce4_keep4_of16: lane r keeps columns [4r, 4r + 4).  reduce8_keep2_of16: the lane with bits (b4 b3 b2) keeps
// columns 8 b4 + 4 b3 + 2 b2 + {0, 1}.
__device__ __forceinline__ void reduce4_keep4_of16(const float (&v)[16], float (&out)[4]) {
  const int lane = threadIdx.x & 31;
  float a8[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const bool up = lane & 2;
    const float keep = up ? v[i + 8] : v[i], send = up ? v[i] : v[i + 8];
    a8[i] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const bool up = lane & 1;
    const float keep = up ? a8[i + 4] : a8[i], send = up ? a8[i] : a8[i + 4];
    out[i] = keep + __shfl_xor_sync(0xffffffffu, send, 1);
  }
}
__device__ __forceinline__ void reduce8_keep2_of16(const float (&v)[16], float (&out)[2]) {
  const int lane = threadIdx.x & 31;
  float a8[8], a4[4];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const bool up = lane & 16;
    const float keep = up ? v[i + 8] : v[i], send = up ? v[i] : v[i + 8];
    a8[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const bool up = lane & 8;
    const float keep = up ? a8[i + 4] : a8[i], send = up ? a8[i] : a8[i + 4];
    a4[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const bool up = lane & 4;
    const float keep = up ? a4[i + 2] : a4[i], send = up ? a4[i] : a4[i + 2];
    out[i] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
  }
}
__device__ __forceinline__ int reduce8_first_col(int lane) { return ((lane >> 4) & 1) * 8 + ((lane >> 3) & 1) * 4 + ((lane >> 2) & 1) * 2; }

__device__ __forceinline__ float fast_silu(float zz) { return __fdividef(zz, 1.f + __expf(-zz)); }

__device__ __forceinline__ void store_half64(uint8_t* slab, const float (&x)[P / 2], float scale) {
  const int i = threadIdx.x & 127, wg = threadIdx.x >> 7;
#pragma unroll
  for (int c = 0; c < P / 16; ++c) {
    float f[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = x[c * 8 + j] * scale;
    *reinterpret_cast<uint4*>(slab + sw_off(i, wg * 4 + c)) = pack8(f);
  }
}

// Per-head constants staged in shared memory (fp32): Q/K bias [R,N] and the three [R,P] MIMO vectors.
template <int N>
struct HeadBias {
  static constexpr int LD = N + 4;           // padded rank stride (see transform_rows)
  float qb[R * LD];
  float kb[R * LD];
};
struct HeadVecs {
  float psi[R * VLD];
  float zeta[R * VLD];
  float phi[R * VLD];
};
template <int N>
__device__ __forceinline__ void load_head_consts(HeadBias<N>* hb, HeadVecs* hv, const float* __restrict__ Qb,
                                                 const float* __restrict__ Kb, const float* __restrict__ Psi,
                                                 const float* __restrict__ Zeta, const float* __restrict__ Phi, int h) {
  for (int x = threadIdx.x; x < R * N; x += blockDim.x) {
    const int dst = (x / N) * HeadBias<N>::LD + (x % N);
    if (Qb) hb->qb[dst] = Qb[(size_t)h * R * N + x];
    hb->kb[dst] = Kb[(size_t)h * R * N + x];
  }
  for (int x = threadIdx.x; x < R * P; x += blockDim.x) {
    hv->psi[vec_idx(x)] = Psi[(size_t)h * R * P + x];
    if (Zeta) hv->zeta[vec_idx(x)] = Zeta[(size_t)h * R * P + x];
    if (Phi) hv->phi[vec_idx(x)] = Phi[(size_t)h * R * P + x];
  }
}

// Store a [128 x 64] operand row (this thread's row, scaled) as bf16 into a swizzled slab.
__device__ __forceinline__ void store_row64(uint8_t* slab, const float (&x)[P], float scale) {
  const int i = threadIdx.x;
#pragma unroll
  for (int c = 0; c < P / 8; ++c) {
    float f[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = x[c * 8 + j] * scale;
    *reinterpret_cast<uint4*>(slab + sw_off(i, c)) = pack8(f);
  }
}

// 5-D tensor map over an operand stored [B, S, G, R, N] bf16; boxes are [32 tokens, 4 ranks, 64 cols].
int make_tmap_qk(CUtensorMap* out, const void* base, int B, int S, int G, int N);
// 2-D map over [rows, 64] bf16 with boxes of [128, 64].
int make_tmap_rows64(CUtensorMap* out, const void* base, uint64_t rows);

// UMMA descriptors for the tiles used here
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t tile_addr, int kstep) {       // [128 x N] operand, K = N
  return umma_desc_sw128(tile_addr + (kstep >> 2) * SLAB + (kstep & 3) * 32, 16, 1024);
}
__device__ __forceinline__ uint64_t desc_mnmajor_rows(uint32_t slab_addr, int kstep) { // [rows(K) x 64] operand, one slab
  return umma_desc_sw128(slab_addr + kstep * 2048, SLAB, 1024);
}
__device__ __forceinline__ uint64_t desc_mnmajor_2slab(uint32_t tile_addr, int kstep) { // [rows(K) x 128(M)] operand
  return umma_desc_sw128(tile_addr + kstep * 2048, SLAB, 1024);
}

}  // namespace mimo
}  // namespace cm
