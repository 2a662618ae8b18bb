// Mamba3 MIMO scan, backward (see mimo_common.cuh for the forward math and notation).
//
//   grad_state   per chunk:  Gc = Qr^T (e^{cs} o dO),  dO[4t+r] = dy[t] * Phi[r] * silu(Z[t] Zeta[r])
//   state_scan   per (b,h), reverse:  dEnd_c = dStart_{c+1},  dStart_c = e^{tot_c} dEnd_c + Gc
//   chunk_grad   per chunk: everything else, on tcgen05 with all accumulators in TMEM:
//       phase 1  S1 = Qr Kr^T | dPm = dO PV^T | O2 = Qr St | X = Kr dEnd | dQb = dO St^T
//       phase A  M, Pm = S1 o M, dS1 = dPm o M -> smem (bf16);  scalar gradients from dPm o S1
//       phase 2  O1 = Pm PV | dPV1 = Pm^T dO | dQ = dS1 Kr
//       epil. B  O = O1 + e O2 + D PV -> dPhi, dZeta, dZ;  dPV = dPV1 + D dO + w X -> dV, dPsi, dD;  dw, de
//       phase 3  dK = dS1^T Qr + (w o PV) dEnd^T
//       epil. C  dQr = dQ + e dQb, dKr;  inverse rotation -> per-head dQ/dK rows, d(angles)
//   Per-token scalar gradients (d cs, d ts, d gamma) are reduced in shared memory and written as
//   d(ADT) (reverse cumulative sum), d(ts), d(gamma) [B,H,S].
// Replaces the two TileLang backward kernels of the reference (bwd_fwd state recompute + bwd_bwd,
// cppmega/megatron/tilelang_mimo_autograd.py:160-219; mathematics restated at
// cppmega/megatron/cute_dsl_mimo/full_bwd_bwd_epilogue.py:9-348).
#include "mimo_common.cuh"

namespace cm {
namespace mimo {

__device__ __forceinline__ void tma_load_5d_b(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2,
                                              int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2),
      "r"(c3), "r"(c4)
      : "memory");
}

struct BwdArgs {
  const __nv_bfloat16* V;       // [B,S,H,P]
  const __nv_bfloat16* Z;
  const __nv_bfloat16* dY;      // [B,S,H,P]
  const float* ADT;             // [B,H,S]
  const float* DT;
  const float* Trap;
  const float* Qb;              // [H,R,N]
  const float* Kb;
  const float* Psi;             // [H,R,P]
  const float* Zeta;
  const float* Phi;
  const float* angles;          // [B,S,H,NROT]
  const float* Dskip;           // [H]
  float* gbuf;                  // [B,H,C,N,P] fp32 (grad_state output)
  __nv_bfloat16* dQh;           // [B,S,H,R,N]
  __nv_bfloat16* dKh;
  __nv_bfloat16* dV;            // [B,S,H,P]
  __nv_bfloat16* dZ;
  float* dAngles;               // [B,S,H,NROT]
  float* dADT;                  // [B,H,S]
  float* dTs;
  float* dGam;
  float* dPsi;                  // [H,R,P] (atomics)
  float* dZeta;
  float* dPhi;
  float* dD;                    // [H]
  int B, S, H, G, C;
  long long ldV, ldZ;           // token strides of V and Z in elements
  int* err;
  int total_blocks;             // B * H * C
};

__device__ __forceinline__ void decode_block_b(const BwdArgs& a, int x, int& b, int& g, int& c, int& h) {
  const int hpg = a.H / a.G;
  const int hl = x % hpg; x /= hpg;
  c = x % a.C; x /= a.C;
  g = x % a.G; x /= a.G;
  b = x;
  h = g * hpg + hl;
}
__device__ __forceinline__ void decode_block_b(const BwdArgs& a, int& b, int& g, int& c, int& h) {
  decode_block_b(a, (int)blockIdx.x, b, g, c, h);
}

// gating of this thread's row: gate[p] = Phi[r,p] * silu(Z[t,p] * Zeta[r,p]); also returns silu' pieces on demand
__device__ __forceinline__ void load_row_bf16(float (&x)[P], const __nv_bfloat16* __restrict__ base) {
  const uint4* v = reinterpret_cast<const uint4*>(base);
#pragma unroll
  for (int c = 0; c < P / 8; ++c) {
    float f[8];
    unpack8(v[c], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[c * 8 + j] = f[j];
  }
}

// this thread's half row (columns [wg*32, wg*32+32)) of a [.., P] bf16 tensor; `base` points at the row start
__device__ __forceinline__ void load_half_bf16(float (&x)[P / 2], const __nv_bfloat16* __restrict__ base) {
  const uint4* v = reinterpret_cast<const uint4*>(base + (threadIdx.x >> 7) * 32);
#pragma unroll
  for (int c = 0; c < P / 16; ++c) {
    float f[8];
    unpack8(v[c], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[c * 8 + j] = f[j];
  }
}

constexpr int NROT_MAX = 32;
constexpr int THREADS2 = 256;      // two warpgroups: thread (i = tid & 127, wg = tid >> 7) owns half of fused row i

// ------------------------------------------------------------------------------------------
// grad_state: Gc[n,p] = sum_i Qr[i,n] e^{cs_ti} dO[i,p]
// ------------------------------------------------------------------------------------------
template <int N, int NROT>
__global__ void __launch_bounds__(THREADS2) mimo_grad_state_kernel(const __grid_constant__ CUtensorMap tmQ, const BwdArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int QT = (N / 64) * SLAB;
  uint8_t* sQ = smem;
  uint8_t* sdO = sQ + QT;
  float* cos_tab = reinterpret_cast<float*>(sdO + SLAB);
  float* sin_tab = cos_tab + tab_floats<NROT>();
  HeadBias<N>* hb = reinterpret_cast<HeadBias<N>*>(sin_tab + tab_floats<NROT>());
  HeadVecs* hv = reinterpret_cast<HeadVecs*>(hb + 1);
  ChunkScalars* sc = reinterpret_cast<ChunkScalars*>(hv + 1);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sc + 1);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  if (a.err && *reinterpret_cast<volatile int*>(a.err) != 0) return;   // an earlier CTA / kernel gave up: drain
  int b, g, c, h;
  decode_block_b(a, b, g, c, h);
  const int t0 = c * LT;
  const int i = threadIdx.x & 127, wg = threadIdx.x >> 7, t = i >> 2, r = i & 3, warp = threadIdx.x >> 5;
  // every global load of the prologue is issued here, ahead of the set-up, and consumed further down
  const ScalarLoads sl = load_chunk_scalars(a.ADT, a.DT, a.Trap, ((size_t)b * a.H + h) * a.S + t0, t0, a.S);
  const float4 ang4 = load_angles4<NROT>(a.angles, b, t0, h, a.S, a.H);
  const HalfRowRaw yraw = load_half_raw(a.dY, b, t0, h, a.S, (long long)a.H * P);
  const HalfRowRaw zraw = load_half_raw(a.Z, b, t0, h, a.S, a.ldZ);
  if (threadIdx.x == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) { tmem_alloc(tmem_slot, 64); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  if (threadIdx.x == 0) {
    mbar_expect_tx(&bars[0], QT);
#pragma unroll
    for (int s = 0; s < N / 64; ++s) tma_load_5d_b(sQ + s * SLAB, &tmQ, &bars[0], s * 64, 0, g, t0, b);
  }
  load_head_consts<N>(hb, hv, a.Qb, a.Qb, a.Phi, a.Zeta, a.Phi, h);
  finish_chunk_scalars(sc, sl, t0, a.S);
  fill_sincos4<NROT>(cos_tab, sin_tab, ang4);
  __syncthreads();
  bool ok = mbar_wait(&bars[0], 0, abort_flag, a.err, ERR_WAIT_FULL);
  if (ok) {
    transform_rows<N, NROT, 2, HeadBias<N>::LD>(sQ, hb->qb, cos_tab, sin_tab);
    float dy[P / 2], z[P / 2];
    half_raw_to_float(dy, yraw);
    half_raw_to_float(z, zraw);
    const float* zeta = hv->zeta + r * VLD + wg * 32;
    const float* phi = hv->phi + r * VLD + wg * 32;
    const float e = __expf(sc->cs[t]);
#pragma unroll
    for (int p = 0; p < P / 2; ++p) dy[p] = dy[p] * phi[p] * fast_silu(z[p] * zeta[p]);
    store_half64(sdO, dy, e);
    fence_proxy_async_smem();
  }
  __syncthreads();
  if (threadIdx.x == 0 && !*abort_flag) {
    constexpr uint32_t idesc = umma_idesc_bf16(N, P, true, true);
    const uint32_t aQ = smem_u32(sQ), aO = smem_u32(sdO);
#pragma unroll
    for (int k = 0; k < ROWS / 16; ++k) umma_f16(tmem, desc_mnmajor_2slab(aQ, k), desc_mnmajor_rows(aO, k), idesc, k != 0);
    umma_commit(&bars[1]);
  }
  ok = mbar_wait(&bars[1], 0, abort_flag, a.err, ERR_WAIT_TMEM_FULL);
  tc_fence_after();
  if (ok) {
    float* dst = a.gbuf + ((((size_t)b * a.H + h) * a.C + c) * N + i) * P + wg * 32;
    uint32_t rr[32];
    tmem_ld_32x32(tmem + (uint32_t((warp & 3) * 32) << 16) + wg * 32, rr);
    tmem_ld_wait();
#pragma unroll
    for (int v = 0; v < 8; ++v)
      reinterpret_cast<float4*>(dst)[v] = make_float4(__uint_as_float(rr[4 * v]), __uint_as_float(rr[4 * v + 1]),
                                                      __uint_as_float(rr[4 * v + 2]), __uint_as_float(rr[4 * v + 3]));
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem, 64); }
}

// reverse scan: dEnd[c] = state; state = e^{tot_c} state + G[c]  for c = C-1 .. 0
__global__ void __launch_bounds__(256) mimo_state_scan_rev_kernel(const float* __restrict__ gbuf, const float* __restrict__ tot,
                                                                  __nv_bfloat16* __restrict__ dend, int C, int NP) {
  const size_t bh = blockIdx.x;
  const int e = (blockIdx.y * 256 + threadIdx.x) * 4;
  if (e >= NP) return;
  float4 st = make_float4(0.f, 0.f, 0.f, 0.f);
  const float* gp = gbuf + bh * (size_t)C * NP + e;
  __nv_bfloat16* dp = dend + bh * (size_t)C * NP + e;
  const float* tp = tot + bh * C;
  for (int c = C - 1; c >= 0; --c) {
    const float4 cur = *reinterpret_cast<const float4*>(gp + (size_t)c * NP);
    uint2 o;
    o.x = pack_bf16(st.x, st.y);
    o.y = pack_bf16(st.z, st.w);
    *reinterpret_cast<uint2*>(dp + (size_t)c * NP) = o;
    const float d = __expf(tp[c]);
    st.x = d * st.x + cur.x; st.y = d * st.y + cur.y; st.z = d * st.z + cur.z; st.w = d * st.w + cur.w;
  }
}

// ------------------------------------------------------------------------------------------
// chunk_grad
// ------------------------------------------------------------------------------------------
struct GradScratch {
  float dcs[LT];
  float dts[LT];
  float dgam[LT];
  float dtot;
  float dD;
  float par[3][4][R][VLD];   // per-lane-quarter partials of dPsi, dZeta, dPhi (each warpgroup fills its own columns)
  float dang[LT][NROT_MAX + 4];  // K-side d(angle) partials (padded rows: eight tokens of a warp write one column) handed from warpgroup 1 to warpgroup 0
};

template <int N, int NROT>
__global__ void __launch_bounds__(THREADS2, 1) mimo_chunk_grad_kernel(const __grid_constant__ CUtensorMap tmQ,
                                                                      const __grid_constant__ CUtensorMap tmK,
                                                                      const __grid_constant__ CUtensorMap tmS,
                                                                      const __grid_constant__ CUtensorMap tmE, const BwdArgs a) {
  static_assert(N == 128, "chunk_grad is written for a 128-wide state");
  static_assert(NROT <= NROT_MAX && NROT / 8 == R, "rank r writes the r-th group of eight angles");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                    // 32 KB
  uint8_t* sK = sQ + 2 * SLAB;           // 32 KB
  uint8_t* sPV = sK + 2 * SLAB;          // 16 KB
  uint8_t* sdO = sPV + SLAB;             // 16 KB
  uint8_t* sSt = sdO + SLAB;             // 16 KB  start state [n x p]
  uint8_t* sdE = sSt + SLAB;             // 16 KB  gradient of the end state [n x p]
  uint8_t* sPm = sdE + SLAB;             // 32 KB
  uint8_t* sdS = sPm + 2 * SLAB;         // 32 KB
  uint8_t* sPVw = sdS + 2 * SLAB;        // 16 KB
  float* cos_tab = reinterpret_cast<float*>(sPVw + SLAB);
  float* sin_tab = cos_tab + tab_floats<NROT>();
  HeadVecs* hv = reinterpret_cast<HeadVecs*>(sin_tab + tab_floats<NROT>());
  ChunkScalars* sc = reinterpret_cast<ChunkScalars*>(hv + 1);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sc + 1);             // tma, ph1, ph2, ph3
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  // colsum [8 warps][2][16] floats follow the abort flag; the head biases and later the reduction scratch alias Pm
  // (biases die before phase A writes Pm; the scratch is used only after phase 2 has read it)
  static_assert(sizeof(GradScratch) <= 2 * SLAB && sizeof(HeadBias<N>) <= 2 * SLAB, "scratch must fit the Pm tile");

  if (a.err && *reinterpret_cast<volatile int*>(a.err) != 0) return;   // an earlier CTA / kernel gave up: drain
  const int tid = threadIdx.x;
  const int i = tid & 127, wg = tid >> 7, t = i >> 2, r = i & 3, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int q = 0; q < 4; ++q) mbar_init(&bars[q], 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  // Persistent: one CTA per SM walks the chunks with a grid stride; barriers, TMEM and the kernel prologue are paid
  // once, and every barrier completes exactly one phase per chunk, so its parity is the iteration's low bit.
  uint32_t par = 0;
#pragma unroll 1
  for (int xblk = blockIdx.x; xblk < a.total_blocks; xblk += gridDim.x, par ^= 1) {
  // Re-derive every shared-memory address from a value the compiler cannot see through: otherwise the addresses and
  // the ~80 MMA descriptors built from them are hoisted out of this loop and spill the 255-register budget.
  uint8_t* smem_l;
  asm volatile("mov.u64 %0, %1;" : "=l"(smem_l) : "l"(smem));
  uint8_t* sQ = smem_l;
  uint8_t* sK = sQ + 2 * SLAB;
  uint8_t* sPV = sK + 2 * SLAB;
  uint8_t* sdO = sPV + SLAB;
  uint8_t* sSt = sdO + SLAB;
  uint8_t* sdE = sSt + SLAB;
  uint8_t* sPm = sdE + SLAB;
  uint8_t* sdS = sPm + 2 * SLAB;
  uint8_t* sPVw = sdS + 2 * SLAB;
  float* cos_tab = reinterpret_cast<float*>(sPVw + SLAB);
  float* sin_tab = cos_tab + tab_floats<NROT>();
  HeadVecs* hv = reinterpret_cast<HeadVecs*>(sin_tab + tab_floats<NROT>());
  ChunkScalars* sc = reinterpret_cast<ChunkScalars*>(hv + 1);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sc + 1);
  float* colsum = reinterpret_cast<float*>(reinterpret_cast<uint32_t*>(bars + 4) + 4);
  HeadBias<N>* hb = reinterpret_cast<HeadBias<N>*>(sPm);
  GradScratch* gs = reinterpret_cast<GradScratch*>(sPm);
  int b, g, c, h;
  decode_block_b(a, xblk, b, g, c, h);
  const int t0 = c * LT;
  // every global load of the prologue is issued here, ahead of the set-up, and consumed further down
  const ScalarLoads sl = load_chunk_scalars(a.ADT, a.DT, a.Trap, ((size_t)b * a.H + h) * a.S + t0, t0, a.S);
  const float4 ang4 = load_angles4<NROT>(a.angles, b, t0, h, a.S, a.H);
  const HalfRowRaw vraw = load_half_raw(a.V, b, t0, h, a.S, a.ldV);
  const HalfRowRaw yraw = load_half_raw(a.dY, b, t0, h, a.S, (long long)a.H * P);
  const HalfRowRaw zraw = load_half_raw(a.Z, b, t0, h, a.S, a.ldZ);
  const uint32_t lane_addr = uint32_t((warp & 3) * 32) << 16;
  // phase 1 accumulators                      phase 2 / 3 accumulators
  const uint32_t tS1 = tmem, tdPm = tmem + 128, tO2 = tmem + 256, tX = tmem + 320, tdQb = tmem + 384;
  const uint32_t tO1 = tmem, tdPV1 = tmem + 64, tdQ = tmem + 128, tdK = tmem + 256;

  if (tid == 0) {
    mbar_expect_tx(&bars[0], 4 * SLAB + 2 * SLAB);
    for (int s = 0; s < 2; ++s) {
      tma_load_5d_b(sQ + s * SLAB, &tmQ, &bars[0], s * 64, 0, g, t0, b);
      tma_load_5d_b(sK + s * SLAB, &tmK, &bars[0], s * 64, 0, g, t0, b);
    }
    const int srow = (int)((((size_t)b * a.H + h) * a.C + c) * N);
    tma_load_2d(sSt, &tmS, &bars[0], 0, srow);
    tma_load_2d(sdE, &tmE, &bars[0], 0, srow);
  }
  load_head_consts<N>(hb, hv, a.Qb, a.Kb, a.Psi, a.Zeta, a.Phi, h);
  finish_chunk_scalars(sc, sl, t0, a.S);
  fill_sincos4<NROT>(cos_tab, sin_tab, ang4);
  __syncthreads();
  const size_t rowoff = (((size_t)b * a.S + t0 + t) * a.H + h) * P + wg * 32;     // this thread's half row
  const float* zeta = hv->zeta + r * VLD + wg * 32;
  const float* phi = hv->phi + r * VLD + wg * 32;
  const float* psi = hv->psi + r * VLD + wg * 32;
  const float csi = sc->cs[t], gi = sc->gam[t], tsi = sc->ts[t], tot = sc->tot;
  const float ei = __expf(csi);
  const float wi = tsi * __expf(tot - csi);
  const float dsk = a.Dskip[h];

  bool ok = mbar_wait(&bars[0], par, abort_flag, a.err, ERR_WAIT_FULL);
  if (ok) {
    transform_rows<N, NROT, 2, HeadBias<N>::LD>(sQ, hb->qb, cos_tab, sin_tab);
    transform_rows<N, NROT, 2, HeadBias<N>::LD>(sK, hb->kb, cos_tab, sin_tab);
    {
      float pv[P / 2];
      pv_from_raw(pv, vraw, hv->psi);
      store_half64(sPV, pv, 1.f);
      store_half64(sPVw, pv, wi);
    }
    {
      float dy[P / 2], z[P / 2];
      half_raw_to_float(dy, yraw);
      half_raw_to_float(z, zraw);
#pragma unroll
      for (int p = 0; p < P / 2; ++p) dy[p] = dy[p] * phi[p] * fast_silu(z[p] * zeta[p]);
      store_half64(sdO, dy, 1.f);
    }
    fence_proxy_async_smem();
  }
  __syncthreads();
  const uint32_t aQ = smem_u32(sQ), aK = smem_u32(sK), aPV = smem_u32(sPV), adO = smem_u32(sdO), aSt = smem_u32(sSt),
                 adE = smem_u32(sdE), aPm = smem_u32(sPm), adS = smem_u32(sdS), aPVw = smem_u32(sPVw);
  constexpr uint32_t id_128_kk = umma_idesc_bf16(ROWS, 128, false, false);
  constexpr uint32_t id_64_km = umma_idesc_bf16(ROWS, P, false, true);
  constexpr uint32_t id_64_mm = umma_idesc_bf16(ROWS, P, true, true);
  constexpr uint32_t id_128_km = umma_idesc_bf16(ROWS, 128, false, true);
  constexpr uint32_t id_128_mm = umma_idesc_bf16(ROWS, 128, true, true);
  if (tid == 0 && !*abort_flag) {
#pragma unroll
    for (int k = 0; k < 8; ++k) umma_f16(tS1, desc_kmajor(aQ, k), desc_kmajor(aK, k), id_128_kk, k != 0);
#pragma unroll
    for (int k = 0; k < 4; ++k) umma_f16(tdPm, desc_kmajor(adO, k), desc_kmajor(aPV, k), id_128_kk, k != 0);
#pragma unroll
    for (int k = 0; k < 8; ++k) umma_f16(tO2, desc_kmajor(aQ, k), desc_mnmajor_rows(aSt, k), id_64_km, k != 0);
#pragma unroll
    for (int k = 0; k < 8; ++k) umma_f16(tX, desc_kmajor(aK, k), desc_mnmajor_rows(adE, k), id_64_km, k != 0);
#pragma unroll
    for (int k = 0; k < 4; ++k) umma_f16(tdQb, desc_kmajor(adO, k), desc_kmajor(aSt, k), id_128_kk, k != 0);
    umma_commit(&bars[1]);
  }
  // while the tensor core works: d tot from the state decay, e^{tot} * <dEnd, St> (state row n = i, half of its columns)
  float dtot_part = 0.f;
  if (ok) {
#pragma unroll
    for (int c2 = 0; c2 < 4; ++c2) {
      const int cidx = wg * 4 + c2;
      float s8[8], e8[8];
      unpack8(*reinterpret_cast<const uint4*>(sSt + sw_off(i, cidx)), s8);
      unpack8(*reinterpret_cast<const uint4*>(sdE + sw_off(i, cidx)), e8);
#pragma unroll
      for (int j = 0; j < 8; ++j) dtot_part += s8[j] * e8[j];
    }
    dtot_part *= __expf(tot);
  }
  ok = __syncthreads_and(mbar_wait(&bars[1], par, abort_flag, a.err, ERR_WAIT_TMEM_FULL));
  tc_fence_after();

  // ---------------- phase A: masks, Pm, dS1, scalar gradients from dM = dPm o S1 ----------------
  // this warpgroup's key tokens: [16 wg, 16 wg + 16)
  float rowR = 0.f, dgam_i = 0.f;
  float colC[LT / 2], colT[LT / 2];
  if (ok) {
#pragma unroll
    for (int c2 = 0; c2 < 2; ++c2) {
      const int cc = wg * 2 + c2;
      uint32_t s1[32], dp[32];
      tmem_ld_32x32(tS1 + lane_addr + cc * 32, s1);
      tmem_ld_32x32(tdPm + lane_addr + cc * 32, dp);
      tmem_ld_wait();
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float fp[8], fd[8];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int tl = c2 * 8 + q * 2 + u;          // local key-token index, 0..15
          const int tj = wg * 16 + tl;
          float ex = 0.f, m = 0.f;
          if (tj < t) { ex = __expf(csi - sc->cs[tj]); m = sc->ts[tj] * ex; }
          else if (tj == t) m = gi;
          float dmsum = 0.f;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const float sv = __uint_as_float(s1[q * 8 + u * 4 + v]);
            const float dv = __uint_as_float(dp[q * 8 + u * 4 + v]);
            fp[u * 4 + v] = sv * m;
            fd[u * 4 + v] = dv * m;
            dmsum += sv * dv;
          }
          if (tj < t) {
            rowR += dmsum * m;
            colC[tl] = dmsum * m;
            colT[tl] = dmsum * ex;
          } else {
            colC[tl] = 0.f;
            colT[tl] = 0.f;
            if (tj == t) dgam_i += dmsum;
          }
        }
        const int col = cc * 32 + q * 8;
        *reinterpret_cast<uint4*>(sPm + (col / 64) * SLAB + sw_off(i, (col % 64) / 8)) = pack8(fp);
        *reinterpret_cast<uint4*>(sdS + (col / 64) * SLAB + sw_off(i, (col % 64) / 8)) = pack8(fd);
      }
    }
    fence_proxy_async_smem();
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && !*abort_flag) {
    tc_fence_after();
#pragma unroll
    for (int k = 0; k < 8; ++k) umma_f16(tO1, desc_kmajor(aPm, k), desc_mnmajor_rows(aPV, k), id_64_km, k != 0);
#pragma unroll
    for (int k = 0; k < 8; ++k) umma_f16(tdPV1, desc_mnmajor_2slab(aPm, k), desc_mnmajor_rows(adO, k), id_64_mm, k != 0);
#pragma unroll
    for (int k = 0; k < 8; ++k) umma_f16(tdQ, desc_kmajor(adS, k), desc_mnmajor_2slab(aK, k), id_128_km, k != 0);
    umma_commit(&bars[2]);
  }
  // column sums over the rows of this warp while phase 2 runs
  if (ok) {
#pragma unroll
    for (int tl = 0; tl < LT / 2; ++tl) {
      const float c_ = warp_sum(colC[tl]);
      const float t_ = warp_sum(colT[tl]);
      if (lane == tl) { colsum[(warp * 2 + 0) * (LT / 2) + tl] = c_; colsum[(warp * 2 + 1) * (LT / 2) + tl] = t_; }
    }
  }
  ok = __syncthreads_and(mbar_wait(&bars[2], par, abort_flag, a.err, ERR_WAIT_TMEM_FULL));
  tc_fence_after();
  // Pm has been consumed by phase 2: its space becomes the reduction scratch
  if (tid < LT) { gs->dcs[tid] = 0.f; gs->dts[tid] = 0.f; gs->dgam[tid] = 0.f; }
  if (tid == 0) { gs->dtot = 0.f; gs->dD = 0.f; }
  __syncthreads();

  // ---------------- epilogue B: gating gradients, dPV, dw, de (this warpgroup's 32 columns) ----------------
  float dw_i = 0.f, de_i = 0.f;
  if (ok) {
    const uint4* vrow = vraw.v;
    const uint4* yrow = yraw.v;
    const uint4* zrow = zraw.v;
    const int wq = warp & 3;
    float dD_part = 0.f;
    float dvrow[32];
    const int pcol = reduce8_first_col(lane);         // first of the two columns (per 16) this lane owns after reduce8
    {   // pass 1: O = O1 + e O2 + D PV  ->  dPhi, dZeta, dZ, de, dD and the D dO part of dPV
      uint32_t o1[32], o2[32];
      tmem_ld_32x32(tO1 + lane_addr + wg * 32, o1);
      tmem_ld_32x32(tO2 + lane_addr + wg * 32, o2);
      tmem_ld_wait();
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        float aphi[16], azeta[16], apsi[16], adz[16];
#pragma unroll
        for (int q2 = 0; q2 < 2; ++q2) {
          const int q = half * 2 + q2;
          float vf[8], yf[8], zf[8];
          unpack8(vrow[q], vf);
          unpack8(yrow[q], yf);
          unpack8(zrow[q], zf);
#pragma unroll
          for (int v = 0; v < 8; ++v) {
            const int e = q * 8 + v, c = q2 * 8 + v;
            const float pvv = vf[v] * psi[e];
            const float o2v = __uint_as_float(o2[e]);
            const float o = __uint_as_float(o1[e]) + ei * o2v + dsk * pvv;
            const float zz = zf[v] * zeta[e];
            const float sg = __fdividef(1.f, 1.f + __expf(-zz));
            const float sil = zz * sg;
            const float dO = yf[v] * phi[e] * sil;
            const float dgate = yf[v] * o;
            const float dzz = dgate * phi[e] * sg * (1.f + zz * (1.f - sg));
            aphi[c] = dgate * sil;
            azeta[c] = dzz * zf[v];
            apsi[c] = dsk * dO * vf[v];
            adz[c] = dzz * zeta[e];
            de_i += dO * o2v;
            dD_part += dO * pvv;
            dvrow[e] = dsk * dO * psi[e];
          }
        }
        float r2[2], mz[4];
        const int col = wg * 32 + half * 16 + pcol;
        reduce8_keep2_of16(apsi, r2);
        gs->par[0][wq][r][col] = r2[0]; gs->par[0][wq][r][col + 1] = r2[1];
        reduce8_keep2_of16(azeta, r2);
        gs->par[1][wq][r][col] = r2[0]; gs->par[1][wq][r][col + 1] = r2[1];
        reduce8_keep2_of16(aphi, r2);
        gs->par[2][wq][r][col] = r2[0]; gs->par[2][wq][r][col + 1] = r2[1];
        reduce4_keep4_of16(adz, mz);
        uint2 oz;
        oz.x = pack_bf16(mz[0], mz[1]);
        oz.y = pack_bf16(mz[2], mz[3]);
        *reinterpret_cast<uint2*>(a.dZ + rowoff + half * 16 + r * 4) = oz;
      }
    }
    {   // pass 2: dPV = dPV1 + w X (+ D dO from pass 1)  ->  dV, dPsi, dw
      uint32_t d1[32], xx[32];
      tmem_ld_32x32(tdPV1 + lane_addr + wg * 32, d1);
      tmem_ld_32x32(tX + lane_addr + wg * 32, xx);
      tmem_ld_wait();
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        float apsi[16];
#pragma unroll
        for (int q2 = 0; q2 < 2; ++q2) {
          const int q = half * 2 + q2;
          float vf[8];
          unpack8(vrow[q], vf);
#pragma unroll
          for (int v = 0; v < 8; ++v) {
            const int e = q * 8 + v;
            const float xv = __uint_as_float(xx[e]);
            const float dpv = __uint_as_float(d1[e]) + wi * xv;
            dw_i += vf[v] * psi[e] * xv;
            apsi[q2 * 8 + v] = dpv * vf[v];
            dvrow[e] += dpv * psi[e];
          }
        }
        float r2[2];
        const int col = wg * 32 + half * 16 + pcol;
        reduce8_keep2_of16(apsi, r2);                 // same lane owns the same columns as in pass 1
        gs->par[0][wq][r][col] += r2[0]; gs->par[0][wq][r][col + 1] += r2[1];
      }
      float mv[8];
      reduce4_keep8(dvrow, mv);
      *reinterpret_cast<uint4*>(a.dV + rowoff + r * 8) = pack8(mv);
    }
    dD_part = warp_sum(dD_part);
    if (lane == 0) atomicAdd(&gs->dD, dD_part);
    // per-token scalar gradients (each warpgroup adds the part that comes from its columns)
    //   cs_ti:  + rowR + e_i de_i - w_i dw_i         ts_ti: + dw_i e^{tot-cs_ti}       gamma_ti: + dgam_i
    const float ewi = __expf(tot - csi);
    float dcs_row = rowR + ei * de_i - wi * dw_i;
    float dts_row = dw_i * ewi;
    float dgm_row = dgam_i;
    float dtot_row = wi * dw_i + dtot_part;
    dcs_row += __shfl_xor_sync(0xffffffffu, dcs_row, 1); dcs_row += __shfl_xor_sync(0xffffffffu, dcs_row, 2);
    dts_row += __shfl_xor_sync(0xffffffffu, dts_row, 1); dts_row += __shfl_xor_sync(0xffffffffu, dts_row, 2);
    dgm_row += __shfl_xor_sync(0xffffffffu, dgm_row, 1); dgm_row += __shfl_xor_sync(0xffffffffu, dgm_row, 2);
    dtot_row = warp_sum(dtot_row);
    if (r == 0) {
      atomicAdd(&gs->dcs[t], dcs_row);
      atomicAdd(&gs->dts[t], dts_row);
      atomicAdd(&gs->dgam[t], dgm_row);
    }
    if (lane == 0) atomicAdd(&gs->dtot, dtot_row);
    // column sums from phase A: lane tl of every warp adds the totals of key token 16 wg + tl
    if (lane < LT / 2) {
      atomicAdd(&gs->dcs[wg * 16 + lane], -colsum[(warp * 2 + 0) * (LT / 2) + lane]);
      atomicAdd(&gs->dts[wg * 16 + lane], colsum[(warp * 2 + 1) * (LT / 2) + lane]);
    }
  }
  tc_fence_before();
  __syncthreads();
  // ---------------- phase 3: dK ----------------
  if (tid == 0 && !*abort_flag) {
    tc_fence_after();
#pragma unroll
    for (int k = 0; k < 8; ++k) umma_f16(tdK, desc_mnmajor_2slab(adS, k), desc_mnmajor_2slab(aQ, k), id_128_mm, k != 0);
#pragma unroll
    for (int k = 0; k < 4; ++k) umma_f16(tdK, desc_kmajor(aPVw, k), desc_kmajor(adE, k), id_128_kk, 1);
    umma_commit(&bars[3]);
  }
  // finish the scalar and parameter gradients while phase 3 runs
  if (ok) {
    if (warp == 0) {
      // d(ADT)[s] = sum_{t >= s} dcs[t]  (+ dtot on the last token)
      float v = gs->dcs[lane] + (lane == LT - 1 ? gs->dtot : 0.f);
#pragma unroll
      for (int o_ = 1; o_ < 32; o_ <<= 1) {
        const float n_ = __shfl_down_sync(0xffffffffu, v, o_);
        if (lane + o_ < 32) v += n_;
      }
      const size_t sb = ((size_t)b * a.H + h) * a.S + t0 + lane;
      a.dADT[sb] = v;
      a.dTs[sb] = gs->dts[lane];
      a.dGam[sb] = gs->dgam[lane];
    }
    {
      const int e = tid;                                   // R * P == 256 == THREADS2
      const int rr = e / P, pp = e % P;
      float s0 = 0.f, s1 = 0.f, s2 = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) { s0 += gs->par[0][w][rr][pp]; s1 += gs->par[1][w][rr][pp]; s2 += gs->par[2][w][rr][pp]; }
      atomicAdd(a.dPsi + (size_t)h * R * P + e, s0);
      atomicAdd(a.dZeta + (size_t)h * R * P + e, s1);
      atomicAdd(a.dPhi + (size_t)h * R * P + e, s2);
    }
    if (tid == 0) atomicAdd(a.dD + h, gs->dD);
  }
  ok = __syncthreads_and(mbar_wait(&bars[3], par, abort_flag, a.err, ERR_WAIT_TMEM_FULL));
  tc_fence_after();
  // ---------------- epilogue C: dQr = dQ + e dQb (warpgroup 0), dKr (warpgroup 1); inverse rotation; d(angles) ----
  float dang[NROT / 8][8];
  if (ok) {
    constexpr int HALF = N / 2;
#pragma unroll
    for (int x = 0; x < NROT / 8; ++x)
#pragma unroll
      for (int j = 0; j < 8; ++j) dang[x][j] = 0.f;
    const bool isq = wg == 0;
    const uint8_t* tile = isq ? sQ : sK;                 // rotated operand rows (bf16) for d(angle)
    __nv_bfloat16* drow = (isq ? a.dQh : a.dKh) + ((((size_t)b * a.S + t0 + t) * a.H + h) * R + r) * N;
    const uint32_t tacc = isq ? tdQ : tdK;
    // columns [0,32) pair with [64,96); [32,64) and [96,128) are not rotated
    uint32_t lo[32], hi[32];
    tmem_ld_32x32(tacc + lane_addr + 0, lo);
    tmem_ld_32x32(tacc + lane_addr + HALF, hi);
    tmem_ld_wait();
    if (isq) {
      uint32_t lob[32], hib[32];
      tmem_ld_32x32(tdQb + lane_addr + 0, lob);
      tmem_ld_32x32(tdQb + lane_addr + HALF, hib);
      tmem_ld_wait();
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        lo[e] = __float_as_uint(__uint_as_float(lo[e]) + ei * __uint_as_float(lob[e]));
        hi[e] = __float_as_uint(__uint_as_float(hi[e]) + ei * __uint_as_float(hib[e]));
      }
    }
#pragma unroll
    for (int x = 0; x < NROT / 8; ++x) {
      float xa[8], xb[8], ga[8], gb[8];
      unpack8(*reinterpret_cast<const uint4*>(tile + sw_off(i, x)), xa);                 // rotated values, cols 8x..
      unpack8(*reinterpret_cast<const uint4*>(tile + SLAB + sw_off(i, x)), xb);          // cols 64+8x..
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float da = __uint_as_float(lo[x * 8 + j]), db = __uint_as_float(hi[x * 8 + j]);
        const float cs_ = cos_tab[t * tab_stride<NROT>() + x * 8 + j], sn_ = sin_tab[t * tab_stride<NROT>() + x * 8 + j];
        dang[x][j] += db * xa[j] - da * xb[j];
        ga[j] = cs_ * da + sn_ * db;
        gb[j] = -sn_ * da + cs_ * db;
      }
      *reinterpret_cast<uint4*>(drow + x * 8) = pack8(ga);
      *reinterpret_cast<uint4*>(drow + HALF + x * 8) = pack8(gb);
    }
    // un-rotated halves
    tmem_ld_32x32(tacc + lane_addr + NROT, lo);
    tmem_ld_32x32(tacc + lane_addr + HALF + NROT, hi);
    tmem_ld_wait();
    if (isq) {
      uint32_t lob[32], hib[32];
      tmem_ld_32x32(tdQb + lane_addr + NROT, lob);
      tmem_ld_32x32(tdQb + lane_addr + HALF + NROT, hib);
      tmem_ld_wait();
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        lo[e] = __float_as_uint(__uint_as_float(lo[e]) + ei * __uint_as_float(lob[e]));
        hi[e] = __float_as_uint(__uint_as_float(hi[e]) + ei * __uint_as_float(hib[e]));
      }
    }
#pragma unroll
    for (int x = 0; x < (HALF - NROT) / 8; ++x) {
      float ga[8], gb[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        ga[j] = __uint_as_float(lo[x * 8 + j]);
        gb[j] = __uint_as_float(hi[x * 8 + j]);
      }
      *reinterpret_cast<uint4*>(drow + NROT + x * 8) = pack8(ga);
      *reinterpret_cast<uint4*>(drow + HALF + NROT + x * 8) = pack8(gb);
    }
    // sum over the four ranks; warpgroup 1 (K side) hands its part over through shared memory
#pragma unroll
    for (int x = 0; x < NROT / 8; ++x) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float v = dang[x][j];
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        dang[x][j] = v;
      }
      if (!isq && x == r) {
#pragma unroll
        for (int j = 0; j < 8; ++j) gs->dang[t][x * 8 + j] = dang[x][j];
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (ok && wg == 0) {
    float* darow = a.dAngles + (((size_t)b * a.S + t0 + t) * a.H + h) * NROT;
#pragma unroll
    for (int x = 0; x < NROT / 8; ++x) {
      if (x == r) {       // NROT/8 == 4 == R: rank r writes the r-th group of 8 angles
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = dang[x][j] + gs->dang[t][x * 8 + j];
        reinterpret_cast<float4*>(darow + x * 8)[0] = make_float4(o[0], o[1], o[2], o[3]);
        reinterpret_cast<float4*>(darow + x * 8)[1] = make_float4(o[4], o[5], o[6], o[7]);
      }
    }
  }
  // the next chunk's TMA loads and MMAs overwrite the tiles and accumulators every thread has just finished with
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (*abort_flag) break;
  }
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

constexpr int grad_state_smem() {
  return 2 * SLAB + SLAB + 2 * tab_floats<32>() * 4 + (int)sizeof(HeadBias<128>) + (int)sizeof(HeadVecs) + (int)sizeof(ChunkScalars) + 64 + 1024;
}
constexpr int chunk_grad_smem() {
  return 13 * SLAB + 2 * tab_floats<32>() * 4 + (int)sizeof(HeadVecs) + (int)sizeof(ChunkScalars) + 64 + 1024 + 1024;
}

}  // namespace mimo
}  // namespace cm

using namespace cm;
using namespace cm::mimo;

// Inputs as in cm_mimo_scan_fwd plus dY [B,S,H,P] bf16, the forward's `states` (start states, bf16) and `tot`.
// Scratch: gbuf [B,H,C,N,P] fp32, dend [B,H,C,N,P] bf16.
// Outputs: dQh, dKh [B,S,H,R,N] bf16 (per head, before the group reduction); dV, dZ [B,S,H,P] bf16;
// dAngles [B,S,H,N/4] fp32; dADT, dTs, dGam [B,H,S] fp32; dPsi, dZeta, dPhi [H,R,P], dD [H] fp32 (accumulated:
// the caller zeroes them).
extern "C" int cm_mimo_scan_bwd(const void* Qn, const void* Kn, const void* V, const void* Z, const void* dY,
                                const float* ADT, const float* DT, const float* Trap, const float* Qb, const float* Kb,
                                const float* Psi, const float* Zeta, const float* Phi, const float* angles,
                                const float* Dskip, const void* states, const float* tot, float* gbuf, void* dend,
                                void* dQh, void* dKh, void* dV, void* dZ, float* dAngles, float* dADT, float* dTs,
                                float* dGam, float* dPsi, float* dZeta, float* dPhi, float* dD_, int B, int S, int H, int G,
                                int N, long long ldV, long long ldZ, int* err, cudaStream_t stream) {
  if (B <= 0 || S <= 0) return 0;
  if (S % LT || N != 128 || H % G) return -10;
  if (ldV < (long long)H * P || ldZ < (long long)H * P || ldV % 8 || ldZ % 8) return -11;
  const int C = S / LT;
  CUtensorMap tmQ, tmK, tmS, tmE;
  int rc = make_tmap_qk(&tmQ, Qn, B, S, G, N);
  if (rc) return rc;
  rc = make_tmap_qk(&tmK, Kn, B, S, G, N);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tmS, states, (uint64_t)B * H * C * N, 64, 64, 128, 64);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tmE, dend, (uint64_t)B * H * C * N, 64, 64, 128, 64);
  if (rc) return rc;
  BwdArgs a{(const __nv_bfloat16*)V, (const __nv_bfloat16*)Z, (const __nv_bfloat16*)dY, ADT, DT, Trap, Qb, Kb, Psi, Zeta,
            Phi, angles, Dskip, gbuf, (__nv_bfloat16*)dQh, (__nv_bfloat16*)dKh, (__nv_bfloat16*)dV, (__nv_bfloat16*)dZ,
            dAngles, dADT, dTs, dGam, dPsi, dZeta, dPhi, dD_, B, S, H, G, C, ldV, ldZ, err, B * H * C};
  auto k0 = mimo_grad_state_kernel<128, 32>;
  auto k2 = mimo_chunk_grad_kernel<128, 32>;
  static PerDevice cfg;
  if (cfg.first()) {
    if (cudaFuncSetAttribute(k0, cudaFuncAttributeMaxDynamicSharedMemorySize, grad_state_smem()) != cudaSuccess) return -2;
    if (cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, chunk_grad_smem()) != cudaSuccess) return -2;
    cfg.done();
  }
  const int grid = B * H * C;
  k0<<<grid, THREADS2, grad_state_smem(), stream>>>(tmQ, a);
  dim3 g2(B * H, (128 * P + 1023) / 1024);
  mimo_state_scan_rev_kernel<<<g2, 256, 0, stream>>>(gbuf, tot, (__nv_bfloat16*)dend, C, 128 * P);
  k2<<<grid < sm_count() ? grid : sm_count(), THREADS2, chunk_grad_smem(), stream>>>(tmQ, tmK, tmS, tmE, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

