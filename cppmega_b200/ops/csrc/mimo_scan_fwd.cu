// Mamba3 MIMO scan, forward: three kernels (see mimo_common.cuh for the math).
//
//   local_state   per chunk:  Lc = Kr^T (w o PV)            -> local [B,H,C,N,P] fp32, tot [B,H,C]
//   state_scan    per (b,h):  St_{c+1} = e^{tot_c} St_c + Lc -> start states [B,H,C,N,P] bf16
//   chunk_out     per chunk:  S1, mask, O = Pm PV + e^{cs}(Qr St) + D PV, gate, reduce over r -> y
//
// GEMMs run on tcgen05 with accumulators in TMEM; Q/K tiles arrive by TMA (5-D tensor map over
// [B,S,G,R,N]) into 128-byte-swizzled shared memory and are bias-added and rotated in place.
// Replaces the TileLang forward kernel the reference imports from mamba_ssm
// (cppmega/megatron/tilelang_mimo_autograd.py:127-135) and its Triton prefix-sum helper (:124).
#include "mimo_common.cuh"

namespace cm {
namespace mimo {

static EncodeTiledFn enc() { return get_encode_tiled(); }

int make_tmap_qk(CUtensorMap* out, const void* base, int B, int S, int G, int N) {
  EncodeTiledFn e = enc();
  if (!e) return -1;
  cuuint64_t dims[5] = {(cuuint64_t)N, (cuuint64_t)R, (cuuint64_t)G, (cuuint64_t)S, (cuuint64_t)B};
  cuuint64_t strides[4] = {(cuuint64_t)N * 2, (cuuint64_t)R * N * 2, (cuuint64_t)G * R * N * 2,
                           (cuuint64_t)S * G * R * N * 2};
  cuuint32_t box[5] = {64, (cuuint32_t)R, 1, (cuuint32_t)LT, 1};
  cuuint32_t es[5] = {1, 1, 1, 1, 1};
  CUresult r = e(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(base), dims, strides, box, es,
                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : int(r);
}

int make_tmap_rows64(CUtensorMap* out, const void* base, uint64_t rows) {
  return make_tmap_2d_bf16(out, base, rows, 64, 64, 128, 64);
}

__device__ __forceinline__ void tma_load_5d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2,
                                            int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2),
      "r"(c3), "r"(c4)
      : "memory");
}

struct FwdArgs {
  const __nv_bfloat16* V;      // [B,S,H,P]
  const __nv_bfloat16* Z;      // [B,S,H,P]
  const float* ADT;            // [B,H,S]
  const float* DT;
  const float* Trap;
  const float* Qb;             // [H,R,N]
  const float* Kb;
  const float* Psi;            // [H,R,P]
  const float* Zeta;
  const float* Phi;
  const float* angles;         // [B,S,H,NROT]
  const float* Dskip;          // [H]
  float* local;                // [B,H,C,N,P] fp32
  float* tot;                  // [B,H,C]
  __nv_bfloat16* y;            // [B,S,H,P]
  int B, S, H, G, C;
  long long ldV, ldZ;          // token strides of V and Z in elements
  int* err;
};

// blockIdx.x -> (b, g, c, head-in-group): CTAs sharing a Q/K tile are adjacent
__device__ __forceinline__ void decode_block(const FwdArgs& a, int& b, int& g, int& c, int& h) {
  const int hpg = a.H / a.G;
  int x = blockIdx.x;
  const int hl = x % hpg; x /= hpg;
  c = x % a.C; x /= a.C;
  g = x % a.G; x /= a.G;
  b = x;
  h = g * hpg + hl;
}

// ------------------------------------------------------------------------------------------
// local_state: Lc[n,p] = sum_j Kr[j,n] * w_j * PV[j,p]
// 256 threads: thread (i = tid & 127, wg = tid >> 7) owns fused row i and half of its columns.
// ------------------------------------------------------------------------------------------
constexpr int THREADS2 = 256;

template <int N, int NROT>
__global__ void __launch_bounds__(THREADS2) mimo_local_state_kernel(const __grid_constant__ CUtensorMap tmK, const FwdArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int KT = (N / 64) * SLAB;
  uint8_t* sK = smem;
  uint8_t* sPVw = sK + KT;
  float* cos_tab = reinterpret_cast<float*>(sPVw + SLAB);
  float* sin_tab = cos_tab + tab_floats<NROT>();
  HeadBias<N>* hb = reinterpret_cast<HeadBias<N>*>(sin_tab + tab_floats<NROT>());
  HeadVecs* hv = reinterpret_cast<HeadVecs*>(hb + 1);
  ChunkScalars* sc = reinterpret_cast<ChunkScalars*>(hv + 1);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sc + 1);            // [0] tma, [1] mma
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  if (a.err && *reinterpret_cast<volatile int*>(a.err) != 0) return;   // an earlier CTA / kernel gave up: drain
  int b, g, c, h;
  decode_block(a, b, g, c, h);
  const int t0 = c * LT;
  const int warp = threadIdx.x >> 5, i = threadIdx.x & 127, wg = threadIdx.x >> 7;
  // every global load of the prologue is issued here, ahead of the set-up, and consumed further down
  const ScalarLoads sl = load_chunk_scalars(a.ADT, a.DT, a.Trap, ((size_t)b * a.H + h) * a.S + t0, t0, a.S);
  const float4 ang4 = load_angles4<NROT>(a.angles, b, t0, h, a.S, a.H);
  const HalfRowRaw vraw = load_half_raw(a.V, b, t0, h, a.S, a.ldV);
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
    mbar_expect_tx(&bars[0], KT);
#pragma unroll
    for (int s = 0; s < N / 64; ++s) tma_load_5d(sK + s * SLAB, &tmK, &bars[0], s * 64, 0, g, t0, b);
  }
  load_head_consts<N>(hb, hv, nullptr, a.Kb, a.Psi, nullptr, nullptr, h);
  finish_chunk_scalars(sc, sl, t0, a.S);
  fill_sincos4<NROT>(cos_tab, sin_tab, ang4);
  __syncthreads();
  bool ok = mbar_wait(&bars[0], 0, abort_flag, a.err, ERR_WAIT_FULL);
  if (ok) {
    transform_rows<N, NROT, 2, HeadBias<N>::LD>(sK, hb->kb, cos_tab, sin_tab);
    float pv[P / 2];
    pv_from_raw(pv, vraw, hv->psi);
    const int t = i >> 2;
    store_half64(sPVw, pv, sc->ts[t] * __expf(sc->tot - sc->cs[t]));
    fence_proxy_async_smem();
  }
  __syncthreads();
  if (threadIdx.x == 0 && !*abort_flag) {
    constexpr uint32_t idesc = umma_idesc_bf16(N, P, true, true);       // M = N (state rows), N = P
    const uint32_t aK = smem_u32(sK), aP = smem_u32(sPVw);
#pragma unroll
    for (int k = 0; k < ROWS / 16; ++k)
      umma_f16(tmem, desc_mnmajor_2slab(aK, k), desc_mnmajor_rows(aP, k), idesc, k != 0);
    umma_commit(&bars[1]);
  }
  ok = mbar_wait(&bars[1], 0, abort_flag, a.err, ERR_WAIT_TMEM_FULL);
  tc_fence_after();
  if (ok) {
    float* dst = a.local + ((((size_t)b * a.H + h) * a.C + c) * N + i) * P + wg * 32;
    uint32_t r[32];
    tmem_ld_32x32(tmem + (uint32_t((warp & 3) * 32) << 16) + wg * 32, r);
    tmem_ld_wait();
#pragma unroll
    for (int v = 0; v < 8; ++v)
      reinterpret_cast<float4*>(dst)[v] = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                                                      __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
  }
  if (threadIdx.x == 0) a.tot[((size_t)b * a.H + h) * a.C + c] = sc->tot;
  tc_fence_before();
  __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem, 64); }
}

// ------------------------------------------------------------------------------------------
// state_scan: start[c] = state; state = e^{tot_c} state + local[c]     (elementwise, sequential in c)
// grid (B*H, N*P/1024), 256 threads x 4 elements
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) mimo_state_scan_kernel(const float* __restrict__ local, const float* __restrict__ tot,
                                                              __nv_bfloat16* __restrict__ start, float* __restrict__ final_state,
                                                              int C, int NP) {
  const size_t bh = blockIdx.x;
  const int e = (blockIdx.y * 256 + threadIdx.x) * 4;
  if (e >= NP) return;
  float4 st = make_float4(0.f, 0.f, 0.f, 0.f);
  const float* lp = local + bh * (size_t)C * NP + e;
  __nv_bfloat16* sp = start + bh * (size_t)C * NP + e;
  const float* tp = tot + bh * C;
  float4 nxt = *reinterpret_cast<const float4*>(lp);
  for (int c = 0; c < C; ++c) {
    const float4 cur = nxt;
    if (c + 1 < C) nxt = *reinterpret_cast<const float4*>(lp + (size_t)(c + 1) * NP);
    uint2 o;
    o.x = pack_bf16(st.x, st.y);
    o.y = pack_bf16(st.z, st.w);
    *reinterpret_cast<uint2*>(sp + (size_t)c * NP) = o;
    const float d = __expf(tp[c]);
    st.x = d * st.x + cur.x; st.y = d * st.y + cur.y; st.z = d * st.z + cur.z; st.w = d * st.w + cur.w;
  }
  if (final_state) *reinterpret_cast<float4*>(final_state + bh * NP + e) = st;
}

// ------------------------------------------------------------------------------------------
// chunk_out (256 threads, two warpgroups splitting the columns of every row-wise phase)
// ------------------------------------------------------------------------------------------
template <int N, int NROT>
__global__ void __launch_bounds__(THREADS2, 2) mimo_chunk_out_kernel(const __grid_constant__ CUtensorMap tmQ,
                                                                     const __grid_constant__ CUtensorMap tmK,
                                                                     const __grid_constant__ CUtensorMap tmS, const FwdArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int QT = (N / 64) * SLAB;            // Q tile bytes (also K tile bytes)
  constexpr int PT = 2 * SLAB;                   // masked scores [128 x 128] bf16
  constexpr int QP = QT > PT ? QT : PT;          // Pm reuses the Q tile's space
  uint8_t* sQ = smem;                            // later: Pm
  uint8_t* sK = sQ + QP;
  uint8_t* sPV = sK + QT;
  uint8_t* sSt = sPV + SLAB;                     // start state [N x 64] bf16
  float* cos_tab = reinterpret_cast<float*>(sSt + (N / 128 > 0 ? N : 128) * 128);
  float* sin_tab = cos_tab + tab_floats<NROT>();
  HeadBias<N>* hb = reinterpret_cast<HeadBias<N>*>(sPV);      // biases die before PV is written (barrier between)
  static_assert(sizeof(HeadBias<N>) <= SLAB, "bias block must fit the PV slab it borrows");
  float* psi_s = sin_tab + tab_floats<NROT>();                 // [R, P]
  float* zeta_s = cos_tab;                                      // zeta / phi move into the sin/cos tables once the
  float* phi_s = cos_tab + R * VLD;                              // rotations are done (registers hold them until then)
  static_assert(2 * R * VLD <= 2 * tab_floats<NROT>(), "zeta and phi must fit the retired tables");
  ChunkScalars* sc = reinterpret_cast<ChunkScalars*>(psi_s + R * VLD);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sc + 1);            // [0] tma, [1] S1+O2, [2] O1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  if (a.err && *reinterpret_cast<volatile int*>(a.err) != 0) return;   // an earlier CTA / kernel gave up: drain
  int b, g, c, h;
  decode_block(a, b, g, c, h);
  const int t0 = c * LT;
  const int i = threadIdx.x & 127, wg = threadIdx.x >> 7, t = i >> 2, r = i & 3;
  const int warp = threadIdx.x >> 5;
  // every global load of the prologue is issued here, ahead of the set-up, and consumed further down
  const ScalarLoads sl = load_chunk_scalars(a.ADT, a.DT, a.Trap, ((size_t)b * a.H + h) * a.S + t0, t0, a.S);
  const float4 ang4 = load_angles4<NROT>(a.angles, b, t0, h, a.S, a.H);
  const HalfRowRaw vraw = load_half_raw(a.V, b, t0, h, a.S, a.ldV);
  const HalfRowRaw zraw = load_half_raw(a.Z, b, t0, h, a.S, a.ldZ);
  const float dsk = a.Dskip[h];
  static_assert(R * P == THREADS2, "one zeta / phi / psi element per thread");
  const float zeta_v = a.Zeta[(size_t)h * R * P + threadIdx.x], phi_v = a.Phi[(size_t)h * R * P + threadIdx.x];
  const float psi_v = a.Psi[(size_t)h * R * P + threadIdx.x];
  if (threadIdx.x == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    mbar_init(&bars[2], 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) { tmem_alloc(tmem_slot, 256); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS1 = tmem, tO2 = tmem + 128, tO1 = tmem + 192;
  if (threadIdx.x == 0) {
    mbar_expect_tx(&bars[0], 2 * QT + N * 128);
#pragma unroll
    for (int s = 0; s < N / 64; ++s) {
      tma_load_5d(sQ + s * SLAB, &tmQ, &bars[0], s * 64, 0, g, t0, b);
      tma_load_5d(sK + s * SLAB, &tmK, &bars[0], s * 64, 0, g, t0, b);
    }
    tma_load_2d(sSt, &tmS, &bars[0], 0, (int)((((size_t)b * a.H + h) * a.C + c) * N));
  }
  for (int x = threadIdx.x; x < R * N; x += THREADS2) {
    const int dst = (x / N) * HeadBias<N>::LD + (x % N);
    hb->qb[dst] = a.Qb[(size_t)h * R * N + x];
    hb->kb[dst] = a.Kb[(size_t)h * R * N + x];
  }
  psi_s[vec_idx(threadIdx.x)] = psi_v;
  finish_chunk_scalars(sc, sl, t0, a.S);
  fill_sincos4<NROT>(cos_tab, sin_tab, ang4);
  __syncthreads();
  bool ok = mbar_wait(&bars[0], 0, abort_flag, a.err, ERR_WAIT_FULL);
  float pv[P / 2];
  if (ok) {
    transform_rows<N, NROT, 2, HeadBias<N>::LD>(sQ, hb->qb, cos_tab, sin_tab);
    transform_rows<N, NROT, 2, HeadBias<N>::LD>(sK, hb->kb, cos_tab, sin_tab);
    pv_from_raw(pv, vraw, psi_s);
  }
  __syncthreads();                               // every thread is done with the biases stored in the PV slab and the tables
  zeta_s[vec_idx(threadIdx.x)] = zeta_v;
  phi_s[vec_idx(threadIdx.x)] = phi_v;
  if (ok) {
    store_half64(sPV, pv, 1.f);
    fence_proxy_async_smem();
  }
  __syncthreads();
  if (threadIdx.x == 0 && !*abort_flag) {
    constexpr uint32_t id_s1 = umma_idesc_bf16(ROWS, ROWS, false, false);
    constexpr uint32_t id_o = umma_idesc_bf16(ROWS, P, false, true);
    const uint32_t aQ = smem_u32(sQ), aK = smem_u32(sK), aSt = smem_u32(sSt);
#pragma unroll
    for (int k = 0; k < N / 16; ++k) umma_f16(tS1, desc_kmajor(aQ, k), desc_kmajor(aK, k), id_s1, k != 0);
#pragma unroll
    for (int k = 0; k < N / 16; ++k) umma_f16(tO2, desc_kmajor(aQ, k), desc_mnmajor_rows(aSt, k), id_o, k != 0);
    umma_commit(&bars[1]);
  }
  ok = mbar_wait(&bars[1], 0, abort_flag, a.err, ERR_WAIT_TMEM_FULL);
  tc_fence_after();
  const uint32_t lane_addr = uint32_t((warp & 3) * 32) << 16;
  if (ok) {
    // mask the scores of this row and store them as the A operand of the second product
    const float csi = sc->cs[t], gi = sc->gam[t];
#pragma unroll
    for (int c2 = 0; c2 < 2; ++c2) {            // 32 columns = 8 key tokens per pass; this warpgroup's two passes
      const int cc = wg * 2 + c2;
      uint32_t rr[32];
      tmem_ld_32x32(tS1 + lane_addr + cc * 32, rr);
      tmem_ld_wait();
#pragma unroll
      for (int q = 0; q < 4; ++q) {             // 8 columns = 2 key tokens per 16-byte store
        float f[8];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int tj = cc * 8 + q * 2 + u;
          float m = 0.f;
          if (tj < t) m = sc->ts[tj] * __expf(csi - sc->cs[tj]);
          else if (tj == t) m = gi;
#pragma unroll
          for (int v = 0; v < 4; ++v) f[u * 4 + v] = __uint_as_float(rr[q * 8 + u * 4 + v]) * m;
        }
        const int col = cc * 32 + q * 8;
        *reinterpret_cast<uint4*>(sQ + (col / 64) * SLAB + sw_off(i, (col % 64) / 8)) = pack8(f);
      }
    }
    fence_proxy_async_smem();
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && !*abort_flag) {
    tc_fence_after();
    constexpr uint32_t id_o = umma_idesc_bf16(ROWS, P, false, true);
    const uint32_t aPm = smem_u32(sQ), aPV = smem_u32(sPV);
#pragma unroll
    for (int k = 0; k < ROWS / 16; ++k) umma_f16(tO1, desc_kmajor(aPm, k), desc_mnmajor_rows(aPV, k), id_o, k != 0);
    umma_commit(&bars[2]);
  }
  ok = mbar_wait(&bars[2], 0, abort_flag, a.err, ERR_WAIT_TMEM_FULL);
  tc_fence_after();
  if (ok) {
    const float ecs = __expf(sc->cs[t]);
    const float* zeta = zeta_s + r * VLD + wg * 32;
    const float* phi = phi_s + r * VLD + wg * 32;
    __nv_bfloat16* yrow = a.y + (((size_t)b * a.S + t0 + t) * a.H + h) * P + wg * 32;
    uint32_t o1[32], o2[32];
    tmem_ld_32x32(tO1 + lane_addr + wg * 32, o1);
    tmem_ld_32x32(tO2 + lane_addr + wg * 32, o2);
    tmem_ld_wait();
    float val[32];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float zf[8];
      unpack8(zraw.v[q], zf);
#pragma unroll
      for (int v = 0; v < 8; ++v) {
        const int p = q * 8 + v;
        const float o = __uint_as_float(o1[p]) + ecs * __uint_as_float(o2[p]) + dsk * pv[p];
        val[p] = o * phi[p] * fast_silu(zf[v] * zeta[p]);
      }
    }
    float mine[8];
    reduce4_keep8(val, mine);
    // lane r holds the sums over the four ranks for columns [8r, 8r + 8) of this warpgroup's half
    *reinterpret_cast<uint4*>(yrow + r * 8) = pack8(mine);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem, 256); }
}

template <int N>
constexpr int local_state_smem() {
  return (N / 64) * SLAB + SLAB + 2 * tab_floats<N / 4>() * 4 + sizeof(HeadBias<N>) + sizeof(HeadVecs) + sizeof(ChunkScalars) + 64 + 1024;
}
template <int N>
constexpr int chunk_out_smem() {
  return ((N / 64) * SLAB > 2 * SLAB ? (N / 64) * SLAB : 2 * SLAB) + (N / 64) * SLAB + SLAB + (N > 128 ? N : 128) * 128 +
         2 * tab_floats<N / 4>() * 4 + R * VLD * 4 + sizeof(ChunkScalars) + 64 + 1024;
}

}  // namespace mimo
}  // namespace cm

using namespace cm;
using namespace cm::mimo;

// Qn, Kn: [B,S,G,R,N] bf16 (already RMS-normalised); V, Z: [B,S,H,P] bf16; ADT, DT, Trap: [B,H,S] fp32;
// Qb, Kb: [H,R,N] fp32; Psi, Zeta, Phi: [H,R,P] fp32; angles: [B,S,H,N/4] fp32 cumulative; D: [H] fp32.
// Scratch: local [B,H,C,N,P] fp32, tot [B,H,C] fp32, states [B,H,C,N,P] bf16 (start state of every chunk).
// Output y [B,S,H,P] bf16.  S % 32 == 0, P == 64, R == 4, N == 128, rotary divisor 4.
// ldV / ldZ: elements between consecutive tokens of V / Z (H*P when packed; V and Z may be column slices of a wider
// [B*S, W] matrix, in which case the batch stride must be S*ld).
extern "C" int cm_mimo_scan_fwd(const void* Qn, const void* Kn, const void* V, const void* Z, const float* ADT,
                                const float* DT, const float* Trap, const float* Qb, const float* Kb, const float* Psi,
                                const float* Zeta, const float* Phi, const float* angles, const float* Dskip, float* local,
                                float* tot, void* states, float* final_state, void* y, int B, int S, int H, int G, int N,
                                long long ldV, long long ldZ, int* err, cudaStream_t stream) {
  if (B <= 0 || S <= 0) return 0;
  if (S % LT || N != 128 || H % G) return -10;   // M = 64 accumulators use a different TMEM lane map
  if (ldV < (long long)H * P || ldZ < (long long)H * P || ldV % 8 || ldZ % 8) return -11;   // 16-byte row loads
  const int C = S / LT;
  CUtensorMap tmQ, tmK, tmS;
  int rc = make_tmap_qk(&tmQ, Qn, B, S, G, N);
  if (rc) return rc;
  rc = make_tmap_qk(&tmK, Kn, B, S, G, N);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tmS, states, (uint64_t)B * H * C * N, 64, 64, 128, 64);
  if (rc) return rc;
  FwdArgs a{(const __nv_bfloat16*)V, (const __nv_bfloat16*)Z, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, angles, Dskip,
            local, tot, (__nv_bfloat16*)y, B, S, H, G, C, ldV, ldZ, err};
  const int grid = B * H * C;
  if (N == 128) {
    auto k1 = mimo_local_state_kernel<128, 32>;
    auto k3 = mimo_chunk_out_kernel<128, 32>;
    static PerDevice cfg;
    if (cfg.first()) {
      if (cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, local_state_smem<128>()) != cudaSuccess) return -2;
      if (cudaFuncSetAttribute(k3, cudaFuncAttributeMaxDynamicSharedMemorySize, chunk_out_smem<128>()) != cudaSuccess) return -2;
      cfg.done();
    }
    k1<<<grid, THREADS2, local_state_smem<128>(), stream>>>(tmK, a);
    dim3 g2(B * H, (128 * P + 1023) / 1024);
    mimo_state_scan_kernel<<<g2, 256, 0, stream>>>(local, tot, (__nv_bfloat16*)states, final_state, C, 128 * P);
    k3<<<grid, THREADS2, chunk_out_smem<128>(), stream>>>(tmQ, tmK, tmS, a);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// ------------------------------------------------------------------------------------------
// Variant with the work buffers in a fixed device array (see mimo_scan_static.h for the contract).
// ------------------------------------------------------------------------------------------
#include <cstdio>

#include "mimo_scan_static.h"

static __device__ __align__(256) unsigned char cm_mimo_static_scratch[CM_MIMO_STATIC_BYTES];

extern "C" int cm_mimo_scan_fwd_static(const void* Qn, const void* Kn, const void* V, const void* Z, const float* ADT,
                                       const float* DT, const float* Trap, const float* Qb, const float* Kb,
                                       const float* Psi, const float* Zeta, const float* Phi, const float* angles,
                                       const float* Dskip, float* final_state, void* y, int B, int S, int H, int G, int N,
                                       int* err, cudaStream_t stream) {
  if (B <= 0 || S <= 0) return 0;
  if (S % LT || N != 128 || H <= 0 || G <= 0 || H % G) return -10;
  const long long chunks = (long long)B * H * (S / LT);
  if (chunks > CM_MIMO_STATIC_MAX_CHUNKS) {
    fprintf(stderr,
            "cm_mimo_scan_fwd_static: B*H*S/32 = %lld chunks exceeds the fixed work array (%d chunks, %zu bytes); "
            "use cm_mimo_scan_fwd with caller-provided scratch for this size\n",
            chunks, CM_MIMO_STATIC_MAX_CHUNKS, (size_t)CM_MIMO_STATIC_BYTES);
    return CM_MIMO_STATIC_E_TOO_LARGE;
  }
  constexpr int MAX_DEV = 64;
  static unsigned char* base[MAX_DEV] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEV) return CM_MIMO_STATIC_E_DEVICE;
  if (base[dev] == nullptr) {
    unsigned char* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress((void**)&p, cm_mimo_static_scratch);
    if (e != cudaSuccess || p == nullptr) {
      fprintf(stderr, "cm_mimo_scan_fwd_static: cudaGetSymbolAddress failed on device %d: %s\n", dev, cudaGetErrorString(e));
      return CM_MIMO_STATIC_E_SYMBOL;
    }
    base[dev] = p;
  }
  // carve: local fp32 | start states bf16 | tot fp32 (each offset a multiple of 256 bytes)
  unsigned char* p = base[dev];
  float* local = reinterpret_cast<float*>(p);
  p += (size_t)CM_MIMO_STATIC_MAX_CHUNKS * CM_MIMO_STATIC_STATE_ELEMS * 4;
  void* states = p;
  p += (size_t)CM_MIMO_STATIC_MAX_CHUNKS * CM_MIMO_STATIC_STATE_ELEMS * 2;
  float* tot = reinterpret_cast<float*>(p);
  return cm_mimo_scan_fwd(Qn, Kn, V, Z, ADT, DT, Trap, Qb, Kb, Psi, Zeta, Phi, angles, Dskip, local, tot, states,
                          final_state, y, B, S, H, G, N, (long long)H * P, (long long)H * P, err, stream);
}
