// Dense causal multi-head attention for the full-attention MLA layers and the MTP layers (q/k head dim 128 = 64 "nope"
// + 64 rope dims, value head dim 64), forward and backward, on tcgen05 with the scores in TMEM.
//
//   s[i,j] = scale * q[i,:] . k[j,:]  (j <= i)      p = softmax_j(s)      o[i,:] = sum_j p[i,j] v[j,:]
//
// forward   one CTA (128 threads, thread r <-> query row r <-> TMEM lane r) per (128-query tile, head, batch); loop over the
//           128-key tiles up to the diagonal:  S = Q K^T (TMEM)  ->  online softmax in registers (exp2 domain), P as bf16
//           into shared memory (it takes the place of the K tile, which is dead once S is complete)  ->  O_j = P V (TMEM)
//           ->  acc = acc * alpha + O_j in registers.  80 KB of shared memory: two CTAs per SM hide each other's waits.
// backward  one CTA per (128-key tile, head, batch) looping over the query tiles at or below the diagonal:
//           S = Q K^T, dP = dO V^T  ->  P = exp2(S - lse), dS = scale * P o (dP - delta)  ->  dV += P^T dO, dK += dS^T Q
//           (both stay in TMEM for the whole loop), dQ_i = dS K, added to an fp32 buffer with one bulk shared->global
//           reduction per row (cp.reduce.async.bulk .add.f32) - the only atomics, issued by the copy engine.
//           Q / dO tiles are double-buffered by TMA.
// All operand tiles are 128-byte-swizzled [128 x 64] bf16 slabs written by TMA (2-D maps over [B*S, H*dim]); the same
// slab is read K-major or MN-major by choosing the descriptor.  Every wait is bounded and reports through the error word.
// The reference takes this operator from cuDNN / FlashAttention (`--attention-backend flash`,
// scripts/remote_smoke_h200_dsa_9_4_m.sh:727-728; MLA adapter at cppmega/megatron/mla_shared.py:39-97).
#include "common.cuh"

namespace cm {
namespace attn {

constexpr int BQ = 128;          // query rows per tile
constexpr int BK = 128;          // key rows per tile
constexpr int D = 128;           // q / k head dim
constexpr int DV = 64;           // v head dim
constexpr int SLAB = 128 * 128;  // bytes of one [128 rows x 64 bf16] swizzled slab
constexpr int THREADS = 128;

__device__ __forceinline__ int sw_off(int row, int c) { return row * 128 + ((c ^ (row & 7)) << 4); }

// [128 x 128] operand, K-major (two slabs side by side along K), 16-element k step `k` (0..7)
__device__ __forceinline__ uint64_t desc_k(uint32_t tile, int k) {
  return umma_desc_sw128(tile + (k >> 2) * SLAB + (k & 3) * 32, 16, 1024);
}
// [128(K) rows x 64] slab read MN-major (M/N = the 64 columns), 16-row k step
__device__ __forceinline__ uint64_t desc_mn1(uint32_t slab, int k) { return umma_desc_sw128(slab + k * 2048, SLAB, 1024); }
// [128(K) rows x 128] two-slab tile read MN-major (M/N = the 128 columns)
__device__ __forceinline__ uint64_t desc_mn2(uint32_t tile, int k) { return umma_desc_sw128(tile + k * 2048, SLAB, 1024); }

__device__ __forceinline__ uint4 pack8f(const float* f) {
  uint4 o;
  o.x = pack_bf16(f[0], f[1]); o.y = pack_bf16(f[2], f[3]);
  o.z = pack_bf16(f[4], f[5]); o.w = pack_bf16(f[6], f[7]);
  return o;
}

struct FwdArgs {
  __nv_bfloat16* out;   // [B, S, H, DV]
  float* lse2;          // [B, H, S]: log2-domain log-sum-exp of the scaled scores
  int S, H, n_qt;
  float scale_log2;     // softmax scale * log2(e)
  int* err;
};

struct FwdShared {
  uint64_t bars[5];     // [0] Q, [1] K, [2] V, [3] S complete, [4] PV complete
  uint32_t tmem_slot;
  int abort_flag;
};

constexpr int fwd_smem() { return 2 * SLAB + 2 * SLAB + SLAB + (int)sizeof(FwdShared) + 1024; }

__global__ void __launch_bounds__(THREADS, 2) attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ,
                                                              const __grid_constant__ CUtensorMap tmK,
                                                              const __grid_constant__ CUtensorMap tmV, const FwdArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                      // [128 x 128]
  uint8_t* sK = sQ + 2 * SLAB;             // K tile, then P
  uint8_t* sV = sK + 2 * SLAB;             // [128 x 64]
  FwdShared* sh = reinterpret_cast<FwdShared*>(sV + SLAB);
  if (a.err && *reinterpret_cast<volatile int*>(a.err) != 0) return;

  // heavy tiles (many key tiles) first
  const int bh = blockIdx.x % (gridDim.x / a.n_qt);
  const int qt = a.n_qt - 1 - blockIdx.x / (gridDim.x / a.n_qt);
  const int h = bh % a.H, b = bh / a.H;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int q0 = qt * BQ;
  if (tid == 0) {
    for (int i = 0; i < 5; ++i) mbar_init(&sh->bars[i], 1);
    sh->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) { tmem_alloc(&sh->tmem_slot, 256); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh->tmem_slot;
  const uint32_t tS = tmem, tO = tmem + 128;
  const uint32_t lane_addr = uint32_t((warp & 3) * 32) << 16;
  volatile int* abort_flag = &sh->abort_flag;
  const uint32_t aQ = smem_u32(sQ), aK = smem_u32(sK), aV = smem_u32(sV);
  const int row0 = b * a.S;                                   // first row of this batch in the [B*S, .] views
  if (tid == 0) {
    mbar_expect_tx(&sh->bars[0], 2 * SLAB);
    tma_load_2d(sQ, &tmQ, &sh->bars[0], h * D, row0 + q0);
    tma_load_2d(sQ + SLAB, &tmQ, &sh->bars[0], h * D + 64, row0 + q0);
  }
  float acc[DV];
#pragma unroll
  for (int e = 0; e < DV; ++e) acc[e] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;
  bool ok = true;
  for (int j = 0; j <= qt && ok; ++j) {
    const uint32_t par = j & 1;
    if (tid == 0) {
      mbar_expect_tx(&sh->bars[1], 2 * SLAB);
      tma_load_2d(sK, &tmK, &sh->bars[1], h * D, row0 + j * BK);
      tma_load_2d(sK + SLAB, &tmK, &sh->bars[1], h * D + 64, row0 + j * BK);
      mbar_expect_tx(&sh->bars[2], SLAB);
      tma_load_2d(sV, &tmV, &sh->bars[2], h * DV, row0 + j * BK);
      bool go = (j != 0) || mbar_wait(&sh->bars[0], 0, abort_flag, a.err, ERR_WAIT_FULL);
      go = go && mbar_wait(&sh->bars[1], par, abort_flag, a.err, ERR_WAIT_FULL);
      if (go) {
        tc_fence_after();
        constexpr uint32_t id_s = umma_idesc_bf16(BQ, BK, false, false);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) umma_f16(tS, desc_k(aQ, k), desc_k(aK, k), id_s, k != 0);
        umma_commit(&sh->bars[3]);
      }
    }
    ok = mbar_wait(&sh->bars[3], par, abort_flag, a.err, ERR_WAIT_TMEM_FULL);
    tc_fence_after();
    float alpha = 1.f;
    if (ok) {
      const bool diag = (j == qt);
      // pass 1: row maximum of this tile
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tS + lane_addr + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const float s = __uint_as_float(r[e]);
          if (!diag || c * 32 + e <= tid) mx = fmaxf(mx, s);
        }
      }
      const float m_new = fmaxf(m_run, mx * a.scale_log2);       // the diagonal tile always has column 0..tid valid
      alpha = exp2f(m_run - m_new);                               // 0 on the first tile (m_run = -inf)
      m_run = m_new;
      // pass 2: probabilities, row sum, P (bf16) over the dead K tile
      float lsum = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tS + lane_addr + c * 32, r);
        tmem_ld_wait();
        float p[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const float s = __uint_as_float(r[e]);
          const bool keep = !diag || c * 32 + e <= tid;
          p[e] = keep ? exp2f(fmaf(s, a.scale_log2, -m_new)) : 0.f;
          lsum += p[e];
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int col = c * 32 + q * 8;
          *reinterpret_cast<uint4*>(sK + (col >> 6) * SLAB + sw_off(tid, (col & 63) >> 3)) = pack8f(p + q * 8);
        }
      }
      l_run = l_run * alpha + lsum;
      fence_proxy_async_smem();
    }
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && !*abort_flag) {
      if (mbar_wait(&sh->bars[2], par, abort_flag, a.err, ERR_WAIT_FULL)) {
        tc_fence_after();
        constexpr uint32_t id_o = umma_idesc_bf16(BQ, DV, false, true);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k) umma_f16(tO, desc_k(aK, k), desc_mn1(aV, k), id_o, k != 0);
        umma_commit(&sh->bars[4]);
      }
    }
    if (ok) {
#pragma unroll
      for (int e = 0; e < DV; ++e) acc[e] *= alpha;              // under the P V product
    }
    ok = mbar_wait(&sh->bars[4], par, abort_flag, a.err, ERR_WAIT_TMEM_FULL) && ok;
    tc_fence_after();
    if (ok) {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tO + lane_addr + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) acc[c * 32 + e] += __uint_as_float(r[e]);
      }
    }
    tc_fence_before();
    __syncthreads();                                              // P and V may be overwritten by the next loads
    tc_fence_after();
  }
  if (ok) {
    const float inv = l_run > 0.f ? __fdividef(1.f, l_run) : 0.f;
    __nv_bfloat16* orow = a.out + ((size_t)(row0 + q0 + tid) * a.H + h) * DV;
#pragma unroll
    for (int c = 0; c < DV / 8; ++c) {
      float f[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = acc[c * 8 + e] * inv;
      reinterpret_cast<uint4*>(orow)[c] = pack8f(f);
    }
    a.lse2[((size_t)b * a.H + h) * a.S + q0 + tid] = m_run + log2f(l_run);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem, 256); }
}

// delta[b,h,s] = sum_d dO[b,s,h,d] * O[b,s,h,d]: one warp per (token, head), two value dims per lane
__global__ void __launch_bounds__(256) attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                                         float* __restrict__ delta, long long rows, int S, int H) {
  const int lane = threadIdx.x & 31;
  const long long w = blockIdx.x * 8LL + (threadIdx.x >> 5);
  if (w >= rows) return;
  const float2 ov = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(o + w * DV + lane * 2));
  const float2 dv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(dout + w * DV + lane * 2));
  const float d = warp_sum(ov.x * dv.x + ov.y * dv.y);
  if (lane == 0) {
    const long long tok = w / H;
    const int h = (int)(w % H);
    const long long b = tok / S, s = tok % S;
    delta[(b * H + h) * S + s] = d;
  }
}

struct BwdArgs {
  const float* lse2;    // [B, H, S]
  const float* delta;   // [B, H, S]
  float* dq;            // [B, S, H, D] fp32, zeroed by the caller; rows are reduced into it
  __nv_bfloat16* dk;    // [B, S, H, D]
  __nv_bfloat16* dv;    // [B, S, H, DV]
  int S, H, n_kt;
  float scale, scale_log2;
  int* err;
};

struct BwdShared {
  uint64_t bars[5];     // [0] K + V, [1] [2] Q + dO stage 0 / 1, [3] S + dP complete, [4] dV + dK + dQ complete
  uint32_t tmem_slot;
  int abort_flag;
};

constexpr int STAGE_LD = 64 * 4 + 16;     // bytes between staging rows of one 64-column half of dQ
constexpr int STAGE_EXTRA = 2 * BQ * STAGE_LD - 4 * SLAB;     // what the two staging halves need beyond the P and dS tiles
static_assert(STAGE_EXTRA > 0 && STAGE_EXTRA % 16 == 0, "staging overhang");
// K 2, V 1, Q 2 x 2, dO 2 x 1, P 2, dS 2 slabs
constexpr int bwd_smem() { return 13 * SLAB + STAGE_EXTRA + (int)sizeof(BwdShared) + 1024; }

__device__ __forceinline__ void bulk_reduce_add_f32(float* gdst, const void* ssrc, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(ssrc)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__global__ void __launch_bounds__(THREADS, 1) attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ,
                                                              const __grid_constant__ CUtensorMap tmK,
                                                              const __grid_constant__ CUtensorMap tmV,
                                                              const __grid_constant__ CUtensorMap tmdO, const BwdArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;                       // [128 keys x 128]
  uint8_t* sV = sK + 2 * SLAB;              // [128 keys x 64]
  uint8_t* sQ = sV + SLAB;                  // 2 stages x [128 queries x 128]
  uint8_t* sdO = sQ + 4 * SLAB;             // 2 stages x [128 queries x 64]
  uint8_t* sP = sdO + 2 * SLAB;             // [128 queries x 128 keys] bf16; with sdS: fp32 dQ staging [128 x 128]
  uint8_t* sdS = sP + 2 * SLAB;
  BwdShared* sh = reinterpret_cast<BwdShared*>(sdS + 2 * SLAB + STAGE_EXTRA);
  if (a.err && *reinterpret_cast<volatile int*>(a.err) != 0) return;

  // key tile 0 has the longest loop: it goes first
  const int bh = blockIdx.x % (gridDim.x / a.n_kt);
  const int kt = blockIdx.x / (gridDim.x / a.n_kt);
  const int h = bh % a.H, b = bh / a.H;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int k0 = kt * BK;
  if (tid == 0) {
    for (int i = 0; i < 5; ++i) mbar_init(&sh->bars[i], 1);
    sh->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) { tmem_alloc(&sh->tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh->tmem_slot;
  const uint32_t tS = tmem, tdP = tmem + 128, tdV = tmem + 256, tdK = tmem + 320, tdQ = tmem;   // dQ reuses the S columns
  const uint32_t lane_addr = uint32_t((warp & 3) * 32) << 16;
  volatile int* abort_flag = &sh->abort_flag;
  const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aP = smem_u32(sP), adS = smem_u32(sdS);
  const int row0 = b * a.S;
  const int n_it = a.n_kt - kt;              // query tiles kt .. n_kt - 1

  auto load_q_stage = [&](int it) {
    const int s = it & 1;
    const int qrow = row0 + (kt + it) * BQ;
    mbar_expect_tx(&sh->bars[1 + s], 3 * SLAB);
    tma_load_2d(sQ + s * 2 * SLAB, &tmQ, &sh->bars[1 + s], h * D, qrow);
    tma_load_2d(sQ + s * 2 * SLAB + SLAB, &tmQ, &sh->bars[1 + s], h * D + 64, qrow);
    tma_load_2d(sdO + s * SLAB, &tmdO, &sh->bars[1 + s], h * DV, qrow);
  };
  if (tid == 0) {
    mbar_expect_tx(&sh->bars[0], 3 * SLAB);
    tma_load_2d(sK, &tmK, &sh->bars[0], h * D, row0 + k0);
    tma_load_2d(sK + SLAB, &tmK, &sh->bars[0], h * D + 64, row0 + k0);
    tma_load_2d(sV, &tmV, &sh->bars[0], h * DV, row0 + k0);
    load_q_stage(0);
  }
  bool ok = true;
  for (int it = 0; it < n_it && ok; ++it) {
    const int s = it & 1;
    const uint32_t par = it & 1;
    const int q0 = (kt + it) * BQ;
    const uint32_t aQ = smem_u32(sQ + s * 2 * SLAB), adO = smem_u32(sdO + s * SLAB);
    // row statistics of this thread's query (consumed after the first products)
    const size_t stat = ((size_t)b * a.H + h) * a.S + q0 + tid;
    const float lse = a.lse2[stat], dlt = a.delta[stat];
    if (tid == 0) {
      if (it + 1 < n_it) load_q_stage(it + 1);       // the other stage was released by the previous iteration's products
      bool go = (it != 0) || mbar_wait(&sh->bars[0], 0, abort_flag, a.err, ERR_WAIT_FULL);
      go = go && mbar_wait(&sh->bars[1 + s], (it >> 1) & 1, abort_flag, a.err, ERR_WAIT_FULL);
      if (go) {
        tc_fence_after();
        constexpr uint32_t id_s = umma_idesc_bf16(BQ, BK, false, false);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) umma_f16(tS, desc_k(aQ, k), desc_k(aK, k), id_s, k != 0);
#pragma unroll
        for (int k = 0; k < DV / 16; ++k)                                 // dP = dO V^T: both K-major over the 64 value dims
          umma_f16(tdP, umma_desc_sw128(adO + k * 32, 16, 1024), umma_desc_sw128(aV + k * 32, 16, 1024), id_s, k != 0);
        umma_commit(&sh->bars[3]);
      }
    }
    ok = mbar_wait(&sh->bars[3], par, abort_flag, a.err, ERR_WAIT_TMEM_FULL);
    tc_fence_after();
    if (ok) {
      const bool diag = (it == 0);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t rs[32], rp[32];
        tmem_ld_32x32(tS + lane_addr + c * 32, rs);
        tmem_ld_32x32(tdP + lane_addr + c * 32, rp);
        tmem_ld_wait();
        float p[32], ds[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const bool keep = !diag || c * 32 + e <= tid;
          const float pe = keep ? exp2f(fmaf(__uint_as_float(rs[e]), a.scale_log2, -lse)) : 0.f;
          p[e] = pe;
          ds[e] = pe * (__uint_as_float(rp[e]) - dlt) * a.scale;
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int col = c * 32 + q * 8;
          const int off = (col >> 6) * SLAB + sw_off(tid, (col & 63) >> 3);
          *reinterpret_cast<uint4*>(sP + off) = pack8f(p + q * 8);
          *reinterpret_cast<uint4*>(sdS + off) = pack8f(ds + q * 8);
        }
      }
      fence_proxy_async_smem();
    }
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && !*abort_flag) {
      tc_fence_after();
      constexpr uint32_t id_dv = umma_idesc_bf16(BK, DV, true, true);     // dV [keys x 64] += P^T dO
      constexpr uint32_t id_dk = umma_idesc_bf16(BK, D, true, true);      // dK [keys x 128] += dS^T Q
      constexpr uint32_t id_dq = umma_idesc_bf16(BQ, D, false, true);     // dQ [queries x 128] = dS K
#pragma unroll
      for (int k = 0; k < BQ / 16; ++k) umma_f16(tdV, desc_mn2(aP, k), desc_mn1(adO, k), id_dv, (it | k) != 0);
#pragma unroll
      for (int k = 0; k < BQ / 16; ++k) umma_f16(tdK, desc_mn2(adS, k), desc_mn2(aQ, k), id_dk, (it | k) != 0);
#pragma unroll
      for (int k = 0; k < BK / 16; ++k) umma_f16(tdQ, desc_k(adS, k), desc_mn2(aK, k), id_dq, k != 0);
      umma_commit(&sh->bars[4]);
    }
    ok = mbar_wait(&sh->bars[4], par, abort_flag, a.err, ERR_WAIT_TMEM_FULL) && ok;
    tc_fence_after();
    if (ok) {
      // dQ row of this thread -> fp32 staging (P and dS are dead) -> bulk reductions into the global buffer, one per
      // 64-column half.  Staging rows are 272 bytes apart: the 16-byte stores of a warp then spread over all banks.
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        float* stage = reinterpret_cast<float*>(sP + half * (BQ * STAGE_LD) + tid * STAGE_LD);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(tdQ + lane_addr + half * 64 + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int v = 0; v < 8; ++v)
            reinterpret_cast<float4*>(stage)[c * 8 + v] = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                                                                      __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
        }
      }
      fence_proxy_async_smem();
      float* grow = a.dq + ((size_t)(row0 + q0 + tid) * a.H + h) * D;
      bulk_reduce_add_f32(grow, sP + tid * STAGE_LD, 64 * 4);
      bulk_reduce_add_f32(grow + 64, sP + BQ * STAGE_LD + tid * STAGE_LD, 64 * 4);
      bulk_commit();
      bulk_wait_read_all();                         // the staging rows may be overwritten once the engine has read them
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
  }
  if (ok) {
    __nv_bfloat16* krow = a.dk + ((size_t)(row0 + k0 + tid) * a.H + h) * D;
    __nv_bfloat16* vrow = a.dv + ((size_t)(row0 + k0 + tid) * a.H + h) * DV;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t r[32];
      tmem_ld_32x32(tdK + lane_addr + c * 32, r);
      tmem_ld_wait();
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float f[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[q * 8 + e]);
        reinterpret_cast<uint4*>(krow)[c * 4 + q] = pack8f(f);
      }
    }
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      uint32_t r[32];
      tmem_ld_32x32(tdV + lane_addr + c * 32, r);
      tmem_ld_wait();
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float f[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[q * 8 + e]);
        reinterpret_cast<uint4*>(vrow)[c * 4 + q] = pack8f(f);
      }
    }
  }
  bulk_wait_all();                                  // this thread's reductions have reached memory
  tc_fence_before();
  __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

}  // namespace attn
}  // namespace cm

using namespace cm;
using namespace cm::attn;

static int attn_shape_ok(int B, int S, int H, int Dq, int Dv) {
  if (Dq != D || Dv != DV || S % BQ || H <= 0) return 0;
  if ((long long)B * S > 0x7fffffffLL / 4) return 0;
  return 1;
}

// q, k [B,S,H,128] bf16, v [B,S,H,64] bf16 (all packed) -> out [B,S,H,64] bf16, lse2 [B,H,S] fp32 (log2 domain).  S % 128 == 0.
extern "C" int cm_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse2, int B, int S, int H, int Dq,
                           int Dv, float scale, int* err, cudaStream_t stream) {
  if (B <= 0 || S <= 0) return 0;
  if (!attn_shape_ok(B, S, H, Dq, Dv)) return -10;
  CUtensorMap tmQ, tmK, tmV;
  const uint64_t rows = (uint64_t)B * S;
  int rc = make_tmap_2d_bf16(&tmQ, q, rows, (uint64_t)H * D, (uint64_t)H * D, BQ, 64);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tmK, k, rows, (uint64_t)H * D, (uint64_t)H * D, BK, 64);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tmV, v, rows, (uint64_t)H * DV, (uint64_t)H * DV, BK, 64);
  if (rc) return rc;
  static PerDevice cfg;
  if (cfg.first()) {
    if (cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, fwd_smem()) != cudaSuccess) return -2;
    cfg.done();
  }
  const int n_qt = S / BQ;
  FwdArgs a{(__nv_bfloat16*)out, lse2, S, H, n_qt, scale * 1.4426950408889634f, err};
  attn_fwd_kernel<<<(unsigned)(n_qt * B * H), THREADS, fwd_smem(), stream>>>(tmQ, tmK, tmV, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// delta [B,H,S] fp32 scratch; dq_acc [B,S,H,128] fp32 ZEROED by the caller (query gradients are reduced into it);
// dk [B,S,H,128], dv [B,S,H,64] bf16 are written.
extern "C" int cm_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse2,
                           float* delta, float* dq_acc, void* dk, void* dv, int B, int S, int H, int Dq, int Dv, float scale,
                           int* err, cudaStream_t stream) {
  if (B <= 0 || S <= 0) return 0;
  if (!attn_shape_ok(B, S, H, Dq, Dv)) return -10;
  CUtensorMap tmQ, tmK, tmV, tmdO;
  const uint64_t rows = (uint64_t)B * S;
  int rc = make_tmap_2d_bf16(&tmQ, q, rows, (uint64_t)H * D, (uint64_t)H * D, BQ, 64);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tmK, k, rows, (uint64_t)H * D, (uint64_t)H * D, BK, 64);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tmV, v, rows, (uint64_t)H * DV, (uint64_t)H * DV, BK, 64);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tmdO, dout, rows, (uint64_t)H * DV, (uint64_t)H * DV, BQ, 64);
  if (rc) return rc;
  static PerDevice cfg;
  if (cfg.first()) {
    if (cudaFuncSetAttribute(attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bwd_smem()) != cudaSuccess) return -2;
    cfg.done();
  }
  const long long nrows = (long long)rows * H;
  attn_delta_kernel<<<(unsigned)((nrows + 7) / 8), 256, 0, stream>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, delta,
                                                                      nrows, S, H);
  const int n_kt = S / BK;
  BwdArgs a{lse2, delta, dq_acc, (__nv_bfloat16*)dk, (__nv_bfloat16*)dv, S, H, n_kt, scale, scale * 1.4426950408889634f, err};
  attn_bwd_kernel<<<(unsigned)(n_kt * B * H), THREADS, bwd_smem(), stream>>>(tmQ, tmK, tmV, tmdO, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
