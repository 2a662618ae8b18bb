// DSA lightning indexer: causal scores and top-k selection.
//
//   score[b,i,j] = sum_h w[b,i,h] * relu(q[b,i,h,:] . k[b,j,:])      (32 heads x 64 dims, j <= i)
//   idx[b,i,:]   = the TOPK keys with the largest score among j <= i  (-1 where fewer are visible)
//
// Scores: a CTA owns 4 consecutive queries = 128 (query, head) rows = one tcgen05 M tile and walks the causal key
// tiles (128 keys, K = 64) through a 3-stage TMA ring with two TMEM accumulators, so the tensor core works on tile
// t+1 while the warps reduce tile t.  In the epilogue a warp is one query and a lane one head: relu, the per-head
// weight and the sum over heads are a transposing shuffle reduction, after which lane l holds the score of key
// column l - stores are 128-byte lines.  The reference computes the same in bf16 bmm + relu + weighted sum per
// head-chunk (cppmega/megatron/dsa_indexer_fused_patch.py:71-133) and selects with torch.topk
// (cppmega/megatron/dsa_splitk_indexer_loss.py:132-192 streams key chunks to bound memory).
// Top-k: one CTA per query row, radix select (4 passes of 8 bits over order-preserving uint32 keys held in
// registers) and an unordered emit; rows that see at most TOPK keys are written directly.
#include "common.cuh"

namespace cm {
namespace idx {

constexpr int HI = 32;          // indexer heads
constexpr int DI = 64;          // indexer head dim
constexpr int QT = 4;           // queries per CTA (QT * HI = 128 rows)
constexpr int KT = 128;         // keys per tile
constexpr int SLAB = 128 * 128; // one [128 x 64] bf16 operand tile
constexpr int STAGES = 3;

struct ScoreArgs {
  const float* w;      // [B, S, HI]
  float* scores;       // [B, S, S]
  int S;
  int* err;
};

struct ScoreShared {
  uint64_t bar_q;
  uint64_t bar_k[STAGES];
  uint64_t bar_m[2];
  uint32_t tmem_slot;
  int abort_flag;
};

constexpr int score_smem() { return (1 + STAGES) * SLAB + (int)sizeof(ScoreShared) + 1024; }

__global__ void __launch_bounds__(128) indexer_scores_kernel(const __grid_constant__ CUtensorMap tmQ,
                                                             const __grid_constant__ CUtensorMap tmK, const ScoreArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = smem + SLAB;
  ScoreShared* sh = reinterpret_cast<ScoreShared*>(sK + STAGES * SLAB);
  if (a.err && *reinterpret_cast<volatile int*>(a.err) != 0) return;
  const int b = blockIdx.y;
  const int qt = gridDim.x - 1 - blockIdx.x;                   // long rows first
  const int i0 = qt * QT;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nkt = min((i0 + QT - 1) / KT + 1, (a.S + KT - 1) / KT);
  const int qi = i0 + warp;
  const float wv = qi < a.S ? a.w[((size_t)b * a.S + qi) * HI + lane] : 0.f;
  if (tid == 0) {
    mbar_init(&sh->bar_q, 1);
    for (int s = 0; s < STAGES; ++s) mbar_init(&sh->bar_k[s], 1);
    mbar_init(&sh->bar_m[0], 1);
    mbar_init(&sh->bar_m[1], 1);
    sh->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) { tmem_alloc(&sh->tmem_slot, 256); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh->tmem_slot;
  const uint32_t lane_addr = uint32_t(warp * 32) << 16;
  volatile int* abort_flag = &sh->abort_flag;
  const uint32_t aQ = smem_u32(sQ), aK = smem_u32(sK);
  if (tid == 0) {
    mbar_expect_tx(&sh->bar_q, SLAB);
    tma_load_2d(sQ, &tmQ, &sh->bar_q, 0, (int)(((size_t)b * a.S + i0) * HI));
    for (int s = 0; s < STAGES && s < nkt; ++s) {
      mbar_expect_tx(&sh->bar_k[s], SLAB);
      tma_load_3d(sK + s * SLAB, &tmK, &sh->bar_k[s], 0, s * KT, b);
    }
  }
  bool ok = true;
  if (tid == 0) ok = mbar_wait(&sh->bar_q, 0, abort_flag, a.err, ERR_WAIT_FULL);
  constexpr uint32_t idesc = umma_idesc_bf16(128, KT, false, false);
#pragma unroll 1
  for (int t = 0; t <= nkt; ++t) {
    if (t < nkt && tid == 0 && ok) {
      const int s = t % STAGES;
      ok = mbar_wait(&sh->bar_k[s], (t / STAGES) & 1, abort_flag, a.err, ERR_WAIT_FULL);
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < DI / 16; ++k)
          umma_f16(tmem + (t & 1) * KT, umma_desc_sw128(aQ + k * 32, 16, 1024), umma_desc_sw128(aK + s * SLAB + k * 32, 16, 1024),
                   idesc, k != 0);
        umma_commit(&sh->bar_m[t & 1]);
      }
    }
    if (t >= 1) {
      const int u = t - 1;
      const bool done = mbar_wait(&sh->bar_m[u & 1], (u >> 1) & 1, abort_flag, a.err, ERR_WAIT_TMEM_FULL);
      tc_fence_after();
      if (done) {
        float* row = a.scores + ((size_t)b * a.S + qi) * a.S + u * KT + lane;
#pragma unroll 1
        for (int cb = 0; cb < KT / 32; ++cb) {
          uint32_t r[32];
          tmem_ld_32x32(tmem + (u & 1) * KT + lane_addr + cb * 32, r);
          tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int c = 0; c < 32; ++c) v[c] = fmaxf(__uint_as_float(r[c]), 0.f) * wv;
          const float sc = xreduce32<false>(v, lane);
          if (qi < a.S && u * KT + cb * 32 + lane < a.S) row[cb * 32] = sc;
        }
      }
      tc_fence_before();
      __syncthreads();                         // accumulator u&1 and key stage u%STAGES are free again
      if (tid == 0 && ok && u + STAGES < nkt) {
        const int s = u % STAGES;
        mbar_expect_tx(&sh->bar_k[s], SLAB);
        tma_load_3d(sK + s * SLAB, &tmK, &sh->bar_k[s], 0, (u + STAGES) * KT, b);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem, 256); }
}

// ------------------------------------------------------------------------------------------
// top-k by radix select
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t orderable(float f) {
  const uint32_t u = __float_as_uint(f);
  return u ^ ((u >> 31) ? 0xffffffffu : 0x80000000u);
}

// NT threads hold PER keys each in registers (S <= NT * PER); the 256-bin histogram is scanned by the first 256 threads.
template <int PER, int NT = 256>
__global__ void __launch_bounds__(NT) indexer_topk_kernel(const float* __restrict__ scores, int* __restrict__ out, int S, int K) {
  __shared__ int hist[256];
  __shared__ int warp_tot[8];
  __shared__ int sel_bin, sel_need, cnt_gt, cnt_eq;
  const size_t row = blockIdx.x;
  const int i = (int)(row % S);
  const int n = i + 1;                         // causal: keys 0..i
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int* orow = out + row * K;
  if (n <= K) {
    for (int t = tid; t < K; t += NT) orow[t] = t < n ? t : -1;
    return;
  }
  const float* srow = scores + row * S;
  uint32_t key[PER];
#pragma unroll
  for (int e = 0; e < PER; ++e) {
    const int j = e * NT + tid;
    key[e] = j < n ? orderable(srow[j]) : 0u;
  }
  uint32_t prefix = 0, mask = 0;
  int need = K;
#pragma unroll 1
  for (int shift = 24; shift >= 0; shift -= 8) {
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
#pragma unroll
    for (int e = 0; e < PER; ++e)
      if (key[e] != 0u && (key[e] & mask) == prefix) atomicAdd(&hist[(key[e] >> shift) & 255], 1);
    __syncthreads();
    // inclusive scan over bins in descending order: thread t < 256 looks at bin 255 - t
    const int h = tid < 256 ? hist[255 - tid] : 0;
    int sc = h;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, sc, o);
      if (lane >= o) sc += v;
    }
    if (lane == 31 && warp < 8) warp_tot[warp] = sc;
    __syncthreads();
    if (tid < 256) {
      int base = 0;
      for (int w2 = 0; w2 < warp; ++w2) base += warp_tot[w2];
      sc += base;                                  // elements in bins >= 255 - tid
      if (sc >= need && sc - h < need) {
        sel_bin = 255 - tid;
        sel_need = need - (sc - h);
      }
    }
    __syncthreads();
    prefix |= (uint32_t)sel_bin << shift;
    mask |= 255u << shift;
    need = sel_need;
    __syncthreads();
  }
  if (tid == 0) { cnt_gt = 0; cnt_eq = 0; }
  __syncthreads();
  const int n_gt = K - need;
#pragma unroll
  for (int e = 0; e < PER; ++e) {
    const int j = e * NT + tid;
    if (key[e] > prefix) {
      const int p = atomicAdd(&cnt_gt, 1);
      if (p < n_gt) orow[p] = j;
    } else if (key[e] == prefix && key[e] != 0u) {
      const int p = atomicAdd(&cnt_eq, 1);
      if (p < need) orow[n_gt + p] = j;
    }
  }
}

}  // namespace idx
}  // namespace cm

using namespace cm;
using namespace cm::idx;

// q [B,S,32,64] bf16, k [B,S,64] bf16, w [B,S,32] fp32 -> scores [B,S,S] fp32 (entries j <= i are defined).
extern "C" int cm_indexer_scores(const void* q, const void* k, const float* w, float* scores, int B, int S, int H, int Dh,
                                 int* err, cudaStream_t stream) {
  if (B <= 0 || S <= 0) return 0;
  if (H != HI || Dh != DI || S % QT) return -10;
  if ((long long)B * S * HI > 0x7fffffffLL) return -11;
  CUtensorMap tmQ, tmK;
  int rc = make_tmap_2d_bf16(&tmQ, q, (uint64_t)B * S * HI, DI, DI, 128, 64);
  if (rc) return rc;
  rc = make_tmap_3d_bf16(&tmK, k, B, S, DI, DI, KT, 64);
  if (rc) return rc;
  static PerDevice cfg;
  if (cfg.first()) {
    if (cudaFuncSetAttribute(indexer_scores_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, score_smem()) != cudaSuccess) return -2;
    cfg.done();
  }
  ScoreArgs a{w, scores, S, err};
  dim3 grid(S / QT, B);
  indexer_scores_kernel<<<grid, 128, score_smem(), stream>>>(tmQ, tmK, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// scores [B,S,S] fp32 -> idx [B,S,K] int32: the K largest causal entries of every row, in no particular order.
extern "C" int cm_indexer_topk(const float* scores, int* out, int B, int S, int K, cudaStream_t stream) {
  if (B <= 0 || S <= 0) return 0;
  if (K <= 0 || K > 2048) return -10;
  const unsigned rows = (unsigned)((long long)B * S);
  if (S <= 256 * 4) indexer_topk_kernel<4><<<rows, 256, 0, stream>>>(scores, out, S, K);
  else if (S <= 256 * 16) indexer_topk_kernel<16><<<rows, 256, 0, stream>>>(scores, out, S, K);
  else if (S <= 256 * 32) indexer_topk_kernel<32><<<rows, 256, 0, stream>>>(scores, out, S, K);
  else if (S <= 512 * 32) indexer_topk_kernel<32, 512><<<rows, 512, 0, stream>>>(scores, out, S, K);
  else if (S <= 1024 * 32) indexer_topk_kernel<32, 1024><<<rows, 1024, 0, stream>>>(scores, out, S, K);
  else return -12;
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
