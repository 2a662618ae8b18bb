// Per-head linear maps on 64-wide heads:  y[t, h, :] = x[t, h, :] . W[h]^T   (forward)   or   x . W[h]   (input gradient),
// and the weight gradient  dW[h] = sum_t dy[t, h, :]^T x[t, h, :].
//
// These are the "absorbed" up-projections of the sparse-attention path: the per-head query is mapped into the KV latent
// (q . W_uk) before the attention and the latent output back to the value space (o . W_uv^T) after it
// (cppmega_b200/models/attention.py; the reference gets them from Megatron's absorbed MLA,
// cppmega/megatron/mla_shared.py:39-97, where they run as batched library GEMMs).  K = 64 makes them pure memory traffic;
// the point of the kernel is to stream x once, with the tokens of a head as the M = 128 rows of a tcgen05 tile:
//
//   forward / dgrad   CTA = 128 tokens, loops over the heads: TMA (3-D map [64, H, T] over the strided activation, so a
//                     head's rows form one [128 x 64] slab) + the head's [64 x 64] weight, one 128x64x64 MMA into one of
//                     two TMEM accumulators, rows converted and stored while the next head's loads and MMA are in flight.
//   wgrad             CTA = (pair of heads, slice of the tokens): D[128 x 128] += [dy_h0 | dy_h1]^T [x_h0 | x_h1] over its
//                     token tiles (both operands read MN-major from the TMA slabs); the two diagonal 64 x 64 blocks are
//                     the two heads' gradients, added to the fp32 result with vector atomics (one add per split).
#include "common.cuh"

namespace cm {
namespace hl {

constexpr int HD = 64;                 // head width (in and out)
constexpr int BT = 128;                // tokens per tile
constexpr int SLAB = BT * 128;         // [128 x 64] bf16
constexpr int WSLAB = HD * 128;        // [64 x 64] bf16
constexpr int THREADS = 128;

static int make_tmap_heads(CUtensorMap* out, const void* base, uint64_t T, uint64_t H, uint64_t head_stride, uint64_t tok_stride) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return -1;
  cuuint64_t dims[3] = {(cuuint64_t)HD, H, T};
  cuuint64_t strides[2] = {head_stride * 2, tok_stride * 2};
  cuuint32_t box[3] = {(cuuint32_t)HD, 1, (cuuint32_t)BT};
  cuuint32_t es[3] = {1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, es,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : int(r);
}

struct Shared {
  uint64_t full[2];       // loads of stage s landed
  uint64_t done[2];       // MMA into accumulator s complete
  uint32_t tmem_slot;
  int abort_flag;
};

struct FwdArgs {
  __nv_bfloat16* y;       // [T, H, 64] with strides (y_tok, y_head)
  long long y_tok, y_head;
  int T, H;
  int* err;
};

constexpr int fwd_smem() { return 2 * SLAB + 2 * WSLAB + (int)sizeof(Shared) + 1024; }

template <bool B_MN>
__global__ void __launch_bounds__(THREADS, 2) head_linear_kernel(const __grid_constant__ CUtensorMap tmX,
                                                                 const __grid_constant__ CUtensorMap tmW, const FwdArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sX = smem;                       // 2 stages
  uint8_t* sW = sX + 2 * SLAB;              // 2 stages
  Shared* sh = reinterpret_cast<Shared*>(sW + 2 * WSLAB);
  if (a.err && *reinterpret_cast<volatile int*>(a.err) != 0) return;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int t0 = blockIdx.x * BT;
  if (tid == 0) {
    for (int i = 0; i < 2; ++i) { mbar_init(&sh->full[i], 1); mbar_init(&sh->done[i], 1); }
    sh->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) { tmem_alloc(&sh->tmem_slot, 128); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh->tmem_slot;
  const uint32_t lane_addr = uint32_t((warp & 3) * 32) << 16;
  volatile int* abort_flag = &sh->abort_flag;
  constexpr uint32_t idesc = umma_idesc_bf16(BT, HD, false, B_MN);

  auto issue_loads = [&](int h) {
    const int s = h & 1;
    mbar_expect_tx(&sh->full[s], SLAB + WSLAB);
    tma_load_3d(sX + s * SLAB, &tmX, &sh->full[s], 0, h, t0);
    tma_load_2d(sW + s * WSLAB, &tmW, &sh->full[s], 0, h * HD);
  };
  auto issue_mma = [&](int h) -> bool {
    const int s = h & 1;
    if (!mbar_wait(&sh->full[s], (h >> 1) & 1, abort_flag, a.err, ERR_WAIT_FULL)) return false;
    tc_fence_after();
    const uint32_t aX = smem_u32(sX + s * SLAB), aW = smem_u32(sW + s * WSLAB);
#pragma unroll
    for (int k = 0; k < HD / 16; ++k) {
      const uint64_t db = B_MN ? umma_desc_sw128(aW + k * 2048, WSLAB, 1024) : umma_desc_sw128(aW + k * 32, 16, 1024);
      umma_f16(tmem + s * HD, umma_desc_sw128(aX + k * 32, 16, 1024), db, idesc, k != 0);
    }
    umma_commit(&sh->done[s]);
    return true;
  };
  if (tid == 0) {
    issue_loads(0);
    if (a.H > 1) issue_loads(1);
    issue_mma(0);
  }
  bool ok = true;
  for (int h = 0; h < a.H && ok; ++h) {
    const int s = h & 1;
    // the next head's product runs while this head's rows are converted and stored
    if (tid == 0 && h + 1 < a.H && !*abort_flag) issue_mma(h + 1);
    ok = __syncthreads_and(mbar_wait(&sh->done[s], (h >> 1) & 1, abort_flag, a.err, ERR_WAIT_TMEM_FULL));   // uniform: the reads below are warp-wide
    tc_fence_after();
    if (ok) {
      // The TMEM read is a warp-wide (.sync.aligned) instruction: every lane takes part, also the lanes whose token is
      // past the end of a partial last tile; only their stores are skipped.
      const bool row_valid = t0 + tid < a.T;
      __nv_bfloat16* yrow = a.y + (size_t)(row_valid ? t0 + tid : 0) * a.y_tok + (size_t)h * a.y_head;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem + lane_addr + s * HD + c * 32, r);
        tmem_ld_wait();
        if (row_valid) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 o;
            o.x = pack_bf16(__uint_as_float(r[q * 8 + 0]), __uint_as_float(r[q * 8 + 1]));
            o.y = pack_bf16(__uint_as_float(r[q * 8 + 2]), __uint_as_float(r[q * 8 + 3]));
            o.z = pack_bf16(__uint_as_float(r[q * 8 + 4]), __uint_as_float(r[q * 8 + 5]));
            o.w = pack_bf16(__uint_as_float(r[q * 8 + 6]), __uint_as_float(r[q * 8 + 7]));
            reinterpret_cast<uint4*>(yrow)[c * 4 + q] = o;
          }
        }
      }
    }
    tc_fence_before();
    __syncthreads();                       // accumulator s and (its MMA being complete) smem stage s are free again
    tc_fence_after();
    if (tid == 0 && h + 2 < a.H && !*abort_flag) issue_loads(h + 2);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem, 128); }
}

struct WgradArgs {
  float* dw;              // [H, 64, 64] fp32, zeroed by the caller
  int T, H, tiles_per_split;
  int* err;
};

constexpr int wgrad_smem() { return 2 * 4 * SLAB + (int)sizeof(Shared) + 1024; }

__global__ void __launch_bounds__(THREADS, 1) head_linear_wgrad_kernel(const __grid_constant__ CUtensorMap tmDY,
                                                                       const __grid_constant__ CUtensorMap tmX, const WgradArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;                       // 2 stages x [dy_h0 | dy_h1]
  uint8_t* sB = sA + 4 * SLAB;              // 2 stages x [x_h0 | x_h1]
  Shared* sh = reinterpret_cast<Shared*>(sB + 4 * SLAB);
  if (a.err && *reinterpret_cast<volatile int*>(a.err) != 0) return;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int hp = blockIdx.x, split = blockIdx.y;
  const int n_tiles_all = (a.T + BT - 1) / BT;
  const int tile0 = split * a.tiles_per_split;
  const int n_tiles = min(a.tiles_per_split, n_tiles_all - tile0);
  if (n_tiles <= 0) return;
  if (tid == 0) {
    for (int i = 0; i < 2; ++i) { mbar_init(&sh->full[i], 1); mbar_init(&sh->done[i], 1); }
    sh->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) { tmem_alloc(&sh->tmem_slot, 128); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh->tmem_slot;
  const uint32_t lane_addr = uint32_t((warp & 3) * 32) << 16;
  volatile int* abort_flag = &sh->abort_flag;
  constexpr uint32_t idesc = umma_idesc_bf16(128, 128, true, true);
  const bool second = 2 * hp + 1 < a.H;     // an odd head count leaves the last pair half empty (TMA fills zeros)

  if (tid == 0) {
    auto issue_loads = [&](int it) {
      const int s = it & 1, t0 = (tile0 + it) * BT;
      mbar_expect_tx(&sh->full[s], 4 * SLAB);
      tma_load_3d(sA + s * 2 * SLAB, &tmDY, &sh->full[s], 0, 2 * hp, t0);
      tma_load_3d(sA + s * 2 * SLAB + SLAB, &tmDY, &sh->full[s], 0, 2 * hp + 1, t0);
      tma_load_3d(sB + s * 2 * SLAB, &tmX, &sh->full[s], 0, 2 * hp, t0);
      tma_load_3d(sB + s * 2 * SLAB + SLAB, &tmX, &sh->full[s], 0, 2 * hp + 1, t0);
    };
    issue_loads(0);
    if (n_tiles > 1) issue_loads(1);
    bool go = true;
    for (int it = 0; it < n_tiles && go; ++it) {
      const int s = it & 1;
      go = mbar_wait(&sh->full[s], (it >> 1) & 1, abort_flag, a.err, ERR_WAIT_FULL);
      if (!go) break;
      tc_fence_after();
      const uint32_t aA = smem_u32(sA + s * 2 * SLAB), aB = smem_u32(sB + s * 2 * SLAB);
#pragma unroll
      for (int k = 0; k < BT / 16; ++k)
        umma_f16(tmem, umma_desc_sw128(aA + k * 2048, SLAB, 1024), umma_desc_sw128(aB + k * 2048, SLAB, 1024), idesc, (it | k) != 0);
      umma_commit(&sh->done[s]);
      if (it + 2 < n_tiles) {               // stage s is reloaded once its products have retired
        go = mbar_wait(&sh->done[s], (it >> 1) & 1, abort_flag, a.err, ERR_WAIT_TMEM_FULL);
        if (go) issue_loads(it + 2);
      }
    }
  }
  // Everyone waits for the last product (the commit of the last tile covers all earlier ones).  A parity wait only tells
  // the two most recent phases apart, so the other threads may look at the barrier only after thread 0 has consumed all
  // earlier phases of it, i.e. after its loop.
  __syncthreads();
  const int last = n_tiles - 1;
  const bool ok = __syncthreads_and(mbar_wait(&sh->done[last & 1], (last >> 1) & 1, abort_flag, a.err, ERR_WAIT_TMEM_FULL));
  tc_fence_after();
  if (ok) {
    // TMEM lane = output feature (0..63: head 2hp, 64..127: head 2hp+1); columns = input features of the two heads
    const int hsel = tid >> 6, o = tid & 63, h = 2 * hp + hsel;
    if (hsel == 0 || second) {
      float* dst = a.dw + ((size_t)h * HD + o) * HD;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem + lane_addr + hsel * HD + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int v = 0; v < 8; ++v)
          atomicAdd(reinterpret_cast<float4*>(dst + c * 32) + v,
                    make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]), __uint_as_float(r[4 * v + 2]),
                                __uint_as_float(r[4 * v + 3])));
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem, 128); }
}

}  // namespace hl
}  // namespace cm

using namespace cm;
using namespace cm::hl;

// x [T, H, 64] bf16 with element strides (x_tok, x_head), innermost contiguous; w [H, 64, 64] bf16 packed;
// y [T, H, 64] bf16 with strides (y_tok, y_head).  transposed = 0: y = x . w[h]^T (w is [out, in]); 1: y = x . w[h].
// Strides must be multiples of 8 elements and the bases 16-byte aligned (TMA).
extern "C" int cm_head_linear(const void* x, const void* w, void* y, int T, int H, long long x_tok, long long x_head,
                              long long y_tok, long long y_head, int transposed, int* err, cudaStream_t stream) {
  if (T <= 0 || H <= 0) return 0;
  if ((x_tok % 8) || (x_head % 8) || (y_tok % 8) || (y_head % 8)) return -10;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(y)) & 15) return -11;
  CUtensorMap tmX, tmW;
  int rc = make_tmap_heads(&tmX, x, (uint64_t)T, (uint64_t)H, (uint64_t)x_head, (uint64_t)x_tok);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tmW, w, (uint64_t)H * HD, HD, HD, HD, 64);
  if (rc) return rc;
  FwdArgs a{(__nv_bfloat16*)y, y_tok, y_head, T, H, err};
  const unsigned grid = (unsigned)((T + BT - 1) / BT);
  static PerDevice cfg;
  if (cfg.first()) {
    if (cudaFuncSetAttribute(head_linear_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, fwd_smem()) != cudaSuccess) return -2;
    if (cudaFuncSetAttribute(head_linear_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, fwd_smem()) != cudaSuccess) return -2;
    cfg.done();
  }
  if (transposed) head_linear_kernel<true><<<grid, THREADS, fwd_smem(), stream>>>(tmX, tmW, a);
  else head_linear_kernel<false><<<grid, THREADS, fwd_smem(), stream>>>(tmX, tmW, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// dw [H, 64, 64] fp32 (ZEROED by the caller) += sum_t dy[t, h, :]^T x[t, h, :];  dy / x as x above.
extern "C" int cm_head_linear_wgrad(const void* dy, const void* x, float* dw, int T, int H, long long dy_tok, long long dy_head,
                                    long long x_tok, long long x_head, int* err, cudaStream_t stream) {
  if (T <= 0 || H <= 0) return 0;
  if ((x_tok % 8) || (x_head % 8) || (dy_tok % 8) || (dy_head % 8)) return -10;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy)) & 15) return -11;
  CUtensorMap tmDY, tmX;
  int rc = make_tmap_heads(&tmDY, dy, (uint64_t)T, (uint64_t)H, (uint64_t)dy_head, (uint64_t)dy_tok);
  if (rc) return rc;
  rc = make_tmap_heads(&tmX, x, (uint64_t)T, (uint64_t)H, (uint64_t)x_head, (uint64_t)x_tok);
  if (rc) return rc;
  static PerDevice cfg;
  if (cfg.first()) {
    if (cudaFuncSetAttribute(head_linear_wgrad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, wgrad_smem()) != cudaSuccess) return -2;
    cfg.done();
  }
  const int pairs = (H + 1) / 2;
  const int n_tiles = (T + BT - 1) / BT;
  int splits = (2 * sm_count() + pairs - 1) / pairs;           // about two CTAs per SM in total
  if (splits > n_tiles) splits = n_tiles;
  if (splits < 1) splits = 1;
  const int per = (n_tiles + splits - 1) / splits;
  splits = (n_tiles + per - 1) / per;
  WgradArgs a{dw, T, H, per, err};
  dim3 grid((unsigned)pairs, (unsigned)splits);
  head_linear_wgrad_kernel<<<grid, THREADS, wgrad_smem(), stream>>>(tmDY, tmX, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
