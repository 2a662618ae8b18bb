// Sparse latent attention (DSA core): every query attends over TOPK gathered rows of one shared KV latent.
//
//   s[h,j] = scale * q[h,:] . kv[idx[j],:]      (D = 128 = 64 latent + 64 rope dims, idx[j] < 0: masked)
//   p      = softmax_j(s)                        o[h,:] = sum_j p[h,j] kv[idx[j], :64]        lse[h] = logsumexp_j s
//
// One CTA per query token.  The 32 heads of a token are too few rows for a tcgen05 tile, so both products are
// computed transposed, with the gathered keys on the M axis:
//   S^T [256 keys x 32 heads]  = KVg [keys x 128]        . Q^T        (2 M=128 tiles, N = 32,  K = 128)
//   O^T [128 dims x 64(32)]    = KVg^T [dims x 256 keys] . P^T        (M = 128, N = 64 (heads, zero padded), K = 256)
// KVg lives once in shared memory (rows gathered with 16-byte async copies into the 128-byte-swizzled layout) and is
// read K-major by the first product and MN-major by the second.  Thread j owns key j between the products: its TMEM
// lane holds the 32 scores of that key, and the softmax statistics per head are all-reduced over the 256 keys with a
// transposing shuffle reduction (31 shuffles for 32 values) plus one shared-memory step.
// Contract of the reference's TileLang kernels (cppmega/megatron/sparse_mla_ops/tilelang_sparse_mla_fwd.py:137-290:
// 64 gathered rows per iteration, online softmax in exp2, heads padded to 16; sparse_mla.py:17-39 for the op).
#include "common.cuh"

namespace cm {
namespace smla {

constexpr int D = 128;        // [latent | rope]
constexpr int DV = 64;        // value = latent part
constexpr int TK = 256;       // gathered keys per query
constexpr int HQ = 32;        // heads per token handled by this kernel
constexpr int SLAB = 128 * 128;
constexpr int THREADS = 256;

__device__ __forceinline__ int sw_off(int row, int c) { return row * 128 + ((c ^ (row & 7)) << 4); }

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}

struct Shared {
  float red[8][32];
  float fin_m[32];
  float fin_l[32];
  uint64_t bars[3];
  uint32_t tmem_slot;
  int abort_flag;
};

struct FwdArgs {
  const __nv_bfloat16* kv;    // [B, Skv, D]
  const int* idx;             // [B, S, TK]
  __nv_bfloat16* out;         // [B, S, HQ, DV]
  float* lse;                 // [B, S, HQ] natural log
  int S, Skv;
  long long tokens;
  float scale_log2;           // softmax scale * log2(e)
  int* err;
};

constexpr int fwd_smem() { return 4 * SLAB + 2 * SLAB + 2 * HQ * 128 + (int)sizeof(Shared) + 1024; }

__global__ void __launch_bounds__(THREADS, 2) sparse_mla_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const FwdArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sKV = smem;                       // 2 key tiles x 2 dim slabs
  uint8_t* sP = sKV + 4 * SLAB;              // 2 key tiles x [128 keys x 64 heads]
  uint8_t* sQ = sP + 2 * SLAB;               // 2 dim slabs x [32 heads x 64]
  Shared* sh = reinterpret_cast<Shared*>(sQ + 2 * HQ * 128);
  if (a.err && *reinterpret_cast<volatile int*>(a.err) != 0) return;

  const long long token = blockIdx.x;
  const int b = (int)(token / a.S);
  const int tid = threadIdx.x, i = tid & 127, wg = tid >> 7, warp = tid >> 5, lane = tid & 31;
  const int kidx = a.idx[token * TK + tid];
  const bool valid = kidx >= 0 && kidx < a.Skv;
  if (tid == 0) {
    mbar_init(&sh->bars[0], 1);
    mbar_init(&sh->bars[1], 1);
    mbar_init(&sh->bars[2], 1);
    sh->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) { tmem_alloc(&sh->tmem_slot, 128); tmem_relinquish(); }
  // gather this thread's key row (16 chunks of 16 bytes) into the swizzled tile of its key half
  {
    uint8_t* tile = sKV + wg * 2 * SLAB;
    if (valid) {
      const __nv_bfloat16* src = a.kv + ((size_t)b * a.Skv + kidx) * D;
#pragma unroll
      for (int c = 0; c < 16; ++c) cp_async16(tile + (c >> 3) * SLAB + sw_off(i, c & 7), src + c * 8);
    } else {
      const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int c = 0; c < 16; ++c) *reinterpret_cast<uint4*>(tile + (c >> 3) * SLAB + sw_off(i, c & 7)) = z;
    }
    const uint4 z = make_uint4(0, 0, 0, 0);     // head columns 32..63 of P^T stay zero
#pragma unroll
    for (int cc = 4; cc < 8; ++cc) *reinterpret_cast<uint4*>(sP + wg * SLAB + sw_off(i, cc)) = z;
  }
  tc_fence_before();
  __syncthreads();                             // barriers initialised, TMEM address published
  tc_fence_after();
  const uint32_t tmem = sh->tmem_slot;
  const uint32_t tS = tmem, tO = tmem + 64;
  const uint32_t lane_addr = uint32_t((warp & 3) * 32) << 16;
  volatile int* abort_flag = &sh->abort_flag;
  if (tid == 0) {
    mbar_expect_tx(&sh->bars[0], 2 * HQ * 128);
    tma_load_2d(sQ, &tmQ, &sh->bars[0], 0, (int)(token * HQ));
    tma_load_2d(sQ + HQ * 128, &tmQ, &sh->bars[0], 64, (int)(token * HQ));
  }
  cp_async_wait_all();
  fence_proxy_async_smem();
  __syncthreads();
  const uint32_t aKV = smem_u32(sKV), aP = smem_u32(sP), aQ = smem_u32(sQ);
  if (tid == 0) {
    if (mbar_wait(&sh->bars[0], 0, abort_flag, a.err, ERR_WAIT_FULL)) {
      constexpr uint32_t id1 = umma_idesc_bf16(128, HQ, false, false);
#pragma unroll
      for (int kt = 0; kt < 2; ++kt)
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          umma_f16(tS + kt * HQ, umma_desc_sw128(aKV + kt * 2 * SLAB + (k >> 2) * SLAB + (k & 3) * 32, 16, 1024),
                   umma_desc_sw128(aQ + (k >> 2) * HQ * 128 + (k & 3) * 32, 16, 1024), id1, k != 0);
      umma_commit(&sh->bars[1]);
    }
  }
  bool ok = mbar_wait(&sh->bars[1], 0, abort_flag, a.err, ERR_WAIT_TMEM_FULL);
  tc_fence_after();
  float x[32];
  if (ok) {
    uint32_t r[32];
    tmem_ld_32x32(tS + lane_addr + wg * HQ, r);
    tmem_ld_wait();
#pragma unroll
    for (int h = 0; h < 32; ++h) x[h] = valid ? __uint_as_float(r[h]) * a.scale_log2 : -INFINITY;
  } else {
#pragma unroll
    for (int h = 0; h < 32; ++h) x[h] = -INFINITY;
  }
  // per-head maximum over the 256 keys
  sh->red[warp][lane] = xreduce32<true>(x, lane);
  __syncthreads();
  if (warp == 0) {
    float m = sh->red[0][lane];
#pragma unroll
    for (int w = 1; w < 8; ++w) m = fmaxf(m, sh->red[w][lane]);
    sh->fin_m[lane] = m;
  }
  __syncthreads();
  {
    float mx[32];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const float4 t = reinterpret_cast<const float4*>(sh->fin_m)[q];
      mx[4 * q] = t.x; mx[4 * q + 1] = t.y; mx[4 * q + 2] = t.z; mx[4 * q + 3] = t.w;
    }
#pragma unroll
    for (int h = 0; h < 32; ++h) x[h] = exp2f(x[h] - (mx[h] == -INFINITY ? 0.f : mx[h]));
  }
  // P^T row of this key (unnormalised) as the B operand of the second product
#pragma unroll
  for (int cc = 0; cc < 4; ++cc) {
    uint4 o;
    o.x = pack_bf16(x[cc * 8 + 0], x[cc * 8 + 1]); o.y = pack_bf16(x[cc * 8 + 2], x[cc * 8 + 3]);
    o.z = pack_bf16(x[cc * 8 + 4], x[cc * 8 + 5]); o.w = pack_bf16(x[cc * 8 + 6], x[cc * 8 + 7]);
    *reinterpret_cast<uint4*>(sP + wg * SLAB + sw_off(i, cc)) = o;
  }
  fence_proxy_async_smem();
  sh->red[warp][lane] = xreduce32<false>(x, lane);     // the maxima in `red` were consumed before the last barrier
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && !*abort_flag) {
    tc_fence_after();
    constexpr uint32_t id2 = umma_idesc_bf16(128, 64, true, true);
#pragma unroll
    for (int kt = 0; kt < 2; ++kt)
#pragma unroll
      for (int k = 0; k < 8; ++k)
        umma_f16(tO, umma_desc_sw128(aKV + kt * 2 * SLAB + k * 2048, SLAB, 1024),
                 umma_desc_sw128(aP + kt * SLAB + k * 2048, SLAB, 1024), id2, (kt | k) != 0);
    umma_commit(&sh->bars[2]);
  }
  if (warp == 0) {
    float l = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) l += sh->red[w][lane];
    sh->fin_l[lane] = l;
    const float m = sh->fin_m[lane];
    a.lse[token * HQ + lane] = l > 0.f ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
  }
  __syncthreads();
  ok = mbar_wait(&sh->bars[2], 0, abort_flag, a.err, ERR_WAIT_TMEM_FULL);
  tc_fence_after();
  if (ok && wg == 0 && i < DV) {                 // TMEM lane = value dim, column = head
    uint32_t r[32];
    tmem_ld_32x32(tO + lane_addr, r);
    tmem_ld_wait();
    __nv_bfloat16* orow = a.out + (size_t)token * HQ * DV + i;
#pragma unroll
    for (int h = 0; h < HQ; ++h) {
      const float l = sh->fin_l[h];
      orow[h * DV] = __float2bfloat16(l > 0.f ? __fdividef(__uint_as_float(r[h]), l) : 0.f);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem, 128); }
}


// ------------------------------------------------------------------------------------------
// backward: dq, and dkv accumulated with vector atomics into an fp32 buffer
//   P = exp(s - lse);  dP = dO V^T;  dS = scale * P o (dP - delta),  delta[h] = dO[h,:] . O[h,:]
//   dQ^T [dims x heads]  = KVg^T . dS^T                      (N = 64: columns 32..63 are a by-product, ignored)
//   dKVg [keys x 128]    = [dS^T | P^T] . [Q ; (dO | 0)]     (one K = 64 product gives dK and adds dV to dims 0..63)
// The combined [dS^T | P^T] row of a key is exactly one 128-byte shared-memory row, written by the thread that
// owns the key.  dKVg rows are scattered to dkv[b, idx[j], :] with 16-byte float atomics, one key tile at a time.
// ------------------------------------------------------------------------------------------
struct BwdShared {
  float delta[32];
  float lse2[32];
  int kidx[TK];
  uint64_t bars[4];
  uint32_t tmem_slot;
  int abort_flag;
};

struct BwdArgs {
  const __nv_bfloat16* kv;    // [B, Skv, D]
  const int* idx;             // [B, S, TK]
  const __nv_bfloat16* o;     // [B, S, HQ, DV] forward output
  const __nv_bfloat16* dout;  // [B, S, HQ, DV]
  const float* lse;           // [B, S, HQ]
  __nv_bfloat16* dq;          // [B, S, HQ, D]
  float* dkv;                 // [B, Skv, D] fp32, accumulated
  int S, Skv;
  float scale, scale_log2;
  int* err;
};

constexpr int bwd_smem() { return 4 * SLAB + 2 * SLAB + 2 * 64 * 128 + (int)sizeof(BwdShared) + 1024; }

__global__ void __launch_bounds__(THREADS, 2) sparse_mla_bwd_kernel(const __grid_constant__ CUtensorMap tmQ,
                                                                    const __grid_constant__ CUtensorMap tmdO, const BwdArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sKV = smem;                       // 2 key tiles x 2 dim slabs
  uint8_t* sA = sKV + 4 * SLAB;              // 2 key tiles x [128 keys x (32 dS | 32 P)]
  uint8_t* sB = sA + 2 * SLAB;               // 2 dim slabs x [64 rows x 64]: rows 0..31 Q, rows 32..63 (dO | 0)
  BwdShared* sh = reinterpret_cast<BwdShared*>(sB + 2 * 64 * 128);
  if (a.err && *reinterpret_cast<volatile int*>(a.err) != 0) return;

  const long long token = blockIdx.x;
  const int b = (int)(token / a.S);
  const int tid = threadIdx.x, i = tid & 127, wg = tid >> 7, warp = tid >> 5, lane = tid & 31;
  const int kidx = a.idx[token * TK + tid];
  const bool valid = kidx >= 0 && kidx < a.Skv;
  sh->kidx[tid] = valid ? kidx : -1;
  if (tid == 0) {
    for (int q = 0; q < 4; ++q) mbar_init(&sh->bars[q], 1);
    sh->abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) { tmem_alloc(&sh->tmem_slot, 256); tmem_relinquish(); }
  {
    uint8_t* tile = sKV + wg * 2 * SLAB;
    if (valid) {
      const __nv_bfloat16* src = a.kv + ((size_t)b * a.Skv + kidx) * D;
#pragma unroll
      for (int c = 0; c < 16; ++c) cp_async16(tile + (c >> 3) * SLAB + sw_off(i, c & 7), src + c * 8);
    } else {
      const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int c = 0; c < 16; ++c) *reinterpret_cast<uint4*>(tile + (c >> 3) * SLAB + sw_off(i, c & 7)) = z;
    }
    // rows 32..63 of the second slab of sB are the zero half of (dO | 0): 4 KB = 256 threads x 16 bytes
    *reinterpret_cast<uint4*>(sB + 64 * 128 + 32 * 128 + tid * 16) = make_uint4(0, 0, 0, 0);
  }
  // delta[h] = dO[h,:] . O[h,:]  (warp w: heads 4w .. 4w+3; lane: two value dims)
  {
#pragma unroll
    for (int hh = 0; hh < 4; ++hh) {
      const int h = warp * 4 + hh;
      const size_t off = ((size_t)token * HQ + h) * DV + lane * 2;
      const float2 ov = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(a.o + off));
      const float2 dv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(a.dout + off));
      const float d = warp_sum(ov.x * dv.x + ov.y * dv.y);
      if (lane == 0) {
        sh->delta[h] = d;
        sh->lse2[h] = a.lse[token * HQ + h] * 1.4426950408889634f;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh->tmem_slot;
  const uint32_t tS = tmem, tdP = tmem + 64, tdQ = tmem, tdKV = tmem + 128;
  const uint32_t lane_addr = uint32_t((warp & 3) * 32) << 16;
  volatile int* abort_flag = &sh->abort_flag;
  if (tid == 0) {
    mbar_expect_tx(&sh->bars[0], 3 * HQ * 128);
    tma_load_2d(sB, &tmQ, &sh->bars[0], 0, (int)(token * HQ));
    tma_load_2d(sB + 64 * 128, &tmQ, &sh->bars[0], 64, (int)(token * HQ));
    tma_load_2d(sB + 32 * 128, &tmdO, &sh->bars[0], 0, (int)(token * HQ));
  }
  cp_async_wait_all();
  fence_proxy_async_smem();
  __syncthreads();
  const uint32_t aKV = smem_u32(sKV), aA = smem_u32(sA), aB = smem_u32(sB);
  if (tid == 0) {
    if (mbar_wait(&sh->bars[0], 0, abort_flag, a.err, ERR_WAIT_FULL)) {
      constexpr uint32_t id1 = umma_idesc_bf16(128, HQ, false, false);
#pragma unroll
      for (int kt = 0; kt < 2; ++kt) {
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          umma_f16(tS + kt * HQ, umma_desc_sw128(aKV + kt * 2 * SLAB + (k >> 2) * SLAB + (k & 3) * 32, 16, 1024),
                   umma_desc_sw128(aB + (k >> 2) * 64 * 128 + (k & 3) * 32, 16, 1024), id1, k != 0);
#pragma unroll
        for (int k = 0; k < DV / 16; ++k)
          umma_f16(tdP + kt * HQ, umma_desc_sw128(aKV + kt * 2 * SLAB + k * 32, 16, 1024),
                   umma_desc_sw128(aB + 32 * 128 + k * 32, 16, 1024), id1, k != 0);
      }
      umma_commit(&sh->bars[1]);
    }
  }
  bool ok = mbar_wait(&sh->bars[1], 0, abort_flag, a.err, ERR_WAIT_TMEM_FULL);
  tc_fence_after();
  if (ok) {
    uint32_t rs[32], rp[32];
    tmem_ld_32x32(tS + lane_addr + wg * HQ, rs);
    tmem_ld_32x32(tdP + lane_addr + wg * HQ, rp);
    tmem_ld_wait();
    float ds[32], pp[32];
#pragma unroll
    for (int h = 0; h < 32; ++h) {
      const float p = valid ? exp2f(__uint_as_float(rs[h]) * a.scale_log2 - sh->lse2[h]) : 0.f;
      pp[h] = p;
      ds[h] = p * (__uint_as_float(rp[h]) - sh->delta[h]) * a.scale;
    }
    uint8_t* slab = sA + wg * SLAB;
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) {
      uint4 o;
      o.x = pack_bf16(ds[cc * 8 + 0], ds[cc * 8 + 1]); o.y = pack_bf16(ds[cc * 8 + 2], ds[cc * 8 + 3]);
      o.z = pack_bf16(ds[cc * 8 + 4], ds[cc * 8 + 5]); o.w = pack_bf16(ds[cc * 8 + 6], ds[cc * 8 + 7]);
      *reinterpret_cast<uint4*>(slab + sw_off(i, cc)) = o;
      uint4 q;
      q.x = pack_bf16(pp[cc * 8 + 0], pp[cc * 8 + 1]); q.y = pack_bf16(pp[cc * 8 + 2], pp[cc * 8 + 3]);
      q.z = pack_bf16(pp[cc * 8 + 4], pp[cc * 8 + 5]); q.w = pack_bf16(pp[cc * 8 + 6], pp[cc * 8 + 7]);
      *reinterpret_cast<uint4*>(slab + sw_off(i, 4 + cc)) = q;
    }
    fence_proxy_async_smem();
  }
  tc_fence_before();
  __syncthreads();
  constexpr uint32_t id_dq = umma_idesc_bf16(128, 64, true, true);
  constexpr uint32_t id_dkv = umma_idesc_bf16(128, 128, false, true);
  if (tid == 0 && !*abort_flag) {
    tc_fence_after();
#pragma unroll
    for (int kt = 0; kt < 2; ++kt)
#pragma unroll
      for (int k = 0; k < 8; ++k)
        umma_f16(tdQ, umma_desc_sw128(aKV + kt * 2 * SLAB + k * 2048, SLAB, 1024),
                 umma_desc_sw128(aA + kt * SLAB + k * 2048, SLAB, 1024), id_dq, (kt | k) != 0);
#pragma unroll
    for (int k = 0; k < 4; ++k)
      umma_f16(tdKV, umma_desc_sw128(aA + k * 32, 16, 1024), umma_desc_sw128(aB + k * 2048, 64 * 128, 1024), id_dkv, k != 0);
    umma_commit(&sh->bars[2]);
  }
  ok = mbar_wait(&sh->bars[2], 0, abort_flag, a.err, ERR_WAIT_TMEM_FULL);
  tc_fence_after();
  if (ok) {
    if (wg == 0) {                                // dQ^T: TMEM lane = dim, column = head
      uint32_t r[32];
      tmem_ld_32x32(tdQ + lane_addr, r);
      tmem_ld_wait();
      __nv_bfloat16* qrow = a.dq + (size_t)token * HQ * D + i;
#pragma unroll
      for (int h = 0; h < HQ; ++h) qrow[h * D] = __float2bfloat16(__uint_as_float(r[h]));
    }
  }
  // scatter the two key tiles: thread (i, wg) adds dims [64 wg, 64 wg + 64) of key kt*128 + i
#pragma unroll 1
  for (int kt = 0; kt < 2; ++kt) {
    if (kt == 1) {
      tc_fence_before();
      __syncthreads();                            // every thread has read tile 0 out of TMEM
      if (tid == 0 && !*abort_flag) {
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_f16(tdKV, umma_desc_sw128(aA + SLAB + k * 32, 16, 1024), umma_desc_sw128(aB + k * 2048, 64 * 128, 1024), id_dkv,
                   k != 0);
        umma_commit(&sh->bars[3]);
      }
      ok = mbar_wait(&sh->bars[3], 0, abort_flag, a.err, ERR_WAIT_TMEM_FULL);
      tc_fence_after();
    }
    const int key = sh->kidx[kt * 128 + i];
    if (ok) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t r[32];
        tmem_ld_32x32(tdKV + lane_addr + wg * 64 + half * 32, r);
        tmem_ld_wait();
        if (key >= 0) {
          float4* dst = reinterpret_cast<float4*>(a.dkv + ((size_t)b * a.Skv + key) * D + wg * 64 + half * 32);
#pragma unroll
          for (int v = 0; v < 8; ++v)
            atomicAdd(dst + v, make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                                           __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3])));
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem, 256); }
}

}  // namespace smla
}  // namespace cm

using namespace cm;
using namespace cm::smla;

// q [B,S,32,128] bf16, kv [B,Skv,128] bf16, idx [B,S,256] int32 (-1 = masked) -> out [B,S,32,64] bf16, lse [B,S,32] fp32
extern "C" int cm_sparse_mla_fwd(const void* q, const void* kv, const int* idx, void* out, float* lse, int B, int S, int Skv,
                                 int Hq, int Dq, int topk, int dv, float scale, int* err, cudaStream_t stream) {
  if (B <= 0 || S <= 0) return 0;
  if (Hq != HQ || Dq != D || topk != TK || dv != DV) return -10;
  const long long tokens = (long long)B * S;
  if (tokens * HQ > 0x7fffffffLL) return -11;
  CUtensorMap tmQ;
  int rc = make_tmap_2d_bf16(&tmQ, q, (uint64_t)tokens * HQ, D, D, HQ, 64);
  if (rc) return rc;
  static PerDevice cfg;
  if (cfg.first()) {
    if (cudaFuncSetAttribute(sparse_mla_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, fwd_smem()) != cudaSuccess) return -2;
    cfg.done();
  }
  FwdArgs a{(const __nv_bfloat16*)kv, idx, (__nv_bfloat16*)out, lse, S, Skv, tokens, scale * 1.4426950408889634f, err};
  sparse_mla_fwd_kernel<<<(unsigned)tokens, THREADS, fwd_smem(), stream>>>(tmQ, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// dkv [B,Skv,128] fp32 must be zeroed by the caller (gradients of all tokens accumulate into it); dq [B,S,32,128] bf16.
extern "C" int cm_sparse_mla_bwd(const void* q, const void* kv, const int* idx, const void* o, const void* dout, const float* lse,
                                 void* dq, float* dkv, int B, int S, int Skv, int Hq, int Dq, int topk, int dv, float scale,
                                 int* err, cudaStream_t stream) {
  if (B <= 0 || S <= 0) return 0;
  if (Hq != HQ || Dq != D || topk != TK || dv != DV) return -10;
  const long long tokens = (long long)B * S;
  if (tokens * HQ > 0x7fffffffLL) return -11;
  CUtensorMap tmQ, tmdO;
  int rc = make_tmap_2d_bf16(&tmQ, q, (uint64_t)tokens * HQ, D, D, HQ, 64);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tmdO, dout, (uint64_t)tokens * HQ, DV, DV, HQ, 64);
  if (rc) return rc;
  static PerDevice cfg;
  if (cfg.first()) {
    if (cudaFuncSetAttribute(sparse_mla_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bwd_smem()) != cudaSuccess) return -2;
    cfg.done();
  }
  BwdArgs a{(const __nv_bfloat16*)kv, idx, (const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, lse, (__nv_bfloat16*)dq, dkv,
            S, Skv, scale, scale * 1.4426950408889634f, err};
  sparse_mla_bwd_kernel<<<(unsigned)tokens, THREADS, bwd_smem(), stream>>>(tmQ, tmdO, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
