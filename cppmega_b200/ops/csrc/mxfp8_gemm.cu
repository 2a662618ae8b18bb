// MXFP8 block-scaled GEMM on the 5th-generation tensor cores:
//
//     C[M,N] (+)= sum_k  (A[m,k] * 2^(SFA[m,k/32]-127)) * (B[n,k] * 2^(SFB[n,k/32]-127))
//
// A [M,K] and B [N,K] are E4M3 payloads with the reduction index contiguous ("TN"); SFA / SFB are the E8M0 scale bytes
// in the 128x4 tile order ([row tile][k tile][32][4][4], 512 bytes per 128 rows x 128 k).  The scaling happens inside
// `tcgen05.mma.kind::mxf8f6f4.block_scale`: the scale bytes of a k tile are copied from shared memory into TMEM with
// `tcgen05.cp.32x128b.warpx4` (4 columns for the 128 rows of A, 8 columns for the 256 rows of B; byte j of a column
// belongs to the j-th 32-wide k block, which the instruction descriptor selects), and the four MMAs of the k tile then
// read payloads through 128-byte-swizzled descriptors exactly like the bf16 kernel, at twice its rate.
//
// Persistent, warp-specialised, one CTA per SM, tile 128 x 256 x 128:
//   warp 0      TMA producer: payload boxes by tensor map, scale tiles by bulk copy, 4-stage ring (198 KB)
//   warp 1      TMEM owner, scale copies and MMA issue (one elected lane)
//   warps 2..9  epilogue: warp w drains lane quarter w%4, column half (w-2)/4 of the accumulator into 128 registers,
//               hands the accumulator back at once and only then converts and stores, so the next tile's main loop
//               runs under the stores although only one 256-column accumulator fits beside the scale columns.
// Grouped modes (experts): GROUPED_ROWS takes the expert of every 128-row tile of A / C from tile_expert[] (-1 = unused
// tile) and addresses B as one [rows, K] matrix in which expert e starts b_row_e rows further down (forward: the
// stacked [E*N, K] weights) or b_k_e columns further right (dgrad: the stacked transposed weights [N, E*K]);
// GROUPED_K reduces over per-expert ranges of the shared K axis (token rows, multiples of 128) into a stack [E, M, N]
// (expert weight gradients from the token-transposed operands).
// The other products of a linear layer use the same kernel on operands quantised along their own reduction
// dimension and stored transposed (dgrad: dy along N with W^T; wgrad: dy^T and x^T along tokens), so no
// MN-major FP8 path is needed.  This is the sm_100 counterpart of the reference's CUTLASS / FlashInfer MXFP8 GEMM
// wrappers (cppmega/megatron/cutlass_mxfp8_gemm.py:102-506, cppmega/megatron/flashinfer_mxfp8_gemm.py:146-160,
// cuda_ext/cutlass_mxfp8_gemm.cu:56-360).
#include "common.cuh"

namespace cm {
namespace mxg {

constexpr int BM = 128, BN = 256, BK = 128;      // BK in elements = bytes
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK, B_BYTES = BN * BK, SFA_BYTES = 512, SFB_BYTES = 1024;
constexpr int SF_OFF = STAGES * (A_BYTES + B_BYTES);
constexpr int BAR_OFF = SF_OFF + STAGES * (SFA_BYTES + SFB_BYTES);
constexpr int SMEM_TOTAL = BAR_OFF + 256 + 1024;
constexpr int THREADS = 320;
constexpr int TMEM_COLS = 512;                   // 256 accumulator + 4 SFA + 8 SFB, rounded up to a power of two
constexpr int SFA_COL = 256, SFB_COL = 260;

enum Mode : int { DENSE = 0, GROUPED_ROWS = 1, GROUPED_K = 2 };

struct Args {
  int M, N, K;               // GROUPED_ROWS: M = allocated rows; GROUPED_K: M, N per expert, K = total reduction length
  long long ldc;
  const uint8_t* sfa;
  const uint8_t* sfb;
  int* err;
  int sfa_nkt, sfb_nkt;      // k tiles per row tile in the two scale buffers
  const int* tile_expert;    // GROUPED_ROWS: [M / 128]
  const int* seg_offsets;    // GROUPED_K: [E + 1], multiples of 128
  int num_experts;
  int b_row_e, b_k_e;        // GROUPED_ROWS: row / column offset of expert e in B is e * b_row_e / e * b_k_e (multiples of 128)
};

struct Tile {
  int mt, nt, e;
  int kt0, nkt;              // k tiles [kt0, kt0 + nkt) of A (and of B, shifted by b_kt0)
  int b_row0, b_kt0;         // first row of the B tile, first k tile of B
  bool two;                  // the second 128-row scale tile of B exists
};

// no-swizzle descriptor of a 32 x 16-byte scale tile: 8-row core matrices 128 bytes apart
__device__ __forceinline__ uint64_t sf_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(128 >> 4) << 32;
  d |= 1ull << 46;
  return d;
}
__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint64_t desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
__device__ __forceinline__ void umma_mxf8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa,
                                          uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
      : "memory");
}
// E4M3 x E4M3, E8M0 scales, K-major operands; the scale-byte selectors are added per k block
__host__ __device__ constexpr uint32_t idesc_mxf8(int m, int n) {
  return (uint32_t(n >> 3) << 17) | (1u << 23) | (uint32_t(m >> 4) << 24);
}
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

template <typename OutT, bool ACC, int MODE>
__global__ void __launch_bounds__(THREADS, 1)
mxfp8_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, OutT* __restrict__ C, const Args args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_BYTES;
  uint8_t* sSF = smem + SF_OFF;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + BAR_OFF);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  if (args.err && *reinterpret_cast<volatile int*>(args.err) != 0) return;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_n = (args.N + BN - 1) / BN;
  const int tiles_m = (args.M + BM - 1) / BM;
  const int tiles_per_problem = tiles_m * tiles_n;
  const int total_tiles = MODE == GROUPED_K ? tiles_per_problem * args.num_experts : tiles_per_problem;
  const int dense_nkt = (args.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(tmem_full, 1);
    mbar_init(tmem_empty, 8);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto decode = [&](int tile) {
    Tile t;
    int local = tile;
    t.e = 0;
    if (MODE == GROUPED_K) {
      t.e = tile / tiles_per_problem;
      local = tile - t.e * tiles_per_problem;
    }
    const int band = 8;                       // bands of 8 row tiles share B tiles in L2
    const int band_tiles = band * tiles_n;
    const int b = local / band_tiles;
    const int r = local - b * band_tiles;
    const int rows_in_band = min(band, tiles_m - b * band);
    t.mt = b * band + r % rows_in_band;
    t.nt = r / rows_in_band;
    t.kt0 = 0;
    t.nkt = dense_nkt;
    t.b_row0 = t.nt * BN;
    t.b_kt0 = 0;
    if (MODE == GROUPED_ROWS) {
      t.e = args.tile_expert[t.mt];
      if (t.e < 0) t.nkt = 0;
      else {
        t.b_row0 += t.e * args.b_row_e;
        t.b_kt0 = t.e * (args.b_k_e / BK);
      }
    }
    if (MODE == GROUPED_K) {
      const int s0 = args.seg_offsets[t.e], s1 = args.seg_offsets[t.e + 1];
      t.kt0 = s0 / BK;
      t.nkt = (s1 - s0) / BK;
      t.b_kt0 = t.kt0;
    }
    t.two = t.nt * BN + 128 < args.N;
    return t;
  };

  if (warp == 0) {
    if (elect_one()) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const Tile t = decode(tile);
        const uint8_t* sfa = args.sfa + ((size_t)t.mt * args.sfa_nkt + t.kt0) * 512;
        const uint8_t* sfb0 = args.sfb + ((size_t)(t.b_row0 / 128) * args.sfb_nkt + t.b_kt0) * 512;
        const uint8_t* sfb1 = sfb0 + (size_t)args.sfb_nkt * 512;
        for (int kt = 0; kt < t.nkt; ++kt) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, args.err, ERR_WAIT_EMPTY);
          if (!ok) break;
          mbar_expect_tx(&full_bar[stage], A_BYTES + B_BYTES + SFA_BYTES + (t.two ? 1024 : 512));
          tma_load_2d(sA + stage * A_BYTES, &tmA, &full_bar[stage], (t.kt0 + kt) * BK, t.mt * BM);
          tma_load_2d(sB + stage * B_BYTES, &tmB, &full_bar[stage], (t.b_kt0 + kt) * BK, t.b_row0);
          uint8_t* sf = sSF + stage * (SFA_BYTES + SFB_BYTES);
          bulk_load(sf, sfa + (size_t)kt * 512, 512, &full_bar[stage]);
          bulk_load(sf + 512, sfb0 + (size_t)kt * 512, 512, &full_bar[stage]);
          if (t.two) bulk_load(sf + 1024, sfb1 + (size_t)kt * 512, 512, &full_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc0 = idesc_mxf8(BM, BN);
      uint32_t stage = 0, phase = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const Tile t = decode(tile);
        if (t.nkt == 0) continue;
        const bool two = t.two;
        ok = mbar_wait(tmem_empty, acc_phase ^ 1, abort_flag, args.err, ERR_WAIT_TMEM_EMPTY);
        if (!ok) break;
        tc_fence_after();
        for (int kt = 0; kt < t.nkt; ++kt) {
          ok = mbar_wait(&full_bar[stage], phase, abort_flag, args.err, ERR_WAIT_FULL);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(sA + stage * A_BYTES);
          const uint32_t sb = smem_u32(sB + stage * B_BYTES);
          const uint32_t sf = smem_u32(sSF + stage * (SFA_BYTES + SFB_BYTES));
          tmem_cp_sf(tmem_base + SFA_COL, sf_desc(sf));
          tmem_cp_sf(tmem_base + SFB_COL, sf_desc(sf + 512));
          if (two) tmem_cp_sf(tmem_base + SFB_COL + 4, sf_desc(sf + 1024));
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint32_t idesc = idesc0 | (uint32_t(k) << 29) | (uint32_t(k) << 4);
            umma_mxf8(tmem_base, umma_desc_sw128(sa + k * 32, 16, 1024), umma_desc_sw128(sb + k * 32, 16, 1024), idesc,
                      tmem_base + SFA_COL, tmem_base + SFB_COL, (kt | k) != 0);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(tmem_full);
        acc_phase ^= 1;
      }
    }
  } else {
    const int q = warp & 3;                    // TMEM lane quarter this warp may read
    const int half = (warp - 2) >> 2;          // which 128 of the 256 accumulator columns
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      const Tile t = decode(tile);
      const int mt = t.mt, nt = t.nt;
      if (t.nkt == 0) {
        if (MODE == GROUPED_K && !ACC) {           // an expert without tokens: its gradient block is zero
          const int row = mt * BM + q * 32 + lane;
          const int col0 = nt * BN + half * 128;
          if (row < args.M) {
            OutT* crow = C + (long long)t.e * args.M * args.ldc + (long long)row * args.ldc;
            for (int c = col0; c < min(col0 + 128, args.N); ++c) crow[c] = OutT(0.f);
          }
        }
        continue;
      }
      ok = mbar_wait(tmem_full, acc_phase, abort_flag, args.err, ERR_WAIT_TMEM_FULL);
      if (!ok) break;
      acc_phase ^= 1;
      tc_fence_after();
      uint32_t r[4][32];
      const uint32_t t_base = tmem_base + half * 128 + (uint32_t(q * 32) << 16);
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32(t_base + c * 32, r[c]);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty);   // the accumulator is in registers: the next tile may start

      const int row = mt * BM + q * 32 + lane;
      const int col0 = nt * BN + half * 128;
      if (row >= args.M || col0 >= args.N) continue;
      OutT* crow = C + (MODE == GROUPED_K ? (long long)t.e * args.M * args.ldc : 0ll) + (long long)row * args.ldc + col0;
      if (col0 + 128 <= args.N && (args.ldc % 8) == 0) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          if constexpr (sizeof(OutT) == 2) {
            uint4* dst = reinterpret_cast<uint4*>(crow + c * 32);
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              float f[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[c][v * 8 + j]);
              if (ACC) {
                const uint4 old = dst[v];
                const __nv_bfloat162* ob = reinterpret_cast<const __nv_bfloat162*>(&old);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float2 t = __bfloat1622float2(ob[j]);
                  f[2 * j] += t.x; f[2 * j + 1] += t.y;
                }
              }
              uint4 o;
              o.x = pack_bf16(f[0], f[1]);
              o.y = pack_bf16(f[2], f[3]);
              o.z = pack_bf16(f[4], f[5]);
              o.w = pack_bf16(f[6], f[7]);
              dst[v] = o;
            }
          } else {
            float4* dst = reinterpret_cast<float4*>(crow + c * 32);
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              float4 o = make_float4(__uint_as_float(r[c][v * 4 + 0]), __uint_as_float(r[c][v * 4 + 1]),
                                     __uint_as_float(r[c][v * 4 + 2]), __uint_as_float(r[c][v * 4 + 3]));
              if (ACC) {
                const float4 old = dst[v];
                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
              }
              dst[v] = o;
            }
          }
        }
      } else {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (col0 + c * 32 + j < args.N) {
              float v = __uint_as_float(r[c][j]);
              if (ACC) v += float(crow[c * 32 + j]);
              crow[c * 32 + j] = OutT(v);
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);      // let copies still in flight land before the CTA goes away
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

static int make_tmap_u8(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld};
  cuuint32_t box[2] = {BK, box_rows};
  cuuint32_t es[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : int(r);
}

template <typename OutT, bool ACC, int MODE = DENSE>
static int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, void* C, const Args& args, cudaStream_t s) {
  auto kern = mxfp8_gemm_kernel<OutT, ACC, MODE>;
  static PerDevice attr_set;
  if (attr_set.first()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL) != cudaSuccess) return -2;
    attr_set.done();
  }
  const int tiles = ((args.M + BM - 1) / BM) * ((args.N + BN - 1) / BN) * (MODE == GROUPED_K ? args.num_experts : 1);
  const int grid = tiles < sm_count() ? tiles : sm_count();
  if (grid <= 0) return 0;
  kern<<<grid, THREADS, SMEM_TOTAL, s>>>(tmA, tmB, reinterpret_cast<OutT*>(C), args);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace mxg
}  // namespace cm

// A [M,K] / B [N,K] E4M3 bytes (row strides lda / ldb bytes, multiples of 16); sfa / sfb swizzled scale tiles of
// ceil(rows/128) x ceil(K/128) x 512 bytes; C [M,N] bf16 (out_fp32 = 0) or fp32, `accumulate` adds to C.
extern "C" int cm_mxfp8_gemm(const void* A, const void* sfa, const void* B, const void* sfb, void* C, int M, int N, int K, long long lda,
                             long long ldb, long long ldc, int out_fp32, int accumulate, int* err, cudaStream_t s) {
  using namespace cm;
  using namespace cm::mxg;
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K % 32) || (lda % 16) || (ldb % 16)) return -10;
  if ((reinterpret_cast<uintptr_t>(sfa) | reinterpret_cast<uintptr_t>(sfb) | reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & 15)
    return -11;
  CUtensorMap tmA, tmB;
  if (int rc = make_tmap_u8(&tmA, A, M, K, lda, BM)) return 100 + rc;
  if (int rc = make_tmap_u8(&tmB, B, N, K, ldb, BN)) return 100 + rc;
  const int nkt = (K + BK - 1) / BK;
  Args args{M, N, K, ldc, (const uint8_t*)sfa, (const uint8_t*)sfb, err, nkt, nkt, nullptr, nullptr, 1, 0, 0};
  if (!out_fp32) return accumulate ? launch<__nv_bfloat16, true>(tmA, tmB, C, args, s) : launch<__nv_bfloat16, false>(tmA, tmB, C, args, s);
  return accumulate ? launch<float, true>(tmA, tmB, C, args, s) : launch<float, false>(tmA, tmB, C, args, s);
}

// Expert products on the 128-row-aligned, expert-sorted token layout.  A [rows, K] E4M3 with scales sfa; tile_expert[rows/128].
//   b_kmode = 0 (forward):  B is the stacked weight [E * N, K]            -> C[r, :N] = A[r] . W[e(r)]^T
//   b_kmode = 1 (dgrad):    B is the stacked transposed weight [N, E * K] -> C[r, :N] = A[r] . Wt[:, e(r) K : (e(r)+1) K]^T
// N % 128 == 0 (forward) / K % 128 == 0 (dgrad) keep the scale tiles of different experts apart.
extern "C" int cm_mxfp8_grouped_rows(const void* A, const void* sfa, const void* B, const void* sfb, void* C, int rows, int N, int K,
                                     int num_experts, int b_kmode, const int* tile_expert, int* err, cudaStream_t s) {
  using namespace cm;
  using namespace cm::mxg;
  if (rows <= 0 || N <= 0) return 0;
  if ((rows % 128) || (K % 32) || (K % 16) || (b_kmode ? (K % 128) : (N % 128))) return -10;
  CUtensorMap tmA, tmB;
  if (int rc = make_tmap_u8(&tmA, A, rows, K, K, BM)) return 100 + rc;
  const long long b_rows = b_kmode ? N : (long long)num_experts * N;
  const long long b_cols = b_kmode ? (long long)num_experts * K : K;
  if (int rc = make_tmap_u8(&tmB, B, b_rows, b_cols, b_cols, BN)) return 100 + rc;
  Args args{rows, N, K, N, (const uint8_t*)sfa, (const uint8_t*)sfb, err, (K + BK - 1) / BK, (int)((b_cols + BK - 1) / BK),
            tile_expert, nullptr, num_experts, b_kmode ? 0 : N, b_kmode ? K : 0};
  return launch<__nv_bfloat16, false, GROUPED_ROWS>(tmA, tmB, C, args, s);
}

// Expert weight gradients: C[e] [M, N] (+)= At[:, seg_e] . Bt[:, seg_e]^T with At [M, R], Bt [N, R] the token-transposed
// E4M3 operands (R = allocated rows, a multiple of 128) and seg_offsets[E + 1] the experts' row ranges.
extern "C" int cm_mxfp8_grouped_k(const void* At, const void* sfa, const void* Bt, const void* sfb, void* C, int R, int M, int N,
                                  int num_experts, const int* seg_offsets, int out_fp32, int accumulate, int* err, cudaStream_t s) {
  using namespace cm;
  using namespace cm::mxg;
  if (M <= 0 || N <= 0 || num_experts <= 0) return 0;
  if (R <= 0 || (R % 128)) return -10;
  CUtensorMap tmA, tmB;
  if (int rc = make_tmap_u8(&tmA, At, M, R, R, BM)) return 100 + rc;
  if (int rc = make_tmap_u8(&tmB, Bt, N, R, R, BN)) return 100 + rc;
  Args args{M, N, R, N, (const uint8_t*)sfa, (const uint8_t*)sfb, err, R / BK, R / BK, nullptr, seg_offsets, num_experts, 0, 0};
  if (!out_fp32)
    return accumulate ? launch<__nv_bfloat16, true, GROUPED_K>(tmA, tmB, C, args, s) : launch<__nv_bfloat16, false, GROUPED_K>(tmA, tmB, C, args, s);
  return accumulate ? launch<float, true, GROUPED_K>(tmA, tmB, C, args, s) : launch<float, false, GROUPED_K>(tmA, tmB, C, args, s);
}
