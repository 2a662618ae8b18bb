// bf16 GEMM family on 5th-generation tensor cores: TMA -> shared memory -> tcgen05.mma with the
// accumulator in TMEM -> tcgen05.ld epilogue.  Persistent, warp-specialised:
//   warp 0      TMA producer (one elected lane)
//   warp 1      TMEM owner + MMA issuer (one elected lane)
//   warps 2..5  epilogue: each reads its 32-lane TMEM quadrant and stores to global memory
// Two 128 x BN fp32 accumulators live in TMEM (2*BN columns) so the epilogue of tile i overlaps
// the main loop of tile i+1.
//
// Operand layouts ("K-major" = reduction index contiguous in memory, "MN-major" = the M or N
// index contiguous) are template parameters, so forward (x W^T), dgrad (dy W) and wgrad
// (dy^T x) all run without a transpose copy:
//   linear fwd   C[M,N]  = A[M,K]  K-major  x  B[N,K] K-major
//   linear dgrad C[M,K'] = A[M,N]  K-major  x  B[N,K'] MN-major
//   linear wgrad C[N,K'] = A[M,N]  MN-major x  B[M,K'] MN-major       (reduction over M)
// Modes:
//   DENSE         one problem
//   GROUPED_ROWS  rows of A/C are grouped by expert in 128-row aligned segments; B (and only B)
//                 is a stack [E, ., .]; tile_expert[m_tile] selects the slice (-1 = unused tile)
//   GROUPED_K     per-expert reduction ranges over the rows of A and B (both MN-major); C is a
//                 stack [E, M, N]  (expert weight gradients)
// This replaces the reference's CUTLASS dense GEMM extension and its scalar grouped kernels
// (cppmega/megatron/cuda_ext/cutlass_mxfp8_gemm.cu:56-360, cuda_ext/grouped_mxfp8_gemm.cu:61-234),
// which have no sm_100 path.
#include "common.cuh"

namespace cm {

constexpr int BM = 128;
constexpr int BK = 64;           // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 192;

// PEER_A: the rows of A live in the symmetric buffers of `n_peers` GPUs (sequence-parallel all-gather fused into the
//         operand loads: row block m0 belongs to segment m0 / rows_per_seg = (batch, peer));
// PEER_C: every output tile is stored into the staging slot `my_slot` of the GPU that owns its rows (the scatter half
//         of a reduce-scatter fused into the epilogue; the owner sums the slots afterwards).
// PEER_KA / PEER_KB: weight gradient of a sequence-parallel linear, C[M,N] (+)= A^T B over the tokens of all ranks; the
//         MN-major operand A (or B) is the gathered one: its reduction rows [k0, k0 + 64) live in the symmetric buffer
//         of the peer that owns token segment k0 / rows_per_seg, the other operand is local.
enum GemmMode : int { DENSE = 0, GROUPED_ROWS = 1, GROUPED_K = 2, PEER_A = 3, PEER_C = 4, PEER_KA = 5, PEER_KB = 6 };
constexpr int MAX_TP_PEERS = 8;
struct PeerMaps {
  CUtensorMap m[MAX_TP_PEERS];
};
struct NoPeerMaps {
  char unused;
};
template <int MODE>
struct PeerParam {
  using type = NoPeerMaps;
};
template <>
struct PeerParam<PEER_A> {
  using type = PeerMaps;
};
template <>
struct PeerParam<PEER_KA> {
  using type = PeerMaps;
};
template <>
struct PeerParam<PEER_KB> {
  using type = PeerMaps;
};

struct GemmArgs {
  int M, N, K;             // DENSE: problem; GROUPED_ROWS: M = allocated rows, N,K per expert;
                           // GROUPED_K: M,N = per-expert output, K unused
  long long ldc;           // elements between rows of C
  int num_experts;
  const int* tile_expert;  // GROUPED_ROWS: [M/128]
  const int* seg_offsets;  // GROUPED_K: [E+1], multiples of BK
  int* err;
  // PEER_A / PEER_C
  int rows_per_seg;        // rows of one (batch, peer) segment; a multiple of BM
  int n_peers;
  int my_slot;             // PEER_C: staging slot this rank writes on every peer
  long long local_rows;    // PEER_C: rows of one staging slot (= batch * rows_per_seg)
  void* c_peers[MAX_TP_PEERS];   // PEER_C: staging buffers [n_peers slots, local_rows, N]
};

template <int BN>
struct SmemLayout {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int TILE_BYTES = STAGES * STAGE_BYTES;
  static constexpr int BAR_BYTES = 256;
  static constexpr int TOTAL = TILE_BYTES + BAR_BYTES + 1024;   // + slack for 1024-byte alignment
};

template <int BN, bool A_MN, bool B_MN, typename OutT, bool ACC, int MODE>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, OutT* __restrict__ C,
                 const GemmArgs args, const __grid_constant__ typename PeerParam<MODE>::type peer_maps) {
  using L = SmemLayout<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::TILE_BYTES);
  uint64_t* empty_bar = full_bar + L::STAGES;
  uint64_t* tmem_full = empty_bar + L::STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  if (args.err && *reinterpret_cast<volatile int*>(args.err) != 0) return;   // an earlier kernel gave up: drain
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int tiles_n = (args.N + BN - 1) / BN;
  const int tiles_m = (args.M + BM - 1) / BM;
  const int tiles_per_problem = tiles_m * tiles_n;
  const int total_tiles = (MODE == GROUPED_K) ? tiles_per_problem * args.num_experts : tiles_per_problem;
  const int dense_kb = (args.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < L::STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 4);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // tile -> (expert, m0, n0, first k block, number of k blocks); identical in every role
  auto decode = [&](int tile, int& e, int& m0, int& n0, int& kb0, int& nkb) {
    int t = tile;
    e = 0;
    if (MODE == GROUPED_K) {
      e = tile / tiles_per_problem;
      t = tile - e * tiles_per_problem;
    }
    // rasterise in bands of 8 m-tiles so concurrently running CTAs share B tiles in L2
    const int band = 8;
    const int band_tiles = band * tiles_n;
    const int b = t / band_tiles;
    const int r = t - b * band_tiles;
    const int rows_in_band = min(band, tiles_m - b * band);
    const int mt = b * band + r % rows_in_band;
    const int nt = r / rows_in_band;
    m0 = mt * BM;
    n0 = nt * BN;
    kb0 = 0;
    nkb = dense_kb;
    if (MODE == GROUPED_ROWS) {
      e = args.tile_expert[mt];
      if (e < 0) nkb = 0;
    }
    if (MODE == GROUPED_K) {
      const int s0 = args.seg_offsets[e], s1 = args.seg_offsets[e + 1];
      kb0 = s0 / BK;
      nkb = (s1 - s0) / BK;
    }
  };

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (elect_one()) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        int e, m0, n0, kb0, nkb;
        decode(tile, e, m0, n0, kb0, nkb);
        for (int kb = 0; kb < nkb; ++kb) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, args.err, ERR_WAIT_EMPTY);
          if (!ok) break;
          uint8_t* sa = smem + stage * L::STAGE_BYTES;
          uint8_t* sb = sa + L::A_BYTES;
          mbar_expect_tx(&full_bar[stage], L::STAGE_BYTES);
          const int k0 = (kb0 + kb) * BK;
          [[maybe_unused]] int peer_k = 0, peer_id = 0;
          if constexpr (MODE == PEER_KA || MODE == PEER_KB) {
            const int seg = k0 / args.rows_per_seg;              // a 64-row k block never straddles segments
            peer_id = seg % args.n_peers;
            peer_k = (seg / args.n_peers) * args.rows_per_seg + (k0 - seg * args.rows_per_seg);
          }
          if constexpr (MODE == PEER_KA) {
            static_assert(MODE != PEER_KA || A_MN, "the gathered operand of a weight gradient is MN-major");
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_2d(sa + c * (BK * 128), &peer_maps.m[peer_id], &full_bar[stage], m0 + c * 64, peer_k);
          } else if constexpr (MODE == PEER_A) {
            // plain (single-CTA) tiled load from the peer that holds this row segment
            const int seg = m0 / args.rows_per_seg;
            const int src_row = (seg / args.n_peers) * args.rows_per_seg + (m0 - seg * args.rows_per_seg);
            tma_load_2d(sa, &peer_maps.m[seg % args.n_peers], &full_bar[stage], k0, src_row);
          } else if (!A_MN) {
            tma_load_2d(sa, &tmA, &full_bar[stage], k0, m0);                       // box [128 rows, 64 k]
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)                                        // boxes [64 k, 64 m]
              tma_load_2d(sa + c * (BK * 128), &tmA, &full_bar[stage], m0 + c * 64, k0);
          }
          if constexpr (MODE == PEER_KB) {
            static_assert(MODE != PEER_KB || B_MN, "the gathered operand of a weight gradient is MN-major");
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sb + c * (BK * 128), &peer_maps.m[peer_id], &full_bar[stage], n0 + c * 64, peer_k);
          } else if (!B_MN) {
            if (MODE == GROUPED_ROWS) tma_load_3d(sb, &tmB, &full_bar[stage], k0, n0, e);
            else tma_load_2d(sb, &tmB, &full_bar[stage], k0, n0);                    // box [BN rows, 64 k]
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) {                                      // boxes [64 k, 64 n]
              if (MODE == GROUPED_ROWS) tma_load_3d(sb + c * (BK * 128), &tmB, &full_bar[stage], n0 + c * 64, k0, e);
              else tma_load_2d(sb + c * (BK * 128), &tmB, &full_bar[stage], n0 + c * 64, k0);
            }
          }
          if (++stage == L::STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, A_MN, B_MN);
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        int e, m0, n0, kb0, nkb;
        decode(tile, e, m0, n0, kb0, nkb);
        if (nkb == 0) continue;
        ok = mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag, args.err, ERR_WAIT_TMEM_EMPTY);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < nkb; ++kb) {
          ok = mbar_wait(&full_bar[stage], phase, abort_flag, args.err, ERR_WAIT_FULL);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * L::STAGE_BYTES);
          const uint32_t sb = sa + L::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t ad = A_MN ? umma_desc_sw128(sa + k * (UMMA_K * 128), BK * 128, 1024)
                                     : umma_desc_sw128(sa + k * (UMMA_K * 2), 16, 1024);
            const uint64_t bd = B_MN ? umma_desc_sw128(sb + k * (UMMA_K * 128), BK * 128, 1024)
                                     : umma_desc_sw128(sb + k * (UMMA_K * 2), 16, 1024);
            umma_f16(d_tmem, ad, bd, idesc, (kb | k) != 0);
          }
          umma_commit(&empty_bar[stage]);          // stage reusable once these MMAs have read it
          if (++stage == L::STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tmem_full[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    const int q = warp & 3;                       // TMEM lane quadrant this warp may read
    uint32_t acc = 0, acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      int e, m0, n0, kb0, nkb;
      decode(tile, e, m0, n0, kb0, nkb);
      const int row = m0 + q * 32 + lane;
      const bool row_ok = row < args.M;
      OutT* crow = C + (MODE == GROUPED_K ? (long long)e * args.M * args.ldc : 0ll) + (long long)row * args.ldc;
      if constexpr (MODE == PEER_C) {
        const int seg = m0 / args.rows_per_seg;
        const long long dst_row = (long long)args.my_slot * args.local_rows + (long long)(seg / args.n_peers) * args.rows_per_seg +
                                  (row - seg * args.rows_per_seg);
        crow = reinterpret_cast<OutT*>(args.c_peers[seg % args.n_peers]) + dst_row * args.ldc;
      }
      if (nkb == 0) {
        if (MODE == GROUPED_K && !ACC && row_ok) {
          for (int c = n0; c < min(n0 + BN, args.N); ++c) crow[c] = OutT(0.f);
        }
        continue;
      }
      ok = mbar_wait(&tmem_full[acc], acc_phase, abort_flag, args.err, ERR_WAIT_TMEM_FULL);
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_base = tmem_base + acc * BN + (uint32_t(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_base + c * 32, r);
        tmem_ld_wait();
        const int col = n0 + c * 32;
        if (!row_ok || col >= args.N) continue;
        if (col + 32 <= args.N && (args.ldc % 8) == 0) {
          if constexpr (sizeof(OutT) == 2) {
            uint4* dst = reinterpret_cast<uint4*>(crow + col);
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 o;
              if (ACC) {
                uint4 old = dst[v];
                const __nv_bfloat162* ob = reinterpret_cast<const __nv_bfloat162*>(&old);
                float2 f0 = __bfloat1622float2(ob[0]), f1 = __bfloat1622float2(ob[1]);
                float2 f2 = __bfloat1622float2(ob[2]), f3 = __bfloat1622float2(ob[3]);
                o.x = pack_bf16(__uint_as_float(r[v * 8 + 0]) + f0.x, __uint_as_float(r[v * 8 + 1]) + f0.y);
                o.y = pack_bf16(__uint_as_float(r[v * 8 + 2]) + f1.x, __uint_as_float(r[v * 8 + 3]) + f1.y);
                o.z = pack_bf16(__uint_as_float(r[v * 8 + 4]) + f2.x, __uint_as_float(r[v * 8 + 5]) + f2.y);
                o.w = pack_bf16(__uint_as_float(r[v * 8 + 6]) + f3.x, __uint_as_float(r[v * 8 + 7]) + f3.y);
              } else {
                o.x = pack_bf16(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]));
                o.y = pack_bf16(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
                o.z = pack_bf16(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
                o.w = pack_bf16(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
              }
              dst[v] = o;
            }
          } else {
            float4* dst = reinterpret_cast<float4*>(crow + col);
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              float4 o = make_float4(__uint_as_float(r[v * 4 + 0]), __uint_as_float(r[v * 4 + 1]),
                                     __uint_as_float(r[v * 4 + 2]), __uint_as_float(r[v * 4 + 3]));
              if (ACC) {
                float4 old = dst[v];
                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
              }
              dst[v] = o;
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (col + j < args.N) {
              float v = __uint_as_float(r[j]);
              if (ACC) v += float(crow[col + j]);
              crow[col + j] = OutT(v);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }

  // ------------------------------ teardown ------------------------------
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // let any TMA copy still in flight land before this CTA's shared memory is released
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

// ------------------------------ host side ------------------------------

static EncodeTiledFn g_encode = nullptr;
EncodeTiledFn get_encode_tiled() {
  // The encode call is a driver entry point and wants the device's primary context current on the calling thread.
  // A thread that has made no runtime call yet (an autograd worker running its first backward) has none bound:
  // one no-op runtime call binds it.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    cudaFree(nullptr);
    ctx_bound = true;
  }
  if (g_encode) return g_encode;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess)
    return nullptr;
  g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  return g_encode;
}

int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                      uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t es[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, es,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : int(r);
}

int make_tmap_3d_bf16(CUtensorMap* out, const void* base, uint64_t batch, uint64_t rows, uint64_t cols, uint64_t ld,
                      uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return -1;
  cuuint64_t dims[3] = {cols, rows, batch};
  cuuint64_t strides[2] = {ld * 2, rows * ld * 2};
  cuuint32_t box[3] = {box_cols, box_rows, 1};
  cuuint32_t es[3] = {1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, es,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : int(r);
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

template <int BN, bool A_MN, bool B_MN, typename OutT, bool ACC, int MODE>
static int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, OutT* C, const GemmArgs& args, int total_tiles,
                  cudaStream_t stream) {
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN, OutT, ACC, MODE>;
  static PerDevice configured;
  if (configured.first()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemLayout<BN>::TOTAL) != cudaSuccess)
      return -2;
    configured.done();
  }
  int grid = total_tiles < sm_count() ? total_tiles : sm_count();
  if (grid <= 0) return 0;
  kern<<<grid, GEMM_THREADS, SmemLayout<BN>::TOTAL, stream>>>(tmA, tmB, C, args, NoPeerMaps{});
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

template <int BN, bool B_MN>
static int launch_peer_a(const PeerMaps& pm, const CUtensorMap& tmB, __nv_bfloat16* C, const GemmArgs& args, int total_tiles,
                         cudaStream_t stream) {
  auto kern = gemm_bf16_kernel<BN, false, B_MN, __nv_bfloat16, false, PEER_A>;
  static PerDevice configured;
  if (configured.first()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemLayout<BN>::TOTAL) != cudaSuccess)
      return -2;
    configured.done();
  }
  int grid = total_tiles < sm_count() ? total_tiles : sm_count();
  if (grid <= 0) return 0;
  kern<<<grid, GEMM_THREADS, SmemLayout<BN>::TOTAL, stream>>>(pm.m[0], tmB, C, args, pm);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

template <int BN, typename OutT, bool ACC, int MODE>
static int dispatch_layout(bool a_mn, bool b_mn, const CUtensorMap& tmA, const CUtensorMap& tmB, OutT* C,
                           const GemmArgs& args, int tiles, cudaStream_t s) {
  if (!a_mn && !b_mn) return launch<BN, false, false, OutT, ACC, MODE>(tmA, tmB, C, args, tiles, s);
  if (!a_mn && b_mn) return launch<BN, false, true, OutT, ACC, MODE>(tmA, tmB, C, args, tiles, s);
  if (a_mn && b_mn) return launch<BN, true, true, OutT, ACC, MODE>(tmA, tmB, C, args, tiles, s);
  return launch<BN, true, false, OutT, ACC, MODE>(tmA, tmB, C, args, tiles, s);
}

}  // namespace cm

using namespace cm;

// C[M,N] (+)= op(A) op(B).  a_mn: A is stored [K,M] (M contiguous) instead of [M,K]; b_mn: B is
// stored [K,N] (N contiguous) instead of [N,K].  lda/ldb/ldc are row pitches in elements.
// out_fp32: C is float (else bf16); accumulate: C += result.  `err` is a device int (may be null).
extern "C" int cm_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                            long long ldc, int a_mn, int b_mn, int out_fp32, int accumulate, int* err,
                            cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return -10;   // TMA needs 16-byte aligned bases and row pitches
  CUtensorMap tmA, tmB;
  int rc;
  rc = a_mn ? make_tmap_2d_bf16(&tmA, A, K, M, lda, 64) : make_tmap_2d_bf16(&tmA, A, M, K, lda, BM);
  if (rc) return rc;
  constexpr int BN = 256;
  rc = b_mn ? make_tmap_2d_bf16(&tmB, B, K, N, ldb, 64) : make_tmap_2d_bf16(&tmB, B, N, K, ldb, BN);
  if (rc) return rc;
  GemmArgs args{M, N, K, ldc, 1, nullptr, nullptr, err, 0, 0, 0, 0, {}};
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  if (out_fp32) {
    if (accumulate) return dispatch_layout<BN, float, true, DENSE>(a_mn, b_mn, tmA, tmB, (float*)C, args, tiles, stream);
    return dispatch_layout<BN, float, false, DENSE>(a_mn, b_mn, tmA, tmB, (float*)C, args, tiles, stream);
  }
  if (accumulate)
    return dispatch_layout<BN, __nv_bfloat16, true, DENSE>(a_mn, b_mn, tmA, tmB, (__nv_bfloat16*)C, args, tiles, stream);
  return dispatch_layout<BN, __nv_bfloat16, false, DENSE>(a_mn, b_mn, tmA, tmB, (__nv_bfloat16*)C, args, tiles, stream);
}

// Grouped over 128-row-aligned expert segments of A / C.
//   b_mn = 0: C[r, :N] = A[r, :K] . W[e(r)][N,K]^T          (expert forward)
//   b_mn = 1: C[r, :N] = A[r, :K] . W[e(r)][K,N]            (expert dgrad; W stored [E, K, N])
// tile_expert[rows/128] gives the expert of each 128-row tile (-1: skip).
extern "C" int cm_grouped_gemm_rows_bf16(const void* A, const void* W, void* C, int rows, int N, int K, int num_experts,
                                         int b_mn, const int* tile_expert, int* err, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (rows % BM) return -11;
  if ((K % 8) || (N % 8)) return -10;
  constexpr int BN = 256;
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d_bf16(&tmA, A, rows, K, K, BM);
  if (rc) return rc;
  rc = b_mn ? make_tmap_3d_bf16(&tmB, W, num_experts, K, N, N, 64) : make_tmap_3d_bf16(&tmB, W, num_experts, N, K, K, BN);
  if (rc) return rc;
  GemmArgs args{rows, N, K, N, num_experts, tile_expert, nullptr, err, 0, 0, 0, 0, {}};
  const int tiles = (rows / BM) * ((N + BN - 1) / BN);
  if (b_mn) return launch<BN, false, true, __nv_bfloat16, false, GROUPED_ROWS>(tmA, tmB, (__nv_bfloat16*)C, args, tiles, stream);
  return launch<BN, false, false, __nv_bfloat16, false, GROUPED_ROWS>(tmA, tmB, (__nv_bfloat16*)C, args, tiles, stream);
}

// Expert weight gradients: C[e][M,N] (+)= sum over rows r in [seg[e], seg[e+1]) of A[r, :M]^T B[r, :N].
// seg offsets are multiples of 64.  out_fp32 / accumulate as in cm_gemm_bf16.
extern "C" int cm_grouped_gemm_k_bf16(const void* A, const void* B, void* C, int rows, int M, int N, int num_experts,
                                      const int* seg_offsets, int out_fp32, int accumulate, int* err,
                                      cudaStream_t stream) {
  if (rows <= 0 || num_experts <= 0) return 0;
  if ((M % 8) || (N % 8)) return -10;
  constexpr int BN = 256;
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d_bf16(&tmA, A, rows, M, M, 64);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tmB, B, rows, N, N, 64);
  if (rc) return rc;
  GemmArgs args{M, N, 0, N, num_experts, nullptr, seg_offsets, err, 0, 0, 0, 0, {}};
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN) * num_experts;
  if (out_fp32) {
    if (accumulate) return launch<BN, true, true, float, true, GROUPED_K>(tmA, tmB, (float*)C, args, tiles, stream);
    return launch<BN, true, true, float, false, GROUPED_K>(tmA, tmB, (float*)C, args, tiles, stream);
  }
  if (accumulate) return launch<BN, true, true, __nv_bfloat16, true, GROUPED_K>(tmA, tmB, (__nv_bfloat16*)C, args, tiles, stream);
  return launch<BN, true, true, __nv_bfloat16, false, GROUPED_K>(tmA, tmB, (__nv_bfloat16*)C, args, tiles, stream);
}

// ---------------------------------------------------------------------------------------------------------
// Tensor parallelism with sequence parallelism, fused with the GEMMs (peer memory; plain single-CTA TMA loads and
// ordinary stores only).  Rows are tokens; M = batch * n_peers * rows_per_seg, and global row block
// (b, p, r) = b * n_peers * rows_per_seg + p * rows_per_seg + r belongs to peer p, local row b * rows_per_seg + r.
// ---------------------------------------------------------------------------------------------------------

// all-gather -> GEMM:  C[M, N] = gather(A)[M, K] . op(B);  a_ptrs[p] = peer p's shard [batch * rows_per_seg, K] bf16.
// Callers make sure (flag barrier) that every peer's shard is complete before the launch and is not overwritten
// until every rank's kernel has finished.
extern "C" int cm_gemm_bf16_peer_a(void* const* a_ptrs, int n_peers, int rows_per_seg, int batch, const void* B, void* C, int N,
                                   int K, long long ldb, long long ldc, int b_mn, int* err, cudaStream_t stream) {
  if (n_peers <= 0 || n_peers > MAX_TP_PEERS || batch <= 0 || rows_per_seg <= 0) return -10;
  if (rows_per_seg % BM || (K % 8) || (ldb % 8)) return -10;
  const int M = batch * n_peers * rows_per_seg;
  PeerMaps pm;
  for (int p = 0; p < n_peers; ++p) {
    if (reinterpret_cast<uintptr_t>(a_ptrs[p]) & 15) return -10;
    int rc = make_tmap_2d_bf16(&pm.m[p], a_ptrs[p], (uint64_t)batch * rows_per_seg, K, K, BM);
    if (rc) return rc;
  }
  for (int p = n_peers; p < MAX_TP_PEERS; ++p) pm.m[p] = pm.m[0];
  constexpr int BN = 256;
  CUtensorMap tmB;
  int rc = b_mn ? make_tmap_2d_bf16(&tmB, B, K, N, ldb, 64) : make_tmap_2d_bf16(&tmB, B, N, K, ldb, BN);
  if (rc) return rc;
  GemmArgs args{M, N, K, ldc, 1, nullptr, nullptr, err, rows_per_seg, n_peers, 0, 0, {}};
  const int tiles = (M / BM) * ((N + BN - 1) / BN);
  if (b_mn) return launch_peer_a<BN, true>(pm, tmB, (__nv_bfloat16*)C, args, tiles, stream);
  return launch_peer_a<BN, false>(pm, tmB, (__nv_bfloat16*)C, args, tiles, stream);
}

template <typename OutT, bool ACC, int MODE>
static int launch_peer_k(const PeerMaps& pm, const CUtensorMap& tmA, const CUtensorMap& tmB, OutT* C, const GemmArgs& args,
                         int total_tiles, cudaStream_t stream) {
  constexpr int BN = 256;
  auto kern = gemm_bf16_kernel<BN, true, true, OutT, ACC, MODE>;
  static PerDevice configured;
  if (configured.first()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemLayout<BN>::TOTAL) != cudaSuccess) return -2;
    configured.done();
  }
  int grid = total_tiles < sm_count() ? total_tiles : sm_count();
  if (grid <= 0) return 0;
  kern<<<grid, GEMM_THREADS, SmemLayout<BN>::TOTAL, stream>>>(tmA, tmB, C, args, pm);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// all-gather -> weight gradient:  C[M,N] (+)= A^T B with A [T, M] and B [T, N] (T = batch * n_peers * rows_per_seg tokens).
// peer_is_a: A is the gathered operand, peer_ptrs[p] = peer p's [batch * rows_per_seg, M] shard and `local` is B [T, N];
// otherwise B is gathered (shards [batch * rows_per_seg, N]) and `local` is A [T, M].
extern "C" int cm_gemm_bf16_peer_k(void* const* peer_ptrs, int n_peers, int rows_per_seg, int batch, int peer_is_a, const void* local,
                                   void* C, int M, int N, long long ld_local, long long ldc, int out_fp32, int accumulate, int* err,
                                   cudaStream_t stream) {
  if (n_peers <= 0 || n_peers > MAX_TP_PEERS || batch <= 0 || rows_per_seg <= 0) return -10;
  if (rows_per_seg % BK || (M % 8) || (N % 8) || (ld_local % 8) || (reinterpret_cast<uintptr_t>(local) & 15)) return -10;
  const int T = batch * n_peers * rows_per_seg;
  const int peer_w = peer_is_a ? M : N;
  PeerMaps pm;
  for (int p = 0; p < n_peers; ++p) {
    if (reinterpret_cast<uintptr_t>(peer_ptrs[p]) & 15) return -10;
    int rc = make_tmap_2d_bf16(&pm.m[p], peer_ptrs[p], (uint64_t)batch * rows_per_seg, peer_w, peer_w, 64);
    if (rc) return rc;
  }
  for (int p = n_peers; p < MAX_TP_PEERS; ++p) pm.m[p] = pm.m[0];
  CUtensorMap tmL;
  int rc = make_tmap_2d_bf16(&tmL, local, T, peer_is_a ? N : M, ld_local, 64);
  if (rc) return rc;
  GemmArgs args{M, N, T, ldc, 1, nullptr, nullptr, err, rows_per_seg, n_peers, 0, 0, {}};
  const int tiles = ((M + BM - 1) / BM) * ((N + 255) / 256);
  const CUtensorMap& tmA = peer_is_a ? pm.m[0] : tmL;
  const CUtensorMap& tmB = peer_is_a ? tmL : pm.m[0];
#define CM_PEER_K(OUT, ACC_)                                                                                         \
  (peer_is_a ? launch_peer_k<OUT, ACC_, PEER_KA>(pm, tmA, tmB, (OUT*)C, args, tiles, stream)                          \
             : launch_peer_k<OUT, ACC_, PEER_KB>(pm, tmA, tmB, (OUT*)C, args, tiles, stream))
  if (out_fp32) return accumulate ? CM_PEER_K(float, true) : CM_PEER_K(float, false);
  return accumulate ? CM_PEER_K(__nv_bfloat16, true) : CM_PEER_K(__nv_bfloat16, false);
#undef CM_PEER_K
}

// GEMM -> scatter:  partial[M, N] = A[M, K] . op(B), every tile stored into slot `my_slot` of the staging buffer of the
// peer that owns its rows; c_ptrs[p] = peer p's staging buffer [n_peers, batch * rows_per_seg, N] bf16.
extern "C" int cm_gemm_bf16_peer_c(const void* A, const void* B, void* const* c_ptrs, int n_peers, int my_slot, int rows_per_seg,
                                   int batch, int N, int K, long long lda, long long ldb, int b_mn, int* err,
                                   cudaStream_t stream) {
  if (n_peers <= 0 || n_peers > MAX_TP_PEERS || batch <= 0 || rows_per_seg <= 0 || my_slot < 0 || my_slot >= n_peers) return -10;
  if (rows_per_seg % BM || (lda % 8) || (ldb % 8) || (N % 8)) return -10;
  const int M = batch * n_peers * rows_per_seg;
  constexpr int BN = 256;
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d_bf16(&tmA, A, M, K, lda, BM);
  if (rc) return rc;
  rc = b_mn ? make_tmap_2d_bf16(&tmB, B, K, N, ldb, 64) : make_tmap_2d_bf16(&tmB, B, N, K, ldb, BN);
  if (rc) return rc;
  GemmArgs args{M, N, K, N, 1, nullptr, nullptr, err, rows_per_seg, n_peers, my_slot, (long long)batch * rows_per_seg, {}};
  for (int p = 0; p < n_peers; ++p) args.c_peers[p] = c_ptrs[p];
  const int tiles = (M / BM) * ((N + BN - 1) / BN);
  if (b_mn) return launch<BN, false, true, __nv_bfloat16, false, PEER_C>(tmA, tmB, (__nv_bfloat16*)nullptr, args, tiles, stream);
  return launch<BN, false, false, __nv_bfloat16, false, PEER_C>(tmA, tmB, (__nv_bfloat16*)nullptr, args, tiles, stream);
}
