// Expert-parallel token movement over peer-mapped memory, fused with the permutation.
//
//  push_rows     dispatch: each routed copy of a token is stored straight into its final row of the
//                owning rank's 128-row-aligned, expert-sorted GEMM input (peer stores).  There is no
//                send buffer, no all-to-all, no receive-side sort.
//  pull_combine  combine: each token reads its k expert outputs from the ranks that computed them
//                (peer loads), applies the routing weights and sums - un-permute, weighting and the
//                return all-to-all in one pass.
//  pull_rowdot   backward of the weighting: dprob[t,j] = dy[t] . y_expert[row(t,j)].
//  zero_pad_rows clears the <=127 padding rows at the end of each expert segment.
// Between push and the expert GEMMs, and between the GEMMs and the pull, ranks synchronise with
// flag words (symm.cu); the grouped tcgen05 GEMMs then run on the padded layout unchanged.
// Baseline replaced: NCCL all-to-all(v) + permute kernels (Megatron alltoall dispatcher selected by
// cppmega/recipes/megatron_args.py:99-135; 3-5 % EP overhead in docs/dsa_ep2_tilelang_sweep_2026_04_12.md:44).
#include "common.cuh"

namespace cm {

constexpr int MOE_MAX_PEERS = 16;
struct MoePeers {
  void* p[MOE_MAX_PEERS];
};

// one warp per copy
__global__ void __launch_bounds__(256) moe_push_rows_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ token_of_copy,
                                                            const int* __restrict__ dest_rank, const long long* __restrict__ dest_row,
                                                            const float* __restrict__ scale, MoePeers dst, int ncopies, int H,
                                                            int world, long long capacity_rows, int* __restrict__ err) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int nvec = H / 8;
  for (int c = blockIdx.x * wpb + (threadIdx.x >> 5); c < ncopies; c += gridDim.x * wpb) {
    const int t = token_of_copy[c];
    const int r = dest_rank[c];
    const long long row = dest_row[c];
    if (row < 0 || row >= capacity_rows || r < 0 || r >= world) {   // receiver buffer too small for this routing: drop + report
      if (lane == 0 && err) atomicCAS(err, 0, ERR_BAD_ARG);
      continue;
    }
    const uint4* s = reinterpret_cast<const uint4*>(src + (size_t)t * H);
    uint4* d = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(dst.p[r]) + row * H);
    if (scale) {
      const float sc = scale[c];
      for (int v = lane; v < nvec; v += 32) {
        uint4 x = s[v];
        __nv_bfloat162* b = reinterpret_cast<__nv_bfloat162*>(&x);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = __bfloat1622float2(b[j]);
          b[j] = __floats2bfloat162_rn(f.x * sc, f.y * sc);
        }
        d[v] = x;
      }
    } else {
      for (int v = lane; v < nvec; v += 32) d[v] = s[v];
    }
  }
}

// one warp per token
__global__ void __launch_bounds__(256) moe_pull_combine_kernel(MoePeers src, const int* __restrict__ dest_rank, const long long* __restrict__ dest_row,
                                                               const float* __restrict__ weights, __nv_bfloat16* __restrict__ out,
                                                               int T, int k, int H, int world, long long capacity_rows,
                                                               int* __restrict__ err) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int nvec = H / 8;
  for (int t = blockIdx.x * wpb + (threadIdx.x >> 5); t < T; t += gridDim.x * wpb) {
    // a copy whose row lies outside the owner's buffer was never stored (push dropped it): it contributes zero and
    // is reported; no address outside the peer mapping is ever formed
    unsigned bad = 0;
    for (int j = 0; j < k; ++j) {
      const int c = t * k + j;
      const long long row = dest_row[c];
      const int r = dest_rank[c];
      if (row < 0 || row >= capacity_rows || r < 0 || r >= world) bad |= 1u << j;
    }
    if (bad && lane == 0 && err) atomicCAS(err, 0, ERR_BAD_ARG);
    for (int v = lane; v < nvec; v += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int j = 0; j < k; ++j) {
        if (bad & (1u << j)) continue;
        const int c = t * k + j;
        const uint4 x = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(src.p[dest_rank[c]]) + dest_row[c] * H)[v];
        const float w = weights ? weights[c] : 1.f;
        const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float2 f = __bfloat1622float2(b[i]);
          acc[2 * i] += w * f.x;
          acc[2 * i + 1] += w * f.y;
        }
      }
      uint4 o;
      o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]);
      o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
      reinterpret_cast<uint4*>(out + (size_t)t * H)[v] = o;
    }
  }
}

// one warp per copy: out[c] = dy[token(c)] . y_rows[row(c)]
__global__ void __launch_bounds__(256) moe_pull_rowdot_kernel(MoePeers src, const int* __restrict__ dest_rank, const long long* __restrict__ dest_row,
                                                              const __nv_bfloat16* __restrict__ dy, float* __restrict__ out, int T, int k, int H,
                                                              int world, long long capacity_rows, int* __restrict__ err) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int nvec = H / 8;
  const int n = T * k;
  for (int c = blockIdx.x * wpb + (threadIdx.x >> 5); c < n; c += gridDim.x * wpb) {
    const int t = c / k;
    {
      const long long row = dest_row[c];
      const int r = dest_rank[c];
      if (row < 0 || row >= capacity_rows || r < 0 || r >= world) {      // dropped copy: zero, reported, never dereferenced
        if (lane == 0) {
          out[c] = 0.f;
          if (err) atomicCAS(err, 0, ERR_BAD_ARG);
        }
        continue;
      }
    }
    const uint4* a = reinterpret_cast<const uint4*>(dy + (size_t)t * H);
    const uint4* b = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(src.p[dest_rank[c]]) + dest_row[c] * H);
    float s = 0.f;
    for (int v = lane; v < nvec; v += 32) {
      const uint4 x = a[v], y = b[v];
      const __nv_bfloat162* xb = reinterpret_cast<const __nv_bfloat162*>(&x);
      const __nv_bfloat162* yb = reinterpret_cast<const __nv_bfloat162*>(&y);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float2 f = __bfloat1622float2(xb[i]), g = __bfloat1622float2(yb[i]);
        s += f.x * g.x + f.y * g.y;
      }
    }
    s = warp_sum(s);
    if (lane == 0) out[c] = s;
  }
}

// grid (num_local_experts, 128): zero row seg_start[e] + tot[e] + j when it is padding
__global__ void __launch_bounds__(256) moe_zero_pad_rows_kernel(__nv_bfloat16* __restrict__ buf, const int* __restrict__ seg_start,
                                                                const int* __restrict__ tot, int H, long long capacity_rows) {
  const int e = blockIdx.x, j = blockIdx.y;
  const int t = tot[e];
  const int padded = (t + 127) / 128 * 128;
  if (t + j >= padded) return;
  const long long row = (long long)seg_start[e] + t + j;
  if (row >= capacity_rows) return;
  uint4* d = reinterpret_cast<uint4*>(buf + row * H);
  const uint4 z = make_uint4(0, 0, 0, 0);
  for (int v = threadIdx.x; v < H / 8; v += blockDim.x) d[v] = z;
}


// ---------------------------------------------------------------------------------------------
// Routing plan.  Two launches replace a few dozen small library kernels per MoE call:
//   moe_count:  counts[e] = number of (token, j) copies routed to expert e on this rank;
//   moe_plan:   from the counts of all source ranks, the destination of every copy and this rank's receive layout.
// Row layout on the owner of expert e: experts in order, each segment padded to a multiple of `tile` rows; inside a
// segment the copies of source rank 0 come first, then rank 1, ...; a rank's copies keep their (token, j) order, so the
// plan is deterministic.  One CTA of 1024 threads per chunk of about 4096 copies: thread t ranks `per` consecutive copies.
// ---------------------------------------------------------------------------------------------
constexpr int PLAN_THREADS = 1024;
constexpr int PLAN_MAX_E = 32;          // 2 * E * 1024 16-bit counters must fit shared memory

__global__ void __launch_bounds__(256) moe_count_kernel(const long long* __restrict__ ids, long long n, long long chunk, int E,
                                                        long long* __restrict__ counts, int* __restrict__ block_counts) {
  __shared__ unsigned int h[PLAN_MAX_E];
  if (threadIdx.x < PLAN_MAX_E) h[threadIdx.x] = 0;
  __syncthreads();
  const long long c0 = blockIdx.x * chunk, c1 = min(n, c0 + chunk);       // the same partition moe_plan_kernel walks
  for (long long i = c0 + threadIdx.x; i < c1; i += blockDim.x) {
    const long long e = ids[i];
    if (e >= 0 && e < E) atomicAdd(&h[e], 1u);
  }
  __syncthreads();
  if (threadIdx.x < E) {
    block_counts[blockIdx.x * E + threadIdx.x] = (int)h[threadIdx.x];
    if (h[threadIdx.x]) atomicAdd(reinterpret_cast<unsigned long long*>(counts) + threadIdx.x, (unsigned long long)h[threadIdx.x]);
  }
}

struct PlanOut {
  long long* dest_row;        // [n]
  int* dest_rank;             // [n]
  int* token_of_copy;         // [n]
  int* seg_start_local;       // [El]
  int* tot_local;             // [El]
  int* seg_offsets;           // [El + 1]
  int* tile_expert;           // [n_tiles]
  long long* counts_global;   // [E]
};

__global__ void __launch_bounds__(PLAN_THREADS) moe_plan_kernel(const long long* __restrict__ ids, long long n, long long chunk, int k, int E, int ep,
                                                                int ep_rank, const long long* __restrict__ allc,
                                                                const int* __restrict__ block_counts, int tile, int n_tiles, PlanOut o) {
  __shared__ long long base[PLAN_MAX_E];          // first row of this rank's copies of expert e on its owner
  __shared__ long long my_end[PLAN_MAX_E];
  __shared__ unsigned int warp_tot[32];
  extern __shared__ unsigned short cnt[];         // [E][PLAN_THREADS] per-thread counts, then exclusive prefixes
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int El = E / ep;
  if (tid < E) {
    long long tot = 0, before = 0;
    for (int r = 0; r < ep; ++r) {
      const long long c = allc[(long long)r * E + tid];
      tot += c;
      if (r < ep_rank) before += c;
    }
    if (blockIdx.x == 0) o.counts_global[tid] = tot;
    for (int g = 0; g < (int)blockIdx.x; ++g) before += block_counts[g * E + tid];     // this rank's copies in earlier CTAs
    const int owner = tid / El;
    long long start = 0;                           // padded sizes of the owner's earlier experts
    for (int e2 = owner * El; e2 < tid; ++e2) {
      long long t2 = 0;
      for (int r = 0; r < ep; ++r) t2 += allc[(long long)r * E + e2];
      start += (t2 + tile - 1) / tile * tile;
    }
    base[tid] = start + before;
    if (owner == ep_rank) {
      const int le = tid - owner * El;
      const long long padded = (tot + tile - 1) / tile * tile;
      my_end[le] = start + padded;
      if (blockIdx.x == 0) {
        // a routing that needs more rows than the buffer holds is reported by the push kernel; the receive layout is
        // clipped to the buffer here so that no GEMM tile or reduction range reaches past it
        const long long cap = (long long)n_tiles * tile;
        const long long s0 = start < cap ? start : cap, s1 = start + padded < cap ? start + padded : cap;
        o.seg_start_local[le] = (int)s0;
        o.tot_local[le] = (int)(tot < s1 - s0 ? tot : s1 - s0);
        o.seg_offsets[le + 1] = (int)s1;
        if (le == 0) o.seg_offsets[0] = 0;
      }
    }
  }
  const long long b0 = blockIdx.x * chunk, b1 = min(n, b0 + chunk);            // this CTA's copies
  const long long per = (chunk + PLAN_THREADS - 1) / PLAN_THREADS;
  const long long c0 = min(b1, b0 + (long long)tid * per), c1 = min(b1, c0 + per);
  for (int e = 0; e < E; ++e) cnt[e * PLAN_THREADS + tid] = 0;
  for (long long c = c0; c < c1; ++c) {
    const long long e = ids[c];
    if (e >= 0 && e < E) cnt[(int)e * PLAN_THREADS + tid] += 1;       // same filter as moe_count_kernel
  }
  __syncthreads();
  // exclusive scan over the threads, one expert at a time
  for (int e = 0; e < E; ++e) {
    const unsigned int v = cnt[e * PLAN_THREADS + tid];
    unsigned int sc = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const unsigned int u = __shfl_up_sync(0xffffffffu, sc, off);
      if (lane >= off) sc += u;
    }
    if (lane == 31) warp_tot[warp] = sc;
    __syncthreads();
    if (warp == 0) {
      unsigned int w = warp_tot[lane], ws = w;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const unsigned int u = __shfl_up_sync(0xffffffffu, ws, off);
        if (lane >= off) ws += u;
      }
      warp_tot[lane] = ws - w;
    }
    __syncthreads();
    cnt[e * PLAN_THREADS + tid] = (unsigned short)0;       // the prefix may exceed 16 bits: keep it in a register below
    const unsigned int excl = warp_tot[warp] + sc - v;
    // stash the 32-bit prefix in two 16-bit halves of the (now free) counter slots of experts e and e + E
    cnt[e * PLAN_THREADS + tid] = (unsigned short)(excl & 0xffffu);
    cnt[(E + e) * PLAN_THREADS + tid] = (unsigned short)(excl >> 16);
    __syncthreads();
  }
  unsigned int run[PLAN_MAX_E / 4];                 // running counts of this thread, 8 bits each (per <= 255 copies)
#pragma unroll
  for (int i = 0; i < PLAN_MAX_E / 4; ++i) run[i] = 0;
  for (long long c = c0; c < c1; ++c) {
    const long long e64 = ids[c];
    if (e64 < 0 || e64 >= E) {                  // not an expert id: the copy gets no row (push and pull skip and report it)
      o.dest_row[c] = -1;
      o.dest_rank[c] = 0;
      o.token_of_copy[c] = (int)(c / k);
      continue;
    }
    const int e = (int)e64;
    const unsigned int excl = (unsigned int)cnt[e * PLAN_THREADS + tid] | ((unsigned int)cnt[(E + e) * PLAN_THREADS + tid] << 16);
    const unsigned int r = (run[e >> 2] >> ((e & 3) * 8)) & 0xffu;
    run[e >> 2] += 1u << ((e & 3) * 8);
    o.dest_row[c] = base[e] + excl + r;
    o.dest_rank[c] = e / El;
    o.token_of_copy[c] = (int)(c / k);
  }
  __syncthreads();
  if (blockIdx.x != 0) return;
  for (int t = tid; t < n_tiles; t += PLAN_THREADS) {
    const long long row = (long long)t * tile;
    int te = 0;
    while (te < El && my_end[te] <= row) ++te;
    o.tile_expert[t] = te < El ? te : -1;
  }
}

}  // namespace cm

using namespace cm;

// Blocks (of 256 threads) per SM that one row-transport launch may occupy.  8 fills every thread slot of the SM: fastest
// alone, but a GEMM CTA launched on another stream then cannot become resident until the transfer drains.  The pipelined
// MoE path lowers it so that transfers and expert GEMMs really share the SMs.
static int g_transport_blocks_per_sm = 8;

extern "C" int cm_moe_set_transport_blocks_per_sm(int n) {
  const int old = g_transport_blocks_per_sm;
  if (n >= 1 && n <= 8) g_transport_blocks_per_sm = n;
  return old;
}

static int grid_for(long long warps_needed) {
  long long blocks = (warps_needed + 7) / 8;
  long long cap = (long long)sm_count() * g_transport_blocks_per_sm;
  return (int)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

extern "C" int cm_moe_push_rows(const void* src, const int* token_of_copy, const int* dest_rank, const long long* dest_row,
                                const float* scale, void* const* dst_ptrs, int world, int ncopies, int H,
                                long long capacity_rows, int* err, cudaStream_t s) {
  if (ncopies <= 0) return 0;
  if (H % 8 || world > MOE_MAX_PEERS) return -10;
  MoePeers p;
  for (int i = 0; i < world; ++i) p.p[i] = dst_ptrs[i];
  moe_push_rows_kernel<<<grid_for(ncopies), 256, 0, s>>>((const __nv_bfloat16*)src, token_of_copy, dest_rank, dest_row, scale, p, ncopies, H, world, capacity_rows, err);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int cm_moe_pull_combine(void* const* src_ptrs, int world, const int* dest_rank, const long long* dest_row,
                                   const float* weights, void* out, int T, int k, int H, long long capacity_rows, int* err,
                                   cudaStream_t s) {
  if (T <= 0) return 0;
  if (H % 8 || world > MOE_MAX_PEERS) return -10;
  MoePeers p;
  for (int i = 0; i < world; ++i) p.p[i] = src_ptrs[i];
  moe_pull_combine_kernel<<<grid_for(T), 256, 0, s>>>(p, dest_rank, dest_row, weights, (__nv_bfloat16*)out, T, k, H, world, capacity_rows, err);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int cm_moe_pull_rowdot(void* const* src_ptrs, int world, const int* dest_rank, const long long* dest_row,
                                  const void* dy, float* out, int T, int k, int H, long long capacity_rows, int* err, cudaStream_t s) {
  if (T <= 0) return 0;
  if (H % 8 || world > MOE_MAX_PEERS) return -10;
  MoePeers p;
  for (int i = 0; i < world; ++i) p.p[i] = src_ptrs[i];
  moe_pull_rowdot_kernel<<<grid_for((long long)T * k), 256, 0, s>>>(p, dest_rank, dest_row, (const __nv_bfloat16*)dy, out, T, k, H, world, capacity_rows, err);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int cm_moe_zero_pad_rows(void* buf, const int* seg_start, const int* tot, int num_local_experts, int H,
                                    long long capacity_rows, cudaStream_t s) {
  if (num_local_experts <= 0) return 0;
  if (H % 8) return -10;
  dim3 grid(num_local_experts, 128);
  moe_zero_pad_rows_kernel<<<grid, 256, 0, s>>>((__nv_bfloat16*)buf, seg_start, tot, H, capacity_rows);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// Both kernels walk the copies in the same contiguous chunks, one CTA per chunk.
static int plan_blocks(long long n) {
  long long g = (n + 4095) / 4096;
  return (int)(g < 1 ? 1 : (g > 64 ? 64 : g));
}
static long long plan_chunk(long long n) { return (n + plan_blocks(n) - 1) / plan_blocks(n); }

// counts [E] int64 (zeroed by the caller) += histogram of ids [n] int64; block_counts [64, E] int32 receives the per-chunk parts
extern "C" int cm_moe_count(const long long* ids, long long n, int E, long long* counts, int* block_counts, cudaStream_t s) {
  if (n <= 0) return 0;
  if (E > cm::PLAN_MAX_E) return -10;
  cm::moe_count_kernel<<<plan_blocks(n), 256, 0, s>>>(ids, n, plan_chunk(n), E, counts, block_counts);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// ids [n = T * k] int64, allc [ep, E] int64 (copies per source rank and expert), block_counts from cm_moe_count -> routing plan
extern "C" int cm_moe_plan(const long long* ids, long long n, int k, int E, int ep, int ep_rank, const long long* allc, const int* block_counts,
                           int tile, int n_tiles, long long* dest_row, int* dest_rank, int* token_of_copy, int* seg_start_local,
                           int* tot_local, int* seg_offsets, int* tile_expert, long long* counts_global, cudaStream_t s) {
  if (n <= 0) return 0;
  const long long chunk = plan_chunk(n);
  if (E > cm::PLAN_MAX_E || E % ep || (chunk + cm::PLAN_THREADS - 1) / cm::PLAN_THREADS > 255) return -10;
  const int smem = 2 * E * cm::PLAN_THREADS * (int)sizeof(unsigned short);
  static cm::PerDevice cfg;
  if (cfg.first()) {
    if (cudaFuncSetAttribute(cm::moe_plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * cm::PLAN_MAX_E * cm::PLAN_THREADS * 2) != cudaSuccess)
      return -2;
    cfg.done();
  }
  cm::PlanOut o{dest_row, dest_rank, token_of_copy, seg_start_local, tot_local, seg_offsets, tile_expert, counts_global};
  cm::moe_plan_kernel<<<plan_blocks(n), cm::PLAN_THREADS, smem, s>>>(ids, n, chunk, k, E, ep, ep_rank, allc, block_counts, tile, n_tiles, o);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
