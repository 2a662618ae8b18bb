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
                                                            long long capacity_rows, int* __restrict__ err) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int nvec = H / 8;
  for (int c = blockIdx.x * wpb + (threadIdx.x >> 5); c < ncopies; c += gridDim.x * wpb) {
    const int t = token_of_copy[c];
    const int r = dest_rank[c];
    const long long row = dest_row[c];
    if (row < 0 || row >= capacity_rows) {          // receiver buffer too small for this routing: drop + report
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
                                                               int T, int k, int H) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int nvec = H / 8;
  for (int t = blockIdx.x * wpb + (threadIdx.x >> 5); t < T; t += gridDim.x * wpb) {
    for (int v = lane; v < nvec; v += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int j = 0; j < k; ++j) {
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
                                                              const __nv_bfloat16* __restrict__ dy, float* __restrict__ out, int T, int k, int H) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  const int nvec = H / 8;
  const int n = T * k;
  for (int c = blockIdx.x * wpb + (threadIdx.x >> 5); c < n; c += gridDim.x * wpb) {
    const int t = c / k;
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

}  // namespace cm

using namespace cm;

static int grid_for(long long warps_needed) {
  long long blocks = (warps_needed + 7) / 8;
  long long cap = (long long)sm_count() * 8;
  return (int)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

extern "C" int cm_moe_push_rows(const void* src, const int* token_of_copy, const int* dest_rank, const long long* dest_row,
                                const float* scale, void* const* dst_ptrs, int world, int ncopies, int H,
                                long long capacity_rows, int* err, cudaStream_t s) {
  if (ncopies <= 0) return 0;
  if (H % 8 || world > MOE_MAX_PEERS) return -10;
  MoePeers p;
  for (int i = 0; i < world; ++i) p.p[i] = dst_ptrs[i];
  moe_push_rows_kernel<<<grid_for(ncopies), 256, 0, s>>>((const __nv_bfloat16*)src, token_of_copy, dest_rank, dest_row, scale, p, ncopies, H, capacity_rows, err);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int cm_moe_pull_combine(void* const* src_ptrs, int world, const int* dest_rank, const long long* dest_row,
                                   const float* weights, void* out, int T, int k, int H, cudaStream_t s) {
  if (T <= 0) return 0;
  if (H % 8 || world > MOE_MAX_PEERS) return -10;
  MoePeers p;
  for (int i = 0; i < world; ++i) p.p[i] = src_ptrs[i];
  moe_pull_combine_kernel<<<grid_for(T), 256, 0, s>>>(p, dest_rank, dest_row, weights, (__nv_bfloat16*)out, T, k, H);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int cm_moe_pull_rowdot(void* const* src_ptrs, int world, const int* dest_rank, const long long* dest_row,
                                  const void* dy, float* out, int T, int k, int H, cudaStream_t s) {
  if (T <= 0) return 0;
  if (H % 8 || world > MOE_MAX_PEERS) return -10;
  MoePeers p;
  for (int i = 0; i < world; ++i) p.p[i] = src_ptrs[i];
  moe_pull_rowdot_kernel<<<grid_for((long long)T * k), 256, 0, s>>>(p, dest_rank, dest_row, (const __nv_bfloat16*)dy, out, T, k, H);
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
