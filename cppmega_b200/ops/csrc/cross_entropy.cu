// Softmax cross-entropy over a chunk of bf16 logits, fused with its own backward:
// per row compute max / log-sum-exp / target logit (one pass, online rescaling), write the
// per-token loss, then overwrite the logits in place with
//     dlogits = weight[row] * (softmax - onehot(label))
// so the caller can feed them straight into the dgrad / wgrad GEMMs.  The logits chunk is read
// twice (second read mostly from L2) and written once; full logits never exist.
// Stands in for the Liger / CCE / native fused linear-CE paths of the reference
// (cppmega/megatron/apply_linear_ce_patch.py:251-527) with a true per-token `none` reduction.
#include "common.cuh"

namespace cm {

constexpr int CE_THREADS = 512;

__global__ void __launch_bounds__(CE_THREADS) ce_fwd_bwd_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels,
                                                                const float* __restrict__ weights, float* __restrict__ loss_out,
                                                                float* __restrict__ lse_out, int rows, int V, long long ld,
                                                                int ignore_index, int write_grad) {
  __shared__ float s_max[CE_THREADS / 32], s_sum[CE_THREADS / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nvec = V / 8;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    __nv_bfloat16* lr = logits + (long long)row * ld;
    uint4* lv = reinterpret_cast<uint4*>(lr);
    const long long label = labels[row];
    const bool ignored = (label == ignore_index) || label < 0 || label >= V;
    if (ignored) {
      if (threadIdx.x == 0) { loss_out[row] = 0.f; if (lse_out) lse_out[row] = 0.f; }
      if (write_grad) {
        const uint4 z = make_uint4(0, 0, 0, 0);
        for (int i = threadIdx.x; i < nvec; i += CE_THREADS) lv[i] = z;
      }
      continue;
    }
    float mx = -INFINITY, sm = 0.f;
    for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
      const uint4 v = lv[i];
      const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v);
      float f[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) { float2 t = __bfloat1622float2(b[j]); f[2 * j] = t.x; f[2 * j + 1] = t.y; }
      float vm = f[0];
#pragma unroll
      for (int j = 1; j < 8; ++j) vm = fmaxf(vm, f[j]);
      if (vm > mx) { sm *= __expf(mx - vm); mx = vm; }
#pragma unroll
      for (int j = 0; j < 8; ++j) sm += __expf(f[j] - mx);
    }
    // block reduce (max, sum)
    float wm = warp_max(mx);
    sm = (mx == -INFINITY) ? 0.f : sm * __expf(mx - wm);     // lanes / warps that saw no element
    sm = warp_sum(sm);
    if (lane == 0) { s_max[warp] = wm; s_sum[warp] = sm; }
    __syncthreads();
    float gm = s_max[0];
#pragma unroll
    for (int i = 1; i < CE_THREADS / 32; ++i) gm = fmaxf(gm, s_max[i]);
    float gs = 0.f;
#pragma unroll
    for (int i = 0; i < CE_THREADS / 32; ++i) gs += (s_max[i] == -INFINITY) ? 0.f : s_sum[i] * __expf(s_max[i] - gm);
    const float lse = gm + __logf(gs);
    const float tgt = __bfloat162float(lr[label]);
    __syncthreads();          // everyone has read the target logit and the shared partials
    if (threadIdx.x == 0) { loss_out[row] = lse - tgt; if (lse_out) lse_out[row] = lse; }
    if (!write_grad) continue;
    const float wgt = weights ? weights[row] : 1.f;
    const int lvec = int(label >> 3), lsub = int(label & 7);
    for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
      const uint4 v = lv[i];
      const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v);
      float f[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) { float2 t = __bfloat1622float2(b[j]); f[2 * j] = t.x; f[2 * j + 1] = t.y; }
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = __expf(f[j] - lse);
      if (i == lvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) if (j == lsub) f[j] -= 1.f;
      }
      uint4 o;
      uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) op[j] = pack_bf16(f[2 * j] * wgt, f[2 * j + 1] * wgt);
      lv[i] = o;
    }
  }
}

}  // namespace cm

// logits [rows, V] bf16 (row pitch ld, V % 8 == 0) are replaced by weighted dlogits when
// write_grad != 0.  loss_out[rows] receives lse - target (0 for ignored rows).
extern "C" int cm_ce_fwd_bwd(void* logits, const long long* labels, const float* weights, float* loss_out,
                             float* lse_out, int rows, int V, long long ld, int ignore_index, int write_grad,
                             cudaStream_t s) {
  if (rows <= 0) return 0;
  if (V % 8 || ld % 8) return -10;
  int grid = rows < cm::sm_count() * 2 ? rows : cm::sm_count() * 2;
  cm::ce_fwd_bwd_kernel<<<grid, cm::CE_THREADS, 0, s>>>((__nv_bfloat16*)logits, labels, weights, loss_out, lse_out, rows, V,
                                                        ld, ignore_index, write_grad);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
