// Small memory-bound operators that PyTorch would run as many tiny launches:
//
//   router top-k     scores = sigmoid | softmax(logits), selection by scores + bias, combine weights from the unbiased
//                    scores (optionally normalised over the selected experts); forward and backward, one thread per token
//                    (the reference enables Megatron's router fusion for this, cppmega/recipes/megatron_args.py:114-135);
//   ngram-hash embed hash of the last `order` tokens per table -> row of one unified table -> concatenated rows
//                    (cppmega/features/engram/ngram_hash.py:117-141), gather forward and atomic scatter backward;
//   rotary embedding rotate-half RoPE over the last dimension with [S, D/2] tables, forward / backward (the backward is
//                    the rotation by the negative angle); the reference runs with RoPE fusion off
//                    (scripts/remote_smoke_h200_dsa_9_4_m.sh:152,621-624).
#include "common.cuh"

namespace cm {

constexpr int RT_MAX_E = 64;
constexpr int RT_MAX_K = 8;

__global__ void __launch_bounds__(256) router_topk_fwd_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                                              float* __restrict__ probs, long long* __restrict__ ids,
                                                              float* __restrict__ scores, long long T, int E, int K, int sigmoid,
                                                              int norm) {
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < T; t += (long long)gridDim.x * blockDim.x) {
    float s[RT_MAX_E];
    const float* lp = logits + t * E;
    if (sigmoid) {
#pragma unroll 4
      for (int e = 0; e < E; ++e) s[e] = 1.f / (1.f + __expf(-lp[e]));
    } else {
      float mx = -INFINITY;
      for (int e = 0; e < E; ++e) mx = fmaxf(mx, lp[e]);
      float z = 0.f;
      for (int e = 0; e < E; ++e) { s[e] = __expf(lp[e] - mx); z += s[e]; }
      const float iz = 1.f / z;
      for (int e = 0; e < E; ++e) s[e] *= iz;
    }
    for (int e = 0; e < E; ++e) scores[t * E + e] = s[e];
    int sel[RT_MAX_K];
    float zsum = 0.f;
    unsigned long long taken = 0ull;
    for (int j = 0; j < K; ++j) {
      int best = -1;
      float bv = -INFINITY;
      for (int e = 0; e < E; ++e) {
        if ((taken >> e) & 1ull) continue;
        const float v = s[e] + (bias ? bias[e] : 0.f);
        if (v > bv) { bv = v; best = e; }
      }
      if (best < 0) best = 0;
      taken |= 1ull << best;
      sel[j] = best;
      zsum += s[best];
    }
    const bool do_norm = norm && (sigmoid || K > 1);
    const float iz = do_norm ? 1.f / fmaxf(zsum, 1e-20f) : 1.f;
    for (int j = 0; j < K; ++j) {
      probs[t * K + j] = s[sel[j]] * iz;
      ids[t * K + j] = sel[j];
    }
  }
}

// dlogits from d(probs) [T,K] and d(scores) [T,E] (either may be null)
__global__ void __launch_bounds__(256) router_topk_bwd_kernel(const float* __restrict__ scores, const long long* __restrict__ ids,
                                                              const float* __restrict__ dprobs, const float* __restrict__ dscores,
                                                              float* __restrict__ dlogits, long long T, int E, int K, int sigmoid,
                                                              int norm) {
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < T; t += (long long)gridDim.x * blockDim.x) {
    float s[RT_MAX_E], ds[RT_MAX_E];
    for (int e = 0; e < E; ++e) {
      s[e] = scores[t * E + e];
      ds[e] = dscores ? dscores[t * E + e] : 0.f;
    }
    if (dprobs) {
      const bool do_norm = norm && (sigmoid || K > 1);
      float z = 0.f, dot = 0.f;
      for (int j = 0; j < K; ++j) z += s[ids[t * K + j]];
      z = fmaxf(z, 1e-20f);
      if (do_norm)
        for (int j = 0; j < K; ++j) dot += dprobs[t * K + j] * s[ids[t * K + j]] / z;
      for (int j = 0; j < K; ++j) {
        const int e = (int)ids[t * K + j];
        ds[e] += do_norm ? (dprobs[t * K + j] - dot) / z : dprobs[t * K + j];
      }
    }
    if (sigmoid) {
      for (int e = 0; e < E; ++e) dlogits[t * E + e] = ds[e] * s[e] * (1.f - s[e]);
    } else {
      float dot = 0.f;
      for (int e = 0; e < E; ++e) dot += ds[e] * s[e];
      for (int e = 0; e < E; ++e) dlogits[t * E + e] = s[e] * (ds[e] - dot);
    }
  }
}

// ---- ngram hash -----------------------------------------------------------------------------
__device__ __forceinline__ long long ngram_row(const long long* __restrict__ tok, long long b, int s, int S, int tb,
                                               const long long* __restrict__ mults, int max_order, const long long* __restrict__ bias,
                                               const long long* __restrict__ sizes, const long long* __restrict__ offsets,
                                               const long long* __restrict__ order) {
  long long h = 0;
  const int ord = (int)order[tb];
  for (int p = 0; p < max_order; ++p) {
    if (p >= ord) break;
    const long long tk = (s - p >= 0) ? tok[b * S + s - p] : 0;
    h ^= tk * mults[tb * max_order + p];
  }
  h ^= bias[tb];
  long long m = h % sizes[tb];
  if (m < 0) m += sizes[tb];            // same sign convention as the tensor library's remainder
  return m + offsets[tb];
}

// one warp per (token, table); lanes cover the embedding dim
template <typename T>
__global__ void __launch_bounds__(256) ngram_embed_fwd_kernel(const long long* __restrict__ tok, const T* __restrict__ table,
                                                              const long long* __restrict__ mults, const long long* __restrict__ bias,
                                                              const long long* __restrict__ sizes, const long long* __restrict__ offsets,
                                                              const long long* __restrict__ order, T* __restrict__ out, long long BS,
                                                              int S, int NT, int D, int max_order) {
  const int lane = threadIdx.x & 31;
  const long long w0 = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nw = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long w = w0; w < BS * NT; w += nw) {
    const long long tokn = w / NT;
    const int tb = (int)(w % NT);
    const long long row = ngram_row(tok, tokn / S, (int)(tokn % S), S, tb, mults, max_order, bias, sizes, offsets, order);
    for (int d = lane; d < D; d += 32) out[(tokn * NT + tb) * D + d] = table[row * D + d];
  }
}

template <typename T>
__global__ void __launch_bounds__(256) ngram_embed_bwd_kernel(const long long* __restrict__ tok, const T* __restrict__ dout,
                                                              const long long* __restrict__ mults, const long long* __restrict__ bias,
                                                              const long long* __restrict__ sizes, const long long* __restrict__ offsets,
                                                              const long long* __restrict__ order, float* __restrict__ dtable,
                                                              long long BS, int S, int NT, int D, int max_order) {
  const int lane = threadIdx.x & 31;
  const long long w0 = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nw = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long w = w0; w < BS * NT; w += nw) {
    const long long tokn = w / NT;
    const int tb = (int)(w % NT);
    const long long row = ngram_row(tok, tokn / S, (int)(tokn % S), S, tb, mults, max_order, bias, sizes, offsets, order);
    for (int d = lane; d < D; d += 32) atomicAdd(dtable + row * D + d, float(dout[(tokn * NT + tb) * D + d]));
  }
}

// ---- RoPE -----------------------------------------------------------------------------------
// x viewed as [B, S, R, D] (R = product of the middle dims); cos/sin [S, D/2] fp32; sign = +1 forward, -1 backward.
// `ldx` / `ldo`: elements between consecutive (b, s, r) rows of the input / output (>= D), so that a column slice of a
// wider head vector can be rotated without a copy.
__global__ void __launch_bounds__(256) rope_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ cosv,
                                                   const float* __restrict__ sinv, __nv_bfloat16* __restrict__ out, long long rows,
                                                   int S, int R, int D, long long ldx, long long ldo, float sign) {
  const int d2 = D / 2;
  const long long total = rows * d2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / d2;
    const int j = (int)(i % d2);
    const int s = (int)((row / R) % S);
    const float c = cosv[(size_t)s * d2 + j], sn = sign * sinv[(size_t)s * d2 + j];
    const float a = __bfloat162float(x[row * ldx + j]), b = __bfloat162float(x[row * ldx + d2 + j]);
    out[row * ldo + j] = __float2bfloat16(a * c - b * sn);
    out[row * ldo + d2 + j] = __float2bfloat16(a * sn + b * c);
  }
}

}  // namespace cm

using namespace cm;

static int grid_1d(long long work, int per_block = 256) {
  long long blocks = (work + per_block - 1) / per_block;
  long long cap = (long long)sm_count() * 16;
  return (int)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

extern "C" int cm_router_topk_fwd(const float* logits, const float* bias, float* probs, long long* ids, float* scores,
                                  long long T, int E, int K, int sigmoid, int norm, cudaStream_t s) {
  if (T <= 0) return 0;
  if (E > RT_MAX_E || K > RT_MAX_K || K > E || E <= 0 || K <= 0) return -10;
  router_topk_fwd_kernel<<<grid_1d(T), 256, 0, s>>>(logits, bias, probs, ids, scores, T, E, K, sigmoid, norm);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int cm_router_topk_bwd(const float* scores, const long long* ids, const float* dprobs, const float* dscores,
                                  float* dlogits, long long T, int E, int K, int sigmoid, int norm, cudaStream_t s) {
  if (T <= 0) return 0;
  if (E > RT_MAX_E || K > RT_MAX_K) return -10;
  router_topk_bwd_kernel<<<grid_1d(T), 256, 0, s>>>(scores, ids, dprobs, dscores, dlogits, T, E, K, sigmoid, norm);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// kind: 0 fp32 table / output, 1 bf16
extern "C" int cm_ngram_embed_fwd(const long long* tok, const void* table, const long long* mults, const long long* bias,
                                  const long long* sizes, const long long* offsets, const long long* order, void* out, int B,
                                  int S, int NT, int D, int max_order, int kind, cudaStream_t s) {
  const long long BS = (long long)B * S;
  if (BS <= 0 || NT <= 0) return 0;
  const int grid = grid_1d(BS * NT * 32);
  if (kind == 0)
    ngram_embed_fwd_kernel<float><<<grid, 256, 0, s>>>(tok, (const float*)table, mults, bias, sizes, offsets, order, (float*)out, BS, S, NT, D, max_order);
  else
    ngram_embed_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(tok, (const __nv_bfloat16*)table, mults, bias, sizes, offsets, order, (__nv_bfloat16*)out, BS, S, NT, D, max_order);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// dtable fp32 [rows, D], zeroed by the caller
extern "C" int cm_ngram_embed_bwd(const long long* tok, const void* dout, const long long* mults, const long long* bias,
                                  const long long* sizes, const long long* offsets, const long long* order, float* dtable, int B,
                                  int S, int NT, int D, int max_order, int kind, cudaStream_t s) {
  const long long BS = (long long)B * S;
  if (BS <= 0 || NT <= 0) return 0;
  const int grid = grid_1d(BS * NT * 32);
  if (kind == 0)
    ngram_embed_bwd_kernel<float><<<grid, 256, 0, s>>>(tok, (const float*)dout, mults, bias, sizes, offsets, order, dtable, BS, S, NT, D, max_order);
  else
    ngram_embed_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(tok, (const __nv_bfloat16*)dout, mults, bias, sizes, offsets, order, dtable, BS, S, NT, D, max_order);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int cm_rope(const void* x, const float* cosv, const float* sinv, void* out, long long rows, int S, int R, int D,
                       long long ldx, long long ldo, float sign, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (D % 2 || ldx < D || ldo < D) return -10;
  rope_kernel<<<grid_1d(rows * (D / 2)), 256, 0, s>>>((const __nv_bfloat16*)x, cosv, sinv, (__nv_bfloat16*)out, rows, S, R, D, ldx, ldo, sign);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// ------------------------------------------------------------------------------------------
// Word embedding: gather forward, and a backward that adds every token's output-gradient row straight into the row of
// the weight's gradient buffer (fp32 or bf16) with vector atomics - no dense [vocab, hidden] gradient tensor, no
// separate accumulation pass.  One warp per token; ids outside [0, vocab) are skipped (forward writes zeros).
// ------------------------------------------------------------------------------------------
namespace cm {

__global__ void __launch_bounds__(256) embedding_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ w,
                                                            __nv_bfloat16* __restrict__ out, long long T, long long vocab, int H) {
  const int lane = threadIdx.x & 31;
  const long long w0 = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nw = ((long long)gridDim.x * blockDim.x) >> 5;
  const int nvec = H / 8;
  for (long long t = w0; t < T; t += nw) {
    const long long id = ids[t];
    uint4* o = reinterpret_cast<uint4*>(out + t * H);
    if (id < 0 || id >= vocab) {
      for (int v = lane; v < nvec; v += 32) o[v] = make_uint4(0u, 0u, 0u, 0u);
      continue;
    }
    const uint4* s = reinterpret_cast<const uint4*>(w + id * H);
    for (int v = lane; v < nvec; v += 32) o[v] = s[v];
  }
}

template <typename G>
__global__ void __launch_bounds__(256) embedding_bwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ dout,
                                                            G* __restrict__ dw, long long T, long long vocab, int H) {
  const int lane = threadIdx.x & 31;
  const long long w0 = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nw = ((long long)gridDim.x * blockDim.x) >> 5;
  const int nvec = H / 8;
  for (long long t = w0; t < T; t += nw) {
    const long long id = ids[t];
    if (id < 0 || id >= vocab) continue;
    const uint4* s = reinterpret_cast<const uint4*>(dout + t * H);
    for (int v = lane; v < nvec; v += 32) {
      const uint4 x = s[v];
      const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&x);
      if constexpr (sizeof(G) == 4) {
        float* d = reinterpret_cast<float*>(dw) + id * H + v * 8;
        const float2 f0 = __bfloat1622float2(b[0]), f1 = __bfloat1622float2(b[1]), f2 = __bfloat1622float2(b[2]),
                     f3 = __bfloat1622float2(b[3]);
        atomicAdd(reinterpret_cast<float4*>(d), make_float4(f0.x, f0.y, f1.x, f1.y));
        atomicAdd(reinterpret_cast<float4*>(d) + 1, make_float4(f2.x, f2.y, f3.x, f3.y));
      } else {
        __nv_bfloat162* d = reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<__nv_bfloat16*>(dw) + id * H + v * 8);
#pragma unroll
        for (int j = 0; j < 4; ++j) atomicAdd(d + j, b[j]);
      }
    }
  }
}

static int embedding_grid(long long T) {
  long long blocks = (T + 7) / 8;
  const long long cap = (long long)sm_count() * 8;
  return (int)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}
}  // namespace cm

// ids [T] int64, w [vocab, H] bf16, out [T, H] bf16; H % 8 == 0
extern "C" int cm_embedding_fwd(const long long* ids, const void* w, void* out, long long T, long long vocab, int H, cudaStream_t s) {
  if (T <= 0) return 0;
  if (H % 8) return -10;
  cm::embedding_fwd_kernel<<<cm::embedding_grid(T), 256, 0, s>>>(ids, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, T, vocab, H);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// dw [vocab, H] (+)= scatter of dout [T, H] bf16 by ids; grad_kind 0: fp32 buffer, 1: bf16 buffer
extern "C" int cm_embedding_bwd(const long long* ids, const void* dout, void* dw, long long T, long long vocab, int H, int grad_kind,
                                cudaStream_t s) {
  if (T <= 0) return 0;
  if (H % 8) return -10;
  if (grad_kind == 0)
    cm::embedding_bwd_kernel<float><<<cm::embedding_grid(T), 256, 0, s>>>(ids, (const __nv_bfloat16*)dout, (float*)dw, T, vocab, H);
  else
    cm::embedding_bwd_kernel<__nv_bfloat16><<<cm::embedding_grid(T), 256, 0, s>>>(ids, (const __nv_bfloat16*)dout, (__nv_bfloat16*)dw, T, vocab, H);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
