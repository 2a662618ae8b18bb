// M2RNN matrix-state recurrence, forward and backward.
//
//   a_t = h_{t-1} W + k_t (x) v_t ;  h_t = f_t h_{t-1} + (1 - f_t) tanh(a_t) ;  y_t = q_t . h_t
//
// One CTA per (batch, head).  The state h [KD x 16] lives in registers for the whole sequence:
// thread (k, quad) owns h[k, 4*quad .. 4*quad+3]; the four threads of a row are adjacent lanes and
// exchange their quads with shuffles for the 16x16 state transition.  Inputs are staged through
// shared memory in blocks of 32 time steps (next block prefetched into registers while the
// current one runs); y partial sums are reduced over k once per block.  The forward pass can
// write the state history (fp32) that the backward pass replays in reverse; the backward pass
// recomputes tanh(a_t) from h_{t-1}, keeps dh in registers, accumulates dW per thread over time
// and reduces it once at the end.  q and k gradients are produced per head (the caller sums the
// head axis when q/k are shared by all heads).
// The reference runs this recurrence as Triton kernels with 64-token checkpoints
// (cppmega/megatron/m2rnn_triton.py:243-415 forward, :662-758 backward).
#include "common.cuh"

namespace cm {

constexpr int VD = 16;       // value head dim (fixed)
constexpr int TB = 32;       // time steps per staging block (forward)
constexpr int TBB = 16;      // backward (more staged arrays)

__device__ __forceinline__ float fast_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Forward.  One CTA owns RS = min(KD, 16) state rows of one (batch, head): 4 * RS threads, thread (row, quad) holds
// h[row, 4 quad .. 4 quad + 3].  The 16 x 16 transition matrix sits in registers, arranged per thread in the order in
// which the row's other three quads arrive by shuffle ("rotation d" brings quad (quad + d) % 4), so a step costs
// 12 shuffles for the matvec and 4 for the reduction of y over the rows of a warp.  With KD > 16 a head is split
// over KD / 16 CTAs; each writes an fp32 partial y and a small kernel adds the parts.
template <int KD>
struct M2Split {
  static constexpr int RS = KD < 16 ? KD : 16;     // 16 rows = 64 threads: B*H*KD/16 CTAs balance over the SMs
  static constexpr int SPLITS = KD / RS;
  static constexpr int NT = RS * 4;
};

template <int KD>
__global__ void __launch_bounds__(M2Split<KD>::NT) m2rnn_fwd_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
    const __nv_bfloat16* __restrict__ W, const float* __restrict__ f, __nv_bfloat16* __restrict__ y, float* __restrict__ y_part,
    float* __restrict__ hist, float* __restrict__ h_last, int B, int S, int H, int Hq, int Hk) {
  constexpr int RS = M2Split<KD>::RS, SPLITS = M2Split<KD>::SPLITS, NT = M2Split<KD>::NT;
  constexpr int NW = NT / 32;
  constexpr int QPT = TB * RS / NT;     // staged q (and k) elements per thread = 8
  constexpr int VPT = (TB * VD + NT - 1) / NT;
  __shared__ float qs[TB][RS], ks[TB][RS], fs[TB];
  __shared__ __align__(16) float vs[TB][VD];
  __shared__ float ypart[TB][NW][VD];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int lrow = tid >> 2, quad = tid & 3;
  const int sp = blockIdx.x % SPLITS;
  const int bh = blockIdx.x / SPLITS;
  const int b = bh / H, h = bh % H;
  const int row = sp * RS + lrow;
  const int hq = Hq == 1 ? 0 : h, hk = Hk == 1 ? 0 : h;
  // wrot[d][u][c] = W[4 * ((quad + d) % 4) + u][4 * quad + c]
  float wrot[4][4][4];
#pragma unroll
  for (int d = 0; d < 4; ++d)
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int c = 0; c < 4; ++c)
        wrot[d][u][c] = __bfloat162float(W[(size_t)h * VD * VD + (4 * ((quad + d) & 3) + u) * VD + 4 * quad + c]);
  float hreg[4] = {0.f, 0.f, 0.f, 0.f};
  float pq[QPT], pk[QPT], pv[VPT], pf = 0.f;

  auto prefetch = [&](int t0) {
#pragma unroll
    for (int i = 0; i < QPT; ++i) {
      const int e = tid + i * NT, t = e / RS, c = e % RS;
      const bool ok = t0 + t < S;
      pq[i] = ok ? __bfloat162float(q[((size_t)(b * S + t0 + t) * Hq + hq) * KD + sp * RS + c]) : 0.f;
      pk[i] = ok ? __bfloat162float(k[((size_t)(b * S + t0 + t) * Hk + hk) * KD + sp * RS + c]) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int e = tid + i * NT;
      const int t = e / VD, c = e % VD;
      pv[i] = (e < TB * VD && t0 + t < S) ? __bfloat162float(v[((size_t)(b * S + t0 + t) * H + h) * VD + c]) : 0.f;
    }
    if (tid < TB) pf = (t0 + tid < S) ? f[(size_t)(b * S + t0 + tid) * H + h] : 1.f;
  };
  auto commit = [&]() {
#pragma unroll
    for (int i = 0; i < QPT; ++i) {
      const int e = tid + i * NT;
      qs[e / RS][e % RS] = pq[i];
      ks[e / RS][e % RS] = pk[i];
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int e = tid + i * NT;
      if (e < TB * VD) vs[e / VD][e % VD] = pv[i];
    }
    if (tid < TB) fs[tid] = pf;
  };

  prefetch(0);
  commit();
  __syncthreads();
  const int src_base = lane & ~3;
  for (int t0 = 0; t0 < S; t0 += TB) {
    if (t0 + TB < S) prefetch(t0 + TB);
    const int nt = min(TB, S - t0);
    for (int t = 0; t < nt; ++t) {
      const float kt = ks[t][lrow], qt = qs[t][lrow], ft = fs[t];
      const float4 vq = *reinterpret_cast<const float4*>(&vs[t][quad * 4]);
      float a[4] = {kt * vq.x, kt * vq.y, kt * vq.z, kt * vq.w};
#pragma unroll
      for (int d = 0; d < 4; ++d) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float hv = d == 0 ? hreg[u] : __shfl_sync(0xffffffffu, hreg[u], src_base | ((quad + d) & 3));
#pragma unroll
          for (int c = 0; c < 4; ++c) a[c] = fmaf(hv, wrot[d][u][c], a[c]);
        }
      }
      float yp[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        hreg[c] = ft * hreg[c] + (1.f - ft) * fast_tanh(a[c]);
        yp[c] = qt * hreg[c];
      }
      if (hist) {
        float4 o = make_float4(hreg[0], hreg[1], hreg[2], hreg[3]);
        *reinterpret_cast<float4*>(hist + (((size_t)(b * H + h) * S + t0 + t) * KD + row) * VD + quad * 4) = o;
      }
      // sum over the 8 rows of this warp (lanes that differ in bits 2..4): 4 shuffles, halving the values kept
      {
        const bool u4 = lane & 16, u3 = lane & 8;
        const float k0 = u4 ? yp[2] : yp[0], k1 = u4 ? yp[3] : yp[1];
        const float s0 = u4 ? yp[0] : yp[2], s1 = u4 ? yp[1] : yp[3];
        const float a0 = k0 + __shfl_xor_sync(0xffffffffu, s0, 16);
        const float a1 = k1 + __shfl_xor_sync(0xffffffffu, s1, 16);
        const float kk = u3 ? a1 : a0, ss = u3 ? a0 : a1;
        float r = kk + __shfl_xor_sync(0xffffffffu, ss, 8);
        r += __shfl_xor_sync(0xffffffffu, r, 4);
        if ((lane & 4) == 0) ypart[t][warp][quad * 4 + (u4 ? 2 : 0) + (u3 ? 1 : 0)] = r;
      }
    }
    __syncthreads();
    for (int e = tid; e < nt * VD; e += NT) {
      const int t = e / VD, c = e % VD;
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) s += ypart[t][w][c];
      const size_t o = ((size_t)(b * S + t0 + t) * H + h) * VD + c;
      if (SPLITS == 1) y[o] = __float2bfloat16(s);
      else y_part[(size_t)sp * B * S * H * VD + o] = s;
    }
    if (t0 + TB < S) commit();
    __syncthreads();
  }
  if (h_last) {
    float4 o = make_float4(hreg[0], hreg[1], hreg[2], hreg[3]);
    *reinterpret_cast<float4*>(h_last + ((size_t)(b * H + h) * KD + row) * VD + quad * 4) = o;
  }
}

__global__ void __launch_bounds__(256) m2rnn_sum_parts_kernel(const float* __restrict__ parts, __nv_bfloat16* __restrict__ y, int nparts,
                                                              long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float s = 0.f;
    for (int p = 0; p < nparts; ++p) s += parts[(size_t)p * n + i];
    y[i] = __float2bfloat16(s);
  }
}

// Backward.  A CTA owns RS state rows of one (batch, head) (thread = (row, quad), W and W^T in shared memory); with
// KD = 64 a head is split over two CTAs of 32 rows so that all CTAs are resident at once, and dv / df / dW, which sum
// over the rows of a head, are accumulated with atomics into zeroed outputs.
// The state history is walked backwards with rolling registers: the row h_{t-1} needed by a step was requested one
// step earlier and h_t (own quad) is a slice of the row used by the previous step, so each step issues one row load
// whose latency hides behind the arithmetic.
template <int KD, int RS>
__global__ void __launch_bounds__(RS * 4) m2rnn_bwd_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
    const __nv_bfloat16* __restrict__ W, const float* __restrict__ f, const float* __restrict__ hist,
    const __nv_bfloat16* __restrict__ dy, float* __restrict__ dq_h, float* __restrict__ dk_h,
    float* __restrict__ dv, float* __restrict__ df, float* __restrict__ dW, int S, int H, int Hq, int Hk) {
  constexpr int NT = RS * 4;
  constexpr int SPLITS = KD / RS;
  constexpr int NW = NT / 32;
  constexpr int QPT = TBB * RS / NT;
  __shared__ float Ws[VD][VD];          // W[u][v]
  __shared__ float Wt[VD][VD];          // W^T: Wt[v][u]
  __shared__ float qs[TBB][RS], ks[TBB][RS], vs[TBB][VD], gs[TBB][VD], fs[TBB];
  __shared__ float dqs[TBB][RS], dks[TBB][RS], dvpart[TBB][NW][VD], dfpart[TBB][NW];
  __shared__ float dWs[VD][VD];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int lrow = tid >> 2, quad = tid & 3;
  const int sp = blockIdx.x % SPLITS;
  const int bh = blockIdx.x / SPLITS;
  const int b = bh / H, h = bh % H;
  const int row = sp * RS + lrow;
  const int hq = Hq == 1 ? 0 : h, hk = Hk == 1 ? 0 : h;
  for (int i = tid; i < VD * VD; i += NT) {
    const float w = __bfloat162float(W[(size_t)h * VD * VD + i]);
    Ws[i / VD][i % VD] = w;
    Wt[i % VD][i / VD] = w;
    dWs[i / VD][i % VD] = 0.f;
  }
  float dh[4] = {0.f, 0.f, 0.f, 0.f};
  float P[4][VD];
#pragma unroll
  for (int c = 0; c < 4; ++c)
#pragma unroll
    for (int j = 0; j < VD; ++j) P[c][j] = 0.f;
  const float* hbase = hist + (size_t)(b * H + h) * S * KD * VD;
  __syncthreads();

  // rolling history registers: row h_{S-2} and own quad of h_{S-1}
  float4 rowbuf[4], quadbuf;
  quadbuf = *reinterpret_cast<const float4*>(hbase + ((size_t)(S - 1) * KD + row) * VD + quad * 4);
  if (S > 1) {
    const float4* hp = reinterpret_cast<const float4*>(hbase + ((size_t)(S - 2) * KD + row) * VD);
#pragma unroll
    for (int j = 0; j < 4; ++j) rowbuf[j] = hp[j];
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) rowbuf[j] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const int nblocks = (S + TBB - 1) / TBB;
  for (int blk = nblocks - 1; blk >= 0; --blk) {
    const int t0 = blk * TBB;
    const int nt = min(TBB, S - t0);
    // stage this block's inputs
#pragma unroll
    for (int i = 0; i < QPT; ++i) {
      const int e = tid + i * NT, t = e / RS, c = e % RS;
      const bool ok = t < nt;
      qs[t][c] = ok ? __bfloat162float(q[((size_t)(b * S + t0 + t) * Hq + hq) * KD + sp * RS + c]) : 0.f;
      ks[t][c] = ok ? __bfloat162float(k[((size_t)(b * S + t0 + t) * Hk + hk) * KD + sp * RS + c]) : 0.f;
    }
    for (int e = tid; e < TBB * VD; e += NT) {
      const int t = e / VD, c = e % VD;
      const bool ok = t < nt;
      vs[t][c] = ok ? __bfloat162float(v[((size_t)(b * S + t0 + t) * H + h) * VD + c]) : 0.f;
      gs[t][c] = ok ? __bfloat162float(dy[((size_t)(b * S + t0 + t) * H + h) * VD + c]) : 0.f;
    }
    if (tid < TBB) fs[tid] = (tid < nt) ? f[(size_t)(b * S + t0 + tid) * H + h] : 1.f;
    __syncthreads();
    for (int t = nt - 1; t >= 0; --t) {
      const int tg = t0 + t;
      // h_{t-1} (full row) was prefetched one step ago and h_t (own quad) is a slice of the row used then; the row
      // for the next step (h_{t-2}) is requested now so that its latency hides behind this step's arithmetic
      float hprev[VD];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        hprev[j * 4 + 0] = rowbuf[j].x; hprev[j * 4 + 1] = rowbuf[j].y; hprev[j * 4 + 2] = rowbuf[j].z; hprev[j * 4 + 3] = rowbuf[j].w;
      }
      const float hcur[4] = {quadbuf.x, quadbuf.y, quadbuf.z, quadbuf.w};
      if (tg > 1) {
        const float4* hp = reinterpret_cast<const float4*>(hbase + ((size_t)(tg - 2) * KD + row) * VD);
#pragma unroll
        for (int j = 0; j < 4; ++j) rowbuf[j] = hp[j];
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) rowbuf[j] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
      const float kt = ks[t][lrow], qt = qs[t][lrow], ft = fs[t];
      // dh_t += q_t (x) dy_t ; dq_t = h_t . dy_t
      float dqp = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float g = gs[t][quad * 4 + c];
        dh[c] += qt * g;
        dqp += hcur[c] * g;
      }
      dqp += __shfl_xor_sync(0xffffffffu, dqp, 1);
      dqp += __shfl_xor_sync(0xffffffffu, dqp, 2);
      if (quad == 0) dqs[t][lrow] = dqp;
      // recompute tanh(a_t) for own columns
      float a[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) a[c] = kt * vs[t][quad * 4 + c];
#pragma unroll
      for (int u = 0; u < VD; ++u) {
        const float4 w = *reinterpret_cast<const float4*>(&Ws[u][quad * 4]);
        a[0] += hprev[u] * w.x; a[1] += hprev[u] * w.y; a[2] += hprev[u] * w.z; a[3] += hprev[u] * w.w;
      }
      float hown[4];                     // h_{t-1}[k, own quad], selected without dynamic indexing
#pragma unroll
      for (int c = 0; c < 4; ++c)
        hown[c] = quad == 0 ? hprev[c] : quad == 1 ? hprev[4 + c] : quad == 2 ? hprev[8 + c] : hprev[12 + c];
      quadbuf = make_float4(hown[0], hown[1], hown[2], hown[3]);      // h_{t-1}[own quad] is next step's h_t
      float da[4], dfp = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float hn = fast_tanh(a[c]);
        dfp += dh[c] * (hown[c] - hn);
        da[c] = dh[c] * (1.f - ft) * (1.f - hn * hn);
      }
      dfp = warp_sum(dfp);
      if (lane == 0) dfpart[t][warp] = dfp;
      // full da row of this k
      float darow[VD];
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) darow[j * 4 + c] = __shfl_sync(0xffffffffu, da[c], (lane & ~3) + j);
      // dk_t[k] = da[k,:] . v_t
      if (quad == 0) {
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < VD; ++j) s += darow[j] * vs[t][j];
        dks[t][lrow] = s;
      }
      // dv_t[v] = sum_k da[k,v] k_t[k]  (own columns; reduce over the 8 rows of this warp)
      float dvp[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        dvp[c] = da[c] * kt;
        dvp[c] += __shfl_xor_sync(0xffffffffu, dvp[c], 4);
        dvp[c] += __shfl_xor_sync(0xffffffffu, dvp[c], 8);
        dvp[c] += __shfl_xor_sync(0xffffffffu, dvp[c], 16);
      }
      if (lane < 4) {
#pragma unroll
        for (int c = 0; c < 4; ++c) dvpart[t][warp][quad * 4 + c] = dvp[c];
      }
      // dW[u,v] += h_{t-1}[k,u] da[k,v]  for own u = 4*quad + c
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float hu = hown[c];
#pragma unroll
        for (int j = 0; j < VD; ++j) P[c][j] += hu * darow[j];
      }
      // dh_{t-1}[k,u] = f dh_t[k,u] + sum_v da[k,v] W[u,v]   for own u
#pragma unroll
      for (int c = 0; c < 4; ++c) dh[c] *= ft;
#pragma unroll
      for (int j = 0; j < VD; ++j) {
        const float4 w = *reinterpret_cast<const float4*>(&Wt[j][quad * 4]);   // W[u=4q..4q+3][v=j]
        dh[0] += darow[j] * w.x; dh[1] += darow[j] * w.y; dh[2] += darow[j] * w.z; dh[3] += darow[j] * w.w;
      }
    }
    __syncthreads();
    // write this block's per-step gradients
    for (int e = tid; e < nt * RS; e += NT) {
      const int t = e / RS, c = e % RS;
      dq_h[((size_t)(b * S + t0 + t) * H + h) * KD + sp * RS + c] = dqs[t][c];
      dk_h[((size_t)(b * S + t0 + t) * H + h) * KD + sp * RS + c] = dks[t][c];
    }
    for (int e = tid; e < nt * VD; e += NT) {
      const int t = e / VD, c = e % VD;
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) s += dvpart[t][w][c];
      float* dst = dv + ((size_t)(b * S + t0 + t) * H + h) * VD + c;
      if (SPLITS == 1) *dst = s; else atomicAdd(dst, s);
    }
    if (tid < nt) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) s += dfpart[tid][w];
      float* dst = df + (size_t)(b * S + t0 + tid) * H + h;
      if (SPLITS == 1) *dst = s; else atomicAdd(dst, s);
    }
    __syncthreads();
  }
  // reduce dW over the rows k of this CTA, then over batch with atomics
#pragma unroll
  for (int c = 0; c < 4; ++c)
#pragma unroll
    for (int j = 0; j < VD; ++j) {
      float s = P[c][j];
      s += __shfl_xor_sync(0xffffffffu, s, 4);
      s += __shfl_xor_sync(0xffffffffu, s, 8);
      s += __shfl_xor_sync(0xffffffffu, s, 16);
      if (lane < 4) atomicAdd(&dWs[quad * 4 + c][j], s);
    }
  __syncthreads();
  for (int i = tid; i < VD * VD; i += NT) atomicAdd(dW + (size_t)h * VD * VD + i, dWs[i / VD][i % VD]);
}

}  // namespace cm

using namespace cm;

// q [B,S,Hq,KD], k [B,S,Hk,KD], v [B,S,H,16], W [H,16,16] (bf16); f [B,S,H] fp32.
// y [B,S,H,16] bf16; y_part: fp32 scratch [KD/16,B,S,H,16] (needed for KD > 16, may be null otherwise);
// hist (nullable) [B,H,S,KD,16] fp32; h_last (nullable) [B,H,KD,16] fp32.
extern "C" int cm_m2rnn_fwd(const void* q, const void* k, const void* v, const void* W, const float* f, void* y,
                            float* y_part, float* hist, float* h_last, int B, int S, int H, int Hq, int Hk, int KD, int VDim,
                            cudaStream_t s) {
  if (B <= 0 || S <= 0) return 0;
  if (VDim != VD) return -10;
  auto qp = (const __nv_bfloat16*)q; auto kp = (const __nv_bfloat16*)k; auto vp = (const __nv_bfloat16*)v;
  auto wp = (const __nv_bfloat16*)W; auto yp = (__nv_bfloat16*)y;
  const int bh = B * H;
  if (KD == 64 || KD == 32) {
    const int splits = KD / 16;
    if (!y_part) return -10;          // several CTAs per head: needs the [KD/16, B, S, H, 16] fp32 partial buffer
    if (KD == 64) m2rnn_fwd_kernel<64><<<bh * splits, 64, 0, s>>>(qp, kp, vp, wp, f, yp, y_part, hist, h_last, B, S, H, Hq, Hk);
    else m2rnn_fwd_kernel<32><<<bh * splits, 64, 0, s>>>(qp, kp, vp, wp, f, yp, y_part, hist, h_last, B, S, H, Hq, Hk);
    const long long n = (long long)B * S * H * VD;
    long long blocks = (n + 255) / 256;
    const int grid = (int)(blocks < (long long)sm_count() * 8 ? blocks : (long long)sm_count() * 8);
    m2rnn_sum_parts_kernel<<<grid, 256, 0, s>>>(y_part, yp, splits, n);
  } else if (KD == 16) {
    m2rnn_fwd_kernel<16><<<bh, 64, 0, s>>>(qp, kp, vp, wp, f, yp, y_part, hist, h_last, B, S, H, Hq, Hk);
  } else {
    return -10;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// dq_h, dk_h [B,S,H,KD] fp32 (per head); dv [B,S,H,16], df [B,S,H] and dW [H,16,16] fp32 are accumulated: the caller zeroes them.
extern "C" int cm_m2rnn_bwd(const void* q, const void* k, const void* v, const void* W, const float* f, const float* hist,
                            const void* dy, float* dq_h, float* dk_h, float* dv, float* df, float* dW, int B, int S, int H,
                            int Hq, int Hk, int KD, int VDim, cudaStream_t s) {
  if (B <= 0 || S <= 0) return 0;
  if (VDim != VD) return -10;
  auto qp = (const __nv_bfloat16*)q; auto kp = (const __nv_bfloat16*)k; auto vp = (const __nv_bfloat16*)v;
  auto wp = (const __nv_bfloat16*)W; auto gp = (const __nv_bfloat16*)dy;
  const int grid = B * H;
  // K = 64: four CTAs of 16 state rows each per (batch, head) (6.3 ms against 6.6 ms with two CTAs of 32 rows and 10.4 ms
  // with one CTA of 64 rows at B 4, S 4096, 51 heads): more resident CTAs hide the per-step dependency chain better
  if (KD == 64) m2rnn_bwd_kernel<64, 16><<<grid * 4, 64, 0, s>>>(qp, kp, vp, wp, f, hist, gp, dq_h, dk_h, dv, df, dW, S, H, Hq, Hk);
  else if (KD == 32) m2rnn_bwd_kernel<32, 32><<<grid, 128, 0, s>>>(qp, kp, vp, wp, f, hist, gp, dq_h, dk_h, dv, df, dW, S, H, Hq, Hk);
  else if (KD == 16) m2rnn_bwd_kernel<16, 16><<<grid, 64, 0, s>>>(qp, kp, vp, wp, f, hist, gp, dq_h, dk_h, dv, df, dW, S, H, Hq, Hk);
  else return -10;
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
