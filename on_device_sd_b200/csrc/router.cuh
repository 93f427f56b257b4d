// K1 - fused router: gate dot products, certified rounding, top-k with torch's CUDA tie order,
// softmax over the kept logits.  Replaces Qwen3MoEGate.forward
// (demo/src/layers/moe_layer.py:25-60 of the reference): nn.Linear + torch.topk + F.softmax.
//
// Logit definition.  A logit is the real-number dot product rounded to fp32 and then to the
// model dtype (the two roundings any fp32-accumulating GEMM applies), plus an optional bias
// added in the model dtype.  For 16-bit models the kernel evaluates the dot product in fp32
// and ACCEPTS the result only when its distance to the nearest rounding boundary of the model
// dtype exceeds a rigorous bound on the fp32 summation error ((H/32+16)*2^-24*|x|*|w|, from
// the Cauchy-Schwarz bound on sum|x_i w_i|); otherwise the logit is recomputed with fp64
// accumulation, where products of 16-bit values are exact.  Every logit therefore equals the
// fp64 definition bit for bit, whatever the summation order.  fp32 models always use fp64
// accumulation.
#pragma once
#include <type_traits>
#include "common.cuh"

namespace b200moe {

constexpr int kRouterTokensPerTile = 4;   // tokens per CTA tile
constexpr int kRouterThreads = 256;       // 8 warps = 8 experts per CTA in phase 1

struct RouterParams {
  const void* x;        // [T,H]
  const void* wg;       // [E,H]
  const void* bias;     // [E] or null (model dtype)
  const float* wnorm2;  // [E] squared row norms of wg
  const void* logits_in;  // [T,E] model dtype (route_from_logits) or null
  float* logit_sum;     // [T,E] fp32 dot products (workspace)
  float* xnorm2;        // [T]
  unsigned* tile_counter;  // [ceil(T/4)], zero between calls
  int64_t* ids64;       // [T,K]
  void* scores;         // [T,K] model dtype
  unsigned long long* bitmap;  // 4 words or null
  int T, H, E, K;
};

template <typename T> __device__ __forceinline__ double exact_dot(const T* xr, const T* wr, int nch, int lane) {
  double acc = 0.0;
  for (int c = lane; c < nch; c += 32) {
    Chunk<T> xc, wc;
    xc.template load<false>(xr + c * 8);
    wc.template load<false>(wr + c * 8);
    float xf[8], wf[8];
    xc.unpack(xf);
    wc.unpack(wf);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc = fma((double)xf[i], (double)wf[i], acc);
  }
  return warp_sum(acc);
}

// Distance (absolute) from an fp32 value to the nearest point where rounding to T changes.
// Returns 0 when no cheap statement is possible (then the caller recomputes exactly).
template <typename T> __device__ __forceinline__ float boundary_distance(float s) {
  const uint32_t u = __float_as_uint(s);
  const int ex = (u >> 23) & 0xff;
  if (ex <= 24 || ex == 0xff) return 0.0f;
  const float ulp32 = __uint_as_float((uint32_t)(ex - 23) << 23);
  if (std::is_same<T, __nv_bfloat16>::value) {
    const int frac = (int)(u & 0xffffu);
    return fabsf((float)(frac - 0x8000)) * ulp32;
  } else {  // fp16: 13 dropped bits, valid inside the normal range of fp16 only
    if (ex < 127 - 14 || ex > 127 + 14) return 0.0f;
    const int frac = (int)(u & 0x1fffu);
    return fabsf((float)(frac - 0x1000)) * ulp32;
  }
}

// One warp turns the E logits of token t into ordered top-k ids and softmax scores.
template <typename T>
__device__ void topk_softmax_token(const RouterParams& p, int t, int lane, float* skey, int* sidx) {
  constexpr int kMaxJ = kMaxExperts / 32;
  const int E = p.E, K = p.K;
  const int nj = (E + 31) / 32;
  float v[kMaxJ];
  const T* bias = reinterpret_cast<const T*>(p.bias);

  if (p.logits_in != nullptr) {
    const T* lg = reinterpret_cast<const T*>(p.logits_in) + (size_t)t * E;
#pragma unroll
    for (int j = 0; j < kMaxJ; ++j) {
      const int e = j * 32 + lane;
      v[j] = (j < nj && e < E) ? Elem<T>::to_float(lg[e]) : -INFINITY;
    }
  } else {
    const int nch = p.H / 8;
    const T* xr = reinterpret_cast<const T*>(p.x) + (size_t)t * p.H;
    const float xn = __ldcg(p.xnorm2 + t);
    const float cH = (float)(p.H / 32 + 16) * 5.9604645e-8f * 1.01f;
#pragma unroll
    for (int j = 0; j < kMaxJ; ++j) {
      if (j >= nj) { v[j] = -INFINITY; continue; }   // uniform across the warp
      const int e = j * 32 + lane;
      float s = 0.0f;
      bool risky = false;
      if (e < E) {
        s = __ldcg(p.logit_sum + (size_t)t * E + e);
        if (!std::is_same<T, float>::value) {
          const float bound = cH * sqrtf(xn * p.wnorm2[e]) + 1e-37f;
          risky = !(boundary_distance<T>(s) > bound);
        }
      }
      unsigned m = __ballot_sync(0xffffffffu, risky);
      while (m) {
        const int src = __ffs(m) - 1;
        m &= m - 1;
        const int e2 = j * 32 + src;
        const double d = exact_dot<T>(xr, reinterpret_cast<const T*>(p.wg) + (size_t)e2 * p.H, nch, lane);
        if (lane == src) s = (float)d;
      }
      float l = rn<T>(s);
      if (bias != nullptr && e < E) l = rn<T>(l + Elem<T>::to_float(bias[e]));
      v[j] = (e < E) ? l : -INFINITY;
      // keep the final logit where b200moe_last_logits can read it back
      if (e < E) p.logit_sum[(size_t)t * E + e] = l;
    }
  }

  // ---- selection: k rounds of (max value, lowest index) ----
  unsigned taken = 0;
  float kth = 0.0f;
  for (int r = 0; r < K; ++r) {
    float bv = -INFINITY;
    int be = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < kMaxJ; ++j) {
      const int e = j * 32 + lane;
      if (j < nj && e < E && !((taken >> j) & 1u)) {
        if (v[j] > bv || be == 0x7fffffff) { bv = v[j]; be = e; }   // ascending e within a lane
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (oe != 0x7fffffff && (be == 0x7fffffff || ov > bv || (ov == bv && oe < be))) { bv = ov; be = oe; }
    }
    if ((be & 31) == lane && be != 0x7fffffff) taken |= 1u << (be >> 5);
    kth = bv;
  }

  // ---- placement before the sort: entries > kth in index order, then entries == kth ----
  const unsigned lt = (1u << lane) - 1u;
  int base = 0;
#pragma unroll
  for (int pass = 0; pass < 2; ++pass) {
#pragma unroll
    for (int j = 0; j < kMaxJ; ++j) {
      if (j >= nj) continue;
      const bool sel = ((taken >> j) & 1u) && (pass == 0 ? (v[j] > kth) : (v[j] == kth));
      const unsigned m = __ballot_sync(0xffffffffu, sel);
      if (sel) {
        const int pos = base + __popc(m & lt);
        skey[pos] = v[j];
        sidx[pos] = j * 32 + lane;
      }
      base += __popc(m);
    }
  }
  __syncwarp();
  float key = (lane < K) ? skey[lane] : 0.0f;
  int idx = (lane < K) ? sidx[lane] : -1;
  bool ok = lane < K;
  __syncwarp();

  // ---- 32-slot bitonic network, the permutation torch's CUDA top-k applies for 1 < k <= 32 ----
  if (K > 1) {
    auto cmpx = [&](int stride, bool flag) {
      const float pk = __shfl_xor_sync(0xffffffffu, key, stride);
      const int pi = __shfl_xor_sync(0xffffffffu, idx, stride);
      const bool pok = __shfl_xor_sync(0xffffffffu, (int)ok, stride) != 0;
      const bool is_lo = (lane & stride) == 0;
      const float k_lo = is_lo ? key : pk, k_hi = is_lo ? pk : key;
      const bool ok_lo = is_lo ? ok : pok, ok_hi = is_lo ? pok : ok;
      const bool pred = (k_lo > k_hi && ok_lo) || !ok_hi;
      if (pred == flag) { key = pk; idx = pi; ok = pok; }
    };
    for (int size = 2; size < 32; size <<= 1)
      for (int stride = size >> 1; stride > 0; stride >>= 1) cmpx(stride, ((lane & ~stride) & size) != 0);
    for (int stride = 16; stride > 0; stride >>= 1) cmpx(stride, false);
  }

  // ---- softmax over the k kept logits (fp32 math, butterfly reductions over next_pow2(k) lanes) ----
  int width = 1;
  while (width < K) width <<= 1;
  float mx = (lane < K) ? key : -INFINITY;
  for (int o = width >> 1; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  const float ex = (lane < K) ? expf(key - mx) : 0.0f;
  float sum = ex;
  for (int o = width >> 1; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (lane < K) {
    const float sc = ex / sum;
    p.ids64[(size_t)t * K + lane] = idx;
    reinterpret_cast<T*>(p.scores)[(size_t)t * K + lane] = Elem<T>::from_float(sc);
    if (p.bitmap != nullptr) atomicOr(p.bitmap + (idx >> 6), 1ull << (idx & 63));
  }
}

// grid = (ceil(T/4), ceil(E/8)), 256 threads.  Phase 1: warp w of CTA (bx,by) computes the dot
// products of expert by*8+w with the 4 tokens of tile bx.  The CTA that finishes a tile last
// runs phase 2 (top-k) for its tokens; the counter returns to zero for the next call.
template <typename T> __global__ void __launch_bounds__(kRouterThreads) router_kernel(RouterParams p) {
  constexpr int TT = kRouterTokensPerTile;
  constexpr bool kExact = std::is_same<T, float>::value;
  using Acc = typename std::conditional<kExact, double, float>::type;
  __shared__ float skey[TT][32];
  __shared__ int sidx[TT][32];
  __shared__ int s_last;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t0 = blockIdx.x * TT;
  const int e = blockIdx.y * (kRouterThreads / 32) + warp;
  const int nch = p.H / 8;
  const T* x = reinterpret_cast<const T*>(p.x);

  if (e < p.E) {
    const T* wrow = reinterpret_cast<const T*>(p.wg) + (size_t)e * p.H;
    const bool do_norm = (blockIdx.y == 0 && warp == 0);
    Acc acc[TT];
    float xn[TT];
#pragma unroll
    for (int tt = 0; tt < TT; ++tt) { acc[tt] = 0; xn[tt] = 0.0f; }
    // two chunk positions per trip, all ten loads issued before the first use: the loop is
    // latency-bound (a warp owns one expert row), so loads in flight are what matter
    constexpr int U = 2;
    for (int c0 = lane; c0 < nch; c0 += 32 * U) {
      Chunk<T> wc[U], xc[U][TT];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int c = c0 + 32 * u;
        if (c < nch) {
          wc[u].template load<false>(wrow + c * 8);
#pragma unroll
          for (int tt = 0; tt < TT; ++tt)
            xc[u][tt].template load<false>(x + (size_t)min(t0 + tt, p.T - 1) * p.H + c * 8);
        } else {
          wc[u].zero();
#pragma unroll
          for (int tt = 0; tt < TT; ++tt) xc[u][tt].zero();
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        float wf[8];
        wc[u].unpack(wf);
#pragma unroll
        for (int tt = 0; tt < TT; ++tt) {
          float xf[8];
          xc[u][tt].unpack(xf);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            if (kExact) acc[tt] = fma((double)xf[i], (double)wf[i], acc[tt]);
            else acc[tt] = fmaf(xf[i], wf[i], acc[tt]);
            if (do_norm) xn[tt] = fmaf(xf[i], xf[i], xn[tt]);
          }
        }
      }
    }
#pragma unroll
    for (int tt = 0; tt < TT; ++tt) {
      const Acc s = warp_sum(acc[tt]);
      if (lane == 0 && t0 + tt < p.T) p.logit_sum[(size_t)(t0 + tt) * p.E + e] = (float)s;
      if (do_norm) {
        const float n2 = warp_sum(xn[tt]);
        if (lane == 0 && t0 + tt < p.T) p.xnorm2[t0 + tt] = n2;
      }
    }
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(p.tile_counter + blockIdx.x, 1u);
    s_last = (prev == gridDim.y - 1);
    if (s_last) p.tile_counter[blockIdx.x] = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (warp < TT && t0 + warp < p.T) topk_softmax_token<T>(p, t0 + warp, lane, skey[warp], sidx[warp]);
}

// Top-k / softmax on caller-supplied logits: one warp per token.
template <typename T> __global__ void __launch_bounds__(kRouterThreads) router_from_logits_kernel(RouterParams p) {
  __shared__ float skey[kRouterThreads / 32][32];
  __shared__ int sidx[kRouterThreads / 32][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (kRouterThreads / 32) + warp;
  if (t < p.T) topk_softmax_token<T>(p, t, lane, skey[warp], sidx[warp]);
}

// Squared row norms of the gate weight, one warp per expert (set_gate).
template <typename T> __global__ void gate_norm_kernel(const T* wg, float* wnorm2, int E, int H) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= E) return;
  float acc = 0.0f;
  for (int c = lane; c < H / 8; c += 32) {
    Chunk<T> wc;
    wc.template load<false>(wg + (size_t)warp * H + c * 8);
    float wf[8];
    wc.unpack(wf);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc = fmaf(wf[i], wf[i], acc);
  }
  acc = warp_sum(acc);
  if (lane == 0) wnorm2[warp] = acc;
}

}  // namespace b200moe
