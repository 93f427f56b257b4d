// K1 - fused router: gate dot products, certified rounding, top-k with torch's CUDA tie order,
// softmax over the kept logits.  Replaces Qwen3MoEGate.forward
// (demo/src/layers/moe_layer.py:25-60 of the reference): nn.Linear + torch.topk + F.softmax.
//
// Logit definition.  A logit is the real-number dot product rounded to fp32 and then to the
// model dtype (the two roundings any fp32-accumulating GEMM applies), plus an optional bias
// added in the model dtype.  For 16-bit models the kernel evaluates the dot product in fp32
// together with sum|x_i w_i|, and ACCEPTS the fp32 result only when its distance to the nearest
// rounding boundary of the model dtype exceeds a rigorous bound on the fp32 summation error,
// (H/128 + 12) * 2^-24 * sum|x_i w_i| (products of 16-bit values are exact in fp32; each of
// the four accumulators of a lane sees at most H/128 + 2 roundings, then 2 + 5 for the tree).
// Otherwise the same warp recomputes the logit with fp64 accumulation, where the products are
// exact and the sum is exact to 2^-53.  Every logit therefore equals the fp64 definition bit
// for bit, whatever the summation order.  fp32 models always use fp64 accumulation.
#pragma once
#include <type_traits>
#include "common.cuh"
#include "ep.cuh"
#include "permute.cuh"
#include "rmsnorm.cuh"

namespace b200moe {

constexpr int kRouterThreads = 256;       // 8 warps = 8 experts per CTA in phase 1

struct RouterParams {
  const void* x;        // [T,H]
  const void* wg;       // [E,H]
  const void* bias;     // [E] or null (model dtype)
  const void* logits_in;  // [T,E] model dtype (route_from_logits) or null
  float* logits;        // [T,E] final logits (rounded to the model dtype, bias added), as fp32
  unsigned* tile_counter;  // one per token tile, zero between calls
  int64_t* ids64;       // [T,K]
  void* scores;         // [T,K] model dtype
  unsigned long long* bitmap;  // 4 words or null
  int T, H, E, K;
  // Fused grouping: when fuse_permute is set, the CTA that finishes the LAST token tile of the grid runs
  // the token-to-expert grouping (permute_block) over the ids the grid has just written, so the permute
  // launch and its dependency edge disappear.  all_done counts finished tiles and returns to zero.
  int fuse_permute;
  unsigned* all_done;
  PermuteParams perm;
  // RMSNorm fused into the load of the tokens (NORM instances of the kernels): x is then the raw hidden state,
  // s = x (+ norm_res), the routed row is T(T(s * rsqrt(mean(s^2) + eps)) * norm_w) - the reference's
  // post_attention_layernorm (demo/src/layers/layernorm.py:21-36, call site demo/src/model/qwen3_runner.py:204).
  // The CTAs of expert group 0 write the normalised rows to normed_out (read by the expert kernels) and
  // T(s) to res_out (the residual the combine adds); either may be null.
  const void* norm_res;
  const void* norm_w;
  void* normed_out;
  void* res_out;
  float norm_eps;
  // Expert-parallel dispatch fused into the tail (ep_dispatch set): the CTA that has just routed a token tile
  // stores each of its tokens' rows into the receive region of the rank that owns the chosen expert, the CTA
  // that finishes the last tile publishes the row counts and raises the flags (the work of ep_dispatch_kernel,
  // without its launch and without its second pass over the ids).  Row positions inside a region are handed
  // out by an atomic counter per destination, so their order varies from run to run; results do not, every
  // row is computed on its own and carries its pair index.
  int ep_dispatch;
  EpGeom epg;
  unsigned* ep_epoch;
  int* ep_dest_count;
  int* ep_status;
};

constexpr int kRouterFuseSmemInts = (kRouterThreads / 32 + 1) * kMaxExperts;

// Expert-parallel tail: called by every thread of a CTA that has just finished the top-k of the tokens
// t0 .. t0+ntok-1.  Pairs are dealt to the CTA's warps; a warp copies one token row (16-byte pieces, eight in
// flight per lane) into the owner's receive region.
template <typename T>
__device__ __forceinline__ void router_dispatch_tail(const RouterParams& p, const EpPeers& peers, int t0, int ntok, unsigned n_tiles) {
  __shared__ int s_alld;
  const EpGeom& g = p.epg;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();                       // the ids of this tile's tokens have been written by this CTA's warps
  const unsigned epoch = *p.ep_epoch + 1u;
  const int npairs = ntok * g.K;
  const int npiece = g.H / 8 * ((int)sizeof(T) == 2 ? 1 : 2);
  for (int pi = warp; pi < npairs; pi += kRouterThreads / 32) {
    const int t = t0 + pi / g.K;
    const int pr = t * g.K + pi % g.K;
    const long long e = __ldcg(reinterpret_cast<const long long*>(p.ids64) + pr);
    if (e < 0 || e >= p.E) continue;
    const int d = (int)e / g.epr;
    int pos = 0;
    if (lane == 0) pos = atomicAdd(p.ep_dest_count + d, 1);
    pos = __shfl_sync(0xffffffffu, pos, 0);
    if (pos >= g.cap) { if (lane == 0) atomicOr(p.ep_status, kDevBadOffsets); continue; }
    const size_t row = (size_t)g.me * g.cap + pos;
    const unsigned char* src = reinterpret_cast<const unsigned char*>(p.x) + (size_t)t * g.H * sizeof(T);
    unsigned char* dst = peers.base[d] + g.off_x + row * (size_t)g.H * sizeof(T);
    for (int c0 = lane; c0 < npiece; c0 += 32 * 8) {
      uint4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (c0 + 32 * u < npiece) v[u] = ldg_cached(src + (size_t)(c0 + 32 * u) * 16);
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (c0 + 32 * u < npiece) *reinterpret_cast<uint4*>(dst + (size_t)(c0 + 32 * u) * 16) = v[u];
    }
    if (lane == 0) reinterpret_cast<int2*>(peers.base[d] + g.off_meta)[row] = make_int2((int)e, pr);
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(p.all_done, 1u);
    s_alld = (prev == n_tiles - 1);
    if (s_alld) *p.all_done = 0u;
  }
  __syncthreads();
  if (!s_alld) return;
  // every tile's CTA fenced its rows before it arrived; the release store orders them, and the count, ahead of the flag
  if (threadIdx.x < g.G) {
    EpHeader* h = reinterpret_cast<EpHeader*>(peers.base[threadIdx.x]);
    h->disp_count[g.me] = min(__ldcg(p.ep_dest_count + threadIdx.x), g.cap);
    st_release_sys(&h->disp_flag[g.me], epoch);
  }
  __syncthreads();
  if (threadIdx.x < kEpMaxRanks) p.ep_dest_count[threadIdx.x] = 0;
  if (threadIdx.x == 0) *p.ep_epoch = epoch;
}

// Tail shared by the router kernels: called by every thread of a CTA that has just finished the top-k of a
// token tile.  Returns after the grouping when this CTA was the last one of the grid.
__device__ __forceinline__ void router_fused_tail(const RouterParams& p, const SlotTable& st, unsigned n_tiles, int* smem) {
  __shared__ int s_all;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(p.all_done, 1u);
    s_all = (prev == n_tiles - 1);
    if (s_all) *p.all_done = 0u;
  }
  __syncthreads();
  if (!s_all) return;
  __threadfence();
  permute_block(p.perm, st, smem);
}

// kSmemX: the token row lives in shared memory (tile kernel, fused norm), else in global memory.
template <typename T, bool kSmemX = false> __device__ __forceinline__ double exact_dot(const T* xr, const T* wr, int nch, int lane) {
  double acc = 0.0;
  for (int c0 = lane; c0 < nch; c0 += 256) {
    Chunk<T> xc[8], wc[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int c = c0 + 32 * u;
      if (c < nch) {
        if (kSmemX) xc[u].from_smem(xr + c * 8); else xc[u].template load<false>(xr + c * 8);
        wc[u].template load<false>(wr + c * 8);
      }
      else { xc[u].zero(); wc[u].zero(); }
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      float xf[8], wf[8];
      xc[u].unpack(xf);
      wc[u].unpack(wf);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc = fma((double)xf[i], (double)wf[i], acc);
    }
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

// Top-k / softmax of up to TT tokens by ALL kRouterThreads threads of a CTA (it synchronises).
//
// Shaped by what this code costs where it runs - once per launch, on the critical path, with cold instruction
// caches and one or a few warps: a straight-line, unrolled one-warp version measured 13 - 24 us per call against
// 4 - 5 us for the same code once resident, and a single warp retires an instruction only every ~7 cycles.  So the
// loops are rolled, the function is not inlined, the O(E^2) part is spread over the whole CTA and the 32-slot
// network runs only for tokens that need it:
//   A  every thread copies logits into shared memory (NaN sorts first, as torch.topk has it);
//   B  one thread per (token, expert) counts the entries ahead of its own in (value descending, index ascending)
//      order - its rank; ranks below k are the kept entries, written to slot `rank` of the token's list;
//   C  warp tt finishes token tt.  With k distinct kept values the descending order IS the result (a sorting
//      network sorts any arrangement of distinct keys to the same order).  With equal values among them the
//      order of the equal ones is whatever torch's CUDA kernel makes of it: the kept entries are arranged as that
//      kernel gathers them (entries > kth in index order, then entries == kth in index order) and passed through
//      the 32-slot bitonic network it applies for 1 < k <= 32.  Then the softmax over the k kept logits.
constexpr int kTopkLogSlots = kMaxExperts + 4;
template <int TT> struct TopkSmem {
  __align__(16) float log[TT][kTopkLogSlots];
  float sel_v[TT][32];
  int sel_i[TT][32];
  float key[TT][32];
  int idx[TT][32];
};
struct TopkArgs {          // by value: passing the kernel's parameter struct by reference would put a copy on the stack
  const void* logits_in;   // [T,E] model dtype, or null
  const float* logits;     // [T,E] fp32
  int64_t* ids64;
  void* scores;
  unsigned long long* bitmap;
  int E, K;
};
__device__ __forceinline__ TopkArgs topk_args(const RouterParams& p) {
  return TopkArgs{p.logits_in, p.logits, p.ids64, p.scores, p.bitmap, p.E, p.K};
}

// ids_s / w_s (shared memory, ntok * K entries; the score as the model dtype holds it) receive a private copy of the
// routing for a caller that goes on to use it; write_global = false leaves ids / scores / bitmap untouched.
template <typename T, int TT>
__device__ __noinline__ void topk_softmax_tile(TopkArgs a, int t0, int ntok, TopkSmem<TT>* sm, int* ids_s, float* w_s, bool write_global) {
  static_assert(TT <= kRouterThreads / 32, "one warp per token in the last step");
  const int E = a.E, K = a.K;
  const int E4 = (E + 3) & ~3;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#pragma unroll 1
  for (int i = tid; i < ntok * E4; i += kRouterThreads) {
    const int tt = i / E4, e = i - tt * E4;
    float v = -INFINITY;                                  // padding up to a multiple of four never wins a comparison
    if (e < E) {
      const size_t at = (size_t)(t0 + tt) * E + e;
      v = a.logits_in != nullptr ? Elem<T>::to_float(reinterpret_cast<const T*>(a.logits_in)[at]) : __ldcg(a.logits + at);
      if (v != v) v = INFINITY;
    }
    sm->log[tt][e] = v;
  }
  __syncthreads();
#pragma unroll 1
  for (int i = tid; i < ntok * E; i += kRouterThreads) {
    const int tt = i / E, e = i - tt * E;
    const float* row = sm->log[tt];
    const float v = row[e];
    int cnt = 0;
#pragma unroll 1
    for (int o = 0; o < E4; o += 4) {
      const float4 w = *reinterpret_cast<const float4*>(row + o);
      cnt += (w.x > v || (w.x == v && o < e)) ? 1 : 0;
      cnt += (w.y > v || (w.y == v && o + 1 < e)) ? 1 : 0;
      cnt += (w.z > v || (w.z == v && o + 2 < e)) ? 1 : 0;
      cnt += (w.w > v || (w.w == v && o + 3 < e)) ? 1 : 0;
    }
    if (cnt < K) { sm->sel_v[tt][cnt] = v; sm->sel_i[tt][cnt] = e; }
  }
  __syncthreads();
  if (warp >= ntok) return;
  const int tt = warp;
  float key = (lane < K) ? sm->sel_v[tt][lane] : 0.0f;
  int idx = (lane < K) ? sm->sel_i[tt][lane] : -1;
  bool ok = lane < K;
  const float below = __shfl_down_sync(0xffffffffu, key, 1);
  if (__any_sync(0xffffffffu, lane + 1 < K && below == key)) {
    const float kth = sm->sel_v[tt][K - 1];
    if (lane < K) {
      int gt_before = 0, eq_before = 0, gt_total = 0;
#pragma unroll 1
      for (int r = 0; r < K; ++r) {
        const float w = sm->sel_v[tt][r];
        const int wi = sm->sel_i[tt][r];
        gt_total += (w > kth) ? 1 : 0;
        gt_before += (w > kth && wi < idx) ? 1 : 0;
        eq_before += (w == kth && wi < idx) ? 1 : 0;
      }
      const int pos = key > kth ? gt_before : gt_total + eq_before;
      sm->key[tt][pos] = key;
      sm->idx[tt][pos] = idx;
    }
    __syncwarp();
    if (lane < K) { key = sm->key[tt][lane]; idx = sm->idx[tt][lane]; }
    // sorting stages of size 2 .. 16 in alternating directions, then the merge of size 32 (its direction flag is clear)
#pragma unroll 1
    for (int size = 2; size <= 32; size <<= 1) {
#pragma unroll 1
      for (int stride = size >> 1; stride > 0; stride >>= 1) {
        const bool flag = ((lane & ~stride) & size) != 0;
        const float pk = __shfl_xor_sync(0xffffffffu, key, stride);
        const int pi = __shfl_xor_sync(0xffffffffu, idx, stride);
        const bool pok = __shfl_xor_sync(0xffffffffu, (int)ok, stride) != 0;
        const bool is_lo = (lane & stride) == 0;
        const float k_lo = is_lo ? key : pk, k_hi = is_lo ? pk : key;
        const bool ok_lo = is_lo ? ok : pok, ok_hi = is_lo ? pok : ok;
        const bool pred = (k_lo > k_hi && ok_lo) || !ok_hi;
        if (pred == flag) { key = pk; idx = pi; ok = pok; }
      }
    }
  }

  // softmax over the k kept logits (fp32 math, butterfly reductions over next_pow2(k) lanes)
  int width = 1;
  while (width < K) width <<= 1;
  float mx = (lane < K) ? key : -INFINITY;
#pragma unroll 1
  for (int o = width >> 1; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  const float ex = (lane < K) ? expf(key - mx) : 0.0f;
  float sum = ex;
#pragma unroll 1
  for (int o = width >> 1; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (lane < K) {
    const float sc = ex / sum;
    const size_t at = (size_t)(t0 + tt) * K + lane;
    if (write_global) {
      a.ids64[at] = idx;
      reinterpret_cast<T*>(a.scores)[at] = Elem<T>::from_float(sc);
      if (a.bitmap != nullptr) atomicOr(a.bitmap + (idx >> 6), 1ull << (idx & 63));
    }
    if (ids_s != nullptr) { ids_s[tt * K + lane] = idx; w_s[tt * K + lane] = rn<T>(sc); }
  }
}

// One warp turns the E logits of token t into ordered top-k ids and softmax scores: the same selection, placement,
// network and softmax as topk_softmax_tile, kept in registers and unrolled.  This is the form for kernels that run
// it many times per SM (token tiles of a large batch, caller-supplied logits), where the code is resident after the
// first tile and one warp per token beats the CTA-wide counting; a launch that runs it once takes the tile form.
template <typename T>
__device__ void topk_softmax_token(const RouterParams& p, int t, int lane, float* skey, int* sidx) {
  constexpr int kMaxJ = kMaxExperts / 32;
  const int E = p.E, K = p.K;
  const int nj = (E + 31) / 32;
  float v[kMaxJ];
#pragma unroll
  for (int j = 0; j < kMaxJ; ++j) {
    const int e = j * 32 + lane;
    if (j < nj && e < E) {
      v[j] = p.logits_in != nullptr ? Elem<T>::to_float(reinterpret_cast<const T*>(p.logits_in)[(size_t)t * E + e])
                                    : __ldcg(p.logits + (size_t)t * E + e);
    } else {
      v[j] = -INFINITY;
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

// grid = (ceil(T/TT), ceil(E/8)), 256 threads.  Phase 1: warp w of CTA (bx,by) computes the
// logits of expert by*8+w for the TT tokens of tile bx and certifies (or recomputes) each.
// The CTA that finishes a tile last runs phase 2 (top-k) for its tokens; the counter returns to
// zero for the next call.  TT = 1 with 8 chunk positions per trip serves small batches
// (latency-bound: every load of a row is in flight at once); TT = 4 amortises the weight row.
template <typename T, int TT, int U, bool NORM = false> __global__ void __launch_bounds__(kRouterThreads) router_kernel(RouterParams p, SlotTable st, EpPeers peers) {
  static_assert(!NORM || TT == 1, "the fused norm stages one token row per CTA");
  static_assert(kNormThreads == kRouterThreads, "rmsnorm_row is written for the router's CTA size");
  extern __shared__ __align__(16) unsigned char xrow_raw[];       // NORM: the normalised row of this CTA's token
  __shared__ float s_part[kNormThreads / 32];
  __shared__ float s_scale;
  __shared__ int s_perm[kRouterFuseSmemInts];
  constexpr bool kExact = std::is_same<T, float>::value;
  using Acc = typename std::conditional<kExact, double, float>::type;
  __shared__ TopkSmem<TT> s_topk;
  __shared__ int s_last;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t0 = blockIdx.x * TT;
  const int e = blockIdx.y * (kRouterThreads / 32) + warp;
  const int nch = p.H / 8;
  const T* x = reinterpret_cast<const T*>(p.x);
  const T* bias = reinterpret_cast<const T*>(p.bias);
  pdl_wait();        // the previous call's combine may still read the ids / scores this kernel rewrites
  pdl_trigger();
  if (NORM) {
    const size_t off = (size_t)t0 * p.H;
    const bool writer = blockIdx.y == 0;
    rmsnorm_row<T>(x + off, p.norm_res ? reinterpret_cast<const T*>(p.norm_res) + off : nullptr, reinterpret_cast<const T*>(p.norm_w), p.norm_eps, p.H,
                   reinterpret_cast<T*>(xrow_raw), (writer && p.normed_out) ? reinterpret_cast<T*>(p.normed_out) + off : nullptr,
                   (writer && p.res_out) ? reinterpret_cast<T*>(p.res_out) + off : nullptr, s_part, &s_scale);
  }

  if (e < p.E) {
    const T* wrow = reinterpret_cast<const T*>(p.wg) + (size_t)e * p.H;
    Acc acc[TT][4];
    float sabs[TT];
#pragma unroll
    for (int tt = 0; tt < TT; ++tt) {
      sabs[tt] = 0.0f;
#pragma unroll
      for (int a = 0; a < 4; ++a) acc[tt][a] = 0;
    }
    for (int c0 = lane; c0 < nch; c0 += 32 * U) {
      Chunk<T> wc[U], xc[U][TT];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int c = c0 + 32 * u;
        if (c < nch) {
          wc[u].template load<false>(wrow + c * 8);
#pragma unroll
          for (int tt = 0; tt < TT; ++tt) {
            if (NORM) xc[u][tt].from_smem(reinterpret_cast<const T*>(xrow_raw) + c * 8);
            else xc[u][tt].template load<false>(x + (size_t)min(t0 + tt, p.T - 1) * p.H + c * 8);
          }
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
            if (kExact) {
              acc[tt][i & 3] = fma((double)xf[i], (double)wf[i], acc[tt][i & 3]);
            } else {
              acc[tt][i & 3] = fmaf(xf[i], wf[i], acc[tt][i & 3]);
              sabs[tt] = fmaf(fabsf(xf[i]), fabsf(wf[i]), sabs[tt]);
            }
          }
        }
      }
    }
    const float cH = (float)(p.H / 128 + 12) * 5.9604645e-8f * 1.01f;
#pragma unroll
    for (int tt = 0; tt < TT; ++tt) {
      const Acc part = (acc[tt][0] + acc[tt][1]) + (acc[tt][2] + acc[tt][3]);
      float s = (float)warp_sum(part);
      if (!kExact) {
        const float bound = cH * warp_sum(sabs[tt]) + 1e-37f;
        const bool risky = !(boundary_distance<T>(s) > bound);    // uniform: every lane holds the same sums
        if (risky && t0 + tt < p.T)
          s = (float)exact_dot<T, NORM>(NORM ? reinterpret_cast<const T*>(xrow_raw) : x + (size_t)(t0 + tt) * p.H, wrow, nch, lane);
      }
      float l = rn<T>(s);
      if (bias != nullptr) l = rn<T>(l + Elem<T>::to_float(bias[e]));
      if (lane == 0 && t0 + tt < p.T) p.logits[(size_t)(t0 + tt) * p.E + e] = l;
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
  topk_softmax_tile<T, TT>(topk_args(p), t0, min(TT, p.T - t0), &s_topk, nullptr, nullptr, true);
  if (p.fuse_permute) router_fused_tail(p, st, gridDim.x, s_perm);
  if (p.ep_dispatch) router_dispatch_tail<T>(p, peers, t0, min(TT, p.T - t0), gridDim.x);
}

// Larger batches (T > 16): a CTA owns a tile of TT tokens x (8 * EPW) experts.  The token tile is staged
// ONCE in shared memory and shared by the eight warps (letting every warp fetch its tokens from L2 again
// made the kernel L2-bound); a warp streams EPW expert rows against all the tile's tokens.  Same
// certificate as above with two accumulators per lane and (token, expert): each sees at most H/64 + 1
// roundings, then 1 + 5 for the pair and the warp tree.  Small tiles (4 tokens x 8 experts) keep a CTA's
// serial chain short - a warp reduces TT * EPW sums one after the other - and give the grid enough CTAs.
constexpr int kTileTokens = 4;
template <typename T, int TT, int EPW, bool NORM = false> __global__ void __launch_bounds__(kRouterThreads) router_tile_kernel(RouterParams p, SlotTable st, EpPeers peers) {
  __shared__ float s_part[kNormThreads / 32];
  __shared__ float s_scale;
  constexpr bool kExact = std::is_same<T, float>::value;
  using Acc = typename std::conditional<kExact, double, float>::type;
  static_assert(TT <= kRouterThreads / 32, "one warp per token in the top-k phase");
  extern __shared__ __align__(16) unsigned char tile_raw[];     // [TT][H] tokens of this tile
  __shared__ float skey[TT][32];
  __shared__ int sidx[TT][32];
  __shared__ int s_last;
  __shared__ int s_perm[kRouterFuseSmemInts];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t0 = blockIdx.x * TT;
  const int e0 = (blockIdx.y * (kRouterThreads / 32) + warp) * EPW;
  const int nch = p.H / 8;
  constexpr int CB = 8 * (int)sizeof(T);
  const T* x = reinterpret_cast<const T*>(p.x);
  const T* bias = reinterpret_cast<const T*>(p.bias);
  pdl_wait();        // the previous call's combine may still read the ids / scores this kernel rewrites
  pdl_trigger();
  if (NORM) {
    const bool writer = blockIdx.y == 0;
    for (int tt = 0; tt < TT; ++tt) {
      const int t = min(t0 + tt, p.T - 1);
      const size_t off = (size_t)t * p.H;
      const bool wr = writer && t0 + tt < p.T;
      rmsnorm_row<T>(x + off, p.norm_res ? reinterpret_cast<const T*>(p.norm_res) + off : nullptr, reinterpret_cast<const T*>(p.norm_w), p.norm_eps, p.H,
                     reinterpret_cast<T*>(tile_raw) + (size_t)tt * p.H, (wr && p.normed_out) ? reinterpret_cast<T*>(p.normed_out) + off : nullptr,
                     (wr && p.res_out) ? reinterpret_cast<T*>(p.res_out) + off : nullptr, s_part, &s_scale);
    }
  } else {
    constexpr int US = 4;                  // staging loads in flight per thread
    for (int i0 = threadIdx.x; i0 < TT * nch; i0 += kRouterThreads * US) {
      Chunk<T> xc[US];
#pragma unroll
      for (int u = 0; u < US; ++u) {
        const int i = i0 + u * kRouterThreads;
        if (i < TT * nch) {
          const int tt = i / nch, c = i - tt * nch;
          xc[u].template load<false>(x + (size_t)min(t0 + tt, p.T - 1) * p.H + c * 8);
        }
      }
#pragma unroll
      for (int u = 0; u < US; ++u) {
        const int i = i0 + u * kRouterThreads;
        if (i < TT * nch) {
          if (sizeof(T) == 2) *reinterpret_cast<uint4*>(tile_raw + (size_t)i * CB) = *reinterpret_cast<const uint4*>(&xc[u]);
          else { reinterpret_cast<uint4*>(tile_raw + (size_t)i * CB)[0] = reinterpret_cast<const uint4*>(&xc[u])[0]; reinterpret_cast<uint4*>(tile_raw + (size_t)i * CB)[1] = reinterpret_cast<const uint4*>(&xc[u])[1]; }
        }
      }
    }
  }
  __syncthreads();

  if (e0 < p.E) {
    const T* wrow[EPW];
#pragma unroll
    for (int ee = 0; ee < EPW; ++ee) wrow[ee] = reinterpret_cast<const T*>(p.wg) + (size_t)min(e0 + ee, p.E - 1) * p.H;
    Acc acc[TT][EPW][2];
    float sabs[TT][EPW];
#pragma unroll
    for (int tt = 0; tt < TT; ++tt)
#pragma unroll
      for (int ee = 0; ee < EPW; ++ee) { acc[tt][ee][0] = 0; acc[tt][ee][1] = 0; sabs[tt][ee] = 0.0f; }
    constexpr int UW = 4;                  // chunk positions per trip: their weight loads are all in flight before the first is used
    for (int c0 = lane; c0 < nch; c0 += 32 * UW) {
      Chunk<T> wc[UW][EPW];
#pragma unroll
      for (int u = 0; u < UW; ++u)
#pragma unroll
        for (int ee = 0; ee < EPW; ++ee) {
          if (c0 + 32 * u < nch) wc[u][ee].template load<false>(wrow[ee] + (c0 + 32 * u) * 8);
          else wc[u][ee].zero();
        }
#pragma unroll
      for (int u = 0; u < UW; ++u) {
        const int c = c0 + 32 * u;
        if (c >= nch) break;
        float wf[EPW][8];
#pragma unroll
        for (int ee = 0; ee < EPW; ++ee) wc[u][ee].unpack(wf[ee]);
#pragma unroll
        for (int tt = 0; tt < TT; ++tt) {
          Chunk<T> xc;
          xc.from_smem(tile_raw + ((size_t)tt * nch + c) * CB);
          float xf[8];
          xc.unpack(xf);
#pragma unroll
          for (int ee = 0; ee < EPW; ++ee)
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              if (kExact) {
                acc[tt][ee][i & 1] = fma((double)xf[i], (double)wf[ee][i], acc[tt][ee][i & 1]);
              } else {
                acc[tt][ee][i & 1] = fmaf(xf[i], wf[ee][i], acc[tt][ee][i & 1]);
                sabs[tt][ee] = fmaf(fabsf(xf[i]), fabsf(wf[ee][i]), sabs[tt][ee]);
              }
            }
        }
      }
    }
    const float cH = (float)(p.H / 64 + 12) * 5.9604645e-8f * 1.01f;
#pragma unroll
    for (int tt = 0; tt < TT; ++tt)
#pragma unroll
      for (int ee = 0; ee < EPW; ++ee) {
        float s = (float)warp_sum(acc[tt][ee][0] + acc[tt][ee][1]);
        const bool live = t0 + tt < p.T && e0 + ee < p.E;
        if (!kExact) {
          const float bound = cH * warp_sum(sabs[tt][ee]) + 1e-37f;
          const bool risky = !(boundary_distance<T>(s) > bound);    // uniform: every lane holds the same sums
          if (risky && live) s = (float)exact_dot<T, true>(reinterpret_cast<const T*>(tile_raw) + (size_t)tt * p.H, wrow[ee], nch, lane);
        }
        float l = rn<T>(s);
        if (bias != nullptr && live) l = rn<T>(l + Elem<T>::to_float(bias[e0 + ee]));
        if (lane == 0 && live) p.logits[(size_t)(t0 + tt) * p.E + e0 + ee] = l;
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
  if (p.fuse_permute) router_fused_tail(p, st, gridDim.x, s_perm);
  if (p.ep_dispatch) router_dispatch_tail<T>(p, peers, t0, min(TT, p.T - t0), gridDim.x);
}

// Top-k / softmax on caller-supplied logits: one warp per token.
template <typename T> __global__ void __launch_bounds__(kRouterThreads) router_from_logits_kernel(RouterParams p) {
  __shared__ float skey[kRouterThreads / 32][32];
  __shared__ int sidx[kRouterThreads / 32][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (kRouterThreads / 32) + warp;
  pdl_wait();
  pdl_trigger();
  if (t < p.T) topk_softmax_token<T>(p, t, lane, skey[warp], sidx[warp]);
}

}  // namespace b200moe
