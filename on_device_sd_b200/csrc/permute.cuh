// K2 - token-to-expert permute / histogram.  Replaces the per-expert
// `torch.where(topk_indices == e)` grouping of Qwen3ModelRunner._execute_moe_with_placement
// (demo/src/model/qwen3_runner.py:303-314 of the reference) with one stable counting sort:
// inside an expert, (token, slot) pairs keep row-major order, which is the order torch.where
// returns them in.
#pragma once
#include "common.cuh"

namespace b200moe {

// Per-call tables passed BY VALUE (kernel parameter space), so that no host buffer has to
// outlive the enqueue: slot[e] = registered expert whose weights serve tokens routed to e
// (-1 = skip), rank[e] = position of e in the accumulation order of the combine step.
struct SlotTable {
  int16_t slot[kMaxExperts];
  uint8_t rank[kMaxExperts];
};

struct PermuteParams {
  const int64_t* ids64;  // [T,K]
  int T, K, E;
  int* offsets;      // [E+1] exclusive prefix of per-expert pair counts
  int* sorted_pair;  // [T*K] pair index (t*K+k) at each sorted position
  int* inv;          // [T*K] sorted position of each pair, -1 for an invalid id
  int* act_list;     // [E] experts that have work (count > 0 and a usable slot), ascending
  int* n_act;        // [1]
  int* status;
  // Expert-parallel source (ep_meta != null): the "pairs" are the rows of this rank's receive buffer,
  // [ep_G][ep_cap] with K = 1; row j of source s holds expert ep_meta[s*cap+j].x when j < ep_count[s], the
  // rest of a region is not visited (its inv entries keep whatever they held).  The kernel first waits
  // (bounded) until every source's dispatch flag has reached *ep_epoch.
  const int2* ep_meta;
  const int* ep_count;
  const unsigned* ep_flags;
  const unsigned* ep_epoch;
  int ep_G, ep_cap;
  long long ep_wait_cycles;
};

constexpr int kPermuteMaxThreads = 1024;

// exclusive prefix sum over the first 256 threads of the block (E <= 256); `warp_tot` has 8 slots
__device__ __forceinline__ int block_exclusive_scan_256(int v, int* warp_tot, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  if (warp < 8 && lane == 31) warp_tot[warp] = inc;
  __syncthreads();
  int base = 0;
  if (warp < 8) {
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const int t = warp_tot[w];
      if (w < warp) base += t;
    }
  }
  if (total != nullptr) {
    int tt = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) tt += warp_tot[w];
    *total = tt;
  }
  __syncthreads();
  return base + inc - v;
}

// The whole grouping, executed by ONE CTA of 256..1024 threads (a multiple of 32, at least 256 so that
// every expert has a thread).  `smem` holds (blockDim/32 + 1) * E ints.  Called by permute_kernel and by
// the tail of the router kernels (the CTA that finishes the last token tile groups the batch it just routed).
__device__ __forceinline__ void permute_block(const PermuteParams& p, const SlotTable& st, int* smem) {
  const int nwarps = blockDim.x >> 5;
  int* cnt = smem;                  // [nwarps][E]
  int* offs = smem + nwarps * p.E;  // [E]
  __shared__ int warp_tot[8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int E = p.E;
  for (int i = threadIdx.x; i < nwarps * E; i += blockDim.x) cnt[i] = 0;
  // Expert-parallel source: only the rows the sources really sent are visited.  ep_start[s] is the number of
  // rows of the sources before s; visit index i in [ep_start[s], ep_start[s+1]) is row s*cap + (i - ep_start[s]).
  __shared__ int ep_start[9];
  if (p.ep_meta != nullptr) {
    if (threadIdx.x < p.ep_G) {
      const bool ok = ep_wait_flag(p.ep_flags + threadIdx.x, *p.ep_epoch, p.ep_wait_cycles);
      if (!ok) atomicOr(p.status, kDevWaitExpired);
      ep_start[threadIdx.x + 1] = ok ? max(0, min(__ldcg(p.ep_count + threadIdx.x), p.ep_cap)) : 0;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      ep_start[0] = 0;
      for (int s = 0; s < p.ep_G; ++s) ep_start[s + 1] += ep_start[s];
    }
  }
  __syncthreads();
  const int npairs = p.ep_meta != nullptr ? ep_start[p.ep_G] : p.T * p.K;     // pairs to visit
  // contiguous, 32-aligned slice of the visit list per warp
  const int per_warp = ((npairs + nwarps - 1) / nwarps + 31) / 32 * 32;
  const int begin = warp * per_warp, end = min(begin + per_warp, npairs);
  // visit index -> pair index (row of the receive buffer in expert-parallel mode)
  auto pair_of = [&](int i) -> int {
    if (p.ep_meta == nullptr) return i;
    int s = 0;
#pragma unroll
    for (int k = 1; k < 8; ++k) s += (k < p.ep_G && i >= ep_start[k]) ? 1 : 0;
    return s * p.ep_cap + (i - ep_start[s]);
  };
  // id of pair pr: anything outside [0,E) is reported (or dropped quietly for a caller that only wants the tables)
  auto load_id = [&](int pr) -> long long {
    if (p.ep_meta == nullptr) return __ldcg(reinterpret_cast<const long long*>(p.ids64) + pr);   // L2: another CTA of this grid may have written it
    const int e = __ldcg(&p.ep_meta[pr]).x;
    return (e < 0) ? -2 : e;
  };
  const bool quiet = p.ep_meta == nullptr && p.ep_cap < 0;

  for (int b = begin; b < end; b += 32) {
    const int vi = b + lane;
    if (vi < end) {
      const long long e = load_id(pair_of(vi));
      if (e >= 0 && e < E) atomicAdd(&cnt[warp * E + (int)e], 1);
      else if (!quiet) atomicOr(p.status, kDevBadExpertId);
    }
  }
  __syncthreads();

  int tot = 0;
  if (threadIdx.x < E) {
    for (int w = 0; w < nwarps; ++w) {
      const int c = cnt[w * E + threadIdx.x];
      cnt[w * E + threadIdx.x] = tot;
      tot += c;
    }
  }
  int grand = 0;
  const int my_off = block_exclusive_scan_256(threadIdx.x < E ? tot : 0, warp_tot, &grand);
  const bool active = threadIdx.x < E && tot > 0 && st.slot[threadIdx.x] >= 0;
  int n_active = 0;
  const int my_rank = block_exclusive_scan_256(active ? 1 : 0, warp_tot, &n_active);
  if (threadIdx.x < E) {
    offs[threadIdx.x] = my_off;
    p.offsets[threadIdx.x] = my_off;
    if (active) p.act_list[my_rank] = threadIdx.x;
  }
  if (threadIdx.x == 0) {
    p.offsets[E] = grand;
    *p.n_act = n_active;
  }
  __syncthreads();

  const int cap_pairs = p.T * p.K;      // size of the tables
  for (int b = begin; b < end; b += 32) {
    const int vi = b + lane;
    int pr = -1;
    long long e = -1;
    if (vi < end) {
      pr = pair_of(vi);
      e = load_id(pr);
      if (e < 0 || e >= E) e = -1;
    }
    const unsigned m = __match_any_sync(0xffffffffu, (int)e);
    const int rank = __popc(m & ((1u << lane) - 1u));
    int pos = -1;
    if (e >= 0) pos = offs[e] + cnt[warp * E + (int)e] + rank;
    __syncwarp();
    if (e >= 0 && rank == 0) cnt[warp * E + (int)e] += __popc(m);
    __syncwarp();
    if (vi < end) {
      p.inv[pr] = pos;
      if (pos >= 0) {
        if (pos < cap_pairs) p.sorted_pair[pos] = pr;
        else atomicOr(p.status, kDevBadOffsets);
      }
    }
  }
}

static __global__ void __launch_bounds__(kPermuteMaxThreads) permute_kernel(PermuteParams p, SlotTable st) {
  extern __shared__ int smem[];
  pdl_wait();        // ids come from the router launched just before
  pdl_trigger();
  permute_block(p, st, smem);
}

}  // namespace b200moe
