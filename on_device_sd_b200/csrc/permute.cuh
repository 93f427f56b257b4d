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
};

constexpr int kPermuteThreads = 1024;
constexpr int kPermuteWarps = kPermuteThreads / 32;

__global__ void __launch_bounds__(kPermuteThreads) permute_kernel(PermuteParams p, SlotTable st) {
  extern __shared__ int smem[];
  int* cnt = smem;                       // [warps][E]
  int* tot = smem + kPermuteWarps * p.E; // [E]
  int* offs = tot + p.E;                 // [E+1]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int E = p.E, npairs = p.T * p.K;
  // contiguous, 32-aligned slice of the pair list per warp
  const int per_warp = ((npairs + kPermuteWarps - 1) / kPermuteWarps + 31) / 32 * 32;
  const int begin = warp * per_warp, end = min(begin + per_warp, npairs);

  for (int i = threadIdx.x; i < kPermuteWarps * E; i += kPermuteThreads) cnt[i] = 0;
  __syncthreads();

  for (int b = begin; b < end; b += 32) {
    const int pr = b + lane;
    if (pr < end) {
      const long long e = p.ids64[pr];
      if (e >= 0 && e < E) atomicAdd(&cnt[warp * E + (int)e], 1);
      else atomicOr(p.status, kDevBadExpertId);
    }
  }
  __syncthreads();

  if (threadIdx.x < E) {
    int run = 0;
    for (int w = 0; w < kPermuteWarps; ++w) {
      const int c = cnt[w * E + threadIdx.x];
      cnt[w * E + threadIdx.x] = run;
      run += c;
    }
    tot[threadIdx.x] = run;
  }
  __syncthreads();
  if (threadIdx.x <= E) {
    int s = 0;
    for (int e = 0; e < (int)threadIdx.x; ++e) s += tot[e];
    offs[threadIdx.x] = s;
    p.offsets[threadIdx.x] = s;
  }
  if (threadIdx.x == kPermuteThreads - 1) {
    int n = 0;
    for (int e = 0; e < E; ++e)
      if (tot[e] > 0 && st.slot[e] >= 0) p.act_list[n++] = e;
    *p.n_act = n;
  }
  __syncthreads();

  for (int b = begin; b < end; b += 32) {
    const int pr = b + lane;
    long long e = -1;
    if (pr < end) {
      e = p.ids64[pr];
      if (e < 0 || e >= E) e = -1;
    }
    const unsigned m = __match_any_sync(0xffffffffu, (int)e);
    const int rank = __popc(m & ((1u << lane) - 1u));
    int pos = -1;
    if (e >= 0) pos = offs[e] + cnt[warp * E + (int)e] + rank;
    __syncwarp();
    if (e >= 0 && rank == 0) cnt[warp * E + (int)e] += __popc(m);
    __syncwarp();
    if (pr < end) {
      p.inv[pr] = pos;
      if (pos >= 0) {
        if (pos < npairs) p.sorted_pair[pos] = pr;
        else atomicOr(p.status, kDevBadOffsets);
      }
    }
  }
}

}  // namespace b200moe
