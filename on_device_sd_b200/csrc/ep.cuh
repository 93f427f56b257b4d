// Expert-parallel dispatch and return over NVLink peer memory (no counterpart in the reference,
// which runs on one GPU; "expert distribution across GPUs" is future work there, demo/others.md:58-62).
//
// Rank r owns experts [r*E/G, (r+1)*E/G).  Every rank holds one "exchange buffer" of identical
// layout that its peers can write (mapped through CUDA IPC handles, or plain pointers inside one process):
//
//   header     disp_flag[G]   epoch of the latest dispatch by source rank s   (written by s)
//              disp_count[G]  rows that source rank s sent in that dispatch   (written by s)
//              ret_flag[G]    epoch of the latest return by owner rank o      (written by o)
//   recv_meta  int2 [G][cap]  (expert id, pair index t_local*K+k on the source) of every received row
//   recv_x     T    [G][cap][H]   the token row of every received (token, expert) pair, one region per source
//   ret_y      T    [cap][H]      expert outputs of this rank's own pairs, in pair order, written by the owners
//
// One layer forward on every rank:
//   route (local tokens) -> ep_dispatch_kernel: each pair's token row goes straight into the owner's
//   recv_x region for this source, then count + flag -> permute (waits for all G flags, groups the received
//   rows by expert) -> expert FFN over the LOCAL receive buffer -> ep_return_kernel: each output row goes
//   straight into its source's ret_y, then flag -> combine on the source (waits for all G flags).
//
// Only plain st.global / ld.global touch peer memory: no TMA, no bulk copy, no multicast, no library
// kernel ever sees a peer address.  Flags are epochs (one per layer call, kept on the device so a call
// sequence can be replayed), written with st.release.sys after a system-scope fence and polled with
// ld.acquire.sys; every poll loop gives up after a cycle budget, sets B200MOE_DEV_WAIT_EXPIRED and
// lets the kernel finish, so nothing can hang.  A rank starts the dispatch of call n+1 only after it
// has seen every owner's return flag of call n, and an owner raises that flag after its expert
// kernels are done with the receive buffer, so one buffer set is enough (no double buffering).
#pragma once
#include "common.cuh"
#include "permute.cuh"

namespace b200moe {

constexpr int kEpMaxRanks = 8;
constexpr int kEpHeaderBytes = 256;
constexpr int kEpThreads = 256;
constexpr int kEpPairsPerCta = 4;

struct EpHeader {
  unsigned disp_flag[kEpMaxRanks];
  int disp_count[kEpMaxRanks];
  unsigned ret_flag[kEpMaxRanks];
};
static_assert(sizeof(EpHeader) <= kEpHeaderBytes, "header");

struct EpPeers { unsigned char* base[kEpMaxRanks]; };   // exchange buffer of every rank as addressed from this GPU

struct EpGeom {
  int G, me, cap, H, K, epr;                 // ranks, this rank, rows per (destination, source) region, hidden, top-k, experts per rank
  unsigned long long off_meta, off_x, off_ret;
};

struct EpDispatchParams {
  const void* x;          // [T_local, H]
  const int64_t* ids;     // [T_local, K] from the router
  int T_local, E;
  EpGeom g;
  unsigned* epoch;        // this rank's call counter (device)
  unsigned* done;         // CTA arrival counter, zero between launches
  int* dest_count;        // [kEpMaxRanks] rows sent to each rank in this call, zero between launches
  int* status;
};

// grid = ceil(pairs / kEpPairsPerCta) (at least 1).  Pair p = t*K+k goes to rank d = ids[p] / epr, row
// "number of earlier pairs with the same destination" of region [d][me]: every source fills its region
// densely and in pair order, so the layout does not depend on timing.  Written for latency: every
// dependent step is one round of loads that are all in flight together.
template <typename T> __global__ void __launch_bounds__(kEpThreads) ep_dispatch_kernel(EpDispatchParams p, EpPeers peers) {
  static_assert(kEpPairsPerCta == 4, "the row copy below is unrolled for four pairs");
  __shared__ int s_cnt[kEpMaxRanks];
  __shared__ int s_dst[kEpPairsPerCta], s_pos[kEpPairsPerCta];
  __shared__ int s_last;
  const EpGeom& g = p.g;
  const int npairs = p.T_local * g.K;
  const int p0 = blockIdx.x * kEpPairsPerCta;
  if (threadIdx.x < kEpMaxRanks) s_cnt[threadIdx.x] = 0;
  pdl_wait();        // ids come from the router launched just before; the previous call's combine is complete too
  pdl_trigger();
  const unsigned epoch = *p.epoch + 1u;      // read early: only the last CTA uses it, and nobody writes it before every CTA has arrived
  __syncthreads();
  // this CTA's own pairs (lanes 0..3 of warp 0) and the destinations of all earlier pairs, in one round of loads
  long long my_e = -1;
  if (threadIdx.x < kEpPairsPerCta && p0 + (int)threadIdx.x < npairs) my_e = p.ids[p0 + threadIdx.x];
  for (int i = threadIdx.x; i < min(p0, npairs); i += kEpThreads) {
    const long long e = p.ids[i];
    if (e >= 0 && e < p.E) atomicAdd(&s_cnt[(int)e / g.epr], 1);
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    const bool mine = threadIdx.x < kEpPairsPerCta && p0 + (int)threadIdx.x < npairs;
    const bool valid = mine && my_e >= 0 && my_e < p.E;
    if (mine && !valid) atomicOr(p.status, kDevBadExpertId);
    const int d = valid ? (int)my_e / g.epr : -1;
    int before = 0;                               // earlier pairs of this CTA with the same destination
#pragma unroll
    for (int j = 0; j < kEpPairsPerCta; ++j) {
      const int dj = __shfl_sync(0xffffffffu, d, j);
      if (j < (int)threadIdx.x && dj == d) ++before;
    }
    if (threadIdx.x < kEpPairsPerCta) {
      s_dst[threadIdx.x] = d;
      s_pos[threadIdx.x] = valid ? s_cnt[d] + before : 0;
      if (valid) {
        atomicAdd(p.dest_count + d, 1);
        const size_t row = (size_t)g.me * g.cap + s_pos[threadIdx.x];
        if (s_pos[threadIdx.x] < g.cap) reinterpret_cast<int2*>(peers.base[d] + g.off_meta)[row] = make_int2((int)my_e, p0 + (int)threadIdx.x);
      }
    }
  }
  __syncthreads();
  const int nch = g.H / 8;
  constexpr int CB = 8 * (int)sizeof(T);
  constexpr int V = (int)sizeof(T) == 2 ? 1 : 2;    // 16-byte pieces per chunk
  const unsigned char* xb = reinterpret_cast<const unsigned char*>(p.x);
  for (int c = threadIdx.x; c < nch * V; c += kEpThreads) {
    uint4 v[kEpPairsPerCta];
#pragma unroll
    for (int i = 0; i < kEpPairsPerCta; ++i)      // the four rows' loads are in flight together
      if (s_dst[i] >= 0) v[i] = ldg_cached(xb + (size_t)((p0 + i) / g.K) * g.H * sizeof(T) + (size_t)c * 16);
#pragma unroll
    for (int i = 0; i < kEpPairsPerCta; ++i) {
      const int d = s_dst[i];
      if (d >= 0 && s_pos[i] < g.cap) {
        const size_t row = (size_t)g.me * g.cap + s_pos[i];
        *reinterpret_cast<uint4*>(peers.base[d] + g.off_x + row * (size_t)g.H * sizeof(T) + (size_t)c * 16) = v[i];
      }
    }
  }
  (void)CB;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(p.done, 1u) == gridDim.x - 1);
  __syncthreads();
  if (!s_last) return;
  // Last CTA: every CTA fenced its rows at system scope before it arrived on `done`, and this CTA has observed
  // all arrivals; the release store below (a system-scope fence followed by the store) therefore orders all of
  // them, and the count written just before it by the same thread, ahead of the flag.
  if (threadIdx.x < g.G) {
    EpHeader* h = reinterpret_cast<EpHeader*>(peers.base[threadIdx.x]);
    h->disp_count[g.me] = min(__ldcg(p.dest_count + threadIdx.x), g.cap);
    st_release_sys(&h->disp_flag[g.me], epoch);
  }
  __syncthreads();
  if (threadIdx.x < kEpMaxRanks) p.dest_count[threadIdx.x] = 0;
  if (threadIdx.x == 0) { *p.epoch = epoch; *p.done = 0u; }
}

struct EpReturnParams {
  const void* y;            // [rows, H] expert outputs in sorted order
  const int* offsets;       // [E+1]
  const int* sorted_pair;   // sorted position -> row of the receive buffer (s*cap + j)
  int E;
  EpGeom g;
  const unsigned* epoch;
  unsigned* done;
  int* status;
};

constexpr int kEpRowsPerTrip = 4;

// A CTA returns kEpRowsPerTrip sorted rows per trip (grid-stride).  Rows of experts this rank does not serve are
// returned as zeros, so that every pair row of every source is rewritten in every call.  One thread per row
// resolves the table entry and the metadata; the copy then keeps the rows' loads in flight together; the
// system-scope fence is paid once per CTA, not once per row.
template <typename T> __global__ void __launch_bounds__(kEpThreads) ep_return_kernel(EpReturnParams p, EpPeers peers, SlotTable st) {
  static_assert(kEpRowsPerTrip == 4, "the copy below is unrolled for four rows");
  __shared__ int s_last;
  __shared__ int s_src[kEpRowsPerTrip], s_pair[kEpRowsPerTrip], s_served[kEpRowsPerTrip];
  const EpGeom& g = p.g;
  pdl_wait();        // y comes from the down projection launched just before
  pdl_trigger();
  const unsigned epoch = *p.epoch;
  const int2* meta = reinterpret_cast<const int2*>(peers.base[g.me] + g.off_meta);
  const int nrows = g.G * g.cap;
  const int total = min(__ldcg(p.offsets + p.E), nrows);
  const int npiece = g.H / 8 * ((int)sizeof(T) == 2 ? 1 : 2);
  const size_t row_bytes = (size_t)g.H * sizeof(T);
  const unsigned char* yb = reinterpret_cast<const unsigned char*>(p.y);
  for (int base = blockIdx.x * kEpRowsPerTrip; base < total; base += gridDim.x * kEpRowsPerTrip) {
    if (threadIdx.x < kEpRowsPerTrip) {
      int src = -1, pair = 0, served = 0;
      const int pos = base + threadIdx.x;
      if (pos < total) {
        const int row = __ldcg(p.sorted_pair + pos);
        if (row >= 0 && row < nrows) {
          const int2 m = __ldcg(meta + row);
          if (m.y >= 0 && m.y < g.cap) {
            src = row / g.cap; pair = m.y;
            served = (m.x >= 0 && m.x < p.E && st.slot[m.x] >= 0) ? 1 : 0;
          }
        }
        if (src < 0) atomicOr(p.status, kDevBadOffsets);
      }
      s_src[threadIdx.x] = src; s_pair[threadIdx.x] = pair; s_served[threadIdx.x] = served;
    }
    __syncthreads();
    for (int c = threadIdx.x; c < npiece; c += kEpThreads) {
      uint4 v[kEpRowsPerTrip];
#pragma unroll
      for (int i = 0; i < kEpRowsPerTrip; ++i) {
        v[i] = make_uint4(0, 0, 0, 0);
        if (s_src[i] >= 0 && s_served[i]) v[i] = ld_cg16(yb + (size_t)(base + i) * row_bytes + (size_t)c * 16);
      }
#pragma unroll
      for (int i = 0; i < kEpRowsPerTrip; ++i)
        if (s_src[i] >= 0) *reinterpret_cast<uint4*>(peers.base[s_src[i]] + g.off_ret + (size_t)s_pair[i] * row_bytes + (size_t)c * 16) = v[i];
    }
    __syncthreads();
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(p.done, 1u) == gridDim.x - 1);
  __syncthreads();
  if (!s_last) return;
  if (threadIdx.x < g.G) st_release_sys(&reinterpret_cast<EpHeader*>(peers.base[threadIdx.x])->ret_flag[g.me], epoch);   // see ep_dispatch_kernel
  if (threadIdx.x == 0) *p.done = 0u;
}

}  // namespace b200moe
