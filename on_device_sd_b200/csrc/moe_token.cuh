// The whole MoE block of ONE token in one cooperative launch: gate logits, top-k / softmax, gate/up projection
// with SwiGLU, down projection and the weighted combine.  Replaces, for a single-token batch (the draft step of
// the reference's speculative decoder), Qwen3MoEGate.forward (demo/src/layers/moe_layer.py:25-60),
// expert_forward_with_weights per chosen expert (demo/src/layers/mlp.py:209-231) and the accumulation of
// _execute_moe_with_placement (demo/src/model/qwen3_runner.py:352-383) - the same arithmetic and the same
// rounding points as the router, GEMV and combine kernels, which stay the path of every other batch size.
//
// Why one launch: a single token moves K experts' weights once (76 MB on the Qwen3-shaped layer, 11.6 us at the
// measured copy rate) and a chain of four dependent kernels spends more than that on its hand-overs.  Here one
// persistent CTA per SM keeps per-warp rings of 1-D bulk copies (the GEMV kernel's scheme) running ACROSS the
// phases: weights do not depend on activations, so while a warp waits at the grid barrier for h to be complete
// its first down-projection rows are already on their way into shared memory.  The down projection's unit is a
// pair of output rows over ALL chosen experts, so the warp that computed a row's K products also runs the combine
// for it and no third hand-over is needed.  The two grid barriers (logits complete, h complete) are counters in
// global memory with a bounded wait; the launch is cooperative, so every CTA is resident and they cannot starve.
#pragma once
#include "common.cuh"
#include "ffn_gemv.cuh"
#include "permute.cuh"
#include "router.cuh"
#include "tma.cuh"

namespace b200moe {

struct TokenParams {
  RouterParams r;              // x, wg, bias, logits, ids64, scores, H, E, K (T = 1); r.perm = tables of the grouping
  const ExpertPtrs* experts;   // table of this layer, [E]
  void* h;                     // [K][I] silu(gate) * up, one row per live slot of the token
  const void* residual;        // [H] or null (with the fused norm: r.res_out)
  void* out;                   // [H]
  int I;
  unsigned* gbar;              // grid barrier word: bit 31 flips once per barrier, the low bits return to zero
  int* status;
  long long wait_cycles;
};

__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Barrier over all CTAs of a cooperative grid.  CTA 0 adds 2^31 - (n - 1), every other CTA adds 1: after the n-th
// arrival bit 31 has flipped and the low bits are back where they were, so the word needs no reset between
// barriers or launches.  Returns false (for every thread of the CTA) when the wait ran out.
__device__ __forceinline__ bool grid_barrier_bounded(unsigned* bar, long long limit, int* s_flag, int* status) {
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned inc = blockIdx.x == 0 ? (0x80000000u - (gridDim.x - 1u)) : 1u;
    __threadfence();
    const unsigned old = atomicAdd(bar, inc);
    bool ok = true;
    const long long t0 = clock64();
    while (((ld_acquire_gpu(bar) ^ old) & 0x80000000u) == 0u) {
      if (clock64() - t0 > limit) { ok = false; break; }
    }
    __threadfence();
    if (!ok) atomicOr(status, kDevWaitExpired);
    *s_flag = ok ? 1 : 0;
  }
  __syncthreads();
  return *s_flag != 0;
}


// One warp: the gate logit of expert row `wrow` for the token row `xr` (shared memory), with router_kernel's
// certificate - four fp32 accumulators per lane, eight chunk positions per trip, sum|x w| beside them; a result
// closer to a rounding boundary of T than the bound on the fp32 summation error is recomputed with fp64
// accumulation.  Returns the logit rounded to T (bias added in T), the same value in every lane.
template <typename T>
__device__ __forceinline__ float token_gate_logit(const unsigned char* xr, const T* wrow, const T* bias, int e, int H, int lane) {
  constexpr int CB = 8 * (int)sizeof(T);
  const int nch = H / 8;
  float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  float sabs = 0.0f;
  for (int c0 = lane; c0 < nch; c0 += 32 * 8) {
    Chunk<T> wc[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (c0 + 32 * u < nch) wc[u].template load<false>(wrow + (size_t)(c0 + 32 * u) * 8);
      else wc[u].zero();
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (c0 + 32 * u >= nch) break;
      Chunk<T> xc;
      xc.from_smem(xr + (size_t)(c0 + 32 * u) * CB);
      float wf[8], xf[8];
      wc[u].unpack(wf);
      xc.unpack(xf);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        acc[i & 3] = fmaf(xf[i], wf[i], acc[i & 3]);
        sabs = fmaf(fabsf(xf[i]), fabsf(wf[i]), sabs);
      }
    }
  }
  const float cH = (float)(H / 128 + 12) * 5.9604645e-8f * 1.01f;
  float s = warp_sum((acc[0] + acc[1]) + (acc[2] + acc[3]));
  const float bound = cH * warp_sum(sabs) + 1e-37f;
  if (!(boundary_distance<T>(s) > bound)) s = (float)exact_dot<T, true>(reinterpret_cast<const T*>(xr), wrow, nch, lane);
  float l = rn<T>(s);
  if (bias != nullptr) l = rn<T>(l + Elem<T>::to_float(bias[e]));
  return l;
}

constexpr int kTokenMaxRowBytes = 16384;   // the token row kept in shared memory beside the rings

template <typename S> constexpr size_t token_smem_bytes() { return S::SMEM + kTokenMaxRowBytes; }

// grid = one CTA per SM (cooperative), S::THREADS threads.  T is a 16-bit type.
template <typename T, typename S>
__global__ void __launch_bounds__(S::THREADS, 1) moe_token_kernel(TokenParams p, SlotTable st) {
  static_assert(sizeof(T) == 2, "fp32 models take the kernel chain");
  static_assert(S::THREADS == kRouterThreads, "the grouping tail is written for the router's CTA size");
  constexpr int SEG = S::SEG, STAGES = S::STAGES;
  constexpr int CB = 8 * (int)sizeof(T);                 // bytes of one 8-element chunk
  constexpr int SEG_ELEMS = SEG / (int)sizeof(T);
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ TopkSmem<1> s_topk;
  __shared__ int s_ids[kMaxTopK];
  __shared__ float s_w[kMaxTopK];
  __shared__ int s_live[kMaxTopK];       // live index j -> slot k of the token
  __shared__ int s_order[kMaxTopK];      // accumulation order of the combine: live indices by rank, stable
  __shared__ const unsigned char* s_wp[3][kMaxTopK];
  __shared__ int s_nlive;
  __shared__ int s_flag;
  __shared__ float s_part[kNormThreads / 32];
  __shared__ float s_scale;
  static_assert(kNormThreads == S::THREADS, "rmsnorm_row is written for this CTA size");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  unsigned char* ring = smem_raw + (size_t)warp * STAGES * 4 * SEG;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw + (size_t)S::WARPS * STAGES * 4 * SEG) + warp * STAGES;
  unsigned char* xrow = smem_raw + (size_t)S::WARPS * STAGES * 4 * SEG + (size_t)S::WARPS * STAGES * 8;
  const int H = p.r.H, E = p.r.E, K = p.r.K, I = p.I;
  const int nch = H / 8;

  // ---- phase 0: the token row into shared memory, one warp per gate row ----
  if (p.r.norm_w != nullptr) {
    // the norm in front of the block (RouterParams): every CTA normalises the row for itself, CTA 0 publishes it
    const bool writer = blockIdx.x == 0;
    rmsnorm_row<T>(reinterpret_cast<const T*>(p.r.x), reinterpret_cast<const T*>(p.r.norm_res), reinterpret_cast<const T*>(p.r.norm_w), p.r.norm_eps, H,
                   reinterpret_cast<T*>(xrow), writer ? reinterpret_cast<T*>(p.r.normed_out) : nullptr,
                   writer ? reinterpret_cast<T*>(p.r.res_out) : nullptr, s_part, &s_scale);
  } else {
    for (int c = threadIdx.x; c < nch; c += S::THREADS)
      *reinterpret_cast<uint4*>(xrow + (size_t)c * CB) = ldg_cached(reinterpret_cast<const unsigned char*>(p.r.x) + (size_t)c * CB);
  }
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < STAGES; ++i) mbar_init(&full[i], 1);
    mbar_fence_init();
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();

  for (int e = blockIdx.x + (int)gridDim.x * warp; e < E; e += (int)gridDim.x * S::WARPS) {
    const float l = token_gate_logit<T>(xrow, reinterpret_cast<const T*>(p.r.wg) + (size_t)e * H, reinterpret_cast<const T*>(p.r.bias), e, H, lane);
    if (lane == 0) p.r.logits[e] = l;
  }
  bool alive = grid_barrier_bounded(p.gbar, p.wait_cycles, &s_flag, p.status);

  // ---- phase 1: every CTA selects the experts for itself; CTA 0 publishes ids, scores and the grouping ----
  if (alive) topk_softmax_tile<T, 1>(topk_args(p.r), 0, 1, &s_topk, s_ids, s_w, blockIdx.x == 0);
  if (warp == 0) {
    int n = 0;
    if (alive) {
      __syncwarp();
      // lane k looks after slot k of the token: the K table entries are fetched side by side, not one after the other
      int slot = -1, e = -1;
      if (lane < K) {
        e = s_ids[lane];
        slot = (e >= 0 && e < E) ? st.slot[e] : -1;   // no weights for this expert in the placement: skipped
      }
      ExpertPtrs ep{};
      if (slot >= 0) ep = p.experts[slot];
      const unsigned live = __ballot_sync(0xffffffffu, slot >= 0);
      n = __popc(live);
      if (slot >= 0) {
        const int j = __popc(live & ((1u << lane) - 1u));
        s_live[j] = lane;
        s_wp[0][j] = reinterpret_cast<const unsigned char*>(ep.w[0]);
        s_wp[1][j] = reinterpret_cast<const unsigned char*>(ep.w[1]);
        s_wp[2][j] = reinterpret_cast<const unsigned char*>(ep.w[2]);
        // position in the combine's accumulation order: by rank, equal ranks in slot order
        const int my_rank = st.rank[e];
        int before = 0;
        for (int k2 = 0; k2 < K; ++k2) {
          if (!((live >> k2) & 1u) || k2 == lane) continue;
          const int r2 = st.rank[s_ids[k2]];
          before += (r2 < my_rank || (r2 == my_rank && k2 < lane)) ? 1 : 0;
        }
        s_order[before] = j;
      }
    }
    if (lane == 0) s_nlive = n;
  }
  __syncthreads();
  if (alive && blockIdx.x == 0) {
    // The grouping tables of this one-token batch, for readers of the last call's grouping (what permute_block
    // leaves): the K pairs in expert order, every id valid and distinct because the top-k above produced them.
    const PermuteParams& t = p.r.perm;
    for (int e = threadIdx.x; e <= E; e += S::THREADS) {
      int c = 0;
      for (int k = 0; k < K; ++k) c += (s_ids[k] < e) ? 1 : 0;
      t.offsets[e] = c;
    }
    if (threadIdx.x < K) {
      const int k = threadIdx.x, e = s_ids[k];
      const bool served = st.slot[e] >= 0;
      int pos = 0, act_pos = 0;
      for (int k2 = 0; k2 < K; ++k2) {
        const int e2 = s_ids[k2];
        pos += (e2 < e) ? 1 : 0;
        act_pos += (e2 < e && st.slot[e2] >= 0) ? 1 : 0;
      }
      t.inv[k] = pos;
      t.sorted_pair[pos] = k;
      if (served) t.act_list[act_pos] = e;
    }
    if (threadIdx.x == 0) *t.n_act = s_nlive;
  }

  // ---- phases 2 and 3 share one list of units and one ring per warp ----
  const int n_live = s_nlive;
  // warp-major: when the units do not divide evenly, the extra ones fall on ONE warp of many SMs, not on every warp of a few
  const int gw = warp * (int)gridDim.x + blockIdx.x;
  const int W = gridDim.x * S::WARPS;
  const int rb2 = H * (int)sizeof(T);
  // gate/up units: rows (r, r+1) of gate_proj and of up_proj of one expert - or, when that leaves the warps with
  // noticeably unequal shares (Mixtral shape: 14336 units on 1184 warps, one warp in nine holds a thirteenth), row r
  // of both matrices with every row cut in two halves along K, which makes twice as many units of half the size
  bool halfrow = false;
  if (n_live > 0 && (rb2 / 2) % SEG == 0) {
    // rounds * W / units is a warp's largest share over the mean; halves are taken when they bring it down by 0.02:
    // rounds_half * W / (2u) + 0.02 < rounds_full * W / u, in integers
    const long long u_full = (long long)n_live * (I / 2);
    const long long rounds_full = (u_full + W - 1) / W, rounds_half = (2 * u_full + W - 1) / W;
    halfrow = 25 * rounds_half * W + u_full < 50 * rounds_full * W;
  }
  const int upe = halfrow ? I : I / 2;                   // units per expert
  const int U2 = n_live * upe;
  const int rb2u = halfrow ? rb2 / 2 : rb2;               // bytes one stream of a gate/up unit covers
  // down projection + combine: rows (r, r+1) of down_proj of EVERY live expert, two experts per stage in the
  // combine's accumulation order, so that the warp holding a row's K products also adds them up
  const int U3 = n_live > 0 ? H / 2 : 0;
  const int npair = (n_live + 1) / 2;
  const int total_units = U2 + U3;
  const int nseg2 = (rb2u + SEG - 1) / SEG;
  const int rb3 = I * (int)sizeof(T), nseg3 = (rb3 + SEG - 1) / SEG;
  const uint64_t policy = l2_policy_evict_first();
  const int sidx4 = lane & 3;

  // producer: STAGES-1 stages ahead of the consumer, across unit and phase boundaries
  int pu = gw, ps = 0, issued = 0;
  const unsigned char* prow = nullptr;     // gate/up unit: this lane's row
  int p_row3 = 0;                          // down unit: this lane's row index
  int p_nstage = 0;
  auto open_unit = [&](int u) {
    if (u < U2) {
      const int j = u / upe, g = u - j * upe;
      // streams: (gate r, gate r+1, up r, up r+1), or (gate r first half, second half, up r first half, second half)
      prow = halfrow ? s_wp[sidx4 >> 1][j] + (size_t)g * rb2 + (size_t)(sidx4 & 1) * rb2u
                     : s_wp[sidx4 >> 1][j] + (size_t)(2 * g + (sidx4 & 1)) * rb2;
      p_nstage = nseg2;
    } else {
      p_row3 = (u - U2) * 2 + (sidx4 & 1);
      p_nstage = npair * nseg3;
    }
  };
  if (alive && pu < total_units) open_unit(pu);
  auto produce = [&]() {
    if (pu >= total_units) return;
    const int slot = issued % STAGES;
    const unsigned char* src;
    uint32_t bytes, streams = 4;
    bool mine = true;
    if (pu < U2) {
      bytes = (uint32_t)min(SEG, rb2u - ps * SEG);
      src = prow + (size_t)ps * SEG;
    } else {
      const int q = ps / nseg3, seg = ps - q * nseg3;
      const int ord = 2 * q + (sidx4 >> 1);             // streams 0,1: expert 2q of the order; streams 2,3: expert 2q+1
      if (2 * q + 1 >= n_live) streams = 2;
      mine = ord < n_live;
      bytes = (uint32_t)min(SEG, rb3 - seg * SEG);
      src = s_wp[2][s_order[min(ord, n_live - 1)]] + (size_t)p_row3 * rb3 + (size_t)seg * SEG;
    }
    if (lane == 0) mbar_expect_tx(&full[slot], streams * bytes);
    __syncwarp();
    if (lane < 4 && mine) bulk_g2s(ring + (size_t)(slot * 4 + lane) * SEG, src, bytes, &full[slot], policy);
    ++issued;
    if (++ps == p_nstage) {
      pu += W;
      ps = 0;
      if (pu < total_units) open_unit(pu);
    }
  };
  if (alive) {
#pragma unroll
    for (int i = 0; i < STAGES - 1; ++i) produce();
  } else {
    pu = total_units;
  }

  int consumed = 0;
  bool dead = !alive;
  // waits for the next stage of this warp's ring; null when the wait ran out
  auto next_stage = [&]() -> const unsigned char* {
    produce();
    const int slot = consumed % STAGES;
    if (!mbar_wait_bounded(&full[slot], (uint32_t)(consumed / STAGES) & 1u)) {
      if (lane == 0) atomicOr(p.status, kDevWaitExpired);
      dead = true;
      return nullptr;
    }
    ++consumed;
    return ring + (size_t)slot * 4 * SEG;
  };

  int cu = gw;
  for (; cu < U2 && !dead; cu += W) {
    const int j = cu / upe, g = cu - j * upe;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int seg = 0; seg < nseg2; ++seg) {
      const unsigned char* sbase = next_stage();
      if (sbase == nullptr) break;
      const int nchunk = min(SEG, rb2u - seg * SEG) / CB;
      for (int cl = lane; cl < nchunk; cl += 32) {
        Chunk<T> xc;
        float xf[2][8];
        xc.from_smem(xrow + (size_t)seg * SEG + (size_t)cl * CB);
        xc.unpack(xf[0]);
        if (halfrow) {                    // the odd streams hold the second half of the row
          xc.from_smem(xrow + (size_t)rb2u + (size_t)seg * SEG + (size_t)cl * CB);
          xc.unpack(xf[1]);
        }
#pragma unroll
        for (int s = 0; s < 4; ++s) {
          Chunk<T> wc;
          wc.from_smem(sbase + (size_t)s * SEG + (size_t)cl * CB);
          float wf[8];
          wc.unpack(wf);
          const float* xs = (halfrow && (s & 1)) ? xf[1] : xf[0];
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[s] = fmaf(wf[i], xs[i], acc[s]);
        }
      }
      __syncwarp();   // every lane is done with the slot before it is refilled
    }
    if (dead) break;
    // rounding points of the reference's SwiGLU
    if (halfrow) {
      const float gs = warp_sum(acc[0] + acc[1]), us = warp_sum(acc[2] + acc[3]);
      if (lane == 0) {
        const float gg = rn<T>(gs), uu = rn<T>(us);
        const float sg = rn<T>(silu_f32(gg));
        reinterpret_cast<T*>(p.h)[(size_t)j * I + g] = Elem<T>::from_float(__fmul_rn(sg, uu));
      }
    } else {
#pragma unroll
      for (int s = 0; s < 4; ++s) acc[s] = warp_sum(acc[s]);
      if (lane < 2) {
        const float gg = rn<T>(lane == 0 ? acc[0] : acc[1]);
        const float uu = rn<T>(lane == 0 ? acc[2] : acc[3]);
        const float sg = rn<T>(silu_f32(gg));
        reinterpret_cast<T*>(p.h)[(size_t)j * I + 2 * g + lane] = Elem<T>::from_float(__fmul_rn(sg, uu));
      }
    }
  }
  if (!grid_barrier_bounded(p.gbar, p.wait_cycles, &s_flag, p.status)) dead = true;     // h is complete

  for (; cu < total_units && !dead; cu += W) {
    const int r0 = (cu - U2) * 2;
    float out_acc[2] = {0.0f, 0.0f};     // the combine's running sums of rows r0, r0+1, each held as the model dtype holds it
    for (int q = 0; q < npair && !dead; ++q) {
      const int ja = s_order[2 * q];
      const bool two = 2 * q + 1 < n_live;
      const int jb = s_order[two ? 2 * q + 1 : 2 * q];
      const T* ha = reinterpret_cast<const T*>(p.h) + (size_t)ja * I;
      const T* hb = reinterpret_cast<const T*>(p.h) + (size_t)jb * I;
      float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      for (int seg = 0; seg < nseg3; ++seg) {
        static_assert(SEG / CB == 32 * 4, "one h chunk per lane and quarter of a segment");
        const int nchunk = min(SEG, rb3 - seg * SEG) / CB;
        // h was written in this launch: plain loads (L2 for the most part - the rings leave little L1), all of the
        // segment's chunks requested before the wait for the weights
        Chunk<T> hca[4], hcb[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (lane + 32 * u < nchunk) {
            hca[u].from_smem(ha + (size_t)seg * SEG_ELEMS + (size_t)(lane + 32 * u) * 8);
            hcb[u].from_smem(hb + (size_t)seg * SEG_ELEMS + (size_t)(lane + 32 * u) * 8);
          }
        const unsigned char* sbase = next_stage();
        if (sbase == nullptr) break;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int cl = lane + 32 * u;
          if (cl >= nchunk) break;
          float hf[8];
          hca[u].unpack(hf);
#pragma unroll
          for (int s = 0; s < 2; ++s) {
            Chunk<T> wc;
            wc.from_smem(sbase + (size_t)s * SEG + (size_t)cl * CB);
            float wf[8];
            wc.unpack(wf);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[s] = fmaf(wf[i], hf[i], acc[s]);
          }
          if (two) {
            hcb[u].unpack(hf);
#pragma unroll
            for (int s = 2; s < 4; ++s) {
              Chunk<T> wc;
              wc.from_smem(sbase + (size_t)s * SEG + (size_t)cl * CB);
              float wf[8];
              wc.unpack(wf);
#pragma unroll
              for (int i = 0; i < 8; ++i) acc[s] = fmaf(wf[i], hf[i], acc[s]);
            }
          }
        }
        __syncwarp();
      }
      if (dead) break;
#pragma unroll
      for (int s = 0; s < 4; ++s) acc[s] = warp_sum(acc[s]);       // every lane holds the four sums
      // the expert's output rounded as F.linear rounds it, times its score, added in rank order: the rounding
      // points of `final_output[tok] += expert_output * weights`
      const float wa = s_w[s_live[ja]], wb = s_w[s_live[jb]];
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        out_acc[rr] = rn<T>(__fadd_rn(out_acc[rr], rn<T>(__fmul_rn(rn<T>(acc[rr]), wa))));
        if (two) out_acc[rr] = rn<T>(__fadd_rn(out_acc[rr], rn<T>(__fmul_rn(rn<T>(acc[2 + rr]), wb))));
      }
    }
    if (dead) break;
    if (lane < 2) {
      float o = lane == 0 ? out_acc[0] : out_acc[1];
      if (p.residual != nullptr)      // plain load: with the fused norm CTA 0 wrote it in this launch
        o = rn<T>(__fadd_rn(Elem<T>::to_float(reinterpret_cast<const T*>(p.residual)[r0 + lane]), o));
      reinterpret_cast<T*>(p.out)[r0 + lane] = Elem<T>::from_float(o);
    }
  }
  if (n_live == 0 && !dead) {
    // nothing served: the block contributes zeros
    for (int c = blockIdx.x * S::THREADS + threadIdx.x; c < H; c += (int)gridDim.x * S::THREADS) {
      float o = 0.0f;
      if (p.residual != nullptr) o = rn<T>(__fadd_rn(Elem<T>::to_float(reinterpret_cast<const T*>(p.residual)[c]), o));
      reinterpret_cast<T*>(p.out)[c] = Elem<T>::from_float(o);
    }
  }
  if (dead) {
    // A wait ran out.  Copies issued earlier may still be in flight towards this warp's ring: give each of them
    // a short, bounded chance to land before the shared memory can pass to another CTA.
    for (int i = consumed; i < issued; ++i) mbar_wait_brief(&full[i % STAGES], (uint32_t)(i / STAGES) & 1u);
  }
}

}  // namespace b200moe
