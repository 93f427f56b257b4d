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
// its first down-projection rows are already on their way into shared memory.  The three grid barriers are
// sense-reversing counters in global memory with a bounded wait; the launch is cooperative, so every CTA is
// resident and the barriers cannot starve.
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
  void* y;                     // [K][H] expert outputs, same rows
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
  __shared__ float skey[32];
  __shared__ int sidx[32];
  __shared__ int s_ids[kMaxTopK];
  __shared__ float s_w[kMaxTopK];
  __shared__ int s_live[kMaxTopK];       // live index j -> slot k of the token
  __shared__ int s_order[kMaxTopK];      // accumulation order of the combine: live indices by rank, stable
  __shared__ const unsigned char* s_wp[3][kMaxTopK];
  __shared__ int s_nlive;
  __shared__ int s_flag;
  __shared__ int s_perm[kRouterFuseSmemInts];
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
    // the certificate of router_kernel: four fp32 accumulators per lane, eight chunk positions per trip
    const T* wrow = reinterpret_cast<const T*>(p.r.wg) + (size_t)e * H;
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
        xc.from_smem(xrow + (size_t)(c0 + 32 * u) * CB);
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
    if (!(boundary_distance<T>(s) > bound)) s = (float)exact_dot<T, true>(reinterpret_cast<const T*>(xrow), wrow, nch, lane);
    float l = rn<T>(s);
    if (p.r.bias != nullptr) l = rn<T>(l + Elem<T>::to_float(reinterpret_cast<const T*>(p.r.bias)[e]));
    if (lane == 0) p.r.logits[e] = l;
  }
  bool alive = grid_barrier_bounded(p.gbar, p.wait_cycles, &s_flag, p.status);

  // ---- phase 1: every CTA selects the experts for itself; CTA 0 publishes ids, scores and the grouping ----
  if (alive && warp == 0) topk_softmax_token<T>(p.r, 0, lane, skey, sidx, s_ids, s_w, blockIdx.x == 0);
  __syncthreads();
  if (threadIdx.x == 0) {
    int n = 0;
    if (alive) {
      for (int k = 0; k < K; ++k) {
        const int e = s_ids[k];
        const int slot = (e >= 0 && e < E) ? st.slot[e] : -1;
        if (slot < 0) continue;                       // no weights for this expert in the placement: skipped
        const ExpertPtrs ep = p.experts[slot];
        s_live[n] = k;
        s_wp[0][n] = reinterpret_cast<const unsigned char*>(ep.w[0]);
        s_wp[1][n] = reinterpret_cast<const unsigned char*>(ep.w[1]);
        s_wp[2][n] = reinterpret_cast<const unsigned char*>(ep.w[2]);
        int i = n;
        while (i > 0 && st.rank[s_ids[s_live[s_order[i - 1]]]] > st.rank[e]) {   // stable insertion by rank
          s_order[i] = s_order[i - 1];
          --i;
        }
        s_order[i] = n;
        ++n;
      }
    }
    s_nlive = n;
  }
  __syncthreads();
  if (alive && blockIdx.x == 0) permute_block(p.r.perm, st, s_perm);

  // ---- phases 2 and 3 share one list of units and one ring per warp ----
  const int n_live = s_nlive;
  const int gw = blockIdx.x * S::WARPS + warp;
  const int W = gridDim.x * S::WARPS;
  const int half_I = I / 2;
  const int U2 = n_live * half_I;                       // gate/up: rows (r, r+1) of gate_proj and of up_proj
  // down projection: one row split into four K quarters when four-row units would leave warps idle (and a
  // quarter still fills a ring segment), else rows (r .. r+3)
  const bool quarter = (I % 32 == 0) && I * (int)sizeof(T) >= 4 * SEG && n_live * (H / 4) < 6 * W;
  const int groups3 = quarter ? H : H / 4;
  const int total_units = U2 + n_live * groups3;
  const int rb2 = H * (int)sizeof(T), nseg2 = (rb2 + SEG - 1) / SEG;
  const int rb3 = (quarter ? I / 4 : I) * (int)sizeof(T), nseg3 = (rb3 + SEG - 1) / SEG;
  const uint64_t policy = l2_policy_evict_first();
  const int sidx4 = lane & 3;

  // producer: STAGES-1 stages ahead of the consumer, across unit and phase boundaries
  int pu = gw, ps = 0, issued = 0;
  const unsigned char* prow = nullptr;
  int p_nseg = 0, p_rb = 0;
  auto open_unit = [&](int u) {
    if (u < U2) {
      const int j = u / half_I, r0 = (u - j * half_I) * 2;
      prow = s_wp[sidx4 >> 1][j] + (size_t)(r0 + (sidx4 & 1)) * rb2;
      p_nseg = nseg2; p_rb = rb2;
    } else {
      const int v = u - U2;
      const int j = v / groups3, g = v - j * groups3;
      if (quarter) prow = s_wp[2][j] + (size_t)g * I * sizeof(T) + (size_t)sidx4 * rb3;
      else prow = s_wp[2][j] + (size_t)(g * 4 + sidx4) * rb3;
      p_nseg = nseg3; p_rb = rb3;
    }
  };
  if (alive && pu < total_units) open_unit(pu);
  auto produce = [&]() {
    if (pu >= total_units) return;
    const int slot = issued % STAGES;
    const uint32_t bytes = (uint32_t)min(SEG, p_rb - ps * SEG);
    if (lane == 0) mbar_expect_tx(&full[slot], 4 * bytes);
    __syncwarp();
    if (lane < 4) bulk_g2s(ring + (size_t)(slot * 4 + lane) * SEG, prow + (size_t)ps * SEG, bytes, &full[slot], policy);
    ++issued;
    if (++ps == p_nseg) {
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
  // waits for the next stage of this warp's ring; false when the wait ran out
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
    const int j = cu / half_I, r0 = (cu - j * half_I) * 2;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int seg = 0; seg < nseg2; ++seg) {
      const unsigned char* sbase = next_stage();
      if (sbase == nullptr) break;
      const int nchunk = min(SEG, rb2 - seg * SEG) / CB;
      for (int cl = lane; cl < nchunk; cl += 32) {
        Chunk<T> xc;
        xc.from_smem(xrow + (size_t)seg * SEG + (size_t)cl * CB);
        float xf[8];
        xc.unpack(xf);
#pragma unroll
        for (int s = 0; s < 4; ++s) {
          Chunk<T> wc;
          wc.from_smem(sbase + (size_t)s * SEG + (size_t)cl * CB);
          float wf[8];
          wc.unpack(wf);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[s] = fmaf(wf[i], xf[i], acc[s]);
        }
      }
      __syncwarp();   // every lane is done with the slot before it is refilled
    }
    if (dead) break;
#pragma unroll
    for (int s = 0; s < 4; ++s) acc[s] = warp_sum(acc[s]);
    if (lane < 2) {
      // stream order is (gate r, gate r+1, up r, up r+1); rounding points of the reference's SwiGLU
      const float g = rn<T>(lane == 0 ? acc[0] : acc[1]);
      const float u = rn<T>(lane == 0 ? acc[2] : acc[3]);
      const float sg = rn<T>(silu_f32(g));
      reinterpret_cast<T*>(p.h)[(size_t)j * I + r0 + lane] = Elem<T>::from_float(__fmul_rn(sg, u));
    }
  }
  if (!grid_barrier_bounded(p.gbar, p.wait_cycles, &s_flag, p.status)) dead = true;     // h is complete

  for (; cu < total_units && !dead; cu += W) {
    const int v = cu - U2;
    const int j = v / groups3, g = v - j * groups3;
    const T* hrow = reinterpret_cast<const T*>(p.h) + (size_t)j * I;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int seg = 0; seg < nseg3; ++seg) {
      const unsigned char* sbase = next_stage();
      if (sbase == nullptr) break;
      const int nchunk = min(SEG, rb3 - seg * SEG) / CB;
      for (int cl = lane; cl < nchunk; cl += 32) {
        if (quarter) {
#pragma unroll
          for (int s = 0; s < 4; ++s) {
            Chunk<T> wc, hc;
            wc.from_smem(sbase + (size_t)s * SEG + (size_t)cl * CB);
            hc.from_smem(hrow + (size_t)s * (I / 4) + (size_t)seg * SEG_ELEMS + (size_t)cl * 8);   // plain load: written in this launch
            float wf[8], hf[8];
            wc.unpack(wf);
            hc.unpack(hf);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[s] = fmaf(wf[i], hf[i], acc[s]);
          }
        } else {
          Chunk<T> hc;
          hc.from_smem(hrow + (size_t)seg * SEG_ELEMS + (size_t)cl * 8);
          float hf[8];
          hc.unpack(hf);
#pragma unroll
          for (int s = 0; s < 4; ++s) {
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
    if (quarter) {
      const float s = warp_sum((acc[0] + acc[1]) + (acc[2] + acc[3]));
      if (lane == 0) reinterpret_cast<T*>(p.y)[(size_t)j * H + g] = Elem<T>::from_float(s);
    } else {
#pragma unroll
      for (int s = 0; s < 4; ++s) acc[s] = warp_sum(acc[s]);
      if (lane < 4) {
        const float s = lane == 0 ? acc[0] : lane == 1 ? acc[1] : lane == 2 ? acc[2] : acc[3];
        reinterpret_cast<T*>(p.y)[(size_t)j * H + g * 4 + lane] = Elem<T>::from_float(s);
      }
    }
  }
  if (!grid_barrier_bounded(p.gbar, p.wait_cycles, &s_flag, p.status)) dead = true;     // y is complete

  // ---- phase 4: out = residual + sum over the live experts, in rank order, rounded where the reference rounds ----
  if (!dead && warp == 0) {
    const T* y = reinterpret_cast<const T*>(p.y);
    for (int c = blockIdx.x * 32 + lane; c < nch; c += (int)gridDim.x * 32) {
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
      for (int j0 = 0; j0 < n_live; j0 += 8) {
        Chunk<T> yc[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (j0 + u < n_live) yc[u].from_smem(y + (size_t)s_order[j0 + u] * H + (size_t)c * 8);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          if (j0 + u >= n_live) break;
          const float w = s_w[s_live[s_order[j0 + u]]];
          float yf[8];
          yc[u].unpack(yf);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] = rn<T>(__fadd_rn(acc[i], rn<T>(__fmul_rn(yf[i], w))));
        }
      }
      if (p.residual != nullptr) {
        Chunk<T> rc;
        rc.from_smem(reinterpret_cast<const T*>(p.residual) + (size_t)c * 8);    // plain load: with the fused norm CTA 0 wrote it in this launch
        float rf[8];
        rc.unpack(rf);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = rn<T>(__fadd_rn(rf[i], acc[i]));
      }
      store_chunk<T>(reinterpret_cast<T*>(p.out) + (size_t)c * 8, acc);
    }
  }
  if (dead) {
    // A wait ran out.  Copies issued earlier may still be in flight towards this warp's ring: give each of them
    // a short, bounded chance to land before the shared memory can pass to another CTA.
    for (int i = consumed; i < issued; ++i) mbar_wait_brief(&full[i % STAGES], (uint32_t)(i / STAGES) & 1u);
  }
}

}  // namespace b200moe
