// The MoE block of a batch of TWO tokens in one cooperative launch: the scheme of moe_token.cuh (gate logits, grid
// barrier, top-k in every CTA, gate/up units through per-warp bulk-copy rings, grid barrier, down units that also
// run the combine) with a token tile in registers.  Replaces the same reference code as moe_token.cuh
// (demo/src/layers/moe_layer.py:25-60, demo/src/layers/mlp.py:209-231, demo/src/model/qwen3_runner.py:352-383)
// for the smallest verify batch.  The token tile NT is a template parameter and the kernel is correct for up to
// four tokens, but only two are dispatched here: on the Qwen3-shaped layer two tokens take 47 us against 54 us for
// the kernel chain, four tokens 88 us against 75 us: global-timer marks put the gate/up phase at 5.8 TB/s but the
// down phase at 2.8 TB/s - a down unit walks ~30 experts, one 6 KB ring stage after the other (2.2 us per stage, of
// which the sixteen warp reductions and the combine arithmetic of every expert pair are about half), and only
// 1024 of the 1184 warps have a unit.
//
// What differs from the single-token kernel:
//  * the (token, expert) pairs - at most 32, one lane each - are grouped by expert in every CTA by counting
//    (sorted position = number of pairs ahead in (expert, pair) order); a served expert's table entry is fetched
//    by the lane of its first pair, all entries side by side;
//  * a gate/up unit (rows r, r+1 of gate_proj and up_proj of one expert) carries up to NT token accumulators;
//  * h (at most 32 rows of I elements) is copied into shared memory after the second barrier, so the down phase
//    reads weights AND activations from shared memory - with h in global memory every ring stage of the down
//    phase paid an L2 round trip, and a down unit walks all served experts one stage after the other;
//  * the ring segments are 1.5 KB instead of 2 KB to make room for h.
// The combine adds a token's experts in ascending expert order, which is the accumulation order of the fused entry
// points (rank[e] = e); callers with another order take the kernel chain.
#pragma once
#include "moe_token.cuh"

namespace b200moe {

constexpr int kTokensMaxPairs = 32;            // (token, expert) pairs of the batch: one lane each
constexpr int kTokensMaxHBytes = 49152;        // h of all pairs, kept in shared memory for the down phase
using TokensShape = GemvShape<8, 1536, 3>;
constexpr size_t kTokensSmemBytes = TokensShape::SMEM + kTokenMaxRowBytes + kTokensMaxHBytes;

// grid = one CTA per SM (cooperative), 256 threads.  T is a 16-bit type; 2 <= p.r.T <= NT,
// p.r.T * K <= kTokensMaxPairs, p.r.T * H * sizeof(T) <= kTokenMaxRowBytes, p.r.T * K * I * sizeof(T) <= kTokensMaxHBytes.
template <typename T, int NT>
__global__ void __launch_bounds__(TokensShape::THREADS, 1) moe_tokens_kernel(TokenParams p, SlotTable st) {
  using S = TokensShape;
  static_assert(sizeof(T) == 2, "fp32 models take the kernel chain");
  static_assert(NT == 2 || NT == 4, "token tile");
  constexpr int SEG = S::SEG, STAGES = S::STAGES;
  constexpr int CB = 8 * (int)sizeof(T);                 // bytes of one 8-element chunk
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ TopkSmem<NT> s_topk;
  __shared__ int s_ids[kTokensMaxPairs];                 // expert of pair p = t * K + k
  __shared__ float s_w[kTokensMaxPairs];                 // its score, as the model dtype holds it
  __shared__ int s_pos_tok[kTokensMaxPairs];             // sorted position (expert ascending, pair ascending) -> token
  __shared__ float s_pos_w[kTokensMaxPairs];             //                                                 -> score
  __shared__ int s_exp_off[kTokensMaxPairs];             // served expert j (ascending id): first sorted position
  __shared__ int s_exp_n[kTokensMaxPairs];               //                                  its number of tokens
  __shared__ const unsigned char* s_wp[3][kTokensMaxPairs];  //                              its three matrices
  __shared__ int s_nexp;
  __shared__ int s_flag;
  __shared__ float s_part[kNormThreads / 32];
  __shared__ float s_scale;
  static_assert(kNormThreads == S::THREADS && kRouterThreads == S::THREADS, "rmsnorm_row and the top-k are written for this CTA size");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  unsigned char* ring = smem_raw + (size_t)warp * STAGES * 4 * SEG;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw + (size_t)S::WARPS * STAGES * 4 * SEG) + warp * STAGES;
  unsigned char* xrows = smem_raw + (size_t)S::WARPS * STAGES * 4 * SEG + (size_t)S::WARPS * STAGES * 8;   // [nt][H]
  unsigned char* hbuf = xrows + kTokenMaxRowBytes;                                                           // [P][I]
  const int H = p.r.H, E = p.r.E, K = p.r.K, I = p.I, nt = p.r.T;
  const int nch = H / 8;
  const int P = nt * K;
  const size_t xrow_bytes = (size_t)H * sizeof(T);
  const size_t hrow_bytes = (size_t)I * sizeof(T);

  // ---- phase 0: the token rows into shared memory, one warp per (token, gate row) ----
  if (p.r.norm_w != nullptr) {
    // the norm in front of the block (RouterParams): every CTA normalises the rows for itself, CTA 0 publishes them
    const bool writer = blockIdx.x == 0;
    for (int t = 0; t < nt; ++t) {
      const size_t off = (size_t)t * H;
      rmsnorm_row<T>(reinterpret_cast<const T*>(p.r.x) + off, p.r.norm_res ? reinterpret_cast<const T*>(p.r.norm_res) + off : nullptr,
                     reinterpret_cast<const T*>(p.r.norm_w), p.r.norm_eps, H, reinterpret_cast<T*>(xrows) + off,
                     (writer && p.r.normed_out) ? reinterpret_cast<T*>(p.r.normed_out) + off : nullptr,
                     (writer && p.r.res_out) ? reinterpret_cast<T*>(p.r.res_out) + off : nullptr, s_part, &s_scale);
    }
  } else {
    for (int c = threadIdx.x; c < nt * nch; c += S::THREADS)
      *reinterpret_cast<uint4*>(xrows + (size_t)c * CB) = ldg_cached(reinterpret_cast<const unsigned char*>(p.r.x) + (size_t)c * CB);
  }
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < STAGES; ++i) mbar_init(&full[i], 1);
    mbar_fence_init();
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();

  for (int it = blockIdx.x + (int)gridDim.x * warp; it < nt * E; it += (int)gridDim.x * S::WARPS) {
    const int t = it / E, e = it - t * E;
    const float l = token_gate_logit<T>(xrows + (size_t)t * xrow_bytes, reinterpret_cast<const T*>(p.r.wg) + (size_t)e * H,
                                        reinterpret_cast<const T*>(p.r.bias), e, H, lane);
    if (lane == 0) p.r.logits[(size_t)t * E + e] = l;
  }
  bool alive = grid_barrier_bounded(p.gbar, p.wait_cycles, &s_flag, p.status);

  // ---- phase 1: every CTA selects the experts for itself and groups the pairs; CTA 0 publishes ids, scores, tables ----
  if (alive) topk_softmax_tile<T, NT>(topk_args(p.r), 0, nt, &s_topk, s_ids, s_w, blockIdx.x == 0);
  __syncthreads();
  if (warp == 0) {
    int n_exp = 0;
    if (alive) {
      // lane q looks after pair q: its sorted position, whether it is the first pair of a served expert (the
      // "head", which fetches the expert's table entry), the expert's index among the served ones and its load
      const int e = lane < P ? s_ids[lane] : 0x7fffffff;
      const int slot = (e >= 0 && e < E) ? st.slot[e] : -1;      // no weights for this expert in the placement: skipped
      int pos = 0, same_before = 0, cnt = 0;
      for (int q = 0; q < P; ++q) {
        const int eq = s_ids[q];
        pos += (eq < e || (eq == e && q < lane)) ? 1 : 0;
        same_before += (eq == e && q < lane) ? 1 : 0;
        cnt += (eq == e) ? 1 : 0;
      }
      const bool head = slot >= 0 && same_before == 0;
      ExpertPtrs ep{};
      if (head) ep = p.experts[slot];
      const unsigned heads = __ballot_sync(0xffffffffu, head);
      n_exp = __popc(heads);
      int j = 0;
      for (int q = 0; q < P; ++q) j += (((heads >> q) & 1u) && s_ids[q] < e) ? 1 : 0;
      if (lane < P) {
        s_pos_tok[pos] = lane / K;
        s_pos_w[pos] = s_w[lane];
      }
      if (head) {
        s_exp_off[j] = pos;
        s_exp_n[j] = cnt;
        s_wp[0][j] = reinterpret_cast<const unsigned char*>(ep.w[0]);
        s_wp[1][j] = reinterpret_cast<const unsigned char*>(ep.w[1]);
        s_wp[2][j] = reinterpret_cast<const unsigned char*>(ep.w[2]);
      }
      if (blockIdx.x == 0) {
        // The grouping tables of the batch, for readers of the last call's grouping (what permute_block leaves);
        // every id is valid because the top-k above produced it.
        const PermuteParams& tb = p.r.perm;
        for (int x = lane; x <= E; x += 32) {
          int c = 0;
          for (int q = 0; q < P; ++q) c += (s_ids[q] < x) ? 1 : 0;
          tb.offsets[x] = c;
        }
        if (lane < P) {
          tb.inv[lane] = pos;
          tb.sorted_pair[pos] = lane;
        }
        if (head) tb.act_list[j] = e;
        if (lane == 0) *tb.n_act = n_exp;
      }
    }
    if (lane == 0) s_nexp = n_exp;
  }
  __syncthreads();

  // ---- phases 2 and 3 share one list of units and one ring per warp ----
  const int n_exp = s_nexp;
  // warp-major: when the units do not divide evenly, the extra ones fall on ONE warp of many SMs, not on every warp of a few
  const int gw = warp * (int)gridDim.x + blockIdx.x;
  const int W = gridDim.x * S::WARPS;
  const int half_I = I / 2;
  const int U2 = n_exp * half_I;                        // gate/up: rows (r, r+1) of gate_proj and of up_proj of one expert
  // down projection + combine: rows (r, r+1) of down_proj of EVERY served expert, two experts per stage in
  // ascending order, so that the warp holding a row's products also adds them up
  const int U3 = n_exp > 0 ? H / 2 : 0;
  const int npair = (n_exp + 1) / 2;
  const int total_units = U2 + U3;
  const int rb2 = H * (int)sizeof(T), nseg2 = (rb2 + SEG - 1) / SEG;
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
      const int j = u / half_I, r0 = (u - j * half_I) * 2;
      prow = s_wp[sidx4 >> 1][j] + (size_t)(r0 + (sidx4 & 1)) * rb2;
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
      bytes = (uint32_t)min(SEG, rb2 - ps * SEG);
      src = prow + (size_t)ps * SEG;
    } else {
      const int q = ps / nseg3, seg = ps - q * nseg3;
      const int ord = 2 * q + (sidx4 >> 1);             // streams 0,1: expert 2q; streams 2,3: expert 2q+1
      if (2 * q + 1 >= n_exp) streams = 2;
      mine = ord < n_exp;
      bytes = (uint32_t)min(SEG, rb3 - seg * SEG);
      src = s_wp[2][min(ord, n_exp - 1)] + (size_t)p_row3 * rb3 + (size_t)seg * SEG;
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
    const int j = cu / half_I, r0 = (cu - j * half_I) * 2;
    const int off = s_exp_off[j], n = min(s_exp_n[j], NT);
    const unsigned char* xr[NT];
#pragma unroll
    for (int i = 0; i < NT; ++i) xr[i] = xrows + (size_t)s_pos_tok[off + min(i, n - 1)] * xrow_bytes;
    float acc[4][NT];
#pragma unroll
    for (int s = 0; s < 4; ++s)
#pragma unroll
      for (int i = 0; i < NT; ++i) acc[s][i] = 0.0f;
    for (int seg = 0; seg < nseg2; ++seg) {
      const unsigned char* sbase = next_stage();
      if (sbase == nullptr) break;
      const int nchunk = min(SEG, rb2 - seg * SEG) / CB;
      for (int cl = lane; cl < nchunk; cl += 32) {
        float wf[4][8];
#pragma unroll
        for (int s = 0; s < 4; ++s) {
          Chunk<T> wc;
          wc.from_smem(sbase + (size_t)s * SEG + (size_t)cl * CB);
          wc.unpack(wf[s]);
        }
#pragma unroll
        for (int i = 0; i < NT; ++i) {
          if (i >= n) break;
          Chunk<T> xc;
          xc.from_smem(xr[i] + (size_t)seg * SEG + (size_t)cl * CB);
          float xf[8];
          xc.unpack(xf);
#pragma unroll
          for (int s = 0; s < 4; ++s)
#pragma unroll
            for (int k8 = 0; k8 < 8; ++k8) acc[s][i] = fmaf(wf[s][k8], xf[k8], acc[s][i]);
        }
      }
      __syncwarp();   // every lane is done with the slot before it is refilled
    }
    if (dead) break;
#pragma unroll
    for (int s = 0; s < 4; ++s)
#pragma unroll
      for (int i = 0; i < NT; ++i) acc[s][i] = warp_sum(acc[s][i]);
    // stream order is (gate r, gate r+1, up r, up r+1); lane rr * NT + i stores (row r0 + rr, token i of the expert)
    // with the rounding points of the reference's SwiGLU
#pragma unroll
    for (int rr = 0; rr < 2; ++rr)
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        if (lane == rr * NT + i && i < n) {
          const float g = rn<T>(acc[rr][i]);
          const float u = rn<T>(acc[2 + rr][i]);
          const float sg = rn<T>(silu_f32(g));
          reinterpret_cast<T*>(p.h)[(size_t)(off + i) * I + r0 + rr] = Elem<T>::from_float(__fmul_rn(sg, u));
        }
      }
  }
  if (!grid_barrier_bounded(p.gbar, p.wait_cycles, &s_flag, p.status)) dead = true;     // h is complete

  // h of all pairs into shared memory (written in this launch by other SMs: plain loads after the barrier's acquire)
  if (!dead) {
    const int nh = P * (I / 8);
    for (int c = threadIdx.x; c < nh; c += S::THREADS)
      *reinterpret_cast<uint4*>(hbuf + (size_t)c * CB) = *reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned char*>(p.h) + (size_t)c * CB);
  }
  __syncthreads();

  for (; cu < total_units && !dead; cu += W) {
    const int r0 = (cu - U2) * 2;
    float out_acc[2][NT];     // the combine's running sums of rows r0, r0+1 per token, each held as the model dtype holds it
#pragma unroll
    for (int rr = 0; rr < 2; ++rr)
#pragma unroll
      for (int t = 0; t < NT; ++t) out_acc[rr][t] = 0.0f;
    for (int q = 0; q < npair && !dead; ++q) {
      const int ja = 2 * q;
      const bool two = 2 * q + 1 < n_exp;
      const int jb = two ? 2 * q + 1 : 2 * q;
      const int off_a = s_exp_off[ja], n_a = min(s_exp_n[ja], NT);
      const int off_b = s_exp_off[jb], n_b = two ? min(s_exp_n[jb], NT) : 0;
      const unsigned char* ha = hbuf + (size_t)off_a * hrow_bytes;
      const unsigned char* hb = hbuf + (size_t)off_b * hrow_bytes;
      float acc[4][NT];
#pragma unroll
      for (int s = 0; s < 4; ++s)
#pragma unroll
        for (int i = 0; i < NT; ++i) acc[s][i] = 0.0f;
      for (int seg = 0; seg < nseg3; ++seg) {
        const unsigned char* sbase = next_stage();
        if (sbase == nullptr) break;
        const int nchunk = min(SEG, rb3 - seg * SEG) / CB;
        for (int cl = lane; cl < nchunk; cl += 32) {
          float wf[4][8];
#pragma unroll
          for (int s = 0; s < 4; ++s) {
            Chunk<T> wc;
            wc.from_smem(sbase + (size_t)s * SEG + (size_t)cl * CB);
            wc.unpack(wf[s]);
          }
          const size_t at = (size_t)seg * SEG + (size_t)cl * CB;
#pragma unroll
          for (int i = 0; i < NT; ++i) {
            Chunk<T> hc;
            float hf[8];
            if (i < n_a) {
              hc.from_smem(ha + (size_t)i * hrow_bytes + at);
              hc.unpack(hf);
#pragma unroll
              for (int s = 0; s < 2; ++s)
#pragma unroll
                for (int k8 = 0; k8 < 8; ++k8) acc[s][i] = fmaf(wf[s][k8], hf[k8], acc[s][i]);
            }
            if (i < n_b) {
              hc.from_smem(hb + (size_t)i * hrow_bytes + at);
              hc.unpack(hf);
#pragma unroll
              for (int s = 2; s < 4; ++s)
#pragma unroll
                for (int k8 = 0; k8 < 8; ++k8) acc[s][i] = fmaf(wf[s][k8], hf[k8], acc[s][i]);
            }
          }
        }
        __syncwarp();
      }
      if (dead) break;
#pragma unroll
      for (int s = 0; s < 4; ++s)
#pragma unroll
        for (int i = 0; i < NT; ++i) acc[s][i] = warp_sum(acc[s][i]);       // every lane holds the sums
      // the expert's output rounded as F.linear rounds it, times the pair's score, added to the token's sum: the
      // rounding points of `final_output[tok] += expert_output * weights`; expert a before expert b
#pragma unroll
      for (int side = 0; side < 2; ++side) {
        const int n_s = side == 0 ? n_a : n_b, off_s = side == 0 ? off_a : off_b;
#pragma unroll
        for (int i = 0; i < NT; ++i) {
          if (i >= n_s) break;
          const int tok = s_pos_tok[off_s + i];
          const float w = s_pos_w[off_s + i];
#pragma unroll
          for (int rr = 0; rr < 2; ++rr) {
            const float prod = rn<T>(__fmul_rn(rn<T>(acc[2 * side + rr][i]), w));
#pragma unroll
            for (int t = 0; t < NT; ++t)
              if (t == tok) out_acc[rr][t] = rn<T>(__fadd_rn(out_acc[rr][t], prod));
          }
        }
      }
    }
    if (dead) break;
#pragma unroll
    for (int rr = 0; rr < 2; ++rr)
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        if (lane == rr * NT + t && t < nt) {
          float o = out_acc[rr][t];
          const size_t at = (size_t)t * H + r0 + rr;
          if (p.residual != nullptr)      // plain load: with the fused norm CTA 0 wrote it in this launch
            o = rn<T>(__fadd_rn(Elem<T>::to_float(reinterpret_cast<const T*>(p.residual)[at]), o));
          reinterpret_cast<T*>(p.out)[at] = Elem<T>::from_float(o);
        }
      }
  }
  if (n_exp == 0 && !dead) {
    // nothing served: the block contributes zeros
    for (int c = blockIdx.x * S::THREADS + threadIdx.x; c < nt * H; c += (int)gridDim.x * S::THREADS) {
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
