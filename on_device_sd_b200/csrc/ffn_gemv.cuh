// K3a - grouped SwiGLU expert FFN as weight-streaming GEMV on CUDA cores, and K4 - the
// weighted combine.  Replaces expert_forward_with_weights (demo/src/layers/mlp.py:209-231 of
// the reference) run once per activated expert, and the `final_output[tok] += y * w`
// accumulation of _execute_moe_with_placement (demo/src/model/qwen3_runner.py:376).
//
// One persistent launch covers every activated expert of the layer: a work item is
// (expert, tile of output rows); each warp streams whole weight rows with 16-byte loads, keeps
// fp32 accumulators for up to NT tokens of that expert and reduces across the warp.  Rounding
// points follow the reference: gate, up, silu(gate), silu*up and the down projection are each
// rounded to the model dtype because the reference materialises each as a tensor.
#pragma once
#include "common.cuh"
#include "permute.cuh"
#include "tma.cuh"

namespace b200moe {

struct ExpertPtrs {
  const void* w[3];  // gate_proj [I,H], up_proj [I,H], down_proj [H,I]
  const void* s[3];  // int4 mode: bf16 scales per matrix, else null
};

struct FfnParams {
  const void* x;     // [T,H] activations
  void* h;           // [pairs, I] silu(gate)*up, in sorted-pair order
  void* y;           // [pairs, H] expert outputs, in sorted-pair order
  const ExpertPtrs* experts;  // table of this layer, [E]
  const int* offsets;
  const int* sorted_pair;
  const int* act_list;
  const int* n_act;
  int H, I, K;
};

// Bytes of one row segment, ring depth and warps per CTA of the streaming kernels.  Every warp
// owns a private ring of STAGES slots x 4 row segments in shared memory, fills it with 1-D bulk
// copies (TMA) and consumes it itself, so no cross-warp synchronisation exists at all.
template <int WARPS_, int SEG_, int STAGES_> struct GemvShape {
  static constexpr int WARPS = WARPS_, SEG = SEG_, STAGES = STAGES_;
  static constexpr int THREADS = WARPS * 32;
  static constexpr size_t SMEM = (size_t)WARPS * STAGES * 4 * SEG + (size_t)WARPS * STAGES * 8 + 128;
};

// DUAL = true : gate/up projections + SwiGLU epilogue; a unit = rows (r, r+1) of gate_proj and up_proj
// DUAL = false: down projection; a unit = rows (r .. r+3) of down_proj
// Units are dealt round-robin to the warps of the whole grid.  For every unit the warp streams the
// four rows once per pass of NT tokens; x (or h) comes through L1 with 16-byte loads.
template <typename T, int NT, bool DUAL, typename S>
__global__ void __launch_bounds__(S::THREADS, 1) ffn_gemv_kernel(FfnParams p, SlotTable st, int* status) {
  constexpr int RW = DUAL ? 2 : 4;
  constexpr int SEG = S::SEG, STAGES = S::STAGES;
  constexpr int SEG_ELEMS = SEG / (int)sizeof(T);
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  unsigned char* ring = smem_raw + (size_t)warp * STAGES * 4 * SEG;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw + (size_t)S::WARPS * STAGES * 4 * SEG) + warp * STAGES;

  const int Kdim = DUAL ? p.H : p.I;
  const int Rdim = DUAL ? p.I : p.H;
  pdl_wait();        // routing tables (and, for the down projection, h) come from the previous kernels
  pdl_trigger();
  const int gw = blockIdx.x * S::WARPS + warp;
  const int W = gridDim.x * S::WARPS;
  // When the down projection has too few four-row units to keep every warp of the grid busy
  // (single-token batches: 2 experts x 1024 units on 1184 warps), a unit becomes ONE row whose
  // four streams are the four quarters of K; the partial sums are added before the reduction.
  // Only for rows long enough that a quarter still fills a whole ring segment.
  const bool ksplit = !DUAL && (Kdim % 32 == 0) && Kdim * (int)sizeof(T) >= 4 * SEG && ((*p.n_act) * ((Rdim + RW - 1) / RW) < 6 * W);
  const int rows_per_unit = ksplit ? 1 : RW;
  const int row_bytes = (ksplit ? Kdim / 4 : Kdim) * (int)sizeof(T);   // bytes one stream covers
  const int full_row_bytes = Kdim * (int)sizeof(T);
  const int nseg = (row_bytes + SEG - 1) / SEG;
  const int groups = (Rdim + rows_per_unit - 1) / rows_per_unit;
  const int total_units = (*p.n_act) * groups;
  if (gw >= total_units) return;

  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < STAGES; ++i) mbar_init(&full[i], 1);
    mbar_fence_init();
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncwarp();
  const uint64_t policy = l2_policy_evict_first();

  // what a unit needs: my stream's row pointer (stream = lane & 3), the expert's pair range
  struct Unit { const unsigned char* row; int pos0, n, r0; };
  auto load_unit = [&](int u) {
    Unit q;
    const int e = p.act_list[u / groups];
    const ExpertPtrs ep = p.experts[st.slot[e]];
    q.r0 = (u % groups) * rows_per_unit;
    q.pos0 = p.offsets[e];
    q.n = p.offsets[e + 1] - q.pos0;
    const int sidx = lane & 3;
    const int row = min(q.r0 + (DUAL ? (sidx & 1) : (ksplit ? 0 : sidx)), Rdim - 1);
    const void* base = DUAL ? ep.w[sidx >> 1] : ep.w[2];
    q.row = reinterpret_cast<const unsigned char*>(base) + (size_t)row * full_row_bytes + (ksplit ? (size_t)sidx * row_bytes : 0);
    return q;
  };

  // ---- producer state: runs STAGES-1 stages ahead of the consumer, across unit boundaries ----
  int pu = gw, ps = 0, issued = 0;
  Unit pq = load_unit(pu);
  int p_stages = ((pq.n + NT - 1) / NT) * nseg;
  auto produce = [&]() {
    if (pu >= total_units) return;
    const int slot = issued % STAGES;
    const int seg = ps % nseg;
    const uint32_t bytes = (uint32_t)min(SEG, row_bytes - seg * SEG);
    if (lane == 0) mbar_expect_tx(&full[slot], 4 * bytes);
    __syncwarp();
    if (lane < 4) bulk_g2s(ring + (size_t)(slot * 4 + lane) * SEG, pq.row + (size_t)seg * SEG, bytes, &full[slot], policy);
    ++issued;
    if (++ps == p_stages) {
      pu += W;
      ps = 0;
      if (pu < total_units) {
        pq = load_unit(pu);
        p_stages = ((pq.n + NT - 1) / NT) * nseg;
      }
    }
  };
#pragma unroll
  for (int i = 0; i < STAGES - 1; ++i) produce();

  int consumed = 0;
  bool dead = false;
  for (int cu = gw; cu < total_units && !dead; cu += W) {
    const Unit cq = load_unit(cu);
    for (int c0 = 0; c0 < cq.n && !dead; c0 += NT) {
      const int nt = min(NT, cq.n - c0);
      const T* xr[NT];
#pragma unroll
      for (int tt = 0; tt < NT; ++tt) {
        const int pos = cq.pos0 + c0 + min(tt, nt - 1);
        if (DUAL) xr[tt] = reinterpret_cast<const T*>(p.x) + (size_t)(p.sorted_pair[pos] / p.K) * p.H;
        else xr[tt] = reinterpret_cast<const T*>(p.h) + (size_t)pos * p.I;
      }
      float acc[4][NT];
#pragma unroll
      for (int s = 0; s < 4; ++s)
#pragma unroll
        for (int tt = 0; tt < NT; ++tt) acc[s][tt] = 0.0f;

      for (int seg = 0; seg < nseg; ++seg) {
        produce();
        const int slot = consumed % STAGES;
        if (!mbar_wait_bounded(&full[slot], (uint32_t)(consumed / STAGES) & 1u)) {
          if (lane == 0) atomicOr(status, kDevWaitExpired);
          dead = true;
          break;
        }
        ++consumed;
        constexpr int CB = 8 * (int)sizeof(T);   // bytes of one 8-element chunk
        const int nchunk = min(SEG, row_bytes - seg * SEG) / CB;
        const unsigned char* sbase = ring + (size_t)slot * 4 * SEG;
        for (int cl = lane; cl < nchunk; cl += 32) {
          float wf[4][8];
#pragma unroll
          for (int s = 0; s < 4; ++s) {
            Chunk<T> wc;
            wc.from_smem(sbase + (size_t)s * SEG + (size_t)cl * CB);
            wc.unpack(wf[s]);
          }
          if (!ksplit) {
#pragma unroll
            for (int tt = 0; tt < NT; ++tt) {
              Chunk<T> xc;
              xc.template load<false>(xr[tt] + (size_t)seg * SEG_ELEMS + (size_t)cl * 8);
              float xf[8];
              xc.unpack(xf);
#pragma unroll
              for (int s = 0; s < 4; ++s)
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[s][tt] = fmaf(wf[s][i], xf[i], acc[s][tt]);
            }
          } else {
#pragma unroll
            for (int s = 0; s < 4; ++s)
#pragma unroll
              for (int tt = 0; tt < NT; ++tt) {
                Chunk<T> xc;
                xc.template load<false>(xr[tt] + (size_t)s * (Kdim / 4) + (size_t)seg * SEG_ELEMS + (size_t)cl * 8);
                float xf[8];
                xc.unpack(xf);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[s][tt] = fmaf(wf[s][i], xf[i], acc[s][tt]);
              }
          }
        }
        __syncwarp();   // every lane is done with the slot before it is refilled
      }
      if (dead) break;

      if (ksplit) {
#pragma unroll
        for (int tt = 0; tt < NT; ++tt) acc[0][tt] = (acc[0][tt] + acc[1][tt]) + (acc[2][tt] + acc[3][tt]);
      }
#pragma unroll
      for (int s = 0; s < 4; ++s)
#pragma unroll
        for (int tt = 0; tt < NT; ++tt) acc[s][tt] = warp_sum(acc[s][tt]);

      // epilogue: lane (rr*NT+tt) stores element (row r0+rr, token tt)
      if (DUAL) {
#pragma unroll
        for (int rr = 0; rr < 2; ++rr)
#pragma unroll
          for (int tt = 0; tt < NT; ++tt) {
            if (lane == rr * NT + tt && tt < nt && cq.r0 + rr < Rdim) {
              // stream order is (gate r, gate r+1, up r, up r+1)
              const float g = rn<T>(acc[rr][tt]);
              const float u = rn<T>(acc[2 + rr][tt]);
              const float sg = rn<T>(silu_f32(g));
              reinterpret_cast<T*>(p.h)[(size_t)(cq.pos0 + c0 + tt) * p.I + cq.r0 + rr] = Elem<T>::from_float(__fmul_rn(sg, u));
            }
          }
      } else {
#pragma unroll
        for (int rr = 0; rr < 4; ++rr)
#pragma unroll
          for (int tt = 0; tt < NT; ++tt) {
            if (lane == rr * NT + tt && tt < nt && cq.r0 + rr < Rdim && rr < rows_per_unit)
              reinterpret_cast<T*>(p.y)[(size_t)(cq.pos0 + c0 + tt) * p.H + cq.r0 + rr] = Elem<T>::from_float(acc[rr][tt]);
          }
      }
    }
  }
  if (dead) {
    // A wait ran out.  Copies issued earlier may still be in flight towards this warp's ring: give each
    // of them a short, bounded chance to land before the shared memory can pass to another CTA.
    for (int i = consumed; i < issued; ++i) mbar_wait_brief(&full[i % STAGES], (uint32_t)(i / STAGES) & 1u);
  }
}

// ---------------------------------------------------------------------------------------------
// K4 combine: out[t] = (residual[t] +) sum over the token's experts, in rank order, of
// y[pair] * score[pair], with every product and every partial sum rounded to the model dtype
// exactly where the reference's `final_output[tok] += expert_output * weights` rounds.
// ---------------------------------------------------------------------------------------------
struct CombineParams {
  const float* ypart;   // K-split down projection: fp32 slices [y_parts][pairs_cap][H], else null
  int y_parts, pairs_cap;
  const void* y;        // [pairs, H] sorted-pair order
  const int* inv;       // [T*K]
  const int64_t* ids64; // [T,K]
  const void* scores;   // [T,K]
  int scores_f32;       // scores are fp32 although activations are 16-bit
  const void* residual; // [T,H] or null
  void* out;            // [T,H]
  int T, H, K, E;
  // Expert-parallel mode (wait_flags != null): y is the return buffer that the owner ranks fill over
  // NVLink while this kernel may already be running; every CTA first waits (bounded) until all n_wait
  // flags have reached *epoch, and reads y through L2 only.
  const unsigned* wait_flags;
  const unsigned* epoch;
  int n_wait;
  long long wait_cycles;
  int* status;
};

template <typename T> __device__ __forceinline__ void store_chunk(T* dst, const float (&f)[8]);
template <> __device__ __forceinline__ void store_chunk<float>(float* dst, const float (&f)[8]) {
  reinterpret_cast<float4*>(dst)[0] = make_float4(f[0], f[1], f[2], f[3]);
  reinterpret_cast<float4*>(dst)[1] = make_float4(f[4], f[5], f[6], f[7]);
}
template <> __device__ __forceinline__ void store_chunk<__nv_bfloat16>(__nv_bfloat16* dst, const float (&f)[8]) {
  uint4 v;
  uint32_t* w = &v.x;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 t = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&t);
  }
  *reinterpret_cast<uint4*>(dst) = v;
}
template <> __device__ __forceinline__ void store_chunk<__half>(__half* dst, const float (&f)[8]) {
  uint4 v;
  uint32_t* w = &v.x;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __half2 t = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&t);
  }
  *reinterpret_cast<uint4*>(dst) = v;
}

constexpr int kCombineThreads = 256;

template <typename T> __global__ void __launch_bounds__(kCombineThreads) combine_kernel(CombineParams p, SlotTable st) {
  __shared__ int s_pos[kMaxTopK];
  __shared__ float s_w[kMaxTopK];
  __shared__ int s_rank[kMaxTopK];
  __shared__ int s_order[kMaxTopK];
  __shared__ int s_n;
  const int t = blockIdx.x;
  pdl_trigger();
  // The routing (ids, scores) and the inverse map were complete before the expert kernels could start (each of
  // them passes its own dependency wait before it lets its successor launch), so this prologue may run while
  // the down projection is still producing y: slot k of the token is read by thread k, thread 0 then orders
  // the live ones by rank.
  if (threadIdx.x < p.K) {
    const int k = threadIdx.x;
    const long long e = p.ids64[(size_t)t * p.K + k];
    int pos = -1, r = 0;
    float w = 0.0f;
    if (e >= 0 && e < p.E && st.slot[e] >= 0) {
      pos = p.inv[(size_t)t * p.K + k];
      w = p.scores_f32 ? reinterpret_cast<const float*>(p.scores)[(size_t)t * p.K + k]
                       : Elem<T>::to_float(reinterpret_cast<const T*>(p.scores)[(size_t)t * p.K + k]);
      r = st.rank[e];
    }
    s_pos[k] = pos; s_w[k] = w; s_rank[k] = r;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int n = 0;
    for (int k = 0; k < p.K; ++k) {
      if (s_pos[k] < 0) continue;
      int i = n++;
      while (i > 0 && s_rank[s_order[i - 1]] > s_rank[k]) {  // stable insertion: equal ranks keep slot order
        s_order[i] = s_order[i - 1];
        --i;
      }
      s_order[i] = k;
    }
    s_n = n;
  }
  pdl_wait();        // y comes from the down projection launched just before
  const bool remote_y = p.wait_flags != nullptr;
  if (remote_y && threadIdx.x >= 32 && threadIdx.x < 32 + p.n_wait) {
    if (!ep_wait_flag(p.wait_flags + (threadIdx.x - 32), *p.epoch, p.wait_cycles)) atomicOr(p.status, kDevWaitExpired);
  }
  __syncthreads();
  const int n = s_n;
  const T* y = reinterpret_cast<const T*>(p.y);
  for (int c = threadIdx.x; c < p.H / 8; c += kCombineThreads) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
    for (int j0 = 0; j0 < n; j0 += 4) {
      Chunk<T> yc[4];
      float w[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (j0 + u < n) {
          const int k = s_order[j0 + u];
          if (p.ypart == nullptr) {
            if (remote_y) yc[u].load_cg(y + (size_t)s_pos[k] * p.H + c * 8);
            else yc[u].template load<false>(y + (size_t)s_pos[k] * p.H + c * 8);
          }
          w[u] = s_w[k];
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (j0 + u < n) {
          float yf[8];
          if (p.ypart == nullptr) {
            yc[u].unpack(yf);
          } else {
            // the down projection's value is the sum of its K slices, added in slice order and
            // rounded to the model dtype once - the rounding point of the reference's F.linear
            const float* src = p.ypart + (size_t)s_pos[s_order[j0 + u]] * p.H + c * 8;
#pragma unroll
            for (int i = 0; i < 8; ++i) yf[i] = 0.0f;
            for (int sl0 = 0; sl0 < p.y_parts; sl0 += 4) {        // four slices' loads in flight, added in slice order
              float4 a[4], b[4];
#pragma unroll
              for (int q = 0; q < 4; ++q)
                if (sl0 + q < p.y_parts) {
                  const float* qp = src + (size_t)(sl0 + q) * p.pairs_cap * p.H;
                  a[q] = __ldg(reinterpret_cast<const float4*>(qp)); b[q] = __ldg(reinterpret_cast<const float4*>(qp) + 1);
                }
#pragma unroll
              for (int q = 0; q < 4; ++q)
                if (sl0 + q < p.y_parts) {
                  if (sl0 + q == 0) { yf[0] = a[q].x; yf[1] = a[q].y; yf[2] = a[q].z; yf[3] = a[q].w; yf[4] = b[q].x; yf[5] = b[q].y; yf[6] = b[q].z; yf[7] = b[q].w; }
                  else { yf[0] += a[q].x; yf[1] += a[q].y; yf[2] += a[q].z; yf[3] += a[q].w; yf[4] += b[q].x; yf[5] += b[q].y; yf[6] += b[q].z; yf[7] += b[q].w; }
                }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) yf[i] = rn<T>(yf[i]);
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            // __fmul_rn / __fadd_rn are never contracted into an FMA: the reference multiplies, then adds
            const float prod = p.scores_f32 ? __fmul_rn(yf[i], w[u]) : rn<T>(__fmul_rn(yf[i], w[u]));
            acc[i] = rn<T>(__fadd_rn(acc[i], prod));
          }
        }
      }
    }
    if (p.residual != nullptr) {
      Chunk<T> rc;
      rc.template load<false>(reinterpret_cast<const T*>(p.residual) + (size_t)t * p.H + c * 8);
      float rf[8];
      rc.unpack(rf);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = rn<T>(__fadd_rn(rf[i], acc[i]));
    }
    store_chunk<T>(reinterpret_cast<T*>(p.out) + (size_t)t * p.H + c * 8, acc);
  }
}

}  // namespace b200moe
