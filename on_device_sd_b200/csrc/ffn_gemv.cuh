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

constexpr int kGemvThreads = 256;
constexpr int kGemvWarps = kGemvThreads / 32;
constexpr int kGemvStreams = 4;   // weight rows a warp streams concurrently
constexpr int kGemvDepth = 3;     // register stages of the load pipeline

// DUAL = true : gate/up projections + SwiGLU epilogue, 2 rows x 2 matrices per warp, 16 rows per item
// DUAL = false: down projection, 4 rows per warp, 32 rows per item
template <typename T, int NT, bool DUAL>
__global__ void __launch_bounds__(kGemvThreads, 2) ffn_gemv_kernel(FfnParams p, SlotTable st) {
  constexpr int RW = DUAL ? 2 : 4;                 // output rows per warp
  constexpr int ROWS_PER_ITEM = RW * kGemvWarps;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int Kdim = DUAL ? p.H : p.I;               // reduction length
  const int Rdim = DUAL ? p.I : p.H;               // output rows of the matrix
  const int nch = Kdim / 8;
  const int nj = (nch + 31) / 32;
  const int tiles = (Rdim + ROWS_PER_ITEM - 1) / ROWS_PER_ITEM;
  const int total = (*p.n_act) * tiles;

  for (int item = blockIdx.x; item < total; item += gridDim.x) {
    const int e = p.act_list[item / tiles];
    const int tile = item % tiles;
    const int slot = st.slot[e];
    const ExpertPtrs ep = p.experts[slot];
    const int pos0 = p.offsets[e];
    const int n = p.offsets[e + 1] - pos0;
    const int r0 = tile * ROWS_PER_ITEM + warp * RW;

    const T* wp[kGemvStreams];
#pragma unroll
    for (int s = 0; s < kGemvStreams; ++s) {
      const int row = min(r0 + (DUAL ? (s & 1) : s), Rdim - 1);
      const T* base = reinterpret_cast<const T*>(DUAL ? ep.w[s >> 1] : ep.w[2]);
      wp[s] = base + (size_t)row * Kdim;
    }

    for (int c0 = 0; c0 < n; c0 += NT) {
      const int nt = min(NT, n - c0);
      const T* xr[NT];
#pragma unroll
      for (int tt = 0; tt < NT; ++tt) {
        const int pos = pos0 + c0 + min(tt, nt - 1);
        if (DUAL) xr[tt] = reinterpret_cast<const T*>(p.x) + (size_t)(p.sorted_pair[pos] / p.K) * p.H;
        else xr[tt] = reinterpret_cast<const T*>(p.h) + (size_t)pos * p.I;
      }
      float acc[kGemvStreams][NT];
#pragma unroll
      for (int s = 0; s < kGemvStreams; ++s)
#pragma unroll
        for (int tt = 0; tt < NT; ++tt) acc[s][tt] = 0.0f;

      Chunk<T> buf[kGemvDepth][kGemvStreams];
      auto issue = [&](Chunk<T>(&dst)[kGemvStreams], int c) {
        if (c < nch) {
#pragma unroll
          for (int s = 0; s < kGemvStreams; ++s) dst[s].template load<true>(wp[s] + (size_t)c * 8);
        }
      };
      auto consume = [&](const Chunk<T>(&src)[kGemvStreams], int c) {
        if (c < nch) {
          float wf[kGemvStreams][8];
#pragma unroll
          for (int s = 0; s < kGemvStreams; ++s) src[s].unpack(wf[s]);
#pragma unroll
          for (int tt = 0; tt < NT; ++tt) {
            Chunk<T> xc;
            xc.template load<false>(xr[tt] + (size_t)c * 8);
            float xf[8];
            xc.unpack(xf);
#pragma unroll
            for (int s = 0; s < kGemvStreams; ++s)
#pragma unroll
              for (int i = 0; i < 8; ++i) acc[s][tt] = fmaf(wf[s][i], xf[i], acc[s][tt]);
          }
        }
      };
#pragma unroll
      for (int d = 0; d < kGemvDepth - 1; ++d) issue(buf[d], d * 32 + lane);
      for (int j = 0; j < nj; j += kGemvDepth) {
#pragma unroll
        for (int d = 0; d < kGemvDepth; ++d) {
          issue(buf[(d + kGemvDepth - 1) % kGemvDepth], (j + d + kGemvDepth - 1) * 32 + lane);
          consume(buf[d], (j + d) * 32 + lane);
        }
      }

#pragma unroll
      for (int s = 0; s < kGemvStreams; ++s)
#pragma unroll
        for (int tt = 0; tt < NT; ++tt) acc[s][tt] = warp_sum(acc[s][tt]);

      // epilogue: lane (rr*NT+tt) stores element (row r0+rr, token tt)
      if (DUAL) {
#pragma unroll
        for (int rr = 0; rr < 2; ++rr)
#pragma unroll
          for (int tt = 0; tt < NT; ++tt) {
            if (lane == rr * NT + tt && tt < nt && r0 + rr < Rdim) {
              const float g = rn<T>(acc[rr][tt]);
              const float u = rn<T>(acc[2 + rr][tt]);
              const float sg = rn<T>(silu_f32(g));
              reinterpret_cast<T*>(p.h)[(size_t)(pos0 + c0 + tt) * p.I + r0 + rr] = Elem<T>::from_float(__fmul_rn(sg, u));
            }
          }
      } else {
#pragma unroll
        for (int rr = 0; rr < 4; ++rr)
#pragma unroll
          for (int tt = 0; tt < NT; ++tt) {
            if (lane == rr * NT + tt && tt < nt && r0 + rr < Rdim)
              reinterpret_cast<T*>(p.y)[(size_t)(pos0 + c0 + tt) * p.H + r0 + rr] = Elem<T>::from_float(acc[rr][tt]);
          }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// K4 combine: out[t] = (residual[t] +) sum over the token's experts, in rank order, of
// y[pair] * score[pair], with every product and every partial sum rounded to the model dtype
// exactly where the reference's `final_output[tok] += expert_output * weights` rounds.
// ---------------------------------------------------------------------------------------------
struct CombineParams {
  const void* y;        // [pairs, H] sorted-pair order
  const int* inv;       // [T*K]
  const int64_t* ids64; // [T,K]
  const void* scores;   // [T,K]
  int scores_f32;       // scores are fp32 although activations are 16-bit
  const void* residual; // [T,H] or null
  void* out;            // [T,H]
  int T, H, K, E;
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
  __shared__ int s_n;
  const int t = blockIdx.x;
  if (threadIdx.x == 0) {
    int rk[kMaxTopK];
    int n = 0;
    for (int k = 0; k < p.K; ++k) {
      const long long e = p.ids64[(size_t)t * p.K + k];
      if (e < 0 || e >= p.E || st.slot[e] < 0) continue;
      const int pos = p.inv[(size_t)t * p.K + k];
      if (pos < 0) continue;
      const float w = p.scores_f32 ? reinterpret_cast<const float*>(p.scores)[(size_t)t * p.K + k]
                                   : Elem<T>::to_float(reinterpret_cast<const T*>(p.scores)[(size_t)t * p.K + k]);
      const int r = st.rank[e];
      int i = n++;
      while (i > 0 && rk[i - 1] > r) {  // stable insertion: equal ranks keep slot order
        rk[i] = rk[i - 1]; s_pos[i] = s_pos[i - 1]; s_w[i] = s_w[i - 1];
        --i;
      }
      rk[i] = r; s_pos[i] = pos; s_w[i] = w;
    }
    s_n = n;
  }
  __syncthreads();
  const int n = s_n;
  const T* y = reinterpret_cast<const T*>(p.y);
  for (int c = threadIdx.x; c < p.H / 8; c += kCombineThreads) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
    for (int j = 0; j < n; ++j) {
      Chunk<T> yc;
      yc.template load<false>(y + (size_t)s_pos[j] * p.H + c * 8);
      float yf[8];
      yc.unpack(yf);
      const float w = s_w[j];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        // __fmul_rn / __fadd_rn are never contracted into an FMA: the reference multiplies, then adds
        const float prod = p.scores_f32 ? __fmul_rn(yf[i], w) : rn<T>(__fmul_rn(yf[i], w));
        acc[i] = rn<T>(__fadd_rn(acc[i], prod));
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
