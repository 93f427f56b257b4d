// RMSNorm of the decoder layer that feeds the MoE block (post_attention_layernorm), optionally fused
// with the residual add in front of it.  Arithmetic and rounding points of the reference's
// RMSNorm.rms_forward / add_rms_forward (demo/src/layers/layernorm.py:21-36):
//   s = float(x) [+ float(residual)];  residual_out = T(s);  var = mean(s^2);
//   out = T( T(s * rsqrt(var + eps)) * weight )           (weight in the model dtype)
// One CTA per row, 16-byte loads; the row stays in registers between the two passes.  A 2 MB
// activation tile is far below what bounds this kernel (launch latency), so no more is done.
#pragma once
#include "common.cuh"

namespace b200moe {

constexpr int kNormThreads = 256;
constexpr int kNormMaxChunks = 8;     // chunks of 8 elements per thread: rows up to 16384 elements

struct NormParams {
  const void* x;
  const void* residual;      // may be null
  const void* weight;        // [H], model dtype
  void* out;
  void* residual_out;        // may be null; written only when residual is given
  float eps;
  int T, H;
};

template <typename T> __device__ __forceinline__ void norm_store_chunk(T* dst, const float (&f)[8]) {
  if constexpr (std::is_same<T, float>::value) {
    reinterpret_cast<float4*>(dst)[0] = make_float4(f[0], f[1], f[2], f[3]);
    reinterpret_cast<float4*>(dst)[1] = make_float4(f[4], f[5], f[6], f[7]);
  } else {
    T v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = Elem<T>::from_float(f[i]);
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(v);
  }
}

// One row, executed by ALL kNormThreads threads of a CTA (it synchronises).  Destinations that are null are
// skipped: out_a / out_b receive the normalised row (either may be shared memory), res_out the sum x + residual.
// rmsnorm_kernel and the router kernels (norm fused into their load of the token) both call this, so the
// fused form produces the same bits as the stand-alone one.
template <typename T>
__device__ __forceinline__ void rmsnorm_row(const T* x, const T* res, const T* w, float eps, int H, T* out_a, T* out_b, T* res_out,
                                            float* s_part, float* s_scale) {
  const int nch = H / 8;
  float v[kNormMaxChunks][8];
  float ss = 0.0f;
#pragma unroll
  for (int j = 0; j < kNormMaxChunks; ++j) {
    const int c = threadIdx.x + j * kNormThreads;
    if (c < nch) {
      Chunk<T> xc;
      xc.template load<false>(x + c * 8);
      xc.unpack(v[j]);
      if (res) {
        Chunk<T> rc;
        float rf[8];
        rc.template load<false>(res + c * 8);
        rc.unpack(rf);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[j][i] = __fadd_rn(v[j][i], rf[i]);
      }
      if (res_out) norm_store_chunk<T>(res_out + c * 8, v[j]);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss = fmaf(v[j][i], v[j][i], ss);
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.0f;
#pragma unroll
    for (int wi = 0; wi < kNormThreads / 32; ++wi) tot += s_part[wi];
    const float var = __fdiv_rn(tot, (float)H);
    *s_scale = __frcp_rn(__fsqrt_rn(__fadd_rn(var, eps)));     // 1 / sqrt: the two correctly rounded steps of torch's CPU rsqrt
  }
  __syncthreads();
  const float scale = *s_scale;
#pragma unroll
  for (int j = 0; j < kNormMaxChunks; ++j) {
    const int c = threadIdx.x + j * kNormThreads;
    if (c < nch) {
      Chunk<T> wc;
      float wf[8], o[8];
      wc.template load<false>(w + c * 8);
      wc.unpack(wf);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = __fmul_rn(rn<T>(__fmul_rn(v[j][i], scale)), wf[i]);
      if (out_a) norm_store_chunk<T>(out_a + c * 8, o);
      if (out_b) norm_store_chunk<T>(out_b + c * 8, o);
    }
  }
  __syncthreads();      // s_part / s_scale may be reused for the next row
}

template <typename T> __global__ void __launch_bounds__(kNormThreads) rmsnorm_kernel(NormParams p) {
  __shared__ float s_part[kNormThreads / 32];
  __shared__ float s_scale;
  pdl_wait();
  pdl_trigger();
  const size_t row = blockIdx.x;
  const T* res = p.residual ? reinterpret_cast<const T*>(p.residual) + row * p.H : nullptr;
  T* res_out = (p.residual && p.residual_out) ? reinterpret_cast<T*>(p.residual_out) + row * p.H : nullptr;
  rmsnorm_row<T>(reinterpret_cast<const T*>(p.x) + row * p.H, res, reinterpret_cast<const T*>(p.weight), p.eps, p.H,
                 reinterpret_cast<T*>(p.out) + row * p.H, nullptr, res_out, s_part, &s_scale);
}

}  // namespace b200moe
