// Shared device helpers: element-type traits, 16-byte chunk loads, rounding points.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200moe {

constexpr int kMaxExperts = 256;
constexpr int kMaxTopK = 32;

// ---------------------------------------------------------------------------------------------
// Element types.  `rn<T>(f)` is the rounding point "a torch op wrote its fp32 result into a
// tensor of dtype T", returned as float again.
// ---------------------------------------------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<float> {
  static constexpr int kBytes = 4;
  __device__ static __forceinline__ float to_float(float v) { return v; }
  __device__ static __forceinline__ float from_float(float v) { return v; }
};
template <> struct Elem<__half> {
  static constexpr int kBytes = 2;
  __device__ static __forceinline__ float to_float(__half v) { return __half2float(v); }
  __device__ static __forceinline__ __half from_float(float v) { return __float2half_rn(v); }
};
template <> struct Elem<__nv_bfloat16> {
  static constexpr int kBytes = 2;
  __device__ static __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
  __device__ static __forceinline__ __nv_bfloat16 from_float(float v) { return __float2bfloat16_rn(v); }
};

template <typename T> __device__ __forceinline__ float rn(float v) {
  return Elem<T>::to_float(Elem<T>::from_float(v));
}
template <> __device__ __forceinline__ float rn<float>(float v) { return v; }

// ---------------------------------------------------------------------------------------------
// A "chunk" is 8 consecutive elements: one 16-byte load for 16-bit types, two for fp32.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  // weights are read exactly once: keep them out of L1
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ldg_cached(const void* p) {
  return __ldg(reinterpret_cast<const uint4*>(p));
}

template <typename T> struct Chunk;  // raw registers of 8 elements

template <> struct Chunk<float> {
  uint4 a, b;
  template <bool kStream> __device__ __forceinline__ void load(const float* p) {
    if (kStream) { a = ldg_stream(p); b = ldg_stream(p + 4); }
    else { a = ldg_cached(p); b = ldg_cached(p + 4); }
  }
  __device__ __forceinline__ void load_cg(const float* p) {     // through L2 only: data another GPU may have just written
    a = __ldcg(reinterpret_cast<const uint4*>(p)); b = __ldcg(reinterpret_cast<const uint4*>(p) + 1);
  }
  __device__ __forceinline__ void from_smem(const void* p) {   // 32 bytes
    a = reinterpret_cast<const uint4*>(p)[0];
    b = reinterpret_cast<const uint4*>(p)[1];
  }
  __device__ __forceinline__ void zero() { a = make_uint4(0, 0, 0, 0); b = a; }
  __device__ __forceinline__ void unpack(float (&f)[8]) const {
    f[0] = __uint_as_float(a.x); f[1] = __uint_as_float(a.y); f[2] = __uint_as_float(a.z); f[3] = __uint_as_float(a.w);
    f[4] = __uint_as_float(b.x); f[5] = __uint_as_float(b.y); f[6] = __uint_as_float(b.z); f[7] = __uint_as_float(b.w);
  }
};

template <> struct Chunk<__nv_bfloat16> {
  uint4 a;
  template <bool kStream> __device__ __forceinline__ void load(const __nv_bfloat16* p) {
    a = kStream ? ldg_stream(p) : ldg_cached(p);
  }
  __device__ __forceinline__ void load_cg(const void* p) { a = __ldcg(reinterpret_cast<const uint4*>(p)); }
  __device__ __forceinline__ void from_smem(const void* p) { a = *reinterpret_cast<const uint4*>(p); }
  __device__ __forceinline__ void zero() { a = make_uint4(0, 0, 0, 0); }
  __device__ __forceinline__ void unpack(float (&f)[8]) const {
    // bf16 -> fp32 is a 16-bit shift
    f[0] = __uint_as_float(a.x << 16); f[1] = __uint_as_float(a.x & 0xffff0000u);
    f[2] = __uint_as_float(a.y << 16); f[3] = __uint_as_float(a.y & 0xffff0000u);
    f[4] = __uint_as_float(a.z << 16); f[5] = __uint_as_float(a.z & 0xffff0000u);
    f[6] = __uint_as_float(a.w << 16); f[7] = __uint_as_float(a.w & 0xffff0000u);
  }
};

template <> struct Chunk<__half> {
  uint4 a;
  template <bool kStream> __device__ __forceinline__ void load(const __half* p) {
    a = kStream ? ldg_stream(p) : ldg_cached(p);
  }
  __device__ __forceinline__ void load_cg(const void* p) { a = __ldcg(reinterpret_cast<const uint4*>(p)); }
  __device__ __forceinline__ void from_smem(const void* p) { a = *reinterpret_cast<const uint4*>(p); }
  __device__ __forceinline__ void zero() { a = make_uint4(0, 0, 0, 0); }
  __device__ __forceinline__ void unpack(float (&f)[8]) const {
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      f[2 * i] = t.x; f[2 * i + 1] = t.y;
    }
  }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// SiLU as torch evaluates it for a low-precision tensor: fp32 math, x / (1 + exp(-x)).
__device__ __forceinline__ float silu_f32(float g) { return g / (1.0f + expf(-g)); }

// Programmatic dependent launch: every kernel of the chain is launched with the
// programmatic-stream-serialization attribute, may start while its predecessor is still
// running, and must call pdl_wait() before it touches anything the predecessor (or, through the
// chain, any earlier kernel) produces or still reads.  pdl_trigger() lets the successor launch.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// Flags that another GPU writes (expert-parallel exchange, ep.cuh): system-scope release / acquire.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_cg16(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }

// Waits until the flag has reached `epoch` (signed distance, so the counter may wrap), for at most
// `limit` cycles.  The flag lives in this GPU's memory; a peer writes it.
__device__ __forceinline__ bool ep_wait_flag(const unsigned* flag, unsigned epoch, long long limit) {
  if ((int)(ld_acquire_sys(flag) - epoch) >= 0) return true;
  const long long t0 = clock64();
  for (;;) {
    __nanosleep(100);
    if ((int)(ld_acquire_sys(flag) - epoch) >= 0) return true;
    if (clock64() - t0 > limit) return false;
  }
}

// Device status word bits (mirrors B200MOE_DEV_* of the public header).
constexpr int kDevBadExpertId = 1;
constexpr int kDevBadOffsets = 2;
constexpr int kDevWaitExpired = 4;

}  // namespace b200moe
