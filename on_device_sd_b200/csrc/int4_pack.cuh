// K5 - int4 g128 packer / unpacker.  The reference has no quantised weights; the format is
// defined by this library: symmetric per-group scales over 128 consecutive `in` elements,
// scale = bf16(amax/7) (1 for an all-zero group), q = clamp(rne(w/scale), -8, 7), two values
// per byte (element 2j in the low nibble, 2j+1 in the high nibble, each stored as q+8).
#pragma once
#include "common.cuh"

namespace b200moe {

// one warp per (row, group): 4 consecutive elements per lane
template <typename T>
__global__ void pack_int4_kernel(const T* w, int out_f, int in_f, uint8_t* q, __nv_bfloat16* scales) {
  const int lane = threadIdx.x & 31;
  const long long gw = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int groups = in_f / 128;
  if (gw >= (long long)out_f * groups) return;
  const int row = (int)(gw / groups), g = (int)(gw % groups);
  const T* src = w + (size_t)row * in_f + g * 128 + lane * 4;
  float v[4];
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    // quantisation starts from the bf16-rounded weight whatever the storage type
    v[i] = __bfloat162float(__float2bfloat16_rn(Elem<T>::to_float(src[i])));
    amax = fmaxf(amax, fabsf(v[i]));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  __nv_bfloat16 sb = __float2bfloat16_rn(__fdiv_rn(amax, 7.0f));
  if (amax == 0.0f) sb = __float2bfloat16_rn(1.0f);
  const float s = __bfloat162float(sb);
  uint32_t nib[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float r = rintf(__fdiv_rn(v[i], s));
    r = fminf(fmaxf(r, -8.0f), 7.0f);
    nib[i] = (uint32_t)((int)r + 8);
  }
  const uint16_t two = (uint16_t)(nib[0] | (nib[1] << 4) | (nib[2] << 8) | (nib[3] << 12));
  *reinterpret_cast<uint16_t*>(q + (size_t)row * (in_f / 2) + g * 64 + lane * 2) = two;
  if (lane == 0) scales[(size_t)row * groups + g] = sb;
}

// one thread per byte (two elements)
template <typename T>
__global__ void unpack_int4_kernel(const uint8_t* q, const __nv_bfloat16* scales, int out_f, int in_f,
                                   int8_t* q_out, T* w_out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nbytes = (long long)out_f * (in_f / 2);
  if (i >= nbytes) return;
  const int row = (int)(i / (in_f / 2)), jb = (int)(i % (in_f / 2));
  const uint8_t b = q[i];
  const int q0 = (int)(b & 0xf) - 8, q1 = (int)(b >> 4) - 8;
  const size_t o = (size_t)row * in_f + 2 * jb;
  if (q_out != nullptr) { q_out[o] = (int8_t)q0; q_out[o + 1] = (int8_t)q1; }
  if (w_out != nullptr) {
    const float s = __bfloat162float(scales[(size_t)row * (in_f / 128) + (2 * jb) / 128]);
    w_out[o] = Elem<T>::from_float(__fmul_rn(s, (float)q0));
    w_out[o + 1] = Elem<T>::from_float(__fmul_rn(s, (float)q1));
  }
}

}  // namespace b200moe
