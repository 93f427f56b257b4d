// K3d - grouped SwiGLU expert FFN over int4 g128 weights on the tcgen05 tensor cores.
// Same contract and numerics as ffn_int4.cuh (the dequantised weight is bf16(scale * q), bit for
// bit), but the tokens ride the MMA's N dimension, so the per-weight work no longer grows with the
// number of tokens an expert holds: used for batches of two or more tokens.
//
// Data flow per stage of 128 k (= one scale group):
//   TMA box (128 rows x 64 bytes of nibbles, 64-byte swizzle) -> shared-memory ring (8 stages)
//   -> 8 dequant warps: thread (row, half) reads 32 bytes, converts 64 nibbles in registers
//      (lop3 magic, exact subtraction, one bf16 multiplication by the group scale) and stores them
//      as the bf16 A tile of the MMA in the canonical 128-byte-swizzle layout (two 64-k atoms)
//   -> tcgen05.mma (A and B from shared memory, accumulator in TMEM), epilogue as in ffn_umma.cuh.
// lop3 extracts nibble pairs (t, t+4); instead of re-ordering the weights, the tokens carry the
// same permutation inside every group of 8 k: a small kernel writes a permuted copy of x once per
// call, and the gate/up epilogue stores h permuted, so the loader warps stay plain cp.async.
//
//   warp 0      TMA producer            warp 1      MMA issuer + TMEM owner
//   warps 2-5   token-tile loaders      warps 6-13  dequant
//   warps 14-17 epilogue
#pragma once
#include <cuda.h>

#include "common.cuh"
#include "ffn_gemv.cuh"
#include "ffn_umma.cuh"
#include "tma.cuh"

namespace b200moe {

constexpr int kI4uThreads = 18 * 32;
constexpr int kI4uLoaders = 128;
constexpr int kI4uDequant = 256;
constexpr int kI4uWStages = 6;            // ring of packed tiles (8 KB each): the bytes in flight from HBM
constexpr int kI4uWTile = 128 * 64;       // 128 rows x 64 bytes = 128 k of nibbles
constexpr int kI4uATile = 2 * 16384;      // bf16 A tile: two atoms of 128 rows x 128 bytes
constexpr int kI4uBK = 128;

// Shared memory: the packed-tile ring, the bf16 A ring (32 KB per stage, few stages) and a separate,
// deeper ring for the small token tiles - the token tiles come from L2 with cp.async and need
// several stages in flight to hide that latency.
template <int NMAX> struct I4uShape {
  static constexpr int B_TILE = 2 * NMAX * 128;                 // two 64-k atoms
  static constexpr int A_STAGES = NMAX <= 32 ? 4 : (NMAX == 64 ? 3 : 2);
  static constexpr int EX_BYTES = 64 * 17 * 4;
  static constexpr int PTR_BYTES = 128 * 8;
  static constexpr int FIXED = 1024 + kI4uWStages * kI4uWTile + A_STAGES * kI4uATile + EX_BYTES + PTR_BYTES + 512;
  static constexpr int B_FIT = (227 * 1024 - FIXED) / B_TILE;
  static constexpr int B_STAGES = B_FIT > 8 ? 8 : B_FIT;
  static constexpr int LOADER_LAG = B_STAGES >= 6 ? 4 : (B_STAGES - 2 > 0 ? B_STAGES - 2 : 1);
  static constexpr size_t SMEM = (size_t)FIXED + (size_t)B_STAGES * B_TILE;
  static constexpr int TMEM_COLS = (2 * NMAX) < 32 ? 32 : 2 * NMAX;
  static_assert(B_STAGES >= 3, "token tile too large for the shared-memory budget");
};

struct I4uParams {
  FfnParams f;
  const void* xperm;          // [T,H] copy of x with every group of 8 k stored as k0,k4,k1,k5,k2,k6,k3,k7
  const CUtensorMap* tmaps;   // [E][3]: uint8 maps with {64 B, 64 rows} (gate, up) / {64 B, 128 rows} (down) boxes, 64-byte swizzle
  int* status;
};

// 8 nibbles -> 4 words holding (q_t, q_{t+4}) * scale as bf16 pairs, t = 0..3 (see ffn_int4.cuh)
__device__ __forceinline__ void i4u_dequant8(uint32_t w, __nv_bfloat162 scale2, uint32_t (&p)[4]) {
  const __nv_bfloat162 bias = __nv_bfloat162(__float2bfloat16_rn(136.0f), __float2bfloat16_rn(136.0f));
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    uint32_t v;
    asm("lop3.b32 %0, %1, 0x000F000F, 0x43004300, 0xEA;" : "=r"(v) : "r"(w >> (4 * t)));
    const __nv_bfloat162 d = __hmul2(__hsub2(*reinterpret_cast<__nv_bfloat162*>(&v), bias), scale2);
    p[t] = *reinterpret_cast<const uint32_t*>(&d);
  }
}

template <int NMAX, bool DUAL>
__global__ void __launch_bounds__(kI4uThreads, 1) ffn_int4_umma_kernel(I4uParams ip, SlotTable st) {
  using S = I4uShape<NMAX>;
  constexpr int STAGES = S::A_STAGES;       // bf16 A ring
  constexpr int BSTAGES = S::B_STAGES;      // token-tile ring
  constexpr int B_TILE = S::B_TILE;
  constexpr int TILE_ROWS = DUAL ? 64 : 128;
  const FfnParams& p = ip.f;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  unsigned char* Ws = smem;                                           // packed tiles
  unsigned char* As = Ws + (size_t)kI4uWStages * kI4uWTile;          // bf16 A tiles
  unsigned char* Bs = As + (size_t)STAGES * kI4uATile;               // token tiles
  float* ex = reinterpret_cast<float*>(Bs + (size_t)BSTAGES * B_TILE);
  const __nv_bfloat16** rowptr = reinterpret_cast<const __nv_bfloat16**>(reinterpret_cast<unsigned char*>(ex) + S::EX_BYTES);
  uint64_t* w_full = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(rowptr) + S::PTR_BYTES);
  uint64_t* w_empty = w_full + kI4uWStages;
  uint64_t* full = w_empty + kI4uWStages;     // A stage written by the dequant warps
  uint64_t* empty = full + STAGES;
  uint64_t* b_full = empty + STAGES;           // token tile landed
  uint64_t* b_empty = b_full + BSTAGES;
  uint64_t* acc_full = b_empty + BSTAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int Kdim = DUAL ? p.H : p.I;
  const int Rdim = DUAL ? p.I : p.H;
  const int nkb = Kdim / kI4uBK;                 // K is a multiple of 128 for int4 weights
  const int tiles = (Rdim + TILE_ROWS - 1) / TILE_ROWS;
  const int sgroups = Kdim / 128;

  if (DUAL) pdl_wait();
  pdl_trigger();
  const int total = (*p.n_act) * tiles;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kI4uWStages; ++i) { mbar_init(&w_full[i], 1); mbar_init(&w_empty[i], kI4uDequant); }
    for (int i = 0; i < STAGES; ++i) { mbar_init(&full[i], kI4uDequant); mbar_init(&empty[i], 1); }
    for (int i = 0; i < BSTAGES; ++i) { mbar_init(&b_full[i], kI4uLoaders); mbar_init(&b_empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 128); }
    *abort_flag = 0;
    mbar_fence_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_holder)), "r"((uint32_t)S::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------ TMA producer: packed tiles ------------------------------
    if (lane == 0) {
      const uint64_t policy = l2_policy_evict_first();
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total && ok; item += gridDim.x) {
        const int e = p.act_list[item / tiles];
        const int tile = item % tiles;
        const int slot = st.slot[e];
        const int n = p.offsets[e + 1] - p.offsets[e];
        const CUtensorMap* m0 = ip.tmaps + (size_t)slot * 3 + (DUAL ? 0 : 2);
        const CUtensorMap* m1 = ip.tmaps + (size_t)slot * 3 + 1;
        tensormap_acquire(m0);
        if (DUAL) tensormap_acquire(m1);
        for (int c0 = 0; c0 < n && ok; c0 += NMAX) {
          for (int kb = 0; kb < nkb; ++kb) {
            if (!wait_or_abort(&w_empty[s], ph ^ 1, abort_flag)) { ok = false; break; }
            mbar_expect_tx(&w_full[s], kI4uWTile);
            unsigned char* dst = Ws + (size_t)s * kI4uWTile;
            if (DUAL) {
              tma_load_2d(dst, m0, kb * 64, tile * 64, &w_full[s], policy);
              tma_load_2d(dst + 4096, m1, kb * 64, tile * 64, &w_full[s], policy);
            } else {
              tma_load_2d(dst, m0, kb * 64, tile * 128, &w_full[s], policy);
            }
            if (++s == kI4uWStages) { s = 0; ph ^= 1; }
          }
        }
      }
      if (!ok) atomicOr(ip.status, kDevWaitExpired);
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      int s = 0, sb = 0, job = 0;
      uint32_t ph = 0, phb = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total && ok; item += gridDim.x) {
        const int e = p.act_list[item / tiles];
        const int n = p.offsets[e + 1] - p.offsets[e];
        for (int c0 = 0; c0 < n && ok; c0 += NMAX, ++job) {
          const int npad = (min(NMAX, n - c0) + 15) & ~15;
          const uint32_t idesc = umma_idesc_bf16(npad);
          const int b = job & 1;
          if (!wait_or_abort(&acc_empty[b], ((job >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + (uint32_t)(b * NMAX);
          for (int kb = 0; kb < nkb; ++kb) {
            if (!wait_or_abort(&full[s], ph, abort_flag) || !wait_or_abort(&b_full[sb], phb, abort_flag)) { ok = false; break; }
            tc_fence_after();
#pragma unroll
            for (int atom = 0; atom < 2; ++atom) {
              const uint64_t adesc = umma_desc_sw128(smem_addr(As + (size_t)s * kI4uATile + atom * 16384));
              const uint64_t bdesc = umma_desc_sw128(smem_addr(Bs + (size_t)sb * B_TILE + atom * NMAX * 128));
#pragma unroll
              for (int k = 0; k < 4; ++k)
                tc_mma_bf16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > 0 || atom > 0 || k > 0) ? 1u : 0u);
            }
            tc_commit(&empty[s]);
            tc_commit(&b_empty[sb]);
            if (++s == STAGES) { s = 0; ph ^= 1; }
            if (++sb == BSTAGES) { sb = 0; phb ^= 1; }
          }
          if (ok) tc_commit(&acc_full[b]);
        }
      }
      if (!ok) atomicOr(ip.status, kDevWaitExpired);
    }
  } else if (warp < 6) {
    // ------------------------------ token-tile loaders (cp.async, inputs already k-permuted) ------------------------------
    const int tl = threadIdx.x - 64;          // 0..127
    constexpr int LOADER_LAG = S::LOADER_LAG;
    if (!DUAL) pdl_wait();                    // h must be complete
    int s = 0, lag_s = 0, issued = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < total; item += gridDim.x) {   // runs to the end even after a failed wait (named barriers)
      const int e = p.act_list[item / tiles];
      const int pos0 = p.offsets[e];
      const int n = p.offsets[e + 1] - pos0;
      for (int c0 = 0; c0 < n; c0 += NMAX) {
        const int nt = min(NMAX, n - c0);
        const int npad = (nt + 15) & ~15;
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (tl < npad) {
          const int pos = pos0 + c0 + min(tl, nt - 1);
          rowptr[tl] = DUAL ? reinterpret_cast<const __nv_bfloat16*>(ip.xperm) + (size_t)(p.sorted_pair[pos] / p.K) * p.H
                            : reinterpret_cast<const __nv_bfloat16*>(p.h) + (size_t)pos * p.I;
        }
        asm volatile("bar.sync 2, 128;" ::: "memory");
        for (int kb = 0; kb < nkb && ok; ++kb) {
          if (!wait_or_abort(&b_empty[s], ph ^ 1, abort_flag)) { ok = false; break; }
          unsigned char* bt = Bs + (size_t)s * B_TILE;
          for (int id = tl; id < npad * 16; id += kI4uLoaders) {
            const int r = id >> 4, c = id & 15;           // chunk c of 16: atom c>>3, 16-byte slot c&7
            const bool live = r < nt;
            const __nv_bfloat16* src = rowptr[r];
            cp_async_16(bt + (c >> 3) * NMAX * 128 + r * 128 + (((c & 7) ^ (r & 7)) << 4),
                        live ? (const void*)(src + kb * kI4uBK + c * 8) : (const void*)src, live ? 16u : 0u);
          }
          cp_async_commit();
          ++issued;
          if (issued > LOADER_LAG) {
            cp_async_wait<LOADER_LAG>();
            fence_proxy_async();
            mbar_arrive(&b_full[lag_s]);
            if (++lag_s == BSTAGES) lag_s = 0;
          }
          if (++s == BSTAGES) { s = 0; ph ^= 1; }
        }
      }
    }
    cp_async_wait<0>();
    fence_proxy_async();
    for (int q = min(issued, LOADER_LAG); q > 0; --q) {
      mbar_arrive(&b_full[lag_s]);
      if (++lag_s == BSTAGES) lag_s = 0;
    }
    if (!ok && tl == 0) atomicOr(ip.status, kDevWaitExpired);
  } else if (warp < 14) {
    // ------------------------------ dequant: packed tile -> bf16 A tile ------------------------------
    const int dt = threadIdx.x - 192;         // 0..255
    const int row = dt & 127, half = dt >> 7; // row of the tile, which 64 k of the 128
    int ws = 0, s = 0;
    uint32_t wph = 0, ph = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < total && ok; item += gridDim.x) {
      const int e = p.act_list[item / tiles];
      const int tile = item % tiles;
      const ExpertPtrs ep = p.experts[st.slot[e]];
      const int n = p.offsets[e + 1] - p.offsets[e];
      // scale row of this thread: DUAL rows 0-63 are gate rows, 64-127 the same rows of up
      const __nv_bfloat16* sc;
      if (DUAL) {
        const int gr = min(tile * 64 + (row & 63), Rdim - 1);
        sc = reinterpret_cast<const __nv_bfloat16*>(ep.s[row >> 6]) + (size_t)gr * sgroups;
      } else {
        const int gr = min(tile * 128 + row, Rdim - 1);
        sc = reinterpret_cast<const __nv_bfloat16*>(ep.s[2]) + (size_t)gr * sgroups;
      }
      for (int c0 = 0; c0 < n && ok; c0 += NMAX) {
        __nv_bfloat16 sv = sc[0];
        for (int kb = 0; kb < nkb; ++kb) {
          const __nv_bfloat16 sv_next = sc[min(kb + 1, nkb - 1)];   // next group's scale, fetched a stage ahead
          if (!wait_or_abort(&w_full[ws], wph, abort_flag)) { ok = false; break; }
          // 64-byte swizzle of the TMA box: 16-byte slot c of row r sits at c ^ ((r >> 1) & 3)
          const unsigned char* wrow = Ws + (size_t)ws * kI4uWTile + row * 64;
          const int sw = (row >> 1) & 3;
          const uint4 q0 = *reinterpret_cast<const uint4*>(wrow + (((half * 2 + 0) ^ sw) << 4));
          const uint4 q1 = *reinterpret_cast<const uint4*>(wrow + (((half * 2 + 1) ^ sw) << 4));
          mbar_arrive(&w_empty[ws]);
          if (++ws == kI4uWStages) { ws = 0; wph ^= 1; }
          if (!wait_or_abort(&empty[s], ph ^ 1, abort_flag)) { ok = false; break; }
          unsigned char* arow = As + (size_t)s * kI4uATile + half * 16384 + row * 128;
          const __nv_bfloat162 s2 = __nv_bfloat162(sv, sv);
          const uint32_t words[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
          for (int c = 0; c < 8; ++c) {       // word c = 8 k = one 16-byte chunk of the bf16 row
            uint32_t o[4];
            i4u_dequant8(words[c], s2, o);
            *reinterpret_cast<uint4*>(arow + ((c ^ (row & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
          }
          fence_proxy_async();
          mbar_arrive(&full[s]);
          if (++s == STAGES) { s = 0; ph ^= 1; }
          sv = sv_next;
        }
      }
    }
    if (!ok && dt == 0) atomicOr(ip.status, kDevWaitExpired);
  } else {
    // ------------------------------ epilogue ------------------------------
    const int q = warp & 3;                       // TMEM lane quarter this warp may read
    const int et = threadIdx.x - 448;             // 0..127
    int job = 0;
    bool ok = true;
    __nv_bfloat16* hout = reinterpret_cast<__nv_bfloat16*>(p.h);
    __nv_bfloat16* yout = reinterpret_cast<__nv_bfloat16*>(p.y);
    for (int item = blockIdx.x; item < total && ok; item += gridDim.x) {
      const int e = p.act_list[item / tiles];
      const int tile = item % tiles;
      const int pos0 = p.offsets[e];
      const int n = p.offsets[e + 1] - pos0;
      for (int c0 = 0; c0 < n && ok; c0 += NMAX, ++job) {
        const int nt = min(NMAX, n - c0);
        const int npad = (nt + 15) & ~15;
        const int b = job & 1;
        if (et == 0) ex[64 * 17 - 1] = wait_or_abort(&acc_full[b], (job >> 1) & 1, abort_flag) ? 1.0f : 0.0f;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        ok = ex[64 * 17 - 1] != 0.0f;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (!ok) break;
        tc_fence_after();
        for (int col = 0; col < npad; col += 16) {
          uint32_t r[16];
          tc_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * NMAX + col), r);
          if (DUAL) {
            if (q >= 2) {
              const int rr = (q - 2) * 32 + lane;
#pragma unroll
              for (int j = 0; j < 16; ++j) ex[rr * 17 + j] = rn<__nv_bfloat16>(__uint_as_float(r[j]));
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (q < 2) {
              const int rr = q * 32 + lane;
              const int grow = tile * 64 + rr;
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                if (col + j < nt && grow < Rdim) {
                  const float g = rn<__nv_bfloat16>(__uint_as_float(r[j]));
                  const float u = ex[rr * 17 + j];
                  const float sg = rn<__nv_bfloat16>(silu_f32(g));
                  // h feeds the down projection of this same kernel family: store it k-permuted
                  const int gperm = (grow & ~7) | ((grow & 3) << 1) | ((grow >> 2) & 1);
                  hout[(size_t)(pos0 + c0 + col + j) * p.I + gperm] = __float2bfloat16_rn(__fmul_rn(sg, u));
                }
              }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
          } else {
            const int grow = tile * 128 + q * 32 + lane;
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (col + j < nt && grow < Rdim)
                yout[(size_t)(pos0 + c0 + col + j) * p.H + grow] = __float2bfloat16_rn(__uint_as_float(r[j]));
          }
        }
        tc_fence_before();
        mbar_arrive(&acc_empty[b]);
      }
    }
    if (!ok && et == 0) atomicOr(ip.status, kDevWaitExpired);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)S::TMEM_COLS) : "memory");
  }
}

// x [T,H] -> copy with every group of 8 elements stored as (x0,x4,x1,x5,x2,x6,x3,x7)
__global__ void i4u_permute_x_kernel(const __nv_bfloat16* x, __nv_bfloat16* xperm, int T, int H) {
  pdl_wait();
  pdl_trigger();
  const size_t nchunks = (size_t)T * (H / 8);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nchunks; i += (size_t)gridDim.x * blockDim.x) {
    const uint4 v = ldg_cached(x + i * 8);
    uint4 o;
    o.x = __byte_perm(v.x, v.z, 0x5410); o.y = __byte_perm(v.x, v.z, 0x7632);
    o.z = __byte_perm(v.y, v.w, 0x5410); o.w = __byte_perm(v.y, v.w, 0x7632);
    *reinterpret_cast<uint4*>(xperm + i * 8) = o;
  }
}

}  // namespace b200moe
