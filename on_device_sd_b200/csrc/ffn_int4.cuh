// K3c - grouped SwiGLU expert FFN over int4 g128 weights (bf16 activations).  Same contract as
// the other FFN kernels (expert_forward_with_weights, demo/src/layers/mlp.py:209-231 of the
// reference, once per activated expert); the reference has no quantised weights, the format is
// this library's (int4_pack.cuh).
//
// Weights are never re-tiled: they stay uint8 [out, in/2] as packed.  A warp owns a tile of 16
// output rows and a private ring of TMA boxes (16 rows x 128 bytes = 256 nibbles, 128-byte
// swizzle); a lane reads 16 bytes = 32 nibbles of row g and of row g+8, turns them into exact
// bf16 integers in registers (lop3 with the 0x4300 magic, one subtraction), scales them and feeds them to
// m16n8k16 tensor-core MMAs as the A operand; the tokens are the B operand (8 per MMA), loaded
// as 16-byte chunks and byte-permuted to the same k order.  The group scale is applied as one
// bf16 multiplication per weight, which reproduces bit for bit the dequantised weight
// bf16(scale * q) that the unpacker materialises.
#pragma once
#include <cuda.h>

#include "common.cuh"
#include "ffn_gemv.cuh"
#include "tma.cuh"

namespace b200moe {

constexpr int kInt4Warps = 16;
constexpr int kInt4Threads = kInt4Warps * 32;
constexpr int kInt4Box = 2048;            // 16 rows x 128 bytes
constexpr int kInt4Stages = 3;            // ring depth per warp; a stage = two boxes
constexpr size_t kInt4Smem = 1024 + (size_t)kInt4Warps * kInt4Stages * 2 * kInt4Box + (size_t)kInt4Warps * kInt4Stages * 8 + 64;

struct Int4Params {
  FfnParams f;
  const CUtensorMap* tmaps;   // [E][3]: uint8 [rows, K/2] maps with a {128 B, 16 rows} box
  int* status;
};

__device__ __forceinline__ void tma_load_2d_plain(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
      ::"r"(smem_addr(dst)), "l"(map), "r"(c0), "r"(c1), "r"(smem_addr(bar)), "l"(policy)
      : "memory");
}

// 8 nibbles (k .. k+7, low nibble first) -> 4 bf16x2 registers holding (q_t, q_{t+4}), t = 0..3,
// as exact integers in [-8, 7]:  (w >> 4t) & 0x000F000F | 0x43004300 is the pair (128 + n_t, 128 + n_{t+4}).
__device__ __forceinline__ void dequant8(uint32_t w, __nv_bfloat162 scale2, uint32_t (&p)[4]) {
  const __nv_bfloat162 bias = __nv_bfloat162(__float2bfloat16_rn(136.0f), __float2bfloat16_rn(136.0f));
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    uint32_t v;
    asm("lop3.b32 %0, %1, 0x000F000F, 0x43004300, 0xEA;" : "=r"(v) : "r"(w >> (4 * t)));
    const __nv_bfloat162 d = __hmul2(__hsub2(*reinterpret_cast<__nv_bfloat162*>(&v), bias), scale2);   // exact integer, then one rounding
    p[t] = *reinterpret_cast<const uint32_t*>(&d);
  }
}

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// DUAL: a unit = rows [r0, r0+16) of gate_proj and of up_proj; a stage = the two boxes of one k-step.
// !DUAL: a unit = rows [r0, r0+16) of down_proj; a stage = the boxes of two consecutive k-steps.
template <bool DUAL, int NTILE>
__global__ void __launch_bounds__(kInt4Threads, 1) ffn_int4_kernel(Int4Params ip, SlotTable st) {
  const FfnParams& p = ip.f;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, q = lane & 3;
  unsigned char* ring = smem + (size_t)warp * kInt4Stages * 2 * kInt4Box;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)kInt4Warps * kInt4Stages * 2 * kInt4Box) + warp * kInt4Stages;

  const int Kdim = DUAL ? p.H : p.I;
  const int Rdim = DUAL ? p.I : p.H;
  const int nks = (Kdim + 255) / 256;                  // boxes along K
  const int nstage = DUAL ? nks : (nks + 1) / 2;       // stages per pass
  const int groups = (Rdim + 15) / 16;
  const int sgroups = Kdim / 128;                      // scales per row

  pdl_wait();
  pdl_trigger();
  const int total_units = (*p.n_act) * groups;
  const int gw = blockIdx.x * kInt4Warps + warp;
  const int W = gridDim.x * kInt4Warps;
  if (gw >= total_units) return;

  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < kInt4Stages; ++i) mbar_init(&full[i], 1);
    mbar_fence_init();
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncwarp();
  const uint64_t policy = l2_policy_evict_first();

  struct Unit { int slot, pos0, n, r0; };
  auto load_unit = [&](int u) {
    Unit v;
    const int e = p.act_list[u / groups];
    v.slot = st.slot[e];
    v.r0 = (u % groups) * 16;
    v.pos0 = p.offsets[e];
    v.n = p.offsets[e + 1] - v.pos0;
    return v;
  };

  // ---- producer state (lane 0 issues; all lanes track it) ----
  int pu = gw, ps = 0, issued = 0;
  Unit pq = load_unit(pu);
  int p_stages = ((pq.n + 8 * NTILE - 1) / (8 * NTILE)) * nstage;
  auto produce = [&]() {
    if (pu >= total_units) return;
    const int slot = issued % kInt4Stages;
    const int sidx = ps % nstage;
    if (lane == 0) {
      mbar_expect_tx(&full[slot], 2 * kInt4Box);
      unsigned char* dst = ring + (size_t)slot * 2 * kInt4Box;
      if (DUAL) {
        tma_load_2d_plain(dst, ip.tmaps + (size_t)pq.slot * 3 + 0, sidx * 128, pq.r0, &full[slot], policy);
        tma_load_2d_plain(dst + kInt4Box, ip.tmaps + (size_t)pq.slot * 3 + 1, sidx * 128, pq.r0, &full[slot], policy);
      } else {
        const CUtensorMap* m = ip.tmaps + (size_t)pq.slot * 3 + 2;
        tma_load_2d_plain(dst, m, (2 * sidx) * 128, pq.r0, &full[slot], policy);
        tma_load_2d_plain(dst + kInt4Box, m, (2 * sidx + 1) * 128, pq.r0, &full[slot], policy);   // may lie past K: zero fill, skipped below
      }
    }
    ++issued;
    if (++ps == p_stages) {
      pu += W;
      ps = 0;
      if (pu < total_units) {
        pq = load_unit(pu);
        p_stages = ((pq.n + 8 * NTILE - 1) / (8 * NTILE)) * nstage;
      }
    }
  };
#pragma unroll
  for (int i = 0; i < kInt4Stages - 1; ++i) produce();

  int consumed = 0;
  bool dead = false;
  const __nv_bfloat16* xbase = reinterpret_cast<const __nv_bfloat16*>(DUAL ? p.x : p.h);
  for (int cu = gw; cu < total_units && !dead; cu += W) {
    const Unit cq = load_unit(cu);
    const ExpertPtrs ep = p.experts[cq.slot];
    const int rowA = min(cq.r0 + g, Rdim - 1), rowB = min(cq.r0 + g + 8, Rdim - 1);
    for (int c0 = 0; c0 < cq.n && !dead; c0 += 8 * NTILE) {
      const int nt = min(8 * NTILE, cq.n - c0);
      // this lane's token row for every n-tile (column g of the tile)
      const __nv_bfloat16* xr[NTILE];
#pragma unroll
      for (int t = 0; t < NTILE; ++t) {
        const int pos = cq.pos0 + c0 + min(t * 8 + g, nt - 1);
        xr[t] = DUAL ? xbase + (size_t)(p.sorted_pair[pos] / p.K) * p.H : xbase + (size_t)pos * p.I;
      }
      constexpr int NM = DUAL ? 2 : 1;
      float acc[NM][NTILE][4];
#pragma unroll
      for (int m = 0; m < NM; ++m)
#pragma unroll
        for (int t = 0; t < NTILE; ++t)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[m][t][j] = 0.0f;

      for (int sidx = 0; sidx < nstage; ++sidx) {
        produce();
        // (box, half) pairs: DUAL shares x between the gate box and the up box of the same k range
        constexpr int NKR = DUAL ? 2 : 4;              // k ranges of 128 in a stage
        // the stage's group scales are fetched before the wait on the weights, so that their
        // latency overlaps the TMA's
        __nv_bfloat16 sca[NM][NKR], scb[NM][NKR];
#pragma unroll
        for (int kr = 0; kr < NKR; ++kr) {
          const int kb = (DUAL ? sidx * 256 : (2 * sidx + (kr >> 1)) * 256) + (kr & 1) * 128;
          const int gi = min(kb >> 7, sgroups - 1);
#pragma unroll
          for (int m = 0; m < NM; ++m) {
            const __nv_bfloat16* sc = reinterpret_cast<const __nv_bfloat16*>(DUAL ? ep.s[m] : ep.s[2]);
            sca[m][kr] = sc[(size_t)rowA * sgroups + gi];
            scb[m][kr] = sc[(size_t)rowB * sgroups + gi];
          }
        }
        const int slot = consumed % kInt4Stages;
        if (!mbar_wait_bounded(&full[slot], (uint32_t)(consumed / kInt4Stages) & 1u)) {
          if (lane == 0) atomicOr(ip.status, kDevWaitExpired);
          dead = true;
          break;
        }
        ++consumed;
        const unsigned char* sbase = ring + (size_t)slot * 2 * kInt4Box;
#pragma unroll
        for (int kr = 0; kr < NKR; ++kr) {
          const int box0 = DUAL ? 0 : (kr >> 1);
          const int half = kr & 1;
          const int kbase = (DUAL ? sidx * 256 : (2 * sidx + box0) * 256) + half * 128;
          if (kbase >= Kdim) continue;                 // beyond K: the box holds fill bytes, not weights
          const int chunk = half * 4 + q;
          uint4 wa[NM], wb[NM];
          __nv_bfloat162 sa[NM], sb[NM];
#pragma unroll
          for (int m = 0; m < NM; ++m) {
            const unsigned char* bx = sbase + (size_t)(DUAL ? m : box0) * kInt4Box;
            wa[m] = *reinterpret_cast<const uint4*>(bx + g * 128 + ((chunk ^ (g & 7)) << 4));
            wb[m] = *reinterpret_cast<const uint4*>(bx + (g + 8) * 128 + ((chunk ^ (g & 7)) << 4));   // (g+8)&7 == g&7
            sa[m] = __nv_bfloat162(sca[m][kr], sca[m][kr]);
            sb[m] = __nv_bfloat162(scb[m][kr], scb[m][kr]);
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint32_t pa[NM][4], pb[NM][4];
#pragma unroll
            for (int m = 0; m < NM; ++m) {
              dequant8((&wa[m].x)[i], sa[m], pa[m]);
              dequant8((&wb[m].x)[i], sb[m], pb[m]);
            }
#pragma unroll
            for (int t = 0; t < NTILE; ++t) {
              const uint4 xv = ldg_cached(xr[t] + kbase + q * 32 + 8 * i);
              const uint32_t x0 = __byte_perm(xv.x, xv.z, 0x5410), x1 = __byte_perm(xv.x, xv.z, 0x7632);
              const uint32_t x2 = __byte_perm(xv.y, xv.w, 0x5410), x3 = __byte_perm(xv.y, xv.w, 0x7632);
#pragma unroll
              for (int m = 0; m < NM; ++m) {
                mma_bf16_16816(acc[m][t], pa[m][0], pb[m][0], pa[m][1], pb[m][1], x0, x1);
                mma_bf16_16816(acc[m][t], pa[m][2], pb[m][2], pa[m][3], pb[m][3], x2, x3);
              }
            }
          }
        }
        __syncwarp();   // every lane is done with the slot before it is refilled
      }
      if (dead) break;

      // epilogue: fragment element j of tile t is (row g + 8*(j>>1), token t*8 + 2q + (j&1))
#pragma unroll
      for (int t = 0; t < NTILE; ++t)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int row = cq.r0 + g + 8 * (j >> 1);
          const int tok = t * 8 + 2 * q + (j & 1);
          if (tok < nt && row < Rdim) {
            if (DUAL) {
              const float gg = rn<__nv_bfloat16>(acc[0][t][j]);
              const float uu = rn<__nv_bfloat16>(acc[NM - 1][t][j]);
              const float sg = rn<__nv_bfloat16>(silu_f32(gg));
              reinterpret_cast<__nv_bfloat16*>(p.h)[(size_t)(cq.pos0 + c0 + tok) * p.I + row] = __float2bfloat16_rn(__fmul_rn(sg, uu));
            } else {
              reinterpret_cast<__nv_bfloat16*>(p.y)[(size_t)(cq.pos0 + c0 + tok) * p.H + row] = __float2bfloat16_rn(acc[0][t][j]);
            }
          }
        }
    }
  }
}

}  // namespace b200moe
