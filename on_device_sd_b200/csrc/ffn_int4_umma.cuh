// K3d - grouped SwiGLU expert FFN over int4 g128 weights on the tcgen05 tensor cores.
// Same contract and numerics as ffn_int4.cuh (the dequantised weight is bf16(scale * q), bit for
// bit), but the tokens ride the MMA's N dimension, so the per-weight work does not grow with the
// number of tokens an expert holds.
//
// Data flow per stage of 128 k (= one scale group):
//   TMA box (128 rows x 64 bytes of nibbles, 64-byte swizzle) -> shared-memory ring
//   -> dequant warps: thread (row, half) reads 32 bytes, converts 64 nibbles in registers
//      (lop3 magic, exact subtraction, one bf16 multiplication by the group scale) and writes them
//      with tcgen05.st into TENSOR MEMORY: lane = weight row, 32 columns = 64 k.  The dequantised
//      tile never touches shared memory - a bf16 copy there would cost eight times the packed
//      bytes in shared-memory traffic (write + read).
//   -> tcgen05.mma with A from tensor memory and B (tokens) from shared memory, accumulator in
//      tensor memory, epilogue as in ffn_umma.cuh.
// Tensor memory (512 columns): accumulators 2 x PARTS x NMAX at column 0, then the A ring of 64-column slots:
// six slots for the 16-token tile (the accumulators take 128 columns there), four otherwise.  With more
// slots than dequant groups a group does not have to wait for the MMAs of its own previous stage to
// release "its" slot before it may store the next tile (measured: a third of a group's time).
//
// Token tiles also arrive by TMA: a small kernel first writes the tokens of every (token, expert)
// pair in sorted-pair order - so an expert's rows are contiguous, like the rows of h - with the k
// permutation the nibble extraction wants (lop3 yields pairs (t, t+4); every group of 8 k is
// stored as k0,k4,k1,k5,k2,k6,k3,k7, and the gate/up epilogue stores h the same way).  A tile is
// then a few plain {64 k, 16 rows} boxes; rows past the expert's last token belong to the next expert
// and only feed accumulator columns nobody reads.  No thread computes addresses per 16 bytes:
// the integer pipe is what bounds this kernel (7 ALU operations per 8 weights for the nibbles).
//
//   warp 0      TMA producer, weights   warp 2      TMA producer, tokens
//   warps 1, 3  MMA issuers: issuer w takes the k-stages whose running index is w modulo 2 (warp 1 owns the TMEM allocation)
//   warps 4-19  dequant: four groups of 4 warps; group g takes every fourth k-stage (running index g modulo 4),
//               thread = one weight row of the stage (64 bytes of nibbles -> 64 columns)
//   warps 20-23 epilogue
// Producer and issuer warps run warp-uniform with one elected lane per instruction (see tc_mma_bf16_w).
#pragma once
#include <cuda.h>

#include "common.cuh"
#include "ffn_gemv.cuh"
#include "ffn_umma.cuh"
#include "tma.cuh"

namespace b200moe {

constexpr int kI4uDeqGroups = 4;                  // groups of dequant warps; group g takes the stages g modulo 4
constexpr int kI4uDeqWarps = 4 * kI4uDeqGroups;   // per group: one warp per TMEM lane quarter
constexpr int kI4uFirstDeq = 4;
constexpr int kI4uFirstEpi = kI4uFirstDeq + kI4uDeqWarps;
constexpr int kI4uThreads = (kI4uFirstEpi + 4) * 32;
constexpr int kI4uWTile = 128 * 64;       // 128 rows x 64 bytes = 128 k of nibbles
constexpr int kI4uBK = 128;
constexpr int kI4uACols = 64;             // 128 k of bf16 = 64 32-bit columns per lane

// Shared memory: the packed-tile ring (the bytes in flight from HBM) and a ring of token tiles.
template <int NMAX> struct I4uShape {
  static constexpr int B_TILE = 2 * NMAX * 128;                 // two 64-k atoms of NMAX rows x 128 bytes
  static constexpr int W_STAGES = NMAX <= 16 ? 20 : (NMAX == 32 ? 16 : (NMAX == 64 ? 12 : 8));   // 8 KB each; a multiple of the number of dequant groups
  static constexpr int A_STAGES = NMAX <= 16 ? 6 : 4;           // dequantised A tiles in tensor memory
  static constexpr int A_COL0 = 512 - A_STAGES * kI4uACols;     // first column of the A ring (accumulators sit below)
  // Successive MMAs into one accumulator serialise on its latency, so the k-steps rotate over
  // PARTS independent accumulators that the epilogue adds up.
  static constexpr int PARTS = NMAX <= 32 ? 4 : (NMAX == 64 ? 2 : 1);
  // One warp issues a tcgen05.mma every 45-150 cycles depending on how the operands reach the
  // uniform registers (measured in this kernel: ~75 per MMA), the tensor pipe takes one every ~38:
  // two issuing warps on interleaved k-stages with disjoint accumulators keep the eight MMAs of a stage
  // inside its HBM time (four issuers measured no faster: 80 against 83 k tokens/s on the Mixtral shape).
  // Issuer w takes the stages whose RUNNING index (over the whole kernel) is w modulo MMA_WARPS: the ring
  // depths are multiples of MMA_WARPS, so a ring slot always belongs to the same issuer and that issuer
  // sees every phase of the slot's barriers (a warp that skipped a phase could not tell it from the next
  // one of the same parity).
  static constexpr int MMA_WARPS = PARTS >= 2 ? 2 : 1;
  static constexpr int PARTS_PER_WARP = PARTS / MMA_WARPS;
  static constexpr int EX_BYTES = 64 * 17 * 4;
  static constexpr int FIXED = 1024 + W_STAGES * kI4uWTile + EX_BYTES + 1024;   // alignment slack, packed ring, epilogue exchange, barriers
  static constexpr int B_FIT = (227 * 1024 - FIXED) / B_TILE;
  static constexpr int B_STAGES = (B_FIT > 8 ? 8 : B_FIT) / MMA_WARPS * MMA_WARPS;
  static constexpr size_t SMEM = (size_t)FIXED + (size_t)B_STAGES * B_TILE;
  static constexpr int TMEM_COLS = 512;
  static_assert(2 * PARTS * NMAX <= A_COL0, "accumulators overlap the A ring");
  static_assert(B_STAGES >= 3 && A_STAGES % MMA_WARPS == 0 && B_STAGES % MMA_WARPS == 0, "ring depths");
};

struct I4uParams {
  FfnParams f;
  const CUtensorMap* tmaps;   // [E][3]: uint8 maps with {64 B, 64 rows} (gate, up) / {64 B, 128 rows} (down) boxes, 64-byte swizzle
  int* status;
  CUtensorMap bmap;           // token rows of this pass in sorted-pair order ([pairs, H] or [pairs, I] bf16), box {64 k, 16 rows}, 128-byte swizzle
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

// D[tmem] (+)= A[tmem] * B[smem]: the A operand is read from tensor memory (lane = row of A).
// Called by a converged warp, one elected lane issues (see tc_mma_bf16_w).
__device__ __forceinline__ void tc_mma_bf16_ts_w(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\telect.sync _|q, 0xffffffff;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// 32 consecutive 32-bit columns of this thread's lane
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
        "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
        "r"(r[30]), "r"(r[31]) : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// Called by a converged warp: one elected lane arms the barrier / issues the copy.
__device__ __forceinline__ void mbar_expect_tx_w(uint64_t* bar, uint32_t bytes) {
  asm volatile("{\n\t.reg .pred q;\n\telect.sync _|q, 0xffffffff;\n\t"
               "@q mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n\t}" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_load_2d_w(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar, uint64_t policy) {
  asm volatile(
      "{\n\t.reg .pred q;\n\telect.sync _|q, 0xffffffff;\n\t"
      "@q cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;\n\t}"
      ::"r"(smem_addr(dst)), "l"(map), "r"(c0), "r"(c1), "r"(smem_addr(bar)), "l"(policy)
      : "memory");
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}

template <int NMAX, bool DUAL>
__global__ void __launch_bounds__(kI4uThreads, 1) ffn_int4_umma_kernel(const __grid_constant__ I4uParams ip, SlotTable st) {
  using S = I4uShape<NMAX>;
  constexpr int STAGES = S::A_STAGES;       // A ring in tensor memory
  constexpr int BSTAGES = S::B_STAGES;      // token-tile ring
  constexpr int WSTAGES = S::W_STAGES;      // packed-tile ring
  constexpr int B_TILE = S::B_TILE;
  constexpr int TILE_ROWS = DUAL ? 64 : 128;
  const FfnParams& p = ip.f;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  unsigned char* Ws = smem;                                           // packed tiles
  unsigned char* Bs = Ws + (size_t)WSTAGES * kI4uWTile;              // token tiles
  float* ex = reinterpret_cast<float*>(Bs + (size_t)BSTAGES * B_TILE);
  uint64_t* w_full = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(ex) + S::EX_BYTES);
  uint64_t* w_empty = w_full + WSTAGES;
  uint64_t* full = w_empty + WSTAGES;          // A stage written by the dequant warps
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

  if (threadIdx.x == 0) {
    for (int i = 0; i < WSTAGES; ++i) { mbar_init(&w_full[i], 1); mbar_init(&w_empty[i], 4); }
    for (int i = 0; i < STAGES; ++i) { mbar_init(&full[i], 4); mbar_init(&empty[i], 1); }
    for (int i = 0; i < BSTAGES; ++i) { mbar_init(&b_full[i], 1); mbar_init(&b_empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], S::MMA_WARPS); mbar_init(&acc_empty[i], 128); }
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
  // the token copy of the gather kernel (and the tables before it) must be complete: gate/up waits here, with its
  // barriers and its tensor memory set up while the predecessor was still running
  if (DUAL) pdl_wait();
  pdl_trigger();
  const int total = (*p.n_act) * tiles;

  if (warp == 0) {
    // ------------------------------ TMA producer: packed weight tiles (whole warp, one elected lane issues) ------------------------------
    const uint64_t policy = l2_policy_evict_first();
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < total && ok; item += gridDim.x) {
      const int e = warp_bcast(p.act_list[item / tiles]);
      const int tile = item % tiles;
      const int slot = st.slot[e];
      const int pos0 = warp_bcast(p.offsets[e]);
      const int n = warp_bcast(p.offsets[e + 1]) - pos0;
      const CUtensorMap* m0 = ip.tmaps + (size_t)slot * 3 + (DUAL ? 0 : 2);
      const CUtensorMap* m1 = ip.tmaps + (size_t)slot * 3 + 1;
      tensormap_acquire(m0);
      if (DUAL) tensormap_acquire(m1);
      for (int c0 = 0; c0 < n && ok; c0 += NMAX) {
        for (int kb = 0; kb < nkb; ++kb) {
          if (!__all_sync(0xffffffffu, wait_or_abort(&w_empty[s], ph ^ 1, abort_flag))) { ok = false; break; }
          mbar_expect_tx_w(&w_full[s], kI4uWTile);
          unsigned char* dst = Ws + (size_t)s * kI4uWTile;
          if (DUAL) {
            tma_load_2d_w(dst, m0, kb * 64, tile * 64, &w_full[s], policy);
            tma_load_2d_w(dst + 4096, m1, kb * 64, tile * 64, &w_full[s], policy);
          } else {
            tma_load_2d_w(dst, m0, kb * 64, tile * 128, &w_full[s], policy);
          }
          if (++s == WSTAGES) { s = 0; ph ^= 1; }
        }
      }
    }
    if (!ok && lane == 0) atomicOr(ip.status, kDevWaitExpired);
  } else if (warp == 2) {
    // ------------------------------ TMA producer: token tiles ------------------------------
    const uint64_t policy_b = l2_policy_evict_last();    // every CTA working on this expert re-reads the token rows
    if (!DUAL) pdl_wait();                               // h must be complete; the weight stream has already started
    int sb = 0;
    uint32_t phb = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < total && ok; item += gridDim.x) {
      const int e = warp_bcast(p.act_list[item / tiles]);
      const int pos0 = warp_bcast(p.offsets[e]);
      const int n = warp_bcast(p.offsets[e + 1]) - pos0;
      for (int c0 = 0; c0 < n && ok; c0 += NMAX) {
        for (int kb = 0; kb < nkb; ++kb) {
          if (!__all_sync(0xffffffffu, wait_or_abort(&b_empty[sb], phb ^ 1, abort_flag))) { ok = false; break; }
          const int npad = (min(NMAX, n - c0) + 15) & ~15;
          mbar_expect_tx_w(&b_full[sb], (uint32_t)(2 * npad * 128));
          unsigned char* bdst = Bs + (size_t)sb * B_TILE;
          for (int r = 0; r < npad; r += 16) {   // boxes of 16 rows: only the rows this pass multiplies are fetched
            tma_load_2d_w(bdst + r * 128, &ip.bmap, kb * kI4uBK, pos0 + c0 + r, &b_full[sb], policy_b);
            tma_load_2d_w(bdst + NMAX * 128 + r * 128, &ip.bmap, kb * kI4uBK + 64, pos0 + c0 + r, &b_full[sb], policy_b);
          }
          if (++sb == BSTAGES) { sb = 0; phb ^= 1; }
        }
      }
    }
    if (!ok && lane == 0) atomicOr(ip.status, kDevWaitExpired);
  } else if (warp == 1 || warp == 3) {
    // ------------------------------ MMA issuers (whole warps, warp-uniform; see tc_mma_bf16_w) ------------------------------
    // Issuer w takes the k-stages whose running index is w modulo MMA_WARPS and owns PARTS_PER_WARP accumulators.
    const int w = warp == 1 ? 0 : 1;
    if (w < S::MMA_WARPS) {
      int s = 0, sb = 0, job = 0, gmod = 0;      // gmod: running stage index modulo MMA_WARPS
      uint32_t ph = 0, phb = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total && ok; item += gridDim.x) {
        const int e = p.act_list[item / tiles];
        const int n = warp_bcast(p.offsets[e + 1] - p.offsets[e]);
        for (int c0 = 0; c0 < n && ok; c0 += NMAX, ++job) {
          const int npad = (min(NMAX, n - c0) + 15) & ~15;
          const uint32_t idesc = umma_idesc_bf16(npad);
          const int b = job & 1;
          if (!__all_sync(0xffffffffu, wait_or_abort(&acc_empty[b], ((job >> 1) & 1) ^ 1, abort_flag))) { ok = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + (uint32_t)((b * S::PARTS + w * S::PARTS_PER_WARP) * NMAX);
          uint32_t started = 0u;                  // this issuer's first stage of the job starts its accumulators
          for (int kb = 0; kb < nkb; ++kb) {
            if (gmod == w) {
              const bool got = wait_or_abort(&full[s], ph, abort_flag) && wait_or_abort(&b_full[sb], phb, abort_flag);
              if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
              tc_fence_after();
              const uint32_t a_tmem = tmem_base + (uint32_t)(S::A_COL0 + s * kI4uACols);
#pragma unroll
              for (int atom = 0; atom < 2; ++atom) {
                const uint64_t bdesc = umma_desc_sw128(smem_addr(Bs + (size_t)sb * B_TILE + atom * NMAX * 128));
#pragma unroll
                for (int k = 0; k < 4; ++k) {   // 16 k per MMA = 8 columns of A
                  const int kk = atom * 4 + k;
                  tc_mma_bf16_ts_w(d_tmem + (uint32_t)((kk % S::PARTS_PER_WARP) * NMAX), a_tmem + (uint32_t)(kk * 8), bdesc + 2 * k, idesc,
                                   kk >= S::PARTS_PER_WARP ? 1u : started);
                }
              }
              started = 1u;
              tc_commit_w(&empty[s]);
              tc_commit_w(&b_empty[sb]);
            }
            if (++gmod == S::MMA_WARPS) gmod = 0;
            if (++s == STAGES) { s = 0; ph ^= 1; }
            if (++sb == BSTAGES) { sb = 0; phb ^= 1; }
          }
          if (ok) tc_commit_w(&acc_full[b]);
        }
      }
      if (!ok && lane == 0) atomicOr(ip.status, kDevWaitExpired);
    }
  } else if (warp < kI4uFirstEpi) {
    // ------------------------------ dequant: packed tile -> bf16 A tile in tensor memory ------------------------------
    // A warp may only touch the 32 TMEM lanes of its quarter (warp % 4): thread = weight row of the stage.
    // Group grp handles the k-stages whose running index is grp modulo 4 and therefore always A stage grp.
    // Group grp handles the k-stages whose running index gi (over the whole kernel) is grp modulo 4.  Stage gi
    // lives in packed-ring slot gi % WSTAGES and goes to A slot gi % STAGES; the phase of a slot's barriers
    // is the parity of how often the slot has been used, (gi / depth) & 1.
    const int q = warp & 3;
    const int row = q * 32 + lane, grp = (warp - kI4uFirstDeq) >> 2;
    const int sw = (row >> 1) & 3;              // 64-byte swizzle of the TMA box: 16-byte slot c of row r sits at c ^ ((r >> 1) & 3)
    const unsigned char* wrow0 = Ws + row * 64;
    const uint32_t a_addr0 = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)S::A_COL0;
    int gi = grp;                                 // running index of this group's next stage
    int first = grp;                              // first k-stage of the next job that belongs to this group
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
        int kb = first;
        __nv_bfloat16 sv = sc[min(kb, nkb - 1)];
        // Software pipeline over this group's stages: the tensor-memory stores of a stage are left in flight while
        // the next stage's packed tile is fetched and its first half converted; only then does the group wait for
        // the stores and hand the earlier stage to the MMA issuers (tcgen05.wait::st covers every store issued so far).
        bool pending = false;
        int pend_as = 0;
        for (; kb < nkb; kb += kI4uDeqGroups, gi += kI4uDeqGroups) {
          const __nv_bfloat16 sv_next = sc[min(kb + kI4uDeqGroups, nkb - 1)];   // the scale of this group's next stage is fetched a stage ahead
          const int ws = gi % WSTAGES, as = gi % STAGES;
          const uint32_t wph = (uint32_t)(gi / WSTAGES) & 1u, aph = (uint32_t)(gi / STAGES) & 1u;
          if (!__all_sync(0xffffffffu, wait_or_abort(&w_full[ws], wph, abort_flag))) { ok = false; break; }   // warp-uniform
          const unsigned char* wrow = wrow0 + (size_t)ws * kI4uWTile;
          uint4 pk[4];
#pragma unroll
          for (int c = 0; c < 4; ++c) pk[c] = *reinterpret_cast<const uint4*>(wrow + ((c ^ sw) << 4));
          __syncwarp();
          if (lane == 0) mbar_arrive(&w_empty[ws]);
          const __nv_bfloat162 s2 = __nv_bfloat162(sv, sv);
          const uint32_t a_addr = a_addr0 + (uint32_t)(as * kI4uACols);
#pragma unroll
          for (int half = 0; half < 2; ++half) {  // 64 k = 32 columns at a time keeps the register count down
            const uint32_t words[8] = {pk[2 * half].x, pk[2 * half].y, pk[2 * half].z, pk[2 * half].w,
                                       pk[2 * half + 1].x, pk[2 * half + 1].y, pk[2 * half + 1].z, pk[2 * half + 1].w};
            uint32_t o[32];
#pragma unroll
            for (int c = 0; c < 8; ++c) {         // word c = 8 k = 4 columns
              uint32_t o4[4];
              i4u_dequant8(words[c], s2, o4);
              o[4 * c + 0] = o4[0]; o[4 * c + 1] = o4[1]; o[4 * c + 2] = o4[2]; o[4 * c + 3] = o4[3];
            }
            if (half == 0) {
              if (pending) {                      // the previous stage's stores have had a conversion's worth of time to land
                tc_wait_st();
                tc_fence_before();
                if (lane == 0) mbar_arrive(&full[pend_as]);
                pending = false;
              }
              if (!__all_sync(0xffffffffu, wait_or_abort(&empty[as], aph ^ 1, abort_flag))) { ok = false; break; }
              tc_fence_after();
            }
            tc_st32(a_addr + (uint32_t)(half * 32), o);
          }
          if (!ok) break;
          pending = true;
          pend_as = as;
          sv = sv_next;
        }
        if (pending) {                            // last stage of the job for this group: hand it over now
          tc_wait_st();
          tc_fence_before();
          if (lane == 0) mbar_arrive(&full[pend_as]);
        }
        first = kb - nkb;                         // the stride carries over into the next job
      }
    }
    if (!ok && lane == 0) atomicOr(ip.status, kDevWaitExpired);
  } else {
    // ------------------------------ epilogue ------------------------------
    const int q = warp & 3;                       // TMEM lane quarter this warp may read
    const int et = threadIdx.x - kI4uFirstEpi * 32;   // 0..127
    int job = 0, gbase = 0;                       // gbase: running index of the job's first k-stage modulo MMA_WARPS
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
          // Sum of the accumulators, in part order.  A job with fewer k-stages than issuers leaves the
          // accumulators of the idle issuers untouched: issuer w worked iff (w - gbase) mod MMA_WARPS < nkb.
          uint32_t r[16];
          bool have = false;
#pragma unroll
          for (int part = 0; part < S::PARTS; ++part) {
            const int wi = part / S::PARTS_PER_WARP;
            if (((wi - gbase + S::MMA_WARPS) % S::MMA_WARPS) >= nkb) continue;
            uint32_t r2[16];
            tc_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)((b * S::PARTS + part) * NMAX + col), r2);
            if (!have) {
#pragma unroll
              for (int j = 0; j < 16; ++j) r[j] = r2[j];
              have = true;
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) r[j] = __float_as_uint(__fadd_rn(__uint_as_float(r[j]), __uint_as_float(r2[j])));
            }
          }
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
        gbase = (gbase + nkb) % S::MMA_WARPS;
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

// Tokens of every (token, expert) pair in sorted-pair order, every group of 8 k stored as
// (x0,x4,x1,x5,x2,x6,x3,x7): row pos of xg = x[sorted_pair[pos] / K].  One warp-sized slice of a row per step.
__global__ void i4u_gather_x_kernel(const __nv_bfloat16* x, __nv_bfloat16* xg, const int* sorted_pair, const int* offsets, int E, int K, int H) {
  pdl_wait();
  pdl_trigger();
  const int pairs = offsets[E];
  const int chunks = H / 8;
  const size_t nchunks = (size_t)pairs * chunks;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nchunks; i += (size_t)gridDim.x * blockDim.x) {
    const int pos = (int)(i / chunks), c = (int)(i % chunks);
    const int tok = sorted_pair[pos] / K;
    const uint4 v = ldg_cached(x + (size_t)tok * H + c * 8);
    uint4 o;
    o.x = __byte_perm(v.x, v.z, 0x5410); o.y = __byte_perm(v.x, v.z, 0x7632);
    o.z = __byte_perm(v.y, v.w, 0x5410); o.w = __byte_perm(v.y, v.w, 0x7632);
    *reinterpret_cast<uint4*>(xg + (size_t)pos * H + c * 8) = o;
  }
}

}  // namespace b200moe
