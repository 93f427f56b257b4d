// K3b - grouped SwiGLU expert FFN on the 5th-generation tensor cores (tcgen05 + TMEM), bf16.
// Same contract as the GEMV kernels (expert_forward_with_weights, demo/src/layers/mlp.py:209-231
// of the reference, once per activated expert), for experts that hold more than a few tokens.
//
// "Swap-AB": the weight rows ride the MMA's M dimension (128 per tile, K-major, staged by TMA
// with the 128-byte swizzle), the expert's tokens ride N (16..128, K-major, gathered into the
// same swizzled layout with cp.async), the accumulator lives in tensor memory.  No weight byte
// passes through a register.  The kernel stays HBM-bound: per 16 KB weight tile it issues four
// 128xNx16 MMAs.
//
//   warp 0     TMA producer (one elected lane): weight tiles -> shared-memory ring
//   warp 1     MMA issuer (one elected lane) + owner of the TMEM allocation
//   warps 2-5  token-tile loaders (cp.async gather of x rows / h rows)
//   warps 6-9  epilogue: tcgen05.ld, rounding points, SwiGLU, stores (overlaps the next tile's
//              main loop through a double-buffered accumulator)
//
// DUAL  (gate/up): one tile = 64 rows of gate_proj stacked on the same 64 rows of up_proj, so one
//                  MMA per k-step serves both and a tile is 1 MB of a Mixtral-sized expert
//                  (fine-grained enough to balance 148 SMs); the epilogue pairs lane r (gate) with
//                  lane r+64 (up) through shared memory.
// !DUAL (down)   : one tile = 128 rows of down_proj.
// Every wait is bounded; on expiry the CTA raises a flag, every role leaves its loop, TMEM is
// freed and the status word reports B200MOE_DEV_WAIT_EXPIRED.
#pragma once
#include <cuda.h>

#include "common.cuh"
#include "ffn_gemv.cuh"
#include "tma.cuh"

namespace b200moe {

constexpr int kUmmaThreads = 320;
constexpr int kUmmaLoaders = 128;        // threads gathering token tiles
constexpr int kUmmaBK = 64;          // k elements per stage (128 bytes of bf16)
constexpr int kUmmaATile = 16384;    // 128 rows x 128 bytes

// NMAX = tokens per pass (the widest MMA N) sizes the token tile of a stage and the TMEM
// allocation; whatever shared memory is left goes to ring depth.
template <int NMAX> struct UmmaShape {
  static constexpr int B_TILE = NMAX * 128;
  static constexpr int STAGE = kUmmaATile + B_TILE;
  static constexpr int STAGES = (200 * 1024 / STAGE) > 12 ? 12 : (200 * 1024 / STAGE);
  static constexpr int EX_BYTES = 64 * 17 * 4;
  static constexpr int PTR_BYTES = 128 * 8;
  static constexpr size_t SMEM = 1024 /*alignment slack*/ + (size_t)STAGES * STAGE + EX_BYTES + PTR_BYTES + (2 * STAGES + 4) * 8 + 64;
  // Successive MMAs into one accumulator serialise on its latency (about 170 cycles each, far more
  // than a 128 x N x 16 product with a small N takes), so the k-steps rotate over PARTS independent
  // accumulators that the epilogue adds up.
  static constexpr int PARTS = NMAX <= 64 ? 4 : 2;
  static constexpr int TMEM_COLS = 2 * PARTS * NMAX;            // 128, 256, 512, 512: powers of two
};

struct UmmaParams {
  FfnParams f;
  const CUtensorMap* tmaps;   // [E][3] for this layer: gate (box 64x64), up (64x64), down (64x128)
  int* status;
  // Down projection only: K split into `ksplit` slices so that few experts still give every SM
  // several work items.  Slice s writes fp32 partial sums to ypart[s][pos][H]; the combine kernel
  // adds the slices in index order (deterministic) and rounds once.  ksplit == 1: bf16 y as usual.
  int ksplit;
  float* ypart;
  int pairs_cap;              // rows of one slice of ypart
};

// ---- PTX wrappers -------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
      ::"r"(smem_addr(dst)), "l"(map), "r"(c0), "r"(c1), "r"(smem_addr(bar)), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tensormap_acquire(const CUtensorMap* map) {
  asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(map) : "memory");
}
__device__ __forceinline__ void cp_async_16(void* dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// tcgen05.commit and tcgen05.mma for a CONVERGED warp: every lane executes the call, one elected lane
// issues.  tcgen05.mma takes its descriptors from uniform registers; issued from a single-thread
// branch each instruction measured 152 cycles on B200 (operands moved over one by one), from a
// converged warp 44 (M = 128, N = 16), so the MMA warps keep their control flow warp-uniform.
__device__ __forceinline__ void tc_commit_w(uint64_t* bar) {
  asm volatile("{\n\t.reg .pred q;\n\telect.sync _|q, 0xffffffff;\n\t"
               "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16_w(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\telect.sync _|q, 0xffffffff;\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// lane 0's value in every lane; also tells the compiler the value is warp-uniform
__device__ __forceinline__ int warp_bcast(int v) { return __shfl_sync(0xffffffffu, v, 0); }
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// K-major operand tile in the canonical 128-byte-swizzle layout: rows of 128 bytes, groups of 8
// rows 1024 bytes apart (stride byte offset), descriptor version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr) {
  const uint64_t lo = (uint64_t)((saddr & 0x3ffffu) >> 4) | (1ull << 16);
  const uint64_t hi = (uint64_t)(1024u >> 4) | (1ull << 14) | (2ull << 29);
  return lo | (hi << 32);
}
// kind::f16 instruction descriptor: fp32 accumulate, bf16 x bf16, both K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t umma_idesc_bf16(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((128u >> 4) << 24);
}
// the same with the operand format of the model dtype: 0 = fp16, 1 = bf16 (bits 7-9 for A, 10-12 for B)
template <typename T> __device__ __forceinline__ uint32_t umma_idesc(int n) {
  constexpr uint32_t fmt = std::is_same<T, __half>::value ? 0u : 1u;
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(n >> 3) << 17) | ((128u >> 4) << 24);
}

// Bounded wait that also leaves when another role has raised the CTA's abort flag.  The first
// probe costs one instruction; after that the warp sleeps between probes - a spinning warp takes
// issue slots and integer-pipe cycles from the warps that do the work (measured on the int4 kernel:
// almost half of all issued instructions were polls), and the clock is only read when the barrier
// was found busy.
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait_hint(bar, parity, 20000u)) return true;
  const long long t0 = clock64();
  for (uint32_t i = 0;; ++i) {
    __nanosleep(i < 8u ? 32u : 128u);
    if (mbar_try_wait_hint(bar, parity, 20000u)) return true;
    if ((i & 15u) == 15u) {
      if (*abort_flag) return false;
      if (clock64() - t0 > (1ll << 31)) { *abort_flag = 1; return false; }
    }
  }
}

template <typename T, int NMAX, bool DUAL>
__global__ void __launch_bounds__(kUmmaThreads, 1) ffn_umma_kernel(UmmaParams up, SlotTable st) {
  static_assert(std::is_same<T, __nv_bfloat16>::value || std::is_same<T, __half>::value, "16-bit model dtypes only");
  using S = UmmaShape<NMAX>;
  constexpr int STAGES = S::STAGES;
  constexpr int B_TILE = S::B_TILE;
  constexpr int TILE_ROWS = DUAL ? 64 : 128;       // output rows per tile
  constexpr int LOADER_LAG = (STAGES >= 8) ? 4 : 2;  // cp.async groups a loader keeps in flight
  static_assert(STAGES > LOADER_LAG + 1, "ring too shallow");
  const FfnParams& p = up.f;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~(uintptr_t)1023);
  unsigned char* As = smem;
  unsigned char* Bs = smem + (size_t)STAGES * kUmmaATile;
  float* ex = reinterpret_cast<float*>(Bs + (size_t)STAGES * B_TILE);
  const T** rowptr = reinterpret_cast<const T**>(reinterpret_cast<unsigned char*>(ex) + S::EX_BYTES);
  uint64_t* full = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(rowptr) + S::PTR_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int Kdim = DUAL ? p.H : p.I;
  const int Rdim = DUAL ? p.I : p.H;
  const int nkb = (Kdim + kUmmaBK - 1) / kUmmaBK;
  const int tiles = (Rdim + TILE_ROWS - 1) / TILE_ROWS;

  const int KS = DUAL ? 1 : up.ksplit;
  // work item -> (expert slot in act_list, row tile, K slice); k-blocks [kb0, kb1) of the slice
#define B200MOE_DECODE_ITEM(item)                                   \
  const int ks_ = (item) % KS;                                      \
  const int tile = ((item) / KS) % tiles;                           \
  const int e = p.act_list[(item) / KS / tiles];                    \
  const int kb0 = ks_ * nkb / KS, kb1 = (ks_ + 1) * nkb / KS;       \
  (void)tile; (void)kb0; (void)kb1;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) { mbar_init(&full[i], 1 + kUmmaLoaders / 32);   /* TMA bytes + one arrival per loader warp */ mbar_init(&empty[i], 1); }
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
  // Gate/up follows the router / permute kernel directly and needs its tables: it waits here, with its barriers
  // and its tensor memory already set up while the predecessor was still running.  The down projection follows
  // gate/up: the tables were complete before gate/up could start, so its weight stream starts immediately and
  // only the loaders (readers of h) wait for gate/up to finish.
  if (DUAL) pdl_wait();
  pdl_trigger();
  const int total = (*p.n_act) * tiles * KS;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      const uint64_t policy = l2_policy_evict_first();
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total && ok; item += gridDim.x) {
        B200MOE_DECODE_ITEM(item)
        const int slot = st.slot[e];
        const int n = p.offsets[e + 1] - p.offsets[e];
        const CUtensorMap* m0 = up.tmaps + (size_t)slot * 3 + (DUAL ? 0 : 2);
        const CUtensorMap* m1 = up.tmaps + (size_t)slot * 3 + 1;
        tensormap_acquire(m0);
        if (DUAL) tensormap_acquire(m1);
        for (int c0 = 0; c0 < n && ok; c0 += NMAX) {
          for (int kb = kb0; kb < kb1; ++kb) {
            if (!wait_or_abort(&empty[s], ph ^ 1, abort_flag)) { ok = false; break; }
            mbar_expect_tx(&full[s], kUmmaATile);
            unsigned char* dst = As + (size_t)s * kUmmaATile;
            if (DUAL) {
              tma_load_2d(dst, m0, kb * kUmmaBK, tile * 64, &full[s], policy);
              tma_load_2d(dst + 8192, m1, kb * kUmmaBK, tile * 64, &full[s], policy);
            } else {
              tma_load_2d(dst, m0, kb * kUmmaBK, tile * 128, &full[s], policy);
            }
            if (++s == STAGES) { s = 0; ph ^= 1; }
          }
        }
      }
      if (!ok) atomicOr(up.status, kDevWaitExpired);
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (whole warp, warp-uniform; see tc_mma_bf16_w) ------------------------------
    int s = 0, job = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < total && ok; item += gridDim.x) {
      B200MOE_DECODE_ITEM(item)
      const int n = warp_bcast(p.offsets[e + 1] - p.offsets[e]);
      for (int c0 = 0; c0 < n && ok; c0 += NMAX, ++job) {
        const int npad = (min(NMAX, n - c0) + 15) & ~15;
        const uint32_t idesc = umma_idesc<T>(npad);
        const int b = job & 1;
        if (!__all_sync(0xffffffffu, wait_or_abort(&acc_empty[b], ((job >> 1) & 1) ^ 1, abort_flag))) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(b * S::PARTS * NMAX);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!__all_sync(0xffffffffu, wait_or_abort(&full[s], ph, abort_flag))) { ok = false; break; }
          tc_fence_after();
          const uint64_t adesc = umma_desc_sw128(smem_addr(As + (size_t)s * kUmmaATile));
          const uint64_t bdesc = umma_desc_sw128(smem_addr(Bs + (size_t)s * B_TILE));
#pragma unroll
          for (int k = 0; k < kUmmaBK / 16; ++k)   // 32 bytes of K per instruction: +2 in the 16-byte address field
            tc_mma_bf16_w(d_tmem + (uint32_t)((k % S::PARTS) * NMAX), adesc + 2 * k, bdesc + 2 * k, idesc, (kb > kb0 || k >= S::PARTS) ? 1u : 0u);
          tc_commit_w(&empty[s]);      // frees the stage when these MMAs have read it
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (ok) tc_commit_w(&acc_full[b]);
      }
    }
    if (!ok && lane == 0) atomicOr(up.status, kDevWaitExpired);
  } else if (warp < 6) {
    // ------------------------------ token-tile loaders ------------------------------
    const int tl = threadIdx.x - 64;          // 0..127
    if (!DUAL) pdl_wait();                    // h must be complete
    int s = 0, lag_s = 0, issued = 0;         // stage being filled; oldest stage not yet signalled
    uint32_t ph = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < total; item += gridDim.x) {   // runs to the end even after a failed wait: the named barriers below need all 128 threads
      B200MOE_DECODE_ITEM(item)
      const int pos0 = p.offsets[e];
      const int n = p.offsets[e + 1] - pos0;
      for (int c0 = 0; c0 < n; c0 += NMAX) {
        const int nt = min(NMAX, n - c0);
        const int npad = (nt + 15) & ~15;
        // row pointers of this pass, shared by the loader threads
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (tl < npad) {
          const int pos = pos0 + c0 + min(tl, nt - 1);
          rowptr[tl] = DUAL ? reinterpret_cast<const T*>(p.x) + (size_t)(p.sorted_pair[pos] / p.K) * p.H
                            : reinterpret_cast<const T*>(p.h) + (size_t)pos * p.I;
        }
        asm volatile("bar.sync 2, 128;" ::: "memory");
        for (int kb = kb0; kb < kb1 && ok; ++kb) {
          if (!__all_sync(0xffffffffu, wait_or_abort(&empty[s], ph ^ 1, abort_flag))) { ok = false; break; }
          unsigned char* bt = Bs + (size_t)s * B_TILE;
          for (int id = tl; id < npad * 8; id += kUmmaLoaders) {
            const int r = id >> 3, chunk = id & 7;
            const int k0 = kb * kUmmaBK + chunk * 8;
            const bool live = (r < nt) && (k0 < Kdim);
            const T* src = rowptr[r];
            cp_async_16(bt + r * 128 + ((chunk ^ (r & 7)) << 4), live ? (const void*)(src + k0) : (const void*)src, live ? 16u : 0u);
          }
          cp_async_commit();
          ++issued;
          if (issued > LOADER_LAG) {              // the group issued LOADER_LAG stages ago has landed
            cp_async_wait<LOADER_LAG>();
            fence_proxy_async();
            __syncwarp();                         // one arrival per warp: 128 arrivals on one barrier serialise for hundreds of cycles
            if (lane == 0) mbar_arrive(&full[lag_s]);
            if (++lag_s == STAGES) lag_s = 0;
          }
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
    cp_async_wait<0>();
    fence_proxy_async();
    __syncwarp();
    for (int q = min(issued, LOADER_LAG); q > 0; --q) {
      if (lane == 0) mbar_arrive(&full[lag_s]);
      if (++lag_s == STAGES) lag_s = 0;
    }
    if (!ok && lane == 0) atomicOr(up.status, kDevWaitExpired);
  } else {
    // ------------------------------ epilogue ------------------------------
    const int q = warp & 3;                       // TMEM lane quarter this warp may read
    const int et = threadIdx.x - 192;             // 0..127
    int job = 0;
    bool ok = true;
    T* hout = reinterpret_cast<T*>(p.h);
    T* yout = reinterpret_cast<T*>(p.y);
    for (int item = blockIdx.x; item < total && ok; item += gridDim.x) {
      B200MOE_DECODE_ITEM(item)
      const int pos0 = p.offsets[e];
      const int n = p.offsets[e + 1] - pos0;
      for (int c0 = 0; c0 < n && ok; c0 += NMAX, ++job) {
        const int nt = min(NMAX, n - c0);
        const int npad = (nt + 15) & ~15;
        const int b = job & 1;
        // one thread waits, all four warps take its verdict: they meet at named barriers below
        if (et == 0) ex[64 * 17 - 1] = wait_or_abort(&acc_full[b], (job >> 1) & 1, abort_flag) ? 1.0f : 0.0f;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        ok = ex[64 * 17 - 1] != 0.0f;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (!ok) break;
        tc_fence_after();
        for (int col = 0; col < npad; col += 16) {
          uint32_t r[16];
          tc_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * S::PARTS * NMAX + col), r);
#pragma unroll
          for (int part = 1; part < S::PARTS; ++part) {
            uint32_t r2[16];
            tc_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)((b * S::PARTS + part) * NMAX + col), r2);
#pragma unroll
            for (int j = 0; j < 16; ++j) r[j] = __float_as_uint(__fadd_rn(__uint_as_float(r[j]), __uint_as_float(r2[j])));
          }
          if (DUAL) {
            // lanes 0-63 hold gate rows, lanes 64-127 the same rows of up: pair them through smem
            if (q >= 2) {
              const int row = (q - 2) * 32 + lane;
#pragma unroll
              for (int j = 0; j < 16; ++j) ex[row * 17 + j] = rn<T>(__uint_as_float(r[j]));
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (q < 2) {
              const int row = q * 32 + lane;
              const int grow = tile * 64 + row;
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                if (col + j < nt && grow < Rdim) {
                  const float g = rn<T>(__uint_as_float(r[j]));
                  const float u = ex[row * 17 + j];
                  const float sg = rn<T>(silu_f32(g));
                  hout[(size_t)(pos0 + c0 + col + j) * p.I + grow] = Elem<T>::from_float(__fmul_rn(sg, u));
                }
              }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
          } else {
            const int grow = tile * 128 + q * 32 + lane;
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (col + j < nt && grow < Rdim) {
                if (KS > 1) up.ypart[((size_t)ks_ * up.pairs_cap + (pos0 + c0 + col + j)) * p.H + grow] = __uint_as_float(r[j]);
                else yout[(size_t)(pos0 + c0 + col + j) * p.H + grow] = Elem<T>::from_float(__uint_as_float(r[j]));
              }
          }
        }
        tc_fence_before();
        mbar_arrive(&acc_empty[b]);
      }
    }
    if (!ok && et == 0) atomicOr(up.status, kDevWaitExpired);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)S::TMEM_COLS) : "memory");
  }
}

#undef B200MOE_DECODE_ITEM

}  // namespace b200moe
