// b200moe_expert_ffn_noalloc: one expert's SwiGLU FFN for callers that must not allocate.
//
// Who that is: an engine step loop that has handed the whole device to its own pools (weights,
// KV cache) and where a cudaMalloc would both fail the memory budget and stall the device -
// cudaMalloc synchronises with everything in flight - or a plugin that is invoked from inside
// somebody else's stream-ordered section and is forbidden to create contexts, workspaces or
// tensors.  b200moe_expert_ffn needs a context (whose creation allocates the workspace); this
// entry point needs none: the SwiGLU intermediate h [n, I] and the few words of bookkeeping the
// kernels read live in ONE file-scope device array that every GPU loading the library holds
// until the process exits.
//
// The price: a fixed ceiling (n <= 64 rows, n * I * sizeof(element) <= 2 MiB) and one array
// shared by every call.  It keeps the previous call's contents; the status word in it is cleared
// by the set-up kernel of each call and h is rewritten before it is read, so nothing stale is
// consumed.  Two calls that overlap on the GPU (different streams, different threads) race on
// the array - serialise them.
#include "../../include/b200moe.h"

#include <cuda_runtime.h>

#include "common.cuh"
#include "ffn_gemv.cuh"
#include "internal.h"

using namespace b200moe;

namespace {

constexpr int kNoAllocMaxRows = 64;
constexpr size_t kNoAllocHBytes = 2u << 20;   // SwiGLU intermediate, n * I elements

struct NoAllocScratch {
  unsigned char h[kNoAllocHBytes];
  ExpertPtrs expert;            // the one expert of this call
  int offsets[2];               // {0, n}
  int n_act;                    // 1
  int act;                      // expert index 0
  int status;                   // bounded-wait failures of the kernels
  int sorted[kNoAllocMaxRows];  // identity: row i of x is pair i
};

// The scratch itself.  In host code this name is only a stand-in for the symbol - its device
// address comes from cudaGetSymbolAddress below; device code may name it directly.
static __device__ __align__(256) unsigned char g_noalloc_scratch[sizeof(NoAllocScratch)];

__global__ void noalloc_setup_kernel(const void* gate, const void* up, const void* down, int n) {
  NoAllocScratch* s = reinterpret_cast<NoAllocScratch*>(g_noalloc_scratch);
  const int i = threadIdx.x;
  if (i < kNoAllocMaxRows) s->sorted[i] = i;
  if (i == 0) {
    s->expert.w[0] = gate; s->expert.w[1] = up; s->expert.w[2] = down;
    s->expert.s[0] = nullptr; s->expert.s[1] = nullptr; s->expert.s[2] = nullptr;
    s->offsets[0] = 0; s->offsets[1] = n;
    s->n_act = 1;
    s->act = 0;
    s->status = 0;              // must start at zero for every call
  }
}

constexpr int kMaxDevices = 64;
// Per device, filled by the first call on that device.  No lock: concurrent first calls on one
// device resolve the same symbol and store the same pointer, so the race is benign.
void* g_scratch_addr[kMaxDevices];

using Shape = GemvShape<8, 2048, 3>;

template <typename T, int NT> int launch_pair(const FfnParams& p, const SlotTable& st, int* status, int sms, cudaStream_t s) {
  auto up = ffn_gemv_kernel<T, NT, true, Shape>;
  auto down = ffn_gemv_kernel<T, NT, false, Shape>;
  cudaError_t e = cudaFuncSetAttribute(up, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Shape::SMEM);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(down, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Shape::SMEM);
  if (e != cudaSuccess) return b200moe_fail_global(B200MOE_E_CUDA, "b200moe_expert_ffn_noalloc: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  up<<<sms, Shape::THREADS, Shape::SMEM, s>>>(p, st, status);
  down<<<sms, Shape::THREADS, Shape::SMEM, s>>>(p, st, status);
  e = cudaGetLastError();
  if (e != cudaSuccess) return b200moe_fail_global(B200MOE_E_CUDA, "b200moe_expert_ffn_noalloc: launch failed: %s", cudaGetErrorString(e));
  return B200MOE_OK;
}

template <typename T> int run(const FfnParams& p, const SlotTable& st, int* status, int n, int sms, cudaStream_t s) {
  if (n <= 1) return launch_pair<T, 1>(p, st, status, sms, s);
  if (n <= 2) return launch_pair<T, 2>(p, st, status, sms, s);
  return launch_pair<T, 4>(p, st, status, sms, s);
}

}  // namespace

extern "C" int b200moe_expert_ffn_noalloc(const void* x, int n, int hidden_size, int intermediate_size, int dtype,
                                          const void* gate_proj, const void* up_proj, const void* down_proj, void* out,
                                          void* stream) {
  if (n < 0 || hidden_size <= 0 || intermediate_size <= 0)
    return b200moe_fail_global(B200MOE_E_ARG, "b200moe_expert_ffn_noalloc: sizes must be positive");
  if (dtype < B200MOE_F32 || dtype > B200MOE_BF16) return b200moe_fail_global(B200MOE_E_ARG, "b200moe_expert_ffn_noalloc: unknown dtype %d", dtype);
  if (hidden_size % 8 || intermediate_size % 8)
    return b200moe_fail_global(B200MOE_E_ARG, "b200moe_expert_ffn_noalloc: hidden_size and intermediate_size must be multiples of 8");
  const size_t eb = dtype == B200MOE_F32 ? 4 : 2;
  if (n > kNoAllocMaxRows || (size_t)n * intermediate_size * eb > kNoAllocHBytes)
    return b200moe_fail_global(B200MOE_E_UNSUPPORTED,
                               "b200moe_expert_ffn_noalloc: n=%d rows x I=%d exceeds the built-in scratch (at most %d rows and %zu bytes of "
                               "intermediate); use b200moe_expert_ffn with a context for larger calls",
                               n, intermediate_size, kNoAllocMaxRows, kNoAllocHBytes);
  if (n == 0) return B200MOE_OK;
  if (!x || !gate_proj || !up_proj || !down_proj || !out) return b200moe_fail_global(B200MOE_E_ARG, "b200moe_expert_ffn_noalloc: null pointer");
  const uintptr_t align_or = (uintptr_t)x | (uintptr_t)gate_proj | (uintptr_t)up_proj | (uintptr_t)down_proj | (uintptr_t)out;
  if (align_or & 15u) return b200moe_fail_global(B200MOE_E_ARG, "b200moe_expert_ffn_noalloc: pointers must be 16-byte aligned");

  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return b200moe_fail_global(B200MOE_E_CUDA, "b200moe_expert_ffn_noalloc: no CUDA device: %s (there is no CPU path)", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return b200moe_fail_global(B200MOE_E_UNSUPPORTED, "b200moe_expert_ffn_noalloc: device ordinal %d not supported", dev);
  // Set-up, once per device, with that device current: resolve the device address of the scratch
  // array.  This first call on a device should come before any stream capture.
  if (g_scratch_addr[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || ptr == nullptr)
      return b200moe_fail_global(B200MOE_E_CUDA, "b200moe_expert_ffn_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    g_scratch_addr[dev] = ptr;
  }
  NoAllocScratch* sc = reinterpret_cast<NoAllocScratch*>(g_scratch_addr[dev]);   // device address: never dereferenced here
  int sms = 0;
  e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess || sms <= 0) return b200moe_fail_global(B200MOE_E_CUDA, "b200moe_expert_ffn_noalloc: cannot query the device: %s", cudaGetErrorString(e));

  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  noalloc_setup_kernel<<<1, kNoAllocMaxRows, 0, st>>>(gate_proj, up_proj, down_proj, n);
  e = cudaGetLastError();
  if (e != cudaSuccess) return b200moe_fail_global(B200MOE_E_CUDA, "b200moe_expert_ffn_noalloc: launch failed: %s", cudaGetErrorString(e));

  FfnParams p{};
  p.x = x;
  p.h = sc->h;
  p.y = out;
  p.experts = &sc->expert;
  p.offsets = sc->offsets;
  p.sorted_pair = sc->sorted;
  p.act_list = &sc->act;
  p.n_act = &sc->n_act;
  p.H = hidden_size; p.I = intermediate_size; p.K = 1;
  SlotTable tab;
  for (int i = 0; i < kMaxExperts; ++i) { tab.slot[i] = -1; tab.rank[i] = 0; }
  tab.slot[0] = 0;
  switch (dtype) {
    case B200MOE_F32: return run<float>(p, tab, &sc->status, n, sms, st);
    case B200MOE_F16: return run<__half>(p, tab, &sc->status, n, sms, st);
    default: return run<__nv_bfloat16>(p, tab, &sc->status, n, sms, st);
  }
}

extern "C" int b200moe_expert_ffn_noalloc_status(int* device_status_out, void* stream) {
  if (!device_status_out) return b200moe_fail_global(B200MOE_E_ARG, "b200moe_expert_ffn_noalloc_status: null argument");
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return b200moe_fail_global(B200MOE_E_CUDA, "b200moe_expert_ffn_noalloc_status: no CUDA device: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return b200moe_fail_global(B200MOE_E_UNSUPPORTED, "b200moe_expert_ffn_noalloc_status: device ordinal %d not supported", dev);
  *device_status_out = 0;
  if (g_scratch_addr[dev] == nullptr) return B200MOE_OK;   // no call has run on this device yet
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const NoAllocScratch* sc = reinterpret_cast<const NoAllocScratch*>(g_scratch_addr[dev]);   // device address
  int v = 0;
  e = cudaMemcpyAsync(&v, &sc->status, sizeof v, cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return b200moe_fail_global(B200MOE_E_CUDA, "b200moe_expert_ffn_noalloc_status: %s", cudaGetErrorString(e));
  *device_status_out = v;
  if (v) return b200moe_fail_global(B200MOE_E_DEVICE, "b200moe_expert_ffn_noalloc: device status word = %d (a bounded wait gave up; the output is incomplete)", v);
  return B200MOE_OK;
}
