// libb200moe.so - host side of the C ABI declared in include/b200moe.h: argument checks,
// workspace, expert pointer tables and kernel launches.  No torch types, no CPU compute path.
#include "../../include/b200moe.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <algorithm>
#include <atomic>
#include <new>
#include <string>
#include <utility>
#include <vector>

#include "common.cuh"
#include "internal.h"
#include "ffn_gemv.cuh"
#include "ep.cuh"
#include "int4_pack.cuh"
#include "permute.cuh"
#include "rmsnorm.cuh"
#include "router.cuh"
#ifdef B200MOE_WITH_INT4
#include "ffn_int4.cuh"
#include "ffn_int4_umma.cuh"
#endif
#ifdef B200MOE_WITH_UMMA
#include "ffn_umma.cuh"
#endif
#include "moe_token.cuh"
#include "moe_tokens.cuh"

using namespace b200moe;

struct b200moe_ctx {
  b200moe_config cfg{};
  int sm_count = 0;
  std::string err;
  int64_t launches = 0;
  // registered weights (host mirror) and the device table
  std::vector<const void*> gate_w, gate_bias;
  std::vector<ExpertPtrs> h_experts;
  std::vector<uint8_t> registered;
  std::vector<uint8_t> dirty;
  ExpertPtrs* d_experts = nullptr;  // [L*E (+1 scratch entry for expert_ffn)]
#ifdef B200MOE_WITH_UMMA
  // TMA descriptors of the registered experts (dense bf16 only): [L*E + 1][3], host mirror + device copy
  std::vector<CUtensorMap> h_tmaps;
  std::vector<uint8_t> tmap_ok;
  CUtensorMap* d_tmaps = nullptr;
  std::vector<CUtensorMap> h_tmaps2;   // int4 only: second set of boxes (tcgen05 int4 kernel)
  CUtensorMap* d_tmaps2 = nullptr;
  void* encode_fn = nullptr;   // cuTensorMapEncodeTiled, resolved through the runtime
#endif
  // workspace
  float* logits = nullptr;          // [Tm,E] rounded logits of the latest router launch, as fp32
  unsigned* tile_counter = nullptr;     // [Tm] one per token tile, [Tm] all tiles done, [Tm+1] grid barrier word of the single-token kernel
  int64_t* ids64 = nullptr;
  void* scores = nullptr;
  int* offsets = nullptr;
  int* sorted_pair = nullptr;
  int* inv = nullptr;
  int* act_list = nullptr;
  int* n_act = nullptr;
  void* h = nullptr;
  void* y = nullptr;
  void* xnorm = nullptr;            // fused-norm entry: normalised token rows [Tm, H]
  void* xres = nullptr;             // fused-norm entry: x + residual rounded to the model dtype [Tm, H]
  void* xperm = nullptr;            // int4 tcgen05 path: k-permuted token rows in sorted-pair order [Tm*K, H]
  float* ypart = nullptr;           // fp32 K-slices of the down projection (tensor-core path)
  int ypart_slices = 0;             // slices ypart has room for
  int last_ksplit = 1;              // K split used by the most recent tensor-core launch
  bool token_kernel = true;         // single-token batches of the fused entry take the one-launch kernel (b200moe_set_token_kernel)
  int* status = nullptr;
  unsigned long long* bitmap = nullptr;
  // second, tiny table set used by b200moe_expert_ffn (one expert, identity permutation)
  int* one_offsets = nullptr;
  int* one_sorted = nullptr;
  int* one_act = nullptr;
  int* one_nact = nullptr;
  std::vector<void*> allocs;
  // expert-parallel exchange (b200moe_ep_*): this rank's exchange buffer, the peers' buffers as this GPU addresses them
  struct Ep {
    int world = 0, rank = 0, max_local = 0;
    bool attached = false;
    EpGeom geom{};
    EpPeers peers{};
    unsigned char* base = nullptr;
    size_t bytes = 0;
    unsigned* counters = nullptr;      // [0] epoch, [1] dispatch arrivals, [2] return arrivals, [8..15] rows sent per destination
    long long wait_cycles = 1ll << 31; // about one second
    std::vector<void*> opened;         // IPC mappings to close
    int last_T_local = 0;
  } ep;
  // optional per-kernel timing (b200moe_profile): one event pair per launch, grouped by kernel class
  bool profiling = false;
  struct ProfRec { int cls; cudaEvent_t a, b; };
  std::vector<ProfRec> prof;
};

// Brackets one kernel launch with CUDA events on the launching stream while profiling is on.
struct ProfScope {
  b200moe_ctx* ctx; cudaStream_t st; int idx = -1;
  ProfScope(b200moe_ctx* c, int cls, cudaStream_t s) : ctx(c), st(s) {
    if (!c || !c->profiling) return;
    b200moe_ctx::ProfRec r{cls, nullptr, nullptr};
    if (cudaEventCreate(&r.a) != cudaSuccess || cudaEventCreate(&r.b) != cudaSuccess) return;
    cudaEventRecord(r.a, s);
    c->prof.push_back(r);
    idx = (int)c->prof.size() - 1;
  }
  ~ProfScope() { if (idx >= 0) cudaEventRecord(ctx->prof[idx].b, st); }
};

static thread_local std::string g_err;

static int fail(b200moe_ctx* ctx, int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (ctx) ctx->err = buf;
  g_err = buf;
  return code;
}

int b200moe_fail_global(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_err = buf;
  return code;
}

#define CUDA_TRY(ctx, call)                                                                        \
  do {                                                                                             \
    cudaError_t e_ = (call);                                                                       \
    if (e_ != cudaSuccess)                                                                         \
      return fail(ctx, B200MOE_E_CUDA, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e_), __FILE__, __LINE__); \
  } while (0)

// Launch with the programmatic-stream-serialization attribute: the kernel may begin while its
// predecessor in the stream is still running and synchronises on the device (pdl_wait).
template <typename... KArgs, typename... Args>
static void launch_chain(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);   // errors surface in post_launch
}

static size_t elem_bytes(int dtype) { return dtype == B200MOE_F32 ? 4 : 2; }

template <typename T> static int dev_alloc(b200moe_ctx* ctx, T** p, size_t count) {
  void* q = nullptr;
  cudaError_t e = cudaMalloc(&q, count * sizeof(T) > 0 ? count * sizeof(T) : 16);
  if (e != cudaSuccess) return fail(ctx, B200MOE_E_CUDA, "cudaMalloc(%zu bytes) failed: %s", count * sizeof(T), cudaGetErrorString(e));
  ctx->allocs.push_back(q);
  *p = reinterpret_cast<T*>(q);
  return B200MOE_OK;
}

extern "C" int b200moe_abi_version(void) { return 2; }

extern "C" const char* b200moe_last_error(const b200moe_ctx* ctx) { return ctx ? ctx->err.c_str() : g_err.c_str(); }

extern "C" int64_t b200moe_launch_count(const b200moe_ctx* ctx) { return ctx ? ctx->launches : 0; }

extern "C" int b200moe_create(const b200moe_config* cfg, b200moe_ctx** out) {
  if (!cfg || !out) return fail(nullptr, B200MOE_E_ARG, "b200moe_create: null argument");
  *out = nullptr;
  const int H = cfg->hidden_size, E = cfg->num_experts, K = cfg->top_k, I = cfg->intermediate_size;
  if (H <= 0 || I <= 0 || E <= 0 || K <= 0 || cfg->num_layers <= 0 || cfg->max_tokens <= 0)
    return fail(nullptr, B200MOE_E_ARG, "b200moe_create: sizes must be positive");
  if (E > B200MOE_MAX_EXPERTS) return fail(nullptr, B200MOE_E_UNSUPPORTED, "num_experts %d > %d", E, B200MOE_MAX_EXPERTS);
  if (K > E || K > B200MOE_MAX_TOPK) return fail(nullptr, B200MOE_E_ARG, "top_k %d must be <= min(num_experts, %d)", K, B200MOE_MAX_TOPK);
  if (cfg->act_dtype < B200MOE_F32 || cfg->act_dtype > B200MOE_BF16) return fail(nullptr, B200MOE_E_ARG, "unknown act_dtype %d", cfg->act_dtype);
  if (cfg->weight_mode != B200MOE_W_DENSE && cfg->weight_mode != B200MOE_W_INT4_G128)
    return fail(nullptr, B200MOE_E_ARG, "unknown weight_mode %d", cfg->weight_mode);
  const int mult = cfg->weight_mode == B200MOE_W_INT4_G128 ? 128 : 8;
  if (H % mult || I % mult) return fail(nullptr, B200MOE_E_ARG, "hidden_size and intermediate_size must be multiples of %d", mult);
  if (cfg->weight_mode == B200MOE_W_INT4_G128 && cfg->act_dtype != B200MOE_BF16)
    return fail(nullptr, B200MOE_E_UNSUPPORTED, "int4 expert weights need bf16 activations");
#ifndef B200MOE_WITH_INT4
  if (cfg->weight_mode == B200MOE_W_INT4_G128) return fail(nullptr, B200MOE_E_UNSUPPORTED, "library built without the int4 kernels");
#endif
  int ndev = 0;
  cudaError_t e = cudaGetDeviceCount(&ndev);
  if (e != cudaSuccess || ndev == 0)
    return fail(nullptr, B200MOE_E_CUDA, "no CUDA device: %s (this library has no CPU path)", cudaGetErrorString(e));
  if (cfg->device < 0 || cfg->device >= ndev) return fail(nullptr, B200MOE_E_ARG, "device %d out of range", cfg->device);
  CUDA_TRY(nullptr, cudaSetDevice(cfg->device));
  cudaDeviceProp prop;
  CUDA_TRY(nullptr, cudaGetDeviceProperties(&prop, cfg->device));
  if (prop.major != 10) return fail(nullptr, B200MOE_E_UNSUPPORTED, "device is sm_%d%d; this library is built for sm_100a only", prop.major, prop.minor);

  b200moe_ctx* ctx = new (std::nothrow) b200moe_ctx();
  if (!ctx) return fail(nullptr, B200MOE_E_CUDA, "out of host memory");
  ctx->cfg = *cfg;
  ctx->sm_count = prop.multiProcessorCount;
  const size_t L = cfg->num_layers, Tm = cfg->max_tokens, eb = elem_bytes(cfg->act_dtype);
  ctx->gate_w.assign(L, nullptr);
  ctx->gate_bias.assign(L, nullptr);
  ctx->h_experts.assign(L * E, ExpertPtrs{});
  ctx->registered.assign(L * E, 0);
  ctx->dirty.assign(L, 0);
  int rc = B200MOE_OK;
  char* hb = nullptr;
  char* yb = nullptr;
  char* sb = nullptr;
  const size_t pairs = Tm * K;
  if ((rc = dev_alloc(ctx, &ctx->d_experts, L * E + 1)) || (rc = dev_alloc(ctx, &ctx->logits, Tm * E)) ||
      (rc = dev_alloc(ctx, &ctx->tile_counter, Tm + 2)) || (rc = dev_alloc(ctx, &ctx->ids64, pairs)) ||
      (rc = dev_alloc(ctx, &sb, pairs * 4)) || (rc = dev_alloc(ctx, &ctx->offsets, (size_t)E + 1)) ||
      (rc = dev_alloc(ctx, &ctx->sorted_pair, pairs)) || (rc = dev_alloc(ctx, &ctx->inv, pairs)) ||
      (rc = dev_alloc(ctx, &ctx->act_list, (size_t)E)) || (rc = dev_alloc(ctx, &ctx->n_act, 4)) ||
      (rc = dev_alloc(ctx, &hb, pairs * I * eb)) || (rc = dev_alloc(ctx, &yb, pairs * H * eb)) ||
      (rc = dev_alloc(ctx, &ctx->status, 4)) || (rc = dev_alloc(ctx, &ctx->bitmap, 4)) ||
      (rc = dev_alloc(ctx, &ctx->one_offsets, 2)) || (rc = dev_alloc(ctx, &ctx->one_sorted, pairs)) ||
      (rc = dev_alloc(ctx, &ctx->one_act, 1)) || (rc = dev_alloc(ctx, &ctx->one_nact, 1))) {
    std::string msg = ctx->err;
    b200moe_destroy(ctx);
    return fail(nullptr, rc, "%s", msg.c_str());
  }
  ctx->h = hb;
  ctx->y = yb;
  ctx->scores = sb;
  {
    char* xn = nullptr;
    char* xr = nullptr;
    if ((rc = dev_alloc(ctx, &xn, Tm * (size_t)H * eb)) || (rc = dev_alloc(ctx, &xr, Tm * (size_t)H * eb))) {
      std::string msg = ctx->err;
      b200moe_destroy(ctx);
      return fail(nullptr, rc, "%s", msg.c_str());
    }
    ctx->xnorm = xn;
    ctx->xres = xr;
  }
#ifdef B200MOE_WITH_UMMA
  if (cfg->act_dtype == B200MOE_BF16 || (cfg->act_dtype == B200MOE_F16 && cfg->weight_mode == B200MOE_W_DENSE)) {   // dense bf16 / fp16 (tcgen05 path) and int4 (TMA boxes of packed nibbles)
    ctx->h_tmaps.assign((L * E + 1) * 3, CUtensorMap{});
    ctx->tmap_ok.assign(L * E + 1, 0);
    if (cfg->weight_mode == B200MOE_W_INT4_G128) {
      char* xp = nullptr;
      if ((rc = dev_alloc(ctx, &xp, pairs * (size_t)H * 2))) {
        std::string msg = ctx->err;
        b200moe_destroy(ctx);
        return fail(nullptr, rc, "%s", msg.c_str());
      }
      ctx->xperm = xp;
      ctx->h_tmaps2.assign((L * E + 1) * 3, CUtensorMap{});
      if ((rc = dev_alloc(ctx, &ctx->d_tmaps2, (L * E + 1) * 3))) {
        std::string msg = ctx->err;
        b200moe_destroy(ctx);
        return fail(nullptr, rc, "%s", msg.c_str());
      }
    }
    if ((rc = dev_alloc(ctx, &ctx->d_tmaps, (L * E + 1) * 3))) {
      std::string msg = ctx->err;
      b200moe_destroy(ctx);
      return fail(nullptr, rc, "%s", msg.c_str());
    }
    if (cfg->weight_mode == B200MOE_W_DENSE) {
      const size_t slice = pairs * (size_t)H * sizeof(float);
      int slices = (int)std::min<size_t>(12, (64u << 20) / std::max<size_t>(slice, 1));
      if (slices >= 2 && dev_alloc(ctx, &ctx->ypart, (size_t)slices * pairs * H) == B200MOE_OK) ctx->ypart_slices = slices;
    }
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ctx->encode_fn, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      ctx->encode_fn = nullptr;   // the tensor-core path then reports itself unsupported
  }
#endif
  cudaMemset(ctx->tile_counter, 0, (Tm + 2) * sizeof(unsigned));
  cudaMemset(ctx->status, 0, sizeof(int));
  cudaMemset(ctx->d_experts, 0, (L * E + 1) * sizeof(ExpertPtrs));
  {
    std::vector<int> iota(pairs);
    for (size_t i = 0; i < pairs; ++i) iota[i] = (int)i;
    cudaMemcpy(ctx->one_sorted, iota.data(), pairs * sizeof(int), cudaMemcpyHostToDevice);
    const int zero_one[2] = {0, 1};
    cudaMemcpy(ctx->one_act, &zero_one[0], sizeof(int), cudaMemcpyHostToDevice);
    cudaMemcpy(ctx->one_nact, &zero_one[1], sizeof(int), cudaMemcpyHostToDevice);
  }
  e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    b200moe_destroy(ctx);
    return fail(nullptr, B200MOE_E_CUDA, "workspace initialisation failed: %s", cudaGetErrorString(e));
  }
  *out = ctx;
  return B200MOE_OK;
}

extern "C" int b200moe_destroy(b200moe_ctx* ctx) {
  if (!ctx) return B200MOE_OK;
  cudaSetDevice(ctx->cfg.device);
  for (auto& r : ctx->prof) { cudaEventDestroy(r.a); cudaEventDestroy(r.b); }
  for (void* p : ctx->ep.opened) cudaIpcCloseMemHandle(p);
  for (void* p : ctx->allocs) cudaFree(p);
  delete ctx;
  return B200MOE_OK;
}

static int check_layer(b200moe_ctx* ctx, int layer, const char* who) {
  if (!ctx) return fail(nullptr, B200MOE_E_ARG, "%s: null context", who);
  if (layer < 0 || layer >= ctx->cfg.num_layers) return fail(ctx, B200MOE_E_ARG, "%s: layer %d out of range [0,%d)", who, layer, ctx->cfg.num_layers);
  return B200MOE_OK;
}
static int check_tokens(b200moe_ctx* ctx, int T, const char* who) {
  if (T < 0) return fail(ctx, B200MOE_E_ARG, "%s: negative token count", who);
  if (T > ctx->cfg.max_tokens) return fail(ctx, B200MOE_E_STATE, "%s: T=%d exceeds the context's max_tokens=%d", who, T, ctx->cfg.max_tokens);
  return B200MOE_OK;
}
static bool misaligned(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) != 0; }

template <typename F> static int dispatch_dtype(b200moe_ctx* ctx, int dtype, F&& f) {
  switch (dtype) {
    case B200MOE_F32: return f(float{});
    case B200MOE_F16: return f(__half{});
    case B200MOE_BF16: return f(__nv_bfloat16{});
  }
  return fail(ctx, B200MOE_E_ARG, "unknown dtype %d", dtype);
}

static int post_launch(b200moe_ctx* ctx, const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(ctx, B200MOE_E_CUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
  if (ctx) ctx->launches++;
  return B200MOE_OK;
}

#ifdef B200MOE_WITH_UMMA
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// bf16 matrix [rows, cols] row-major -> 2-D tensor map with a {64 cols, box_rows} box, 128-byte swizzle
static bool encode_map(b200moe_ctx* ctx, CUtensorMap* out, const void* base, int rows, int cols, int box_rows, bool fp16 = false) {
  if (!ctx->encode_fn) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  const cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1u, 1u};
  CUresult r = reinterpret_cast<EncodeTiledFn>(ctx->encode_fn)(out, fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                                                               estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// packed int4 matrix, uint8 [rows, bytes_per_row] -> 2-D map with a {128 bytes, 16 rows} box, 128-byte swizzle
static bool encode_map_u8(b200moe_ctx* ctx, CUtensorMap* out, const void* base, int rows, int bytes_per_row, int box_bytes = 128,
                          int box_rows = 16) {
  if (!ctx->encode_fn) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)bytes_per_row, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)bytes_per_row};
  const cuuint32_t box[2] = {(cuuint32_t)box_bytes, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1u, 1u};
  CUresult r = reinterpret_cast<EncodeTiledFn>(ctx->encode_fn)(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box,
                                                               estr, CU_TENSOR_MAP_INTERLEAVE_NONE, box_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                                                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

static bool encode_expert_maps(b200moe_ctx* ctx, CUtensorMap* three, const void* gate, const void* up, const void* down) {
  const int H0 = ctx->cfg.hidden_size, I0 = ctx->cfg.intermediate_size;
  if (ctx->cfg.weight_mode == B200MOE_W_INT4_G128)
    return encode_map_u8(ctx, &three[0], gate, I0, H0 / 2) && encode_map_u8(ctx, &three[1], up, I0, H0 / 2) &&
           encode_map_u8(ctx, &three[2], down, H0, I0 / 2);
  const int H = ctx->cfg.hidden_size, I = ctx->cfg.intermediate_size;
  const bool fp16 = ctx->cfg.act_dtype == B200MOE_F16;
  return encode_map(ctx, &three[0], gate, I, H, 64, fp16) && encode_map(ctx, &three[1], up, I, H, 64, fp16) &&
         encode_map(ctx, &three[2], down, H, I, 128, fp16);
}
#endif

extern "C" int b200moe_set_gate(b200moe_ctx* ctx, int layer, const void* gate_weight, const void* bias_or_null, void* stream) {
  int rc = check_layer(ctx, layer, "b200moe_set_gate");
  if (rc) return rc;
  if (!gate_weight || misaligned(gate_weight)) return fail(ctx, B200MOE_E_ARG, "b200moe_set_gate: gate weight must be a 16-byte aligned device pointer");
  CUDA_TRY(ctx, cudaSetDevice(ctx->cfg.device));
  ctx->gate_w[layer] = gate_weight;
  ctx->gate_bias[layer] = bias_or_null;
  (void)stream;  // nothing is enqueued: the pointers are read by later router launches
  return B200MOE_OK;
}

extern "C" int b200moe_set_expert(b200moe_ctx* ctx, int layer, int expert, const void* gate_proj, const void* up_proj,
                                  const void* down_proj, const void* gate_scales, const void* up_scales,
                                  const void* down_scales) {
  int rc = check_layer(ctx, layer, "b200moe_set_expert");
  if (rc) return rc;
  const int E = ctx->cfg.num_experts;
  if (expert < 0 || expert >= E) return fail(ctx, B200MOE_E_ARG, "b200moe_set_expert: expert %d out of range [0,%d)", expert, E);
  if (!gate_proj || !up_proj || !down_proj) return fail(ctx, B200MOE_E_ARG, "b200moe_set_expert: null weight pointer");
  if (misaligned(gate_proj) || misaligned(up_proj) || misaligned(down_proj))
    return fail(ctx, B200MOE_E_ARG, "b200moe_set_expert: weight pointers must be 16-byte aligned");
  const bool int4 = ctx->cfg.weight_mode == B200MOE_W_INT4_G128;
  if (int4 && (!gate_scales || !up_scales || !down_scales)) return fail(ctx, B200MOE_E_ARG, "b200moe_set_expert: int4 mode needs the three scale pointers");
  if (!int4 && (gate_scales || up_scales || down_scales)) return fail(ctx, B200MOE_E_ARG, "b200moe_set_expert: scales given but the context holds dense weights");
  if (int4 && (misaligned(gate_scales) || misaligned(up_scales) || misaligned(down_scales)))
    return fail(ctx, B200MOE_E_ARG, "b200moe_set_expert: scale pointers must be 16-byte aligned");
  ExpertPtrs& ep = ctx->h_experts[(size_t)layer * E + expert];
  ep.w[0] = gate_proj; ep.w[1] = up_proj; ep.w[2] = down_proj;
  ep.s[0] = gate_scales; ep.s[1] = up_scales; ep.s[2] = down_scales;
  ctx->registered[(size_t)layer * E + expert] = 1;
  ctx->dirty[layer] = 1;
#ifdef B200MOE_WITH_UMMA
  if (!ctx->h_tmaps.empty()) {
    const size_t idx = (size_t)layer * E + expert;
    bool ok = encode_expert_maps(ctx, &ctx->h_tmaps[idx * 3], gate_proj, up_proj, down_proj);
    if (ok && !ctx->h_tmaps2.empty()) {   // 128 k x 64/128 rows boxes for the tcgen05 int4 kernel
      const int H0 = ctx->cfg.hidden_size, I0 = ctx->cfg.intermediate_size;
      CUtensorMap* m = &ctx->h_tmaps2[idx * 3];
      ok = encode_map_u8(ctx, &m[0], gate_proj, I0, H0 / 2, 64, 64) && encode_map_u8(ctx, &m[1], up_proj, I0, H0 / 2, 64, 64) &&
           encode_map_u8(ctx, &m[2], down_proj, H0, I0 / 2, 64, 128);
    }
    ctx->tmap_ok[idx] = ok ? 1 : 0;
  }
#endif
  return B200MOE_OK;
}

extern "C" int b200moe_clear_expert(b200moe_ctx* ctx, int layer, int expert) {
  int rc = check_layer(ctx, layer, "b200moe_clear_expert");
  if (rc) return rc;
  const int E = ctx->cfg.num_experts;
  if (expert < 0 || expert >= E) return fail(ctx, B200MOE_E_ARG, "b200moe_clear_expert: expert %d out of range", expert);
  ctx->h_experts[(size_t)layer * E + expert] = ExpertPtrs{};
  ctx->registered[(size_t)layer * E + expert] = 0;
  ctx->dirty[layer] = 1;
  return B200MOE_OK;
}

// ------------------------------------------------------------------------------------------
// router
// ------------------------------------------------------------------------------------------
// The opt-in dynamic shared-memory size is a property of a kernel ON ONE DEVICE: remember per template
// instance which devices have been configured (one bit each), not just that some device was.
struct ConfiguredDevices {
  std::atomic<unsigned long long> mask{0};
  bool needs(int device) const { return device < 0 || device >= 64 || !((mask.load(std::memory_order_acquire) >> device) & 1ull); }
  void done(int device) { if (device >= 0 && device < 64) mask.fetch_or(1ull << device, std::memory_order_release); }
};

static void identity_slots(SlotTable& tab) {
  for (int e = 0; e < kMaxExperts; ++e) { tab.slot[e] = -1; tab.rank[e] = (uint8_t)(e & 255); }
}

// Largest batch (in pairs) whose grouping the router's last CTA takes over: its 256 threads group that
// many pairs about as fast as the separate kernel's CTA does, and one launch plus one dependency edge go.
constexpr int kFusePermuteMaxPairs = 512;

// Batches up to this size take the one-token-per-CTA router (grid T x E/8), larger ones the token-tile router.
constexpr int kRouterRowKernelMaxTokens = 32;   // measured on the Qwen3 shape: 32 tokens 21 against 24 us, 64 tokens 29 against 26 us

// `fuse` (with `tab`): the grouping tables of the batch are built by the router grid itself.
struct RouterNorm {          // RMSNorm fused into the router's load of the tokens (null weight = off)
  const void* residual = nullptr;
  const void* weight = nullptr;
  float eps = 0.0f;
  void* normed_out = nullptr;
  void* res_out = nullptr;
};

static int launch_router(b200moe_ctx* ctx, int layer, const void* x, const void* logits, int T, int64_t* ids_out,
                         void* scores_out, unsigned long long* bitmap_dev, cudaStream_t st, const PermuteParams* fuse = nullptr,
                         const SlotTable* tab = nullptr, const RouterNorm* norm = nullptr, bool ep_dispatch = false) {
  const b200moe_config& c = ctx->cfg;
  RouterParams p{};
  p.x = x;
  p.logits_in = logits;
  if (!logits) {
    p.wg = ctx->gate_w[layer];
    p.bias = ctx->gate_bias[layer];
  }
  p.logits = ctx->logits;
  p.tile_counter = ctx->tile_counter;
  p.ids64 = ids_out;
  p.scores = scores_out;
  p.bitmap = bitmap_dev;
  p.T = T; p.H = c.hidden_size; p.E = c.num_experts; p.K = c.top_k;
  p.all_done = ctx->tile_counter + c.max_tokens;
  const bool with_norm = norm != nullptr && norm->weight != nullptr;
  if (with_norm) {
    p.norm_res = norm->residual; p.norm_w = norm->weight; p.norm_eps = norm->eps; p.normed_out = norm->normed_out; p.res_out = norm->res_out;
    if (c.hidden_size % 8 || c.hidden_size > kNormThreads * kNormMaxChunks * 8)
      return fail(ctx, B200MOE_E_UNSUPPORTED, "fused norm: hidden size %d (multiples of 8 up to %d)", c.hidden_size, kNormThreads * kNormMaxChunks * 8);
  }
  EpPeers peers{};
  if (ep_dispatch) {       // the routed rows leave for their owners from the router's own tail
    p.ep_dispatch = 1; p.epg = ctx->ep.geom; p.ep_epoch = ctx->ep.counters; p.ep_dest_count = reinterpret_cast<int*>(ctx->ep.counters + 8);
    p.ep_status = ctx->status;
    peers = ctx->ep.peers;
  }
  SlotTable none;
  if (fuse && tab) { p.fuse_permute = 1; p.perm = *fuse; }
  else { identity_slots(none); tab = &none; }
  return dispatch_dtype(ctx, c.act_dtype, [&](auto tag) {
    using Tt = decltype(tag);
    ProfScope prof(ctx, B200MOE_KERNEL_ROUTER, st);
    if (logits) {
      launch_chain(router_from_logits_kernel<Tt>, dim3((T + 7) / 8), dim3(kRouterThreads), 0, st, p);
      return post_launch(ctx, "router_from_logits_kernel");
    }
    if (T <= kRouterRowKernelMaxTokens) {   // small batch: one token per tile, every load of a row in flight at once
      const unsigned ey = (c.num_experts + 7) / 8;
      if (with_norm) {
        const size_t row = (size_t)c.hidden_size * sizeof(Tt);
        auto kn = router_kernel<Tt, 1, 8, true>;
        static ConfiguredDevices configured_n;
        if (configured_n.needs(c.device)) {
          CUDA_TRY(ctx, cudaFuncSetAttribute(kn, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
          configured_n.done(c.device);
        }
        launch_chain(kn, dim3(T, ey), dim3(kRouterThreads), row, st, p, *tab, peers);
      } else {
        launch_chain(router_kernel<Tt, 1, 8>, dim3(T, ey), dim3(kRouterThreads), 0, st, p, *tab, peers);
      }
      return post_launch(ctx, "router_kernel");
    }
    // larger batches: token tile staged in shared memory, one expert row per warp
    const size_t smem = (size_t)kTileTokens * c.hidden_size * sizeof(Tt);
    auto k1 = router_tile_kernel<Tt, kTileTokens, 1>;
    auto k1n = router_tile_kernel<Tt, kTileTokens, 1, true>;
    static ConfiguredDevices configured;   // per template instance (one per element type)
    if (configured.needs(c.device)) {
      CUDA_TRY(ctx, cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
      CUDA_TRY(ctx, cudaFuncSetAttribute(k1n, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
      // several CTAs per SM: ask for the shared-memory end of the L1 / shared split
      CUDA_TRY(ctx, cudaFuncSetAttribute(k1, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
      CUDA_TRY(ctx, cudaFuncSetAttribute(k1n, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
      configured.done(c.device);
    }
    if (smem > 160 * 1024) return fail(ctx, B200MOE_E_UNSUPPORTED, "router: hidden size %d too large for the token tile", c.hidden_size);
    const dim3 grid((T + kTileTokens - 1) / kTileTokens, (c.num_experts + 7) / 8);
    launch_chain(with_norm ? k1n : k1, grid, dim3(kRouterThreads), smem, st, p, *tab, peers);
    return post_launch(ctx, "router_tile_kernel");
  });
}

static int route_common(b200moe_ctx* ctx, int layer, const void* x, const void* logits, int T, int64_t* ids_out,
                        void* scores_out, uint64_t* bitmap_out, void* stream, const char* who) {
  int rc = check_layer(ctx, layer, who);
  if (rc) return rc;
  if ((rc = check_tokens(ctx, T, who))) return rc;
  if (T > 0 && (!ids_out || !scores_out || (!x && !logits))) return fail(ctx, B200MOE_E_ARG, "%s: null pointer", who);
  if (!logits && x && !ctx->gate_w[layer]) return fail(ctx, B200MOE_E_STATE, "%s: no gate weight registered for layer %d", who, layer);
  if (x && misaligned(x)) return fail(ctx, B200MOE_E_ARG, "%s: x must be 16-byte aligned", who);
  CUDA_TRY(ctx, cudaSetDevice(ctx->cfg.device));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (T == 0) {
    if (bitmap_out) CUDA_TRY(ctx, cudaMemsetAsync(ctx->bitmap, 0, 32, st));
  } else {
    if (bitmap_out) CUDA_TRY(ctx, cudaMemsetAsync(ctx->bitmap, 0, 32, st));
    rc = launch_router(ctx, layer, x, logits, T, ids_out, scores_out, bitmap_out ? ctx->bitmap : nullptr, st);
    if (rc) return rc;
  }
  if (bitmap_out) CUDA_TRY(ctx, cudaMemcpyAsync(bitmap_out, ctx->bitmap, 32, cudaMemcpyDefault, st));
  return B200MOE_OK;
}

extern "C" int b200moe_route(b200moe_ctx* ctx, int layer, const void* x, int T, int64_t* ids_out, void* scores_out,
                             uint64_t* active_bitmap_out, void* stream) {
  if (!x && T > 0) return fail(ctx, B200MOE_E_ARG, "b200moe_route: null x");
  return route_common(ctx, layer, x, nullptr, T, ids_out, scores_out, active_bitmap_out, stream, "b200moe_route");
}

extern "C" int b200moe_route_from_logits(b200moe_ctx* ctx, const void* logits, int T, int64_t* ids_out, void* scores_out,
                                         uint64_t* active_bitmap_out, void* stream) {
  if (!logits && T > 0) return fail(ctx, B200MOE_E_ARG, "b200moe_route_from_logits: null logits");
  return route_common(ctx, 0, nullptr, logits, T, ids_out, scores_out, active_bitmap_out, stream, "b200moe_route_from_logits");
}

extern "C" int b200moe_last_logits(b200moe_ctx* ctx, int T, float* logits_out, void* stream) {
  if (!ctx || !logits_out) return fail(ctx, B200MOE_E_ARG, "b200moe_last_logits: null argument");
  int rc = check_tokens(ctx, T, "b200moe_last_logits");
  if (rc) return rc;
  CUDA_TRY(ctx, cudaSetDevice(ctx->cfg.device));
  CUDA_TRY(ctx, cudaMemcpyAsync(logits_out, ctx->logits, (size_t)T * ctx->cfg.num_experts * sizeof(float),
                                cudaMemcpyDeviceToDevice, reinterpret_cast<cudaStream_t>(stream)));
  return B200MOE_OK;
}

extern "C" int b200moe_last_tables(b200moe_ctx* ctx, int T, int32_t* offsets_out, int32_t* sorted_pair_out, int32_t* inv_out,
                                   int32_t* act_list_out, int32_t* n_act_out, void* stream) {
  if (!ctx) return fail(nullptr, B200MOE_E_ARG, "b200moe_last_tables: null context");
  int rc = check_tokens(ctx, T, "b200moe_last_tables");
  if (rc) return rc;
  CUDA_TRY(ctx, cudaSetDevice(ctx->cfg.device));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const size_t pairs = (size_t)T * ctx->cfg.top_k, E = ctx->cfg.num_experts;
  if (offsets_out) CUDA_TRY(ctx, cudaMemcpyAsync(offsets_out, ctx->offsets, (E + 1) * sizeof(int), cudaMemcpyDefault, st));
  if (sorted_pair_out && pairs) CUDA_TRY(ctx, cudaMemcpyAsync(sorted_pair_out, ctx->sorted_pair, pairs * sizeof(int), cudaMemcpyDefault, st));
  if (inv_out && pairs) CUDA_TRY(ctx, cudaMemcpyAsync(inv_out, ctx->inv, pairs * sizeof(int), cudaMemcpyDefault, st));
  if (act_list_out) CUDA_TRY(ctx, cudaMemcpyAsync(act_list_out, ctx->act_list, E * sizeof(int), cudaMemcpyDefault, st));
  if (n_act_out) CUDA_TRY(ctx, cudaMemcpyAsync(n_act_out, ctx->n_act, sizeof(int), cudaMemcpyDefault, st));
  return B200MOE_OK;
}

extern "C" int b200moe_group_pairs(b200moe_ctx* ctx, const int64_t* ids, int T, int32_t* tables_out, void* stream) {
  if (!ctx) return fail(nullptr, B200MOE_E_ARG, "b200moe_group_pairs: null context");
  int rc = check_tokens(ctx, T, "b200moe_group_pairs");
  if (rc) return rc;
  if (T == 0) return B200MOE_OK;
  if (!ids || !tables_out) return fail(ctx, B200MOE_E_ARG, "b200moe_group_pairs: null pointer");
  const b200moe_config& c = ctx->cfg;
  CUDA_TRY(ctx, cudaSetDevice(c.device));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int E = c.num_experts;
  SlotTable tab;
  for (int e = 0; e < kMaxExperts; ++e) { tab.slot[e] = (int16_t)(e < E ? e : -1); tab.rank[e] = (uint8_t)(e & 255); }
  PermuteParams pp{};
  pp.ids64 = ids; pp.T = T; pp.K = c.top_k; pp.E = E;
  pp.offsets = ctx->offsets; pp.sorted_pair = ctx->sorted_pair; pp.inv = ctx->inv;
  pp.act_list = ctx->act_list; pp.n_act = ctx->n_act; pp.status = ctx->status;
  pp.ep_cap = -1;                                    // ids outside [0,E) are dropped without a status bit, as the reference's `==` test drops them
  const int pthreads = std::min(kPermuteMaxThreads, std::max(256, (T * c.top_k + 31) / 32 * 32));
  const size_t smem = (size_t)((pthreads / 32) * E + E) * sizeof(int);
  launch_chain(permute_kernel, dim3(1), dim3(pthreads), smem, st, pp, tab);
  if ((rc = post_launch(ctx, "permute_kernel"))) return rc;
  CUDA_TRY(ctx, cudaMemcpyAsync(tables_out, ctx->offsets, (size_t)(E + 1) * sizeof(int), cudaMemcpyDefault, st));
  CUDA_TRY(ctx, cudaMemcpyAsync(tables_out + E + 1, ctx->sorted_pair, (size_t)T * c.top_k * sizeof(int), cudaMemcpyDefault, st));
  return B200MOE_OK;
}

// ------------------------------------------------------------------------------------------
// expert execution
// ------------------------------------------------------------------------------------------
static int upload_layer_table(b200moe_ctx* ctx, int layer, cudaStream_t st) {
  if (!ctx->dirty[layer]) return B200MOE_OK;
  const int E = ctx->cfg.num_experts;
  // pageable source: the runtime stages the bytes before returning, and the copy is ordered
  // behind earlier work of `st` that may still read the old table
  CUDA_TRY(ctx, cudaMemcpyAsync(ctx->d_experts + (size_t)layer * E, ctx->h_experts.data() + (size_t)layer * E,
                                E * sizeof(ExpertPtrs), cudaMemcpyHostToDevice, st));
#ifdef B200MOE_WITH_UMMA
  if (!ctx->h_tmaps.empty())
    CUDA_TRY(ctx, cudaMemcpyAsync(ctx->d_tmaps + (size_t)layer * E * 3, ctx->h_tmaps.data() + (size_t)layer * E * 3,
                                  (size_t)E * 3 * sizeof(CUtensorMap), cudaMemcpyHostToDevice, st));
  if (!ctx->h_tmaps2.empty())
    CUDA_TRY(ctx, cudaMemcpyAsync(ctx->d_tmaps2 + (size_t)layer * E * 3, ctx->h_tmaps2.data() + (size_t)layer * E * 3,
                                  (size_t)E * 3 * sizeof(CUtensorMap), cudaMemcpyHostToDevice, st));
#endif
  ctx->dirty[layer] = 0;
  return B200MOE_OK;
}

struct FfnLaunch {
  const ExpertPtrs* experts;
  const int* offsets;
  const int* sorted_pair;
  const int* act_list;
  const int* n_act;
  const void* x;
  void* h;
  void* y;
  int K;        // pairs per token in sorted_pair
  const void* tmaps;  // tensor maps matching `experts` (null when the tensor-core path cannot run)
  const void* tmaps2 = nullptr;  // int4: boxes of the tcgen05 int4 kernel
  int max_n;    // tokens per expert the kernels size their token tile for; experts holding more take several passes
  int n_tokens = 0;      // rows of x (only the int4 tcgen05 path needs it)
  int n_act_bound = 1;   // upper bound on the number of experts with work
  bool ksplit_ok = false;   // the consumer of y accepts fp32 K-slices (the combine kernel does)
};

using GemvDefault = GemvShape<8, 2048, 3>;

// which: bit 0 = gate/up projection, bit 1 = down projection
template <typename T, int NT, typename S> static int launch_gemv_pair_shape(b200moe_ctx* ctx, const FfnParams& p, const SlotTable& st, cudaStream_t s, int which = 3) {
  const int grid = ctx->sm_count;   // one persistent CTA per SM: the rings take most of its shared memory
  auto up = ffn_gemv_kernel<T, NT, true, S>;
  auto down = ffn_gemv_kernel<T, NT, false, S>;
  static ConfiguredDevices configured;   // per template instance
  if (configured.needs(ctx->cfg.device)) {
    CUDA_TRY(ctx, cudaFuncSetAttribute(up, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)S::SMEM));
    CUDA_TRY(ctx, cudaFuncSetAttribute(down, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)S::SMEM));
    configured.done(ctx->cfg.device);
  }
  if (which & 1) {
    {
      ProfScope prof(ctx, B200MOE_KERNEL_FFN_GATEUP, s);
      launch_chain(up, dim3(grid), dim3(S::THREADS), S::SMEM, s, p, st, ctx->status);
    }
    int rc = post_launch(ctx, "ffn_gemv_kernel<gate/up>");
    if (rc) return rc;
  }
  if (!(which & 2)) return B200MOE_OK;
  {
    ProfScope prof(ctx, B200MOE_KERNEL_FFN_DOWN, s);
    launch_chain(down, dim3(grid), dim3(S::THREADS), S::SMEM, s, p, st, ctx->status);
  }
  return post_launch(ctx, "ffn_gemv_kernel<down>");
}

template <typename T, int NT> static int launch_gemv_pair(b200moe_ctx* ctx, const FfnParams& p, const SlotTable& st, cudaStream_t s, int which = 3) {
  return launch_gemv_pair_shape<T, NT, GemvDefault>(ctx, p, st, s, which);
}

#ifdef B200MOE_WITH_UMMA
template <typename T, int NMAX> static int launch_umma_pair(b200moe_ctx* ctx, const UmmaParams& up, const SlotTable& st, cudaStream_t s, int which = 3) {
  using S = UmmaShape<NMAX>;
  auto k_up = ffn_umma_kernel<T, NMAX, true>;
  auto k_down = ffn_umma_kernel<T, NMAX, false>;
  static ConfiguredDevices configured;   // per template instance
  if (configured.needs(ctx->cfg.device)) {
    CUDA_TRY(ctx, cudaFuncSetAttribute(k_up, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)S::SMEM));
    CUDA_TRY(ctx, cudaFuncSetAttribute(k_down, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)S::SMEM));
    configured.done(ctx->cfg.device);
  }
  if (which & 1) {
    {
      ProfScope prof(ctx, B200MOE_KERNEL_FFN_GATEUP, s);
      launch_chain(k_up, dim3(ctx->sm_count), dim3(kUmmaThreads), S::SMEM, s, up, st);
    }
    int rc = post_launch(ctx, "ffn_umma_kernel<gate/up>");
    if (rc) return rc;
  }
  if (!(which & 2)) return B200MOE_OK;
  {
    ProfScope prof(ctx, B200MOE_KERNEL_FFN_DOWN, s);
    launch_chain(k_down, dim3(ctx->sm_count), dim3(kUmmaThreads), S::SMEM, s, up, st);
  }
  return post_launch(ctx, "ffn_umma_kernel<down>");
}

// max_n bounds the tokens any expert can hold in this call (the batch size); a pass of the
// kernel covers NMAX tokens, so larger per-expert counts only cost extra passes.
static int launch_ffn_umma(b200moe_ctx* ctx, const FfnParams& p, const void* tmaps, const SlotTable& st, int max_n, int n_act_bound,
                           bool ksplit_ok, cudaStream_t s, int which = 3) {
  if (!tmaps) return fail(ctx, B200MOE_E_UNSUPPORTED, "tensor-core path unavailable: no TMA descriptors for these experts");
  UmmaParams up{};
  up.f = p;
  up.tmaps = reinterpret_cast<const CUtensorMap*>(tmaps);
  up.status = ctx->status;
  // K split of the down projection: aim at >= 8 work items per SM (n_act_bound experts x H/128 tiles)
  up.ksplit = 1;
  up.ypart = ctx->ypart;
  up.pairs_cap = ctx->cfg.max_tokens * ctx->cfg.top_k;
  if (ksplit_ok && ctx->ypart_slices >= 2) {
    const int tiles = (p.H + 127) / 128, nkb = (p.I + 63) / 64;
    const int items = std::max(1, n_act_bound * tiles);
    int want = (8 * ctx->sm_count + items - 1) / items;
    const int cap = std::min(std::min(want, ctx->ypart_slices), std::max(1, nkb / 16));   // a slice keeps >= 16 k-blocks (1024 of K)
    // Among the allowed splits take the one whose work items fill whole rounds of the grid best: the items
    // are equal-sized, so the launch lasts ceil(items * ks / SMs) rounds whatever the last round holds.
    int best = 1;
    double best_eff = 0.0;
    for (int ks = std::max(1, cap / 2); ks <= cap; ++ks) {
      const long long n = (long long)items * ks;
      const long long rounds = (n + ctx->sm_count - 1) / ctx->sm_count;
      const double eff = (double)n / (double)(rounds * ctx->sm_count);
      if (eff > best_eff + 1e-9) { best_eff = eff; best = ks; }
    }
    up.ksplit = std::max(1, best);
  }
  ctx->last_ksplit = up.ksplit;
  if (ctx->cfg.act_dtype == B200MOE_F16) {
    if (max_n <= 16) return launch_umma_pair<__half, 16>(ctx, up, st, s, which);
    if (max_n <= 32) return launch_umma_pair<__half, 32>(ctx, up, st, s, which);
    if (max_n <= 64) return launch_umma_pair<__half, 64>(ctx, up, st, s, which);
    return launch_umma_pair<__half, 128>(ctx, up, st, s, which);
  }
  if (max_n <= 16) return launch_umma_pair<__nv_bfloat16, 16>(ctx, up, st, s, which);
  if (max_n <= 32) return launch_umma_pair<__nv_bfloat16, 32>(ctx, up, st, s, which);
  if (max_n <= 64) return launch_umma_pair<__nv_bfloat16, 64>(ctx, up, st, s, which);
  return launch_umma_pair<__nv_bfloat16, 128>(ctx, up, st, s, which);
}
#endif

#ifdef B200MOE_WITH_INT4
template <int NTILE> static int launch_int4_pair(b200moe_ctx* ctx, const Int4Params& ip, const SlotTable& st, cudaStream_t s) {
  auto k_up = ffn_int4_kernel<true, NTILE>;
  auto k_down = ffn_int4_kernel<false, NTILE>;
  static ConfiguredDevices configured;   // per template instance
  if (configured.needs(ctx->cfg.device)) {
    CUDA_TRY(ctx, cudaFuncSetAttribute(k_up, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kInt4Smem));
    CUDA_TRY(ctx, cudaFuncSetAttribute(k_down, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kInt4Smem));
    configured.done(ctx->cfg.device);
  }
  {
    ProfScope prof(ctx, B200MOE_KERNEL_FFN_GATEUP, s);
    launch_chain(k_up, dim3(ctx->sm_count), dim3(kInt4Threads), kInt4Smem, s, ip, st);
  }
  int rc = post_launch(ctx, "ffn_int4_kernel<gate/up>");
  if (rc) return rc;
  {
    ProfScope prof(ctx, B200MOE_KERNEL_FFN_DOWN, s);
    launch_chain(k_down, dim3(ctx->sm_count), dim3(kInt4Threads), kInt4Smem, s, ip, st);
  }
  return post_launch(ctx, "ffn_int4_kernel<down>");
}

template <int NMAX> static int launch_i4u_pair(b200moe_ctx* ctx, const I4uParams& ip_up, const I4uParams& ip_down, const SlotTable& st, cudaStream_t s) {
  using S = I4uShape<NMAX>;
  auto k_up = ffn_int4_umma_kernel<NMAX, true>;
  auto k_down = ffn_int4_umma_kernel<NMAX, false>;
  static ConfiguredDevices configured;   // per template instance
  if (configured.needs(ctx->cfg.device)) {
    CUDA_TRY(ctx, cudaFuncSetAttribute(k_up, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)S::SMEM));
    CUDA_TRY(ctx, cudaFuncSetAttribute(k_down, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)S::SMEM));
    configured.done(ctx->cfg.device);
  }
  {
    ProfScope prof(ctx, B200MOE_KERNEL_FFN_GATEUP, s);
    launch_chain(k_up, dim3(ctx->sm_count), dim3(kI4uThreads), S::SMEM, s, ip_up, st);
  }
  int rc = post_launch(ctx, "ffn_int4_umma_kernel<gate/up>");
  if (rc) return rc;
  {
    ProfScope prof(ctx, B200MOE_KERNEL_FFN_DOWN, s);
    launch_chain(k_down, dim3(ctx->sm_count), dim3(kI4uThreads), S::SMEM, s, ip_down, st);
  }
  return post_launch(ctx, "ffn_int4_umma_kernel<down>");
}

static int launch_ffn_int4_umma(b200moe_ctx* ctx, const FfnParams& p, const void* tmaps, const SlotTable& st, int max_n, int n_tokens,
                                cudaStream_t s) {
  const size_t pairs_cap = (size_t)ctx->cfg.max_tokens * ctx->cfg.top_k;
  I4uParams ip_up{}, ip_down{};
  ip_up.f = p;
  ip_up.tmaps = reinterpret_cast<const CUtensorMap*>(tmaps);
  ip_up.status = ctx->status;
  ip_down = ip_up;
  // token rows of the two passes as TMA tensors: the gathered copy of x, and h
  if (!encode_map(ctx, &ip_up.bmap, ctx->xperm, (int)pairs_cap, p.H, 16) || !encode_map(ctx, &ip_down.bmap, p.h, (int)pairs_cap, p.I, 16))
    return fail(ctx, B200MOE_E_STATE, "int4 tensor-core path: cuTensorMapEncodeTiled failed for the token tiles");
  {
    ProfScope prof(ctx, B200MOE_KERNEL_PERMUTE, s);
    const long long chunks = (long long)n_tokens * p.K * (p.H / 8);
    const int grid = (int)std::min<long long>(4LL * ctx->sm_count, std::max<long long>(1, (chunks + 255) / 256));
    launch_chain(i4u_gather_x_kernel, dim3(grid), dim3(256), 0, s, reinterpret_cast<const __nv_bfloat16*>(p.x),
                 reinterpret_cast<__nv_bfloat16*>(ctx->xperm), p.sorted_pair, p.offsets, ctx->cfg.num_experts, p.K, p.H);
  }
  int rc0 = post_launch(ctx, "i4u_gather_x_kernel");
  if (rc0) return rc0;
  if (max_n <= 16) return launch_i4u_pair<16>(ctx, ip_up, ip_down, st, s);
  if (max_n <= 32) return launch_i4u_pair<32>(ctx, ip_up, ip_down, st, s);
  if (max_n <= 64) return launch_i4u_pair<64>(ctx, ip_up, ip_down, st, s);
  return launch_i4u_pair<128>(ctx, ip_up, ip_down, st, s);
}

static int launch_ffn_int4(b200moe_ctx* ctx, const FfnParams& p, const void* tmaps, const SlotTable& st, int max_n, cudaStream_t s) {
  if (!tmaps) return fail(ctx, B200MOE_E_STATE, "int4 path: no TMA descriptors for these experts (cuTensorMapEncodeTiled unavailable or failed)");
  Int4Params ip{};
  ip.f = p;
  ip.tmaps = reinterpret_cast<const CUtensorMap*>(tmaps);
  ip.status = ctx->status;
  if (max_n <= 8) return launch_int4_pair<1>(ctx, ip, st, s);
  if (max_n <= 16) return launch_int4_pair<2>(ctx, ip, st, s);
  return launch_int4_pair<4>(ctx, ip, st, s);
}
#endif

static int launch_ffn(b200moe_ctx* ctx, const FfnLaunch& f, const SlotTable& st, int ffn_kind, cudaStream_t s) {
  const b200moe_config& c = ctx->cfg;
  FfnParams p{};
  p.x = f.x; p.h = f.h; p.y = f.y;
  p.experts = f.experts; p.offsets = f.offsets; p.sorted_pair = f.sorted_pair; p.act_list = f.act_list; p.n_act = f.n_act;
  p.H = c.hidden_size; p.I = c.intermediate_size; p.K = f.K;
  if (c.weight_mode == B200MOE_W_INT4_G128) {
#ifdef B200MOE_WITH_INT4
    // The tcgen05 kernel (dequantised tiles in tensor memory) is faster than the register-fragment
    // kernel at every measured batch (Mixtral-shaped T = 1..64, Qwen3-shaped T = 1..256); the latter
    // stays reachable as B200MOE_FFN_GEMV and is what runs when no TMA descriptor could be made.
    if (f.tmaps2 && ffn_kind != B200MOE_FFN_GEMV)
      return launch_ffn_int4_umma(ctx, p, f.tmaps2, st, f.max_n, f.n_tokens, s);
    return launch_ffn_int4(ctx, p, f.tmaps, st, f.max_n, s);
#else
    return fail(ctx, B200MOE_E_UNSUPPORTED, "library built without the int4 kernels");
#endif
  }
#ifdef B200MOE_WITH_UMMA
  if ((c.act_dtype == B200MOE_BF16 || c.act_dtype == B200MOE_F16) && ffn_kind == B200MOE_FFN_AUTO && f.max_n <= 1 && f.tmaps) {
    // Single token: the GEMV kernel is the faster gate/up projection (2 rows per warp unit fill the GPU),
    // the tensor-core kernel with its K split the faster down projection (measured 47 against 65 us on the
    // Mixtral-shaped layer, 13 against 16.5 us on the Qwen3-shaped one).  Both use the same h layout.
    int rc = dispatch_dtype(ctx, c.act_dtype, [&](auto tag) {
      using T = decltype(tag);
      return launch_gemv_pair<T, 1>(ctx, p, st, s, 1);
    });
    if (rc) return rc;
    return launch_ffn_umma(ctx, p, f.tmaps, st, f.max_n, f.n_act_bound, f.ksplit_ok, s, 2);
  }
  if ((c.act_dtype == B200MOE_BF16 || c.act_dtype == B200MOE_F16) && ffn_kind != B200MOE_FFN_GEMV && (ffn_kind == B200MOE_FFN_MMA || f.max_n > 1)) {
    int rc = launch_ffn_umma(ctx, p, f.tmaps, st, f.max_n, f.n_act_bound, f.ksplit_ok, s);
    if (rc != B200MOE_E_UNSUPPORTED) return rc;
    if (ffn_kind == B200MOE_FFN_MMA) return rc;
  }
#else
  if (ffn_kind == B200MOE_FFN_MMA) return fail(ctx, B200MOE_E_UNSUPPORTED, "library built without the tensor-core kernels");
#endif
  return dispatch_dtype(ctx, c.act_dtype, [&](auto tag) {
    using T = decltype(tag);
    if (f.max_n <= 1) return launch_gemv_pair<T, 1>(ctx, p, st, s);
    if (f.max_n <= 2) return launch_gemv_pair<T, 2>(ctx, p, st, s);
    return launch_gemv_pair<T, 4>(ctx, p, st, s);
  });
}

// Single-token batch of a dense 16-bit model through the fused entry: one cooperative launch (moe_token.cuh).
// Returns B200MOE_E_UNSUPPORTED (without recording an error) when the shape or the device cannot take it.
static int launch_token(b200moe_ctx* ctx, int layer, const void* x, int64_t* ids, void* scores, const void* residual, void* out,
                        const PermuteParams& pp, const SlotTable& tab, const RouterNorm* norm, cudaStream_t st) {
  const b200moe_config& c = ctx->cfg;
  if (c.weight_mode != B200MOE_W_DENSE || c.act_dtype == B200MOE_F32) return B200MOE_E_UNSUPPORTED;
  if (c.hidden_size % 8 || c.intermediate_size % 8 || (size_t)c.hidden_size * 2 > (size_t)kTokenMaxRowBytes) return B200MOE_E_UNSUPPORTED;
  using S = GemvDefault;
  TokenParams p{};
  p.r.x = x; p.r.wg = ctx->gate_w[layer]; p.r.bias = ctx->gate_bias[layer];
  p.r.logits = ctx->logits; p.r.ids64 = ids; p.r.scores = scores;
  p.r.T = 1; p.r.H = c.hidden_size; p.r.E = c.num_experts; p.r.K = c.top_k;
  p.r.perm = pp;
  if (norm && norm->weight) {
    if (c.hidden_size > kNormMaxChunks * kNormThreads * 8) return B200MOE_E_UNSUPPORTED;
    p.r.norm_res = norm->residual; p.r.norm_w = norm->weight; p.r.norm_eps = norm->eps;
    p.r.normed_out = norm->normed_out; p.r.res_out = norm->res_out;
  }
  p.experts = ctx->d_experts + (size_t)layer * c.num_experts;
  p.h = ctx->h; p.residual = residual; p.out = out; p.I = c.intermediate_size;
  p.gbar = ctx->tile_counter + c.max_tokens + 1;
  p.status = ctx->status;
  p.wait_cycles = 1ll << 31;
  return dispatch_dtype(ctx, c.act_dtype, [&](auto tag) -> int {
    using Tt = decltype(tag);
    if constexpr (sizeof(Tt) != 2) {
      return B200MOE_E_UNSUPPORTED;
    } else {
      auto kn = moe_token_kernel<Tt, S>;
      constexpr size_t smem = token_smem_bytes<S>();
      static ConfiguredDevices configured, usable;   // per template instance
      if (configured.needs(c.device)) {
        int coop = 0, per_sm = 0;
        cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, c.device);
        if (cudaFuncSetAttribute(kn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess &&
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kn, S::THREADS, smem) == cudaSuccess && coop && per_sm >= 1)
          usable.done(c.device);
        cudaGetLastError();
        configured.done(c.device);
      }
      if (usable.needs(c.device)) return B200MOE_E_UNSUPPORTED;
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(ctx->sm_count);
      cfg.blockDim = dim3(S::THREADS);
      cfg.dynamicSmemBytes = smem;
      cfg.stream = st;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeCooperative;     // every CTA resident: the grid barriers cannot starve
      attr[0].val.cooperative = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      {
        ProfScope prof(ctx, B200MOE_KERNEL_TOKEN, st);
        cudaLaunchKernelEx(&cfg, kn, p, tab);
      }
      return post_launch(ctx, "moe_token_kernel");
    }
  });
}

// Batches of two tokens of a dense 16-bit model through the fused entry: one cooperative launch (moe_tokens.cuh).
// Same contract as launch_token.
template <typename Tt, int NT>
static int launch_tokens_nt(b200moe_ctx* ctx, const TokenParams& p, const SlotTable& tab, cudaStream_t st) {
  const b200moe_config& c = ctx->cfg;
  auto kn = moe_tokens_kernel<Tt, NT>;
  static ConfiguredDevices configured, usable;   // per template instance
  if (configured.needs(c.device)) {
    int coop = 0, per_sm = 0;
    cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, c.device);
    if (cudaFuncSetAttribute(kn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTokensSmemBytes) == cudaSuccess &&
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kn, TokensShape::THREADS, kTokensSmemBytes) == cudaSuccess && coop && per_sm >= 1)
      usable.done(c.device);
    cudaGetLastError();
    configured.done(c.device);
  }
  if (usable.needs(c.device)) return B200MOE_E_UNSUPPORTED;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ctx->sm_count);
  cfg.blockDim = dim3(TokensShape::THREADS);
  cfg.dynamicSmemBytes = kTokensSmemBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;     // every CTA resident: the grid barriers cannot starve
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  {
    ProfScope prof(ctx, B200MOE_KERNEL_TOKEN, st);
    cudaLaunchKernelEx(&cfg, kn, p, tab);
  }
  return post_launch(ctx, "moe_tokens_kernel");
}

static int launch_tokens(b200moe_ctx* ctx, int layer, const void* x, int T, int64_t* ids, void* scores, const void* residual, void* out,
                         const PermuteParams& pp, const SlotTable& tab, const RouterNorm* norm, cudaStream_t st) {
  const b200moe_config& c = ctx->cfg;
  if (c.weight_mode != B200MOE_W_DENSE || c.act_dtype == B200MOE_F32) return B200MOE_E_UNSUPPORTED;
  if (c.hidden_size % 8 || c.intermediate_size % 8) return B200MOE_E_UNSUPPORTED;
  if (T != 2 || T * c.top_k > kTokensMaxPairs || (size_t)T * c.hidden_size * 2 > (size_t)kTokenMaxRowBytes ||
      (size_t)T * c.top_k * c.intermediate_size * 2 > (size_t)kTokensMaxHBytes)
    return B200MOE_E_UNSUPPORTED;
  TokenParams p{};
  p.r.x = x; p.r.wg = ctx->gate_w[layer]; p.r.bias = ctx->gate_bias[layer];
  p.r.logits = ctx->logits; p.r.ids64 = ids; p.r.scores = scores;
  p.r.T = T; p.r.H = c.hidden_size; p.r.E = c.num_experts; p.r.K = c.top_k;
  p.r.perm = pp;
  if (norm && norm->weight) {
    if (c.hidden_size > kNormMaxChunks * kNormThreads * 8) return B200MOE_E_UNSUPPORTED;
    p.r.norm_res = norm->residual; p.r.norm_w = norm->weight; p.r.norm_eps = norm->eps;
    p.r.normed_out = norm->normed_out; p.r.res_out = norm->res_out;
  }
  p.experts = ctx->d_experts + (size_t)layer * c.num_experts;
  p.h = ctx->h; p.residual = residual; p.out = out; p.I = c.intermediate_size;
  p.gbar = ctx->tile_counter + c.max_tokens + 1;
  p.status = ctx->status;
  p.wait_cycles = 1ll << 31;
  return dispatch_dtype(ctx, c.act_dtype, [&](auto tag) -> int {
    using Tt = decltype(tag);
    if constexpr (sizeof(Tt) != 2) {
      return B200MOE_E_UNSUPPORTED;
    } else {
      return launch_tokens_nt<Tt, 2>(ctx, p, tab, st);
    }
  });
}

// route_first: the ids / scores buffers are OUTPUTS of the router, which this call launches first (fused entry).
static int run_experts(b200moe_ctx* ctx, int layer, const void* x, int T, const int64_t* ids, const void* scores,
                       int scores_dtype, const int32_t* expert_slot, const int32_t* order, const void* residual,
                       void* out, int ffn_kind, cudaStream_t st, bool route_first = false, const void* route_x = nullptr,
                       const RouterNorm* norm = nullptr) {
  const b200moe_config& c = ctx->cfg;
  const int E = c.num_experts;
  SlotTable tab;
  for (int e = 0; e < kMaxExperts; ++e) { tab.slot[e] = -1; tab.rank[e] = (uint8_t)(e & 255); }
  for (int e = 0; e < E; ++e) {
    int s = expert_slot ? expert_slot[e] : e;
    if (s >= E) return fail(ctx, B200MOE_E_ARG, "expert_slot[%d]=%d out of range", e, s);
    if (s >= 0 && !ctx->registered[(size_t)layer * E + s]) s = -1;
    tab.slot[e] = (int16_t)(s < 0 ? -1 : s);
    if (order) {
      if (order[e] < 0 || order[e] > 255) return fail(ctx, B200MOE_E_ARG, "order[%d]=%d out of range [0,255]", e, order[e]);
      tab.rank[e] = (uint8_t)order[e];
    }
  }
  int rc = upload_layer_table(ctx, layer, st);
  if (rc) return rc;

  PermuteParams pp{};
  pp.ids64 = ids; pp.T = T; pp.K = c.top_k; pp.E = E;
  pp.offsets = ctx->offsets; pp.sorted_pair = ctx->sorted_pair; pp.inv = ctx->inv;
  pp.act_list = ctx->act_list; pp.n_act = ctx->n_act; pp.status = ctx->status;
  if (route_first && T == 1 && ffn_kind == B200MOE_FFN_AUTO && ctx->token_kernel) {
    rc = launch_token(ctx, layer, route_x ? route_x : x, const_cast<int64_t*>(ids), const_cast<void*>(scores), residual, out, pp, tab, norm, st);
    if (rc != B200MOE_E_UNSUPPORTED) return rc;
  }
  if (route_first && T == 2 && !order && !expert_slot && ffn_kind == B200MOE_FFN_AUTO && ctx->token_kernel) {
    rc = launch_tokens(ctx, layer, route_x ? route_x : x, T, const_cast<int64_t*>(ids), const_cast<void*>(scores), residual, out, pp, tab, norm, st);
    if (rc != B200MOE_E_UNSUPPORTED) return rc;
  }
  const bool fused_grouping = route_first && T * c.top_k <= kFusePermuteMaxPairs;
  if (route_first &&
      (rc = launch_router(ctx, layer, route_x ? route_x : x, nullptr, T, const_cast<int64_t*>(ids), const_cast<void*>(scores), nullptr, st,
                          fused_grouping ? &pp : nullptr, &tab, norm)))
    return rc;
  if (!fused_grouping) {
    const int pthreads = std::min(kPermuteMaxThreads, std::max(256, (T * c.top_k + 31) / 32 * 32));
    const size_t smem = (size_t)((pthreads / 32) * E + E) * sizeof(int);
    {
      ProfScope prof(ctx, B200MOE_KERNEL_PERMUTE, st);
      launch_chain(permute_kernel, dim3(1), dim3(pthreads), smem, st, pp, tab);
    }
    if ((rc = post_launch(ctx, "permute_kernel"))) return rc;
  }

  FfnLaunch f{};
  f.experts = ctx->d_experts + (size_t)layer * E;
  f.offsets = ctx->offsets; f.sorted_pair = ctx->sorted_pair; f.act_list = ctx->act_list; f.n_act = ctx->n_act;
  f.x = x; f.h = ctx->h; f.y = ctx->y; f.K = c.top_k;
  {
    // Token-tile size: four times the mean load of an expert (measured best on uniform and on
    // Zipf-skewed routing), at least 16, never more than the batch.  A popular expert that holds
    // more tokens is processed in several passes over its weights, which then come from L2.
    const long long n_mean = ((long long)T * c.top_k + E - 1) / E;
    f.max_n = (int)std::min<long long>(T, std::max<long long>(16, 4 * n_mean));
  }
  f.n_tokens = T;
  f.n_act_bound = (int)std::min<long long>(E, (long long)T * c.top_k);
  f.ksplit_ok = true;
  ctx->last_ksplit = 1;
#ifdef B200MOE_WITH_UMMA
  if (!ctx->h_tmaps.empty()) {
    bool all_ok = true;
    for (int e = 0; e < E; ++e)
      if (tab.slot[e] >= 0 && !ctx->tmap_ok[(size_t)layer * E + tab.slot[e]]) all_ok = false;
    if (all_ok) f.tmaps = ctx->d_tmaps + (size_t)layer * E * 3;
    if (all_ok && ctx->d_tmaps2) f.tmaps2 = ctx->d_tmaps2 + (size_t)layer * E * 3;
  }
#endif
  if ((rc = launch_ffn(ctx, f, tab, ffn_kind, st))) return rc;

  CombineParams cp{};
  if (ctx->last_ksplit > 1) { cp.ypart = ctx->ypart; cp.y_parts = ctx->last_ksplit; cp.pairs_cap = c.max_tokens * c.top_k; }
  cp.y = ctx->y; cp.inv = ctx->inv; cp.ids64 = ids; cp.scores = scores;
  cp.scores_f32 = (scores_dtype == B200MOE_F32 && c.act_dtype != B200MOE_F32) ? 1 : 0;
  cp.residual = residual; cp.out = out; cp.T = T; cp.H = c.hidden_size; cp.K = c.top_k; cp.E = E;
  return dispatch_dtype(ctx, c.act_dtype, [&](auto tag) {
    using Tt = decltype(tag);
    ProfScope prof(ctx, B200MOE_KERNEL_COMBINE, st);
    launch_chain(combine_kernel<Tt>, dim3(T), dim3(kCombineThreads), 0, st, cp, tab);
    return post_launch(ctx, "combine_kernel");
  });
}

extern "C" int b200moe_forward(b200moe_ctx* ctx, int layer, const void* x, int T, const int64_t* ids, const void* scores,
                               int scores_dtype, const int32_t* expert_slot, const int32_t* order, const void* residual,
                               void* out, int ffn_kind, void* stream) {
  int rc = check_layer(ctx, layer, "b200moe_forward");
  if (rc) return rc;
  if ((rc = check_tokens(ctx, T, "b200moe_forward"))) return rc;
  if (T == 0) return B200MOE_OK;
  if (!x || !ids || !scores || !out) return fail(ctx, B200MOE_E_ARG, "b200moe_forward: null pointer");
  if (misaligned(x) || misaligned(out) || (residual && misaligned(residual)))
    return fail(ctx, B200MOE_E_ARG, "b200moe_forward: x, out and residual must be 16-byte aligned");
  if (scores_dtype != ctx->cfg.act_dtype && scores_dtype != B200MOE_F32)
    return fail(ctx, B200MOE_E_ARG, "b200moe_forward: scores must be in the activation dtype or fp32");
  if (ffn_kind < B200MOE_FFN_AUTO || ffn_kind > B200MOE_FFN_MMA) return fail(ctx, B200MOE_E_ARG, "b200moe_forward: unknown ffn_kind %d", ffn_kind);
  CUDA_TRY(ctx, cudaSetDevice(ctx->cfg.device));
  return run_experts(ctx, layer, x, T, ids, scores, scores_dtype, expert_slot, order, residual, out, ffn_kind,
                     reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int b200moe_forward_fused(b200moe_ctx* ctx, int layer, const void* x, int T, const void* residual, void* out,
                                     int64_t* ids_out, void* scores_out, int ffn_kind, void* stream) {
  int rc = check_layer(ctx, layer, "b200moe_forward_fused");
  if (rc) return rc;
  if ((rc = check_tokens(ctx, T, "b200moe_forward_fused"))) return rc;
  if (T == 0) return B200MOE_OK;
  if (!x || !out) return fail(ctx, B200MOE_E_ARG, "b200moe_forward_fused: null pointer");
  if (misaligned(x) || misaligned(out) || (residual && misaligned(residual)))
    return fail(ctx, B200MOE_E_ARG, "b200moe_forward_fused: x, out and residual must be 16-byte aligned");
  if (!ctx->gate_w[layer]) return fail(ctx, B200MOE_E_STATE, "b200moe_forward_fused: no gate weight registered for layer %d", layer);
  if (ffn_kind < B200MOE_FFN_AUTO || ffn_kind > B200MOE_FFN_MMA) return fail(ctx, B200MOE_E_ARG, "b200moe_forward_fused: unknown ffn_kind %d", ffn_kind);
  CUDA_TRY(ctx, cudaSetDevice(ctx->cfg.device));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int64_t* ids = ids_out ? ids_out : ctx->ids64;
  void* scores = scores_out ? scores_out : ctx->scores;
  return run_experts(ctx, layer, x, T, ids, scores, ctx->cfg.act_dtype, nullptr, nullptr, residual, out, ffn_kind, st, true);
}

extern "C" int b200moe_forward_fused_norm(b200moe_ctx* ctx, int layer, const void* hidden, const void* residual, const void* norm_weight, float eps,
                                          int T, void* out, void* residual_out, void* normed_out, int64_t* ids_out, void* scores_out, int ffn_kind,
                                          void* stream) {
  int rc = check_layer(ctx, layer, "b200moe_forward_fused_norm");
  if (rc) return rc;
  if ((rc = check_tokens(ctx, T, "b200moe_forward_fused_norm"))) return rc;
  if (T == 0) return B200MOE_OK;
  if (!hidden || !norm_weight || !out) return fail(ctx, B200MOE_E_ARG, "b200moe_forward_fused_norm: null pointer");
  if (misaligned(hidden) || misaligned(norm_weight) || misaligned(out) || (residual && misaligned(residual)) || (residual_out && misaligned(residual_out)) ||
      (normed_out && misaligned(normed_out)))
    return fail(ctx, B200MOE_E_ARG, "b200moe_forward_fused_norm: pointers must be 16-byte aligned");
  if (!ctx->gate_w[layer]) return fail(ctx, B200MOE_E_STATE, "b200moe_forward_fused_norm: no gate weight registered for layer %d", layer);
  if (ffn_kind < B200MOE_FFN_AUTO || ffn_kind > B200MOE_FFN_MMA) return fail(ctx, B200MOE_E_ARG, "b200moe_forward_fused_norm: unknown ffn_kind %d", ffn_kind);
  CUDA_TRY(ctx, cudaSetDevice(ctx->cfg.device));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  RouterNorm nm;
  nm.residual = residual; nm.weight = norm_weight; nm.eps = eps;
  nm.normed_out = normed_out ? normed_out : ctx->xnorm;
  nm.res_out = residual_out ? residual_out : ctx->xres;       // without an incoming residual this is a copy of `hidden`, the residual the block adds
  int64_t* ids = ids_out ? ids_out : ctx->ids64;
  void* scores = scores_out ? scores_out : ctx->scores;
  return run_experts(ctx, layer, nm.normed_out, T, ids, scores, ctx->cfg.act_dtype, nullptr, nullptr, nm.res_out, out, ffn_kind, st, true, hidden, &nm);
}

// ------------------------------------------------------------------------------------------
// expert parallelism: peer-store dispatch / return (ep.cuh)
// ------------------------------------------------------------------------------------------
static size_t ep_align(size_t v) { return (v + 255) & ~(size_t)255; }

extern "C" int b200moe_ep_create(b200moe_ctx* ctx, int world, int rank, int max_local_tokens, void* handle_out) {
  if (!ctx) return fail(nullptr, B200MOE_E_ARG, "b200moe_ep_create: null context");
  const b200moe_config& c = ctx->cfg;
  if (ctx->ep.base) return fail(ctx, B200MOE_E_STATE, "b200moe_ep_create: this context already has an exchange buffer");
  if (world < 1 || world > kEpMaxRanks) return fail(ctx, B200MOE_E_UNSUPPORTED, "b200moe_ep_create: world=%d (1..%d ranks)", world, kEpMaxRanks);
  if (rank < 0 || rank >= world) return fail(ctx, B200MOE_E_ARG, "b200moe_ep_create: rank %d out of range [0,%d)", rank, world);
  if (c.num_experts % world) return fail(ctx, B200MOE_E_ARG, "b200moe_ep_create: num_experts=%d is not divisible by world=%d", c.num_experts, world);
  if (max_local_tokens < 1) return fail(ctx, B200MOE_E_ARG, "b200moe_ep_create: max_local_tokens must be positive");
  if ((long long)world * max_local_tokens > c.max_tokens)
    return fail(ctx, B200MOE_E_STATE, "b200moe_ep_create: world*max_local_tokens=%d exceeds the context's max_tokens=%d (the workspace holds every rank's pairs)",
                world * max_local_tokens, c.max_tokens);
  CUDA_TRY(ctx, cudaSetDevice(c.device));
  b200moe_ctx::Ep& ep = ctx->ep;
  const size_t eb = elem_bytes(c.act_dtype);
  const int cap = max_local_tokens * c.top_k;
  EpGeom g{};
  g.G = world; g.me = rank; g.cap = cap; g.H = c.hidden_size; g.K = c.top_k; g.epr = c.num_experts / world;
  g.off_meta = kEpHeaderBytes;
  g.off_x = ep_align(g.off_meta + (size_t)world * cap * sizeof(int2));
  g.off_ret = ep_align(g.off_x + (size_t)world * cap * c.hidden_size * eb);
  const size_t bytes = ep_align(g.off_ret + (size_t)cap * c.hidden_size * eb);
  void* base = nullptr;
  cudaError_t e = cudaMalloc(&base, bytes);
  if (e != cudaSuccess) return fail(ctx, B200MOE_E_CUDA, "b200moe_ep_create: cudaMalloc(%zu bytes) failed: %s", bytes, cudaGetErrorString(e));
  ctx->allocs.push_back(base);
  int rc = dev_alloc(ctx, &ep.counters, 16);
  if (rc) return rc;
  CUDA_TRY(ctx, cudaMemset(base, 0, bytes));
  CUDA_TRY(ctx, cudaMemset(ep.counters, 0, 16 * sizeof(unsigned)));
  CUDA_TRY(ctx, cudaDeviceSynchronize());
  if (handle_out) {
    cudaIpcMemHandle_t h;
    static_assert(sizeof(cudaIpcMemHandle_t) == B200MOE_EP_HANDLE_BYTES, "handle size");
    e = cudaIpcGetMemHandle(&h, base);
    if (e != cudaSuccess) return fail(ctx, B200MOE_E_CUDA, "b200moe_ep_create: cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e));
    memcpy(handle_out, &h, sizeof h);
  }
  ep.world = world; ep.rank = rank; ep.max_local = max_local_tokens; ep.geom = g;
  ep.base = reinterpret_cast<unsigned char*>(base); ep.bytes = bytes;
  for (int r = 0; r < kEpMaxRanks; ++r) ep.peers.base[r] = nullptr;
  ep.peers.base[rank] = ep.base;
  ep.attached = world == 1;
  return B200MOE_OK;
}

extern "C" int b200moe_ep_attach_ipc(b200moe_ctx* ctx, const void* handles_all) {
  if (!ctx || !handles_all) return fail(ctx, B200MOE_E_ARG, "b200moe_ep_attach_ipc: null argument");
  b200moe_ctx::Ep& ep = ctx->ep;
  if (!ep.base) return fail(ctx, B200MOE_E_STATE, "b200moe_ep_attach_ipc: call b200moe_ep_create first");
  if (ep.attached && ep.world > 1) return fail(ctx, B200MOE_E_STATE, "b200moe_ep_attach_ipc: already attached");
  CUDA_TRY(ctx, cudaSetDevice(ctx->cfg.device));
  const unsigned char* hb = reinterpret_cast<const unsigned char*>(handles_all);
  for (int r = 0; r < ep.world; ++r) {
    if (r == ep.rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, hb + (size_t)r * B200MOE_EP_HANDLE_BYTES, sizeof h);
    void* ptr = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return fail(ctx, B200MOE_E_CUDA, "b200moe_ep_attach_ipc: cudaIpcOpenMemHandle for rank %d failed: %s", r, cudaGetErrorString(e));
    ep.opened.push_back(ptr);
    ep.peers.base[r] = reinterpret_cast<unsigned char*>(ptr);
  }
  ep.attached = true;
  return B200MOE_OK;
}

extern "C" int b200moe_ep_attach_local(b200moe_ctx* ctx, b200moe_ctx* const* ranks) {
  if (!ctx || !ranks) return fail(ctx, B200MOE_E_ARG, "b200moe_ep_attach_local: null argument");
  b200moe_ctx::Ep& ep = ctx->ep;
  if (!ep.base) return fail(ctx, B200MOE_E_STATE, "b200moe_ep_attach_local: call b200moe_ep_create first");
  CUDA_TRY(ctx, cudaSetDevice(ctx->cfg.device));
  for (int r = 0; r < ep.world; ++r) {
    if (r == ep.rank) continue;
    const b200moe_ctx* o = ranks[r];
    if (!o || !o->ep.base) return fail(ctx, B200MOE_E_STATE, "b200moe_ep_attach_local: rank %d has no exchange buffer", r);
    if (o->ep.world != ep.world || o->ep.rank != r || o->ep.bytes != ep.bytes)
      return fail(ctx, B200MOE_E_ARG, "b200moe_ep_attach_local: rank %d was created with a different geometry", r);
    if (o->cfg.device != ctx->cfg.device) {
      cudaError_t e = cudaDeviceEnablePeerAccess(o->cfg.device, 0);
      if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); e = cudaSuccess; }
      if (e != cudaSuccess) return fail(ctx, B200MOE_E_CUDA, "b200moe_ep_attach_local: no peer access from device %d to %d: %s", ctx->cfg.device, o->cfg.device, cudaGetErrorString(e));
    }
    ep.peers.base[r] = o->ep.base;
  }
  ep.attached = true;
  return B200MOE_OK;
}

extern "C" int b200moe_ep_set_wait_ms(b200moe_ctx* ctx, int milliseconds) {
  if (!ctx) return fail(nullptr, B200MOE_E_ARG, "b200moe_ep_set_wait_ms: null context");
  if (milliseconds < 1 || milliseconds > 2000) return fail(ctx, B200MOE_E_ARG, "b200moe_ep_set_wait_ms: 1..2000 ms");
  int khz = 0;
  if (cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, ctx->cfg.device) != cudaSuccess || khz <= 0) khz = 1965000;
  ctx->ep.wait_cycles = (long long)khz * milliseconds;
  return B200MOE_OK;
}

extern "C" int b200moe_ep_detach(b200moe_ctx* ctx) {
  if (!ctx) return fail(nullptr, B200MOE_E_ARG, "b200moe_ep_detach: null context");
  cudaSetDevice(ctx->cfg.device);
  for (void* p : ctx->ep.opened) cudaIpcCloseMemHandle(p);
  ctx->ep.opened.clear();
  for (int r = 0; r < kEpMaxRanks; ++r)
    if (r != ctx->ep.rank) ctx->ep.peers.base[r] = nullptr;
  ctx->ep.attached = ctx->ep.world == 1;
  return B200MOE_OK;
}

static int ep_ready(b200moe_ctx* ctx, const char* who) {
  if (!ctx) return fail(nullptr, B200MOE_E_ARG, "%s: null context", who);
  if (!ctx->ep.base) return fail(ctx, B200MOE_E_STATE, "%s: no exchange buffer (b200moe_ep_create)", who);
  if (!ctx->ep.attached) return fail(ctx, B200MOE_E_STATE, "%s: peers not attached (b200moe_ep_attach_ipc / _local)", who);
  return B200MOE_OK;
}

// phase 1: route this rank's tokens, then store every (token, expert) pair's row into its owner's receive buffer
extern "C" int b200moe_ep_dispatch(b200moe_ctx* ctx, int layer, const void* x_local, int T_local, void* stream) {
  int rc = ep_ready(ctx, "b200moe_ep_dispatch");
  if (rc) return rc;
  if ((rc = check_layer(ctx, layer, "b200moe_ep_dispatch"))) return rc;
  b200moe_ctx::Ep& ep = ctx->ep;
  const b200moe_config& c = ctx->cfg;
  if (T_local < 0 || T_local > ep.max_local) return fail(ctx, B200MOE_E_STATE, "b200moe_ep_dispatch: T_local=%d outside [0, max_local_tokens=%d]", T_local, ep.max_local);
  if (T_local > 0 && (!x_local || misaligned(x_local))) return fail(ctx, B200MOE_E_ARG, "b200moe_ep_dispatch: x_local must be a 16-byte aligned device pointer");
  if (!ctx->gate_w[layer]) return fail(ctx, B200MOE_E_STATE, "b200moe_ep_dispatch: no gate weight registered for layer %d", layer);
  CUDA_TRY(ctx, cudaSetDevice(c.device));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  ep.last_T_local = T_local;
  if (T_local > 0)       // router + dispatch in one launch: each routed tile's rows leave from the router's tail
    return launch_router(ctx, layer, x_local, nullptr, T_local, ctx->ids64, ctx->scores, nullptr, st, nullptr, nullptr, nullptr, true);
  // no tokens on this rank: it still has to tell every peer so
  EpDispatchParams dp{};
  dp.x = x_local; dp.ids = ctx->ids64; dp.T_local = 0; dp.E = c.num_experts; dp.g = ep.geom;
  dp.epoch = ep.counters; dp.done = ep.counters + 1; dp.dest_count = reinterpret_cast<int*>(ep.counters + 8); dp.status = ctx->status;
  return dispatch_dtype(ctx, c.act_dtype, [&](auto tag) {
    using Tt = decltype(tag);
    ProfScope prof(ctx, B200MOE_KERNEL_EP_DISPATCH, st);
    launch_chain(ep_dispatch_kernel<Tt>, dim3(1), dim3(kEpThreads), 0, st, dp, ep.peers);
    return post_launch(ctx, "ep_dispatch_kernel");
  });
}

// phase 2: wait for every source's rows, group them by expert, run the local experts, store every output row into its source's return buffer
extern "C" int b200moe_ep_experts(b200moe_ctx* ctx, int layer, int ffn_kind, void* stream) {
  int rc = ep_ready(ctx, "b200moe_ep_experts");
  if (rc) return rc;
  if ((rc = check_layer(ctx, layer, "b200moe_ep_experts"))) return rc;
  if (ffn_kind < B200MOE_FFN_AUTO || ffn_kind > B200MOE_FFN_MMA) return fail(ctx, B200MOE_E_ARG, "b200moe_ep_experts: unknown ffn_kind %d", ffn_kind);
  b200moe_ctx::Ep& ep = ctx->ep;
  const b200moe_config& c = ctx->cfg;
  const int E = c.num_experts;
  CUDA_TRY(ctx, cudaSetDevice(c.device));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  SlotTable tab;
  for (int e = 0; e < kMaxExperts; ++e) { tab.slot[e] = -1; tab.rank[e] = (uint8_t)(e & 255); }
  for (int e = 0; e < E; ++e) tab.slot[e] = (int16_t)(ctx->registered[(size_t)layer * E + e] ? e : -1);
  if ((rc = upload_layer_table(ctx, layer, st))) return rc;
  const EpGeom& g = ep.geom;
  const int rows = g.G * g.cap;                      // every row of the receive buffer is a "pair" with K = 1
  const EpHeader* hdr = reinterpret_cast<const EpHeader*>(ep.base);
  PermuteParams pp{};
  pp.ids64 = nullptr; pp.T = rows; pp.K = 1; pp.E = E;
  pp.offsets = ctx->offsets; pp.sorted_pair = ctx->sorted_pair; pp.inv = ctx->inv;
  pp.act_list = ctx->act_list; pp.n_act = ctx->n_act; pp.status = ctx->status;
  pp.ep_meta = reinterpret_cast<const int2*>(ep.base + g.off_meta);
  pp.ep_count = hdr->disp_count; pp.ep_flags = hdr->disp_flag; pp.ep_epoch = ep.counters;
  pp.ep_G = g.G; pp.ep_cap = g.cap; pp.ep_wait_cycles = ep.wait_cycles;
  // the CTA is sized for the rows this rank can expect (about T_local*K when the routing is balanced), not for
  // the capacity of its receive buffer: fewer warps mean shorter scans; any number of rows is still handled
  const int expect_rows = (int)std::min<long long>(rows, 2LL * std::max(1, ep.last_T_local) * c.top_k + 64);
  const int pthreads = std::min(kPermuteMaxThreads, std::max(256, (expect_rows + 31) / 32 * 32));
  const size_t smem = (size_t)((pthreads / 32) * E + E) * sizeof(int);
  {
    ProfScope prof(ctx, B200MOE_KERNEL_PERMUTE, st);
    launch_chain(permute_kernel, dim3(1), dim3(pthreads), smem, st, pp, tab);
  }
  if ((rc = post_launch(ctx, "permute_kernel"))) return rc;

  FfnLaunch f{};
  f.experts = ctx->d_experts + (size_t)layer * E;
  f.offsets = ctx->offsets; f.sorted_pair = ctx->sorted_pair; f.act_list = ctx->act_list; f.n_act = ctx->n_act;
  f.x = ep.base + g.off_x; f.h = ctx->h; f.y = ctx->y; f.K = 1;
  {
    // same token-tile rule as on one GPU, from the whole batch (all ranks' tokens), so that the same
    // kernel instance - and with it the same summation order - serves an expert wherever it lives
    const long long T_all = (long long)g.G * std::max(1, ep.last_T_local);
    const long long n_mean = (T_all * c.top_k + E - 1) / E;
    f.max_n = (int)std::min<long long>(T_all, std::max<long long>(16, 4 * n_mean));
  }
  f.n_tokens = rows;
  f.n_act_bound = std::min(g.epr, rows);
  f.ksplit_ok = false;                               // the return kernel ships y rows in the model dtype
  ctx->last_ksplit = 1;
#ifdef B200MOE_WITH_UMMA
  if (!ctx->h_tmaps.empty()) {
    bool all_ok = true;
    for (int e = 0; e < E; ++e)
      if (tab.slot[e] >= 0 && !ctx->tmap_ok[(size_t)layer * E + tab.slot[e]]) all_ok = false;
    if (all_ok) f.tmaps = ctx->d_tmaps + (size_t)layer * E * 3;
    if (all_ok && ctx->d_tmaps2) f.tmaps2 = ctx->d_tmaps2 + (size_t)layer * E * 3;
  }
#endif
  if ((rc = launch_ffn(ctx, f, tab, ffn_kind, st))) return rc;

  EpReturnParams rp{};
  rp.y = ctx->y; rp.offsets = ctx->offsets; rp.sorted_pair = ctx->sorted_pair; rp.E = E; rp.g = g;
  rp.epoch = ep.counters; rp.done = ep.counters + 2; rp.status = ctx->status;
  // rows actually received are about T_all*K/G; CTAs beyond them leave after one load
  const int expect = (int)std::min<long long>(rows, 2LL * std::max(1, ep.last_T_local) * c.top_k + 64);
  const int grid = std::max(1, std::min((expect + kEpRowsPerTrip - 1) / kEpRowsPerTrip, 4 * ctx->sm_count));
  return dispatch_dtype(ctx, c.act_dtype, [&](auto tag) {
    using Tt = decltype(tag);
    ProfScope prof(ctx, B200MOE_KERNEL_EP_RETURN, st);
    launch_chain(ep_return_kernel<Tt>, dim3(grid), dim3(kEpThreads), 0, st, rp, ep.peers, tab);
    return post_launch(ctx, "ep_return_kernel");
  });
}

// phase 3: wait for every owner's rows, then the weighted accumulation of this rank's own tokens
extern "C" int b200moe_ep_combine(b200moe_ctx* ctx, int T_local, const int32_t* order, const void* residual, void* out, void* stream) {
  int rc = ep_ready(ctx, "b200moe_ep_combine");
  if (rc) return rc;
  b200moe_ctx::Ep& ep = ctx->ep;
  const b200moe_config& c = ctx->cfg;
  if (T_local != ep.last_T_local) return fail(ctx, B200MOE_E_STATE, "b200moe_ep_combine: T_local=%d but the matching dispatch had %d tokens", T_local, ep.last_T_local);
  if (T_local == 0) return B200MOE_OK;
  if (!out || misaligned(out) || (residual && misaligned(residual))) return fail(ctx, B200MOE_E_ARG, "b200moe_ep_combine: out and residual must be 16-byte aligned device pointers");
  CUDA_TRY(ctx, cudaSetDevice(c.device));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  SlotTable tab;
  for (int e = 0; e < kMaxExperts; ++e) { tab.slot[e] = (int16_t)(e < c.num_experts ? e : -1); tab.rank[e] = (uint8_t)(e & 255); }
  if (order)
    for (int e = 0; e < c.num_experts; ++e) {
      if (order[e] < 0 || order[e] > 255) return fail(ctx, B200MOE_E_ARG, "order[%d]=%d out of range [0,255]", e, order[e]);
      tab.rank[e] = (uint8_t)order[e];
    }
  const EpHeader* hdr = reinterpret_cast<const EpHeader*>(ep.base);
  CombineParams cp{};
  cp.y = ep.base + ep.geom.off_ret; cp.inv = ctx->one_sorted;   // identity: pair p lives in row p of the return buffer
  cp.ids64 = ctx->ids64; cp.scores = ctx->scores; cp.scores_f32 = 0;
  cp.residual = residual; cp.out = out; cp.T = T_local; cp.H = c.hidden_size; cp.K = c.top_k; cp.E = c.num_experts;
  cp.wait_flags = hdr->ret_flag; cp.epoch = ep.counters; cp.n_wait = ep.geom.G; cp.wait_cycles = ep.wait_cycles; cp.status = ctx->status;
  return dispatch_dtype(ctx, c.act_dtype, [&](auto tag) {
    using Tt = decltype(tag);
    ProfScope prof(ctx, B200MOE_KERNEL_COMBINE, st);
    launch_chain(combine_kernel<Tt>, dim3(T_local), dim3(kCombineThreads), 0, st, cp, tab);
    return post_launch(ctx, "combine_kernel");
  });
}

extern "C" int b200moe_ep_forward(b200moe_ctx* ctx, int layer, const void* x_local, int T_local, const int32_t* order, const void* residual,
                                  void* out, int ffn_kind, void* stream) {
  int rc = b200moe_ep_dispatch(ctx, layer, x_local, T_local, stream);
  if (rc) return rc;
  if ((rc = b200moe_ep_experts(ctx, layer, ffn_kind, stream))) return rc;
  return b200moe_ep_combine(ctx, T_local, order, residual, out, stream);
}

extern "C" int b200moe_ep_last_routing(b200moe_ctx* ctx, int T_local, int64_t* ids_out, void* scores_out, void* stream) {
  int rc = ep_ready(ctx, "b200moe_ep_last_routing");
  if (rc) return rc;
  if (T_local < 0 || T_local > ctx->ep.max_local) return fail(ctx, B200MOE_E_ARG, "b200moe_ep_last_routing: T_local out of range");
  CUDA_TRY(ctx, cudaSetDevice(ctx->cfg.device));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const size_t n = (size_t)T_local * ctx->cfg.top_k;
  if (ids_out && n) CUDA_TRY(ctx, cudaMemcpyAsync(ids_out, ctx->ids64, n * sizeof(int64_t), cudaMemcpyDefault, st));
  if (scores_out && n) CUDA_TRY(ctx, cudaMemcpyAsync(scores_out, ctx->scores, n * elem_bytes(ctx->cfg.act_dtype), cudaMemcpyDefault, st));
  return B200MOE_OK;
}

extern "C" int b200moe_rmsnorm(b200moe_ctx* ctx, const void* x, const void* residual_or_null, const void* weight, float eps, int T,
                               void* out, void* residual_out_or_null, void* stream) {
  if (!ctx) return fail(nullptr, B200MOE_E_ARG, "b200moe_rmsnorm: null context");
  const b200moe_config& c = ctx->cfg;
  if (T < 0) return fail(ctx, B200MOE_E_ARG, "b200moe_rmsnorm: negative row count");
  if (T == 0) return B200MOE_OK;
  if (!x || !weight || !out) return fail(ctx, B200MOE_E_ARG, "b200moe_rmsnorm: null pointer");
  if (misaligned(x) || misaligned(weight) || misaligned(out) || (residual_or_null && misaligned(residual_or_null)) ||
      (residual_out_or_null && misaligned(residual_out_or_null)))
    return fail(ctx, B200MOE_E_ARG, "b200moe_rmsnorm: pointers must be 16-byte aligned");
  if (c.hidden_size % 8 || c.hidden_size > kNormThreads * kNormMaxChunks * 8)
    return fail(ctx, B200MOE_E_UNSUPPORTED, "b200moe_rmsnorm: hidden size %d (multiples of 8 up to %d)", c.hidden_size, kNormThreads * kNormMaxChunks * 8);
  CUDA_TRY(ctx, cudaSetDevice(c.device));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  NormParams p{};
  p.x = x; p.residual = residual_or_null; p.weight = weight; p.out = out;
  p.residual_out = residual_or_null ? residual_out_or_null : nullptr;
  p.eps = eps; p.T = T; p.H = c.hidden_size;
  return dispatch_dtype(ctx, c.act_dtype, [&](auto tag) {
    using Tt = decltype(tag);
    launch_chain(rmsnorm_kernel<Tt>, dim3(T), dim3(kNormThreads), 0, st, p);
    return post_launch(ctx, "rmsnorm_kernel");
  });
}

extern "C" int b200moe_expert_ffn(b200moe_ctx* ctx, const void* x, int n, const void* gate_proj, const void* up_proj,
                                  const void* down_proj, void* out, void* stream) {
  if (!ctx) return fail(nullptr, B200MOE_E_ARG, "b200moe_expert_ffn: null context");
  const b200moe_config& c = ctx->cfg;
  if (c.weight_mode != B200MOE_W_DENSE) return fail(ctx, B200MOE_E_UNSUPPORTED, "b200moe_expert_ffn: dense weights only");
  if (n < 0) return fail(ctx, B200MOE_E_ARG, "b200moe_expert_ffn: negative row count");
  if ((size_t)n > (size_t)c.max_tokens * c.top_k) return fail(ctx, B200MOE_E_STATE, "b200moe_expert_ffn: n=%d exceeds max_tokens*top_k=%d", n, c.max_tokens * c.top_k);
  if (n == 0) return B200MOE_OK;
  if (!x || !gate_proj || !up_proj || !down_proj || !out) return fail(ctx, B200MOE_E_ARG, "b200moe_expert_ffn: null pointer");
  if (misaligned(x) || misaligned(gate_proj) || misaligned(up_proj) || misaligned(down_proj) || misaligned(out))
    return fail(ctx, B200MOE_E_ARG, "b200moe_expert_ffn: pointers must be 16-byte aligned");
  CUDA_TRY(ctx, cudaSetDevice(c.device));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  ExpertPtrs ep{};
  ep.w[0] = gate_proj; ep.w[1] = up_proj; ep.w[2] = down_proj;
  ExpertPtrs* slot = ctx->d_experts + (size_t)c.num_layers * c.num_experts;
  const int offs[2] = {0, n};
  CUDA_TRY(ctx, cudaMemcpyAsync(slot, &ep, sizeof ep, cudaMemcpyHostToDevice, st));
  CUDA_TRY(ctx, cudaMemcpyAsync(ctx->one_offsets, offs, sizeof offs, cudaMemcpyHostToDevice, st));
  SlotTable tab;
  for (int e = 0; e < kMaxExperts; ++e) { tab.slot[e] = -1; tab.rank[e] = 0; }
  tab.slot[0] = 0;
  FfnLaunch f{};
  f.experts = slot; f.offsets = ctx->one_offsets; f.sorted_pair = ctx->one_sorted; f.act_list = ctx->one_act; f.n_act = ctx->one_nact;
  f.x = x; f.h = ctx->h; f.y = out; f.K = 1; f.max_n = n;
#ifdef B200MOE_WITH_UMMA
  if (!ctx->h_tmaps.empty() && n > 1) {
    const size_t idx = (size_t)c.num_layers * c.num_experts;
    if (encode_expert_maps(ctx, &ctx->h_tmaps[idx * 3], gate_proj, up_proj, down_proj)) {
      CUDA_TRY(ctx, cudaMemcpyAsync(ctx->d_tmaps + idx * 3, &ctx->h_tmaps[idx * 3], 3 * sizeof(CUtensorMap), cudaMemcpyHostToDevice, st));
      f.tmaps = ctx->d_tmaps + idx * 3;
    }
  }
#endif
  return launch_ffn(ctx, f, tab, B200MOE_FFN_AUTO, st);
}

// ------------------------------------------------------------------------------------------
// int4 pack / unpack, status
// ------------------------------------------------------------------------------------------
extern "C" int b200moe_pack_int4(const void* w, int out_features, int in_features, int dtype, void* q, void* scales, void* stream) {
  if (!w || !q || !scales) return fail(nullptr, B200MOE_E_ARG, "b200moe_pack_int4: null pointer");
  if (out_features <= 0 || in_features <= 0 || in_features % 128) return fail(nullptr, B200MOE_E_ARG, "b200moe_pack_int4: in_features must be a positive multiple of 128");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const long long warps = (long long)out_features * (in_features / 128);
  const long long blocks = (warps * 32 + 255) / 256;
  if (blocks > 0x7fffffffLL) return fail(nullptr, B200MOE_E_ARG, "b200moe_pack_int4: matrix too large");
  return dispatch_dtype(nullptr, dtype, [&](auto tag) {
    using T = decltype(tag);
    pack_int4_kernel<T><<<(unsigned)blocks, 256, 0, st>>>(reinterpret_cast<const T*>(w), out_features, in_features,
                                                           reinterpret_cast<uint8_t*>(q), reinterpret_cast<__nv_bfloat16*>(scales));
    return post_launch(nullptr, "pack_int4_kernel");
  });
}

extern "C" int b200moe_unpack_int4(const void* q, const void* scales, int out_features, int in_features, int dtype,
                                   void* q_out, void* w_out, void* stream) {
  if (!q || (!q_out && !w_out)) return fail(nullptr, B200MOE_E_ARG, "b200moe_unpack_int4: null pointer");
  if (w_out && !scales) return fail(nullptr, B200MOE_E_ARG, "b200moe_unpack_int4: scales needed to dequantise");
  if (out_features <= 0 || in_features <= 0 || in_features % 128) return fail(nullptr, B200MOE_E_ARG, "b200moe_unpack_int4: in_features must be a positive multiple of 128");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const long long nbytes = (long long)out_features * (in_features / 2);
  const long long blocks = (nbytes + 255) / 256;
  if (blocks > 0x7fffffffLL) return fail(nullptr, B200MOE_E_ARG, "b200moe_unpack_int4: matrix too large");
  return dispatch_dtype(nullptr, dtype, [&](auto tag) {
    using T = decltype(tag);
    unpack_int4_kernel<T><<<(unsigned)blocks, 256, 0, st>>>(reinterpret_cast<const uint8_t*>(q), reinterpret_cast<const __nv_bfloat16*>(scales),
                                                             out_features, in_features, reinterpret_cast<int8_t*>(q_out), reinterpret_cast<T*>(w_out));
    return post_launch(nullptr, "unpack_int4_kernel");
  });
}

extern "C" int b200moe_profile(b200moe_ctx* ctx, int enable) {
  if (!ctx) return fail(nullptr, B200MOE_E_ARG, "b200moe_profile: null context");
  ctx->profiling = enable != 0;
  return B200MOE_OK;
}

extern "C" int b200moe_profile_read(b200moe_ctx* ctx, float* total_ms, int32_t* launches) {
  if (!ctx || !total_ms || !launches) return fail(ctx, B200MOE_E_ARG, "b200moe_profile_read: null argument");
  for (int i = 0; i < B200MOE_KERNEL_CLASSES; ++i) { total_ms[i] = 0.0f; launches[i] = 0; }
  int rc = B200MOE_OK;
  for (auto& r : ctx->prof) {
    float ms = 0.0f;
    cudaError_t e = cudaEventSynchronize(r.b);
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, r.a, r.b);
    if (e != cudaSuccess) rc = fail(ctx, B200MOE_E_CUDA, "b200moe_profile_read: %s", cudaGetErrorString(e));
    else if (r.cls >= 0 && r.cls < B200MOE_KERNEL_CLASSES) { total_ms[r.cls] += ms; launches[r.cls]++; }
    cudaEventDestroy(r.a);
    cudaEventDestroy(r.b);
  }
  ctx->prof.clear();
  return rc;
}

extern "C" int b200moe_set_token_kernel(b200moe_ctx* ctx, int enable) {
  if (!ctx) return fail(nullptr, B200MOE_E_ARG, "b200moe_set_token_kernel: null context");
  ctx->token_kernel = enable != 0;
  return B200MOE_OK;
}

extern "C" int b200moe_status(b200moe_ctx* ctx, int* device_status_out, void* stream) {
  if (!ctx || !device_status_out) return fail(ctx, B200MOE_E_ARG, "b200moe_status: null argument");
  CUDA_TRY(ctx, cudaSetDevice(ctx->cfg.device));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int v = 0;
  CUDA_TRY(ctx, cudaMemcpyAsync(&v, ctx->status, sizeof v, cudaMemcpyDeviceToHost, st));
  CUDA_TRY(ctx, cudaMemsetAsync(ctx->status, 0, sizeof v, st));
  CUDA_TRY(ctx, cudaStreamSynchronize(st));
  if (v & B200MOE_DEV_WAIT_EXPIRED)   // a grid barrier that gave up leaves its word between two states
    CUDA_TRY(ctx, cudaMemsetAsync(ctx->tile_counter + ctx->cfg.max_tokens + 1, 0, sizeof(unsigned), st));
  *device_status_out = v;
  if (v) return fail(ctx, B200MOE_E_DEVICE, "device status word = %d", v);
  return B200MOE_OK;
}
