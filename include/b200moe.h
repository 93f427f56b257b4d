/*
 * b200moe.h - C ABI of libb200moe.so: the MoE block forward of on_device_sd's demo engine
 * (router -> token-to-expert permute -> grouped SwiGLU expert FFN -> weighted combine),
 * written for NVIDIA B200 (sm_100a) only.
 *
 * Conventions
 *   - Every function returns an int status: 0 = B200MOE_OK, otherwise one of the B200MOE_E_*
 *     codes; b200moe_last_error() then returns a message.  Nothing throws, traps or waits
 *     without a bound.  There is no CPU fallback: without a usable CUDA device every compute
 *     entry point fails with B200MOE_E_CUDA.
 *   - All data pointers are DEVICE pointers unless the comment says "host".  Matrices are
 *     row-major [out_features, in_features], one allocation per matrix, as the reference's
 *     ParameterLoader hands them out (demo/src/memory/parameter_loader.py:478-497).
 *   - Pointers registered with set_gate / set_expert are BORROWED: the caller keeps them alive
 *     until clear_expert / destroy, or re-registers after moving them (the reference's
 *     ExpertCache may evict between calls, demo/src/memory/expert_cache.py:125-139).
 *   - Work is enqueued on the cudaStream_t passed as `stream` (a void* here so that the header
 *     needs no CUDA include) and is asynchronous unless stated.
 *   - A context is bound to one device and is not re-entrant: one thread drives it, the same
 *     rule as the engine's single GPU thread (demo/src/api/inference.py:340-369).
 */
#ifndef B200MOE_H_
#define B200MOE_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200MOE_OK 0
#define B200MOE_E_ARG 1      /* bad argument (null pointer, shape, alignment, unknown enum)   */
#define B200MOE_E_CUDA 2     /* a CUDA runtime call failed, or no CUDA device                  */
#define B200MOE_E_STATE 3    /* call order: gate / expert not registered, context too small    */
#define B200MOE_E_DEVICE 4   /* a kernel's own bounds check or bounded wait reported a problem */
#define B200MOE_E_UNSUPPORTED 5

/* activation / dense-weight element types (MoEConfig.get_dtype, demo/src/core/model.py:122-129) */
#define B200MOE_F32 0
#define B200MOE_F16 1
#define B200MOE_BF16 2

/* expert weight storage */
#define B200MOE_W_DENSE 0      /* same element type as the activations                         */
#define B200MOE_W_INT4_G128 1  /* symmetric int4, groups of 128 along `in`, bf16 scales        */

/* which expert-FFN kernel family b200moe_forward may pick */
#define B200MOE_FFN_AUTO 0
#define B200MOE_FFN_GEMV 1     /* CUDA-core weight-streaming kernels (any dtype, any count)     */
#define B200MOE_FFN_MMA 2      /* tensor-core kernels (bf16 activations)                        */

#define B200MOE_MAX_EXPERTS 256
#define B200MOE_MAX_TOPK 32

typedef struct b200moe_ctx b200moe_ctx;

/* The five numbers of MoEConfig the path consumes (demo/src/core/model.py:33-45) plus storage. */
typedef struct b200moe_config {
  int32_t hidden_size;        /* H, multiple of 8 (128 for int4 weights)                       */
  int32_t num_experts;        /* E <= B200MOE_MAX_EXPERTS                                      */
  int32_t top_k;              /* K <= min(E, B200MOE_MAX_TOPK)                                 */
  int32_t intermediate_size;  /* I (moe_intermediate_size), multiple of 8 (128 for int4)       */
  int32_t act_dtype;          /* B200MOE_F32 / F16 / BF16                                      */
  int32_t weight_mode;        /* B200MOE_W_DENSE / B200MOE_W_INT4_G128 (needs BF16)            */
  int32_t num_layers;         /* layers whose gate / experts can be registered                 */
  int32_t max_tokens;         /* largest T of any call; sizes the workspace                    */
  int32_t device;             /* CUDA device ordinal                                           */
  int32_t reserved;
} b200moe_config;

/* Library ABI version; bumped on any incompatible change of this header. */
int b200moe_abi_version(void);

/* Message for the last non-zero status returned on this context (ctx may be NULL: the last
 * error of b200moe_create or of a context-free function in the calling thread). */
const char* b200moe_last_error(const b200moe_ctx* ctx);

/* Allocates the context and its workspace on cfg->device (synchronous).  Replaces the
 * per-call temporaries of Qwen3ModelRunner._execute_moe_with_placement
 * (demo/src/model/qwen3_runner.py:295-314). */
int b200moe_create(const b200moe_config* cfg, b200moe_ctx** out);
int b200moe_destroy(b200moe_ctx* ctx);

/* Registers the router weight Wg [E, H] of `layer` (nn.Linear.weight of Qwen3MoEGate,
 * demo/src/layers/moe_layer.py:20-23, loaded by load_weights :62-65) and an optional logit
 * bias [E] in the activation dtype (NULL in the reference; used by the popularity-skew
 * stress configuration).  Host-side bookkeeping only; `stream` is unused. */
int b200moe_set_gate(b200moe_ctx* ctx, int layer, const void* gate_weight, const void* bias_or_null,
                     void* stream);

/* Registers expert `expert` of `layer`: gate_proj [I,H], up_proj [I,H], down_proj [H,I]
 * (the dict handed over in ExpertPlacement.gpu_expert_params,
 * demo/src/core/model_runner.py:30-43).  Dense mode: the three *_scales are NULL.  Int4 mode:
 * the matrices are uint8 [out, in/2] (element 2j in the low nibble of byte j, 2j+1 in the high
 * nibble, each stored as q+8) and the scales are bf16 [out, in/128].  Host-side bookkeeping
 * only; the device table is refreshed by the next forward call. */
int b200moe_set_expert(b200moe_ctx* ctx, int layer, int expert, const void* gate_proj, const void* up_proj,
                       const void* down_proj, const void* gate_scales, const void* up_scales,
                       const void* down_scales);
int b200moe_clear_expert(b200moe_ctx* ctx, int layer, int expert);

/* Router: Qwen3MoEGate.forward (demo/src/layers/moe_layer.py:25-60) as called by
 * Qwen3ModelRunner.route_experts (demo/src/model/qwen3_runner.py:86-119).
 *   x [T,H] activations; ids_out int64 [T,K]; scores_out [T,K] in the activation dtype;
 *   active_bitmap_out: NULL, or 4 uint64 words (device, or pinned host) receiving one bit per
 *   expert that at least one token selected (the content of RoutingResult.activated_expert_ids).
 * Logits are the correctly rounded dot products (see b200moe_route_from_logits for callers
 * that want a particular GEMM's roundings); top-k order and tie order are those of torch.topk
 * on CUDA; scores are softmax over the k kept logits. */
int b200moe_route(b200moe_ctx* ctx, int layer, const void* x, int T, int64_t* ids_out, void* scores_out,
                  uint64_t* active_bitmap_out, void* stream);

/* Same top-k / softmax stage on logits [T,E] (activation dtype) the caller computed itself,
 * e.g. with the library GEMM the reference uses (moe_layer.py:44).  No counterpart of its own
 * in the reference: it is lines :49-54 of Qwen3MoEGate.forward alone. */
int b200moe_route_from_logits(b200moe_ctx* ctx, const void* logits, int T, int64_t* ids_out, void* scores_out,
                              uint64_t* active_bitmap_out, void* stream);

/* Copies the logits [T,E] of the most recent b200moe_route / b200moe_forward_fused call on this
 * context (after rounding to the activation dtype and adding the bias), widened to fp32, into
 * logits_out (device).  Lets a caller check moe_layer.py:44 separately from the top-k. */
int b200moe_last_logits(b200moe_ctx* ctx, int T, float* logits_out, void* stream);

/* Copies the grouping tables the most recent b200moe_forward / b200moe_forward_fused call on this
 * context built for its T tokens (each destination may be NULL; device or pinned host memory):
 *   offsets [E+1]      exclusive prefix of the per-expert pair counts, offsets[E] = valid pairs
 *   sorted_pair [T*K]  pair index t*K+k at each sorted position: expert e owns positions
 *                      offsets[e] .. offsets[e+1]-1, in row-major (t, k) order - the order in which
 *                      torch.where(topk_indices == e) lists them (demo/src/model/qwen3_runner.py:305-308)
 *   inv [T*K]          sorted position of each pair, -1 for an id outside [0,E)
 *   act_list [E]       experts with work and a usable slot, ascending; n_act [1] = how many
 * Debug / test read; the reference has no such structure (it re-derives the grouping per expert). */
int b200moe_last_tables(b200moe_ctx* ctx, int T, int32_t* offsets_out, int32_t* sorted_pair_out, int32_t* inv_out,
                        int32_t* act_list_out, int32_t* n_act_out, void* stream);

/* K2 alone: groups the (token, slot) pairs of ids [T,K] by expert and copies the result to tables_out
 * (int32, device or pinned host): offsets [E+1] followed by sorted_pair [T*K] as described above; ids
 * outside [0,E) are dropped.  It is the device form of the K x E loop of torch.where calls with which
 * the reference builds LayerExpertActivations (demo/src/execution/model_runner_utils.py:13-41). */
int b200moe_group_pairs(b200moe_ctx* ctx, const int64_t* ids, int T, int32_t* tables_out, void* stream);

/* Expert execution for a given routing: Qwen3ModelRunner._execute_moe_with_placement
 * (demo/src/model/qwen3_runner.py:269-385) plus, with `residual`, forward_moe's add (:226).
 *   x [T,H]; ids int64 [T,K]; scores [T,K] of scores_dtype (activation dtype or B200MOE_F32);
 *   expert_slot: host int32 [E] or NULL.  expert_slot[e] = index of the registered expert whose
 *     weights serve tokens routed to e (e itself normally, a substitute in the draft phase,
 *     :322-329), or -1 to skip e silently (:330-333).  NULL = identity; unregistered experts
 *     are skipped as the reference skips experts missing from the placement.
 *   order: host int32 [E] or NULL.  order[e] = rank of expert e in the sequence in which the
 *     per-expert results are accumulated into the output (the reference accumulates in the
 *     model dtype, so the order is part of the result).  NULL = ascending expert index
 *     (the order of Qwen3MoELayer.forward, demo/src/layers/moe_layer.py:127).
 *   residual: NULL or [T,H]; out [T,H].
 *   ffn_kind: B200MOE_FFN_AUTO or a forced kernel family. */
int b200moe_forward(b200moe_ctx* ctx, int layer, const void* x, int T, const int64_t* ids, const void* scores,
                    int scores_dtype, const int32_t* expert_slot, const int32_t* order, const void* residual,
                    void* out, int ffn_kind, void* stream);

/* Router + expert execution with no host round trip: Qwen3MoELayer.forward
 * (demo/src/layers/moe_layer.py:93-170) in one enqueue.  ids_out / scores_out may be NULL. */
int b200moe_forward_fused(b200moe_ctx* ctx, int layer, const void* x, int T, const void* residual, void* out,
                          int64_t* ids_out, void* scores_out, int ffn_kind, void* stream);

/* The decoder layer's post-attention RMSNorm, the router, the experts, the combine and the residual add
 * in one enqueue: what the reference does with `post_attention_layernorm` at the end of forward_attention
 * (demo/src/model/qwen3_runner.py:204, demo/src/layers/layernorm.py:21-36), route_experts (:86-119) and
 * forward_moe (:212-226).  The norm is fused into the router kernel's load of the tokens; no separate
 * norm launch and no extra pass over [T,H].
 *   s = hidden (+ residual);  new_residual = T(s);  normed = T( T(s * rsqrt(mean(s^2) + eps)) * norm_weight )
 *   out = new_residual + MoE(normed)
 *   hidden, residual (may be NULL), out [T,H]; norm_weight [H]; all in the activation dtype.
 *   residual_out / normed_out (device, [T,H]) receive new_residual / normed when not NULL;
 *   ids_out / scores_out as in b200moe_forward_fused.
 * normed equals b200moe_rmsnorm's output bit for bit (same code), the rest equals b200moe_forward_fused
 * on it. */
int b200moe_forward_fused_norm(b200moe_ctx* ctx, int layer, const void* hidden, const void* residual, const void* norm_weight, float eps,
                               int T, void* out, void* residual_out, void* normed_out, int64_t* ids_out, void* scores_out, int ffn_kind,
                               void* stream);

/* Expert parallelism.  No counterpart in the reference, which runs on one GPU ("expert distribution
 * across GPUs" is future work there, demo/others.md:58-62); the single-GPU result is the oracle.
 *
 * One process (or context) per GPU; rank r registers only the experts [r*E/G, (r+1)*E/G) it owns, the
 * router weight is replicated, every rank holds its own slice of the token batch.  Tokens travel to the
 * experts and results travel back by plain stores into the peers' memory over NVLink, issued by this
 * library's own kernels - no collective library on the data path, no multicast, no bulk/TMA copy with a
 * peer address.  Ranks meet through epoch flags in device memory; every wait on a flag is bounded
 * (about one second unless b200moe_ep_set_wait_ms says otherwise): when a peer never arrives the kernels
 * finish, b200moe_status reports B200MOE_DEV_WAIT_EXPIRED and the output of that call is not to be used.
 *
 * Set-up:
 *   b200moe_ep_create       allocates this rank's exchange buffer (receive regions for world x
 *                           max_local_tokens x top_k rows, return rows for its own pairs) and writes a
 *                           B200MOE_EP_HANDLE_BYTES-byte handle for the other processes (handle_out may
 *                           be NULL).  The context's max_tokens must be >= world * max_local_tokens.
 *   b200moe_ep_attach_ipc   handles_all = the handles of all ranks, rank-major (world x 64 bytes, host);
 *                           the caller exchanges them with whatever it has (torch.distributed, MPI, a file).
 *   b200moe_ep_attach_local the ranks are contexts of this same process (same GPU, or GPUs with peer access).
 *   b200moe_ep_detach       unmaps the peers; call it on every rank, after a barrier, before destroy.
 * Every rank must make the same sequence of layer calls (the flags count them).
 *
 * A layer call, b200moe_ep_forward(layer, x_local [T_local,H]) -> out [T_local,H], is three phases that
 * can also be enqueued one by one (a host that drives several ranks from one thread runs phase by phase):
 *   b200moe_ep_dispatch  router on the local tokens, then each (token, expert) pair's row is stored into
 *                        the owner rank's receive region, then count + flag
 *   b200moe_ep_experts   waits for all sources, groups the received rows by expert (K2), runs the local
 *                        experts (K3), stores each output row into its source rank's return rows, then flag
 *   b200moe_ep_combine   waits for all owners, then the weighted accumulation (K4) with the same order /
 *                        rounding rules as b200moe_forward; residual may be NULL
 * Results are bit-identical to b200moe_forward_fused on one GPU holding all experts whenever the same
 * kernel family serves the batch (it is chosen from world * T_local, as on one GPU).
 * b200moe_ep_last_routing copies the ids / scores the latest dispatch computed for the local tokens. */
#define B200MOE_EP_HANDLE_BYTES 64
int b200moe_ep_create(b200moe_ctx* ctx, int world, int rank, int max_local_tokens, void* handle_out);
int b200moe_ep_attach_ipc(b200moe_ctx* ctx, const void* handles_all);
int b200moe_ep_attach_local(b200moe_ctx* ctx, b200moe_ctx* const* ranks);
int b200moe_ep_set_wait_ms(b200moe_ctx* ctx, int milliseconds);
int b200moe_ep_detach(b200moe_ctx* ctx);
int b200moe_ep_dispatch(b200moe_ctx* ctx, int layer, const void* x_local, int T_local, void* stream);
int b200moe_ep_experts(b200moe_ctx* ctx, int layer, int ffn_kind, void* stream);
int b200moe_ep_combine(b200moe_ctx* ctx, int T_local, const int32_t* order, const void* residual, void* out, void* stream);
int b200moe_ep_forward(b200moe_ctx* ctx, int layer, const void* x_local, int T_local, const int32_t* order, const void* residual,
                       void* out, int ffn_kind, void* stream);
int b200moe_ep_last_routing(b200moe_ctx* ctx, int T_local, int64_t* ids_out, void* scores_out, void* stream);

/* One expert's SwiGLU FFN on n rows: expert_forward_with_weights (demo/src/layers/mlp.py:209-231).
 * Dense weights in the activation dtype; x [n,H] -> out [n,H]. */
int b200moe_expert_ffn(b200moe_ctx* ctx, const void* x, int n, const void* gate_proj, const void* up_proj,
                       const void* down_proj, void* out, void* stream);

/* RMSNorm in front of the MoE block, optionally fused with the residual add before it
 * (RMSNorm.rms_forward / add_rms_forward, demo/src/layers/layernorm.py:21-36; the call site is
 * `layer.post_attention_layernorm`, demo/src/model/qwen3_runner.py:204).
 *   s = float(x) [+ float(residual)];  residual_out = T(s);  out = T( T(s * rsqrt(mean(s^2) + eps)) * weight )
 *   x, residual, out, residual_out [T,H] and weight [H] in the context's activation dtype, H = hidden_size.
 *   residual_out is written only when residual is given; out may alias x, residual_out may alias residual. */
int b200moe_rmsnorm(b200moe_ctx* ctx, const void* x, const void* residual_or_null, const void* weight, float eps, int T,
                    void* out, void* residual_out_or_null, void* stream);

/* The same FFN for callers that cannot allocate device memory.  It has no counterpart in the
 * reference.  b200moe_expert_ffn needs a context, and creating one allocates its workspace; an
 * engine that has already handed the whole GPU to its own pools, or code running inside a section
 * where cudaMalloc's device-wide synchronisation is not acceptable, cannot do that.  This entry
 * point takes no context and calls no allocator of any kind: the SwiGLU intermediate and the
 * kernels' bookkeeping live in one fixed device array inside the library (about 2 MiB, held by
 * every GPU that loads the library until the process exits).
 *   x [n,H], out [n,H], gate_proj / up_proj [I,H], down_proj [H,I], all of `dtype`, on the CURRENT
 *   device, 16-byte aligned; H and I multiples of 8.
 *   Limits: n <= 64 and n * I * sizeof(element) <= 2 MiB; larger calls fail with
 *   B200MOE_E_UNSUPPORTED and a message (use b200moe_expert_ffn then).
 *   The first call on a device looks up the device address of the array; make that first call
 *   before starting any stream capture.
 *   All calls share the array, which keeps the last call's contents (each call clears the words
 *   that must start at zero): calls that overlap on the GPU race - serialise them.
 *   The per-device address table behind the look-up is filled without a lock: two host threads
 *   making the first call on one device at the same time both store the same address. */
int b200moe_expert_ffn_noalloc(const void* x, int n, int hidden_size, int intermediate_size, int dtype,
                               const void* gate_proj, const void* up_proj, const void* down_proj, void* out,
                               void* stream);

/* Companion of b200moe_expert_ffn_noalloc, equally allocation-free: waits for `stream`, then copies
 * the status word the kernels of that entry point keep in the built-in scratch (B200MOE_DEV_* bits of
 * the most recent call on the current device; each call clears it before its kernels run) to
 * *device_status_out (host).  Returns B200MOE_E_DEVICE when the word is non-zero - a bounded wait of
 * a kernel gave up and `out` of that call is not to be trusted.  No counterpart in the reference. */
int b200moe_expert_ffn_noalloc_status(int* device_status_out, void* stream);

/* Int4 g128 packer / unpacker.  Not in the reference (it has no quantised weights); the format
 * is the one documented at b200moe_set_expert.  w [out,in] in `dtype`; q uint8 [out,in/2];
 * scales bf16 [out,in/128].  unpack writes q_out int8 [out,in] (values -8..7, may be NULL) and
 * w_out [out,in] in `dtype` = scale*q rounded once (may be NULL). */
int b200moe_pack_int4(const void* w, int out_features, int in_features, int dtype, void* q, void* scales,
                      void* stream);
int b200moe_unpack_int4(const void* q, const void* scales, int out_features, int in_features, int dtype,
                        void* q_out, void* w_out, void* stream);

/* Batches of one or two tokens of b200moe_forward_fused / _fused_norm on a dense 16-bit model with ffn_kind AUTO run as ONE
 * cooperative launch that covers router, experts and combine (same results contract as the kernel chain; the
 * expert sums are taken in a different order, so outputs agree to rounding, routing bit for bit).  enable = 0
 * sends them through the kernel chain again (comparisons, per-kernel timing).  Default: enabled.  No counterpart
 * in the reference, whose draft step runs the same Python loop as every other batch
 * (demo/src/model/qwen3_runner.py:269-385). */
int b200moe_set_token_kernel(b200moe_ctx* ctx, int enable);

/* Synchronises `stream`, then reads the device status word: 0 when no kernel of this context
 * reported a failed bounds check since the last call.  Bit values are B200MOE_DEV_*. */
int b200moe_status(b200moe_ctx* ctx, int* device_status_out, void* stream);
#define B200MOE_DEV_BAD_EXPERT_ID 1   /* an id outside [0,E) was supplied; the pair was skipped */
#define B200MOE_DEV_BAD_OFFSETS 2     /* permute produced inconsistent offsets                   */
#define B200MOE_DEV_WAIT_EXPIRED 4    /* a bounded on-chip wait gave up                          */

/* Per-kernel timing for benchmarks.  While enabled, every kernel launch of this context is
 * bracketed by a pair of CUDA events on the launching stream.  b200moe_profile_read waits for
 * the recorded events, adds up elapsed milliseconds and launch counts per kernel class into
 * arrays of B200MOE_KERNEL_CLASSES entries, and forgets the records.  No counterpart in the
 * reference (its MetricsCollector takes host wall-clock times, demo/src/utils/metrics.py:76-112). */
#define B200MOE_KERNEL_ROUTER 0
#define B200MOE_KERNEL_PERMUTE 1
#define B200MOE_KERNEL_FFN_GATEUP 2
#define B200MOE_KERNEL_FFN_DOWN 3
#define B200MOE_KERNEL_COMBINE 4
#define B200MOE_KERNEL_EP_DISPATCH 5
#define B200MOE_KERNEL_EP_RETURN 6
#define B200MOE_KERNEL_TOKEN 7        /* the one-launch block of a batch of one or two tokens */
#define B200MOE_KERNEL_CLASSES 8
int b200moe_profile(b200moe_ctx* ctx, int enable);
int b200moe_profile_read(b200moe_ctx* ctx, float* total_ms, int32_t* launches);

/* Counts kernels this context has launched (monotonic); the benchmark reports the difference
 * over its timed region. */
int64_t b200moe_launch_count(const b200moe_ctx* ctx);

#ifdef __cplusplus
}
#endif
#endif /* B200MOE_H_ */
