/*
 * fmoe.h - C ABI of libfmoe_sm100a.so: the hot path of the FlashMoE layer
 * (product-key router -> fine-grained experts -> shared SwiGLU MLP; the fused forward and
 * the backward of the three ops) as hand-written CUDA kernels for NVIDIA B200 (sm_100a).
 *
 * Conventions
 *   - every data pointer is a DEVICE pointer, row-major and contiguous unless stated;
 *   - `stream` is a cudaStream_t passed as void*; all work is enqueued on it and the
 *     functions return without synchronising the host;
 *   - nothing is allocated inside: scratch memory comes from the caller through
 *     (`workspace`, `workspace_bytes`), sized by the matching *_workspace_bytes query;
 *   - return value: 0 = ok, > 0 = argument error found on the host (FMOE_ERR_*),
 *     < 0 = a CUDA runtime/driver error code, negated;
 *   - `status` (nullable) points to one int32 in device memory that kernels OR flags
 *     into (FMOE_STATUS_*): out-of-range expert ids are skipped and reported there, a
 *     device-side wait that ran out is reported there; the caller zeroes and reads it.
 *
 * Reference interfaces replaced (paths inside the flash-algo/flash-moe project) are
 * cited on each entry point.
 */
#ifndef FMOE_H_
#define FMOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* fmoe_stream_t; /* cudaStream_t */

enum fmoe_dtype { FMOE_DTYPE_F32 = 0, FMOE_DTYPE_BF16 = 1, FMOE_DTYPE_F16 = 2 };

enum fmoe_error {
  FMOE_OK = 0,
  FMOE_ERR_BAD_ARG = 1,     /* null pointer, negative size, k > num_keys ... */
  FMOE_ERR_UNSUPPORTED = 2, /* a shape/dtype combination no kernel covers */
  FMOE_ERR_WORKSPACE = 3,   /* workspace missing or too small */
  FMOE_ERR_ALIGNMENT = 4    /* pointer or row pitch not 16-byte aligned */
};

enum fmoe_status_bits {
  FMOE_STATUS_BAD_EXPERT_ID = 1, /* an index outside [0, num_experts) was skipped */
  FMOE_STATUS_WAIT_TIMEOUT = 2,  /* a bounded device-side wait gave up */
  FMOE_STATUS_BAD_ROW_INDEX = 4  /* fmoe_combine_partial_rows skipped a slot >= num_rows */
};

/* Library version (major*10000 + minor*100 + patch). */
int fmoe_version(void);
/* Static string for a return code of this library. */
const char* fmoe_error_string(int code);

/*
 * Product-key router top-k.
 * Replaces triton_flash_router_func(router_logits, num_expert_keys, num_experts_per_tok)
 *   flash_moe/ops/triton/flash_router.py:381-382 (forward: :252-314, kernels :8-194).
 * log_probs [2, T, num_keys] of `dtype`; scores [T, top_k] of `dtype`; indices [T, top_k] int64.
 * Result = the top_k candidates (i, j) of log_probs[0,t,i] + log_probs[1,t,j] (sum formed in
 * `dtype`), flat id i*num_keys + j, in descending score order, equal scores ordered by
 * ascending flat id - the order the reference's repeated arg-max produces.
 * gates (nullable) [T, top_k] of `dtype`: exp(score) rounded to `dtype`, divided by its row
 * sum when norm_topk_prob != 0 (flash_moe/modules/flash_moe.py:80-85).
 * Requires 0 <= top_k <= num_keys (flash_router.py:261).
 */
int fmoe_router_topk(const void* log_probs, int dtype, int64_t num_tokens, int num_keys, int top_k, void* scores,
                     int64_t* indices, void* gates, int norm_topk_prob, fmoe_stream_t stream);

/*
 * Router front end: BatchNorm1d(affine=False) -> Linear(H, 2*num_keys, bias=False) -> per-half log-softmax.
 * Replaces flash_moe/modules/flash_moe.py:65-72 (router_norm :49, router_gate :48).
 * x [T, H]; router_weight [2*num_keys, H]; running_mean / running_var [H] in `dtype` (the module
 * casts its buffers with its parameters); training != 0 uses batch statistics (biased variance)
 * and updates the running buffers in place with `momentum` (unbiased variance), as torch does.
 * logits [T, 2*num_keys] (half h = columns h*num_keys ..), log_probs [2, T, num_keys], both `dtype`.
 */
size_t fmoe_router_front_workspace_bytes(int64_t num_tokens, int hidden, int num_keys, int dtype);
int fmoe_router_front(const void* x, const void* router_weight, void* running_mean, void* running_var, int training,
                      float momentum, float eps, void* logits, void* log_probs, int dtype, int64_t num_tokens,
                      int hidden, int num_keys, void* workspace, size_t workspace_bytes, int32_t* status,
                      fmoe_stream_t stream);

/*
 * Per-feature batch statistics of this rank's rows for the router batch-norm under token sharding:
 * sums[0:H] = sum_r x[r, c], sums[H:2H] = sum_r x[r, c]^2 (float32).  The ranks all-reduce these 2*H
 * floats and hand the result to fmoe_layer_forward (bn_global_sums / bn_global_count), which then
 * normalises with the statistics of the WHOLE batch like the unsharded nn.BatchNorm1d in training
 * mode does (flash_moe/modules/flash_moe.py:49,:65).
 */
size_t fmoe_bn_batch_sums_workspace_bytes(int hidden);
int fmoe_bn_batch_sums(const void* x, int dtype, int64_t num_tokens, int hidden, float* sums, void* workspace,
                       size_t workspace_bytes, fmoe_stream_t stream);

/*
 * Fine-grained experts: out[t] = sum_j silu(<x[t], down[idx[t,j]]>) * gates[t,j] * up[idx[t,j]].
 * Replaces triton_flash_expert_func(hidden_states, down_weights, up_weights, indices, routing_weights)
 *   flash_moe/ops/triton/flash_expert.py:831-836 (forward :580-649, preprocessing :528-577,
 *   kernels :13-211).
 * x [T, H], down/up [N, H], gates [T, k] of `dtype`; indices [T, k] int64 (duplicates inside a
 * token accumulate; -1 marks an empty slot and is skipped silently; other ids outside [0, N) are
 * skipped and flagged in *status).
 * out [T, H] of `out_dtype`: `dtype` (one rounding of the fp32 sum) or FMOE_DTYPE_F32.
 */
size_t fmoe_expert_workspace_bytes(int64_t num_tokens, int hidden, int64_t num_experts, int top_k);
int fmoe_expert_forward(const void* x, const void* down, const void* up, const int64_t* indices, const void* gates,
                        void* out, int dtype, int out_dtype, int64_t num_tokens, int hidden, int64_t num_experts,
                        int top_k, void* workspace, size_t workspace_bytes, int32_t* status, fmoe_stream_t stream);

/*
 * The two retrieval baselines the reference ships beside its layer, on the same gather kernels.
 * fmoe_peer_forward - triton_peer_func(hidden_states, down_embed, up_embed, routing_weights, indices),
 *   flash_moe/ops/triton/peer.py:151-255: out[t] = sum_j gelu(<x[t], down[idx]>) * w[t,j] * up[idx] with the exact
 *   (erf) GELU; workspace as for fmoe_expert_forward (fmoe_expert_workspace_bytes).
 * fmoe_pkm_forward - triton_pkm_func(values, routing_weights, indices), flash_moe/ops/triton/pkm.py:123-200:
 *   out[t] = sum_j w[t,j] * values[idx[t,j]]; workspace fmoe_pkm_workspace_bytes.
 * float32 accumulation, one rounding to `dtype`; ids outside [0, num_experts) are skipped.
 */
int fmoe_peer_forward(const void* x, const void* down, const void* up, const void* routing_weights,
                      const int64_t* indices, void* out, int dtype, int64_t num_tokens, int hidden, int64_t num_experts,
                      int top_k, void* workspace, size_t workspace_bytes, int32_t* status, fmoe_stream_t stream);
size_t fmoe_pkm_workspace_bytes(int64_t num_tokens, int top_k);
int fmoe_pkm_forward(const void* values, const void* routing_weights, const int64_t* indices, void* out, int dtype,
                     int64_t num_tokens, int hidden, int64_t num_experts, int top_k, void* workspace,
                     size_t workspace_bytes, int32_t* status, fmoe_stream_t stream);

/*
 * Backward of the three ops (the reference's autograd Functions).  Gradients have the dtype of their tensors;
 * every sum is formed in float32 in a fixed order and rounded once (the reference scatters with atomics).
 *
 * fmoe_router_topk_backward - flash_moe/ops/triton/flash_router.py:197-249,:316-345:
 *   dlog_probs [2, T, num_keys] (fully written): dlog_probs[0,t,i] / [1,t,j] = sum of dscores[t,s] over the slots
 *   whose index is i*num_keys + j.
 * fmoe_expert_forward_saving_scores - fmoe_expert_forward that also writes scores_out [T,k] float32, the
 *   pre-activation scores <x[t], down[e]> the reference saves for its backward (flash_expert.py:784-794).
 * fmoe_expert_backward - flash_moe/ops/triton/flash_expert.py:214-525,:653-745: from dout [T,H], the forward's
 *   inputs and saved_scores (nullable: recomputed when absent) dx [T,H], ddown / dup [N,H] (every row written;
 *   rows of experts nobody selected are zero), dgates [T,k].  Skipped (out-of-range) ids get zero gradient.
 * fmoe_swiglu_backward - flash_moe/ops/triton/flash_mlp.py:52-102: da = dh * b * silu'(a), db = dh * silu(a)
 *   over num_elements values (a multiple of 16 bytes); h (nullable) receives silu(a) * b.
 */
int fmoe_router_topk_backward(const void* dscores, const int64_t* indices, int dtype, int64_t num_tokens, int num_keys,
                              int top_k, void* dlog_probs, fmoe_stream_t stream);
int fmoe_expert_forward_saving_scores(const void* x, const void* down, const void* up, const int64_t* indices,
                                      const void* gates, void* out, float* scores_out, int dtype, int out_dtype,
                                      int64_t num_tokens, int hidden, int64_t num_experts, int top_k, void* workspace,
                                      size_t workspace_bytes, int32_t* status, fmoe_stream_t stream);
size_t fmoe_expert_backward_workspace_bytes(int64_t num_tokens, int hidden, int64_t num_experts, int top_k);
int fmoe_expert_backward(const void* dout, const void* x, const void* down, const void* up, const int64_t* indices,
                         const void* gates, const float* saved_scores, void* dx, void* ddown, void* dup, void* dgates,
                         int dtype, int64_t num_tokens, int hidden, int64_t num_experts, int top_k, void* workspace,
                         size_t workspace_bytes, int32_t* status, fmoe_stream_t stream);
int fmoe_swiglu_backward(const void* dh, const void* a, const void* b, void* da, void* db, void* h, int dtype,
                         int64_t num_elements, fmoe_stream_t stream);

/*
 * NOT PART OF THE LAYER - a measurement aid with no counterpart in the reference, exported only so that the
 * benchmark can state the ceiling of the expert step on the GPU it runs on.  A load-only kernel with the access
 * pattern of that step: the rows row_ids[count] (each in [0, num_rows); others read row 0 and raise
 * FMOE_STATUS_BAD_ROW_INDEX in *status) of `row_bytes` bytes of `table` are brought to the SMs and dropped.
 *   mode 0: 16-byte loads into registers by device_sms * ctas_per_sm CTAs of 128 threads (row_bytes = 512, 1024,
 *           2048 or 4096);
 *   mode 1: one bulk asynchronous copy per row into a shared-memory ring, one CTA per SM (row_bytes a multiple of
 *           16 up to 6144; ctas_per_sm ignored);
 *   mode 2: the same ring filled with 16-byte cp.async copies by four producer warps - the way the fused expert
 *           kernel fetches its rows (row_bytes = 512, 1024 or 2048).
 * count * row_bytes / duration is the rate at which this GPU can bring gathered rows to its SMs.  `sink` (nullable)
 * is one float that is never written in practice.
 */
int fmoe_gather_probe(const void* table, int64_t num_rows, const int32_t* row_ids, int64_t count, int row_bytes,
                      int ctas_per_sm, int mode, float* sink, int32_t* status, fmoe_stream_t stream);

/*
 * RMS pre-norm of the decoder block that surrounds the layer: out[r] = dtype(x[r] * rsqrt(mean(x[r]^2) + eps) * weight),
 * float32 inside, one rounding; weight (nullable) [hidden] in `dtype`.  The reference leaves normalisation to its caller
 * (flash_moe/modules/flash_moe.py:55-59 receives already-normalised hidden states); together with the `residual`
 * of fmoe_layer_forward this is the caller's `x + layer(norm(x))` in two library calls.
 */
int fmoe_rms_norm(const void* x, const void* weight, void* out, int dtype, int64_t num_tokens, int hidden, float eps,
                  fmoe_stream_t stream);

/*
 * Self-test of the bounded device-side waits (no counterpart in the reference): a one-thread kernel waits on a
 * barrier that nothing completes, gives up after limit_ns (clamped to 10 ms), ORs FMOE_STATUS_WAIT_TIMEOUT into
 * *status, writes 2 to *result (1 would mean the barrier completed) and returns; later launches work as usual.
 * It exercises the give-up path that keeps a stuck copy or peer from hanging a shared GPU.
 */
int fmoe_selftest_wait_timeout(uint64_t limit_ns, int32_t* status, int32_t* result, fmoe_stream_t stream);

/*
 * Combine step of the expert-sharded layout (tables split over GPUs by expert id, token rows sent to
 * the owners, partial results sent back): out[t] = sum_g rows[slot[g * num_tokens + t]], skipping
 * slot < 0, sources added in ascending g in float32.  rows [num_rows, hidden] float32 are the partial
 * sums received from the owners, slot [num_sources, num_tokens] int32 maps (owner, token) to its row.
 * The reference has no multi-GPU code; this finishes the sum of flash_expert.py:13-211 when the
 * experts of one token live on several GPUs.  hidden must be a multiple of 4.
 */
int fmoe_combine_partial_rows(const float* rows, int64_t num_rows, const int32_t* slot, int num_sources,
                              int64_t num_tokens, int hidden, float* out, int32_t* status, fmoe_stream_t stream);

/*
 * fmoe_expert_forward with both tables sharded over the GPUs of one node by expert id: shard r = id % num_shards
 * holds expert id at row id / num_shards.  down_shards / up_shards are DEVICE arrays of num_shards pointers to row
 * 0 of each shard; the entries of the other GPUs are peer-mapped pointers (CUDA IPC / symmetric memory), which the
 * gather kernels read with plain loads over NVLink - no dispatch, no all-to-all, no host planning.  Every GPU calls
 * it for its own tokens.  bf16 / fp16 only; workspace as for fmoe_expert_forward.  The reference has no multi-GPU
 * code; the result equals fmoe_expert_forward on the unsharded tables bit for bit.
 * hot_down / hot_up (nullable, [num_hot, hidden], local memory): copies of the most frequently selected experts kept
 * on every GPU so that their rows never cross NVLink; the caller rewrites the id of hot expert j to num_experts + j.
 */
int fmoe_expert_forward_sharded(const void* x, const void* const* down_shards, const void* const* up_shards,
                                int num_shards, const int64_t* indices, const void* gates, void* out, int dtype,
                                int out_dtype, int64_t num_tokens, int hidden, int64_t num_experts, int top_k,
                                void* workspace, size_t workspace_bytes, int32_t* status, fmoe_stream_t stream,
                                const void* hot_down, const void* hot_up, int64_t num_hot);

/*
 * fmoe_expert_forward without a caller-supplied workspace.  It has no counterpart in the
 * reference; it exists for hosts that cannot allocate device memory where they call the library
 * (a frozen memory plan after warm-up, a fixed real-time budget, a language binding without a
 * device allocator).  Same arguments and results as fmoe_expert_forward; the scratch is a
 * fmoe_expert_static_scratch_bytes() = 8 MiB array inside the library image that each GPU using
 * the library holds until the process exits.  Shapes with fmoe_expert_workspace_bytes(...) above
 * that limit return FMOE_ERR_WORKSPACE.  All calls share the array: calls that overlap on the GPU
 * race, so order them on one stream or with events.  The first call on a device looks up the
 * array's device address (which, with CUDA's lazy module loading, may be the moment the driver
 * loads this library's device code and the 8 MiB with it): make it during warm-up and outside any
 * stream capture.  After that first call nothing is allocated.
 */
size_t fmoe_expert_static_scratch_bytes(void);
int fmoe_expert_forward_static(const void* x, const void* down, const void* up, const int64_t* indices,
                               const void* gates, void* out, int dtype, int out_dtype, int64_t num_tokens, int hidden,
                               int64_t num_experts, int top_k, int32_t* status, fmoe_stream_t stream);

/*
 * Shared SwiGLU MLP: out = (silu(x Wg^T) * (x Wu^T)) Wd^T  (+ addend).
 * Replaces triton_flash_mlp_func(x, gate_weight, up_weight, down_weight)
 *   flash_moe/ops/triton/flash_mlp.py:169-181 and the final add flash_moe/modules/flash_moe.py:101.
 * x [T, H], gate_w / up_w [I, H], down_w [H, I], out [T, H] of `dtype`;
 * addend (nullable) [T, H] float32 is added to the fp32 accumulator before the single rounding.
 */
size_t fmoe_mlp_workspace_bytes(int64_t num_tokens, int hidden, int intermediate, int dtype);
int fmoe_mlp_forward(const void* x, const void* gate_w, const void* up_w, const void* down_w, const float* addend,
                     void* out, int dtype, int64_t num_tokens, int hidden, int intermediate, void* workspace,
                     size_t workspace_bytes, int32_t* status, fmoe_stream_t stream);

/*
 * fmoe_mlp_forward that also keeps the two pre-activations pre_gate = x Wg^T and pre_up = x Wu^T ([T, I] of `dtype`),
 * the tensors the reference's TritonSwiGLUFunc saves for its backward (flash_moe/ops/triton/flash_mlp.py:150-156).
 * They are written by the epilogue of the fused gate/up GEMM, which only its CTA-pair form supports: 16-bit dtypes,
 * T >= 512, I >= 256, H >= 256 - other shapes return FMOE_ERR_UNSUPPORTED (callers then recompute in the backward).
 */
int fmoe_mlp_forward_saving_preacts(const void* x, const void* gate_w, const void* up_w, const void* down_w,
                                    void* out, void* pre_gate, void* pre_up, int dtype, int64_t num_tokens, int hidden,
                                    int intermediate, void* workspace, size_t workspace_bytes, int32_t* status,
                                    fmoe_stream_t stream);

/*
 * Whole layer forward.  Replaces FlashMoE.forward, flash_moe/modules/flash_moe.py:55-105.
 * Parameter names follow the module: gate_proj/up_proj [I,H], down_proj [H,I], router_gate
 * [2*num_keys, H], down_embed/up_embed [N, H], router_norm running buffers [H].
 * Outputs: y [T, H]; router_logits [T, 2*num_keys] (the module returns it viewed as
 * (2, T, num_keys)); optional indices [T,k] int64 and gates [T,k] for inspection.
 * residual (nullable) is added in the last GEMM's epilogue: the reference leaves the skip connection of the
 * surrounding decoder block to its caller (flash_moe/modules/flash_moe.py:55-59 takes **kwargs for such callers).
 * aux_stream (nullable): a second stream the shared MLP may run on concurrently with routing.
 * stage_events (nullable): host array of 2*FMOE_NUM_STAGES cudaEvent_t handles; entry 2*s is
 * recorded before and 2*s+1 after stage s (enum fmoe_stage) on the stream that stage runs on,
 * so a caller can time the stages of a real forward with cudaEventElapsedTime.
 */
enum fmoe_stage {
  FMOE_STAGE_ROUTER_FRONT = 0, /* batch-norm + sub-key GEMM + log-softmax */
  FMOE_STAGE_ROUTER_TOPK = 1,
  FMOE_STAGE_EXPERT_SCORES = 2, /* (sort +) gs = silu(<x, down[e]>) * gate */
  FMOE_STAGE_EXPERT_ACCUM = 3,  /* acc = sum gs * up[e] */
  FMOE_STAGE_MLP_UP = 4,        /* h = silu(x Wg^T) * (x Wu^T) */
  FMOE_STAGE_MLP_DOWN = 5,      /* y = h Wd^T + acc */
  FMOE_NUM_STAGES = 6
};

typedef struct fmoe_layer_args {
  const void* x;
  const void* gate_proj;
  const void* up_proj;
  const void* down_proj;
  const void* router_gate;
  const void* down_embed;
  const void* up_embed;
  void* running_mean;
  void* running_var;
  void* y;
  void* router_logits;
  int64_t* indices_out; /* nullable */
  void* gates_out;      /* nullable */
  void* workspace;
  size_t workspace_bytes;
  int32_t* status; /* nullable */
  fmoe_stream_t stream;
  fmoe_stream_t aux_stream; /* nullable */
  void* const* stage_events; /* nullable */
  int64_t num_tokens;
  int64_t num_experts;
  int32_t hidden;
  int32_t intermediate;
  int32_t num_keys;
  int32_t top_k;
  int32_t dtype;
  int32_t training;
  int32_t norm_topk_prob;
  float bn_momentum;
  float bn_eps;
  const float* bn_global_sums; /* nullable; training only: [2*H] sums over all shards (fmoe_bn_batch_sums) */
  int64_t bn_global_count;     /* rows behind bn_global_sums */
  const void* residual;        /* nullable: [T, H] in `dtype`; y = dtype(shared MLP + experts + residual), the
                                  caller's `x + layer(x)` (a decoder block's skip connection) with ONE rounding */
} fmoe_layer_args;

size_t fmoe_layer_workspace_bytes(int64_t num_tokens, int hidden, int intermediate, int64_t num_experts, int num_keys,
                                  int top_k, int dtype);
int fmoe_layer_forward(const fmoe_layer_args* args);

#ifdef __cplusplus
}
#endif
#endif /* FMOE_H_ */
