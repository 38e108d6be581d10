// extern "C" entry points of libfmoe_sm100a.so (declared in include/fmoe.h) and the host-side
// orchestration of the layer forward.
#include <cstdlib>

#include "common.cuh"

namespace fmoe {

size_t bn_workspace_bytes(int H);
int launch_bn(const void* x, void* xn, void* running_mean, void* running_var, int training, float momentum, float eps,
              int dtype, int64_t ntok, int H, float* ws, const float* global_sums, int64_t global_count,
              cudaStream_t stream);
int launch_bn_sums(const void* x, int dtype, int64_t ntok, int H, float* ws, float* sums, cudaStream_t stream);
void bn_stats_in_workspace(float* ws, int H, const float** mean, const float** invstd);

int device_sm_count() {
  static int cache[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cache[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cache[dev] = n;
  }
  return cache[dev];
}

// read on every launch (a getenv costs well under a microsecond), so a process can compare settings: FMOE_PDL is a
// bit mask of kernel classes (see common.cuh) that are launched with programmatic stream serialisation
bool pdl_enabled(int kernel_class) {
  const char* v = std::getenv("FMOE_PDL");
  const int mask = v == nullptr ? kPdlDefaultMask : std::atoi(v);
  return (mask & kernel_class) != 0;
}

namespace {

bool is16(int dtype) { return dtype == FMOE_DTYPE_BF16 || dtype == FMOE_DTYPE_F16; }
bool valid_dtype(int dtype) { return dtype == FMOE_DTYPE_F32 || is16(dtype); }

struct Carver {
  char* base;
  size_t off = 0;
  explicit Carver(void* p) : base(static_cast<char*>(p)) {}
  void* take(size_t bytes) {
    void* p = base ? base + off : nullptr;
    off += align_up(bytes, 256);
    return p;
  }
};

// fork/join events for the optional second stream, one pair per device and host thread
struct ForkJoin {
  cudaEvent_t fork = nullptr, join = nullptr;
};
ForkJoin* fork_join_events() {
  thread_local ForkJoin ev[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (ev[dev].fork == nullptr) {
    if (cudaEventCreateWithFlags(&ev[dev].fork, cudaEventDisableTiming) != cudaSuccess) return nullptr;
    if (cudaEventCreateWithFlags(&ev[dev].join, cudaEventDisableTiming) != cudaSuccess) return nullptr;
  }
  return &ev[dev];
}

size_t router_front_ws(int64_t T, int H, int dtype) {
  Carver c(nullptr);
  c.take(static_cast<size_t>(T) * H * dtype_size(dtype));
  c.take(bn_workspace_bytes(H));
  return c.off;
}

// logp == nullptr: stop after the logits (the caller applies the log-softmax elsewhere)
int router_front(const void* x, const void* w, void* rm, void* rv, int training, float momentum, float eps,
                 void* logits, void* logp, int dtype, int64_t T, int H, int nk, void* ws, size_t ws_bytes,
                 int32_t* status, cudaStream_t stream, const float* bn_sums = nullptr, int64_t bn_count = 0) {
  if (!valid_dtype(dtype) || T < 0 || H <= 0 || nk <= 0) return FMOE_ERR_BAD_ARG;
  if (T == 0) return FMOE_OK;
  if (x == nullptr || w == nullptr || logits == nullptr) return FMOE_ERR_BAD_ARG;
  if (ws == nullptr || ws_bytes < router_front_ws(T, H, dtype)) return FMOE_ERR_WORKSPACE;
  Carver c(ws);
  void* xn = c.take(static_cast<size_t>(T) * H * dtype_size(dtype));
  float* bnws = static_cast<float*>(c.take(bn_workspace_bytes(H)));
  const bool tc = is16(dtype) && (H % 8 == 0) && aligned16(w);
  int rc;
  if (logp == nullptr && tc && aligned16(x) && aligned16(logits) && router_bn_gemm_supported(dtype, T, 2 * nk, H)) {
    // one kernel: the GEMM normalises its x tiles in shared memory (training: after the statistics pre-pass)
    const float *mean = nullptr, *invstd = nullptr;
    if (training) {
      rc = launch_bn(x, nullptr, rm, rv, training, momentum, eps, dtype, T, H, bnws, bn_sums, bn_count, stream);
      if (rc != FMOE_OK) return rc;
      bn_stats_in_workspace(bnws, H, &mean, &invstd);
    } else if (rm == nullptr || rv == nullptr) {
      return FMOE_ERR_BAD_ARG;
    }
    return launch_router_bn_gemm(x, w, mean, invstd, training ? nullptr : rm, training ? nullptr : rv, eps, logits, dtype,
                                 T, 2 * nk, H, status, stream);
  }
  rc = launch_bn(x, xn, rm, rv, training, momentum, eps, dtype, T, H, bnws, bn_sums, bn_count, stream);
  if (rc != FMOE_OK) return rc;
  if (logp != nullptr && tc && gemm_router_fused_supported(nk) && aligned16(logits) && aligned16(logp))
    return launch_gemm_router(xn, H, 0, w, logits, logp, dtype, T, nk, H, status, stream);
  if (tc && (2 * nk) % 8 == 0 && aligned16(logits))
    rc = launch_gemm_add(xn, w, nullptr, logits, dtype, T, 2 * nk, H, status, stream);
  else
    rc = launch_simt_gemm(xn, H, w, nullptr, nullptr, logits, 2 * static_cast<int64_t>(nk), dtype, 0, T, 2 * nk, H,
                          stream);
  if (rc != FMOE_OK) return rc;
  if (logp == nullptr) return FMOE_OK;
  return launch_log_softmax_halves(logits, logp, dtype, T, nk, stream);
}

size_t mlp_ws(int64_t T, int I, int dtype) { return align_up(static_cast<size_t>(T) * I * dtype_size(dtype), 256); }

int mlp_up(const void* x, const void* gw, const void* uw, void* h, int dtype, int64_t T, int H, int I, int32_t* status,
           cudaStream_t stream, void* pre_gate = nullptr, void* pre_up = nullptr) {
  const bool tc = is16(dtype) && (H % 8 == 0) && (I % 8 == 0) && aligned16(x) && aligned16(gw) && aligned16(uw);
  if (tc && gemm_pair_supported(T, I, H))
    return launch_gemm_swiglu_pair(x, gw, uw, h, dtype, T, I, H, status, stream, pre_gate, pre_up);
  if (pre_gate != nullptr || pre_up != nullptr) return FMOE_ERR_UNSUPPORTED;  // only the CTA-pair kernel keeps them
  if (tc) return launch_gemm_swiglu(x, gw, uw, h, dtype, T, I, H, status, stream);
  return launch_simt_gemm(x, H, gw, uw, nullptr, h, I, dtype, 1, T, I, H, stream);
}

// residual (nullable): [T, H] in the module dtype, added with the float32 addend before the single rounding
int mlp_down(const void* h, const void* dw, const float* addend, void* out, int dtype, int64_t T, int H, int I,
             int32_t* status, cudaStream_t stream, const void* residual = nullptr) {
  const bool tc = is16(dtype) && (H % 8 == 0) && (I % 8 == 0) && aligned16(dw) && aligned16(out) &&
                  (addend == nullptr || aligned16(addend)) && (residual == nullptr || aligned16(residual));
  if (tc && gemm_pair_supported(T, H, I))
    return launch_gemm_add_pair(h, dw, addend, out, dtype, T, H, I, status, stream, residual);
  if (tc) return launch_gemm_add(h, dw, addend, out, dtype, T, H, I, status, stream, residual);
  return launch_simt_gemm(h, I, dw, nullptr, addend, out, H, dtype, 0, T, H, I, stream, residual);
}

struct LayerWs {
  void *front, *logp, *scores, *indices, *gates, *acc, *h, *expert;
  size_t front_bytes, expert_bytes, total;
};

LayerWs carve_layer(void* ws, int64_t T, int H, int I, int64_t N, int nk, int k, int dtype) {
  Carver c(ws);
  LayerWs w;
  const size_t es = dtype_size(dtype);
  w.front_bytes = router_front_ws(T, H, dtype);
  w.front = c.take(w.front_bytes);
  w.logp = c.take(static_cast<size_t>(2) * T * nk * es);
  w.scores = c.take(static_cast<size_t>(T) * k * es);
  w.indices = c.take(static_cast<size_t>(T) * k * 8);
  w.gates = c.take(static_cast<size_t>(T) * k * es);
  w.acc = c.take(static_cast<size_t>(T) * H * 4);
  w.h = c.take(static_cast<size_t>(T) * I * es);
  w.expert_bytes = expert_workspace_bytes(T, H, N, k);
  w.expert = c.take(w.expert_bytes);
  w.total = c.off;
  return w;
}

}  // namespace
}  // namespace fmoe

using namespace fmoe;

extern "C" {

int fmoe_version(void) { return 100; }

const char* fmoe_error_string(int code) {
  if (code < 0) return cudaGetErrorString(static_cast<cudaError_t>(-code));
  switch (code) {
    case FMOE_OK: return "ok";
    case FMOE_ERR_BAD_ARG: return "bad argument";
    case FMOE_ERR_UNSUPPORTED: return "unsupported shape or dtype";
    case FMOE_ERR_WORKSPACE: return "workspace missing or too small";
    case FMOE_ERR_ALIGNMENT: return "pointer or row size not 16-byte aligned";
    default: return "unknown error";
  }
}

int fmoe_router_topk(const void* log_probs, int dtype, int64_t num_tokens, int num_keys, int top_k, void* scores,
                     int64_t* indices, void* gates, int norm_topk_prob, fmoe_stream_t stream) {
  return launch_router_topk(log_probs, dtype, num_tokens, num_keys, top_k, scores, indices, gates,
                            norm_topk_prob ? 1 : 0, static_cast<cudaStream_t>(stream));
}

size_t fmoe_router_front_workspace_bytes(int64_t num_tokens, int hidden, int num_keys, int dtype) {
  (void)num_keys;
  if (num_tokens < 0 || hidden <= 0) return 0;
  return router_front_ws(num_tokens, hidden, dtype);
}

int fmoe_router_front(const void* x, const void* router_weight, void* running_mean, void* running_var, int training,
                      float momentum, float eps, void* logits, void* log_probs, int dtype, int64_t num_tokens,
                      int hidden, int num_keys, void* workspace, size_t workspace_bytes, int32_t* status,
                      fmoe_stream_t stream) {
  if (log_probs == nullptr && num_tokens > 0) return FMOE_ERR_BAD_ARG;
  return router_front(x, router_weight, running_mean, running_var, training, momentum, eps, logits, log_probs, dtype,
                      num_tokens, hidden, num_keys, workspace, workspace_bytes, status,
                      static_cast<cudaStream_t>(stream));
}

size_t fmoe_bn_batch_sums_workspace_bytes(int hidden) { return hidden > 0 ? bn_workspace_bytes(hidden) : 0; }

int fmoe_bn_batch_sums(const void* x, int dtype, int64_t num_tokens, int hidden, float* sums, void* workspace,
                       size_t workspace_bytes, fmoe_stream_t stream) {
  if (!valid_dtype(dtype) || hidden <= 0 || num_tokens <= 0) return FMOE_ERR_BAD_ARG;
  if (workspace == nullptr || workspace_bytes < bn_workspace_bytes(hidden)) return FMOE_ERR_WORKSPACE;
  return launch_bn_sums(x, dtype, num_tokens, hidden, static_cast<float*>(workspace), sums,
                        static_cast<cudaStream_t>(stream));
}

int fmoe_expert_forward_sharded(const void* x, const void* const* down_shards, const void* const* up_shards,
                                int num_shards, const int64_t* indices, const void* gates, void* out, int dtype,
                                int out_dtype, int64_t num_tokens, int hidden, int64_t num_experts, int top_k,
                                void* workspace, size_t workspace_bytes, int32_t* status, fmoe_stream_t stream,
                                const void* hot_down, const void* hot_up, int64_t num_hot) {
  if (!valid_dtype(dtype)) return FMOE_ERR_BAD_ARG;
  return launch_expert_forward_peer(x, down_shards, up_shards, num_shards, indices, gates, out, dtype, out_dtype,
                                    num_tokens, hidden, num_experts, top_k, workspace, workspace_bytes, status,
                                    static_cast<cudaStream_t>(stream), hot_down, hot_up, num_hot);
}

int fmoe_peer_forward(const void* x, const void* down, const void* up, const void* routing_weights,
                      const int64_t* indices, void* out, int dtype, int64_t num_tokens, int hidden, int64_t num_experts,
                      int top_k, void* workspace, size_t workspace_bytes, int32_t* status, fmoe_stream_t stream) {
  if (!valid_dtype(dtype)) return FMOE_ERR_BAD_ARG;
  return launch_expert_forward(x, down, up, indices, routing_weights, out, dtype, dtype, num_tokens, hidden, num_experts,
                               top_k, workspace, workspace_bytes, status, static_cast<cudaStream_t>(stream), nullptr,
                               kActGelu);
}

size_t fmoe_pkm_workspace_bytes(int64_t num_tokens, int top_k) {
  return (num_tokens < 0 || top_k < 0) ? 0 : static_cast<size_t>(num_tokens) * top_k * 4;
}

int fmoe_pkm_forward(const void* values, const void* routing_weights, const int64_t* indices, void* out, int dtype,
                     int64_t num_tokens, int hidden, int64_t num_experts, int top_k, void* workspace,
                     size_t workspace_bytes, int32_t* status, fmoe_stream_t stream) {
  if (!valid_dtype(dtype)) return FMOE_ERR_BAD_ARG;
  return launch_weighted_rows(values, routing_weights, indices, out, dtype, num_tokens, hidden, num_experts, top_k,
                              workspace, workspace_bytes, status, static_cast<cudaStream_t>(stream));
}

int fmoe_router_topk_backward(const void* dscores, const int64_t* indices, int dtype, int64_t num_tokens, int num_keys,
                              int top_k, void* dlog_probs, fmoe_stream_t stream) {
  if (!valid_dtype(dtype)) return FMOE_ERR_BAD_ARG;
  return launch_router_topk_backward(dscores, indices, dtype, num_tokens, num_keys, top_k, dlog_probs,
                                     static_cast<cudaStream_t>(stream));
}

int fmoe_expert_forward_saving_scores(const void* x, const void* down, const void* up, const int64_t* indices,
                                      const void* gates, void* out, float* scores_out, int dtype, int out_dtype,
                                      int64_t num_tokens, int hidden, int64_t num_experts, int top_k, void* workspace,
                                      size_t workspace_bytes, int32_t* status, fmoe_stream_t stream) {
  if (!valid_dtype(dtype)) return FMOE_ERR_BAD_ARG;
  return launch_expert_forward(x, down, up, indices, gates, out, dtype, out_dtype, num_tokens, hidden, num_experts,
                               top_k, workspace, workspace_bytes, status, static_cast<cudaStream_t>(stream), nullptr,
                               kActSilu, scores_out);
}

size_t fmoe_expert_backward_workspace_bytes(int64_t num_tokens, int hidden, int64_t num_experts, int top_k) {
  return expert_backward_workspace_bytes(num_tokens, hidden, num_experts, top_k);
}

int fmoe_expert_backward(const void* dout, const void* x, const void* down, const void* up, const int64_t* indices,
                         const void* gates, const float* saved_scores, void* dx, void* ddown, void* dup, void* dgates,
                         int dtype, int64_t num_tokens, int hidden, int64_t num_experts, int top_k, void* workspace,
                         size_t workspace_bytes, int32_t* status, fmoe_stream_t stream) {
  if (!valid_dtype(dtype)) return FMOE_ERR_BAD_ARG;
  return launch_expert_backward(dout, x, down, up, indices, gates, dx, ddown, dup, dgates, dtype, num_tokens, hidden,
                                num_experts, top_k, workspace, workspace_bytes, status, static_cast<cudaStream_t>(stream),
                                saved_scores);
}

int fmoe_swiglu_backward(const void* dh, const void* a, const void* b, void* da, void* db, void* h, int dtype,
                         int64_t num_elements, fmoe_stream_t stream) {
  if (!valid_dtype(dtype)) return FMOE_ERR_BAD_ARG;
  return launch_swiglu_backward(dh, a, b, da, db, h, dtype, num_elements, static_cast<cudaStream_t>(stream));
}

int fmoe_gather_probe(const void* table, int64_t num_rows, const int32_t* row_ids, int64_t count, int row_bytes,
                      int ctas_per_sm, int mode, float* sink, int32_t* status, fmoe_stream_t stream) {
  return launch_gather_probe(table, num_rows, row_ids, count, row_bytes, ctas_per_sm, mode, sink, status,
                             static_cast<cudaStream_t>(stream));
}

int fmoe_rms_norm(const void* x, const void* weight, void* out, int dtype, int64_t num_tokens, int hidden, float eps,
                  fmoe_stream_t stream) {
  if (!valid_dtype(dtype)) return FMOE_ERR_BAD_ARG;
  return launch_rms_norm(x, weight, out, dtype, num_tokens, hidden, eps, static_cast<cudaStream_t>(stream));
}

int fmoe_combine_partial_rows(const float* rows, int64_t num_rows, const int32_t* slot, int num_sources,
                              int64_t num_tokens, int hidden, float* out, int32_t* status, fmoe_stream_t stream) {
  return launch_combine_rows(rows, num_rows, slot, num_sources, num_tokens, hidden, out, status,
                             static_cast<cudaStream_t>(stream));
}

size_t fmoe_expert_workspace_bytes(int64_t num_tokens, int hidden, int64_t num_experts, int top_k) {
  return expert_workspace_bytes(num_tokens, hidden, num_experts, top_k);
}

int fmoe_expert_forward(const void* x, const void* down, const void* up, const int64_t* indices, const void* gates,
                        void* out, int dtype, int out_dtype, int64_t num_tokens, int hidden, int64_t num_experts,
                        int top_k, void* workspace, size_t workspace_bytes, int32_t* status, fmoe_stream_t stream) {
  if (!valid_dtype(dtype)) return FMOE_ERR_BAD_ARG;
  return launch_expert_forward(x, down, up, indices, gates, out, dtype, out_dtype, num_tokens, hidden, num_experts,
                               top_k, workspace, workspace_bytes, status, static_cast<cudaStream_t>(stream));
}

size_t fmoe_mlp_workspace_bytes(int64_t num_tokens, int hidden, int intermediate, int dtype) {
  (void)hidden;
  if (num_tokens < 0 || intermediate <= 0) return 0;
  return mlp_ws(num_tokens, intermediate, dtype);
}

int fmoe_mlp_forward(const void* x, const void* gate_w, const void* up_w, const void* down_w, const float* addend,
                     void* out, int dtype, int64_t num_tokens, int hidden, int intermediate, void* workspace,
                     size_t workspace_bytes, int32_t* status, fmoe_stream_t stream) {
  if (!valid_dtype(dtype) || num_tokens < 0 || hidden <= 0 || intermediate <= 0) return FMOE_ERR_BAD_ARG;
  if (num_tokens == 0) return FMOE_OK;
  if (x == nullptr || gate_w == nullptr || up_w == nullptr || down_w == nullptr || out == nullptr)
    return FMOE_ERR_BAD_ARG;
  if (workspace == nullptr || workspace_bytes < mlp_ws(num_tokens, intermediate, dtype)) return FMOE_ERR_WORKSPACE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int rc = mlp_up(x, gate_w, up_w, workspace, dtype, num_tokens, hidden, intermediate, status, s);
  if (rc != FMOE_OK) return rc;
  return mlp_down(workspace, down_w, addend, out, dtype, num_tokens, hidden, intermediate, status, s);
}

int fmoe_mlp_forward_saving_preacts(const void* x, const void* gate_w, const void* up_w, const void* down_w,
                                    void* out, void* pre_gate, void* pre_up, int dtype, int64_t num_tokens, int hidden,
                                    int intermediate, void* workspace, size_t workspace_bytes, int32_t* status,
                                    fmoe_stream_t stream) {
  if (!valid_dtype(dtype) || num_tokens < 0 || hidden <= 0 || intermediate <= 0) return FMOE_ERR_BAD_ARG;
  if (num_tokens == 0) return FMOE_OK;
  if (x == nullptr || gate_w == nullptr || up_w == nullptr || down_w == nullptr || out == nullptr || pre_gate == nullptr ||
      pre_up == nullptr)
    return FMOE_ERR_BAD_ARG;
  if (!aligned16(pre_gate) || !aligned16(pre_up)) return FMOE_ERR_ALIGNMENT;
  if (workspace == nullptr || workspace_bytes < mlp_ws(num_tokens, intermediate, dtype)) return FMOE_ERR_WORKSPACE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int rc = mlp_up(x, gate_w, up_w, workspace, dtype, num_tokens, hidden, intermediate, status, s, pre_gate, pre_up);
  if (rc != FMOE_OK) return rc;
  return mlp_down(workspace, down_w, nullptr, out, dtype, num_tokens, hidden, intermediate, status, s);
}

size_t fmoe_layer_workspace_bytes(int64_t num_tokens, int hidden, int intermediate, int64_t num_experts, int num_keys,
                                  int top_k, int dtype) {
  if (num_tokens < 0 || hidden <= 0 || intermediate <= 0 || num_experts <= 0 || num_keys <= 0 || top_k < 0) return 0;
  return carve_layer(nullptr, num_tokens, hidden, intermediate, num_experts, num_keys, top_k, dtype).total;
}

int fmoe_layer_forward(const fmoe_layer_args* a) {
  if (a == nullptr) return FMOE_ERR_BAD_ARG;
  const int64_t T = a->num_tokens;
  const int H = a->hidden, I = a->intermediate, nk = a->num_keys, k = a->top_k, dtype = a->dtype;
  const int64_t N = a->num_experts;
  if (!valid_dtype(dtype) || T < 0 || H <= 0 || I <= 0 || N <= 0 || nk <= 0 || k < 0 || k > nk) return FMOE_ERR_BAD_ARG;
  if (static_cast<int64_t>(nk) * nk > N) return FMOE_ERR_BAD_ARG;  // flat ids must address the tables
  if (T == 0) return FMOE_OK;
  if (!a->x || !a->gate_proj || !a->up_proj || !a->down_proj || !a->router_gate || !a->down_embed || !a->up_embed ||
      !a->y || !a->router_logits)
    return FMOE_ERR_BAD_ARG;
  const LayerWs w = carve_layer(a->workspace, T, H, I, N, nk, k, dtype);
  if (a->workspace == nullptr || a->workspace_bytes < w.total) return FMOE_ERR_WORKSPACE;
  cudaStream_t s = static_cast<cudaStream_t>(a->stream);
  cudaStream_t s2 = static_cast<cudaStream_t>(a->aux_stream);
  int64_t* indices = a->indices_out ? a->indices_out : static_cast<int64_t*>(w.indices);
  void* gates = a->gates_out ? a->gates_out : w.gates;
  int rc;
  auto mark = [&](int stage, int end, cudaStream_t st) -> int {
    if (a->stage_events == nullptr) return FMOE_OK;
    void* ev = a->stage_events[2 * stage + end];
    if (ev == nullptr) return FMOE_OK;
    FMOE_CUDA_TRY(cudaEventRecord(static_cast<cudaEvent_t>(ev), st));
    return FMOE_OK;
  };
#define FMOE_MARK(stage, end, st)                         \
  do {                                                    \
    if ((rc = mark(stage, end, st)) != FMOE_OK) return rc; \
  } while (0)

  // router front end: batch-norm -> sub-key GEMM.  For 16-bit dtypes and num_keys <= 1024 the top-k
  // kernel applies the per-half log-softmax itself (each warp already holds both halves of its
  // token in registers), which saves a [2, T, nk] round trip and a serial GEMM epilogue.
  const bool topk_from_logits = is16(dtype) && nk <= 1024;
  FMOE_MARK(FMOE_STAGE_ROUTER_FRONT, 0, s);
  rc = router_front(a->x, a->router_gate, a->running_mean, a->running_var, a->training, a->bn_momentum, a->bn_eps,
                    a->router_logits, topk_from_logits ? nullptr : w.logp, dtype, T, H, nk, w.front, w.front_bytes,
                    a->status, s, a->training ? a->bn_global_sums : nullptr, a->bn_global_count);
  if (rc != FMOE_OK) return rc;
  FMOE_MARK(FMOE_STAGE_ROUTER_FRONT, 1, s);

  // shared MLP, first half: h = silu(x Wg^T) * (x Wu^T).  It is independent of routing; on the side
  // stream it is forked AFTER the router GEMM (both want a whole SM's shared memory and its tensor memory) so that
  // the tensor-core GEMM overlaps the issue-bound top-k that follows.
  ForkJoin* fj = nullptr;
  // after the fork every early return first joins the side stream back into the caller's, so that a failed call
  // never leaves a dangling branch (which would also invalidate a stream capture in progress)
  auto fail = [&](int code) -> int {
    if (fj != nullptr) {
      if (cudaEventRecord(fj->join, s2) == cudaSuccess) (void)cudaStreamWaitEvent(s, fj->join, 0);
    }
    return code;
  };
  if (s2 != nullptr && s2 != s) {
    fj = fork_join_events();
    if (fj == nullptr) return -static_cast<int>(cudaErrorUnknown);
    FMOE_CUDA_TRY(cudaEventRecord(fj->fork, s));
    FMOE_CUDA_TRY(cudaStreamWaitEvent(s2, fj->fork, 0));
    FMOE_MARK(FMOE_STAGE_MLP_UP, 0, s2);
    rc = mlp_up(a->x, a->gate_proj, a->up_proj, w.h, dtype, T, H, I, a->status, s2);
    if (rc != FMOE_OK) return fail(rc);
    FMOE_MARK(FMOE_STAGE_MLP_UP, 1, s2);
    FMOE_CUDA_TRY(cudaEventRecord(fj->join, s2));
  }

  // product-key top-k (+ gates)
  FMOE_MARK(FMOE_STAGE_ROUTER_TOPK, 0, s);
  rc = FMOE_ERR_UNSUPPORTED;
  if (topk_from_logits)
    rc = launch_router_topk(a->router_logits, dtype, T, nk, k, w.scores, indices, gates,
                            (a->norm_topk_prob ? 1 : 0) | 2, s);
  if (rc == FMOE_ERR_UNSUPPORTED) {
    if (topk_from_logits) {  // shapes the register kernel does not cover: explicit log-softmax pass
      rc = launch_log_softmax_halves(a->router_logits, w.logp, dtype, T, nk, s);
      if (rc != FMOE_OK) return fail(rc);
    }
    rc = launch_router_topk(w.logp, dtype, T, nk, k, w.scores, indices, gates, a->norm_topk_prob ? 1 : 0, s);
  }
  if (rc != FMOE_OK) return fail(rc);
  FMOE_MARK(FMOE_STAGE_ROUTER_TOPK, 1, s);
  // The side stream is joined HERE, before the experts: the two gather passes compete with the GEMM for the same
  // L2 -> SM bandwidth and are slower beside it than after it.  (Measured at the benchmark shape the fork does not
  // pay either way - 230 vs 226 us: the top-k's CTAs fill the shared memory first and the GEMM's wait for them; with
  // the top-k held to one CTA per SM so that the GEMM fits beside it, the top-k itself takes 165 us, because one
  // token costs a warp about 20 us of dependent instructions and all 4096 tokens must be resident at once; and with
  // the GEMM's ring cut to four stages, so that four top-k CTAs fit beside it, the step takes 224 against 216 us.)
  bool joined = false;
  if (fj != nullptr) {
    if (cudaStreamWaitEvent(s, fj->join, 0) != cudaSuccess) return fail(-static_cast<int>(cudaErrorUnknown));
    fj = nullptr;
    joined = true;
  }
  FMOE_MARK(FMOE_STAGE_EXPERT_SCORES, 0, s);

  // routed experts into an fp32 accumulator; the scores stage ends and the accumulate stage starts
  // between the two passes, inside the launcher
  void* between[2] = {nullptr, nullptr};
  if (a->stage_events != nullptr) {
    between[0] = a->stage_events[2 * FMOE_STAGE_EXPERT_SCORES + 1];
    between[1] = a->stage_events[2 * FMOE_STAGE_EXPERT_ACCUM + 0];
    if (T == 0 || k == 0) {  // the launcher returns before it reaches the marks
      FMOE_MARK(FMOE_STAGE_EXPERT_SCORES, 1, s);
      FMOE_MARK(FMOE_STAGE_EXPERT_ACCUM, 0, s);
    }
  }
  rc = launch_expert_forward(a->x, a->down_embed, a->up_embed, indices, gates, w.acc, dtype, FMOE_DTYPE_F32, T, H, N, k,
                             w.expert, w.expert_bytes, a->status, s, between);
  if (rc != FMOE_OK) return fail(rc);
  FMOE_MARK(FMOE_STAGE_EXPERT_ACCUM, 1, s);

  if (!joined) {
    FMOE_MARK(FMOE_STAGE_MLP_UP, 0, s);
    rc = mlp_up(a->x, a->gate_proj, a->up_proj, w.h, dtype, T, H, I, a->status, s);
    if (rc != FMOE_OK) return fail(rc);
    FMOE_MARK(FMOE_STAGE_MLP_UP, 1, s);
  }
  // y = h Wd^T + experts, one rounding
  FMOE_MARK(FMOE_STAGE_MLP_DOWN, 0, s);
  rc = mlp_down(w.h, a->down_proj, static_cast<const float*>(w.acc), a->y, dtype, T, H, I, a->status, s, a->residual);
  if (rc != FMOE_OK) return fail(rc);
  FMOE_MARK(FMOE_STAGE_MLP_DOWN, 1, s);
#undef FMOE_MARK
  return FMOE_OK;
}

}  // extern "C"
