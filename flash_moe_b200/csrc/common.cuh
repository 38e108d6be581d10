// Shared helpers for the FlashMoE forward kernels (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "../../include/fmoe.h"

namespace fmoe {

#define FMOE_CUDA_TRY(expr)                         \
  do {                                              \
    cudaError_t _e = (expr);                        \
    if (_e != cudaSuccess) return -static_cast<int>(_e); \
  } while (0)

#define FMOE_LAUNCH_CHECK()                         \
  do {                                              \
    cudaError_t _e = cudaGetLastError();            \
    if (_e != cudaSuccess) return -static_cast<int>(_e); \
  } while (0)

inline int dtype_size(int dtype) { return dtype == FMOE_DTYPE_F32 ? 4 : 2; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
inline int next_pow2(int v) {
  int p = 1;
  while (p < v) p <<= 1;
  return p;
}

int device_sm_count();  // cached per device (api.cu)

// ---- programmatic dependent launch ----------------------------------------------------------
// The six kernels of a layer forward run back to back on one stream.  Launched with programmatic stream
// serialisation, a kernel's CTAs may become resident, and run their set-up (barrier init, tensor-map prefetch, tensor
// memory allocation, index tables), while the previous kernel is still draining; pdl_wait() then blocks until the
// previous kernel has finished and its writes are visible.  Rules every kernel launched through launch_pdl keeps:
// all threads call pdl_launch_dependents() first and pdl_wait() before their first access to global memory that is
// not a launch-time constant (weights are read by kernels only, so even those accesses sit behind the wait).  Because
// each kernel waits for its predecessor before it finishes, completion is transitive along the stream.
// FMOE_PDL=<bit mask of kernel classes> in the environment chooses which kernels get the attribute (0: none; the
// device-side instructions are no-ops without it).
// measured: the scores pass (4) is slower when it is made resident early - at the benchmark shape 215 vs 213 us per
// step, at 131072 tokens x 2048 columns 15.4 vs 13.4 ms per layer - so it keeps the plain stream order; the other four
// together give 211 vs 213 us in a graph and 214 vs 224 us launched eagerly
constexpr int kPdlDefaultMask = 27;
bool pdl_enabled(int kernel_class);  // api.cu; classes: 1 router GEMM, 2 top-k, 4 scores, 8 accumulate, 16 MLP GEMMs
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// cudaLaunchKernelEx with the programmatic-serialisation attribute (plus a cluster width when cluster_x > 1)
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(int kernel_class, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, int cluster_x, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  unsigned n = 0;
  if (cluster_x > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = static_cast<unsigned>(cluster_x);
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  if (pdl_enabled(kernel_class)) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// ---- scalar conversions -------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

// value after one rounding to T, as float
template <typename T> __device__ __forceinline__ float round_to(float v) { return to_f32<T>(from_f32<T>(v)); }

__device__ __forceinline__ float silu_f32(float v) { return __fdividef(v, 1.0f + __expf(-v)); }
// exact (erf) GELU, the activation of the PEER comparison op (flash_moe/ops/triton/peer.py:116-118)
__device__ __forceinline__ float gelu_f32(float v) { return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f)); }
enum ExpertAct { kActSilu = 0, kActGelu = 1 };
__device__ __forceinline__ float expert_act(float v, int act) { return act == kActGelu ? gelu_f32(v) : silu_f32(v); }

// ---- 16-byte vectors of T -----------------------------------------------------------------
template <typename T> struct Vec16 { static constexpr int N = 16 / sizeof(T); };

// unpack a 16-byte register quad into floats
template <typename T> __device__ __forceinline__ void unpack16(const uint4& q, float (&f)[Vec16<T>::N]);
template <> __device__ __forceinline__ void unpack16<float>(const uint4& q, float (&f)[4]) {
  f[0] = __uint_as_float(q.x); f[1] = __uint_as_float(q.y); f[2] = __uint_as_float(q.z); f[3] = __uint_as_float(q.w);
}
template <> __device__ __forceinline__ void unpack16<__nv_bfloat16>(const uint4& q, float (&f)[8]) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
template <> __device__ __forceinline__ void unpack16<__half>(const uint4& q, float (&f)[8]) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
    const float2 v = __half22float2(h);
    f[2 * i] = v.x; f[2 * i + 1] = v.y;
  }
}

template <typename T> __device__ __forceinline__ uint4 pack16(const float (&f)[Vec16<T>::N]);
template <> __device__ __forceinline__ uint4 pack16<float>(const float (&f)[4]) {
  return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
}
template <> __device__ __forceinline__ uint4 pack16<__nv_bfloat16>(const float (&f)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}
template <> __device__ __forceinline__ uint4 pack16<__half>(const float (&f)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

__device__ __forceinline__ uint4 ldg16(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

// ---- order-preserving float <-> uint32 map (larger float <=> larger unsigned) ---------------
__device__ __forceinline__ uint32_t f32_to_ord(float v) {
  const uint32_t b = __float_as_uint(v);
  return b ^ ((b >> 31) ? 0xFFFFFFFFu : 0x80000000u);
}
__device__ __forceinline__ float ord_to_f32(uint32_t u) {
  return __uint_as_float(u ^ ((u >> 31) ? 0x80000000u : 0xFFFFFFFFu));
}

// ---- internal launchers (one per .cu) -----------------------------------------------------
int launch_router_topk(const void* log_probs, int dtype, int64_t T, int nk, int k, void* scores, int64_t* indices,
                       void* gates, int norm, cudaStream_t stream);

size_t expert_workspace_bytes(int64_t T, int H, int64_t N, int k);
int launch_expert_forward(const void* x, const void* down, const void* up, const int64_t* indices, const void* gates,
                          void* out, int dtype, int out_dtype, int64_t T, int H, int64_t N, int k, void* ws,
                          size_t ws_bytes, int32_t* status, cudaStream_t stream, void* const* between_passes = nullptr,
                          int act = 0, float* raw_scores = nullptr);
// raw_scores (nullable) [T, k] float32 receives <x[t], down[e]> before the activation, for the backward pass.
// both steps in one kernel for 16-bit tables (expert_fused.cu): rows streamed through a shared-memory ring
bool expert_fused_supported(int dtype, int64_t T, int H, int k);
int launch_expert_fused(const void* x, const void* down, const void* up, const int64_t* idx, const void* gates,
                        void* out, int dtype, int out_f32, int64_t T, int H, int64_t N, int k, int act,
                        float* raw_scores, int32_t* status, cudaStream_t stream);
// the same sum with both tables sharded by e % world over the GPUs of a node; *_shards are DEVICE arrays of `world`
// row-0 pointers (peer pointers for the other GPUs); 16-bit dtypes only
// hot_down / hot_up (nullable): hot_rows rows replicated on every GPU, addressed by the ids N .. N + hot_rows - 1
int launch_expert_forward_peer(const void* x, const void* const* down_shards, const void* const* up_shards, int world,
                               const int64_t* indices, const void* gates, void* out, int dtype, int out_dtype, int64_t T,
                               int H, int64_t N, int k, void* ws, size_t ws_bytes, int32_t* status, cudaStream_t stream,
                               const void* hot_down = nullptr, const void* hot_up = nullptr, int64_t hot_rows = 0);
// out[t] = sum_j weights[t,j] * values[indices[t,j]] (the PKM comparison op)
int launch_weighted_rows(const void* values, const void* weights, const int64_t* indices, void* out, int dtype,
                         int64_t T, int H, int64_t N, int k, void* ws, size_t ws_bytes, int32_t* status,
                         cudaStream_t stream);
// between_passes (nullable): two cudaEvent_t handles (each nullable) recorded back to back after the scores pass
// and before the accumulate pass.

// C[M,N] = A[M,K] * B[N,K]^T on tcgen05 with a fused epilogue (gemm_sm100.cu); bf16/fp16 only.
int launch_gemm_swiglu(const void* x, const void* gate_w, const void* up_w, void* h, int dtype, int64_t M, int I, int K,
                       int32_t* status, cudaStream_t stream);
// residual (nullable): [M, N] in the module dtype, added to the float32 sum before the single rounding
int launch_gemm_add(const void* a, const void* b, const float* addend, void* out, int dtype, int64_t M, int N, int K,
                    int32_t* status, cudaStream_t stream, const void* residual = nullptr);
// router: per half h: logits[:, h*nk:(h+1)*nk] = A[:, h*a_half_koff : +K] * W[h*nk:(h+1)*nk, :K]^T, then log-softmax
int launch_gemm_router(const void* xn, int64_t a_cols, int a_half_koff, const void* w, void* logits, void* log_probs,
                       int dtype, int64_t M, int nk, int K, int32_t* status, cudaStream_t stream);
bool gemm_router_fused_supported(int nk);
// logits = T(batch_norm(x)) * W^T with the normalisation applied to the x tiles in shared memory (gemm_router_bn.cu)
bool router_bn_gemm_supported(int dtype, int64_t M, int N, int K);
int launch_router_bn_gemm(const void* x, const void* w, const float* mean, const float* invstd,
                          const void* running_mean, const void* running_var, float eps, void* logits, int dtype,
                          int64_t M, int N, int K, int32_t* status, cudaStream_t stream);
// CTA-pair (cta_group::2) versions of the two shared-MLP GEMMs (gemm_sm100_pair.cu)
bool gemm_pair_supported(int64_t M, int N, int K);
int launch_gemm_swiglu_pair(const void* x, const void* gate_w, const void* up_w, void* h, int dtype, int64_t M, int I,
                            int K, int32_t* status, cudaStream_t stream, void* pre_gate = nullptr,
                            void* pre_up = nullptr);
int launch_gemm_add_pair(const void* a, const void* b, const float* addend, void* out, int dtype, int64_t M, int N,
                         int K, int32_t* status, cudaStream_t stream, const void* residual = nullptr);

// fp32-FMA GEMM on CUDA cores (simt_gemm.cu): float32 modules and shapes TMA cannot address.
int launch_simt_gemm(const void* a, int64_t lda, const void* b0, const void* b1, const float* addend, void* out,
                     int64_t ldo, int dtype, int swiglu, int64_t M, int N, int K, cudaStream_t stream,
                     const void* residual = nullptr);

// elementwise.cu
int launch_log_softmax_halves(const void* logits, void* log_probs, int dtype, int64_t T, int nk, cudaStream_t stream);
size_t expert_backward_workspace_bytes(int64_t T, int H, int64_t N, int k);
int launch_expert_backward(const void* dout, const void* x, const void* down, const void* up, const int64_t* indices,
                           const void* gates, void* dx, void* ddown, void* dup, void* dgates, int dtype, int64_t T,
                           int H, int64_t N, int k, void* ws, size_t ws_bytes, int32_t* status, cudaStream_t stream,
                           const float* saved_scores = nullptr);
int launch_router_topk_backward(const void* dscores, const int64_t* indices, int dtype, int64_t T, int nk, int k,
                                void* dlog_probs, cudaStream_t stream);
int launch_swiglu_backward(const void* dh, const void* a, const void* b, void* da, void* db, void* h, int dtype,
                           int64_t n, cudaStream_t stream);
int launch_gather_probe(const void* table, int64_t num_rows, const int32_t* row_ids, int64_t count, int row_bytes,
                        int ctas_per_sm, int mode, float* sink, int32_t* status, cudaStream_t stream);
int launch_rms_norm(const void* x, const void* weight, void* out, int dtype, int64_t ntok, int H, float eps,
                    cudaStream_t stream);
int launch_combine_rows(const float* rows, int64_t num_rows, const int32_t* slot, int num_sources, int64_t ntok, int H,
                        float* out, int32_t* status, cudaStream_t stream);

}  // namespace fmoe
