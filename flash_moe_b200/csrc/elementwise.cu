// Small memory-bound stages of the router front end:
//   batch-norm (affine=False) statistics / normalisation  (flash_moe/modules/flash_moe.py:49,:65)
//   per-half log-softmax of the router logits              (flash_moe/modules/flash_moe.py:72)
#include "common.cuh"

namespace fmoe {
namespace {

constexpr unsigned kFull = 0xFFFFFFFFu;
constexpr int kBnSplits = 32;  // row splits of the statistics pass (fixed => deterministic sums)

// partial[s][c] = sum over the rows of split s of x[r][c]; same for squares.
template <typename T>
__global__ void bn_partial_kernel(const T* __restrict__ x, int64_t ntok, int H, float* __restrict__ psum,
                                  float* __restrict__ psq) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int s = blockIdx.y;
  if (c >= H) return;
  const int64_t rows_per = (ntok + kBnSplits - 1) / kBnSplits;
  const int64_t r0 = s * rows_per;
  const int64_t r1 = r0 + rows_per < ntok ? r0 + rows_per : ntok;
  float a = 0.f, b = 0.f;
  for (int64_t r = r0; r < r1; ++r) {
    const float v = to_f32<T>(x[r * H + c]);
    a += v;
    b = fmaf(v, v, b);
  }
  psum[static_cast<int64_t>(s) * H + c] = a;
  psq[static_cast<int64_t>(s) * H + c] = b;
}

// mean / inverse std per feature.  Training: from the batch partials (biased variance) and the
// running buffers are updated (momentum, unbiased variance).  Eval: from the running buffers.
template <typename T>
__global__ void bn_finalize_kernel(const float* __restrict__ psum, const float* __restrict__ psq, T* running_mean,
                                   T* running_var, int training, float momentum, float eps, int64_t ntok, int H,
                                   float* __restrict__ mean_out, float* __restrict__ invstd_out,
                                   const float* __restrict__ global_sums) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float mean, var;
  if (training) {
    double s = 0.0, q = 0.0;
    if (global_sums != nullptr) {  // sums over ALL shards' rows (ntok is then the global row count)
      s = static_cast<double>(global_sums[c]);
      q = static_cast<double>(global_sums[H + c]);
    } else {
      for (int i = 0; i < kBnSplits; ++i) {
        s += static_cast<double>(psum[static_cast<int64_t>(i) * H + c]);
        q += static_cast<double>(psq[static_cast<int64_t>(i) * H + c]);
      }
    }
    const double m = s / static_cast<double>(ntok);
    double v = q / static_cast<double>(ntok) - m * m;
    if (v < 0.0) v = 0.0;
    mean = static_cast<float>(m);
    var = static_cast<float>(v);
    if (running_mean != nullptr && running_var != nullptr) {
      const double unbiased = ntok > 1 ? v * static_cast<double>(ntok) / static_cast<double>(ntok - 1) : v;
      const float rm = to_f32<T>(running_mean[c]);
      const float rv = to_f32<T>(running_var[c]);
      running_mean[c] = from_f32<T>((1.f - momentum) * rm + momentum * mean);
      running_var[c] = from_f32<T>((1.f - momentum) * rv + momentum * static_cast<float>(unbiased));
    }
  } else {
    mean = to_f32<T>(running_mean[c]);
    var = to_f32<T>(running_var[c]);
  }
  mean_out[c] = mean;
  invstd_out[c] = 1.0f / sqrtf(var + eps);
}

// sums[c] = sum_r x[r][c], sums[H + c] = sum_r x[r][c]^2 from the split partials (for the cross-rank all-reduce)
__global__ void bn_sums_kernel(const float* __restrict__ psum, const float* __restrict__ psq, int H,
                               float* __restrict__ sums) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  double s = 0.0, q = 0.0;
  for (int i = 0; i < kBnSplits; ++i) {
    s += static_cast<double>(psum[static_cast<int64_t>(i) * H + c]);
    q += static_cast<double>(psq[static_cast<int64_t>(i) * H + c]);
  }
  sums[c] = static_cast<float>(s);
  sums[H + c] = static_cast<float>(q);
}

// blockIdx.x / threadIdx.x pick a fixed group of VEC columns (mean / inv-std stay in registers),
// blockIdx.y strides over the rows; consecutive threads read consecutive 16-byte pieces of a row.
template <typename T>
__global__ void __launch_bounds__(128) bn_apply_kernel(const T* __restrict__ x, T* __restrict__ xn,
                                                      const float* __restrict__ mean,
                                                      const float* __restrict__ invstd,
                                                      const T* __restrict__ running_mean,
                                                      const T* __restrict__ running_var, float eps, int64_t ntok,
                                                      int H) {
  constexpr int VEC = Vec16<T>::N;
  const int cv = blockIdx.x * blockDim.x + threadIdx.x;
  if (cv * VEC >= H) return;
  float m[VEC], s[VEC];
#pragma unroll
  for (int j = 0; j < VEC; ++j) {
    if (running_mean != nullptr) {  // eval mode: statistics straight from the running buffers
      m[j] = to_f32<T>(running_mean[cv * VEC + j]);
      s[j] = 1.0f / sqrtf(to_f32<T>(running_var[cv * VEC + j]) + eps);
    } else {
      m[j] = mean[cv * VEC + j];
      s[j] = invstd[cv * VEC + j];
    }
  }
  constexpr int ROWS = 4;
  for (int64_t r0 = static_cast<int64_t>(blockIdx.y) * ROWS; r0 < ntok; r0 += static_cast<int64_t>(gridDim.y) * ROWS) {
    uint4 q[ROWS];
#pragma unroll
    for (int u = 0; u < ROWS; ++u)
      q[u] = (r0 + u < ntok) ? ldg16(x + (r0 + u) * H + cv * VEC) : make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int u = 0; u < ROWS; ++u) {
      if (r0 + u < ntok) {
        float f[VEC];
        unpack16<T>(q[u], f);
#pragma unroll
        for (int j = 0; j < VEC; ++j) f[j] = (f[j] - m[j]) * s[j];
        *reinterpret_cast<uint4*>(xn + (r0 + u) * H + cv * VEC) = pack16<T>(f);
      }
    }
  }
}

// one warp per (token, half): lp = (l - max) - log(sum exp(l - max)), rounded to T
template <typename T>
__global__ void log_softmax_halves_kernel(const T* __restrict__ logits, T* __restrict__ logp, int64_t ntok, int nk) {
  const int lane = threadIdx.x & 31;
  const int64_t warps_total = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  for (int64_t task = warp_global; task < 2 * ntok; task += warps_total) {
    const int64_t t = task >> 1;
    const int h = static_cast<int>(task & 1);
    const T* src = logits + t * 2 * nk + static_cast<int64_t>(h) * nk;
    T* dst = logp + (static_cast<int64_t>(h) * ntok + t) * nk;
    float vmax = -INFINITY;
    for (int i = lane; i < nk; i += 32) vmax = fmaxf(vmax, to_f32<T>(src[i]));
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) vmax = fmaxf(vmax, __shfl_xor_sync(kFull, vmax, d));
    float vsum = 0.f;
    for (int i = lane; i < nk; i += 32) vsum += expf(to_f32<T>(src[i]) - vmax);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) vsum += __shfl_xor_sync(kFull, vsum, d);
    const float lsum = logf(vsum);
    for (int i = lane; i < nk; i += 32) dst[i] = from_f32<T>((to_f32<T>(src[i]) - vmax) - lsum);
  }
}

template <typename T>
int bn_typed(const void* x, void* xn, void* rm, void* rv, int training, float momentum, float eps, int64_t ntok, int H,
             float* ws, const float* global_sums, int64_t global_count, cudaStream_t stream) {
  float* psum = ws;
  float* psq = ws + static_cast<size_t>(kBnSplits) * H;
  float* mean = psq + static_cast<size_t>(kBnSplits) * H;
  float* invstd = mean + H;
  if (training && global_sums == nullptr) {
    dim3 grid((H + 127) / 128, kBnSplits);
    bn_partial_kernel<T><<<grid, 128, 0, stream>>>(static_cast<const T*>(x), ntok, H, psum, psq);
    FMOE_LAUNCH_CHECK();
  }
  if (training) {
    bn_finalize_kernel<T><<<(H + 127) / 128, 128, 0, stream>>>(
        psum, psq, static_cast<T*>(rm), static_cast<T*>(rv), training, momentum, eps,
        global_sums != nullptr ? global_count : ntok, H, mean, invstd, global_sums);
    FMOE_LAUNCH_CHECK();
  }
  if (xn == nullptr) return FMOE_OK;  // statistics only: the caller normalises inside its GEMM
  constexpr int VEC = Vec16<T>::N;
  const int hv = H / VEC;
  const int gx = (hv + 127) / 128;
  int64_t gy = (ntok + 3) / 4;
  const int64_t cap = static_cast<int64_t>(device_sm_count()) * 16 / gx;
  if (gy > cap) gy = cap > 0 ? cap : 1;
  if (gy > 65535) gy = 65535;
  bn_apply_kernel<T><<<dim3(gx, static_cast<unsigned>(gy)), 128, 0, stream>>>(
      static_cast<const T*>(x), static_cast<T*>(xn), mean, invstd, training ? nullptr : static_cast<const T*>(rm),
      training ? nullptr : static_cast<const T*>(rv), eps, ntok, H);
  FMOE_LAUNCH_CHECK();
  return FMOE_OK;
}

// RMS pre-norm of a decoder block in front of the layer: out[r] = T(x[r] * rsqrt(mean(x[r]^2) + eps) * weight).
// One warp per row, float32 inside, one rounding; 16-byte loads and stores.
template <typename T>
__global__ void __launch_bounds__(256) rms_norm_kernel(const T* __restrict__ x, const T* __restrict__ weight,
                                                      T* __restrict__ out, int64_t ntok, int H, float eps) {
  constexpr int VEC = Vec16<T>::N;
  const int lane = threadIdx.x & 31;
  const int64_t warps_total = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  for (int64_t r = warp_global; r < ntok; r += warps_total) {
    const T* xr = x + r * H;
    float ss = 0.f;
    for (int c = lane * VEC; c < H; c += 32 * VEC) {
      float f[VEC];
      unpack16<T>(ldg16(xr + c), f);
#pragma unroll
      for (int i = 0; i < VEC; ++i) ss = fmaf(f[i], f[i], ss);
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) ss += __shfl_xor_sync(kFull, ss, d);
    const float scale = rsqrtf(ss / static_cast<float>(H) + eps);
    for (int c = lane * VEC; c < H; c += 32 * VEC) {
      float f[VEC], w[VEC];
      unpack16<T>(ldg16(xr + c), f);
      if (weight != nullptr) unpack16<T>(ldg16(weight + c), w);
#pragma unroll
      for (int i = 0; i < VEC; ++i) f[i] = f[i] * scale * (weight != nullptr ? w[i] : 1.0f);
      *reinterpret_cast<uint4*>(out + r * H + c) = pack16<T>(f);
    }
  }
}

// out[t] = sum over sources g of rows[slot[g * ntok + t]] (slot < 0: source g holds nothing for token t).
// One thread per 16 bytes of an output row; sources are added in ascending g, so the sum is reproducible.
__global__ void __launch_bounds__(256) combine_rows_kernel(const float4* __restrict__ rows, int64_t num_rows,
                                                           const int32_t* __restrict__ slot, int num_sources,
                                                           int64_t ntok, int h4, float4* __restrict__ out,
                                                           int32_t* status) {
  const int64_t total = ntok * h4;
  bool bad = false;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t t = i / h4;
    const int c = static_cast<int>(i - t * h4);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int g = 0; g < num_sources; ++g) {
      const int64_t r = slot[static_cast<int64_t>(g) * ntok + t];
      if (r < 0) continue;
      if (r >= num_rows) {
        bad = true;
        continue;
      }
      const float4 v = __ldg(rows + r * h4 + c);
      acc.x += v.x;
      acc.y += v.y;
      acc.z += v.z;
      acc.w += v.w;
    }
    out[i] = acc;
  }
  if (bad && status != nullptr) atomicOr(status, FMOE_STATUS_BAD_ROW_INDEX);
}

}  // namespace

size_t bn_workspace_bytes(int H) { return static_cast<size_t>(2 * kBnSplits + 2) * H * sizeof(float); }

// where launch_bn leaves the per-feature mean and inverse standard deviation of a training-mode batch (float32 [H])
void bn_stats_in_workspace(float* ws, int H, const float** mean, const float** invstd) {
  *mean = ws + static_cast<size_t>(2 * kBnSplits) * H;
  *invstd = *mean + H;
}

// per-feature sum and sum of squares of this rank's rows: sums[0:H], sums[H:2H] (float32)
int launch_bn_sums(const void* x, int dtype, int64_t ntok, int H, float* ws, float* sums, cudaStream_t stream) {
  if (x == nullptr || ws == nullptr || sums == nullptr || ntok <= 0 || H <= 0) return FMOE_ERR_BAD_ARG;
  float* psum = ws;
  float* psq = ws + static_cast<size_t>(kBnSplits) * H;
  dim3 grid((H + 127) / 128, kBnSplits);
  switch (dtype) {
    case FMOE_DTYPE_F32: bn_partial_kernel<float><<<grid, 128, 0, stream>>>(static_cast<const float*>(x), ntok, H, psum, psq); break;
    case FMOE_DTYPE_BF16: bn_partial_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), ntok, H, psum, psq); break;
    case FMOE_DTYPE_F16: bn_partial_kernel<__half><<<grid, 128, 0, stream>>>(static_cast<const __half*>(x), ntok, H, psum, psq); break;
    default: return FMOE_ERR_BAD_ARG;
  }
  FMOE_LAUNCH_CHECK();
  bn_sums_kernel<<<(H + 127) / 128, 128, 0, stream>>>(psum, psq, H, sums);
  FMOE_LAUNCH_CHECK();
  return FMOE_OK;
}

int launch_bn(const void* x, void* xn, void* running_mean, void* running_var, int training, float momentum, float eps,
              int dtype, int64_t ntok, int H, float* ws, const float* global_sums, int64_t global_count,
              cudaStream_t stream) {
  if (x == nullptr || ws == nullptr || ntok <= 0 || H <= 0) return FMOE_ERR_BAD_ARG;
  if (!training && (running_mean == nullptr || running_var == nullptr)) return FMOE_ERR_BAD_ARG;
  if (H % (16 / dtype_size(dtype)) != 0 || !aligned16(x) || (xn != nullptr && !aligned16(xn))) return FMOE_ERR_ALIGNMENT;
  switch (dtype) {
    case FMOE_DTYPE_F32: return bn_typed<float>(x, xn, running_mean, running_var, training, momentum, eps, ntok, H, ws, global_sums, global_count, stream);
    case FMOE_DTYPE_BF16: return bn_typed<__nv_bfloat16>(x, xn, running_mean, running_var, training, momentum, eps, ntok, H, ws, global_sums, global_count, stream);
    case FMOE_DTYPE_F16: return bn_typed<__half>(x, xn, running_mean, running_var, training, momentum, eps, ntok, H, ws, global_sums, global_count, stream);
    default: return FMOE_ERR_BAD_ARG;
  }
}

int launch_log_softmax_halves(const void* logits, void* log_probs, int dtype, int64_t ntok, int nk,
                              cudaStream_t stream) {
  if (logits == nullptr || log_probs == nullptr || ntok <= 0 || nk <= 0) return FMOE_ERR_BAD_ARG;
  const int64_t want = (2 * ntok + 7) / 8;
  const int64_t cap = static_cast<int64_t>(device_sm_count()) * 8;
  const int grid = static_cast<int>(want < cap ? want : cap);
  switch (dtype) {
    case FMOE_DTYPE_F32:
      log_softmax_halves_kernel<float><<<grid, 256, 0, stream>>>(static_cast<const float*>(logits), static_cast<float*>(log_probs), ntok, nk);
      break;
    case FMOE_DTYPE_BF16:
      log_softmax_halves_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(logits), static_cast<__nv_bfloat16*>(log_probs), ntok, nk);
      break;
    case FMOE_DTYPE_F16:
      log_softmax_halves_kernel<__half><<<grid, 256, 0, stream>>>(static_cast<const __half*>(logits), static_cast<__half*>(log_probs), ntok, nk);
      break;
    default: return FMOE_ERR_BAD_ARG;
  }
  FMOE_LAUNCH_CHECK();
  return FMOE_OK;
}

int launch_rms_norm(const void* x, const void* weight, void* out, int dtype, int64_t ntok, int H, float eps,
                    cudaStream_t stream) {
  if (ntok < 0 || H <= 0 || !(eps >= 0.f)) return FMOE_ERR_BAD_ARG;
  if (ntok == 0) return FMOE_OK;
  if (x == nullptr || out == nullptr) return FMOE_ERR_BAD_ARG;
  if (H % (16 / dtype_size(dtype)) != 0 || !aligned16(x) || !aligned16(out) || (weight != nullptr && !aligned16(weight)))
    return FMOE_ERR_ALIGNMENT;
  const int64_t want = (ntok + 7) / 8;
  const int64_t cap = static_cast<int64_t>(device_sm_count()) * 8;
  const int grid = static_cast<int>(want < cap ? want : cap);
  switch (dtype) {
    case FMOE_DTYPE_F32:
      rms_norm_kernel<float><<<grid, 256, 0, stream>>>(static_cast<const float*>(x), static_cast<const float*>(weight),
                                                       static_cast<float*>(out), ntok, H, eps);
      break;
    case FMOE_DTYPE_BF16:
      rms_norm_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x),
                                                               static_cast<const __nv_bfloat16*>(weight),
                                                               static_cast<__nv_bfloat16*>(out), ntok, H, eps);
      break;
    case FMOE_DTYPE_F16:
      rms_norm_kernel<__half><<<grid, 256, 0, stream>>>(static_cast<const __half*>(x), static_cast<const __half*>(weight),
                                                        static_cast<__half*>(out), ntok, H, eps);
      break;
    default: return FMOE_ERR_BAD_ARG;
  }
  FMOE_LAUNCH_CHECK();
  return FMOE_OK;
}

int launch_combine_rows(const float* rows, int64_t num_rows, const int32_t* slot, int num_sources, int64_t ntok, int H,
                        float* out, int32_t* status, cudaStream_t stream) {
  if (num_rows < 0 || num_sources < 0 || ntok < 0 || H <= 0) return FMOE_ERR_BAD_ARG;
  if (ntok == 0) return FMOE_OK;
  if (out == nullptr || (num_sources > 0 && slot == nullptr) || (num_rows > 0 && rows == nullptr)) return FMOE_ERR_BAD_ARG;
  if (H % 4 != 0 || !aligned16(rows) || !aligned16(out)) return FMOE_ERR_ALIGNMENT;
  const int h4 = H / 4;
  const int64_t want = (ntok * h4 + 255) / 256;
  const int64_t cap = static_cast<int64_t>(device_sm_count()) * 16;
  const int grid = static_cast<int>(want < cap ? want : cap);
  combine_rows_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const float4*>(rows), num_rows, slot, num_sources, ntok,
                                                h4, reinterpret_cast<float4*>(out), status);
  FMOE_LAUNCH_CHECK();
  return FMOE_OK;
}

}  // namespace fmoe
