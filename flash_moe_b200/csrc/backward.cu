// Backward kernels of the router op and of the SwiGLU activation (sm_100a).  The expert op's backward lives
// with its forward in expert.cu.
#include "common.cuh"

namespace fmoe {
namespace {

// d log_probs[h, t, c] = sum over the token's selected slots j whose sub-key of half h is c of dscores[t, j]
// (flash_moe/ops/triton/flash_router.py:197-249 scatters with atomics in the gradient's dtype; here every
// output element is a float32 sum over the slots in ascending j, rounded once).
template <typename T>
__global__ void __launch_bounds__(128) router_bwd_kernel(const T* __restrict__ dscores, const int64_t* __restrict__ idx,
                                                         T* __restrict__ dlogp, int64_t ntok, int nk, int k) {
  extern __shared__ unsigned char smem_raw[];
  float* ds = reinterpret_cast<float*>(smem_raw);  // [k]
  int* ix = reinterpret_cast<int*>(ds + k);        // [k]
  int* iy = ix + k;                                // [k]
  for (int64_t t = blockIdx.x; t < ntok; t += gridDim.x) {
    __syncthreads();
    for (int j = threadIdx.x; j < k; j += blockDim.x) {
      const int64_t e = idx[t * k + j];
      const bool ok = e >= 0 && e < static_cast<int64_t>(nk) * nk;
      ds[j] = ok ? to_f32<T>(dscores[t * k + j]) : 0.f;
      ix[j] = ok ? static_cast<int>(e / nk) : -1;
      iy[j] = ok ? static_cast<int>(e % nk) : -1;
    }
    __syncthreads();
    for (int c = threadIdx.x; c < 2 * nk; c += blockDim.x) {
      const int half = c >= nk ? 1 : 0;
      const int key = c - half * nk;
      const int* sel = half ? iy : ix;
      float acc = 0.f;
      for (int j = 0; j < k; ++j)
        if (sel[j] == key) acc += ds[j];
      dlogp[(static_cast<int64_t>(half) * ntok + t) * nk + key] = from_f32<T>(acc);
    }
  }
}

// h = silu(a) * b;  da = dh * b * silu'(a);  db = dh * silu(a)   (flash_moe/ops/triton/flash_mlp.py:52-102)
template <typename T>
__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const T* __restrict__ dh, const T* __restrict__ a,
                                                         const T* __restrict__ b, T* __restrict__ da,
                                                         T* __restrict__ db, T* __restrict__ h, int64_t nvec) {
  constexpr int VEC = Vec16<T>::N;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    float fd[VEC], fa[VEC], fb[VEC], oa[VEC], ob[VEC], oh[VEC];
    unpack16<T>(ldg16(dh + i * VEC), fd);
    unpack16<T>(ldg16(a + i * VEC), fa);
    unpack16<T>(ldg16(b + i * VEC), fb);
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      const float sig = __fdividef(1.0f, 1.0f + __expf(-fa[j]));
      const float act = fa[j] * sig;
      oa[j] = fd[j] * fb[j] * (sig * (1.0f + fa[j] * (1.0f - sig)));
      ob[j] = fd[j] * act;
      oh[j] = act * fb[j];
    }
    *reinterpret_cast<uint4*>(da + i * VEC) = pack16<T>(oa);
    *reinterpret_cast<uint4*>(db + i * VEC) = pack16<T>(ob);
    if (h != nullptr) *reinterpret_cast<uint4*>(h + i * VEC) = pack16<T>(oh);
  }
}

template <typename T>
int router_bwd_typed(const void* dscores, const int64_t* idx, void* dlogp, int64_t ntok, int nk, int k,
                     cudaStream_t stream) {
  const size_t smem = static_cast<size_t>(k) * 12;
  auto kern = router_bwd_kernel<T>;
  if (smem > 48 * 1024) FMOE_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  const int64_t cap = static_cast<int64_t>(device_sm_count()) * 16;
  const int grid = static_cast<int>(ntok < cap ? ntok : cap);
  kern<<<grid, 128, smem, stream>>>(static_cast<const T*>(dscores), idx, static_cast<T*>(dlogp), ntok, nk, k);
  FMOE_LAUNCH_CHECK();
  return FMOE_OK;
}

template <typename T>
int swiglu_bwd_typed(const void* dh, const void* a, const void* b, void* da, void* db, void* h, int64_t n,
                     cudaStream_t stream) {
  constexpr int VEC = Vec16<T>::N;
  const int64_t nvec = n / VEC;
  const int64_t want = (nvec + 255) / 256;
  const int64_t cap = static_cast<int64_t>(device_sm_count()) * 16;
  const int grid = static_cast<int>(want < cap ? want : cap);
  swiglu_bwd_kernel<T><<<grid, 256, 0, stream>>>(static_cast<const T*>(dh), static_cast<const T*>(a),
                                                 static_cast<const T*>(b), static_cast<T*>(da), static_cast<T*>(db),
                                                 static_cast<T*>(h), nvec);
  FMOE_LAUNCH_CHECK();
  return FMOE_OK;
}

}  // namespace

int launch_router_topk_backward(const void* dscores, const int64_t* indices, int dtype, int64_t T, int nk, int k,
                                void* dlog_probs, cudaStream_t stream) {
  if (T < 0 || nk <= 0 || k < 0 || k > nk) return FMOE_ERR_BAD_ARG;
  if (T == 0) return FMOE_OK;
  if (dlog_probs == nullptr || (k > 0 && (dscores == nullptr || indices == nullptr))) return FMOE_ERR_BAD_ARG;
  if (static_cast<size_t>(k) * 12 > 200 * 1024) return FMOE_ERR_UNSUPPORTED;
  switch (dtype) {
    case FMOE_DTYPE_F32: return router_bwd_typed<float>(dscores, indices, dlog_probs, T, nk, k, stream);
    case FMOE_DTYPE_BF16: return router_bwd_typed<__nv_bfloat16>(dscores, indices, dlog_probs, T, nk, k, stream);
    case FMOE_DTYPE_F16: return router_bwd_typed<__half>(dscores, indices, dlog_probs, T, nk, k, stream);
    default: return FMOE_ERR_BAD_ARG;
  }
}

int launch_swiglu_backward(const void* dh, const void* a, const void* b, void* da, void* db, void* h, int dtype,
                           int64_t n, cudaStream_t stream) {
  if (dtype != FMOE_DTYPE_F32 && dtype != FMOE_DTYPE_BF16 && dtype != FMOE_DTYPE_F16) return FMOE_ERR_BAD_ARG;
  if (n < 0) return FMOE_ERR_BAD_ARG;
  if (n == 0) return FMOE_OK;
  if (dh == nullptr || a == nullptr || b == nullptr || da == nullptr || db == nullptr) return FMOE_ERR_BAD_ARG;
  if (n % (16 / dtype_size(dtype)) != 0) return FMOE_ERR_ALIGNMENT;
  if (!aligned16(dh) || !aligned16(a) || !aligned16(b) || !aligned16(da) || !aligned16(db) || !aligned16(h))
    return FMOE_ERR_ALIGNMENT;
  switch (dtype) {
    case FMOE_DTYPE_F32: return swiglu_bwd_typed<float>(dh, a, b, da, db, h, n, stream);
    case FMOE_DTYPE_BF16: return swiglu_bwd_typed<__nv_bfloat16>(dh, a, b, da, db, h, n, stream);
    case FMOE_DTYPE_F16: return swiglu_bwd_typed<__half>(dh, a, b, da, db, h, n, stream);
    default: return FMOE_ERR_BAD_ARG;
  }
}

}  // namespace fmoe
