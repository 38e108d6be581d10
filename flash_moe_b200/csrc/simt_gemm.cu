// C[M, N] = A[M, K] * B[N, K]^T with fp32 FMA accumulation on the CUDA cores.
// Used where the tensor-core path does not apply: float32 modules (tcgen05 has no fp32-exact
// mode) and operand shapes TMA cannot address (K not a multiple of 8 elements).  Same fused
// epilogues as the tcgen05 kernels: plain store (+ optional fp32 addend) and SwiGLU.
#include "common.cuh"

namespace fmoe {
namespace {

constexpr int TM = 64, TN = 64, TK = 16;

template <typename T, bool SWIGLU>
__global__ void __launch_bounds__(256) simt_gemm_kernel(const T* __restrict__ A, int64_t lda, const T* __restrict__ B0,
                                                       const T* __restrict__ B1, int64_t ldb,
                                                       const float* __restrict__ addend,
                                                       const T* __restrict__ residual, T* __restrict__ out,
                                                       int64_t ldo, int M, int N, int K) {
  __shared__ float As[TK][TM + 4];
  __shared__ float Bs0[TK][TN + 4];
  __shared__ float Bs1[SWIGLU ? TK : 1][TN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  float acc0[4][4] = {}, acc1[4][4] = {};
  const int lr = tid >> 2;        // 0..63: row of the tile this thread stages
  const int lk = (tid & 3) * 4;   // 0,4,8,12
  for (int k0 = 0; k0 < K; k0 += TK) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int kk = k0 + lk + j;
      const int am = m0 + lr, bn = n0 + lr;
      As[lk + j][lr] = (am < M && kk < K) ? to_f32<T>(A[static_cast<int64_t>(am) * lda + kk]) : 0.f;
      Bs0[lk + j][lr] = (bn < N && kk < K) ? to_f32<T>(B0[static_cast<int64_t>(bn) * ldb + kk]) : 0.f;
      if (SWIGLU) Bs1[lk + j][lr] = (bn < N && kk < K) ? to_f32<T>(B1[static_cast<int64_t>(bn) * ldb + kk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < TK; ++k) {
      float a[4], b[4], c[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs0[k][tx * 4 + j];
      if (SWIGLU) {
#pragma unroll
        for (int j = 0; j < 4; ++j) c[j] = Bs1[k][tx * 4 + j];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc0[i][j] = fmaf(a[i], b[j], acc0[i][j]);
          if (SWIGLU) acc1[i][j] = fmaf(a[i], c[j], acc1[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v = acc0[i][j];
      if (SWIGLU) {
        v = (v / (1.0f + expf(-v))) * acc1[i][j];
      } else {
        if (addend != nullptr) v += addend[static_cast<int64_t>(m) * ldo + n];
        if (residual != nullptr) v += to_f32<T>(residual[static_cast<int64_t>(m) * ldo + n]);
      }
      out[static_cast<int64_t>(m) * ldo + n] = from_f32<T>(v);
    }
  }
}

template <typename T>
int run(const void* a, int64_t lda, const void* b0, const void* b1, const float* addend, void* out, int64_t ldo,
        int swiglu, int64_t M, int N, int K, cudaStream_t stream, const void* residual) {
  dim3 grid((N + TN - 1) / TN, static_cast<unsigned>((M + TM - 1) / TM));
  if (swiglu)
    simt_gemm_kernel<T, true><<<grid, 256, 0, stream>>>(static_cast<const T*>(a), lda, static_cast<const T*>(b0),
                                                        static_cast<const T*>(b1), K, nullptr, nullptr,
                                                        static_cast<T*>(out), ldo, static_cast<int>(M), N, K);
  else
    simt_gemm_kernel<T, false><<<grid, 256, 0, stream>>>(static_cast<const T*>(a), lda, static_cast<const T*>(b0),
                                                         nullptr, K, addend, static_cast<const T*>(residual),
                                                         static_cast<T*>(out), ldo, static_cast<int>(M), N, K);
  FMOE_LAUNCH_CHECK();
  return FMOE_OK;
}

}  // namespace

int launch_simt_gemm(const void* a, int64_t lda, const void* b0, const void* b1, const float* addend, void* out,
                     int64_t ldo, int dtype, int swiglu, int64_t M, int N, int K, cudaStream_t stream,
                     const void* residual) {
  if (a == nullptr || b0 == nullptr || out == nullptr || (swiglu && b1 == nullptr)) return FMOE_ERR_BAD_ARG;
  if (M <= 0 || N <= 0 || K <= 0 || M > 0x7FFFFFFFll - TM || (M + TM - 1) / TM > 65535) return FMOE_ERR_UNSUPPORTED;
  switch (dtype) {
    case FMOE_DTYPE_F32: return run<float>(a, lda, b0, b1, addend, out, ldo, swiglu, M, N, K, stream, residual);
    case FMOE_DTYPE_BF16: return run<__nv_bfloat16>(a, lda, b0, b1, addend, out, ldo, swiglu, M, N, K, stream, residual);
    case FMOE_DTYPE_F16: return run<__half>(a, lda, b0, b1, addend, out, ldo, swiglu, M, N, K, stream, residual);
    default: return FMOE_ERR_BAD_ARG;
  }
}

}  // namespace fmoe
