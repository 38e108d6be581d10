// Dense contractions of the FlashMoE forward on the 5th-generation tensor cores (sm_100a):
//   C[M, N] = A[M, K] * B[N, K]^T,  bf16/fp16 operands (both K-major), fp32 accumulate in TMEM.
//
// One persistent CTA per SM, 192 threads, warp-specialised:
//   warp 0 (one lane)  TMA producer: 128x64 A tile + BLOCK_N x 64 B tile per stage, 128-byte swizzle,
//                      mbarrier ring of STAGES slots;
//   warp 1 (one lane)  issues tcgen05.mma (128 x BLOCK_N x 16 per instruction) into one of two
//                      TMEM accumulators, frees smem slots / publishes accumulators via tcgen05.commit;
//   warps 2..5         epilogue: tcgen05.ld the finished accumulator (one row per thread) while the
//                      next tile's MMAs fill the other accumulator.
// Fused epilogues:
//   SWIGLU  B tile = 128 gate rows + 128 up rows of the same columns -> h = silu(g) * u   (bf16)
//   ADD     out = acc (+ fp32 addend), one rounding                                        (bf16)
//   ROUTER  one router half per N tile: logits rounded to the module dtype, then the per-half
//           log-softmax of those rounded logits (flash_moe/modules/flash_moe.py:65-72)
// Every mbarrier wait is bounded; on a timeout the CTA flags FMOE_STATUS_WAIT_TIMEOUT, drains and exits.
// (tcgen05.alloc itself blocks until tensor memory is free, i.e. until an earlier CTA on the SM has released it.)
// No cluster launch and no multicast: each CTA loads its own operands.
#include "gemm_epilogue.cuh"

namespace fmoe {
namespace {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_K = 64;  // 64 x 2 B = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int kThreads = 192;
constexpr unsigned kFull = 0xFFFFFFFFu;
constexpr int kSmemLimit = 227 * 1024;

enum { EPI_ADD = 0, EPI_SWIGLU = 1, EPI_ROUTER = 2 };

struct EpiParams {
  void* out;            // ADD: out[M, ldo]; SWIGLU: h[M, ldo]; ROUTER: logits[M, ldo]
  void* out2;           // ROUTER: log_probs[2, M, n_valid]
  const float* addend;  // ADD: optional fp32 [M, ldo]
  const void* residual; // ADD: optional [M, ldo] in the module dtype, added before the single rounding
  int64_t ldo;
  int n_valid;      // ADD: N; SWIGLU: I; ROUTER: num_keys
  int a_half_koff;  // ROUTER: K offset of half 1 inside a row of A
};

template <int BLOCK_N> struct Cfg {
  static constexpr int A_BYTES = BLOCK_M * BLOCK_K * 2;
  static constexpr int B_BYTES = BLOCK_N * BLOCK_K * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES_RAW = (kSmemLimit - 2048) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int TMEM_COLS = 2 * BLOCK_N < 32 ? 32 : 2 * BLOCK_N;
  static constexpr int BAR_BYTES = 256;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + BAR_BYTES + 1024;
};

using epi::UmmaFmt;

template <int BLOCK_N, int EPI, typename T>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB0,
                    const __grid_constant__ CUtensorMap tmB1, EpiParams ep, int M, int num_m_tiles, int num_n_tiles,
                    int num_k_blocks, int32_t* status) {
  using C = Cfg<BLOCK_N>;
  constexpr int STAGES = C::STAGES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_u32 = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw_u32 + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - raw_u32);
  const uint32_t bar_base = base + STAGES * C::STAGE_BYTES;
  auto a_smem = [&](int s) { return base + s * C::STAGE_BYTES; };
  auto b_smem = [&](int s) { return base + s * C::STAGE_BYTES + C::A_BYTES; };
  auto full_bar = [&](int s) { return bar_base + s * 8; };
  auto empty_bar = [&](int s) { return bar_base + (STAGES + s) * 8; };
  auto tfull_bar = [&](int a) { return bar_base + (2 * STAGES + a) * 8; };
  auto tempty_bar = [&](int a) { return bar_base + (2 * STAGES + 2 + a) * 8; };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + STAGES * C::STAGE_BYTES + (2 * STAGES + 4) * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + STAGES * C::STAGE_BYTES + (2 * STAGES + 4) * 8 + 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = num_m_tiles * num_n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(tfull_bar(a), 1);
      ptx::mbar_init(tempty_bar(a), 4);
    }
    *abort_flag = 0;
    ptx::mbar_fence_init();
    ptx::prefetch_tensormap(&tmA);
    ptx::prefetch_tensormap(&tmB0);
    if (EPI == EPI_SWIGLU) ptx::prefetch_tensormap(&tmB1);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), C::TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m_tile = tile % num_m_tiles;
        const int n_tile = tile / num_m_tiles;
        const int a_k0 = (EPI == EPI_ROUTER) ? n_tile * ep.a_half_koff : 0;
        for (int kb = 0; kb < num_k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!ptx::mbar_wait_bounded(empty_bar(s), ph ^ 1u, abort_flag)) { ok = false; break; }
          ptx::mbar_arrive_expect_tx(full_bar(s), C::STAGE_BYTES);
          ptx::tma_load_2d(a_smem(s), &tmA, full_bar(s), a_k0 + kb * BLOCK_K, m_tile * BLOCK_M);
          if (EPI == EPI_SWIGLU) {
            ptx::tma_load_2d(b_smem(s), &tmB0, full_bar(s), kb * BLOCK_K, n_tile * (BLOCK_N / 2));
            ptx::tma_load_2d(b_smem(s) + C::B_BYTES / 2, &tmB1, full_bar(s), kb * BLOCK_K, n_tile * (BLOCK_N / 2));
          } else if (EPI == EPI_ROUTER) {
            ptx::tma_load_2d(b_smem(s), &tmB0, full_bar(s), kb * BLOCK_K, n_tile * ep.n_valid);
          } else {
            ptx::tma_load_2d(b_smem(s), &tmB0, full_bar(s), kb * BLOCK_K, n_tile * BLOCK_N);
          }
        }
      }
      if (!ok) {
        // let the copies already issued land before the CTA goes away (bounded)
        const uint32_t first = it > static_cast<uint32_t>(STAGES) ? it - STAGES : 0u;
        for (uint32_t j = first; j < it; ++j)
          ptx::mbar_wait_drain(full_bar(j % STAGES), (j / STAGES) & 1u);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = (1u << 4) | (UmmaFmt<T>::v << 7) | (UmmaFmt<T>::v << 10) |
                                 (static_cast<uint32_t>(BLOCK_N >> 3) << 17) |
                                 (static_cast<uint32_t>(BLOCK_M >> 4) << 24);
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tcount) {
        const int acc = tcount & 1u;
        const uint32_t aph = (tcount >> 1) & 1u;
        if (!ptx::mbar_wait_bounded(tempty_bar(acc), aph ^ 1u, abort_flag)) { ok = false; break; }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BLOCK_N;
        for (int kb = 0; kb < num_k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!ptx::mbar_wait_bounded(full_bar(s), ph, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint64_t da = ptx::umma_desc_kmajor_sw128(a_smem(s));
          const uint64_t db = ptx::umma_desc_kmajor_sw128(b_smem(s));
#pragma unroll
          for (int kk = 0; kk < BLOCK_K / UMMA_K; ++kk) {
            // advance 16 elements = 32 B inside the swizzle row: +2 in 16-byte address units
            ptx::umma_bf16_ss(d_tmem, da + 2 * kk, db + 2 * kk, idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          ptx::umma_commit(empty_bar(s));
        }
        if (ok) ptx::umma_commit(tfull_bar(acc));
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const int row_in_tile = q * 32 + lane;
    uint32_t tcount = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++tcount) {
      const int m_tile = tile % num_m_tiles;
      const int n_tile = tile / num_m_tiles;
      const int acc = tcount & 1u;
      const uint32_t aph = (tcount >> 1) & 1u;
      bool ok = ptx::mbar_wait_bounded(tfull_bar(acc), aph, abort_flag);
      ok = __all_sync(kFull, ok);
      if (!ok) break;
      ptx::tc_fence_after();
      const uint32_t taddr = tmem_base + acc * BLOCK_N + (static_cast<uint32_t>(q * 32) << 16);
      const int64_t row = static_cast<int64_t>(m_tile) * BLOCK_M + row_in_tile;
      const bool row_ok = row < M;

      if constexpr (EPI == EPI_SWIGLU) {
        T* orow = static_cast<T*>(ep.out) + row * ep.ldo;
        epi::store_swiglu_row<T, BLOCK_N>(taddr, orow, nullptr, nullptr, n_tile * (BLOCK_N / 2), ep.n_valid, row_ok);
      } else if constexpr (EPI == EPI_ADD) {
        T* orow = static_cast<T*>(ep.out) + row * ep.ldo;
        const float* arow = (ep.addend != nullptr && row_ok) ? ep.addend + row * ep.ldo : nullptr;
        const T* rrow = (ep.residual != nullptr && row_ok) ? static_cast<const T*>(ep.residual) + row * ep.ldo : nullptr;
        epi::store_add_row<T, BLOCK_N>(taddr, orow, arow, rrow, n_tile * BLOCK_N, ep.n_valid, row_ok);
      } else {  // EPI_ROUTER: n_tile is the router half
        const int nk = ep.n_valid;
        const bool vec_ok = (nk % 8) == 0;
        T* lrow = static_cast<T*>(ep.out) + row * ep.ldo + static_cast<int64_t>(n_tile) * nk;
        T* prow = static_cast<T*>(ep.out2) + (static_cast<int64_t>(n_tile) * M + row) * nk;
        float vmax = -INFINITY;
#pragma unroll 1
        for (int c = 0; c < BLOCK_N / 32; ++c) {  // pass 1: round, store logits, row max
          uint32_t a[32];
          ptx::tmem_ld_32x32(taddr + c * 32, a);
          ptx::tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const int col = c * 32 + v * 8;
              float f[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                f[i] = round_to<T>(__uint_as_float(a[v * 8 + i]));
                if (col + i < nk) vmax = fmaxf(vmax, f[i]);
              }
              if (vec_ok) {
                if (col < nk) *reinterpret_cast<uint4*>(lrow + col) = pack16<T>(f);
              } else {
#pragma unroll
                for (int i = 0; i < 8; ++i)
                  if (col + i < nk) lrow[col + i] = from_f32<T>(f[i]);
              }
            }
          }
        }
        float vsum = 0.f;
#pragma unroll 1
        for (int c = 0; c < BLOCK_N / 32; ++c) {  // pass 2: sum of exp
          uint32_t a[32];
          ptx::tmem_ld_32x32(taddr + c * 32, a);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i < nk) vsum += expf(round_to<T>(__uint_as_float(a[i])) - vmax);
        }
        const float lsum = logf(vsum);
#pragma unroll 1
        for (int c = 0; c < BLOCK_N / 32; ++c) {  // pass 3: log-probabilities
          uint32_t a[32];
          ptx::tmem_ld_32x32(taddr + c * 32, a);
          ptx::tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const int col = c * 32 + v * 8;
              float f[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) f[i] = (round_to<T>(__uint_as_float(a[v * 8 + i])) - vmax) - lsum;
              if (vec_ok) {
                if (col < nk) *reinterpret_cast<uint4*>(prow + col) = pack16<T>(f);
              } else {
#pragma unroll
                for (int i = 0; i < 8; ++i)
                  if (col + i < nk) prow[col + i] = from_f32<T>(f[i]);
              }
            }
          }
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(tempty_bar(acc));
    }
  }

  // ---------------------------------------------------------------- teardown
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_flag != 0 && status != nullptr) atomicOr(status, FMOE_STATUS_WAIT_TIMEOUT);
}

// ------------------------------------------------------------------ host side
// 2-D K-major operand: `rows` rows of `cols` elements, row pitch `pitch` elements; box = 64 x box_rows.
int make_tmap(CUtensorMap* m, const void* basep, int dtype, uint64_t cols, uint64_t rows, uint64_t pitch,
              uint32_t box_rows) {
  return epi::make_tensor_map(m, basep, dtype, cols, rows, pitch, box_rows);
}

template <int BLOCK_N, int EPI, typename T>
int launch(const CUtensorMap& tA, const CUtensorMap& tB0, const CUtensorMap& tB1, const EpiParams& ep, int64_t M,
           int num_n_tiles, int K, int32_t* status, cudaStream_t stream) {
  using C = Cfg<BLOCK_N>;
  auto kern = gemm_tcgen05_kernel<BLOCK_N, EPI, T>;
  FMOE_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
  const int num_m_tiles = static_cast<int>((M + BLOCK_M - 1) / BLOCK_M);
  const int num_k_blocks = (K + BLOCK_K - 1) / BLOCK_K;
  const int64_t tiles = static_cast<int64_t>(num_m_tiles) * num_n_tiles;
  const int sms = device_sm_count();
  const int grid = static_cast<int>(tiles < sms ? tiles : sms);
  kern<<<grid, kThreads, C::SMEM_BYTES, stream>>>(tA, tB0, tB1, ep, static_cast<int>(M), num_m_tiles, num_n_tiles,
                                                  num_k_blocks, status);
  FMOE_LAUNCH_CHECK();
  return FMOE_OK;
}

int check_gemm_args(const void* a, const void* b, const void* out, int dtype, int64_t M, int K) {
  if (dtype != FMOE_DTYPE_BF16 && dtype != FMOE_DTYPE_F16) return FMOE_ERR_UNSUPPORTED;
  if (a == nullptr || b == nullptr || out == nullptr) return FMOE_ERR_BAD_ARG;
  if (M <= 0 || M > 0x7FFFFFFFll - BLOCK_M || K <= 0) return FMOE_ERR_BAD_ARG;
  if (K % 8 != 0) return FMOE_ERR_ALIGNMENT;
  if (!aligned16(a) || !aligned16(b) || !aligned16(out)) return FMOE_ERR_ALIGNMENT;
  return FMOE_OK;
}

}  // namespace

int launch_gemm_swiglu(const void* x, const void* gate_w, const void* up_w, void* h, int dtype, int64_t M, int I, int K,
                       int32_t* status, cudaStream_t stream) {
  int rc = check_gemm_args(x, gate_w, h, dtype, M, K);
  if (rc != FMOE_OK) return rc;
  if (up_w == nullptr || I <= 0) return FMOE_ERR_BAD_ARG;
  if (I % 8 != 0 || !aligned16(up_w)) return FMOE_ERR_ALIGNMENT;
  CUtensorMap tA, tG, tU;
  if ((rc = make_tmap(&tA, x, dtype, K, M, K, BLOCK_M)) != FMOE_OK) return rc;
  if ((rc = make_tmap(&tG, gate_w, dtype, K, I, K, 128)) != FMOE_OK) return rc;
  if ((rc = make_tmap(&tU, up_w, dtype, K, I, K, 128)) != FMOE_OK) return rc;
  EpiParams ep{h, nullptr, nullptr, nullptr, I, I, 0};
  const int n_tiles = (I + 127) / 128;
  if (dtype == FMOE_DTYPE_BF16)
    return launch<256, EPI_SWIGLU, __nv_bfloat16>(tA, tG, tU, ep, M, n_tiles, K, status, stream);
  return launch<256, EPI_SWIGLU, __half>(tA, tG, tU, ep, M, n_tiles, K, status, stream);
}

int launch_gemm_add(const void* a, const void* b, const float* addend, void* out, int dtype, int64_t M, int N, int K,
                    int32_t* status, cudaStream_t stream, const void* residual) {
  int rc = check_gemm_args(a, b, out, dtype, M, K);
  if (rc != FMOE_OK) return rc;
  if (N <= 0) return FMOE_ERR_BAD_ARG;
  if (N % 8 != 0 || (addend != nullptr && !aligned16(addend)) || (residual != nullptr && !aligned16(residual)))
    return FMOE_ERR_ALIGNMENT;
  CUtensorMap tA, tB;
  if ((rc = make_tmap(&tA, a, dtype, K, M, K, BLOCK_M)) != FMOE_OK) return rc;
  EpiParams ep{out, nullptr, addend, residual, N, N, 0};
  const int64_t m_tiles = (M + BLOCK_M - 1) / BLOCK_M;
  const bool wide = N > 128 && m_tiles * ((N + 255) / 256) * 2 > device_sm_count();
  if (wide) {
    if ((rc = make_tmap(&tB, b, dtype, K, N, K, 256)) != FMOE_OK) return rc;
    const int n_tiles = (N + 255) / 256;
    if (dtype == FMOE_DTYPE_BF16)
      return launch<256, EPI_ADD, __nv_bfloat16>(tA, tB, tB, ep, M, n_tiles, K, status, stream);
    return launch<256, EPI_ADD, __half>(tA, tB, tB, ep, M, n_tiles, K, status, stream);
  }
  if ((rc = make_tmap(&tB, b, dtype, K, N, K, 128)) != FMOE_OK) return rc;
  const int n_tiles = (N + 127) / 128;
  if (dtype == FMOE_DTYPE_BF16)
    return launch<128, EPI_ADD, __nv_bfloat16>(tA, tB, tB, ep, M, n_tiles, K, status, stream);
  return launch<128, EPI_ADD, __half>(tA, tB, tB, ep, M, n_tiles, K, status, stream);
}

bool gemm_router_fused_supported(int nk) { return nk >= 1 && nk <= 256; }

int launch_gemm_router(const void* xn, int64_t a_cols, int a_half_koff, const void* w, void* logits, void* log_probs,
                       int dtype, int64_t M, int nk, int K, int32_t* status, cudaStream_t stream) {
  int rc = check_gemm_args(xn, w, logits, dtype, M, K);
  if (rc != FMOE_OK) return rc;
  if (log_probs == nullptr || nk <= 0 || a_cols < K) return FMOE_ERR_BAD_ARG;
  if (!gemm_router_fused_supported(nk)) return FMOE_ERR_UNSUPPORTED;
  if (a_cols % 8 != 0 || a_half_koff % 8 != 0 || !aligned16(log_probs)) return FMOE_ERR_ALIGNMENT;
  const int bn = nk <= 32 ? 32 : nk <= 64 ? 64 : nk <= 128 ? 128 : 256;
  CUtensorMap tA, tB;
  if ((rc = make_tmap(&tA, xn, dtype, a_cols, M, a_cols, BLOCK_M)) != FMOE_OK) return rc;
  if ((rc = make_tmap(&tB, w, dtype, K, 2 * static_cast<uint64_t>(nk), K, bn)) != FMOE_OK) return rc;
  EpiParams ep{logits, log_probs, nullptr, nullptr, 2 * static_cast<int64_t>(nk), nk, a_half_koff};
#define FMOE_ROUTER_CASE(BN)                                                                               \
  case BN:                                                                                                 \
    if (dtype == FMOE_DTYPE_BF16)                                                                          \
      return launch<BN, EPI_ROUTER, __nv_bfloat16>(tA, tB, tB, ep, M, 2, K, status, stream);               \
    return launch<BN, EPI_ROUTER, __half>(tA, tB, tB, ep, M, 2, K, status, stream);
  switch (bn) {
    FMOE_ROUTER_CASE(32)
    FMOE_ROUTER_CASE(64)
    FMOE_ROUTER_CASE(128)
    FMOE_ROUTER_CASE(256)
  }
#undef FMOE_ROUTER_CASE
  return FMOE_ERR_UNSUPPORTED;
}

}  // namespace fmoe
