// Router front end in one kernel for 16-bit modules on sm_100a:
//   logits[M, N] = T(batch_norm(x))[M, K] * W[N, K]^T          (flash_moe/modules/flash_moe.py:49,:65-66)
// The batch-norm (affine=False) is applied to the A tile in shared memory between its TMA arrival and the MMA, with
// the arithmetic and the rounding of the stand-alone normalisation pass (xn = T((x - mean) * inv_std), float32
// inside), so the logits are bit-equal to normalise-then-GEMM while x is read once and xn never exists in memory.
//
// One 128 x BLOCK_N tile per CTA, 320 threads:
//   warp 0 (one lane)  TMA producer: raw 128 x 64 x tile + BLOCK_N x 64 weight tile per stage, 128-byte swizzle;
//   warps 2..9         normalise the x tile in place (each thread owns 16-byte pieces of fixed features), make the
//                      writes visible to the tensor core (fence.proxy.async) and arrive on the stage's `ready`;
//   warp 1 (one lane)  waits for `ready`, issues tcgen05.mma into TMEM, frees the stage with tcgen05.commit;
//   warps 2..5         epilogue: tcgen05.ld the accumulator (one row per thread), round, store.
// Columns of x beyond K arrive as zeros from TMA and are normalised with mean 0 / scale 0, so they stay zero.
// Every wait is bounded; a wait that runs out raises FMOE_STATUS_WAIT_TIMEOUT and the CTA drains and leaves.
#include <cstdlib>

#include "gemm_epilogue.cuh"

namespace fmoe {
namespace {

constexpr int BLOCK_K = 64;
constexpr int UMMA_K = 16;
constexpr int kXformWarps = 8;
constexpr int kThreads = (2 + kXformWarps) * 32;
constexpr unsigned kFull = 0xFFFFFFFFu;

using epi::UmmaFmt;

__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ring depth: 6 x 24 KB or 6 x 32 KB stages for 128-column tiles, 4 x 48 KB for 256-column tiles.  Deeper does not
// help (8 stages measured the same): timestamps taken inside the kernel show the tiles landed and normalised well ahead
// of the MMA thread, which needs about 700 cycles per k-block (four tcgen05.mma of K = 16 and a commit) whether the
// tile has 64 or 128 rows - the issue pace of the MMAs, not the operand feed, sets the length of the main loop here.
template <int BLOCK_M, int BLOCK_N> struct RingDepth { static constexpr int v = BLOCK_N <= 128 ? 6 : 4; };

// BLOCK_M = 128, or 64 for small problems (twice the CTAs, half the x tile to fetch and normalise per CTA).  With
// M = 64 the accumulator's row i sits in TMEM lane 32 * (i / 16) + i % 16: each of the four epilogue warps finds 16
// rows in the first 16 lanes of its lane quarter.
template <int BLOCK_M, int BLOCK_N, typename T>
__global__ void __launch_bounds__(kThreads, 1)
router_gemm_bn_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const float* __restrict__ mean, const float* __restrict__ invstd,
                      const T* __restrict__ running_mean, const T* __restrict__ running_var, float eps, T* __restrict__ out,
                      int M, int N, int K, int num_m_tiles, int num_k_blocks, int32_t* status) {
  constexpr int A_BYTES = BLOCK_M * BLOCK_K * 2;
  constexpr int B_BYTES = BLOCK_N * BLOCK_K * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int kStages = RingDepth<BLOCK_M, BLOCK_N>::v;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_u32 = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw_u32 + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - raw_u32);
  const uint32_t bar_base = base + kStages * STAGE_BYTES;
  auto a_smem = [&](int s) { return base + s * STAGE_BYTES; };
  auto b_smem = [&](int s) { return base + s * STAGE_BYTES + A_BYTES; };
  auto full_bar = [&](int s) { return bar_base + s * 8; };
  auto ready_bar = [&](int s) { return bar_base + (kStages + s) * 8; };
  auto empty_bar = [&](int s) { return bar_base + (2 * kStages + s) * 8; };
  const uint32_t tfull_bar = bar_base + 3 * kStages * 8;
  uint8_t* gen_tail = gen + kStages * STAGE_BYTES + (3 * kStages + 1) * 8;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen_tail);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_tail + 8);
  float2* stats = reinterpret_cast<float2*>(gen_tail + 24);  // (mean, inv_std) per feature, padded to whole k-blocks; 16-byte aligned

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_tile = blockIdx.x % num_m_tiles;
  const int n_tile = blockIdx.x / num_m_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(ready_bar(s), kXformWarps / 2);  // one group of four warps normalises a k-block
      ptx::mbar_init(empty_bar(s), 1);
    }
    ptx::mbar_init(tfull_bar, 1);
    *abort_flag = 0;
    ptx::mbar_fence_init();
    ptx::prefetch_tensormap(&tmA);
    ptx::prefetch_tensormap(&tmB);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), BLOCK_N);
    ptx::tmem_relinquish();
  }
  // everything above is independent of earlier kernels; from here on global memory is read
  pdl_wait();
  // the first ring of operand tiles is requested before the statistics are fetched, so that the two cold reads overlap
  int kb_issued = 0;
  if (threadIdx.x == 0) {
    for (; kb_issued < kStages && kb_issued < num_k_blocks; ++kb_issued) {
      ptx::mbar_arrive_expect_tx(full_bar(kb_issued), STAGE_BYTES);
      ptx::tma_load_2d(a_smem(kb_issued), &tmA, full_bar(kb_issued), kb_issued * BLOCK_K, m_tile * BLOCK_M);
      ptx::tma_load_2d(b_smem(kb_issued), &tmB, full_bar(kb_issued), kb_issued * BLOCK_K, n_tile * BLOCK_N);
    }
  }
  // statistics: eval mode straight from the running buffers, training mode from the finalised batch statistics.
  // One thread fetches the eight features 8 p .. 8 p + 7 of a k-block with vector loads (all of a thread's loads are in
  // flight together: the buffers are cold, and fetching them one feature at a time took four DRAM round trips), and
  // writes them as four 16-byte entries: within a k-block the pairs (i, i + 1) of those eight features sit at
  // [i / 2][p], so the eight 16-byte reads a warp makes for one i cover 128 consecutive bytes instead of one bank group.
  const bool vec_stats = (running_mean != nullptr)
                             ? (sizeof(T) == 2 && ((reinterpret_cast<uintptr_t>(running_mean) | reinterpret_cast<uintptr_t>(running_var)) & 15u) == 0)
                             : (((reinterpret_cast<uintptr_t>(mean) | reinterpret_cast<uintptr_t>(invstd)) & 15u) == 0);
  for (int ch = threadIdx.x; ch < num_k_blocks * (BLOCK_K / 8); ch += kThreads) {
    const int c0 = ch * 8;
    float m[8], sd[8];
    if (vec_stats && c0 + 8 <= K) {
      if (running_mean != nullptr) {
        float v[8];
        unpack16<T>(ldg16(running_mean + c0), m);
        unpack16<T>(ldg16(running_var + c0), v);
#pragma unroll
        for (int i = 0; i < 8; ++i) sd[i] = 1.0f / sqrtf(v[i] + eps);
      } else {
        const float4 m0 = *reinterpret_cast<const float4*>(mean + c0), m1 = *reinterpret_cast<const float4*>(mean + c0 + 4);
        const float4 s0 = *reinterpret_cast<const float4*>(invstd + c0), s1 = *reinterpret_cast<const float4*>(invstd + c0 + 4);
        m[0] = m0.x; m[1] = m0.y; m[2] = m0.z; m[3] = m0.w; m[4] = m1.x; m[5] = m1.y; m[6] = m1.z; m[7] = m1.w;
        sd[0] = s0.x; sd[1] = s0.y; sd[2] = s0.z; sd[3] = s0.w; sd[4] = s1.x; sd[5] = s1.y; sd[6] = s1.z; sd[7] = s1.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int c = c0 + i;
        m[i] = 0.f;
        sd[i] = 0.f;
        if (c < K) {
          if (running_mean != nullptr) {
            m[i] = to_f32<T>(running_mean[c]);
            sd[i] = 1.0f / sqrtf(to_f32<T>(running_var[c]) + eps);
          } else {
            m[i] = mean[c];
            sd[i] = invstd[c];
          }
        }
      }
    }
    const int kb0 = (c0 / BLOCK_K) * BLOCK_K, pp = (c0 % BLOCK_K) >> 3;
#pragma unroll
    for (int j = 0; j < 4; ++j)
      *reinterpret_cast<float4*>(&stats[kb0 + j * 16 + pp * 2]) = make_float4(m[2 * j], sd[2 * j], m[2 * j + 1], sd[2 * j + 1]);
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int kb = kb_issued;
      bool ok = true;
      for (; kb < num_k_blocks; ++kb) {
        const int s = kb % kStages;
        const uint32_t ph = (kb / kStages) & 1u;
        if (!ptx::mbar_wait_bounded(empty_bar(s), ph ^ 1u, abort_flag)) { ok = false; break; }
        ptx::mbar_arrive_expect_tx(full_bar(s), STAGE_BYTES);
        ptx::tma_load_2d(a_smem(s), &tmA, full_bar(s), kb * BLOCK_K, m_tile * BLOCK_M);
        ptx::tma_load_2d(b_smem(s), &tmB, full_bar(s), kb * BLOCK_K, n_tile * BLOCK_N);
      }
      if (!ok) {  // let the copies already issued land before the CTA goes away (bounded)
        const int first = kb > kStages ? kb - kStages : 0;
        for (int j = first; j < kb; ++j)
          ptx::mbar_wait_drain(full_bar(j % kStages), (j / kStages) & 1u);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = (1u << 4) | (UmmaFmt<T>::v << 7) | (UmmaFmt<T>::v << 10) |
                                 (static_cast<uint32_t>(BLOCK_N >> 3) << 17) |
                                 (static_cast<uint32_t>(BLOCK_M >> 4) << 24);
      bool ok = true;
      for (int kb = 0; kb < num_k_blocks; ++kb) {
        const int s = kb % kStages;
        if (!ptx::mbar_wait_bounded(ready_bar(s), (kb / kStages) & 1u, abort_flag)) { ok = false; break; }
        ptx::tc_fence_after();
        const uint64_t da = ptx::umma_desc_kmajor_sw128(a_smem(s));
        const uint64_t db = ptx::umma_desc_kmajor_sw128(b_smem(s));
#pragma unroll
        for (int kk = 0; kk < BLOCK_K / UMMA_K; ++kk)
          ptx::umma_bf16_ss(tmem_base, da + 2 * kk, db + 2 * kk, idesc, (kb | kk) != 0 ? 1u : 0u);
        ptx::umma_commit(empty_bar(s));
      }
      if (ok) ptx::umma_commit(tfull_bar);
    }
  } else {
    // ------------------------------------------------------------ normalise the x tiles (warps 2..9)
    // Two groups of four warps take alternate k-blocks, so that two tiles are being normalised at any time (one
    // group's load -> arithmetic -> store -> proxy fence -> arrive chain took about 600 cycles per k-block and was the
    // pace of the whole kernel).  Thread i of a group owns the 16-byte pieces i, i + 128, ... of the BLOCK_M x
    // 128-byte tile: row (i >> 3) + 16 j, position i & 7.  With the 128-byte swizzle position p of row r holds the
    // features 8 * (p ^ (r & 7)) .. + 7 of the k-block, and r & 7 does not depend on j, so one thread always handles the
    // same eight features.
    constexpr int kGroupThreads = (kXformWarps / 2) * 32;
    constexpr int kGroupPieces = BLOCK_M * 8 / kGroupThreads;
    const int group = (warp - 2) / (kXformWarps / 2);
    const int xt = threadIdx.x - 64 - group * kGroupThreads;
    const int feat0 = 8 * ((xt & 7) ^ ((xt >> 3) & 7));
    bool ok = true;
    for (int kb = group; kb < num_k_blocks; kb += 2) {
      const int s = kb % kStages;
      float mm[8], ss[8];
#pragma unroll
      for (int i = 0; i < 8; i += 2) {
        const float4 v = *reinterpret_cast<const float4*>(&stats[kb * BLOCK_K + (i >> 1) * 16 + (feat0 >> 3) * 2]);
        mm[i] = v.x; ss[i] = v.y; mm[i + 1] = v.z; ss[i + 1] = v.w;
      }
      ok = ok && ptx::mbar_wait_bounded(full_bar(s), (kb / kStages) & 1u, abort_flag);
      uint4* tile = reinterpret_cast<uint4*>(gen + s * STAGE_BYTES);
      uint4 q[kGroupPieces];
#pragma unroll
      for (int j = 0; j < kGroupPieces; ++j) q[j] = tile[xt + kGroupThreads * j];
#pragma unroll
      for (int j = 0; j < kGroupPieces; ++j) {
        float f[8];
        unpack16<T>(q[j], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = (f[i] - mm[i]) * ss[i];
        tile[xt + kGroupThreads * j] = pack16<T>(f);
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(ready_bar(s));
    }

    if (warp < 6) {
      // ---------------------------------------------------------- epilogue (warps 2..5)
      const int q4 = warp & 3;  // TMEM lane quarter this warp may read
      bool done = ptx::mbar_wait_bounded(tfull_bar, 0u, abort_flag);
      done = __all_sync(kFull, done);
      if (done) {
        ptx::tc_fence_after();
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q4 * 32) << 16);
        constexpr int kRowsPerWarp = BLOCK_M / 4;  // 32, or 16 (the lower half of the warp's lanes) for M = 64
        const int64_t row = static_cast<int64_t>(m_tile) * BLOCK_M + q4 * kRowsPerWarp + lane;
        epi::store_add_row<T, BLOCK_N>(taddr, out + row * N, nullptr, nullptr, n_tile * BLOCK_N, N,
                                       lane < kRowsPerWarp && row < M);
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  __syncwarp();
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, BLOCK_N);
  }
  if (threadIdx.x == 0 && *abort_flag != 0 && status != nullptr) atomicOr(status, FMOE_STATUS_WAIT_TIMEOUT);
}

int make_map(CUtensorMap* m, const void* basep, int dtype, uint64_t cols, uint64_t rows, uint32_t box_rows) {
  return epi::make_tensor_map(m, basep, dtype, cols, rows, cols, box_rows);
}

template <int BLOCK_M, int BLOCK_N, typename T>
int launch_bn_gemm(const void* x, const void* w, const float* mean, const float* invstd, const void* rm, const void* rv,
                   float eps, void* out, int dtype, int64_t M, int N, int K, int32_t* status, cudaStream_t stream) {
  CUtensorMap tA, tB;
  int rc;
  if ((rc = make_map(&tA, x, dtype, K, M, BLOCK_M)) != FMOE_OK) return rc;
  if ((rc = make_map(&tB, w, dtype, K, N, BLOCK_N)) != FMOE_OK) return rc;
  const int num_k_blocks = (K + BLOCK_K - 1) / BLOCK_K;
  constexpr int kStages = RingDepth<BLOCK_M, BLOCK_N>::v;
  const int smem = kStages * (BLOCK_M * BLOCK_K * 2 + BLOCK_N * BLOCK_K * 2) + (3 * kStages + 1) * 8 + 24 + num_k_blocks * BLOCK_K * 8 + 1024;
  auto kern = router_gemm_bn_kernel<BLOCK_M, BLOCK_N, T>;
  FMOE_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  const int num_m_tiles = static_cast<int>((M + BLOCK_M - 1) / BLOCK_M);
  const int num_n_tiles = (N + BLOCK_N - 1) / BLOCK_N;
  FMOE_CUDA_TRY(launch_pdl(1, kern, dim3(num_m_tiles * num_n_tiles), dim3(kThreads), smem, stream, 1, tA, tB, mean, invstd,
                           static_cast<const T*>(rm), static_cast<const T*>(rv), eps, static_cast<T*>(out),
                           static_cast<int>(M), N, K, num_m_tiles, num_k_blocks, status));
  return FMOE_OK;
}

}  // namespace

// 16-bit dtypes, 16-byte aligned rows (K % 8, N % 8), K small enough for the statistics table beside the ring.
bool router_bn_gemm_supported(int dtype, int64_t M, int N, int K) {
  if (dtype != FMOE_DTYPE_BF16 && dtype != FMOE_DTYPE_F16) return false;
  return M > 0 && M < 0x7FFFFF00ll && N > 0 && K > 0 && K % 8 == 0 && N % 8 == 0 && K <= 3072;
}

// Statistics: running_mean / running_var (module dtype, eval mode) when non-null, else mean / invstd (float32 [K]).
int launch_router_bn_gemm(const void* x, const void* w, const float* mean, const float* invstd,
                          const void* running_mean, const void* running_var, float eps, void* logits, int dtype,
                          int64_t M, int N, int K, int32_t* status, cudaStream_t stream) {
  if (!router_bn_gemm_supported(dtype, M, N, K)) return FMOE_ERR_UNSUPPORTED;
  if (x == nullptr || w == nullptr || logits == nullptr) return FMOE_ERR_BAD_ARG;
  if ((running_mean == nullptr) != (running_var == nullptr)) return FMOE_ERR_BAD_ARG;
  if (running_mean == nullptr && (mean == nullptr || invstd == nullptr)) return FMOE_ERR_BAD_ARG;
  if (!aligned16(x) || !aligned16(w) || !aligned16(logits)) return FMOE_ERR_ALIGNMENT;
  // wide tiles once there are several waves of them: the x tile is then normalised once per 256 output columns
  const int64_t m_tiles = (M + 127) / 128;
  const int64_t tiles128 = m_tiles * ((N + 127) / 128);
  const bool wide = N > 128 && tiles128 >= 4 * static_cast<int64_t>(device_sm_count());
  // fewer 128 x 128 tiles than SMs: 64-row tiles put twice as many CTAs to work, each with half the x tile
  bool small = tiles128 < device_sm_count();
  if (const char* e = std::getenv("FMOE_BN_TILE")) small = e[0] == '6';  // measurement aid: 64 or 128 rows
#define FMOE_BN_GEMM(BM_, BN_)                                                                                       \
  (dtype == FMOE_DTYPE_BF16                                                                                          \
       ? launch_bn_gemm<BM_, BN_, __nv_bfloat16>(x, w, mean, invstd, running_mean, running_var, eps, logits, dtype, M, N, \
                                                 K, status, stream)                                                  \
       : launch_bn_gemm<BM_, BN_, __half>(x, w, mean, invstd, running_mean, running_var, eps, logits, dtype, M, N, K, \
                                          status, stream))
  if (wide) return FMOE_BN_GEMM(128, 256);
  if (small) return FMOE_BN_GEMM(64, 128);
  return FMOE_BN_GEMM(128, 128);
#undef FMOE_BN_GEMM
}

}  // namespace fmoe
