// CTA-pair tcgen05 GEMM for the two shared-MLP contractions:
//   C[M, N] = A[M, K] * B[N, K]^T, bf16/fp16, fp32 accumulate in TMEM, 256 x 256 tile per CTA pair.
//
// Why pairs: the single-CTA kernel feeds 48 KB per 128x256x64 MMA block from L2 (96 B/clk per SM at
// full tensor rate); its 4-stage ring cannot cover the L2 latency at that rate and the tensor pipe
// idles a third of the time.  With tcgen05 cta_group::2 the two CTAs of a 2-CTA cluster share one
// 256-row MMA: each loads its own 128 rows of A and only HALF of the B tile (its 128 of the 256 N
// rows), i.e. 32 KB per block and six stages in the same shared memory.
//
// Protocol (rank 0 = leader):
//   * both producers wait on their own `empty` barrier and issue their TMA loads; the byte counts
//     of both CTAs land on the LEADER's `full` barrier (armed with twice the per-CTA bytes);
//   * the leader's MMA thread issues the pair MMAs and commits to `empty` in both CTAs and, after
//     the last k-block, to `tmem_full` in both CTAs;
//   * each CTA's epilogue warps drain their own 128 accumulator rows and arrive on the leader's
//     `tmem_empty` barrier (8 arrivals);
//   * cluster barriers bracket set-up and tear-down so no CTA touches a peer that is not there.
// No multicast loads anywhere; every wait is bounded like in the single-CTA kernel.
#include <cuda.h>

#include "common.cuh"
#include "ptx_sm100.cuh"

namespace fmoe {
namespace {

constexpr int BLOCK_M = 128;  // rows per CTA; the pair covers 256
constexpr int BLOCK_N = 256;
constexpr int BLOCK_K = 64;
constexpr int UMMA_K = 16;
constexpr int kThreads = 192;
constexpr unsigned kFull = 0xFFFFFFFFu;
constexpr int A_BYTES = BLOCK_M * BLOCK_K * 2;
constexpr int B_BYTES = (BLOCK_N / 2) * BLOCK_K * 2;  // this CTA's half of the B tile
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;        // 32 KB
constexpr int STAGES = 6;
constexpr int TMEM_COLS = 512;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 256 + 1024;

enum { PAIR_EPI_ADD = 0, PAIR_EPI_SWIGLU = 1 };

struct PairEpi {
  void* out;
  const float* addend;
  int64_t ldo;
  int n_valid;
  void* pre_gate;  // SWIGLU only, nullable: x Wg^T and x Wu^T rounded to T, kept for the backward pass
  void* pre_up;
};

template <typename T> struct UmmaFmt;
template <> struct UmmaFmt<__nv_bfloat16> { static constexpr uint32_t v = 1; };
template <> struct UmmaFmt<__half> { static constexpr uint32_t v = 0; };

template <int EPI, typename T>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB0,
                         const __grid_constant__ CUtensorMap tmB1, PairEpi ep, int M, int num_m_tiles, int num_n_tiles,
                         int num_k_blocks, int32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_u32 = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw_u32 + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - raw_u32);
  const uint32_t bar_base = base + STAGES * STAGE_BYTES;
  auto a_smem = [&](int s) { return base + s * STAGE_BYTES; };
  auto b_smem = [&](int s) { return base + s * STAGE_BYTES + A_BYTES; };
  auto full_bar = [&](int s) { return bar_base + s * 8; };
  auto empty_bar = [&](int s) { return bar_base + (STAGES + s) * 8; };
  auto tfull_bar = [&](int a) { return bar_base + (2 * STAGES + a) * 8; };
  auto tempty_bar = [&](int a) { return bar_base + (2 * STAGES + 2 + a) * 8; };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + STAGES * STAGE_BYTES + (2 * STAGES + 4) * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + STAGES * STAGE_BYTES + (2 * STAGES + 4) * 8 + 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();
  const int pair = blockIdx.x >> 1;
  const int npairs = gridDim.x >> 1;
  const int num_tiles = num_m_tiles * num_n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(full_bar(s), 1);   // leader only is used: its producer's arrive + bytes of both CTAs
      ptx::mbar_init(empty_bar(s), 1);  // one commit per use
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(tfull_bar(a), 1);
      ptx::mbar_init(tempty_bar(a), 8);  // leader only is used: 4 epilogue warps of each CTA
    }
    *abort_flag = 0;
    ptx::mbar_fence_init();
    ptx::prefetch_tensormap(&tmA);
    ptx::prefetch_tensormap(&tmB0);
    if (EPI == PAIR_EPI_SWIGLU) ptx::prefetch_tensormap(&tmB1);
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before();
  ptx::cluster_sync();  // barriers of both CTAs are initialised before anyone signals them
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += npairs) {
        const int m_tile = tile % num_m_tiles;
        const int n_tile = tile / num_m_tiles;
        const int a_row = m_tile * (2 * BLOCK_M) + static_cast<int>(rank) * BLOCK_M;
        for (int kb = 0; kb < num_k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!ptx::mbar_wait_bounded(empty_bar(s), ph ^ 1u, abort_flag)) { ok = false; break; }
          if (rank == 0) ptx::mbar_arrive_expect_tx(full_bar(s), 2 * STAGE_BYTES);
          const uint32_t leader_full = ptx::map_to_cta(full_bar(s), 0);
          ptx::tma_load_2d_pair(a_smem(s), &tmA, leader_full, kb * BLOCK_K, a_row);
          if (EPI == PAIR_EPI_SWIGLU) {
            // N columns 0..127 = gate rows (leader), 128..255 = up rows (peer) of the same 128 outputs
            ptx::tma_load_2d_pair(b_smem(s), rank == 0 ? &tmB0 : &tmB1, leader_full, kb * BLOCK_K,
                                  n_tile * (BLOCK_N / 2));
          } else {
            ptx::tma_load_2d_pair(b_smem(s), &tmB0, leader_full, kb * BLOCK_K,
                                  n_tile * BLOCK_N + static_cast<int>(rank) * (BLOCK_N / 2));
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = (1u << 4) | (UmmaFmt<T>::v << 7) | (UmmaFmt<T>::v << 10) |
                                 (static_cast<uint32_t>(BLOCK_N >> 3) << 17) |
                                 (static_cast<uint32_t>((2 * BLOCK_M) >> 4) << 24);
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += npairs, ++tcount) {
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
          for (int kk = 0; kk < BLOCK_K / UMMA_K; ++kk)
            ptx::umma_bf16_ss_pair(d_tmem, da + 2 * kk, db + 2 * kk, idesc, (kb | kk) != 0 ? 1u : 0u);
          ptx::umma_commit_pair(empty_bar(s), 3);  // frees the slot in both CTAs
        }
        if (ok) ptx::umma_commit_pair(tfull_bar(acc), 3);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int q = warp & 3;
    const int row_in_tile = q * 32 + lane;
    uint32_t tcount = 0;
    for (int tile = pair; tile < num_tiles; tile += npairs, ++tcount) {
      const int m_tile = tile % num_m_tiles;
      const int n_tile = tile / num_m_tiles;
      const int acc = tcount & 1u;
      const uint32_t aph = (tcount >> 1) & 1u;
      bool ok = ptx::mbar_wait_bounded(tfull_bar(acc), aph, abort_flag);
      ok = __all_sync(kFull, ok);
      if (!ok) break;
      ptx::tc_fence_after();
      const uint32_t taddr = tmem_base + acc * BLOCK_N + (static_cast<uint32_t>(q * 32) << 16);
      const int64_t row = static_cast<int64_t>(m_tile) * (2 * BLOCK_M) + rank * BLOCK_M + row_in_tile;
      const bool row_ok = row < M;

      if constexpr (EPI == PAIR_EPI_SWIGLU) {
        T* orow = static_cast<T*>(ep.out) + row * ep.ldo;
        T* grow = ep.pre_gate != nullptr ? static_cast<T*>(ep.pre_gate) + row * ep.ldo : nullptr;
        T* urow = ep.pre_up != nullptr ? static_cast<T*>(ep.pre_up) + row * ep.ldo : nullptr;
#pragma unroll 1
        for (int c = 0; c < BLOCK_N / 64; ++c) {
          uint32_t g[32], u[32];
          ptx::tmem_ld_32x32(taddr + c * 32, g);
          ptx::tmem_ld_32x32(taddr + BLOCK_N / 2 + c * 32, u);
          ptx::tmem_ld_wait();
          const int col0 = n_tile * (BLOCK_N / 2) + c * 32;
          if (row_ok) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              float f[8];
#pragma unroll
              for (int i = 0; i < 8; ++i)
                f[i] = silu_f32(__uint_as_float(g[v * 8 + i])) * __uint_as_float(u[v * 8 + i]);
              if (col0 + v * 8 < ep.n_valid) {
                *reinterpret_cast<uint4*>(orow + col0 + v * 8) = pack16<T>(f);
                if (grow != nullptr) {
                  float fg[8], fu[8];
#pragma unroll
                  for (int i = 0; i < 8; ++i) {
                    fg[i] = __uint_as_float(g[v * 8 + i]);
                    fu[i] = __uint_as_float(u[v * 8 + i]);
                  }
                  *reinterpret_cast<uint4*>(grow + col0 + v * 8) = pack16<T>(fg);
                  *reinterpret_cast<uint4*>(urow + col0 + v * 8) = pack16<T>(fu);
                }
              }
            }
          }
        }
      } else {
        T* orow = static_cast<T*>(ep.out) + row * ep.ldo;
        const float* arow = (ep.addend != nullptr && row_ok) ? ep.addend + row * ep.ldo : nullptr;
        constexpr int NCHUNK = BLOCK_N / 32;
        float4 nxt[8];
        auto fetch = [&](int c) {
          const int col0 = n_tile * BLOCK_N + c * 32;
#pragma unroll
          for (int v = 0; v < 8; ++v)
            nxt[v] = (arow != nullptr && col0 + v * 4 < ep.n_valid)
                         ? __ldg(reinterpret_cast<const float4*>(arow + col0 + v * 4))
                         : make_float4(0.f, 0.f, 0.f, 0.f);
        };
        fetch(0);
#pragma unroll 1
        for (int c = 0; c < NCHUNK; ++c) {
          float4 cur[8];
#pragma unroll
          for (int v = 0; v < 8; ++v) cur[v] = nxt[v];
          if (c + 1 < NCHUNK) fetch(c + 1);
          uint32_t a[32];
          ptx::tmem_ld_32x32(taddr + c * 32, a);
          ptx::tmem_ld_wait();
          const int col0 = n_tile * BLOCK_N + c * 32;
          if (row_ok) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              if (col0 + v * 8 < ep.n_valid) {
                float f[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(a[v * 8 + i]);
                f[0] += cur[2 * v].x; f[1] += cur[2 * v].y; f[2] += cur[2 * v].z; f[3] += cur[2 * v].w;
                f[4] += cur[2 * v + 1].x; f[5] += cur[2 * v + 1].y; f[6] += cur[2 * v + 1].z; f[7] += cur[2 * v + 1].w;
                *reinterpret_cast<uint4*>(orow + col0 + v * 8) = pack16<T>(f);
              }
            }
          }
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive_cluster(ptx::map_to_cta(tempty_bar(acc), 0));
    }
  }

  // ---------------------------------------------------------------- teardown
  __syncwarp();  // the single-lane roles rejoin their warps before the warp-aligned cluster barrier
  ptx::tc_fence_before();
  ptx::cluster_sync();  // nobody frees TMEM or exits while the peer may still signal it
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_flag != 0 && status != nullptr) atomicOr(status, FMOE_STATUS_WAIT_TIMEOUT);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

int make_map(CUtensorMap* m, const void* basep, int dtype, uint64_t cols, uint64_t rows, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return -static_cast<int>(cudaErrorNotSupported);
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 2};
  const cuuint32_t box[2] = {BLOCK_K, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = dtype == FMOE_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUresult r = fn(m, dt, 2, const_cast<void*>(basep), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FMOE_OK : FMOE_ERR_BAD_ARG;
}

template <int EPI, typename T>
int launch_pair(const CUtensorMap& tA, const CUtensorMap& tB0, const CUtensorMap& tB1, const PairEpi& ep, int64_t M,
                int num_n_tiles, int K, int32_t* status, cudaStream_t stream) {
  auto kern = gemm_tcgen05_pair_kernel<EPI, T>;
  FMOE_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
  const int num_m_tiles = static_cast<int>((M + 2 * BLOCK_M - 1) / (2 * BLOCK_M));
  const int num_k_blocks = (K + BLOCK_K - 1) / BLOCK_K;
  const int64_t tiles = static_cast<int64_t>(num_m_tiles) * num_n_tiles;
  const int max_pairs = device_sm_count() / 2;
  const int pairs = static_cast<int>(tiles < max_pairs ? tiles : max_pairs);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  FMOE_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, tA, tB0, tB1, ep, static_cast<int>(M), num_m_tiles, num_n_tiles,
                                   num_k_blocks, status));
  return FMOE_OK;
}

}  // namespace

// The pair kernels cover the two big shared-MLP GEMMs; callers fall back to the single-CTA kernels
// when this returns false.
bool gemm_pair_supported(int64_t M, int N, int K) { return M >= 512 && N >= 256 && K >= 256; }

int launch_gemm_swiglu_pair(const void* x, const void* gate_w, const void* up_w, void* h, int dtype, int64_t M, int I,
                            int K, int32_t* status, cudaStream_t stream, void* pre_gate, void* pre_up) {
  CUtensorMap tA, tG, tU;
  int rc;
  if ((rc = make_map(&tA, x, dtype, K, M, BLOCK_M)) != FMOE_OK) return rc;
  if ((rc = make_map(&tG, gate_w, dtype, K, I, BLOCK_N / 2)) != FMOE_OK) return rc;
  if ((rc = make_map(&tU, up_w, dtype, K, I, BLOCK_N / 2)) != FMOE_OK) return rc;
  if ((pre_gate == nullptr) != (pre_up == nullptr)) return FMOE_ERR_BAD_ARG;
  PairEpi ep{h, nullptr, I, I, pre_gate, pre_up};
  const int n_tiles = (I + 127) / 128;
  if (dtype == FMOE_DTYPE_BF16)
    return launch_pair<PAIR_EPI_SWIGLU, __nv_bfloat16>(tA, tG, tU, ep, M, n_tiles, K, status, stream);
  return launch_pair<PAIR_EPI_SWIGLU, __half>(tA, tG, tU, ep, M, n_tiles, K, status, stream);
}

int launch_gemm_add_pair(const void* a, const void* b, const float* addend, void* out, int dtype, int64_t M, int N,
                         int K, int32_t* status, cudaStream_t stream) {
  CUtensorMap tA, tB;
  int rc;
  if ((rc = make_map(&tA, a, dtype, K, M, BLOCK_M)) != FMOE_OK) return rc;
  if ((rc = make_map(&tB, b, dtype, K, N, BLOCK_N / 2)) != FMOE_OK) return rc;
  PairEpi ep{out, addend, N, N, nullptr, nullptr};
  const int n_tiles = (N + 255) / 256;
  if (dtype == FMOE_DTYPE_BF16)
    return launch_pair<PAIR_EPI_ADD, __nv_bfloat16>(tA, tB, tB, ep, M, n_tiles, K, status, stream);
  return launch_pair<PAIR_EPI_ADD, __half>(tA, tB, tB, ep, M, n_tiles, K, status, stream);
}

}  // namespace fmoe
