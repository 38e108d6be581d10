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
// No multicast loads anywhere; every mbarrier wait is bounded like in the single-CTA kernel (tcgen05.alloc blocks
// until tensor memory is free on the SM, which an earlier CTA of this library always releases).
#include "gemm_epilogue.cuh"

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
constexpr int RING_BYTES = STAGES * STAGE_BYTES;
constexpr int ADDEND_CHUNK_BYTES = BLOCK_M * 32 * 4;  // this CTA's 128 rows x 32 float32 columns of the addend
constexpr int ADDEND_BUFS = 2;  // four (with a five-stage ring) measured the same: 35.4 vs 35.8 us
constexpr int ADDEND_BYTES = ADDEND_BUFS * ADDEND_CHUNK_BYTES;  // chunks on their way while one is being added
constexpr int SMEM_BYTES = RING_BYTES + ADDEND_BYTES + 256 + 1024;

enum { PAIR_EPI_ADD = 0, PAIR_EPI_SWIGLU = 1 };

struct PairEpi {
  void* out;
  const float* addend;
  const void* residual;  // ADD only, nullable: [M, ldo] in the module dtype, added before the single rounding
  int64_t ldo;
  int n_valid;
  void* pre_gate;  // SWIGLU only, nullable: x Wg^T and x Wu^T rounded to T, kept for the backward pass
  void* pre_up;
};

using epi::UmmaFmt;

template <int EPI, typename T>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB0,
                         const __grid_constant__ CUtensorMap tmB1, PairEpi ep, int M, int num_m_tiles, int num_n_tiles,
                         int num_k_blocks, int32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_u32 = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw_u32 + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - raw_u32);
  const uint32_t bar_base = base + RING_BYTES + ADDEND_BYTES;
  auto a_smem = [&](int s) { return base + s * STAGE_BYTES; };
  auto b_smem = [&](int s) { return base + s * STAGE_BYTES + A_BYTES; };
  auto full_bar = [&](int s) { return bar_base + s * 8; };
  auto empty_bar = [&](int s) { return bar_base + (STAGES + s) * 8; };
  auto tfull_bar = [&](int a) { return bar_base + (2 * STAGES + a) * 8; };
  auto tempty_bar = [&](int a) { return bar_base + (2 * STAGES + 2 + a) * 8; };
  auto cfull_bar = [&](int b) { return bar_base + (2 * STAGES + 4 + b) * 8; };  // addend chunk b has landed
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + RING_BYTES + ADDEND_BYTES + (2 * STAGES + 4 + ADDEND_BUFS) * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + RING_BYTES + ADDEND_BYTES + (2 * STAGES + 4 + ADDEND_BUFS) * 8 + 8);

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
    for (int b = 0; b < ADDEND_BUFS; ++b) ptx::mbar_init(cfull_bar(b), 1);
    *abort_flag = 0;
    ptx::mbar_fence_init();
    ptx::prefetch_tensormap(&tmA);
    ptx::prefetch_tensormap(&tmB0);
    if (EPI == PAIR_EPI_SWIGLU || ep.addend != nullptr) ptx::prefetch_tensormap(&tmB1);  // ADD: the addend's map
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before();
  ptx::cluster_sync();  // barriers of both CTAs are initialised before anyone signals them
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();  // barriers, tensor memory and tensor maps are ready; the operands come from the kernel before this one

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
      if (!ok && rank == 0) {
        // gave up: the leader's `full` barriers count the bytes of BOTH CTAs, so once the leader has seen the
        // stages still in flight complete, neither CTA has a copy on its way; the peer stays until the cluster
        // barrier of the teardown, which the leader reaches only after this loop
        const uint32_t first = it > static_cast<uint32_t>(STAGES) ? it - STAGES : 0u;
        for (uint32_t j = first; j < it; ++j) ptx::mbar_wait_drain(full_bar(j % STAGES), (j / STAGES) & 1u);
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
      // the tile's accumulator is complete when the leader's last commit lands; the ADD epilogue calls this AFTER it
      // has requested its first addend and residual chunks, so that they travel during the end of the main loop
      auto wait_accumulator = [&]() {
        bool ok = ptx::mbar_wait_bounded(tfull_bar(acc), aph, abort_flag);
        ok = __all_sync(kFull, ok);
        if (ok) {
          ptx::tc_fence_after();
          if (tile + npairs >= num_tiles) pdl_launch_dependents();  // last tile: only this epilogue is left
        }
        return ok;
      };
      const uint32_t taddr = tmem_base + acc * BLOCK_N + (static_cast<uint32_t>(q * 32) << 16);
      const int64_t row = static_cast<int64_t>(m_tile) * (2 * BLOCK_M) + rank * BLOCK_M + row_in_tile;
      const bool row_ok = row < M;

      T* orow = static_cast<T*>(ep.out) + row * ep.ldo;
      if constexpr (EPI == PAIR_EPI_SWIGLU) {
        if (!wait_accumulator()) break;
        T* grow = ep.pre_gate != nullptr ? static_cast<T*>(ep.pre_gate) + row * ep.ldo : nullptr;
        T* urow = ep.pre_up != nullptr ? static_cast<T*>(ep.pre_up) + row * ep.ldo : nullptr;
        epi::store_swiglu_row<T, BLOCK_N>(taddr, orow, grow, urow, n_tile * (BLOCK_N / 2), ep.n_valid, row_ok);
      } else {
        const T* rrow = (ep.residual != nullptr && row_ok) ? static_cast<const T*>(ep.residual) + row * ep.ldo : nullptr;
        if (ep.addend == nullptr) {
          if (!epi::store_add_row<T, BLOCK_N>(taddr, orow, nullptr, rrow, n_tile * BLOCK_N, ep.n_valid, row_ok, wait_accumulator))
            break;
        } else {
          // The float32 addend comes through shared memory: one thread asks TMA for this CTA's 128 rows x 32 columns
          // of it, two chunks ahead (the first two before the accumulator is complete), and every thread reads its
          // own row from the swizzled box.  Fetched one row per thread from global memory, 16 bytes per access, the
          // addend cost 6 us of the 37 (measured by taking the loads out); tmB1 carries its tensor map here.
          constexpr int NCHUNK = BLOCK_N / 32;
          const int a_row0 = m_tile * (2 * BLOCK_M) + static_cast<int>(rank) * BLOCK_M;
          auto request = [&](int c) {  // by thread 64 only
            const int b = c % ADDEND_BUFS;
            ptx::mbar_arrive_expect_tx(cfull_bar(b), ADDEND_CHUNK_BYTES);
            ptx::tma_load_2d(base + RING_BYTES + b * ADDEND_CHUNK_BYTES, &tmB1, cfull_bar(b), n_tile * BLOCK_N + c * 32, a_row0);
          };
          if (threadIdx.x == 64) {
#pragma unroll
            for (int c = 0; c < ADDEND_BUFS; ++c) request(c);
          }
          // every warp walks all chunks and meets the others at the barrier even after a wait has given up (the
          // waits then return at once: the abort flag is up), so that the named barrier can never be left hanging
          bool cok = wait_accumulator();
          int requested = ADDEND_BUFS;
#pragma unroll 1
          for (int c = 0; c < NCHUNK; ++c) {
            const int b = c % ADDEND_BUFS;
            const uint32_t cph = (tcount * (NCHUNK / ADDEND_BUFS) + c / ADDEND_BUFS) & 1u;  // uses of buffer b so far
            if (c < requested) cok = ptx::mbar_wait_bounded(cfull_bar(b), cph, abort_flag) && cok;
            else cok = false;
            cok = __all_sync(kFull, cok);
            uint4 rcur[4];
            const int col0 = n_tile * BLOCK_N + c * 32;
#pragma unroll
            for (int v = 0; v < 4; ++v)
              rcur[v] = (rrow != nullptr && col0 + v * 8 < ep.n_valid) ? ldg16(rrow + col0 + v * 8) : make_uint4(0, 0, 0, 0);
            if (cok)
              epi::store_add_chunk_smem<T>(taddr + c * 32, orow, gen + RING_BYTES + b * ADDEND_CHUNK_BYTES, row_in_tile, rcur,
                                           rrow != nullptr, col0, ep.n_valid, row_ok);
            // all four epilogue warps are done with buffer b before it is refilled
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (c + ADDEND_BUFS < NCHUNK && *abort_flag == 0) {
              if (threadIdx.x == 64) request(c + ADDEND_BUFS);
              requested = c + ADDEND_BUFS + 1;
            }
          }
          if (!__all_sync(kFull, cok)) {
            // gave up: let the addend boxes already requested land before this CTA's shared memory goes away (bounded)
            if (threadIdx.x == 64) {
              for (int c = requested - ADDEND_BUFS > 0 ? requested - ADDEND_BUFS : 0; c < requested && c < NCHUNK; ++c)
                ptx::mbar_wait_drain(cfull_bar(c % ADDEND_BUFS), (tcount * (NCHUNK / ADDEND_BUFS) + c / ADDEND_BUFS) & 1u);
            }
            break;
          }
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive_cluster(ptx::map_to_cta(tempty_bar(acc), 0));
    }
  }

  // ---------------------------------------------------------------- teardown
  pdl_launch_dependents();
  __syncwarp();  // the single-lane roles rejoin their warps before the warp-aligned cluster barrier
  ptx::tc_fence_before();
  ptx::cluster_sync();  // nobody frees TMEM or exits while the peer may still signal it
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_flag != 0 && status != nullptr) atomicOr(status, FMOE_STATUS_WAIT_TIMEOUT);
}

int make_map(CUtensorMap* m, const void* basep, int dtype, uint64_t cols, uint64_t rows, uint32_t box_rows) {
  return epi::make_tensor_map(m, basep, dtype, cols, rows, cols, box_rows);
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
  FMOE_CUDA_TRY(launch_pdl(16, kern, dim3(2 * pairs), dim3(kThreads), SMEM_BYTES, stream, 2, tA, tB0, tB1, ep,
                           static_cast<int>(M), num_m_tiles, num_n_tiles, num_k_blocks, status));
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
  PairEpi ep{h, nullptr, nullptr, I, I, pre_gate, pre_up};
  const int n_tiles = (I + 127) / 128;
  if (dtype == FMOE_DTYPE_BF16)
    return launch_pair<PAIR_EPI_SWIGLU, __nv_bfloat16>(tA, tG, tU, ep, M, n_tiles, K, status, stream);
  return launch_pair<PAIR_EPI_SWIGLU, __half>(tA, tG, tU, ep, M, n_tiles, K, status, stream);
}

int launch_gemm_add_pair(const void* a, const void* b, const float* addend, void* out, int dtype, int64_t M, int N,
                         int K, int32_t* status, cudaStream_t stream, const void* residual) {
  CUtensorMap tA, tB;
  int rc;
  if ((rc = make_map(&tA, a, dtype, K, M, BLOCK_M)) != FMOE_OK) return rc;
  if ((rc = make_map(&tB, b, dtype, K, N, BLOCK_N / 2)) != FMOE_OK) return rc;
  PairEpi ep{out, addend, residual, N, N, nullptr, nullptr};
  const int n_tiles = (N + 255) / 256;
  CUtensorMap tC = tB;  // third slot: the float32 addend's map (unused without an addend)
  if (addend != nullptr && (rc = epi::make_tensor_map_f32(&tC, addend, N, M, N, BLOCK_M)) != FMOE_OK) return rc;
  if (dtype == FMOE_DTYPE_BF16)
    return launch_pair<PAIR_EPI_ADD, __nv_bfloat16>(tA, tB, tC, ep, M, n_tiles, K, status, stream);
  return launch_pair<PAIR_EPI_ADD, __half>(tA, tB, tC, ep, M, n_tiles, K, status, stream);
}

}  // namespace fmoe
