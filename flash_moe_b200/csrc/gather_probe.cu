// Measurement aid, not part of the layer: load-only kernels with the access pattern of the expert step - random
// rows of a table brought to the SMs - whose rate is the ceiling the expert kernel is measured against while its
// tables sit in L2.  Two ways of fetching a row:
//   mode 0  16-byte loads into registers (4 rows x row_bytes / 512 loads per lane in flight, many CTAs per SM);
//   mode 1  one bulk asynchronous copy per row into a shared-memory ring (one CTA per SM, a producer warp issuing
//           groups of 16 rows on an mbarrier, a consumer warp handing the slots back), the way the fused expert
//           kernel could fetch its rows;
//   mode 2  the same ring filled by four producer warps with 16-byte cp.async copies whose completion arrives on
//           the group's mbarrier - the way the fused expert kernel does fetch them.
// Row ids outside [0, num_rows) read row 0 instead and raise FMOE_STATUS_BAD_ROW_INDEX.
#include "common.cuh"
#include "ptx_sm100.cuh"

namespace fmoe {
namespace {

constexpr unsigned kFull = 0xFFFFFFFFu;

template <int C>
__global__ void __launch_bounds__(128) gather_probe_kernel(const uint4* __restrict__ table, int64_t num_rows,
                                                           const int32_t* __restrict__ ids, int64_t count, int row_u4,
                                                           float* sink, int32_t* status) {
  const int lane = threadIdx.x & 31;
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t warps_total = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  uint32_t acc = 0;
  bool bad = false;
  for (int64_t r0 = warp_global * 4; r0 + 4 <= count; r0 += warps_total * 4) {
    uint4 q[4][C];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      int64_t id = ids[r0 + u];
      if (id < 0 || id >= num_rows) {
        bad = true;
        id = 0;
      }
      const uint4* row = table + id * row_u4;
#pragma unroll
      for (int c = 0; c < C; ++c) q[u][c] = __ldg(row + c * 32 + lane);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int c = 0; c < C; ++c) acc += q[u][c].x ^ q[u][c].y ^ q[u][c].z ^ q[u][c].w;
  }
  if (acc == 0x12345u && sink != nullptr) sink[0] = static_cast<float>(acc);  // keeps the loads alive
  if (bad && status != nullptr) atomicOr(status, FMOE_STATUS_BAD_ROW_INDEX);
}

constexpr int kRingGroupRows = 16;
constexpr int kRingMaxGroups = 32;

// CTA c takes the id range [c * per_cta, (c + 1) * per_cta) in groups of 16 rows.
__global__ void __launch_bounds__(64, 1)
gather_probe_ring_kernel(const uint8_t* __restrict__ table, int64_t num_rows, const int32_t* __restrict__ ids,
                         int64_t count, int row_bytes, int groups, float* sink, int32_t* status) {
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t ring = ptx::smem_u32(smem);
  const int group_bytes = kRingGroupRows * row_bytes;
  const uint32_t bars = ring + groups * group_bytes;
  auto full_bar = [&](int s) { return bars + s * 8; };
  auto empty_bar = [&](int s) { return bars + (kRingMaxGroups + s) * 8; };
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + groups * group_bytes + 2 * kRingMaxGroups * 8);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < groups; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    *abort_flag = 0;
    ptx::mbar_fence_init();
  }
  __syncthreads();
  const int64_t per_cta = (count + gridDim.x - 1) / gridDim.x;
  const int64_t first = blockIdx.x * per_cta;
  const int64_t last = first + per_cta < count ? first + per_cta : count;
  const int64_t ngroups = last > first ? (last - first + kRingGroupRows - 1) / kRingGroupRows : 0;
  if (warp == 0) {
    bool bad = false;
    uint32_t issued = 0;
    for (int64_t g = 0; g < ngroups; ++g, ++issued) {
      const int s = static_cast<int>(g % groups);
      const uint32_t ph = static_cast<uint32_t>(g / groups) & 1u;
      const int64_t r = first + g * kRingGroupRows + lane;
      const int nrows = static_cast<int>(last - (first + g * kRingGroupRows) < kRingGroupRows
                                             ? last - (first + g * kRingGroupRows)
                                             : kRingGroupRows);
      int64_t id = (lane < nrows) ? ids[r] : 0;
      if (id < 0 || id >= num_rows) {
        bad = true;
        id = 0;
      }
      if (!ptx::mbar_wait_bounded(empty_bar(s), ph ^ 1u, abort_flag, 1000000000ull)) break;
      if (lane == 0) ptx::mbar_arrive_expect_tx(full_bar(s), static_cast<uint32_t>(nrows) * row_bytes);
      __syncwarp();
      if (lane < nrows) {
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                         ring + s * group_bytes + lane * row_bytes),
                     "l"(reinterpret_cast<uint64_t>(table + id * row_bytes)), "r"(row_bytes), "r"(full_bar(s))
                     : "memory");
      }
    }
    if (bad && status != nullptr) atomicOr(status, FMOE_STATUS_BAD_ROW_INDEX);
    if (*abort_flag != 0 && lane == 0) {  // let the copies in flight land before the CTA leaves
      const uint32_t lo = issued > static_cast<uint32_t>(groups) ? issued - groups : 0u;
      for (uint32_t g = lo; g < issued; ++g) {
        const uint64_t t0 = ptx::globaltimer_ns();
        while (!ptx::mbar_try_wait(full_bar(g % groups), (g / groups) & 1u) && ptx::globaltimer_ns() - t0 < 100000000ull) {
        }
      }
    }
  } else {
    uint32_t acc = 0;
    for (int64_t g = 0; g < ngroups; ++g) {
      const int s = static_cast<int>(g % groups);
      if (!ptx::mbar_wait_bounded(full_bar(s), static_cast<uint32_t>(g / groups) & 1u, abort_flag, 1000000000ull)) break;
      if (lane < kRingGroupRows) acc += *reinterpret_cast<const uint32_t*>(smem + s * group_bytes + lane * row_bytes);
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(empty_bar(s));
    }
    if (acc == 0x12345u && sink != nullptr) sink[0] = static_cast<float>(acc);
  }
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag != 0 && status != nullptr) atomicOr(status, FMOE_STATUS_WAIT_TIMEOUT);
}

constexpr int kCpProducers = 4;

// mode 2: warps 0..3 fill the groups g with g % 4 == warp, warp 4 hands the slots back.  C = row_bytes / 512:
// 16-byte pieces per lane and row (the copy loop is unrolled; a rolled loop issued too slowly to show the roof).
template <int C>
__global__ void __launch_bounds__((kCpProducers + 1) * 32, 1)
gather_probe_cpasync_kernel(const uint8_t* __restrict__ table, int64_t num_rows, const int32_t* __restrict__ ids,
                            int64_t count, int row_bytes, int groups, float* sink, int32_t* status) {
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t ring = ptx::smem_u32(smem);
  const int group_bytes = kRingGroupRows * row_bytes;
  const uint32_t bars = ring + groups * group_bytes;
  auto full_bar = [&](int s) { return bars + s * 8; };
  auto empty_bar = [&](int s) { return bars + (kRingMaxGroups + s) * 8; };
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + groups * group_bytes + 2 * kRingMaxGroups * 8);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < groups; ++s) {
      ptx::mbar_init(full_bar(s), 32);
      ptx::mbar_init(empty_bar(s), 1);
    }
    *abort_flag = 0;
    ptx::mbar_fence_init();
  }
  __syncthreads();
  const int64_t per_cta = (count + gridDim.x - 1) / gridDim.x;
  const int64_t first = blockIdx.x * per_cta;
  const int64_t last = first + per_cta < count ? first + per_cta : count;
  const int64_t ngroups = last > first ? (last - first + kRingGroupRows - 1) / kRingGroupRows : 0;
  if (warp < kCpProducers) {
    bool bad = false;
    for (int64_t g = warp; g < ngroups; g += kCpProducers) {
      const int s = static_cast<int>(g % groups);
      const uint32_t ph = static_cast<uint32_t>(g / groups) & 1u;
      const int64_t r0 = first + g * kRingGroupRows;
      const int nrows = static_cast<int>(last - r0 < kRingGroupRows ? last - r0 : kRingGroupRows);
      int64_t id = (lane < nrows) ? ids[r0 + lane] : 0;
      if (id < 0 || id >= num_rows) {
        bad = true;
        id = 0;
      }
      if (!ptx::mbar_wait_bounded(empty_bar(s), ph ^ 1u, abort_flag, 1000000000ull)) break;
#pragma unroll 4
      for (int rr = 0; rr < kRingGroupRows; ++rr) {
        if (rr < nrows) {
          const int64_t e = __shfl_sync(kFull, id, rr);
          const uint8_t* src = table + e * row_bytes + lane * 16;
          const uint32_t dst = ring + s * group_bytes + rr * row_bytes + lane * 16;
#pragma unroll
          for (int j = 0; j < C; ++j)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + j * 512),
                         "l"(reinterpret_cast<uint64_t>(src + j * 512))
                         : "memory");
        }
      }
      asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(full_bar(s)) : "memory");
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
    if (bad && status != nullptr) atomicOr(status, FMOE_STATUS_BAD_ROW_INDEX);
  } else {
    uint32_t acc = 0;
    for (int64_t g = 0; g < ngroups; ++g) {
      const int s = static_cast<int>(g % groups);
      if (!ptx::mbar_wait_bounded(full_bar(s), static_cast<uint32_t>(g / groups) & 1u, abort_flag, 1000000000ull)) break;
      if (lane < kRingGroupRows) acc += *reinterpret_cast<const uint32_t*>(smem + s * group_bytes + lane * row_bytes);
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(empty_bar(s));
    }
    if (acc == 0x12345u && sink != nullptr) sink[0] = static_cast<float>(acc);
  }
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag != 0 && status != nullptr) atomicOr(status, FMOE_STATUS_WAIT_TIMEOUT);
}

}  // namespace

int launch_gather_probe(const void* table, int64_t num_rows, const int32_t* row_ids, int64_t count, int row_bytes,
                        int ctas_per_sm, int mode, float* sink, int32_t* status, cudaStream_t stream) {
  if (table == nullptr || row_ids == nullptr || count < 0 || num_rows < 1) return FMOE_ERR_BAD_ARG;
  if (!aligned16(table)) return FMOE_ERR_ALIGNMENT;
  if (mode == 1 || mode == 2) {
    if (row_bytes < 16 || row_bytes % 16 != 0) return FMOE_ERR_ALIGNMENT;
    const int group_bytes = kRingGroupRows * row_bytes;
    int groups = (220 * 1024) / group_bytes;
    if (groups > kRingMaxGroups) groups = kRingMaxGroups;
    if (groups < 2) return FMOE_ERR_UNSUPPORTED;
    const int smem = groups * group_bytes + 2 * kRingMaxGroups * 8 + 64;
    if (mode == 1) {
      FMOE_CUDA_TRY(cudaFuncSetAttribute(gather_probe_ring_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      gather_probe_ring_kernel<<<device_sm_count(), 64, smem, stream>>>(static_cast<const uint8_t*>(table), num_rows,
                                                                        row_ids, count, row_bytes, groups, sink, status);
    } else {
      if (row_bytes % 512 != 0) return FMOE_ERR_ALIGNMENT;
      if (groups < kCpProducers) return FMOE_ERR_UNSUPPORTED;  // a producer must never lap the ring
#define FMOE_PROBE_CP(C_)                                                                                              \
  do {                                                                                                                 \
    FMOE_CUDA_TRY(cudaFuncSetAttribute(gather_probe_cpasync_kernel<C_>, cudaFuncAttributeMaxDynamicSharedMemorySize,   \
                                       smem));                                                                         \
    gather_probe_cpasync_kernel<C_><<<device_sm_count(), (kCpProducers + 1) * 32, smem, stream>>>(                     \
        static_cast<const uint8_t*>(table), num_rows, row_ids, count, row_bytes, groups, sink, status);                \
  } while (0)
      switch (row_bytes / 512) {
        case 1: FMOE_PROBE_CP(1); break;
        case 2: FMOE_PROBE_CP(2); break;
        case 4: FMOE_PROBE_CP(4); break;
        default: return FMOE_ERR_UNSUPPORTED;
      }
#undef FMOE_PROBE_CP
    }
    FMOE_LAUNCH_CHECK();
    return FMOE_OK;
  }
  if (mode != 0 || ctas_per_sm < 1 || ctas_per_sm > 32) return FMOE_ERR_BAD_ARG;
  if (row_bytes % 512 != 0) return FMOE_ERR_ALIGNMENT;
  const int grid = device_sm_count() * ctas_per_sm;
  const uint4* t = static_cast<const uint4*>(table);
  switch (row_bytes / 512) {
    case 1: gather_probe_kernel<1><<<grid, 128, 0, stream>>>(t, num_rows, row_ids, count, row_bytes / 16, sink, status); break;
    case 2: gather_probe_kernel<2><<<grid, 128, 0, stream>>>(t, num_rows, row_ids, count, row_bytes / 16, sink, status); break;
    case 4: gather_probe_kernel<4><<<grid, 128, 0, stream>>>(t, num_rows, row_ids, count, row_bytes / 16, sink, status); break;
    case 8: gather_probe_kernel<8><<<grid, 128, 0, stream>>>(t, num_rows, row_ids, count, row_bytes / 16, sink, status); break;
    default: return FMOE_ERR_UNSUPPORTED;
  }
  FMOE_LAUNCH_CHECK();
  return FMOE_OK;
}

}  // namespace fmoe
