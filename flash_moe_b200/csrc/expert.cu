// Fine-grained expert forward for sm_100a:
//   out[t] = sum_j silu(<x[t], D[e_tj]>) * g[t,j] * U[e_tj]
// (flash_moe/ops/triton/flash_expert.py:13-211, preprocessing :528-577).
//
// Two schedules, picked by dtype
//   A. 16-bit dtypes: no sort.  Scores per token on the tensor cores
//      (mma.sync, groups of 16 gathered down rows against the token's x row), then the per-token
//      accumulate of step 3.
//   B. float32: expert-centric order of the (token, slot) pairs by a
//      device-side counting sort (histogram with warp-aggregated atomics -> exclusive scan ->
//      scatter; no host sync; ids outside [0, N) are dropped and flagged), then a scores pass over
//      the SORTED pairs: a warp walks a contiguous run of pairs, keeps the current expert's down
//      row in registers (loaded once per run of equal ids with 128-bit loads), gathers each pair's
//      x row and reduces the dot product in fp32; empty experts cost nothing, a hot expert is
//      split over many warps.
//   Both store gs = silu(s) * gate at the pair's (token, slot) position (4 bytes per pair).
//   3. accumulate pass per token: out[t] = sum_j gs[t,j] * U[e_tj] in fp32 (packed f32x2 FMAs),
//      fixed slot order, one rounding on store - no atomics, run-to-run deterministic.
#include <cub/device/device_radix_sort.cuh>

#include <cstdlib>

#include "common.cuh"

namespace fmoe {
namespace {

constexpr unsigned kFull = 0xFFFFFFFFu;
constexpr int kScanThreads = 256;
constexpr int kScanItems = 8;
constexpr int kScanTile = kScanThreads * kScanItems;

// ---------------------------------------------------------------- 1. counting sort
__global__ void expert_hist_kernel(const int64_t* __restrict__ idx, int64_t P, int64_t N, int* __restrict__ counts,
                                   int* __restrict__ rank, int32_t* status) {
  const int lane = threadIdx.x & 31;
  const int64_t warps_total = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  bool bad = false;
  for (int64_t base = warp_global * 32; base < P; base += warps_total * 32) {
    const int64_t p = base + lane;
    int64_t e = -1;
    if (p < P) e = idx[p];
    const bool valid = (p < P) && (e >= 0) && (e < N);
    if (p < P && !valid && e != -1) bad = true;  // -1 is the empty-slot value: skipped without a flag
    // lanes holding the same expert id share one atomic; invalid lanes get distinct keys
    const unsigned key = valid ? static_cast<unsigned>(e) : (0x80000000u | lane);
    const unsigned peers = __match_any_sync(kFull, key);
    const int leader = __ffs(peers) - 1;
    int basecnt = 0;
    if (valid && lane == leader) basecnt = atomicAdd(&counts[e], __popc(peers));
    basecnt = __shfl_sync(kFull, basecnt, leader);
    if (p < P) rank[p] = valid ? basecnt + __popc(peers & ((1u << lane) - 1u)) : -1;
  }
  if (bad && status != nullptr) atomicOr(status, FMOE_STATUS_BAD_EXPERT_ID);
}

__device__ __forceinline__ int block_reduce_sum(int v, int* sh) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(kFull, v, d);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  int tot = 0;
  for (int w = 0; w < (blockDim.x >> 5); ++w) tot += sh[w];
  __syncthreads();
  return tot;
}

__global__ void __launch_bounds__(kScanThreads) scan_tile_sums_kernel(const int* __restrict__ counts, int64_t N,
                                                                     int* __restrict__ tile_sums) {
  __shared__ int sh[kScanThreads / 32];
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kScanTile;
  int v = 0;
  for (int i = threadIdx.x; i < kScanTile; i += kScanThreads)
    if (base + i < N) v += counts[base + i];
  const int tot = block_reduce_sum(v, sh);
  if (threadIdx.x == 0) tile_sums[blockIdx.x] = tot;
}

// offsets[i] = sum(counts[0..i)), offsets[N] = total.  tile_sums == nullptr: the prefix of the
// preceding tiles is recomputed from counts (cheap when there are only a few tiles).
__global__ void __launch_bounds__(kScanThreads) scan_apply_kernel(const int* __restrict__ counts, int64_t N,
                                                                  const int* __restrict__ tile_sums,
                                                                  int* __restrict__ offsets) {
  __shared__ int sh[kScanThreads / 32];
  __shared__ int warp_pref[kScanThreads / 32];
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kScanTile;
  int v = 0;
  if (tile_sums != nullptr) {
    for (int i = threadIdx.x; i < static_cast<int>(blockIdx.x); i += kScanThreads) v += tile_sums[i];
  } else {
    for (int64_t i = threadIdx.x; i < base; i += kScanThreads) v += counts[i];
  }
  const int prefix = block_reduce_sum(v, sh);

  int item[kScanItems];
  int tsum = 0;
  const int64_t first = base + static_cast<int64_t>(threadIdx.x) * kScanItems;
#pragma unroll
  for (int i = 0; i < kScanItems; ++i) {
    item[i] = (first + i < N) ? counts[first + i] : 0;
    tsum += item[i];
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = tsum;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int up = __shfl_up_sync(kFull, incl, d);
    if (lane >= d) incl += up;
  }
  if (lane == 31) warp_pref[warp] = incl;
  __syncthreads();
  int wbase = 0;
  for (int w = 0; w < warp; ++w) wbase += warp_pref[w];
  int run = prefix + wbase + incl - tsum;
#pragma unroll
  for (int i = 0; i < kScanItems; ++i) {
    if (first + i < N) offsets[first + i] = run;
    run += item[i];
    if (first + i == N - 1) offsets[N] = run;
  }
}

__global__ void expert_scatter_kernel(const int64_t* __restrict__ idx, const int* __restrict__ rank,
                                      const int* __restrict__ offsets, int64_t P, int* __restrict__ sorted_pair,
                                      int* __restrict__ sorted_expert) {
  for (int64_t p = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; p < P;
       p += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int r = rank[p];
    if (r < 0) continue;
    const int e = static_cast<int>(idx[p]);
    const int pos = offsets[e] + r;
    sorted_pair[pos] = static_cast<int>(p);
    sorted_expert[pos] = e;
  }
}

// ---------------------------------------------------------------- 2. scores over sorted pairs
// NCH > 0: the row fits NCH 16-byte chunks per lane and the down row is cached in registers.
// NCH == 0: any H, the down row is re-read (L1-resident) for every pair.
template <typename T, int NCH>
__global__ void __launch_bounds__(256) expert_scores_kernel(const T* __restrict__ x, const T* __restrict__ down,
                                                           const int* __restrict__ sorted_pair,
                                                           const int* __restrict__ sorted_expert,
                                                           const int* __restrict__ total_ptr,
                                                           const T* __restrict__ gates, float* __restrict__ gs, int H,
                                                           int k, int chunk, int act, float* __restrict__ raw_out) {
  constexpr int VEC = Vec16<T>::N;
  constexpr int R = NCH > 0 ? NCH : 1;
  const int lane = threadIdx.x & 31;
  const int64_t warps_total = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int total = *total_ptr;

  for (int64_t task = warp_global; task * chunk < total; task += warps_total) {
    const int pos0 = static_cast<int>(task * chunk);
    const int pos1 = min(pos0 + chunk, total);
    int cur_e = -1;
    float dreg[R][VEC];
    uint4 xq[R], xn[R];
    // prefetch the first pair's x row
    int p_next = sorted_pair[pos0];
    if (NCH > 0) {
      const T* xr = x + static_cast<int64_t>(p_next / k) * H;
#pragma unroll
      for (int c = 0; c < R; ++c) {
        const int col = (c * 32 + lane) * VEC;
        xn[c] = (col < H) ? ldg16(xr + col) : make_uint4(0, 0, 0, 0);
      }
    }
    for (int pos = pos0; pos < pos1; ++pos) {
      const int p = p_next;
      const int e = sorted_expert[pos];
      float acc = 0.f;
      if (NCH > 0) {
#pragma unroll
        for (int c = 0; c < R; ++c) xq[c] = xn[c];
        if (pos + 1 < pos1) {  // issue the next pair's gather before the math of this one
          p_next = sorted_pair[pos + 1];
          const T* xr = x + static_cast<int64_t>(p_next / k) * H;
#pragma unroll
          for (int c = 0; c < R; ++c) {
            const int col = (c * 32 + lane) * VEC;
            xn[c] = (col < H) ? ldg16(xr + col) : make_uint4(0, 0, 0, 0);
          }
        }
        if (e != cur_e) {  // warp-uniform
          cur_e = e;
          const T* dr = down + static_cast<int64_t>(e) * H;
#pragma unroll
          for (int c = 0; c < R; ++c) {
            const int col = (c * 32 + lane) * VEC;
            const uint4 q = (col < H) ? ldg16(dr + col) : make_uint4(0, 0, 0, 0);
            unpack16<T>(q, dreg[c]);
          }
        }
#pragma unroll
        for (int c = 0; c < R; ++c) {
          float xf[VEC];
          unpack16<T>(xq[c], xf);
#pragma unroll
          for (int i = 0; i < VEC; ++i) acc = fmaf(xf[i], dreg[c][i], acc);
        }
      } else {
        if (pos + 1 < pos1) p_next = sorted_pair[pos + 1];
        const T* xr = x + static_cast<int64_t>(p / k) * H;
        const T* dr = down + static_cast<int64_t>(e) * H;
        for (int col = lane * VEC; col < H; col += 32 * VEC) {
          float xf[VEC], df[VEC];
          unpack16<T>(ldg16(xr + col), xf);
          unpack16<T>(ldg16(dr + col), df);
#pragma unroll
          for (int i = 0; i < VEC; ++i) acc = fmaf(xf[i], df[i], acc);
        }
      }
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) acc += __shfl_xor_sync(kFull, acc, d);
      if (lane == 0) {
        gs[p] = gates != nullptr ? expert_act(acc, act) * to_f32<T>(gates[p]) : acc;  // nullptr: raw dot product
        if (raw_out != nullptr) raw_out[p] = acc;  // kept for the backward pass
      }
    }
  }
}

// ---------------------------------------------------------------- 2b. scores per token on mma.sync
// Token-centric scores for 16-bit dtypes when the tables are small enough to stay in L2: no
// sort.  One warp per token; groups of 16 of its experts form the A operand (their down rows,
// gathered with 128-bit loads), the token's x row is every column of B, so each accumulator
// column holds <x, D[e]> for the 16 rows (fp32 accumulate).  The k index inside a 32-column
// block is permuted identically for A and B so that every thread's 16-byte load feeds two MMAs.
template <typename T> struct Mma16816;
template <> struct Mma16816<__nv_bfloat16> {
  static __device__ __forceinline__ void run(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
};
template <> struct Mma16816<__half> {
  static __device__ __forceinline__ void run(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
};

// Row e of a table that is either one array or, PEER, sharded over the GPUs of a node by e % world (shard r holds
// expert e at row e / world; shards[r] may point into a peer GPU's memory, read with plain loads over NVLink).
// In the sharded form ids at or above `sharded` address a small table replicated on every GPU (the hottest
// experts, copied once): row e - sharded of `table`, which is local memory.
template <typename T, bool PEER>
__device__ __forceinline__ const T* table_row(const T* table, const T* const* shards, int world, int64_t e, int H,
                                              int64_t sharded = 0) {
  if constexpr (PEER) {
    if (e >= sharded) return table + (e - sharded) * H;
    const int64_t local = e / world;
    return shards[e - local * world] + local * H;
  } else {
    return table + e * H;
  }
}

// One warp per (token, group of 16 of its experts).  The token's x row is parked in the warp's
// slice of shared memory (read back as B fragments right before each MMA; fetched with cp.async one task ahead,
// together with the next task's expert ids), so every register that
// waits for data waits for a gathered down row: batches of UNROLL 32-column blocks (2 * UNROLL x 16 B per lane) in
// STAGES register buffers keep gathers in flight across batches to cover the L2 latency (measured at the
// benchmark shape: 4 x 2 buffers 57.7 us, 8 x 1 61.9 us, 4 x 3 62.6 us, 2 x 2 57.8 us).
template <typename T, int UNROLL, bool PEER = false, int STAGES = 1>
__global__ void __launch_bounds__(128) expert_scores_mma_kernel(const T* __restrict__ x, const T* __restrict__ down,
                                                               const int64_t* __restrict__ idx,
                                                               const T* __restrict__ gates, float* __restrict__ gs,
                                                               int64_t ntok, int H, int64_t N, int k, int xs_stride,
                                                               int32_t* status, int act,
                                                               const T* const* __restrict__ shards = nullptr,
                                                               int world = 1, float* __restrict__ raw_out = nullptr,
                                                               int64_t sharded = 0) {
  extern __shared__ uint4 xs_all[];
  pdl_wait();  // ids and gates come from the kernel before this one
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2, tq = lane & 3;
  // two x-row buffers per warp (xs_stride uint4 each, >= ceil(H/256)*32): while one task is computed, the next
  // task's ids and x row are already on their way (cp.async), so a task does not start with an exposed round trip
  uint4* xs_buf = xs_all + (threadIdx.x >> 5) * 2 * xs_stride;
  const int64_t warps_total = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int groups = (k + 15) >> 4;
  const int64_t tasks = ntok * groups;
  const int hv = H >> 3;  // 16-byte pieces per row
  bool bad = false;
  auto fetch_ids = [&](int64_t task_, int64_t& ea_, int64_t& eb_) {
    const int64_t t_ = task_ / groups;
    const int ja_ = static_cast<int>(task_ - t_ * groups) * 16 + g, jb_ = ja_ + 8;
    ea_ = ja_ < k ? idx[t_ * k + ja_] : 0;
    eb_ = jb_ < k ? idx[t_ * k + jb_] : 0;
  };
  auto fetch_x = [&](int64_t t_, uint4* dst) {
    const T* xr = x + t_ * H;
    for (int c = lane; c < xs_stride; c += 32) {
      if (c < hv) {
        asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst + c))),
                     "l"(reinterpret_cast<uint64_t>(xr + c * 8))
                     : "memory");
      } else {
        dst[c] = make_uint4(0, 0, 0, 0);
      }
    }
  };
  int cur = 0;
  int64_t ea_next = 0, eb_next = 0;
  if (warp_global < tasks) {
    fetch_ids(warp_global, ea_next, eb_next);
    fetch_x(warp_global / groups, xs_buf);
  }
  for (int64_t task = warp_global; task < tasks; task += warps_total) {
    if (task + warps_total >= tasks) pdl_launch_dependents();  // last task of this warp: the next kernel may set up
    const int64_t t = task / groups;
    const int G = static_cast<int>(task - t * groups);
    const int ja = G * 16 + g, jb = ja + 8;
    const int64_t ea = ea_next, eb = eb_next;
    const uint4* xs = xs_buf + cur * xs_stride;
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncwarp();  // this task's x row has landed; the other buffer is free (its task is finished)
    if (task + warps_total < tasks) {
      fetch_ids(task + warps_total, ea_next, eb_next);
      fetch_x((task + warps_total) / groups, xs_buf + (cur ^ 1) * xs_stride);
    }
    cur ^= 1;
    const bool oka = (ja < k) && ea >= 0 && ea < N;
    const bool okb = (jb < k) && eb >= 0 && eb < N;
    if ((ja < k && !oka && ea != -1) || (jb < k && !okb && eb != -1)) bad = true;  // -1: empty slot, no flag
    const T* ra = table_row<T, PEER>(down, shards, world, oka ? ea : 0, H, sharded) + 8 * tq;
    const T* rb = table_row<T, PEER>(down, shards, world, okb ? eb : 0, H, sharded) + 8 * tq;
    float c[4] = {0.f, 0.f, 0.f, 0.f};
    auto load = [&](uint4 (&qa)[UNROLL], uint4 (&qb)[UNROLL], int c0) {
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int col = c0 + 32 * u;
        const bool in = col + 8 * tq < H;
        qa[u] = in ? ldg16(ra + col) : make_uint4(0, 0, 0, 0);
        qb[u] = in ? ldg16(rb + col) : make_uint4(0, 0, 0, 0);
      }
    };
    auto consume = [&](const uint4 (&qa)[UNROLL], const uint4 (&qb)[UNROLL], int c0) {
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int piece = ((c0 + 32 * u) >> 3) + tq;
        const uint4 xq = piece < xs_stride ? xs[piece] : make_uint4(0, 0, 0, 0);
        Mma16816<T>::run(c, qa[u].x, qb[u].x, qa[u].y, qb[u].y, xq.x, xq.y);
        Mma16816<T>::run(c, qa[u].z, qb[u].z, qa[u].w, qb[u].w, xq.z, xq.w);
      }
    };
    if constexpr (STAGES == 2) {
      // two register buffers: the next batch of gathers is issued before the current one is consumed, so the
      // loads in flight never drain between batches (same column order, hence the same sums)
      constexpr int STEP = 32 * UNROLL;
      uint4 a0[UNROLL], b0[UNROLL], a1[UNROLL], b1[UNROLL];
      load(a0, b0, 0);
      for (int c0 = 0; c0 < H; c0 += 2 * STEP) {
        if (c0 + STEP < H) load(a1, b1, c0 + STEP);
        consume(a0, b0, c0);
        if (c0 + 2 * STEP < H) load(a0, b0, c0 + 2 * STEP);
        if (c0 + STEP < H) consume(a1, b1, c0 + STEP);
      }
    } else {
      for (int c0 = 0; c0 < H; c0 += 32 * UNROLL) {
        uint4 qa[UNROLL], qb[UNROLL];
        load(qa, qb, c0);
        consume(qa, qb, c0);
      }
    }
    if (tq == 0) {
      if (gates != nullptr) {
        if (ja < k) gs[t * k + ja] = oka ? expert_act(c[0], act) * to_f32<T>(gates[t * k + ja]) : 0.f;
        if (jb < k) gs[t * k + jb] = okb ? expert_act(c[2], act) * to_f32<T>(gates[t * k + jb]) : 0.f;
        if (raw_out != nullptr) {  // pre-activation scores kept for the backward pass
          if (ja < k) raw_out[t * k + ja] = oka ? c[0] : 0.f;
          if (jb < k) raw_out[t * k + jb] = okb ? c[2] : 0.f;
        }
      } else {  // raw dot products (backward pass)
        if (ja < k) gs[t * k + ja] = oka ? c[0] : 0.f;
        if (jb < k) gs[t * k + jb] = okb ? c[2] : 0.f;
      }
    }
  }
  if (bad && status != nullptr) atomicOr(status, FMOE_STATUS_BAD_EXPERT_ID);
}

// ---------------------------------------------------------------- 3. per-token accumulate
// One warp per (token, column block of 32*VEC*NCH elements); 16 x 16 B of gathered rows in flight
// per lane, packed f32x2 FMAs (two accumulators per instruction).  The launch bound keeps the kernel at 120
// registers so that four CTAs (not three) fit an SM: a third more gathers in flight, 52 -> 48 us at the benchmark
// shape (a fifth CTA would need spills and is slower: 120 vs 105 us for both passes).
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ void ffma2(uint64_t& acc, uint64_t a, uint64_t b) {
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(a), "l"(b));
}

template <typename T, typename OutT, int NCH, bool PEER = false>
__global__ void __launch_bounds__(128, 4) expert_accum_kernel(const T* __restrict__ up, const int64_t* __restrict__ idx,
                                                          const float* __restrict__ gs, OutT* __restrict__ out,
                                                          int64_t ntok, int H, int64_t N, int k, int colblocks,
                                                          const T* const* __restrict__ shards = nullptr,
                                                          int world = 1, int64_t sharded = 0) {
  constexpr int VEC = Vec16<T>::N;
  constexpr int SLOTS = NCH >= 4 ? 4 : 8;
  pdl_wait();  // the weights gs come from the scores pass
  const int lane = threadIdx.x & 31;
  const int64_t warps_total = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t tasks = ntok * colblocks;
  // each lane fetches one slot's (expert id, weight) - one batch of 32 slots AHEAD of the batch being gathered,
  // also across tasks, so that the gathers of a batch never wait for their own ids; invalid or absent slots get
  // weight 0
  auto fetch_slot = [&](int64_t t_, int j0_, int& e_, float& w_) {
    e_ = 0;
    w_ = 0.f;
    const int j = j0_ + lane;
    if (j < k) {
      const int64_t e = idx[t_ * k + j];
      if (e >= 0 && e < N) {
        e_ = static_cast<int>(e);
        w_ = gs[t_ * k + j];
      }
    }
  };
  int e_next = 0;
  float w_next = 0.f;
  if (warp_global < tasks) fetch_slot(warp_global / colblocks, 0, e_next, w_next);
  for (int64_t task = warp_global; task < tasks; task += warps_total) {
    if (task + warps_total >= tasks) pdl_launch_dependents();  // last task of this warp: the next kernel may set up
    const int64_t t = task / colblocks;
    const int cb = static_cast<int>(task - t * colblocks);
    const int col0 = cb * (32 * VEC * NCH);
    bool in[NCH];
#pragma unroll
    for (int c = 0; c < NCH; ++c) in[c] = col0 + (c * 32 + lane) * VEC < H;
    uint64_t acc[NCH][VEC / 2];
#pragma unroll
    for (int c = 0; c < NCH; ++c)
#pragma unroll
      for (int i = 0; i < VEC / 2; ++i) acc[c][i] = 0ull;

    for (int j0 = 0; j0 < k; j0 += 32) {
      const int e_l = e_next;
      const float w_l = w_next;
      if (j0 + 32 < k) fetch_slot(t, j0 + 32, e_next, w_next);
      else if (task + warps_total < tasks) fetch_slot((task + warps_total) / colblocks, 0, e_next, w_next);
      const int nslots = min(32, k - j0);
      auto load = [&](uint4 (&q)[SLOTS][NCH], uint64_t (&ww)[SLOTS], int s) {
#pragma unroll
        for (int u = 0; u < SLOTS; ++u) {
          const int e = __shfl_sync(kFull, e_l, s + u);
          const float w = __shfl_sync(kFull, w_l, s + u);
          ww[u] = pack_f32x2(w, w);
          const T* row = table_row<T, PEER>(up, shards, world, e, H, sharded) + col0 + lane * VEC;
#pragma unroll
          for (int c = 0; c < NCH; ++c) q[u][c] = in[c] ? ldg16(row + c * 32 * VEC) : make_uint4(0, 0, 0, 0);
        }
      };
      auto consume = [&](const uint4 (&q)[SLOTS][NCH], const uint64_t (&ww)[SLOTS]) {
#pragma unroll
        for (int u = 0; u < SLOTS; ++u)
#pragma unroll
          for (int c = 0; c < NCH; ++c) {
            float f[VEC];
            unpack16<T>(q[u][c], f);
#pragma unroll
            for (int i = 0; i < VEC / 2; ++i) ffma2(acc[c][i], pack_f32x2(f[2 * i], f[2 * i + 1]), ww[u]);
          }
      };
      // one batch of SLOTS gathered rows at a time (a second register buffer was measured slower: 64 vs 52 us)
      for (int s = 0; s < nslots; s += SLOTS) {
        uint4 q[SLOTS][NCH];
        uint64_t ww[SLOTS];
        load(q, ww, s);
        consume(q, ww);
      }
    }
    OutT* orow = out + t * H + col0;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int col = (c * 32 + lane) * VEC;
      if (in[c]) {
        float f[VEC];
#pragma unroll
        for (int i = 0; i < VEC / 2; ++i) unpack_f32x2(acc[c][i], f[2 * i], f[2 * i + 1]);
        if constexpr (sizeof(OutT) == 4) {
#pragma unroll
          for (int i = 0; i < VEC; i += 4)
            *reinterpret_cast<float4*>(reinterpret_cast<float*>(orow) + col + i) =
                make_float4(f[i], f[i + 1], f[i + 2], f[i + 3]);
        } else {
          *reinterpret_cast<uint4*>(orow + col) = pack16<OutT>(f);
        }
      }
    }
  }
}

struct ExpertWs {
  int* counts;
  int* offsets;
  int* tile_sums;
  int* rank;
  int* sorted_pair;
  int* sorted_expert;
  float* gs;
  size_t bytes;
};

ExpertWs carve(void* ws, int64_t T, int64_t N, int k) {
  const int64_t P = T * k;
  const int64_t ntiles = (N + kScanTile - 1) / kScanTile;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    void* p = ws ? static_cast<char*>(ws) + off : nullptr;
    off += align_up(bytes, 256);
    return p;
  };
  ExpertWs w;
  w.counts = static_cast<int*>(take(static_cast<size_t>(N) * 4));
  w.offsets = static_cast<int*>(take(static_cast<size_t>(N + 1) * 4));
  w.tile_sums = static_cast<int*>(take(static_cast<size_t>(ntiles) * 4));
  w.rank = static_cast<int*>(take(static_cast<size_t>(P) * 4));
  w.sorted_pair = static_cast<int*>(take(static_cast<size_t>(P) * 4));
  w.sorted_expert = static_cast<int*>(take(static_cast<size_t>(P) * 4));
  w.gs = static_cast<float*>(take(static_cast<size_t>(P) * 4));
  w.bytes = off;
  return w;
}

template <typename T, int NCH>
void launch_scores(const void* x, const void* down, const ExpertWs& w, int64_t N, const void* gates, float* gs_out,
                   int H, int k, int64_t P, cudaStream_t stream, int act, float* raw_out) {
  const int chunk = 16;
  const int64_t tasks = (P + chunk - 1) / chunk;
  const int64_t want = (tasks + 7) / 8;
  const int64_t cap = static_cast<int64_t>(device_sm_count()) * 8;
  const int grid = static_cast<int>(want < cap ? (want > 0 ? want : 1) : cap);
  expert_scores_kernel<T, NCH><<<grid, 256, 0, stream>>>(static_cast<const T*>(x), static_cast<const T*>(down),
                                                         w.sorted_pair, w.sorted_expert, w.offsets + N,
                                                         static_cast<const T*>(gates), gs_out, H, k, chunk, act, raw_out);
}

template <typename T, typename OutT, int NCH>
void launch_accum(const void* up, const int64_t* idx, const float* gs, void* out, int64_t T_, int H, int64_t N, int k,
                  cudaStream_t stream) {
  constexpr int VEC = Vec16<T>::N;
  const int colblocks = (H + 32 * VEC * NCH - 1) / (32 * VEC * NCH);
  const int64_t tasks = T_ * colblocks;
  const int64_t want = (tasks + 3) / 4;
  const int64_t cap = static_cast<int64_t>(device_sm_count()) * 16;
  const int grid = static_cast<int>(want < cap ? (want > 0 ? want : 1) : cap);
  auto kern = expert_accum_kernel<T, OutT, NCH>;
  (void)launch_pdl(8, kern, dim3(grid), dim3(128), 0, stream, 1, static_cast<const T*>(up), idx, gs, static_cast<OutT*>(out), T_,
                   H, N, k, colblocks, nullptr, 1, 0);  // launch errors surface through the caller's launch check
}

// 16-bit tables are gathered per token (no sort, tensor-core dot products) whatever their size: measured against
// the expert-centric order at 2^16 experts x 131072 tokens (3.07 vs 3.94 ms) and at 2^20 experts with Zipf ids
// (0.54 vs 0.83 ms; uniform ids 1.23 vs 1.16 ms).  float32 takes the expert-centric order.
// debugging / measurement aid: FMOE_EXPERT_SCHEDULE=token|sorted|fused forces one schedule for 16-bit tables (read
// once per process; `fused` only where that kernel applies); anything else leaves the default choice
int forced_schedule() {
  static const int forced = [] {
    const char* v = std::getenv("FMOE_EXPERT_SCHEDULE");
    if (v == nullptr) return 0;
    return v[0] == 't' ? 1 : (v[0] == 's' ? 2 : (v[0] == 'f' ? 3 : 0));
  }();
  return forced;
}

template <typename T> bool use_token_centric(int64_t N, int H) {
  if (sizeof(T) != 2) return false;
  if (forced_schedule() == 1 || forced_schedule() == 2) return forced_schedule() == 1;
  (void)N;
  (void)H;
  return true;
}

// counting sort of the (token, slot) pairs by expert id: w.offsets[0..N], w.sorted_pair, w.sorted_expert
int run_sort(const int64_t* idx, int64_t P, int64_t N, const ExpertWs& w, int32_t* status, cudaStream_t stream) {
  const int sms = device_sm_count();
  FMOE_CUDA_TRY(cudaMemsetAsync(w.counts, 0, static_cast<size_t>(N) * 4, stream));
  {
    const int64_t want = (P + 255) / 256;
    const int grid = static_cast<int>(want < sms * 8 ? want : sms * 8);
    expert_hist_kernel<<<grid, 256, 0, stream>>>(idx, P, N, w.counts, w.rank, status);
    FMOE_LAUNCH_CHECK();
  }
  {
    const int ntiles = static_cast<int>((N + kScanTile - 1) / kScanTile);
    if (ntiles > 16) {
      scan_tile_sums_kernel<<<ntiles, kScanThreads, 0, stream>>>(w.counts, N, w.tile_sums);
      FMOE_LAUNCH_CHECK();
      scan_apply_kernel<<<ntiles, kScanThreads, 0, stream>>>(w.counts, N, w.tile_sums, w.offsets);
    } else {
      scan_apply_kernel<<<ntiles, kScanThreads, 0, stream>>>(w.counts, N, nullptr, w.offsets);
    }
    FMOE_LAUNCH_CHECK();
  }
  {
    const int64_t want = (P + 255) / 256;
    const int grid = static_cast<int>(want < sms * 8 ? want : sms * 8);
    expert_scatter_kernel<<<grid, 256, 0, stream>>>(idx, w.rank, w.offsets, P, w.sorted_pair, w.sorted_expert);
    FMOE_LAUNCH_CHECK();
  }
  return FMOE_OK;
}

// per-pair dot products <rows[t], table[e]>: gates != nullptr stores silu(dot) * gate (forward), nullptr the
// raw dot product.  `sorted` says whether run_sort has filled w for these indices.
template <typename T>
int run_scores(const void* rows, const void* table, const int64_t* idx, const void* gates, float* out, int64_t T_, int H,
               int64_t N, int k, const ExpertWs& w, bool sorted, int32_t* status, cudaStream_t stream, int act = 0,
               float* raw_out = nullptr) {
  constexpr int VEC = Vec16<T>::N;
  const int64_t P = T_ * k;
  const int sms = device_sm_count();
  const int need = (H + 32 * VEC - 1) / (32 * VEC);
  if (use_token_centric<T>(N, H)) {
    if constexpr (sizeof(T) == 2) {
      const int64_t want = (T_ * ((k + 15) / 16) + 3) / 4;
      // exactly the CTAs that are resident at once (four per SM at 121 registers): every warp walks its tasks with
      // the next one's ids and x row already in flight, and the work ends evenly (53.7 vs 55.7 us with 16 per SM)
      const int64_t cap = static_cast<int64_t>(sms) * 4;
      const int grid = static_cast<int>(want < cap ? want : cap);
      const int xs_stride = ((H + 255) / 256) * 32;  // uint4 per warp, rows padded to 256 columns
      const int smem = 4 * 2 * xs_stride * 16;  // two x-row buffers per warp
      auto kern = expert_scores_mma_kernel<T, 4, false, 2>;
      if (smem > 48 * 1024) FMOE_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      FMOE_CUDA_TRY(launch_pdl(4, kern, dim3(grid), dim3(128), smem, stream, 1, static_cast<const T*>(rows),
                               static_cast<const T*>(table), idx, static_cast<const T*>(gates), out, T_, H, N, k, xs_stride,
                               status, act, nullptr, 1, raw_out, 0));
    }
    return FMOE_OK;
  }
  if (!sorted) {
    const int rc = run_sort(idx, P, N, w, status, stream);
    if (rc != FMOE_OK) return rc;
  }
  if (need <= 1) launch_scores<T, 1>(rows, table, w, N, gates, out, H, k, P, stream, act, raw_out);
  else if (need <= 2) launch_scores<T, 2>(rows, table, w, N, gates, out, H, k, P, stream, act, raw_out);
  else if (need <= 4) launch_scores<T, 4>(rows, table, w, N, gates, out, H, k, P, stream, act, raw_out);
  else if (need <= 8) launch_scores<T, 8>(rows, table, w, N, gates, out, H, k, P, stream, act, raw_out);
  else launch_scores<T, 0>(rows, table, w, N, gates, out, H, k, P, stream, act, raw_out);
  FMOE_LAUNCH_CHECK();
  return FMOE_OK;
}

// out[t] = sum_j coef[t,j] * table[idx[t,j]] (float32 accumulation, one rounding)
template <typename T>
int run_accum(const void* table, const int64_t* idx, const float* coef, void* out, int out_f32, int64_t T_, int H,
              int64_t N, int k, cudaStream_t stream) {
  constexpr int VEC = Vec16<T>::N;
  const int need = (H + 32 * VEC - 1) / (32 * VEC);
#define FMOE_ACCUM(NCH_)                                                                       \
  do {                                                                                         \
    if (out_f32) launch_accum<T, float, NCH_>(table, idx, coef, out, T_, H, N, k, stream);     \
    else launch_accum<T, T, NCH_>(table, idx, coef, out, T_, H, N, k, stream);                 \
  } while (0)
  // narrow column blocks: more warps per token, i.e. more gathers in flight
  if (need <= 1) FMOE_ACCUM(1);
  else FMOE_ACCUM(2);
#undef FMOE_ACCUM
  FMOE_LAUNCH_CHECK();
  return FMOE_OK;
}

template <typename T>
int run_typed(const void* x, const void* down, const void* up, const int64_t* idx, const void* gates, void* out,
              int out_f32, int64_t T_, int H, int64_t N, int k, const ExpertWs& w, int32_t* status,
              cudaStream_t stream, void* const* between_passes, int act, float* raw_scores, int dtype) {
  auto mark_between = [&]() -> int {
    if (between_passes != nullptr)
      for (int i = 0; i < 2; ++i)
        if (between_passes[i] != nullptr)
          FMOE_CUDA_TRY(cudaEventRecord(static_cast<cudaEvent_t>(between_passes[i]), stream));
    return FMOE_OK;
  };
  // The fused kernel pays off once the tables are far larger than L2 (its deep ring of asynchronous copies covers
  // the DRAM latency: 0.71 vs 0.93 ms at 2^20 experts x 2048); while they sit in L2 the two passes are faster
  // (110 vs 162 us at 2^14 experts x 1024), so tables below 1 GiB each take the two-pass path.
  const bool big_tables = static_cast<double>(N) * H * sizeof(T) >= 1073741824.0;
  const bool want_fused = forced_schedule() == 3 || (forced_schedule() == 0 && big_tables);
  if (sizeof(T) == 2 && want_fused && expert_fused_supported(dtype, T_, H, k)) {
    // one kernel for both steps: the marks that separate the two passes fall in front of it
    const int rc = mark_between();
    if (rc != FMOE_OK) return rc;
    return launch_expert_fused(x, down, up, idx, gates, out, dtype, out_f32, T_, H, N, k, act, raw_scores, status, stream);
  }
  int rc = run_scores<T>(x, down, idx, gates, w.gs, T_, H, N, k, w, false, status, stream, act, raw_scores);
  if (rc != FMOE_OK) return rc;
  if ((rc = mark_between()) != FMOE_OK) return rc;
  return run_accum<T>(up, idx, w.gs, out, out_f32, T_, H, N, k, stream);
}

// ---------------------------------------------------------------- backward
// Gradients of out[t] = sum_j silu(s_tj) * g_tj * U[e_tj], s_tj = <x[t], D[e_tj]>
// (flash_moe/ops/triton/flash_expert.py:214-525, host side :653-745):
//   q_tj  = <dout[t], U[e]>                      dg_tj = q * silu(s)
//   ds_tj = q * g * silu'(s)                     dx[t] = sum_j ds_tj * D[e]
//   dD[e] = sum_{pairs of e} ds * x[t]           dU[e] = sum_{pairs of e} silu(s) * g * dout[t]
// s is recomputed (nothing but the forward's inputs is saved).  All sums are float32 in a fixed order with one
// rounding on store: no atomics (the reference scatters with atomics), run-to-run deterministic.
constexpr int kBwdChunk = 64;  // sorted pairs per warp task of the table-gradient pass

// The forward's counting sort orders the pairs of one expert by atomic arrival, which is fine for per-pair
// results but would make the order of the gradient sums vary from run to run.  The backward therefore sorts
// (expert id, pair id) with a stable radix sort (CUB, from the CUDA toolkit headers): pairs of one expert end up
// in ascending pair id, skipped ids (key N) at the end.
__global__ void expert_sort_keys_kernel(const int64_t* __restrict__ idx, int64_t P, int64_t N,
                                        unsigned* __restrict__ keys, int* __restrict__ vals, int* __restrict__ counts,
                                        int32_t* status) {
  bool bad = false;
  for (int64_t p = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; p < P;
       p += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t e = idx[p];
    const bool valid = e >= 0 && e < N;
    bad |= !valid && e != -1;
    keys[p] = valid ? static_cast<unsigned>(e) : static_cast<unsigned>(N);
    vals[p] = static_cast<int>(p);
    if (valid) atomicAdd(&counts[e], 1);  // integer counts: the result does not depend on the order
  }
  if (bad && status != nullptr) atomicOr(status, FMOE_STATUS_BAD_EXPERT_ID);
}

int key_bits(int64_t N) {
  int b = 1;
  while ((int64_t{1} << b) <= N) ++b;  // keys run from 0 to N inclusive
  return b;
}

size_t stable_sort_temp_bytes(int64_t P, int64_t N) {
  size_t bytes = 0;
  const cudaError_t e = cub::DeviceRadixSort::SortPairs(nullptr, bytes, static_cast<const unsigned*>(nullptr),
                                                        static_cast<unsigned*>(nullptr), static_cast<const int*>(nullptr),
                                                        static_cast<int*>(nullptr), static_cast<int>(P), 0, key_bits(N));
  if (e != cudaSuccess) {  // no device to ask (host-only size query): a bound that covers CUB's histograms
    (void)cudaGetLastError();
    bytes = static_cast<size_t>(P) * 8 + (size_t{4} << 20);
  }
  return bytes;
}

// in: s_in (raw <x, D>; may alias s_ds), q (raw <dout, U>), gates.  out: s_ds = ds, gs = silu(s) * g (over q), dgates.
template <typename T>
__global__ void expert_bwd_pairs_kernel(const float* s_in, float* s_ds, float* __restrict__ q_gs,
                                        const T* __restrict__ gates, const int64_t* __restrict__ idx, int64_t N,
                                        T* __restrict__ dgates, int64_t P) {
  for (int64_t p = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; p < P;
       p += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t e = idx[p];
    if (e < 0 || e >= N) {  // a skipped pair contributes nothing and receives no gradient
      s_ds[p] = 0.f;
      q_gs[p] = 0.f;
      dgates[p] = from_f32<T>(0.f);
      continue;
    }
    const float s = s_in[p], q = q_gs[p], g = to_f32<T>(gates[p]);
    const float sig = __fdividef(1.0f, 1.0f + __expf(-s));
    const float act = s * sig;
    s_ds[p] = q * g * (sig * (1.0f + s * (1.0f - sig)));
    q_gs[p] = act * g;
    dgates[p] = from_f32<T>(q * act);
  }
}

// One warp per (chunk of kBwdChunk sorted pairs, block of 32*VEC*NCH columns).  The warp walks its pairs in sorted
// order with the running sums of the current expert's two gradient rows in registers.  A row whose pairs all lie
// inside the chunk is stored directly; otherwise the partial sum goes to `partial` (slot 0: the expert began in an
// earlier chunk, slot 1: it began here and continues) and expert_bwd_finish_kernel adds the pieces in chunk order.
template <typename T, int NCH>
__global__ void __launch_bounds__(128) expert_bwd_tables_kernel(
    const T* __restrict__ x, const T* __restrict__ dout, const float* __restrict__ ds, const float* __restrict__ gs,
    const int* __restrict__ sorted_pair, const int* __restrict__ sorted_expert, const int* __restrict__ offsets,
    int64_t N, T* __restrict__ ddown, T* __restrict__ dup, float* __restrict__ partial_d, float* __restrict__ partial_u,
    int H, int k, int colblocks) {
  constexpr int VEC = Vec16<T>::N;
  const int lane = threadIdx.x & 31;
  const int64_t warps_total = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int total = offsets[N];
  const int64_t nchunks = (total + kBwdChunk - 1) / kBwdChunk;
  for (int64_t task = warp_global; task < nchunks * colblocks; task += warps_total) {
    const int64_t chunk = task / colblocks;
    const int cb = static_cast<int>(task - chunk * colblocks);
    const int col0 = cb * (32 * VEC * NCH);
    const int pos0 = static_cast<int>(chunk * kBwdChunk);
    const int pos1 = min(pos0 + kBwdChunk, total);
    bool in[NCH];
#pragma unroll
    for (int c = 0; c < NCH; ++c) in[c] = col0 + (c * 32 + lane) * VEC < H;
    uint64_t ad[NCH][VEC / 2], au[NCH][VEC / 2];  // packed pairs of float32 sums (fma.rn.f32x2)
#pragma unroll
    for (int c = 0; c < NCH; ++c)
#pragma unroll
      for (int i = 0; i < VEC / 2; ++i) ad[c][i] = au[c][i] = 0ull;

    int cur_e = sorted_expert[pos0];
    bool began_earlier = offsets[cur_e] < pos0;
    // flush the running sums of expert e: final row, or a partial sum for the finishing pass
    auto flush = [&](int e, bool partial, int slot) {
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        const int col = col0 + (c * 32 + lane) * VEC;
        if (!in[c]) continue;
        float fd[VEC], fu[VEC];
#pragma unroll
        for (int i = 0; i < VEC / 2; ++i) {
          unpack_f32x2(ad[c][i], fd[2 * i], fd[2 * i + 1]);
          unpack_f32x2(au[c][i], fu[2 * i], fu[2 * i + 1]);
          ad[c][i] = au[c][i] = 0ull;
        }
        if (partial) {
          float* pd = partial_d + (chunk * 2 + slot) * H + col;
          float* pu = partial_u + (chunk * 2 + slot) * H + col;
#pragma unroll
          for (int i = 0; i < VEC; i += 4) {
            *reinterpret_cast<float4*>(pd + i) = make_float4(fd[i], fd[i + 1], fd[i + 2], fd[i + 3]);
            *reinterpret_cast<float4*>(pu + i) = make_float4(fu[i], fu[i + 1], fu[i + 2], fu[i + 3]);
          }
        } else {
          *reinterpret_cast<uint4*>(ddown + static_cast<int64_t>(e) * H + col) = pack16<T>(fd);
          *reinterpret_cast<uint4*>(dup + static_cast<int64_t>(e) * H + col) = pack16<T>(fu);
        }
      }
    };

    uint4 xn[NCH], on[NCH];
    int p_next = sorted_pair[pos0];
    {
      const int64_t t = p_next / k;
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        const int col = col0 + (c * 32 + lane) * VEC;
        xn[c] = in[c] ? ldg16(x + t * H + col) : make_uint4(0, 0, 0, 0);
        on[c] = in[c] ? ldg16(dout + t * H + col) : make_uint4(0, 0, 0, 0);
      }
    }
    for (int pos = pos0; pos < pos1; ++pos) {
      const int p = p_next;
      const int e = sorted_expert[pos];
      uint4 xq[NCH], oq[NCH];
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        xq[c] = xn[c];
        oq[c] = on[c];
      }
      if (pos + 1 < pos1) {  // issue the next pair's row gathers before this pair's math
        p_next = sorted_pair[pos + 1];
        const int64_t t = p_next / k;
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          const int col = col0 + (c * 32 + lane) * VEC;
          xn[c] = in[c] ? ldg16(x + t * H + col) : make_uint4(0, 0, 0, 0);
          on[c] = in[c] ? ldg16(dout + t * H + col) : make_uint4(0, 0, 0, 0);
        }
      }
      if (e != cur_e) {  // warp-uniform: cur_e ends inside this chunk
        flush(cur_e, began_earlier, 0);
        cur_e = e;
        began_earlier = false;
      }
      const float wd = ds[p], wu = gs[p];
      const uint64_t wd2 = pack_f32x2(wd, wd), wu2 = pack_f32x2(wu, wu);
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        float xf[VEC], of[VEC];
        unpack16<T>(xq[c], xf);
        unpack16<T>(oq[c], of);
#pragma unroll
        for (int i = 0; i < VEC / 2; ++i) {
          ffma2(ad[c][i], pack_f32x2(xf[2 * i], xf[2 * i + 1]), wd2);
          ffma2(au[c][i], pack_f32x2(of[2 * i], of[2 * i + 1]), wu2);
        }
      }
    }
    const bool continues = offsets[cur_e + 1] > pos1;
    flush(cur_e, began_earlier || continues, began_earlier ? 0 : 1);
  }
}

// One CTA per expert: rows of experts without pairs are zeroed, rows of experts whose pairs span several chunks are
// the sum of their partial rows in chunk order; rows stored directly by the pass above are left alone.
template <typename T>
__global__ void __launch_bounds__(256) expert_bwd_finish_kernel(const int* __restrict__ offsets, int64_t N,
                                                                const float* __restrict__ partial_d,
                                                                const float* __restrict__ partial_u,
                                                                T* __restrict__ ddown, T* __restrict__ dup, int H) {
  constexpr int VEC = Vec16<T>::N;
  for (int64_t e = blockIdx.x; e < N; e += gridDim.x) {
    const int b = offsets[e], en = offsets[e + 1];
    T* rd = ddown + e * H;
    T* ru = dup + e * H;
    if (b == en) {
      for (int col = threadIdx.x * VEC; col < H; col += blockDim.x * VEC) {
        *reinterpret_cast<uint4*>(rd + col) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(ru + col) = make_uint4(0, 0, 0, 0);
      }
      continue;
    }
    const int c0 = b / kBwdChunk, c1 = (en - 1) / kBwdChunk;
    if (c0 == c1) continue;
    for (int col = threadIdx.x * VEC; col < H; col += blockDim.x * VEC) {
      float sd[VEC], su[VEC];
#pragma unroll
      for (int i = 0; i < VEC; ++i) sd[i] = su[i] = 0.f;
      for (int c = c0; c <= c1; ++c) {
        const int64_t row = static_cast<int64_t>(c) * 2 + (c == c0 ? 1 : 0);
        const float* pd = partial_d + row * H + col;
        const float* pu = partial_u + row * H + col;
#pragma unroll
        for (int i = 0; i < VEC; i += 4) {
          const float4 a = *reinterpret_cast<const float4*>(pd + i);
          const float4 u = *reinterpret_cast<const float4*>(pu + i);
          sd[i] += a.x; sd[i + 1] += a.y; sd[i + 2] += a.z; sd[i + 3] += a.w;
          su[i] += u.x; su[i + 1] += u.y; su[i + 2] += u.z; su[i + 3] += u.w;
        }
      }
      *reinterpret_cast<uint4*>(rd + col) = pack16<T>(sd);
      *reinterpret_cast<uint4*>(ru + col) = pack16<T>(su);
    }
  }
}

// Tables sharded over the GPUs of one node, rows of the other GPUs read through peer pointers: the two gather
// kernels of the per-token schedule with the row address computed from (e % world, e / world).
// hot_down / hot_up (nullable, hot_rows rows): tables replicated on every GPU, addressed by the ids N .. N + hot_rows - 1
template <typename T>
int run_typed_peer(const void* x, const void* const* down_shards, const void* const* up_shards, int world,
                   const int64_t* idx, const void* gates, void* out, int out_f32, int64_t T_, int H, int64_t N, int k,
                   const ExpertWs& w, int32_t* status, cudaStream_t stream, const void* hot_down, const void* hot_up,
                   int64_t hot_rows) {
  if constexpr (sizeof(T) != 2) {
    return FMOE_ERR_UNSUPPORTED;
  } else {
    constexpr int VEC = Vec16<T>::N;
    const int sms = device_sm_count();
    {
      const int64_t want = (T_ * ((k + 15) / 16) + 3) / 4;
      const int64_t cap = static_cast<int64_t>(sms) * 16;
      const int grid = static_cast<int>(want < cap ? want : cap);
      const int xs_stride = ((H + 255) / 256) * 32;
      const int smem = 4 * 2 * xs_stride * 16;  // two x-row buffers per warp
      auto kern = expert_scores_mma_kernel<T, 4, true, 2>;
      if (smem > 48 * 1024) FMOE_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      kern<<<grid, 128, smem, stream>>>(static_cast<const T*>(x), static_cast<const T*>(hot_down), idx,
                                        static_cast<const T*>(gates), w.gs, T_, H, N + hot_rows, k, xs_stride, status,
                                        kActSilu, reinterpret_cast<const T* const*>(down_shards), world, nullptr, N);
      FMOE_LAUNCH_CHECK();
    }
    const int need = (H + 32 * VEC - 1) / (32 * VEC);
    const int nch = need <= 1 ? 1 : 2;
    const int colblocks = (H + 32 * VEC * nch - 1) / (32 * VEC * nch);
    const int64_t want = (T_ * colblocks + 3) / 4;
    const int64_t cap = static_cast<int64_t>(sms) * 16;
    const int grid = static_cast<int>(want < cap ? (want > 0 ? want : 1) : cap);
    const T* const* us = reinterpret_cast<const T* const*>(up_shards);
#define FMOE_PEER_ACCUM(OUT_, NCH_)                                                                            \
  expert_accum_kernel<T, OUT_, NCH_, true><<<grid, 128, 0, stream>>>(static_cast<const T*>(hot_up), idx, w.gs,    \
                                                                     static_cast<OUT_*>(out), T_, H, N + hot_rows, k, \
                                                                     colblocks, us, world, N)
    if (out_f32) {
      if (nch == 1) FMOE_PEER_ACCUM(float, 1);
      else FMOE_PEER_ACCUM(float, 2);
    } else {
      if (nch == 1) FMOE_PEER_ACCUM(T, 1);
      else FMOE_PEER_ACCUM(T, 2);
    }
#undef FMOE_PEER_ACCUM
    FMOE_LAUNCH_CHECK();
    return FMOE_OK;
  }
}

template <typename T>
__global__ void weights_to_f32_kernel(const T* __restrict__ w, float* __restrict__ out, int64_t n) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    out[i] = to_f32<T>(w[i]);
}

template <typename T>
int run_weighted_rows(const void* values, const void* weights, const int64_t* idx, void* out, int64_t T_, int H,
                      int64_t N, int k, float* coef, cudaStream_t stream) {
  const int64_t P = T_ * k;
  const int64_t want = (P + 255) / 256;
  const int64_t cap = static_cast<int64_t>(device_sm_count()) * 8;
  weights_to_f32_kernel<T><<<static_cast<int>(want < cap ? want : cap), 256, 0, stream>>>(static_cast<const T*>(weights),
                                                                                          coef, P);
  FMOE_LAUNCH_CHECK();
  return run_accum<T>(values, idx, coef, out, sizeof(T) == 4 ? 1 : 0, T_, H, N, k, stream);
}

struct ExpertBwdWs {
  ExpertWs fwd;  // sort arrays; fwd.gs holds s, then ds
  float* q;      // <dout, U>, then silu(s) * g
  unsigned* keys_in;
  int* vals_in;
  void* sort_temp;
  size_t sort_temp_bytes;
  float* partial_d;
  float* partial_u;
  size_t bytes;
};

ExpertBwdWs carve_bwd(void* ws, int64_t T, int H, int64_t N, int k) {
  ExpertBwdWs w;
  w.fwd = carve(ws, T, N, k);
  size_t off = w.fwd.bytes;
  auto take = [&](size_t bytes) {
    void* p = ws ? static_cast<char*>(ws) + off : nullptr;
    off += align_up(bytes, 256);
    return p;
  };
  const int64_t P = T * k;
  const int64_t nchunks = (P + kBwdChunk - 1) / kBwdChunk;
  w.q = static_cast<float*>(take(static_cast<size_t>(P) * 4));
  w.keys_in = static_cast<unsigned*>(take(static_cast<size_t>(P) * 4));
  w.vals_in = static_cast<int*>(take(static_cast<size_t>(P) * 4));
  w.sort_temp_bytes = stable_sort_temp_bytes(P, N);
  w.sort_temp = take(w.sort_temp_bytes);
  w.partial_d = static_cast<float*>(take(static_cast<size_t>(nchunks) * 2 * H * 4));
  w.partial_u = static_cast<float*>(take(static_cast<size_t>(nchunks) * 2 * H * 4));
  w.bytes = off;
  return w;
}

template <typename T, int NCH>
void launch_bwd_tables(const void* x, const void* dout, const ExpertBwdWs& w, int64_t N, void* ddown, void* dup, int H,
                       int k, int64_t P, cudaStream_t stream) {
  constexpr int VEC = Vec16<T>::N;
  const int colblocks = (H + 32 * VEC * NCH - 1) / (32 * VEC * NCH);
  const int64_t tasks = ((P + kBwdChunk - 1) / kBwdChunk) * colblocks;
  const int64_t want = (tasks + 3) / 4;
  const int64_t cap = static_cast<int64_t>(device_sm_count()) * 16;
  const int grid = static_cast<int>(want < cap ? (want > 0 ? want : 1) : cap);
  expert_bwd_tables_kernel<T, NCH><<<grid, 128, 0, stream>>>(
      static_cast<const T*>(x), static_cast<const T*>(dout), w.fwd.gs, w.q, w.fwd.sorted_pair, w.fwd.sorted_expert,
      w.fwd.offsets, N, static_cast<T*>(ddown), static_cast<T*>(dup), w.partial_d, w.partial_u, H, k, colblocks);
}

template <typename T>
int run_backward(const void* dout, const void* x, const void* down, const void* up, const int64_t* idx,
                 const void* gates, void* dx, void* ddown, void* dup, void* dgates, int64_t T_, int H, int64_t N, int k,
                 const ExpertBwdWs& w, int32_t* status, cudaStream_t stream, const float* saved_scores) {
  constexpr int VEC = Vec16<T>::N;
  const int64_t P = T_ * k;
  const int sms = device_sm_count();
  int rc;
  {  // stable sort of the pairs by expert id + segment offsets
    FMOE_CUDA_TRY(cudaMemsetAsync(w.fwd.counts, 0, static_cast<size_t>(N) * 4, stream));
    const int64_t want = (P + 255) / 256;
    const int grid = static_cast<int>(want < sms * 8 ? want : sms * 8);
    expert_sort_keys_kernel<<<grid, 256, 0, stream>>>(idx, P, N, w.keys_in, w.vals_in, w.fwd.counts, status);
    FMOE_LAUNCH_CHECK();
    const int ntiles = static_cast<int>((N + kScanTile - 1) / kScanTile);
    if (ntiles > 16) {
      scan_tile_sums_kernel<<<ntiles, kScanThreads, 0, stream>>>(w.fwd.counts, N, w.fwd.tile_sums);
      FMOE_LAUNCH_CHECK();
      scan_apply_kernel<<<ntiles, kScanThreads, 0, stream>>>(w.fwd.counts, N, w.fwd.tile_sums, w.fwd.offsets);
    } else {
      scan_apply_kernel<<<ntiles, kScanThreads, 0, stream>>>(w.fwd.counts, N, nullptr, w.fwd.offsets);
    }
    FMOE_LAUNCH_CHECK();
    size_t need = 0;
    FMOE_CUDA_TRY(cub::DeviceRadixSort::SortPairs(nullptr, need, w.keys_in,
                                                  reinterpret_cast<unsigned*>(w.fwd.sorted_expert), w.vals_in,
                                                  w.fwd.sorted_pair, static_cast<int>(P), 0, key_bits(N), stream));
    if (need > w.sort_temp_bytes) return FMOE_ERR_WORKSPACE;
    size_t have = w.sort_temp_bytes;
    FMOE_CUDA_TRY(cub::DeviceRadixSort::SortPairs(w.sort_temp, have, w.keys_in,
                                                  reinterpret_cast<unsigned*>(w.fwd.sorted_expert), w.vals_in,
                                                  w.fwd.sorted_pair, static_cast<int>(P), 0, key_bits(N), stream));
  }
  if (saved_scores == nullptr) {  // s = <x, D[e]> was not kept by the forward: recompute it
    rc = run_scores<T>(x, down, idx, nullptr, w.fwd.gs, T_, H, N, k, w.fwd, true, status, stream);
    if (rc != FMOE_OK) return rc;
  }
  rc = run_scores<T>(dout, up, idx, nullptr, w.q, T_, H, N, k, w.fwd, true, status, stream);
  if (rc != FMOE_OK) return rc;
  {
    const int64_t want = (P + 255) / 256;
    const int grid = static_cast<int>(want < sms * 8 ? want : sms * 8);
    expert_bwd_pairs_kernel<T><<<grid, 256, 0, stream>>>(saved_scores != nullptr ? saved_scores : w.fwd.gs, w.fwd.gs, w.q,
                                                        static_cast<const T*>(gates), idx, N, static_cast<T*>(dgates), P);
    FMOE_LAUNCH_CHECK();
  }
  rc = run_accum<T>(down, idx, w.fwd.gs, dx, sizeof(T) == 4 ? 1 : 0, T_, H, N, k, stream);
  if (rc != FMOE_OK) return rc;
  const int need = (H + 32 * VEC - 1) / (32 * VEC);
  if (need <= 1) launch_bwd_tables<T, 1>(x, dout, w, N, ddown, dup, H, k, P, stream);
  else if (need <= 2) launch_bwd_tables<T, 2>(x, dout, w, N, ddown, dup, H, k, P, stream);
  else launch_bwd_tables<T, 4>(x, dout, w, N, ddown, dup, H, k, P, stream);
  FMOE_LAUNCH_CHECK();
  {
    const int64_t cap = static_cast<int64_t>(sms) * 16;
    const int grid = static_cast<int>(N < cap ? N : cap);
    expert_bwd_finish_kernel<T><<<grid, 256, 0, stream>>>(w.fwd.offsets, N, w.partial_d, w.partial_u,
                                                          static_cast<T*>(ddown), static_cast<T*>(dup), H);
    FMOE_LAUNCH_CHECK();
  }
  return FMOE_OK;
}

}  // namespace

size_t expert_workspace_bytes(int64_t T, int H, int64_t N, int k) {
  (void)H;
  if (T < 0 || N < 0 || k < 0) return 0;
  return carve(nullptr, T, N, k).bytes;
}

int launch_expert_forward(const void* x, const void* down, const void* up, const int64_t* indices, const void* gates,
                          void* out, int dtype, int out_dtype, int64_t T, int H, int64_t N, int k, void* ws,
                          size_t ws_bytes, int32_t* status, cudaStream_t stream, void* const* between_passes, int act,
                          float* raw_scores) {
  if (T < 0 || H <= 0 || N <= 0 || k < 0) return FMOE_ERR_BAD_ARG;
  if (act != kActSilu && act != kActGelu) return FMOE_ERR_BAD_ARG;
  if (out_dtype != dtype && out_dtype != FMOE_DTYPE_F32) return FMOE_ERR_BAD_ARG;
  if (T == 0) return FMOE_OK;
  if (x == nullptr || down == nullptr || up == nullptr || out == nullptr) return FMOE_ERR_BAD_ARG;
  if (k > 0 && (indices == nullptr || gates == nullptr)) return FMOE_ERR_BAD_ARG;
  if (N > 0x7FFFFFFFll || T * static_cast<int64_t>(k) > 0x7FFFFFFFll) return FMOE_ERR_UNSUPPORTED;
  const int vec = 16 / dtype_size(dtype);
  if (H % vec != 0) return FMOE_ERR_ALIGNMENT;
  if (!aligned16(x) || !aligned16(down) || !aligned16(up) || !aligned16(out)) return FMOE_ERR_ALIGNMENT;
  if (k == 0) {
    FMOE_CUDA_TRY(cudaMemsetAsync(out, 0, static_cast<size_t>(T) * H * dtype_size(out_dtype), stream));
    return FMOE_OK;
  }
  const ExpertWs w = carve(ws, T, N, k);
  if (ws == nullptr || ws_bytes < w.bytes) return FMOE_ERR_WORKSPACE;
  const int out_f32 = (out_dtype == FMOE_DTYPE_F32) ? 1 : 0;
  switch (dtype) {
    case FMOE_DTYPE_F32:
      return run_typed<float>(x, down, up, indices, gates, out, 1, T, H, N, k, w, status, stream, between_passes, act,
                              raw_scores, dtype);
    case FMOE_DTYPE_BF16:
      return run_typed<__nv_bfloat16>(x, down, up, indices, gates, out, out_f32, T, H, N, k, w, status, stream,
                                      between_passes, act, raw_scores, dtype);
    case FMOE_DTYPE_F16:
      return run_typed<__half>(x, down, up, indices, gates, out, out_f32, T, H, N, k, w, status, stream, between_passes,
                               act, raw_scores, dtype);
    default:
      return FMOE_ERR_BAD_ARG;
  }
}

size_t expert_backward_workspace_bytes(int64_t T, int H, int64_t N, int k) {
  if (T < 0 || N < 0 || k < 0 || H <= 0) return 0;
  return carve_bwd(nullptr, T, H, N, k).bytes;
}

int launch_expert_backward(const void* dout, const void* x, const void* down, const void* up, const int64_t* indices,
                           const void* gates, void* dx, void* ddown, void* dup, void* dgates, int dtype, int64_t T,
                           int H, int64_t N, int k, void* ws, size_t ws_bytes, int32_t* status, cudaStream_t stream,
                           const float* saved_scores) {
  if (T < 0 || H <= 0 || N <= 0 || k < 0) return FMOE_ERR_BAD_ARG;
  if (dx == nullptr || ddown == nullptr || dup == nullptr) return FMOE_ERR_BAD_ARG;
  if (N > 0x7FFFFFFFll || T * static_cast<int64_t>(k) > 0x7FFFFFFFll) return FMOE_ERR_UNSUPPORTED;
  const int vec = 16 / dtype_size(dtype);
  if (H % vec != 0) return FMOE_ERR_ALIGNMENT;
  if (!aligned16(dx) || !aligned16(ddown) || !aligned16(dup)) return FMOE_ERR_ALIGNMENT;
  const size_t table_bytes = static_cast<size_t>(N) * H * dtype_size(dtype);
  if (T == 0 || k == 0) {  // no pairs: every gradient is zero
    FMOE_CUDA_TRY(cudaMemsetAsync(ddown, 0, table_bytes, stream));
    FMOE_CUDA_TRY(cudaMemsetAsync(dup, 0, table_bytes, stream));
    if (T > 0) FMOE_CUDA_TRY(cudaMemsetAsync(dx, 0, static_cast<size_t>(T) * H * dtype_size(dtype), stream));
    return FMOE_OK;
  }
  if (dout == nullptr || x == nullptr || down == nullptr || up == nullptr || indices == nullptr || gates == nullptr ||
      dgates == nullptr)
    return FMOE_ERR_BAD_ARG;
  if (!aligned16(dout) || !aligned16(x) || !aligned16(down) || !aligned16(up)) return FMOE_ERR_ALIGNMENT;
  const ExpertBwdWs w = carve_bwd(ws, T, H, N, k);
  if (ws == nullptr || ws_bytes < w.bytes) return FMOE_ERR_WORKSPACE;
  switch (dtype) {
    case FMOE_DTYPE_F32:
      return run_backward<float>(dout, x, down, up, indices, gates, dx, ddown, dup, dgates, T, H, N, k, w, status, stream,
                                 saved_scores);
    case FMOE_DTYPE_BF16:
      return run_backward<__nv_bfloat16>(dout, x, down, up, indices, gates, dx, ddown, dup, dgates, T, H, N, k, w, status,
                                         stream, saved_scores);
    case FMOE_DTYPE_F16:
      return run_backward<__half>(dout, x, down, up, indices, gates, dx, ddown, dup, dgates, T, H, N, k, w, status, stream,
                                  saved_scores);
    default:
      return FMOE_ERR_BAD_ARG;
  }
}

int launch_weighted_rows(const void* values, const void* weights, const int64_t* indices, void* out, int dtype,
                         int64_t T, int H, int64_t N, int k, void* ws, size_t ws_bytes, int32_t* status,
                         cudaStream_t stream) {
  (void)status;  // ids outside [0, N) contribute nothing (the accumulate pass skips them)
  if (T < 0 || H <= 0 || N <= 0 || k < 0) return FMOE_ERR_BAD_ARG;
  if (T == 0) return FMOE_OK;
  if (values == nullptr || out == nullptr) return FMOE_ERR_BAD_ARG;
  if (T * static_cast<int64_t>(k) > 0x7FFFFFFFll) return FMOE_ERR_UNSUPPORTED;
  if (H % (16 / dtype_size(dtype)) != 0 || !aligned16(values) || !aligned16(out)) return FMOE_ERR_ALIGNMENT;
  if (k == 0) {
    FMOE_CUDA_TRY(cudaMemsetAsync(out, 0, static_cast<size_t>(T) * H * dtype_size(dtype), stream));
    return FMOE_OK;
  }
  if (weights == nullptr || indices == nullptr) return FMOE_ERR_BAD_ARG;
  const size_t need = static_cast<size_t>(T) * k * 4;
  if (ws == nullptr || ws_bytes < need) return FMOE_ERR_WORKSPACE;
  float* coef = static_cast<float*>(ws);
  switch (dtype) {
    case FMOE_DTYPE_F32: return run_weighted_rows<float>(values, weights, indices, out, T, H, N, k, coef, stream);
    case FMOE_DTYPE_BF16: return run_weighted_rows<__nv_bfloat16>(values, weights, indices, out, T, H, N, k, coef, stream);
    case FMOE_DTYPE_F16: return run_weighted_rows<__half>(values, weights, indices, out, T, H, N, k, coef, stream);
    default: return FMOE_ERR_BAD_ARG;
  }
}

int launch_expert_forward_peer(const void* x, const void* const* down_shards, const void* const* up_shards, int world,
                               const int64_t* indices, const void* gates, void* out, int dtype, int out_dtype, int64_t T,
                               int H, int64_t N, int k, void* ws, size_t ws_bytes, int32_t* status, cudaStream_t stream,
                               const void* hot_down, const void* hot_up, int64_t hot_rows) {
  if (T < 0 || H <= 0 || N <= 0 || k < 0 || world < 1 || hot_rows < 0) return FMOE_ERR_BAD_ARG;
  if (hot_rows > 0 && (hot_down == nullptr || hot_up == nullptr || !aligned16(hot_down) || !aligned16(hot_up)))
    return FMOE_ERR_BAD_ARG;
  if (out_dtype != dtype && out_dtype != FMOE_DTYPE_F32) return FMOE_ERR_BAD_ARG;
  if (dtype == FMOE_DTYPE_F32) return FMOE_ERR_UNSUPPORTED;
  if (T == 0) return FMOE_OK;
  if (x == nullptr || down_shards == nullptr || up_shards == nullptr || out == nullptr) return FMOE_ERR_BAD_ARG;
  if (k > 0 && (indices == nullptr || gates == nullptr)) return FMOE_ERR_BAD_ARG;
  if (N + hot_rows > 0x7FFFFFFFll || T * static_cast<int64_t>(k) > 0x7FFFFFFFll) return FMOE_ERR_UNSUPPORTED;
  if (H % 8 != 0 || !aligned16(x) || !aligned16(out)) return FMOE_ERR_ALIGNMENT;
  if (k == 0) {
    FMOE_CUDA_TRY(cudaMemsetAsync(out, 0, static_cast<size_t>(T) * H * dtype_size(out_dtype), stream));
    return FMOE_OK;
  }
  const ExpertWs w = carve(ws, T, N, k);
  if (ws == nullptr || ws_bytes < w.bytes) return FMOE_ERR_WORKSPACE;
  const int out_f32 = (out_dtype == FMOE_DTYPE_F32) ? 1 : 0;
  if (dtype == FMOE_DTYPE_BF16)
    return run_typed_peer<__nv_bfloat16>(x, down_shards, up_shards, world, indices, gates, out, out_f32, T, H, N, k, w,
                                         status, stream, hot_down, hot_up, hot_rows);
  if (dtype == FMOE_DTYPE_F16)
    return run_typed_peer<__half>(x, down_shards, up_shards, world, indices, gates, out, out_f32, T, H, N, k, w, status,
                                  stream, hot_down, hot_up, hot_rows);
  return FMOE_ERR_BAD_ARG;
}

}  // namespace fmoe
