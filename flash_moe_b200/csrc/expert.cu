// Fine-grained expert forward for sm_100a:
//   out[t] = sum_j silu(<x[t], D[e_tj]>) * g[t,j] * U[e_tj]
// (flash_moe/ops/triton/flash_expert.py:13-211, preprocessing :528-577).
//
// Two schedules, picked by table size
//   A. tables resident in L2 (16-bit dtypes): no sort.  Scores per token on the tensor cores
//      (mma.sync, groups of 16 gathered down rows against the token's x row), then the per-token
//      accumulate of step 3.
//   B. larger tables (and float32): expert-centric order of the (token, slot) pairs by a
//      device-side counting sort (histogram with warp-aggregated atomics -> exclusive scan ->
//      scatter; no host sync; ids outside [0, N) are dropped and flagged), then a scores pass over
//      the SORTED pairs: a warp walks a contiguous run of pairs, keeps the current expert's down
//      row in registers (loaded once per run of equal ids with 128-bit loads), gathers each pair's
//      x row and reduces the dot product in fp32; empty experts cost nothing, a hot expert is
//      split over many warps.
//   Both store gs = silu(s) * gate at the pair's (token, slot) position (4 bytes per pair).
//   3. accumulate pass per token: out[t] = sum_j gs[t,j] * U[e_tj] in fp32 (packed f32x2 FMAs),
//      fixed slot order, one rounding on store - no atomics, run-to-run deterministic.
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
    if (p < P && !valid) bad = true;
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
                                                           int k, int chunk) {
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
      if (lane == 0) gs[p] = silu_f32(acc) * to_f32<T>(gates[p]);
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

// One warp per (token, group of 16 of its experts).  The token's x row is parked in the warp's
// slice of shared memory (read back as B fragments right before each MMA), so every register that
// waits for data waits for a gathered down row: batches of UNROLL 32-column blocks keep
// 2 * UNROLL x 16 B per lane in flight to cover the L2 latency of the gather.
template <typename T, int UNROLL>
__global__ void __launch_bounds__(128) expert_scores_mma_kernel(const T* __restrict__ x, const T* __restrict__ down,
                                                               const int64_t* __restrict__ idx,
                                                               const T* __restrict__ gates, float* __restrict__ gs,
                                                               int64_t ntok, int H, int64_t N, int k, int xs_stride,
                                                               int32_t* status) {
  extern __shared__ uint4 xs_all[];
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2, tq = lane & 3;
  uint4* xs = xs_all + (threadIdx.x >> 5) * xs_stride;  // xs_stride uint4 per warp, >= ceil(H/256)*32
  const int64_t warps_total = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int groups = (k + 15) >> 4;
  const int64_t tasks = ntok * groups;
  const int hv = H >> 3;  // 16-byte pieces per row
  bool bad = false;
  int64_t t_in_smem = -1;
  for (int64_t task = warp_global; task < tasks; task += warps_total) {
    const int64_t t = task / groups;
    const int G = static_cast<int>(task - t * groups);
    const int ja = G * 16 + g, jb = ja + 8;
    int64_t ea = 0, eb = 0;
    if (ja < k) ea = idx[t * k + ja];
    if (jb < k) eb = idx[t * k + jb];
    const bool oka = (ja < k) && ea >= 0 && ea < N;
    const bool okb = (jb < k) && eb >= 0 && eb < N;
    if ((ja < k && !oka) || (jb < k && !okb)) bad = true;
    const T* ra = down + (oka ? ea : 0) * H + 8 * tq;
    const T* rb = down + (okb ? eb : 0) * H + 8 * tq;
    if (t != t_in_smem) {  // warp-uniform
      __syncwarp();
      const T* xr = x + t * H;
      for (int c = lane; c < xs_stride; c += 32) xs[c] = (c < hv) ? ldg16(xr + c * 8) : make_uint4(0, 0, 0, 0);
      __syncwarp();
      t_in_smem = t;
    }
    float c[4] = {0.f, 0.f, 0.f, 0.f};
    for (int c0 = 0; c0 < H; c0 += 32 * UNROLL) {
      uint4 qa[UNROLL], qb[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int col = c0 + 32 * u;
        const bool in = col + 8 * tq < H;
        qa[u] = in ? ldg16(ra + col) : make_uint4(0, 0, 0, 0);
        qb[u] = in ? ldg16(rb + col) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int piece = ((c0 + 32 * u) >> 3) + tq;
        const uint4 xq = piece < xs_stride ? xs[piece] : make_uint4(0, 0, 0, 0);
        Mma16816<T>::run(c, qa[u].x, qb[u].x, qa[u].y, qb[u].y, xq.x, xq.y);
        Mma16816<T>::run(c, qa[u].z, qb[u].z, qa[u].w, qb[u].w, xq.z, xq.w);
      }
    }
    if (tq == 0) {
      if (ja < k) gs[t * k + ja] = oka ? silu_f32(c[0]) * to_f32<T>(gates[t * k + ja]) : 0.f;
      if (jb < k) gs[t * k + jb] = okb ? silu_f32(c[2]) * to_f32<T>(gates[t * k + jb]) : 0.f;
    }
  }
  if (bad && status != nullptr) atomicOr(status, FMOE_STATUS_BAD_EXPERT_ID);
}

// ---------------------------------------------------------------- 3. per-token accumulate
// One warp per (token, column block of 32*VEC*NCH elements); 16 x 16 B of gathered rows in flight
// per lane, packed f32x2 FMAs (two accumulators per instruction).
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

template <typename T, typename OutT, int NCH>
__global__ void __launch_bounds__(128) expert_accum_kernel(const T* __restrict__ up, const int64_t* __restrict__ idx,
                                                          const float* __restrict__ gs, OutT* __restrict__ out,
                                                          int64_t ntok, int H, int64_t N, int k, int colblocks) {
  constexpr int VEC = Vec16<T>::N;
  constexpr int SLOTS = NCH >= 4 ? 4 : 8;
  const int lane = threadIdx.x & 31;
  const int64_t warps_total = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  const int64_t warp_global = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t tasks = ntok * colblocks;
  for (int64_t task = warp_global; task < tasks; task += warps_total) {
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
      // each lane fetches one slot's (expert id, weight); invalid or absent slots get weight 0
      const int j = j0 + lane;
      int e_l = 0;
      float w_l = 0.f;
      if (j < k) {
        const int64_t e = idx[t * k + j];
        if (e >= 0 && e < N) {
          e_l = static_cast<int>(e);
          w_l = gs[t * k + j];
        }
      }
      const int nslots = min(32, k - j0);
      for (int s = 0; s < nslots; s += SLOTS) {
        uint4 q[SLOTS][NCH];
        uint64_t ww[SLOTS];
#pragma unroll
        for (int u = 0; u < SLOTS; ++u) {
          const int e = __shfl_sync(kFull, e_l, s + u);
          const float w = __shfl_sync(kFull, w_l, s + u);
          ww[u] = pack_f32x2(w, w);
          const T* row = up + static_cast<int64_t>(e) * H + col0 + lane * VEC;
#pragma unroll
          for (int c = 0; c < NCH; ++c) q[u][c] = in[c] ? ldg16(row + c * 32 * VEC) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < SLOTS; ++u)
#pragma unroll
          for (int c = 0; c < NCH; ++c) {
            float f[VEC];
            unpack16<T>(q[u][c], f);
#pragma unroll
            for (int i = 0; i < VEC / 2; ++i) ffma2(acc[c][i], pack_f32x2(f[2 * i], f[2 * i + 1]), ww[u]);
          }
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
void launch_scores(const void* x, const void* down, const ExpertWs& w, int64_t N, const void* gates, int H, int k,
                   int64_t P, cudaStream_t stream) {
  const int chunk = 16;
  const int64_t tasks = (P + chunk - 1) / chunk;
  const int64_t want = (tasks + 7) / 8;
  const int64_t cap = static_cast<int64_t>(device_sm_count()) * 8;
  const int grid = static_cast<int>(want < cap ? (want > 0 ? want : 1) : cap);
  expert_scores_kernel<T, NCH><<<grid, 256, 0, stream>>>(static_cast<const T*>(x), static_cast<const T*>(down),
                                                         w.sorted_pair, w.sorted_expert, w.offsets + N,
                                                         static_cast<const T*>(gates), w.gs, H, k, chunk);
}

template <typename T, typename OutT, int NCH>
void launch_accum(const void* up, const int64_t* idx, const ExpertWs& w, void* out, int64_t T_, int H, int64_t N, int k,
                  cudaStream_t stream) {
  constexpr int VEC = Vec16<T>::N;
  const int colblocks = (H + 32 * VEC * NCH - 1) / (32 * VEC * NCH);
  const int64_t tasks = T_ * colblocks;
  const int64_t want = (tasks + 3) / 4;
  const int64_t cap = static_cast<int64_t>(device_sm_count()) * 16;
  const int grid = static_cast<int>(want < cap ? (want > 0 ? want : 1) : cap);
  expert_accum_kernel<T, OutT, NCH><<<grid, 128, 0, stream>>>(static_cast<const T*>(up), idx, w.gs,
                                                              static_cast<OutT*>(out), T_, H, N, k, colblocks);
}

template <typename T>
int run_typed(const void* x, const void* down, const void* up, const int64_t* idx, const void* gates, void* out,
              int out_f32, int64_t T_, int H, int64_t N, int k, const ExpertWs& w, int32_t* status,
              cudaStream_t stream, void* const* between_passes) {
  constexpr int VEC = Vec16<T>::N;
  const int64_t P = T_ * k;
  const int sms = device_sm_count();
  const int per_chunk = 32 * VEC;
  const int need = (H + per_chunk - 1) / per_chunk;
  // Tables that stay resident in the 126 MB L2 are gathered per token (no sort, tensor-core dot
  // products); larger tables take the expert-centric order so each down row leaves HBM once.
  const bool token_centric = sizeof(T) == 2 && (2.0 * static_cast<double>(N) * H * sizeof(T) <= 96.0 * 1024 * 1024);
  if (token_centric) {
    if constexpr (sizeof(T) == 2) {
      const int64_t want = (T_ * ((k + 15) / 16) + 3) / 4;
      const int64_t cap = static_cast<int64_t>(sms) * 16;
      const int grid = static_cast<int>(want < cap ? want : cap);
      const int xs_stride = ((H + 255) / 256) * 32;  // uint4 per warp, rows padded to 256 columns
      const int smem = 4 * xs_stride * 16;
      auto kern = expert_scores_mma_kernel<T, 8>;
      if (smem > 48 * 1024) FMOE_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      kern<<<grid, 128, smem, stream>>>(static_cast<const T*>(x), static_cast<const T*>(down), idx,
                                        static_cast<const T*>(gates), w.gs, T_, H, N, k, xs_stride, status);
      FMOE_LAUNCH_CHECK();
    }
  } else {
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
    if (need <= 1) launch_scores<T, 1>(x, down, w, N, gates, H, k, P, stream);
    else if (need <= 2) launch_scores<T, 2>(x, down, w, N, gates, H, k, P, stream);
    else if (need <= 4) launch_scores<T, 4>(x, down, w, N, gates, H, k, P, stream);
    else if (need <= 8) launch_scores<T, 8>(x, down, w, N, gates, H, k, P, stream);
    else launch_scores<T, 0>(x, down, w, N, gates, H, k, P, stream);
    FMOE_LAUNCH_CHECK();
  }
  if (between_passes != nullptr)
    for (int i = 0; i < 2; ++i)
      if (between_passes[i] != nullptr) FMOE_CUDA_TRY(cudaEventRecord(static_cast<cudaEvent_t>(between_passes[i]), stream));

#define FMOE_ACCUM(NCH_)                                                                       \
  do {                                                                                         \
    if (out_f32) launch_accum<T, float, NCH_>(up, idx, w, out, T_, H, N, k, stream);           \
    else launch_accum<T, T, NCH_>(up, idx, w, out, T_, H, N, k, stream);                       \
  } while (0)
  // narrow column blocks: more warps per token, i.e. more gathers in flight
  if (need <= 1) FMOE_ACCUM(1);
  else FMOE_ACCUM(2);
#undef FMOE_ACCUM
  FMOE_LAUNCH_CHECK();
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
                          size_t ws_bytes, int32_t* status, cudaStream_t stream, void* const* between_passes) {
  if (T < 0 || H <= 0 || N <= 0 || k < 0) return FMOE_ERR_BAD_ARG;
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
      return run_typed<float>(x, down, up, indices, gates, out, 1, T, H, N, k, w, status, stream, between_passes);
    case FMOE_DTYPE_BF16:
      return run_typed<__nv_bfloat16>(x, down, up, indices, gates, out, out_f32, T, H, N, k, w, status, stream,
                                      between_passes);
    case FMOE_DTYPE_F16:
      return run_typed<__half>(x, down, up, indices, gates, out, out_f32, T, H, N, k, w, status, stream,
                                      between_passes);
    default:
      return FMOE_ERR_BAD_ARG;
  }
}

}  // namespace fmoe
