// Fused fine-grained expert forward for 16-bit tables on sm_100a (one kernel instead of a scores pass and an
// accumulate pass):
//   out[t] = sum_j act(<x[t], D[e_tj]>) * g[t,j] * U[e_tj]      (flash_moe/ops/triton/flash_expert.py:13-211)
//
// What bounds this op is not HBM but the L2 -> SM path: every (token, expert) pair needs one down row and one up row
// (2 * H bytes each) on the SM that holds the token, whatever the schedule.  The rate an SM draws is
// (bytes in flight) / latency, so the rows are kept out of the register file: four producer warps stream them into a
// ring in shared memory with 16-byte asynchronous copies (cp.async global -> shared, whose completion arrives on an
// mbarrier), close to 200 KB in flight per SM, and eight consumer warps work from shared memory.  (One bulk copy
// per row - cp.async.bulk - was measured first: the copy engine handles about one 2 KB row per 60 ns per SM, 5 TB/s
// over the GPU against 15 TB/s for plain loads, so rows are fetched through the load/store path instead.)
//
// One persistent CTA per SM walks tokens t = blockIdx.x, blockIdx.x + gridDim.x, ...  Per token, in rounds of up to 64
// of its k slots (groups of 16 rows, one mbarrier pair per group):
//   producers x row -> xbuf; the round's down rows, then its up rows, group by group into the ring (the groups
//             are dealt to the producer warps round-robin);
//   scores    every consumer warp takes one eighth of the columns of each down group: the 16 rows are the A operand
//             of mma.sync.m16n8k16 (fp32 accumulate), its slice of the x row every column of B; the eight partial
//             dot products per slot meet in shared memory;
//   gates     gs = act(s) * gate per slot, kept in registers (two slots per lane) - it never leaves the SM;
//   sum       every consumer warp owns 128-column slices of the output row and adds gs * up row in fp32 (packed
//             f32x2 FMAs) in slot order: fixed order, one rounding on store, no atomics, bit-equal reruns.
// Ids outside [0, N) are skipped and flagged (-1: skipped silently) like in the two-pass kernels.
// Every mbarrier wait is bounded; a wait that runs out raises FMOE_STATUS_WAIT_TIMEOUT, the CTA finishes its loop
// without waiting any more (results are then garbage), waits for its copies in flight and exits.
#include "common.cuh"
#include "ptx_sm100.cuh"

namespace fmoe {
namespace {

constexpr unsigned kFull = 0xFFFFFFFFu;
constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kProducerWarps = 4;
constexpr int kThreads = kConsumerThreads + kProducerWarps * 32;
constexpr int kGroupRows = 16;                   // rows per ring group = M of the MMA
constexpr int kRoundSlots = 64;                  // slots of one token handled per round (two per lane)
constexpr int kMaxGroups = 16;                   // ring depth limit (barrier array size)
constexpr int kSmemLimit = 227 * 1024;
constexpr uint64_t kWaitLimitNs = 1000000000ull;

struct FusedLayout {
  int stride;       // bytes between rows of a group (row + padding; = 64 mod 128 so that 16-byte reads of 8 rows x 4
                    // column pieces hit distinct banks)
  int group_bytes;  // kGroupRows * stride
  int groups;       // ring depth
  int xbuf_bytes;   // one x row, padded
  int off_x, off_part, off_bar, total;
};

FusedLayout fused_layout(int H) {
  FusedLayout L;
  const int row = 2 * H;
  L.stride = row + ((64 - row % 128) + 128) % 128;
  L.group_bytes = kGroupRows * L.stride;
  L.xbuf_bytes = static_cast<int>(align_up(static_cast<size_t>(row), 128));
  const int fixed = 2 * L.xbuf_bytes + 2 * kConsumerWarps * kRoundSlots * 4 + (2 * kMaxGroups + 4) * 8 + 128;
  int g = (kSmemLimit - fixed) / L.group_bytes;
  L.groups = g > kMaxGroups ? kMaxGroups : g;
  L.off_x = L.groups * L.group_bytes;
  L.off_part = L.off_x + 2 * L.xbuf_bytes;
  L.off_bar = L.off_part + 2 * kConsumerWarps * kRoundSlots * 4;
  L.total = L.off_bar + (2 * kMaxGroups + 4) * 8 + 128;
  return L;
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)) : "memory");
}
// this thread arrives on `bar` once all its cp.async issued so far have landed (the barrier's count includes it)
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
// one row copied by the 32 lanes of a warp: lane l takes the 16-byte pieces l, l + 32, ... (NB of them; H <= 256 * NB)
template <typename T, int NB>
__device__ __forceinline__ void copy_row(uint32_t dst, const T* src, int H, int lane) {
#pragma unroll
  for (int j = 0; j < NB; ++j) {
    const int col = (j * 32 + lane) * 8;
    if (col < H) cp_async16(dst + col * 2, src + col);
  }
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ void consumer_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory"); }

// mbarrier wait for the warps of this kernel: polls with a short sleep between attempts, so that the (up to twelve)
// waiting warps of a CTA leave the issue slots to the ones that have work; bounded like ptx::mbar_wait_bounded
__device__ __forceinline__ bool ring_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (ptx::mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = ptx::globaltimer_ns();
  for (uint32_t it = 1; it < (1u << 28); ++it) {
    __nanosleep(40);
    if (ptx::mbar_try_wait(bar, parity)) return true;
    if ((it & 255u) == 0u) {
      if (*abort_flag) return false;
      if (ptx::globaltimer_ns() - t0 > kWaitLimitNs) break;
    }
  }
  *abort_flag = 1;
  return false;
}

// Consumer-side wait: only the first consumer warp polls the mbarrier; the other seven sleep in a hardware barrier
// (bar.sync costs no issue slots while blocked) and are released together with it.  With all eight warps polling,
// about half of the kernel's issued instructions were polls; removing them did not change the kernel's duration,
// which is set by the in-order hand-over of ring slots, not by issue slots.
__device__ __forceinline__ void consumer_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int warp) {
  if (warp == 0) ring_wait(bar, parity, abort_flag);
  asm volatile("bar.sync 2, %0;" ::"n"(kConsumerThreads) : "memory");
}

template <typename T> struct MmaK16;
template <> struct MmaK16<__nv_bfloat16> {
  static __device__ __forceinline__ void run(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
};
template <> struct MmaK16<__half> {
  static __device__ __forceinline__ void run(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
};

template <typename T> __device__ __forceinline__ void unpack8(const uint2& q, float (&f)[4]);
template <> __device__ __forceinline__ void unpack8<__nv_bfloat16>(const uint2& q, float (&f)[4]) {
  f[0] = __uint_as_float(q.x << 16);
  f[1] = __uint_as_float(q.x & 0xFFFF0000u);
  f[2] = __uint_as_float(q.y << 16);
  f[3] = __uint_as_float(q.y & 0xFFFF0000u);
}
template <> __device__ __forceinline__ void unpack8<__half>(const uint2& q, float (&f)[4]) {
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&q.x));
  const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&q.y));
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ void fma2(uint64_t& acc, uint64_t a, uint64_t b) {
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(a), "l"(b));
}

// NB: 32-column blocks of the x row per consumer warp in the scores step (8 * 32 * NB >= H);
// NS: 128-column slices of the output row per consumer warp in the sum step (8 * 128 * NS >= H).
template <typename T, typename OutT, int NB, int NS>
__global__ void __launch_bounds__(kThreads, 1)
expert_fused_kernel(const T* __restrict__ x, const T* __restrict__ down, const T* __restrict__ up,
                    const int64_t* __restrict__ idx, const T* __restrict__ gates, OutT* __restrict__ out,
                    float* __restrict__ raw_out, int64_t ntok, int H, int64_t N, int k, int act, int32_t* status,
                    int stride, int group_bytes, int groups, int off_x, int xbuf_bytes, int off_part, int off_bar) {
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t ring = ptx::smem_u32(smem);
  const uint32_t xbuf = ring + off_x;
  float* part = reinterpret_cast<float*>(smem + off_part);  // [2][kConsumerWarps][kRoundSlots]
  const uint32_t bars = ring + off_bar;
  auto full_bar = [&](int s) { return bars + s * 8; };
  auto empty_bar = [&](int s) { return bars + (kMaxGroups + s) * 8; };
  auto xfull_bar = [&](int b) { return bars + (2 * kMaxGroups + b) * 8; };
  auto xempty_bar = [&](int b) { return bars + (2 * kMaxGroups + 2 + b) * 8; };
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + off_bar + (2 * kMaxGroups + 4) * 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < groups; ++s) {
      ptx::mbar_init(full_bar(s), 32);               // every lane of the producer warp that filled the group
      ptx::mbar_init(empty_bar(s), kConsumerWarps);  // one arrive per consumer warp
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(xfull_bar(b), 32);
      ptx::mbar_init(xempty_bar(b), kConsumerWarps);
    }
    *abort_flag = 0;
    ptx::mbar_fence_init();
  }
  __syncthreads();

  const int rounds = (k + kRoundSlots - 1) / kRoundSlots;

  if (warp >= kConsumerWarps) {
    // ------------------------------------------------------------------ producer warps
    // Every producer warp walks the same sequence of groups and fills those with q % np == its number.  np <= groups:
    // a warp that waits for a slot has then seen the slot's previous use released, so the parity it waits for is
    // never two phases ahead of the barrier.
    const int pw = warp - kConsumerWarps;
    const int np = groups < kProducerWarps ? groups : kProducerWarps;
    bool bad = false;
    uint32_t q = 0;    // groups so far (ring position and phase follow from it)
    uint32_t ti = 0;   // tokens started so far
    // ids of the slots lane and lane + 32 of a round
    auto load_ids = [&](int64_t t, int r, int64_t& e_lo, int64_t& e_hi) {
      const int n = min(kRoundSlots, k - r * kRoundSlots);
      const int64_t* p = idx + t * k + r * kRoundSlots;
      e_lo = lane < n ? p[lane] : 0;
      e_hi = lane + 32 < n ? p[lane + 32] : 0;
    };
    int64_t t = blockIdx.x;
    int64_t e_lo = 0, e_hi = 0;
    if (t < ntok) load_ids(t, 0, e_lo, e_hi);
    for (; t < ntok; t += gridDim.x, ++ti) {
      if (pw == 0) {  // x rows stay with one warp: their two buffers are then filled in order
        const int b = ti & 1u;
        ring_wait(xempty_bar(b), ((ti >> 1) & 1u) ^ 1u, abort_flag);
        copy_row<T, NB>(xbuf + b * xbuf_bytes, x + t * H, H, lane);
        cp_async_arrive(xfull_bar(b));
      }
      for (int r = 0; r < rounds; ++r) {
        const int n = min(kRoundSlots, k - r * kRoundSlots);
        const int ng = (n + kGroupRows - 1) / kGroupRows;
        // validate this round's ids; fetch the next round's (or next token's) while this one is issued
        const bool ok_lo = e_lo >= 0 && e_lo < N, ok_hi = e_hi >= 0 && e_hi < N;
        bad |= (lane < n && !ok_lo && e_lo != -1) || (lane + 32 < n && !ok_hi && e_hi != -1);
        const int64_t row_lo = ok_lo ? e_lo : 0, row_hi = ok_hi ? e_hi : 0;
        if (r + 1 < rounds) load_ids(t, r + 1, e_lo, e_hi);
        else if (t + gridDim.x < ntok) load_ids(t + gridDim.x, 0, e_lo, e_hi);
#pragma unroll 1
        for (int pass = 0; pass < 2; ++pass) {
          const T* table = pass == 0 ? down : up;
#pragma unroll 1
          for (int gi = 0; gi < ng; ++gi, ++q) {
            if (static_cast<int>(q % np) != pw) continue;
            const int s = q % groups;
            const uint32_t ph = (q / groups) & 1u;
            const int nrows = min(kGroupRows, n - gi * kGroupRows);
            ring_wait(empty_bar(s), ph ^ 1u, abort_flag);
            const uint32_t dst = ring + s * group_bytes;
            const int64_t mine = gi < 2 ? row_lo : row_hi;
            if (nrows == kGroupRows) {
#pragma unroll 4
              for (int rr = 0; rr < kGroupRows; ++rr) {
                const int64_t e = __shfl_sync(kFull, mine, (gi * kGroupRows + rr) & 31);
                copy_row<T, NB>(dst + rr * stride, table + e * H, H, lane);
              }
            } else {
              for (int rr = 0; rr < nrows; ++rr) {
                const int64_t e = __shfl_sync(kFull, mine, (gi * kGroupRows + rr) & 31);
                copy_row<T, NB>(dst + rr * stride, table + e * H, H, lane);
              }
            }
            cp_async_arrive(full_bar(s));
          }
        }
      }
    }
    cp_async_wait_all();  // nothing of this warp is in flight when the CTA's shared memory goes away
    if (bad && pw == 0 && status != nullptr) atomicOr(status, FMOE_STATUS_BAD_EXPERT_ID);
  } else {
    // ------------------------------------------------------------------ consumer warps
    const int g = lane >> 2, tq = lane & 3;
    const int kslice = NB * 32;  // columns of the x row this warp multiplies in the scores step
    uint32_t q = 0, ti = 0, step = 0;  // step: rounds done so far (picks the buffer of partial sums)
    for (int64_t t = blockIdx.x; t < ntok; t += gridDim.x, ++ti) {
      const int b = ti & 1u;
      // this warp's slice of the token's x row, as B fragments
      consumer_wait(xfull_bar(b), (ti >> 1) & 1u, abort_flag, warp);
      uint4 xf[NB];
#pragma unroll
      for (int i = 0; i < NB; ++i) {
        const int col = warp * kslice + 32 * i + 8 * tq;
        xf[i] = col < H ? lds128(xbuf + b * xbuf_bytes + col * 2) : make_uint4(0, 0, 0, 0);
      }
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(xempty_bar(b));

      uint64_t acc[NS][2];
#pragma unroll
      for (int i = 0; i < NS; ++i) acc[i][0] = acc[i][1] = 0ull;
      bool in[NS];
#pragma unroll
      for (int i = 0; i < NS; ++i) in[i] = (warp + kConsumerWarps * i) * 128 + 4 * lane < H;

      for (int r = 0; r < rounds; ++r, ++step) {
        const int n = min(kRoundSlots, k - r * kRoundSlots);
        const int ng = (n + kGroupRows - 1) / kGroupRows;
        const int64_t p0 = t * k + r * kRoundSlots;
        // ids and gates of this lane's two slots (needed after the scores step: latency hidden behind it)
        int64_t e_lo = -1, e_hi = -1;
        float g_lo = 0.f, g_hi = 0.f;
        if (lane < n) {
          e_lo = idx[p0 + lane];
          g_lo = to_f32<T>(gates[p0 + lane]);
        }
        if (lane + 32 < n) {
          e_hi = idx[p0 + lane + 32];
          g_hi = to_f32<T>(gates[p0 + lane + 32]);
        }
        // two buffers of partial sums, alternating per round: the barrier of round i + 1 separates the reads of
        // round i from the writes of round i + 2
        float* allpart = part + (step & 1u) * (kConsumerWarps * kRoundSlots);
        float* mypart = allpart + warp * kRoundSlots;

        // ---- scores: partial dot products of this warp's column slice for every down group
#pragma unroll 1
        for (int gi = 0; gi < ng; ++gi, ++q) {
          const int s = q % groups;
          consumer_wait(full_bar(s), (q / groups) & 1u, abort_flag, warp);
          const uint32_t ra = ring + s * group_bytes + g * stride;
          const uint32_t rb = ra + 8 * stride;
          float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
          uint4 qa[NB], qb[NB];
#pragma unroll
          for (int i = 0; i < NB; ++i) {
            const int col = warp * kslice + 32 * i + 8 * tq;
            qa[i] = qb[i] = make_uint4(0, 0, 0, 0);
            if (col < H) {
              qa[i] = lds128(ra + col * 2);
              qb[i] = lds128(rb + col * 2);
            }
          }
#pragma unroll
          for (int i = 0; i < NB; ++i) {
            MmaK16<T>::run(c0, qa[i].x, qb[i].x, qa[i].y, qb[i].y, xf[i].x, xf[i].y);
            MmaK16<T>::run(c1, qa[i].z, qb[i].z, qa[i].w, qb[i].w, xf[i].z, xf[i].w);
          }
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(empty_bar(s));
          if (tq == 0) {  // every accumulator column holds the same dot product: row g, row g + 8
            mypart[gi * kGroupRows + g] = c0[0] + c1[0];
            mypart[gi * kGroupRows + g + 8] = c0[2] + c1[2];
          }
        }
        consumer_barrier();

        // ---- gs = act(s) * gate for this lane's two slots (every warp computes all of them)
        float s_lo = 0.f, s_hi = 0.f;
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) {
          s_lo += allpart[w * kRoundSlots + lane];
          s_hi += allpart[w * kRoundSlots + lane + 32];
        }
        const bool ok_lo = lane < n && e_lo >= 0 && e_lo < N;
        const bool ok_hi = lane + 32 < n && e_hi >= 0 && e_hi < N;
        if (raw_out != nullptr && warp == 0) {  // pre-activation scores kept for the backward pass
          if (lane < n) raw_out[p0 + lane] = ok_lo ? s_lo : 0.f;
          if (lane + 32 < n) raw_out[p0 + lane + 32] = ok_hi ? s_hi : 0.f;
        }
        const float gs_lo = ok_lo ? expert_act(s_lo, act) * g_lo : 0.f;
        const float gs_hi = ok_hi ? expert_act(s_hi, act) * g_hi : 0.f;

        // ---- sum: acc += gs * up row over this warp's column slices, slot by slot
#pragma unroll 1
        for (int gi = 0; gi < ng; ++gi, ++q) {
          const int s = q % groups;
          const int nrows = min(kGroupRows, n - gi * kGroupRows);
          const float sel = gi < 2 ? gs_lo : gs_hi;
          const int src0 = (gi & 1) * kGroupRows;
          consumer_wait(full_bar(s), (q / groups) & 1u, abort_flag, warp);
          const uint32_t base = ring + s * group_bytes + (warp * 128 + 4 * lane) * 2;
          // batches of 8 rows: all their shared-memory loads are issued before the first multiply-add, so the
          // load latency is paid once per batch and not once per row
#pragma unroll
          for (int r0 = 0; r0 < kGroupRows; r0 += 8) {
            if (r0 < nrows) {
              uint2 qv[8][NS];
#pragma unroll
              for (int rr = 0; rr < 8; ++rr)
#pragma unroll
                for (int i = 0; i < NS; ++i)
                  qv[rr][i] = (in[i] && r0 + rr < nrows) ? lds64(base + (r0 + rr) * stride + i * (kConsumerWarps * 256))
                                                         : make_uint2(0u, 0u);
#pragma unroll
              for (int rr = 0; rr < 8; ++rr) {
                float wv = __shfl_sync(kFull, sel, src0 + r0 + rr);
                if (r0 + rr >= nrows) wv = 0.f;  // slots past the end of a short group
                const uint64_t ww = pack2(wv, wv);
#pragma unroll
                for (int i = 0; i < NS; ++i) {
                  float f[4];
                  unpack8<T>(qv[rr][i], f);
                  fma2(acc[i][0], pack2(f[0], f[1]), ww);
                  fma2(acc[i][1], pack2(f[2], f[3]), ww);
                }
              }
            }
          }
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(empty_bar(s));
        }
      }

      // ---- one rounding, one store per output element
#pragma unroll
      for (int i = 0; i < NS; ++i) {
        if (!in[i]) continue;
        float f[4];
        unpack2(acc[i][0], f[0], f[1]);
        unpack2(acc[i][1], f[2], f[3]);
        OutT* o = out + t * H + (warp + kConsumerWarps * i) * 128 + 4 * lane;
        if constexpr (sizeof(OutT) == 4) {
          *reinterpret_cast<float4*>(o) = make_float4(f[0], f[1], f[2], f[3]);
        } else {
          __align__(8) OutT h[4] = {from_f32<OutT>(f[0]), from_f32<OutT>(f[1]), from_f32<OutT>(f[2]), from_f32<OutT>(f[3])};
          *reinterpret_cast<uint2*>(o) = *reinterpret_cast<const uint2*>(h);
        }
      }
    }
  }

  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag != 0 && status != nullptr) atomicOr(status, FMOE_STATUS_WAIT_TIMEOUT);
}

template <typename T, typename OutT, int NB, int NS>
int launch_fused_nb(const void* x, const void* down, const void* up, const int64_t* idx, const void* gates, void* out,
                    float* raw_out, int64_t T_, int H, int64_t N, int k, int act, int32_t* status, cudaStream_t stream) {
  const FusedLayout L = fused_layout(H);
  auto kern = expert_fused_kernel<T, OutT, NB, NS>;
  FMOE_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L.total));
  const int sms = device_sm_count();
  const int grid = static_cast<int>(T_ < sms ? T_ : sms);
  kern<<<grid, kThreads, L.total, stream>>>(static_cast<const T*>(x), static_cast<const T*>(down),
                                            static_cast<const T*>(up), idx, static_cast<const T*>(gates),
                                            static_cast<OutT*>(out), raw_out, T_, H, N, k, act, status, L.stride,
                                            L.group_bytes, L.groups, L.off_x, L.xbuf_bytes, L.off_part, L.off_bar);
  FMOE_LAUNCH_CHECK();
  return FMOE_OK;
}

template <typename T, typename OutT>
int launch_fused_out(const void* x, const void* down, const void* up, const int64_t* idx, const void* gates, void* out,
                     float* raw_out, int64_t T_, int H, int64_t N, int k, int act, int32_t* status,
                     cudaStream_t stream) {
  if (H <= 256) return launch_fused_nb<T, OutT, 1, 1>(x, down, up, idx, gates, out, raw_out, T_, H, N, k, act, status, stream);
  if (H <= 512) return launch_fused_nb<T, OutT, 2, 1>(x, down, up, idx, gates, out, raw_out, T_, H, N, k, act, status, stream);
  if (H <= 1024) return launch_fused_nb<T, OutT, 4, 1>(x, down, up, idx, gates, out, raw_out, T_, H, N, k, act, status, stream);
  return launch_fused_nb<T, OutT, 8, 2>(x, down, up, idx, gates, out, raw_out, T_, H, N, k, act, status, stream);
}

}  // namespace

// The fused kernel covers 16-bit tables whose rows fit the ring at least three groups deep and batches with at least
// one token per few SMs; everything else (float32, very wide rows, a handful of tokens) takes the two-pass kernels.
bool expert_fused_supported(int dtype, int64_t T, int H, int k) {
  if (dtype != FMOE_DTYPE_BF16 && dtype != FMOE_DTYPE_F16) return false;
  if (H % 8 != 0 || H > 2048 || k < 1 || T < 64) return false;
  return fused_layout(H).groups >= 3;
}

int launch_expert_fused(const void* x, const void* down, const void* up, const int64_t* idx, const void* gates,
                        void* out, int dtype, int out_f32, int64_t T, int H, int64_t N, int k, int act,
                        float* raw_scores, int32_t* status, cudaStream_t stream) {
  if (dtype == FMOE_DTYPE_BF16) {
    if (out_f32) return launch_fused_out<__nv_bfloat16, float>(x, down, up, idx, gates, out, raw_scores, T, H, N, k, act, status, stream);
    return launch_fused_out<__nv_bfloat16, __nv_bfloat16>(x, down, up, idx, gates, out, raw_scores, T, H, N, k, act, status, stream);
  }
  if (dtype == FMOE_DTYPE_F16) {
    if (out_f32) return launch_fused_out<__half, float>(x, down, up, idx, gates, out, raw_scores, T, H, N, k, act, status, stream);
    return launch_fused_out<__half, __half>(x, down, up, idx, gates, out, raw_scores, T, H, N, k, act, status, stream);
  }
  return FMOE_ERR_UNSUPPORTED;
}

}  // namespace fmoe
