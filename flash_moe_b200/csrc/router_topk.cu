// Product-key router top-k for sm_100a.
//
// For every token the reference evaluates all nk*nk sums lp0[i] + lp1[j] and extracts the k
// largest by k rounds of arg-max (flash_moe/ops/triton/flash_router.py:8-194).  This kernel gets
// the same answer - same scores, same indices, same order, including the order among equal
// scores (ascending flat id i*nk + j) - from far less work:
//
//   1. sort each half descending (value, then lower index first);
//   2. a candidate at ranks (p, q) (0-based) has (p+1)*(q+1)-1 candidates that score at least
//      as high, so only the "staircase" (p+1)*(q+1) <= k can hold a score above the k-th
//      largest; its ~k ln k sums are formed in the input dtype like the reference does;
//   3. tau = k-th largest staircase score, found by a bitwise search on order-preserving keys;
//      every candidate scoring above tau is inside the staircase and is emitted;
//   4. the remaining slots go to candidates scoring exactly tau with the lowest flat ids.  These
//      may lie outside the staircase, so they are located exactly: per row i a binary search in
//      the sorted second half counts its ties, then rows are visited in index order.
//   5. the k winners are sorted by (score desc, flat id asc) and written out, optionally with
//      gates = exp(score) (and the row renormalisation of flash_moe/modules/flash_moe.py:80-85).
//
// One warp owns one token; all scratch lives in shared memory.
#include <cstdlib>

#include "common.cuh"

namespace fmoe {
namespace {

constexpr unsigned kFull = 0xFFFFFFFFu;

template <typename T> struct OrdLowBits;  // low bits of the order key that carry no information
template <> struct OrdLowBits<float> { static constexpr int value = 0; };
template <> struct OrdLowBits<__nv_bfloat16> { static constexpr int value = 16; };
template <> struct OrdLowBits<__half> { static constexpr int value = 13; };

__device__ __forceinline__ uint64_t make_key(uint32_t ord, uint32_t id) {
  return (static_cast<uint64_t>(ord) << 32) | static_cast<uint64_t>(0xFFFFFFFFu - id);
}
__device__ __forceinline__ uint32_t key_id(uint64_t key) { return 0xFFFFFFFFu - static_cast<uint32_t>(key); }
__device__ __forceinline__ float key_val(uint64_t key) { return ord_to_f32(static_cast<uint32_t>(key >> 32)); }

// Warp-cooperative bitonic sort (descending) of one or two arrays of n = 2^m keys in shared memory.
__device__ __forceinline__ void bitonic_desc(uint64_t* a, uint64_t* b, int n, int lane) {
  for (int size = 2; size <= n; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = lane; i < (n >> 1); i += 32) {
        const int lo = ((i & ~(stride - 1)) << 1) | (i & (stride - 1));
        const int hi = lo | stride;
        const bool desc = (lo & size) == 0;
        uint64_t x = a[lo], y = a[hi];
        if ((x < y) == desc) { a[lo] = y; a[hi] = x; }
        if (b != nullptr) {
          x = b[lo]; y = b[hi];
          if ((x < y) == desc) { b[lo] = y; b[hi] = x; }
        }
      }
      __syncwarp();
    }
  }
}

struct RouterSmemLayout {
  int cta_bytes;   // staircase table + row starts (shared by the CTA)
  int warp_bytes;  // per-warp scratch
  int off_keys, off_win, off_cs, off_cnt;
  int nkp, kp, kq, C, Cp;
};

template <typename T>
__global__ void router_topk_smem_kernel(const T* __restrict__ logp, int64_t ntok, int nk, int k, RouterSmemLayout L,
                                   T* __restrict__ scores, int64_t* __restrict__ indices, T* __restrict__ gates,
                                   int norm) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int nwarps = blockDim.x >> 5;
  const int kq = L.kq, C = L.C, nkp = L.nkp, kp = L.kp;

  // ---- staircase table, built once per CTA: entry c -> (p << 16) | q with (p+1)(q+1) <= k
  uint32_t* pq = reinterpret_cast<uint32_t*>(smem);
  int* rowstart = reinterpret_cast<int*>(smem) + L.Cp;
  if (warp == 0) {
    int running = 0;
    for (int base = 0; base < kq; base += 32) {
      const int p = base + lane;
      const int len = (p < kq) ? min(k / (p + 1), kq) : 0;
      int incl = len;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int up = __shfl_up_sync(kFull, incl, d);
        if (lane >= d) incl += up;
      }
      if (p < kq) rowstart[p] = running + incl - len;
      running += __shfl_sync(kFull, incl, 31);
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < C; c += blockDim.x) {  // entry c lies in the last row whose start is <= c
    int lo = 0, hi = kq - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (rowstart[mid] <= c) lo = mid; else hi = mid - 1;
    }
    pq[c] = (static_cast<uint32_t>(lo) << 16) | static_cast<uint32_t>(c - rowstart[lo]);
  }
  __syncthreads();

  unsigned char* wbase = smem + L.cta_bytes + warp * L.warp_bytes;
  float* va = reinterpret_cast<float*>(wbase);
  float* vb = va + nk;
  uint64_t* ka = reinterpret_cast<uint64_t*>(wbase + L.off_keys);
  uint64_t* kb = ka + nkp;
  uint64_t* win = reinterpret_cast<uint64_t*>(wbase + L.off_win);
  uint32_t* cs = reinterpret_cast<uint32_t*>(wbase + L.off_cs);
  uint32_t* cnt = reinterpret_cast<uint32_t*>(wbase + L.off_cnt);
  constexpr int LOW = OrdLowBits<T>::value;

  for (int64_t t = static_cast<int64_t>(blockIdx.x) * nwarps + warp; t < ntok;
       t += static_cast<int64_t>(gridDim.x) * nwarps) {
    const T* a_row = logp + t * nk;
    const T* b_row = logp + (ntok + t) * nk;
    // 1. load (canonicalising -0 to +0) and build sort keys
    for (int i = lane; i < nkp; i += 32) {
      if (i < nk) {
        const float a = to_f32<T>(a_row[i]) + 0.0f;
        const float b = to_f32<T>(b_row[i]) + 0.0f;
        va[i] = a;
        vb[i] = b;
        ka[i] = make_key(f32_to_ord(a), i);
        kb[i] = make_key(f32_to_ord(b), i);
      } else {
        ka[i] = 0;
        kb[i] = 0;
      }
    }
    __syncwarp();
    bitonic_desc(ka, kb, nkp, lane);

    // 2. staircase candidate scores, rounded to T like the reference's in-dtype add
    for (int c = lane; c < C; c += 32) {
      const uint32_t e = pq[c];
      const float s = round_to<T>(__fadd_rn(key_val(ka[e >> 16]), key_val(kb[e & 0xFFFFu])));
      cs[c] = f32_to_ord(s + 0.0f);
    }
    __syncwarp();

    // 3. tau = k-th largest candidate score (bitwise search over the order key)
    uint32_t tau = 0;
    for (int bit = 31; bit >= LOW; --bit) {
      const uint32_t trial = tau | (1u << bit);
      int n_ge = 0;
      for (int c = lane; c < C; c += 32) n_ge += (cs[c] >= trial) ? 1 : 0;
      n_ge = __reduce_add_sync(kFull, n_ge);
      if (n_ge >= k) tau = trial;
    }
    if (LOW > 0 && (tau >> 31) == 0) tau |= (1u << LOW) - 1u;  // negative values: dropped bits are all ones

    // emit everything strictly above tau
    int filled = 0;
    for (int base = 0; base < C; base += 32) {
      const int c = base + lane;
      const bool g = (c < C) && (cs[c] > tau);
      const unsigned bal = __ballot_sync(kFull, g);
      if (g) {
        const int pos = filled + __popc(bal & ((1u << lane) - 1u));
        const uint32_t e = pq[c];
        const uint32_t flat = key_id(ka[e >> 16]) * static_cast<uint32_t>(nk) + key_id(kb[e & 0xFFFFu]);
        if (pos < k) win[pos] = make_key(cs[c], flat);
      }
      filled += __popc(bal);
    }
    int need = k - filled;

    // 4. candidates equal to tau, lowest flat id first.  Row i ties with sorted-b positions [gt, ge).
    for (int i = lane; i < nk; i += 32) {
      const float a = va[i];
      int lo = 0, hi = nk;
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (f32_to_ord(round_to<T>(__fadd_rn(a, key_val(kb[mid]))) + 0.0f) >= tau) lo = mid + 1; else hi = mid;
      }
      const int ge = lo;
      lo = 0; hi = ge;
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (f32_to_ord(round_to<T>(__fadd_rn(a, key_val(kb[mid]))) + 0.0f) > tau) lo = mid + 1; else hi = mid;
      }
      cnt[i] = static_cast<uint32_t>(ge - lo);
    }
    __syncwarp();
    for (int base = 0; base < nk && need > 0; base += 32) {
      const int i = base + lane;
      unsigned has = __ballot_sync(kFull, (i < nk) && (cnt[i] > 0));
      while (has != 0 && need > 0) {
        const int row = base + __ffs(has) - 1;
        has &= has - 1;
        const float a = va[row];
        for (int jb = 0; jb < nk && need > 0; jb += 32) {
          const int j = jb + lane;
          const bool tie = (j < nk) && (f32_to_ord(round_to<T>(__fadd_rn(a, vb[j])) + 0.0f) == tau);
          const unsigned bal = __ballot_sync(kFull, tie);
          const int rank = __popc(bal & ((1u << lane) - 1u));
          if (tie && rank < need)
            win[filled + rank] = make_key(tau, static_cast<uint32_t>(row) * static_cast<uint32_t>(nk) + j);
          const int took = min(__popc(bal), need);
          filled += took;
          need -= took;
        }
      }
    }
    for (int r = filled + lane; r < kp; r += 32) win[r] = 0;
    __syncwarp();

    // 5. order the winners and write out
    bitonic_desc(win, nullptr, kp, lane);
    float gsum = 0.f;
    for (int r = lane; r < k; r += 32) {
      const uint64_t key = win[r];
      const float s = key_val(key);
      scores[t * k + r] = from_f32<T>(s);
      indices[t * k + r] = static_cast<int64_t>(key_id(key));
      if (gates != nullptr) {
        const T g = from_f32<T>(expf(s));
        gsum += to_f32<T>(g);
        if (!norm) gates[t * k + r] = g;
      }
    }
    if (gates != nullptr && norm) {
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) gsum += __shfl_xor_sync(kFull, gsum, d);
      const float denom = round_to<T>(gsum);
      for (int r = lane; r < k; r += 32) {
        const float g = round_to<T>(expf(key_val(win[r])));
        gates[t * k + r] = from_f32<T>(g / denom);
      }
    }
    __syncwarp();
  }
}


// ------------------------------------------------------------------------------------------
// Register-resident variant for num_keys <= 1024: each half is sorted by a shuffle-based bitonic
// network (E = padded num_keys / 32 keys per lane), sort keys are 32-bit for 16-bit dtypes
// (16-bit order key | inverted index) and 64-bit for float32.  Shared memory only holds the
// sorted halves (for the candidate gathers and binary searches), the index-order values, the
// candidate scores and the winners.
// ------------------------------------------------------------------------------------------
template <typename T> struct HalfKey;  // sort key of one router half
template <> struct HalfKey<float> {
  using type = uint64_t;
  static __device__ __forceinline__ uint64_t make(float v, uint32_t i) { return make_key(f32_to_ord(v), i); }
  static __device__ __forceinline__ float value(uint64_t k) { return key_val(k); }
  static __device__ __forceinline__ uint32_t id(uint64_t k) { return key_id(k); }
};
template <typename T16> struct HalfKey16 {
  using type = uint32_t;
  static __device__ __forceinline__ uint32_t make(float v, uint32_t i) {
    const T16 h = from_f32<T16>(v);  // exact: v came from a T16
    uint32_t b = *reinterpret_cast<const uint16_t*>(&h);
    b ^= (b >> 15) ? 0xFFFFu : 0x8000u;
    return (b << 16) | (0xFFFFu - i);
  }
  static __device__ __forceinline__ float value(uint32_t k) {
    uint32_t b = k >> 16;
    b ^= (b >> 15) ? 0x8000u : 0xFFFFu;
    const uint16_t raw = static_cast<uint16_t>(b);
    return to_f32<T16>(*reinterpret_cast<const T16*>(&raw));
  }
  static __device__ __forceinline__ uint32_t id(uint32_t k) { return 0xFFFFu - (k & 0xFFFFu); }
};
template <> struct HalfKey<__nv_bfloat16> : HalfKey16<__nv_bfloat16> {};
template <> struct HalfKey<__half> : HalfKey16<__half> {};

__device__ __forceinline__ uint32_t shfl_xor_key(uint32_t v, int m) { return __shfl_xor_sync(kFull, v, m); }
__device__ __forceinline__ uint64_t shfl_xor_key(uint64_t v, int m) {
  return static_cast<uint64_t>(__shfl_xor_sync(kFull, static_cast<unsigned long long>(v), m));
}

// Descending bitonic sort of 32*E keys in the lane-blocked layout: element i = lane * E + r sits in a[r].  Strides
// below E exchange two registers of one lane (no shuffle: 15 shuffle stages for any E >= 1 instead of up to 35 with
// the keys dealt round-robin over the lanes); the direction of a block folds into the comparison predicate, so an
// exchange costs one compare and two selects per pair and a shuffle stage one shuffle, one compare and one select per key.
template <int E, typename K>
__device__ __forceinline__ void bitonic_desc_regs(K (&a)[E], int lane) {
  constexpr int n = 32 * E;
#pragma unroll
  for (int size = 2; size <= n; size <<= 1) {
#pragma unroll
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      if (stride >= E) {
        const int ls = stride / E;
        const bool desc = (size == n) || (((lane * E) & size) == 0);  // size >= 2 E here: decided by the lane
        const bool keep_max = ((lane & ls) == 0) == desc;
#pragma unroll
        for (int r = 0; r < E; ++r) {
          const K other = shfl_xor_key(a[r], ls);
          a[r] = ((other > a[r]) == keep_max) ? other : a[r];
        }
      } else {
#pragma unroll
        for (int r = 0; r < E; ++r) {
          if ((r & stride) == 0) {
            const bool desc = (size == n) || (size < E ? ((r & size) == 0) : (((lane * E) & size) == 0));
            const K x = a[r], y = a[r | stride];
            const bool sw = (x < y) == desc;
            a[r] = sw ? y : x;
            a[r | stride] = sw ? x : y;
          }
        }
      }
    }
  }
}

// One lane's E consecutive elements of a row (element lane * E + r -> v[r]); entries past nk read as -inf.  Whole
// rows of 32 E elements at a 16-byte aligned address are fetched with one or a few vector loads.
template <typename T, int E>
__device__ __forceinline__ void load_blocked(const T* __restrict__ row, int nk, int lane, float (&v)[E]) {
  constexpr int BYTES = E * static_cast<int>(sizeof(T));
  if (BYTES >= 4 && nk == 32 * E && (reinterpret_cast<uintptr_t>(row) & 15u) == 0) {
    __align__(16) T tmp[E];
    const T* src = row + lane * E;
    if constexpr (BYTES % 16 == 0) {
#pragma unroll
      for (int j = 0; j < BYTES / 16; ++j) reinterpret_cast<uint4*>(tmp)[j] = reinterpret_cast<const uint4*>(src)[j];
    } else if constexpr (BYTES == 8) {
      *reinterpret_cast<uint2*>(tmp) = *reinterpret_cast<const uint2*>(src);
    } else if constexpr (BYTES == 4) {
      *reinterpret_cast<uint32_t*>(tmp) = *reinterpret_cast<const uint32_t*>(src);
    }
#pragma unroll
    for (int r = 0; r < E; ++r) v[r] = to_f32<T>(tmp[r]);
  } else {
#pragma unroll
    for (int r = 0; r < E; ++r) {
      const int i = lane * E + r;
      v[r] = (i < nk) ? to_f32<T>(row[i]) : -INFINITY;
    }
  }
}

// One lane's E consecutive entries of a per-warp shared-memory array (16-byte aligned base, 32 E entries)
template <int E>
__device__ __forceinline__ void store_blocked(float* base, int lane, const float (&v)[E]) {
  float* dst = base + lane * E;
  if constexpr (E % 4 == 0) {
#pragma unroll
    for (int j = 0; j < E / 4; ++j)
      reinterpret_cast<float4*>(dst)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
  } else if constexpr (E == 2) {
    *reinterpret_cast<float2*>(dst) = make_float2(v[0], v[1]);
  } else {
#pragma unroll
    for (int r = 0; r < E; ++r) dst[r] = v[r];
  }
}
template <int E>
__device__ __forceinline__ void store_blocked(uint16_t* base, int lane, const uint32_t (&v)[E]) {  // v[r] < 65536
  uint16_t* dst = base + lane * E;
  if constexpr (E % 8 == 0) {
#pragma unroll
    for (int j = 0; j < E / 8; ++j)
      reinterpret_cast<uint4*>(dst)[j] =
          make_uint4(v[8 * j] | (v[8 * j + 1] << 16), v[8 * j + 2] | (v[8 * j + 3] << 16),
                     v[8 * j + 4] | (v[8 * j + 5] << 16), v[8 * j + 6] | (v[8 * j + 7] << 16));
  } else if constexpr (E == 4) {
    *reinterpret_cast<uint2*>(dst) = make_uint2(v[0] | (v[1] << 16), v[2] | (v[3] << 16));
  } else if constexpr (E == 2) {
    *reinterpret_cast<uint32_t*>(dst) = v[0] | (v[1] << 16);
  } else {
#pragma unroll
    for (int r = 0; r < E; ++r) dst[r] = static_cast<uint16_t>(v[r]);
  }
}

constexpr int kTieCap = 256;  // entries of the per-warp list of candidates that tie with tau

struct RouterRegLayout {
  int cta_bytes, warp_bytes;
  int off_sorted, off_ids, off_win, off_cs, off_tl;
  int nkp, kp, kq, C, Cp;
};

// CPL > 0: the staircase candidates (at most 32 * CPL of them) stay in registers, CPL per lane, through the threshold
// search and the emit step, whose loops then have compile-time bounds and no shared-memory round trips between rounds.
template <typename T, int E, int CPL = 0>
__global__ void __launch_bounds__(256) router_topk_reg_kernel(const T* __restrict__ logp, int64_t ntok, int nk, int k,
                                                             RouterRegLayout L, T* __restrict__ scores,
                                                             int64_t* __restrict__ indices, T* __restrict__ gates,
                                                             int flags) {
  const int norm = flags & 1;
  const bool from_logits = (flags & 2) != 0;
  using HK = HalfKey<T>;
  using K = typename HK::type;
  extern __shared__ __align__(16) unsigned char smem[];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int nwarps = blockDim.x >> 5;
  const int kq = L.kq, C = L.C, nkp = L.nkp, kp = L.kp;

  uint32_t* pq = reinterpret_cast<uint32_t*>(smem);
  int* rowstart = reinterpret_cast<int*>(smem) + L.Cp;
  if (warp == 0) {
    int running = 0;
    for (int base = 0; base < kq; base += 32) {
      const int p = base + lane;
      const int len = (p < kq) ? min(k / (p + 1), kq) : 0;
      int incl = len;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int up = __shfl_up_sync(kFull, incl, d);
        if (lane >= d) incl += up;
      }
      if (p < kq) rowstart[p] = running + incl - len;
      running += __shfl_sync(kFull, incl, 31);
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < C; c += blockDim.x) {  // entry c lies in the last row whose start is <= c
    int lo = 0, hi = kq - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (rowstart[mid] <= c) lo = mid; else hi = mid - 1;
    }
    pq[c] = (static_cast<uint32_t>(lo) << 16) | static_cast<uint32_t>(c - rowstart[lo]);
  }
  __syncthreads();
  pdl_wait();  // the staircase table above depends on k alone; the logits come from the previous kernel

  unsigned char* wbase = smem + L.cta_bytes + warp * L.warp_bytes;
  float* va = reinterpret_cast<float*>(wbase);  // index order
  float* vb = va + nkp;
  float* sa = reinterpret_cast<float*>(wbase + L.off_sorted);  // sorted, descending
  float* sb = sa + nkp;
  uint16_t* ia = reinterpret_cast<uint16_t*>(wbase + L.off_ids);
  uint16_t* ib = ia + nkp;
  uint64_t* win = reinterpret_cast<uint64_t*>(wbase + L.off_win);
  uint32_t* cs = reinterpret_cast<uint32_t*>(wbase + L.off_cs);
  uint32_t* tl = reinterpret_cast<uint32_t*>(wbase + L.off_tl);  // flat ids of candidates equal to tau
  int* tcnt = reinterpret_cast<int*>(tl + kTieCap);
  constexpr int LOW = OrdLowBits<T>::value;
  int nsteps = 0;  // binary-search steps covering [0, nk]
  while ((1 << nsteps) <= nk) ++nsteps;

  for (int64_t t = static_cast<int64_t>(blockIdx.x) * nwarps + warp; t < ntok;
       t += static_cast<int64_t>(gridDim.x) * nwarps) {
    if (t + static_cast<int64_t>(gridDim.x) * nwarps >= ntok) pdl_launch_dependents();  // last token of this warp
    // from_logits: the input is the raw router logits [T, 2*nk]; the per-half log-softmax
    // (flash_moe/modules/flash_moe.py:72) is applied here, rounded to T like torch does
    const T* a_row = from_logits ? logp + t * 2 * nk : logp + t * nk;
    const T* b_row = from_logits ? a_row + nk : logp + (ntok + t) * nk;
    // 1. per half: load (lane-blocked: element lane * E + r in register r), optional log-softmax, keep the
    //    index-order copy, sort in registers, store the rank-order values and ids.  The two halves run through ONE copy
    //    of this code (the loop is not unrolled): the unrolled sorting network is most of the kernel's instructions -
    //    at 16 keys per lane two copies alone exceed 70 KB - and only one half's keys are live at a time.
    //    Measured, 16384 tokens x 512 keys top-128 | 16384 x 1024 top-16 | 131072 x 256 top-32 | 4096 x 128 top-64 (us):
    //    this form 330 | 532 | 559 | 21.5; both halves unrolled side by side 348 | 663 | 539 | 22.5; keys dealt round-robin
    //    over the lanes (r * 32 + lane, 25-35 shuffle stages) unrolled side by side 304 | 584 | 803 | 25.6, in one copy
    //    476 | 962 - with 16 or 32 keys per lane few warps are resident and the two halves' independent chains hide
    //    each other's latency, which the single copy gives up and the smaller code buys back.
#pragma unroll 1
    for (int h = 0; h < 2; ++h) {
      const T* row = h == 0 ? a_row : b_row;
      float* vh = h == 0 ? va : vb;
      float* sh = h == 0 ? sa : sb;
      uint16_t* ih = h == 0 ? ia : ib;
      K key[E];
      float lv[E];
      load_blocked<T, E>(row, nk, lane, lv);
      if (from_logits) {
        float m = -INFINITY;
#pragma unroll
        for (int r = 0; r < E; ++r) m = fmaxf(m, lv[r]);
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(kFull, m, d));
        float sum = 0.f;
#pragma unroll
        for (int r = 0; r < E; ++r)
          if (lane * E + r < nk) sum += expf(lv[r] - m);
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(kFull, sum, d);
        const float lg = logf(sum);
#pragma unroll
        for (int r = 0; r < E; ++r) lv[r] = round_to<T>((lv[r] - m) - lg);
      }
#pragma unroll
      for (int r = 0; r < E; ++r) {
        const int i = lane * E + r;
        lv[r] += 0.0f;  // -0 -> +0
        key[r] = (i < nk) ? HK::make(lv[r], i) : K(0);
      }
      store_blocked<E>(vh, lane, lv);  // index order (entries past nk are never read)
      bitonic_desc_regs<E, K>(key, lane);
      uint32_t idr[E];
#pragma unroll
      for (int r = 0; r < E; ++r) {
        lv[r] = HK::value(key[r]);
        idr[r] = HK::id(key[r]) & 0xFFFFu;
      }
      store_blocked<E>(sh, lane, lv);  // rank order
      store_blocked<E>(ih, lane, idr);
    }
    __syncwarp();

    // 2. staircase candidate scores; track the smallest to narrow the threshold search
    uint32_t cmin = 0xFFFFFFFFu;
    uint32_t csr[CPL > 0 ? CPL : 1], pqr[CPL > 0 ? CPL : 1];
    if constexpr (CPL > 0) {
#pragma unroll
      for (int j = 0; j < CPL; ++j) {
        const int c = 32 * j + lane;
        const bool in = c < C;
        const uint32_t e = in ? pq[c] : 0u;
        const uint32_t o = f32_to_ord(round_to<T>(__fadd_rn(sa[e >> 16], sb[e & 0xFFFFu])) + 0.0f);
        pqr[j] = e;
        csr[j] = in ? o : 0u;  // 0 is below the key of every float, -inf included
        if (in) {
          cs[c] = o;  // the tie search below looks up single cells
          cmin = min(cmin, o);
        }
      }
    } else {
      for (int c = lane; c < C; c += 32) {
        const uint32_t e = pq[c];
        const uint32_t o = f32_to_ord(round_to<T>(__fadd_rn(sa[e >> 16], sb[e & 0xFFFFu])) + 0.0f);
        cs[c] = o;
        cmin = min(cmin, o);
      }
    }
    cmin = __reduce_min_sync(kFull, cmin);
    __syncwarp();
    const uint32_t cmax = cs[0];  // ranks (0, 0): the largest sum

    // 3. tau = k-th largest candidate; all candidates agree on the bits above the top differing one
    uint32_t tau = cmax;
    if (cmax != cmin) {
      const int top = 31 - __clz(cmax ^ cmin);
      tau = cmax & ~((2u << top) - 1u);
      for (int bit = top; bit >= LOW; --bit) {
        const uint32_t trial = tau | (1u << bit);
        int n_ge = 0;
        if constexpr (CPL > 0) {
#pragma unroll
          for (int j = 0; j < CPL; ++j) n_ge += (csr[j] >= trial) ? 1 : 0;
        } else {
          for (int c = lane; c < C; c += 32) n_ge += (cs[c] >= trial) ? 1 : 0;
        }
        n_ge = __reduce_add_sync(kFull, n_ge);
        if (n_ge >= k) tau = trial;
      }
      if (LOW > 0 && (tau >> 31) == 0) tau |= (1u << LOW) - 1u;
    }

    // emit everything above tau; collect the staircase candidates equal to tau in the tie list
    int filled = 0, nties = 0;
    auto emit = [&](int c, uint32_t v, uint32_t e, bool known) {
      const bool g = (c < C) && (v > tau);
      const bool eq = (c < C) && (v == tau);
      const unsigned bal = __ballot_sync(kFull, g);
      const unsigned beq = __ballot_sync(kFull, eq);
      if (g || eq) {
        if (!known) e = pq[c];
        const uint32_t flat = static_cast<uint32_t>(ia[e >> 16]) * static_cast<uint32_t>(nk) + ib[e & 0xFFFFu];
        if (g) {
          const int pos = filled + __popc(bal & ((1u << lane) - 1u));
          if (pos < k) win[pos] = make_key(v, flat);
        } else {
          const int pos = nties + __popc(beq & ((1u << lane) - 1u));
          if (pos < kTieCap) tl[pos] = flat;
        }
      }
      filled += __popc(bal);
      nties += __popc(beq);
    };
    if constexpr (CPL > 0) {
#pragma unroll
      for (int j = 0; j < CPL; ++j)
        if (32 * j < C) emit(32 * j + lane, csr[j], pqr[j], true);
    } else {
      for (int base = 0; base < C; base += 32) {
        const int c = base + lane;
        emit(c, (c < C) ? cs[c] : 0u, 0u, false);
      }
    }
    int need = k - filled;

    // 4. the remaining `need` slots go to the candidates equal to tau with the lowest flat ids.
    //    Outside the staircase every score is <= tau, and along a row (fixed rank p of the first
    //    half) the scores do not increase, so the ties outside the staircase are the runs that
    //    continue a row past its last staircase cell, plus runs from q = 0 in the rows below the
    //    staircase.  They are gathered in rank space into the tie list; if the list overflows, the
    //    exhaustive per-row search below takes over.
    if (lane == 0) *tcnt = nties;
    __syncwarp();
    for (int p = lane; p < kq; p += 32) {
      const int rs = rowstart[p];
      const int len = ((p + 1 < kq) ? rowstart[p + 1] : C) - rs;  // = min(k / (p + 1), kq) without the division
      if (len < nk && cs[rs + len - 1] >= tau) {
        const float a = sa[p];
        const uint32_t ida = static_cast<uint32_t>(ia[p]) * static_cast<uint32_t>(nk);
        for (int q = len; q < nk; ++q) {
          if (f32_to_ord(round_to<T>(__fadd_rn(a, sb[q])) + 0.0f) != tau) break;
          const int pos = atomicAdd(tcnt, 1);
          if (pos < kTieCap) tl[pos] = ida + ib[q];
        }
      }
    }
    {
      const float b0 = sb[0];
      for (int base = kq; base < nk; base += 32) {  // rows below the staircase: tie runs start at q = 0
        const int p = base + lane;
        const bool hit = (p < nk) && (f32_to_ord(round_to<T>(__fadd_rn(sa[p < nk ? p : 0], b0)) + 0.0f) == tau);
        if (hit) {
          const float a = sa[p];
          const uint32_t ida = static_cast<uint32_t>(ia[p]) * static_cast<uint32_t>(nk);
          for (int q = 0; q < nk; ++q) {
            if (f32_to_ord(round_to<T>(__fadd_rn(a, sb[q])) + 0.0f) != tau) break;
            const int pos = atomicAdd(tcnt, 1);
            if (pos < kTieCap) tl[pos] = ida + ib[q];
          }
        }
        if (__ballot_sync(kFull, hit) == 0u) break;  // the rows are sorted: no later row can tie
      }
    }
    __syncwarp();
    nties = *tcnt;
    __syncwarp();
    const bool tie_list_ok = nties <= kTieCap;
    if (tie_list_ok && need > 0 && nties <= 32) {
      // the usual case, a handful of ties: one id per lane, its rank among them by a round of shuffles
      const uint32_t id = lane < nties ? tl[lane] : 0xFFFFFFFFu;
      int rank = 0;
      for (int j = 0; j < nties; ++j) rank += (__shfl_sync(kFull, id, j) < id) ? 1 : 0;
      if (lane < nties && rank < need) win[filled + rank] = make_key(tau, id);
      filled += min(nties, need);
      need = k - filled;
    } else if (tie_list_ok && need > 0) {
      uint32_t phi = 0xFFFFFFFFu;  // ids <= phi are taken
      if (nties > need) {
        // phi = the need-th smallest id = the largest v with fewer than `need` ids below v
        uint32_t v = 0;
        const int topbit = 31 - __clz(static_cast<unsigned>(nk) * static_cast<unsigned>(nk));
        for (int bit = topbit; bit >= 0; --bit) {
          const uint32_t trial = v | (1u << bit);
          int below = 0;
          for (int i = lane; i < nties; i += 32) below += (tl[i] < trial) ? 1 : 0;
          below = __reduce_add_sync(kFull, below);
          if (below < need) v = trial;
        }
        phi = v;
      }
      for (int base = 0; base < nties; base += 32) {
        const int i = base + lane;
        const uint32_t id = (i < nties) ? tl[i] : 0xFFFFFFFFu;
        const bool take = (i < nties) && (id <= phi);
        const unsigned bal = __ballot_sync(kFull, take);
        if (take) win[filled + __popc(bal & ((1u << lane) - 1u))] = make_key(tau, id);
        filled += __popc(bal);
      }
      need = k - filled;
    }

    // 4b. overflow path (more than kTieCap ties, e.g. constant inputs): row i = r*32 + lane ties with
    //     sorted-b positions [gt, ge); rows are then visited in index order
    if (!tie_list_ok) {
    int lo_ge[E], hi_ge[E], lo_gt[E], hi_gt[E];
    float arow[E];
#pragma unroll
    for (int r = 0; r < E; ++r) {
      const int i = (r << 5) | lane;
      arow[r] = (i < nk) ? va[i] : 0.f;
      lo_ge[r] = 0; hi_ge[r] = (i < nk) ? nk : 0;
      lo_gt[r] = 0; hi_gt[r] = (i < nk) ? nk : 0;
    }
    for (int step = 0; step < nsteps; ++step) {
#pragma unroll
      for (int r = 0; r < E; ++r) {
        if (lo_ge[r] < hi_ge[r]) {
          const int mid = (lo_ge[r] + hi_ge[r]) >> 1;
          const uint32_t o = f32_to_ord(round_to<T>(__fadd_rn(arow[r], sb[mid])) + 0.0f);
          if (o >= tau) lo_ge[r] = mid + 1; else hi_ge[r] = mid;
        }
        if (lo_gt[r] < hi_gt[r]) {
          const int mid = (lo_gt[r] + hi_gt[r]) >> 1;
          const uint32_t o = f32_to_ord(round_to<T>(__fadd_rn(arow[r], sb[mid])) + 0.0f);
          if (o > tau) lo_gt[r] = mid + 1; else hi_gt[r] = mid;
        }
      }
    }
#pragma unroll
    for (int r = 0; r < E; ++r) {
      const int cnt = lo_ge[r] - lo_gt[r];
      unsigned has = __ballot_sync(kFull, cnt > 0);
      while (has != 0 && need > 0) {
        const int row = (r << 5) + __ffs(has) - 1;
        has &= has - 1;
        const float a = va[row];
        for (int jb = 0; jb < nk && need > 0; jb += 32) {
          const int j = jb + lane;
          const bool tie = (j < nk) && (f32_to_ord(round_to<T>(__fadd_rn(a, vb[j])) + 0.0f) == tau);
          const unsigned bal = __ballot_sync(kFull, tie);
          const int rank = __popc(bal & ((1u << lane) - 1u));
          if (tie && rank < need)
            win[filled + rank] = make_key(tau, static_cast<uint32_t>(row) * static_cast<uint32_t>(nk) + j);
          const int took = min(__popc(bal), need);
          filled += took;
          need -= took;
        }
      }
    }
    }  // overflow path
    for (int r = filled + lane; r < kp; r += 32) win[r] = 0;
    __syncwarp();

    // 5. order the winners (registers when they fit, shared memory otherwise) and write out
    if (sizeof(T) == 2 && kp == 64 && nk <= 256) {
      // 16-bit scores and 16-bit flat ids: sort 32-bit keys
      uint32_t w[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const uint64_t key = win[lane * 2 + r];
        w[r] = key == 0 ? 0u : static_cast<uint32_t>(HalfKey<T>::make(key_val(key), key_id(key)));
      }
      bitonic_desc_regs<2, uint32_t>(w, lane);
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const uint32_t key32 = w[r];
        const float sc = static_cast<float>(HalfKey<T>::value(static_cast<typename HalfKey<T>::type>(key32)));
        win[lane * 2 + r] = make_key(f32_to_ord(sc + 0.0f), HalfKey<T>::id(static_cast<typename HalfKey<T>::type>(key32)));
      }
    } else if (kp <= 32) {
      uint64_t w[1] = {lane < kp ? win[lane] : 0};
      bitonic_desc_regs<1, uint64_t>(w, lane);
      if (lane < kp) win[lane] = w[0];
    } else if (kp == 64) {
      uint64_t w[2] = {win[2 * lane], win[2 * lane + 1]};
      bitonic_desc_regs<2, uint64_t>(w, lane);
      win[2 * lane] = w[0]; win[2 * lane + 1] = w[1];
    } else if (kp == 128) {
      uint64_t w[4] = {win[4 * lane], win[4 * lane + 1], win[4 * lane + 2], win[4 * lane + 3]};
      bitonic_desc_regs<4, uint64_t>(w, lane);
      win[4 * lane] = w[0]; win[4 * lane + 1] = w[1]; win[4 * lane + 2] = w[2]; win[4 * lane + 3] = w[3];
    } else {
      bitonic_desc(win, nullptr, kp, lane);
    }
    __syncwarp();
    float gsum = 0.f;
    for (int r = lane; r < k; r += 32) {
      const uint64_t key = win[r];
      const float s = key_val(key);
      scores[t * k + r] = from_f32<T>(s);
      indices[t * k + r] = static_cast<int64_t>(key_id(key));
      if (gates != nullptr) {
        const T g = from_f32<T>(expf(s));
        gsum += to_f32<T>(g);
        if (!norm) gates[t * k + r] = g;
      }
    }
    if (gates != nullptr && norm) {
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) gsum += __shfl_xor_sync(kFull, gsum, d);
      const float denom = round_to<T>(gsum);
      for (int r = lane; r < k; r += 32) {
        const float g = round_to<T>(expf(key_val(win[r])));
        gates[t * k + r] = from_f32<T>(g / denom);
      }
    }
    __syncwarp();
  }
}

RouterRegLayout make_reg_layout(int nk, int k) {
  RouterRegLayout L{};
  L.nkp = next_pow2(nk) < 32 ? 32 : next_pow2(nk);
  L.kp = next_pow2(k);
  L.kq = k < nk ? k : nk;
  int C = 0;
  for (int p = 0; p < L.kq; ++p) C += (k / (p + 1) < L.kq) ? k / (p + 1) : L.kq;
  L.C = C;
  L.Cp = (C + 3) / 4 * 4;
  L.cta_bytes = static_cast<int>(align_up(static_cast<size_t>(L.Cp) * 4 + static_cast<size_t>(L.kq) * 4, 16));
  int off = 2 * L.nkp * 4;
  L.off_sorted = off;
  off += 2 * L.nkp * 4;
  L.off_ids = off;
  off += 2 * L.nkp * 2;
  off = static_cast<int>(align_up(off, 16));
  L.off_win = off;
  off += (L.kp < 32 ? 32 : L.kp) * 8;
  L.off_cs = off;
  off += L.Cp * 4;
  L.off_tl = off;
  off += (kTieCap + 4) * 4;
  L.warp_bytes = static_cast<int>(align_up(off, 16));
  return L;
}

template <typename T, int E, int CPL = 0>
int launch_reg_cpl(const void* logp, int64_t T_, int nk, int k, const RouterRegLayout& L, int warps, void* scores,
                   int64_t* indices, void* gates, int norm, cudaStream_t stream) {
  const int smem = L.cta_bytes + warps * L.warp_bytes;
  auto kern = router_topk_reg_kernel<T, E, CPL>;
  FMOE_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  int per_sm = 1;
  FMOE_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, warps * 32, smem));
  if (per_sm < 1) per_sm = 1;
  const int64_t want = (T_ + warps - 1) / warps;
  const int64_t cap = static_cast<int64_t>(device_sm_count()) * per_sm;
  const int grid = static_cast<int>(want < cap ? want : cap);
  FMOE_CUDA_TRY(launch_pdl(2, kern, dim3(grid), dim3(warps * 32), smem, stream, 1, static_cast<const T*>(logp), T_, nk, k, L,
                           static_cast<T*>(scores), indices, static_cast<T*>(gates), norm));
  return FMOE_OK;
}

// 16-bit dtypes with at least 128 keys per half (the shapes of real layers) keep the candidates in registers when
// there are at most 320 of them (top-k up to 64: 22.5 vs 23.4 us at 4096 tokens x 128 keys, 539 vs 629 us at
// 131072 x 256 keys, top-32); with 22 per lane (top-128) the shared-memory walk measured faster (348 vs 382 us)
template <typename T, int E>
int launch_reg(const void* logp, int64_t T_, int nk, int k, const RouterRegLayout& L, int warps, void* scores,
               int64_t* indices, void* gates, int norm, cudaStream_t stream) {
  const char* force = std::getenv("FMOE_TOPK_CANDIDATES");  // measurement aid: "smem" forces the shared-memory walk
  const bool in_regs = force == nullptr || force[0] != 's';
  if constexpr (sizeof(T) == 2 && E >= 4) {
    if (!in_regs) return launch_reg_cpl<T, E, 0>(logp, T_, nk, k, L, warps, scores, indices, gates, norm, stream);
    if (L.C <= 32 * 4) return launch_reg_cpl<T, E, 4>(logp, T_, nk, k, L, warps, scores, indices, gates, norm, stream);
    if (L.C <= 32 * 10) return launch_reg_cpl<T, E, 10>(logp, T_, nk, k, L, warps, scores, indices, gates, norm, stream);
  }
  return launch_reg_cpl<T, E, 0>(logp, T_, nk, k, L, warps, scores, indices, gates, norm, stream);
}

// register kernel when the halves fit 32 keys per lane and the per-warp scratch stays small
template <typename T>
int launch_typed(const void* logp, int64_t T_, int nk, int k, void* scores, int64_t* indices, void* gates, int norm,
                 cudaStream_t stream);

RouterSmemLayout make_layout(int nk, int k) {
  RouterSmemLayout L{};
  L.nkp = next_pow2(nk);
  L.kp = next_pow2(k);
  L.kq = k < nk ? k : nk;
  int C = 0;
  for (int p = 0; p < L.kq; ++p) C += (k / (p + 1) < L.kq) ? k / (p + 1) : L.kq;
  L.C = C;
  L.Cp = (C + 3) / 4 * 4;
  L.cta_bytes = static_cast<int>(align_up(static_cast<size_t>(L.Cp) * 4 + static_cast<size_t>(L.kq) * 4, 16));
  int off = 2 * nk * 4;
  off = static_cast<int>(align_up(off, 16));
  L.off_keys = off;
  off += 2 * L.nkp * 8;
  L.off_win = off;
  off += L.kp * 8;
  L.off_cs = off;
  off += L.Cp * 4;
  L.off_cnt = off;
  off += nk * 4;
  L.warp_bytes = static_cast<int>(align_up(off, 16));
  return L;
}

template <typename T>
int launch_smem(const void* logp, int64_t T_, int nk, int k, void* scores, int64_t* indices, void* gates, int norm,
                 cudaStream_t stream) {
  const RouterSmemLayout L = make_layout(nk, k);
  constexpr int kMaxSmem = 227 * 1024;
  int warps = 8;
  while (warps > 1 && L.cta_bytes + warps * L.warp_bytes > kMaxSmem / 2) warps >>= 1;  // keep >= 2 CTAs/SM if possible
  if (L.cta_bytes + warps * L.warp_bytes > kMaxSmem) return FMOE_ERR_UNSUPPORTED;
  const int smem = L.cta_bytes + warps * L.warp_bytes;
  auto kern = router_topk_smem_kernel<T>;
  FMOE_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  int per_sm = 1;
  FMOE_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, warps * 32, smem));
  if (per_sm < 1) per_sm = 1;
  const int64_t want = (T_ + warps - 1) / warps;
  const int64_t cap = static_cast<int64_t>(device_sm_count()) * per_sm;
  const int grid = static_cast<int>(want < cap ? want : cap);
  kern<<<grid, warps * 32, smem, stream>>>(static_cast<const T*>(logp), T_, nk, k, L, static_cast<T*>(scores), indices,
                                           static_cast<T*>(gates), norm);
  FMOE_LAUNCH_CHECK();
  return FMOE_OK;
}


template <typename T>
int launch_typed(const void* logp, int64_t T_, int nk, int k, void* scores, int64_t* indices, void* gates, int norm,
                 cudaStream_t stream) {
  if (nk <= 1024) {
    const RouterRegLayout L = make_reg_layout(nk, k);
    // few tokens per SM: small CTAs spread them over more SMs
    int warps = 4;
    while (warps > 1 && L.cta_bytes + warps * L.warp_bytes > 96 * 1024) warps >>= 1;
    if (L.cta_bytes + warps * L.warp_bytes <= 200 * 1024) {
      switch (L.nkp / 32) {
        case 1: return launch_reg<T, 1>(logp, T_, nk, k, L, warps, scores, indices, gates, norm, stream);
        case 2: return launch_reg<T, 2>(logp, T_, nk, k, L, warps, scores, indices, gates, norm, stream);
        case 4: return launch_reg<T, 4>(logp, T_, nk, k, L, warps, scores, indices, gates, norm, stream);
        case 8: return launch_reg<T, 8>(logp, T_, nk, k, L, warps, scores, indices, gates, norm, stream);
        case 16: return launch_reg<T, 16>(logp, T_, nk, k, L, warps, scores, indices, gates, norm, stream);
        case 32: return launch_reg<T, 32>(logp, T_, nk, k, L, warps, scores, indices, gates, norm, stream);
        default: break;
      }
    }
  }
  if (norm & 2) return FMOE_ERR_UNSUPPORTED;  // raw logits are only accepted by the register kernel
  return launch_smem<T>(logp, T_, nk, k, scores, indices, gates, norm, stream);
}

}  // namespace

// norm: bit 0 = renormalise the gates per token, bit 1 = `log_probs` holds raw logits [T, 2*nk]
int launch_router_topk(const void* log_probs, int dtype, int64_t T, int nk, int k, void* scores, int64_t* indices,
                       void* gates, int norm, cudaStream_t stream) {
  if (T < 0 || nk <= 0 || k < 0 || k > nk) return FMOE_ERR_BAD_ARG;
  if (nk > 32768) return FMOE_ERR_UNSUPPORTED;  // flat ids and the (p, q) table are 32/16-bit
  if (T == 0 || k == 0) return FMOE_OK;
  if (log_probs == nullptr || scores == nullptr || indices == nullptr) return FMOE_ERR_BAD_ARG;
  switch (dtype) {
    case FMOE_DTYPE_F32: return launch_typed<float>(log_probs, T, nk, k, scores, indices, gates, norm, stream);
    case FMOE_DTYPE_BF16: return launch_typed<__nv_bfloat16>(log_probs, T, nk, k, scores, indices, gates, norm, stream);
    case FMOE_DTYPE_F16: return launch_typed<__half>(log_probs, T, nk, k, scores, indices, gates, norm, stream);
    default: return FMOE_ERR_BAD_ARG;
  }
}

}  // namespace fmoe
