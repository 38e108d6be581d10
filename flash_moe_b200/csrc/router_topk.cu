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
__global__ void router_topk_kernel(const T* __restrict__ logp, int64_t ntok, int nk, int k, RouterSmemLayout L,
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
  for (int p = warp; p < kq; p += nwarps) {
    const int len = min(k / (p + 1), kq);
    const int rs = rowstart[p];
    for (int q = lane; q < len; q += 32) pq[rs + q] = (static_cast<uint32_t>(p) << 16) | static_cast<uint32_t>(q);
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
int launch_typed(const void* logp, int64_t T_, int nk, int k, void* scores, int64_t* indices, void* gates, int norm,
                 cudaStream_t stream) {
  const RouterSmemLayout L = make_layout(nk, k);
  constexpr int kMaxSmem = 227 * 1024;
  int warps = 8;
  while (warps > 1 && L.cta_bytes + warps * L.warp_bytes > kMaxSmem / 2) warps >>= 1;  // keep >= 2 CTAs/SM if possible
  if (L.cta_bytes + warps * L.warp_bytes > kMaxSmem) return FMOE_ERR_UNSUPPORTED;
  const int smem = L.cta_bytes + warps * L.warp_bytes;
  auto kern = router_topk_kernel<T>;
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

}  // namespace

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
