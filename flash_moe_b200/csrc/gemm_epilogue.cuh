// Shared pieces of the tcgen05 GEMM kernels (gemm_sm100.cu, gemm_sm100_pair.cu, gemm_router_bn.cu): the fused
// epilogues, in which one thread drains one accumulator row from TMEM, and the TMA tensor-map encoder.
#pragma once
#include <cuda.h>

#include "common.cuh"
#include "ptx_sm100.cuh"

namespace fmoe {
namespace epi {

// out[row, col_base .. col_base + NCOLS) = T(acc + addend + residual): float32 sum, one rounding.
// taddr: TMEM address of the row's first column; arow (nullable): float32 addend row; rrow (nullable): residual row
// in the module dtype; columns at or beyond n_valid are skipped (n_valid is a multiple of 8).
// The addend and the residual travel two 32-column chunks ahead of the chunk being converted and stored, and the
// first two chunks are requested BEFORE `wait_accumulator()` is called (the caller's wait for the tile's last MMA):
// timestamps taken inside the down GEMM showed the epilogue warps, one per scheduler and idle through the main loop,
// spending ~2250 cycles per chunk when the operands were requested only one chunk ahead and only after the wait -
// a full L2 round trip each, 18 000 cycles for a 128 x 256 tile.  `wait_accumulator` returns false to give up.
template <typename T, int NCOLS, typename WaitFn>
__device__ __forceinline__ bool store_add_row(uint32_t taddr, T* orow, const float* arow, const T* rrow, int col_base,
                                              int n_valid, bool row_ok, WaitFn&& wait_accumulator) {
  constexpr int NCHUNK = NCOLS / 32;
  constexpr int DEPTH = 3;
  float4 ad[DEPTH][8];
  uint4 rs[DEPTH][4];
  auto fetch = [&](int c, float4 (&a)[8], uint4 (&r)[4]) {
    const int col0 = col_base + c * 32;
#pragma unroll
    for (int v = 0; v < 8; ++v)
      a[v] = (arow != nullptr && col0 + v * 4 < n_valid) ? __ldg(reinterpret_cast<const float4*>(arow + col0 + v * 4))
                                                         : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int v = 0; v < 4; ++v)
      r[v] = (rrow != nullptr && col0 + v * 8 < n_valid) ? ldg16(rrow + col0 + v * 8) : make_uint4(0, 0, 0, 0);
  };
  fetch(0, ad[0], rs[0]);
  if (NCHUNK > 1) fetch(1, ad[1], rs[1]);
  if (!wait_accumulator()) return false;
#pragma unroll
  for (int c = 0; c < NCHUNK; ++c) {  // fully unrolled: the buffer a chunk uses is a compile-time choice
    if (c + 2 < NCHUNK) fetch(c + 2, ad[(c + 2) % DEPTH], rs[(c + 2) % DEPTH]);
    const float4 (&cur)[8] = ad[c % DEPTH];
    const uint4 (&rcur)[4] = rs[c % DEPTH];
    uint32_t a[32];
    ptx::tmem_ld_32x32(taddr + c * 32, a);
    ptx::tmem_ld_wait();
    const int col0 = col_base + c * 32;
    if (row_ok) {
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        if (col0 + v * 8 < n_valid) {
          float f[8], r[8];
          unpack16<T>(rcur[v], r);
#pragma unroll
          for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(a[v * 8 + i]);
          f[0] += cur[2 * v].x; f[1] += cur[2 * v].y; f[2] += cur[2 * v].z; f[3] += cur[2 * v].w;
          f[4] += cur[2 * v + 1].x; f[5] += cur[2 * v + 1].y; f[6] += cur[2 * v + 1].z; f[7] += cur[2 * v + 1].w;
          if (rrow != nullptr) {
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] += r[i];
          }
          *reinterpret_cast<uint4*>(orow + col0 + v * 8) = pack16<T>(f);
        }
      }
    }
  }
  return true;
}
// the same for a caller that has already waited for the accumulator
template <typename T, int NCOLS>
__device__ __forceinline__ void store_add_row(uint32_t taddr, T* orow, const float* arow, const T* rrow, int col_base,
                                              int n_valid, bool row_ok) {
  (void)store_add_row<T, NCOLS>(taddr, orow, arow, rrow, col_base, n_valid, row_ok, [] { return true; });
}

// One 32-column chunk of the ADD epilogue with the float32 addend already in shared memory: `achunk` is a
// [rows x 32] float32 box written by TMA with the 128-byte swizzle (16-byte piece j of row r sits at piece
// j ^ (r & 7)), `srow` this thread's row inside it.  Same sums in the same order as store_add_row.
template <typename T>
__device__ __forceinline__ void store_add_chunk_smem(uint32_t taddr_chunk, T* orow, const uint8_t* achunk, int srow,
                                                     const uint4 (&rcur)[4], bool has_residual, int col0, int n_valid,
                                                     bool row_ok) {
  uint32_t a[32];
  ptx::tmem_ld_32x32(taddr_chunk, a);
  ptx::tmem_ld_wait();
  if (!row_ok) return;
  const uint8_t* rowp = achunk + srow * 128;
  uint4 pk[4];
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    const float4 c0 = *reinterpret_cast<const float4*>(rowp + (((2 * v) ^ (srow & 7)) << 4));
    const float4 c1 = *reinterpret_cast<const float4*>(rowp + (((2 * v + 1) ^ (srow & 7)) << 4));
    float f[8], r[8];
    unpack16<T>(rcur[v], r);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(a[v * 8 + i]);
    f[0] += c0.x; f[1] += c0.y; f[2] += c0.z; f[3] += c0.w;
    f[4] += c1.x; f[5] += c1.y; f[6] += c1.z; f[7] += c1.w;
    if (has_residual) {
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] += r[i];
    }
    pk[v] = pack16<T>(f);
  }
  // 32-byte stores (one whole sector per instruction) where the row is 32-byte aligned, 16-byte stores otherwise
  T* dst = orow + col0;
  const bool wide = (reinterpret_cast<uintptr_t>(dst) & 31u) == 0;
#pragma unroll
  for (int v = 0; v < 4; v += 2) {
    if (wide && col0 + v * 8 + 8 < n_valid) {
      asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst + v * 8), "r"(pk[v].x), "r"(pk[v].y),
                   "r"(pk[v].z), "r"(pk[v].w), "r"(pk[v + 1].x), "r"(pk[v + 1].y), "r"(pk[v + 1].z), "r"(pk[v + 1].w)
                   : "memory");
    } else {
      if (col0 + v * 8 < n_valid) *reinterpret_cast<uint4*>(dst + v * 8) = pk[v];
      if (col0 + v * 8 + 8 < n_valid) *reinterpret_cast<uint4*>(dst + v * 8 + 8) = pk[v + 1];
    }
  }
}

// The accumulator holds NCOLS / 2 gate columns followed by NCOLS / 2 up columns of the same outputs:
// out[row, col_base .. col_base + NCOLS / 2) = T(silu(gate) * up); grow / urow (nullable, both or neither) receive
// the two pre-activations rounded to T.
template <typename T, int NCOLS>
__device__ __forceinline__ void store_swiglu_row(uint32_t taddr, T* orow, T* grow, T* urow, int col_base, int n_valid,
                                                 bool row_ok) {
#pragma unroll 1
  for (int c = 0; c < NCOLS / 64; ++c) {
    uint32_t g[32], u[32];
    ptx::tmem_ld_32x32(taddr + c * 32, g);
    ptx::tmem_ld_32x32(taddr + NCOLS / 2 + c * 32, u);
    ptx::tmem_ld_wait();
    const int col0 = col_base + c * 32;
    if (row_ok) {
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        float f[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = silu_f32(__uint_as_float(g[v * 8 + i])) * __uint_as_float(u[v * 8 + i]);
        if (col0 + v * 8 < n_valid) {
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
}

template <typename T> struct UmmaFmt;
template <> struct UmmaFmt<__nv_bfloat16> { static constexpr uint32_t v = 1; };
template <> struct UmmaFmt<__half> { static constexpr uint32_t v = 0; };

// ---------------------------------------------------------------- host side: TMA tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
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

// 2-D K-major 16-bit operand: `rows` rows of `cols` elements, row pitch `pitch` elements; box = 64 columns (one
// 128-byte swizzle row) x box_rows rows; out-of-range elements read as zero.
inline int make_tensor_map(CUtensorMap* m, const void* basep, int dtype, uint64_t cols, uint64_t rows, uint64_t pitch,
                           uint32_t box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return -static_cast<int>(cudaErrorNotSupported);
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {pitch * 2};
  const cuuint32_t box[2] = {64, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = dtype == FMOE_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUresult r = fn(m, dt, 2, const_cast<void*>(basep), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FMOE_OK : FMOE_ERR_BAD_ARG;
}

// float32 [rows, cols] row-major, boxes of 32 columns (128 bytes) x box_rows rows, 128-byte swizzle: the addend tile of
// the down GEMM's epilogue
inline int make_tensor_map_f32(CUtensorMap* m, const void* basep, uint64_t cols, uint64_t rows, uint64_t pitch,
                               uint32_t box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return -static_cast<int>(cudaErrorNotSupported);
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {pitch * 4};
  const cuuint32_t box[2] = {32, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(basep), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FMOE_OK : FMOE_ERR_BAD_ARG;
}

}  // namespace epi
}  // namespace fmoe
