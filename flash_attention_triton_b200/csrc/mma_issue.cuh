// MMA issue sequences shared by the attention kernels.  They are deliberately not inlined:
// each call site would otherwise keep a set of 64-bit descriptors live in the single issuing
// thread and drive up the register count of the whole kernel.
#pragma once
#include "common.cuh"
#include "ptx.cuh"

namespace fa2 {

// acc[128, 128] = A[128 rows, D] * B[128 rows, D]^T.  Both tiles are K-major (row = M / N
// index, the contiguous dimension is the reduction index d), as TMA stages a [128, D] tile.
template <int D, bool BF16>
__device__ __forceinline__ void issue_rows_x_rows(uint32_t d_tmem, uint32_t a_addr, uint32_t b_addr) {
  using T = Tile<D>;
  constexpr uint32_t idesc = make_idesc(128, 128, BF16, false, false);
#pragma unroll
  for (int k = 0; k < D / 16; ++k) {
    const uint32_t off =
        (k / T::kKStepsPerChunk) * T::kChunkTileBytes + (k % T::kKStepsPerChunk) * 32;
    mma_ss(d_tmem, make_smem_desc(a_addr + off, 16, T::kAtomBytes, T::kSwizzleMode),
           make_smem_desc(b_addr + off, 16, T::kAtomBytes, T::kSwizzleMode), idesc, k > 0);
  }
}

// acc[128, D] (+)= A[128, 128] * B[128 rows, D].  A is 16-bit in tensor memory, two values per
// column: reduction indices 0..63 at columns a_col .. a_col+31 and 64..127 at a_col+a_col_half ..
// (+31).  B is a staged [128, D] tile used MN-major (row = reduction index, d contiguous).
template <int D, bool BF16>
__device__ __forceinline__ void issue_tmem_x_tile(uint32_t d_tmem, uint32_t a_tmem,
                                               uint32_t a_col_half, uint32_t b_addr,
                                               uint32_t accumulate) {
  using T = Tile<D>;
  constexpr uint32_t idesc = make_idesc(128, D, BF16, false, true);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const uint32_t a = a_tmem + (k < 4 ? k * 8 : a_col_half + (k - 4) * 8);
    mma_ts(d_tmem, a,
           make_smem_desc(b_addr + k * 2 * T::kAtomBytes, T::kChunkTileBytes, T::kAtomBytes,
                          T::kSwizzleMode),
           idesc, (accumulate || k > 0) ? 1u : 0u);
  }
}

// acc[128, D] = A^T * B with A = [128 rows (reduction), 128] 16-bit tile written by threads as
// two swizzled [128][64] chunk tiles (MN-major A) and B a staged [128, D] tile (MN-major B).
template <int D, bool BF16>
__device__ __forceinline__ void issue_tileT_x_tile(uint32_t d_tmem, uint32_t a_addr, uint32_t b_addr) {
  using T = Tile<D>;
  constexpr uint32_t idesc = make_idesc(128, D, BF16, true, true);
#pragma unroll
  for (int k = 0; k < 8; ++k)
    mma_ss(d_tmem, make_smem_desc(a_addr + k * 2048, 16384, 1024, kSwizzle128B),
           make_smem_desc(b_addr + k * 2 * T::kAtomBytes, T::kChunkTileBytes, T::kAtomBytes,
                          T::kSwizzleMode),
           idesc, k > 0);
}

}  // namespace fa2
