// MMA issue sequences shared by the attention kernels.
//
// Every function here is called by the WHOLE MMA warp, converged; `elected` (elect_one())
// is non-zero in the one lane that actually issues.  The issuing warp shares its scheduler
// with busy compute warps, so every instruction it spends per MMA delays the tensor pipe.  Each sequence therefore builds the
// constant upper word of its shared-memory descriptors once and derives the eight per-step
// descriptors with one 32-bit add each (the start-address field is the only part that moves,
// and it cannot carry out of its 14 bits for addresses below 256 KiB).
//
// Operand types: tiles staged from the caller's tensors (Q, K, V, dO) and the operands the kernels
// produce themselves (P and dS, in tensor memory, in shared memory or spilled to global memory)
// all have the tensors' dtype (kInterBF16 in ptx.cuh).
#pragma once
#include "common.cuh"
#include "ptx.cuh"

namespace fa2 {

// 64-bit shared-memory descriptor from its two words.
__device__ __forceinline__ uint64_t desc_from_words(uint32_t lo, uint32_t hi) {
  return (static_cast<uint64_t>(hi) << 32) | lo;
}
// Upper word: stride byte offset >> 4 in bits [0,14), version 1 at bit 14, swizzle at [29,32).
__host__ __device__ constexpr uint32_t desc_hi_word(uint32_t sbo_bytes, uint32_t swizzle) {
  return ((sbo_bytes >> 4) & 0x3FFFu) | (1u << 14) | (swizzle << 29);
}
// Lower word: start address >> 4 in bits [0,14), leading byte offset >> 4 in bits [16,30).
__device__ __forceinline__ uint32_t desc_lo_word(uint32_t saddr, uint32_t lbo_bytes) {
  return ((saddr & 0x3FFFFu) >> 4) | (((lbo_bytes >> 4) & 0x3FFFu) << 16);
}

// acc[128, 128] (+)= A[128 rows, D] * B[128 rows, D]^T.  Both tiles are K-major (row = M / N
// index, the contiguous dimension is the reduction index d), as TMA stages a [128, D] tile.
template <int D, bool BF16>
__device__ __forceinline__ void issue_rows_x_rows(uint32_t elected, uint32_t d_tmem,
                                                  uint32_t a_addr, uint32_t b_addr,
                                                  uint32_t accumulate = 0u) {
  using T = Tile<D>;
  constexpr uint32_t idesc = make_idesc(128, 128, BF16, false, false);
  constexpr uint32_t hi = desc_hi_word(T::kAtomBytes, T::kSwizzleMode);
  const uint32_t a_lo = desc_lo_word(a_addr, 16), b_lo = desc_lo_word(b_addr, 16);
#pragma unroll
  for (int k = 0; k < D / 16; ++k) {
    constexpr int kpc = T::kKStepsPerChunk;
    const uint32_t off16 = ((k / kpc) * T::kChunkTileBytes + (k % kpc) * 32) >> 4;
    if (elected)
      mma_ss(d_tmem, desc_from_words(a_lo + off16, hi), desc_from_words(b_lo + off16, hi), idesc,
             k > 0 ? 1u : accumulate);
  }
}

// acc[128, D] (+)= A[128, 128] * B[128 rows, D].  A is 16-bit in tensor memory, two values per
// column: reduction indices 0..63 at columns a_tmem .. +31 and 64..127 at a_tmem + a_col_half ..
// (+31).  B is a staged [128, D] tile used MN-major (row = reduction index, d contiguous).
template <int D, bool BF16>
__device__ __forceinline__ void issue_tmem_x_tile(uint32_t elected, uint32_t d_tmem,
                                                  uint32_t a_tmem, uint32_t a_col_half,
                                                  uint32_t b_addr, uint32_t accumulate) {
  using T = Tile<D>;
  constexpr uint32_t idesc = make_idesc_ab(128, D, kInterBF16<BF16>, BF16, false, true);
  constexpr uint32_t hi = desc_hi_word(T::kAtomBytes, T::kSwizzleMode);
  const uint32_t b_lo = desc_lo_word(b_addr, T::kChunkTileBytes);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const uint32_t a = a_tmem + (k < 4 ? k * 8 : a_col_half + (k - 4) * 8);
    if (elected)
      mma_ts(d_tmem, a, desc_from_words(b_lo + ((k * 2 * T::kAtomBytes) >> 4), hi), idesc,
             k > 0 ? 1u : accumulate);
  }
}

// acc[128, D] (+)= A^T * B with A = [128 rows (reduction), 128] 16-bit tile written by threads as
// two swizzled [128][64] chunk tiles (MN-major A) and B a staged [128, D] tile (MN-major B).
template <int D, bool BF16>
__device__ __forceinline__ void issue_tileT_x_tile(uint32_t elected, uint32_t d_tmem,
                                                   uint32_t a_addr, uint32_t b_addr,
                                                   uint32_t accumulate = 0u) {
  using T = Tile<D>;
  constexpr uint32_t idesc = make_idesc_ab(128, D, kInterBF16<BF16>, BF16, true, true);
  constexpr uint32_t a_hi = desc_hi_word(1024, kSwizzle128B);
  constexpr uint32_t b_hi = desc_hi_word(T::kAtomBytes, T::kSwizzleMode);
  const uint32_t a_lo = desc_lo_word(a_addr, 16384), b_lo = desc_lo_word(b_addr, T::kChunkTileBytes);
#pragma unroll
  for (int k = 0; k < 8; ++k)
    if (elected)
      mma_ss(d_tmem, desc_from_words(a_lo + ((k * 2048) >> 4), a_hi),
             desc_from_words(b_lo + ((k * 2 * T::kAtomBytes) >> 4), b_hi), idesc,
             k > 0 ? 1u : accumulate);
}

// acc[128, D] (+)= A^T * B like issue_tileT_x_tile, but with A in the unswizzled "piece-major"
// layout the spill mode keeps in global memory and copies linearly into shared memory:
// element (reduction row r, column c) at byte (c / 8) * 2048 + r * 16 + (c % 8) * 2, i.e. core
// matrices of 8 rows x 16 bytes, consecutive along the reduction rows (128 bytes apart) and
// 2048 bytes apart along the columns.
constexpr uint32_t kPiecesT_Lbo = 128;   // stride between core matrices along the reduction (K) index
constexpr uint32_t kPiecesT_Sbo = 2048;  // stride between core matrices along the M index
template <int D, bool BF16>
__device__ __forceinline__ void issue_piecesT_x_tile(uint32_t elected, uint32_t d_tmem,
                                                     uint32_t a_addr, uint32_t b_addr,
                                                     uint32_t accumulate) {
  using T = Tile<D>;
  constexpr uint32_t idesc = make_idesc_ab(128, D, kInterBF16<BF16>, BF16, true, true);
  constexpr uint32_t a_hi = desc_hi_word(kPiecesT_Sbo, 0u);  // no swizzle
  constexpr uint32_t b_hi = desc_hi_word(T::kAtomBytes, T::kSwizzleMode);
  const uint32_t a_lo = desc_lo_word(a_addr, kPiecesT_Lbo), b_lo = desc_lo_word(b_addr, T::kChunkTileBytes);
#pragma unroll
  for (int k = 0; k < 8; ++k)
    if (elected)
      mma_ss(d_tmem, desc_from_words(a_lo + ((k * 256) >> 4), a_hi),
             desc_from_words(b_lo + ((k * 2 * T::kAtomBytes) >> 4), b_hi), idesc,
             k > 0 ? 1u : accumulate);
}

// acc[128, D] (+)= A * B with A = a piece-major tile used the other way round: row r of the tile
// is the M index and its columns are the reduction index (K-major, unswizzled: core matrices of
// 8 rows x 16 bytes, 128 bytes apart along M and 2048 bytes apart along the reduction index);
// B a staged [128, D] tile (MN-major).
constexpr uint32_t kPieces_Lbo = 2048;  // stride between core matrices along the reduction (K) index
constexpr uint32_t kPieces_Sbo = 128;   // stride between core matrices along the M index
template <int D, bool BF16>
__device__ __forceinline__ void issue_pieces_x_tile(uint32_t elected, uint32_t d_tmem,
                                                    uint32_t a_addr, uint32_t b_addr,
                                                    uint32_t accumulate) {
  using T = Tile<D>;
  constexpr uint32_t idesc = make_idesc_ab(128, D, kInterBF16<BF16>, BF16, false, true);
  constexpr uint32_t a_hi = desc_hi_word(kPieces_Sbo, 0u);  // no swizzle
  constexpr uint32_t b_hi = desc_hi_word(T::kAtomBytes, T::kSwizzleMode);
  const uint32_t a_lo = desc_lo_word(a_addr, kPieces_Lbo), b_lo = desc_lo_word(b_addr, T::kChunkTileBytes);
#pragma unroll
  for (int k = 0; k < 8; ++k)
    if (elected)
      mma_ss(d_tmem, desc_from_words(a_lo + ((k * 4096) >> 4), a_hi),
             desc_from_words(b_lo + ((k * 2 * T::kAtomBytes) >> 4), b_hi), idesc,
             k > 0 ? 1u : accumulate);
}

}  // namespace fa2
