// Tile geometry shared by the attention kernels, and the host-side launcher interface
// between the translation units of the library.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace fa2 {

// A 128-row tile of a [.., N, D] tensor is staged in shared memory as D/CH "chunk tiles" of
// [128 rows][CH elements]; CH*2 bytes is the swizzle span (128 B for D >= 64, 64 B for D = 32).
// This is exactly what one TMA box of (CH, 128, 1) with the matching swizzle mode produces,
// and what the tensor-core shared-memory descriptors below describe.
template <int D>
struct Tile {
  static_assert(D == 32 || D == 64 || D == 128 || D == 256, "tile width must be 32, 64, 128 or 256");
  static constexpr int kRows = 128;
  static constexpr int kChunkElems = D >= 64 ? 64 : 32;
  static constexpr int kChunks = D / kChunkElems;
  static constexpr int kRowBytes = kChunkElems * 2;             // 128 or 64
  static constexpr int kChunkTileBytes = kRows * kRowBytes;     // 16384 or 8192
  static constexpr int kTileBytes = kChunks * kChunkTileBytes;  // 128 * D * 2
  static constexpr int kAtomBytes = 8 * kRowBytes;              // 8-row swizzle atom
  static constexpr uint32_t kSwizzleMode = kRowBytes == 128 ? 2u : 4u;
  static constexpr uint32_t kSwizzleMask = kRowBytes == 128 ? 7u : 3u;
  static constexpr int kKStepsPerChunk = kChunkElems / 16;  // MMAs (K = 16) per chunk tile
};

// Byte offset of the 16-byte piece `piece` of row `row` inside one chunk tile, after the
// hardware XOR swizzle (address bits [4,7) ^= bits [7,10), restricted to the swizzle span).
template <int D>
__host__ __device__ __forceinline__ uint32_t swizzled_offset(uint32_t row, uint32_t piece) {
  const uint32_t off = row * Tile<D>::kRowBytes + piece * 16u;
  return off ^ (((off >> 7) & Tile<D>::kSwizzleMask) << 4);
}

// Same for a [128 rows][64 elements] 16-bit tile with 128-byte rows, whatever D is (used
// for the score-gradient tile, whose row length is the tile width 128, not D).
__host__ __device__ __forceinline__ uint32_t swizzled_offset_128B(uint32_t row, uint32_t piece) {
  const uint32_t off = row * 128u + piece * 16u;
  return off ^ (((off >> 7) & 7u) << 4);
}

// ----------------------------------------------------------------------------------------
// Host launchers (one per kernel family), defined in the .cu files of this directory.
// Tensor maps describe [B, H, N, D] tensors with box (CH, 128 or 32, 1, 1).
// ----------------------------------------------------------------------------------------
struct AttnShape {
  int B, H;
  int N;      // query rows (rows of q, o, dout, dq, lse)
  int D;      // head dim the kernels are instantiated for: 32, 64, 128 or 256
  int dtype;  // 0 = fp16, 1 = bf16
  float scale;
  int Dg;     // head dim of the tensors in memory (a multiple of 8, <= D); the columns
              // Dg..D-1 are zeros on TMA loads and dropped on TMA stores
  int Nk;     // key rows (rows of k, v, dk, dv), 1 <= Nk <= N; the causal mask is aligned at
              // the top left: query row i sees keys 0 .. min(i, Nk - 1)
};

// Element strides of one [B, H, N, D] tensor (the last dimension is contiguous).
struct Strides {
  long long b, h, n;
};

// What the backward preprocess leaves for the backward kernels: the tile-blocked row statistics
// and, one word per 128-row tile, the largest |dout| of the tile (16-bit pattern, sign cleared),
// both indexed from the first (batch, head) problem of the launch.
struct RowStats {
  const float* stats;         // [B*H][T][2][128]
  const unsigned* tile_amax;  // [B*H][T]
};

// Smallest instantiated head dim that holds `d` columns.
inline int padded_head_dim(int d) { return d <= 32 ? 32 : (d <= 64 ? 64 : (d <= 128 ? 128 : 256)); }

// Order in which the causal kernels take their (head, tile) work items.  A tile's work shrinks
// with its rank (rank 0 is the tile that meets the most tiles of the other kind), so for an even
// finish the long items must start first; but the items of one head share its tensors through
// the L2 cache, so they must also run close together.  Heads are therefore taken in groups of
// `group` whose tensors fit a share of the L2 cache together, and inside a group every head's
// rank-0 item comes first, then every head's rank-1 item, and so on.  Against the plain
// head-by-head order this removes most of the causal tail (the last head's longest item no
// longer starts last): the fewer heads a launch has, the more it gains.
struct HeadTile {
  int bh;    // flattened (batch, head) index
  int rank;  // 0 = the heaviest tile of the head
};
__host__ __device__ __forceinline__ HeadTile grouped_order(long long id, int num_bh, int tiles,
                                                           int group) {
  const long long per_group = static_cast<long long>(group) * tiles;
  const int g0 = static_cast<int>(id / per_group) * group;
  const int n = num_bh - g0 < group ? num_bh - g0 : group;  // heads of this group
  const int local = static_cast<int>(id - (id / per_group) * per_group);
  return HeadTile{g0 + local % n, local / n};
}
// Heads per group: q, dout (or o) and k, v of the group's heads in 64 MiB of the 126 MiB L2.
inline int heads_per_group(const AttnShape& s) {
  const long long per_head = (2ll * s.N + 2ll * s.Nk) * s.D * 2;
  const long long g = (64ll << 20) / per_head;
  const long long bh = static_cast<long long>(s.B) * s.H;
  return static_cast<int>(g < 1 ? 1 : (g > bh ? bh : g));
}

// Per-launch context of the forward kernel.  It runs one CTA per SM; each CTA fetches work
// items (pairs of Q tiles) from `work_counter` until none are left, so tensor memory is
// allocated once and no SM idles between items.  The counter is zero before the launch and the kernel
// leaves it at zero (see fetch_work_item), so no memset sits between launches.
struct LaunchCtx {
  int* status;                 // device status word (bounded-wait failures)
  unsigned int* work_counter;  // device word, 0 at kernel start and again at kernel end
  int num_sms;
};

// Next work item of this CTA (called by one thread).  With a counter, CTAs draw items in launch
// order until the counter passes `total_items`; the launch draws total_items + gridDim.x numbers
// in all, and whoever draws the last one puts the counter back to zero for the next launch that
// uses it.  Without a counter every CTA handles the single item blockIdx.x.
__device__ __forceinline__ int fetch_work_item(unsigned int* work_counter, int total_items,
                                               bool first) {
  if (work_counter == nullptr) return first ? static_cast<int>(blockIdx.x) : total_items;
  const unsigned int next = atomicAdd(work_counter, 1u);
  if (next == static_cast<unsigned int>(total_items) + gridDim.x - 1u) atomicExch(work_counter, 0u);
  return next < static_cast<unsigned int>(total_items) ? static_cast<int>(next) : total_items;
}

cudaError_t launch_fwd(const AttnShape& s, const CUtensorMap& tq, const CUtensorMap& tk,
                       const CUtensorMap& tv, const CUtensorMap& to, float* lse,
                       const LaunchCtx& ctx, cudaStream_t stream);

// rowstats[bh][t][0][r] = -lse * log2(e) (-inf for padded rows), rowstats[bh][t][1][r] = -delta;
// behind the last tile, one 32-bit word per tile: the largest |dout| of the tile's rows as its
// 16-bit pattern with the sign cleared.
cudaError_t launch_bwd_preprocess(const AttnShape& s, const void* o, const Strides& so,
                                  const void* dout, const Strides& sdo, const float* lse,
                                  float* rowstats, int* status, int num_sms,
                                  cudaStream_t stream);

// dK/dV per KV tile.  mode 1 also accumulates dQ into dq_accum with fp32 atomic adds
// (dq_accum layout: [bh][t][w = 4][k = D/4][lane = 32][4] floats, holding element
// (row 128*t + 32*w + lane, col 4*k + 0..3)); mode 2 also stores every 16-bit dS^T tile to the
// scratch tensor dq_accum then points to (32 KiB per (KV tile, Q tile) pair, pairs numbered
// per head KV tile by KV tile, see dstile_pairs), from which launch_bwd_consume (form 2) forms dQ.
cudaError_t launch_bwd_dkdv(const AttnShape& s, const CUtensorMap& tq, const CUtensorMap& tk,
                            const CUtensorMap& tv, const CUtensorMap& tdo,
                            const CUtensorMap& tdk, const CUtensorMap& tdv,
                            const RowStats& rowstats, float* dq_accum, int mode, int* status,
                            cudaStream_t stream);

// Head dim 256: P^T and dS^T of every (KV tile, Q tile) pair as 16-bit piece-major tiles into two
// scratch tensors (pair numbering as in the spill mode); launch_bwd_consume forms 0, 1 and 2 then
// give dV, dK and dQ.
cudaError_t launch_bwd_scores_wide(const AttnShape& s, const CUtensorMap& tq, const CUtensorMap& tk,
                                   const CUtensorMap& tv, const CUtensorMap& tdo,
                                   const RowStats& rowstats, void* p_scratch, void* ds_scratch,
                                   int* status, cudaStream_t stream);

// One output tile per CTA from spilled 16-bit score-gradient / probability tiles, one product
// per tile pair in ascending order (deterministic):
//   form 2: dQ(qt) = sum_j dS(j, qt) K_j     (scratch = dS tiles, tb = K, tout = dQ)
//   form 0: dV(jt) = sum_i P(jt, i)^T dO_i   (scratch = P tiles,  tb = dO, tout = dV)  head dim 256
//   form 1: dK(jt) = sum_i dS(jt, i)^T Q_i   (scratch = dS tiles, tb = Q,  tout = dK)  head dim 256
cudaError_t launch_bwd_consume(const AttnShape& s, int form, const void* scratch,
                               const CUtensorMap& tb, const CUtensorMap& tout, const RowStats& rowstats,
                               int* status, cudaStream_t stream);

// (KV tile, Q tile) pairs of one head: KV tile t < nktiles meets Q tiles t .. ntiles-1.
inline long long dstile_pairs(int N, int Nk) {
  const long long nt = (N + 127) / 128, nk = (Nk + 127) / 128;
  return nk * nt - nk * (nk - 1) / 2;
}

// dQ per Q tile, ascending KV order (deterministic path).
cudaError_t launch_bwd_dq(const AttnShape& s, const CUtensorMap& tq, const CUtensorMap& tk,
                          const CUtensorMap& tv, const CUtensorMap& tdo, const CUtensorMap& tdq,
                          const RowStats& rowstats, int* status, cudaStream_t stream);

// dq = convert(dq_accum) (non-deterministic path).
cudaError_t launch_dq_convert(const AttnShape& s, const float* dq_accum, void* dq,
                              const Strides& sdq, cudaStream_t stream);

// One CTA whose waits run into the time limit on purpose (nothing ever arrives); it must end
// by itself with the status word set.
cudaError_t launch_selftest_wait(int* status, cudaStream_t stream);

cudaError_t launch_selftest_mma(int form, const CUtensorMap& ta, const CUtensorMap& tb,
                                const void* a_raw, float* c, int D, int dtype, int* status,
                                cudaStream_t stream);

}  // namespace fa2
