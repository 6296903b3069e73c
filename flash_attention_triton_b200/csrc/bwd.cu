// Causal attention backward for sm_100a.
//
// Replaces _backward_kernel_one_col_block and its launcher
// (src/flash_attention_triton/_triton_kernels_v2.py:192-529 of the reference).  Per
// (KV tile j, Q tile i >= j) the maths is that of lines 312-343 there:
//     S = Q K^T, P = exp(scale*S - lse), dP = dO V^T, dS = P o (dP - delta) * scale,
//     dV += P^T dO, dK += dS^T Q, dQ += dS K.
//
// bwd_dkdv_kernel (one CTA per KV tile) works on the TRANSPOSED score tile so that everything
// a later MMA consumes as its A operand already sits in tensor memory with kv rows on lanes:
//     St  = K  Q_i^T      (smem x smem)  -> tensor memory, 128 columns
//     dPt = V  dO_i^T     (smem x smem)  -> tensor memory, 128 columns
//     dV += Pt  dO_i      (tmem x smem)     Pt  = 16-bit P^T written over St by the compute warps
//     dK += dSt Q_i       (tmem x smem)     dSt = 16-bit dS^T written over dPt
//     dQ_i = dS K         (smem x smem)     fused variant only: dS^T also goes to shared memory,
//                                           the tile lands over dPt and is added to the fp32
//                                           workspace with vector atomics
// bwd_dq_kernel (one CTA per Q tile, deterministic path) recomputes S and dP untransposed and
// accumulates dQ_i over ascending j in tensor memory, so each dQ tile has one owner and one
// summation order.
//
// -lse*log2(e) and -delta of a Q tile arrive in shared memory as one 1 KiB bulk copy from the
// tile-blocked rowstats array; padded rows carry -lse = -inf, which makes their P exactly 0.
#include "common.cuh"
#include "mma_issue.cuh"
#include "ptx.cuh"

#ifndef FA2_BWD_POLY_PAIRS_PER_8
#define FA2_BWD_POLY_PAIRS_PER_8 4  // of every 8 column pairs, this many use ex2_poly2
#endif

namespace fa2 {
namespace {

// 2^x for column pair `c` (compile-time index after unrolling): a fixed share of the pairs
// goes to the FMA-pipe polynomial, the rest to the MUFU, because 128 x 128 exponentials per
// tile pair would otherwise keep the MUFU (16 / clk / SM) busy for 1024 cycles.
__device__ __forceinline__ float2 exp2_pair(float2 x, int c) {
  if ((c & 7) < FA2_BWD_POLY_PAIRS_PER_8) return ex2_poly2(x);
  return make_float2(ex2(x.x), ex2(x.y));
}

__device__ __forceinline__ void bulk_load_1d(uint32_t dst_smem, const void* src, uint32_t bytes,
                                             uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(dst_smem),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c),
               "f"(d)
               : "memory");
}

// The transposed-score kernels (bwd_dkdv_kernel, bwd_scores_wide_kernel) give each thread one kv
// row and 64 q columns of a tile.  probabilities_of_row: p = 2^(s * c - lse2[q]) from the raw
// scores `sr` and the negated, log2-scaled row statistics of the 64 columns (`nlse`, read with
// warp-wide broadcasts).  mask_row: keep only the q columns >= `first` (128 keeps nothing).
__device__ __forceinline__ void probabilities_of_row(const uint32_t (&sr)[64], const float4* nlse,
                                                     float2 sc2, float2 (&p)[32]) {
#pragma unroll
  for (int c4 = 0; c4 < 16; ++c4) {
    const float4 l = nlse[c4];
    const float2 t0 = __ffma2_rn(
        make_float2(__uint_as_float(sr[4 * c4]), __uint_as_float(sr[4 * c4 + 1])), sc2,
        make_float2(l.x, l.y));
    const float2 t1 = __ffma2_rn(
        make_float2(__uint_as_float(sr[4 * c4 + 2]), __uint_as_float(sr[4 * c4 + 3])), sc2,
        make_float2(l.z, l.w));
    p[2 * c4] = exp2_pair(t0, 2 * c4);
    p[2 * c4 + 1] = exp2_pair(t1, 2 * c4 + 1);
  }
}
__device__ __forceinline__ void mask_row(float2 (&p)[32], int first_column, int column0) {
#pragma unroll
  for (int c = 0; c < 32; ++c) {
    p[c].x = (column0 + 2 * c >= first_column) ? p[c].x : 0.f;
    p[c].y = (column0 + 2 * c + 1 >= first_column) ? p[c].y : 0.f;
  }
}

// Epilogue helper: one warp converts its 32 rows of a [128, D] fp32 accumulator to 16 bits,
// stages them swizzled in `stage` (a free tile buffer) and stores them with one TMA per chunk.
template <int D, bool BF16>
__device__ __forceinline__ void store_rows_16bit(uint32_t tmem_row_addr, uint8_t* stage, int warp4,
                                                 int lane, const CUtensorMap* map, int row_base,
                                                 HeadCoord hc, int N) {
  using T = Tile<D>;
  const int r = warp4 * 32 + lane;
#pragma unroll
  for (int c0 = 0; c0 < D; c0 += 32) {
    uint32_t v[32];
    tmem_ld_x32(tmem_row_addr + c0, v);
    tmem_wait_ld();
    const int chunk = c0 / T::kChunkElems;
    const int piece0 = (c0 % T::kChunkElems) / 8;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      uint4 val;
      val.x = pack2<BF16>(__uint_as_float(v[8 * p + 0]), __uint_as_float(v[8 * p + 1]));
      val.y = pack2<BF16>(__uint_as_float(v[8 * p + 2]), __uint_as_float(v[8 * p + 3]));
      val.z = pack2<BF16>(__uint_as_float(v[8 * p + 4]), __uint_as_float(v[8 * p + 5]));
      val.w = pack2<BF16>(__uint_as_float(v[8 * p + 6]), __uint_as_float(v[8 * p + 7]));
      *reinterpret_cast<uint4*>(stage + chunk * T::kChunkTileBytes +
                                swizzled_offset<D>(r, piece0 + p)) = val;
    }
  }
  fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0 && row_base + warp4 * 32 < N) {
    for (int ch = 0; ch < T::kChunks; ++ch)
      tma_store_4d(map, ch * T::kChunkElems, row_base + warp4 * 32, hc,
                   smem_u32(stage + ch * T::kChunkTileBytes + warp4 * 32 * T::kRowBytes));
    tma_store_commit();
    tma_store_wait_all();
  }
}

// =========================================================================================
// dK / dV (+ fused dQ) kernel
// =========================================================================================
// Number of (KV tile, Q tile) pairs of one head whose KV tile index is below `jt`, with
// `ntiles` Q tiles: KV tile t meets Q tiles t .. ntiles-1.  Also the index of the first pair
// of KV tile jt in the dS scratch tensor of the spill mode.
__host__ __device__ __forceinline__ int dstile_count(int ntiles, int jt) {
  return jt * ntiles - jt * (jt - 1) / 2;
}

// MODE 0: dK, dV only (dQ comes from bwd_dq_kernel).  MODE 1 (fused): also dQ, accumulated into
// an fp32 buffer with atomic adds by a fourth warp group.  MODE 2 (spill): also stores every
// 16-bit dS^T tile to a scratch tensor (dq_accum then points to it), from which
// bwd_consume_kernel forms dQ with one product per tile pair instead of recomputing S, P, dP.
template <int D, int MODE>
struct DkdvCfg {
  using T = Tile<D>;
  static constexpr bool FUSE = MODE == 1;
  static constexpr bool SPILL = MODE == 2;
  static constexpr int kStages = 2;  // Q (+rowstats) ring and dO ring (the code relies on 2)
  static constexpr int kThreads = FUSE ? 512 : 384;
  static constexpr int kMmaWarp = FUSE ? 12 : 8;
  static constexpr int kLoadWarp = kMmaWarp + 1;
  static constexpr int kOffK = 0;
  static constexpr int kOffV = kOffK + T::kTileBytes;
  static constexpr int kOffQ = kOffV + T::kTileBytes;
  static constexpr int kOffDO = kOffQ + kStages * T::kTileBytes;
  static constexpr int kOffDS = kOffDO + kStages * T::kTileBytes;  // [2][128 kv][64 q] 16-bit
  static constexpr int kOffStats = kOffDS + (FUSE ? 32768 : 0);    // [kStages][256] fp32
  static constexpr int kOffBar = kOffStats + kStages * 1024;
  static constexpr int kBarKV = 0;
  static constexpr int kBarQFull = 1;                      // kStages
  static constexpr int kBarQEmpty = kBarQFull + kStages;   // kStages
  static constexpr int kBarDOFull = kBarQEmpty + kStages;  // kStages
  static constexpr int kBarDOEmpty = kBarDOFull + kStages;
  static constexpr int kBarStFull = kBarDOEmpty + kStages;
  static constexpr int kBarDptFull = kBarStFull + 1;
  static constexpr int kBarPtReady = kBarDptFull + 1;   // 8 arrivals (one per compute warp)
  static constexpr int kBarDsReady = kBarPtReady + 1;   // 8 arrivals
  static constexpr int kBarDqFull = kBarDsReady + 1;
  static constexpr int kBarDqDrained = kBarDqFull + 1;  // 4 arrivals
  static constexpr int kBarDone = kBarDqDrained + 1;
  static constexpr int kNumBars = kBarDone + 1;
  static constexpr int kSmemBytes = kOffBar + kNumBars * 8 + 16;
  static_assert(kSmemBytes <= 232448, "shared memory budget of one CTA");
  static constexpr int kColSt = 0;
  static constexpr int kColDpt = 128;  // dQ (fused) reuses these columns
  static constexpr int kColDV = 256;
  static constexpr int kColDK = 256 + D;
  static constexpr int kTmemCols = 512;
};

enum BwdSite {
  kBSiteLoadQ = 32,
  kBSiteLoadDO,
  kBSiteMmaKV,
  kBSiteMmaQ,
  kBSiteMmaDO,
  kBSiteMmaPt,
  kBSiteMmaDs,
  kBSiteMmaDrain,
  kBSiteCmpQ,
  kBSiteCmpSt,
  kBSiteCmpDpt,
  kBSiteCmpDone,
  kBSiteRedDq,
  kBSiteAlign
};

template <int D, bool BF16, int MODE>
__global__ void __launch_bounds__(DkdvCfg<D, MODE>::kThreads, 1)
    bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                    const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo,
                    const __grid_constant__ CUtensorMap tdk,
                    const __grid_constant__ CUtensorMap tdv, const float* __restrict__ rowstats,
                    float* __restrict__ dq_accum, int N, int Nk, float scale, float scale_log2,
                    int* status) {
  using C = DkdvCfg<D, MODE>;
  constexpr bool FUSE = C::FUSE;
  constexpr bool SPILL = C::SPILL;
  using T = Tile<D>;
  extern __shared__ __align__(1024) uint8_t smem[];
  // Role index: the producer / MMA group takes hardware warps 0-3 (lowest ids on their
  // schedulers), the compute and reduction groups follow; shifts are multiples of 4, so
  // role % 4 is still the tensor-memory lane quarter of the hardware warp.
  constexpr int kWarps = C::kThreads / 32;
  const int warp = ((threadIdx.x >> 5) + C::kMmaWarp) % kWarps, lane = threadIdx.x & 31;
  const uint32_t smem_base = smem_u32(smem);
  if (smem_base & 1023u) {
    if (threadIdx.x == 0) atomicCAS(status, 0, 0x20000 | kBSiteAlign);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kOffBar);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + C::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  auto bar = [&](int i) { return smem_base + C::kOffBar + 8u * i; };

  const int ntiles = (N + 127) >> 7;
  const int jt = blockIdx.x;  // KV tile; tile 0 has the most Q tiles and is scheduled first
  const HeadCoord hc{static_cast<int>(blockIdx.y), static_cast<int>(blockIdx.z)};  // grid (tiles, H, B)
  const int bh = hc.b * static_cast<int>(gridDim.y) + hc.h;
  const int nq = ntiles - jt;  // Q tiles jt .. ntiles-1 (N = query rows, Nk <= N = key rows)
  const bool kv_ragged = jt * 128 + 128 > Nk;  // this KV tile has rows beyond the last key
  // Spill mode: tiles of a head are numbered KV tile by KV tile, Q tiles ascending inside.
  const int nktiles = (Nk + 127) >> 7;
  const int tile0 = bh * dstile_count(ntiles, nktiles) + dstile_count(ntiles, jt);
  (void)tile0;

  if (threadIdx.x == 0) {
    mbar_init(bar(C::kBarKV), 1);
    for (int i = 0; i < C::kStages; ++i) {
      mbar_init(bar(C::kBarQFull + i), 1);
      mbar_init(bar(C::kBarQEmpty + i), 2);   // St (warp X) and dK (warp Y) both done
      mbar_init(bar(C::kBarDOFull + i), 1);
      mbar_init(bar(C::kBarDOEmpty + i), 2);  // dV (warp X) and dPt (warp Y) both done
    }
    mbar_init(bar(C::kBarStFull), 1);
    mbar_init(bar(C::kBarDptFull), 1);
    mbar_init(bar(C::kBarPtReady), 8);
    mbar_init(bar(C::kBarDsReady), 8);
    mbar_init(bar(C::kBarDqFull), 1);
    mbar_init(bar(C::kBarDqDrained), 4);
    mbar_init(bar(C::kBarDone), 2);  // last dV (warp X) and last dK (warp Y)
    *abort_flag = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == C::kMmaWarp) {
    tmem_alloc(smem_u32(tmem_slot), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const WaitCtx w{abort_flag, status};

  if (warp >= C::kMmaWarp) {
    // ---------------------------------------------------------------- producer / MMA group
    reg_dec<72>();
    if (warp == C::kLoadWarp) {
      // TMA producer: whole warp, converged; the elected lane arms barriers and issues copies.
      const uint32_t elected = elect_one();
      if (elected) {
        prefetch_tensormap(&tq);
        prefetch_tensormap(&tk);
        prefetch_tensormap(&tv);
        prefetch_tensormap(&tdo);
        mbar_arrive_expect_tx(bar(C::kBarKV), 2 * T::kTileBytes);
        for (int ch = 0; ch < T::kChunks; ++ch) {
          tma_load_4d(smem_base + C::kOffK + ch * T::kChunkTileBytes, &tk, ch * T::kChunkElems,
                      jt * 128, hc, bar(C::kBarKV));
          tma_load_4d(smem_base + C::kOffV + ch * T::kChunkTileBytes, &tv, ch * T::kChunkElems,
                      jt * 128, hc, bar(C::kBarKV));
        }
      }
      for (int ii = 0; ii < nq; ++ii) {
        const int s = ii % C::kStages, ph = (ii / C::kStages) & 1;
        const int qt = jt + ii;
        if (!mbar_wait_warp(bar(C::kBarQEmpty + s), ph ^ 1, w, kBSiteLoadQ)) break;
        if (elected) {
          mbar_arrive_expect_tx(bar(C::kBarQFull + s), T::kTileBytes + 1024);
#pragma unroll
          for (int ch = 0; ch < T::kChunks; ++ch)
            tma_load_4d(smem_base + C::kOffQ + s * T::kTileBytes + ch * T::kChunkTileBytes, &tq,
                        ch * T::kChunkElems, qt * 128, hc, bar(C::kBarQFull + s));
          bulk_load_1d(smem_base + C::kOffStats + s * 1024,
                       rowstats + (static_cast<size_t>(bh) * ntiles + qt) * 256, 1024,
                       bar(C::kBarQFull + s));
        }
        if (!mbar_wait_warp(bar(C::kBarDOEmpty + s), ph ^ 1, w, kBSiteLoadDO)) break;
        if (elected) {
          mbar_arrive_expect_tx(bar(C::kBarDOFull + s), T::kTileBytes);
#pragma unroll
          for (int ch = 0; ch < T::kChunks; ++ch)
            tma_load_4d(smem_base + C::kOffDO + s * T::kTileBytes + ch * T::kChunkTileBytes, &tdo,
                        ch * T::kChunkElems, qt * 128, hc, bar(C::kBarDOFull + s));
        }
      }
    } else if (warp == C::kMmaWarp || warp == C::kMmaWarp + 2) {
      // Two MMA-issuing warps, one per dependency chain (whole warp converged, the elected
      // lane issues).  The chains touch disjoint tensor-memory columns, so no ordering
      // between the two instruction streams is needed and neither waits behind the other:
      //   warp X:  [Pt(i) ready]  dV += Pt dO_i,  St(i+1) = K Q_(i+1)^T         (St / Pt / dV)
      //   warp Y:  [dSt(i) ready] dK += dSt Q_i, (dQ_i = dS K), dPt(i+1) = V dO_(i+1)^T
      //            (dPt / dSt / dK; in the fused kernel dQ shares the dPt columns, so dPt(i+1)
      //            waits until the reduction group has drained dQ_i)
      // Within a chain the in-order tensor pipe protects the write-after-read hazards
      // (St(i+1) over Pt(i), dPt(i+1) / dQ_i over dSt(i)).
      const uint32_t elected = elect_one();
      const uint32_t ka = smem_base + C::kOffK, va = smem_base + C::kOffV;
      auto commit = [&](int b) {
        if (elected) mma_commit(bar(b));
      };
      bool ok = mbar_wait(bar(C::kBarKV), 0, w, kBSiteMmaKV);
      int s = 0, ph = 0;  // ring stage / phase of Q tile ii (both rings advance together)
      if (warp == C::kMmaWarp) {
        // ------------------------------------------------------------ warp X
        if (ok && (ok = mbar_wait(bar(C::kBarQFull + 0), 0, w, kBSiteMmaQ))) {
          issue_rows_x_rows<D, BF16>(elected, tmem_base + C::kColSt, ka, smem_base + C::kOffQ);
          commit(C::kBarStFull);
          commit(C::kBarQEmpty + 0);
        }
        for (int ii = 0; ok && ii < nq; ++ii) {
          const int s1 = s ^ 1, ph1 = ph ^ s;  // stage / phase of tile ii+1 (two stages)
          const uint32_t doa = smem_base + C::kOffDO + s * T::kTileBytes;
          if (!(ok = mbar_wait(bar(C::kBarDOFull + s), ph, w, kBSiteMmaDO))) break;
          if (!(ok = mbar_wait(bar(C::kBarPtReady), ii & 1, w, kBSiteMmaPt))) break;
          tc_fence_after();
          issue_tmem_x_tile<D, BF16>(elected, tmem_base + C::kColDV, tmem_base + C::kColSt, 64, doa,
                                     ii > 0);  // dV += Pt dO_i
          commit(C::kBarDOEmpty + s);
          if (ii + 1 < nq) {
            if (!(ok = mbar_wait(bar(C::kBarQFull + s1), ph1, w, kBSiteMmaQ))) break;
            issue_rows_x_rows<D, BF16>(elected, tmem_base + C::kColSt, ka,
                                       smem_base + C::kOffQ + s1 * T::kTileBytes);  // St(i+1)
            commit(C::kBarStFull);
            commit(C::kBarQEmpty + s1);
          }
          ph ^= s;
          s ^= 1;
        }
        if (ok) commit(C::kBarDone);
      } else {
        // ------------------------------------------------------------ warp Y
        if (ok && (ok = mbar_wait(bar(C::kBarDOFull + 0), 0, w, kBSiteMmaDO))) {
          issue_rows_x_rows<D, BF16>(elected, tmem_base + C::kColDpt, va, smem_base + C::kOffDO);
          commit(C::kBarDptFull);
          commit(C::kBarDOEmpty + 0);
        }
        for (int ii = 0; ok && ii < nq; ++ii) {
          const int s1 = s ^ 1, ph1 = ph ^ s;
          const uint32_t qa = smem_base + C::kOffQ + s * T::kTileBytes;
          if (!(ok = mbar_wait(bar(C::kBarQFull + s), ph, w, kBSiteMmaQ))) break;
          if (!(ok = mbar_wait(bar(C::kBarDsReady), ii & 1, w, kBSiteMmaDs))) break;
          if constexpr (!FUSE) {
            // St(i+1) sits on the critical chain St -> Pt -> dV -> St; let warp X get it into
            // the in-order pipe first, dK and dPt(i+1) then run under the next exponentials.
            if (ii + 1 < nq) {
              if (!(ok = mbar_wait(bar(C::kBarStFull), (ii + 1) & 1, w, kBSiteMmaQ))) break;
            }
          }
          tc_fence_after();
          issue_tmem_x_tile<D, BF16>(elected, tmem_base + C::kColDK, tmem_base + C::kColDpt, 64, qa,
                                     ii > 0);  // dK += dSt Q_i
          commit(C::kBarQEmpty + s);
          if constexpr (FUSE) {
            // dQ_i[128 q, D] = dS[q, kv] * K[kv, d]: A = dS^T tile in smem (q contiguous ->
            // MN-major), B = K tile (d contiguous -> MN-major); lands over the dPt columns.
            issue_tileT_x_tile<D, BF16>(elected, tmem_base + C::kColDpt, smem_base + C::kOffDS, ka);
            commit(C::kBarDqFull);
          }
          if (ii + 1 < nq) {
            if constexpr (FUSE) {
              if (!(ok = mbar_wait(bar(C::kBarDqDrained), ii & 1, w, kBSiteMmaDrain))) break;
              tc_fence_after();
            }
            if (!(ok = mbar_wait(bar(C::kBarDOFull + s1), ph1, w, kBSiteMmaDO))) break;
            issue_rows_x_rows<D, BF16>(elected, tmem_base + C::kColDpt, va,
                                       smem_base + C::kOffDO + s1 * T::kTileBytes);  // dPt(i+1)
            commit(C::kBarDptFull);
            commit(C::kBarDOEmpty + s1);
          }
          ph ^= s;
          s ^= 1;
        }
        if (ok) commit(C::kBarDone);
      }
    }
    __syncwarp();
  } else if (FUSE && warp >= 8) {
    // ---------------------------------------------------------------- dQ reduction group
    reg_inc<136>();  // 512-thread kernel starts at 128 registers per thread
    const int w4 = warp & 3;
    const uint32_t lane_base = static_cast<uint32_t>(w4 * 32) << 16;
    for (int ii = 0; ii < nq; ++ii) {
      if (!mbar_wait_warp(bar(C::kBarDqFull), ii & 1, w, kBSiteRedDq)) break;
      tc_fence_after();
      const int qt = jt + ii;
      float* dst = dq_accum + (((static_cast<size_t>(bh) * ntiles + qt) * 4 + w4) * (D / 4)) * 128 +
                   lane * 4;
      // Whole dQ tile into registers first, so the MMA warp can reuse the columns at once;
      // the atomics follow at leisure.
      uint32_t v[D];
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 32) tmem_ld_x32(tmem_base + lane_base + C::kColDpt + c0, v + c0);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(C::kBarDqDrained));
#pragma unroll
      for (int k = 0; k < D / 4; ++k)
        red_add_v4(dst + k * 128, __uint_as_float(v[4 * k]), __uint_as_float(v[4 * k + 1]),
                   __uint_as_float(v[4 * k + 2]), __uint_as_float(v[4 * k + 3]));
    }
  } else {
    // ---------------------------------------------------------------- compute groups
    if constexpr (FUSE) reg_inc<152>(); else reg_inc<208>();
    const int wg = warp >> 2;  // 0: score columns (q) 0..63, 1: 64..127
    const int w4 = warp & 3;
    const int r = w4 * 32 + lane;  // kv row in the tile = tensor-memory lane
    const uint32_t lane_base = static_cast<uint32_t>(w4 * 32) << 16;
    const uint32_t tSt = tmem_base + lane_base + C::kColSt + wg * 64;
    const uint32_t tDpt = tmem_base + lane_base + C::kColDpt + wg * 64;
    const float2 sc2 = make_float2(scale_log2, scale_log2);
    const float2 scale2 = make_float2(scale, scale);
    bool ok = true;
    for (int ii = 0; ii < nq; ++ii) {
      const int s = ii % C::kStages, ph = (ii / C::kStages) & 1;
      const float* stats = reinterpret_cast<const float*>(smem + C::kOffStats + s * 1024);
      const float4* nlse = reinterpret_cast<const float4*>(stats + wg * 64);        // -lse*log2e
      const float4* ndlt = reinterpret_cast<const float4*>(stats + 128 + wg * 64);  // -delta
      if (!(ok = mbar_wait_warp(bar(C::kBarQFull + s), ph, w, kBSiteCmpQ))) break;
      if (!(ok = mbar_wait_warp(bar(C::kBarStFull), ii & 1, w, kBSiteCmpSt))) break;
      tc_fence_after();
      float2 p[32];  // P^T for this thread's kv row, q columns wg*64 .. wg*64+63
      {
        uint32_t sr[64];
        tmem_ld_x32(tSt, sr);
        tmem_ld_x32(tSt + 32, sr + 32);
        tmem_wait_ld();
        probabilities_of_row(sr, nlse, sc2, p);
      }
      if (ii == 0 || kv_ragged) {
        // diagonal tile: keep q >= kv; rows beyond the last key (zero-filled K, V) keep nothing,
        // so that a huge 2^(-lse) never meets their zeros
        mask_row(p, (jt * 128 + r >= Nk) ? 128 : (ii == 0 ? r : 0), wg * 64);
      }
      {
        uint32_t pk[32];
#pragma unroll
        for (int c = 0; c < 32; ++c) pk[c] = pack2<BF16>(p[c].x, p[c].y);
        tmem_st_x32(tSt, pk);  // columns wg*64 .. wg*64+31 of the St region
        tmem_wait_st();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(C::kBarPtReady));

      if (!(ok = mbar_wait_warp(bar(C::kBarDptFull), ii & 1, w, kBSiteCmpDpt))) break;
      tc_fence_after();
      uint32_t dsk[32];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t dp[32];
        tmem_ld_x32(tDpt + 32 * h, dp);
        tmem_wait_ld();
#pragma unroll
        for (int c4 = 0; c4 < 8; ++c4) {
          const float4 nd = ndlt[8 * h + c4];
          // dS = P * (dP - delta) * scale, scale folded in before the 16-bit rounding
          float2 u0 = __fadd2_rn(make_float2(__uint_as_float(dp[4 * c4]), __uint_as_float(dp[4 * c4 + 1])),
                                 make_float2(nd.x, nd.y));
          float2 u1 = __fadd2_rn(make_float2(__uint_as_float(dp[4 * c4 + 2]), __uint_as_float(dp[4 * c4 + 3])),
                                 make_float2(nd.z, nd.w));
          u0 = __fmul2_rn(__fmul2_rn(p[16 * h + 2 * c4], u0), scale2);
          u1 = __fmul2_rn(__fmul2_rn(p[16 * h + 2 * c4 + 1], u1), scale2);
          dsk[16 * h + 2 * c4] = pack2<BF16>(u0.x, u0.y);
          dsk[16 * h + 2 * c4 + 1] = pack2<BF16>(u1.x, u1.y);
        }
      }
      tmem_st_x32(tDpt, dsk);  // columns 128 + wg*64 .. +31
      if constexpr (SPILL) {
        // This thread's 64 values of dS^T(jt, jt+ii) (kv row r, q columns wg*64 ..) straight to
        // pair `tile0 + ii` of the scratch tensor.  A tile is stored piece-major: the 16-byte
        // piece (kv row r, q columns 8g .. 8g+7) at byte g * 2048 + r * 16, so one warp
        // instruction writes 512 contiguous bytes, and the tile can later be copied linearly
        // into shared memory as an unswizzled tensor-core operand.  Going through registers
        // keeps the copy out of shared memory, whose bandwidth the operand reads already use up.
        uint4* dst = reinterpret_cast<uint4*>(dq_accum) +
                     (static_cast<size_t>(tile0 + ii) * 2048 + wg * 1024 + r);
#pragma unroll
        for (int pc = 0; pc < 8; ++pc)
          dst[pc * 128] = make_uint4(dsk[4 * pc], dsk[4 * pc + 1], dsk[4 * pc + 2], dsk[4 * pc + 3]);
      }
      if constexpr (FUSE) {
        uint8_t* ds_tile = smem + C::kOffDS + wg * 16384;
#pragma unroll
        for (int pc = 0; pc < 8; ++pc)
          *reinterpret_cast<uint4*>(ds_tile + swizzled_offset_128B(r, pc)) =
              make_uint4(dsk[4 * pc], dsk[4 * pc + 1], dsk[4 * pc + 2], dsk[4 * pc + 3]);
        fence_proxy_async_smem();
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(C::kBarDsReady));
    }
    // epilogue: group 0 stores dV, group 1 stores dK, staged through the idle dO / Q buffers
    if (ok && mbar_wait_warp(bar(C::kBarDone), 0, w, kBSiteCmpDone)) {
      tc_fence_after();
      if (wg == 0)
        store_rows_16bit<D, BF16>(tmem_base + lane_base + C::kColDV, smem + C::kOffDO, w4, lane,
                                  &tdv, jt * 128, hc, Nk);
      else
        store_rows_16bit<D, BF16>(tmem_base + lane_base + C::kColDK, smem + C::kOffQ, w4, lane,
                                  &tdk, jt * 128, hc, Nk);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == C::kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// =========================================================================================
// dQ kernel (deterministic path): one CTA per Q tile, KV tiles in ascending order
// =========================================================================================
// Pipeline per KV tile j:  S(j) = Q K_j^T lands in score buffer j%2, dP(j) = dO V_j^T in the dP
// columns.  The compute warps turn S into P (registers), read dP, release the dP columns
// (so dP(j+1) can be issued while they still work), write dS(j) as 16-bit pairs over the score
// buffer they just read, and the MMA warp then issues dQ += dS(j) K_j followed by S(j+2) into
// the same buffer.  S(j+1) is already in the other buffer, so the tensor pipe and the compute
// warps overlap instead of alternating.
template <int D>
struct DqCfg {
  using T = Tile<D>;
  static constexpr int kKStages = 3;  // K_j is needed by S(j) and, later, by dQ(j)
  static constexpr int kVStages = 2;
  static constexpr int kThreads = 384;
  static constexpr int kMmaWarp = 8;
  static constexpr int kLoadWarp = 9;
  static constexpr int kOffQ = 0;
  static constexpr int kOffDO = kOffQ + T::kTileBytes;
  static constexpr int kOffK = kOffDO + T::kTileBytes;
  static constexpr int kOffV = kOffK + kKStages * T::kTileBytes;
  static constexpr int kOffStats = kOffV + kVStages * T::kTileBytes;  // [256] fp32
  static constexpr int kOffBar = kOffStats + 1024;
  static constexpr int kBarQ = 0;  // Q, dO and rowstats
  static constexpr int kBarKFull = 1;
  static constexpr int kBarKEmpty = kBarKFull + kKStages;
  static constexpr int kBarVFull = kBarKEmpty + kKStages;
  static constexpr int kBarVEmpty = kBarVFull + kVStages;
  static constexpr int kBarSFull = kBarVEmpty + kVStages;  // 2 (one per score buffer)
  static constexpr int kBarDpFull = kBarSFull + 2;
  static constexpr int kBarDpConsumed = kBarDpFull + 1;  // 8 arrivals (one per compute warp)
  static constexpr int kBarDsReady = kBarDpConsumed + 1;  // 8 arrivals
  static constexpr int kBarDqDone = kBarDsReady + 1;      // 2: dQ += dS(j) K_j completed, by j%2
  static constexpr int kBarDone = kBarDqDone + 2;
  static constexpr int kNumBars = kBarDone + 1;
  static constexpr int kSmemBytes = kOffBar + kNumBars * 8 + 16;
  static constexpr int kColS = 0;     // score buffers at 0 and 128; dS (16-bit) overwrites them
  static constexpr int kColDp = 256;
  static constexpr int kColDQ = 384;
  static constexpr int kTmemCols = 512;
};

template <int D, bool BF16>
__global__ void __launch_bounds__(DqCfg<D>::kThreads, 1)
    bwd_dq_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                  const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo,
                  const __grid_constant__ CUtensorMap tdq, const float* __restrict__ rowstats, int N,
                  int Nk,
                  float scale, float scale_log2, int* status) {
  using C = DqCfg<D>;
  using T = Tile<D>;
  extern __shared__ __align__(1024) uint8_t smem[];
  // Role index: producer / MMA group on hardware warps 0-3, compute groups on 4-11.
  const int warp = ((threadIdx.x >> 5) + C::kMmaWarp) % (C::kThreads / 32), lane = threadIdx.x & 31;
  const uint32_t smem_base = smem_u32(smem);
  if (smem_base & 1023u) {
    if (threadIdx.x == 0) atomicCAS(status, 0, 0x20000 | kBSiteAlign);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kOffBar);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + C::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  auto bar = [&](int i) { return smem_base + C::kOffBar + 8u * i; };

  const int ntiles = (N + 127) >> 7;
  const int qt = ntiles - 1 - static_cast<int>(blockIdx.x);  // heaviest Q tile first
  const HeadCoord hc{static_cast<int>(blockIdx.y), static_cast<int>(blockIdx.z)};  // grid (tiles, H, B)
  const int bh = hc.b * static_cast<int>(gridDim.y) + hc.h;
  const int nktiles = (Nk + 127) >> 7;               // N = query rows, Nk <= N = key rows
  const int nkv = qt + 1 < nktiles ? qt + 1 : nktiles;  // KV tiles 0 .. min(qt, last)

  if (threadIdx.x == 0) {
    mbar_init(bar(C::kBarQ), 1);
    for (int i = 0; i < C::kKStages; ++i) {
      mbar_init(bar(C::kBarKFull + i), 1);
      mbar_init(bar(C::kBarKEmpty + i), 2);  // S(j) (warp X) and dQ(j) (warp Y) both done
    }
    for (int i = 0; i < C::kVStages; ++i) {
      mbar_init(bar(C::kBarVFull + i), 1);
      mbar_init(bar(C::kBarVEmpty + i), 1);
    }
    mbar_init(bar(C::kBarSFull + 0), 1);
    mbar_init(bar(C::kBarSFull + 1), 1);
    mbar_init(bar(C::kBarDpFull), 1);
    mbar_init(bar(C::kBarDpConsumed), 8);
    mbar_init(bar(C::kBarDsReady), 8);
    mbar_init(bar(C::kBarDqDone + 0), 1);
    mbar_init(bar(C::kBarDqDone + 1), 1);
    mbar_init(bar(C::kBarDone), 1);
    *abort_flag = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == C::kMmaWarp) {
    tmem_alloc(smem_u32(tmem_slot), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const WaitCtx w{abort_flag, status};

  if (warp >= C::kMmaWarp) {
    reg_dec<72>();
    if (warp == C::kLoadWarp) {
      // TMA producer: whole warp, converged; the elected lane arms barriers and issues copies.
      const uint32_t elected = elect_one();
      if (elected) {
        prefetch_tensormap(&tq);
        prefetch_tensormap(&tk);
        prefetch_tensormap(&tv);
        prefetch_tensormap(&tdo);
        mbar_arrive_expect_tx(bar(C::kBarQ), 2 * T::kTileBytes + 1024);
        for (int ch = 0; ch < T::kChunks; ++ch) {
          tma_load_4d(smem_base + C::kOffQ + ch * T::kChunkTileBytes, &tq, ch * T::kChunkElems,
                      qt * 128, hc, bar(C::kBarQ));
          tma_load_4d(smem_base + C::kOffDO + ch * T::kChunkTileBytes, &tdo, ch * T::kChunkElems,
                      qt * 128, hc, bar(C::kBarQ));
        }
        bulk_load_1d(smem_base + C::kOffStats,
                     rowstats + (static_cast<size_t>(bh) * ntiles + qt) * 256, 1024, bar(C::kBarQ));
      }
      for (int j = 0; j < nkv; ++j) {
        const int ks = j % C::kKStages, kph = (j / C::kKStages) & 1;
        if (!mbar_wait_warp(bar(C::kBarKEmpty + ks), kph ^ 1, w, kBSiteLoadQ)) break;
        if (elected) {
          mbar_arrive_expect_tx(bar(C::kBarKFull + ks), T::kTileBytes);
#pragma unroll
          for (int ch = 0; ch < T::kChunks; ++ch)
            tma_load_4d(smem_base + C::kOffK + ks * T::kTileBytes + ch * T::kChunkTileBytes, &tk,
                        ch * T::kChunkElems, j * 128, hc, bar(C::kBarKFull + ks));
        }
        const int vs = j % C::kVStages, vph = (j / C::kVStages) & 1;
        if (!mbar_wait_warp(bar(C::kBarVEmpty + vs), vph ^ 1, w, kBSiteLoadDO)) break;
        if (elected) {
          mbar_arrive_expect_tx(bar(C::kBarVFull + vs), T::kTileBytes);
#pragma unroll
          for (int ch = 0; ch < T::kChunks; ++ch)
            tma_load_4d(smem_base + C::kOffV + vs * T::kTileBytes + ch * T::kChunkTileBytes, &tv,
                        ch * T::kChunkElems, j * 128, hc, bar(C::kBarVFull + vs));
        }
      }
    } else if (warp == C::kMmaWarp) {
      // ------------------------------------------------------------ warp X: dP(j) = dO V_j^T
      // (whole warp converged, the elected lane issues).  The three products of a KV step are
      // issued by three warps (X: dP, Z: S, Y: dQ), so none of them waits behind another
      // one's barrier: dP(j+1) only needs the compute warps to have read dP(j), S(j+2) only
      // needs dQ(j) to have consumed dS(j) (both live in score buffer j%2), dQ(j) only needs
      // dS(j).  The tensor pipe executes whatever is issued first.
      const uint32_t elected = elect_one();
      auto commit = [&](int b) {
        if (elected) mma_commit(bar(b));
      };
      const uint32_t doa = smem_base + C::kOffDO;
      int vs = 0, vph = 0;  // ring position of the next V tile
      bool ok = mbar_wait(bar(C::kBarQ), 0, w, kBSiteMmaQ);
      for (int j = 0; ok && j < nkv; ++j) {
        if (j > 0) {
          // dP columns are free once every compute warp has read dP(j-1)
          if (!(ok = mbar_wait(bar(C::kBarDpConsumed), (j - 1) & 1, w, kBSiteMmaDrain))) break;
          tc_fence_after();
        }
        if (!(ok = mbar_wait(bar(C::kBarVFull + vs), vph, w, kBSiteMmaDO))) break;
        issue_rows_x_rows<D, BF16>(elected, tmem_base + C::kColDp, doa,
                                   smem_base + C::kOffV + vs * T::kTileBytes);
        commit(C::kBarDpFull);
        commit(C::kBarVEmpty + vs);  // V is free once dP has read it
        if (++vs == C::kVStages) {
          vs = 0;
          vph ^= 1;
        }
      }
    } else if (warp == C::kMmaWarp + 3) {
      // ------------------------------------------------------------ warp Z: S(j) = Q K_j^T
      const uint32_t elected = elect_one();
      auto commit = [&](int b) {
        if (elected) mma_commit(bar(b));
      };
      const uint32_t qa = smem_base + C::kOffQ;
      int ks = 0, kph = 0;  // ring position of the next K tile
      bool ok = mbar_wait(bar(C::kBarQ), 0, w, kBSiteMmaQ);
      for (int j = 0; ok && j < nkv; ++j) {
        if (j >= 2) {
          // score buffer j%2 holds dS(j-2) until dQ += dS(j-2) K_(j-2) has completed
          if (!(ok = mbar_wait(bar(C::kBarDqDone + (j & 1)), ((j - 2) >> 1) & 1, w, kBSiteMmaDs)))
            break;
          tc_fence_after();
        }
        if (!(ok = mbar_wait(bar(C::kBarKFull + ks), kph, w, kBSiteMmaKV))) break;
        issue_rows_x_rows<D, BF16>(elected, tmem_base + C::kColS + (j & 1) * 128, qa,
                                   smem_base + C::kOffK + ks * T::kTileBytes);
        commit(C::kBarSFull + (j & 1));
        commit(C::kBarKEmpty + ks);
        if (++ks == C::kKStages) {
          ks = 0;
          kph ^= 1;
        }
      }
    } else if (warp == C::kMmaWarp + 2) {
      // ------------------------------------------------------------ warp Y: dQ += dS(j) K_j
      const uint32_t elected = elect_one();
      auto commit = [&](int b) {
        if (elected) mma_commit(bar(b));
      };
      bool ok = true;
      int ks = 0, kph = 0;
      for (int j = 0; ok && j < nkv; ++j) {
        if (!(ok = mbar_wait(bar(C::kBarKFull + ks), kph, w, kBSiteMmaKV))) break;
        if (!(ok = mbar_wait(bar(C::kBarDsReady), j & 1, w, kBSiteMmaDs))) break;
        tc_fence_after();
        // A = 16-bit dS over score buffer j%2, B = K_j as MN-major tile
        issue_tmem_x_tile<D, BF16>(elected, tmem_base + C::kColDQ, tmem_base + C::kColS + (j & 1) * 128,
                                   64, smem_base + C::kOffK + ks * T::kTileBytes, j > 0);
        commit(C::kBarDqDone + (j & 1));
        commit(C::kBarKEmpty + ks);
        if (++ks == C::kKStages) {
          ks = 0;
          kph ^= 1;
        }
      }
      if (ok) commit(C::kBarDone);
    }
    __syncwarp();
  } else {
    reg_inc<208>();
    const int wg = warp >> 2;
    const int w4 = warp & 3;
    const int r = w4 * 32 + lane;  // q row in the tile = tensor-memory lane
    const uint32_t lane_base = static_cast<uint32_t>(w4 * 32) << 16;
    const uint32_t tDp = tmem_base + lane_base + C::kColDp + wg * 64;
    const float2 sc2 = make_float2(scale_log2, scale_log2);
    const float2 scale2 = make_float2(scale, scale);
    bool ok = mbar_wait_warp(bar(C::kBarQ), 0, w, kBSiteCmpQ);
    float2 nlse2 = make_float2(0.f, 0.f), ndlt2 = make_float2(0.f, 0.f);
    if (ok) {
      const float* stats = reinterpret_cast<const float*>(smem + C::kOffStats);
      nlse2 = make_float2(stats[r], stats[r]);              // -lse*log2e of this row
      ndlt2 = make_float2(stats[128 + r], stats[128 + r]);  // -delta of this row
    }
    for (int j = 0; ok && j < nkv; ++j) {
      const uint32_t tS = tmem_base + lane_base + C::kColS + (j & 1) * 128 + wg * 64;
      if (!(ok = mbar_wait_warp(bar(C::kBarSFull + (j & 1)), (j >> 1) & 1, w, kBSiteCmpSt))) break;
      tc_fence_after();
      float2 p[32];
      {
        uint32_t sr[64];
        tmem_ld_x32(tS, sr);
        tmem_ld_x32(tS + 32, sr + 32);
        tmem_wait_ld();
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const float2 t = __ffma2_rn(
              make_float2(__uint_as_float(sr[2 * c]), __uint_as_float(sr[2 * c + 1])), sc2, nlse2);
          p[c] = exp2_pair(t, c);
        }
      }
      if (j == qt || j * 128 + 128 > Nk) {
        // diagonal tile: keep kv <= q; last KV tile: drop the columns beyond the last key
        int last = j == qt ? r : 127;
        last = last < Nk - 1 - j * 128 ? last : Nk - 1 - j * 128;
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          p[c].x = (wg * 64 + 2 * c <= last) ? p[c].x : 0.f;
          p[c].y = (wg * 64 + 2 * c + 1 <= last) ? p[c].y : 0.f;
        }
      }
      if (!(ok = mbar_wait_warp(bar(C::kBarDpFull), j & 1, w, kBSiteCmpDpt))) break;
      tc_fence_after();
      uint32_t dp[64];
      tmem_ld_x32(tDp, dp);
      tmem_ld_x32(tDp + 32, dp + 32);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(C::kBarDpConsumed));
      uint32_t dsk[32];
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        float2 u = __fadd2_rn(
            make_float2(__uint_as_float(dp[2 * c]), __uint_as_float(dp[2 * c + 1])), ndlt2);
        u = __fmul2_rn(__fmul2_rn(p[c], u), scale2);
        dsk[c] = pack2<BF16>(u.x, u.y);
      }
      tmem_st_x32(tS, dsk);  // over the score columns this thread has already read
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(C::kBarDsReady));
    }
    if (ok && wg == 0 && mbar_wait_warp(bar(C::kBarDone), 0, w, kBSiteCmpDone)) {
      tc_fence_after();
      store_rows_16bit<D, BF16>(tmem_base + lane_base + C::kColDQ, smem + C::kOffDO, w4, lane, &tdq,
                                qt * 128, hc, N);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == C::kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// =========================================================================================
// One output tile from spilled 16-bit tiles (spill mode).  A CTA owns one output tile and adds
// one tensor-core product per tile pair in ascending order, no exponentials; the kernel is bound
// by reading the 32 KiB scratch tile per product from HBM.
//   FORM 2: dQ(qt) = sum_j dS(j, qt) K_j      A = dS^T tile transposed (MN-major pieces)
//   FORM 0: dV(jt) = sum_i P(jt, i)^T dO_i    A = P^T tile as stored   (K-major pieces)
//   FORM 1: dK(jt) = sum_i dS(jt, i)^T Q_i    A = dS^T tile as stored  (K-major pieces)
// (forms 0 and 1 serve head dim 256, where dK and dV do not fit next to the scores in tensor
// memory.)
//   warps 0-3  epilogue (tensor memory -> 16 bit -> TMA store)
//   warp  4    TMA producer: ring of kStages x (scratch tile + operand tile)
//   warp  5    MMA issue
// =========================================================================================
template <int D>
struct ConsumeCfg {
  using T = Tile<D>;
  static constexpr int kStages = D == 256 ? 2 : (D == 128 ? 3 : 4);
  static constexpr int kThreads = 192;
  static constexpr int kLoadWarp = 4;
  static constexpr int kMmaWarp = 5;
  static constexpr int kStageBytes = 32768 + T::kTileBytes;  // scratch tile, then the operand tile
  static constexpr int kOffBar = kStages * kStageBytes;
  static constexpr int kBarFull = 0;
  static constexpr int kBarEmpty = kStages;
  static constexpr int kBarDone = 2 * kStages;
  static constexpr int kNumBars = kBarDone + 1;
  static constexpr int kSmemBytes = kOffBar + kNumBars * 8 + 16;
  static constexpr int kTmemCols = D < 32 ? 32 : D;
  static_assert(kSmemBytes <= 232448, "shared memory budget of one CTA");
};

template <int D, bool BF16, int FORM>
__global__ void __launch_bounds__(ConsumeCfg<D>::kThreads, 1)
    bwd_consume_kernel(const uint4* __restrict__ scratch, const __grid_constant__ CUtensorMap tb,
                       const __grid_constant__ CUtensorMap tout, int N, int Nk, int* status) {
  using C = ConsumeCfg<D>;
  using T = Tile<D>;
  extern __shared__ __align__(1024) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = smem_u32(smem);
  if (smem_base & 1023u) {
    if (threadIdx.x == 0) atomicCAS(status, 0, 0x20000 | kBSiteAlign);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kOffBar);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + C::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  auto bar = [&](int i) { return smem_base + C::kOffBar + 8u * i; };

  const int ntiles = (N + 127) >> 7;     // Q tiles
  const int nktiles = (Nk + 127) >> 7;   // KV tiles
  const HeadCoord hc{static_cast<int>(blockIdx.y), static_cast<int>(blockIdx.z)};  // grid (tiles, H, B)
  const int bh = hc.b * static_cast<int>(gridDim.y) + hc.h;
  const int head_tile0 = bh * dstile_count(ntiles, nktiles);
  // The output tile and the range of tiles it is summed over (heaviest output tile first).
  const int ot = FORM == 2 ? ntiles - 1 - static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x);
  const int first = FORM == 2 ? 0 : ot;
  const int count = FORM == 2 ? (ot + 1 < nktiles ? ot + 1 : nktiles) : ntiles - ot;
  const int out_rows = FORM == 2 ? N : Nk;

  if (threadIdx.x == 0) {
    for (int i = 0; i < C::kStages; ++i) {
      mbar_init(bar(C::kBarFull + i), 1);
      mbar_init(bar(C::kBarEmpty + i), 1);
    }
    mbar_init(bar(C::kBarDone), 1);
    *abort_flag = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == C::kMmaWarp) {
    tmem_alloc(smem_u32(tmem_slot), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const WaitCtx w{abort_flag, status};

  if (warp == C::kLoadWarp) {
    const uint32_t elected = elect_one();
    if (elected) prefetch_tensormap(&tb);
    for (int n = 0; n < count; ++n) {
      const int st = n % C::kStages, ph = (n / C::kStages) & 1;
      if (!mbar_wait_warp(bar(C::kBarEmpty + st), ph ^ 1, w, kBSiteLoadQ)) break;
      if (elected) {
        const uint32_t dst = smem_base + st * C::kStageBytes;
        const int other = first + n;  // the KV tile (form 2) or Q tile (forms 0, 1) of this product
        // pair (KV tile, Q tile) -> scratch tile: pairs of a head are numbered KV tile by KV tile
        const int tile = FORM == 2 ? head_tile0 + dstile_count(ntiles, other) + (ot - other)
                                   : head_tile0 + dstile_count(ntiles, ot) + n;
        mbar_arrive_expect_tx(bar(C::kBarFull + st), C::kStageBytes);
        bulk_load_1d(dst, scratch + static_cast<size_t>(tile) * 2048, 32768,
                     bar(C::kBarFull + st));  // a tile is 32 KiB, stored as it is used
#pragma unroll
        for (int ch = 0; ch < T::kChunks; ++ch)
          tma_load_4d(dst + 32768 + ch * T::kChunkTileBytes, &tb, ch * T::kChunkElems, other * 128,
                      hc, bar(C::kBarFull + st));
      }
    }
    __syncwarp();
  } else if (warp == C::kMmaWarp) {
    const uint32_t elected = elect_one();
    bool ok = true;
    for (int n = 0; ok && n < count; ++n) {
      const int st = n % C::kStages, ph = (n / C::kStages) & 1;
      if (!(ok = mbar_wait(bar(C::kBarFull + st), ph, w, kBSiteMmaKV))) break;
      const uint32_t src = smem_base + st * C::kStageBytes;
      // out[128, D] += A * B; B = the operand tile (d contiguous, MN-major)
      if constexpr (FORM == 2)
        issue_piecesT_x_tile<D, BF16>(elected, tmem_base, src, src + 32768, n > 0);
      else
        issue_pieces_x_tile<D, BF16>(elected, tmem_base, src, src + 32768, n > 0);
      if (elected) mma_commit(bar(C::kBarEmpty + st));
    }
    if (ok && elected) mma_commit(bar(C::kBarDone));
    __syncwarp();
  } else {
    if (mbar_wait_warp(bar(C::kBarDone), 0, w, kBSiteCmpDone)) {
      tc_fence_after();
      const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
      // every product has completed, so the ring is idle: stage through its first buffer
      store_rows_16bit<D, BF16>(tmem_base + lane_base, smem, warp, lane, &tout, ot * 128, hc,
                                out_rows);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == C::kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// =========================================================================================
// Head dim 256: scores only.  dK and dV alone would fill the 512 tensor-memory columns, so the
// backward is split: this kernel forms P^T and dS^T for every (KV tile, Q tile) pair and writes
// both as 16-bit piece-major tiles to two scratch tensors; bwd_consume_kernel then forms dV, dK
// and dQ from them.  CTA = one KV tile.  K and V stay in shared memory as two half tiles each
// (128 KiB); Q and dO stream through a ring of three half-tile slots; St and dPt are double
// buffered in tensor memory (4 x 128 columns) and accumulate over the two halves of the head dim.
//   warps 0-7  compute (as in bwd_dkdv_kernel: kv row per thread, two groups of 64 q columns)
//   warp  8    MMA issue: St(i) = K_lo Q_lo^T + K_hi Q_hi^T, dPt(i) = V_lo dO_lo^T + V_hi dO_hi^T
//   warp  9    TMA producer
// =========================================================================================
struct ScoresCfg {
  using T = Tile<128>;
  static constexpr int kThreads = 384;
  static constexpr int kMmaWarp = 8;
  static constexpr int kLoadWarp = 9;
  static constexpr int kRing = 3;
  static constexpr int kOffK = 0;                                   // K_lo, K_hi
  static constexpr int kOffV = 2 * T::kTileBytes;                   // V_lo, V_hi
  static constexpr int kOffRing = 4 * T::kTileBytes;                // Q_lo, Q_hi, dO_lo, dO_hi stream
  static constexpr int kOffStats = kOffRing + kRing * T::kTileBytes;  // [2][256] fp32
  static constexpr int kOffBar = kOffStats + 2 * 1024;
  static constexpr int kBarKV = 0;
  static constexpr int kBarRingFull = 1;
  static constexpr int kBarRingEmpty = kBarRingFull + kRing;
  static constexpr int kBarStFull = kBarRingEmpty + kRing;  // 2
  static constexpr int kBarStFree = kBarStFull + 2;         // 2, 8 arrivals
  static constexpr int kBarDptFull = kBarStFree + 2;        // 2
  static constexpr int kBarDptFree = kBarDptFull + 2;       // 2, 8 arrivals
  static constexpr int kBarStatsFull = kBarDptFree + 2;     // 2
  static constexpr int kBarStatsFree = kBarStatsFull + 2;   // 2, 8 arrivals
  static constexpr int kNumBars = kBarStatsFree + 2;
  static constexpr int kSmemBytes = kOffBar + kNumBars * 8 + 16;
  static_assert(kSmemBytes <= 232448, "shared memory budget of one CTA");
  static constexpr int kColSt = 0;     // 2 x 128
  static constexpr int kColDpt = 256;  // 2 x 128
  static constexpr int kTmemCols = 512;
};

template <bool BF16>
__global__ void __launch_bounds__(ScoresCfg::kThreads, 1)
    bwd_scores_wide_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                           const __grid_constant__ CUtensorMap tv,
                           const __grid_constant__ CUtensorMap tdo, const float* __restrict__ rowstats,
                           uint4* __restrict__ p_scratch, uint4* __restrict__ ds_scratch, int N, int Nk,
                           float scale, float scale_log2, int* status) {
  using C = ScoresCfg;
  using T = Tile<128>;
  extern __shared__ __align__(1024) uint8_t smem[];
  constexpr int kWarps = C::kThreads / 32;
  const int warp = ((threadIdx.x >> 5) + C::kMmaWarp) % kWarps, lane = threadIdx.x & 31;
  const uint32_t smem_base = smem_u32(smem);
  if (smem_base & 1023u) {
    if (threadIdx.x == 0) atomicCAS(status, 0, 0x20000 | kBSiteAlign);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kOffBar);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + C::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  auto bar = [&](int i) { return smem_base + C::kOffBar + 8u * i; };

  const int ntiles = (N + 127) >> 7;
  const int nktiles = (Nk + 127) >> 7;
  const int jt = blockIdx.x;  // KV tile
  const HeadCoord hc{static_cast<int>(blockIdx.y), static_cast<int>(blockIdx.z)};  // grid (tiles, H, B)
  const int bh = hc.b * static_cast<int>(gridDim.y) + hc.h;
  const int nq = ntiles - jt;  // Q tiles jt .. ntiles-1
  const bool kv_ragged = jt * 128 + 128 > Nk;
  const int tile0 = bh * dstile_count(ntiles, nktiles) + dstile_count(ntiles, jt);

  if (threadIdx.x == 0) {
    mbar_init(bar(C::kBarKV), 1);
    for (int i = 0; i < C::kRing; ++i) {
      mbar_init(bar(C::kBarRingFull + i), 1);
      mbar_init(bar(C::kBarRingEmpty + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(C::kBarStFull + i), 1);
      mbar_init(bar(C::kBarStFree + i), 8);
      mbar_init(bar(C::kBarDptFull + i), 1);
      mbar_init(bar(C::kBarDptFree + i), 8);
      mbar_init(bar(C::kBarStatsFull + i), 1);
      mbar_init(bar(C::kBarStatsFree + i), 8);
    }
    *abort_flag = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == C::kMmaWarp) {
    tmem_alloc(smem_u32(tmem_slot), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const WaitCtx w{abort_flag, status};

  if (warp >= C::kMmaWarp) {
    reg_dec<72>();
    if (warp == C::kLoadWarp) {
      const uint32_t elected = elect_one();
      if (elected) {
        prefetch_tensormap(&tq);
        prefetch_tensormap(&tk);
        prefetch_tensormap(&tv);
        prefetch_tensormap(&tdo);
        mbar_arrive_expect_tx(bar(C::kBarKV), 4 * T::kTileBytes);
        for (int half = 0; half < 2; ++half)
          for (int ch = 0; ch < T::kChunks; ++ch) {
            tma_load_4d(smem_base + C::kOffK + half * T::kTileBytes + ch * T::kChunkTileBytes, &tk,
                        half * 128 + ch * T::kChunkElems, jt * 128, hc, bar(C::kBarKV));
            tma_load_4d(smem_base + C::kOffV + half * T::kTileBytes + ch * T::kChunkTileBytes, &tv,
                        half * 128 + ch * T::kChunkElems, jt * 128, hc, bar(C::kBarKV));
          }
      }
      bool ok = true;
      for (int i = 0; ok && i < nq; ++i) {
        const int qt = jt + i;
        // rowstats of Q tile qt -> stats buffer i % 2, once the compute warps are done with
        // tile i - 2
        if (!(ok = mbar_wait_warp(bar(C::kBarStatsFree + (i & 1)), ((i >> 1) & 1) ^ 1, w, kBSiteLoadQ)))
          break;
        if (elected) {
          mbar_arrive_expect_tx(bar(C::kBarStatsFull + (i & 1)), 1024);
          bulk_load_1d(smem_base + C::kOffStats + (i & 1) * 1024,
                       rowstats + (static_cast<size_t>(bh) * ntiles + qt) * 256, 1024,
                       bar(C::kBarStatsFull + (i & 1)));
        }
        for (int sub = 0; sub < 4; ++sub) {  // Q_lo, Q_hi, dO_lo, dO_hi
          const int t = 4 * i + sub, slot = t % C::kRing, ph = (t / C::kRing) & 1;
          if (!(ok = mbar_wait_warp(bar(C::kBarRingEmpty + slot), ph ^ 1, w, kBSiteLoadDO))) break;
          if (elected) {
            mbar_arrive_expect_tx(bar(C::kBarRingFull + slot), T::kTileBytes);
#pragma unroll
            for (int ch = 0; ch < T::kChunks; ++ch)
              tma_load_4d(smem_base + C::kOffRing + slot * T::kTileBytes + ch * T::kChunkTileBytes,
                          sub < 2 ? &tq : &tdo, (sub & 1) * 128 + ch * T::kChunkElems, qt * 128, hc,
                          bar(C::kBarRingFull + slot));
          }
        }
      }
    } else if (warp == C::kMmaWarp) {
      const uint32_t elected = elect_one();
      auto commit = [&](int b) {
        if (elected) mma_commit(bar(b));
      };
      bool ok = mbar_wait(bar(C::kBarKV), 0, w, kBSiteMmaKV);
      for (int i = 0; ok && i < nq; ++i) {
        const int b = i & 1, u = i >> 1;  // tensor-memory buffer and its use count
        for (int prod = 0; ok && prod < 2; ++prod) {  // 0: St(i), 1: dPt(i)
          if (u > 0) {
            // the compute warps have copied use u - 1 of this buffer into registers
            if (!(ok = mbar_wait(bar((prod ? C::kBarDptFree : C::kBarStFree) + b), (u - 1) & 1, w,
                                 kBSiteMmaDrain)))
              break;
            tc_fence_after();
          }
          for (int half = 0; ok && half < 2; ++half) {
            const int t = 4 * i + 2 * prod + half, slot = t % C::kRing, ph = (t / C::kRing) & 1;
            if (!(ok = mbar_wait(bar(C::kBarRingFull + slot), ph, w, kBSiteMmaQ))) break;
            issue_rows_x_rows<128, BF16>(
                elected, tmem_base + (prod ? C::kColDpt : C::kColSt) + b * 128,
                smem_base + (prod ? C::kOffV : C::kOffK) + half * T::kTileBytes,
                smem_base + C::kOffRing + slot * T::kTileBytes, half);
            commit(C::kBarRingEmpty + slot);
          }
          if (ok) commit((prod ? C::kBarDptFull : C::kBarStFull) + b);
        }
      }
    }
    __syncwarp();
  } else {
    reg_inc<208>();
    const int wg = warp >> 2;  // 0: q columns 0..63 of the tile, 1: 64..127
    const int w4 = warp & 3;
    const int r = w4 * 32 + lane;  // kv row in the tile = tensor-memory lane
    const uint32_t lane_base = static_cast<uint32_t>(w4 * 32) << 16;
    const float2 sc2 = make_float2(scale_log2, scale_log2);
    const float2 scale2 = make_float2(scale, scale);
    bool ok = true;
    for (int i = 0; i < nq; ++i) {
      const int b = i & 1, u = i >> 1;
      const uint32_t tSt = tmem_base + lane_base + C::kColSt + b * 128 + wg * 64;
      const uint32_t tDpt = tmem_base + lane_base + C::kColDpt + b * 128 + wg * 64;
      const float* stats = reinterpret_cast<const float*>(smem + C::kOffStats + b * 1024);
      const float4* nlse = reinterpret_cast<const float4*>(stats + wg * 64);        // -lse*log2e
      const float4* ndlt = reinterpret_cast<const float4*>(stats + 128 + wg * 64);  // -delta
      const size_t out_off = static_cast<size_t>(tile0 + i) * 2048 + wg * 1024 + r;
      if (!(ok = mbar_wait_warp(bar(C::kBarStatsFull + b), u & 1, w, kBSiteCmpQ))) break;
      if (!(ok = mbar_wait_warp(bar(C::kBarStFull + b), u & 1, w, kBSiteCmpSt))) break;
      tc_fence_after();
      float2 p[32];  // P^T for this thread's kv row, q columns wg*64 .. wg*64+63
      {
        uint32_t sr[64];
        tmem_ld_x32(tSt, sr);
        tmem_ld_x32(tSt + 32, sr + 32);
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(C::kBarStFree + b));  // St(i + 2) may overwrite the buffer
        probabilities_of_row(sr, nlse, sc2, p);
      }
      if (i == 0 || kv_ragged) {
        // diagonal tile: keep q >= kv; rows beyond the last key keep nothing
        mask_row(p, (jt * 128 + r >= Nk) ? 128 : (i == 0 ? r : 0), wg * 64);
      }
      {
        // P^T rounded to 16 bits, piece-major (see bwd_dkdv_kernel's spill store)
        uint4* dst = p_scratch + out_off;
#pragma unroll
        for (int pc = 0; pc < 8; ++pc)
          dst[pc * 128] = make_uint4(pack2<BF16>(p[4 * pc].x, p[4 * pc].y),
                                     pack2<BF16>(p[4 * pc + 1].x, p[4 * pc + 1].y),
                                     pack2<BF16>(p[4 * pc + 2].x, p[4 * pc + 2].y),
                                     pack2<BF16>(p[4 * pc + 3].x, p[4 * pc + 3].y));
      }
      if (!(ok = mbar_wait_warp(bar(C::kBarDptFull + b), u & 1, w, kBSiteCmpDpt))) break;
      tc_fence_after();
      uint32_t dp[64];
      tmem_ld_x32(tDpt, dp);
      tmem_ld_x32(tDpt + 32, dp + 32);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(C::kBarDptFree + b));
      uint32_t dsk[32];
#pragma unroll
      for (int c4 = 0; c4 < 16; ++c4) {
        const float4 nd = ndlt[c4];
        // dS = P * (dP - delta) * scale, scale folded in before the 16-bit rounding
        float2 u0 = __fadd2_rn(make_float2(__uint_as_float(dp[4 * c4]), __uint_as_float(dp[4 * c4 + 1])),
                               make_float2(nd.x, nd.y));
        float2 u1 = __fadd2_rn(make_float2(__uint_as_float(dp[4 * c4 + 2]), __uint_as_float(dp[4 * c4 + 3])),
                               make_float2(nd.z, nd.w));
        u0 = __fmul2_rn(__fmul2_rn(p[2 * c4], u0), scale2);
        u1 = __fmul2_rn(__fmul2_rn(p[2 * c4 + 1], u1), scale2);
        dsk[2 * c4] = pack2<BF16>(u0.x, u0.y);
        dsk[2 * c4 + 1] = pack2<BF16>(u1.x, u1.y);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(C::kBarStatsFree + b));  // the row statistics are consumed
      {
        uint4* dst = ds_scratch + out_off;
#pragma unroll
        for (int pc = 0; pc < 8; ++pc)
          dst[pc * 128] = make_uint4(dsk[4 * pc], dsk[4 * pc + 1], dsk[4 * pc + 2], dsk[4 * pc + 3]);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == C::kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

template <bool BF16>
cudaError_t launch_scores_wide_t(const AttnShape& s, const CUtensorMap& tq, const CUtensorMap& tk,
                                 const CUtensorMap& tv, const CUtensorMap& tdo, const float* rowstats,
                                 void* p_scratch, void* ds_scratch, int* status,
                                 cudaStream_t stream) {
  using C = ScoresCfg;
  auto kern = bwd_scores_wide_kernel<BF16>;
  cudaError_t e =
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
  if (e != cudaSuccess) return e;
  dim3 grid((s.Nk + 127) / 128, s.H, s.B);  // one CTA per KV tile
  kern<<<grid, C::kThreads, C::kSmemBytes, stream>>>(
      tq, tk, tv, tdo, rowstats, static_cast<uint4*>(p_scratch), static_cast<uint4*>(ds_scratch),
      s.N, s.Nk, s.scale, s.scale * 1.4426950408889634f, status);
  return cudaGetLastError();
}

template <int D, bool BF16, int MODE>
cudaError_t launch_dkdv_t(const AttnShape& s, const CUtensorMap& tq, const CUtensorMap& tk,
                          const CUtensorMap& tv, const CUtensorMap& tdo, const CUtensorMap& tdk,
                          const CUtensorMap& tdv, const float* rowstats, float* dq_accum,
                          int* status, cudaStream_t stream) {
  using C = DkdvCfg<D, MODE>;
  auto kern = bwd_dkdv_kernel<D, BF16, MODE>;
  cudaError_t e =
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
  if (e != cudaSuccess) return e;
  dim3 grid((s.Nk + 127) / 128, s.H, s.B);  // one CTA per KV tile
  kern<<<grid, C::kThreads, C::kSmemBytes, stream>>>(tq, tk, tv, tdo, tdk, tdv, rowstats, dq_accum,
                                                     s.N, s.Nk, s.scale,
                                                     s.scale * 1.4426950408889634f, status);
  return cudaGetLastError();
}

template <int D, bool BF16, int FORM>
cudaError_t launch_consume_t(const AttnShape& s, const void* scratch, const CUtensorMap& tb,
                             const CUtensorMap& tout, int* status, cudaStream_t stream) {
  using C = ConsumeCfg<D>;
  auto kern = bwd_consume_kernel<D, BF16, FORM>;
  cudaError_t e =
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
  if (e != cudaSuccess) return e;
  dim3 grid(((FORM == 2 ? s.N : s.Nk) + 127) / 128, s.H, s.B);  // one CTA per output tile
  kern<<<grid, C::kThreads, C::kSmemBytes, stream>>>(static_cast<const uint4*>(scratch), tb, tout,
                                                     s.N, s.Nk, status);
  return cudaGetLastError();
}

template <int D, bool BF16>
cudaError_t launch_dq_t(const AttnShape& s, const CUtensorMap& tq, const CUtensorMap& tk,
                        const CUtensorMap& tv, const CUtensorMap& tdo, const CUtensorMap& tdq,
                        const float* rowstats, int* status, cudaStream_t stream) {
  using C = DqCfg<D>;
  auto kern = bwd_dq_kernel<D, BF16>;
  cudaError_t e =
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
  if (e != cudaSuccess) return e;
  const int ntiles = (s.N + 127) / 128;
  dim3 grid(ntiles, s.H, s.B);
  kern<<<grid, C::kThreads, C::kSmemBytes, stream>>>(tq, tk, tv, tdo, tdq, rowstats, s.N, s.Nk,
                                                     s.scale, s.scale * 1.4426950408889634f,
                                                     status);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_bwd_dkdv(const AttnShape& s, const CUtensorMap& tq, const CUtensorMap& tk,
                            const CUtensorMap& tv, const CUtensorMap& tdo,
                            const CUtensorMap& tdk, const CUtensorMap& tdv,
                            const float* rowstats, float* dq_accum, int mode, int* status,
                            cudaStream_t stream) {
  // modes: 0 dK/dV only, 1 fused atomic dQ (dq_accum = fp32 accumulator), 2 spill dS tiles
  // (dq_accum = the 16-bit scratch tensor)
#define FA2_ARGS s, tq, tk, tv, tdo, tdk, tdv, rowstats, dq_accum, status, stream
#define FA2_CASE(DD)                                                                        \
  case DD:                                                                                  \
    if (mode == 1)                                                                          \
      return s.dtype ? launch_dkdv_t<DD, true, 1>(FA2_ARGS)                                 \
                     : launch_dkdv_t<DD, false, 1>(FA2_ARGS);                               \
    if (mode == 2)                                                                          \
      return s.dtype ? launch_dkdv_t<DD, true, 2>(FA2_ARGS)                                 \
                     : launch_dkdv_t<DD, false, 2>(FA2_ARGS);                               \
    return s.dtype ? launch_dkdv_t<DD, true, 0>(FA2_ARGS)                                   \
                   : launch_dkdv_t<DD, false, 0>(FA2_ARGS);
  switch (s.D) {
    FA2_CASE(32)
    FA2_CASE(64)
    FA2_CASE(128)
  }
#undef FA2_CASE
#undef FA2_ARGS
  return cudaErrorInvalidValue;
}

cudaError_t launch_bwd_dq(const AttnShape& s, const CUtensorMap& tq, const CUtensorMap& tk,
                          const CUtensorMap& tv, const CUtensorMap& tdo, const CUtensorMap& tdq,
                          const float* rowstats, int* status, cudaStream_t stream) {
#define FA2_ARGS s, tq, tk, tv, tdo, tdq, rowstats, status, stream
#define FA2_CASE(DD)                                                   \
  case DD:                                                             \
    return s.dtype ? launch_dq_t<DD, true>(FA2_ARGS)                   \
                   : launch_dq_t<DD, false>(FA2_ARGS);
  switch (s.D) {
    FA2_CASE(32)
    FA2_CASE(64)
    FA2_CASE(128)
  }
#undef FA2_CASE
#undef FA2_ARGS
  return cudaErrorInvalidValue;
}

cudaError_t launch_bwd_scores_wide(const AttnShape& s, const CUtensorMap& tq, const CUtensorMap& tk,
                                   const CUtensorMap& tv, const CUtensorMap& tdo,
                                   const float* rowstats, void* p_scratch, void* ds_scratch,
                                   int* status, cudaStream_t stream) {
  return s.dtype ? launch_scores_wide_t<true>(s, tq, tk, tv, tdo, rowstats, p_scratch, ds_scratch,
                                              status, stream)
                 : launch_scores_wide_t<false>(s, tq, tk, tv, tdo, rowstats, p_scratch, ds_scratch,
                                               status, stream);
}

cudaError_t launch_bwd_consume(const AttnShape& s, int form, const void* scratch,
                               const CUtensorMap& tb, const CUtensorMap& tout, int* status,
                               cudaStream_t stream) {
#define FA2_ARGS s, scratch, tb, tout, status, stream
#define FA2_CASE(DD)                                                      \
  case DD:                                                                \
    return s.dtype ? launch_consume_t<DD, true, 2>(FA2_ARGS)              \
                   : launch_consume_t<DD, false, 2>(FA2_ARGS);
  if (s.D == 256) {
    if (form == 0)
      return s.dtype ? launch_consume_t<256, true, 0>(FA2_ARGS) : launch_consume_t<256, false, 0>(FA2_ARGS);
    if (form == 1)
      return s.dtype ? launch_consume_t<256, true, 1>(FA2_ARGS) : launch_consume_t<256, false, 1>(FA2_ARGS);
    return s.dtype ? launch_consume_t<256, true, 2>(FA2_ARGS) : launch_consume_t<256, false, 2>(FA2_ARGS);
  }
  if (form != 2) return cudaErrorInvalidValue;
  switch (s.D) {
    FA2_CASE(32)
    FA2_CASE(64)
    FA2_CASE(128)
  }
#undef FA2_CASE
#undef FA2_ARGS
  return cudaErrorInvalidValue;
}

}  // namespace fa2
