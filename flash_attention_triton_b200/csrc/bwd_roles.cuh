// Device-side building blocks of the backward kernels: the per-tile arithmetic helpers, and the
// warp-role bodies of the two work-item kinds that more than one kernel runs:
//   dkdv_roles     one KV tile of one (batch, head): dK, dV (and, by mode, dQ atomics or the
//                  spilled dS^T tiles), used by bwd_dkdv_kernel;
//   consume_roles  one output tile summed from spilled 16-bit tiles, used by bwd_consume_kernel.
// The maths is that of _backward_kernel_one_col_block
// (src/flash_attention_triton/_triton_kernels_v2.py:312-343 of the reference).
#pragma once
#include "common.cuh"
#include "mma_issue.cuh"
#include "ptx.cuh"

#ifndef FA2_BWD_POLY_PAIRS_PER_8
#define FA2_BWD_POLY_PAIRS_PER_8 4  // of every 8 column pairs, this many use ex2_poly2
#endif

namespace fa2 {

// 2^x for column pair `c` (compile-time index after unrolling): SHARE of every 8 pairs go to
// the FMA-pipe polynomial, the rest to the MUFU, because 128 x 128 exponentials per tile pair
// would otherwise keep the MUFU (16 / clk / SM) busy for 1024 cycles.
template <int SHARE = FA2_BWD_POLY_PAIRS_PER_8>
__device__ __forceinline__ float2 exp2_pair(float2 x, int c) {
  if ((c & 7) < SHARE) return ex2_poly2(x);
  return make_float2(ex2(x.x), ex2(x.y));
}
// Share used by the transposed-score kernels.  At head dims up to 64 the tensor pipe has time to
// spare and the compute warps' instruction stream is what a tile pair waits for, so fewer
// exponentials go to the (longer) polynomial: measured on the fused-atomics kernel 6-8 % faster
// with 2 than with 4, the other modes within 3 % either way.  A function of the head dim only, so
// that P, and with it dK and dV, have the same bits in every mode.
template <int D>
constexpr int kPolyShareT = D <= 64 ? 2 : FA2_BWD_POLY_PAIRS_PER_8;

__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c),
               "f"(d)
               : "memory");
}

// The transposed-score kernels (bwd_dkdv_kernel, bwd_scores_wide_kernel) give each thread one kv
// row and 64 q columns of a tile.  probabilities_of_row: p = 2^(s * c - lse2[q]) from the raw
// scores `sr` and the negated, log2-scaled row statistics of the 64 columns (`nlse`, read with
// warp-wide broadcasts).  mask_row: keep only the q columns >= `first` (128 keeps nothing).
template <int SHARE = FA2_BWD_POLY_PAIRS_PER_8>
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
    p[2 * c4] = exp2_pair<SHARE>(t0, 2 * c4);
    p[2 * c4 + 1] = exp2_pair<SHARE>(t1, 2 * c4 + 1);
  }
}
__device__ __forceinline__ void mask_row(float2 (&p)[32], int first_column, int column0) {
#pragma unroll
  for (int c = 0; c < 32; ++c) {
    p[c].x = (column0 + 2 * c >= first_column) ? p[c].x : 0.f;
    p[c].y = (column0 + 2 * c + 1 >= first_column) ? p[c].y : 0.f;
  }
}

// Epilogue helper: one warp multiplies its 32 rows of a [128, D] fp32 accumulator by `mul` (a power
// of two, see head_dscale), converts them to 16 bits, stages them swizzled in `stage` (a free
// tile buffer) and stores them with one TMA per chunk.
template <int D, bool BF16>
__device__ __forceinline__ void store_rows_16bit(uint32_t tmem_row_addr, uint8_t* stage, int warp4,
                                                 int lane, const CUtensorMap* map, int row_base,
                                                 HeadCoord hc, int N, float mul = 1.0f) {
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
      val.x = pack2<BF16>(__uint_as_float(v[8 * p + 0]) * mul, __uint_as_float(v[8 * p + 1]) * mul);
      val.y = pack2<BF16>(__uint_as_float(v[8 * p + 2]) * mul, __uint_as_float(v[8 * p + 3]) * mul);
      val.z = pack2<BF16>(__uint_as_float(v[8 * p + 4]) * mul, __uint_as_float(v[8 * p + 5]) * mul);
      val.w = pack2<BF16>(__uint_as_float(v[8 * p + 6]) * mul, __uint_as_float(v[8 * p + 7]) * mul);
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

// dS is rounded to 16 bits; in fp16 the exponent range (6e-8 .. 65504) is narrow, and upstream
// gradients dO of 1e-4 already push dS into the subnormals.  dS is linear in dO, so the kernels
// form dS * 2^k with the power of two that brings the largest |dO| of the (batch, head) problem
// into [1, 2) and multiply the dK and dQ accumulators, which are linear in dS, by 2^-k before
// the final rounding: exact, as long as nothing leaves the 16-bit range, and independent of how the
// (batch, head) problems are partitioned.  `tile_amax` holds, per Q tile of the head, the largest
// |dO| as its 16-bit pattern with the sign cleared (written by the preprocess kernel); called by
// a whole warp.  Returns 2^k and stores 2^-k in *inverse; 1 for an all-zero or non-finite head.
template <bool BF16>
__device__ __forceinline__ float head_dscale(const unsigned* __restrict__ tile_amax, int ntiles,
                                             int lane, float* inverse) {
  unsigned m = 0;
  for (int t = lane; t < ntiles; t += 32) m = max(m, __ldg(tile_amax + t));
  m = __reduce_max_sync(0xffffffffu, m);
  int k = 0;
  if constexpr (BF16) {
    const int e = static_cast<int>((m >> 7) & 0xffu);  // biased by 127
    if (e != 0 && e != 255) k = 127 - e;
  } else {
    const int e = static_cast<int>((m >> 10) & 0x1fu);  // biased by 15
    if (e != 31 && m != 0) k = 15 - (e == 0 ? 1 : e);   // subnormal: the smallest normal exponent
  }
  k = k < -100 ? -100 : (k > 100 ? 100 : k);
  *inverse = __uint_as_float(static_cast<unsigned>(127 - k) << 23);
  return __uint_as_float(static_cast<unsigned>(127 + k) << 23);
}

// Number of (KV tile, Q tile) pairs of one head whose KV tile index is below `jt`, with
// `ntiles` Q tiles: KV tile t meets Q tiles t .. ntiles-1.  Also the index of the first pair
// of KV tile jt among a head's tiles in the dS scratch tensor.
__host__ __device__ __forceinline__ int dstile_count(int ntiles, int jt) {
  return jt * ntiles - jt * (jt - 1) / 2;
}

// =========================================================================================
// dK / dV work item
// =========================================================================================
// MODE 0: dK, dV only (dQ comes from bwd_dq_kernel).  MODE 1 (fused): also dQ, accumulated into
// an fp32 buffer with atomic adds by a fourth warp group.  MODE 2 (spill): also stores every
// 16-bit dS^T tile to a scratch tensor, from which a consumer forms dQ with one product per tile
// pair instead of recomputing S, P, dP.
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

// One dK/dV work item: KV tile `jt` of (batch, head) `hc` (flattened index `bh`).
struct DkdvItem {
  int jt;
  HeadCoord hc;
  int bh;
  const unsigned* tile_amax;  // largest |dO| per Q tile of this head (see head_dscale)
  size_t tile0;         // spill modes: scratch index of the item's first pair (jt, jt)
};

template <int D, int MODE>
__device__ __forceinline__ void dkdv_init_barriers(uint32_t bar0) {
  using C = DkdvCfg<D, MODE>;
  auto bar = [&](int i) { return bar0 + 8u * i; };
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
}

// The warp roles of one dK/dV item.  Called by every thread of the CTA after the barriers of the
// item have been initialised and a CTA-wide barrier has made them visible.  The CTA walks the
// Q tiles of its KV tile from the LAST one down to the diagonal one (ii = 0 is Q tile ntiles-1), so
// that the CTAs of a head, which start at about the same time, read the same Q / dO tiles at about
// the same time (one L2 fill serves them all).  The order is the same in every mode, so dK and dV
// do not depend on the mode bit for bit.
//
// It works on the TRANSPOSED score tile so that everything a later MMA consumes as its A operand
// already sits in tensor memory with kv rows on lanes:
//     St  = K  Q_i^T      (smem x smem)  -> tensor memory, 128 columns
//     dPt = V  dO_i^T     (smem x smem)  -> tensor memory, 128 columns
//     dV += Pt  dO_i      (tmem x smem)     Pt  = 16-bit P^T written over St by the compute warps
//     dK += dSt Q_i       (tmem x smem)     dSt = 16-bit dS^T written over dPt
//     dQ_i = dS K         (smem x smem)     fused variant only: dS^T also goes to shared memory,
//                                           the tile lands over dPt and is added to the fp32
//                                           workspace with vector atomics
// -lse*log2(e) and -delta of a Q tile arrive in shared memory as one 1 KiB bulk copy from the
// tile-blocked rowstats array; padded rows carry -lse = -inf, which makes their P exactly 0.
template <int D, bool BF16, int MODE>
__device__ __forceinline__ void dkdv_roles(
    uint8_t* smem, uint32_t smem_base, uint32_t tmem_base, int warp, int lane,
    const CUtensorMap* tq, const CUtensorMap* tk, const CUtensorMap* tv, const CUtensorMap* tdo,
    const CUtensorMap* tdk, const CUtensorMap* tdv, const float* __restrict__ rowstats,
    float* __restrict__ dq_accum, int N, int Nk, float scale, float scale_log2, const WaitCtx& w,
    const DkdvItem& item) {
  using C = DkdvCfg<D, MODE>;
  constexpr bool FUSE = C::FUSE;
  constexpr bool SPILL = C::SPILL;
  using T = Tile<D>;
  auto bar = [&](int i) { return smem_base + C::kOffBar + 8u * i; };
  const int ntiles = (N + 127) >> 7;
  const int jt = item.jt;
  const HeadCoord hc = item.hc;
  const int bh = item.bh;
  const int nq = ntiles - jt;  // Q tiles ntiles-1 down to jt (N = query rows, Nk <= N = key rows)
  const bool kv_ragged = jt * 128 + 128 > Nk;  // this KV tile has rows beyond the last key

  if (warp >= C::kMmaWarp) {
    // ---------------------------------------------------------------- producer / MMA group
    reg_dec<72>();
    if (warp == C::kLoadWarp) {
      // TMA producer: whole warp, converged; the elected lane arms barriers and issues copies.
      const uint32_t elected = elect_one();
      if (elected) {
        prefetch_tensormap(tq);
        prefetch_tensormap(tk);
        prefetch_tensormap(tv);
        prefetch_tensormap(tdo);
        mbar_arrive_expect_tx(bar(C::kBarKV), 2 * T::kTileBytes);
        for (int ch = 0; ch < T::kChunks; ++ch) {
          tma_load_4d(smem_base + C::kOffK + ch * T::kChunkTileBytes, tk, ch * T::kChunkElems,
                      jt * 128, hc, bar(C::kBarKV));
          tma_load_4d(smem_base + C::kOffV + ch * T::kChunkTileBytes, tv, ch * T::kChunkElems,
                      jt * 128, hc, bar(C::kBarKV));
        }
      }
      for (int ii = 0; ii < nq; ++ii) {
        const int s = ii % C::kStages, ph = (ii / C::kStages) & 1;
        const int qt = ntiles - 1 - ii;
        if (!mbar_wait_warp(bar(C::kBarQEmpty + s), ph ^ 1, w, kBSiteLoadQ)) break;
        if (elected) {
          mbar_arrive_expect_tx(bar(C::kBarQFull + s), T::kTileBytes + 1024);
#pragma unroll
          for (int ch = 0; ch < T::kChunks; ++ch)
            tma_load_4d(smem_base + C::kOffQ + s * T::kTileBytes + ch * T::kChunkTileBytes, tq,
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
            tma_load_4d(smem_base + C::kOffDO + s * T::kTileBytes + ch * T::kChunkTileBytes, tdo,
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
      int s = 0, ph = 0;  // ring stage / phase of step ii (both rings advance together)
      if (warp == C::kMmaWarp) {
        // ------------------------------------------------------------ warp X
        if (ok && (ok = mbar_wait(bar(C::kBarQFull + 0), 0, w, kBSiteMmaQ))) {
          issue_rows_x_rows<D, BF16>(elected, tmem_base + C::kColSt, ka, smem_base + C::kOffQ);
          commit(C::kBarStFull);
          commit(C::kBarQEmpty + 0);
        }
        for (int ii = 0; ok && ii < nq; ++ii) {
          const int s1 = s ^ 1, ph1 = ph ^ s;  // stage / phase of step ii+1 (two stages)
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
    float inv_dscale;
    head_dscale<BF16>(item.tile_amax, ntiles, lane, &inv_dscale);  // dS carries 2^k, dQ gives it back
    for (int ii = 0; ii < nq; ++ii) {
      if (!mbar_wait_warp(bar(C::kBarDqFull), ii & 1, w, kBSiteRedDq)) break;
      tc_fence_after();
      const int qt = ntiles - 1 - ii;
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
        red_add_v4(dst + k * 128, __uint_as_float(v[4 * k]) * inv_dscale,
                   __uint_as_float(v[4 * k + 1]) * inv_dscale, __uint_as_float(v[4 * k + 2]) * inv_dscale,
                   __uint_as_float(v[4 * k + 3]) * inv_dscale);
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
    float inv_dscale;
    const float dscale = head_dscale<BF16>(item.tile_amax, ntiles, lane, &inv_dscale);
    const float2 scale2 = make_float2(scale * dscale, scale * dscale);  // dS = P (dP - delta) scale 2^k
    bool ok = true;
    for (int ii = 0; ii < nq; ++ii) {
      const int s = ii % C::kStages, ph = (ii / C::kStages) & 1;
      const int qt = ntiles - 1 - ii;
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
        probabilities_of_row<kPolyShareT<D>>(sr, nlse, sc2, p);
      }
      if (qt == jt || kv_ragged) {
        // diagonal tile: keep q >= kv; rows beyond the last key (zero-filled K, V) keep nothing,
        // so that a huge 2^(-lse) never meets their zeros
        mask_row(p, (jt * 128 + r >= Nk) ? 128 : (qt == jt ? r : 0), wg * 64);
      }
      {
        uint32_t pk[32];
#pragma unroll
        for (int c = 0; c < 32; ++c) pk[c] = pack2<kInterBF16<BF16>>(p[c].x, p[c].y);
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
          dsk[16 * h + 2 * c4] = pack2<kInterBF16<BF16>>(u0.x, u0.y);
          dsk[16 * h + 2 * c4 + 1] = pack2<kInterBF16<BF16>>(u1.x, u1.y);
        }
      }
      tmem_st_x32(tDpt, dsk);  // columns 128 + wg*64 .. +31
      if constexpr (SPILL) {
        // This thread's 64 values of dS^T(jt, qt) (kv row r, q columns wg*64 ..) straight to pair
        // `tile0 + (qt - jt)` of the scratch tensor.  A tile is stored piece-major: the 16-byte
        // piece (kv row r, q columns 8g .. 8g+7) at byte g * 2048 + r * 16, so one warp
        // instruction writes 512 contiguous bytes, and the tile can later be copied linearly
        // into shared memory as an unswizzled tensor-core operand.  Going through registers
        // keeps the copy out of shared memory, whose bandwidth the operand reads already use up.
        uint4* dst = reinterpret_cast<uint4*>(dq_accum) +
                     ((item.tile0 + static_cast<size_t>(qt - jt)) * 2048 + wg * 1024 + r);
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
                                  tdv, jt * 128, hc, Nk);
      else
        store_rows_16bit<D, BF16>(tmem_base + lane_base + C::kColDK, smem + C::kOffQ, w4, lane,
                                  tdk, jt * 128, hc, Nk, inv_dscale);
    }
  }
}

// =========================================================================================
// One output tile from spilled 16-bit tiles.  The item adds one tensor-core product per tile
// pair in ascending order, no exponentials; its cost is reading the 32 KiB scratch tile (and the
// operand tile) per product.
//   FORM 2: dQ(qt) = sum_j dS(j, qt) K_j      A = dS^T tile transposed (MN-major pieces)
//   FORM 0: dV(jt) = sum_i P(jt, i)^T dO_i    A = P^T tile as stored   (K-major pieces)
//   FORM 1: dK(jt) = sum_i dS(jt, i)^T Q_i    A = dS^T tile as stored  (K-major pieces)
// (forms 0 and 1 serve head dim 256, where dK and dV do not fit next to the scores in tensor
// memory.)  Roles: one producer warp (ring of kStages x (scratch tile + operand tile)), one
// MMA-issuing warp, four epilogue warps (tensor memory -> 16 bit -> TMA store).
// =========================================================================================
template <int STAGES>
__device__ __forceinline__ void consume_init_barriers(uint32_t bar0) {
  for (int i = 0; i < 2 * STAGES; ++i) mbar_init(bar0 + 8u * i, 1);  // full[STAGES], empty[STAGES]
  mbar_init(bar0 + 8u * (2 * STAGES), 1);                            // done
}

struct ConsumeItem {
  int ot;             // output tile
  HeadCoord hc;
  size_t head_tile0;  // scratch index of the head's first pair
  const unsigned* tile_amax;  // forms 1, 2: largest |dO| per Q tile of the head (the tiles are dS * 2^k,
                              // see head_dscale); nullptr for form 0 (P tiles)
};

// epi_warp: 0..3 for the four epilogue warps (warp e owns tensor-memory lanes 32e .. 32e+31),
// -1 for every other warp.
template <int D, bool BF16, int FORM, int STAGES>
__device__ __forceinline__ void consume_roles(uint8_t* ring, uint32_t ring_base, uint32_t bar0,
                                              uint32_t tmem_acc, bool is_load_warp, bool is_mma_warp,
                                              int epi_warp, int lane, const uint4* __restrict__ scratch,
                                              const CUtensorMap* tb, const CUtensorMap* tout, int N,
                                              int Nk, const WaitCtx& w, const ConsumeItem& item) {
  using T = Tile<D>;
  constexpr int kStageBytes = 32768 + T::kTileBytes;  // scratch tile, then the operand tile
  auto full = [&](int i) { return bar0 + 8u * i; };
  auto empty = [&](int i) { return bar0 + 8u * (STAGES + i); };
  const uint32_t done = bar0 + 8u * (2 * STAGES);
  const int ntiles = (N + 127) >> 7;     // Q tiles
  const int nktiles = (Nk + 127) >> 7;   // KV tiles
  const int ot = item.ot;
  // the range of scratch tiles the output tile is summed over
  const int first = FORM == 2 ? 0 : ot;
  const int count = FORM == 2 ? (ot + 1 < nktiles ? ot + 1 : nktiles) : ntiles - ot;
  const int out_rows = FORM == 2 ? N : Nk;

  if (is_load_warp) {
    const uint32_t elected = elect_one();
    if (elected) prefetch_tensormap(tb);
    for (int n = 0; n < count; ++n) {
      const int st = n % STAGES, ph = (n / STAGES) & 1;
      if (!mbar_wait_warp(empty(st), ph ^ 1, w, kBSiteLoadQ)) break;
      if (elected) {
        const uint32_t dst = ring_base + st * kStageBytes;
        const int other = first + n;  // the KV tile (form 2) or Q tile (forms 0, 1) of this product
        // pair (KV tile, Q tile) -> scratch tile: pairs of a head are numbered KV tile by KV tile
        const size_t tile = item.head_tile0 + (FORM == 2 ? dstile_count(ntiles, other) + (ot - other)
                                                         : dstile_count(ntiles, ot) + n);
        mbar_arrive_expect_tx(full(st), kStageBytes);
        bulk_load_1d(dst, scratch + tile * 2048, 32768, full(st));  // 32 KiB, stored as it is used
#pragma unroll
        for (int ch = 0; ch < T::kChunks; ++ch)
          tma_load_4d(dst + 32768 + ch * T::kChunkTileBytes, tb, ch * T::kChunkElems, other * 128,
                      item.hc, full(st));
      }
    }
    __syncwarp();
  } else if (is_mma_warp) {
    const uint32_t elected = elect_one();
    bool ok = true;
    for (int n = 0; ok && n < count; ++n) {
      const int st = n % STAGES, ph = (n / STAGES) & 1;
      if (!(ok = mbar_wait(full(st), ph, w, kBSiteMmaKV))) break;
      const uint32_t src = ring_base + st * kStageBytes;
      // out[128, D] += A * B; B = the operand tile (d contiguous, MN-major)
      if constexpr (FORM == 2)
        issue_piecesT_x_tile<D, BF16>(elected, tmem_acc, src, src + 32768, n > 0);
      else
        issue_pieces_x_tile<D, BF16>(elected, tmem_acc, src, src + 32768, n > 0);
      if (elected) mma_commit(empty(st));
    }
    if (ok && elected) mma_commit(done);
    __syncwarp();
  } else if (epi_warp >= 0) {
    float inv_dscale = 1.0f;
    if (item.tile_amax != nullptr) head_dscale<BF16>(item.tile_amax, ntiles, lane, &inv_dscale);
    if (mbar_wait_warp(done, 0, w, kBSiteCmpDone)) {
      tc_fence_after();
      const uint32_t lane_base = static_cast<uint32_t>(epi_warp * 32) << 16;
      // every product has completed, so the ring is idle: stage through its first buffer
      store_rows_16bit<D, BF16>(tmem_acc + lane_base, ring, epi_warp, lane, tout, ot * 128, item.hc,
                                out_rows, inv_dscale);
    }
  }
}

}  // namespace fa2
