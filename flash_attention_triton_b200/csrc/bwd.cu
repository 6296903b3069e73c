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
#include "bwd_roles.cuh"

namespace fa2 {
namespace {

// =========================================================================================
// dK / dV (+ fused dQ) kernel: one CTA per KV tile of one (batch, head); see dkdv_roles.
// =========================================================================================
template <int D, bool BF16, int MODE>
__global__ void __launch_bounds__(DkdvCfg<D, MODE>::kThreads, 1)
    bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                    const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo,
                    const __grid_constant__ CUtensorMap tdk,
                    const __grid_constant__ CUtensorMap tdv, const float* __restrict__ rowstats,
                    const unsigned* __restrict__ tile_amax, float* __restrict__ dq_accum, int N,
                    int Nk, int num_bh, int num_heads, int group, float scale, float scale_log2,
                    int* status) {
  using C = DkdvCfg<D, MODE>;
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

  const int ntiles = (N + 127) >> 7;
  const int nktiles = (Nk + 127) >> 7;
  DkdvItem item;
  const HeadTile ht = grouped_order(blockIdx.x, num_bh, nktiles, group);
  item.jt = ht.rank;  // KV tile; tile 0 has the most Q tiles
  item.bh = ht.bh;
  item.hc = HeadCoord{ht.bh % num_heads, ht.bh / num_heads};
  // Spill mode: tiles of a head are numbered KV tile by KV tile, Q tiles ascending inside.
  item.tile0 = static_cast<size_t>(item.bh) * dstile_count(ntiles, nktiles) + dstile_count(ntiles, item.jt);
  item.tile_amax = tile_amax + static_cast<size_t>(item.bh) * ntiles;

  if (threadIdx.x == 0) {
    dkdv_init_barriers<D, MODE>(smem_base + C::kOffBar);
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

  dkdv_roles<D, BF16, MODE>(smem, smem_base, tmem_base, warp, lane, &tq, &tk, &tv, &tdo, &tdk, &tdv,
                            rowstats, dq_accum, N, Nk, scale, scale_log2, w, item);

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
                  const __grid_constant__ CUtensorMap tdq, const float* __restrict__ rowstats,
                  const unsigned* __restrict__ tile_amax, int N, int Nk, int num_bh, int num_heads,
                  int group, float scale, float scale_log2, int* status) {
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
  const HeadTile ht = grouped_order(blockIdx.x, num_bh, ntiles, group);
  const int qt = ntiles - 1 - ht.rank;  // the last Q tile meets the most KV tiles
  const int bh = ht.bh;
  const HeadCoord hc{bh % num_heads, bh / num_heads};
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
    // dS is formed as dS * 2^k in fp16 and dQ multiplied by 2^-k at the end (head_dscale)
    float inv_dscale;
    const float dscale =
        head_dscale<BF16>(tile_amax + static_cast<size_t>(bh) * ntiles, ntiles, lane, &inv_dscale);
    const float2 scale2 = make_float2(scale * dscale, scale * dscale);
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
        dsk[c] = pack2<kInterBF16<BF16>>(u.x, u.y);
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
                                qt * 128, hc, N, inv_dscale);
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
// One output tile per CTA from spilled 16-bit tiles (head dim 256: dV, dK and dQ; see
// consume_roles).  warps 0-3 epilogue, warp 4 producer, warp 5 MMA issue.
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
  static constexpr int kNumBars = 2 * kStages + 1;
  static constexpr int kSmemBytes = kOffBar + kNumBars * 8 + 16;
  static constexpr int kTmemCols = D < 32 ? 32 : D;
  static_assert(kSmemBytes <= 232448, "shared memory budget of one CTA");
};

template <int D, bool BF16, int FORM>
__global__ void __launch_bounds__(ConsumeCfg<D>::kThreads, 1)
    bwd_consume_kernel(const uint4* __restrict__ scratch, const __grid_constant__ CUtensorMap tb,
                       const __grid_constant__ CUtensorMap tout,
                       const unsigned* __restrict__ tile_amax, int N, int Nk, int num_bh,
                       int num_heads, int group, int* status) {
  using C = ConsumeCfg<D>;
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

  const int ntiles = (N + 127) >> 7;     // Q tiles
  const int nktiles = (Nk + 127) >> 7;   // KV tiles
  ConsumeItem item;
  const HeadTile ht = grouped_order(blockIdx.x, num_bh, FORM == 2 ? ntiles : nktiles, group);
  const int bh = ht.bh;
  item.hc = HeadCoord{bh % num_heads, bh / num_heads};
  item.head_tile0 = static_cast<size_t>(bh) * dstile_count(ntiles, nktiles);
  // the last Q tile (form 2) and the first KV tile (forms 0, 1) are summed over the most tiles
  item.ot = FORM == 2 ? ntiles - 1 - ht.rank : ht.rank;
  // dS tiles carry the head's power-of-two factor (head_dscale); P tiles (form 0) do not
  item.tile_amax = FORM == 0 ? nullptr : tile_amax + static_cast<size_t>(bh) * ntiles;

  if (threadIdx.x == 0) {
    consume_init_barriers<C::kStages>(smem_base + C::kOffBar);
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

  consume_roles<D, BF16, FORM, C::kStages>(smem, smem_base, smem_base + C::kOffBar, tmem_base,
                                           warp == C::kLoadWarp, warp == C::kMmaWarp,
                                           warp < 4 ? warp : -1, lane, scratch, &tb, &tout, N, Nk, w,
                                           item);

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
                           const unsigned* __restrict__ tile_amax, uint4* __restrict__ p_scratch,
                           uint4* __restrict__ ds_scratch, int N, int Nk, int num_bh,
                           int num_heads, int group, float scale, float scale_log2, int* status) {
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
  const HeadTile ht = grouped_order(blockIdx.x, num_bh, nktiles, group);
  const int jt = ht.rank;  // KV tile
  const int bh = ht.bh;
  const HeadCoord hc{bh % num_heads, bh / num_heads};
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
    float inv_dscale;
    const float dscale =
        head_dscale<BF16>(tile_amax + static_cast<size_t>(bh) * ntiles, ntiles, lane, &inv_dscale);
    const float2 scale2 = make_float2(scale * dscale, scale * dscale);  // dS * 2^k, see head_dscale
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
          dst[pc * 128] = make_uint4(pack2<kInterBF16<BF16>>(p[4 * pc].x, p[4 * pc].y),
                                     pack2<kInterBF16<BF16>>(p[4 * pc + 1].x, p[4 * pc + 1].y),
                                     pack2<kInterBF16<BF16>>(p[4 * pc + 2].x, p[4 * pc + 2].y),
                                     pack2<kInterBF16<BF16>>(p[4 * pc + 3].x, p[4 * pc + 3].y));
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
        dsk[2 * c4] = pack2<kInterBF16<BF16>>(u0.x, u0.y);
        dsk[2 * c4 + 1] = pack2<kInterBF16<BF16>>(u1.x, u1.y);
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
                                 const CUtensorMap& tv, const CUtensorMap& tdo, const RowStats& rowstats,
                                 void* p_scratch, void* ds_scratch, int* status,
                                 cudaStream_t stream) {
  using C = ScoresCfg;
  auto kern = bwd_scores_wide_kernel<BF16>;
  cudaError_t e =
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
  if (e != cudaSuccess) return e;
  const unsigned grid = static_cast<unsigned>((s.Nk + 127) / 128) * s.B * s.H;  // one CTA per KV tile
  kern<<<grid, C::kThreads, C::kSmemBytes, stream>>>(
      tq, tk, tv, tdo, rowstats.stats, rowstats.tile_amax, static_cast<uint4*>(p_scratch),
      static_cast<uint4*>(ds_scratch), s.N, s.Nk, s.B * s.H, s.H, heads_per_group(s), s.scale,
      s.scale * 1.4426950408889634f, status);
  return cudaGetLastError();
}

template <int D, bool BF16, int MODE>
cudaError_t launch_dkdv_t(const AttnShape& s, const CUtensorMap& tq, const CUtensorMap& tk,
                          const CUtensorMap& tv, const CUtensorMap& tdo, const CUtensorMap& tdk,
                          const CUtensorMap& tdv, const RowStats& rowstats, float* dq_accum,
                          int* status, cudaStream_t stream) {
  using C = DkdvCfg<D, MODE>;
  auto kern = bwd_dkdv_kernel<D, BF16, MODE>;
  cudaError_t e =
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
  if (e != cudaSuccess) return e;
  const unsigned grid = static_cast<unsigned>((s.Nk + 127) / 128) * s.B * s.H;  // one CTA per KV tile
  kern<<<grid, C::kThreads, C::kSmemBytes, stream>>>(
      tq, tk, tv, tdo, tdk, tdv, rowstats.stats, rowstats.tile_amax, dq_accum, s.N, s.Nk, s.B * s.H,
      s.H, heads_per_group(s), s.scale, s.scale * 1.4426950408889634f, status);
  return cudaGetLastError();
}

template <int D, bool BF16, int FORM>
cudaError_t launch_consume_t(const AttnShape& s, const void* scratch, const CUtensorMap& tb,
                             const CUtensorMap& tout, const RowStats& rowstats, int* status,
                             cudaStream_t stream) {
  using C = ConsumeCfg<D>;
  auto kern = bwd_consume_kernel<D, BF16, FORM>;
  cudaError_t e =
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
  if (e != cudaSuccess) return e;
  const unsigned grid =
      static_cast<unsigned>(((FORM == 2 ? s.N : s.Nk) + 127) / 128) * s.B * s.H;  // one CTA per output tile
  kern<<<grid, C::kThreads, C::kSmemBytes, stream>>>(static_cast<const uint4*>(scratch), tb, tout,
                                                     rowstats.tile_amax, s.N, s.Nk, s.B * s.H, s.H,
                                                     heads_per_group(s), status);
  return cudaGetLastError();
}

template <int D, bool BF16>
cudaError_t launch_dq_t(const AttnShape& s, const CUtensorMap& tq, const CUtensorMap& tk,
                        const CUtensorMap& tv, const CUtensorMap& tdo, const CUtensorMap& tdq,
                        const RowStats& rowstats, int* status, cudaStream_t stream) {
  using C = DqCfg<D>;
  auto kern = bwd_dq_kernel<D, BF16>;
  cudaError_t e =
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
  if (e != cudaSuccess) return e;
  const unsigned grid = static_cast<unsigned>((s.N + 127) / 128) * s.B * s.H;  // one CTA per Q tile
  kern<<<grid, C::kThreads, C::kSmemBytes, stream>>>(
      tq, tk, tv, tdo, tdq, rowstats.stats, rowstats.tile_amax, s.N, s.Nk, s.B * s.H, s.H,
      heads_per_group(s), s.scale, s.scale * 1.4426950408889634f, status);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_bwd_dkdv(const AttnShape& s, const CUtensorMap& tq, const CUtensorMap& tk,
                            const CUtensorMap& tv, const CUtensorMap& tdo,
                            const CUtensorMap& tdk, const CUtensorMap& tdv,
                            const RowStats& rowstats, float* dq_accum, int mode, int* status,
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
                          const RowStats& rowstats, int* status, cudaStream_t stream) {
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
                                   const RowStats& rowstats, void* p_scratch, void* ds_scratch,
                                   int* status, cudaStream_t stream) {
  return s.dtype ? launch_scores_wide_t<true>(s, tq, tk, tv, tdo, rowstats, p_scratch, ds_scratch,
                                              status, stream)
                 : launch_scores_wide_t<false>(s, tq, tk, tv, tdo, rowstats, p_scratch, ds_scratch,
                                               status, stream);
}

cudaError_t launch_bwd_consume(const AttnShape& s, int form, const void* scratch,
                               const CUtensorMap& tb, const CUtensorMap& tout, const RowStats& rowstats,
                               int* status, cudaStream_t stream) {
#define FA2_ARGS s, scratch, tb, tout, rowstats, status, stream
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
