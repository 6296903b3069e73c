// Causal attention forward for sm_100a.
//
// Replaces _forward_kernel (src/flash_attention_triton/_triton_kernels_v2.py:11-189 of the
// reference).  One CTA owns two adjacent 128-row Q tiles of one (batch, head) and walks the KV
// tiles 0..diagonal.  Warp roles:
//   warps 0-3   softmax for Q tile 0   (thread = one score row = one tensor-memory lane)
//   warps 4-7   softmax for Q tile 1
//   warp  8     issues S = Q_i K_j^T          } one elected lane each; two warps so that neither
//   warp  10    issues O_i += P_i V_j         } MMA stream waits behind the other's barriers
//   warp  9     TMA producer: Q once, then a K ring and a V ring
//   warp  11    idle; warps 8-11 give registers to the softmax groups (setmaxnreg)
// (role numbers; hardware warps 0-3 take roles 8-11, see below)
//
// Tensor memory: ONE score buffer S shared by both Q tiles, a 16-bit probability buffer P_i per
// tile and an output accumulator O_i per tile.  A softmax group copies its score row into
// registers as soon as S is complete and hands the buffer back at once, so the next S product
// (for the other tile) runs while the group is still exponentiating; because P_i has its own
// columns, S_i(j+1) does not wait for O_i += P_i(j) V_j either.  Neither softmax group ever
// waits for its own MMAs in steady state: the tensor pipe sees four tile products per KV step
// back to back.
//
// The online softmax works in the exp2 domain with the scale folded in, and rescales O only
// when the running maximum has moved by more than 2^8 ("lazy rescale"); masking code runs on
// the diagonal tile only.  A fixed fraction of the exponentials is evaluated with a
// polynomial on the FMA pipe because the MUFU rate (16 / clk / SM) would otherwise bound the
// kernel: 2 x 128 x 128 exponentials per KV step cost as many cycles as the four MMAs.
#include "common.cuh"
#include "mma_issue.cuh"
#include "ptx.cuh"

#ifndef FA2_FWD_POLY_PAIRS_PER_8
#define FA2_FWD_POLY_PAIRS_PER_8 3  // of every 8 column pairs, this many use ex2_poly2
#endif

namespace fa2 {
namespace {

constexpr int kFwdThreads = 384;
constexpr float kRescaleThreshold = 8.0f;  // log2 units
constexpr float kLn2 = 0.6931471805599453f;

template <int D>
struct FwdCfg {
  using T = Tile<D>;
  static constexpr int kKStages = D == 128 ? 3 : 4;
  static constexpr int kVStages = D == 128 ? 2 : 4;
  static constexpr int kOffQ = 0;
  static constexpr int kOffK = kOffQ + 2 * T::kTileBytes;
  static constexpr int kOffV = kOffK + kKStages * T::kTileBytes;
  static constexpr int kOffBar = kOffV + kVStages * T::kTileBytes;
  // barrier slots
  static constexpr int kBarQFull = 0;
  static constexpr int kBarKFull = 1;
  static constexpr int kBarKEmpty = kBarKFull + kKStages;
  static constexpr int kBarVFull = kBarKEmpty + kKStages;
  static constexpr int kBarVEmpty = kBarVFull + kVStages;
  static constexpr int kBarSFull = kBarVEmpty + kVStages;  // 2: S holds tile i's scores
  static constexpr int kBarSFree = kBarSFull + 2;    // 2: group i has copied S out (4 arrivals)
  static constexpr int kBarPFull = kBarSFree + 2;    // 2: P_i written, O_i rescaled (4 arrivals)
  static constexpr int kBarPvDone = kBarPFull + 2;   // 2: O_i += P_i V completed
  static constexpr int kNumBars = kBarPvDone + 2;
  static constexpr int kSmemBytes = kOffBar + kNumBars * 8 + 16;  // + tmem slot, abort, work slot
  // tensor-memory columns
  static constexpr int kColS = 0;
  static constexpr int kColP = 128;  // P0 at 128, P1 at 192 (64 columns of 16-bit pairs each)
  static constexpr int kColO = 256;  // O0 at 256, O1 at 256 + D
  static constexpr int kTmemCols = 512;
};

enum FwdSite {
  kSiteLoadK = 1,
  kSiteLoadV,
  kSiteMmaQ,
  kSiteMmaK,
  kSiteMmaV,
  kSiteMmaP,
  kSiteMmaSFree,
  kSiteSoftS,
  kSiteSoftPv,
  kSiteSoftO,
  kSiteAlign
};

template <int D, bool BF16>
__global__ void __launch_bounds__(kFwdThreads, 1)
    fwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
               const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap to,
               float* __restrict__ lse, int N, int Nk, int num_bh, int num_heads, int group,
               float scale_log2, int* status, unsigned int* work_counter) {
  // Head dim 256 ("wide") runs on the staging and tensor-memory plan of head dim 128 with ONE
  // Q tile per work item: the two Q slots hold the two 128-column halves of that tile, K and V
  // tiles stream through their rings as half tiles, S = Q_lo K_lo^T + Q_hi K_hi^T accumulates
  // over two products and O_lo / O_hi take the places of O0 / O1.  Only softmax group 0 works.
  constexpr bool WIDE = D == 256;
  constexpr int DT = WIDE ? 128 : D;    // columns of one staged tile
  constexpr int HALVES = WIDE ? 2 : 1;  // staged tiles per 128 rows
  using C = FwdCfg<DT>;
  using T = Tile<DT>;
  extern __shared__ __align__(1024) uint8_t smem[];

  // Role index: hardware warps 0-3 take roles 8-11 (MMA, TMA, idle, idle) and hardware warps
  // 4-11 the softmax roles 0-7, so the latency-critical MMA / TMA warps have the lowest
  // hardware warp ids on their schedulers.  The shift is a multiple of 4, so role % 4 is
  // still the tensor-memory lane quarter the hardware warp may access.
  const int warp = ((threadIdx.x >> 5) + 8) % 12;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = smem_u32(smem);
  if (smem_base & 1023u) {  // swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0) atomicCAS(status, 0, 0x20000 | kSiteAlign);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kOffBar);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + C::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* work_slot = reinterpret_cast<volatile int*>(tmem_slot + 2);
  auto bar = [&](int i) { return smem_base + C::kOffBar + 8u * i; };

  const int ntiles = (N + 127) >> 7;
  const int nktiles = (Nk + 127) >> 7;
  const int npairs = WIDE ? ntiles : (ntiles + 1) >> 1;  // work items per (batch, head)
  const int total_items = npairs * num_bh;

  if (threadIdx.x == 0) *abort_flag = 0;
  if (warp == 8) {
    tmem_alloc(smem_u32(tmem_slot), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const WaitCtx w{abort_flag, status};

  // One CTA per SM; work items (one Q-tile pair of one (batch, head)) are fetched from a
  // global counter in head-major, heavy-pair-first order, like a hardware block scheduler
  // would hand them out, but without the launch gap and with tensor memory kept allocated.
  // Between items all roles meet at a barrier and the mbarriers are re-initialised, so each
  // item starts from phase 0.
  for (bool first = true;; first = false) {
    __syncthreads();  // every role has finished the previous item
    if (threadIdx.x == 0) {
      const int next = fetch_work_item(work_counter, total_items, first);
      *work_slot = next;
      if (next < total_items && !*abort_flag) {
        if (!first)
          for (int i = 0; i < C::kNumBars; ++i) mbar_inval(bar(i));
        mbar_init(bar(C::kBarQFull), 1);
        for (int i = 0; i < C::kKStages; ++i) {
          mbar_init(bar(C::kBarKFull + i), 1);
          mbar_init(bar(C::kBarKEmpty + i), 1);
        }
        for (int i = 0; i < C::kVStages; ++i) {
          mbar_init(bar(C::kBarVFull + i), 1);
          mbar_init(bar(C::kBarVEmpty + i), 1);
        }
        for (int i = 0; i < 2; ++i) {
          mbar_init(bar(C::kBarSFull + i), 1);
          mbar_init(bar(C::kBarSFree + i), 4);
          mbar_init(bar(C::kBarPFull + i), 4);
          mbar_init(bar(C::kBarPvDone + i), 1);
        }
        fence_mbar_init();
        fence_proxy_async_smem();
      }
    }
    __syncthreads();
    const int item = *work_slot;
    if (item >= total_items) break;
    if (*abort_flag) continue;  // keep drawing so that the counter is left at zero
    const HeadTile ht = grouped_order(item, num_bh, npairs, group);
    const int bh = ht.bh;
    const HeadCoord hc{bh % num_heads, bh / num_heads};
    const int pair = npairs - 1 - ht.rank;  // the last pair of Q tiles meets the most KV tiles
    const int qt0 = WIDE ? pair : 2 * pair, qt1 = qt0 + 1;
    const bool has1 = !WIDE && qt1 < ntiles;
    // KV tiles of Q tile i: 0 .. min(i, last KV tile)  (N = query rows, Nk <= N = key rows)
    const int n0 = qt0 + 1 < nktiles ? qt0 + 1 : nktiles;
    const int n1 = has1 ? (qt1 + 1 < nktiles ? qt1 + 1 : nktiles) : 0;
    const int nkv = n1 > n0 ? n1 : n0;

  if (warp >= 8) {
    reg_dec<72>();  // whole warpgroup (warps 8-11) gives registers to the softmax groups
    if (warp == 9) {
      // ---------------------------------------------------------------- TMA producer
      // (whole warp, converged; only the elected lane arms barriers and issues copies)
      const uint32_t elected = elect_one();
      if (elected) {
        prefetch_tensormap(&tq);
        prefetch_tensormap(&tk);
        prefetch_tensormap(&tv);
        const int nslots = (WIDE || has1) ? 2 : 1;
        mbar_arrive_expect_tx(bar(C::kBarQFull), nslots * T::kTileBytes);
        for (int i = 0; i < nslots; ++i)
          for (int ch = 0; ch < T::kChunks; ++ch)
            tma_load_4d(smem_base + C::kOffQ + i * T::kTileBytes + ch * T::kChunkTileBytes, &tq,
                        (WIDE ? i * 128 : 0) + ch * T::kChunkElems, (WIDE ? qt0 : qt0 + i) * 128, hc,
                        bar(C::kBarQFull));
      }
      // K runs one KV tile ahead of V: S(j+1) is issued during KV step j.  Ring entries are
      // staged tiles: entry t holds columns (t % HALVES) * 128 .. of KV tile t / HALVES.
      const int nsub = nkv * HALVES;
      for (int t = 0; t < nsub + HALVES; ++t) {
        if (t < nsub) {
          const int ks = t % C::kKStages, kph = (t / C::kKStages) & 1;
          if (!mbar_wait_warp(bar(C::kBarKEmpty + ks), kph ^ 1, w, kSiteLoadK)) break;
          if (elected) {
            mbar_arrive_expect_tx(bar(C::kBarKFull + ks), T::kTileBytes);
#pragma unroll
            for (int ch = 0; ch < T::kChunks; ++ch)
              tma_load_4d(smem_base + C::kOffK + ks * T::kTileBytes + ch * T::kChunkTileBytes, &tk,
                          (t % HALVES) * 128 + ch * T::kChunkElems, (t / HALVES) * 128, hc,
                          bar(C::kBarKFull + ks));
          }
        }
        if (t >= HALVES) {
          const int tv_ = t - HALVES;
          const int vs = tv_ % C::kVStages, vph = (tv_ / C::kVStages) & 1;
          if (!mbar_wait_warp(bar(C::kBarVEmpty + vs), vph ^ 1, w, kSiteLoadV)) break;
          if (elected) {
            mbar_arrive_expect_tx(bar(C::kBarVFull + vs), T::kTileBytes);
#pragma unroll
            for (int ch = 0; ch < T::kChunks; ++ch)
              tma_load_4d(smem_base + C::kOffV + vs * T::kTileBytes + ch * T::kChunkTileBytes, &tv,
                          (tv_ % HALVES) * 128 + ch * T::kChunkElems, (tv_ / HALVES) * 128, hc,
                          bar(C::kBarVFull + vs));
          }
        }
      }
    } else if (warp == 8) {
      // ---------------------------------------------------------------- S = Q_i K_j^T issuer
      // Whole warp, converged; only the elected lane issues MMAs and commits.  The score
      // products and the P V products are issued by two different warps (this one and warp
      // 10): they touch disjoint tensor-memory columns and are ordered against each other
      // only through the softmax groups, so neither stream waits behind the other's barriers.
      // Order: S0(0) S1(0) S0(1) S1(1) ...; each product waits until the previous one has
      // been copied out of the single score buffer.
      const uint32_t elected = elect_one();
      bool ok = mbar_wait(bar(C::kBarQFull), 0, w, kSiteMmaQ);
      int ks = 0, kph = 0;          // K ring position of tile j
      int prev_i = -1, prev_ph = 0;  // group and phase of the previous score product
      auto next_k = [&]() {
        if (++ks == C::kKStages) {
          ks = 0;
          kph ^= 1;
        }
      };
      for (int j = 0; ok && j < nkv; ++j) {
        if constexpr (!WIDE) {
          if (!(ok = mbar_wait(bar(C::kBarKFull + ks), kph, w, kSiteMmaK))) break;
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          if (j >= (i == 0 ? n0 : n1)) continue;
          if (prev_i >= 0) {
            if (!(ok = mbar_wait(bar(C::kBarSFree + prev_i), prev_ph, w, kSiteMmaSFree))) break;
            tc_fence_after();
          }
          if constexpr (WIDE) {
            // S = Q_lo K_lo^T + Q_hi K_hi^T: the Q slots hold the halves, K arrives half by half
            for (int half = 0; ok && half < 2; ++half) {
              if (!(ok = mbar_wait(bar(C::kBarKFull + ks), kph, w, kSiteMmaK))) break;
              issue_rows_x_rows<DT, BF16>(elected, tmem_base + C::kColS,
                                          smem_base + C::kOffQ + half * T::kTileBytes,
                                          smem_base + C::kOffK + ks * T::kTileBytes, half);
              if (elected) mma_commit(bar(C::kBarKEmpty + ks));
              next_k();
            }
            if (!ok) break;
          } else {
            issue_rows_x_rows<DT, BF16>(elected, tmem_base + C::kColS,
                                        smem_base + C::kOffQ + i * T::kTileBytes,
                                        smem_base + C::kOffK + ks * T::kTileBytes);
          }
          if (elected) mma_commit(bar(C::kBarSFull + i));
          prev_i = i;
          prev_ph = j & 1;
        }
        if (!ok) break;
        if constexpr (!WIDE) {
          if (elected) mma_commit(bar(C::kBarKEmpty + ks));  // both products that read K_j issued
          next_k();
        }
      }
    } else if (warp == 10) {
      // ---------------------------------------------------------------- O_i += P_i V_j issuer
      const uint32_t elected = elect_one();
      bool ok = true;
      int vs = 0, vph = 0;  // V ring position of tile j
      auto next_v = [&]() {
        if (++vs == C::kVStages) {
          vs = 0;
          vph ^= 1;
        }
      };
      for (int j = 0; ok && j < nkv; ++j) {
        if constexpr (!WIDE) {
          if (!(ok = mbar_wait(bar(C::kBarVFull + vs), vph, w, kSiteMmaV))) break;
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          if (j >= (i == 0 ? n0 : n1)) continue;
          if (!(ok = mbar_wait(bar(C::kBarPFull + i), j & 1, w, kSiteMmaP))) break;
          tc_fence_after();
          if constexpr (WIDE) {
            // O_lo += P V_lo, O_hi += P V_hi: the O0 / O1 columns hold the two halves of O
            for (int half = 0; ok && half < 2; ++half) {
              if (!(ok = mbar_wait(bar(C::kBarVFull + vs), vph, w, kSiteMmaV))) break;
              issue_tmem_x_tile<DT, BF16>(elected, tmem_base + C::kColO + half * DT,
                                          tmem_base + C::kColP, 32,
                                          smem_base + C::kOffV + vs * T::kTileBytes, j > 0);
              if (elected) mma_commit(bar(C::kBarVEmpty + vs));
              next_v();
            }
            if (!ok) break;
          } else {
            issue_tmem_x_tile<DT, BF16>(elected, tmem_base + C::kColO + i * DT,
                                        tmem_base + C::kColP + i * 64, 32,
                                        smem_base + C::kOffV + vs * T::kTileBytes, j > 0);
          }
          if (elected) mma_commit(bar(C::kBarPvDone + i));
        }
        if (!ok) break;
        if constexpr (!WIDE) {
          if (elected) mma_commit(bar(C::kBarVEmpty + vs));
          next_v();
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ softmax groups
    reg_inc<208>();
    const int wg = warp >> 2;
    const int qt = wg == 0 ? qt0 : qt1;
    const int nj = wg == 0 ? n0 : n1;
    const int r = (warp & 3) * 32 + lane;  // row inside the Q tile = tensor-memory lane
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem_base + lane_base + C::kColS;
    const uint32_t tP = tmem_base + lane_base + C::kColP + wg * 64;
    const uint32_t tO = tmem_base + lane_base + C::kColO + wg * DT;  // wide: 256 columns, wg 0 only
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < nj; ++j) {
      if (!(ok = mbar_wait_warp(bar(C::kBarSFull + wg), j & 1, w, kSiteSoftS))) break;
      tc_fence_after();
      uint32_t sr[128];
      tmem_ld_x32(tS + 0, sr + 0);
      tmem_ld_x32(tS + 32, sr + 32);
      tmem_ld_x32(tS + 64, sr + 64);
      tmem_ld_x32(tS + 96, sr + 96);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(C::kBarSFree + wg));  // S may be overwritten now
      float* s = reinterpret_cast<float*>(sr);
      if (j == qt || j * 128 + 128 > Nk) {
        // diagonal tile: keep col <= row; last KV tile: drop the columns beyond the last key
        int last = j == qt ? r : 127;
        last = last < Nk - 1 - j * 128 ? last : Nk - 1 - j * 128;
#pragma unroll
        for (int c = 0; c < 128; ++c) s[c] = (c <= last) ? s[c] : -INFINITY;
      }
      float mx[4];
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        mx[q4] = max3(s[32 * q4], s[32 * q4 + 1], s[32 * q4 + 2]);
#pragma unroll
        for (int c = 3; c < 31; c += 2) mx[q4] = max3(mx[q4], s[32 * q4 + c], s[32 * q4 + c + 1]);
        mx[q4] = fmaxf(mx[q4], s[32 * q4 + 31]);
      }
      const float m_new = fmaxf(max3(m_run, mx[0], mx[1]), fmaxf(mx[2], mx[3]));
      const bool need = (m_new - m_run) * scale_log2 > kRescaleThreshold;
      bool pv_waited = false;
      if (__any_sync(0xffffffffu, need)) {
        const float alpha = ex2((m_run - m_new) * scale_log2);
        l_run *= alpha;
        m_run = m_new;
        if (j > 0) {
          // O_i must be at rest: wait for O_i += P_i(j-1) V_(j-1)
          if (!(ok = mbar_wait_warp(bar(C::kBarPvDone + wg), (j - 1) & 1, w, kSiteSoftPv))) break;
          tc_fence_after();
          pv_waited = true;
#pragma unroll
          for (int c0 = 0; c0 < D; c0 += 32) {
            uint32_t orr[32];
            tmem_ld_x32(tO + c0, orr);
            tmem_wait_ld();
#pragma unroll
            for (int c = 0; c < 32; ++c) orr[c] = __float_as_uint(__uint_as_float(orr[c]) * alpha);
            tmem_st_x32(tO + c0, orr);
          }
        }
      }
      // p = 2^(s*c - m*c) with packed fp32x2 FMAs; row sum in four independent packed chains.
      const float2 sc2 = make_float2(scale_log2, scale_log2);
      const float2 nm2 = make_float2(-m_run * scale_log2, -m_run * scale_log2);
      float2 acc[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
      uint32_t pk[64];
#pragma unroll
      for (int c = 0; c < 64; ++c) {
        float2 t = __ffma2_rn(make_float2(s[2 * c], s[2 * c + 1]), sc2, nm2);
        if ((c & 7) < FA2_FWD_POLY_PAIRS_PER_8) {
          t = ex2_poly2(t);
        } else {
          t.x = ex2(t.x);
          t.y = ex2(t.y);
        }
        acc[c & 3] = __fadd2_rn(acc[c & 3], t);
        pk[c] = pack2<kInterBF16<BF16>>(t.x, t.y);
      }
      if (j > 0 && !pv_waited) {
        // P_i still feeds O_i += P_i(j-1) V_(j-1) until that product has completed
        if (!(ok = mbar_wait_warp(bar(C::kBarPvDone + wg), (j - 1) & 1, w, kSiteSoftPv))) break;
      }
      tmem_st_x32(tP, pk);
      tmem_st_x32(tP + 32, pk + 32);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(C::kBarPFull + wg));
      const float2 a01 = __fadd2_rn(acc[0], acc[1]), a23 = __fadd2_rn(acc[2], acc[3]);
      l_run += (a01.x + a01.y) + (a23.x + a23.y);
    }
    if (ok && nj > 0 && mbar_wait_warp(bar(C::kBarPvDone + wg), (nj - 1) & 1, w, kSiteSoftO)) {
      tc_fence_after();
      const float inv_l = 1.0f / l_run;
      // Stage the tile through the (now idle) Q buffer in the swizzled layout the output
      // tensor map expects; each warp stores its own 32 rows.
      uint8_t* sO = smem + C::kOffQ + wg * T::kTileBytes;
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t orr[32];
        tmem_ld_x32(tO + c0, orr);
        tmem_wait_ld();
        const int chunk = c0 / T::kChunkElems;
        const int piece0 = (c0 % T::kChunkElems) / 8;
#pragma unroll
        for (int p = 0; p < 4; ++p) {
          uint4 val;
          val.x = pack2<BF16>(__uint_as_float(orr[8 * p + 0]) * inv_l,
                              __uint_as_float(orr[8 * p + 1]) * inv_l);
          val.y = pack2<BF16>(__uint_as_float(orr[8 * p + 2]) * inv_l,
                              __uint_as_float(orr[8 * p + 3]) * inv_l);
          val.z = pack2<BF16>(__uint_as_float(orr[8 * p + 4]) * inv_l,
                              __uint_as_float(orr[8 * p + 5]) * inv_l);
          val.w = pack2<BF16>(__uint_as_float(orr[8 * p + 6]) * inv_l,
                              __uint_as_float(orr[8 * p + 7]) * inv_l);
          *reinterpret_cast<uint4*>(sO + chunk * T::kChunkTileBytes +
                                    swizzled_offset<DT>(r, piece0 + p)) = val;
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        const int row0 = (warp & 3) * 32;
        if (qt * 128 + row0 < N) {
          for (int ch = 0; ch < D / T::kChunkElems; ++ch)
            tma_store_4d(&to, ch * T::kChunkElems, qt * 128 + row0, hc,
                         smem_u32(sO + ch * T::kChunkTileBytes + row0 * T::kRowBytes));
          tma_store_commit();
          // the staging buffer may be refilled once the store has READ it; the write itself
          // completes on its own before the grid does
          tma_store_wait_read();
        }
      }
      const int row = qt * 128 + r;
      if (row < N)
        lse[static_cast<size_t>(bh) * N + row] = (m_run * scale_log2 + lg2(l_run)) * kLn2;
    }
  }

  }  // work-item loop

  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

template <int D, bool BF16>
cudaError_t launch_fwd_t(const AttnShape& s, const CUtensorMap& tq, const CUtensorMap& tk,
                         const CUtensorMap& tv, const CUtensorMap& to, float* lse,
                         const LaunchCtx& ctx, cudaStream_t stream) {
  using C = FwdCfg<D == 256 ? 128 : D>;  // head dim 256 runs on the plan of head dim 128
  auto kern = fwd_kernel<D, BF16>;
  cudaError_t e =
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
  if (e != cudaSuccess) return e;
  const int ntiles = (s.N + 127) / 128;
  const int npairs = D == 256 ? ntiles : (ntiles + 1) / 2;
  const long long items = static_cast<long long>(npairs) * s.B * s.H;
  const unsigned grid = static_cast<unsigned>(items < ctx.num_sms ? items : ctx.num_sms);
  const float scale_log2 = s.scale * 1.4426950408889634f;
  kern<<<grid, kFwdThreads, C::kSmemBytes, stream>>>(tq, tk, tv, to, lse, s.N, s.Nk, s.B * s.H, s.H,
                                                     heads_per_group(s), scale_log2, ctx.status,
                                                     ctx.work_counter);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_fwd(const AttnShape& s, const CUtensorMap& tq, const CUtensorMap& tk,
                       const CUtensorMap& tv, const CUtensorMap& to, float* lse,
                       const LaunchCtx& ctx, cudaStream_t stream) {
#define FA2_CASE(DD)                                                                 \
  case DD:                                                                           \
    return s.dtype ? launch_fwd_t<DD, true>(s, tq, tk, tv, to, lse, ctx, stream)     \
                   : launch_fwd_t<DD, false>(s, tq, tk, tv, to, lse, ctx, stream);
  switch (s.D) {
    FA2_CASE(32)
    FA2_CASE(64)
    FA2_CASE(128)
    FA2_CASE(256)
  }
#undef FA2_CASE
  return cudaErrorInvalidValue;
}

}  // namespace fa2
