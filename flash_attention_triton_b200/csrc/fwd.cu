// Causal attention forward for sm_100a.
//
// Replaces _forward_kernel (src/flash_attention_triton/_triton_kernels_v2.py:11-189 of the
// reference).  One CTA owns two adjacent 128-row Q tiles of one (batch, head) and walks the KV
// tiles 0..diagonal.  Warp roles:
//   warps 0-3  softmax for Q tile 0   (thread = one score row = one tensor-memory lane)
//   warps 4-7  softmax for Q tile 1
//   warp  8    MMA issue (one elected thread): S_i = Q_i K_j^T, O_i += P_i V_j
//   warp  9    TMA producer: Q once, then a K ring and a V ring
//   warps 10-11 idle; with warps 8-9 they give registers to the softmax groups (setmaxnreg)
// While one softmax group turns S_i into P_i the tensor cores run the other tile's MMAs.
// S, P and O live in tensor memory; P overwrites S in place as 16-bit pairs.  The online
// softmax works in the exp2 domain with the scale folded in, and rescales O only when the
// running maximum has moved by more than 2^8 ("lazy rescale"); masking code runs on the
// diagonal tile only.
#include "common.cuh"
#include "mma_issue.cuh"
#include "ptx.cuh"

namespace fa2 {
namespace {

constexpr int kFwdThreads = 384;  // warps 10, 11 idle: register donors for the softmax groups
constexpr float kRescaleThreshold = 8.0f;  // log2 units
constexpr float kLn2 = 0.6931471805599453f;

template <int D>
struct FwdCfg {
  using T = Tile<D>;
  static constexpr int kKStages = D == 128 ? 2 : (D == 64 ? 3 : 4);
  static constexpr int kVStages = kKStages;
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
  static constexpr int kBarSFull = kBarVEmpty + kVStages;  // 2
  static constexpr int kBarPFull = kBarSFull + 2;          // 2
  static constexpr int kBarOFull = kBarPFull + 2;          // 2
  static constexpr int kNumBars = kBarOFull + 2;
  static constexpr int kSmemBytes = kOffBar + kNumBars * 8 + 16;
  // tensor-memory columns
  static constexpr int kColS = 0;    // S0 at 0, S1 at 128 (P_i aliases the first 64 of S_i)
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
  kSiteSoftS,
  kSiteSoftO,
  kSiteAlign
};

template <int D, bool BF16>
__global__ void __launch_bounds__(kFwdThreads, 1)
    fwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
               const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap to,
               float* __restrict__ lse, int N, float scale_log2, int* status) {
  using C = FwdCfg<D>;
  using T = Tile<D>;
  extern __shared__ __align__(1024) uint8_t smem[];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = smem_u32(smem);
  if (smem_base & 1023u) {  // swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0) atomicCAS(status, 0, 0x20000 | kSiteAlign);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kOffBar);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + C::kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  auto bar = [&](int i) { return smem_base + C::kOffBar + 8u * i; };

  const int ntiles = (N + 127) >> 7;
  const int pair = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);  // heavy first
  const int bh = blockIdx.y;
  const int qt0 = 2 * pair, qt1 = 2 * pair + 1;
  const bool has1 = qt1 < ntiles;
  const int n0 = qt0 + 1;
  const int n1 = has1 ? qt1 + 1 : 0;
  const int nkv = has1 ? n1 : n0;

  if (threadIdx.x == 0) {
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
      mbar_init(bar(C::kBarPFull + i), 4);
      mbar_init(bar(C::kBarOFull + i), 1);
    }
    *abort_flag = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == 8) {
    tmem_alloc(smem_u32(tmem_slot), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const WaitCtx w{abort_flag, status};

  if (warp >= 8) {
    reg_dec<72>();  // whole warpgroup (warps 8-11) gives registers to the softmax groups
  if (warp == 9) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tensormap(&tq);
      prefetch_tensormap(&tk);
      prefetch_tensormap(&tv);
      mbar_arrive_expect_tx(bar(C::kBarQFull), (has1 ? 2 : 1) * T::kTileBytes);
      for (int i = 0; i < (has1 ? 2 : 1); ++i)
        for (int ch = 0; ch < T::kChunks; ++ch)
          tma_load_3d(smem_base + C::kOffQ + i * T::kTileBytes + ch * T::kChunkTileBytes, &tq,
                      ch * T::kChunkElems, (qt0 + i) * 128, bh, bar(C::kBarQFull));
      for (int j = 0; j < nkv; ++j) {
        const int ks = j % C::kKStages, kph = (j / C::kKStages) & 1;
        if (!mbar_wait(bar(C::kBarKEmpty + ks), kph ^ 1, w, kSiteLoadK)) break;
        mbar_arrive_expect_tx(bar(C::kBarKFull + ks), T::kTileBytes);
        for (int ch = 0; ch < T::kChunks; ++ch)
          tma_load_3d(smem_base + C::kOffK + ks * T::kTileBytes + ch * T::kChunkTileBytes, &tk,
                      ch * T::kChunkElems, j * 128, bh, bar(C::kBarKFull + ks));
        const int vs = j % C::kVStages, vph = (j / C::kVStages) & 1;
        if (!mbar_wait(bar(C::kBarVEmpty + vs), vph ^ 1, w, kSiteLoadV)) break;
        mbar_arrive_expect_tx(bar(C::kBarVFull + vs), T::kTileBytes);
        for (int ch = 0; ch < T::kChunks; ++ch)
          tma_load_3d(smem_base + C::kOffV + vs * T::kTileBytes + ch * T::kChunkTileBytes, &tv,
                      ch * T::kChunkElems, j * 128, bh, bar(C::kBarVFull + vs));
      }
    }
    __syncwarp();
  } else if (warp == 8) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // S_i = Q_i K^T (both K-major); O_i += P_i V with P_i from tensor memory (16-bit
      // pairs over the first 64 columns of S_i) and V as the MN-major B operand.
      auto issue_s = [&](int i, int kstage) {
        issue_rows_x_rows<D, BF16>(tmem_base + C::kColS + i * 128,
                                   smem_base + C::kOffQ + i * T::kTileBytes,
                                   smem_base + C::kOffK + kstage * T::kTileBytes);
      };
      auto issue_pv = [&](int i, int vstage, bool accumulate) {
        issue_tmem_x_tile<D, BF16>(tmem_base + C::kColO + i * D, tmem_base + C::kColS + i * 128, 32,
                                   smem_base + C::kOffV + vstage * T::kTileBytes, accumulate);
      };
      bool ok = mbar_wait(bar(C::kBarQFull), 0, w, kSiteMmaQ) &&
                mbar_wait(bar(C::kBarKFull + 0), 0, w, kSiteMmaK);
      if (ok) {
        issue_s(0, 0);
        mma_commit(bar(C::kBarSFull + 0));
        if (has1) {
          issue_s(1, 0);
          mma_commit(bar(C::kBarSFull + 1));
        }
        mma_commit(bar(C::kBarKEmpty + 0));
      }
      for (int j = 0; ok && j < nkv; ++j) {
        const int vs = j % C::kVStages, vph = (j / C::kVStages) & 1;
        const int ks1 = (j + 1) % C::kKStages, kph1 = ((j + 1) / C::kKStages) & 1;
        if (!(ok = mbar_wait(bar(C::kBarVFull + vs), vph, w, kSiteMmaV))) break;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int ni = i == 0 ? n0 : n1;
          if (j < ni) {
            if (!(ok = mbar_wait(bar(C::kBarPFull + i), j & 1, w, kSiteMmaP))) break;
            tc_fence_after();
            issue_pv(i, vs, j > 0);
            if (j + 1 < ni) {
              if (!(ok = mbar_wait(bar(C::kBarKFull + ks1), kph1, w, kSiteMmaK))) break;
              issue_s(i, ks1);
              mma_commit(bar(C::kBarSFull + i));
            } else {
              mma_commit(bar(C::kBarOFull + i));
            }
          }
        }
        if (!ok) break;
        mma_commit(bar(C::kBarVEmpty + vs));
        if (j + 1 < nkv) mma_commit(bar(C::kBarKEmpty + ks1));
      }
    }
    __syncwarp();
  }
  } else {
    // ------------------------------------------------------------------ softmax groups
    reg_inc<208>();
    const int wg = warp >> 2;
    const int qt = wg == 0 ? qt0 : qt1;
    const int nj = wg == 0 ? n0 : n1;
    const int r = (warp & 3) * 32 + lane;  // row inside the Q tile = tensor-memory lane
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem_base + lane_base + C::kColS + wg * 128;
    const uint32_t tO = tmem_base + lane_base + C::kColO + wg * D;
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
      float* s = reinterpret_cast<float*>(sr);
      if (j == qt) {  // diagonal tile: keep col <= row
#pragma unroll
        for (int c = 0; c < 128; ++c) s[c] = (c <= r) ? s[c] : -INFINITY;
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
      if (__any_sync(0xffffffffu, need)) {
        const float alpha = ex2((m_run - m_new) * scale_log2);
        l_run *= alpha;
        m_run = m_new;
        if (j > 0) {
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
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t pk[32];
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          float2 t = __ffma2_rn(make_float2(s[64 * h + 2 * c], s[64 * h + 2 * c + 1]), sc2, nm2);
          t.x = ex2(t.x);
          t.y = ex2(t.y);
          acc[c & 3] = __fadd2_rn(acc[c & 3], t);
          pk[c] = pack2<BF16>(t.x, t.y);
        }
        tmem_st_x32(tS + 32 * h, pk);
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(C::kBarPFull + wg));
      const float2 a01 = __fadd2_rn(acc[0], acc[1]), a23 = __fadd2_rn(acc[2], acc[3]);
      l_run += (a01.x + a01.y) + (a23.x + a23.y);
    }
    if (ok && nj > 0 && mbar_wait_warp(bar(C::kBarOFull + wg), 0, w, kSiteSoftO)) {
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
                                    swizzled_offset<D>(r, piece0 + p)) = val;
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        const int row0 = (warp & 3) * 32;
        if (qt * 128 + row0 < N) {
          for (int ch = 0; ch < T::kChunks; ++ch)
            tma_store_3d(&to, ch * T::kChunkElems, qt * 128 + row0, bh,
                         smem_u32(sO + ch * T::kChunkTileBytes + row0 * T::kRowBytes));
          tma_store_commit();
          tma_store_wait_all();
        }
      }
      const int row = qt * 128 + r;
      if (row < N)
        lse[static_cast<size_t>(bh) * N + row] = (m_run * scale_log2 + lg2(l_run)) * kLn2;
    }
  }

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
                         const CUtensorMap& tv, const CUtensorMap& to, float* lse, int* status,
                         cudaStream_t stream) {
  using C = FwdCfg<D>;
  auto kern = fwd_kernel<D, BF16>;
  cudaError_t e =
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
  if (e != cudaSuccess) return e;
  const int ntiles = (s.N + 127) / 128;
  const int npairs = (ntiles + 1) / 2;
  dim3 grid(npairs, s.B * s.H);
  const float scale_log2 = s.scale * 1.4426950408889634f;
  kern<<<grid, kFwdThreads, C::kSmemBytes, stream>>>(tq, tk, tv, to, lse, s.N, scale_log2, status);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_fwd(const AttnShape& s, const CUtensorMap& tq, const CUtensorMap& tk,
                       const CUtensorMap& tv, const CUtensorMap& to, float* lse, int* status,
                       cudaStream_t stream) {
#define FA2_CASE(DD)                                                                    \
  case DD:                                                                              \
    return s.dtype ? launch_fwd_t<DD, true>(s, tq, tk, tv, to, lse, status, stream)     \
                   : launch_fwd_t<DD, false>(s, tq, tk, tv, to, lse, status, stream);
  switch (s.D) {
    FA2_CASE(32)
    FA2_CASE(64)
    FA2_CASE(128)
  }
#undef FA2_CASE
  return cudaErrorInvalidValue;
}

}  // namespace fa2
