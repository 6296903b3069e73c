// Single-tile tensor-core self-test: one kernel per operand form the attention kernels use.
// It exists so that a wrong descriptor encoding shows up as a wrong 128 x N tile that a test
// can compare with a plain matrix product, instead of as subtly wrong attention gradients.
//   form 0: C[128,128] = A[128,D] * B[128,D]^T   A, B staged by TMA, both K-major
//   form 1: C[128,D]   = P[128,128] * B[128,D]   P written to tensor memory by the threads
//                                                (16-bit pairs), B staged by TMA, MN-major
//   form 2: C[128,D]   = A[128,128]^T * B[128,D] A written to shared memory by the threads
//                                                with the 128-byte swizzle, MN-major; B as form 1
#include "common.cuh"
#include "ptx.cuh"

namespace fa2 {
namespace {

constexpr int kSelfThreads = 160;

template <int D>
struct SelfCfg {
  using T = Tile<D>;
  static constexpr int kOffA = 0;                      // form 0: A tile [128][D]; form 2: 2 x [128][64]
  static constexpr int kOffB = 32768;                  // B tile [128][D]
  static constexpr int kOffBar = kOffB + 32768;
  static constexpr int kSmemBytes = kOffBar + 64;
};

template <int D, bool BF16>
__global__ void __launch_bounds__(kSelfThreads, 1)
    selftest_kernel(int form, const __grid_constant__ CUtensorMap ta,
                    const __grid_constant__ CUtensorMap tb, const uint16_t* __restrict__ a_raw,
                    float* __restrict__ c, int* status) {
  using C = SelfCfg<D>;
  using T = Tile<D>;
  extern __shared__ __align__(1024) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = smem_u32(smem);
  if (smem_base & 1023u) {
    if (threadIdx.x == 0) atomicCAS(status, 0, 0x20000 | 99);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kOffBar);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t bar_load = smem_base + C::kOffBar, bar_mma = bar_load + 8;
  if (threadIdx.x == 0) {
    mbar_init(bar_load, 1);
    mbar_init(bar_mma, 1);
    *abort_flag = 0;
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == 4) {
    tmem_alloc(smem_u32(tmem_slot), 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const WaitCtx w{abort_flag, status};
  const int r = (warp & 3) * 32 + lane;
  const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
  constexpr int kColC = 0, kColP = 128;

  // Stage the thread-written operand.
  if (warp < 4) {
    if (form == 1) {
      const uint32_t* row = reinterpret_cast<const uint32_t*>(a_raw + r * 128);
      uint32_t pk[32];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
#pragma unroll
        for (int i = 0; i < 32; ++i) pk[i] = row[32 * h + i];
        tmem_st_x32(tmem_base + lane_base + kColP + 32 * h, pk);
      }
      tmem_wait_st();
    } else if (form == 2) {
      const uint4* row = reinterpret_cast<const uint4*>(a_raw + r * 128);
#pragma unroll
      for (int p = 0; p < 16; ++p)
        *reinterpret_cast<uint4*>(smem + C::kOffA + (p >> 3) * 16384 +
                                  swizzled_offset_128B(r, p & 7)) = row[p];
      fence_proxy_async_smem();
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  if (warp == 4 && lane == 0) {
    uint32_t bytes = T::kTileBytes;
    if (form == 0) bytes += T::kTileBytes;
    mbar_arrive_expect_tx(bar_load, bytes);
    for (int ch = 0; ch < T::kChunks; ++ch) {
      if (form == 0)
        tma_load_4d(smem_base + C::kOffA + ch * T::kChunkTileBytes, &ta, ch * T::kChunkElems, 0, HeadCoord{0, 0}, bar_load);
      tma_load_4d(smem_base + C::kOffB + ch * T::kChunkTileBytes, &tb, ch * T::kChunkElems, 0, HeadCoord{0, 0},
                  bar_load);
    }
    if (mbar_wait(bar_load, 0, w, 1)) {
      if (form == 0) {
        constexpr uint32_t idesc = make_idesc(128, 128, BF16, false, false);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off =
              (k / T::kKStepsPerChunk) * T::kChunkTileBytes + (k % T::kKStepsPerChunk) * 32;
          mma_ss(tmem_base + kColC,
                 make_smem_desc(smem_base + C::kOffA + off, 16, T::kAtomBytes, T::kSwizzleMode),
                 make_smem_desc(smem_base + C::kOffB + off, 16, T::kAtomBytes, T::kSwizzleMode),
                 idesc, k > 0);
        }
      } else if (form == 1) {
        constexpr uint32_t idesc = make_idesc(128, D, BF16, false, true);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          mma_ts(tmem_base + kColC, tmem_base + kColP + k * 8,
                 make_smem_desc(smem_base + C::kOffB + k * 2 * T::kAtomBytes, T::kChunkTileBytes,
                                T::kAtomBytes, T::kSwizzleMode),
                 idesc, k > 0);
      } else {
        constexpr uint32_t idesc = make_idesc(128, D, BF16, true, true);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          mma_ss(tmem_base + kColC,
                 make_smem_desc(smem_base + C::kOffA + k * 2048, 16384, 1024, kSwizzle128B),
                 make_smem_desc(smem_base + C::kOffB + k * 2 * T::kAtomBytes, T::kChunkTileBytes,
                                T::kAtomBytes, T::kSwizzleMode),
                 idesc, k > 0);
      }
      mma_commit(bar_mma);
    }
  }
  __syncwarp();
  if (warp < 4) {
    if (mbar_wait_warp(bar_mma, 0, w, 2)) {
      tc_fence_after();
      const int ncols = form == 0 ? 128 : D;
      for (int c0 = 0; c0 < ncols; c0 += 32) {
        uint32_t v[32];
        tmem_ld_x32(tmem_base + lane_base + kColC + c0, v);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) c[r * ncols + c0 + i] = __uint_as_float(v[i]);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

// Bounded-wait self-test: two warps wait on an mbarrier that nobody arrives at.  The first
// waiter to reach the time limit sets the CTA's abort flag and the device status word; the
// other one sees the flag and leaves; the kernel ends normally and the context stays usable.
constexpr int kSiteWaitProbe = 120;
__global__ void __launch_bounds__(64, 1) wait_probe_kernel(int* status) {
  __shared__ __align__(8) uint64_t bar_storage;
  __shared__ int abort_storage;
  const uint32_t bar = smem_u32(&bar_storage);
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    abort_storage = 0;
    fence_mbar_init();
  }
  __syncthreads();
  const WaitCtx w{&abort_storage, status};
  const bool ok = mbar_wait_warp(bar, 0, w, kSiteWaitProbe);  // never completes: returns false
  if (ok && threadIdx.x == 0) atomicCAS(status, 0, 0x30000 | kSiteWaitProbe);  // must not happen
  __syncthreads();
}

template <int D, bool BF16>
cudaError_t launch_t(int form, const CUtensorMap& ta, const CUtensorMap& tb, const void* a_raw,
                     float* c, int* status, cudaStream_t stream) {
  using C = SelfCfg<D>;
  auto kern = selftest_kernel<D, BF16>;
  cudaError_t e =
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
  if (e != cudaSuccess) return e;
  kern<<<1, kSelfThreads, C::kSmemBytes, stream>>>(form, ta, tb,
                                                   static_cast<const uint16_t*>(a_raw), c, status);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_selftest_mma(int form, const CUtensorMap& ta, const CUtensorMap& tb,
                                const void* a_raw, float* c, int D, int dtype, int* status,
                                cudaStream_t stream) {
#define FA2_CASE(DD)                                                                \
  case DD:                                                                          \
    return dtype ? launch_t<DD, true>(form, ta, tb, a_raw, c, status, stream)       \
                 : launch_t<DD, false>(form, ta, tb, a_raw, c, status, stream);
  switch (D) {
    FA2_CASE(32)
    FA2_CASE(64)
    FA2_CASE(128)
  }
#undef FA2_CASE
  return cudaErrorInvalidValue;
}

cudaError_t launch_selftest_wait(int* status, cudaStream_t stream) {
  wait_probe_kernel<<<1, 64, 0, stream>>>(status);
  return cudaGetLastError();
}

}  // namespace fa2
