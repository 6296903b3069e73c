// Bandwidth-bound helpers of the backward pass.
//
//   bwd_preprocess_kernel  delta[row] = sum_d float(o[row,d]) * float(dout[row,d])
//       replaces _backward_preprocess_do_o_dot (_triton_kernels_v2.py:532-608 of the
//       reference).  Algorithmic traffic per row: 2 * D * 2 bytes read + 4 bytes (lse) read +
//       8 bytes written.
//   dq_convert_kernel      dq = 16-bit(dq_accum), the single fp32 -> 16-bit rounding the
//       reference performs with dq.copy_(dq_accum) (flash_attention_2.py:277).
#include "common.cuh"
#include "ptx.cuh"

namespace fa2 {
namespace {

template <bool BF16>
__device__ __forceinline__ float dot8(const uint4& a, const uint4& b) {
  const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
  const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 fa, fb;
    if constexpr (BF16) {
      fa = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&aw[i]));
      fb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&bw[i]));
    } else {
      fa = __half22float2(*reinterpret_cast<const __half2*>(&aw[i]));
      fb = __half22float2(*reinterpret_cast<const __half2*>(&bw[i]));
    }
    acc = fmaf(fa.x, fb.x, acc);
    acc = fmaf(fa.y, fb.y, acc);
  }
  return acc;
}

__device__ __forceinline__ uint4 ld_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

constexpr int kPreThreads = 256;
constexpr int kPreMaxInFlight = 8;  // rows a thread group has in flight at once (2 x 16 bytes each)
constexpr float kLog2e = 1.4426950408889634f;

// One block per 128-row tile of one (batch, head).  A group of D/8 adjacent lanes owns a row: each
// lane reads one 16-byte piece of o and of dout, multiplies, and the group reduces with shuffles
// in a fixed order (deterministic).  The block's 256 threads cover 2048 / D rows per pass and a
// thread issues the loads of up to kPreMaxInFlight passes (16 independent 16-byte loads) before it
// uses the first one, which is what keeps enough bytes in flight to fill the HBM pipe.
// D is the padded head dim; a row in memory has d8 <= D/8 pieces and the lanes beyond it
// contribute zeros.  Rows beyond N are written too: -lse2 = -inf makes every probability of a
// padded row exactly 0 downstream.  Both vectors are stored NEGATED so the consumers can use them
// as FMA / ADD addends directly.  The block also leaves the largest |dout| of its rows, as the
// 16-bit pattern with the sign cleared, in tile_amax[tile] (see head_dscale in bwd_roles.cuh).
template <int D, bool BF16>
__global__ void __launch_bounds__(kPreThreads)
    bwd_preprocess_kernel(const uint4* __restrict__ o, const uint4* __restrict__ dout,
                          const float* __restrict__ lse, float* __restrict__ rowstats,
                          unsigned* __restrict__ tile_amax, int N, int ntiles, int d8, int H,
                          Strides so, Strides sdo) {
  constexpr int kLanesPerRow = D / 8;
  constexpr int kRowsPerPass = kPreThreads / kLanesPerRow;  // 64, 32, 16 or 8
  constexpr int kPasses = 128 / kRowsPerPass;               // 2, 4, 8 or 16
  constexpr int kBatch = kPasses < kPreMaxInFlight ? kPasses : kPreMaxInFlight;
  __shared__ unsigned warp_max[kPreThreads / 32];
  const long long tile = blockIdx.x;  // = bh * ntiles + t
  const long long bh = tile / ntiles;
  const int t = static_cast<int>(tile - bh * ntiles);
  const long long bb = bh / H, hh = bh - bb * H;
  const int sub = threadIdx.x % kLanesPerRow;
  const int row_in_pass = threadIdx.x / kLanesPerRow;
  // strides are in 16-byte units (the host divides the element strides by 8)
  const uint4* o_head = o + bb * so.b + hh * so.h;
  const uint4* do_head = dout + bb * sdo.b + hh * sdo.h;
  float* out = rowstats + tile * 256;
  unsigned amax2 = 0;  // two running maxima of 15-bit magnitudes, one per 16-bit half
#pragma unroll
  for (int p0 = 0; p0 < kPasses; p0 += kBatch) {
    uint4 a[kBatch], b[kBatch];
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
      const int r = (p0 + i) * kRowsPerPass + row_in_pass;  // row inside the tile
      const long long row = static_cast<long long>(t) * 128 + r;
      if (row < N && sub < d8) {
        a[i] = ld_stream(o_head + row * so.n + sub);
        b[i] = ld_stream(do_head + row * sdo.n + sub);
      } else {
        a[i] = make_uint4(0, 0, 0, 0);
        b[i] = make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
      float acc = dot8<BF16>(a[i], b[i]);
#pragma unroll
      for (int off = kLanesPerRow / 2; off > 0; off >>= 1)
        acc += __shfl_xor_sync(0xffffffffu, acc, off);
      amax2 = __vmaxu2(amax2, b[i].x & 0x7fff7fffu);
      amax2 = __vmaxu2(amax2, b[i].y & 0x7fff7fffu);
      amax2 = __vmaxu2(amax2, b[i].z & 0x7fff7fffu);
      amax2 = __vmaxu2(amax2, b[i].w & 0x7fff7fffu);
      const int r = (p0 + i) * kRowsPerPass + row_in_pass;
      if (sub == 0) {
        const long long row = static_cast<long long>(t) * 128 + r;
        const bool valid = row < N;
        out[r] = valid ? -lse[bh * N + row] * kLog2e : -INFINITY;
        out[128 + r] = valid ? -acc : 0.f;
      }
    }
  }
  // largest magnitude of the block: halves, warp, block (a NaN or inf pattern wins, which
  // head_dscale treats as "do not scale")
  unsigned m = max(amax2 & 0xffffu, amax2 >> 16);
  m = __reduce_max_sync(0xffffffffu, m);
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
#pragma unroll
    for (int i = 1; i < kPreThreads / 32; ++i) m = max(m, warp_max[i]);
    tile_amax[tile] = m;
  }
}

// ----------------------------------------------------------------------------------------
// The same computation as a persistent kernel fed by the copy engine (head dims up to 128).
//
// One CTA per SM walks the 128-row tiles blockIdx.x, blockIdx.x + gridDim.x, ...  A producer warp
// keeps a ring of shared-memory stages full with untiled bulk copies (one stage = the o rows and
// the dout rows of one tile; one copy per tensor when its rows are contiguous in memory, else one
// copy per row), so the bytes in flight per SM stay near the ring size (128 - 192 KiB) whatever
// the eight consumer warps are doing; the block-per-tile kernel above has nothing in flight while
// a block reduces and stores, and reaches less than half of the HBM rate.  Consumers read their
// pieces from shared memory with the row / lane assignment of the kernel above, free the stage as
// soon as the pieces are in registers, and hand the tile's 256 results to the next iteration,
// which stores them with one coalesced 1 KiB write.  lse of the next tile is fetched one
// iteration ahead.  Rows in shared memory are packed at their true width (d8 pieces).
// ----------------------------------------------------------------------------------------
template <int D>
struct PreRing {
  static constexpr int kTileBytes = 128 * D * 2;      // one tensor's rows at the padded width
  static constexpr int kStageBytes = 2 * kTileBytes;  // o, then dout
  static constexpr int kStages = D == 128 ? 3 : (D == 64 ? 6 : 8);
  static constexpr int kConsumers = 256;
  static constexpr int kThreads = kConsumers + 32;
  // after the stages: full / empty barriers, two result buffers of 256 floats, two of 8 maxima
  static constexpr int kOffBars = kStages * kStageBytes;
  static constexpr int kOffStat = kOffBars + 16 * kStages;
  static constexpr int kOffMax = kOffStat + 2 * 256 * 4;
  static constexpr int kOffAbort = kOffMax + 2 * 8 * 4;
  static constexpr int kSmemBytes = kOffAbort + 16;
};

enum PreSite { kPSiteProducer = 64, kPSiteConsumer };

// All consumer threads learn whether every one of them got its stage (they leave together).
__device__ __forceinline__ bool consumers_all(bool ok, int nthreads) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "barrier.cta.red.and.pred p, 1, %2, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"(static_cast<uint32_t>(ok)), "r"(nthreads)
      : "memory");
  return r != 0;
}

template <int D, bool BF16>
__global__ void __launch_bounds__(PreRing<D>::kThreads, 1)
    bwd_preprocess_ring_kernel(const uint4* __restrict__ o, const uint4* __restrict__ dout,
                               const float* __restrict__ lse, float* __restrict__ rowstats,
                               unsigned* __restrict__ tile_amax, int N, int ntiles,
                               long long tiles, int d8, int H, Strides so, Strides sdo,
                               int* status) {
  using R = PreRing<D>;
  constexpr int kLanesPerRow = D / 8;
  constexpr int kRowsPerPass = R::kConsumers / kLanesPerRow;  // 64, 32 or 16
  constexpr int kPasses = 128 / kRowsPerPass;                 // 2, 4 or 8
  extern __shared__ __align__(128) unsigned char smem[];
  const uint32_t base = smem_u32(smem);
  auto full = [&](int s) { return base + R::kOffBars + 16u * s; };
  auto empty = [&](int s) { return base + R::kOffBars + 16u * s + 8u; };
  float* stat = reinterpret_cast<float*>(smem + R::kOffStat);
  unsigned* wmax = reinterpret_cast<unsigned*>(smem + R::kOffMax);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + R::kOffAbort);
  const WaitCtx w{abort_flag, status};
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < R::kStages; ++s) {
      mbar_init(full(s), 1);
      mbar_init(empty(s), R::kConsumers / 32);
    }
    fence_mbar_init();
  }
  __syncthreads();
  const uint32_t row_bytes = static_cast<uint32_t>(d8) * 16u;

  if (warp == R::kConsumers / 32) {
    // ---------------- producer warp ----------------
    int it = 0;
    for (long long tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++it) {
      const int s = it % R::kStages;
      const uint32_t ph = (it / R::kStages) & 1;
      if (!mbar_wait_warp(empty(s), ph ^ 1, w, kPSiteProducer)) break;
      const long long bh = tile / ntiles;
      const int t = static_cast<int>(tile - bh * ntiles);
      const long long bb = bh / H, hh = bh - bb * H;
      const int rows = min(128, N - t * 128);
      if (lane == 0) mbar_arrive_expect_tx(full(s), 2u * rows * row_bytes);
      __syncwarp();
      const uint32_t dst = base + s * R::kStageBytes;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const Strides& st = which ? sdo : so;
        const uint4* src = (which ? dout : o) + bb * st.b + hh * st.h +
                           static_cast<long long>(t) * 128 * st.n;
        const uint32_t d0 = dst + which * R::kTileBytes;
        if (st.n == d8) {
          if (lane == 0) bulk_load_1d(d0, src, rows * row_bytes, full(s));
        } else {
          for (int r = lane; r < rows; r += 32)
            bulk_load_1d(d0 + r * row_bytes, src + static_cast<long long>(r) * st.n, row_bytes,
                         full(s));
        }
      }
    }
    return;
  }

  // ---------------- consumer warps ----------------
  const int sub = threadIdx.x % kLanesPerRow;
  const int row_in_pass = threadIdx.x / kLanesPerRow;
  float lse_cur[kPasses], lse_nxt[kPasses];
  auto fetch_lse = [&](long long tile, float* dst) {
    const long long bh = tile / ntiles;
    const int t = static_cast<int>(tile - bh * ntiles);
#pragma unroll
    for (int i = 0; i < kPasses; ++i) {
      const int row = t * 128 + i * kRowsPerPass + row_in_pass;
      dst[i] = (sub == 0 && tile < tiles && row < N) ? __ldg(lse + bh * N + row) : INFINITY;
    }
  };
  fetch_lse(blockIdx.x, lse_cur);
  int it = 0;
  long long prev_tile = -1;
  for (long long tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++it) {
    const int s = it % R::kStages;
    const uint32_t ph = (it / R::kStages) & 1;
    fetch_lse(tile + gridDim.x, lse_nxt);
    const bool ok = mbar_wait(full(s), ph, w, kPSiteConsumer);
    if (!consumers_all(ok, R::kConsumers)) return;
    // the previous tile's results are complete in shared memory: one coalesced store
    if (prev_tile >= 0) {
      const int pb = (it - 1) & 1;
      rowstats[prev_tile * 256 + threadIdx.x] = stat[pb * 256 + threadIdx.x];
      if (threadIdx.x == 0) {
        unsigned m = wmax[pb * 8];
#pragma unroll
        for (int i = 1; i < 8; ++i) m = max(m, wmax[pb * 8 + i]);
        tile_amax[prev_tile] = m;
      }
    }
    const int t = static_cast<int>(tile % ntiles);
    const int rows = min(128, N - t * 128);
    const uint4* so_ = reinterpret_cast<const uint4*>(smem + s * R::kStageBytes);
    const uint4* sdo_ = reinterpret_cast<const uint4*>(smem + s * R::kStageBytes + R::kTileBytes);
    uint4 a[kPasses], b[kPasses];
#pragma unroll
    for (int i = 0; i < kPasses; ++i) {
      const int r = i * kRowsPerPass + row_in_pass;
      if (r < rows && sub < d8) {
        a[i] = so_[r * d8 + sub];
        b[i] = sdo_[r * d8 + sub];
      } else {
        a[i] = make_uint4(0, 0, 0, 0);
        b[i] = make_uint4(0, 0, 0, 0);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty(s));  // the pieces are in registers
    unsigned amax2 = 0;
    const int cb = it & 1;
#pragma unroll
    for (int i = 0; i < kPasses; ++i) {
      float acc = dot8<BF16>(a[i], b[i]);
#pragma unroll
      for (int off = kLanesPerRow / 2; off > 0; off >>= 1)
        acc += __shfl_xor_sync(0xffffffffu, acc, off);
      amax2 = __vmaxu2(amax2, b[i].x & 0x7fff7fffu);
      amax2 = __vmaxu2(amax2, b[i].y & 0x7fff7fffu);
      amax2 = __vmaxu2(amax2, b[i].z & 0x7fff7fffu);
      amax2 = __vmaxu2(amax2, b[i].w & 0x7fff7fffu);
      const int r = i * kRowsPerPass + row_in_pass;
      if (sub == 0) {
        const bool valid = r < rows;
        stat[cb * 256 + r] = valid ? -lse_cur[i] * kLog2e : -INFINITY;
        stat[cb * 256 + 128 + r] = valid ? -acc : 0.f;
      }
    }
    unsigned m = max(amax2 & 0xffffu, amax2 >> 16);
    m = __reduce_max_sync(0xffffffffu, m);
    if (lane == 0) wmax[cb * 8 + warp] = m;
#pragma unroll
    for (int i = 0; i < kPasses; ++i) lse_cur[i] = lse_nxt[i];
    prev_tile = tile;
  }
  if (prev_tile >= 0) {
    named_bar_sync(1, R::kConsumers);
    const int pb = (it - 1) & 1;
    rowstats[prev_tile * 256 + threadIdx.x] = stat[pb * 256 + threadIdx.x];
    if (threadIdx.x == 0) {
      unsigned m = wmax[pb * 8];
#pragma unroll
      for (int i = 1; i < 8; ++i) m = max(m, wmax[pb * 8 + i]);
      tile_amax[prev_tile] = m;
    }
  }
}

// One thread converts 8 consecutive head-dim elements of one row.  Consecutive lanes take
// consecutive rows of the same 32-row group, so the fp32 reads are contiguous 512-byte runs
// (the layout the fused backward kernel accumulates into).
template <int D, bool BF16>
__global__ void __launch_bounds__(256)
    dq_convert_kernel(const float4* __restrict__ acc, uint4* __restrict__ dq, int N, int ntiles,
                      long long total, int d8, int H, Strides sdq) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  // idx = ((tile_global * 4 + w) * (D/8) + k8) * 32 + lane
  const int lane = static_cast<int>(idx & 31);
  long long t = idx >> 5;
  const int k8 = static_cast<int>(t % (D / 8));
  t /= (D / 8);
  const int w = static_cast<int>(t & 3);
  const long long tile_global = t >> 2;
  const long long bh = tile_global / ntiles;
  const int tile = static_cast<int>(tile_global - bh * ntiles);
  const int row = tile * 128 + w * 32 + lane;
  if (row >= N || k8 >= d8) return;  // padding rows / padding columns of the accumulator
  const long long blk = (tile_global * 4 + w) * (D / 4);  // in units of [32 lanes][float4]
  const float4 x = acc[(blk + 2 * k8) * 32 + lane];
  const float4 y = acc[(blk + 2 * k8 + 1) * 32 + lane];
  uint4 r;
  r.x = pack2<BF16>(x.x, x.y);
  r.y = pack2<BF16>(x.z, x.w);
  r.z = pack2<BF16>(y.x, y.y);
  r.w = pack2<BF16>(y.z, y.w);
  const long long bb = bh / H, hh = bh - bb * H;
  dq[bb * sdq.b + hh * sdq.h + row * sdq.n + k8] = r;  // strides in 16-byte units
}

// Element strides -> strides in 16-byte pieces (every stride is a multiple of 8 elements).
Strides in_vec8(const Strides& st) { return Strides{st.b / 8, st.h / 8, st.n / 8}; }

template <int D, bool BF16>
cudaError_t launch_pre_t(const AttnShape& s, const void* o, const Strides& so, const void* dout,
                         const Strides& sdo, const float* lse, float* rowstats, int* status,
                         int num_sms, cudaStream_t stream) {
  const int ntiles = (s.N + 127) / 128;
  const long long tiles = static_cast<long long>(s.B) * s.H * ntiles;
  unsigned* tile_amax = reinterpret_cast<unsigned*>(rowstats + tiles * 256);  // behind the last tile
  if constexpr (D <= 128) {
    using R = PreRing<D>;
    auto* kernel = bwd_preprocess_ring_kernel<D, BF16>;
    const cudaError_t attr = cudaFuncSetAttribute(
        kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, R::kSmemBytes);
    if (attr != cudaSuccess) return attr;
    const unsigned grid = static_cast<unsigned>(tiles < num_sms ? tiles : num_sms);
    kernel<<<grid, R::kThreads, R::kSmemBytes, stream>>>(
        static_cast<const uint4*>(o), static_cast<const uint4*>(dout), lse, rowstats, tile_amax,
        s.N, ntiles, tiles, s.Dg / 8, s.H, in_vec8(so), in_vec8(sdo), status);
  } else {
    bwd_preprocess_kernel<D, BF16><<<static_cast<unsigned>(tiles), kPreThreads, 0, stream>>>(
        static_cast<const uint4*>(o), static_cast<const uint4*>(dout), lse, rowstats, tile_amax,
        s.N, ntiles, s.Dg / 8, s.H, in_vec8(so), in_vec8(sdo));
  }
  return cudaGetLastError();
}

template <int D, bool BF16>
cudaError_t launch_cvt_t(const AttnShape& s, const float* dq_accum, void* dq, const Strides& sdq,
                         cudaStream_t stream) {
  const int ntiles = (s.N + 127) / 128;
  const long long total = static_cast<long long>(s.B) * s.H * ntiles * 128 * (D / 8);
  const long long blocks = (total + 255) / 256;
  dq_convert_kernel<D, BF16><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
      reinterpret_cast<const float4*>(dq_accum), static_cast<uint4*>(dq), s.N, ntiles, total,
      s.Dg / 8, s.H, in_vec8(sdq));
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_bwd_preprocess(const AttnShape& s, const void* o, const Strides& so,
                                  const void* dout, const Strides& sdo, const float* lse,
                                  float* rowstats, int* status, int num_sms,
                                  cudaStream_t stream) {
#define FA2_CASE(DD)                                                                          \
  case DD:                                                                                    \
    return s.dtype                                                                            \
               ? launch_pre_t<DD, true>(s, o, so, dout, sdo, lse, rowstats, status, num_sms,  \
                                        stream)                                               \
               : launch_pre_t<DD, false>(s, o, so, dout, sdo, lse, rowstats, status, num_sms, \
                                         stream);
  switch (s.D) {
    FA2_CASE(32)
    FA2_CASE(64)
    FA2_CASE(128)
    FA2_CASE(256)
  }
#undef FA2_CASE
  return cudaErrorInvalidValue;
}

cudaError_t launch_dq_convert(const AttnShape& s, const float* dq_accum, void* dq,
                              const Strides& sdq, cudaStream_t stream) {
#define FA2_CASE(DD)                                                        \
  case DD:                                                                  \
    return s.dtype ? launch_cvt_t<DD, true>(s, dq_accum, dq, sdq, stream)   \
                   : launch_cvt_t<DD, false>(s, dq_accum, dq, sdq, stream);
  switch (s.D) {
    FA2_CASE(32)
    FA2_CASE(64)
    FA2_CASE(128)
  }
#undef FA2_CASE
  return cudaErrorInvalidValue;
}

}  // namespace fa2
