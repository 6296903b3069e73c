// Inline-PTX layer for sm_100a: mbarrier, TMA (tiled bulk tensor copies), tcgen05 (tensor
// memory allocation, MMA issue, commit, load/store, fences) and descriptor encoders.
// Everything here is a thin wrapper; protocol logic lives in the kernels.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>

namespace fa2 {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ----------------------------------------------------------------------------------------
// Bounded waits.  No wait in this library spins forever: after kWaitLimitCycles a waiter
// raises the CTA-wide abort flag and records where it gave up in the device status word;
// every other waiter of the CTA sees the flag and leaves too, the CTA drains and frees its
// tensor memory, and the host reads the status word (fa2_device_status).
// ----------------------------------------------------------------------------------------
constexpr long long kWaitLimitCycles = 4000000000LL;  // ~2 s at 1.9 GHz

struct WaitCtx {
  volatile int* abort_flag;  // shared memory, one per CTA
  int* status;               // global memory, one per device
};

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_inval(uint32_t bar) {
  asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Returns false when the wait was abandoned (CTA abort).  `site` identifies the caller in
// the status word.
__device__ __forceinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, const WaitCtx& w,
                                               int site) {
  const long long t0 = clock64();
  uint32_t it = 0;
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++it & 63u) == 0) {
      if (*w.abort_flag) return false;
      if (clock64() - t0 > kWaitLimitCycles) {
        *w.abort_flag = 1;
        atomicCAS(w.status, 0, 0x10000 | site);
        return false;
      }
    }
  }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const WaitCtx& w,
                                          int site) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, w, site);
}
// Warp-uniform variant for warps that go on to execute .sync.aligned instructions.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, const WaitCtx& w,
                                               int site) {
  const bool ok = mbar_wait(bar, parity, w, site);
  return __all_sync(0xffffffffu, ok);
}

// ----------------------------------------------------------------------------------------
// Proxy fences and named barriers
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void named_bar_sync(uint32_t id, uint32_t nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ----------------------------------------------------------------------------------------
// TMA: tiled 4-D tensor copies, coordinates {x = element in row, y = row, head, batch}.
// Batch and head are separate dimensions so that the tensors may have any batch / head /
// row strides (multiples of 16 bytes); boxes are always one head of one batch wide.
// ----------------------------------------------------------------------------------------
struct HeadCoord {
  int h, b;
};
__device__ __forceinline__ void tma_load_4d(uint32_t dst_smem, const CUtensorMap* map, int x,
                                            int y, HeadCoord hc, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(dst_smem),
      "l"(map), "r"(x), "r"(y), "r"(hc.h), "r"(hc.b), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, int x, int y, HeadCoord hc,
                                             uint32_t src_smem) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3, %4}], [%5];" ::
          "l"(map),
      "r"(x), "r"(y), "r"(hc.h), "r"(hc.b), "r"(src_smem)
      : "memory");
}
// 3-D variants for the library's own dense scratch tensors: {x, y, tile index}.
__device__ __forceinline__ void tma_load_3d(uint32_t dst_smem, const CUtensorMap* map, int x,
                                            int y, int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst_smem),
      "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, int x, int y, int z,
                                             uint32_t src_smem) {
  asm volatile(
      "cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];" ::"l"(
          map),
      "r"(x), "r"(y), "r"(z), "r"(src_smem)
      : "memory");
}
// All bulk stores of this thread have finished READING shared memory (the data may still be
// in flight to global memory): the source buffer can be rewritten.
// Untiled bulk copy global -> shared: both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_load_1d(uint32_t dst_smem, const void* src, uint32_t bytes,
                                             uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(dst_smem),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ----------------------------------------------------------------------------------------
// tcgen05: tensor memory + MMA
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// One lane of a converged warp gets a non-zero result.  The MMA warp runs its whole role
// convergently and predicates only the tcgen05.mma / commit instructions on this flag: that
// keeps descriptor arithmetic warp-uniform (cheap for the scheduler) instead of burying it in
// a single-lane divergent branch, where the issuing warp is starved by busy compute warps.
__device__ __forceinline__ uint32_t elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred;
}
// Arrive on `bar` once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// 32 lanes x 32-bit, N consecutive columns per thread: thread t of warp w reads lane
// 32*(w%4)+t of tensor memory.  The lane field of `taddr` must be 32*(w%4).
#define FA2_R4(a, i) a(i), a(i + 1), a(i + 2), a(i + 3)
#define FA2_R16(a, i) FA2_R4(a, i), FA2_R4(a, i + 4), FA2_R4(a, i + 8), FA2_R4(a, i + 12)
#define FA2_OUT(i) "=r"(r[i])
#define FA2_IN(i) "r"(r[i])

__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : FA2_R16(FA2_OUT, 0), FA2_R16(FA2_OUT, 16)
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : FA2_R16(FA2_OUT, 0)
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_x32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};" ::
          FA2_R16(FA2_IN, 0),
      FA2_R16(FA2_IN, 16), "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15};" ::FA2_R16(FA2_IN,
                                                                                         0),
      "r"(taddr)
      : "memory");
}

// ----------------------------------------------------------------------------------------
// Descriptors
// ----------------------------------------------------------------------------------------
// Shared-memory matrix descriptor (64-bit): [0,14) start>>4, [16,30) leading byte offset>>4,
// [32,46) stride byte offset>>4, [46,48) version = 1, [61,64) swizzle (2 = 128 B, 4 = 64 B).
constexpr uint32_t kSwizzle128B = 2;
constexpr uint32_t kSwizzle64B = 4;

__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes,
                                                   uint32_t sbo_bytes, uint32_t swizzle) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;
  d |= static_cast<uint64_t>(swizzle) << 61;
  return d;
}

// Instruction descriptor for kind::f16 with fp32 accumulation: [4,6) D format (1 = f32),
// [7,10) A format, [10,13) B format (0 = f16, 1 = bf16; the two are independent fields), bit 15 /
// 16 = A / B is MN-major, [17,23) N>>3, [24,29) M>>4.
__host__ __device__ constexpr uint32_t make_idesc_ab(int m, int n, bool a_bf16, bool b_bf16,
                                                     bool a_mn_major, bool b_mn_major) {
  return (1u << 4) | ((a_bf16 ? 1u : 0u) << 7) | ((b_bf16 ? 1u : 0u) << 10) |
         ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}
// Both operands of the tensors' dtype.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, bool bf16, bool a_mn_major,
                                                  bool b_mn_major) {
  return make_idesc_ab(m, n, bf16, bf16, a_mn_major, b_mn_major);
}

// ----------------------------------------------------------------------------------------
// Small math helpers
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float lg2(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// 2^x for a pair of values on the FMA pipe instead of the MUFU: round-to-nearest split
// x = n + f, f in [-0.5, 0.5], degree-3 minimax polynomial for 2^f (relative error 7.5e-5,
// below half an ulp of both 16-bit formats), exponent added with integer arithmetic.  Inputs
// are clamped at -126, so -inf gives 2^-126 (~1e-38) rather than exactly 0.
__device__ __forceinline__ float2 ex2_poly2(float2 x) {
  const float2 magic = make_float2(12582912.f, 12582912.f);  // 1.5 * 2^23
  const float2 nmagic = make_float2(-12582912.f, -12582912.f);
  x.x = fmaxf(x.x, -126.f);
  x.y = fmaxf(x.y, -126.f);
  const float2 t = __fadd2_rn(x, magic);
  const float2 n = __fadd2_rn(t, nmagic);
  const float2 f = __fadd2_rn(x, make_float2(-n.x, -n.y));
  float2 p = __ffma2_rn(make_float2(0.055171407759189606f, 0.055171407759189606f), f,
                        make_float2(0.2426110953092575f, 0.2426110953092575f));
  p = __ffma2_rn(p, f, make_float2(0.6932610273361206f, 0.6932610273361206f));
  p = __ffma2_rn(p, f, make_float2(0.9999280571937561f, 0.9999280571937561f));
  p.x = __uint_as_float(__float_as_uint(p.x) + (__float_as_uint(t.x) << 23));
  p.y = __uint_as_float(__float_as_uint(p.y) + (__float_as_uint(t.y) << 23));
  return p;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
template <int N>
__device__ __forceinline__ void reg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
// Type of the operands the kernels produce themselves (probabilities P, score gradients dS):
// that of the tensors.  (fp16 P and dS next to bf16 tensors would give bf16 problems the 11
// significant bits the reference's all-fp16 arithmetic has, flash_attention_2.py:316, but
// tcgen05.mma.kind::f16 takes an fp16 A operand with a bf16 B operand as an illegal instruction
// on this part, although the descriptor has one format field per operand.)
template <bool BF16>
constexpr bool kInterBF16 = BF16;

// Two fp32 -> one 32-bit word holding two 16-bit values, `lo` in bits [0,16).
template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  uint32_t r;
  if constexpr (BF16) {
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  } else {
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  }
  return r;
}

}  // namespace fa2
