// C ABI of the library (declared in include/fa2_b200.h): argument validation, tensor-map
// construction and kernel dispatch.  Nothing here allocates device memory or synchronises,
// except fa2_device_status which reads the status word back.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <mutex>

#include "../../include/fa2_b200.h"
#include "common.cuh"

namespace fa2 {

// One status word per device: kernels write here when a bounded wait expires.
__device__ int g_status_word;
// Work counters of the tile-fetching kernels.  Every launch takes the next slot of this ring, so
// launches that overlap on the device do not share a counter (unless more than
// kWorkCounterSlots of them are in flight at once).  No launch zeroes its slot: the slots are
// zero at module load and every kernel puts its counter back to zero when it draws its last
// number (fetch_work_item), so a slot is only left non-zero by a kernel that did not run to
// its end.
constexpr int kWorkCounterSlots = 1024;
__device__ unsigned int g_work_counters[kWorkCounterSlots];

namespace {

constexpr int kMaxDevices = 64;

// fa2_bwd_mark_between: event the next two-kernel backward of this thread records between its
// kernels (one-shot).
thread_local cudaEvent_t t_mark_between = nullptr;
void record_mark_between(cudaStream_t st) {
  if (t_mark_between) {
    cudaEventRecord(t_mark_between, st);
    t_mark_between = nullptr;
  }
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn g_encode = nullptr;
std::once_flag g_encode_once;

EncodeTiledFn get_encode() {
  std::call_once(g_encode_once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  });
  return g_encode;
}

struct DeviceState {
  std::once_flag once;
  int cc_major = 0;
  int num_sms = 0;
  int* status = nullptr;
  unsigned int* counters = nullptr;
  std::atomic<unsigned> next_counter{0};
  cudaError_t err = cudaSuccess;
};
DeviceState g_dev[kMaxDevices];

// Per-device set-up on first use: compute capability and the address of the status word.
int device_state(DeviceState** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kMaxDevices) return FA2_ERR_ARCH;
  // cudaGetDevice alone does not make the device's primary context current in a thread that
  // has made no other runtime call yet (a freshly started worker thread whose allocations all
  // came from a cache); cuTensorMapEncodeTiled, a driver call, then refuses the tensor.
  // cudaSetDevice binds the context and costs nothing when it is bound already.
  e = cudaSetDevice(dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  DeviceState& d = g_dev[dev];
  std::call_once(d.once, [&] {
    d.err = cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev);
    if (d.err == cudaSuccess)
      d.err = cudaDeviceGetAttribute(&d.num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (d.err == cudaSuccess)
      d.err = cudaGetSymbolAddress(reinterpret_cast<void**>(&d.status), g_status_word);
    if (d.err == cudaSuccess)
      d.err = cudaGetSymbolAddress(reinterpret_cast<void**>(&d.counters), g_work_counters);
  });
  if (d.err != cudaSuccess) return static_cast<int>(d.err);
  if (d.cc_major != 10) return FA2_ERR_ARCH;
  *out = &d;
  return FA2_OK;
}

// Strides of tensor `idx` of a call: the caller's triple, or dense when the array is NULL or
// the triple is all zeros.  Strides of size-1 dimensions carry no information (frameworks
// put anything there) and are replaced by the dense ones.
int get_strides(const long long* user, int idx, int B, int H, int N, int D, Strides* out) {
  const Strides dense{static_cast<long long>(H) * N * D, static_cast<long long>(N) * D, D};
  *out = dense;
  if (!user) return FA2_OK;
  const long long* u = user + 3 * idx;
  if (u[0] == 0 && u[1] == 0 && u[2] == 0) return FA2_OK;
  if (B > 1) out->b = u[0];
  if (H > 1) out->h = u[1];
  if (N > 1) out->n = u[2];
  const long long v[3] = {out->b, out->h, out->n};
  for (long long x : v)
    if (x <= 0 || x % 8 != 0 || x >= (1ll << 38)) return FA2_ERR_STRIDE;
  if (out->n < D) return FA2_ERR_STRIDE;
  return FA2_OK;
}

// Tensor map over a [B, H, N, D] 16-bit tensor with box (chunk, box_rows, 1, 1).  The chunk
// follows the padded head dim, so for D = 48 or 96 the last box of a row hangs over the
// tensor: those columns read as zeros and are not written.
int make_map(CUtensorMap* m, const void* base, int dtype, int B, int H, int N, int D,
             const Strides& st, int box_rows) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return FA2_ERR_DRIVER;
  const int chunk = padded_head_dim(D) >= 64 ? 64 : 32;
  const cuuint64_t gdim[4] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(N),
                              static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(B)};
  const cuuint64_t gstride[3] = {static_cast<cuuint64_t>(st.n) * 2,
                                 static_cast<cuuint64_t>(st.h) * 2,
                                 static_cast<cuuint64_t>(st.b) * 2};
  const cuuint32_t box[4] = {static_cast<cuuint32_t>(chunk), static_cast<cuuint32_t>(box_rows), 1,
                             1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r =
      enc(m, dtype ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
          const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
          chunk == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FA2_OK : FA2_ERR_DRIVER;
}

// Map of tensor `idx` of a call (strides as get_strides resolves them).
int make_map_of(CUtensorMap* m, const void* base, const long long* user, int idx, int dtype,
                int B, int H, int N, int D, int box_rows) {
  Strides st;
  if (int e = get_strides(user, idx, B, H, N, D, &st)) return e;
  return make_map(m, base, dtype, B, H, N, D, st, box_rows);
}

// Context for one kernel launch.  Launches rotate through a ring of work counters (all zero
// at module load, each left at zero by the kernel that used it), so kernels that overlap on
// different streams do not share one.
void make_ctx(DeviceState* d, LaunchCtx* ctx) {
  ctx->status = d->status;
  ctx->work_counter = d->counters + (d->next_counter.fetch_add(1) % kWorkCounterSlots);
  ctx->num_sms = d->num_sms;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int check_shape(int B, int H, int N, int D, int dtype) {
  if (D < 8 || D > 256 || D % 8 != 0) return FA2_ERR_HEAD_DIM;
  if (dtype != FA2_DTYPE_FP16 && dtype != FA2_DTYPE_BF16) return FA2_ERR_DTYPE;
  if (B <= 0 || H <= 0 || N <= 0) return FA2_ERR_SHAPE;
  if (static_cast<long long>(B) * H > 65535) return FA2_ERR_SHAPE;
  if (N > (1 << 24)) return FA2_ERR_SHAPE;
  return FA2_OK;
}

// Scratch of the spilling backward modes: one 32 KiB dS tile per (KV tile, Q tile) pair of a
// head, and a P tile as well for head dims above 128.
long long spill_bytes_per_head(int N, int Nk, int D) {
  return dstile_pairs(N, Nk) * 32768 * (D > 128 ? 2 : 1);
}
// What fa2_bwd_workspace_bytes recommends at most (fa2_set_spill_budget); a workspace of any size
// that holds one head is accepted by fa2_bwd.
std::atomic<long long> g_spill_budget{8ll << 30};
// Tiles (= CTAs of the dK/dV and of the dQ kernel) a chunk should have.  Smaller chunks leave SMs
// idle at the end of every launch: at N = 8192, d = 128 on 148 SMs, chunks of 2048 tiles cost
// 0.5 % against a single chunk of 4096, 1024 tiles 3 %, 512 tiles 11 %, 256 tiles 21 %, 64 tiles
// (one head) 290 %.  More scratch than this buys nothing, so the recommendation grows with N
// (about 256 KiB per row of a head), not with B * H * N^2.
constexpr long long kSpillChunkTiles = 2048;

// Spill mode (and head dims above 128, which have no other backward): the problem is worked
// through in chunks of whole batch entries, or of head ranges of one batch entry, that fit the
// workspace.  The split never changes a bit of the results (every (batch, head) problem is
// independent).
struct SpillPlan {
  int nb, nh;  // batch entries and heads per chunk; nb == 0: not even one head fits
};
SpillPlan spill_plan(int B, int H, long long per_head, long long bytes) {
  const long long heads_fit = bytes / per_head;
  if (heads_fit < 1) return SpillPlan{0, 0};
  if (heads_fit >= H)
    return SpillPlan{static_cast<int>(std::min<long long>(B, heads_fit / H)), H};
  const long long nchunks = (H + heads_fit - 1) / heads_fit;
  return SpillPlan{1, static_cast<int>((H + nchunks - 1) / nchunks)};
}

AttnShape make_shape(int B, int H, int N, int Nk, int D, int dtype, float scale) {
  return AttnShape{B, H, N, padded_head_dim(D), dtype, scale, D, Nk};
}

}  // namespace
}  // namespace fa2

using namespace fa2;

extern "C" {

int fa2_abi_version(void) { return FA2_ABI_VERSION; }

const char* fa2_strerror(int code) {
  switch (code) {
    case FA2_OK: return "success";
    case FA2_ERR_NULL_POINTER: return "a required pointer is NULL";
    case FA2_ERR_HEAD_DIM: return "head dimension must be a multiple of 8 between 8 and 256";
    case FA2_ERR_DTYPE: return "dtype must be 0 (fp16) or 1 (bf16)";
    case FA2_ERR_MISALIGNED: return "tensor pointers must be 16-byte aligned";
    case FA2_ERR_SHAPE: return "B, H, N must be positive, B*H <= 65535, N <= 2^24, 1 <= Nk <= N";
    case FA2_ERR_ARCH: return "the current device is not compute capability 10.x (B200)";
    case FA2_ERR_DEVICE_STATUS: return "a kernel abandoned a bounded wait (see fa2_device_status)";
    case FA2_ERR_DRIVER: return "cuTensorMapEncodeTiled is unavailable or rejected the tensor";
    case FA2_ERR_SCALE: return "softmax scale must be finite and > 0";
    case FA2_ERR_WORKSPACE:
      return "this backward mode needs a workspace of at least its minimum size (fa2_bwd_workspace_bytes)";
    case FA2_ERR_STRIDE:
      return "strides must be positive multiples of 8 elements (16 bytes), row stride >= D";
    case FA2_ERR_TOO_LARGE: return "problem exceeds the built-in scratch (B*H*ceil(N/128) > 4096)";
    default: break;
  }
  if (code > 0) return cudaGetErrorString(static_cast<cudaError_t>(code));
  return "unknown fa2 error code";
}

int fa2_fwd_strided(const void* q, const void* k, const void* v, void* o, float* lse, int B, int H,
                    int N, int Nk, int D, int dtype, float scale, const long long* strides,
                    fa2_stream_t stream) {
  if (!q || !k || !v || !o || !lse) return FA2_ERR_NULL_POINTER;
  if (int e = check_shape(B, H, N, D, dtype)) return e;
  if (Nk < 1 || Nk > N) return FA2_ERR_SHAPE;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o)) return FA2_ERR_MISALIGNED;
  if (!std::isfinite(scale) || !(scale > 0.f)) return FA2_ERR_SCALE;
  for (int idx = 0; idx < 4; ++idx) {
    Strides unused;
    if (int e = get_strides(strides, idx, B, H, idx == 1 || idx == 2 ? Nk : N, D, &unused)) return e;
  }
  DeviceState* d = nullptr;
  if (int e = device_state(&d)) return e;
  CUtensorMap tq, tk, tv, to;
  if (int e = make_map_of(&tq, q, strides, 0, dtype, B, H, N, D, 128)) return e;
  if (int e = make_map_of(&tk, k, strides, 1, dtype, B, H, Nk, D, 128)) return e;
  if (int e = make_map_of(&tv, v, strides, 2, dtype, B, H, Nk, D, 128)) return e;
  if (int e = make_map_of(&to, o, strides, 3, dtype, B, H, N, D, 32)) return e;
  const AttnShape s = make_shape(B, H, N, Nk, D, dtype, scale);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  LaunchCtx ctx;
  make_ctx(d, &ctx);
  return static_cast<int>(launch_fwd(s, tq, tk, tv, to, lse, ctx, st));
}

int fa2_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int H, int N,
            int D, int dtype, float scale, fa2_stream_t stream) {
  return fa2_fwd_strided(q, k, v, o, lse, B, H, N, N, D, dtype, scale, nullptr, stream);
}

size_t fa2_rowstats_bytes(int B, int H, int N) {
  if (B <= 0 || H <= 0 || N <= 0) return 0;
  const size_t ntiles = (static_cast<size_t>(N) + 127) / 128;
  return static_cast<size_t>(B) * H * ntiles * (256 + 1) * sizeof(float);  // two vectors + one word per tile
}

int fa2_bwd_preprocess_strided(const void* o, const void* dout, const float* lse, float* rowstats,
                               int B, int H, int N, int D, int dtype, const long long* strides,
                               fa2_stream_t stream) {
  if (!o || !dout || !lse || !rowstats) return FA2_ERR_NULL_POINTER;
  if (int e = check_shape(B, H, N, D, dtype)) return e;
  if (!aligned16(o) || !aligned16(dout) || !aligned16(rowstats)) return FA2_ERR_MISALIGNED;
  if (static_cast<long long>(B) * H * ((N + 127) / 128) > 0x7fffffffll) return FA2_ERR_SHAPE;  // one block per tile (head dim 256)
  Strides so, sdo;
  if (int e = get_strides(strides, 0, B, H, N, D, &so)) return e;
  if (int e = get_strides(strides, 1, B, H, N, D, &sdo)) return e;
  DeviceState* d = nullptr;
  if (int e = device_state(&d)) return e;
  const AttnShape s = make_shape(B, H, N, N, D, dtype, 1.f);
  return static_cast<int>(launch_bwd_preprocess(s, o, so, dout, sdo, lse, rowstats, d->status,
                                                d->num_sms, static_cast<cudaStream_t>(stream)));
}

int fa2_bwd_preprocess(const void* o, const void* dout, const float* lse, float* rowstats, int B,
                       int H, int N, int D, int dtype, fa2_stream_t stream) {
  return fa2_bwd_preprocess_strided(o, dout, lse, rowstats, B, H, N, D, dtype, nullptr, stream);
}

size_t fa2_bwd_workspace_bytes(int B, int H, int N, int D, int deterministic) {
  if (B <= 0 || H <= 0 || N <= 0 || D <= 0) return 0;
  const long long BH = static_cast<long long>(B) * H;
  if (deterministic == 2 || D > 128) {
    // 16-bit [128 x 128] tiles of whole heads: as many heads as make a chunk of
    // kSpillChunkTiles tiles, within the budget, never less than one head; then what the chunk
    // plan uses of that
    const long long per_head = spill_bytes_per_head(N, N, D);
    const long long ntiles = (static_cast<long long>(N) + 127) / 128;
    const long long want = (kSpillChunkTiles + ntiles - 1) / ntiles * per_head;
    const SpillPlan plan =
        spill_plan(B, H, per_head, std::max(per_head, std::min(want, g_spill_budget.load())));
    return static_cast<size_t>(plan.nb) * plan.nh * static_cast<size_t>(per_head);
  }
  if (deterministic == 1) return 0;
  const size_t ntiles = (static_cast<size_t>(N) + 127) / 128;
  return static_cast<size_t>(BH) * ntiles * 128 * padded_head_dim(D) * sizeof(float);
}

// fa2_bwd_strided with the two parts of the preprocess output given separately, so that a chunk of
// a larger problem (see the chunk loop below) can point into the arrays of the whole problem.
static int bwd_strided(const void* q, const void* k, const void* v, const void* dout,
                       const float* rowstats_ptr, const unsigned* tile_amax, void* dq, void* dk,
                       void* dv, void* workspace, size_t workspace_bytes, int B, int H, int N, int Nk,
                       int D, int dtype, float scale, int deterministic, const long long* strides,
                       fa2_stream_t stream) {
  const float* rowstats = rowstats_ptr;
  if (!q || !k || !v || !dout || !rowstats || !dq || !dk || !dv) return FA2_ERR_NULL_POINTER;
  if (int e = check_shape(B, H, N, D, dtype)) return e;
  if (Nk < 1 || Nk > N) return FA2_ERR_SHAPE;
  if (deterministic < 0 || deterministic > 2) return FA2_ERR_SHAPE;
  // Head dims above 128 have one backward (scores kernel + three consumer kernels over two
  // scratch tensors, in chunks); it is deterministic and serves every value of `deterministic`.
  if (D > 128) deterministic = 2;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(dout) || !aligned16(dq) ||
      !aligned16(dk) || !aligned16(dv) || !aligned16(rowstats))
    return FA2_ERR_MISALIGNED;
  if (!std::isfinite(scale) || !(scale > 0.f)) return FA2_ERR_SCALE;
  if (static_cast<long long>(B) * H * ((N + 127) / 128) > 0x7fffffffll) return FA2_ERR_SHAPE;  // one CTA per tile
  if (deterministic != 1 && !workspace) return FA2_ERR_WORKSPACE;
  if (deterministic != 1 && (reinterpret_cast<uintptr_t>(workspace) & 255u)) return FA2_ERR_MISALIGNED;
  // The workspace must hold what the mode needs at least; what lies beyond is used when it
  // helps (more scratch slots, larger chunks) and never written otherwise.
  const long long BH = static_cast<long long>(B) * H;
  const long long per_head = spill_bytes_per_head(N, Nk, D);
  const long long ws = static_cast<long long>(std::min<size_t>(workspace_bytes, size_t(1) << 62));
  if (deterministic == 0 && workspace_bytes < fa2_bwd_workspace_bytes(B, H, N, D, 0))
    return FA2_ERR_WORKSPACE;
  if (deterministic == 2 && ws < per_head) return FA2_ERR_WORKSPACE;
  const int rows_of[7] = {N, Nk, Nk, N, N, Nk, Nk};  // q, k, v, dout, dq, dk, dv
  long long st_all[21];
  for (int idx = 0; idx < 7; ++idx) {
    Strides t;
    if (int e = get_strides(strides, idx, B, H, rows_of[idx], D, &t)) return e;
    st_all[3 * idx] = t.b, st_all[3 * idx + 1] = t.h, st_all[3 * idx + 2] = t.n;
  }
  DeviceState* d = nullptr;
  if (int e = device_state(&d)) return e;
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  if (deterministic == 2) {
    const SpillPlan plan = spill_plan(B, H, per_head, ws);
    if (plan.nb < B || plan.nh < H) {
      // more than one chunk: the same call on sub-ranges, one after the other on the stream
      // (they share the scratch), with the caller's strides spelled out
      const void* in[4] = {q, k, v, dout};
      void* out[3] = {dq, dk, dv};
      const size_t stats_per_head = static_cast<size_t>((N + 127) / 128) * 256;
      for (int b0 = 0; b0 < B; b0 += plan.nb)
        for (int h0 = 0; h0 < H; h0 += plan.nh) {
          const int nb = std::min(plan.nb, B - b0), nh = std::min(plan.nh, H - h0);
          auto at = [&](const void* p, int idx) {
            return static_cast<const char*>(p) + 2 * (b0 * st_all[3 * idx] + h0 * st_all[3 * idx + 1]);
          };
          const int e = bwd_strided(
              at(in[0], 0), at(in[1], 1), at(in[2], 2), at(in[3], 3),
              rowstats + (static_cast<size_t>(b0) * H + h0) * stats_per_head,
              tile_amax + (static_cast<size_t>(b0) * H + h0) * ((N + 127) / 128),
              const_cast<char*>(at(out[0], 4)), const_cast<char*>(at(out[1], 5)),
              const_cast<char*>(at(out[2], 6)), workspace, workspace_bytes, nb, nh, N, Nk, D, dtype,
              scale, 2, st_all, stream);
          if (e) return e;
        }
      return FA2_OK;
    }
    if (BH * dstile_pairs(N, Nk) >= (1ll << 31)) return FA2_ERR_SHAPE;
  }

  CUtensorMap tq, tk, tv, tdo, tdq, tdk, tdv;
  if (int e = make_map_of(&tq, q, strides, 0, dtype, B, H, N, D, 128)) return e;
  if (int e = make_map_of(&tk, k, strides, 1, dtype, B, H, Nk, D, 128)) return e;
  if (int e = make_map_of(&tv, v, strides, 2, dtype, B, H, Nk, D, 128)) return e;
  if (int e = make_map_of(&tdo, dout, strides, 3, dtype, B, H, N, D, 128)) return e;
  if (int e = make_map_of(&tdk, dk, strides, 5, dtype, B, H, Nk, D, 32)) return e;
  if (int e = make_map_of(&tdv, dv, strides, 6, dtype, B, H, Nk, D, 32)) return e;
  const Strides sdq{st_all[12], st_all[13], st_all[14]};
  const AttnShape s = make_shape(B, H, N, Nk, D, dtype, scale);
  const RowStats rs{rowstats, tile_amax};
  if (deterministic != 0)
    if (int e = make_map(&tdq, dq, dtype, B, H, N, D, sdq, 32)) return e;

  if (deterministic == 1) {
    cudaError_t ce =
        launch_bwd_dkdv(s, tq, tk, tv, tdo, tdk, tdv, rs, nullptr, 0, d->status, st);
    if (ce != cudaSuccess) return static_cast<int>(ce);
    record_mark_between(st);
    return static_cast<int>(launch_bwd_dq(s, tq, tk, tv, tdo, tdq, rs, d->status, st));
  }
  if (deterministic == 2) {
    float* scratch = static_cast<float*>(workspace);
    if (D > 128) {
      // P tiles first, dS tiles behind them
      const long long pairs = BH * dstile_pairs(N, Nk);
      char* p_scratch = static_cast<char*>(workspace);
      char* ds_scratch = p_scratch + static_cast<size_t>(pairs) * 32768;
      cudaError_t ce = launch_bwd_scores_wide(s, tq, tk, tv, tdo, rs, p_scratch, ds_scratch,
                                              d->status, st);
      if (ce != cudaSuccess) return static_cast<int>(ce);
      if ((ce = launch_bwd_consume(s, 0, p_scratch, tdo, tdv, rs, d->status, st)) != cudaSuccess)
        return static_cast<int>(ce);
      if ((ce = launch_bwd_consume(s, 1, ds_scratch, tq, tdk, rs, d->status, st)) != cudaSuccess)
        return static_cast<int>(ce);
      return static_cast<int>(launch_bwd_consume(s, 2, ds_scratch, tk, tdq, rs, d->status, st));
    }
    cudaError_t ce =
        launch_bwd_dkdv(s, tq, tk, tv, tdo, tdk, tdv, rs, scratch, 2, d->status, st);
    if (ce != cudaSuccess) return static_cast<int>(ce);
    record_mark_between(st);
    return static_cast<int>(launch_bwd_consume(s, 2, scratch, tk, tdq, rs, d->status, st));
  }
  float* dq_accum = static_cast<float*>(workspace);
  cudaError_t ce = cudaMemsetAsync(dq_accum, 0, fa2_bwd_workspace_bytes(B, H, N, D, 0), st);
  if (ce != cudaSuccess) return static_cast<int>(ce);
  ce = launch_bwd_dkdv(s, tq, tk, tv, tdo, tdk, tdv, rs, dq_accum, 1, d->status, st);
  if (ce != cudaSuccess) return static_cast<int>(ce);
  return static_cast<int>(launch_dq_convert(s, dq_accum, dq, sdq, st));
}

int fa2_bwd_strided(const void* q, const void* k, const void* v, const void* dout,
                    const float* rowstats, void* dq, void* dk, void* dv, void* workspace,
                    size_t workspace_bytes, int B, int H, int N, int Nk, int D, int dtype,
                    float scale, int deterministic, const long long* strides,
                    fa2_stream_t stream) {
  if (!rowstats) return FA2_ERR_NULL_POINTER;
  if (int e = check_shape(B, H, N, D, dtype)) return e;
  // the per-tile maxima of |dout| follow the last tile of the row statistics (fa2_bwd_preprocess)
  const unsigned* tile_amax = reinterpret_cast<const unsigned*>(
      rowstats + static_cast<size_t>(B) * H * ((N + 127) / 128) * 256);
  return bwd_strided(q, k, v, dout, rowstats, tile_amax, dq, dk, dv, workspace, workspace_bytes, B,
                     H, N, Nk, D, dtype, scale, deterministic, strides, stream);
}

int fa2_bwd(const void* q, const void* k, const void* v, const void* dout, const float* rowstats,
            void* dq, void* dk, void* dv, void* workspace, size_t workspace_bytes, int B, int H,
            int N, int D, int dtype, float scale, int deterministic, fa2_stream_t stream) {
  return fa2_bwd_strided(q, k, v, dout, rowstats, dq, dk, dv, workspace, workspace_bytes, B, H, N,
                         N, D, dtype, scale, deterministic, nullptr, stream);
}

int fa2_bwd_mark_between(void* event) {
  t_mark_between = static_cast<cudaEvent_t>(event);
  return FA2_OK;
}

size_t fa2_set_spill_budget(size_t bytes) {
  return static_cast<size_t>(g_spill_budget.exchange(static_cast<long long>(bytes)));
}

int fa2_device_status(int* status_out) {
  if (!status_out) return FA2_ERR_NULL_POINTER;
  DeviceState* d = nullptr;
  if (int e = device_state(&d)) return e;
  cudaError_t ce = cudaDeviceSynchronize();
  if (ce != cudaSuccess) return static_cast<int>(ce);
  ce = cudaMemcpy(status_out, d->status, sizeof(int), cudaMemcpyDeviceToHost);
  if (ce != cudaSuccess) return static_cast<int>(ce);
  if (*status_out != 0) ce = cudaMemset(d->status, 0, sizeof(int));
  return static_cast<int>(ce);
}

int fa2_selftest_wait_timeout(fa2_stream_t stream) {
  DeviceState* d = nullptr;
  if (int e = device_state(&d)) return e;
  return static_cast<int>(launch_selftest_wait(d->status, static_cast<cudaStream_t>(stream)));
}

int fa2_selftest_mma(int form, const void* a, const void* b, float* c, int D, int dtype,
                     fa2_stream_t stream) {
  if (!a || !b || !c) return FA2_ERR_NULL_POINTER;
  if (form < 0 || form > 2) return FA2_ERR_SHAPE;
  if (int e = check_shape(1, 1, 128, D, dtype)) return e;
  if (D != padded_head_dim(D)) return FA2_ERR_HEAD_DIM;  // the self-test takes 32, 64, 128 only
  if (!aligned16(a) || !aligned16(b)) return FA2_ERR_MISALIGNED;
  DeviceState* d = nullptr;
  if (int e = device_state(&d)) return e;
  CUtensorMap ta, tb;
  // form 0 reads A [128, D] through TMA; forms 1 and 2 read A [128, 128] with plain loads.
  if (int e = make_map_of(&ta, form == 0 ? a : b, nullptr, 0, dtype, 1, 1, 128, D, 128)) return e;
  if (int e = make_map_of(&tb, b, nullptr, 0, dtype, 1, 1, 128, D, 128)) return e;
  return static_cast<int>(launch_selftest_mma(form, ta, tb, a, c, D, dtype, d->status,
                                              static_cast<cudaStream_t>(stream)));
}

}  // extern "C"

// ---------------------------------------------------------------------------------------
// Backward without any caller-provided or allocated workspace.
// ---------------------------------------------------------------------------------------
namespace fa2 {
// Row statistics (-lse*log2e, -delta) of up to kStaticRowstatTiles Q tiles live here instead
// of in a caller buffer.  In HOST code this name is only a handle for the runtime: the real
// device address comes from cudaGetSymbolAddress, once per device, below.
constexpr int kStaticRowstatTiles = 4096;  // 4096 tiles x 257 words = 4.02 MiB per GPU
static __device__ __align__(256) float g_static_rowstats[kStaticRowstatTiles * (256 + 1)];

namespace {
struct StaticScratch {
  std::once_flag once;
  float* ptr = nullptr;
  cudaError_t err = cudaSuccess;
};
StaticScratch g_static_scratch[kMaxDevices];

// Device address of g_static_rowstats on the CURRENT device (looked up on first use).
int static_rowstats(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kMaxDevices) return FA2_ERR_ARCH;
  StaticScratch& sc = g_static_scratch[dev];
  std::call_once(sc.once, [&] {
    sc.err = cudaGetSymbolAddress(reinterpret_cast<void**>(&sc.ptr), g_static_rowstats);
  });
  if (sc.err != cudaSuccess) return static_cast<int>(sc.err);
  if (sc.ptr == nullptr) return FA2_ERR_DRIVER;
  *out = sc.ptr;
  return FA2_OK;
}
}  // namespace
}  // namespace fa2

extern "C" int fa2_bwd_static_scratch(const void* q, const void* k, const void* v, const void* o,
                                      const void* dout, const float* lse, void* dq, void* dk,
                                      void* dv, int B, int H, int N, int D, int dtype, float scale,
                                      fa2_stream_t stream) {
  if (!q || !k || !v || !o || !dout || !lse || !dq || !dk || !dv) return FA2_ERR_NULL_POINTER;
  if (int e = check_shape(B, H, N, D, dtype)) return e;
  // Everything fa2_bwd would refuse is refused here, before the first launch: the preprocess
  // kernel writes the shared array, and a call that is going to fail must not touch it.
  if (D > 128) return FA2_ERR_WORKSPACE;  // that backward needs a caller workspace
  if (!std::isfinite(scale) || !(scale > 0.f)) return FA2_ERR_SCALE;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) || !aligned16(dout) ||
      !aligned16(dq) || !aligned16(dk) || !aligned16(dv))
    return FA2_ERR_MISALIGNED;
  const long long tiles = static_cast<long long>(B) * H * ((N + 127) / 128);
  if (tiles > kStaticRowstatTiles) return FA2_ERR_TOO_LARGE;
  float* rowstats = nullptr;
  if (int e = static_rowstats(&rowstats)) return e;
  // Every element of the part of the array that the kernels read is rewritten by the
  // preprocess launch (padding rows included), so nothing has to be cleared first.
  if (int e = fa2_bwd_preprocess(o, dout, lse, rowstats, B, H, N, D, dtype, stream)) return e;
  return fa2_bwd(q, k, v, dout, rowstats, dq, dk, dv, nullptr, 0, B, H, N, D, dtype, scale,
                 /*deterministic=*/1, stream);
}
