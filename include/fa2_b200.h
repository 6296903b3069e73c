/*
 * fa2_b200.h — C ABI of the B200 (sm_100a) causal FlashAttention-2 library.
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes, launches on the
 * stream it is given and returns without synchronising (the one exception,
 * fa2_device_status, says so).  The caller owns every buffer.  All tensors are dense
 * row-major [B, H, N, D] (strides implied) on the current CUDA device; lse is dense fp32
 * [B, H, N].  D is a multiple of 8 between 8 and 256 (32, 64, 128 and 256 are the native tile
 * widths; sizes in between run zero-padded to the next one through TMA out-of-bounds fill, with
 * no extra memory traffic); dtype 0 = fp16, 1 = bf16.  Above D = 128 the backward has a single,
 * deterministic strategy that needs a workspace (fa2_bwd_workspace_bytes) whatever
 * `deterministic` says, and fa2_bwd_static_scratch is not available (FA2_ERR_WORKSPACE).
 *
 * Return value: 0 = success; negative = argument / environment error (table below);
 * positive = a cudaError_t from a launch or attribute call.
 *
 * The functions below replace these pieces of flash-attention-triton (paths inside that
 * project):
 *   fa2_fwd             src/flash_attention_triton/flash_attention_2.py:61-144
 *                       (_flash_attention_forward) + _triton_kernels_v2.py:11-189
 *   fa2_bwd_preprocess  _triton_kernels_v2.py:532-608 (_backward_preprocess_do_o_dot),
 *                       launched from flash_attention_2.py:218-234
 *   fa2_bwd             flash_attention_2.py:147-277 (_flash_attention_backward) +
 *                       _triton_kernels_v2.py:192-529; `deterministic` mirrors
 *                       SEQUENCE_PARALLEL=False of the reference's config tables
 *                       (flash_attention_2.py:570-589)
 */
#ifndef FA2_B200_H_
#define FA2_B200_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FA2_ABI_VERSION 3

#define FA2_DTYPE_FP16 0
#define FA2_DTYPE_BF16 1

#define FA2_OK 0
#define FA2_ERR_NULL_POINTER (-1)      /* a required pointer is NULL */
#define FA2_ERR_HEAD_DIM (-2)          /* D not a multiple of 8 in [8, 256] */
#define FA2_ERR_DTYPE (-3)             /* dtype not FA2_DTYPE_FP16 / FA2_DTYPE_BF16 */
#define FA2_ERR_MISALIGNED (-4)        /* a tensor pointer is not 16-byte aligned */
#define FA2_ERR_SHAPE (-5)             /* B, H or N <= 0, B*H > 65535, N too large, Nk not in [1, N] */
#define FA2_ERR_ARCH (-6)              /* current device is not compute capability 10.x */
#define FA2_ERR_DEVICE_STATUS (-7)     /* a kernel gave up on a bounded wait */
#define FA2_ERR_DRIVER (-8)            /* cuTensorMapEncodeTiled unavailable or failed */
#define FA2_ERR_SCALE (-9)             /* softmax scale not finite or not > 0 */
#define FA2_ERR_WORKSPACE (-10)        /* the mode needs a workspace: NULL, or smaller than its minimum */
#define FA2_ERR_TOO_LARGE (-11)        /* fa2_bwd_static_scratch: B*H*ceil(N/128) > 4096 */
#define FA2_ERR_STRIDE (-12)           /* a stride is <= 0, not a multiple of 8 elements, or row < D */

/* Opaque stream handle: pass a cudaStream_t (NULL = legacy default stream). */
typedef void* fa2_stream_t;

int fa2_abi_version(void);

/* Static, human-readable text for a return code of this library. */
const char* fa2_strerror(int code);

/*
 * Forward: O = softmax_causal(scale * Q K^T) V, lse[b,h,i] = log sum_j exp(scale * s_ij)
 * (natural log).  Replaces _flash_attention_forward / _forward_kernel; unlike the
 * reference (flash_attention_2.py:98-100) lse is not padded and no scratch buffer is used.
 * The kernel runs one CTA per SM; the CTAs draw their work items from a device counter that
 * the library takes from a ring of 1024 (a new one per call, so calls on different streams do
 * not share one).  A call captured into a CUDA graph keeps its counter: replays of that graph
 * must not overlap each other.
 */
int fa2_fwd(const void* q, const void* k, const void* v, void* o, float* lse,
            int B, int H, int N, int D, int dtype, float scale, fa2_stream_t stream);

/*
 * Backward preprocess.  Computes delta[b,h,i] = sum_d float(o[b,h,i,d]) * float(dout[b,h,i,d])
 * (replaces _backward_preprocess_do_o_dot) and stores it, together with lse * log2(e), both
 * NEGATED (the kernels use them as FMA / ADD addends), in the tile-blocked fp32 array
 * `rowstats` that fa2_bwd consumes:
 *     rowstats[(b*H + h)][t][0][r] = -lse[b,h,128*t + r] * log2(e)  (-inf for rows >= N)
 *     rowstats[(b*H + h)][t][1][r] = -delta[b,h,128*t + r]          (0    for rows >= N)
 * with t in [0, ceil(N/128)), r in [0, 128).  One 1 KiB bulk copy then stages both vectors of
 * a Q tile; the padding plays the role of the reference's seqlen_q_rounded buffers
 * (flash_attention_2.py:98-100,180).  rowstats must hold fa2_rowstats_bytes() bytes and be
 * 16-byte aligned.
 */
int fa2_bwd_preprocess(const void* o, const void* dout, const float* lse, float* rowstats,
                       int B, int H, int N, int D, int dtype, fa2_stream_t stream);

size_t fa2_rowstats_bytes(int B, int H, int N);

/*
 * Backward main.  Inputs q,k,v,dout and rowstats (from fa2_bwd_preprocess); outputs
 * dq,dk,dv in the input dtype.  dK and dV are the same bits in every mode (every KV tile sums
 * its Q tiles from the last one down to the diagonal); the modes differ in how dQ is formed and
 * in the workspace they need (`workspace`, 256-byte aligned, `workspace_bytes` long; the call
 * never writes beyond it and returns FA2_ERR_WORKSPACE when it is below the mode's minimum).
 *   deterministic == 1 ("recompute"): dK/dV kernel + a separate dQ kernel that recomputes S and
 *     dP; every output tile has one owner and a fixed accumulation order, so results are
 *     bit-identical across runs, SM counts and (batch, head) partitionings.  No workspace
 *     (memory O(N) like the reference, flash_attention_2.py:195-196).
 *   deterministic == 2 ("spill"): equally deterministic, and the fastest mode at D = 128 when the
 *     scratch can be afforded.  The dK/dV kernel also writes every 16-bit dS tile (32 KiB per
 *     (KV tile, Q tile) pair) to the workspace and a second kernel forms dQ from those tiles with
 *     one tensor-core product per pair in ascending KV order, bound by reading them back from
 *     HBM.  Trades memory (quadratic in N per head: 68 MB at N = 8192) for time.  The problem is
 *     worked through in chunks of whole (batch, head) problems that fit the workspace given, one
 *     after the other on the stream; chunks of 2048 or more 128-row tiles run within 1 % of a
 *     single chunk (1024 tiles: 3 % slower, 512: 11 %, one head of 64 tiles: 3.9x), the minimum
 *     is one head's tiles, and the split never changes a bit of the results.  dQ differs from mode 1 in the last bit at
 *     most (other polynomial / MUFU assignment of the exponentials).  It is the only backward
 *     for head dims above 128, where it is a scores kernel plus dV, dK and dQ kernels over two
 *     scratch tensors (64 KiB per tile pair) and serves every value of `deterministic`.  No
 *     counterpart in the reference.
 *   deterministic == 0 ("atomic"): one fused kernel per KV tile adds its dQ contributions into
 *     the fp32 workspace with atomic adds (the reference's SEQUENCE_PARALLEL mode,
 *     _triton_kernels_v2.py:337-339), then a convert pass writes dq, rounding once like
 *     dq.copy_(dq_accum) (flash_attention_2.py:277).  The workspace is the fp32 accumulator
 *     [B*H][ceil(N/128)*128][D padded to 32/64/128]; this call zeroes it itself.  Its layout is
 *     private (tile-blocked so that every warp-wide atomic is one contiguous 512-byte run).
 */
int fa2_bwd(const void* q, const void* k, const void* v, const void* dout,
            const float* rowstats,
            void* dq, void* dk, void* dv, void* workspace, size_t workspace_bytes,
            int B, int H, int N, int D, int dtype, float scale, int deterministic,
            fa2_stream_t stream);

/*
 * Bytes of workspace fa2_bwd should be given for a value of `deterministic` (see there): the
 * exact size for modes 0 and 1 (0 bytes), the recommended size for mode 2: the tiles of as
 * many heads as make a chunk of 2048 128-row tiles (32 heads at N = 8192: 2.2 GB; about 256 KiB
 * per row of a head, so linear in N and independent of B * H), capped by fa2_set_spill_budget,
 * never less than one head.
 */
size_t fa2_bwd_workspace_bytes(int B, int H, int N, int D, int deterministic);

/*
 * Upper bound of what fa2_bwd_workspace_bytes recommends for mode 2, in bytes (default 8 GiB);
 * returns the previous value.  fa2_bwd itself never reads it: it works with the
 * workspace it is given.  Process-wide.  No counterpart in the reference.
 */
size_t fa2_set_spill_budget(size_t bytes);

/*
 * The same three operations on tensors that are not dense: any batch, head and row strides
 * with a contiguous last dimension (for instance a [B, N, H, D] buffer viewed as
 * [B, H, N, D]).  The reference makes such inputs contiguous with a copy
 * (flash_attention_2.py:316, 170-171); here the strides go into the TMA descriptors and the
 * copy disappears.
 *
 * `strides` holds one (batch, head, row) triple of ELEMENT strides per tensor argument, in
 * argument order:
 *     fa2_fwd_strided             q, k, v, o                      (12 values)
 *     fa2_bwd_preprocess_strided  o, dout                         ( 6 values)
 *     fa2_bwd_strided             q, k, v, dout, dq, dk, dv       (21 values)
 * A triple of zeros means "dense"; strides == NULL means every tensor is dense (the plain
 * entry points above are exactly that).  Every stride must be a positive multiple of 8
 * elements (16 bytes) and the row stride at least D, else FA2_ERR_STRIDE; strides of
 * dimensions of size 1 are ignored.  lse, rowstats and the workspace keep their own layouts.
 *
 * They also take the number of key rows separately: q, o, dout, dq and lse have N rows, k, v,
 * dk and dv have Nk rows, 1 <= Nk <= N.  The causal mask is aligned at the top left like the
 * reference's (_triton_kernels_v2.py:139-147): query row i sees keys 0 .. min(i, Nk - 1).
 * Keys beyond row N - 1 would never be seen by any query, which is why Nk > N is refused
 * (FA2_ERR_SHAPE): pass the first N rows of k and v and zero the rest of dk and dv.
 */
int fa2_fwd_strided(const void* q, const void* k, const void* v, void* o, float* lse,
                    int B, int H, int N, int Nk, int D, int dtype, float scale,
                    const long long* strides, fa2_stream_t stream);
int fa2_bwd_preprocess_strided(const void* o, const void* dout, const float* lse,
                               float* rowstats, int B, int H, int N, int D, int dtype,
                               const long long* strides, fa2_stream_t stream);
int fa2_bwd_strided(const void* q, const void* k, const void* v, const void* dout,
                    const float* rowstats,
                    void* dq, void* dk, void* dv, void* workspace, size_t workspace_bytes,
                    int B, int H, int N, int Nk, int D, int dtype, float scale,
                    int deterministic, const long long* strides, fa2_stream_t stream);

/*
 * Diagnostics for benchmarks: the next fa2_bwd call of the calling thread that runs two kernels
 * (deterministic == 1: dK/dV kernel, dQ kernel; deterministic == 2 at D <= 128: dK/dV kernel,
 * dQ consumer kernel; the first chunk when the call is chunked) records `event`, a cudaEvent_t, on
 * its stream between the two, so that the two parts of one call can be timed in place.  One
 * shot: the event is forgotten once recorded; NULL cancels.  No counterpart in the reference.
 */
int fa2_bwd_mark_between(void* event);

/*
 * Reads and clears the per-device status word that kernels set when a bounded wait
 * expires (they then drain and return instead of hanging).  Synchronises the device.
 * *status_out = 0 when every kernel since the last call ran to completion.
 * No counterpart in the reference (Triton kernels have no such protocol).
 */
int fa2_device_status(int* status_out);

/*
 * Diagnostics: runs one tensor-core tile product through a single operand form used by the
 * attention kernels and writes the fp32 result, so that a driver / toolkit change that
 * breaks a descriptor encoding shows up as a wrong tile rather than as wrong gradients.
 *   form 0: C[128,128] = A[128,D] * B[128,D]^T      (both operands row-major, "K-major")
 *   form 1: C[128,D]   = P[128,128] * B[128,D]      (P from tensor memory, B row-major)
 *   form 2: C[128,D]   = A[128,128]^T * B[128,D]    (A staged transposed in shared memory)
 * a, b: 16-bit inputs of `dtype`; c: fp32 output.  No counterpart in the reference.
 */
/*
 * Diagnostics: launches one small CTA whose threads wait for a barrier that nobody arrives at.
 * The wait is bounded like every wait in this library: after about two seconds the kernel sets
 * the status word (fa2_device_status then reports 0x10000 | 120), its other waiters leave, and it
 * ends normally; the context stays usable.  Shows that a lost signal cannot hang the GPU.
 * No counterpart in the reference.
 */
int fa2_selftest_wait_timeout(fa2_stream_t stream);

int fa2_selftest_mma(int form, const void* a, const void* b, float* c,
                     int D, int dtype, fa2_stream_t stream);

/*
 * Whole deterministic backward (preprocess + dK/dV + dQ) for callers that must not allocate
 * device memory and have no workspace to hand in: code running inside a CUDA-graph replay
 * loop, a plugin called from a framework that owns the allocator, a real-time serving loop
 * in which cudaMalloc (a device-wide synchronising call) is off limits.  The row statistics
 * that fa2_bwd_preprocess normally writes into a caller buffer go into a 4 MiB array that
 * is part of the library image on every GPU that loads it.  The caller passes only inputs
 * (q, k, v, o, dout, lse from fa2_fwd) and outputs (dq, dk, dv); results are bit-identical
 * to fa2_bwd_preprocess + fa2_bwd(deterministic = 1).
 *   Limit: B*H*ceil(N/128) <= 4096 Q tiles (e.g. B*H = 64 at N = 8192); larger problems
 *   return FA2_ERR_TOO_LARGE and launch nothing.
 *   The first call on each device looks up the array's device address (one runtime query,
 *   no allocation); make that first call outside any stream capture.
 *   All calls on a device share the one array: two calls whose kernels may overlap on the
 *   GPU (different streams, no dependency) race on it.  Calls on one stream are safe; the
 *   array keeps the last call's contents and each call rewrites every value it reads.
 * This entry point has no counterpart in the reference.
 */
int fa2_bwd_static_scratch(const void* q, const void* k, const void* v, const void* o,
                           const void* dout, const float* lse, void* dq, void* dk, void* dv,
                           int B, int H, int N, int D, int dtype, float scale,
                           fa2_stream_t stream);

#ifdef __cplusplus
}
#endif

#endif /* FA2_B200_H_ */
