/*
 * attnres_b200.h -- C ABI of the B200 (sm_100a) AttnRes read kernels.
 *
 * The reference project (jon123boss/fast-attnres) is pure Python + Triton and
 * has no FFI of its own.  The seam this library plugs into is the pair of
 * torch.library operators that sit between its public `attnres()` function and
 * its Triton launches:
 *
 *   packed values : attnres::_fixed_tail_forward_with_aux / _fixed_tail_backward
 *                   (src/attnres/_kernels/fixed_tail.py:904-1034)
 *   source lists  : attnres::_fixed_tail_sources_forward_with_aux /
 *                   _fixed_tail_sources_backward
 *                   (src/attnres/_kernels/fixed_tail_sources.py:78-101, launched by
 *                   src/attnres/_kernels/fla_full_sources.py:752-894)
 *
 * Every entry point below takes plain pointers, sizes and a CUDA stream.  The
 * caller allocates inputs, outputs and the dquery workspace and keeps them alive
 * until the stream has run the work; the library allocates nothing (the one
 * piece of device memory it owns is the fixed scratch array documented at
 * attnres_b200_backward_static_scratch).  No compute entry point synchronises,
 * and every argument error is found on the host before a kernel is launched.
 * Calls are re-entrant; calls on different streams may run concurrently as long
 * as they do not share output or workspace buffers.
 *
 * Math (per flattened position n, sources s = 0..S-1, BF16 storage, FP32
 * arithmetic; validation/oracle.py:5-19):
 *
 *   t_s   = v_s[D-R : D]                       the "tail key" of source s
 *   r_s   = rsqrt(mean(t_s^2) + eps)
 *   z_s   = scale * r_s * sum(t_s * q)         saved in `logits`
 *   p     = softmax_s(z)                       (max, 1/sum) saved in `stats`
 *   out   = bf16(sum_s p_s * v_s)
 */
#ifndef ATTNRES_B200_H_
#define ATTNRES_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ATTNRES_B200_ABI_VERSION 3
/* Envelope of the reference operator (src/attnres/_sources.py:12-13). */
#define ATTNRES_B200_MAX_SOURCES 129
#define ATTNRES_B200_MAX_WIDTH 8192

/* Status codes returned by every entry point (0 = success). */
#define ATTNRES_B200_OK 0
#define ATTNRES_B200_ERR_NULL_POINTER 1
#define ATTNRES_B200_ERR_BAD_SOURCE_COUNT 2   /* S outside 1..129 */
#define ATTNRES_B200_ERR_BAD_WIDTH 3          /* D outside 1..8192 */
#define ATTNRES_B200_ERR_BAD_RANK 4           /* R outside 1..D */
#define ATTNRES_B200_ERR_BAD_ROWS 5           /* N < 1 */
#define ATTNRES_B200_ERR_BAD_SCALAR 6         /* eps <= 0 or non-finite, scale non-finite */
#define ATTNRES_B200_ERR_MISALIGNED 7         /* a BF16 pointer that is not 2-byte aligned */
#define ATTNRES_B200_ERR_WORKSPACE 8          /* dquery workspace too small */
#define ATTNRES_B200_ERR_CUDA 9               /* a CUDA runtime call failed (launch, attribute) */
#define ATTNRES_B200_ERR_BAD_FLAGS 10
#define ATTNRES_B200_ERR_NOTHING_TO_DO 11     /* backward with neither value nor query gradient */
#define ATTNRES_B200_ERR_STATIC_SCRATCH 12    /* shape needs more than the built-in dquery scratch */

/* `flags` bits. */
#define ATTNRES_B200_FLAG_DEFAULT 0u
/* Use the layout-generic kernels even when the inputs qualify for the
 * TMA-staged fast path (used by tests to cover both families). */
#define ATTNRES_B200_FLAG_FORCE_GENERIC 1u
/* Backward: take the one-pass streaming kernel whenever the saved output is given and the
 * shape allows it, whatever the library's own choice would be (tests, tuning). */
#define ATTNRES_B200_FLAG_PREFER_STREAM 2u
/* Backward: ACCUMULATE the value gradients.  Every `dsrc_ptrs[s]` row is read, the gradient of
 * this call is added to it in FP32 and the sum is rounded to BF16 once: dsrc[s] += dV_s.  For
 * training loops that own one running gradient buffer per source and read the same sources
 * many times (the role of autograd's accumulation of the per-read gradients after
 * src/attnres/_kernels/fixed_tail_sources.py:141-183; the reference has no fused form).
 * Needs `dsrc_ptrs`.  Runs in the one-pass kernel when the saved output is given and the
 * layout is in the fast class (pass the forward's `out` and `out_residual`; the forward
 * writes the residual for any shape when asked), otherwise in the layout-generic kernel.
 * The query gradient is not accumulated: `dq_*` are overwritten as usual. */
#define ATTNRES_B200_FLAG_ACCUMULATE_DV 4u

/* Replaces nothing in the reference; lets a binding check it loaded the
 * library it was written against. */
int attnres_b200_abi_version(void);

/* Human-readable text for a status code (static storage, never NULL). */
const char* attnres_b200_status_string(int status);

/*
 * Forward read.  Replaces the Triton launches
 * `_packed_online_forward_kernel` (src/attnres/_kernels/fixed_tail.py:927-958)
 * and `_fla_standard_forward_kernel`
 * (src/attnres/_kernels/fla_full_sources.py:776-804).
 *
 *   src_ptrs[s]        device address of row 0 of source s (BF16)
 *   src_row_stride[s]  elements between consecutive rows of source s (may be 0)
 *   src_feat_stride[s] elements between consecutive features of source s
 *                      (the three arrays live in HOST memory, length S; a packed
 *                      [S,N,D] tensor is passed as base + s*stride(0))
 *   query              device BF16 [R], element stride `query_stride`
 *   out                device BF16 [N,D], row stride `out_row_stride`, feature stride 1
 *   out_residual       optional device uint16 [N,D] contiguous: what the BF16 rounding of
 *                      `out` dropped, so that the pair is a full FP32 copy of the result in
 *                      the space of two BF16 rows:
 *                        float_bits(result) = ((bf16_bits(out) << 16) | out_residual) - 0x8000
 *                      (exact except for the one-in-2^17 tie that rounds down, which is one
 *                      FP32 ulp off).  Ask attnres_b200_wants_output_residual
 *                      whether the backward of this shape profits from it; NULL skips it.
 *                      The reference saves a separate FP32 copy of the output
 *                      (fixed_tail.py:917-919); its backward and this one then form
 *                      delta = sum_d dO * result from the same FP32 values.
 *   logits             device FP32 [S,N] contiguous: scaled logits z_s
 *   stats              device FP32 [2,N] contiguous: row max, then 1/sum(exp(z-max))
 *   stream             a cudaStream_t (0 = legacy default stream)
 */
int attnres_b200_forward(
    const void* const* src_ptrs, const int64_t* src_row_stride,
    const int64_t* src_feat_stride,
    int32_t S, int64_t N, int32_t D, int32_t R,
    const void* query, int64_t query_stride,
    float eps, float scale,
    void* out, int64_t out_row_stride, void* out_residual,
    float* logits, float* stats,
    uint32_t flags, void* stream);

/*
 * Forward read with the consumer's LayerNorm computed in the epilogue.  In the reference's
 * model every read is followed by a LayerNorm of its result before the sublayer consumes it
 * (benchmarks/model.py:156, 170 of the reference); the reference has no fused form, its
 * LayerNorm re-reads `out` from memory.  Here the row is normalised while it is still in
 * registers.  Everything attnres_b200_forward writes is written unchanged; in addition
 *
 *   normed_out   device BF16 [N,D] contiguous:
 *                  (out - mean) * rstd * norm_weight + norm_bias
 *                over the D features of the BF16-rounded `out` row (so the result equals a
 *                LayerNorm applied to `out` afterwards, computed in FP32)
 *   norm_stats   device FP32 [2,N] contiguous: mean, then rstd = 1/sqrt(var + norm_eps)
 *                (biased variance), what a LayerNorm backward needs
 *   norm_weight, device FP32 [D] contiguous; NULL means ones / zeros
 *   norm_bias
 *
 * The backward of the pair is the LayerNorm backward (from `out`, `norm_stats` and the
 * gradient of `normed_out`) followed by attnres_b200_backward.
 */
int attnres_b200_forward_layer_norm(
    const void* const* src_ptrs, const int64_t* src_row_stride,
    const int64_t* src_feat_stride,
    int32_t S, int64_t N, int32_t D, int32_t R,
    const void* query, int64_t query_stride,
    float eps, float scale,
    void* out, int64_t out_row_stride, void* out_residual,
    float* logits, float* stats,
    const float* norm_weight, const float* norm_bias, float norm_eps,
    void* normed_out, float* norm_stats,
    uint32_t flags, void* stream);

/*
 * Backward of the LayerNorm that attnres_b200_forward_layer_norm applies, from what that
 * forward wrote (no counterpart in the reference, which runs a separate LayerNorm and leaves
 * its backward to the framework):
 *
 *   grad_normed       device BF16 [N,D], row stride `grad_row_stride`, feature stride 1
 *   out, norm_stats   as written by the forward; norm_weight as passed to it (NULL = ones)
 *   grad_out          device BF16 [N,D] contiguous: the gradient with respect to `out`
 *                     (add any gradient that reaches `out` directly, then hand the sum to
 *                     attnres_b200_backward as its `grad_out`)
 *   partials          device FP32 workspace [partial_rows, 2 D], partial_rows >=
 *                     attnres_b200_layer_norm_workspace_rows(N, D, device)
 *   grad_weight_bias  device FP32 [2 D]: the weight gradient, then the bias gradient, summed
 *                     in a fixed order
 *
 * Needs D % 8 == 0 and 16-byte aligned rows (ATTNRES_B200_ERR_MISALIGNED otherwise; a caller
 * with another layout computes the LayerNorm backward itself).
 */
int32_t attnres_b200_layer_norm_workspace_rows(int64_t N, int32_t D, int32_t device);
int attnres_b200_layer_norm_backward(
    const void* grad_normed, int64_t grad_row_stride, const void* out, const float* norm_stats,
    const float* norm_weight, int64_t N, int32_t D,
    void* grad_out, float* partials, int32_t partial_rows, float* grad_weight_bias,
    void* stream);

/*
 * 1 when the backward of this shape (aligned layout assumed) is faster with the forward's
 * output and residual (it then finishes every source in one pass instead of staging the
 * whole position in shared memory), 0 otherwise.  Pure host function; plays the role of the
 * reference's save-versus-recompute policy (fla_full_sources.py:146-161).
 */
int32_t attnres_b200_wants_output_residual(int32_t S, int32_t D, int32_t R);

/*
 * Rows the dquery workspace must hold for a backward call of this shape on
 * `device`: `dq_partials` is FP32 [rows, R].  Pure host function (replaces the
 * `[N,R]` token partial buffer the reference allocates,
 * src/attnres/_kernels/fixed_tail.py:981-984).  Returns a negative status on
 * error.
 */
int32_t attnres_b200_dq_workspace_rows(int64_t N, int32_t S, int32_t D, int32_t R,
                                       int32_t device);

/*
 * Backward read.  Replaces `_packed_online_backward_kernel` +
 * `_packed_query_reduce_kernel` (src/attnres/_kernels/fixed_tail.py:987-1034)
 * and `_fla_standard_backward_kernel` + the query reducers
 * (src/attnres/_kernels/fla_full_sources.py:845-893).
 *
 *   grad_out           device BF16 [N,D] with arbitrary row/feature strides
 *   logits, stats      as written by attnres_b200_forward for the same inputs
 *   out_saved,         optional: `out` and `out_residual` of the forward (16-bit [N,D]
 *   out_residual       contiguous).  Both or neither; NULL for both is always correct.
 *   dsrc_ptrs[s]       device BF16 [N,D] gradient of source s, row stride
 *                      dsrc_row_stride[s], feature stride 1 (host arrays, length S).
 *                      NULL skips the value gradients.  Overwritten, or with
 *                      ATTNRES_B200_FLAG_ACCUMULATE_DV added to (the S buffers must
 *                      then be distinct and must not overlap: a row is fetched before
 *                      it is updated).
 *   dq_partials        device FP32 workspace [dq_partial_rows, R]
 *   dq_bf16, dq_f32    device [R] outputs, contiguous; either may be NULL.  The
 *                      FP32 form is the one to all-reduce across GPUs before the
 *                      BF16 cast.  Both NULL skips the query gradient.
 *
 * The query gradient is reduced in a fixed order, so repeated calls are
 * bit-identical; the second stage adds the partial rows in FP64 and rounds once.
 */
int attnres_b200_backward(
    const void* const* src_ptrs, const int64_t* src_row_stride,
    const int64_t* src_feat_stride,
    int32_t S, int64_t N, int32_t D, int32_t R,
    const void* query, int64_t query_stride,
    float eps, float scale,
    const void* grad_out, int64_t go_row_stride, int64_t go_feat_stride,
    const float* logits, const float* stats,
    const void* out_saved, const void* out_residual,
    void* const* dsrc_ptrs, const int64_t* dsrc_row_stride,
    float* dq_partials, int32_t dq_partial_rows,
    void* dq_bf16, float* dq_f32,
    uint32_t flags, void* stream);

/*
 * Name of the kernel family the library would pick for a call of this shape
 * ("tma" or "generic"), for logs and tests.  `aligned` is nonzero when every
 * pointer is 16-byte aligned, every row stride a multiple of 8 elements and
 * every feature stride 1.  `backward` selects the backward policy, for a caller
 * that follows attnres_b200_wants_output_residual (a backward that is handed no
 * saved output although the shape wants one may fall back to "generic").
 */
const char* attnres_b200_kernel_family(int32_t S, int32_t D, int32_t R, int32_t aligned,
                                       int32_t backward);

/*
 * Backward read for callers that cannot hand the library a dquery workspace.
 * It has no counterpart in the reference.
 *
 * Some hosts may not allocate device memory at the point where they call the
 * operator: an inference or training runtime that reserves the whole GPU in
 * one arena at start-up and forbids cudaMalloc afterwards, a plugin running
 * inside someone else's captured region or real-time loop, or a binding from a
 * language whose tensors cannot be created from inside a callback.  For them the
 * FP32 [rows, R] scratch of the two-stage dquery reduction lives inside the
 * library, in a fixed device array of ATTNRES_B200_STATIC_SCRATCH_FLOATS floats
 * (9.25 MiB, held by every GPU that loads the library until the process exits).
 *
 * Arguments and results are those of attnres_b200_backward without
 * `dq_partials` / `dq_partial_rows`; inputs and outputs still belong to the
 * caller.  The call allocates nothing and frees nothing.
 *
 *   - Limit: attnres_b200_dq_workspace_rows(N, S, D, R, device) * R must not
 *     exceed ATTNRES_B200_STATIC_SCRATCH_FLOATS (any N up to R = 2048; larger R
 *     only with few rows).  Otherwise nothing is launched and the call returns
 *     ATTNRES_B200_ERR_STATIC_SCRATCH; use attnres_b200_backward instead.
 *   - The first call on each device that asks for a query gradient looks up
 *     the device address of the array (one driver query, cached per device for
 *     the life of the process; a process that calls cudaDeviceReset must reload
 *     the library).  Make that first call outside any CUDA stream capture.
 *   - Arguments are checked exactly as attnres_b200_backward checks them, before
 *     the size limit is looked at; a call with both `dq_*` NULL needs no scratch
 *     and is never refused for its size.
 *   - All calls on a device share the one array.  Its contents are whatever the
 *     previous call left; this is harmless because every element the second
 *     stage reads is written by the first stage of the same call, so nothing has
 *     to be cleared.  Two calls that overlap on the GPU (different streams, or
 *     graphs replayed concurrently) race on the array: serialise them.
 */
#define ATTNRES_B200_STATIC_SCRATCH_FLOATS 2424832 /* 148 SMs: 1184 rows x 2048, 1776 rows x 1024 */
int attnres_b200_backward_static_scratch(
    const void* const* src_ptrs, const int64_t* src_row_stride,
    const int64_t* src_feat_stride,
    int32_t S, int64_t N, int32_t D, int32_t R,
    const void* query, int64_t query_stride,
    float eps, float scale,
    const void* grad_out, int64_t go_row_stride, int64_t go_feat_stride,
    const float* logits, const float* stats,
    const void* out_saved, const void* out_residual,
    void* const* dsrc_ptrs, const int64_t* dsrc_row_stride,
    void* dq_bf16, float* dq_f32,
    uint32_t flags, void* stream);

/*
 * Diagnostics (no counterpart in the reference).  The TMA-staged kernels bound
 * every wait on a shared-memory barrier; a CTA that gives up sets a sticky
 * device-side flag and finishes with meaningless results instead of hanging.
 * This call copies the flag of the current device to `*flag` (0 = no kernel ever
 * gave up) and optionally clears it.  It SYNCHRONISES the device: use it in
 * tests and after failures, not on the hot path.  A launch whose kernel gives
 * up has long returned ATTNRES_B200_OK (launches are asynchronous), so a
 * training loop should read the flag at step boundaries or before it trusts a
 * checkpoint.
 */
int attnres_b200_error_flag(int32_t* flag, int32_t clear);

/*
 * Self-test of the give-up path (no counterpart in the reference).  Launches one
 * tiny CTA on `stream` that announces 32 bytes on a shared-memory barrier, copies
 * only 16, and waits on it with the kernels' own bounded wait and a limit of
 * `limit_ns` nanoseconds (1 000 .. 100 000 000).  The wait runs out, the CTA
 * raises the device error flag and returns; nothing hangs and no memory outside
 * the CTA is written.  `scratch16` is any 16-byte aligned device buffer of at
 * least 16 readable bytes.  Afterwards attnres_b200_error_flag reports 1.
 */
int attnres_b200_selftest_wait_limit(const void* scratch16, uint64_t limit_ns, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ATTNRES_B200_H_ */
